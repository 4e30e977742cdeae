"""Pipeline parallelism hand-off: stage-to-stage activation/gradient transfer on NCCL point-to-point,
issued on a dedicated stream so that it overlaps with the stage's compute.  This path stays on NCCL by
design (it is one producer and one consumer per link; there is nothing to fuse), the library's own
kernels serve the collectives."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class PipelineP2P:
    def __init__(self, group=None):
        self.group = group
        self.stream = torch.cuda.Stream()
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    @property
    def prev_rank(self) -> Optional[int]:
        return self.rank - 1 if self.rank > 0 else None

    @property
    def next_rank(self) -> Optional[int]:
        return self.rank + 1 if self.rank + 1 < self.world else None

    def send_forward(self, t: torch.Tensor) -> Optional["torch.cuda.Event"]:
        """Queue `t` for the next stage; returns an event that fires when the send has finished."""
        if self.next_rank is None:
            return None
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            dist.send(t, self.next_rank, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        t.record_stream(self.stream)
        return ev

    def recv_forward(self, shape, dtype=torch.bfloat16) -> Optional[torch.Tensor]:
        """Activations from the previous stage; the current stream waits for their arrival only."""
        if self.prev_rank is None:
            return None
        buf = torch.empty(tuple(shape), dtype=dtype, device="cuda")
        with torch.cuda.stream(self.stream):
            dist.recv(buf, self.prev_rank, group=self.group)
        torch.cuda.current_stream().wait_stream(self.stream)
        return buf

    def send_backward(self, g: torch.Tensor):
        if self.prev_rank is None:
            return None
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            dist.send(g, self.prev_rank, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        g.record_stream(self.stream)
        return ev

    def recv_backward(self, shape, dtype=torch.bfloat16) -> Optional[torch.Tensor]:
        if self.next_rank is None:
            return None
        buf = torch.empty(tuple(shape), dtype=dtype, device="cuda")
        with torch.cuda.stream(self.stream):
            dist.recv(buf, self.next_rank, group=self.group)
        torch.cuda.current_stream().wait_stream(self.stream)
        return buf

    def run_gpipe(self, stage_fn, microbatches: List[torch.Tensor], act_shape, dtype=torch.bfloat16) -> List[torch.Tensor]:
        """Forward-only GPipe schedule over `microbatches` (used on the first stage; later stages receive)."""
        outs = []
        for i in range(len(microbatches)):
            x = microbatches[i] if self.prev_rank is None else self.recv_forward(act_shape, dtype)
            y = stage_fn(x)
            if self.next_rank is not None:
                self.send_forward(y)
            outs.append(y)
        torch.cuda.current_stream().wait_stream(self.stream)
        return outs
