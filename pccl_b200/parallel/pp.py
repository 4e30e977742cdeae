"""Pipeline parallelism hand-off: stage-to-stage activation/gradient transfer on torch.distributed point-to-point
(NCCL between GPUs; gloo between CPU ranks, which is how the schedules are tested), issued on a dedicated stream so
that it overlaps with the stage's compute.  This path stays on the library that owns point-to-point by design (it is
one producer and one consumer per link; there is nothing to fuse); the library's own kernels serve the collectives.

Two schedules: ``run_gpipe`` (forward only) and ``run_1f1b`` (training: warm-up forwards, one forward and one backward
alternating, cool-down backwards; a stage holds at most ``stages - index`` activations).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class PipelineP2P:
    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.cuda = dist.get_backend(group) == "nccl"
        self.device = torch.device("cuda", torch.cuda.current_device()) if self.cuda else torch.device("cpu")
        self.stream = torch.cuda.Stream() if self.cuda else None

    @property
    def prev_rank(self) -> Optional[int]:
        return self.rank - 1 if self.rank > 0 else None

    @property
    def next_rank(self) -> Optional[int]:
        return self.rank + 1 if self.rank + 1 < self.world else None

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    # ---- one-directional hand-offs -------------------------------------------------------------------------------
    def _send(self, t: torch.Tensor, peer: int):
        if not self.cuda:
            dist.send(t.contiguous(), self._global(peer), group=self.group)
            return None
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            dist.send(t, self._global(peer), group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        t.record_stream(self.stream)
        return ev

    def _recv(self, shape, dtype, peer: int) -> torch.Tensor:
        buf = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        if not self.cuda:
            dist.recv(buf, self._global(peer), group=self.group)
            return buf
        with torch.cuda.stream(self.stream):
            dist.recv(buf, self._global(peer), group=self.group)
        torch.cuda.current_stream().wait_stream(self.stream)
        return buf

    def send_forward(self, t: torch.Tensor):
        """Queue `t` for the next stage; on GPUs returns an event that fires when the send has finished."""
        return None if self.next_rank is None else self._send(t, self.next_rank)

    def recv_forward(self, shape, dtype=torch.bfloat16) -> Optional[torch.Tensor]:
        """Activations from the previous stage; the current stream waits for their arrival only."""
        return None if self.prev_rank is None else self._recv(shape, dtype, self.prev_rank)

    def send_backward(self, g: torch.Tensor):
        return None if self.prev_rank is None else self._send(g, self.prev_rank)

    def recv_backward(self, shape, dtype=torch.bfloat16) -> Optional[torch.Tensor]:
        return None if self.next_rank is None else self._recv(shape, dtype, self.next_rank)

    # ---- two-directional hand-offs: a send and a receive posted together, so that two neighbours that both want to
    # send first cannot block each other --------------------------------------------------------------------------------
    def _exchange(self, send: Optional[torch.Tensor], send_peer: Optional[int], recv_shape, dtype,
                  recv_peer: Optional[int]) -> Optional[torch.Tensor]:
        ops, buf = [], None
        if send is not None and send_peer is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), self._global(send_peer), self.group))
        if recv_peer is not None:
            buf = torch.empty(tuple(recv_shape), dtype=dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, buf, self._global(recv_peer), self.group))
        if not ops:
            return None
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                for req in dist.batch_isend_irecv(ops):
                    req.wait()
            if send is not None:
                send.record_stream(self.stream)
            torch.cuda.current_stream().wait_stream(self.stream)
        else:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return buf

    def send_forward_recv_backward(self, y: torch.Tensor, shape, dtype) -> Optional[torch.Tensor]:
        return self._exchange(y, self.next_rank, shape, dtype, self.next_rank)

    def send_backward_recv_forward(self, gx: Optional[torch.Tensor], shape, dtype) -> Optional[torch.Tensor]:
        return self._exchange(gx, self.prev_rank, shape, dtype, self.prev_rank)

    # ---- schedules ---------------------------------------------------------------------------------------------------
    def run_gpipe(self, stage_fn, microbatches: List[torch.Tensor], act_shape, dtype=torch.bfloat16) -> List[torch.Tensor]:
        """Forward-only GPipe schedule over `microbatches` (used on the first stage; later stages receive)."""
        outs = []
        for i in range(len(microbatches)):
            x = microbatches[i] if self.prev_rank is None else self.recv_forward(act_shape, dtype)
            y = stage_fn(x)
            if self.next_rank is not None:
                self.send_forward(y)
            outs.append(y)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)
        return outs

    def run_1f1b(self, stage: Callable[[torch.Tensor], torch.Tensor], n_micro: int,
                 inputs: Optional[Sequence[torch.Tensor]] = None, in_shape=None, out_shape=None,
                 loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None,
                 dtype=torch.bfloat16) -> List[torch.Tensor]:
        """One training step of ``n_micro`` microbatches through this stage: forward and backward, gradients accumulate
        in the stage's parameters (scale the loss by 1/n_micro in ``loss_fn`` for a mean).

        ``inputs``: the microbatches, on the first stage.  ``in_shape`` / ``out_shape``: shape of one microbatch of
        activations entering / leaving this stage (not needed at the two ends).  ``loss_fn(output, index)``: on the last
        stage.  Returns the last stage's losses (detached), an empty list elsewhere."""
        first, last = self.prev_rank is None, self.next_rank is None
        if first and (inputs is None or len(inputs) != n_micro):
            raise ValueError("run_1f1b: the first stage needs one input per microbatch")
        if last and loss_fn is None:
            raise ValueError("run_1f1b: the last stage needs loss_fn")
        warmup = min(self.world - self.rank - 1, n_micro)
        steady = n_micro - warmup
        held: List[tuple] = []          # (input, output) of forwards whose backward is still to come, oldest first
        losses: List[torch.Tensor] = []
        fwd_index = 0

        def forward(x: Optional[torch.Tensor]) -> torch.Tensor:
            nonlocal fwd_index
            if first:
                x = inputs[fwd_index]
            else:
                x = x.requires_grad_(True)
            y = stage(x)
            if last:
                y = loss_fn(y, fwd_index)
                losses.append(y.detach())
            fwd_index += 1
            held.append((x, y))
            return y

        def backward(g: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
            x, y = held.pop(0)
            if last:
                y.backward()
            else:
                y.backward(g)
            return None if first else x.grad

        for _ in range(warmup):
            y = forward(self.recv_forward(in_shape, dtype))
            self.send_forward(y.detach())
        x = self.recv_forward(in_shape, dtype) if steady > 0 else None
        for i in range(steady):
            y = forward(x)
            g = self.send_forward_recv_backward(None if last else y.detach(), out_shape, dtype)
            gx = backward(g)
            if i + 1 < steady:
                x = self.send_backward_recv_forward(gx, in_shape, dtype)
            elif gx is not None:
                self.send_backward(gx)
        for _ in range(warmup):
            gx = backward(self.recv_backward(out_shape, dtype))
            if gx is not None:
                self.send_backward(gx)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)
        return losses
