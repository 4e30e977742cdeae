"""Data parallelism with bucketed gradient reduce-scatter overlapped with backward.

Gradients live in flat bf16 buckets (25 MB by default) inside the symmetric heap.  The moment the
last gradient of a bucket has been written (the weight-gradient GEMMs write there directly), ONE
kernel is queued on a high-priority side stream: each rank reduces its 1/world slice of the bucket
(multimem.ld_reduce through the switch, or loads from every peer over NVLink), multiplies by
1/world and applies AdamW to its fp32 master slice -- reduction, scaling, cast and optimizer in one
pass -- and writes the new bf16 parameters, which the bucket's all-gather kernel then pushes to
every rank (ZeRO-1).  The kernels run as short, wide bursts (64 to 128 CTAs) that slip in between
two GEMM kernels of backward.  With a world of one the same kernels run (the reduce-scatter
degenerates to the scale/cast/update pass), so single-GPU and multi-GPU steps share one code path.
``fuse_optimizer=False`` keeps the reduce-scatter (with scale and fp32 cast) and the optimizer apart.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..engine import Engine
from ..ops import collectives as coll
from ..ops.elementwise import adamw_step


class _Bucket:
    def __init__(self, index: int):
        self.index = index
        self.params: List[nn.Parameter] = []
        self.offsets: List[int] = []
        self.numel = 0            # padded
        self.pending = 0
        self.grads: torch.Tensor = None      # bf16 view in the symmetric heap
        self.values: torch.Tensor = None     # bf16 view of the flat parameters
        self.grad_shard: torch.Tensor = None  # fp32, numel / world
        self.master: torch.Tensor = None
        self.exp_avg: torch.Tensor = None
        self.exp_avg_sq: torch.Tensor = None
        self.decay = True


class ShardedDataParallel:
    """Wraps a model for data-parallel training over an ``Engine`` (one process per GPU).

    ``train_step(inputs, targets)`` runs forward, backward (with overlapped gradient reduction) and
    the sharded optimizer step, and returns the loss tensor.
    """

    def __init__(self, model: nn.Module, engine: Optional[Engine] = None, *, lr: float = 3e-4, betas=(0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.1, bucket_mb: float = 25.0, heap_bytes: int = 0,
                 comm_blocks: Optional[int] = None, algo: str = "auto", group=None, fuse_optimizer: bool = True,
                 schedule: str = "auto", topology=None):
        """``schedule``: "auto" asks the MILP synthesiser (pccl_b200.synth) for the reduce-scatter schedule of one
        bucket on ``topology`` (default: this world behind an NVSwitch at the measured port bandwidth).  When the
        optimum is the one-step direct exchange -- it is on NVSwitch -- the hand-written kernel that fuses that
        exchange with scaling and AdamW runs it; a multi-step optimum (a ring or a partial mesh) is registered
        with the engine and executed by the interpreter kernel, followed by the unfused optimizer.  "fused" and
        "interpreter" force one or the other."""
        self.model = model
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.algo = algo
        # fused: the bucket's reduce-scatter kernel also performs the AdamW update of this rank's slice and
        # the parameter all-gather follows at once, all while backward is still running
        self.fuse_optimizer = fuse_optimizer
        params = []
        seen = set()
        for p in model.parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                params.append(p)
        total = sum(p.numel() for p in params)
        if engine is None:
            need = 2 * 2 * (total + 64 * len(params)) + (64 << 20)
            engine = Engine(0, 1)
            os.environ.setdefault("PCCL_WORKSPACE_MB", "64")
            engine.initEngine("cuda", max(heap_bytes, need + (512 << 20)))
        self.engine = engine
        self.world, self.rank = engine.world, engine.rank
        # Communication kernels run as short, wide bursts on a high-priority stream: they slip in at the
        # boundary between two GEMM kernels and delay the next one by their own (tens of microseconds)
        # duration.  A narrow long-running kernel would instead hold a few SMs for the whole GEMM and make
        # the persistent GEMM's last CTAs start a full wave late.
        self.comm_blocks = comm_blocks if comm_blocks else (128 if engine.world == 1 else 64)
        self.comm_stream = torch.cuda.Stream(priority=-1)
        self.step_count = 0
        self._plan_schedule(int(bucket_mb * (1 << 20)), schedule, topology)
        self._build_buckets(params, int(bucket_mb * (1 << 20)) // 2)
        self._ready_events: Dict[int, torch.cuda.Event] = {}
        # opt-in per-bucket timing (CUDA events on both streams); see timed_step()
        self._timing = False
        self._marks: Dict[str, object] = {}

    # ------------------------------------------------------------------------------------------
    def _plan_schedule(self, bucket_bytes: int, schedule: str, topology) -> None:
        self.schedule = {"source": "none", "mode": "fused"}
        self.interpreted = False
        if self.world == 1:
            return
        if schedule not in ("auto", "fused", "interpreter"):
            raise ValueError("ShardedDataParallel: schedule must be auto, fused or interpreter")
        from ..synth import Topology, synthesize
        topo = topology or Topology.nvswitch(self.world)
        # deterministic, so every rank arrives at the same schedule without exchanging it
        res = synthesize("reduce_scatter", topo, bucket_bytes, chunks=1, time_limit=10.0)
        direct = res.steps_used == 1 and len(res.sends[0]) == self.world * (self.world - 1)
        self.interpreted = schedule == "interpreter" or (schedule == "auto" and not direct)
        self.schedule = {"source": "milp", "topology": topo.name, "steps": res.steps_used, "direct": direct,
                         "objective_us": res.objective_seconds * 1e6, "lower_bound_us": res.lower_bound_seconds * 1e6,
                         "mode": "interpreter" if self.interpreted else "fused"}
        if self.interpreted:
            self.engine.regOp("dp_grad_reduce_scatter", res.ir)
            self.fuse_optimizer = False

    # ------------------------------------------------------------------------------------------
    def _build_buckets(self, params: List[nn.Parameter], cap_elems: int) -> None:
        world = self.world
        align = 8 * world                      # every rank's slice starts on a 16-byte boundary
        self.buckets: List[_Bucket] = []
        # Matrices (weight decay) and vectors (no decay) go to separate buckets, so that one fused
        # AdamW launch per bucket has one decay setting.
        open_buckets: Dict[bool, _Bucket] = {}
        for p in reversed(params):             # gradients arrive roughly in reverse parameter order
            decay = p.dim() >= 2
            n = (p.numel() + 7) // 8 * 8
            cur = open_buckets.get(decay)
            if cur is None or (cur.params and cur.numel + n > cap_elems):
                cur = _Bucket(len(self.buckets))
                cur.decay = decay
                self.buckets.append(cur)
                open_buckets[decay] = cur
            cur.params.append(p)
            cur.offsets.append(cur.numel)
            cur.numel += n
        eng = self.engine
        for b in self.buckets:
            b.numel = (b.numel + align - 1) // align * align
        total = sum(b.numel for b in self.buckets)
        flat_g = eng.symmetric_tensor((total,), torch.bfloat16, align=256)
        flat_p = eng.symmetric_tensor((total,), torch.bfloat16, align=256)
        flat_g.zero_()
        flat_p.zero_()
        self.flat_grads, self.flat_params = flat_g, flat_p
        base = 0
        for b in self.buckets:
            b.grads = flat_g[base:base + b.numel]
            b.values = flat_p[base:base + b.numel]
            shard = b.numel // world
            for p, off in zip(b.params, b.offsets):
                view = b.values[off:off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = b.grads[off:off + p.numel()].view(p.shape)
                p._pccl_written = False
                p._pccl_seen = 0
                if not hasattr(p, "_pccl_uses"):
                    p._pccl_uses = 1           # a model sets 2 on a weight it uses twice (tied embeddings)
                p._pccl_ready = self._make_ready(b, p)
                if not getattr(p, "_pccl_hooked", False):
                    p.register_post_accumulate_grad_hook(self._autograd_hook)
                    p._pccl_hooked = True
            lo = self.rank * shard
            b.master = b.values[lo:lo + shard].float().clone()
            b.exp_avg = torch.zeros_like(b.master)
            b.exp_avg_sq = torch.zeros_like(b.master)
            b.grad_shard = torch.empty_like(b.master)
            if self.interpreted:
                b.rs_out = eng.symmetric_tensor((shard,), torch.bfloat16, align=256)
            base += b.numel
        torch.cuda.synchronize()

    def _make_ready(self, bucket: _Bucket, p: torch.Tensor):
        def ready():
            p._pccl_seen += 1
            if p._pccl_seen < p._pccl_uses:
                return
            bucket.pending -= 1
            if bucket.pending == 0:
                self._launch_reduce(bucket)
        return ready

    @staticmethod
    def _autograd_hook(p: torch.Tensor) -> None:
        """Parameters whose gradient autograd produced (norms, biases without a fused path)."""
        g = p.grad
        if g is None:
            return
        if p._pccl_written:
            p.main_grad.add_(g.to(p.main_grad.dtype))
        else:
            p.main_grad.copy_(g)
        p.grad = None
        p._pccl_written = True
        p._pccl_ready()

    def _launch_reduce(self, b: _Bucket) -> None:
        ev = torch.cuda.Event(enable_timing=self._timing)
        ev.record(torch.cuda.current_stream())
        self.comm_stream.wait_event(ev)
        if self._timing:
            marks = {"ready": ev, "start": torch.cuda.Event(enable_timing=True), "reduced": torch.cuda.Event(enable_timing=True),
                     "done": torch.cuda.Event(enable_timing=True)}
            self._marks[b.index] = marks
            marks["start"].record(self.comm_stream)
            try:
                self._launch_reduce_inner(b, marks["reduced"])
            finally:
                marks["done"].record(self.comm_stream)
            return
        self._launch_reduce_inner(b, None)

    def _launch_reduce_inner(self, b: _Bucket, reduced_mark) -> None:
        if self.interpreted:
            # the synthesised multi-step schedule, run by the interpreter kernel; scale and cast follow
            self.engine.exeOp("dp_grad_reduce_scatter", b.grads, b.rs_out, width=4, lane=1, stream=self.comm_stream)
            with torch.cuda.stream(self.comm_stream):
                torch.mul(b.rs_out, 1.0 / self.world, out=b.grad_shard)
            return
        if not self.fuse_optimizer:
            coll.reduce_scatter(self.engine, b.grads, b.grad_shard, scale=1.0 / self.world, algo=self.algo,
                                blocks=self.comm_blocks, lane=1, stream=self.comm_stream)
            return
        shard = b.numel // self.world
        dst = b.values[self.rank * shard:(self.rank + 1) * shard]
        coll.reduce_scatter_adamw(self.engine, b.grads, b.master, b.exp_avg, b.exp_avg_sq, dst, lr=self.lr, betas=self.betas,
                                  eps=self.eps, weight_decay=self.weight_decay if b.decay else 0.0, step=self.step_count,
                                  scale=1.0 / self.world, algo=self.algo, blocks=self.comm_blocks, lane=1, stream=self.comm_stream)
        if reduced_mark is not None:
            reduced_mark.record(self.comm_stream)
        if self.world > 1:
            # every gradient of the bucket exists, so backward no longer reads these parameters on any rank
            # that has reached this point; the all-gather's entry barrier waits for the others
            coll.all_gather(self.engine, dst, b.values, algo=self.algo, blocks=self.comm_blocks, lane=2, stream=self.comm_stream)

    # ------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        if self.fuse_optimizer:
            self.step_count += 1          # the optimizer runs inside backward: this is the step being taken
        for b in self.buckets:
            b.pending = len(b.params)
            for p in b.params:
                p._pccl_written = False
                p._pccl_seen = 0
                p.grad = None

    def optimizer_step(self) -> None:
        """Sharded AdamW + parameter all-gather, on the communication stream behind the reductions.  In
        fused mode both already ran bucket by bucket during backward; this only joins the streams."""
        if self.fuse_optimizer:
            for b in self.buckets:
                if b.pending != 0:
                    raise RuntimeError(f"bucket {b.index}: {b.pending} gradient(s) never arrived "
                                       "(a parameter took no part in the loss)")
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            return
        self.step_count += 1
        with torch.cuda.stream(self.comm_stream):
            for b in self.buckets:
                if b.pending != 0:
                    raise RuntimeError(f"bucket {b.index}: {b.pending} gradient(s) never arrived "
                                       "(a parameter took no part in the loss)")
                shard = b.numel // self.world
                lo = self.rank * shard
                dst = b.values[lo:lo + shard]
                adamw_step(b.master, b.exp_avg, b.exp_avg_sq, b.grad_shard, dst, lr=self.lr, betas=self.betas,
                           eps=self.eps, weight_decay=self.weight_decay if b.decay else 0.0,
                           step=self.step_count, stream=self.comm_stream)
                if self.world > 1:
                    coll.all_gather(self.engine, dst, b.values, algo=self.algo, blocks=self.comm_blocks, lane=2,
                                    stream=self.comm_stream)
        torch.cuda.current_stream().wait_stream(self.comm_stream)

    def train_step(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.zero_grad()
        loss = self.model(inputs, targets)
        loss.backward()
        self.optimizer_step()
        return loss.detach()

    def timed_step(self, inputs: torch.Tensor, targets: torch.Tensor) -> Dict[str, object]:
        """One training step with CUDA events around forward, backward and every bucket's kernels on the communication
        stream.  Returns, in milliseconds from the start of the step: ``forward_end``, ``backward_end``, ``step_end`` (after
        the join with the communication stream) and per bucket ``ready`` (its last gradient was written), ``start``,
        ``reduced`` (reduce-scatter + AdamW done; equals ``start`` where the mode does not fuse them) and ``done``
        (parameter all-gather done).  ``exposed_ms`` is what the step waits for after backward has ended;
        ``comm_busy_ms`` is the time the communication stream spent in these kernels."""
        if not self.fuse_optimizer or self.interpreted:
            raise RuntimeError("timed_step covers the fused reduce-scatter + AdamW + all-gather mode")
        ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
        t0, t_fwd, t_bwd, t_end = ev(), ev(), ev(), ev()
        self._timing, self._marks = True, {}
        try:
            cur = torch.cuda.current_stream()
            t0.record(cur)
            self.zero_grad()
            loss = self.model(inputs, targets)
            t_fwd.record(cur)
            loss.backward()
            t_bwd.record(cur)
            self.optimizer_step()
            t_end.record(cur)
            torch.cuda.synchronize()
        finally:
            self._timing = False
        at = lambda e: t0.elapsed_time(e)  # noqa: E731
        rows = []
        for b in self.buckets:
            m = self._marks.get(b.index)
            if m is None:
                continue
            rows.append({"bucket": b.index, "mbytes": b.numel * 2 / 2**20, "ready": at(m["ready"]), "start": at(m["start"]),
                         "reduced": at(m["reduced"]), "done": at(m["done"])})
        rows.sort(key=lambda r: r["ready"])
        self._marks = {}
        busy = sum(r["done"] - r["start"] for r in rows)
        return {"loss": float(loss.detach()), "forward_end": at(t_fwd), "backward_end": at(t_bwd), "step_end": at(t_end),
                "exposed_ms": at(t_end) - at(t_bwd), "comm_busy_ms": busy,
                "reduce_ms": sum(r["reduced"] - r["start"] for r in rows), "allgather_ms": sum(r["done"] - r["reduced"] for r in rows),
                "queue_delay_ms_max": max((r["start"] - r["ready"] for r in rows), default=0.0), "buckets": rows}

    def gather_full_state(self) -> Dict[str, torch.Tensor]:
        """Checkpoint helper: this rank's optimizer shards plus the (replicated) bf16 parameters."""
        return {"step": torch.tensor(self.step_count), "flat_params": self.flat_params.clone(),
                **{f"master.{b.index}": b.master.clone() for b in self.buckets},
                **{f"exp_avg.{b.index}": b.exp_avg.clone() for b in self.buckets},
                **{f"exp_avg_sq.{b.index}": b.exp_avg_sq.clone() for b in self.buckets}}

    def load_full_state(self, state: Dict[str, torch.Tensor]) -> None:
        self.step_count = int(state["step"])
        self.flat_params.copy_(state["flat_params"])
        for b in self.buckets:
            b.master.copy_(state[f"master.{b.index}"])
            b.exp_avg.copy_(state[f"exp_avg.{b.index}"])
            b.exp_avg_sq.copy_(state[f"exp_avg_sq.{b.index}"])
