"""Hand-written collectives over the engine's symmetric heap (csrc/kernels/collectives.cu).

Tensors that peers touch must come from ``Engine.symmetric_tensor`` (same heap offset on every
rank).  ``algo``: ``"nvls"`` uses multimem through the switch (needs the multicast binding made by
``Engine.connect``), ``"p2p"`` plain loads/stores over NVLink, ``"auto"`` picks NVLS when it exists
and the dtype/op has an in-switch form.
"""
from __future__ import annotations

from typing import Optional

import torch

from .._native import C
from ..engine import Engine, dtype_name
from .gemm import count_launch

_NVLS_OK = {("f32", "sum"), ("bf16", "sum"), ("bf16", "max"), ("bf16", "min"), ("f16", "sum"), ("f16", "max"), ("f16", "min")}


def _algo(eng: Engine, algo: str, dt: str, op: str, nbytes: int, kind: str = "allreduce") -> str:
    if algo == "auto":
        ok = eng.has_nvls and (dt, op) in _NVLS_OK and nbytes % 16 == 0
        # reduce-scatter on up to four GPUs: from 64 MiB in total on, pulling the slice from each peer beats the
        # in-switch reduction (measured 595 against 495 GB/s at 256 MiB on four GPUs; equal on eight)
        if ok and kind == "reduce_scatter" and eng.world <= 4 and nbytes * eng.world >= (64 << 20):
            ok = False
        # Between two GPUs the switch has nothing to add: one peer load per element beats a multimem
        # round trip once the message is bandwidth-bound (measured cross-over near 8 MiB).
        if ok and eng.world == 2 and nbytes >= (8 << 20):
            ok = False
        return "nvls" if ok else "p2p"
    if algo == "nvls" and not eng.has_nvls:
        raise RuntimeError("NVLS requested but the heap is not bound to a multicast object")
    return algo


def _blocks(nbytes: int, blocks: Optional[int]) -> int:
    """CTAs for a collective that moves `nbytes` per rank: one CTA (512 threads, 4 x 16 bytes each in
    flight) per 32 KiB keeps small messages to a single pass, 128 CTAs saturate NVLink for large ones."""
    if blocks:
        return blocks
    return max(1, min(128, (nbytes + (32 << 10) - 1) // (32 << 10)))


def all_reduce(eng: Engine, inp: torch.Tensor, out: Optional[torch.Tensor] = None, op: str = "sum", algo: str = "auto",
               blocks: Optional[int] = None, threads: int = 512, lane: int = 0, stream=None) -> torch.Tensor:
    out = inp if out is None else out
    dt = dtype_name(inp.dtype)
    nbytes = inp.numel() * inp.element_size()
    a = _algo(eng, algo, dt, op, nbytes)
    s = (stream or torch.cuda.current_stream()).cuda_stream
    C.collective(eng.raw, "allreduce", a, dt, op, eng.heap_offset(inp), eng.heap_offset(out), inp.numel(), lane, 1.0, "",
                 _blocks(nbytes if (nbytes <= ((64 << 10) if a == "nvls" else (256 << 10)) and out is not inp) else nbytes // eng.world, blocks),
                 threads, s, 0, 0, 0)
    count_launch()
    return out


def reduce_scatter(eng: Engine, inp: torch.Tensor, out: torch.Tensor, op: str = "sum", scale: float = 1.0,
                   algo: str = "auto", blocks: Optional[int] = None, threads: int = 512, lane: int = 0, stream=None) -> torch.Tensor:
    """``out = cast(scale * reduce_over_ranks(inp[rank * n : (rank + 1) * n]))`` with n = out.numel().
    ``inp`` is symmetric; ``out`` may be any local tensor of inp's dtype or fp32 (fused cast)."""
    dt = dtype_name(inp.dtype)
    n = out.numel()
    if inp.numel() != n * eng.world:
        raise ValueError("reduce_scatter: inp must hold world * out.numel() elements")
    a = _algo(eng, algo, dt, op, n * inp.element_size(), "reduce_scatter")
    s = (stream or torch.cuda.current_stream()).cuda_stream
    sym_out = eng.is_symmetric(out)
    C.collective(eng.raw, "reduce_scatter", a, dt, op, eng.heap_offset(inp), eng.heap_offset(out) if sym_out else 0, n, lane,
                 float(scale), dtype_name(out.dtype), _blocks(n * inp.element_size(), blocks), threads, s, 0,
                 0 if sym_out else out.data_ptr(), 0)
    count_launch()
    return out


def reduce_scatter_adamw(eng: Engine, grads: torch.Tensor, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                         param_bf16: torch.Tensor, *, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                         step: int = 1, scale: float = 1.0, algo: str = "auto", blocks: Optional[int] = None, threads: int = 512,
                         lane: int = 0, stream=None) -> None:
    """Gradient-bucket reduce-scatter fused with the sharded AdamW step.  ``grads`` is the symmetric bf16
    bucket (world * n elements); ``master`` / ``exp_avg`` / ``exp_avg_sq`` are this rank's fp32 slices (n
    elements, n % 8 == 0); the updated parameters are written to ``param_bf16`` (bf16, n elements)."""
    n = master.numel()
    if grads.dtype != torch.bfloat16 or grads.numel() != n * eng.world or n % 8:
        raise ValueError("reduce_scatter_adamw: bf16 bucket of world * n elements with n % 8 == 0 expected")
    a = _algo(eng, algo, "bf16", "sum", n * 2)
    s = (stream or torch.cuda.current_stream()).cuda_stream
    C.reduce_scatter_adamw(eng.raw, a, eng.heap_offset(grads), n, lane, float(scale), master.data_ptr(), exp_avg.data_ptr(),
                           exp_avg_sq.data_ptr(), param_bf16.data_ptr(), lr, betas[0], betas[1], eps, weight_decay, step,
                           _blocks(n * 2, blocks), threads, s)
    count_launch()


def all_reduce_fp8(eng: Engine, q: torch.Tensor, s: torch.Tensor, out_q: Optional[torch.Tensor] = None,
                   out_s: Optional[torch.Tensor] = None, op: str = "sum", blocks: Optional[int] = None, threads: int = 512,
                   lane: int = 0, stream=None):
    """All-reduce of a block-scaled fp8 vector: ``q`` e4m3 bytes (symmetric, n elements, n % 128 == 0) with ``s`` fp32
    scales (symmetric, n / 128).  Every 128-value block is dequantised, accumulated in fp32 over the ranks and
    re-quantised with a fresh scale inside the transfer; the result lands in ``out_q`` / ``out_s`` on every rank
    (default: in place).  Returns ``(out_q, out_s)``."""
    out_q = q if out_q is None else out_q
    out_s = s if out_s is None else out_s
    n = q.numel()
    if q.element_size() != 1 or n % 128 or s.dtype != torch.float32 or s.numel() != n // 128:
        raise ValueError("all_reduce_fp8: q must be one-byte elements (n % 128 == 0) and s fp32 with n / 128 entries")
    st = (stream or torch.cuda.current_stream()).cuda_stream
    C.collective(eng.raw, "allreduce_fp8", "p2p", "e4m3", op, eng.heap_offset(q), eng.heap_offset(out_q), n, lane, 1.0, "",
                 _blocks(n // eng.world, blocks), threads, st, 0, 0, 0, eng.heap_offset(s), eng.heap_offset(out_s))
    count_launch()
    return out_q, out_s


def reduce_scatter_fp8(eng: Engine, q: torch.Tensor, s: torch.Tensor, out_q: torch.Tensor, out_s: torch.Tensor, op: str = "sum",
                       blocks: Optional[int] = None, threads: int = 512, lane: int = 0, stream=None):
    """Reduce-scatter of a block-scaled fp8 vector (see ``all_reduce_fp8``): rank r receives blocks
    [r * m, (r + 1) * m) with m = out_q.numel(); all four tensors are symmetric."""
    m = out_q.numel()
    if q.element_size() != 1 or m % 128 or q.numel() != m * eng.world or s.numel() != q.numel() // 128 or out_s.numel() != m // 128:
        raise ValueError("reduce_scatter_fp8: shapes do not match world * shard with 128-value blocks")
    st = (stream or torch.cuda.current_stream()).cuda_stream
    C.collective(eng.raw, "reduce_scatter_fp8", "p2p", "e4m3", op, eng.heap_offset(q), eng.heap_offset(out_q), m, lane, 1.0, "",
                 _blocks(m, blocks), threads, st, 0, 0, 0, eng.heap_offset(s), eng.heap_offset(out_s))
    count_launch()
    return out_q, out_s


def all_gather(eng: Engine, inp: torch.Tensor, out: torch.Tensor, algo: str = "auto", blocks: Optional[int] = None,
               threads: int = 512, lane: int = 0, stream=None) -> torch.Tensor:
    """``out`` (symmetric, world * inp.numel()) receives every rank's ``inp`` at its rank's slot."""
    nbytes = inp.numel() * inp.element_size()
    a = "nvls" if (algo in ("auto", "nvls") and eng.has_nvls and nbytes % 16 == 0 and inp.data_ptr() % 16 == 0) else "p2p"
    # measured on 4 and 8 GPUs: from a few MiB per rank on, plain posted stores to each peer fill the ports
    # better than the multicast store (which also comes back to the sender)
    if algo == "auto" and nbytes >= (4 << 20):
        a = "p2p"
    s = (stream or torch.cuda.current_stream()).cuda_stream
    C.collective(eng.raw, "allgather", a, "u8", "sum", 0, eng.heap_offset(out), nbytes, lane, 1.0, "",
                 _blocks(nbytes, blocks), threads, s, inp.data_ptr(), 0, 0)
    count_launch()
    return out


def all_to_all(eng: Engine, inp: torch.Tensor, out: torch.Tensor, blocks: Optional[int] = None, threads: int = 512,
               lane: int = 0, stream=None) -> torch.Tensor:
    """Block d of ``inp`` goes to rank d; ``out`` (symmetric) receives block s from rank s."""
    nbytes = inp.numel() * inp.element_size() // eng.world
    s = (stream or torch.cuda.current_stream()).cuda_stream
    C.collective(eng.raw, "alltoall", "p2p", "u8", "sum", 0, eng.heap_offset(out), nbytes, lane, 1.0, "",
                 _blocks(nbytes * eng.world, blocks), threads, s, inp.data_ptr(), 0, 0)
    count_launch()
    return out


# ---------------------------------------------------------------------------------------------
# Rooted and point-to-point collectives: library programs of pccl_b200.lang run by the engine (the
# interpreter kernel on a CUDA engine, the host executor on a CPU engine).  Data travels through the
# engine's workspace, so the tensors may be ordinary ones.  Every rank makes every call.
# ---------------------------------------------------------------------------------------------
def _library_op(eng: Engine, algo: str, **kw) -> str:
    """Registers ``lang.build(algo, world, **kw)`` with the engine on first use and returns its name."""
    from ..lang import DeviceType, build
    name = "lib." + algo + "".join(f".{k}={v}" for k, v in sorted(kw.items()))
    done = eng.__dict__.setdefault("_library_ops", set())
    if name not in done:
        dev = DeviceType.CUDA if eng.device == "cuda" else DeviceType.CPU
        eng.regOp(name, build(algo, eng.world, device_type=dev, **kw))
        done.add(name)
    return name


def _run_library_op(eng: Engine, name: str, inp: torch.Tensor, out: torch.Tensor, width: int, lane: int, stream) -> None:
    eng.exeOp(name, inp, out, width=width, lane=lane, stream=stream)
    if inp.is_cuda:
        count_launch()


def broadcast(eng: Engine, t: torch.Tensor, root: int = 0, out: Optional[torch.Tensor] = None, algo: str = "direct",
              channels: int = 1, width: int = 1, lane: int = 0, stream=None) -> torch.Tensor:
    """``t`` of rank ``root`` reaches ``out`` (default: ``t`` itself, in place) on every rank.  ``algo``: ``"direct"``
    (the root stores to every peer: shortest, right for small messages), ``"tree"`` (binomial relay), ``"scatter_allgather"``
    (the root's port carries the vector once: right for long vectors), or ``"auto"``: the cheapest of the three by the
    cost model on an NVSwitch of this world's size."""
    out = t if out is None else out
    if algo == "auto":
        from ..synth import Topology, choose
        ranked = choose("broadcast", Topology.nvswitch(eng.world), t.numel() * t.element_size(), channels=channels, root=root)
        algo = {"broadcast": "direct", "broadcast[tree]": "tree"}.get(ranked[0][0], "scatter_allgather") if ranked else "direct"
    if algo == "scatter_allgather":
        name = _library_op(eng, "scatter_allgather_broadcast", root=root, channels=channels)
    elif algo in ("direct", "tree"):
        name = _library_op(eng, "broadcast", root=root, tree=(algo == "tree"), channels=channels)
    else:
        raise ValueError(f"broadcast: unknown algo {algo!r}")
    _run_library_op(eng, name, t, out, width, lane, stream)
    return out


def reduce(eng: Engine, inp: torch.Tensor, out: torch.Tensor, root: int = 0, op: str = "sum", algo: str = "tree",
           channels: int = 1, width: int = 1, lane: int = 0, stream=None) -> torch.Tensor:
    """The reduction of every rank's ``inp`` lands in ``out`` of rank ``root``; the other ranks' ``out`` is not written.
    ``algo``: ``"tree"`` (binomial, log2(world) hops of the whole vector: small messages), ``"pieces"`` (piece d is reduced
    on rank d and handed to the root: long vectors), or ``"auto"`` (the cheaper of the two by the cost model)."""
    if algo == "auto":
        from ..synth import Topology, choose
        ranked = choose("reduce", Topology.nvswitch(eng.world), inp.numel() * inp.element_size(), channels=channels, root=root)
        algo = "pieces" if ranked and ranked[0][0] == "reduce_scatter_gather_reduce" else "tree"
    if algo not in ("tree", "pieces"):
        raise ValueError(f"reduce: unknown algo {algo!r}")
    name = _library_op(eng, "reduce" if algo == "tree" else "reduce_scatter_gather_reduce", root=root, redop=op, channels=channels)
    _run_library_op(eng, name, inp, out, width, lane, stream)
    return out


def scatter(eng: Engine, inp: torch.Tensor, out: torch.Tensor, root: int = 0, channels: int = 1, width: int = 1,
            lane: int = 0, stream=None) -> torch.Tensor:
    """Block d of ``root``'s ``inp`` (world * out.numel() elements; only read on the root) becomes rank d's ``out``."""
    if inp.numel() != out.numel() * eng.world:
        raise ValueError("scatter: inp must hold world blocks of out's size (on every rank, although only the root's is read)")
    _run_library_op(eng, _library_op(eng, "scatter", root=root, channels=channels), inp, out, width, lane, stream)
    return out


def gather(eng: Engine, inp: torch.Tensor, out: torch.Tensor, root: int = 0, channels: int = 1, width: int = 1,
           lane: int = 0, stream=None) -> torch.Tensor:
    """Rank s's ``inp`` becomes block s of ``root``'s ``out`` (world * inp.numel() elements; only written on the root)."""
    if out.numel() != inp.numel() * eng.world:
        raise ValueError("gather: out must hold world blocks of inp's size (on every rank, although only the root's is written)")
    _run_library_op(eng, _library_op(eng, "gather", root=root, channels=channels), inp, out, width, lane, stream)
    return out


def send_recv(eng: Engine, inp: torch.Tensor, out: torch.Tensor, src: int, dst: int, channels: int = 1, width: int = 1,
              lane: int = 0, stream=None) -> torch.Tensor:
    """``inp`` of rank ``src`` becomes ``out`` of rank ``dst``.  All ranks call it (the others run an empty program),
    so it can sit in a sequence of collectives without a separate group."""
    _run_library_op(eng, _library_op(eng, "send_recv", src=src, dst=dst, channels=channels), inp, out, width, lane, stream)
    return out


def ring_shift(eng: Engine, inp: torch.Tensor, out: torch.Tensor, shift: int = 1, channels: int = 1, width: int = 1,
               lane: int = 0, stream=None) -> torch.Tensor:
    """``inp`` of rank r becomes ``out`` of rank (r + shift) mod world: one hop of a ring (the KV rotation of ring
    attention, when a block's attention is computed between hops)."""
    _run_library_op(eng, _library_op(eng, "ring_shift", shift=shift % eng.world, channels=channels), inp, out, width, lane, stream)
    return out
