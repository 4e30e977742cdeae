"""The two headline measurements of this library, in a form that rides along with ``bench.py`` at N >= 2:

* ``collectives``: all-reduce, reduce-scatter and all-gather (bf16) at 1 MB, 16 MB, 256 MB and 1 GB with
  ``algo="auto"`` (what a caller gets without choosing) next to NCCL on the same GPUs; bus GB/s and
  microseconds, median of five trains of back-to-back calls, device-timed, maximum over the ranks.
* ``fused_tp``: the tensor-parallel MLP shapes (8192 tokens x 8192, d_ff 28672 / TP): all-gather -> GEMM
  and GEMM -> reduce-scatter as ONE kernel each, next to NCCL + cuBLAS run back to back and next to a
  stream-overlapped NCCL + cuBLAS arm (the collective in pieces on a side stream, one matmul per piece),
  with the largest element-wise difference against the sequential baseline's result.

(The reference library publishes no number and has no benchmark; NCCL and cuBLAS on the same box are the bar.)
"""
from __future__ import annotations

import json
import os
from typing import Optional, Dict, List

import torch
import torch.distributed as dist

from .bench_collectives import bench_size
from .engine import Engine
from .ops import check_status
from .ops.fused_tp import AllGatherGemm, GemmReduceScatter
from .ops.gemm import gemm
from .utils import L2Flusher

SIZES = (1 << 20, 16 << 20, 256 << 20, 1 << 30)


def collectives_block(eng: Engine, sizes=SIZES, trains: int = 5) -> List[Dict]:
    rows = []
    for kind in ("allreduce", "reduce_scatter", "allgather"):
        for nbytes in sizes:
            iters = 100 if nbytes <= (1 << 20) else (30 if nbytes <= (16 << 20) else (10 if nbytes <= (256 << 20) else 5))
            r = bench_size(eng, kind, torch.bfloat16, nbytes, ["auto", "nccl"], iters=iters, trains=trains)
            r["speedup_vs_nccl"] = r["nccl"]["us"] / r["auto"]["us"]
            rows.append(r)
    return rows


def _time_us(fn, iters: int, warmup: int, flush, trains: int = 3) -> float:
    """Microseconds per call: every call is preceded by an L2 flush and a barrier and timed by its own pair of CUDA
    events; mean over `iters` calls, maximum over the ranks, median over `trains` repetitions."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    meds = []
    for _ in range(trains):
        total = 0.0
        for _i in range(iters):
            flush()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            total += a.elapsed_time(b)
        t = torch.tensor([total / iters], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        meds.append(float(t.item()) * 1e3)
    meds.sort()
    return meds[len(meds) // 2]


def _peaks() -> Dict:
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def fused_tp_block(eng: Engine, tokens: int = 8192, d_model: int = 8192, d_ff: int = 28672, iters: int = 8, warmup: int = 3,
                   n_copy: Optional[int] = None, pieces: int = 4, link_gbs: float = 770.0) -> List[Dict]:
    world, rank = eng.world, eng.rank
    pk = _peaks()
    peak_tflops = float(pk.get("bf16_tflops", 1590.0))
    peak_src = "measured" if "bf16_tflops" in pk else "fallback"
    n1 = d_ff // world // 8 * 8
    m_local = tokens // world
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x_local = torch.randn(m_local, d_model, generator=g, device="cuda").bfloat16()
    w1 = (torch.randn(n1, d_model, generator=g, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(d_model, n1, generator=g, device="cuda") * 0.02).bfloat16()
    flush = L2Flusher()
    side = torch.cuda.Stream()
    rows = []
    mark = eng.symmetric_mark()

    # ---- all-gather -> GEMM ------------------------------------------------------------------------------
    ag = AllGatherGemm(eng, tokens, d_model, n_copy=n_copy)
    ag.x_local.copy_(x_local)
    y = torch.empty(tokens, n1, dtype=torch.bfloat16, device="cuda")
    xg = torch.empty(tokens, d_model, dtype=torch.bfloat16, device="cuda")
    y_ref = torch.empty_like(y)

    def seq_ag_gemm():
        dist.all_gather_into_tensor(xg, x_local)
        torch.matmul(xg, w1.t(), out=y_ref)

    mp = m_local // pieces
    xg_p = [torch.empty(world * mp, d_model, dtype=torch.bfloat16, device="cuda") for _ in range(pieces)]
    y_p = [torch.empty(world * mp, n1, dtype=torch.bfloat16, device="cuda") for _ in range(pieces)]
    ev = [torch.cuda.Event() for _ in range(pieces)]

    def overlapped_ag_gemm():
        # piece i of every rank's rows is gathered on the side stream while piece i-1 is multiplied; the output
        # rows come out piece-major (a real layer would index them accordingly), the work is the same
        cur = torch.cuda.current_stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for i in range(pieces):
                dist.all_gather_into_tensor(xg_p[i], x_local[i * mp:(i + 1) * mp])
                ev[i].record(side)
        for i in range(pieces):
            cur.wait_event(ev[i])
            torch.matmul(xg_p[i], w1.t(), out=y_p[i])

    fused = _time_us(lambda: ag(w1, out=y), iters, warmup, flush)
    check_status("headline ag_gemm")
    seq = _time_us(seq_ag_gemm, iters, warmup, flush)
    ovl = _time_us(overlapped_ag_gemm, iters, warmup, flush)
    own = _time_us(lambda: gemm(xg, w1, out=y_ref), iters, warmup, flush, trains=1)
    seq_ag_gemm()
    ag(w1, out=y)
    torch.cuda.synchronize()
    err = (y.float() - y_ref.float()).abs().max().item()
    flops = 2.0 * tokens * n1 * d_model
    comm_bytes = (world - 1) * m_local * d_model * 2
    roof = max(flops / (peak_tflops * 1e12), comm_bytes / (link_gbs * 1e9)) * 1e6
    rows.append({"op": "allgather_gemm", "tp": world, "M": tokens, "N": n1, "K": d_model, "fused_us": fused,
                 "nccl_cublas_sequential_us": seq, "nccl_cublas_overlapped_us": ovl, "overlap_pieces": pieces, "own_gemm_alone_us": own,
                 "speedup_vs_sequential": seq / fused, "speedup_vs_overlapped": ovl / fused, "roofline_us": roof,
                 "fraction_of_roofline": roof / fused, "roofline_peaks": f"{peak_tflops:.0f} TFLOP/s ({peak_src} cuBLAS burst), {link_gbs:.0f} GB/s link",
                 "max_abs_diff_vs_baseline": err})
    del ag, xg_p, y_p

    # ---- GEMM -> reduce-scatter --------------------------------------------------------------------------
    rs = GemmReduceScatter(eng, tokens, d_model)
    h = (torch.randn(tokens, n1, generator=g, device="cuda") * 0.5).bfloat16()
    z = torch.empty(m_local, d_model, dtype=torch.bfloat16, device="cuda")
    part = torch.empty(tokens, d_model, dtype=torch.bfloat16, device="cuda")
    z_ref = torch.empty_like(z)

    def seq_gemm_rs():
        torch.matmul(h, w2.t(), out=part)
        dist.reduce_scatter_tensor(z_ref, part)

    dc = d_model // pieces
    part_p = [torch.empty(tokens, dc, dtype=torch.bfloat16, device="cuda") for _ in range(pieces)]
    z_p = [torch.empty(m_local, dc, dtype=torch.bfloat16, device="cuda") for _ in range(pieces)]
    w2_p = [w2[i * dc:(i + 1) * dc] for i in range(pieces)]
    ev2 = [torch.cuda.Event() for _ in range(pieces)]

    def overlapped_gemm_rs():
        # a block of output columns is multiplied while the previous block is reduce-scattered on the side stream
        cur = torch.cuda.current_stream()
        for i in range(pieces):
            torch.matmul(h, w2_p[i].t(), out=part_p[i])
            ev2[i].record(cur)
            side.wait_event(ev2[i])
            with torch.cuda.stream(side):
                dist.reduce_scatter_tensor(z_p[i], part_p[i])
        cur.wait_stream(side)

    fused = _time_us(lambda: rs(h, w2, out=z), iters, warmup, flush)
    check_status("headline gemm_rs")
    seq = _time_us(seq_gemm_rs, iters, warmup, flush)
    ovl = _time_us(overlapped_gemm_rs, iters, warmup, flush)
    own = _time_us(lambda: gemm(h, w2, out=part), iters, warmup, flush, trains=1)
    seq_gemm_rs()
    rs(h, w2, out=z)
    torch.cuda.synchronize()
    err = (z.float() - z_ref.float()).abs().max().item()
    flops = 2.0 * tokens * d_model * n1
    roof = max(flops / (peak_tflops * 1e12), comm_bytes / (link_gbs * 1e9)) * 1e6
    rows.append({"op": "gemm_reduce_scatter", "tp": world, "M": tokens, "N": d_model, "K": n1, "fused_us": fused,
                 "nccl_cublas_sequential_us": seq, "nccl_cublas_overlapped_us": ovl, "overlap_pieces": pieces, "own_gemm_alone_us": own,
                 "speedup_vs_sequential": seq / fused, "speedup_vs_overlapped": ovl / fused, "roofline_us": roof,
                 "fraction_of_roofline": roof / fused, "roofline_peaks": f"{peak_tflops:.0f} TFLOP/s ({peak_src} cuBLAS burst), {link_gbs:.0f} GB/s link",
                 "max_abs_diff_vs_baseline": err})
    del rs
    eng.symmetric_reset(mark)
    return rows


def headline(eng: Engine) -> Dict:
    """Both blocks; a failure in one is reported in its place and does not take the other (or the caller) down."""
    out: Dict = {"metric": "bus GB/s vs message size against NCCL; fused TP all-gather+GEMM / GEMM+reduce-scatter microseconds "
                           "against NCCL+cuBLAS", "timing": "CUDA events, max over ranks; collectives: median of 5 trains over a buffer "
                           "pool larger than L2; fused TP: L2 flushed before every call, median of 3 repetitions"}
    for name, fn in (("collectives", collectives_block), ("fused_tp", fused_tp_block)):
        try:
            out[name] = fn(eng)
        except Exception as e:  # noqa: BLE001 - the training number must still be printed
            out[name] = {"error": f"{type(e).__name__}: {e}"}
    return out
