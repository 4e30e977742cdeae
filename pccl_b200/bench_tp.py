"""Tensor-parallel MLP micro-benchmark: the fused all-gather->GEMM and GEMM->reduce-scatter kernels
against NCCL + torch.matmul (cuBLAS) on the same GPUs and shapes.

Shapes (bf16): X is [tokens, d_model] sharded over ranks by rows; W1 is [d_ff / TP, d_model],
W2 is [d_model, d_ff / TP].  Defaults: tokens 8192, d_model 8192, d_ff 28672.  Device-timed with
CUDA events, max over ranks; every iteration is preceded by an L2 flush.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m pccl_b200.bench_tp --out tp.json
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Optional

import torch
import torch.distributed as dist

from .engine import Engine
from .ops import check_status
from .ops.fused_tp import AllGatherGemm, AllGatherGemmFp8, GemmReduceScatter, GemmReduceScatterFp8, default_copy_ctas
from .ops.gemm import gemm, gemm_fp8, quant_blocks, quant_rows
from .utils import L2Flusher


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
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
    return float(t.item()) * 1e3      # microseconds


def run(eng: Engine, tokens: int, d_model: int, d_ff: int, iters: int = 20, warmup: int = 5, n_copy: Optional[int] = None,
        peak_tflops: float = 1701.7, link_gbs: float = 770.0, fp8: bool = True):
    world, rank = eng.world, eng.rank
    n1 = d_ff // world
    m_local = tokens // world
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x_local = torch.randn(m_local, d_model, generator=g, device="cuda").bfloat16()
    w1 = (torch.randn(n1, d_model, generator=g, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(d_model, n1, generator=g, device="cuda") * 0.02).bfloat16()
    flush = L2Flusher()
    rows = []

    # ---- all-gather -> GEMM -------------------------------------------------------------------
    ag = AllGatherGemm(eng, tokens, d_model, n_copy=n_copy)
    ag.x_local.copy_(x_local)
    y = torch.empty(tokens, n1, dtype=torch.bfloat16, device="cuda")
    xg = torch.empty(tokens, d_model, dtype=torch.bfloat16, device="cuda")
    y_ref = torch.empty_like(y)

    def nccl_ag_gemm():
        dist.all_gather_into_tensor(xg, x_local)
        torch.matmul(xg, w1.t(), out=y_ref)

    fused = _time(lambda: ag(w1, out=y), iters, warmup, flush)
    check_status("ag_gemm")
    base = _time(nccl_ag_gemm, iters, warmup, flush)
    gemm_cublas = _time(lambda: torch.matmul(xg, w1.t(), out=y_ref), iters, warmup, flush)
    gemm_ours = _time(lambda: gemm(xg, w1, out=y_ref), iters, warmup, flush)
    comm_only = _time(lambda: dist.all_gather_into_tensor(xg, x_local), iters, warmup, flush)
    err = (y.float() - y_ref.float()).abs().max().item()
    flops = 2.0 * tokens * n1 * d_model
    comm_bytes = (world - 1) * m_local * d_model * 2
    roof = max(flops / (peak_tflops * 1e12), comm_bytes / (link_gbs * 1e9)) * 1e6
    rows.append({"op": "allgather_gemm", "n_gpus": world, "M": tokens, "N": n1, "K": d_model, "fused_us": fused,
                 "nccl_plus_cublas_us": base, "cublas_gemm_us": gemm_cublas, "own_gemm_us": gemm_ours, "nccl_allgather_us": comm_only,
                 "speedup_vs_nccl_cublas": base / fused, "roofline_us": roof, "fraction_of_roofline": roof / fused,
                 "max_abs_diff_vs_baseline": err})

    # ---- GEMM -> reduce-scatter ---------------------------------------------------------------
    rs = GemmReduceScatter(eng, tokens, d_model)
    h = (torch.randn(tokens, n1, generator=g, device="cuda") * 0.5).bfloat16()
    z = torch.empty(m_local, d_model, dtype=torch.bfloat16, device="cuda")
    part = torch.empty(tokens, d_model, dtype=torch.bfloat16, device="cuda")
    z_ref = torch.empty_like(z)

    def nccl_gemm_rs():
        torch.matmul(h, w2.t(), out=part)
        dist.reduce_scatter_tensor(z_ref, part)

    fused = _time(lambda: rs(h, w2, out=z), iters, warmup, flush)
    check_status("gemm_rs")
    base = _time(nccl_gemm_rs, iters, warmup, flush)
    gemm_cublas = _time(lambda: torch.matmul(h, w2.t(), out=part), iters, warmup, flush)
    gemm_ours = _time(lambda: gemm(h, w2, out=part), iters, warmup, flush)
    comm_only = _time(lambda: dist.reduce_scatter_tensor(z_ref, part), iters, warmup, flush)
    nccl_gemm_rs()
    rs(h, w2, out=z)
    torch.cuda.synchronize()
    err = (z.float() - z_ref.float()).abs().max().item()
    flops = 2.0 * tokens * d_model * n1
    comm_bytes = (world - 1) * m_local * d_model * 2
    roof = max(flops / (peak_tflops * 1e12), comm_bytes / (link_gbs * 1e9)) * 1e6
    rows.append({"op": "gemm_reduce_scatter", "n_gpus": world, "M": tokens, "N": d_model, "K": n1, "fused_us": fused,
                 "nccl_plus_cublas_us": base, "cublas_gemm_us": gemm_cublas, "own_gemm_us": gemm_ours,
                 "nccl_reduce_scatter_us": comm_only, "speedup_vs_nccl_cublas": base / fused, "roofline_us": roof,
                 "fraction_of_roofline": roof / fused, "max_abs_diff_vs_baseline": err})
    if fp8:
        rows += run_fp8(eng, tokens, d_model, d_ff, x_local, w1, w2, h, iters, warmup, n_copy, link_gbs, flush)
    return rows


def _scaled_mm_us(a_q, b_q, iters, warmup, flush):
    """cuBLASLt fp8 with ONE scale per tensor (torch._scaled_mm): the library's fp8 GEMM on this box; it has no
    1x128 / 128x128 block-scaled form here, so this is a speed reference only, not the same arithmetic."""
    one = torch.ones((), device="cuda")
    a8, b8 = a_q.view(torch.float8_e4m3fn), b_q.view(torch.float8_e4m3fn)
    try:
        return _time(lambda: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), iters, warmup, flush)
    except Exception:       # noqa: BLE001 - an unsupported shape or build leaves the reference out
        return None


def run_fp8(eng, tokens, d_model, d_ff, x_local, w1, w2, h, iters, warmup, n_copy, link_gbs, flush):
    """Block-scaled fp8 (1x128 activations, 128x128 weights) forms of the two fused paths."""
    n_copy = n_copy or default_copy_ctas(eng.world)
    world = eng.world
    n1 = d_ff // world
    m_local = tokens // world
    rows = []
    w1q, w1s = quant_blocks(w1)
    w2q, w2s = quant_blocks(w2)
    # ---- all-gather -> GEMM -------------------------------------------------------------------
    ag = AllGatherGemmFp8(eng, tokens, d_model, n_copy=max(2, n_copy // 2))
    ag.quantize_local(x_local)
    y = torch.empty(tokens, n1, dtype=torch.bfloat16, device="cuda")
    xg = torch.empty(tokens, d_model, dtype=torch.bfloat16, device="cuda")
    xgq = torch.empty(tokens, d_model, dtype=torch.uint8, device="cuda")
    xgs = torch.empty(tokens, d_model // 128, dtype=torch.float32, device="cuda")
    y_ref = torch.empty_like(y)
    xq_l, xs_l = ag.xq_local.clone(), ag.xs_local.clone()

    def nccl_bf16():
        dist.all_gather_into_tensor(xg, x_local)
        torch.matmul(xg, w1.t(), out=y_ref)

    def nccl_fp8_then_own_gemm():
        dist.all_gather_into_tensor(xgq, xq_l)
        dist.all_gather_into_tensor(xgs, xs_l)
        gemm_fp8(xgq, xgs, w1q, w1s, out=y_ref)

    fused = _time(lambda: ag(w1q, w1s, out=y), iters, warmup, flush)
    check_status("ag_gemm_fp8")
    fused_q = _time(lambda: ag(w1q, w1s, gelu=True, quant_out=True), iters, warmup, flush)
    base = _time(nccl_bf16, iters, warmup, flush)
    unfused = _time(nccl_fp8_then_own_gemm, iters, warmup, flush)
    torch.cuda.synchronize()
    err = (y.float() - y_ref.float()).abs().max().item()
    own = _time(lambda: gemm_fp8(xgq, xgs, w1q, w1s, out=y_ref), iters, warmup, flush)
    lt = _scaled_mm_us(xgq, w1q, iters, warmup, flush)
    flops = 2.0 * tokens * n1 * d_model
    comm_bytes = (world - 1) * m_local * (d_model + d_model // 128 * 4)
    peak = flops / (lt * 1e-6) if lt else None
    roof = max(flops / peak if peak else 0.0, comm_bytes / (link_gbs * 1e9)) * 1e6
    rows.append({"op": "allgather_gemm_fp8", "n_gpus": world, "M": tokens, "N": n1, "K": d_model, "fused_us": fused,
                 "fused_gelu_quant_out_us": fused_q, "nccl_bf16_plus_cublas_bf16_us": base, "nccl_fp8_plus_own_fp8_gemm_us": unfused,
                 "own_fp8_gemm_us": own, "cublaslt_fp8_tensorwise_gemm_us": lt, "speedup_vs_nccl_cublas_bf16": base / fused,
                 "speedup_vs_unfused_fp8": unfused / fused, "roofline_us": roof, "fraction_of_roofline": roof / fused,
                 "roofline_note": "compute term at the measured cuBLASLt tensorwise-fp8 rate of the same shape",
                 "max_abs_diff_vs_unfused": err})

    # ---- the same all-gather GEMM with power-of-two scales applied by the tensor core --------------
    try:
        from .ops.gemm import gemm_mx8, quant_blocks_mx
        agx = AllGatherGemmFp8(eng, tokens, d_model, n_copy=max(2, n_copy // 2), mx=True)
        agx.quantize_local(x_local)
        wxq, wxs = quant_blocks_mx(w1)
        fused_x = _time(lambda: agx(wxq, wxs, out=y), iters, warmup, flush)
        check_status("ag_gemm_mx8")
        own_x = _time(lambda: gemm_mx8(agx.xq_full, agx.xs_full, wxq, wxs, out=y_ref), iters, warmup, flush)
        roof_x = max(flops / peak if peak else 0.0, (world - 1) * m_local * (d_model + d_model // 128) / (link_gbs * 1e9)) * 1e6
        rows.append({"op": "allgather_gemm_mx8", "n_gpus": world, "M": tokens, "N": n1, "K": d_model, "fused_us": fused_x,
                     "nccl_bf16_plus_cublas_bf16_us": base, "own_mx8_gemm_us": own_x, "cublaslt_fp8_tensorwise_gemm_us": lt,
                     "speedup_vs_nccl_cublas_bf16": base / fused_x, "roofline_us": roof_x, "fraction_of_roofline": roof_x / fused_x,
                     "note": "e4m3 with UE8M0 (power-of-two) 1x128 / 128x128 scales, tcgen05 kind::mxf8f6f4.block_scale"})
    except Exception as e:      # noqa: BLE001 - the row is optional; the other rows must still be reported
        rows.append({"op": "allgather_gemm_mx8", "n_gpus": world, "error": f"{type(e).__name__}: {e}"})

    # ---- GEMM -> reduce-scatter ---------------------------------------------------------------
    rs = GemmReduceScatterFp8(eng, tokens, d_model)
    hq, hs = quant_rows(h)
    z = torch.empty(m_local, d_model, dtype=torch.bfloat16, device="cuda")
    part = torch.empty(tokens, d_model, dtype=torch.bfloat16, device="cuda")
    z_ref = torch.empty_like(z)

    def nccl_bf16_rs():
        torch.matmul(h, w2.t(), out=part)
        dist.reduce_scatter_tensor(z_ref, part)

    def own_gemm_then_nccl():
        gemm_fp8(hq, hs, w2q, w2s, out=part)
        dist.reduce_scatter_tensor(z_ref, part)

    fused = _time(lambda: rs(hq, hs, w2q, w2s, out=z), iters, warmup, flush)
    check_status("gemm_rs_fp8")
    base = _time(nccl_bf16_rs, iters, warmup, flush)
    unfused = _time(own_gemm_then_nccl, iters, warmup, flush)
    own = _time(lambda: gemm_fp8(hq, hs, w2q, w2s, out=part), iters, warmup, flush)
    lt = _scaled_mm_us(hq, w2q, iters, warmup, flush)
    own_gemm_then_nccl()
    rs(hq, hs, w2q, w2s, out=z)
    torch.cuda.synchronize()
    err = (z.float() - z_ref.float()).abs().max().item()
    flops = 2.0 * tokens * d_model * n1
    comm_bytes = (world - 1) * m_local * d_model * 2
    peak = flops / (lt * 1e-6) if lt else None
    roof = max(flops / peak if peak else 0.0, comm_bytes / (link_gbs * 1e9)) * 1e6
    rows.append({"op": "gemm_reduce_scatter_fp8", "n_gpus": world, "M": tokens, "N": d_model, "K": n1, "fused_us": fused,
                 "nccl_bf16_plus_cublas_bf16_us": base, "own_fp8_gemm_plus_nccl_us": unfused, "own_fp8_gemm_us": own,
                 "cublaslt_fp8_tensorwise_gemm_us": lt, "speedup_vs_nccl_cublas_bf16": base / fused,
                 "speedup_vs_unfused_fp8": unfused / fused, "roofline_us": roof, "fraction_of_roofline": roof / fused,
                 "roofline_note": "compute term at the measured cuBLASLt tensorwise-fp8 rate of the same shape",
                 "max_abs_diff_vs_unfused": err})
    return rows


def probe_fused(eng: Engine, tokens: int, d_model: int, d_ff: int, n_copy: int):
    """One launch of each bf16 fused kernel with the wait-time probes on (csrc/kernels/fused_api.h: setFusedProbe):
    per rank, the mean and maximum over CTAs of the nanoseconds spent in each kind of wait, the spread of CTA start
    times, and the kernel's span from the first CTA's start to the last CTA's end."""
    from ._native import C
    world, rank = eng.world, eng.rank
    n1, m_local = d_ff // world, tokens // world
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    w1 = (torch.randn(n1, d_model, generator=g, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(d_model, n1, generator=g, device="cuda") * 0.02).bfloat16()
    h = (torch.randn(tokens, n1, generator=g, device="cuda") * 0.5).bfloat16()
    ag = AllGatherGemm(eng, tokens, d_model, n_copy=n_copy)
    ag.x_local.normal_()
    rs = GemmReduceScatter(eng, tokens, d_model)
    ctas = C.sm_count()
    buf = torch.zeros(ctas * C.PROBE_WORDS, dtype=torch.int64, device="cuda")
    rows = []
    for name, fn in (("allgather_gemm", lambda: ag(w1)), ("gemm_reduce_scatter", lambda: rs(h, w2))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        buf.zero_()
        C.fused_set_probe(buf.data_ptr())
        fn()
        torch.cuda.synchronize()
        C.fused_set_probe(0)
        p = buf.view(ctas, C.PROBE_WORDS).double().cpu()
        live = p[:, 4] > 0
        start, end = p[live, 4], p[live, 5]
        rec = {"op": name + "_probe", "rank": rank, "n_gpus": world, "ctas": int(live.sum()),
               "span_us": float(end.max() - start.min()) / 1e3, "start_spread_us": float(start.max() - start.min()) / 1e3}
        for i, key in ((0, "gate_wait"), (1, "own_tile_wait"), (2, "stage_drain_wait"), (3, "tile_done_wait"), (6, "copy_role")):
            col = p[live, i] / 1e3
            rec[key + "_us_mean"] = float(col.mean())
            rec[key + "_us_max"] = float(col.max())
        rec["tiles_max_per_cta"] = float(p[live, 7].max())
        gathered = [None] * world
        dist.all_gather_object(gathered, rec)
        rows += gathered if rank == 0 else []
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=8192)
    ap.add_argument("--d-ff", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--n-copy", type=int, default=0, help="copy CTAs of the fused all-gather (0 = the default for this world size)")
    ap.add_argument("--no-fp8", action="store_true")
    ap.add_argument("--probe", action="store_true", help="after the timed runs, one launch of each bf16 fused kernel with the "
                    "in-kernel wait-time probes on; prints where the CTAs waited")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=180))
    os.environ.setdefault("PCCL_WORKSPACE_MB", "64")
    eng = Engine(rank, world)
    heap = 5 * args.tokens * args.d_model * 2 + (1 << 30)
    eng.initEngine("cuda", heap_bytes=heap)
    eng.connect()
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    rows = run(eng, args.tokens, args.d_model, args.d_ff, iters=args.iters, n_copy=args.n_copy or None,
               peak_tflops=float(peaks.get("bf16_tflops", 1590.0)), fp8=not args.no_fp8)
    if args.probe:
        rows += probe_fused(eng, args.tokens, args.d_model, args.d_ff, args.n_copy or None)
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump(rows, f)
    dist.barrier()
    del eng
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
