"""Small single-GPU runs of the communication kernels with all ranks emulated in one launch, sized for
`ncu` captures (a few hundred MB on the device, a handful of launches):

    python -m pccl_b200.profile_targets ag_gemm   [--world 2 --rows 1024 --k 8192 --n 3584]
    python -m pccl_b200.profile_targets ag_gemm_fp8 [--world 2 --rows 1024 --k 8192 --n 3584]
    python -m pccl_b200.profile_targets gemm_rs   [--world 2 --rows 1024 --k 3584 --n 8192]
    python -m pccl_b200.profile_targets allreduce [--world 4 --mbytes 64]
    python -m pccl_b200.profile_targets moe       [--world 2 --tokens 2048 --hidden 7168]

Each prints device times (CUDA events) of its launches and raises if a kernel reported a status.
"""
from __future__ import annotations

import argparse

import torch

from ._native import C

SIGNAL_OFF, FLAG_OFF, DATA_OFF = 0, 64 * 1024, 512 * 1024


def _timed(fn, iters):
    out = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); b.synchronize()
        out.append(round(a.elapsed_time(b) * 1e3, 1))
    return out


def _check(st):
    bad = [s.tolist() for s in st if int(s[0]) != 0]
    if bad:
        raise RuntimeError(f"kernel status {bad}")


def ag_gemm(a):
    w, ml, K, N = a.world, a.rows, a.k, a.n
    M = ml * w
    ready_off = DATA_OFF + M * K * 2
    heaps = [torch.zeros(ready_off + 4096, dtype=torch.uint8, device="cuda") for _ in range(w)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(w)]
    ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(w)]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(w)]
    for r in range(w):
        heaps[r][DATA_OFF:ready_off].view(torch.bfloat16).view(M, K)[r * ml:(r + 1) * ml].normal_()
    ctas = (C.sm_count() // w) & ~1
    ep = [0]

    def run():
        ep[0] += 1
        C.emu_ag_gemm([h.data_ptr() for h in heaps], FLAG_OFF, DATA_OFF, M, N, K, [x.data_ptr() for x in ws], K,
                      [o.data_ptr() for o in outs], N, ready_off, ep[0], a.n_copy, ctas, [s.data_ptr() for s in st], 0,
                      torch.cuda.current_stream().cuda_stream)
    print({"op": "ag_gemm", "world": w, "M": M, "N": N, "K": K, "ctas_per_rank": ctas, "us": _timed(run, a.iters)})
    _check(st)


def ag_gemm_fp8(a):
    """The block-scaled fp8 all-gather GEMM, emulated ranks, next to the plain fp8 GEMM of one rank's shape on the
    same number of CTAs (what the fused kernel would cost if the rows were already there)."""
    from .ops.gemm import gemm_fp8, quant_blocks, quant_rows
    w, ml, K, N = a.world, a.rows, a.k, a.n
    M = ml * w
    xs_off = DATA_OFF + M * K
    ready_off = xs_off + M * (K // 128) * 4
    heaps = [torch.zeros(ready_off + 4096, dtype=torch.uint8, device="cuda") for _ in range(w)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(w)]
    ws = [quant_blocks((torch.randn(N, K, device="cuda") * 0.02).bfloat16()) for _ in range(w)]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(w)]
    for r in range(w):
        q, s_ = quant_rows(torch.randn(ml, K, device="cuda").bfloat16())
        heaps[r][DATA_OFF:xs_off].view(M, K)[r * ml:(r + 1) * ml] = q
        heaps[r][xs_off:ready_off].view(torch.float32).view(M, K // 128)[r * ml:(r + 1) * ml] = s_
    ctas = (C.sm_count() // w) & ~1
    ep = [0]

    def run():
        ep[0] += 1
        C.ag_gemm_fp8(None, [h.data_ptr() for h in heaps], FLAG_OFF, DATA_OFF, xs_off, M, N, K, [x[0].data_ptr() for x in ws], K,
                      [x[1].data_ptr() for x in ws], K // 128, [o.data_ptr() for o in outs], N, [], [], 0, 0, 0, ready_off, ep[0],
                      a.n_copy if w > 1 else 0, ctas, 0, [s.data_ptr() for s in st], 0, torch.cuda.current_stream().cuda_stream)
    fused = _timed(run, a.iters)
    _check(st)
    aq = heaps[0][DATA_OFF:xs_off].view(M, K)
    a_s = heaps[0][xs_off:ready_off].view(torch.float32).view(M, K // 128)
    plain = _timed(lambda: gemm_fp8(aq, a_s, ws[0][0], ws[0][1], out=outs[0], sms=ctas - (a.n_copy if w > 1 else 0)), a.iters)
    print({"op": "ag_gemm_fp8", "world": w, "M": M, "N": N, "K": K, "ctas_per_rank": ctas, "us": fused,
           "plain_fp8_gemm_one_rank_same_ctas_us": plain})


def gemm_rs(a):
    w, ml, K, N = a.world, a.rows, a.k, a.n
    M = ml * w
    stage = w * ml * N * 2
    nflags = w * (ml // 128) * (N // 256)
    heaps = [torch.zeros(DATA_OFF + stage + nflags * 8, dtype=torch.uint8, device="cuda") for _ in range(w)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(w)]
    ys = [(torch.randn(M, K, device="cuda") * 0.5).bfloat16() for _ in range(w)]
    ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(w)]
    outs = [torch.empty(ml, N, dtype=torch.bfloat16, device="cuda") for _ in range(w)]
    ctas = (C.sm_count() // w) & ~1
    ep = [0]

    def run():
        ep[0] += 1
        C.emu_gemm_rs([h.data_ptr() for h in heaps], [y.data_ptr() for y in ys], K, [x.data_ptr() for x in ws], K,
                      [o.data_ptr() for o in outs], N, M, N, K, DATA_OFF, DATA_OFF + stage, ep[0], ctas, [s.data_ptr() for s in st], 0,
                      torch.cuda.current_stream().cuda_stream)
    print({"op": "gemm_rs", "world": w, "M": M, "N": N, "K": K, "ctas_per_rank": ctas, "us": _timed(run, a.iters)})
    _check(st)


def allreduce(a):
    w = a.world
    nbytes = a.mbytes << 20
    heaps = [torch.zeros(DATA_OFF + 2 * nbytes, dtype=torch.uint8, device="cuda") for _ in range(w)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(w)]
    for h in heaps:
        h[DATA_OFF:DATA_OFF + nbytes].view(torch.bfloat16).normal_()
    ep = [0]

    def run():
        ep[0] += 1
        C.emu_collective("allreduce", [h.data_ptr() for h in heaps], SIGNAL_OFF, FLAG_OFF, "bf16", "sum", DATA_OFF, DATA_OFF + nbytes,
                         nbytes // 2, ep[0], 0, 1.0, "", max(1, 128 // w), 512, torch.cuda.current_stream().cuda_stream,
                         [s.data_ptr() for s in st], [], [], 0)
    print({"op": "allreduce_p2p_emulated", "world": w, "bytes": nbytes, "us": _timed(run, a.iters)})
    _check(st)


def moe(a):
    w, T, H, Kt, epr = a.world, a.tokens, a.hidden, 8, 4
    cap = T * Kt * w
    q_off, s_off = DATA_OFF, DATA_OFF + cap * H
    y_off = s_off + cap * (H // 128) * 4
    heaps = [torch.zeros(y_off + cap * H * 2, dtype=torch.uint8, device="cuda") for _ in range(w)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(w)]
    xs = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(w)]
    ids = [torch.randint(0, w * epr, (T, Kt), device="cuda", dtype=torch.int32) for _ in range(w)]
    rows = [(torch.arange(T * Kt, device="cuda", dtype=torch.int32) + r * T * Kt).view(T, Kt).contiguous() for r in range(w)]
    probs = [torch.rand(T, Kt, device="cuda") for _ in range(w)]
    outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(w)]
    ep = [0]
    blocks = min(C.sm_count() // w, C.MAX_BLOCKS_PER_COLL)

    def run(kind):
        ep[0] += 1
        C.moe_exchange(kind, None, [h.data_ptr() for h in heaps], FLAG_OFF, T, H, Kt, epr, q_off, s_off, y_off, ep[0], 0,
                       [x.data_ptr() for x in xs], [i.data_ptr() for i in ids], [r.data_ptr() for r in rows],
                       [p.data_ptr() for p in probs], [o.data_ptr() for o in outs], [s.data_ptr() for s in st], blocks, 0,
                       torch.cuda.current_stream().cuda_stream)
    print({"op": "moe_dispatch", "world": w, "tokens": T, "hidden": H, "us": _timed(lambda: run("dispatch"), a.iters)})
    print({"op": "moe_combine", "world": w, "tokens": T, "hidden": H, "us": _timed(lambda: run("combine"), a.iters)})
    _check(st)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("target", choices=["ag_gemm", "ag_gemm_fp8", "gemm_rs", "allreduce", "moe"])
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--rows", type=int, default=1024, help="rows per rank")
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--n-copy", type=int, default=8)
    ap.add_argument("--mbytes", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    if a.target in ("ag_gemm", "ag_gemm_fp8"):
        a.k, a.n = a.k or 8192, a.n or 3584
    if a.target == "gemm_rs":
        a.k, a.n = a.k or 3584, a.n or 8192
    {"ag_gemm": ag_gemm, "ag_gemm_fp8": ag_gemm_fp8, "gemm_rs": gemm_rs, "allreduce": allreduce, "moe": moe}[a.target](a)


if __name__ == "__main__":
    main()
