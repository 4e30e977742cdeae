"""Small single-GPU runs of the communication kernels with all ranks emulated in one launch, sized for
`ncu` captures (a few hundred MB on the device, a handful of launches):

    python -m pccl_b200.profile_targets ag_gemm   [--world 2 --rows 1024 --k 8192 --n 3584]
    python -m pccl_b200.profile_targets ag_gemm_fp8 [--world 2 --rows 1024 --k 8192 --n 3584]
    python -m pccl_b200.profile_targets gemm_rs   [--world 2 --rows 1024 --k 3584 --n 8192]
    python -m pccl_b200.profile_targets allreduce [--world 4 --mbytes 64]
    python -m pccl_b200.profile_targets moe       [--world 2 --tokens 2048 --hidden 7168]
    python -m pccl_b200.profile_targets train_kernels   (GEMM with the GELU-backward epilogue, LayerNorm backward with
                                                         the residual and bias-gradient extras, column sums; GPT-1.3B shapes)
    python -m pccl_b200.profile_targets grouped_gemm [--tokens 8192 --hidden 7168]   (expert FFN, 32 experts)

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


def train_kernels(a):
    """The fused kernels of the training step at the GPT-1.3B shapes (16384 tokens, d = 2048, d_ff = 8192)."""
    from .nn.norm import _ln_backward, _ln_forward
    from .ops.elementwise import colsum
    from .ops.gemm import gemm, gemm_dgelu, gemm_dual
    T, D, H = 16384, 2048, 8192
    r = lambda *s: torch.randn(*s, device="cuda").bfloat16()  # noqa: E731
    dz, w2, pre = r(T, D), r(D, H) * 0.02, r(T, H)
    out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    sums = torch.zeros(H, device="cuda")
    print({"op": "gemm_dgelu_colsum", "M": T, "N": H, "K": D, "us": _timed(lambda: gemm_dgelu(dz, w2, pre, b_t=True, colsum=sums, out=out), a.iters)})
    print({"op": "gemm_plain_same_shape", "us": _timed(lambda: gemm(dz, w2, b_t=True, out=out), a.iters)})
    act, xin, dy1 = r(T, H), r(T, D), r(T, H)
    dw1, dw2 = torch.empty(H, D, device="cuda", dtype=torch.bfloat16), torch.empty(D, H, device="cuda", dtype=torch.bfloat16)
    print({"op": "gemm_dual_two_weight_gradients", "K": T, "shapes": [[H, D], [D, H]],
           "us": _timed(lambda: gemm_dual(dy1, xin, dw1, dz, act, dw2, a_t=True, b_t=True), a.iters)})
    print({"op": "gemm_weight_gradients_two_launches",
           "us": _timed(lambda: (gemm(dy1, xin, a_t=True, b_t=True, out=dw1), gemm(dz, act, a_t=True, b_t=True, out=dw2)), a.iters)})
    x, delta, g = r(T, D), r(T, D), r(T, D)
    gamma, beta = torch.ones(D, device="cuda", dtype=torch.bfloat16), torch.zeros(D, device="cuda", dtype=torch.bfloat16)
    s, _, mean, rstd = _ln_forward(x, delta, gamma, beta, 1e-5)
    print({"op": "ln_fwd_add", "rows": T, "D": D, "us": _timed(lambda: _ln_forward(x, delta, gamma, beta, 1e-5), a.iters)})
    print({"op": "ln_bwd_add_colsum", "rows": T, "D": D, "us": _timed(lambda: _ln_backward(g, s, gamma, mean, rstd, delta, True), a.iters)})
    q = r(T, 3 * D)
    print({"op": "colsum", "rows": T, "N": 3 * D, "us": _timed(lambda: colsum(q), a.iters)})
    from .ops import check_status
    check_status("train kernels")


def grouped_gemm(a):
    """Expert FFN of the MoE layer: 32 experts, 7168 -> 2048 (GELU) -> 7168; rows spread unevenly, or (--balanced) the way a
    router with many tokens spreads them: the mean per expert give or take a few per cent."""
    from .ops.moe import grouped_gemm as gg
    E, H, Fd, rows = 32, a.hidden, 2048, a.tokens
    if a.balanced:
        sizes = (torch.randn(E) * 0.04 * rows / E + rows / E).round().clamp(min=1).long()
        sizes[-1] = max(1, rows - int(sizes[:-1].sum()))
        row_off = torch.cat([torch.zeros(1, dtype=torch.long), sizes.cumsum(0)]).to(torch.int32).cuda()
        rows = int(row_off[-1])
    else:
        cuts = torch.sort(torch.randint(0, rows, (E - 1,), device="cuda")).values
        row_off = torch.cat([torch.zeros(1, device="cuda", dtype=torch.long), cuts, torch.tensor([rows], device="cuda")]).to(torch.int32)
    x = torch.randn(rows, H, device="cuda").bfloat16()
    w1 = (torch.randn(E * Fd, H, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(E * H, Fd, device="cuda") * 0.02).bfloat16()
    h = torch.empty(rows, Fd, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(rows, H, device="cuda", dtype=torch.bfloat16)
    print({"op": "grouped_gemm_up_gelu", "rows": rows, "N": Fd, "K": H, "experts": E, "us": _timed(lambda: gg(x, w1, row_off, Fd, out=h, gelu=True), a.iters)})
    print({"op": "grouped_gemm_down", "rows": rows, "N": H, "K": Fd, "experts": E, "us": _timed(lambda: gg(h, w2, row_off, H, out=y), a.iters)})
    from .ops import check_status
    check_status("grouped gemm")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("target", choices=["ag_gemm", "ag_gemm_fp8", "gemm_rs", "allreduce", "moe", "train_kernels", "grouped_gemm"])
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--rows", type=int, default=1024, help="rows per rank")
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--n-copy", type=int, default=8)
    ap.add_argument("--mbytes", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--balanced", action="store_true", help="grouped_gemm: expert sizes near the mean instead of random cuts")
    a = ap.parse_args()
    if a.target in ("ag_gemm", "ag_gemm_fp8"):
        a.k, a.n = a.k or 8192, a.n or 3584
    if a.target == "gemm_rs":
        a.k, a.n = a.k or 3584, a.n or 8192
    {"ag_gemm": ag_gemm, "ag_gemm_fp8": ag_gemm_fp8, "gemm_rs": gemm_rs, "allreduce": allreduce, "moe": moe,
     "train_kernels": train_kernels, "grouped_gemm": grouped_gemm}[a.target](a)


if __name__ == "__main__":
    main()
