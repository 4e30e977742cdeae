"""tcgen05 GEMM against an fp32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_t, b_t):
    A = a.float().t() if a_t else a.float()
    B = b.float() if b_t else b.float().t()
    return A @ B


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).bfloat16()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (1000, 520, 200), (72, 40, 136)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_matches_fp32_reference(M, N, K, a_t, b_t):
    from pccl_b200.ops import gemm, check_status
    a = _rand((K, M) if a_t else (M, K), 1)
    b = _rand((K, N) if b_t else (N, K), 2)
    out = gemm(a, b, a_t=a_t, b_t=b_t)
    check_status("gemm")
    ref = _ref(a, b, a_t, b_t)
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * (K ** 0.5) * 0.25 + 1e-2 * ref.abs().max().item()
    assert err <= tol, f"max err {err} > {tol}"
    # fp32 output is compared tightly: products of bf16 are exact in fp32, only the sum order differs
    out32 = gemm(a, b, a_t=a_t, b_t=b_t, out_dtype=torch.float32)
    assert (out32 - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())


def test_gemm_epilogues():
    from pccl_b200.ops import gemm, check_status
    M, N, K = 512, 1024, 512
    a, b = _rand((M, K), 3), _rand((N, K), 4, 0.05)
    bias = _rand((N,), 5)
    act = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pre = gemm(a, b, bias=bias, gelu_out=act)
    check_status("gemm")
    ref = a.float() @ b.float().t() + bias.float()
    assert (pre.float() - ref).abs().max().item() < 0.05
    ref_act = torch.nn.functional.gelu(ref, approximate="tanh")    # the kernel applies GELU before rounding
    assert ((act.float() - ref_act).abs() <= 0.01 + 0.01 * ref_act.abs()).all()
    acc = torch.ones((M, N), dtype=torch.float32, device="cuda")
    gemm(a, b, out=acc, accumulate=True)
    assert (acc - (a.float() @ b.float().t() + 1)).abs().max().item() < 1e-2


def test_gemm_padded_leading_dimension():
    from pccl_b200.ops import gemm
    M, N, K = 300, 1001, 264                     # N not a multiple of 8: row stride is padded
    a, b = _rand((M, K), 6), _rand((N, K), 7)
    out = gemm(a, b)
    assert out.shape == (M, N) and out.stride(0) == 1008
    assert (out.float() - a.float() @ b.float().t()).abs().max().item() < 0.5
    # consume it again as a K-padded operand
    w = _rand((128, N), 8, 0.1)
    wp = torch.zeros((128, 1008), dtype=torch.bfloat16, device="cuda")[:, :N]
    wp.copy_(w)
    y = gemm(out, wp)
    assert (y.float() - out.float() @ w.float().t()).abs().max().item() < 1.0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 512), (1000, 520, 200), (72, 40, 136), (2048, 1024, 1024)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True), (True, False)])
def test_cta_pair_gemm_matches_fp32_reference(M, N, K, a_t, b_t):
    """cta_group::2 kernel: two CTAs per 256 x 256 tile."""
    from pccl_b200.ops import gemm, check_status
    a = _rand((K, M) if a_t else (M, K), 11)
    b = _rand((K, N) if b_t else (N, K), 12)
    out32 = gemm(a, b, a_t=a_t, b_t=b_t, out_dtype=torch.float32, pair=True)
    check_status("pair gemm")
    ref = _ref(a, b, a_t, b_t)
    assert (out32 - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())
    bias = _rand((N,), 13)
    out = gemm(a, b, a_t=a_t, b_t=b_t, bias=bias, pair=True)
    assert (out.float() - (ref + bias.float())).abs().max().item() <= 0.02 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (384, 768, 2048), (1000, 640, 512), (72, 128, 256)])
def test_fp8_block_scaled_gemm_matches_fp32_reference_of_the_quantised_operands(M, N, K):
    from pccl_b200.ops import check_status
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, gemm_fp8, quant_blocks, quant_rows
    a = _rand((M, K), 3)
    w = _rand((N, K), 4, scale=0.02)
    # per-block magnitudes that differ by orders of magnitude, so that a wrong scale index shows
    a = (a.float() * torch.logspace(-2, 2, K // 128, device="cuda").repeat_interleave(128)[None, :]).bfloat16()
    aq, a_s = quant_rows(a)
    wq, w_s = quant_blocks(w)
    out32 = gemm_fp8(aq, a_s, wq, w_s, out_dtype=torch.float32)
    check_status("gemm_fp8")
    ref = dequant_rows(aq, a_s) @ dequant_blocks(wq, w_s).t()
    scale = max(1.0, ref.abs().max().item())
    # the kernel's sum is exact products of e4m3 values accumulated in fp32: only the order differs
    assert (out32 - ref).abs().max().item() <= 2e-3 * scale
    out = gemm_fp8(aq, a_s, wq, w_s)
    assert (out.float() - ref).abs().max().item() <= 1e-2 * scale
    # and the quantised product stays close to the bf16 one
    full = a.float() @ w.float().t()
    assert (ref - full).abs().max().item() <= 0.08 * full.abs().max().item()


def test_fp8_gemm_bias_and_accumulate():
    from pccl_b200.ops import check_status
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, gemm_fp8, quant_blocks, quant_rows
    M, N, K = 256, 384, 512
    aq, a_s = quant_rows(_rand((M, K), 5))
    wq, w_s = quant_blocks(_rand((N, K), 6, scale=0.05))
    bias = _rand((N,), 7)
    ref = dequant_rows(aq, a_s) @ dequant_blocks(wq, w_s).t()
    out = torch.ones((M, N), device="cuda", dtype=torch.float32)
    gemm_fp8(aq, a_s, wq, w_s, out=out, bias=bias, accumulate=True)
    check_status("gemm_fp8")
    assert (out - (ref + bias.float()[None, :] + 1.0)).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item())


def test_mx_quantisers_give_power_of_two_scales_that_cover_the_block():
    from pccl_b200.ops.gemm import dequant_rows, quant_blocks_mx, quant_rows_mx, ue8m0_to_float
    x = _rand((200, 512), 11, scale=3.0)
    q, s = quant_rows_mx(x)
    sc = ue8m0_to_float(s)
    amax = x.float().view(200, 4, 128).abs().amax(-1)
    assert torch.all(sc * 448.0 >= amax) and torch.all(sc * 224.0 < amax.clamp_min(1e-30) * 1.0000001)
    back = dequant_rows(q, sc)
    assert (back - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    w = _rand((256, 384), 12, scale=0.02)
    qw, sw = quant_blocks_mx(w)
    amaxw = w.float().view(2, 128, 3, 128).abs().amax((1, 3))
    assert torch.all(ue8m0_to_float(sw) * 448.0 >= amaxw)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 256, 512), (256, 512, 1024), (384, 768, 2048), (1000, 640, 640), (72, 128, 256)])
def test_mx_fp8_gemm_matches_fp32_reference_of_the_quantised_operands(M, N, K):
    from pccl_b200.ops import check_status
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, gemm_mx8, quant_blocks_mx, quant_rows_mx, ue8m0_to_float
    a = _rand((M, K), 13)
    w = _rand((N, K), 14, scale=0.02)
    # magnitudes that differ per K block AND per row group / column block, so that a wrong scale index shows
    a = (a.float() * torch.logspace(-2, 2, K // 128, device="cuda").repeat_interleave(128)[None, :]
         * (1.0 + (torch.arange(M, device="cuda") // 32 % 4).float())[:, None]).bfloat16()
    w = (w.float() * (1.0 + 3.0 * (torch.arange(N, device="cuda") // 128).float())[:, None]).bfloat16()
    aq, a_s = quant_rows_mx(a)
    wq, w_s = quant_blocks_mx(w)
    out32 = gemm_mx8(aq, a_s, wq, w_s, out_dtype=torch.float32)
    check_status("gemm_mx8")
    ref = dequant_rows(aq, ue8m0_to_float(a_s)) @ dequant_blocks(wq, ue8m0_to_float(w_s)).t()
    scale = max(1.0, ref.abs().max().item())
    assert (out32 - ref).abs().max().item() <= 2e-3 * scale
    out = gemm_mx8(aq, a_s, wq, w_s)
    assert (out.float() - ref).abs().max().item() <= 1e-2 * scale


def test_gemm_residual_epilogue_adds_the_residual_stream():
    """out = a @ b.T + bias + residual in the GEMM epilogue (full and ragged tiles)."""
    from pccl_b200.ops import gemm, check_status
    for (M, N, K) in [(512, 1024, 256), (300, 264, 128)]:
        a, b = _rand((M, K), 21), _rand((N, K), 22, 0.05)
        bias, res = _rand((N,), 23), _rand((M, N), 24)
        out = gemm(a, b, bias=bias, residual=res)
        check_status("gemm residual")
        ref = a.float() @ b.float().t() + bias.float() + res.float()
        assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("b_t", [True, False])
def test_gemm_dgelu_epilogue_and_column_sums(b_t):
    """(a @ op(b)) * gelu_tanh'(pre) with the column sums of the result, against fp32 PyTorch."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.gemm import gemm_dgelu
    M, N, K = 512, 768, 256
    a = _rand((M, K), 31)
    b = _rand((K, N) if b_t else (N, K), 32, 0.05)
    pre = _rand((M, N), 33, 1.5)
    sums = torch.zeros(N, dtype=torch.float32, device="cuda")
    out = gemm_dgelu(a, b, pre, b_t=b_t, colsum=sums)
    check_status("gemm dgelu")
    prod = a.float() @ (b.float() if b_t else b.float().t())
    x = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(x, approximate="tanh").backward(prod)
    ref = x.grad
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert (sums - ref.sum(0)).abs().max().item() <= 2e-2 * max(1.0, ref.sum(0).abs().max().item())
    # without column sums the product is the same
    out2 = gemm_dgelu(a, b, pre, b_t=b_t)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("shapes", [((512, 256), (256, 768)), ((304, 520), (1032, 136)), ((2048, 8192), (8192, 2048))])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_dual_two_weight_gradients_one_launch(shapes, out_dtype):
    """Two dW = dy^T x products of one row count as a single launch, fresh and accumulating, against fp32 PyTorch."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.gemm import gemm_dual
    rows = 1024
    (m0, n0), (m1, n1) = shapes
    dy0, x0 = _rand((rows, m0), 51, 0.1), _rand((rows, n0), 52)
    dy1, x1 = _rand((rows, m1), 53, 0.1), _rand((rows, n1), 54)
    o0 = torch.full((m0, n0), 3.0, dtype=out_dtype, device="cuda")
    o1 = torch.full((m1, n1), -2.0, dtype=out_dtype, device="cuda")
    gemm_dual(dy0, x0, o0, dy1, x1, o1, a_t=True, b_t=True, accumulate1=True)
    check_status("gemm dual")
    r0 = dy0.float().t() @ x0.float()
    r1 = dy1.float().t() @ x1.float() - 2.0
    for got, ref in ((o0, r0), (o1, r1)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    # the plain (K-major) operand forms go through the same scheduler
    a0, b0 = _rand((m0, 192), 55), _rand((n0, 192), 56)
    a1, b1 = _rand((m1, 192), 57), _rand((n1, 192), 58)
    p0 = torch.empty((m0, n0), dtype=out_dtype, device="cuda")
    p1 = torch.empty((m1, n1), dtype=out_dtype, device="cuda")
    gemm_dual(a0, b0, p0, a1, b1, p1)
    check_status("gemm dual k-major")
    for got, ref in ((p0, a0.float() @ b0.float().t()), (p1, a1.float() @ b1.float().t())):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("rows,N", [(16384, 2048), (1000, 520), (37, 8)])
def test_colsum_kernel_matches_torch(rows, N):
    from pccl_b200.ops.elementwise import colsum
    x = _rand((rows, N), 41)
    got = colsum(x)
    ref = x.float().sum(0)
    assert (got.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())
    view = _rand((rows, N + 24), 42)[:, 8:8 + N] if N % 8 == 0 and N > 8 else None     # a column slice of a wider buffer
    if view is not None and view.data_ptr() % 16 == 0:
        assert (colsum(view).float() - view.float().sum(0)).abs().max().item() <= 1e-2 * max(1.0, view.float().sum(0).abs().max().item())
