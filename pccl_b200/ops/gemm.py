"""bf16 GEMM on the tcgen05/TMEM pipeline (csrc/kernels/gemm_tc05.cu).

``gemm(a, b, a_t=False, b_t=False)`` computes ``op(a) @ op(b)`` for row-major tensors, where the
flags say which operand is consumed in its transposed ("MN-major") form — the kernel reads such an
operand through a different TMA box and shared-memory descriptor, no transpose pass is made.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .._native import C

import os

_PAIR_DEFAULT = os.environ.get("PCCL_GEMM_PAIR", "1") != "0"      # CTA pairs unless switched off
_status: Dict[int, torch.Tensor] = {}
_launches = 0


def status_words(device=None) -> torch.Tensor:
    """Per-device status words that kernels write when a bounded wait runs out (all zero = fine)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx not in _status:
        _status[idx] = torch.zeros(64, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_status(what: str = "kernel") -> None:
    """Synchronises and raises if a kernel reported a failure since the last check."""
    st = status_words()
    vals = st[:4].tolist()
    if vals[0] != 0:
        st.zero_()
        C.gemm_reset_tile_counters()      # a GEMM that gave up leaves its run-time tile counter where it was
        raise RuntimeError(f"{what}: device status {vals} (1 = bounded wait timed out)")


def launch_count() -> int:
    """Number of kernels of this package launched by this process (benchmarks report it)."""
    return _launches


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def _check(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"gemm: {name} must be a 2-D CUDA bf16 tensor with unit inner stride")
    if t.stride(0) % 8 or t.data_ptr() % 16:
        raise ValueError(f"gemm: {name} needs a row stride that is a multiple of 8 and a 16-byte aligned base")


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         bias: Optional[torch.Tensor] = None, gelu_out: Optional[torch.Tensor] = None,
         accumulate: bool = False, sms: int = 0, pair: Optional[bool] = None,
         residual: Optional[torch.Tensor] = None, row_stores: bool = False) -> torch.Tensor:
    """``out = op(a) @ op(b)`` with ``op(a) = a.T if a_t else a`` (a: [M,K] or [K,M]) and
    ``op(b) = b if b_t else b.T`` (b: [N,K], or [K,N] when ``b_t``).  So the default is the linear
    layer form ``a @ b.T``.  ``bias`` (bf16 [N]) is added; ``gelu_out`` receives gelu_tanh(out).
    ``pair`` selects the CTA-pair kernel (cta_group::2, 256 x 256 tiles); default from PCCL_GEMM_PAIR.
    ``residual`` (bf16, out's shape and strides) is added in the epilogue: ``out = a @ b.T + bias + residual``.
    ``row_stores`` turns the epilogue's coalescing patch off (comparison runs)."""
    _check(a, "a")
    _check(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_t else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_t else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    if out is None:
        ldd = (N + 7) // 8 * 8
        store = torch.empty((M, ldd), dtype=out_dtype, device=a.device)
        out = store[:, :N] if ldd != N else store
    if out.dtype not in (torch.bfloat16, torch.float32) or out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError("gemm: out must be [M,N] bf16/fp32 with unit inner stride")
    flags = 0
    if a_t:
        flags |= C.GEMM_A_MN
    if b_t:
        flags |= C.GEMM_B_MN
    if out.dtype == torch.float32:
        flags |= C.GEMM_OUT_F32
    if accumulate:
        flags |= C.GEMM_ACCUMULATE
    if (_PAIR_DEFAULT and M > 128) if pair is None else pair:
        flags |= C.GEMM_PAIR
    if row_stores:
        flags |= C.GEMM_ROW_STORES
    bias_ptr = 0
    if bias is not None:
        if bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous():
            raise ValueError("gemm: bias must be a contiguous bf16 vector of length N")
        flags |= C.GEMM_BIAS
        bias_ptr = bias.data_ptr()
    d2 = 0
    if gelu_out is not None:
        if gelu_out.shape != out.shape or gelu_out.stride() != out.stride() or gelu_out.dtype != torch.bfloat16:
            raise ValueError("gemm: gelu_out must match out")
        flags |= C.GEMM_GELU
        d2 = gelu_out.data_ptr()
    if residual is not None:
        if gelu_out is not None or out.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16 or residual.shape != out.shape \
                or residual.stride() != out.stride() or residual.data_ptr() % 16:
            raise ValueError("gemm: residual must be bf16 with out's shape and strides (and excludes gelu_out)")
        flags |= C.GEMM_ADD_D2
        d2 = residual.data_ptr()
    C.gemm_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), M, N, K, flags,
                bias_ptr, d2, sms, status_words(a.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch()
    return out


def gemm_dual(a0: torch.Tensor, b0: torch.Tensor, out0: torch.Tensor, a1: torch.Tensor, b1: torch.Tensor, out1: torch.Tensor, *,
              a_t: bool = False, b_t: bool = False, accumulate0: bool = False, accumulate1: bool = False, sms: int = 0) -> None:
    """Two GEMMs ``out_i (+)= op(a_i) @ op(b_i)`` with one reduction length and operand form, as a single launch: their tiles
    form one list for the persistent CTA pairs, so the partly filled last wave is paid once (the two weight-gradient GEMMs
    of an MLP are the case in mind)."""
    for t, name in ((a0, "a0"), (b0, "b0"), (a1, "a1"), (b1, "b1")):
        _check(t, name)
    dims = []
    for a, b, out in ((a0, b0, out0), (a1, b1, out1)):
        M, K = (a.shape[1], a.shape[0]) if a_t else (a.shape[0], a.shape[1])
        N, Kb = (b.shape[1], b.shape[0]) if b_t else (b.shape[0], b.shape[1])
        if K != Kb or out.shape != (M, N) or out.stride(1) != 1 or out.dtype != out0.dtype or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("gemm_dual: shapes do not match, or the outputs differ in dtype")
        dims.append((M, N, K))
    if dims[0][2] != dims[1][2]:
        raise ValueError("gemm_dual: both products must have the same inner dimension")
    flags = (C.GEMM_A_MN if a_t else 0) | (C.GEMM_B_MN if b_t else 0) | (C.GEMM_OUT_F32 if out0.dtype == torch.float32 else 0)
    C.gemm_bf16_dual(a0.data_ptr(), a0.stride(0), b0.data_ptr(), b0.stride(0), out0.data_ptr(), out0.stride(0), dims[0][0], dims[0][1], accumulate0,
                     a1.data_ptr(), a1.stride(0), b1.data_ptr(), b1.stride(0), out1.data_ptr(), out1.stride(0), dims[1][0], dims[1][1], accumulate1,
                     dims[0][2], flags, sms, status_words(a0.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch()


def gemm_dgelu(a: torch.Tensor, b: torch.Tensor, pre: torch.Tensor, *, b_t: bool = False, colsum: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, sms: int = 0) -> torch.Tensor:
    """``out = (a @ op(b)) * gelu_tanh'(pre)`` in one kernel (the GELU derivative is applied in the GEMM epilogue), and,
    when ``colsum`` (fp32 [N], zeroed by the caller) is given, ``colsum += out.sum(0)``.  This is the step of an MLP's
    backward pass that turns the gradient of the second layer's input into the gradient of the first layer's output;
    the column sums are the first layer's bias gradient.  M and N must be multiples of 256."""
    _check(a, "a")
    _check(b, "b")
    M, K = a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_t else (b.shape[0], b.shape[1])
    if K != Kb or pre.shape != (M, N) or pre.dtype != torch.bfloat16 or pre.stride(1) != 1:
        raise ValueError("gemm_dgelu: shapes of a, b and pre do not match")
    if out is None:
        out = torch.empty_strided((M, N), pre.stride(), dtype=torch.bfloat16, device=a.device)
    if out.stride() != pre.stride() or out.dtype != torch.bfloat16:
        raise ValueError("gemm_dgelu: out must have pre's strides")
    if colsum is not None and (colsum.dtype != torch.float32 or colsum.numel() != N or not colsum.is_contiguous()):
        raise ValueError("gemm_dgelu: colsum must be a contiguous fp32 vector of length N")
    C.gemm_bf16_dgelu(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), pre.data_ptr(),
                      colsum.data_ptr() if colsum is not None else 0, M, N, K, C.GEMM_B_MN if b_t else 0, sms,
                      status_words(a.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch()
    return out


def quant_rows(x: torch.Tensor):
    """bf16 [rows, K] -> (e4m3 bytes [rows, K], fp32 scales [rows, K/128]): one scale per row and 128 values."""
    rows, k = x.shape
    if k % 128 or not x.is_contiguous() or x.dtype != torch.bfloat16:
        raise ValueError("quant_rows: contiguous bf16 with K % 128 == 0")
    q = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, k // 128), dtype=torch.float32, device=x.device)
    C.quant_fp8_rows(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, k, torch.cuda.current_stream().cuda_stream)
    count_launch()
    return q, s


def quant_blocks(w: torch.Tensor):
    """bf16 [N, K] weights -> (e4m3 bytes, fp32 scales [N/128, K/128]): one scale per 128 x 128 block."""
    n, k = w.shape
    if n % 128 or k % 128 or not w.is_contiguous() or w.dtype != torch.bfloat16:
        raise ValueError("quant_blocks: contiguous bf16 with both sizes multiples of 128")
    q = torch.empty((n, k), dtype=torch.uint8, device=w.device)
    s = torch.empty((n // 128, k // 128), dtype=torch.float32, device=w.device)
    C.quant_fp8_blocks(w.data_ptr(), q.data_ptr(), s.data_ptr(), n, k, torch.cuda.current_stream().cuda_stream)
    count_launch()
    return q, s


def gemm_fp8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, *,
             out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
             bias: Optional[torch.Tensor] = None, gelu_inplace: bool = False, accumulate: bool = False,
             sms: int = 0) -> torch.Tensor:
    """Block-scaled fp8 linear form ``a @ b.T``: ``a_q`` e4m3 bytes [M, K] with ``a_s`` fp32 [M, K/128]
    (1 x 128 scales), ``b_q`` e4m3 bytes [N, K] with ``b_s`` fp32 [ceil(N/128), K/128] (128 x 128 scales).
    The partial product of every 128-wide K block is scaled and accumulated in fp32 (csrc/kernels/gemm_fp8.cu)."""
    for t, name in ((a_q, "a_q"), (b_q, "b_q")):
        if not t.is_cuda or t.element_size() != 1 or t.dim() != 2 or t.stride(1) != 1 or t.stride(0) % 16 or t.data_ptr() % 16:
            raise ValueError(f"gemm_fp8: {name} must be 2-D one-byte elements, unit inner stride, 16-byte aligned rows")
    M, K = a_q.shape
    N, Kb = b_q.shape
    if K != Kb or K % 128:
        raise ValueError("gemm_fp8: inner sizes must agree and be a multiple of 128")
    if a_s.dtype != torch.float32 or a_s.shape != (M, K // 128) or a_s.stride(1) != 1:
        raise ValueError("gemm_fp8: a_s must be fp32 [M, K/128]")
    if b_s.dtype != torch.float32 or b_s.shape != ((N + 127) // 128, K // 128) or b_s.stride(1) != 1:
        raise ValueError("gemm_fp8: b_s must be fp32 [ceil(N/128), K/128]")
    if out is None:
        ldd = (N + 7) // 8 * 8
        store = torch.empty((M, ldd), dtype=out_dtype, device=a_q.device)
        out = store[:, :N] if ldd != N else store
    if out.dtype not in (torch.bfloat16, torch.float32) or out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError("gemm_fp8: out must be [M,N] bf16/fp32 with unit inner stride")
    flags = 0
    if out.dtype == torch.float32:
        flags |= C.GEMM_OUT_F32
    if accumulate:
        flags |= C.GEMM_ACCUMULATE
    if gelu_inplace:
        flags |= C.GEMM_GELU_INPLACE
    bias_ptr = 0
    if bias is not None:
        if bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous():
            raise ValueError("gemm_fp8: bias must be a contiguous bf16 vector of length N")
        flags |= C.GEMM_BIAS
        bias_ptr = bias.data_ptr()
    C.gemm_fp8(a_q.data_ptr(), a_q.stride(0), a_s.data_ptr(), a_s.stride(0), b_q.data_ptr(), b_q.stride(0), b_s.data_ptr(),
               b_s.stride(0), out.data_ptr(), out.stride(0), M, N, K, flags, bias_ptr, 0, sms,
               status_words(a_q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch()
    return out


def quant_rows_mx(x: torch.Tensor):
    """bf16 [rows, K] -> (e4m3 bytes [rows, K], UE8M0 scale bytes [rows, K/128]): power-of-two scales for the
    hardware block-scaled GEMM (``gemm_mx8``)."""
    rows, k = x.shape
    if k % 128 or not x.is_contiguous() or x.dtype != torch.bfloat16:
        raise ValueError("quant_rows_mx: contiguous bf16 with K % 128 == 0")
    q = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, k // 128), dtype=torch.uint8, device=x.device)
    C.quant_mx8_rows(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, k, torch.cuda.current_stream().cuda_stream)
    count_launch()
    return q, s


def quant_blocks_mx(w: torch.Tensor):
    """bf16 [N, K] weights -> (e4m3 bytes, UE8M0 scale bytes [N/128, K/128])."""
    n, k = w.shape
    if n % 128 or k % 128 or not w.is_contiguous() or w.dtype != torch.bfloat16:
        raise ValueError("quant_blocks_mx: contiguous bf16 with both sizes multiples of 128")
    q = torch.empty((n, k), dtype=torch.uint8, device=w.device)
    s = torch.empty((n // 128, k // 128), dtype=torch.uint8, device=w.device)
    C.quant_mx8_blocks(w.data_ptr(), q.data_ptr(), s.data_ptr(), n, k, torch.cuda.current_stream().cuda_stream)
    count_launch()
    return q, s


def ue8m0_to_float(s: torch.Tensor) -> torch.Tensor:
    """2^(byte - 127) as fp32."""
    return torch.exp2(s.float() - 127.0)


def gemm_mx8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, *,
             out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
             bias: Optional[torch.Tensor] = None, gelu_inplace: bool = False, accumulate: bool = False,
             sms: int = 0) -> torch.Tensor:
    """``a @ b.T`` for e4m3 operands with power-of-two block scales applied by the tensor core
    (tcgen05 ``kind::mxf8f6f4.block_scale``; csrc/kernels/gemm_mx8.cu): ``a_s`` uint8 [M, K/128], ``b_s`` uint8
    [ceil(N/128), K/128], bytes in UE8M0 (``quant_rows_mx`` / ``quant_blocks_mx``)."""
    for t, name in ((a_q, "a_q"), (b_q, "b_q")):
        if not t.is_cuda or t.element_size() != 1 or t.dim() != 2 or t.stride(1) != 1 or t.stride(0) % 16 or t.data_ptr() % 16:
            raise ValueError(f"gemm_mx8: {name} must be 2-D one-byte elements, unit inner stride, 16-byte aligned rows")
    M, K = a_q.shape
    N, Kb = b_q.shape
    if K != Kb or K % 128:
        raise ValueError("gemm_mx8: inner sizes must agree and be a multiple of 128")
    if a_s.dtype != torch.uint8 or a_s.shape != (M, K // 128) or a_s.stride(1) != 1:
        raise ValueError("gemm_mx8: a_s must be uint8 [M, K/128]")
    if b_s.dtype != torch.uint8 or b_s.shape != ((N + 127) // 128, K // 128) or b_s.stride(1) != 1:
        raise ValueError("gemm_mx8: b_s must be uint8 [ceil(N/128), K/128]")
    if out is None:
        ldd = (N + 7) // 8 * 8
        store = torch.empty((M, ldd), dtype=out_dtype, device=a_q.device)
        out = store[:, :N] if ldd != N else store
    if out.dtype not in (torch.bfloat16, torch.float32) or out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError("gemm_mx8: out must be [M,N] bf16/fp32 with unit inner stride")
    flags = 0
    if out.dtype == torch.float32:
        flags |= C.GEMM_OUT_F32
    if accumulate:
        flags |= C.GEMM_ACCUMULATE
    if gelu_inplace:
        flags |= C.GEMM_GELU_INPLACE
    bias_ptr = 0
    if bias is not None:
        if bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous():
            raise ValueError("gemm_mx8: bias must be a contiguous bf16 vector of length N")
        flags |= C.GEMM_BIAS
        bias_ptr = bias.data_ptr()
    C.gemm_mx8(a_q.data_ptr(), a_q.stride(0), a_s.data_ptr(), a_s.stride(0), b_q.data_ptr(), b_q.stride(0), b_s.data_ptr(),
               b_s.stride(0), out.data_ptr(), out.stride(0), M, N, K, flags, bias_ptr, 0, sms,
               status_words(a_q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch()
    return out


def dequant_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """fp32 values of a 1 x 128 block-scaled e4m3 tensor (reference for tests; tensor ops)."""
    v = q.view(torch.float8_e4m3fn).float()
    return (v.view(q.shape[0], -1, 128) * s.unsqueeze(-1)).view(q.shape)


def dequant_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """fp32 values of a 128 x 128 block-scaled e4m3 tensor (reference for tests; tensor ops)."""
    n, k = q.shape
    v = q.view(torch.float8_e4m3fn).float().view(n // 128, 128, k // 128, 128)
    return (v * s.view(n // 128, 1, k // 128, 1)).view(n, k)


def gemm_nt(a, b, **kw):
    """a[M,K] @ b[N,K].T"""
    return gemm(a, b, **kw)


def gemm_nn(a, b, **kw):
    """a[M,K] @ b[K,N]"""
    return gemm(a, b, b_t=True, **kw)


def gemm_tn(a, b, **kw):
    """a[K,M].T @ b[K,N]"""
    return gemm(a, b, a_t=True, b_t=True, **kw)


if __name__ == "__main__":      # python -m pccl_b200.ops.gemm --m 4096 --n 4096 --k 4096 [--iters 3] [--a-t] [--b-t]
    import argparse
    ap = argparse.ArgumentParser(description="run the tcgen05 GEMM a few times (profiling / timing target)")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--a-t", action="store_true")
    ap.add_argument("--b-t", action="store_true")
    ap.add_argument("--pair", action="store_true")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 operands (1x128 / 128x128 scales)")
    ap.add_argument("--mx", action="store_true", help="with --fp8: power-of-two scales applied by the tensor core")
    a_ = ap.parse_args()
    if a_.fp8:
        qr, qb, gemm_fp8 = (quant_rows_mx, quant_blocks_mx, gemm_mx8) if a_.mx else (quant_rows, quant_blocks, gemm_fp8)
        Aq, As = qr(torch.randn((a_.m, a_.k), device="cuda").bfloat16())
        Bq, Bs = qb((torch.randn((a_.n, a_.k), device="cuda") * 0.02).bfloat16())
        D = torch.empty((a_.m, a_.n), device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(a_.iters + 1)]
        ev[0].record()
        for i in range(a_.iters):
            gemm_fp8(Aq, As, Bq, Bs, out=D)
            ev[i + 1].record()
        torch.cuda.synchronize()
        check_status("gemm_fp8")
        ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(a_.iters)]
        print({"fp8": True, "mx": a_.mx, "ms": ms, "tflops": [2 * a_.m * a_.n * a_.k / t / 1e9 for t in ms]})
        raise SystemExit(0)
    A = torch.randn((a_.k, a_.m) if a_.a_t else (a_.m, a_.k), device="cuda").bfloat16()
    B = torch.randn((a_.k, a_.n) if a_.b_t else (a_.n, a_.k), device="cuda").bfloat16()
    D = torch.empty((a_.m, a_.n), device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(a_.iters + 1)]
    ev[0].record()
    for i in range(a_.iters):
        gemm(A, B, a_t=a_.a_t, b_t=a_.b_t, out=D, pair=a_.pair)
        ev[i + 1].record()
    torch.cuda.synchronize()
    check_status("gemm")
    ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(a_.iters)]
    print({"ms": ms, "tflops": [2 * a_.m * a_.n * a_.k / t / 1e9 for t in ms]})
