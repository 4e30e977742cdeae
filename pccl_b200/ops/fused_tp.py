"""Tensor/sequence-parallel GEMMs with the collective fused in (csrc/kernels/fused_tp.cu).

``AllGatherGemm``: ``Y = all_gather_rows(X) @ W^T``.  ``GemmReduceScatter``: ``Z_r = reduce_scatter_rows(
Y @ W^T)``.  Each object owns the symmetric buffers of one layer shape and counts its launches (the
kernels' flags are epoch-valued and never reset).
"""
from __future__ import annotations

from typing import Optional

import torch

from .._native import C
from ..engine import Engine
from .gemm import count_launch, status_words


def default_copy_ctas(world: int) -> int:
    """Copy CTAs of the fused all-gather kernels: each peer's share of the rows shrinks with the world size while the
    number of receivers grows, so larger worlds want more of them."""
    return 8 if world <= 4 else 16


class AllGatherGemm:
    """Rows of X are sharded over the ranks.  Write this rank's rows into ``self.x_local`` (a view of
    the symmetric gathered buffer), then ``out = self(w)``; afterwards ``self.x_full`` holds all rows
    (the backward pass of a column-parallel layer needs them for the weight gradient)."""

    def __init__(self, eng: Engine, rows_total: int, k: int, n_copy: Optional[int] = None, ctas: Optional[int] = None, flag_lane: int = 4):
        """``n_copy``: CTAs that push this rank's rows to the peers while the others multiply.  Default from measurements
        at the 8192 x 8192 row block: 8 on up to four GPUs (703 us against 757 with 16 at TP=4), 16 on eight."""
        if n_copy is None:
            n_copy = default_copy_ctas(eng.world)
        if rows_total % (128 * eng.world) or k % 8:
            raise ValueError("AllGatherGemm: rows per rank must be a multiple of 128 and K a multiple of 8")
        self.eng, self.M, self.K = eng, rows_total, k
        self.x_full = eng.symmetric_tensor((rows_total, k), torch.bfloat16)
        m_local = rows_total // eng.world
        self.x_local = self.x_full[eng.rank * m_local:(eng.rank + 1) * m_local]
        self.ready = eng.symmetric_tensor((rows_total // 128,), torch.int32)     # peers bump these counters
        self.ready.zero_()
        torch.cuda.synchronize()
        eng.barrier()
        self.epoch = 0
        self.n_copy = n_copy if eng.world > 1 else 0
        self.ctas = ctas or C.sm_count()
        self.flag_lane = flag_lane

    def __call__(self, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 w_t: bool = False) -> torch.Tensor:
        """``w`` is [N, K]; with ``w_t`` it is stored [K, N] and consumed transposed (no copy)."""
        n = w.shape[1] if w_t else w.shape[0]
        if w.dtype != torch.bfloat16 or w.shape[0 if w_t else 1] != self.K or w.stride(1) != 1:
            raise ValueError("AllGatherGemm: w must be bf16 [N, K] (or [K, N] with w_t)")
        if out is None:
            out = torch.empty((self.M, n), dtype=torch.bfloat16, device="cuda")
        self.epoch += 1
        C.ag_gemm(self.eng.raw, self.eng.heap_offset(self.x_full), self.M, n, self.K, w.data_ptr(), w.stride(0), out.data_ptr(),
                  out.stride(0), bias.data_ptr() if bias is not None else 0, self.eng.heap_offset(self.ready), self.epoch, self.n_copy,
                  self.ctas, self.flag_lane, status_words().data_ptr(), torch.cuda.current_stream().cuda_stream, w_t)
        count_launch()
        return out


class GemmReduceScatter:
    """``out[rows of this rank] = sum over ranks of (y @ w^T)[those rows]`` for y [M, K] and w [N, K] local."""

    def __init__(self, eng: Engine, rows_total: int, n: int, ctas: Optional[int] = None):
        if rows_total % (128 * eng.world) or n % 256:
            raise ValueError("GemmReduceScatter: rows per rank must be a multiple of 128 and N a multiple of 256")
        self.eng, self.M, self.N = eng, rows_total, n
        m_local = rows_total // eng.world
        self.stage = eng.symmetric_tensor((eng.world, m_local, n), torch.bfloat16)
        self.flags = eng.symmetric_tensor((eng.world, (m_local // 128) * (n // 256)), torch.int64)
        self.flags.zero_()
        torch.cuda.synchronize()
        eng.barrier()
        self.epoch = 0
        self.ctas = ctas or C.sm_count()

    def __call__(self, y: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, w_t: bool = False) -> torch.Tensor:
        """``w`` is [N, K]; with ``w_t`` it is stored [K, N] and consumed transposed (no copy)."""
        wn, wk = (w.shape[1], w.shape[0]) if w_t else (w.shape[0], w.shape[1])
        if y.shape[0] != self.M or wn != self.N or y.shape[1] != wk:
            raise ValueError("GemmReduceScatter: shape mismatch")
        if out is None:
            out = torch.empty((self.M // self.eng.world, self.N), dtype=torch.bfloat16, device="cuda")
        self.epoch += 1
        C.gemm_rs(self.eng.raw, y.data_ptr(), y.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), self.M, self.N,
                  y.shape[1], self.eng.heap_offset(self.stage), self.eng.heap_offset(self.flags), self.epoch, self.ctas,
                  status_words().data_ptr(), torch.cuda.current_stream().cuda_stream, w_t)
        count_launch()
        return out


class AllGatherGemmFp8:
    """Block-scaled fp8 form of ``AllGatherGemm``: the rank's activations are quantised (e4m3, one fp32 scale
    per row and 128 values) straight into the symmetric gathered buffers, the kernel moves bytes and scales
    to the peers, and the weight shard comes as e4m3 with 128 x 128 scales (``ops.gemm.quant_blocks``).
    With ``quant_out`` the result (after bias / GELU) is returned quantised the same way, ready for the
    second GEMM of the layer."""

    def __init__(self, eng: Engine, rows_total: int, k: int, n_copy: int = 8, ctas: Optional[int] = None, flag_lane: int = 4,
                 mx: bool = False):
        """``mx``: power-of-two scale bytes (UE8M0) applied by the tensor core (``ops.gemm.quant_blocks_mx`` weights,
        224-column tiles, bf16 output only) instead of fp32 scales applied by promotion."""
        if rows_total % (128 * eng.world) or k % 128:
            raise ValueError("AllGatherGemmFp8: rows per rank must be a multiple of 128 and K a multiple of 128")
        self.eng, self.M, self.K, self.mx = eng, rows_total, k, mx
        self.xq_full = eng.symmetric_tensor((rows_total, k), torch.uint8)
        self.xs_full = eng.symmetric_tensor((rows_total, k // 128), torch.uint8 if mx else torch.float32)
        m_local = rows_total // eng.world
        self.m_local = m_local
        self.xq_local = self.xq_full[eng.rank * m_local:(eng.rank + 1) * m_local]
        self.xs_local = self.xs_full[eng.rank * m_local:(eng.rank + 1) * m_local]
        self.ready = eng.symmetric_tensor((rows_total // 128,), torch.int32)
        self.ready.zero_()
        torch.cuda.synchronize()
        eng.barrier()
        self.epoch = 0
        self.n_copy = n_copy if eng.world > 1 else 0
        self.ctas = ctas or C.sm_count()
        self.flag_lane = flag_lane

    def quantize_local(self, x: torch.Tensor) -> None:
        """bf16 [M/world, K] -> this rank's rows of the gathered fp8 buffer and its scales (one kernel)."""
        if x.shape != (self.m_local, self.K) or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("AllGatherGemmFp8.quantize_local: contiguous bf16 [M/world, K]")
        quant = C.quant_mx8_rows if self.mx else C.quant_fp8_rows
        quant(x.data_ptr(), self.xq_local.data_ptr(), self.xs_local.data_ptr(), self.m_local, self.K,
              torch.cuda.current_stream().cuda_stream)
        count_launch()

    def __call__(self, wq: torch.Tensor, ws: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
                 quant_out: bool = False, out=None):
        n = wq.shape[0]
        if wq.element_size() != 1 or wq.shape[1] != self.K or n % (128 if self.mx else 256) or ws.shape != (n // 128, self.K // 128):
            raise ValueError("AllGatherGemmFp8: wq e4m3 [N, K] with N % 256 == 0 (128 with mx) and ws [N/128, K/128]")
        if ws.dtype != (torch.uint8 if self.mx else torch.float32) or (self.mx and (quant_out or gelu)):
            raise ValueError("AllGatherGemmFp8: scales must be fp32 (uint8 with mx); mx has the plain bf16 epilogue only")
        d, dq, ds, ldd, ldq = [], [], [], 0, 0
        if quant_out:
            q = torch.empty((self.M, n), dtype=torch.uint8, device="cuda") if out is None else out[0]
            s = torch.empty((self.M, n // 128), dtype=torch.float32, device="cuda") if out is None else out[1]
            dq, ds, ldq, result = [q.data_ptr()], [s.data_ptr()], q.stride(0), (q, s)
        else:
            o = torch.empty((self.M, n), dtype=torch.bfloat16, device="cuda") if out is None else out
            d, ldd, result = [o.data_ptr()], o.stride(0), o
        self.epoch += 1
        C.ag_gemm_fp8(self.eng.raw, [], 0, self.eng.heap_offset(self.xq_full), self.eng.heap_offset(self.xs_full), self.M, n, self.K,
                      [wq.data_ptr()], wq.stride(0), [ws.data_ptr()], ws.stride(0), d, ldd, dq, ds, ldq,
                      bias.data_ptr() if bias is not None else 0, C.GEMM_GELU_INPLACE if gelu else 0, self.eng.heap_offset(self.ready),
                      self.epoch, self.n_copy, self.ctas, self.flag_lane, [status_words().data_ptr()], 0,
                      torch.cuda.current_stream().cuda_stream, self.mx)
        count_launch()
        return result


class GemmReduceScatterFp8:
    """Block-scaled fp8 form of ``GemmReduceScatter``: y is e4m3 [M, K] with 1 x 128 scales, w e4m3 [N, K] with
    128 x 128 scales; the partial tiles cross NVLink in bf16 and are folded in fp32 by their owner."""

    def __init__(self, eng: Engine, rows_total: int, n: int, ctas: Optional[int] = None):
        if rows_total % (128 * eng.world) or n % 256:
            raise ValueError("GemmReduceScatterFp8: rows per rank must be a multiple of 128 and N a multiple of 256")
        self.eng, self.M, self.N = eng, rows_total, n
        m_local = rows_total // eng.world
        self.stage = eng.symmetric_tensor((eng.world, m_local, n), torch.bfloat16)
        self.flags = eng.symmetric_tensor((eng.world, (m_local // 128) * (n // 256)), torch.int64)
        self.flags.zero_()
        torch.cuda.synchronize()
        eng.barrier()
        self.epoch = 0
        self.ctas = ctas or C.sm_count()

    def __call__(self, yq: torch.Tensor, ys: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        k = yq.shape[1]
        if yq.shape[0] != self.M or wq.shape != (self.N, k) or k % 128 or ys.shape != (self.M, k // 128) or ws.shape != (self.N // 128, k // 128):
            raise ValueError("GemmReduceScatterFp8: shape mismatch")
        if out is None:
            out = torch.empty((self.M // self.eng.world, self.N), dtype=torch.bfloat16, device="cuda")
        self.epoch += 1
        C.gemm_rs_fp8(self.eng.raw, [], [yq.data_ptr()], yq.stride(0), [ys.data_ptr()], ys.stride(0), [wq.data_ptr()], wq.stride(0),
                      [ws.data_ptr()], ws.stride(0), [out.data_ptr()], out.stride(0), self.M, self.N, k,
                      self.eng.heap_offset(self.stage), self.eng.heap_offset(self.flags), self.epoch, self.ctas,
                      [status_words().data_ptr()], 0, torch.cuda.current_stream().cuda_stream)
        count_launch()
        return out
