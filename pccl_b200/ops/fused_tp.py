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


class AllGatherGemm:
    """Rows of X are sharded over the ranks.  Write this rank's rows into ``self.x_local`` (a view of
    the symmetric gathered buffer), then ``out = self(w)``; afterwards ``self.x_full`` holds all rows
    (the backward pass of a column-parallel layer needs them for the weight gradient)."""

    def __init__(self, eng: Engine, rows_total: int, k: int, n_copy: int = 16, ctas: Optional[int] = None, flag_lane: int = 4):
        if rows_total % (128 * eng.world) or k % 8:
            raise ValueError("AllGatherGemm: rows per rank must be a multiple of 128 and K a multiple of 8")
        self.eng, self.M, self.K = eng, rows_total, k
        self.x_full = eng.symmetric_tensor((rows_total, k), torch.bfloat16)
        m_local = rows_total // eng.world
        self.x_local = self.x_full[eng.rank * m_local:(eng.rank + 1) * m_local]
        self.ready = eng.symmetric_tensor((rows_total // 128,), torch.int32)     # peers bump these counters
        self.ready.zero_()
        torch.cuda.synchronize()
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
