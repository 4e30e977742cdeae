"""LayerNorm on this package's kernels (csrc/kernels/layernorm.cu): bf16 activations, fp32 statistics,
one pass over the activations per direction."""
from __future__ import annotations

import torch
import torch.nn as nn

from .._native import C
from ..ops.gemm import count_launch


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        C.layernorm_fwd(x2.data_ptr(), weight.data_ptr(), bias.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, D,
                        eps, torch.cuda.current_stream().cuda_stream)
        count_launch()
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        dg = torch.empty_like(weight)
        db = torch.empty_like(weight)
        partials = torch.empty(2 * C.layernorm_bwd_parts(rows) * D, dtype=torch.float32, device=x2.device)
        C.layernorm_bwd(dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                        dg.data_ptr(), db.data_ptr(), partials.data_ptr(), rows, D, torch.cuda.current_stream().cuda_stream)
        count_launch(2)
        return dx.view(ctx.shape), dg, db, None


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=torch.bfloat16):
        super().__init__()
        if dim % 8 or dim > 8192 or dtype != torch.bfloat16:
            raise ValueError("LayerNorm: bf16, dim % 8 == 0 and dim <= 8192")
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _LayerNormFn.apply(x, self.weight, self.bias, self.eps)
