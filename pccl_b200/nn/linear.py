"""Linear layers whose three GEMMs (y = xW^T, dx = dy W, dW = dy^T x) run on the tcgen05 kernel.

The weight gradient is written by the GEMM epilogue straight into ``weight.main_grad`` when the
data-parallel wrapper has attached one (a view into a flat gradient bucket in the symmetric heap),
so the bucket is ready for its reduce-scatter the moment the GEMM retires; no ``.grad`` tensor, no
copy.  Operands are never transposed in memory: dx and dW use the kernel's MN-major operand forms.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops.gemm import gemm


def _as_operand(t: torch.Tensor) -> torch.Tensor:
    """2-D view usable as a GEMM operand: unit inner stride, row stride % 8 == 0, 16-byte aligned
    (a column slice of a padded buffer qualifies; anything else is made contiguous)."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def _grad_target(p: torch.Tensor):
    return getattr(p, "main_grad", None)


def _finish_main_grad(p: torch.Tensor) -> None:
    p._pccl_written = True
    cb = getattr(p, "_pccl_ready", None)
    if cb is not None:
        cb()


def _weight_grad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    mg = _grad_target(weight)
    if mg is None:
        return gemm(dy2, x2, a_t=True, b_t=True)
    gemm(dy2, x2, a_t=True, b_t=True, out=mg, accumulate=bool(getattr(weight, "_pccl_written", False)))
    _finish_main_grad(weight)
    return None


def _bias_grad(dy2: torch.Tensor, bias: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if bias is None:
        return None
    db = dy2.sum(0, dtype=torch.float32).to(bias.dtype)
    mg = _grad_target(bias)
    if mg is None:
        return db
    if getattr(bias, "_pccl_written", False):
        mg.add_(db)
    else:
        mg.copy_(db)
    _finish_main_grad(bias)
    return None


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = _as_operand(x)
        y = gemm(x2, weight, bias=bias)
        ctx.save_for_backward(x2, weight, bias)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, bias = ctx.saved_tensors
        dy2 = _as_operand(dy)
        dx = gemm(dy2, weight, b_t=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dy2, x2, weight)
        db = _bias_grad(dy2, bias)
        return dx, dw, db


class _LinearGeluFn(torch.autograd.Function):
    """act = gelu_tanh(x W^T + b); the activation is produced by the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = _as_operand(x)
        act = torch.empty((x2.shape[0], weight.shape[0]), dtype=torch.bfloat16, device=x.device)
        pre = gemm(x2, weight, bias=bias, gelu_out=act)
        ctx.save_for_backward(x2, weight, bias, pre)
        ctx.x_shape = x.shape
        return act.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dact):
        x2, weight, bias, pre = ctx.saved_tensors
        dact2 = dact.reshape(-1, dact.shape[-1])
        dy2 = torch.ops.aten.gelu_backward(dact2, pre, approximate="tanh")
        dx = gemm(dy2, weight, b_t=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dy2, x2, weight)
        db = _bias_grad(dy2, bias)
        return dx, dw, db


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=torch.bfloat16,
                 init_std: float = 0.02):
        super().__init__()
        if in_features % 8 or dtype != torch.bfloat16:
            raise ValueError("Linear: bf16 and in_features % 8 == 0 required by the TMA descriptors")
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty((out_features, in_features), device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _LinearFn.apply(x, self.weight, self.bias)


class LinearGelu(Linear):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _LinearGeluFn.apply(x, self.weight, self.bias)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids, weight)
        return weight[ids]

    @staticmethod
    def backward(ctx, dy):
        ids, weight = ctx.saved_tensors
        mg = _grad_target(weight)
        flat_ids, flat_dy = ids.reshape(-1), dy.reshape(-1, dy.shape[-1])
        if mg is None:
            g = torch.zeros_like(weight)
            g.index_add_(0, flat_ids, flat_dy.to(weight.dtype))
            return None, g
        if not getattr(weight, "_pccl_written", False):
            mg.zero_()
        mg.index_add_(0, flat_ids, flat_dy.to(mg.dtype))
        _finish_main_grad(weight)
        return None, None


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, dim: int, device=None, dtype=torch.bfloat16, init_std: float = 0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty((num_embeddings, dim), device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return _EmbeddingFn.apply(ids, self.weight)
