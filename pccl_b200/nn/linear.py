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

from ..ops.elementwise import colsum
from ..ops.gemm import gemm, gemm_dgelu, gemm_dual


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


def _weight_grad_pair(dy_a: torch.Tensor, x_a: torch.Tensor, w_a: torch.Tensor, dy_b: torch.Tensor, x_b: torch.Tensor, w_b: torch.Tensor):
    """The weight gradients of two layers over the same rows as one launch (``gemm_dual``)."""
    mg_a, mg_b = _grad_target(w_a), _grad_target(w_b)
    if (mg_a is None) != (mg_b is None) or dy_a.shape[0] != dy_b.shape[0] or (mg_a is not None and mg_a.dtype != mg_b.dtype):
        return _weight_grad(dy_a, x_a, w_a), _weight_grad(dy_b, x_b, w_b)
    if mg_a is None:
        ga = torch.empty((dy_a.shape[1], x_a.shape[1]), dtype=torch.bfloat16, device=dy_a.device)
        gb = torch.empty((dy_b.shape[1], x_b.shape[1]), dtype=torch.bfloat16, device=dy_b.device)
        gemm_dual(dy_a, x_a, ga, dy_b, x_b, gb, a_t=True, b_t=True)
        return ga, gb
    gemm_dual(dy_a, x_a, mg_a, dy_b, x_b, mg_b, a_t=True, b_t=True, accumulate0=bool(getattr(w_a, "_pccl_written", False)),
              accumulate1=bool(getattr(w_b, "_pccl_written", False)))
    _finish_main_grad(w_a)
    _finish_main_grad(w_b)
    return None, None


def _bias_grad(dy2: torch.Tensor, bias: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if bias is None:
        return None
    if dy2.shape[1] % 8 == 0 and dy2.is_cuda:
        db = colsum(dy2)
    else:
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
    """y = x W^T + b (+ residual).  ``defer_bias_grad``: the bias gradient is produced elsewhere (by the fused
    residual-add + LayerNorm that consumes y, which sums the same rows anyway), so backward skips it."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual=None, defer_bias_grad=False):
        x2 = _as_operand(x)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, weight.shape[0])
        y = gemm(x2, weight, bias=bias, residual=res2)
        ctx.save_for_backward(x2, weight, bias)
        ctx.x_shape = x.shape
        ctx.defer_bias_grad = defer_bias_grad
        ctx.has_residual = residual is not None
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, bias = ctx.saved_tensors
        dy2 = _as_operand(dy)
        dx = gemm(dy2, weight, b_t=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dy2, x2, weight)
        db = None if ctx.defer_bias_grad else _bias_grad(dy2, bias)
        return dx, dw, db, (dy if ctx.has_residual else None), None


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


class _MlpFn(torch.autograd.Function):
    """out = gelu_tanh(x W1^T + b1) W2^T + b2 as one autograd node, so that backward can fuse across the two layers:
    the GEMM that turns the output gradient into the activation gradient applies gelu' in its epilogue and sums the
    columns of its result (the first bias gradient) on the way out -- no GELU-backward kernel, no separate reduction,
    and the activation gradient never visits memory."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, defer_b2_grad=False):
        x2 = _as_operand(x)
        act = torch.empty((x2.shape[0], w1.shape[0]), dtype=torch.bfloat16, device=x.device)
        pre = gemm(x2, w1, bias=b1, gelu_out=act)
        out = gemm(act, w2, bias=b2)
        ctx.save_for_backward(x2, w1, b1, w2, b2, pre, act)
        ctx.x_shape = x.shape
        ctx.defer_b2_grad = defer_b2_grad
        return out.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dz):
        x2, w1, b1, w2, b2, pre, act = ctx.saved_tensors
        dz2 = _as_operand(dz)
        rows, n1 = pre.shape
        if rows % 256 == 0 and n1 % 256 == 0:
            sums = torch.zeros(n1, dtype=torch.float32, device=pre.device) if b1 is not None else None
            dy2 = gemm_dgelu(dz2, w2, pre, b_t=True, colsum=sums)
            db1 = _deliver_bias(b1, sums.to(b1.dtype)) if b1 is not None else None
        else:
            dact = gemm(dz2, w2, b_t=True)
            dy2 = torch.ops.aten.gelu_backward(dact, pre, approximate="tanh")
            db1 = _bias_grad(dy2, b1)
        db2 = None if ctx.defer_b2_grad else _bias_grad(dz2, b2)
        dx = gemm(dy2, w1, b_t=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw1, dw2 = _weight_grad_pair(dy2, x2, w1, dz2, act, w2)          # both weight gradients in one launch
        return dx, dw1, db1, dw2, db2, None


def _deliver_bias(bias: torch.Tensor, db: torch.Tensor) -> Optional[torch.Tensor]:
    mg = _grad_target(bias)
    if mg is None:
        return db
    if getattr(bias, "_pccl_written", False):
        mg.add_(db)
    else:
        mg.copy_(db)
    _finish_main_grad(bias)
    return None


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

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, defer_bias_grad: bool = False) -> torch.Tensor:
        """``residual`` is added in the GEMM epilogue.  ``defer_bias_grad=True`` promises that the consumer of the output
        (``LayerNorm.add_norm(..., prev_bias=self.bias)``) produces this layer's bias gradient."""
        return _LinearFn.apply(x, self.weight, self.bias, residual, defer_bias_grad)


def mlp(x: torch.Tensor, fc1: "Linear", fc2: "Linear", defer_fc2_bias_grad: bool = False) -> torch.Tensor:
    """``fc2(gelu_tanh(fc1(x)))`` with the two layers' backward passes fused (see ``_MlpFn``)."""
    return _MlpFn.apply(x, fc1.weight, fc1.bias, fc2.weight, fc2.bias, defer_fc2_bias_grad)


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
