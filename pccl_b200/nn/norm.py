"""LayerNorm on this package's kernels (csrc/kernels/layernorm.cu): bf16 activations, fp32 statistics,
one pass over the activations per direction.  ``add_layer_norm`` is the residual connection of a pre-norm
transformer block and the norm that follows it as one kernel per direction."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .._native import C
from ..ops.gemm import count_launch


def _deliver(param: Optional[torch.Tensor], grad: torch.Tensor):
    """Hands a parameter's gradient to the data-parallel wrapper's flat bucket when there is one (and returns None),
    else returns it for autograd to accumulate."""
    if param is None:
        return None
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return grad
    if getattr(param, "_pccl_written", False):
        mg.add_(grad.to(mg.dtype).view_as(mg))
    else:
        mg.copy_(grad.view_as(mg))
    param._pccl_written = True
    cb = getattr(param, "_pccl_ready", None)
    if cb is not None:
        cb()
    return None


def _ln_forward(x2, delta2, weight, bias, eps):
    rows, D = x2.shape
    y = torch.empty_like(x2)
    s = torch.empty_like(x2) if delta2 is not None else None
    mean = torch.empty(rows, dtype=torch.float32, device=x2.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    C.layernorm_fwd(x2.data_ptr(), delta2.data_ptr() if delta2 is not None else 0, s.data_ptr() if s is not None else 0,
                    weight.data_ptr(), bias.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, D, eps,
                    torch.cuda.current_stream().cuda_stream)
    count_launch()
    return s, y, mean, rstd


def _ln_backward(dy2, x2, weight, mean, rstd, dres2, want_colsum):
    rows, D = x2.shape
    dx = torch.empty_like(x2)
    dg = torch.empty_like(weight)
    db = torch.empty_like(weight)
    dc = torch.empty_like(weight) if want_colsum else None
    partials = torch.empty(3 * C.layernorm_bwd_parts(rows) * D, dtype=torch.float32, device=x2.device)
    C.layernorm_bwd(dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                    dres2.data_ptr() if dres2 is not None else 0, dx.data_ptr(), dg.data_ptr(), db.data_ptr(),
                    dc.data_ptr() if dc is not None else 0, partials.data_ptr(), rows, D, torch.cuda.current_stream().cuda_stream)
    count_launch(2)
    return dx, dg, db, dc


def _rows(t: torch.Tensor, D: int) -> torch.Tensor:
    t2 = t.reshape(-1, D)
    return t2 if t2.is_contiguous() else t2.contiguous()


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x2 = _rows(x, x.shape[-1])
        _, y, mean, rstd = _ln_forward(x2, None, weight, bias, eps)
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        dx, dg, db, _ = _ln_backward(_rows(dy, x2.shape[1]), x2, weight, mean, rstd, None, False)
        return dx.view(ctx.shape), dg, db, None


class _AddLayerNormFn(torch.autograd.Function):
    """(x, delta) -> (s, y) with s = x + delta and y = LayerNorm(s).  ``prev_bias`` is the bias of the linear layer that
    produced ``delta`` (or None): the gradient of ``delta`` summed over rows is that bias's gradient, and backward computes
    it while it has the rows in registers, so that layer does not make a pass of its own for it."""

    @staticmethod
    def forward(ctx, x, delta, weight, bias, prev_bias, eps):
        D = x.shape[-1]
        x2, d2 = _rows(x, D), _rows(delta, D)
        s, y, mean, rstd = _ln_forward(x2, d2, weight, bias, eps)
        ctx.save_for_backward(s, weight, mean, rstd)
        ctx.prev_bias = prev_bias
        ctx.shape = x.shape
        return s.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, ds, dy):
        s, weight, mean, rstd = ctx.saved_tensors
        D = s.shape[1]
        if dy is None:
            dy = torch.zeros_like(s)
        dres = _rows(ds, D) if ds is not None else None
        want = ctx.prev_bias is not None and ctx.needs_input_grad[4]
        dx, dg, db, dc = _ln_backward(_rows(dy, D), s, weight, mean, rstd, dres, want)
        dxv = dx.view(ctx.shape)
        return dxv, dxv, dg, db, (_deliver(ctx.prev_bias, dc) if want else None), None


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

    def add_norm(self, x: torch.Tensor, delta: torch.Tensor, prev_bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(x + delta, LayerNorm(x + delta))``.  Pass the bias of the linear layer that produced ``delta`` as
        ``prev_bias`` when that layer was told to leave its bias gradient to this norm (``Linear(..., defer_bias_grad=True)``)."""
        return _AddLayerNormFn.apply(x, delta, self.weight, self.bias, prev_bias, self.eps)
