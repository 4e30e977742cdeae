"""Cross-entropy whose forward also produces the logits' gradient, in place (one pass over HBM)."""
from __future__ import annotations

import torch

from ..ops.elementwise import cross_entropy_


class _FusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index, unit_grad):
        if ignore_index is None:
            scale, ign = 1.0 / targets.numel(), -(1 << 62)
        else:
            scale, ign = 1.0 / max(1, int((targets != ignore_index).sum())), int(ignore_index)
        # The kernel writes through the raw pointer: after it, `logits` holds d(mean loss)/d(logits).
        losses = cross_entropy_(logits.detach(), targets, grad_scale=scale, ignore_index=ign)
        ctx.save_for_backward(logits.detach())
        ctx.unit_grad = unit_grad
        return losses.sum() * scale

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        if ctx.unit_grad:
            return dlogits, None, None, None
        return dlogits * dloss.to(dlogits.dtype), None, None, None


def fused_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index=None,
                        unit_grad: bool = True) -> torch.Tensor:
    """Mean cross-entropy of bf16 ``logits`` [rows, vocab] (row stride a multiple of 8; a column
    slice of a padded buffer is fine).  ``logits`` is consumed: it is overwritten by its gradient.
    ``unit_grad=True`` states that the loss is differentiated with an upstream gradient of exactly 1
    (``loss.backward()``), which lets backward hand the stored gradient on without another pass; pass
    False when the loss is scaled or combined before ``backward``."""
    return _FusedCE.apply(logits, targets.reshape(-1), ignore_index, unit_grad)
