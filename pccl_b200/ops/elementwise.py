"""Memory-bound training kernels (csrc/kernels/elementwise.cu): fused AdamW, fused cross-entropy."""
from __future__ import annotations

import torch

from .._native import C
from .gemm import count_launch, status_words


def adamw_step(master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, grad: torch.Tensor,
               param_bf16: torch.Tensor, *, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
               step: int = 1, grad_scale: float = 1.0, stream=None) -> None:
    """One AdamW step on flat fp32 tensors; the new parameters are also written to ``param_bf16``."""
    n = master.numel()
    for t in (master, exp_avg, exp_avg_sq, grad):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise ValueError("adamw_step: fp32 contiguous tensors of one length expected")
    if param_bf16.dtype != torch.bfloat16 or param_bf16.numel() != n or not param_bf16.is_contiguous():
        raise ValueError("adamw_step: param_bf16 must be a contiguous bf16 tensor of the same length")
    s = (stream or torch.cuda.current_stream()).cuda_stream
    C.adamw(master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad.data_ptr(), param_bf16.data_ptr(), n,
            lr, betas[0], betas[1], eps, weight_decay, step, grad_scale, s)
    count_launch()


def cross_entropy_(logits: torch.Tensor, targets: torch.Tensor, *, grad_scale: float = 1.0,
                   ignore_index: int = -100) -> torch.Tensor:
    """Per-row losses of ``logits`` (bf16 [rows, vocab], row stride a multiple of 8); the logits are
    replaced in place by ``(softmax - onehot) * grad_scale``.  Targets must lie in [0, vocab) or equal
    ``ignore_index``; any other value yields an ignored row (loss 0, zero gradient) and sets the device status
    words, so the next ``check_status`` raises."""
    if logits.dtype != torch.bfloat16 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("cross_entropy_: bf16 [rows, vocab] logits with unit inner stride expected")
    rows, vocab = logits.shape
    targets = targets.reshape(-1)
    if targets.dtype != torch.int64 or targets.numel() != rows:
        raise ValueError("cross_entropy_: int64 targets, one per row")
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    C.cross_entropy(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), rows, vocab, logits.stride(0), grad_scale,
                    ignore_index, status_words(logits.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch()
    return loss


def colsum(x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Column sums (fp32 accumulation) of a bf16 matrix [rows, N] with unit inner stride, as bf16 [N]: the bias gradient of
    a linear layer.  Two short kernels (partial rows, then their sum) that run near memory bandwidth."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1 or x.stride(0) % 8 or x.shape[1] % 8 or x.data_ptr() % 16:
        raise ValueError("colsum: bf16 [rows, N] with unit inner stride, N and the row stride multiples of 8, 16-byte aligned")
    rows, n = x.shape
    if out is None:
        out = torch.empty(n, dtype=torch.bfloat16, device=x.device)
    partials = torch.empty(C.colsum_parts(rows) * n, dtype=torch.float32, device=x.device)
    C.colsum(x.data_ptr(), x.stride(0), rows, n, out.data_ptr(), partials.data_ptr(), torch.cuda.current_stream().cuda_stream)
    count_launch(2)
    return out
