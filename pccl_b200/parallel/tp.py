"""Tensor parallelism with sequence-parallel activations (Megatron's g / g-bar pair), every
collective fused into its GEMM kernel:

    forward   x_local --[all-gather -> GEMM]--> h = gelu(.) --[GEMM -> reduce-scatter]--> z_local
    backward  dz_local --[all-gather -> GEMM]--> dh ... --[GEMM -> reduce-scatter]--> dx_local

``ColumnParallelLinear`` holds W1[d_ff / TP, d_model], ``RowParallelLinear`` W2[d_model, d_ff / TP];
tokens (rows) are sharded over the ranks between the layers.  The backward GEMMs consume the weights
in transposed form through the kernels' MN-major operand path; weight gradients are local GEMMs on
the gathered activations that the forward kernels leave behind.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..engine import Engine
from ..ops.fused_tp import AllGatherGemm, GemmReduceScatter
from ..ops.gemm import gemm


class _ColumnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, bias, layer):
        layer.ag.x_local.copy_(x_local)
        y = layer.ag(weight, bias)
        ctx.layer = layer
        ctx.save_for_backward(weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        (weight,) = ctx.saved_tensors
        layer = ctx.layer
        dy = dy.contiguous()
        # dx_local = reduce_scatter_rows(dy @ W): W is [N1, K] = the [K_gemm, N_gemm] form -> w_t
        dx = layer.rs_bwd(dy, weight, w_t=True)
        dw = gemm(dy, layer.ag.x_full, a_t=True, b_t=True)            # [N1, K]
        db = dy.sum(0, dtype=torch.float32).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db, None


class _RowFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, layer):
        z = layer.rs(h, weight)
        ctx.layer = layer
        ctx.save_for_backward(h, weight)
        return z

    @staticmethod
    def backward(ctx, dz_local):
        h, weight = ctx.saved_tensors
        layer = ctx.layer
        layer.ag_bwd.x_local.copy_(dz_local)
        dh = layer.ag_bwd(weight, w_t=True)                           # all_gather(dz) @ W2, W2 is [D, N1]
        dw = gemm(layer.ag_bwd.x_full, h, a_t=True, b_t=True)         # [D, N1]
        return dh, dw, None


class ColumnParallelLinear(nn.Module):
    """y[tokens, out/TP] = all_gather_rows(x_local) @ W^T + b."""

    def __init__(self, eng: Engine, tokens: int, in_features: int, out_features: int, bias: bool = True, n_copy: int = 12,
                 init_std: float = 0.02):
        super().__init__()
        if out_features % eng.world:
            raise ValueError("ColumnParallelLinear: out_features must divide over the ranks")
        self.eng, self.tokens = eng, tokens
        n_local = out_features // eng.world
        self.weight = nn.Parameter(torch.empty((n_local, in_features), device="cuda", dtype=torch.bfloat16))
        nn.init.normal_(self.weight, std=init_std)
        self.bias = nn.Parameter(torch.zeros(n_local, device="cuda", dtype=torch.bfloat16)) if bias else None
        self.ag = AllGatherGemm(eng, tokens, in_features, n_copy=n_copy, flag_lane=4)
        self.rs_bwd = GemmReduceScatter(eng, tokens, in_features)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        return _ColumnFn.apply(x_local, self.weight, self.bias, self)


class RowParallelLinear(nn.Module):
    """z_local[tokens/TP, out] = reduce_scatter_rows(h @ W^T)  (+ b on every rank's rows)."""

    def __init__(self, eng: Engine, tokens: int, in_features: int, out_features: int, bias: bool = True, n_copy: int = 12,
                 init_std: float = 0.02):
        super().__init__()
        if in_features % eng.world:
            raise ValueError("RowParallelLinear: in_features must divide over the ranks")
        self.eng, self.tokens = eng, tokens
        k_local = in_features // eng.world
        self.weight = nn.Parameter(torch.empty((out_features, k_local), device="cuda", dtype=torch.bfloat16))
        nn.init.normal_(self.weight, std=init_std)
        self.bias = nn.Parameter(torch.zeros(out_features, device="cuda", dtype=torch.bfloat16)) if bias else None
        self.rs = GemmReduceScatter(eng, tokens, out_features)
        self.ag_bwd = AllGatherGemm(eng, tokens, out_features, n_copy=n_copy, flag_lane=6)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        z = _RowFn.apply(h, self.weight, self)
        return z if self.bias is None else z + self.bias


class TensorParallelMLP(nn.Module):
    """x_local -> ColumnParallel -> GELU -> RowParallel -> z_local, rows sharded outside, d_ff sharded inside."""

    def __init__(self, eng: Engine, tokens: int, d_model: int, d_ff: int, n_copy: int = 12):
        super().__init__()
        self.fc1 = ColumnParallelLinear(eng, tokens, d_model, d_ff, n_copy=n_copy)
        self.fc2 = RowParallelLinear(eng, tokens, d_ff, d_model, n_copy=n_copy)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        return self.fc2(torch.nn.functional.gelu(self.fc1(x_local), approximate="tanh"))
