"""Expert parallelism: a mixture-of-experts feed-forward layer whose token exchange runs on this
library's dispatch / combine kernels (fp8 payload with per-128 scales out, gate-weighted bf16 back)
and whose experts run as one grouped tcgen05 GEMM per projection.  Forward only in this version: the
layer is built for serving and for measuring the exchange; its gradient path is not written yet."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..engine import Engine
from ..ops.moe import MoEExchange


class MoELayer(nn.Module):
    def __init__(self, eng: Engine, tokens: int, d_model: int, d_ff: int, n_experts: int, topk: int = 8,
                 capacity_factor: float = 2.0, init_std: float = 0.02):
        super().__init__()
        self.eng, self.topk = eng, topk
        epr = n_experts // eng.world
        self.gate = nn.Parameter(torch.randn(n_experts, d_model, device="cuda", dtype=torch.bfloat16) * init_std)
        self.w1 = nn.Parameter(torch.randn(epr * d_ff, d_model, device="cuda", dtype=torch.bfloat16) * init_std)
        self.w2 = nn.Parameter(torch.randn(epr * d_model, d_ff, device="cuda", dtype=torch.bfloat16) * init_std)
        self.exchange = MoEExchange(eng, tokens, d_model, n_experts, topk, capacity_factor)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, gate_logits: torch.Tensor = None) -> torch.Tensor:
        if gate_logits is None:
            gate_logits = (x @ self.gate.t()).float()
        return self.exchange.forward(x, gate_logits, self.w1, self.w2)
