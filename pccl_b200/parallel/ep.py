"""Expert parallelism: a mixture-of-experts feed-forward layer whose token exchange runs on this
library's dispatch / combine kernels (fp8 payload with per-128 scales out, gate-weighted bf16 back)
and whose experts run as one grouped tcgen05 GEMM per projection.

The layer trains: its backward pass reuses the same exchange.  The gradient of the output goes to the
experts' ranks through the dispatch kernel, weighted by the gate probability of each assignment (the
e4m3 payload of a row is the same for all of its destinations, only the block scales are multiplied);
the experts' input gradients come back through the combine kernel; the gradients of the gate weights
are dot products of the upstream gradient with the expert output rows, taken by a third kernel that
pulls the rows like the combine does.  The expert GEMMs of the backward pass are the grouped kernel
again (input gradients) and one tcgen05 GEMM per expert (weight gradients, whose reduction dimension
is the expert's row count).  The reference has no model code; this is the EP strategy it names.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..engine import Engine
from ..ops.gemm import gemm
from ..ops.moe import MoEExchange, grouped_gemm


class _MoEFn(torch.autograd.Function):
    """out[t] = sum_k p[t,k] * W2_e gelu(W1_e x[t]) over the top-k experts e of token t.  One forward per backward:
    the expert outputs stay in the exchange's symmetric buffer until the backward pass has read them."""

    @staticmethod
    def forward(ctx, x, gate_logits, w1, w2, ex: MoEExchange):
        ids, probs, plan = ex.route_and_plan(gate_logits)
        ex.dispatch(x, ids, plan)
        xr = ex.received(plan)                                   # what the experts see (after the e4m3 round trip)
        d_ff = w1.shape[0] // ex.epr
        h_pre = grouped_gemm(xr, w1, plan["row_off"], d_ff)
        h = F.gelu(h_pre, approximate="tanh")
        grouped_gemm(h, w2, plan["row_off"], ex.H, out=ex.y)
        out = ex.combine(ids, probs, plan)
        ctx.save_for_backward(gate_logits, w1, w2, ids, probs, plan["rows"], plan["row_off"], plan["n_rows"], xr, h_pre, h)
        ctx.ex = ex
        return out

    @staticmethod
    def backward(ctx, dout):
        gate_logits, w1, w2, ids, probs, rows, row_off, n_rows, xr, h_pre, h = ctx.saved_tensors
        ex = ctx.ex
        plan = {"rows": rows, "row_off": row_off, "n_rows": n_rows}
        epr, H = ex.epr, ex.H
        d_ff = w1.shape[0] // epr
        dout = dout.contiguous()
        # gate weights: d p[t,k] = <dout[t], expert output row>, while the forward outputs are still in ex.y
        dp = ex.combine_dot(dout, ids, plan)
        # output gradients to the experts, each weighted by its gate probability
        ex.dispatch(dout, ids, plan, probs=probs)
        g = ex.received(plan)
        # experts: input gradients with the grouped kernel (it multiplies by B^T, so the weights are laid out transposed)
        w2t = w2.view(epr, H, d_ff).transpose(1, 2).reshape(epr * d_ff, H).contiguous()
        dh = grouped_gemm(g, w2t, row_off, d_ff)
        dh_pre = torch.ops.aten.gelu_backward(dh, h_pre, approximate="tanh")
        w1t = w1.view(epr, d_ff, H).transpose(1, 2).reshape(epr * H, d_ff).contiguous()
        grouped_gemm(dh_pre, w1t, row_off, H, out=ex.y)
        # weight gradients: per expert, reduced over that expert's rows (the one place the host needs the row counts)
        offs = row_off.tolist()
        dw1 = torch.zeros_like(w1)
        dw2 = torch.zeros_like(w2)
        for e in range(epr):
            r0, r1 = offs[e], offs[e + 1]
            if r1 > r0:
                gemm(dh_pre[r0:r1], xr[r0:r1], a_t=True, b_t=True, out=dw1[e * d_ff:(e + 1) * d_ff])
                gemm(g[r0:r1], h[r0:r1], a_t=True, b_t=True, out=dw2[e * H:(e + 1) * H])
        # input gradients back to the tokens: a plain sum over the k assignments (the gate weight went out with dout)
        dx = ex.combine(ids, torch.ones_like(probs), plan)
        # softmax over all experts, top-k taken: chain rule through the softmax for the selected probabilities
        pf = torch.softmax(gate_logits.float(), dim=-1)
        dfull = torch.zeros_like(pf).scatter_(1, ids.long(), dp)
        dlogits = pf * (dfull - (dfull * pf).sum(-1, keepdim=True))
        return dx, dlogits.to(gate_logits.dtype), dw1, dw2, None


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

    def forward(self, x: torch.Tensor, gate_logits: torch.Tensor = None) -> torch.Tensor:
        """With gradients enabled the layer runs as an autograd node (see ``_MoEFn``); under ``torch.no_grad()`` it takes
        the serving path, which fuses the GELU into the first grouped GEMM and keeps nothing for a backward pass."""
        if gate_logits is None:
            gate_logits = (x @ self.gate.t()).float()
        if torch.is_grad_enabled() and (x.requires_grad or gate_logits.requires_grad or self.w1.requires_grad):
            return _MoEFn.apply(x, gate_logits, self.w1, self.w2, self.exchange)
        with torch.no_grad():
            return self.exchange.forward(x, gate_logits, self.w1, self.w2)
