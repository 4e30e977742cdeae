"""GPT-style decoder whose linear layers, loss and optimizer run on this package's sm_100a kernels.

The reference has no model at all; this is the data-parallel training workload the framework is
measured on (24 layers, d=2048, 16 heads, sequence 2048, vocabulary 50257 gives 1.3 B parameters).
Attention itself uses PyTorch's fused scaled-dot-product attention; every GEMM (QKV, projection,
MLP, LM head, and their input/weight gradients), the GELU epilogue, the cross-entropy and AdamW are
this package's kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.linear import Embedding, Linear, LinearGelu, _LinearFn, mlp
from ..nn.loss import fused_cross_entropy
from ..nn.norm import LayerNorm


@dataclass
class GPTConfig:
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 2048
    seq_len: int = 2048
    vocab_size: int = 50257
    mlp_ratio: int = 4
    tie_embeddings: bool = True
    # Residual adds inside the LayerNorm kernels, the MLP as one autograd node (GELU backward and bias gradients in
    # GEMM epilogues), bias gradients of proj / fc2 as a by-product of the next norm's backward.  False keeps every
    # layer a separate node with element-wise PyTorch kernels between them (for comparison and debugging).
    fuse_blocks: bool = True

    @staticmethod
    def gpt_1p3b() -> "GPTConfig":
        return GPTConfig()

    @staticmethod
    def tiny() -> "GPTConfig":
        return GPTConfig(n_layer=2, n_head=4, d_model=256, seq_len=128, vocab_size=1001)

    def num_params(self) -> int:
        d = self.d_model
        per_layer = 4 * d * d + 4 * d + 2 * self.mlp_ratio * d * d + (self.mlp_ratio + 1) * d + 4 * d
        emb = self.vocab_size * d + self.seq_len * d
        return self.n_layer * per_layer + emb + 2 * d + (0 if self.tie_embeddings else self.vocab_size * d)

    def flops_per_token(self) -> float:
        """Training FLOPs per token: 6 x (non-embedding + LM-head parameters) + attention."""
        d = self.d_model
        dense = self.n_layer * (4 * d * d + 2 * self.mlp_ratio * d * d) + self.vocab_size * d
        attn = self.n_layer * 2 * self.seq_len * d      # QK^T and PV, causal counted in full as usual
        return 6.0 * dense + 6.0 * attn


class Block(nn.Module):
    def __init__(self, cfg: GPTConfig, device=None):
        super().__init__()
        d = cfg.d_model
        self.n_head = cfg.n_head
        self.fuse = cfg.fuse_blocks
        self.ln1 = LayerNorm(d, device=device)
        self.qkv = Linear(d, 3 * d, device=device)
        self.proj = Linear(d, d, device=device, init_std=0.02 / math.sqrt(2 * cfg.n_layer))
        self.ln2 = LayerNorm(d, device=device)
        self.fc1 = LinearGelu(d, cfg.mlp_ratio * d, device=device)
        self.fc2 = Linear(cfg.mlp_ratio * d, d, device=device, init_std=0.02 / math.sqrt(2 * cfg.n_layer))

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], prev_bias: Optional[torch.Tensor]):
        """The residual stream travels as ``(x, delta)``: the sum is formed inside the LayerNorm kernel that needs it.
        Returns the block's own ``(x, delta, bias of the layer that made delta)`` for the next norm to finish."""
        B, T, D = x.shape
        if not self.fuse:
            qkv = self.qkv(self.ln1(x)).view(B, T, 3, self.n_head, D // self.n_head)
            q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.proj(a.transpose(1, 2).reshape(B, T, D))
            return x + self.fc2(self.fc1(self.ln2(x))), None, None
        if delta is None:
            h = self.ln1(x)
        else:
            x, h = self.ln1.add_norm(x, delta, prev_bias)
        qkv = self.qkv(h).view(B, T, 3, self.n_head, D // self.n_head)
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))    # unbind: one stacked gradient, no zero-fills
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        d_attn = self.proj(a.transpose(1, 2).reshape(B, T, D), defer_bias_grad=True)
        x, h = self.ln2.add_norm(x, d_attn, self.proj.bias)
        return x, mlp(h, self.fc1, self.fc2, defer_fc2_bias_grad=True), self.fc2.bias


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.wte = Embedding(cfg.vocab_size, cfg.d_model, device=device)
        self.wpe = Embedding(cfg.seq_len, cfg.d_model, device=device)
        self.blocks = nn.ModuleList(Block(cfg, device) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.d_model, device=device)
        if cfg.tie_embeddings:
            self.wte.weight._pccl_uses = 2     # gradient arrives from the LM head and from the lookup
        else:
            self.lm_head = Linear(cfg.d_model, cfg.vocab_size, bias=False, device=device)

    def logits(self, ids: torch.Tensor) -> torch.Tensor:
        B, T = ids.shape
        pos = torch.arange(T, device=ids.device)
        x = self.wte(ids) + self.wpe(pos)[None]
        delta, prev_bias = None, None
        for blk in self.blocks:
            x, delta, prev_bias = blk(x, delta, prev_bias)
        x = self.ln_f(x) if delta is None else self.ln_f.add_norm(x, delta, prev_bias)[1]
        w = self.wte.weight if self.cfg.tie_embeddings else self.lm_head.weight
        return _LinearFn.apply(x, w, None)          # [B, T, vocab]; rows padded to a multiple of 8

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None):
        lg = self.logits(ids)
        if targets is None:
            return lg
        return fused_cross_entropy(lg.view(-1, lg.shape[-1]), targets.reshape(-1))


def smoke_step() -> float:
    """One tiny forward + backward + sharded-AdamW step on cuda:0 (world of one)."""
    from ..parallel.dp import ShardedDataParallel
    torch.manual_seed(0)
    cfg = GPTConfig.tiny()
    model = GPT(cfg, device="cuda")
    dp = ShardedDataParallel(model, lr=1e-3, heap_bytes=256 << 20)
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
    losses = []
    for _ in range(3):
        loss = dp.train_step(ids, ids.roll(-1, 1))
        losses.append(float(loss))
    assert all(math.isfinite(l) for l in losses) and losses[-1] < losses[0], losses
    return losses[-1]
