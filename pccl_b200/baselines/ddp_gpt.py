"""The opponent for the data-parallel training benchmark: the same GPT decoder written with plain
``torch.nn`` modules (cuBLAS GEMMs, cuDNN / flash scaled-dot-product attention, eager element-wise
kernels), wrapped in ``torch.nn.parallel.DistributedDataParallel`` (NCCL all-reduce of 25 MB gradient
buckets overlapped with backward) and stepped by ``torch.optim.AdamW(fused=True)``.

Nothing of this package's kernels or engine is on this path; it exists so that the framework's
tokens/s has a number to stand against that was measured on the same GPUs, in the same process
launch, on the same shapes.  (The reference library has no model and no training loop to time.)

``precision="bf16"`` keeps the parameters, gradients and AdamW state in bf16, the least work PyTorch
can do per step; ``"amp"`` keeps fp32 parameters under ``torch.autocast`` (the usual mixed-precision
recipe, closer to this framework's fp32 master weights but slower).  The default is the faster one,
so the baseline is not handicapped.
"""
from __future__ import annotations

import math
import time
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class _Block(nn.Module):
    def __init__(self, d: int, n_head: int, mlp_ratio: int, n_layer: int):
        super().__init__()
        self.n_head = n_head
        self.ln1 = nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln2 = nn.LayerNorm(d)
        self.fc1 = nn.Linear(d, mlp_ratio * d)
        self.fc2 = nn.Linear(mlp_ratio * d, d)
        for lin in (self.qkv, self.fc1):
            nn.init.normal_(lin.weight, std=0.02)
        for lin in (self.proj, self.fc2):
            nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * n_layer))
        for lin in (self.qkv, self.proj, self.fc1, self.fc2):
            nn.init.zeros_(lin.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.n_head, D // self.n_head).unbind(2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, D))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class TorchGPT(nn.Module):
    """Same architecture as ``pccl_b200.models.GPT`` (tied input / output embeddings, learned positions,
    pre-LayerNorm blocks, tanh GELU), in stock PyTorch modules."""

    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.wte = nn.Embedding(cfg.vocab_size, d)
        self.wpe = nn.Embedding(cfg.seq_len, d)
        self.blocks = nn.ModuleList(_Block(d, cfg.n_head, cfg.mlp_ratio, cfg.n_layer) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(d)
        nn.init.normal_(self.wte.weight, std=0.02)
        nn.init.normal_(self.wpe.weight, std=0.02)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        T = ids.shape[1]
        x = self.wte(ids) + self.wpe(torch.arange(T, device=ids.device))[None]
        for blk in self.blocks:
            x = blk(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1))


class DDPTrainer:
    """``train_step(ids, targets) -> loss`` of the PyTorch baseline (forward, backward with DDP's
    overlapped all-reduce, fused AdamW)."""

    def __init__(self, cfg, world: int, local_rank: int, *, lr: float = 1e-4, precision: str = "bf16",
                 bucket_cap_mb: float = 25.0, zero: bool = False):
        if precision not in ("bf16", "amp"):
            raise ValueError("precision must be 'bf16' or 'amp'")
        self.precision = precision
        torch.manual_seed(1234)
        model = TorchGPT(cfg).to("cuda")
        if precision == "bf16":
            model = model.to(torch.bfloat16)
        self.params = sum(p.numel() for p in model.parameters())
        self.model = model
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel
            self.model = DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=bucket_cap_mb,
                                                 gradient_as_bucket_view=True, static_graph=True)
        decay = [p for p in model.parameters() if p.dim() >= 2]
        no_decay = [p for p in model.parameters() if p.dim() < 2]
        groups = [{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}]
        if zero and world > 1:
            from torch.distributed.optim import ZeroRedundancyOptimizer
            self.opt = ZeroRedundancyOptimizer(model.parameters(), optimizer_class=torch.optim.AdamW, lr=lr, betas=(0.9, 0.95),
                                               eps=1e-8, weight_decay=0.1, fused=True)
        else:
            self.opt = torch.optim.AdamW(groups, lr=lr, betas=(0.9, 0.95), eps=1e-8, fused=True)

    def train_step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.opt.zero_grad(set_to_none=True)
        if self.precision == "amp":
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = self.model(ids, targets)
        else:
            loss = self.model(ids, targets)
        loss.backward()
        self.opt.step()
        return loss.detach()


def measure(cfg, world: int, rank: int, local_rank: int, batch: int, steps: int, warmup: int, *, precision: str = "bf16",
            zero: bool = False, e2e: bool = True, seed_base: int = 1000) -> Dict:
    """Times the baseline like ``bench.py`` times the framework: ``warmup`` untimed steps, then ``steps``
    steps between CUDA events with a barrier and a synchronize on both sides, maximum over ranks; then
    (``e2e``) the same with the step's token ids copied from pinned host memory and the loss read back."""
    import torch.distributed as dist
    trainer = DDPTrainer(cfg, world, local_rank, precision=precision, zero=zero)
    S = cfg.seq_len
    g = torch.Generator().manual_seed(seed_base + rank)
    host = [torch.randint(0, cfg.vocab_size, (batch, S + 1), generator=g).pin_memory() for _ in range(warmup + steps)]
    dev = [h.cuda() for h in host[:2]]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(warmup):
        b = dev[i % 2]
        trainer.train_step(b[:, :-1], b[:, 1:])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        b = dev[i % 2]
        loss = trainer.train_step(b[:, :-1], b[:, 1:])
    e1.record()
    barrier()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    out = {"tokens_per_s": world * batch * S * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps, "final_loss": float(loss),
           "params": trainer.params, "precision": precision, "optimizer": "ZeroRedundancyOptimizer(AdamW fused)" if zero else "AdamW(fused=True)",
           "wrapper": "DistributedDataParallel(bucket_cap_mb=25, gradient_as_bucket_view, static_graph)" if world > 1 else "none (one GPU)"}
    if e2e:
        loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        f0.record()
        for i in range(steps):
            ids = host[warmup + i].to("cuda", non_blocking=True)
            loss = trainer.train_step(ids[:, :-1], ids[:, 1:])
            loss_host.copy_(loss.reshape(1).float(), non_blocking=True)
            torch.cuda.current_stream().synchronize()
            _ = float(loss_host[0])
        f1.record()
        barrier()
        ms = max(max_over_ranks(f0.elapsed_time(f1)), max_over_ranks((time.perf_counter() - t0) * 1e3))
        out["e2e_tokens_per_s"] = world * batch * S * steps / (ms / 1e3)
        out["e2e_ms_per_step"] = ms / steps
    del trainer
    torch.cuda.empty_cache()
    return out


def recorded(n_gpus: int) -> Optional[float]:
    """Tokens/s of this baseline as recorded for this GPU pool (``ddp_gpt1p3b_b200.json`` beside this file), or None."""
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ddp_gpt1p3b_b200.json")
    try:
        with open(path) as f:
            table = json.load(f)
    except OSError:
        return None
    v = table.get("tokens_per_s", {}).get(str(n_gpus))
    return float(v) if v else None
