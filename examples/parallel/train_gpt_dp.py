#!/usr/bin/env python
"""Data-parallel GPT training with bucketed gradient reduce-scatter fused with AdamW, plus checkpoint / resume.

    python examples/parallel/train_gpt_dp.py --steps 10                                   # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/parallel/train_gpt_dp.py --steps 10
    ... --save ckpt.pt      /      ... --resume ckpt.pt        (every rank writes / reads ckpt.pt.rank<r>)
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from pccl_b200.engine import Engine  # noqa: E402
from pccl_b200.models import GPT, GPTConfig  # noqa: E402
from pccl_b200.parallel import ShardedDataParallel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["tiny", "gpt-1.3b"], default="tiny")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--save", default="")
    ap.add_argument("--resume", default="")
    a = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))     # rendezvous only
    cfg = GPTConfig.tiny() if a.model == "tiny" else GPTConfig.gpt_1p3b()
    torch.manual_seed(0)
    model = GPT(cfg, device="cuda")
    n_params = sum(p.numel() for p in model.parameters())
    eng = Engine(rank, world)
    eng.initEngine("cuda", heap_bytes=8 * n_params + (1 << 30))      # bf16 gradients + parameters live in the symmetric heap
    if world > 1:
        eng.connect()
    dp = ShardedDataParallel(model, eng, lr=3e-4, bucket_mb=25.0)
    if a.resume:
        dp.load_full_state(torch.load(f"{a.resume}.rank{rank}"))
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    for step in range(a.steps):
        ids = torch.randint(0, cfg.vocab_size, (a.batch, cfg.seq_len + 1), device="cuda", generator=g)
        loss = dp.train_step(ids[:, :-1], ids[:, 1:])
        if rank == 0:
            print(f"step {dp.step_count}: loss {float(loss):.4f}  (reduce-scatter schedule: {dp.schedule['mode']})")
    if a.save:
        torch.cuda.synchronize()
        torch.save(dp.gather_full_state(), f"{a.save}.rank{rank}")
    if world > 1:
        dist.barrier()
        del dp, model, eng
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
