#!/usr/bin/env python
"""Expert-parallel MoE layer: routing, fp8 dispatch all-to-all, grouped expert FFN, weighted combine all-to-all.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/parallel/moe_layer.py
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from pccl_b200.engine import Engine  # noqa: E402
from pccl_b200.ops import check_status  # noqa: E402
from pccl_b200.ops.moe import MoEExchange  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tokens, hidden, d_ff, experts, topk = 2048, 2048, 1024, 8 * world, 4
    eng = Engine(rank, world)
    eng.initEngine("cuda", heap_bytes=2 << 30)
    eng.connect()
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).bfloat16()
    logits = torch.randn(tokens, experts, device="cuda", generator=g)
    epr = experts // world
    w1 = (torch.randn(epr * d_ff, hidden, device="cuda", generator=g) * 0.05).bfloat16()      # this rank's experts, stacked
    w2 = (torch.randn(epr * hidden, d_ff, device="cuda", generator=g) * 0.05).bfloat16()
    moe = MoEExchange(eng, tokens, hidden, experts, topk)
    out = moe.forward(x, logits, w1, w2)
    torch.cuda.synchronize()
    check_status("moe")
    if rank == 0:
        print(f"output {tuple(out.shape)}, mean |y| {out.float().abs().mean().item():.4f}")
    dist.barrier()
    del moe, eng
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
