#!/usr/bin/env python
"""A model cut into pipeline stages, trained with the one-forward-one-backward schedule.

CPU ranks over gloo (no GPU needed), three stages:

    python -m torch.distributed.run --nproc-per-node 3 --master-addr 127.0.0.1 --master-port 29710 \
        examples/parallel/pipeline_1f1b.py --backend gloo

On GPUs leave the backend at nccl: the hand-offs then run on the pipeline's own stream and overlap the stage's compute.
Every rank builds the whole model from one seed and keeps its own stage, so rank 0 can also train the whole model by
itself and the example can say how far the two parameter sets are apart after the steps (they should agree).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from pccl_b200.parallel.pp import PipelineP2P  # noqa: E402


def make_stages(n, width):
    torch.manual_seed(0)
    return [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.GELU(), torch.nn.Linear(width, width)) for _ in range(n)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--width", type=int, default=64)
    ap.add_argument("--rows", type=int, default=8, help="rows of one microbatch")
    ap.add_argument("--micro", type=int, default=6, help="microbatches per step")
    ap.add_argument("--steps", type=int, default=5)
    a = ap.parse_args()
    dist.init_process_group(a.backend)
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cpu")
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda")
    stages = make_stages(world, a.width)
    whole = [s.to(dev) for s in make_stages(world, a.width)] if rank == 0 else None       # the comparison copy
    stage = stages[rank].to(dev)
    opt = torch.optim.SGD(stage.parameters(), lr=0.05)
    pp = PipelineP2P()
    shape = (a.rows, a.width)
    g = torch.Generator().manual_seed(1)
    for step in range(a.steps):
        xs = [torch.randn(*shape, generator=g).to(dev) for _ in range(a.micro)]
        ts = [torch.randn(*shape, generator=g).to(dev) for _ in range(a.micro)]
        opt.zero_grad(set_to_none=True)
        losses = pp.run_1f1b(stage, a.micro, inputs=xs if rank == 0 else None, in_shape=shape, out_shape=shape,
                             loss_fn=lambda y, i: ((y - ts[i]) ** 2).mean() / a.micro, dtype=torch.float32)
        opt.step()
        if rank == world - 1:
            print(f"step {step}: loss {sum(float(v) for v in losses):.5f}", flush=True)
        if rank == 0:                                   # the same step on the whole model
            params = [p for s in whole for p in s.parameters()]
            for p in params:
                p.grad = None
            for x, t in zip(xs, ts):
                y = x
                for s in whole:
                    y = s(y)
                (((y - t) ** 2).mean() / a.micro).backward()
            with torch.no_grad():
                for p in params:
                    p -= 0.05 * p.grad
    if rank == 0:
        diff = max((p - q).abs().max().item() for p, q in zip(stage.parameters(), whole[0].parameters()))
        print(f"stage 0 after {a.steps} steps differs from the whole-model run by {diff:.2e}")
        assert diff < 1e-5
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
