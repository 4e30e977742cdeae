#!/usr/bin/env python
"""Write a ring all-reduce in the DSL, prove it symbolically, save it as a schedule file, and run it.

CPU ranks (no GPU needed), two processes on this host:

    python examples/collective/allreduce.py --rank 0 --world 2 --master 127.0.0.1:29700 &
    python examples/collective/allreduce.py --rank 1 --world 2 --master 127.0.0.1:29700

The same program runs on GPUs through the interpreter kernel when the engine is initialised with
device="cuda" under torch.distributed.run (see tests/mp_worker.py, case "interp").
"""
import argparse
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402

from pccl.engine import Engine  # noqa: E402
from pccl.lang import Chunk, CollectiveIR, Device, DeviceType, Link, PrimitiveOpType, to_schedule, verify  # noqa: E402


def ring_allreduce(n: int) -> CollectiveIR:
    """n chunks; n-1 reduce steps around the ring, then n-1 copy steps.  Remote ranks only touch `scratch`."""
    ir = CollectiveIR("example_ring_allreduce", "allreduce", units=n, buffers={"input": n, "output": n, "scratch": n})
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CPU, memory_bandwidth=50e9, compute_capability=0))
    for r in range(n):
        ir.add_link(Link(r, (r + 1) % n, bandwidth=10e9, latency=20e-6))
    ir.set_precondition([Chunk({r}, r, n, 0, "input") for r in range(n)])
    ir.set_postcondition([Chunk(set(range(n)), r, n, 0, "output") for r in range(n)])
    last = {}
    for r in range(n):
        for c in range(n):
            last[(r, c)] = ir.create_operation(PrimitiveOpType.COPY, Chunk({r}, r, 1, c, "input"), Chunk({r}, r, 1, c, "output"))
    for s in range(n - 1):                      # reduce-scatter
        new = {}
        for r in range(n):
            c, nxt = (r - s) % n, (r + 1) % n
            have = {(r - k) % n for k in range(s + 1)}
            push = ir.create_operation(PrimitiveOpType.COPY, Chunk(have, r, 1, c, "output"), Chunk(have, nxt, 1, c, "scratch"),
                                       dependencies=[last[(r, c)]])
            new[(nxt, c)] = ir.create_operation(PrimitiveOpType.REDUCE, Chunk(have, nxt, 1, c, "scratch"),
                                                Chunk(have | {nxt}, nxt, 1, c, "output"), dependencies=[push, last[(nxt, c)]])
        last.update(new)
    everyone = set(range(n))
    for s in range(n - 1):                      # all-gather
        new = {}
        for r in range(n):
            c, nxt = (r + 1 - s) % n, (r + 1) % n
            push = ir.create_operation(PrimitiveOpType.COPY, Chunk(everyone, r, 1, c, "output"), Chunk(everyone, nxt, 1, c, "scratch"),
                                       dependencies=[last[(r, c)], last[(nxt, c)]])
            new[(nxt, c)] = ir.create_operation(PrimitiveOpType.COPY, Chunk(everyone, nxt, 1, c, "scratch"),
                                                Chunk(everyone, nxt, 1, c, "output"), dependencies=[push])
        last.update(new)
    return ir


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--master", default="127.0.0.1:29700")
    ap.add_argument("--elems", type=int, default=1 << 20)
    args = ap.parse_args()

    ir = ring_allreduce(args.world)
    assert ir.validate_dag() and ir.validate_topology()
    report = verify(ir)                                   # symbolic proof: every rank ends with every contribution once
    assert report.ok, report.errors
    path = os.path.join(tempfile.gettempdir(), f"example_ring_allreduce_{args.world}.json")
    with open(path, "w") as f:
        json.dump(to_schedule(ir), f)                     # the file Engine.regOp reads

    eng = Engine(args.rank, args.world)
    eng.initEngine("cpu")
    if args.world > 1:
        eng.joinCluster(args.master)
    eng.regOp("ring", path)
    x = torch.full((args.elems,), float(args.rank + 1))
    y = torch.empty_like(x)
    eng.exeOp("ring", x, y)
    want = args.world * (args.world + 1) / 2
    print(f"rank {args.rank}: allreduce -> {y[0].item()} (expected {want}); ops={report.num_ops} steps={report.num_steps}")
    assert torch.all(y == want)
    eng.exitCluster()


if __name__ == "__main__":
    main()
