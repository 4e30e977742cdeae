"""Host-side plumbing benchmark: ring all-reduce (sum) of fp32 vectors between CPU ranks of one host, through the
engine's CPU executor over shared memory and over TCP, next to gloo's all_reduce on the same ranks.

    python -m pccl_b200.bench_cpu --world 2 --elems 4194304 --iters 10

It is the configuration "ring all-reduce, 4 M fp32, world 2, host memory / TCP" end to end: DSL program -> schedule ->
engine -> executor.  Times are wall-clock on the host (there is no device here), the median over ``--iters`` calls after
``--warmup`` calls, and the maximum over ranks; bus bandwidth = bytes * 2 (n-1)/n / time.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import time


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, gloo_port: int, transport: str, elems: int, iters: int, warmup: int, width: int, q) -> None:
    import torch
    import torch.distributed as dist
    os.environ["PCCL_TRANSPORT"] = transport
    os.environ.setdefault("PCCL_WORKSPACE_MB", str(max(64, (elems * 4 * 4) >> 20)))
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{gloo_port}", rank=rank, world_size=world)
    e = Engine(rank, world)
    e.initEngine("cpu")
    e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ring", build("ring_allreduce", world, channels=2, device_type=DeviceType.CPU))
    g = torch.Generator().manual_seed(rank)
    x = torch.rand(elems, generator=g) * 2 - 1
    y = torch.empty_like(x)

    def timed(fn):
        ts = []
        for i in range(warmup + iters):
            dist.barrier()
            t0 = time.perf_counter()
            fn()
            t1 = time.perf_counter()
            if i >= warmup:
                ts.append(t1 - t0)
        return statistics.median(ts)

    ours = timed(lambda: e.exeOp("ring", x, y, width=width))
    ref = x.clone()
    dist.all_reduce(ref)
    err = (y - ref).abs().max().item()
    z = x.clone()
    theirs = timed(lambda: dist.all_reduce(z))
    both = torch.tensor([ours, theirs], dtype=torch.float64)
    dist.all_reduce(both, op=dist.ReduceOp.MAX)
    stats = e.stats()
    e.exitCluster()
    dist.destroy_process_group()
    if rank == 0:
        q.put({"ours_s": both[0].item(), "gloo_s": both[1].item(), "max_err": err, "tcp_bytes_sent": stats.get("tcp_bytes_sent", 0)})


def main() -> None:
    import torch.multiprocessing as mp
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--elems", type=int, default=4 * 1024 * 1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--width", type=int, default=2, help="threads per channel in the CPU executor")
    ap.add_argument("--transports", default="shm,tcp")
    a = ap.parse_args()
    ctx = mp.get_context("spawn")
    nbytes = a.elems * 4
    for transport in a.transports.split(","):
        q = ctx.Queue()
        port, gloo_port = _free_port(), _free_port()
        procs = [ctx.Process(target=_rank, args=(r, a.world, port, gloo_port, transport, a.elems, a.iters, a.warmup, a.width, q))
                 for r in range(a.world)]
        for p in procs:
            p.start()
        res = q.get(timeout=600)
        for p in procs:
            p.join(60)
        bus = nbytes * 2 * (a.world - 1) / a.world
        print(json.dumps({"collective": "allreduce", "algorithm": "ring", "transport": transport, "world": a.world, "dtype": "fp32",
                          "bytes": nbytes, "ms": round(res["ours_s"] * 1e3, 3), "bus_gbs": round(bus / res["ours_s"] / 1e9, 2),
                          "gloo_ms": round(res["gloo_s"] * 1e3, 3), "gloo_bus_gbs": round(bus / res["gloo_s"] / 1e9, 2),
                          "speedup_vs_gloo": round(res["gloo_s"] / res["ours_s"], 2), "max_err_vs_gloo": res["max_err"],
                          "tcp_bytes_sent_rank0": res["tcp_bytes_sent"], "timing": "host wall clock, median, max over ranks"}))


if __name__ == "__main__":
    main()
