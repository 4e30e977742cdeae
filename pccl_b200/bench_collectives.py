"""Collective micro-benchmarks: this library's kernels (NVLS and P2P forms) against NCCL on the same
GPUs, same sizes.  Device-timed with CUDA events, maximum over ranks; buffers rotate through a pool
larger than the 126 MB L2 so that consecutive iterations do not find their data cached.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m pccl_b200.bench_collectives \\
        --min-bytes 1024 --max-bytes 1073741824 --out sweep.json
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .engine import Engine, dtype_name
from .ops import collectives as C

POOL_BYTES = 320 << 20


def _time(fn_at, n_slots: int, iters: int, warmup: int, trains: int = 1) -> float:
    """Milliseconds per call: a train of `iters` back-to-back calls between two CUDA events, maximum over the
    ranks; with `trains` > 1 the median of that many trains (one slow train, e.g. a clock dip, does not decide)."""
    for i in range(warmup):
        fn_at(i % n_slots)
    per_train = []
    k = warmup
    for _ in range(max(1, trains)):
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _i in range(iters):
            fn_at(k % n_slots)
            k += 1
        b.record()
        b.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_train.append(float(t.item()))
    per_train.sort()
    return per_train[len(per_train) // 2]


def bus_factor(kind: str, n: int) -> float:
    return 2.0 * (n - 1) / n if kind == "allreduce" else (n - 1) / n


_PROGRAMS: Dict[str, List[str]] = {}


def interp_programs(eng: Engine, kind: str) -> List[str]:
    """Registers (once) the ``pccl_b200.lang`` programs the interpreter kernel is timed on: the NVLS and direct forms of
    the collective and the MILP-synthesised schedule for this world behind an NVSwitch."""
    if kind in _PROGRAMS:
        return _PROGRAMS[kind]
    from .lang import build
    from .synth import Topology, synthesize
    lang_kind = {"allreduce": "allreduce", "reduce_scatter": "reduce_scatter", "allgather": "allgather"}[kind]
    names = []
    if eng.has_nvls:
        eng.regOp(f"bench_nvls_{kind}", build(f"nvls_{lang_kind}", eng.world, channels=2))
        names.append(f"bench_nvls_{kind}")
    eng.regOp(f"bench_direct_{kind}", build(f"direct_{lang_kind}", eng.world, channels=2))
    names.append(f"bench_direct_{kind}")
    # the same exchange on symmetric buffers: peers' inputs are read (outputs written) in place, nothing is staged
    eng.regOp(f"bench_pull_{kind}", build(f"direct_{lang_kind}", eng.world, channels=2, direct=True))
    names.append(f"bench_pull_{kind}")
    res = synthesize(lang_kind, Topology.nvswitch(eng.world), 16 << 20, chunks=1, time_limit=10.0)
    eng.regOp(f"bench_milp_{kind}", res.ir)
    names.append(f"bench_milp_{kind}")
    _PROGRAMS[kind] = names
    return names


def bench_size(eng: Engine, kind: str, dtype: torch.dtype, nbytes: int, impls: List[str], iters: Optional[int] = None,
               trains: int = 1) -> Dict:
    """`nbytes` = bytes of the full vector (all-reduce) or of the gathered/scattered whole (RS/AG)."""
    world = eng.world
    es = torch.empty((), dtype=dtype).element_size()
    n = max(world * 16 // es, nbytes // es // (world * 16 // es) * (world * 16 // es))
    nbytes = n * es
    if iters is None:
        iters = 200 if nbytes <= (1 << 20) else (50 if nbytes <= (64 << 20) else 10)
    warmup = max(3, iters // 10)
    slot = (nbytes + 255) // 256 * 256
    n_slots = max(1, min(64, POOL_BYTES // (2 * slot)))
    mark = eng.symmetric_mark()
    pool_in = eng.symmetric_tensor((n_slots * slot,), torch.uint8)
    pool_out = eng.symmetric_tensor((n_slots * slot,), torch.uint8)
    pool_in.view(torch.int16)[:] = 0x3C00 if dtype != torch.float32 else 0     # finite values in every dtype
    shard = n // world
    ins = [pool_in[i * slot:i * slot + nbytes].view(dtype) for i in range(n_slots)]
    outs = [pool_out[i * slot:i * slot + nbytes].view(dtype) for i in range(n_slots)]
    res = {"kind": kind, "dtype": str(dtype).replace("torch.", ""), "bytes": nbytes, "n_gpus": world}
    for impl in impls:
        if impl == "interp":
            # the same collective as a lowered pccl_b200.lang program run by the persistent interpreter kernel:
            # best program and width (runtime CTA budget) for this size
            best = None
            for name in interp_programs(eng, kind):
                if nbytes > (64 << 20) and "nvls" not in name and "pull" not in name:   # the staged forms need that much workspace
                    continue
                for width in ((4, 16, 32) if nbytes <= (64 << 20) else (32,)):
                    if kind == "allreduce":
                        fn = lambda i, n_=name, w_=width: eng.exeOp(n_, ins[i], outs[i], width=w_)  # noqa: E731
                    elif kind == "reduce_scatter":
                        fn = lambda i, n_=name, w_=width: eng.exeOp(n_, ins[i], outs[i][:shard], width=w_)  # noqa: E731
                    else:
                        fn = lambda i, n_=name, w_=width: eng.exeOp(n_, ins[i][:shard], outs[i], width=w_)  # noqa: E731
                    try:
                        ms = _time(fn, n_slots, max(5, iters // 4), 3)
                    except Exception as e:  # noqa: BLE001 - a program that does not fit the workspace is left out
                        if eng.rank == 0:
                            print(f"# interp {name} width {width} at {nbytes} bytes: {type(e).__name__}: {e}", flush=True)
                        continue
                    st = eng.check_status(0)
                    if st[0] != 0:        # the kernel gave up (bounds check, time-out): not a timing
                        if eng.rank == 0:
                            print(f"# interp {name} width {width} at {nbytes} bytes: device status {list(st)}", flush=True)
                        continue
                    if best is None or ms < best[0]:
                        best = (ms, name, width)
            if best is not None:
                alg = nbytes / (best[0] * 1e-3) / 1e9
                res[impl] = {"us": best[0] * 1e3, "algbw_gbs": alg, "busbw_gbs": alg * bus_factor(kind, world),
                             "program": best[1].replace("bench_", ""), "width": best[2]}
            continue
        if impl == "nccl":
            if kind == "allreduce":
                fn = lambda i: dist.all_reduce(ins[i])  # noqa: E731
            elif kind == "reduce_scatter":
                fn = lambda i: dist.reduce_scatter_tensor(outs[i][:shard], ins[i])  # noqa: E731
            else:
                fn = lambda i: dist.all_gather_into_tensor(outs[i], ins[i][:shard])  # noqa: E731
        else:
            if impl == "nvls" and not eng.has_nvls:
                continue
            if kind == "allreduce":
                fn = lambda i, a=impl: C.all_reduce(eng, ins[i], outs[i], algo=a)  # noqa: E731
            elif kind == "reduce_scatter":
                fn = lambda i, a=impl: C.reduce_scatter(eng, ins[i], outs[i][:shard], algo=a)  # noqa: E731
            else:
                fn = lambda i, a=impl: C.all_gather(eng, ins[i][:shard], outs[i], algo=a)  # noqa: E731
        ms = _time(fn, n_slots, iters, warmup, trains)
        alg = nbytes / (ms * 1e-3) / 1e9
        res[impl] = {"us": ms * 1e3, "algbw_gbs": alg, "busbw_gbs": alg * bus_factor(kind, world)}
        if impl == "auto":          # what `algo="auto"` resolved to at this size
            per_rank = nbytes if kind == "allreduce" else nbytes // world
            if kind == "allgather":
                res[impl]["algo"] = "nvls" if (eng.has_nvls and per_rank % 16 == 0 and per_rank < (4 << 20)) else "p2p"
            else:
                res[impl]["algo"] = C._algo(eng, "auto", dtype_name(dtype), "sum", per_rank, kind)
                if kind == "allreduce" and nbytes <= (64 << 10) and nbytes % 4 == 0 and os.environ.get("PCCL_LL", "1") != "0":
                    res[impl]["algo"] = "ll"          # flag-in-data packets, no barrier (csrc/kernels/collectives.cu)
    eng.symmetric_reset(mark)
    return res


def bench_rooted(eng: Engine, kind: str, dtype: torch.dtype, nbytes: int, iters: Optional[int] = None, root: int = 0) -> Dict:
    """Broadcast or rooted reduce of a vector of `nbytes`: the library programs run by the interpreter kernel (every
    form, best width) next to NCCL's.  Bandwidth is bytes of the vector over time."""
    es = torch.empty((), dtype=dtype).element_size()
    n = max(eng.world * 16 // es, nbytes // es // (eng.world * 16 // es) * (eng.world * 16 // es))
    nbytes = n * es
    if iters is None:
        iters = 100 if nbytes <= (1 << 20) else (30 if nbytes <= (64 << 20) else 10)
    n_slots = max(1, min(32, (256 << 20) // nbytes))            # rotate through more than the L2 holds
    xs = [torch.ones(n, dtype=dtype, device="cuda") for _ in range(n_slots)]
    ys = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(n_slots)]
    res = {"kind": kind, "dtype": str(dtype).replace("torch.", ""), "bytes": nbytes, "n_gpus": eng.world, "root": root}
    forms = ("direct", "tree", "scatter_allgather") if kind == "broadcast" else ("tree", "pieces")
    best = None
    for form in forms:
        for width in (4, 16):
            if kind == "broadcast":
                fn = lambda i, f=form, w=width: C.broadcast(eng, xs[i], root=root, out=ys[i], algo=f, channels=2, width=w)  # noqa: E731
            else:
                fn = lambda i, f=form, w=width: C.reduce(eng, xs[i], ys[i], root=root, algo=f, channels=2, width=w)  # noqa: E731
            try:
                ms = _time(fn, n_slots, iters, 3)
            except Exception as e:  # noqa: BLE001 - a form that does not fit the workspace at this size is left out
                if eng.rank == 0:
                    print(f"# {kind} {form} width {width} at {nbytes} bytes: {type(e).__name__}: {e}", flush=True)
                continue
            if eng.check_status(0)[0] != 0:
                continue
            if best is None or ms < best[0]:
                best = (ms, form, width)
    if best is not None:
        res["interp"] = {"us": best[0] * 1e3, "algbw_gbs": nbytes / (best[0] * 1e-3) / 1e9, "form": best[1], "width": best[2]}
    nccl = (lambda i: dist.broadcast(xs[i], root)) if kind == "broadcast" else (lambda i: dist.reduce(xs[i], root))
    ms = _time(nccl, n_slots, iters, 3)
    res["nccl"] = {"us": ms * 1e3, "algbw_gbs": nbytes / (ms * 1e-3) / 1e9}
    return res


def quick_micro(eng: Engine) -> Dict:
    """Three all-reduce sizes, ours against NCCL; cheap enough to ride along with bench.py."""
    out = []
    for nbytes in (1 << 20, 16 << 20, 256 << 20):
        out.append(bench_size(eng, "allreduce", torch.bfloat16, nbytes, ["nvls", "p2p", "nccl"], iters=20 if nbytes > (1 << 24) else 50))
    return {"allreduce_bf16": out}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--kinds", default="allreduce,reduce_scatter,allgather")
    ap.add_argument("--dtypes", default="bf16,f32")
    ap.add_argument("--impls", default="nvls,p2p,nccl")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=180))
    interp = "interp" in args.impls.split(",") or any(k in ("broadcast", "reduce") for k in args.kinds.split(","))
    os.environ.setdefault("PCCL_WORKSPACE_MB", "1024" if interp else "64")      # scratch of the direct programs
    eng = Engine(rank, world)
    eng.initEngine("cuda", heap_bytes=(2 * POOL_BYTES) + 4 * args.max_bytes + (512 << 20) + ((2 << 30) if interp else 0))
    eng.connect()
    dtypes = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}
    rows = []
    for kind in args.kinds.split(","):
        for dn in args.dtypes.split(","):
            nbytes = args.min_bytes
            while nbytes <= args.max_bytes:
                if kind in ("broadcast", "reduce"):
                    if nbytes > (64 << 20):          # the programs stage through the workspace
                        break
                    r = bench_rooted(eng, kind, dtypes[dn], nbytes)
                else:
                    r = bench_size(eng, kind, dtypes[dn], nbytes, args.impls.split(","))
                rows.append(r)
                if rank == 0:
                    print(json.dumps(r), flush=True)
                nbytes *= 2
    eng.raise_on_status(8, "sweep")
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"n_gpus": world, "nvls": eng.has_nvls, "rows": rows}, f)
    dist.barrier()
    del eng
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
