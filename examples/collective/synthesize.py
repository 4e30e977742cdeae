#!/usr/bin/env python
"""Synthesise collective schedules with the MILP (no GPU needed): pick a topology, a collective and a size, get a
verified program, its cost against the port lower bound, and a schedule file that ``Engine.regOp`` accepts.

    python examples/collective/synthesize.py --topology nvswitch --world 8 --collective allreduce --mbytes 64
    python examples/collective/synthesize.py --topology ring --world 4 --collective allgather --mbytes 1 --out ag.json
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from pccl.lang import Cluster, check_lowered_deadlock_free, to_schedule  # noqa: E402
from pccl_b200.synth import ScheduleCache, Topology, synthesize  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--topology", choices=["nvswitch", "ring"], default="nvswitch")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--collective", choices=["allreduce", "reduce_scatter", "allgather", "alltoall", "broadcast", "reduce"], default="allreduce")
    ap.add_argument("--mbytes", type=float, default=64.0)
    ap.add_argument("--chunks", type=int, default=1, help="pieces per shard (broadcast / reduce: pieces of the vector; try --chunks = --world)")
    ap.add_argument("--root", type=int, default=0, help="broadcast / reduce only")
    ap.add_argument("--out", default="")
    ap.add_argument("--cache-dir", default="")
    a = ap.parse_args()
    topo = Topology.nvswitch(a.world) if a.topology == "nvswitch" else Topology.ring(a.world)
    nbytes = int(a.mbytes * (1 << 20))
    rooted = {"root": a.root} if a.collective in ("broadcast", "reduce") else {}
    res = synthesize(a.collective, topo, nbytes, chunks=a.chunks, time_limit=20.0, **rooted)
    doc = to_schedule(res.ir)
    assert check_lowered_deadlock_free(doc["lowered"])
    report = {"program": res.ir.name, "steps": res.steps_used, "transfers_per_step": [len(s) for s in res.sends],
              "model_time_us": round(res.objective_seconds * 1e6, 2), "port_lower_bound_us": round(res.lower_bound_seconds * 1e6, 2),
              "instructions_per_rank": [sum(len(stream) for stream in rank_prog) for rank_prog in doc["lowered"]["programs"]][:4],
              "links_in_cluster": len(Cluster.from_topology(topo).links)}
    if a.cache_dir:                         # the on-disk cache that a trainer would consult at start-up
        cache = ScheduleCache(a.cache_dir)
        cache.get_or_synthesize(a.collective, topo, nbytes, chunks=a.chunks, **rooted)
        cache.get_or_synthesize(a.collective, topo, nbytes, chunks=a.chunks, **rooted)
        report["cache_hits"], report["cache_misses"] = cache.hits, cache.misses
    if a.out:
        with open(a.out, "w") as f:
            json.dump(doc, f)
        report["schedule_file"] = a.out
    print(json.dumps(report))


if __name__ == "__main__":
    main()
