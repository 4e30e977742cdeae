"""Multi-process CPU ranks: lang -> JSON schedule -> C++ engine -> CPU executor over shm and TCP."""
import json

import pytest
import torch

from _ranks import run_ranks


def _collective_rank(rank, world, port, algos, transport, dtype_name, n_elems, channels, width):
    """Every (algorithm, arguments) of ``algos`` in one set of ranks: three launches each, against torch."""
    from pccl_b200.engine import Engine
    e = Engine(rank, world)
    e.initEngine("cpu")
    e.joinCluster(f"127.0.0.1:{port}")
    out = {}
    for i, (algo, kwargs) in enumerate(algos):
        out[f"{algo}{kwargs or ''}"] = _one_collective(e, f"op{i}", rank, world, algo, dtype_name, n_elems, channels, width, kwargs)
    e.exitCluster()
    return out


def _one_collective(e, name, rank, world, algo, dtype_name, n_elems, channels, width, kwargs):
    import torch
    from pccl_b200.lang import DeviceType, build
    dtype = getattr(torch, dtype_name)
    ir = build(algo, world, channels=channels, device_type=DeviceType.CPU, **kwargs)
    e.regOp(name, ir)
    g = torch.Generator().manual_seed(0)
    coll = ir.collective
    per_rank = {"allreduce": n_elems, "reduce_scatter": n_elems * world, "allgather": n_elems,
                "alltoall": n_elems * world, "send_recv": n_elems, "broadcast": n_elems, "reduce": n_elems,
                "scatter": n_elems * world, "gather": n_elems}[coll]
    xs = [((torch.rand(per_rank, generator=g) * 2 - 1) * 4).to(dtype) for _ in range(world)]
    out_elems = {"allreduce": n_elems, "reduce_scatter": n_elems, "allgather": n_elems * world,
                 "alltoall": n_elems * world, "send_recv": n_elems, "broadcast": n_elems, "reduce": n_elems,
                 "scatter": n_elems, "gather": n_elems * world}[coll]
    root = ir.attrs.get("root", 0)
    untouched = torch.full((out_elems,), -777.0)
    errs = []
    for it in range(3):     # repeated launches exercise the epoch-counting signals and scratch halves
        x = (xs[rank].float() + it).to(dtype)
        y = torch.full((out_elems,), -777, dtype=dtype)
        e.exeOp(name, x, y, width=width)
        full = [(v.float() + it).to(dtype).float() for v in xs]
        if coll == "allreduce":
            ref = torch.stack(full).sum(0)
        elif coll == "reduce_scatter":
            ref = torch.stack(full).sum(0)[rank * n_elems:(rank + 1) * n_elems]
        elif coll == "allgather":
            ref = torch.cat(full)
        elif coll == "alltoall":
            ref = torch.cat([f[rank * n_elems:(rank + 1) * n_elems] for f in full])
        elif coll == "send_recv":           # only the receiver's output is written
            ref = full[ir.attrs["src"]] if rank == ir.attrs["dst"] else untouched
        elif coll == "broadcast":
            ref = full[root]
        elif coll == "reduce":
            ref = torch.stack(full).sum(0) if rank == root else untouched
        elif coll == "scatter":
            ref = full[root][rank * n_elems:(rank + 1) * n_elems]
        else:
            ref = torch.cat(full) if rank == root else untouched
        errs.append((y.float() - ref).abs().max().item())
    st = e.stats()
    return {"err": max(errs), "launches": st["ops"][name]["launches"], "tcp": st.get("tcp_bytes_sent", 0)}


def _baseline_rank(rank, world, port, transport):
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, algorithms
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ring", algorithms.ring_allreduce(world, channels=2, device_type=DeviceType.CPU))
    g = torch.Generator().manual_seed(0)
    xs = [torch.rand(4 * 1024 * 1024, generator=g) * 2 - 1 for _ in range(world)]
    y = torch.empty_like(xs[rank])
    e.exeOp("ring", xs[rank], y, width=2)
    ref = xs[0] + xs[1]
    tcp = e.stats()["tcp_bytes_sent"]
    e.exitCluster()
    return (torch.equal(y, ref), (y - ref).abs().max().item(), tcp)


def _mixed_width_rank(rank, world, port):
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, channels=2, device_type=DeviceType.CPU))
    g = torch.Generator().manual_seed(3)
    xs = [torch.rand(6 * 1024, generator=g) for _ in range(world)]
    errs = []
    for it, width in enumerate([1, 3, 1, 2, 3, 3, 1]):     # the runtime CTA/thread budget changes from launch to launch
        y = torch.empty_like(xs[rank])
        e.exeOp("ar", xs[rank] + it, y, width=width)
        errs.append((y - (sum(xs) + it * world)).abs().max().item())
    e.exitCluster()
    return max(errs)


def _operator_rank(rank, world, port):
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, Operator
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    op = Operator.from_algorithm("direct_allreduce", world, name="ar", channels=2, device_type=DeviceType.CPU).register(e)
    g = torch.Generator().manual_seed(9)
    xs = [torch.rand(4096, generator=g) for _ in range(world)]
    y = torch.empty_like(xs[rank])
    st = op(xs[rank], y, width=2)
    e.exitCluster()
    return st, (y - sum(xs)).abs().max().item()


def test_operator_object_registers_and_runs_on_cpu_ranks():
    res = run_ranks(_operator_rank, 2, env={"PCCL_WORKSPACE_MB": "16"})
    for r in (0, 1):
        assert res[r][0] == 0 and res[r][1] < 1e-5


def _two_hosts_rank(rank, world, port):
    """Ranks 0,1 pretend to sit on one host and ranks 2,3 on another: shared memory inside a host, TCP between them."""
    import torch
    from pccl_b200.engine import Engine, LaunchEnvironments
    from pccl_b200.lang import DeviceType, build
    LaunchEnvironments.setOverride("PCCL_HOST_ID", f"host{rank // 2}")
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, channels=1, device_type=DeviceType.CPU))
    e.regOp("a2a", build("alltoall", world, channels=1, device_type=DeviceType.CPU))
    g = torch.Generator().manual_seed(6)
    xs = [torch.rand(8 * 1024, generator=g) for _ in range(world)]
    y = torch.empty_like(xs[rank])
    e.exeOp("ar", xs[rank], y)
    err = (y - sum(xs)).abs().max().item()
    z = torch.empty_like(xs[rank])
    e.exeOp("a2a", xs[rank], z)
    blk = xs[rank].numel() // world
    err = max(err, (z - torch.cat([x[rank * blk:(rank + 1) * blk] for x in xs])).abs().max().item())
    tcp = e.stats().get("tcp_bytes_sent", 0)
    e.exitCluster()
    return err, tcp


def test_shared_memory_inside_a_host_and_tcp_between_hosts_in_one_collective():
    res = run_ranks(_two_hosts_rank, 4, env={"PCCL_WORKSPACE_MB": "16"}, timeout=120)
    for r in range(4):
        assert res[r][0] < 1e-5
    # in the ring 0-1-2-3-0 only the hops 1->2 and 3->0 cross hosts: those senders use TCP, ranks 0 and 2 send the ring
    # traffic over shared memory (their all-to-all blocks for the other host still travel by TCP)
    assert res[1][1] > res[0][1] > 0 and res[3][1] > res[2][1] > 0


def _hier_rank(rank, world, port, algo):
    import torch
    from pccl_b200.engine import Engine, LaunchEnvironments
    from pccl_b200.lang import DeviceType, build
    LaunchEnvironments.setOverride("PCCL_HOST_ID", f"host{rank // 2}")
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    kw = {"per_host": 2} if algo == "hierarchical_allreduce" else {}
    e.regOp("ar", build(algo, world, channels=1, device_type=DeviceType.CPU, **kw))
    g = torch.Generator().manual_seed(8)
    xs = [torch.rand(32 * 1024, generator=g) for _ in range(world)]
    y = torch.empty_like(xs[rank])
    e.exeOp("ar", xs[rank], y)
    tcp = e.stats().get("tcp_bytes_sent", 0)
    e.exitCluster()
    return (y - sum(xs)).abs().max().item(), tcp


def test_hierarchical_allreduce_sends_less_over_the_network_than_the_direct_one():
    """Four ranks on two pretended hosts: only the middle phase of the hierarchical algorithm uses TCP."""
    sent = {}
    for algo in ("hierarchical_allreduce", "direct_allreduce"):
        res = run_ranks(_hier_rank, 4, args=(algo,), env={"PCCL_WORKSPACE_MB": "16"}, timeout=120)
        assert all(res[r][0] < 1e-5 for r in range(4)), (algo, res)
        sent[algo] = sum(res[r][1] for r in range(4))
    vector = 32 * 1024 * 4
    # hierarchical: each rank sends 2 * (hosts - 1) / n of the vector across = 1/2 vector per rank; direct: 2 * 2/4 = 1 vector per rank
    assert sent["hierarchical_allreduce"] <= 0.6 * sent["direct_allreduce"], sent
    assert sent["hierarchical_allreduce"] >= 4 * vector // 2


def _overlap_rank(rank, world, port):
    """Two collectives at once, from two host threads, on two workspace lanes."""
    import threading
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, channels=2, device_type=DeviceType.CPU))
    e.regOp("ag", build("ring_allgather", world, channels=2, device_type=DeviceType.CPU))
    e.prepareOp("ar", 2); e.prepareOp("ag", 1)           # same order on every rank
    g = torch.Generator().manual_seed(4)
    xs = [torch.rand(64 * 1024, generator=g) for _ in range(world)]
    errs = []

    def allreduce():
        for it in range(6):
            y = torch.empty_like(xs[rank])
            e.exeOp("ar", xs[rank] + it, y, width=2, lane=0)
            errs.append((y - (sum(xs) + it * world)).abs().max().item())

    def allgather():
        for it in range(6):
            y = torch.empty(world * 4096)
            e.exeOp("ag", xs[rank][:4096] * (it + 1), y, width=1, lane=1)
            errs.append((y - torch.cat([x[:4096] * (it + 1) for x in xs])).abs().max().item())

    ts = [threading.Thread(target=allreduce), threading.Thread(target=allgather)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    st = e.stats()["ops"]
    e.exitCluster()
    return max(errs), st["ar"]["launches"], st["ag"]["launches"]


def test_two_ops_overlap_on_two_lanes_from_two_threads():
    res = run_ranks(_overlap_rank, 3, env={"PCCL_WORKSPACE_MB": "16"}, timeout=120)
    for r in range(3):
        assert res[r][0] < 1e-5 and res[r][1] == 6 and res[r][2] == 6, res[r]


def test_one_op_may_run_at_a_different_width_on_every_launch():
    res = run_ranks(_mixed_width_rank, 2, env={"PCCL_WORKSPACE_MB": "16"})
    assert max(res.values() if isinstance(res, dict) else res) < 1e-5


def test_baseline_config_ring_allreduce_4m_fp32_world2_shm_and_tcp():
    # ring allreduce (sum) of 4M fp32 per rank, uniform[-1,1) from seed 0, world 2, checked against torch sum
    for transport in ("shm", "tcp"):
        env = {"PCCL_WORKSPACE_MB": "128", "PCCL_TRANSPORT": transport}
        res = run_ranks(_baseline_rank, 2, args=(transport,), env=env)
        for r in (0, 1):
            assert res[r][0], f"{transport}: rank {r} differs from torch sum by {res[r][1]}"
            assert (res[r][2] > 0) == (transport == "tcp")


_SYMMETRIC = [
    ("ring_allreduce", {}), ("direct_allreduce", {}), ("oneshot_allreduce", {}), ("tree_allreduce", {}),
    ("direct_reduce_scatter", {}), ("direct_allgather", {}), ("ring_allgather", {}), ("ring_kv_rotation", {}),
    ("alltoall", {}), ("ulysses_alltoall", {}), ("ring_reduce_scatter", {}), ("recursive_doubling_allgather", {}),
    ("halving_doubling_allreduce", {}), ("hierarchical_allreduce", {"per_host": 2}),
    ("hierarchical_allgather", {"per_host": 2})]
_ROOTED = [
    ("send_recv", {"src": 2, "dst": 1}), ("broadcast", {"root": 1}), ("broadcast", {"root": 3, "tree": True}),
    ("reduce", {"root": 2}), ("scatter", {"root": 1}), ("gather", {"root": 3}),
    ("scatter_allgather_broadcast", {"root": 2}), ("reduce_scatter_gather_reduce", {"root": 1})]


@pytest.mark.parametrize("algos", [_SYMMETRIC, _ROOTED], ids=["symmetric", "rooted"])
def test_algorithms_on_cpu_ranks_shm(algos):
    """One set of four ranks runs the whole group, one program after the other (starting ranks is what costs time)."""
    res = run_ranks(_collective_rank, 4, args=(algos, "shm", "float32", 1000 + 17, 2, 2),
                    env={"PCCL_WORKSPACE_MB": "16"}, timeout=300)
    for r, per_algo in res.items():
        assert len(per_algo) == len(algos)
        for label, v in per_algo.items():
            assert v["err"] < 1e-4 and v["launches"] == 3, (label, r, v)


def test_algorithms_on_cpu_ranks_tcp_bf16():
    algos = [("ring_allreduce", {}), ("direct_reduce_scatter", {}), ("alltoall", {})]
    res = run_ranks(_collective_rank, 3, args=(algos, "tcp", "bfloat16", 4096 + 8, 1, 1),
                    env={"PCCL_WORKSPACE_MB": "16", "PCCL_TRANSPORT": "tcp"}, timeout=300)
    for r, per_algo in res.items():
        for label, v in per_algo.items():
            assert v["err"] <= 0.26 and v["tcp"] > 0, (label, r, v)   # bf16 rounding of sums up to ~24


def test_regop_accepts_file_and_rejects_garbage(tmp_path):
    from pccl_b200.engine import Engine
    from pccl_b200.lang import build, to_schedule
    e = Engine(0, 1)
    e.initEngine("cpu")
    path = tmp_path / "ar.json"
    path.write_text(json.dumps(to_schedule(build("ring_allreduce", 1))))
    e.regOp("from_file", str(path))
    x = torch.arange(10, dtype=torch.float32); y = torch.zeros(10)
    e.exeOp("from_file", x, y)
    assert torch.equal(x, y)
    with pytest.raises(RuntimeError):
        e.regOp("from_file", str(path))            # duplicate name
    with pytest.raises(RuntimeError):
        e.regOp("bad", "{\"name\": \"x\"}")         # no lowered section
    with pytest.raises(RuntimeError):
        e.exeOp("nope", x, y)
    doc = json.loads(e.exportEndpoint())
    assert doc["rank"] == 0 and "ipc.cpu.handle" in doc["endpoint_configs"] and "host_id" in doc["endpoint_configs"]
    lay = e.layout()
    assert lay["signal_off"] == lay["workspace_bytes"] and lay["total"] % (2 << 20) == 0


def test_exeop_reports_scratch_overflow():
    from pccl_b200.engine import Engine
    from pccl_b200.lang import build
    from pccl_b200.engine import LaunchEnvironments
    LaunchEnvironments.setOverride("PCCL_WORKSPACE_MB", "4")   # the environment is snapshotted at load
    try:
        e = Engine(0, 1); e.initEngine("cpu")
    finally:
        LaunchEnvironments.setOverride("PCCL_WORKSPACE_MB", "64")
    ir = build("oneshot_allreduce", 1)
    ir.buffers["scratch"] = 1
    e.regOp("big", ir, check=False)
    x = torch.zeros(2 << 20)
    with pytest.raises(RuntimeError, match="scratch"):
        e.exeOp("big", x, torch.empty_like(x))


def test_instruction_trace_is_chrome_trace_json(tmp_path):
    from pccl_b200.engine import Engine, LaunchEnvironments
    from pccl_b200.lang import build
    LaunchEnvironments.setOverride("PCCL_TRACE", "1")
    try:
        e = Engine(0, 1); e.initEngine("cpu")
    finally:
        LaunchEnvironments.setOverride("PCCL_TRACE", "0")
    e.regOp("ar", build("ring_allreduce", 1))
    x = torch.ones(1000); y = torch.zeros(1000)
    e.exeOp("ar", x, y)
    doc = e.trace(str(tmp_path / "t.json"))
    ev = doc["traceEvents"]
    assert ev and ev[0]["ph"] == "X" and ev[0]["name"] == "COPY" and ev[0]["args"]["bytes"] == 4000
    assert json.loads((tmp_path / "t.json").read_text())["traceEvents"] == ev
    assert e.trace()["traceEvents"] == []       # reading clears the record


def test_device_stamps_become_trace_events():
    """The interpreter kernel leaves two timer words per instruction; the engine pairs them with the program it
    launched.  Here the stamp buffer is made by hand: reached instructions get spans, END and the unreached do not."""
    import re
    from pccl_b200.engine import Engine
    from pccl_b200.lang import build
    e = Engine(0, 2); e.initEngine("cpu")
    e.regOp("ar", build("ring_allreduce", 2))
    in_bytes = 4 * 4096
    with pytest.raises(RuntimeError) as err:
        e._e.ingestDeviceTrace("ar", in_bytes, 1, [0])
    n = int(re.search(r"for (\d+) instructions", str(err.value)).group(1))
    assert n >= 6
    stamps = []
    for i in range(n):
        reached = i < n - 3                   # the last instructions never ran (a stream that gave up early)
        stamps += [1_000_000 + 100 * i, 1_000_000 + 100 * i + 40] if reached else [0, 0]
    e._e.ingestDeviceTrace("ar", in_bytes, 1, stamps)
    ev = e.trace()["traceEvents"]
    assert 0 < len(ev) <= n - 3 and all(x["name"] != "END" and x["cat"] == "ar" and x["dur"] == pytest.approx(0.04) for x in ev)
    assert [x["ts"] for x in ev] == sorted(x["ts"] for x in ev)
    moved = [x for x in ev if x["name"] in ("COPY", "REDUCE")]
    assert moved and all(x["args"]["bytes"] == in_bytes // 2 for x in moved)
    assert all(x["args"]["bytes"] == 0 for x in ev if x["name"] in ("NOTIFY", "WAIT"))
    with pytest.raises(RuntimeError, match="no operator"):
        e._e.ingestDeviceTrace("nope", in_bytes, 1, stamps)


def _runahead_rank(rank, world, port):
    """A sender that is never slowed down by its own work against a receiver that dawdles before every launch."""
    import time
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("p2p", build("send_recv", world, channels=1, device_type=DeviceType.CPU, src=0, dst=1))
    bad = 0
    t0 = time.monotonic()
    for it in range(6):
        if rank == 1:
            time.sleep(0.15)
        x = torch.full((2048,), float(it + 1))
        y = torch.zeros(2048)
        e.exeOp("p2p", x, y)
        if rank == 1:
            bad += int((y != it + 1).any())
    took = time.monotonic() - t0
    e.exitCluster()
    return bad, took


def test_a_rank_that_only_sends_cannot_overrun_the_receivers_workspace():
    """Workspace halves alternate by launch, so a sender two launches ahead would overwrite data its receiver has not
    taken yet: the rooted programs end with an acknowledgement, which holds the sender to at most one launch ahead."""
    res = run_ranks(_runahead_rank, 2, env={"PCCL_WORKSPACE_MB": "8"})
    assert res[1][0] == 0
    assert res[0][1] > 0.5          # the sender was held back by the receiver's pace (6 x 0.15 s)


def _rooted_api_rank(rank, world, port):
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.ops import collectives as C
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    n = 3000 + 5
    mine = torch.arange(n, dtype=torch.float32) + 1000 * rank
    errs = {}
    for it in range(2):                              # the second round reuses the registered programs
        for algo in ("direct", "tree", "scatter_allgather", "auto"):
            t = mine.clone() + it
            C.broadcast(e, t, root=1, algo=algo)
            errs["broadcast_" + algo] = (t - (torch.arange(n) + 1000 + it)).abs().max().item()
        for algo in ("tree", "pieces", "auto"):
            out = torch.full((n,), -1.0)
            C.reduce(e, mine + it, out, root=2, algo=algo)
            want = sum(torch.arange(n, dtype=torch.float32) + 1000 * r + it for r in range(world)) if rank == 2 else torch.full((n,), -1.0)
            errs["reduce_" + algo] = (out - want).abs().max().item()
        big = torch.arange(n * world, dtype=torch.float32) + 7 * rank + it
        part = torch.zeros(n)
        C.scatter(e, big, part, root=0)
        errs["scatter"] = (part - (torch.arange(n * world, dtype=torch.float32) + it)[rank * n:(rank + 1) * n]).abs().max().item()
        allv = torch.full((n * world,), -1.0)
        C.gather(e, mine + it, allv, root=1, width=2)
        want = torch.cat([torch.arange(n, dtype=torch.float32) + 1000 * r + it for r in range(world)]) if rank == 1 else torch.full((n * world,), -1.0)
        errs["gather"] = (allv - want).abs().max().item()
        got = torch.full((n,), -1.0)
        C.send_recv(e, mine + it, got, src=2, dst=0)
        want = torch.arange(n, dtype=torch.float32) + 2000 + it if rank == 0 else torch.full((n,), -1.0)
        errs["send_recv"] = (got - want).abs().max().item()
        if max(errs.values()) > 0:
            break
    ops = sorted(k for k in e.stats()["ops"] if k.startswith("lib."))
    e.exitCluster()
    return errs, ops


def test_rooted_collectives_through_the_ops_api_on_cpu_ranks():
    res = run_ranks(_rooted_api_rank, 3, env={"PCCL_WORKSPACE_MB": "16"}, timeout=120)
    for r in range(3):
        errs, ops = res[r]
        assert max(errs.values()) == 0, (r, errs)
        assert len(ops) == 8            # one registration per (program, arguments), reused by the second round and by "auto"
    with pytest.raises(ValueError):
        from pccl_b200.ops import collectives as C

        class _E:
            world = 4
        C.scatter(_E(), torch.zeros(7), torch.zeros(2))


def _traced_rank(rank, world, port):
    import torch
    from pccl_b200.engine import Engine, LaunchEnvironments
    from pccl_b200.lang import DeviceType, build
    LaunchEnvironments.setOverride("PCCL_TRACE", "1")
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, device_type=DeviceType.CPU))
    x = torch.ones(4096); y = torch.zeros(4096)
    e.exeOp("ar", x, y)
    doc = e.trace()
    e.exitCluster()
    return doc


def test_traces_of_all_ranks_merge_into_one_document(tmp_path):
    from pccl_b200.utils.trace import merge_traces, summarize
    res = run_ranks(_traced_rank, 2, env={"PCCL_WORKSPACE_MB": "8"})
    merged = merge_traces([res[0], res[1]], out=str(tmp_path / "all.json"), align=True)
    ev = merged["traceEvents"]
    assert {e["pid"] for e in ev} == {0, 1}
    assert sorted(e["args"]["name"] for e in ev if e["ph"] == "M") == ["rank 0", "rank 1"]
    for pid in (0, 1):
        assert min(e["ts"] for e in ev if e["ph"] == "X" and e["pid"] == pid) == 0.0
    stats = summarize(str(tmp_path / "all.json"))
    assert stats["COPY"]["count"] >= 4 and stats["REDUCE"]["count"] == 2 and stats["REDUCE"]["bytes"] == 2 * 8192
    assert stats["WAIT"]["bytes"] == 0 and stats["COPY"]["gbs"] > 0


def _interleaved_rank(rank, world, port):
    """all-reduce, then a send between two OTHER ranks, then the all-reduce again, on one workspace lane; one rank is
    slowed down before every instruction."""
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, channels=1, device_type=DeviceType.CPU))
    e.regOp("p2p", build("send_recv", world, channels=1, device_type=DeviceType.CPU, src=0, dst=1))
    g = torch.Generator().manual_seed(11)
    xs = [torch.rand(3 * 4096, generator=g) for _ in range(world)]
    errs = []
    for it in range(4):
        y = torch.zeros_like(xs[rank])
        e.exeOp("ar", xs[rank] + it, y)
        errs.append((y - (sum(xs) + it * world)).abs().max().item())
        z = torch.zeros(64)
        e.exeOp("p2p", torch.full((64,), float(it)), z)        # ranks other than 0 and 1 run an empty program
        if rank == 1:
            errs.append((z - it).abs().max().item())
    e.exitCluster()
    return max(errs)


def test_programs_interleaved_on_one_lane_do_not_overrun_a_slow_ranks_scratch():
    """The scratch half of launch n is the half of launch n - 2.  Between two all-reduces sits a program that does not
    involve rank 2, so nothing in the programs themselves keeps rank 2 from starting the second all-reduce while the
    slowed-down rank still reads the first one's scratch; the engine's per-lane turn-taking does."""
    res = run_ranks(_interleaved_rank, 3, env={"PCCL_WORKSPACE_MB": "8", "PCCL_EXEC_DELAY_US": "3000", "PCCL_EXEC_DELAY_RANK": "0"},
                    timeout=300)
    for r in range(3):
        assert res[r] < 1e-5, res


def _rebind_rank(rank, world, port):
    """Launch, rebind to the same world (every counter starts over), reconnect, launch again."""
    import torch
    from _ranks import free_port  # noqa: F401
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, channels=1, device_type=DeviceType.CPU))
    xs = [torch.arange(2048, dtype=torch.float32) * (r + 1) for r in range(world)]
    errs = []
    for it in range(3):
        y = torch.zeros(2048)
        e.exeOp("ar", xs[rank], y)
        errs.append((y - sum(xs)).abs().max().item())
    docs_before = e.exportEndpoint()
    e.exitCluster()
    e.rebind(rank, world)
    e.joinCluster(f"127.0.0.1:{port + 1}")
    for it in range(3):                      # after a rebind the signal words were cleared and the epochs restarted
        y = torch.zeros(2048)
        st = e.exeOp("ar", xs[rank] + it, y)
        errs.append(float(st))
        errs.append((y - (sum(xs) + it * world)).abs().max().item())
    e.exitCluster()
    return max(errs), len(docs_before) > 0


def test_rebind_restarts_every_counter_and_the_engine_runs_again():
    res = run_ranks(_rebind_rank, 2, env={"PCCL_WORKSPACE_MB": "8"})
    for r in (0, 1):
        assert res[r][0] < 1e-5, res
