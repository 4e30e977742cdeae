"""Failure detection and elastic membership on CPU ranks.  Every failure is made on the host: a rank
that exits, a rank whose control connection is dropped, a rank that goes silent, a rank that never
joins a collective.  No GPU takes part."""
import time

import pytest

from _ranks import run_ranks


def _leaver(rank, world, port, mode):
    import torch
    from pccl_b200.engine import Engine, PcclTimeout
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("direct_allreduce", world, device_type=DeviceType.CPU))
    x = torch.full((1024,), float(rank + 1)); y = torch.empty_like(x)
    e.exeOp("ar", x, y)
    assert y[0].item() == sum(range(1, world + 1))
    victim = world - 1
    if rank == victim:
        if mode == "graceful":
            e.exitCluster()
        elif mode == "close":
            e.inject_fault("close")          # socket dropped without a goodbye
            time.sleep(1.0)
        elif mode == "silent":
            e.inject_fault("silence")        # alive but no heartbeats
            time.sleep(3.0)
        return {"left": True}
    # survivors: the departure is announced on the host (QuitNode), before any further launch
    assert e.wait_for_departure(victim, 8000), "departure was not detected"
    assert victim not in e.alive_ranks()
    out = {"alive": e.alive_ranks()}
    # a collective of the old world cannot complete: the bounded wait returns a time-out status
    try:
        e.exeOp("ar", x, y)
        out["second"] = "completed"
    except PcclTimeout:
        out["second"] = "timeout"
    # shrink: the master renumbers the survivors and announces the new world
    if rank == 0:
        time.sleep(0.3)
        mapping = e.resize_world()
    else:
        deadline = time.time() + 8
        mapping = {}
        while time.time() < deadline and len(mapping) != world - 1:
            mapping = e.last_resize()
            time.sleep(0.05)
    out["mapping"] = mapping
    e.exitCluster()
    return out


@pytest.mark.parametrize("mode", ["graceful", "close", "silent"])
def test_departure_is_detected_and_world_shrinks(mode):
    env = {"PCCL_WORKSPACE_MB": "8", "PCCL_WAIT_TIMEOUT_MS": "1500", "PCCL_HEARTBEAT_MS": "100", "PCCL_HEARTBEAT_MISSES": "5"}
    res = run_ranks(_leaver, 3, args=(mode,), env=env, timeout=60)
    for r in (0, 1):
        assert res[r]["alive"] == [0, 1]
        assert res[r]["second"] == "timeout"
        assert res[r]["mapping"] == {0: 0, 1: 1}


def _rejoin(rank, world, port, phase_port):
    """After a shrink the survivors build a new engine of the new world and run again."""
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    if rank == world - 1:
        e.exitCluster()
        return {"left": True}
    assert e.wait_for_departure(world - 1, 8000)
    e.exitCluster()
    new_world = world - 1
    e2 = Engine(rank, new_world); e2.initEngine("cpu"); e2.joinCluster(f"127.0.0.1:{phase_port}")
    e2.regOp("ar", build("ring_allreduce", new_world, device_type=DeviceType.CPU))
    x = torch.full((256,), float(rank + 1)); y = torch.empty_like(x)
    e2.exeOp("ar", x, y)
    e2.exitCluster()
    return {"sum": y[0].item()}


def test_survivors_run_in_the_resized_world():
    from _ranks import free_port
    res = run_ranks(_rejoin, 3, args=(free_port(),), env={"PCCL_WORKSPACE_MB": "8", "PCCL_HEARTBEAT_MS": "100"}, timeout=60)
    assert res[0]["sum"] == 3.0 and res[1]["sum"] == 3.0


def _recover(rank, world, port, next_port, cache_dir):
    """The packaged flow: departure -> time-out -> resize -> new engine with re-synthesised schedules."""
    import torch
    from pccl_b200.engine import Engine, PcclTimeout
    from pccl_b200.engine.elastic import cached_schedule, recover
    from pccl_b200.lang import DeviceType, build
    from pccl_b200.synth import ScheduleCache, Topology
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("direct_allreduce", world, device_type=DeviceType.CPU))
    x = torch.full((512,), float(rank + 1)); y = torch.empty_like(x)
    e.exeOp("ar", x, y)
    if rank == 1:                            # a middle rank leaves: the survivors are renumbered 0, 1
        e.exitCluster()
        return {"left": True}
    assert e.wait_for_departure(1, 8000)
    try:
        e.exeOp("ar", x, y)
        second = "completed"
    except PcclTimeout:
        second = "timeout"
    cache = ScheduleCache(cache_dir)
    e2 = recover(e, f"127.0.0.1:{next_port}", {"ar": cached_schedule("allreduce", 1 << 16, lambda n: Topology.ring(n, 50.0), cache)})
    y2 = torch.empty_like(x)
    e2.exeOp("ar", x, y2)
    out = {"second": second, "new_rank": e2.rank, "new_world": e2.world, "sum": y2[0].item(), "misses": cache.misses}
    e2.exitCluster()
    return out


def test_recover_builds_the_new_world_with_resynthesised_schedules(tmp_path):
    from _ranks import free_port
    res = run_ranks(_recover, 3, args=(free_port(), str(tmp_path)), timeout=90,
                    env={"PCCL_WORKSPACE_MB": "8", "PCCL_WAIT_TIMEOUT_MS": "1500", "PCCL_HEARTBEAT_MS": "100", "PCCL_HEARTBEAT_MISSES": "5"})
    assert res[0]["second"] == res[2]["second"] == "timeout"
    assert (res[0]["new_rank"], res[2]["new_rank"]) == (0, 1) and res[0]["new_world"] == res[2]["new_world"] == 2
    assert res[0]["sum"] == res[2]["sum"] == 1.0 + 3.0          # ranks 0 and 2 of the old world
    assert res[0]["misses"] + res[2]["misses"] >= 1             # the schedule for two ranks did not exist before


def _never_joins(rank, world, port):
    import torch
    from pccl_b200.engine import Engine, PcclTimeout
    from pccl_b200.lang import DeviceType, build
    e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
    e.regOp("ar", build("ring_allreduce", world, device_type=DeviceType.CPU))
    x = torch.ones(64); y = torch.zeros(64)
    status = "skipped"
    if rank == 0:
        try:
            e.exeOp("ar", x, y)
            status = "completed"
        except PcclTimeout:
            status = "timeout"
        st = e.stats()["ops"]["ar"]
        assert st["timeouts"] == 1
    else:
        time.sleep(1.5)           # rank 1 never launches the collective
    e.exitCluster()
    return status


def test_wait_on_a_rank_that_never_launches_times_out():
    res = run_ranks(_never_joins, 2, env={"PCCL_WORKSPACE_MB": "8", "PCCL_WAIT_TIMEOUT_MS": "500"}, timeout=60)
    assert res[0] == "timeout"


def test_join_times_out_when_a_rank_is_missing():
    from pccl_b200.engine import Engine
    from _ranks import free_port
    e = Engine(0, 2); e.initEngine("cpu")
    t0 = time.time()
    with pytest.raises(RuntimeError, match="1 of 2"):
        e.joinCluster(f"127.0.0.1:{free_port()}", 700)
    assert time.time() - t0 < 5
    e.exitCluster()


def _recover_with_spare(rank, nprocs, port, next_port):
    """Three ranks and a stand-by process; rank 1 leaves, the stand-by takes the last rank of a new world of three."""
    import torch
    from pccl_b200.engine import Engine
    from pccl_b200.engine.elastic import join_as_spare, recover
    from pccl_b200.lang import DeviceType, build
    world = nprocs - 1
    programs = {"ar": lambda n: build("direct_allreduce", n, device_type=DeviceType.CPU)}
    value = float(10 * (rank + 1))
    x = torch.full((512,), value); y = torch.empty_like(x)
    if rank == world:                        # the stand-by: joins whenever the new world's master appears
        e2 = join_as_spare(f"127.0.0.1:{next_port}", world - 1, world, programs, device="cpu", timeout_ms=60000)
    else:
        e = Engine(rank, world); e.initEngine("cpu"); e.joinCluster(f"127.0.0.1:{port}")
        e.regOp("ar", programs["ar"](world))
        e.exeOp("ar", x, y)
        assert y[0].item() == 10.0 + 20.0 + 30.0
        if rank == 1:
            e.exitCluster()
            return {"left": True}
        assert e.wait_for_departure(1, 8000)
        e2 = recover(e, f"127.0.0.1:{next_port}", programs, spares=1)
    e2.exeOp("ar", x, y)
    out = {"new_rank": e2.rank, "new_world": e2.world, "sum": y[0].item()}
    e2.exitCluster()
    return out


def test_a_stand_by_process_takes_the_place_of_a_rank_that_left():
    from _ranks import free_port
    res = run_ranks(_recover_with_spare, 4, args=(free_port(),), timeout=120,
                    env={"PCCL_WORKSPACE_MB": "8", "PCCL_WAIT_TIMEOUT_MS": "3000", "PCCL_HEARTBEAT_MS": "100", "PCCL_HEARTBEAT_MISSES": "5"})
    assert res[1] == {"left": True}
    assert [res[r]["new_rank"] for r in (0, 2, 3)] == [0, 1, 2] and all(res[r]["new_world"] == 3 for r in (0, 2, 3))
    assert all(res[r]["sum"] == 10.0 + 30.0 + 40.0 for r in (0, 2, 3))       # old ranks 0 and 2, and the stand-by
