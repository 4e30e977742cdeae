"""Elastic recovery: what the survivors do after a rank has left.

The control plane announces a departure on the host (``QuitNode``: a goodbye, a dropped connection, or missed
heartbeats) and collectives of the old world end in ``PcclTimeout`` instead of hanging.  ``recover`` then performs the
steps the reference only names in its event vocabulary (``ResizeWorld`` ..., include/cluster/daemon.h:16-25): the
master renumbers the survivors, every survivor tears its engine down, builds one of the new world size, joins the new
cluster, and registers the programs of the new size -- each taken from a factory, so a schedule is re-synthesised (or
fetched from the on-disk cache) for the world it will actually run in.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Optional, Union

from . import Engine, PcclError

ProgramFactory = Callable[[int], Union[object, dict, str]]     # world size -> CollectiveIR / schedule dict / JSON / path


def wait_for_resize(engine: Engine, survivors: int, timeout_s: float = 10.0) -> Dict[int, int]:
    """Old rank -> new rank, as announced by the master (rank 0 announces it itself)."""
    if engine.rank == 0:
        time.sleep(0.3)                      # lets every survivor see the departure first
        return engine.resize_world()
    deadline = time.time() + timeout_s
    mapping: Dict[int, int] = {}
    while time.time() < deadline:
        mapping = engine.last_resize()
        if len(mapping) == survivors:
            return mapping
        time.sleep(0.05)
    raise PcclError(f"no ResizeWorld for {survivors} survivors within {timeout_s} s (got {mapping})")


def recover(engine: Engine, next_master: str, programs: Dict[str, ProgramFactory], *, device: Optional[str] = None,
            heap_bytes: int = 0, timeout_s: float = 10.0, spares: int = 0) -> Engine:
    """Called by every survivor once ``engine.alive_ranks()`` has shrunk.  Returns the engine of the new world with
    ``programs`` registered (``{name: factory(new_world)}``).  ``next_master`` is the endpoint ("host:port") on which
    the new rank 0 serves the new cluster; the old cluster is left.

    ``spares``: processes that stood by and now take the ranks after the survivors' (``join_as_spare``), so that a job
    can go on at its old size: the replacement that the reference's ReplaceOld / BeReplaced events stand for
    (include/cluster/daemon.h:16-25), done by forming the new world instead of patching the old one."""
    alive = engine.alive_ranks()
    if engine.rank not in alive:
        raise PcclError("recover: this rank is not among the survivors")
    mapping = wait_for_resize(engine, len(alive), timeout_s)
    new_rank, new_world = mapping[engine.rank], len(mapping) + int(spares)
    dev = device or engine.device
    engine.exitCluster()
    fresh = Engine(new_rank, new_world)
    fresh.initEngine(dev, heap_bytes) if heap_bytes else fresh.initEngine(dev)
    fresh.joinCluster(next_master)
    for name, factory in programs.items():
        fresh.regOp(name, factory(new_world))
    return fresh


def join_as_spare(next_master: str, new_rank: int, new_world: int, programs: Dict[str, ProgramFactory], *,
                  device: str = "auto", heap_bytes: int = 0, timeout_ms: int = 60000) -> Engine:
    """The stand-by's side of ``recover(..., spares=k)``: wait for the new world's master (the connection is retried
    until ``timeout_ms``), join as ``new_rank`` (survivors come first, spares after them) and register the programs."""
    fresh = Engine(new_rank, new_world)
    fresh.initEngine(device, heap_bytes) if heap_bytes else fresh.initEngine(device)
    fresh.joinCluster(next_master, timeout_ms)
    for name, factory in programs.items():
        fresh.regOp(name, factory(new_world))
    return fresh


def cached_schedule(collective: str, nbytes: int, topology_of: Callable[[int], object], cache=None, **kw) -> ProgramFactory:
    """A program factory that asks the schedule cache (and through it the MILP synthesiser) for ``collective`` on the
    topology of the new world: ``recover(..., programs={"ar": cached_schedule("allreduce", 1 << 20, Topology.ring)})``."""
    def factory(world: int):
        from ..synth import ScheduleCache
        c = cache or ScheduleCache()
        return c.get_or_synthesize(collective, topology_of(world), nbytes, **kw)
    return factory


__all__ = ["recover", "join_as_spare", "wait_for_resize", "cached_schedule"]
