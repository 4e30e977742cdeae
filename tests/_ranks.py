"""Helper that runs a function as N CPU ranks in child processes and collects their results."""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
import traceback


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(fn, rank, world, port, env, q, args):
    try:
        os.environ.update(env)
        q.put((rank, "ok", fn(rank, world, port, *args)))
    except BaseException as e:  # noqa: BLE001 - report everything to the parent
        q.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def run_ranks(fn, world, args=(), env=None, timeout=120, allow_missing=()):
    """Returns {rank: result}.  Raises if a rank failed (ranks in `allow_missing` may die silently)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, dict(env or {}), q, args)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    want = world - len(allow_missing)
    try:
        while len([r for r in results if r not in allow_missing]) < want:
            rank, status, payload = q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return results
