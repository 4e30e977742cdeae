"""On-disk cache of synthesised schedules, keyed by (collective, world, size bucket, chunks, topology
fingerprint) through the library's FNV-1a hash (csrc/common/hash.h; the reference has the same hash,
csrc/common/hash.cc:3-15, and never uses it).  A cached entry is a schedule document ready for
``Engine.regOp``; nothing else of a collective library's state needs to survive a restart."""
from __future__ import annotations

import json
import os
from typing import Optional

from ..lang import to_schedule
from .milp import synthesize
from .topology import Topology


def _fnv1a(text: str) -> int:
    try:
        from .._native import C
        return int(C.utils.fnv1a(text))
    except Exception:  # noqa: BLE001 - pure-python fallback keeps the cache usable without the extension
        h = 14695981039346656037
        for b in text.encode():
            h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        return h


class ScheduleCache:
    def __init__(self, directory: Optional[str] = None):
        self.dir = directory or os.environ.get("PCCL_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "pccl_b200")
        os.makedirs(self.dir, exist_ok=True)
        self.hits = self.misses = 0

    @staticmethod
    def size_bucket(nbytes: int) -> int:
        return max(0, int(nbytes).bit_length() - 1)        # floor(log2)

    def key(self, collective: str, topo: Topology, nbytes: int, chunks: int, root: Optional[int] = None) -> str:
        text = f"{collective}|{topo.n}|{self.size_bucket(nbytes)}|{chunks}|{topo.fingerprint()}"
        if root is not None:                 # rooted collectives: one schedule per root
            text += f"|root{root}"
        return f"{_fnv1a(text):016x}"

    def path(self, key: str) -> str:
        return os.path.join(self.dir, f"{key}.json")

    def get_or_synthesize(self, collective: str, topo: Topology, nbytes: int, chunks: int = 1, **kw) -> dict:
        k = self.key(collective, topo, nbytes, chunks, kw.get("root") if collective in ("broadcast", "reduce") else None)
        p = self.path(k)
        if os.path.exists(p):
            self.hits += 1
            with open(p) as f:
                return json.load(f)
        self.misses += 1
        res = synthesize(collective, topo, nbytes, chunks=chunks, **kw)
        doc = to_schedule(res.ir)
        tmp = p + f".tmp{os.getpid()}"
        with open(tmp, "w") as f:
            json.dump(doc, f)
        os.replace(tmp, p)
        return doc
