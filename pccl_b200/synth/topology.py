"""Topology model fed to the synthesiser.

The reference reserves two empty headers for this (include/topology/cache.h, local_node.h) and vendors
hwloc without using it; its IR carries ``Link.bandwidth`` / ``Link.latency`` (pccl/lang/chunk.py:39-44).
On an NVSwitch machine every GPU pair has the same bandwidth and what limits a schedule is each GPU's
port (egress and ingress), so the model has both per-link and per-port capacities.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class Topology:
    n: int
    link_bw: Dict[Tuple[int, int], float]            # bytes/s for every usable directed pair
    egress_bw: List[float]                           # bytes/s per device port, sending
    ingress_bw: List[float]                          # bytes/s per device port, receiving
    alpha: float = 4.0e-6                            # seconds per step (launch + flag round trip)
    name: str = "custom"
    rotation_symmetric: bool = False                 # relabelling r -> r+1 (mod n) maps the topology onto itself
    # Extra shared capacities: (directed links that share it, bytes/s).  A host's network card is one: every flow that
    # leaves the host goes through it, whichever GPU sends and whichever remote GPU receives.
    shared_caps: List[Tuple[Tuple[Tuple[int, int], ...], float]] = field(default_factory=list)

    @staticmethod
    def nvswitch(n: int, port_gbs: float = 770.0, alpha: float = 4.0e-6) -> "Topology":
        """All-to-all through a switch: any pair at full port rate, ports shared by all of a GPU's flows."""
        bw = port_gbs * 1e9
        return Topology(n, {(a, b): bw for a in range(n) for b in range(n) if a != b}, [bw] * n, [bw] * n, alpha,
                        f"nvswitch{n}", True)

    @staticmethod
    def ring(n: int, link_gbs: float = 50.0, alpha: float = 4.0e-6, bidirectional: bool = True) -> "Topology":
        bw = link_gbs * 1e9
        links = {}
        for a in range(n):
            links[(a, (a + 1) % n)] = bw
            if bidirectional:
                links[(a, (a - 1) % n)] = bw
        port = bw * (2 if bidirectional else 1)
        return Topology(n, links, [port] * n, [port] * n, alpha, f"ring{n}", True)

    @staticmethod
    def from_matrix(gbs: List[List[float]], alpha: float = 4.0e-6, port_gbs: Optional[float] = None) -> "Topology":
        """From a measured pairwise copy-bandwidth matrix in GB/s (0 or None = no direct path)."""
        n = len(gbs)
        links = {(a, b): gbs[a][b] * 1e9 for a in range(n) for b in range(n) if a != b and gbs[a][b]}
        port = [(port_gbs or max((gbs[a][b] or 0) for b in range(n) if b != a)) * 1e9 for a in range(n)]
        sym = all(abs((gbs[a][b] or 0) - (gbs[(a + 1) % n][(b + 1) % n] or 0)) <= 0.1 * max(1.0, gbs[a][b] or 0)
                  for a in range(n) for b in range(n) if a != b)
        return Topology(n, links, list(port), list(port), alpha, "measured", sym)

    @staticmethod
    def two_level(hosts: int, per_host: int, intra_gbs: float = 770.0, nic_gbs: float = 50.0, alpha: float = 4.0e-6,
                  inter_alpha: float = 12.0e-6) -> "Topology":
        """``hosts`` machines of ``per_host`` GPUs: inside a machine every pair at the NVSwitch port rate, between
        machines every pair at the network card's rate, and one card per machine and direction shared by all of its
        GPUs' remote flows.  Rank r sits on host r // per_host."""
        n = hosts * per_host
        intra, nic = intra_gbs * 1e9, nic_gbs * 1e9
        host = lambda r: r // per_host  # noqa: E731
        links = {(a, b): (intra if host(a) == host(b) else nic) for a in range(n) for b in range(n) if a != b}
        caps = []
        for h in range(hosts):
            out = tuple((a, b) for (a, b) in sorted(links) if host(a) == h and host(b) != h)
            inn = tuple((a, b) for (a, b) in sorted(links) if host(b) == h and host(a) != h)
            if out:
                caps.append((out, nic))
                caps.append((inn, nic))
        t = Topology(n, links, [intra] * n, [intra] * n, max(alpha, inter_alpha) if hosts > 1 else alpha,
                     f"hosts{hosts}x{per_host}", False, caps)
        return t

    def fingerprint(self) -> str:
        doc = {"n": self.n, "links": sorted((a, b, round(v / 1e9)) for (a, b), v in self.link_bw.items()),
               "shared": sorted((sorted(ls), round(c / 1e9)) for ls, c in self.shared_caps),
               "egress": [round(v / 1e9) for v in self.egress_bw], "ingress": [round(v / 1e9) for v in self.ingress_bw],
               "alpha_us": round(self.alpha * 1e6, 1)}
        return hashlib.sha1(json.dumps(doc, sort_keys=True).encode()).hexdigest()[:16]


def probe_topology(engine, nbytes: int = 64 << 20, iters: int = 3) -> Topology:
    """Measures this rank's copy bandwidth from every peer's heap (device-timed) and all-gathers the rows
    into a matrix.  Needs a connected CUDA engine and an initialised torch.distributed group."""
    import torch
    import torch.distributed as dist
    from .._native import C
    n, me = engine.world, engine.rank
    dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    row = [0.0] * n
    s = torch.cuda.current_stream().cuda_stream
    for p in range(n):
        if p == me:
            continue
        src = engine.raw.heapBase(p)
        C.memcpy_d2d(dst.data_ptr(), src, nbytes, s)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            C.memcpy_d2d(dst.data_ptr(), src, nbytes, s)
        b.record()
        b.synchronize()
        row[p] = nbytes * iters / (a.elapsed_time(b) * 1e-3) / 1e9
    rows = [None] * n
    dist.all_gather_object(rows, row)
    return Topology.from_matrix(rows)
