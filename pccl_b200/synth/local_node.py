"""What this host looks like, and a cache of measured topologies.

The reference reserves two empty headers for this (include/topology/local_node.h, include/topology/cache.h) and
vendors hwloc for it without a line that uses it.  Here the host is read from sysfs (CPUs, NUMA nodes, the NUMA node
of each GPU's PCI function) and from the CUDA runtime (GPUs, peer access), and a measured bandwidth matrix
(``probe_topology``) is kept on disk per host, so that a job measures its links once per machine and not per start.
Nothing here needs a GPU: without one the node has no devices and ``to_topology`` has nothing to return.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional

from .topology import Topology


@dataclass
class GpuInfo:
    index: int
    name: str
    sm_count: int
    memory_bytes: int
    pci_bus_id: str                # "0000:1b:00.0" (lower case, as sysfs spells it); "" when unknown
    numa_node: int                 # -1 when the platform does not say
    peers: List[int] = field(default_factory=list)      # devices this one can load from and store to directly


@dataclass
class LocalNode:
    host_id: str
    cpus: int
    numa_cpus: Dict[int, List[int]]          # NUMA node -> CPU ids
    gpus: List[GpuInfo]

    # ---- probing ----------------------------------------------------------------------------------------------
    @staticmethod
    def probe(sysfs: str = "/sys", proc: str = "/proc", cuda=None) -> "LocalNode":
        """``cuda``: an object with ``device_count()``, ``get_device_properties(i)`` and
        ``can_device_access_peer(a, b)`` (``torch.cuda`` when it is usable, else no GPUs); a stand-in serves the tests."""
        host_id = os.environ.get("PCCL_HOST_ID") or _read(os.path.join(proc, "sys", "kernel", "random", "boot_id")) or "unknown"
        numa_cpus: Dict[int, List[int]] = {}
        node_dir = os.path.join(sysfs, "devices", "system", "node")
        if os.path.isdir(node_dir):
            for entry in sorted(os.listdir(node_dir)):
                if entry.startswith("node") and entry[4:].isdigit():
                    numa_cpus[int(entry[4:])] = parse_cpu_list(_read(os.path.join(node_dir, entry, "cpulist")))
        cpus = sum(len(v) for v in numa_cpus.values()) or (os.cpu_count() or 1)
        if cuda is None:
            cuda = _torch_cuda()
        gpus: List[GpuInfo] = []
        n = cuda.device_count() if cuda is not None else 0
        for i in range(n):
            p = cuda.get_device_properties(i)
            bus = _bus_id(p)
            numa = _read(os.path.join(sysfs, "bus", "pci", "devices", bus, "numa_node")) if bus else ""
            peers = [j for j in range(n) if j != i and cuda.can_device_access_peer(i, j)]
            gpus.append(GpuInfo(i, str(getattr(p, "name", "gpu")), int(getattr(p, "multi_processor_count", 0)),
                                int(getattr(p, "total_memory", 0)), bus, int(numa) if numa.lstrip("-").isdigit() else -1, peers))
        return LocalNode(host_id, cpus, numa_cpus, gpus)

    # ---- use --------------------------------------------------------------------------------------------------
    def fully_peered(self) -> bool:
        """Every GPU reaches every other directly: what a switch (or a full mesh) gives."""
        n = len(self.gpus)
        return n > 0 and all(sorted(g.peers) == [j for j in range(n) if j != g.index] for g in self.gpus)

    def to_topology(self, port_gbs: float = 770.0, pcie_gbs: float = 50.0) -> Optional[Topology]:
        """Nominal model before anything is measured: pairs with peer access at the port rate, the rest at a host
        bridge's rate.  ``None`` without GPUs."""
        n = len(self.gpus)
        if n == 0:
            return None
        if self.fully_peered():
            return Topology.nvswitch(n, port_gbs)
        gbs = [[0.0 if a == b else (port_gbs if b in self.gpus[a].peers else pcie_gbs) for b in range(n)] for a in range(n)]
        return Topology.from_matrix(gbs, port_gbs=port_gbs)

    def cpus_near(self, gpu: int) -> List[int]:
        """CPUs of the GPU's NUMA node (all CPUs when the platform does not say): where its host threads belong."""
        node = self.gpus[gpu].numa_node
        return list(self.numa_cpus.get(node, [])) or [c for v in self.numa_cpus.values() for c in v] or list(range(self.cpus))

    def to_json(self) -> str:
        return json.dumps(asdict(self), sort_keys=True)

    @staticmethod
    def from_json(text: str) -> "LocalNode":
        d = json.loads(text)
        return LocalNode(d["host_id"], d["cpus"], {int(k): v for k, v in d["numa_cpus"].items()},
                         [GpuInfo(**g) for g in d["gpus"]])


def parse_cpu_list(text: str) -> List[int]:
    """sysfs list format: "0-3,8,10-11"."""
    out: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.extend(range(int(lo), int(hi or lo) + 1))
    return out


def _read(path: str) -> str:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return ""


def _bus_id(props) -> str:
    """torch gives domain, bus and device numbers; sysfs names the function "dddd:bb:dd.0"."""
    try:
        return f"{int(props.pci_domain_id):04x}:{int(props.pci_bus_id):02x}:{int(props.pci_device_id):02x}.0"
    except (AttributeError, TypeError, ValueError):
        return ""


def _torch_cuda():
    try:
        import torch
        return torch.cuda if torch.cuda.is_available() else None
    except Exception:  # noqa: BLE001 - a host without a usable CUDA runtime simply has no GPUs
        return None


# -------------------------------------------------------------------------------------------------------------------
# cache of measured topologies
# -------------------------------------------------------------------------------------------------------------------
def topology_to_doc(t: Topology) -> dict:
    return {"n": t.n, "links": [[a, b, v] for (a, b), v in sorted(t.link_bw.items())], "egress": list(t.egress_bw),
            "ingress": list(t.ingress_bw), "alpha": t.alpha, "name": t.name, "rotation_symmetric": t.rotation_symmetric,
            "shared": [[[list(l) for l in links], cap] for links, cap in t.shared_caps]}


def topology_from_doc(d: dict) -> Topology:
    return Topology(int(d["n"]), {(int(a), int(b)): float(v) for a, b, v in d["links"]}, [float(x) for x in d["egress"]],
                    [float(x) for x in d["ingress"]], float(d["alpha"]), str(d["name"]), bool(d["rotation_symmetric"]),
                    [(tuple((int(a), int(b)) for a, b in links), float(cap)) for links, cap in d.get("shared", [])])


class TopologyCache:
    """One file per (host, world size) under the schedule cache's directory.  A host that reboots gets a new boot id
    and therefore measures again, which is what one wants after hardware was reseated."""

    def __init__(self, directory: Optional[str] = None):
        self.dir = directory or os.environ.get("PCCL_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "pccl_b200")
        os.makedirs(self.dir, exist_ok=True)
        self.hits = self.misses = 0

    def path(self, host_id: str, world: int) -> str:
        safe = "".join(c if c.isalnum() else "_" for c in host_id)[:64]
        return os.path.join(self.dir, f"topology_{safe}_{world}.json")

    def load(self, host_id: str, world: int) -> Optional[Topology]:
        try:
            with open(self.path(host_id, world)) as f:
                return topology_from_doc(json.load(f))
        except (OSError, ValueError, KeyError):
            return None

    def store(self, host_id: str, topo: Topology) -> str:
        p = self.path(host_id, topo.n)
        tmp = p + f".tmp{os.getpid()}"
        with open(tmp, "w") as f:
            json.dump(topology_to_doc(topo), f)
        os.replace(tmp, p)
        return p

    def get_or_measure(self, host_id: str, world: int, measure: Callable[[], Topology]) -> Topology:
        """``measure`` is called on a miss (``lambda: probe_topology(engine)`` on a GPU job; every rank calls it,
        since the measurement is itself collective, and every rank of the host writes the same file)."""
        t = self.load(host_id, world)
        if t is not None:
            self.hits += 1
            return t
        self.misses += 1
        t = measure()
        self.store(host_id, t)
        return t


__all__ = ["GpuInfo", "LocalNode", "TopologyCache", "parse_cpu_list", "topology_to_doc", "topology_from_doc"]
