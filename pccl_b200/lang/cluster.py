"""Cluster descriptions for collective programs (the reference's ``pccl/lang/cluster.py`` is an empty file).

A ``Cluster`` is the device-and-link graph that a ``CollectiveIR`` carries (chunk.py:32-44 in the reference:
``Device`` and ``Link`` records), built once and stamped onto any number of programs, and convertible to the
``Topology`` the MILP synthesiser consumes, so that the program, its verifier (port loads) and the synthesiser
all talk about the same machine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .ir import CollectiveIR, Device, DeviceType, Link


@dataclass
class Cluster:
    devices: List[Device] = field(default_factory=list)
    links: List[Link] = field(default_factory=list)
    name: str = "cluster"

    # -- canned shapes --------------------------------------------------------------------------
    @staticmethod
    def nvswitch(n: int, link_gbs: float = 770.0, latency: float = 2.0e-6, device_type: DeviceType = DeviceType.CUDA) -> "Cluster":
        """n GPUs behind an NVSwitch: every ordered pair has a link at the full per-direction port rate."""
        c = Cluster([Device(r, device_type) for r in range(n)], [], f"nvswitch{n}")
        c.links = [Link(a, b, link_gbs * 1e9, latency) for a in range(n) for b in range(n) if a != b]
        return c

    @staticmethod
    def ring(n: int, link_gbs: float = 50.0, latency: float = 2.0e-6, bidirectional: bool = True,
             device_type: DeviceType = DeviceType.CUDA) -> "Cluster":
        c = Cluster([Device(r, device_type) for r in range(n)], [], f"ring{n}")
        pairs = set()
        for r in range(n):
            pairs.add((r, (r + 1) % n))
            if bidirectional:
                pairs.add(((r + 1) % n, r))
        c.links = [Link(a, b, link_gbs * 1e9, latency) for a, b in sorted(pairs) if a != b]
        return c

    @staticmethod
    def from_topology(topo, device_type: DeviceType = DeviceType.CUDA) -> "Cluster":
        """From a ``pccl_b200.synth.Topology`` (canned or measured)."""
        c = Cluster([Device(r, device_type) for r in range(topo.n)], [], topo.name)
        for (a, b), bw in sorted(topo.link_bw.items()):
            if a != b and bw > 0:
                c.links.append(Link(a, b, bw, topo.alpha))
        return c

    @staticmethod
    def from_local_node(node=None, port_gbs: float = 770.0, pcie_gbs: float = 50.0) -> "Cluster":
        """The GPUs of this host as a cluster: ``node`` is a ``pccl_b200.synth.LocalNode`` (probed when omitted); pairs
        with peer access get the port rate, the others a host bridge's; each device carries its SM count as
        ``compute_capability`` and nothing is measured.  Refuses a host without GPUs."""
        if node is None:
            from ..synth.local_node import LocalNode
            node = LocalNode.probe()
        topo = node.to_topology(port_gbs, pcie_gbs)
        if topo is None:
            raise ValueError("this host has no GPUs to make a cluster of")
        c = Cluster.from_topology(topo)
        c.name = f"host_{len(node.gpus)}gpu"
        for d, g in zip(c.devices, node.gpus):
            d.compute_capability = g.sm_count
        return c

    # -- use -------------------------------------------------------------------------------------
    @property
    def world_size(self) -> int:
        return len(self.devices)

    def apply(self, ir: CollectiveIR) -> CollectiveIR:
        """Replaces the device/link graph of ``ir`` by this cluster (device ids must cover the program's ranks)."""
        have = {d.device_id for d in self.devices}
        need = set(ir.devices)
        if need and not need <= have:
            raise ValueError(f"cluster lacks devices {sorted(need - have)} that the program uses")
        ir.devices.clear()
        ir.links.clear()
        ir.device_topology = type(ir.device_topology)()
        for d in self.devices:
            ir.add_device(d)
        for l in self.links:
            ir.add_link(l)
        ir.attrs["cluster"] = self.name
        return ir

    def to_topology(self, port_gbs: Optional[float] = None):
        """The synthesiser's view: link matrix in bytes/s; port capacity = ``port_gbs`` or the largest link of each device."""
        from ..synth.topology import Topology
        n = self.world_size
        gbs = [[0.0] * n for _ in range(n)]
        alpha = 0.0
        for l in self.links:
            gbs[l.src_device][l.dst_device] = l.bandwidth / 1e9
            alpha = max(alpha, l.latency)
        return Topology.from_matrix(gbs, alpha=alpha or 2.0e-6, port_gbs=port_gbs)


__all__ = ["Cluster"]
