"""Topology of the machine as the DSL and the synthesiser see it (the reference's ``pccl/lang/topology.py`` is an
empty file next to an empty ``include/topology/``): per-GPU port capacities and pairwise link bandwidths, canned
NVSwitch / ring shapes, a measured matrix, and the probe that measures it through an engine."""
from ..synth.topology import Topology, probe_topology  # noqa: F401

__all__ = ["Topology", "probe_topology"]
