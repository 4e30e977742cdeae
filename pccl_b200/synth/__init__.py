"""Schedule synthesis: topology model, MILP over (chunk, link, step), cost model and algorithm choice, on-disk schedule cache."""
from .topology import Topology, probe_topology
from .milp import SynthesisResult, synthesize
from .cache import ScheduleCache
from .simulate import Estimate, choose, estimate
from .local_node import GpuInfo, LocalNode, TopologyCache

__all__ = ["Topology", "probe_topology", "SynthesisResult", "synthesize", "ScheduleCache", "Estimate", "choose", "estimate",
           "GpuInfo", "LocalNode", "TopologyCache"]
