"""Schedule synthesis: topology model, MILP over (chunk, link, step), on-disk schedule cache."""
from .topology import Topology, probe_topology
from .milp import SynthesisResult, synthesize
from .cache import ScheduleCache

__all__ = ["Topology", "probe_topology", "SynthesisResult", "synthesize", "ScheduleCache"]
