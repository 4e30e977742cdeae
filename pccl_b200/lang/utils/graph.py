"""``DirectedGraph`` under the module name of the reference (pccl/lang/utils/graph.py:17-134); defined in ``dag.py``."""
from ..dag import DirectedGraph  # noqa: F401

__all__ = ["DirectedGraph"]
