"""``pccl.lang.utils.graph`` -> ``pccl_b200.lang.utils.graph``."""
from pccl_b200.lang.utils.graph import DirectedGraph  # noqa: F401

__all__ = ["DirectedGraph"]
