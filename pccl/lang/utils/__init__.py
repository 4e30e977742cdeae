"""``pccl.lang.utils`` -> ``pccl_b200.lang.utils``."""
from pccl_b200.lang.utils import DirectedGraph  # noqa: F401
