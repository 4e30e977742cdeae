"""``pccl.lang.cluster`` (module name of the reference) -> ``pccl_b200.lang.cluster``."""
from pccl_b200.lang.cluster import *  # noqa: F401,F403
from pccl_b200.lang.cluster import __all__  # noqa: F401
