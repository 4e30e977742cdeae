"""``pccl.lang.topology`` (module name of the reference) -> ``pccl_b200.lang.topology``."""
from pccl_b200.lang.topology import *  # noqa: F401,F403
from pccl_b200.lang.topology import __all__  # noqa: F401
