"""``pccl.lang.chunk`` (module name of the reference) -> ``pccl_b200.lang.chunk``."""
from pccl_b200.lang.chunk import *  # noqa: F401,F403
from pccl_b200.lang.chunk import __all__  # noqa: F401
