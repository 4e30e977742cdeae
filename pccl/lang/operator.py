"""``pccl.lang.operator`` (module name of the reference) -> ``pccl_b200.lang.operator``."""
from pccl_b200.lang.operator import *  # noqa: F401,F403
from pccl_b200.lang.operator import __all__  # noqa: F401
