"""Drop-in names of the reference project: ``import pccl.lang`` / ``import pccl.engine`` resolve to
the B200-native implementation in ``pccl_b200``."""
from pccl_b200 import lang, engine  # noqa: F401

__version__ = "0.1.0"
