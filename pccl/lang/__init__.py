"""``pccl.lang``: same vocabulary as the reference's pccl/lang/chunk.py (PrimitiveOpType, DeviceType, Chunk,
Device, Link, PrimitiveOp, CollectiveIR) plus the algorithm library, verifier and lowering."""
from pccl_b200.lang import *  # noqa: F401,F403
from pccl_b200.lang import algorithms  # noqa: F401
