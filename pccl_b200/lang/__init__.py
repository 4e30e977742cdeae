"""``pccl.lang``: the collective-program DSL (IR, algorithm library, verifier, lowering)."""
from .dag import DirectedGraph
from .ir import (BUFFER_KINDS, Chunk, CollectiveIR, Device, DeviceType, Link, PrimitiveOp,
                 PrimitiveOpType)
from .verify import Report, VerificationError, add_acknowledgements, port_load, relaunch_hazards, verify
from .lower import LoweringError, OPCODES, check_lowered_deadlock_free, lower, to_schedule
from . import algorithms
from .algorithms import ALGORITHMS, build
from .cluster import Cluster
from .operator import Operator

__all__ = ["DirectedGraph", "BUFFER_KINDS", "Chunk", "CollectiveIR", "Device", "DeviceType", "Link",
           "PrimitiveOp", "PrimitiveOpType", "Report", "VerificationError", "port_load", "relaunch_hazards", "add_acknowledgements", "verify",
           "LoweringError", "OPCODES", "check_lowered_deadlock_free", "lower", "to_schedule",
           "algorithms", "ALGORITHMS", "build", "Cluster", "Operator"]
