"""The vocabulary of the reference's ``pccl/lang/chunk.py`` under its module name: ``PrimitiveOpType``,
``DeviceType``, ``Chunk``, ``Device``, ``Link``, ``PrimitiveOp`` and ``CollectiveIR`` (chunk.py:6-135).  The
definitions live in ``ir.py``."""
from .ir import (BUFFER_KINDS, Chunk, CollectiveIR, Device, DeviceType, Link, PrimitiveOp,  # noqa: F401
                 PrimitiveOpType)

__all__ = ["BUFFER_KINDS", "Chunk", "CollectiveIR", "Device", "DeviceType", "Link", "PrimitiveOp", "PrimitiveOpType"]
