"""Parallelism strategies built on the collectives and fused kernels."""
from .dp import ShardedDataParallel

__all__ = ["ShardedDataParallel", "tp", "ep", "pp"]
