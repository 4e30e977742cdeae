"""Helpers of the DSL (the reference keeps its graph class under ``pccl/lang/utils``)."""
from .graph import DirectedGraph  # noqa: F401
