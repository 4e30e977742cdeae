"""PyTorch framework layer on top of the sm_100a kernels."""
from .linear import Embedding, Linear, LinearGelu
from .loss import fused_cross_entropy
from .norm import LayerNorm

__all__ = ["Embedding", "Linear", "LinearGelu", "fused_cross_entropy", "LayerNorm"]
