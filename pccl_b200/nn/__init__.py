"""PyTorch framework layer on top of the sm_100a kernels."""
from .linear import Embedding, Linear, LinearGelu, mlp
from .loss import fused_cross_entropy
from .norm import LayerNorm

__all__ = ["Embedding", "Linear", "LinearGelu", "mlp", "fused_cross_entropy", "LayerNorm"]
