"""Drop-in for ``q8_kernels.modules`` (reference: q8_kernels/modules/)."""
from .activations import GELU
from .attention import Attention
from .ffn import FeedForward
from .linear import FP8Linear, Q8Linear, Q8LinearLora
from .rms_norm import RMSNorm

__all__ = ["Attention", "FeedForward", "FP8Linear", "GELU", "Q8Linear", "Q8LinearLora", "RMSNorm"]
