"""Mixed-precision multiply-add (reference: q8_kernels/functional/fma.py:9)."""
import torch

from ..native import fma_8bit


def multiply_add(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, scale_add: float = 0.0) -> torch.Tensor:
    """``e4m3(float(x) * (y + scale_add) + z)`` with y, z broadcast over tokens."""
    return fma_8bit(x, y, z, scale_add)
