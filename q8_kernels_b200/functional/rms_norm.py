"""RMS norm without eps (reference: q8_kernels/functional/rms_norm.py:23)."""
from typing import Optional

import torch

from ..native import rms_norm


def rms_norm_8bit(x: torch.Tensor, weights: Optional[torch.Tensor] = None,
                  out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    assert weights is None or weights.dtype == torch.float, "RMSNorm8bit: dtype missmatch"
    return rms_norm(x, weights, out_type)[0]
