"""Fast Hadamard transform (reference: q8_kernels/functional/fast_hadamard.py:24-38)."""
import math
from typing import Optional

import torch

from ..native import fast_hadamard_transform


def hadamard_transform(x: torch.Tensor, scale: Optional[float] = None,
                       out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """Multiply each row of ``x`` (..., dim) by the Sylvester-Hadamard matrix and
    by ``scale`` (default ``1/sqrt(dim)``).  A dim that is not a power of two is
    implicitly zero-padded to the next one.  ``out_type`` defaults to x.dtype."""
    if scale is None:
        scale = 1 / math.sqrt(x.shape[-1])
    return fast_hadamard_transform(x, scale, out_type)
