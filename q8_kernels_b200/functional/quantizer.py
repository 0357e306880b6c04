"""Per-token absmax quantizer (reference: q8_kernels/functional/quantizer.py)."""
from typing import Tuple

import torch

from ..native import tokenwise_quant


def quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """int8 values (round half away from zero) and fp32 per-row dequant scales."""
    q, s = tokenwise_quant(x, None)
    return q, s


def quantize_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """float8_e4m3fn values and fp32 per-row dequant scales."""
    q, s = tokenwise_quant(x, torch.float8_e4m3fn)
    return q, s
