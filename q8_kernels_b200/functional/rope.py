"""Rotary embedding over interleaved pairs (reference: q8_kernels/functional/rope.py).

The reference's ``apply_rope`` bypasses its own kernel and returns the torch
promotion of ``x*cos + rot(x)*sin`` (fp32 for fp32 tables), ignoring
``out_type``.  Here the kernel runs and ``out_type`` is honoured; with
``out_type=None`` the result is fp32 for bf16 inputs to keep the values the
reference produces, bit for bit.
"""
from typing import Optional

import torch

from ..native import rope


def apply_rope(x: torch.Tensor, cos_freqs: torch.Tensor, sin_freqs: torch.Tensor,
               out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    assert (x.dtype == torch.float8_e4m3fn or x.dtype == torch.bfloat16) and \
        cos_freqs.dtype == torch.float and sin_freqs.dtype == torch.float
    if out_type is None:
        out_type = torch.float32 if x.dtype == torch.bfloat16 else x.dtype
    return rope(x, cos_freqs, sin_freqs, out_type)
