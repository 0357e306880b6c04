"""Rotary embedding over interleaved pairs (reference: q8_kernels/functional/rope.py).

The reference's ``apply_rope`` bypasses its own kernel and returns the torch
promotion of ``x*cos + rot(x)*sin`` (fp32 for fp32 tables), ignoring
``out_type``.  Here the kernel runs and ``out_type`` is honoured; with
``out_type=None`` the result is fp32 for bf16 inputs to keep the values the
reference produces, bit for bit.
"""
from typing import Optional

import torch

from ..native import rope, rope_backward


class ROPE(torch.autograd.Function):
    """q8_kernels/functional/rope.py:10-23: kernel forward, ``rope_backward`` for the gradient."""

    @staticmethod
    def forward(ctx, x, cos_freqs, sin_freqs, out_type):
        ctx.save_for_backward(cos_freqs, sin_freqs)
        ctx.out_type = out_type
        return rope(x, cos_freqs, sin_freqs, out_type)

    @staticmethod
    def backward(ctx, grad_output):
        cos_freqs, sin_freqs = ctx.saved_tensors
        out_type = ctx.out_type if ctx.out_type in (torch.bfloat16, torch.float8_e4m3fn) else torch.bfloat16
        g = grad_output if grad_output.dtype in (torch.bfloat16, torch.float8_e4m3fn) else grad_output.to(torch.bfloat16)
        return rope_backward(g, cos_freqs, sin_freqs, out_type), None, None, None


def apply_rope(x: torch.Tensor, cos_freqs: torch.Tensor, sin_freqs: torch.Tensor,
               out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    assert (x.dtype == torch.float8_e4m3fn or x.dtype == torch.bfloat16) and \
        cos_freqs.dtype == torch.float and sin_freqs.dtype == torch.float
    if out_type is None:
        out_type = torch.float32 if x.dtype == torch.bfloat16 else x.dtype
    if torch.is_grad_enabled() and x.requires_grad:
        return ROPE.apply(x, cos_freqs, sin_freqs, out_type)
    return rope(x, cos_freqs, sin_freqs, out_type)
