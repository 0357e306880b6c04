"""RMS norm without eps (reference: q8_kernels/functional/rms_norm.py:8-26), with the reference's
autograd rule: the backward pass runs ``rms_norm_backward`` on the saved output and row norms."""
from typing import Optional

import torch

from ..native import rms_norm, rms_norm_backward


class RMSNorm8bit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, out_type):
        x_normed, x_norms = rms_norm(x, weights, out_type)
        ctx.save_for_backward(x_normed, x_norms, weights)
        ctx.out_type = out_type
        return x_normed

    @staticmethod
    def backward(ctx, grad_output):
        x_normed, x_norms, weights = ctx.saved_tensors
        return rms_norm_backward(x_normed, x_norms, grad_output, weights, ctx.out_type), None, None


def rms_norm_8bit(x: torch.Tensor, weights: Optional[torch.Tensor] = None,
                  out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    assert weights is None or weights.dtype == torch.float, "RMSNorm8bit: dtype missmatch"
    if torch.is_grad_enabled() and x.requires_grad:
        return RMSNorm8bit.apply(x, weights, out_type)
    return rms_norm(x, weights, out_type)[0]
