"""GELU projection (reference: q8_kernels/modules/activations.py:9-16): a
Q8Linear whose GEMM epilogue applies tanh-GELU."""
import torch.nn as nn

from .linear import Q8Linear


class GELU(nn.Module):
    def __init__(self, dim_in: int, dim_out: int, approximate: str = "none", bias: bool = True):
        super().__init__()
        self.proj = Q8Linear(dim_in, dim_out, bias=bias)

    def forward(self, hidden_states, out_dtype=None):
        return self.proj(hidden_states, fuse_gelu=True, out_dtype=out_dtype)
