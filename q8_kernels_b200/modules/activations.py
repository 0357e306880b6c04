"""GELU projection (reference: q8_kernels/modules/activations.py:9-16): a
quantised linear whose GEMM epilogue applies tanh-GELU (``linear="fp8"`` builds it
from FP8Linear instead of Q8Linear)."""
import torch.nn as nn

from .linear import make_linear


class GELU(nn.Module):
    def __init__(self, dim_in: int, dim_out: int, approximate: str = "none", bias: bool = True, linear: str = "int8"):
        super().__init__()
        self.proj = make_linear(linear, dim_in, dim_out, bias=bias)

    def forward(self, hidden_states, out_dtype=None):
        return self.proj(hidden_states, fuse_gelu=True, out_dtype=out_dtype)
