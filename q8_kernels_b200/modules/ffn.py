"""FeedForward (reference: q8_kernels/modules/ffn.py:10-17)."""
import torch.nn as nn

from .activations import GELU
from .linear import make_linear


class FeedForward(nn.Module):
    def __init__(self, dim: int, mult: int = 4, bias: bool = True, linear: str = "int8"):
        super().__init__()
        self.inner_dim = dim * mult
        self.act = GELU(dim, self.inner_dim, bias=bias, linear=linear)
        self.proj_down = make_linear(linear, self.inner_dim, dim, bias=bias)

    def forward(self, x, out_dtype=None):
        return self.proj_down(self.act(x, out_dtype=out_dtype), out_dtype=out_dtype)
