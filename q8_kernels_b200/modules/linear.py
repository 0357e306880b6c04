"""Q8Linear / FP8Linear (reference: q8_kernels/modules/linear.py:11-49,117-146).

Parameter layout and state-dict keys match the reference: ``weight`` int8 or
e4m3 [out, in] (frozen), ``bias`` fp32 [out] or None, buffer ``scales`` fp32 [out].
"""
import math

import torch
import torch.nn as nn

from .. import functional as Q8F
from .. import native


def is_16bit(x) -> bool:
    return x.dtype == torch.float16 or x.dtype == torch.bfloat16


class Q8Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=torch.int8),
                                   requires_grad=False)
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=torch.float), requires_grad=False)
        else:
            self.register_parameter("bias", None)
        self.register_buffer("scales", torch.empty(out_features, device=device, dtype=torch.float))

    def forward(self, x, x_scales=None, fuse_gelu=False, out_dtype=None):
        return Q8F.linear.q8_linear(x, self.weight.data, self.bias.data if self.bias is not None else None,
                                    x_scales, self.scales, fuse_gelu, out_dtype)

    @classmethod
    def from_linear(cls, linear: nn.Linear, quant_with_hadamard=True):
        assert linear.weight.data.is_cuda, "input linear layer must be in cuda device"
        assert linear.weight.data.dtype == torch.float8_e4m3fn or is_16bit(linear.weight.data)
        layer = cls(linear.in_features, linear.out_features, linear.bias is not None, linear.weight.device)
        w = linear.weight.data
        if w.dtype == torch.float16:
            w = w.to(torch.bfloat16)
        if quant_with_hadamard:
            w_quant, w_scale = native.hadamard_quant(w, 1 / math.sqrt(w.shape[-1]), torch.int8)
        else:
            w_quant, w_scale = Q8F.quantizer.quantize(w)
        layer.weight.data = w_quant
        layer.scales.data = w_scale
        if linear.bias is not None:
            layer.bias.data = linear.bias.data.float()
        return layer


class FP8Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, use_hadamard: bool = False,
                 device=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=torch.float8_e4m3fn),
                                   requires_grad=False)
        self.use_hadamard = use_hadamard
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=torch.float), requires_grad=False)
        else:
            self.register_parameter("bias", None)
        self.register_buffer("scales", torch.empty(out_features, device=device, dtype=torch.float))

    def forward(self, x):
        return Q8F.linear.fp8_linear(x, self.weight.data, self.bias.data if self.bias is not None else None,
                                     None, self.scales, self.use_hadamard, x.dtype)

    @classmethod
    def from_linear(cls, linear: nn.Linear, force_cuda=True, use_hadamard=False):
        assert linear.weight.data.is_cuda or force_cuda, "input linear layer must be in cuda device"
        assert is_16bit(linear.weight.data)
        w = linear.weight.data.cuda() if force_cuda else linear.weight.data
        layer = cls(linear.in_features, linear.out_features, linear.bias is not None, use_hadamard, w.device)
        w = w.to(torch.bfloat16)
        if use_hadamard:
            w_quant, w_scale = native.hadamard_quant(w, 1 / math.sqrt(w.shape[-1]), torch.float8_e4m3fn)
        else:
            w_quant, w_scale = Q8F.quantizer.quantize_fp8(w)
        layer.weight.data = w_quant
        layer.scales.data = w_scale
        if linear.bias is not None:
            layer.bias.data = linear.bias.data.float().to(w.device)
        return layer
