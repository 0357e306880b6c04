"""Q8Linear / Q8LinearLora / FP8Linear (reference: q8_kernels/modules/linear.py:11-146).

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


class Q8LinearLora(nn.Module):
    """Frozen INT8 linear with a trainable 16-bit low-rank branch (q8_kernels/modules/linear.py:53-114)."""

    def __init__(self, in_features: int, out_features: int, r: int, bias: bool = True, device=None,
                 dtype=torch.bfloat16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.r = r
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=torch.int8),
                                   requires_grad=False)
        self.lora_a = nn.Parameter(torch.empty(r, in_features, device=device, dtype=dtype))
        self.lora_b = nn.Parameter(torch.empty(out_features, r, device=device, dtype=dtype))
        nn.init.normal_(self.lora_a, std=1 / r)
        nn.init.zeros_(self.lora_b)
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=torch.float), requires_grad=False)
        else:
            self.register_parameter("bias", None)
        self.register_buffer("scales", torch.empty(out_features, device=device, dtype=torch.float))

    def forward(self, x, x_scales=None, fuse_gelu=False, out_dtype=None):
        return Q8F.linear.q8_linear_lora(x, self.weight.data, self.bias.data if self.bias is not None else None,
                                         x_scales, self.scales, self.lora_a, self.lora_b, fuse_gelu, True, out_dtype)

    @classmethod
    def from_linear(cls, linear, r: int, quant_with_hadamard=True):
        if isinstance(linear, Q8Linear):
            layer = cls(linear.in_features, linear.out_features, r, linear.bias is not None, linear.weight.device)
            layer.weight.data = linear.weight.data
            layer.scales.data = linear.scales.data
            if linear.bias is not None:
                layer.bias.data = linear.bias.data
            return layer
        base = Q8Linear.from_linear(linear, quant_with_hadamard)
        return cls.from_linear(base, r)


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

    def forward(self, x, x_scales=None, fuse_gelu=False, out_dtype=None):
        """``forward(x)`` is the reference's call (16-bit activation in, same dtype out).  The optional
        arguments follow Q8Linear's convention so that the attention / feed-forward modules can drive
        either kind: an already quantised e4m3 activation with its row scales, a tanh-GELU in the GEMM
        epilogue, and the output dtype."""
        bias = self.bias.data if self.bias is not None else None
        e4m3 = torch.float8_e4m3fn
        if x_scales is None and not fuse_gelu and x.dtype != e4m3:
            return Q8F.linear.fp8_linear(x, self.weight.data, bias, None, self.scales, self.use_hadamard,
                                         x.dtype if out_dtype is None else out_dtype)
        if x_scales is None:                                   # e4m3 activation without scales (e.g. an attention output), or GELU wanted
            src = x.to(torch.bfloat16) if x.dtype == torch.float16 else x
            x, x_scales = (native.hadamard_quant(src, 1 / math.sqrt(src.shape[-1]), e4m3) if self.use_hadamard
                           else Q8F.quantizer.quantize_fp8(src))
        out_dtype = torch.bfloat16 if out_dtype is None else out_dtype
        if bias is not None:
            return native.fp8_mm_bias(x, self.weight.data, bias, x_scales, self.scales, fuse_gelu, out_dtype)
        return native.fp8_mm(x, self.weight.data, x_scales, self.scales, fuse_gelu, out_dtype)

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


def make_linear(kind: str, in_features: int, out_features: int, bias: bool = True, device=None) -> nn.Module:
    """The quantised linear a DiT module is built from: ``"int8"`` -> Q8Linear (the reference's
    block), ``"fp8"`` -> FP8Linear with Hadamard-rotated per-token e4m3 activations."""
    if kind == "int8":
        return Q8Linear(in_features, out_features, bias=bias, device=device)
    if kind == "fp8":
        return FP8Linear(in_features, out_features, bias=bias, use_hadamard=True, device=device)
    raise ValueError(f"linear kind {kind!r} is not 'int8' or 'fp8'")
