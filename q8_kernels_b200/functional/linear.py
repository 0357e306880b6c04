"""8-bit linear layers (reference: q8_kernels/functional/linear.py:24-42,138-196).

Forward only.  Where the reference launches Hadamard, quantizer and GEMM as
three kernels with two intermediate tensors, the 16-bit / e4m3 activation path
here is one native call: a fused Hadamard+quantizer producer writing into a
cached scratch buffer, then the tcgen05 GEMM.
"""
import math
from typing import Optional

import torch

from .. import native
from .fast_hadamard import hadamard_transform
from .quantizer import quantize, quantize_fp8

E4M3 = torch.float8_e4m3fn


def is_16bit(x) -> bool:
    d = x.dtype if hasattr(x, "dtype") else x
    return d == torch.float16 or d == torch.bfloat16


def q8_linear(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
              scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
              fuse_gelu: bool = False, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """INT8 linear: ``a`` is either int8 with ``scale_a`` or a bf16/fp16/e4m3
    activation that is Hadamard-rotated (scale 1/sqrt(K)) and quantised per
    token first; same for the weight ``b`` [N,K].  Output is [batch, M, N],
    e4m3 unless ``out_dtype`` says bf16."""
    assert ((a.dtype == E4M3 or is_16bit(a)) and scale_a is None) or (a.dtype == torch.int8 and scale_a is not None), \
        "Q8LinearFunc: a dtype missmatch"
    assert ((b.dtype == E4M3 or is_16bit(b)) and scale_b is None) or (b.dtype == torch.int8 and scale_b is not None), \
        "Q8LinearFunc: b dtype missmatch"
    assert a.shape[-1] == b.shape[-1], "Q8LinearFunc: mnk missmatch"
    assert bias is None or bias.dtype == torch.float, "Q8LinearFunc: bias must be in fp32"

    if b.dtype != torch.int8:
        b, scale_b = native.hadamard_quant(b, 1 / math.sqrt(b.shape[-1]), torch.int8)
    if a.dtype != torch.int8:
        if a.dtype in (torch.bfloat16, E4M3) and b.dim() == 2 and 2 <= a.dim() <= 3:
            return native.linear(a, b, scale_b, bias, True, fuse_gelu, E4M3 if out_dtype is None else out_dtype)
        if a.dtype == torch.float16:
            a, scale_a = quantize(hadamard_transform(a.to(torch.bfloat16)).to(torch.float16))
        else:
            a, scale_a = native.hadamard_quant(a, 1 / math.sqrt(a.shape[-1]), torch.int8)
    a = a.contiguous()
    scale_a = scale_a.contiguous()
    if bias is not None:
        return native.q8_mm_bias(a, b, bias, scale_a, scale_b, fuse_gelu, out_dtype)
    return native.q8_mm(a, b, scale_a, scale_b, fuse_gelu, out_dtype)


def fp8_linear(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
               scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
               use_hadamard: bool = False, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """FP8 linear: per-token e4m3 activations (optionally Hadamard-rotated),
    per-channel e4m3 weights, fp32 accumulation, 16-bit output, never GELU."""
    assert (is_16bit(a) and scale_a is None) or (a.dtype == E4M3 and scale_a is not None), \
        "FP8LinearFunc: a dtype missmatch"
    assert (is_16bit(b) and scale_b is None) or (b.dtype == E4M3 and scale_b is not None), \
        "FP8LinearFunc: b dtype missmatch"
    assert a.shape[-1] == b.shape[-1], "FP8LinearFunc: mnk missmatch"
    assert bias is None or bias.dtype == torch.float, "FP8LinearFunc: bias must be in fp32"
    assert is_16bit(out_dtype), "FP8LinearFunc: out_dtype must be in 16bit, FIXME: LATER MAYBE"
    if out_dtype != torch.bfloat16:
        raise native.Q8KernelError("fp8_linear: only bfloat16 output is implemented on sm_100a")

    def quant(x):
        if use_hadamard:
            return native.hadamard_quant(x, 1 / math.sqrt(x.shape[-1]), E4M3)
        return quantize_fp8(x)

    if is_16bit(b):
        b, scale_b = quant(b)
    if is_16bit(a):
        if a.dtype == torch.bfloat16 and b.dim() == 2 and 2 <= a.dim() <= 3:
            return native.linear(a, b, scale_b, bias, use_hadamard, False, out_dtype)
        a, scale_a = quant(a.to(torch.bfloat16))
    a = a.contiguous()
    scale_a = scale_a.contiguous()
    if bias is not None:
        return native.fp8_mm_bias(a, b, bias, scale_a, scale_b, False, out_dtype)
    return native.fp8_mm(a, b, scale_a, scale_b, False, out_dtype)


def q8_linear_lora(*args, **kwargs):
    """The LoRA fine-tuning path of the reference (functional/linear.py:56-133)
    is outside the inference hot path and is not provided."""
    raise NotImplementedError("q8_linear_lora (fine-tuning path) is not part of the sm_100a inference package")
