"""8-bit linear layers (reference: q8_kernels/functional/linear.py:24-196).

Inference: where the reference launches Hadamard, quantizer and GEMM as three
kernels with two intermediate tensors, the 16-bit / e4m3 activation path here is
one native call: a fused Hadamard+quantizer producer writing into a cached
scratch buffer, then the tcgen05 GEMM.

Training side (the activation gradient only, as in the reference: weights are
frozen): when the activation requires grad the call goes through an autograd
function whose backward is the reference's -- the incoming gradient and the
de-quantised weight are re-quantised per row to e4m3 and multiplied by the FP8
GEMM (functional/linear.py:44-53,161-178); ``q8_linear_lora`` adds a 16-bit
low-rank branch with gradients for ``lora_a`` / ``lora_b`` (:56-133).
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
    e4m3 unless ``out_dtype`` says bf16.  Differentiable in ``a`` (see the module docstring)."""
    if _needs_grad(a):
        return Q8LinearFunc.apply(a, b, bias, scale_a, scale_b, fuse_gelu, out_dtype)
    return _q8_linear_forward(a, b, bias, scale_a, scale_b, fuse_gelu, out_dtype)


def _q8_linear_forward(a, b, bias, scale_a, scale_b, fuse_gelu, out_dtype):
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
    per-channel e4m3 weights, fp32 accumulation, 16-bit output, never GELU.
    Differentiable in ``a`` (see the module docstring)."""
    if _needs_grad(a):
        return FP8LinearFunc.apply(a, b, bias, scale_a, scale_b, out_dtype, use_hadamard)
    return _fp8_linear_forward(a, b, bias, scale_a, scale_b, use_hadamard, out_dtype)


def _fp8_linear_forward(a, b, bias, scale_a, scale_b, use_hadamard, out_dtype):
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


# --------------------------------------------------------------------------- training side

def _needs_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def _dequant_t(b: torch.Tensor, scale_b: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``(b.to(dtype) * scale_b[:, None]).T`` of the reference's backward passes: the de-quantised
    weight with the input dim leading, so that its rows are what the FP8 GEMM contracts over."""
    return (b.to(dtype) * scale_b[:, None]).T


class Q8LinearFunc(torch.autograd.Function):
    """q8_kernels/functional/linear.py:24-53."""

    @staticmethod
    def forward(ctx, a, b, bias, scale_a, scale_b, fuse_gelu, out_dtype):
        if b.dtype != torch.int8:
            b, scale_b = native.hadamard_quant(b, 1 / math.sqrt(b.shape[-1]), torch.int8)
        ctx.save_for_backward(b, scale_b)
        ctx.out_dtype = out_dtype
        return _q8_linear_forward(a, b, bias, scale_a, scale_b, fuse_gelu, out_dtype)

    @staticmethod
    def backward(ctx, grad_output):
        b, scale_b = ctx.saved_tensors
        g8, gs = quantize_fp8(grad_output.contiguous())
        w8, ws = quantize_fp8(_dequant_t(b, scale_b, ctx.out_dtype).contiguous())
        grad_x = hadamard_transform(native.fp8_mm(g8, w8, gs, ws, False, ctx.out_dtype))
        return grad_x, None, None, None, None, None, None


class FP8LinearFunc(torch.autograd.Function):
    """q8_kernels/functional/linear.py:138-178."""

    @staticmethod
    def forward(ctx, a, b, bias, scale_a, scale_b, out_dtype, use_hadamard):
        if is_16bit(b):
            b, scale_b = (native.hadamard_quant(b, 1 / math.sqrt(b.shape[-1]), E4M3) if use_hadamard
                          else quantize_fp8(b))
        ctx.save_for_backward(b, scale_b)
        ctx.out_dtype = out_dtype
        ctx.use_hadamard = use_hadamard
        return _fp8_linear_forward(a, b, bias, scale_a, scale_b, use_hadamard, out_dtype)

    @staticmethod
    def backward(ctx, grad_output):
        b, scale_b = ctx.saved_tensors
        g8, gs = quantize_fp8(grad_output.contiguous())
        w = _dequant_t(b, scale_b, ctx.out_dtype)
        # the reference rotates and THEN transposes here (linear.py:165), which only type-checks for
        # square weights; kept as it is
        w8, ws = quantize_fp8((hadamard_transform(w.contiguous()).T if ctx.use_hadamard else w).contiguous())
        grad_x = native.fp8_mm(g8, w8, gs, ws, False, ctx.out_dtype)
        return grad_x, None, None, None, None, None, None


class Q8LinearLora(torch.autograd.Function):
    """q8_kernels/functional/linear.py:56-133: INT8 base linear plus ``lora_b(lora_a(a))`` in 16 bit,
    optional tanh-GELU on the sum; gradients for the activation and the two low-rank factors."""

    @staticmethod
    def forward(ctx, a, b, bias, scale_a, scale_b, lora_a, lora_b, fuse_gelu, use_hadamard, out_dtype):
        assert (a.dtype == E4M3 or is_16bit(a)) and scale_a is None, \
            "Q8LinearFuncLora: the activation must be 16-bit or e4m3 (the low-rank branch needs it un-quantised)"
        assert ((b.dtype == E4M3 or is_16bit(b)) and scale_b is None) or (b.dtype == torch.int8 and scale_b is not None), \
            "Q8LinearFuncLora: b dtype missmatch"
        assert a.shape[-1] == b.shape[-1], "Q8LinearFuncLora: mnk missmatch"
        assert bias is None or bias.dtype == torch.float, "Q8LinearFuncLora: bias must be in fp32"
        assert lora_a is not None and lora_b is not None, "Q8LinearFuncLora: lora_a and lora_b must be provided"
        assert is_16bit(lora_a) and is_16bit(lora_b), "Q8LinearFuncLora: lora_a and lora_b must be in 16bit"
        assert lora_a.shape[0] == lora_b.shape[-1], "Q8LinearFuncLora: lora_a and lora_b shape missmatch"
        assert out_dtype in (torch.float16, torch.bfloat16), "Q8LinearFuncLora: out_dtype must be float16 or bfloat16"
        if b.dtype != torch.int8:
            b, scale_b = native.hadamard_quant(b, 1 / math.sqrt(b.shape[-1]), torch.int8)
        ctx.fuse_gelu = fuse_gelu
        ctx.out_dtype = out_dtype
        ctx.use_hadamard = use_hadamard
        lora_y = torch.nn.functional.linear(torch.nn.functional.linear(a, lora_a), lora_b)
        o = _q8_linear_forward(a, b, bias, None, scale_b, False, out_dtype)
        o = o.reshape(lora_y.shape) + lora_y
        if fuse_gelu:
            ctx.save_for_backward(o, a, b, scale_b, lora_a, lora_b)
            o = native.gelu_forward(o, out_dtype)
        else:
            ctx.save_for_backward(None, a, b, scale_b, lora_a, lora_b)
        return o

    @staticmethod
    def backward(ctx, grad_output):
        o, a, b, scale_b, lora_a, lora_b = ctx.saved_tensors
        out_dtype = ctx.out_dtype
        if ctx.fuse_gelu:
            grad_output = native.gelu_backward(o, grad_output, out_dtype)
        grad_out_lora_b = grad_output @ lora_b                                  # [.., s, d] @ [d, r]
        w = (b * scale_b[:, None]).to(out_dtype)
        if not ctx.use_hadamard:
            raise NotImplementedError("q8_linear_lora backward: only use_hadamard=True is defined "
                                      "(the reference's other branch reads an unset variable)")
        w8, ws = quantize_fp8(hadamard_transform(w).T.contiguous())
        g8, gs = quantize_fp8(grad_output.contiguous())
        grad_x = native.fp8_mm(g8, w8, gs, ws, False, out_dtype).reshape(a.shape) + grad_out_lora_b @ lora_a
        grad_lora_a = grad_out_lora_b.transpose(-1, -2) @ a                     # [.., r, s] @ [.., s, h]
        grad_lora_b = grad_output.transpose(-1, -2) @ (a @ lora_a.T)            # [.., d, s] @ [.., s, r]
        return grad_x, None, None, None, None, grad_lora_a, grad_lora_b, None, None, None


def q8_linear_lora(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
                   lora_a: Optional[torch.Tensor] = None, lora_b: Optional[torch.Tensor] = None,
                   fuse_gelu: bool = False, use_hadamard: bool = True,
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """q8_kernels/functional/linear.py:181-186."""
    return Q8LinearLora.apply(a, b, bias, scale_a, scale_b, lora_a, lora_b, fuse_gelu, use_hadamard, out_dtype)
