"""CPU oracle for the 8-bit DiT inference path of q8_kernels.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA kernels are
compared against; nothing in the product package imports it.  It is a torch-CPU
/ numpy restatement of the reference's CUDA kernel semantics, one function per
native entry point, each citing the reference source it follows.

PARITY UNPINNED: the reference ships no tests, golden vectors or CPU
implementation for this path and its CUDA extensions cannot be built here
(un-vendored CUTLASS submodule, sm_89-only build), so this restatement is
anchored on a reading of the kernel sources only.

Conventions
  c10 cast : fp32 -> float8_e4m3fn as torch's ``.to(torch.float8_e4m3fn)``
             (round to nearest even, overflow -> NaN, no saturation)
  sat cast : clamp to +-448, then round to nearest even (``cvt.rn.satfinite``)
  rha      : round half away from zero (C ``round``)
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

E4M3 = torch.float8_e4m3fn
E4M3_MAX = 448.0
INT8_MAX = 127.0
LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------- casts

def c10_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 the way c10::Float8_e4m3fn(float) does it (overflow -> NaN)."""
    return x.to(torch.float32).to(E4M3)


def sat_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 with saturation to +-448 (``__nv_cvt_float2_to_fp8x2`` with
    ``__NV_SATFINITE``; csrc/gemm/q8_matmul_bias.cu:46)."""
    x = x.to(torch.float32)
    return torch.clamp(x, -E4M3_MAX, E4M3_MAX).to(E4M3)


def round_half_away(x: torch.Tensor) -> torch.Tensor:
    """C ``round``: halves go away from zero.  Done in float64 so that
    ``|x| + 0.5`` is exact for every fp32 ``x``."""
    xd = x.to(torch.float64)
    return (torch.sign(xd) * torch.floor(torch.abs(xd) + 0.5)).to(torch.float32)


def cast_out(y: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Output cast used by the SIMT ops (quantizer, Hadamard, RMSNorm, RoPE,
    FMA, GELU): plain C++ conversion to the c10 scalar type."""
    if out_dtype == E4M3:
        return c10_e4m3(y)
    return y.to(out_dtype)


# --------------------------------------------------------------------------- a1 quantizer

def tokenwise_quant(x: torch.Tensor, out_dtype: Optional[torch.dtype] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row absmax quantizer (csrc/quantizer/tokenwise_quant_cuda.cu:115-148,
    csrc/quantizer/tokenwise_quant.cpp:74-111).

    ``scale = QMAX / absmax`` (IEEE fp32 divide), ``q = round(x*scale)`` for
    int8 (half away from zero) or ``c10(x*scale)`` for e4m3, and the returned
    per-row dequant scale is ``1/scale``.  An all-zero row is undefined in the
    reference (0*inf); here it is defined as q = 0, scale = 0.
    """
    if out_dtype is None:
        out_dtype = torch.int8
    shape = x.shape
    xf = x.reshape(-1, shape[-1]).to(torch.float32)
    amax = xf.abs().amax(dim=-1, keepdim=True)
    qmax = torch.tensor(INT8_MAX if out_dtype == torch.int8 else E4M3_MAX, dtype=torch.float32)
    scale = qmax / amax                       # inf for an all-zero row
    y = xf * scale
    zero_row = amax == 0
    y = torch.where(zero_row, torch.zeros_like(y), y)
    if out_dtype == torch.int8:
        q = round_half_away(y).to(torch.int8)
    else:
        q = c10_e4m3(y)
    out_scale = (torch.tensor(1.0, dtype=torch.float32) / scale).reshape(-1)
    return q.reshape(shape), out_scale.reshape(shape[:-1])


# --------------------------------------------------------------------------- a2 Hadamard

def fwht_fp32(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Sylvester-Hadamard transform of the last dim (a power of
    two) in fp32, butterflies (a+b, a-b) applied for stride 1, 2, 4, ... exactly
    as csrc/fast_hadamard/fast_hadamard_transform_common.h:86-124 orders them
    (in-thread strides, then lanes, then warps, then chunks).  Every butterfly
    is a single fp32 add or subtract, so the result is bit-reproducible."""
    n = x.shape[-1]
    assert n & (n - 1) == 0
    y = x.to(torch.float32).reshape(-1, n).clone()
    rows = y.shape[0]
    stride = 1
    while stride < n:
        v = y.view(rows, n // (2 * stride), 2, stride)
        a = v[:, :, 0, :]
        b = v[:, :, 1, :]
        y = torch.stack((a + b, a - b), dim=2).reshape(rows, n)
        stride *= 2
    return y.reshape(x.shape)


def hadamard_transform(x: torch.Tensor, scale: Optional[float] = None,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/fast_hadamard/fast_hadamard_transform.cpp:70-121 with the Python
    default scale of q8_kernels/functional/fast_hadamard.py:36-37.

    Rows are zero-padded to the next power of two, transformed in fp32,
    multiplied by ``scale`` (as a C float) and cast to ``out_dtype`` (default:
    the input dtype); the padding is sliced off again."""
    dim = x.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(dim)
    if out_dtype is None:
        out_dtype = x.dtype
    n = 1 << max(3, math.ceil(math.log2(dim)))
    xf = x.to(torch.float32)
    if n != dim:
        xf = torch.nn.functional.pad(xf, (0, n - dim))
    y = fwht_fp32(xf) * torch.tensor(scale, dtype=torch.float32)
    return cast_out(y[..., :dim], out_dtype)


# --------------------------------------------------------------------------- a3 / a4 GEMM

def gelu_tanh(y: torch.Tensor) -> torch.Tensor:
    """csrc/gemm/q8_matmul_bias.cu:29-33."""
    y = y.to(torch.float32)
    return 0.5 * y * (1.0 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y * y * y)))


def _gemm_epilogue(acc: torch.Tensor, a_scales, b_scales, bias, fuse_gelu, out_dtype):
    # csrc/gemm/q8_matmul_bias.cu:360-368: acc * (sa*sb) + bias, product of the scales first
    y = acc * (a_scales.to(torch.float32)[..., :, None] * b_scales.to(torch.float32)[..., None, :])
    if bias is not None:
        y = y + bias.to(torch.float32)
    if fuse_gelu:
        y = gelu_tanh(y)
    if out_dtype is None:
        out_dtype = E4M3                      # csrc/gemm/q8_gemm_api.cpp:146-151
    if out_dtype == E4M3:
        return sat_e4m3(y)
    return y.to(out_dtype)


def _as_batched(t: torch.Tensor) -> torch.Tensor:
    return t if t.dim() == 3 else t.unsqueeze(0)


def q8_mm(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
          fuse_gelu: bool = False, out_dtype: Optional[torch.dtype] = None,
          bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """INT8 GEMM ``C = act((A.B^T) * sa (x) sb + bias)`` with exact integer
    accumulation (csrc/gemm/q8_gemm_api.cpp:40-164, q8_matmul_bias.cu:95-415).
    A is [batch?, M, K], B is [batch?, N, K]; the result is always 3-D."""
    a3, b3 = _as_batched(a), _as_batched(b)
    # float64 matmul of int8 values is exact: |sum| <= 127^2 * K < 2^53
    acc = torch.matmul(a3.to(torch.float64), b3.to(torch.float64).transpose(-1, -2)).to(torch.float32)
    sa = a_scales.reshape(a3.shape[0], a3.shape[1])
    sb = b_scales.reshape(b3.shape[0], b3.shape[1])
    return _gemm_epilogue(acc, sa, sb, bias, fuse_gelu, out_dtype)


def fp8_mm(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
           fuse_gelu: bool = False, out_dtype: Optional[torch.dtype] = None,
           bias: Optional[torch.Tensor] = None, exact: bool = False) -> torch.Tensor:
    """FP8-e4m3 GEMM with fp32 accumulation (csrc/gemm/q8_gemm_api.cpp:167-291,
    fp8_matmul_bias.cu:97-415).  ``exact=True`` accumulates in float64."""
    a3, b3 = _as_batched(a), _as_batched(b)
    acc_t = torch.float64 if exact else torch.float32
    acc = torch.matmul(a3.to(acc_t), b3.to(acc_t).transpose(-1, -2)).to(torch.float32)
    sa = a_scales.reshape(a3.shape[0], a3.shape[1])
    sb = b_scales.reshape(b3.shape[0], b3.shape[1])
    return _gemm_epilogue(acc, sa, sb, bias, fuse_gelu, out_dtype)


# --------------------------------------------------------------------------- a12 linear chains

def q8_linear(a, b, bias=None, scale_a=None, scale_b=None, fuse_gelu=False, out_dtype=None):
    """q8_kernels/functional/linear.py:24-42 (Q8LinearFunc.forward)."""
    if a.dtype != torch.int8:
        a, scale_a = tokenwise_quant(hadamard_transform(a))
    if b.dtype != torch.int8:
        b, scale_b = tokenwise_quant(hadamard_transform(b))
    return q8_mm(a, b, scale_a, scale_b, fuse_gelu, out_dtype, bias=bias)


def fp8_linear(a, b, bias=None, scale_a=None, scale_b=None, use_hadamard=False, out_dtype=None):
    """q8_kernels/functional/linear.py:138-159 (FP8LinearFunc.forward)."""
    def quant(x):
        return tokenwise_quant(hadamard_transform(x) if use_hadamard else x, E4M3)
    if a.dtype != E4M3:
        a, scale_a = quant(a)
    if b.dtype != E4M3:
        b, scale_b = quant(b)
    return fp8_mm(a, b, scale_a, scale_b, False, out_dtype, bias=bias)


def q8_linear_backward(grad_output, b, scale_b, out_dtype):
    """Q8LinearFunc.backward (q8_kernels/functional/linear.py:44-53): grad and de-quantised rotated
    weight re-quantised per row to e4m3, FP8 GEMM, Hadamard back."""
    g8, gs = tokenwise_quant(grad_output, E4M3)
    w8, ws = tokenwise_quant((b.to(out_dtype) * scale_b[:, None]).T, E4M3)
    return hadamard_transform(fp8_mm(g8, w8, gs, ws, False, out_dtype))


def fp8_linear_backward(grad_output, b, scale_b, out_dtype, use_hadamard=False):
    """FP8LinearFunc.backward (q8_kernels/functional/linear.py:161-178)."""
    g8, gs = tokenwise_quant(grad_output, E4M3)
    w = (b.to(out_dtype) * scale_b[:, None]).T
    w8, ws = tokenwise_quant(hadamard_transform(w).T if use_hadamard else w, E4M3)
    return fp8_mm(g8, w8, gs, ws, False, out_dtype)


def q8_linear_lora(a, b, bias, scale_b, lora_a, lora_b, fuse_gelu, out_dtype, grad_output=None):
    """Q8LinearLora forward and, with ``grad_output``, backward (use_hadamard=True)
    (q8_kernels/functional/linear.py:56-133).  Returns ``out`` or
    ``(out, grad_a, grad_lora_a, grad_lora_b)``."""
    aq, sa = tokenwise_quant(hadamard_transform(a))
    lora_y = torch.nn.functional.linear(torch.nn.functional.linear(a, lora_a), lora_b)
    pre = q8_mm(aq, b, sa, scale_b, False, out_dtype, bias=bias) + lora_y
    out = gelu_forward(pre, out_dtype) if fuse_gelu else pre
    if grad_output is None:
        return out
    g = gelu_backward(pre, grad_output, out_dtype) if fuse_gelu else grad_output
    g_lb = g @ lora_b
    w = hadamard_transform((b * scale_b[:, None]).to(out_dtype)).T
    w8, ws = tokenwise_quant(w, E4M3)
    g8, gs = tokenwise_quant(g, E4M3)
    grad_a = fp8_mm(g8, w8, gs, ws, False, out_dtype) + g_lb @ lora_a
    # per-batch gradients of the factors; autograd sums them down to the parameters' shapes
    gla, glb = g_lb.transpose(-1, -2) @ a, g.transpose(-1, -2) @ (a @ lora_a.T)
    return out, grad_a, gla.sum_to_size(lora_a.shape), glb.sum_to_size(lora_b.shape)


# --------------------------------------------------------------------------- a8..a11 row-wise ops

def rms_norm(x: torch.Tensor, weights: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """csrc/ops/rms_norm_cuda.cu:127-169: ``r = rsqrt(mean(x^2))`` with no eps,
    ``out = (x*r)*w``; also returns ``r`` per row.  The sum of squares is
    taken in float64 here (the kernel's fp32 summation order is not part of the
    semantics); compare with a tolerance."""
    if out_dtype is None:
        out_dtype = x.dtype
    xf = x.to(torch.float32)
    ms = (xf.to(torch.float64) ** 2).sum(dim=-1, keepdim=True) / x.shape[-1]
    r = (1.0 / torch.sqrt(ms)).to(torch.float32)
    y = xf * r
    if weights is not None:
        y = y * weights.to(torch.float32)
    return cast_out(y, out_dtype), r.squeeze(-1)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
         out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/rope_cuda.cu:99-103: interleaved pairs with per-element fp32
    tables, ``o[2i] = -x[2i+1]*s[2i] + x[2i]*c[2i]`` and
    ``o[2i+1] = x[2i]*s[2i+1] + x[2i+1]*c[2i+1]``, each product rounded to fp32
    before the add (the CUDA kernel here uses non-contracted arithmetic)."""
    if out_dtype is None:
        out_dtype = x.dtype
    xf = x.to(torch.float32)
    x0, x1 = xf[..., 0::2], xf[..., 1::2]
    c0, c1 = cos[..., 0::2].float(), cos[..., 1::2].float()
    s0, s1 = sin[..., 0::2].float(), sin[..., 1::2].float()
    o0 = (-x1) * s0 + x0 * c0
    o1 = x0 * s1 + x1 * c1
    out = torch.stack((o0, o1), dim=-1).reshape(x.shape)
    return cast_out(out, out_dtype)


# --------------------------------------------------------------------------- training-side gradients

def gelu_backward(x: torch.Tensor, grad_output: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/gelu_backward_cuda.cu:88-100: with tau = k (x + f x x x), phi = tanh(tau),
    phi' = (1 - phi^2) k (1 + 3 f x^2):  out = g (0.5 (1 + phi) + 0.5 x phi'), fp32, g read in the
    output dtype."""
    if out_dtype is None:
        out_dtype = x.dtype
    k, f = 0.7978845608028654, 0.044715
    v = x.to(torch.float32)
    g = grad_output.to(out_dtype).to(torch.float32)
    f32 = lambda c: torch.tensor(c, dtype=torch.float32)  # noqa: E731
    tau = f32(k) * (v + f32(f) * v * v * v)
    phi = torch.tanh(tau)
    phi_prime = (1.0 - phi * phi) * (f32(k) * (1.0 + (f32(f) * f32(3.0)) * v * v))
    return cast_out(g * (0.5 * (1.0 + phi) + 0.5 * v * phi_prime), out_dtype)


def rope_backward(grad_out: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/rope_backward_cuda.cu:101-110: ``o[2i] = g[2i] c[2i] + g[2i+1] s[2i+1]``,
    ``o[2i+1] = -g[2i] s[2i] + g[2i+1] c[2i+1]``, each product rounded to fp32 before the add."""
    if out_dtype is None:
        out_dtype = grad_out.dtype
    g = grad_out.to(torch.float32)
    g0, g1 = g[..., 0::2], g[..., 1::2]
    c0, c1 = cos[..., 0::2].float(), cos[..., 1::2].float()
    s0, s1 = sin[..., 0::2].float(), sin[..., 1::2].float()
    o0 = g0 * c0 + g1 * s1
    o1 = (-g0) * s0 + g1 * c1
    return cast_out(torch.stack((o0, o1), dim=-1).reshape(grad_out.shape), out_dtype)


def rms_norm_backward(x_normed: torch.Tensor, x_norms: torch.Tensor, grad_out: torch.Tensor,
                      weights: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/rms_norm_backward_cuda.cu:135-160: ``r / dim * (dim g_i w_i - y_i / w_i * sum_j g_j y_j)``
    with y the forward output, r the saved per-row rsqrt, g read in the output dtype; the row sum is
    taken in float64 here (the kernel's fp32 summation order is not part of the semantics)."""
    if out_dtype is None:
        out_dtype = x_normed.dtype
    dim = x_normed.shape[-1]
    y = x_normed.to(torch.float32)
    g = grad_out.to(out_dtype).to(torch.float32)
    w = torch.ones(dim, dtype=torch.float32) if weights is None else weights.to(torch.float32)
    dot = (g.to(torch.float64) * y.to(torch.float64)).sum(dim=-1, keepdim=True).to(torch.float32)
    fdim = torch.tensor(float(dim), dtype=torch.float32)
    r = x_norms.to(torch.float32).unsqueeze(-1) / fdim
    return cast_out(r * (fdim * g * w - y / w * dot), out_dtype)


def apply_rotary_emb_torch(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """The pure-torch path the reference's ``apply_rope`` actually runs
    (q8_kernels/functional/rope.py:27-43); result dtype follows torch promotion."""
    t = x.reshape(*x.shape[:-1], -1, 2)
    t1, t2 = t.unbind(dim=-1)
    rot = torch.stack((-t2, t1), dim=-1).reshape(x.shape)
    return x * cos + rot * sin


def fma_8bit(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, scale_add: float = 0.0) -> torch.Tensor:
    """csrc/ops/fma_cuda.cu:92-95, csrc/ops/fma.cpp:72-118:
    ``out = c10(float(x) * (y + scale_add) + z)`` with y, z broadcast over the
    token dim (``row / (S / S_y)``); x is e4m3 [B, S, dim]."""
    assert x.dim() == 3
    xf = x.to(torch.float32)
    yf = y.to(torch.float32) + torch.tensor(scale_add, dtype=torch.float32)
    zf = z.to(torch.float32)
    return c10_e4m3(xf * yf + zf)


def gelu_forward(x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/gelu_forward_cuda.cu:12-16,72-100."""
    if out_dtype is None:
        out_dtype = x.dtype
    return cast_out(gelu_tanh(x.to(torch.float32)), out_dtype)


# --------------------------------------------------------------------------- a5 / a6 attention

def flash_attention(q8: torch.Tensor, k8: torch.Tensor, v8t: torch.Tensor, softmax_scale: float,
                    batch_mask: Optional[torch.Tensor] = None, out_dtype: torch.dtype = E4M3,
                    block_n: int = 64) -> torch.Tensor:
    """Reference-faithful FP8 flash attention forward
    (csrc/flash_attention/flash_attention_cuda.cu:197-248,395-497,
    flash_attention_cuda_mask.cu:244,319, flash_attention.cpp:31-32).

    q8 [B,H,M,D], k8 [B,H,N,D], v8t [B,H,D,ceil16(N)] are e4m3.  KV blocks of
    ``block_n`` keys are visited from the LAST to the FIRST; per block
    ``m' = max(m, rowmax s)``, ``alpha = 2^((m-m')c)``, ``p = 2^(s c - m' c)``
    (fp32), ``l = l alpha + sum p``, ``o = o alpha + sat(p) v``.  Columns >= N
    get -inf; with a mask, columns >= valid_len[b] get -1e6.  The final
    ``o / l`` is cast with saturation to e4m3 (reference) or rounded to
    ``out_dtype``."""
    B, H, M, D = q8.shape
    N = k8.shape[2]
    c = torch.tensor(softmax_scale * LOG2E, dtype=torch.float32)
    q = q8.to(torch.float32)
    k = k8.to(torch.float32)
    v = v8t.to(torch.float32)[..., :N].transpose(-1, -2)        # [B,H,N,D]
    out = torch.empty(B, H, M, D, dtype=torch.float32)
    n_blocks = (N + block_n - 1) // block_n
    for b in range(B):
        valid = int(batch_mask[b]) if batch_mask is not None else None
        m = torch.full((H, M, 1), float("-inf"))
        l = torch.zeros(H, M, 1)
        o = torch.zeros(H, M, D)
        for blk in range(n_blocks - 1, -1, -1):
            lo, hi = blk * block_n, min((blk + 1) * block_n, N)
            s = torch.matmul(q[b], k[b, :, lo:hi].transpose(-1, -2))      # [H,M,nb]
            if valid is not None:
                cols = torch.arange(lo, hi)
                s = torch.where(cols[None, None, :] >= valid, torch.tensor(-1.0e6), s)
            m_new = torch.maximum(m, s.amax(dim=-1, keepdim=True))
            m_scaled = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new * c)
            alpha = torch.exp2((m - m_new) * c)
            alpha = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(alpha), alpha)
            p = torch.exp2(s * c - m_scaled)
            l = l * alpha + p.sum(dim=-1, keepdim=True)
            p8 = sat_e4m3(p).to(torch.float32)
            o = o * alpha + torch.matmul(p8, v[b, :, lo:hi])
            m = m_new
        inv = torch.where((l == 0) | torch.isnan(l), torch.ones_like(l), 1.0 / l)
        out[b] = o * inv
    if out_dtype == E4M3:
        return sat_e4m3(out)
    return out.to(out_dtype)


def attention_exact(q8, k8, v8t, softmax_scale, batch_mask=None):
    """Exact softmax attention on the dequantised e4m3 operands (float64);
    reported as a distance, not used as a gate."""
    N = k8.shape[2]
    q, k = q8.to(torch.float64), k8.to(torch.float64)
    v = v8t.to(torch.float64)[..., :N].transpose(-1, -2)
    s = torch.matmul(q, k.transpose(-1, -2)) * softmax_scale
    if batch_mask is not None:
        cols = torch.arange(N)
        for b in range(q.shape[0]):
            s[b][..., cols >= int(batch_mask[b])] = float("-inf")
    return torch.matmul(torch.softmax(s, dim=-1), v).to(torch.float32)


def flash_attn_func(q, k, v, softmax_scale=None, batch_mask=None, apply_qk_hadamard=False,
                    out_dtype: torch.dtype = E4M3) -> torch.Tensor:
    """q8_kernels/functional/flash_attention.py:16-61 (FlashAttnFunc.forward):
    pad D to a multiple of 32, V -> [B,H,D,S] padded to a multiple of 16 keys and
    cast c10 to e4m3 unscaled, Q/K either Hadamard-rotated with the softmax
    scale folded in (kernel scale 1) or cast c10 (kernel scale softmax_scale)."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    d_og = q.shape[3]
    if d_og % 32 != 0:
        pad = 32 - d_og % 32
        q, k, v = (torch.nn.functional.pad(t, [0, pad]) for t in (q, k, v))
    vt = v.transpose(2, 3).contiguous()
    if vt.shape[-1] % 16 != 0:
        vt = torch.nn.functional.pad(vt, (0, 16 - vt.shape[-1] % 16))
    if vt.dtype != E4M3:
        vt = c10_e4m3(vt)
    if apply_qk_hadamard:
        hd = math.sqrt(1 / q.shape[-1]) * math.sqrt(softmax_scale)
        q8 = hadamard_transform(q, scale=hd, out_dtype=E4M3)
        k8 = hadamard_transform(k, scale=hd, out_dtype=E4M3)
        o = flash_attention(q8, k8, vt, 1.0, batch_mask, out_dtype)
    else:
        q8 = q if q.dtype == E4M3 else c10_e4m3(q)
        k8 = k if k.dtype == E4M3 else c10_e4m3(k)
        o = flash_attention(q8, k8, vt, softmax_scale, batch_mask, out_dtype)
    return o[..., :d_og]


# --------------------------------------------------------------------------- a14 RoPE table

def precompute_freqs_cis(indices_grid: torch.Tensor, dim: int = 2048, theta: float = 10000.0,
                         max_pos=(20, 2048, 2048)) -> Tuple[torch.Tensor, torch.Tensor]:
    """q8_kernels/models/LTXVideo.py:95-148 ("exp" spacing): fractional 3-D
    positions, dim//6 exponentially spaced frequencies times pi/2, cos/sin
    repeated per interleaved pair and left-padded with cos=1, sin=0."""
    frac = torch.stack([indices_grid[:, i] / max_pos[i] for i in range(3)], dim=-1)   # [B,S,3]
    idx = theta ** torch.linspace(math.log(1, theta), math.log(theta, theta), dim // 6, dtype=torch.float32)
    idx = idx * math.pi / 2
    freqs = (idx * (frac.unsqueeze(-1) * 2 - 1)).transpose(-1, -2).flatten(2)
    cos = freqs.cos().repeat_interleave(2, dim=-1)
    sin = freqs.sin().repeat_interleave(2, dim=-1)
    if dim % 6 != 0:
        cos = torch.cat([torch.ones_like(cos[:, :, : dim % 6]), cos], dim=-1)
        sin = torch.cat([torch.zeros_like(sin[:, :, : dim % 6]), sin], dim=-1)
    return cos.float(), sin.float()


# --------------------------------------------------------------------------- metrics

def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative Frobenius error ||a-b|| / ||b|| in float64."""
    a64, b64 = a.to(torch.float64), b.to(torch.float64)
    den = torch.linalg.norm(b64)
    return float(torch.linalg.norm(a64 - b64) / den) if den > 0 else float(torch.linalg.norm(a64))
