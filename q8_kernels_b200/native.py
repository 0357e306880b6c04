"""Tensor-level mirror of the reference's four pybind extension modules
(``q8_kernels_cuda.{quantizer,ops,gemm,flash_attention}._C``): same function
names, positional arguments, ``None`` for ``std::optional`` and the same output
shapes / default dtypes.  Each function checks its arguments, allocates the
output with torch's caching allocator on the input's device and launches the
sm_100a kernel through the C ABI on torch's current stream.  Nothing here
synchronises.
"""
from __future__ import annotations

import math
from typing import Sequence, List, Optional, Tuple

import ctypes

import torch

from . import _lib
from ._lib import Q8KernelError, check, dt, lib, ptr, require_cuda, stream_ptr

E4M3 = torch.float8_e4m3fn


def _rows_view(x: torch.Tensor) -> torch.Tensor:
    """[..., dim] -> [rows, dim] with a contiguous last dim, as the reference's
    ``x.reshape({-1, dim}); if (x.stride(-1) != 1) x = x.contiguous()``."""
    x2 = x.reshape(-1, x.shape[-1])
    row_bytes = x2.stride(0) * x2.element_size()
    if (x2.stride(-1) != 1 or (x2.shape[0] > 1 and (x2.stride(0) < x2.shape[1] or row_bytes % 16))
            or x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


def _row_stride(x2: torch.Tensor) -> int:
    return x2.stride(0) if x2.shape[0] > 1 else x2.shape[1]


# ---------------------------------------------------------------- quantizer._C

def tokenwise_quant(x: torch.Tensor, out_type: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """csrc/quantizer/tokenwise_quant.cpp:74-111.  Returns ``[q, scales]`` with
    q shaped like x (int8 by default, or e4m3) and fp32 scales shaped x.shape[:-1]."""
    dev = require_cuda(x)
    out_type = torch.int8 if out_type is None else out_type
    if out_type not in (torch.int8, E4M3):
        raise Q8KernelError(f"tokenwise_quant: out_type {out_type} must be int8 or float8_e4m3fn")
    shape = x.shape
    x2 = _rows_view(x)
    rows, dim = x2.shape
    q = torch.empty((rows, dim), dtype=out_type, device=dev)
    scales = torch.empty((rows,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_tokenwise_quant(ptr(x2), dt(x2.dtype), ptr(q), dt(out_type), ptr(scales), rows, dim,
                                      _row_stride(x2), stream_ptr(dev)), "tokenwise_quant")
    return [q.reshape(shape), scales.reshape(shape[:-1])]


# ---------------------------------------------------------------- ops._C

def fast_hadamard_transform(x: torch.Tensor, scale: float, out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/fast_hadamard/fast_hadamard_transform.cpp:70-121."""
    dev = require_cuda(x)
    if x.dtype not in (torch.bfloat16, E4M3):
        raise Q8KernelError(f"fast_hadamard_transform: input dtype {x.dtype} must be bfloat16 or float8_e4m3fn")
    out_type = x.dtype if out_type is None else out_type
    shape = x.shape
    x2 = _rows_view(x)
    dim_og = x2.shape[1]
    if dim_og % 8 != 0:
        x2 = torch.nn.functional.pad(x2, (0, 8 - dim_og % 8))
    rows, dim = x2.shape
    out = torch.empty((rows, dim), dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_fast_hadamard_transform(ptr(x2), dt(x2.dtype), ptr(out), dt(out_type), rows, dim,
                                              _row_stride(x2), float(scale), stream_ptr(dev)),
              "fast_hadamard_transform")
    if dim != dim_og:
        out = out[:, :dim_og]
    return out.reshape(shape)


def hadamard_quant(x: torch.Tensor, scale: float, out_type: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """Fused ``tokenwise_quant(fast_hadamard_transform(x, scale), out_type)`` in
    one pass; bit-identical to the two-kernel chain of
    q8_kernels/functional/linear.py:30-31."""
    dev = require_cuda(x)
    out_type = torch.int8 if out_type is None else out_type
    shape = x.shape
    x2 = _rows_view(x)
    rows, dim = x2.shape
    q = torch.empty((rows, dim), dtype=out_type, device=dev)
    scales = torch.empty((rows,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_hadamard_quant(ptr(x2), dt(x2.dtype), ptr(q), dt(out_type), ptr(scales), rows, dim,
                                     _row_stride(x2), float(scale), stream_ptr(dev)), "hadamard_quant")
    return [q.reshape(shape), scales.reshape(shape[:-1])]


def norm_modulate_quant(x: torch.Tensor, mod_scale: torch.Tensor, mod_shift: torch.Tensor,
                        out_type: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """RMS norm (no affine weight) -> ``n * (1 + mod_scale) + mod_shift`` -> Hadamard (1/sqrt(dim)) ->
    per-token quantizer in one kernel, keeping the bf16 roundings of the separate ops
    (q8_kernels/blocks/ltx_transformer_block.py:38-39,53-54 + functional/linear.py:30-31).
    x bf16 [B, S, dim]; mod_scale / mod_shift bf16 [B, 1, dim].  Returns ``[q, scales]``."""
    dev = require_cuda(x, mod_scale, mod_shift)
    out_type = torch.int8 if out_type is None else out_type
    if x.dtype != torch.bfloat16 or mod_scale.dtype != torch.bfloat16 or mod_shift.dtype != torch.bfloat16:
        raise Q8KernelError("norm_modulate_quant: x and the modulation rows must be bfloat16")
    if x.dim() != 3 or tuple(mod_scale.shape) != (x.shape[0], 1, x.shape[2]) or mod_shift.shape != mod_scale.shape:
        raise Q8KernelError("norm_modulate_quant: x must be [B,S,dim] and the modulation rows [B,1,dim]")
    B, S, dim = x.shape
    x = x.contiguous()
    mod_scale = mod_scale.contiguous()
    mod_shift = mod_shift.contiguous()
    q = torch.empty((B, S, dim), dtype=out_type, device=dev)
    scales = torch.empty((B, S), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_norm_modulate_quant(ptr(x), ptr(mod_scale), ptr(mod_shift), ptr(q), dt(out_type), ptr(scales),
                                          B * S, dim, S, float(1.0 / math.sqrt(dim)), stream_ptr(dev)),
              "norm_modulate_quant")
    return [q, scales]


def rms_norm(x: torch.Tensor, weights: Optional[torch.Tensor] = None,
             out_type: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """csrc/ops/rms_norm.cpp:103-154.  Returns ``[out, rsqrt_per_row]``."""
    dev = require_cuda(x, weights)
    if weights is not None and weights.dtype != torch.float32:
        raise Q8KernelError("rms_norm: weights must be float32")
    out_type = x.dtype if out_type is None else out_type
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    rows, dim = x2.shape
    if weights is not None:
        weights = weights.contiguous()
        if weights.numel() != dim:
            raise Q8KernelError("rms_norm: weights size does not match the last dim")
    out = torch.empty((rows, dim), dtype=out_type, device=dev)
    rrms = torch.empty((rows,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_rms_norm(ptr(x2), dt(x2.dtype), ptr(weights), ptr(out), dt(out_type), ptr(rrms), rows, dim,
                               stream_ptr(dev)), "rms_norm")
    return [out.reshape(shape), rrms.reshape(shape[:-1])]


def rope(x: torch.Tensor, cos_freqs: torch.Tensor, sin_freqs: torch.Tensor,
         out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/rope.cpp:96-146.  cos/sin are fp32 with x's shape, or with a
    leading batch of 1 that is shared by every batch entry of x."""
    dev = require_cuda(x, cos_freqs, sin_freqs)
    if cos_freqs.dtype != torch.float32 or sin_freqs.dtype != torch.float32:
        raise Q8KernelError("rope: cos/sin tables must be float32")
    if cos_freqs.shape != sin_freqs.shape:
        raise Q8KernelError("rope: cos and sin shapes differ")
    out_type = x.dtype if out_type is None else out_type
    shape = x.shape
    dim = shape[-1]
    x2 = x.reshape(-1, dim).contiguous()
    rows = x2.shape[0]
    c2 = cos_freqs.reshape(-1, dim).contiguous()
    s2 = sin_freqs.reshape(-1, dim).contiguous()
    if c2.shape[0] == rows:
        freq_rows = 0
    elif rows % c2.shape[0] == 0 and cos_freqs.dim() == x.dim() and cos_freqs.shape[0] == 1:
        freq_rows = c2.shape[0]
    else:
        raise Q8KernelError(f"rope: table shape {tuple(cos_freqs.shape)} does not match x {tuple(shape)}")
    out = torch.empty((rows, dim), dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_rope(ptr(x2), dt(x2.dtype), ptr(c2), ptr(s2), ptr(out), dt(out_type), rows, dim, freq_rows,
                           stream_ptr(dev)), "rope")
    return out.reshape(shape)


def fma_8bit(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, scale_add: float) -> torch.Tensor:
    """csrc/ops/fma.cpp:72-118: ``e4m3(float(x) * (y + scale_add) + z)``, x e4m3
    [B,S,dim], y and z [B, S or 1, dim]."""
    dev = require_cuda(x, y, z)
    if x.dtype != E4M3:
        raise Q8KernelError("fma_8bit: x must be float8_e4m3fn")
    if x.dim() != 3:
        raise Q8KernelError("fma_8bit: x must be 3-D")
    dim = x.shape[-1]
    if y.shape[-1] != dim or z.shape[-1] != dim:
        raise Q8KernelError("fma: channels missmatch")
    if y.shape[-2] not in (x.shape[-2], 1) or z.shape[-2] not in (x.shape[-2], 1):
        raise Q8KernelError("fma: token missmatch")
    y_every = x.shape[-2] // y.shape[-2]
    z_every = x.shape[-2] // z.shape[-2]
    x2 = x.reshape(-1, dim).contiguous()
    y2 = y.reshape(-1, dim).contiguous()
    z2 = z.reshape(-1, dim).contiguous()
    out = torch.empty_like(x2)
    with torch.cuda.device(dev):
        check(lib.q8k_fma_8bit(ptr(x2), ptr(y2), dt(y2.dtype), ptr(z2), dt(z2.dtype), ptr(out), x2.shape[0], dim,
                               y_every, z_every, float(scale_add), stream_ptr(dev)), "fma_8bit")
    return out.reshape(x.shape)


def gelu_forward(x: torch.Tensor, out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/gelu_act.cpp:132-172."""
    dev = require_cuda(x)
    out_type = x.dtype if out_type is None else out_type
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    out = torch.empty(x2.shape, dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_gelu_forward(ptr(x2), dt(x2.dtype), ptr(out), dt(out_type), x2.shape[0], x2.shape[1],
                                   stream_ptr(dev)), "gelu_forward")
    return out.reshape(shape)


def gelu_backward(x: torch.Tensor, grad_output: torch.Tensor, out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/gelu_act.cpp:84-129: ``grad_output * d gelu_tanh(x) / dx``.  The reference kernel reads
    ``grad_output`` in the output dtype; a gradient of another dtype is cast to it first."""
    dev = require_cuda(x, grad_output)
    if grad_output.shape != x.shape:
        raise Q8KernelError("gelu_backward: grad_output and x shapes differ")
    out_type = x.dtype if out_type is None else out_type
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    g2 = grad_output.reshape(-1, shape[-1]).to(out_type).contiguous()
    out = torch.empty(x2.shape, dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_gelu_backward(ptr(x2), dt(x2.dtype), ptr(g2), ptr(out), dt(out_type), x2.shape[0], x2.shape[1],
                                    stream_ptr(dev)), "gelu_backward")
    return out.reshape(shape)


def rope_backward(grad_out: torch.Tensor, cos_freqs: torch.Tensor, sin_freqs: torch.Tensor,
                  out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/rope.cpp:150-199: the transposed rotation applied to the incoming gradient."""
    dev = require_cuda(grad_out, cos_freqs, sin_freqs)
    if cos_freqs.dtype != torch.float32 or sin_freqs.dtype != torch.float32:
        raise Q8KernelError("rope_backward: cos/sin tables must be float32")
    if cos_freqs.shape != sin_freqs.shape:
        raise Q8KernelError("rope_backward: cos and sin shapes differ")
    out_type = grad_out.dtype if out_type is None else out_type
    shape = grad_out.shape
    dim = shape[-1]
    g2 = grad_out.reshape(-1, dim).contiguous()
    rows = g2.shape[0]
    c2 = cos_freqs.reshape(-1, dim).contiguous()
    s2 = sin_freqs.reshape(-1, dim).contiguous()
    if c2.shape[0] == rows:
        freq_rows = 0
    elif rows % c2.shape[0] == 0 and cos_freqs.dim() == grad_out.dim() and cos_freqs.shape[0] == 1:
        freq_rows = c2.shape[0]
    else:
        raise Q8KernelError(f"rope_backward: table shape {tuple(cos_freqs.shape)} does not match {tuple(shape)}")
    out = torch.empty((rows, dim), dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_rope_backward(ptr(g2), dt(g2.dtype), ptr(c2), ptr(s2), ptr(out), dt(out_type), rows, dim,
                                    freq_rows, stream_ptr(dev)), "rope_backward")
    return out.reshape(shape)


def rms_norm_backward(x_normed: torch.Tensor, x_norms: torch.Tensor, grad_out: torch.Tensor,
                      weights: Optional[torch.Tensor] = None, out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/ops/rms_norm.cpp:157-214: gradient w.r.t. the input of ``rms_norm`` from its saved output
    ``x_normed`` and per-row ``x_norms``.  ``grad_out`` is read in the output dtype, as in the reference."""
    dev = require_cuda(x_normed, x_norms, grad_out, weights)
    if weights is not None and weights.dtype != torch.float32:
        raise Q8KernelError("rms_norm_backward: weights must be float32")
    if grad_out.shape != x_normed.shape:
        raise Q8KernelError("rms_norm_backward: grad_out and x_normed shapes differ")
    out_type = x_normed.dtype if out_type is None else out_type
    shape = x_normed.shape
    y2 = x_normed.reshape(-1, shape[-1]).contiguous()
    g2 = grad_out.reshape(-1, shape[-1]).to(out_type).contiguous()
    rows, dim = y2.shape
    r = x_norms.reshape(-1).to(torch.float32).contiguous()
    if r.numel() != rows:
        raise Q8KernelError("rms_norm_backward: x_norms must hold one value per row")
    if weights is not None:
        weights = weights.contiguous()
        if weights.numel() != dim:
            raise Q8KernelError("rms_norm_backward: weights size does not match the last dim")
    out = torch.empty((rows, dim), dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_rms_norm_backward(ptr(y2), dt(y2.dtype), ptr(r), ptr(g2), ptr(weights), ptr(out), dt(out_type),
                                        rows, dim, stream_ptr(dev)), "rms_norm_backward")
    return out.reshape(shape)


# ---------------------------------------------------------------- gemm._C

def _gemm(fn, name, a, b, bias, a_scales, b_scales, fuse_gelu, out_type, in_dtype):
    dev = require_cuda(a, b, bias, a_scales, b_scales)
    for t, what in ((a, "a"), (b, "b"), (bias, "bias"), (a_scales, "a_scales"), (b_scales, "b_scales")):
        if t is not None and not t.is_contiguous():
            raise Q8KernelError(f"{name}: {what} must be contiguous")
    if a.dtype != in_dtype or b.dtype != in_dtype:
        raise Q8KernelError(f"{name}: a and b must be {in_dtype}")
    if a_scales.dtype != torch.float32 or b_scales.dtype != torch.float32:
        raise Q8KernelError(f"{name}: scales must be float32")
    if bias is not None and bias.dtype != torch.float32:
        raise Q8KernelError(f"{name}: bias must be float32")
    bs_a, m = (a.shape[0], a.shape[1]) if a.dim() == 3 else (1, a.shape[0])
    bs_b, n = (b.shape[0], b.shape[1]) if b.dim() == 3 else (1, b.shape[0])
    k = a.shape[-1]
    if b.shape[-1] != k:
        raise Q8KernelError(f"{name}: K mismatch ({k} vs {b.shape[-1]})")
    if not (bs_a == bs_b or bs_a == 1 or bs_b == 1):
        raise Q8KernelError("Batch missmatch")
    if a_scales.numel() != bs_a * m or b_scales.numel() != bs_b * n:
        raise Q8KernelError(f"{name}: scale sizes do not match the operands")
    if bias is not None and bias.numel() != n:
        raise Q8KernelError(f"{name}: bias size does not match N")
    batch = max(bs_a, bs_b)
    out_type = E4M3 if out_type is None else out_type
    out = torch.empty((batch, m, n), dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(fn(ptr(a), ptr(b), ptr(bias), ptr(a_scales), ptr(b_scales), ptr(out), dt(out_type), bs_a, bs_b,
                 m, n, k, int(bool(fuse_gelu)), ptr(_lib.status_word(dev)), stream_ptr(dev)), name)
    return out


def q8_mm(a, b, a_scales, b_scales, fuse_gelu: bool, out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/gemm/q8_gemm_api.cpp:40-97."""
    return _gemm(lib.q8k_q8_mm, "q8_mm", a, b, None, a_scales, b_scales, fuse_gelu, out_type, torch.int8)


def q8_mm_bias(a, b, bias, a_scales, b_scales, fuse_gelu: bool, out_type: Optional[torch.dtype] = None):
    """csrc/gemm/q8_gemm_api.cpp:100-164."""
    return _gemm(lib.q8k_q8_mm, "q8_mm_bias", a, b, bias, a_scales, b_scales, fuse_gelu, out_type, torch.int8)


def fp8_mm(a, b, a_scales, b_scales, fuse_gelu: bool, out_type: Optional[torch.dtype] = None) -> torch.Tensor:
    """csrc/gemm/q8_gemm_api.cpp:167-224."""
    return _gemm(lib.q8k_fp8_mm, "fp8_mm", a, b, None, a_scales, b_scales, fuse_gelu, out_type, E4M3)


def fp8_mm_bias(a, b, bias, a_scales, b_scales, fuse_gelu: bool, out_type: Optional[torch.dtype] = None):
    """csrc/gemm/q8_gemm_api.cpp:227-291."""
    return _gemm(lib.q8k_fp8_mm, "fp8_mm_bias", a, b, bias, a_scales, b_scales, fuse_gelu, out_type, E4M3)


def mm_gate_residual(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], a_scales: torch.Tensor,
                     b_scales: torch.Tensor, gate: Optional[torch.Tensor], resid: torch.Tensor) -> torch.Tensor:
    """``bf16(bf16(gate * bf16(linear)) + resid)`` with the gate/residual in the GEMM epilogue: the
    q8_mm_bias (or fp8_mm_bias) call plus the two torch ops of
    q8_kernels/blocks/ltx_transformer_block.py:41,52,56, bit-identical to running them separately.
    a int8|e4m3 [B,S,K] (or [M,K]); b [N,K]; gate bf16 [B,1,N] or None; resid bf16 shaped like the output."""
    dev = require_cuda(a, b, bias, a_scales, b_scales, gate, resid)
    if a.dtype != b.dtype or a.dtype not in (torch.int8, E4M3):
        raise Q8KernelError("mm_gate_residual: a and b must both be int8 or both float8_e4m3fn")
    bs_a, m = (a.shape[0], a.shape[1]) if a.dim() == 3 else (1, a.shape[0])
    n, k = b.shape
    if b.dim() != 2 or a.shape[-1] != k:
        raise Q8KernelError("mm_gate_residual: b must be [N,K] with K matching a")
    if resid.dtype != torch.bfloat16 or resid.numel() != bs_a * m * n:
        raise Q8KernelError("mm_gate_residual: resid must be bfloat16 with the output's shape")
    rows_per_gate = 1
    if gate is not None:
        if gate.dtype != torch.bfloat16 or gate.numel() != bs_a * n:
            raise Q8KernelError("mm_gate_residual: gate must be bfloat16 [B,1,N]")
        gate = gate.contiguous()
        rows_per_gate = m
    a, b, resid = a.contiguous(), b.contiguous(), resid.contiguous()
    a_scales, b_scales = a_scales.contiguous(), b_scales.contiguous()
    out = torch.empty((bs_a, m, n), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_mm_gate_residual(int(a.dtype == torch.int8), ptr(a), ptr(b), ptr(bias), ptr(a_scales), ptr(b_scales),
                                       ptr(gate), ptr(resid), rows_per_gate, ptr(out), bs_a, 1, m, n, k,
                                       ptr(_lib.status_word(dev)), stream_ptr(dev)), "mm_gate_residual")
    return out


# ---------------------------------------------------------------- flash_attention._C

def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                    batch_mask: Optional[torch.Tensor] = None,
                    out_type: Optional[torch.dtype] = None, token_major_out: bool = False,
                    v_rows: bool = False) -> torch.Tensor:
    """csrc/flash_attention/flash_attention.cpp:18-48: q [B,H,M,64], k [B,H,N,64],
    v [B,H,64,ceil16(N)] e4m3, optional int32 [B] valid-key counts; the output is
    e4m3 [B,H,M,64] like the reference unless ``out_type`` asks for bfloat16.
    ``token_major_out`` stores the result as [B,M,H,64] and returns its [B,H,M,64] view, so the
    caller's ``transpose(1,2).reshape(B,M,H*64)`` is free.  ``v_rows``: v is [B,H,N,64] (rows, like k)
    instead of the reference's transposed layout; same result, no transpose pass needed."""
    dev = require_cuda(q, k, v, batch_mask)
    if q.dtype != E4M3 or k.dtype != E4M3 or v.dtype != E4M3:
        raise Q8KernelError("flash_attention: q, k, v must be float8_e4m3fn")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise Q8KernelError("flash_attention: q, k, v must be 4-D")
    B, H, M, D = q.shape
    N = k.shape[2]
    if D != 64 or k.shape[3] != 64:
        raise Q8KernelError("flash_attention: head dim must be 64")
    n_pad = (N + 15) // 16 * 16
    if v_rows:
        if tuple(v.shape) != (B, H, N, 64) or tuple(k.shape[:2]) != (B, H):
            raise Q8KernelError("flash_attention: with v_rows, v must be [B,H,N,64] like k")
    elif tuple(v.shape) != (B, H, 64, n_pad) or tuple(k.shape[:2]) != (B, H):
        raise Q8KernelError(f"flash_attention: v must be [B,H,64,{n_pad}] (transposed, keys padded to 16)")
    if batch_mask is not None:
        if batch_mask.dtype != torch.int32:
            raise Q8KernelError("flash_attention: batch_mask must be int32")
        if batch_mask.dim() != 1 or batch_mask.shape[0] != B:
            raise Q8KernelError("flash_attention: batch_mask must have shape [B]")
        batch_mask = batch_mask.contiguous()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out_type = E4M3 if out_type is None else out_type
    if token_major_out:
        buf = torch.empty((B, M, H, 64), dtype=out_type, device=dev)
        strides = (M * H * 64, 64, H * 64)
    else:
        buf = torch.empty((B, H, M, 64), dtype=out_type, device=dev)
        strides = (H * M * 64, M * 64, 64)
    with torch.cuda.device(dev):
        if v_rows:
            outs = (ctypes.c_void_p * 1)(buf.data_ptr())
            check(lib.q8k_flash_attention_v_rows(ptr(q), ptr(k), ptr(v), ctypes.cast(outs, ctypes.c_void_p), 1,
                                                 dt(out_type), B, H, M, N, *strides, float(softmax_scale),
                                                 ptr(batch_mask), ptr(_lib.status_word(dev)), stream_ptr(dev)),
                  "flash_attention")
        else:
            check(lib.q8k_flash_attention_strided(ptr(q), ptr(k), ptr(v), ptr(buf), dt(out_type), B, H, M, N, *strides,
                                                  float(softmax_scale), ptr(batch_mask), ptr(_lib.status_word(dev)),
                                                  stream_ptr(dev)), "flash_attention")
    return buf.transpose(1, 2) if token_major_out else buf


def flash_attention_into(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                         batch_mask: Optional[torch.Tensor], out_type: torch.dtype, dest_ptrs: Sequence[int],
                         total_heads: int, first_head: int, v_rows: bool = False) -> None:
    """Head-sharded attention writing straight into full token-major buffers: q, k, v hold this rank's
    heads ([B,h,M,64] etc.); every address in ``dest_ptrs`` is the start of a [B,M,total_heads,64] buffer
    of ``out_type`` (this GPU's, or a peer's mapped with ``q8k_ipc_open``) and receives heads
    ``first_head .. first_head+h`` of the result.  Returns nothing: the buffers are the result."""
    dev = require_cuda(q, k, v, batch_mask)
    if q.dtype != E4M3 or k.dtype != E4M3 or v.dtype != E4M3:
        raise Q8KernelError("flash_attention: q, k, v must be float8_e4m3fn")
    B, h, M, D = q.shape
    N = k.shape[2]
    n_pad = (N + 15) // 16 * 16
    if D != 64 or tuple(k.shape) != (B, h, N, 64) or tuple(v.shape) != ((B, h, N, 64) if v_rows else (B, h, 64, n_pad)):
        raise Q8KernelError("flash_attention: q [B,h,M,64], k [B,h,N,64], v [B,h,64,ceil16(N)] (or [B,h,N,64] with v_rows) expected")
    if not (0 <= first_head and first_head + h <= total_heads):
        raise Q8KernelError("flash_attention: head range outside the destination buffers")
    if not 1 <= len(dest_ptrs) <= 8:
        raise Q8KernelError("flash_attention: between 1 and 8 destinations")
    if batch_mask is not None:
        if batch_mask.dtype != torch.int32 or batch_mask.dim() != 1 or batch_mask.shape[0] != B:
            raise Q8KernelError("flash_attention: batch_mask must be int32 [B]")
        batch_mask = batch_mask.contiguous()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    esz = 1 if out_type == E4M3 else 2
    head_off = first_head * 64 * esz
    outs = (ctypes.c_void_p * len(dest_ptrs))(*[int(a) + head_off for a in dest_ptrs])
    strides = (M * total_heads * 64, 64, total_heads * 64)
    with torch.cuda.device(dev):
        fn = lib.q8k_flash_attention_v_rows if v_rows else lib.q8k_flash_attention_multi_out
        check(fn(ptr(q), ptr(k), ptr(v), ctypes.cast(outs, ctypes.c_void_p), len(dest_ptrs), dt(out_type), B, h, M, N,
                 *strides, float(softmax_scale), ptr(batch_mask), ptr(_lib.status_word(dev)), stream_ptr(dev)),
              "flash_attention")


def attention_prep(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, apply_hadamard: bool,
                   qk_scale: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One launch group replacing the torch glue of
    q8_kernels/functional/flash_attention.py:30-60 for bf16 inputs with head dim
    64: q, k, v are [B,H,S,64] tensors or views (any batch / token / head
    strides, last dim contiguous).  Returns q8, k8 [B,H,S,64] and
    vt8 [B,H,64,ceil16(S_kv)] in e4m3."""
    dev = require_cuda(q, k, v)
    B, H, S_q, D = q.shape
    S_kv = k.shape[2]
    if D != 64 or k.shape[3] != 64 or v.shape[3] != 64:
        raise Q8KernelError("attention_prep: head dim must be 64")
    if v.shape[2] != S_kv:
        raise Q8KernelError("v tokens != k tokens")
    fixed = []
    for t in (q, k, v):
        if t.dtype != torch.bfloat16:
            raise Q8KernelError("attention_prep: inputs must be bfloat16")
        if t.stride(3) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
            t = t.contiguous()
        fixed.append(t)
    q, k, v = fixed
    s_pad = (S_kv + 15) // 16 * 16
    q8 = torch.empty((B, H, S_q, 64), dtype=E4M3, device=dev)
    k8 = torch.empty((B, H, S_kv, 64), dtype=E4M3, device=dev)
    vt8 = torch.empty((B, H, 64, s_pad), dtype=E4M3, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_attention_prep(ptr(q), ptr(k), ptr(v), ptr(q8), ptr(k8), ptr(vt8), B, H, S_q, S_kv,
                                     q.stride(0), q.stride(2), q.stride(1),
                                     k.stride(0), k.stride(2), k.stride(1),
                                     v.stride(0), v.stride(2), v.stride(1),
                                     int(bool(apply_hadamard)), float(qk_scale), stream_ptr(dev)), "attention_prep")
    return q8, k8, vt8


def qk_norm_rope_prep(x: torch.Tensor, norm_w: torch.Tensor, freqs_cis, num_heads: int, apply_hadamard: bool,
                      qk_scale: float) -> torch.Tensor:
    """q_norm / k_norm (RMS norm with fp32 weight over all heads) + optional RoPE + per-head Hadamard +
    e4m3 cast in one kernel: x bf16 [B,S,H*64] (row-strided views allowed) -> e4m3 [B,H,S,64], with the
    bf16 roundings of q8_kernels/modules/attention.py:54-68 and functional/flash_attention.py:50-54.
    ``freqs_cis`` is None or (cos, sin) fp32 [1,S,H*64]."""
    dev = require_cuda(x, norm_w)
    if x.dtype != torch.bfloat16 or x.dim() != 3 or x.shape[2] != num_heads * 64 or x.stride(2) != 1:
        raise Q8KernelError("qk_norm_rope_prep: x must be bfloat16 [B,S,H*64] with contiguous channels")
    if norm_w.dtype != torch.float32 or norm_w.numel() != x.shape[2]:
        raise Q8KernelError("qk_norm_rope_prep: norm weight must be float32 [H*64]")
    B, S, C = x.shape
    if x.stride(0) != S * x.stride(1) or x.stride(1) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    cos = sin = None
    if freqs_cis is not None:
        cos, sin = freqs_cis
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.numel() != S * C or sin.numel() != S * C:
            raise Q8KernelError("qk_norm_rope_prep: rotary tables must be float32 [1,S,H*64]")
        cos, sin = cos.contiguous(), sin.contiguous()
    out = torch.empty((B, num_heads, S, 64), dtype=E4M3, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_qk_norm_rope_prep(ptr(x), x.stride(1), ptr(norm_w.contiguous()), ptr(cos), ptr(sin), ptr(out), B, S,
                                        num_heads, int(bool(apply_hadamard)), float(qk_scale), stream_ptr(dev)),
              "qk_norm_rope_prep")
    return out


def kv_prep(xk: torch.Tensor, xv: torch.Tensor, norm_wk: torch.Tensor, num_heads: int, apply_hadamard: bool,
            qk_scale: float):
    """K and V of a cross-attention (two column slices of one fused projection output, same strides) in one
    launch: K as qk_norm_rope_prep without rotation, V cast to e4m3 rows; returns (k8, v8), each [B,H,S,64]."""
    dev = require_cuda(xk, xv, norm_wk)
    C = num_heads * 64
    for x in (xk, xv):
        if x.dtype != torch.bfloat16 or x.dim() != 3 or x.shape[2] != C or x.stride(2) != 1:
            raise Q8KernelError("kv_prep: inputs must be bfloat16 [B,S,H*64] with contiguous channels")
    if xk.shape != xv.shape:
        raise Q8KernelError("kv_prep: k and v must have the same shape")
    B, S, _ = xk.shape
    ok = all(x.stride(0) == S * x.stride(1) and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0 for x in (xk, xv))
    if not ok or xk.stride() != xv.stride():
        xk, xv = xk.contiguous(), xv.contiguous()
    if norm_wk.dtype != torch.float32 or norm_wk.numel() != C:
        raise Q8KernelError("kv_prep: the norm weight must be float32 [H*64]")
    outk = torch.empty((B, num_heads, S, 64), dtype=E4M3, device=dev)
    outv = torch.empty((B, num_heads, S, 64), dtype=E4M3, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_qkv_prep(None, ptr(xk), ptr(xv), xk.stride(1), None, ptr(norm_wk.contiguous()), None, None, None,
                               ptr(outk), ptr(outv), B, S, num_heads, int(bool(apply_hadamard)), float(qk_scale),
                               stream_ptr(dev)), "qkv_prep")
    return outk, outv


def qk_norm_rope_prep_pair(xq: torch.Tensor, xk: torch.Tensor, norm_wq: torch.Tensor, norm_wk: torch.Tensor, freqs_cis,
                           num_heads: int, apply_hadamard: bool, qk_scale: float, xv: Optional[torch.Tensor] = None):
    """qk_norm_rope_prep for the Q and K of one self-attention in a single launch (same shape and
    strides, e.g. column slices of a fused projection output); returns (q8, k8), each e4m3 [B,H,S,64],
    byte-identical to two separate calls.  With ``xv`` (a third slice of the same kind) the launch also
    casts V to e4m3 rows [B,H,S,64] (what attention_cast_rows gives) and (q8, k8, v8) is returned."""
    dev = require_cuda(xq, xk, norm_wq, norm_wk, xv)
    C = num_heads * 64
    xs = (xq, xk) if xv is None else (xq, xk, xv)
    for x in xs:
        if x.dtype != torch.bfloat16 or x.dim() != 3 or x.shape[2] != C or x.stride(2) != 1:
            raise Q8KernelError("qk_norm_rope_prep_pair: inputs must be bfloat16 [B,S,H*64] with contiguous channels")
    if any(x.shape != xq.shape for x in xs):
        raise Q8KernelError("qk_norm_rope_prep_pair: q, k (and v) must have the same shape")
    B, S, _ = xq.shape
    ok = all(x.stride(0) == S * x.stride(1) and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0 for x in xs)
    if not ok or any(x.stride() != xq.stride() for x in xs):
        xs = tuple(x.contiguous() for x in xs)
        xq, xk = xs[0], xs[1]
        xv = xs[2] if xv is not None else None
    cos = sin = None
    if freqs_cis is not None:
        cos, sin = freqs_cis
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.numel() != S * C or sin.numel() != S * C:
            raise Q8KernelError("qk_norm_rope_prep_pair: rotary tables must be float32 [1,S,H*64]")
        cos, sin = cos.contiguous(), sin.contiguous()
    for w in (norm_wq, norm_wk):
        if w.dtype != torch.float32 or w.numel() != C:
            raise Q8KernelError("qk_norm_rope_prep_pair: norm weights must be float32 [H*64]")
    outq = torch.empty((B, num_heads, S, 64), dtype=E4M3, device=dev)
    outk = torch.empty((B, num_heads, S, 64), dtype=E4M3, device=dev)
    with torch.cuda.device(dev):
        if xv is None:
            check(lib.q8k_qk_norm_rope_prep_pair(ptr(xq), ptr(xk), xq.stride(1), ptr(norm_wq.contiguous()),
                                                 ptr(norm_wk.contiguous()), ptr(cos), ptr(sin), ptr(outq), ptr(outk), B, S,
                                                 num_heads, int(bool(apply_hadamard)), float(qk_scale), stream_ptr(dev)),
                  "qk_norm_rope_prep_pair")
            return outq, outk
        outv = torch.empty((B, num_heads, S, 64), dtype=E4M3, device=dev)
        check(lib.q8k_qkv_prep(ptr(xq), ptr(xk), ptr(xv), xq.stride(1), ptr(norm_wq.contiguous()),
                               ptr(norm_wk.contiguous()), ptr(cos), ptr(sin), ptr(outq), ptr(outk), ptr(outv), B, S,
                               num_heads, int(bool(apply_hadamard)), float(qk_scale), stream_ptr(dev)), "qkv_prep")
    return outq, outk, outv


def attention_prep_v(v: torch.Tensor) -> torch.Tensor:
    """V half of attention_prep: bf16 [B,H,S,64] view -> e4m3 [B,H,64,ceil16(S)] (transposed, zero padded)."""
    dev = require_cuda(v)
    B, H, S, D = v.shape
    if D != 64 or v.dtype != torch.bfloat16:
        raise Q8KernelError("attention_prep_v: v must be bfloat16 with head dim 64")
    if v.stride(3) != 1 or any(s % 8 for s in v.stride()[:3]) or v.data_ptr() % 16:
        v = v.contiguous()
    s_pad = (S + 15) // 16 * 16
    vt8 = torch.empty((B, H, 64, s_pad), dtype=E4M3, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_attention_prep_v(ptr(v), ptr(vt8), B, H, S, v.stride(0), v.stride(2), v.stride(1), stream_ptr(dev)),
              "attention_prep_v")
    return vt8


def attention_cast_rows(v: torch.Tensor) -> torch.Tensor:
    """bf16 [B,H,S,64] view -> e4m3 [B,H,S,64] contiguous (the unscaled ``.to(float8_e4m3fn)`` the
    reference applies to V, q8_kernels/functional/flash_attention.py:47-48), for ``flash_attention(v_rows=True)``."""
    dev = require_cuda(v)
    B, H, S, D = v.shape
    if D != 64 or v.dtype != torch.bfloat16:
        raise Q8KernelError("attention_cast_rows: v must be bfloat16 with head dim 64")
    if v.stride(3) != 1 or any(s % 8 for s in v.stride()[:3]) or v.data_ptr() % 16:
        v = v.contiguous()
    out = torch.empty((B, H, S, 64), dtype=E4M3, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_attention_cast_rows(ptr(v), ptr(out), B, H, S, v.stride(0), v.stride(2), v.stride(1),
                                          stream_ptr(dev)), "attention_cast_rows")
    return out


# ---------------------------------------------------------------- fused linear chain

_workspaces = {}


def linear(x: torch.Tensor, w: torch.Tensor, w_scales: torch.Tensor, bias: Optional[torch.Tensor],
           use_hadamard: bool, fuse_gelu: bool, out_type: torch.dtype) -> torch.Tensor:
    """Hadamard + per-token quantizer + GEMM in one native call over a cached
    per-device scratch buffer (q8_kernels/functional/linear.py:24-42,138-159)."""
    dev = require_cuda(x, w, w_scales, bias)
    K = x.shape[-1]
    x2 = x.reshape(-1, K).contiguous()
    M, N = x2.shape[0], w.shape[0]
    need = lib.q8k_linear_workspace_bytes(M, K)
    if torch.cuda.is_current_stream_capturing():
        # a buffer allocated during capture belongs to that graph's private pool: never cache it
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    else:
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
            _workspaces[key] = ws
    out_shape = (x.shape[0], x.shape[1], N) if x.dim() == 3 else (1, M, N)
    out = torch.empty(out_shape, dtype=out_type, device=dev)
    with torch.cuda.device(dev):
        check(lib.q8k_linear(ptr(x2), dt(x2.dtype), ptr(w), dt(w.dtype), ptr(w_scales), ptr(bias), ptr(out),
                             dt(out_type), M, N, K, int(bool(use_hadamard)), int(bool(fuse_gelu)), ptr(ws),
                             ws.numel(), ptr(_lib.status_word(dev)), stream_ptr(dev)), "linear")
    return out
