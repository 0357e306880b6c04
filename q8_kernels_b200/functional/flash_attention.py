"""FP8 flash attention (reference: q8_kernels/functional/flash_attention.py:16-73).

For bf16 inputs with head dim 64 the reference's torch glue (transpose + pad +
cast of V, Hadamard or cast of Q/K: five full-tensor passes) is one pre-pass
kernel group; the attention kernel itself is the tcgen05 one.
"""
import math
from typing import Optional

import torch

from .. import native
from .fast_hadamard import hadamard_transform

E4M3 = torch.float8_e4m3fn


def is_16bit(x) -> bool:
    return x.dtype == torch.float16 or x.dtype == torch.bfloat16


def flash_attn_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: Optional[float] = None,
                    batch_mask: Optional[torch.Tensor] = None, apply_qk_hadamard: bool = False,
                    out_dtype: Optional[torch.dtype] = None, token_major_out: bool = False) -> torch.Tensor:
    """q [B,H,Sq,D], k,v [B,H,Skv,D] (views allowed); ``batch_mask`` is int32 [B]
    with the number of valid keys per batch entry.  Returns [B,H,Sq,D] in e4m3
    (the reference's output dtype) unless ``out_dtype=torch.bfloat16``.  With ``token_major_out``
    the same values are stored as [B,Sq,H,D] and the [B,H,Sq,D] view of that buffer is returned."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    assert batch_mask is None or (batch_mask.shape[0] == q.shape[0] and batch_mask.ndim == 1)
    assert k.shape[2] == v.shape[2], "v tokens != k tokens"
    head_size_og = q.size(3)

    if head_size_og == 64 and all(t.dtype == torch.bfloat16 for t in (q, k, v)) and v.shape == k.shape:
        if apply_qk_hadamard:
            qk_scale = math.sqrt(1 / 64) * math.sqrt(softmax_scale)
            kernel_scale = 1.0
        else:
            qk_scale, kernel_scale = 1.0, softmax_scale
        q8, k8, vt8 = native.attention_prep(q, k, v, apply_qk_hadamard, qk_scale)
        return native.flash_attention(q8, k8, vt8, kernel_scale, batch_mask, out_dtype, token_major_out)

    # general path, same steps as the reference
    if head_size_og % 32 != 0:
        pad = 32 - head_size_og % 32
        q, k, v = (torch.nn.functional.pad(t, [0, pad]) for t in (q, k, v))
    if q.shape[-1] != 64:
        raise native.Q8KernelError("flash_attn_func: only head dims up to 64 are implemented on sm_100a")
    if v.shape == k.shape:
        v = v.transpose(2, 3).contiguous()
    if v.shape[-1] % 16 != 0:
        v = torch.nn.functional.pad(v, (0, 16 - v.shape[-1] % 16))
    if is_16bit(v):
        v = v.to(E4M3)
    if apply_qk_hadamard:
        hd_scale = math.sqrt(1 / q.shape[-1])
        q = hadamard_transform(q.to(torch.bfloat16) if q.dtype == torch.float16 else q,
                               scale=hd_scale * math.sqrt(softmax_scale), out_type=E4M3)
        k = hadamard_transform(k.to(torch.bfloat16) if k.dtype == torch.float16 else k,
                               scale=hd_scale * math.sqrt(softmax_scale), out_type=E4M3)
        o = native.flash_attention(q, k, v, 1.0, batch_mask, out_dtype)
    else:
        if is_16bit(q):
            q = q.to(E4M3)
        if is_16bit(k):
            k = k.to(E4M3)
        o = native.flash_attention(q.contiguous(), k.contiguous(), v, softmax_scale, batch_mask, out_dtype)
    return o[..., :head_size_og]
