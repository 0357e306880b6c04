"""CPU oracle for the module level of the 8-bit DiT path: Q8Linear, Attention
and LTXTransformerBlock forward, written as plain functions over a state dict
and the op-level oracle in ``q8_oracle``.

TEST INFRASTRUCTURE ONLY (see q8_oracle.py).  PARITY UNPINNED: restated from
q8_kernels/modules/{linear,attention,ffn,activations,rms_norm}.py and
q8_kernels/blocks/ltx_transformer_block.py of the reference; the reference has
no tests for these modules.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import q8_oracle as O


def q8_linear_module(sd: Dict[str, torch.Tensor], prefix: str, x: torch.Tensor, fuse_gelu: bool = False,
                     out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Q8Linear.forward (q8_kernels/modules/linear.py:31-32); with an e4m3 weight the FP8Linear
    counterpart with Hadamard-rotated per-token e4m3 activations (:129-133 with use_hadamard, plus the
    GEMM's optional GELU)."""
    w = sd[prefix + "weight"]
    if w.dtype == O.E4M3:
        xq, xs = O.tokenwise_quant(O.hadamard_transform(x), O.E4M3)
        return O.fp8_mm(xq, w, xs, sd[prefix + "scales"], fuse_gelu, torch.bfloat16 if out_dtype is None else out_dtype,
                        bias=sd.get(prefix + "bias"))
    return O.q8_linear(x, w, sd.get(prefix + "bias"), None, sd[prefix + "scales"], fuse_gelu, out_dtype)


def attention_module(sd, prefix, hidden_states, freqs_cis=None, encoder_hidden_states=None, attention_mask=None,
                     num_heads=32, head_dim=64, non_mm_precision=torch.bfloat16, mm_out_dtype=None,
                     apply_qk_hadamard=True, attn_type="q8_kernels", use_rope=False):
    """Attention.forward (q8_kernels/modules/attention.py:45-106).  RoPE output is
    cast to ``non_mm_precision`` (the kernel semantics of csrc/ops/rope.cpp:125-131;
    the reference's torch fallback leaves fp32, which its q8 attention rejects)."""
    if attention_mask is not None and attention_mask.ndim > 1 and attn_type == "q8_kernels":
        attention_mask = attention_mask.argmin(-1).reshape(-1).int()
    q = q8_linear_module(sd, prefix + "to_q.", hidden_states, out_dtype=mm_out_dtype)
    q = O.rms_norm(q, sd[prefix + "q_norm.weight"], non_mm_precision)[0]
    kv = encoder_hidden_states if encoder_hidden_states is not None else hidden_states
    k = q8_linear_module(sd, prefix + "to_k.", kv, out_dtype=mm_out_dtype)
    k = O.rms_norm(k, sd[prefix + "k_norm.weight"], non_mm_precision)[0]
    v = q8_linear_module(sd, prefix + "to_v.", kv, out_dtype=mm_out_dtype)
    if encoder_hidden_states is None and use_rope:
        q = O.rope(q, freqs_cis[0].expand_as(q), freqs_cis[1].expand_as(q), non_mm_precision)
        k = O.rope(k, freqs_cis[0].expand_as(k), freqs_cis[1].expand_as(k), non_mm_precision)
    B = q.shape[0]
    q = q.view(B, -1, num_heads, head_dim).transpose(1, 2)
    k = k.view(B, -1, num_heads, head_dim).transpose(1, 2)
    v = v.view(B, -1, num_heads, head_dim).transpose(1, 2)
    if attn_type == "q8_kernels":
        h = O.flash_attn_func(q, k, v, batch_mask=attention_mask, apply_qk_hadamard=apply_qk_hadamard)
    else:
        q, k, v = (t.to(non_mm_precision) for t in (q, k, v))
        mask = None
        if attention_mask is not None:
            pos = torch.arange(k.shape[2]).expand(B, -1)
            keep = pos < attention_mask.unsqueeze(-1)
            mask = torch.where(keep, 0.0, float("-inf")).unsqueeze(1).unsqueeze(1).expand(-1, num_heads, -1, -1)
            mask = mask.to(q.dtype)
        h = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    h = h.transpose(1, 2).reshape(B, -1, num_heads * head_dim).contiguous()
    h = q8_linear_module(sd, prefix + "to_out.", h, out_dtype=mm_out_dtype)
    return h.to(non_mm_precision)


def ltx_block(sd, hidden_states, freqs_cis, attention_mask, encoder_hidden_states, encoder_attention_mask, timestep,
              num_heads=32, head_dim=64, mm_out_dtype=torch.bfloat16, non_mm_precision=torch.bfloat16,
              attn_type="q8_kernels"):
    """LTXTransformerBlock.forward (q8_kernels/blocks/ltx_transformer_block.py:21-58)."""
    table = sd["scale_shift_table"]
    ada = table[None, None] + timestep.reshape(hidden_states.shape[0], timestep.shape[1], table.shape[0], -1)
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = ada.unbind(dim=2)
    kw = dict(num_heads=num_heads, head_dim=head_dim, non_mm_precision=non_mm_precision, mm_out_dtype=mm_out_dtype,
              attn_type=attn_type)
    n = O.rms_norm(hidden_states, None, non_mm_precision)[0]
    n = n * (1 + scale_msa) + shift_msa
    a = attention_module(sd, "attn1.", n, freqs_cis, None, attention_mask, use_rope=True, **kw)
    hidden_states = gate_msa * a + hidden_states
    a = attention_module(sd, "attn2.", hidden_states, freqs_cis, encoder_hidden_states, encoder_attention_mask,
                         use_rope=False, **kw)
    hidden_states = a + hidden_states
    n = O.rms_norm(hidden_states, None, non_mm_precision)[0]
    n = n * (1 + scale_mlp) + shift_mlp
    f = q8_linear_module(sd, "ff.act.proj.", n, fuse_gelu=True, out_dtype=mm_out_dtype)
    f = q8_linear_module(sd, "ff.proj_down.", f, out_dtype=mm_out_dtype).to(non_mm_precision)
    return gate_mlp * f + hidden_states
