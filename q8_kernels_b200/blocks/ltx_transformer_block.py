"""LTX-Video transformer block (reference:
q8_kernels/blocks/ltx_transformer_block.py:9-58): adaLN-single modulated
self-attention with RoPE, cross-attention on the text states and a tanh-GELU
feed-forward, all linears INT8 with Hadamard-rotated per-token activations.

``attn_type`` selects the attention core for both attention layers and defaults
to the FP8 kernel (``"q8_kernels"``); the reference block never forwards it and so
always runs torch SDPA, which remains available as ``attn_type="torch"``.
"""
import math

import torch
import torch.nn as nn

from .. import native

from ..modules.attention import Attention
from ..modules.ffn import FeedForward
from ..modules.rms_norm import RMSNorm


class LTXTransformerBlock(nn.Module):
    def __init__(self, dim, num_heads, head_dim, kv_dim, bias=True, use_rope=True, norm_affine=False, linear="int8"):
        """``linear``: ``"int8"`` (the reference's block: Q8Linear everywhere) or ``"fp8"`` (the same block
        built from FP8Linear with Hadamard-rotated per-token e4m3 activations)."""
        super().__init__()
        self.linear_kind = linear
        self.norm1 = RMSNorm(dim, norm_affine)
        self.attn1 = Attention(dim, num_heads, head_dim, bias, bias, qk_rms_norm=True, kv_dim=None, use_rope=use_rope,
                               linear=linear)
        self.attn2 = Attention(dim, num_heads, head_dim, bias, bias, qk_rms_norm=True, kv_dim=kv_dim, use_rope=False,
                               linear=linear)
        self.norm2 = RMSNorm(dim, norm_affine)
        self.ff = FeedForward(dim, bias=bias, linear=linear)
        self.scale_shift_table = nn.Parameter(torch.randn(6, dim) / dim ** 0.5)

    def forward(self, hidden_states, freqs_cis, attention_mask, encoder_hidden_states, encoder_attention_mask,
                timestep, mm_out_dtype=torch.bfloat16, non_mm_precision=torch.bfloat16, attn_type="q8_kernels",
                head_shard=None, gather_heads=None, fuse=True, peer_buffers=None):
        num_ada_params = self.scale_shift_table.shape[0]
        ada_values = self.scale_shift_table[None, None] + timestep.reshape(
            hidden_states.shape[0], timestep.shape[1], num_ada_params, -1)
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = ada_values.unbind(dim=2)

        # Fused path (same values, fewer passes over the activations): RMS norm + modulation + Hadamard +
        # quantizer in one kernel in front of attn1 and the feed-forward, and gate * out + residual in
        # the epilogue of the three output projections.  Needs bf16 activations and norms without affine
        # weight; anything else takes the op-by-op path of the reference.
        fused = (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and ada_values.dtype == torch.bfloat16
                 and self.norm1.weight is None and self.norm2.weight is None and mm_out_dtype == torch.bfloat16
                 and non_mm_precision == torch.bfloat16 and hidden_states.dim() == 3 and timestep.shape[1] == 1
                 and hidden_states.shape[-1] >= 512)
        if fused and fuse:
            qt = self.ff.proj_down.weight.dtype                  # int8 or e4m3: the activations follow the weights
            nq = native.norm_modulate_quant(hidden_states, scale_msa, shift_msa, qt)
            hidden_states = self.attn1(None, freqs_cis, None, attention_mask, non_mm_precision, mm_out_dtype,
                                       attn_type=attn_type, head_shard=head_shard, gather_heads=gather_heads,
                                       hidden_states_q=nq, out_gate=gate_msa, out_residual=hidden_states,
                                       peer_buffers=peer_buffers)
            hidden_states = self.attn2(hidden_states, freqs_cis=freqs_cis, encoder_hidden_states=encoder_hidden_states,
                                       attention_mask=encoder_attention_mask, non_mm_precision=non_mm_precision,
                                       mm_out_dtype=mm_out_dtype, attn_type=attn_type, out_residual=hidden_states)
            fq, fs = native.norm_modulate_quant(hidden_states, scale_mlp, shift_mlp, qt)
            act = self.ff.act.proj(fq, fs, fuse_gelu=True, out_dtype=mm_out_dtype)
            aq, as_ = native.hadamard_quant(act, 1 / math.sqrt(act.shape[-1]), qt)
            down = self.ff.proj_down
            return native.mm_gate_residual(aq, down.weight.data, down.bias.data if down.bias is not None else None,
                                           as_, down.scales, gate_mlp, hidden_states)

        norm_hidden_states = self.norm1(hidden_states, non_mm_precision)
        norm_hidden_states = norm_hidden_states * (1 + scale_msa) + shift_msa
        attn_output = self.attn1(norm_hidden_states, freqs_cis, None, attention_mask, non_mm_precision, mm_out_dtype,
                                 attn_type=attn_type, head_shard=head_shard, gather_heads=gather_heads)
        hidden_states = gate_msa * attn_output + hidden_states

        attn_output = self.attn2(hidden_states, freqs_cis=freqs_cis, encoder_hidden_states=encoder_hidden_states,
                                 attention_mask=encoder_attention_mask, non_mm_precision=non_mm_precision,
                                 mm_out_dtype=mm_out_dtype, attn_type=attn_type)
        hidden_states = attn_output + hidden_states

        norm_hidden_states = self.norm2(hidden_states, non_mm_precision)
        norm_hidden_states = norm_hidden_states * (1 + scale_mlp) + shift_mlp
        ff_output = self.ff(norm_hidden_states, out_dtype=mm_out_dtype).to(non_mm_precision)
        hidden_states = gate_mlp * ff_output + hidden_states
        return hidden_states
