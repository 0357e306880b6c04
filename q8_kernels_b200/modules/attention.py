"""Attention module (reference: q8_kernels/modules/attention.py:14-106).

Same constructor, parameters and forward signature.  Differences that do not
change results: ``apply_rope`` runs the RoPE kernel and returns
``non_mm_precision`` (the reference's torch fallback returns fp32, which its own
Hadamard kernel then rejects), and ``head_shard=(rank, world)`` lets a caller
run the attention core on a slice of the heads (the q/k norm spans all heads, so
slicing happens after norm and RoPE); the caller gathers the slices.  ``attn_type``
defaults to ``"q8_kernels"`` (the FP8 kernel; the reference's default is ``"torch"``,
which stays selectable as the eager comparison path).
"""
import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import functional as Q8F
from .. import native
from .linear import make_linear
from .rms_norm import RMSNorm


class Attention(nn.Module):
    def __init__(self, query_dim: int, num_heads: int, head_dim: int, bias: bool = False, out_bias: bool = False,
                 out_dim: Optional[int] = None, qk_rms_norm: bool = False, kv_dim: Optional[int] = None,
                 use_rope: bool = False, linear: str = "int8"):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.query_dim = query_dim
        self.bias = bias
        self.out_bias = out_bias
        self.inner_dim = self.num_heads * self.head_dim
        self.qk_rms_norm = qk_rms_norm
        if qk_rms_norm:
            self.q_norm = RMSNorm(self.inner_dim)
            self.k_norm = RMSNorm(self.inner_dim)
        self.use_rope = use_rope
        kv_dim = query_dim if kv_dim is None else kv_dim
        out_dim = query_dim if out_dim is None else out_dim
        # the reference builds these from Q8Linear; linear="fp8" selects FP8Linear (Hadamard + per-token e4m3)
        self.to_q = make_linear(linear, query_dim, self.inner_dim, bias=bias)
        self.to_k = make_linear(linear, kv_dim, self.inner_dim, bias=bias)
        self.to_v = make_linear(linear, kv_dim, self.inner_dim, bias=bias)
        self.to_out = make_linear(linear, self.inner_dim, out_dim, out_bias)

    def _stacked(self, key, layers):
        """Weights, biases and scales of projections that share an input, stacked along the output
        dim; rebuilt whenever one of the layers' tensors is replaced or modified in place."""
        cache = self.__dict__.setdefault("_stacked_cache", {})
        tag = tuple((l.weight.data_ptr(), l.weight._version, l.scales.data_ptr(), l.scales._version,
                     None if l.bias is None else (l.bias.data_ptr(), l.bias._version)) for l in layers)
        hit = cache.get(key)
        if hit is None or hit[0] != tag:
            w = torch.cat([l.weight.data for l in layers], dim=0)
            sc = torch.cat([l.scales for l in layers], dim=0)
            b = None
            if any(l.bias is not None for l in layers):
                b = torch.cat([l.bias.data if l.bias is not None else
                               torch.zeros(l.out_features, dtype=torch.float32, device=w.device) for l in layers], dim=0)
            hit = (tag, w, b, sc)
            cache[key] = hit
        return hit[1], hit[2], hit[3]

    @staticmethod
    def _mm(xq, w, b, xs, ws):
        mm, mmb = (native.q8_mm, native.q8_mm_bias) if w.dtype == torch.int8 else (native.fp8_mm, native.fp8_mm_bias)
        if b is not None:
            return mmb(xq, w, b, xs, ws, False, torch.bfloat16)
        return mm(xq, w, xs, ws, False, torch.bfloat16)

    def _quantize_once(self, x):
        """Hadamard (scale 1/sqrt(K)) + per-token quantizer of an activation to the weights' 8-bit type
        (INT8 as q8_linear applies to a 16-bit / e4m3 input, or e4m3 for FP8 linears)."""
        if x.dtype == torch.int8:
            raise ValueError("Attention expects un-quantised activations")
        if x.dtype == torch.float16:
            x = x.to(torch.bfloat16)
        q, s = native.hadamard_quant(x, 1 / math.sqrt(x.shape[-1]), self.to_q.weight.dtype)
        return q, s

    def forward(self, hidden_states, freqs_cis=None, encoder_hidden_states=None, attention_mask=None,
                non_mm_precision=torch.bfloat16, mm_out_dtype=None, apply_qk_hadamard=True, attn_type="q8_kernels",
                head_shard: Optional[Tuple[int, int]] = None, gather_heads=None,
                hidden_states_q=None, out_gate=None, out_residual=None, peer_buffers=None):
        """Reference signature plus: ``head_shard`` / ``gather_heads`` (attention core on a slice of the
        heads), ``hidden_states_q = (int8, scales)`` when the caller already holds the Hadamard-rotated,
        quantised ``hidden_states`` (the fused norm + modulation producer), and ``out_gate`` /
        ``out_residual`` to fold ``gate * out + residual`` into the output projection's epilogue;
        ``peer_buffers`` (``sharding.PeerBuffers``) instead of ``gather_heads``: the attention kernel stores
        this rank's heads into every rank's buffer and a barrier replaces the all-gather."""
        if attention_mask is not None and attention_mask.ndim > 1 and attn_type == "q8_kernels":
            attention_mask = attention_mask.argmin(-1).squeeze().int()
            if attention_mask.ndim == 0:
                attention_mask = attention_mask.reshape(1)

        # The reference quantises the same activation once per projection (q8_linear re-runs
        # Hadamard + quantizer on every call); here each distinct input is quantised once and the
        # int8 rows + scales are shared, which is bit-identical.
        kv_src = encoder_hidden_states if encoder_hidden_states is not None else hidden_states
        hq, hs = hidden_states_q if hidden_states_q is not None else self._quantize_once(hidden_states)
        if encoder_hidden_states is not None:
            kq, ks = self._quantize_once(kv_src)
        else:
            kq, ks = hq, hs
        batch_size = hq.shape[0]
        heads = self.num_heads
        rope_here = encoder_hidden_states is None and self.use_rope

        # Fast path: projections that share an input run as ONE GEMM over row-stacked weights (same
        # bits: every output column only sees its own weight row), and q/k norm + RoPE + per-head
        # Hadamard + e4m3 cast are one kernel writing the attention kernel's operand layout (same
        # roundings as the op-by-op path below).
        if (attn_type == "q8_kernels" and self.qk_rms_norm and self.head_dim == 64
                and apply_qk_hadamard and mm_out_dtype == torch.bfloat16 and non_mm_precision == torch.bfloat16
                and hq.dim() == 3 and (not rope_here or freqs_cis[0].shape[0] == 1)):
            scale = math.sqrt(1 / 64) * math.sqrt(64 ** -0.5)
            C = self.inner_dim
            if encoder_hidden_states is None:
                w, b, sc = self._stacked("qkv", (self.to_q, self.to_k, self.to_v))
                qkv = self._mm(hq, w, b, hs, sc)
                # V as rows [B,H,S,64]: the tensor core reads it MN-major, so the reference's transpose is never made
                q8_, k8_, vt8 = native.qk_norm_rope_prep_pair(qkv[..., :C], qkv[..., C:2 * C], self.q_norm.weight,
                                                              self.k_norm.weight, freqs_cis if rope_here else None,
                                                              heads, True, scale, xv=qkv[..., 2 * C:])
            else:
                query = self.to_q(hq, hs, out_dtype=mm_out_dtype)
                w, b, sc = self._stacked("kv", (self.to_k, self.to_v))
                kv = self._mm(kq, w, b, ks, sc)
                q8_ = native.qk_norm_rope_prep(query, self.q_norm.weight, None, heads, True, scale)
                k8_, vt8 = native.kv_prep(kv[..., :C], kv[..., C:], self.k_norm.weight, heads, True, scale)
            if head_shard is not None:
                # projections, q/k norm (it spans all heads) and RoPE ran replicated; the attention core
                # takes this rank's heads and the channel slices are gathered before the output projection
                if gather_heads is None and peer_buffers is None:
                    raise ValueError("head_shard needs gather_heads or peer_buffers to reassemble the channel dim")
                rank, world = head_shard
                heads = heads // world
                sl = slice(rank * heads, (rank + 1) * heads)
                q8_, k8_, vt8 = q8_[:, sl].contiguous(), k8_[:, sl].contiguous(), vt8[:, sl].contiguous()
                if peer_buffers is not None:
                    seq = q8_.shape[2]
                    local, addrs = peer_buffers.next(batch_size * seq * self.inner_dim)
                    native.flash_attention_into(q8_, k8_, vt8, 1.0, attention_mask, torch.float8_e4m3fn, addrs,
                                                self.num_heads, rank * heads, v_rows=True)
                    peer_buffers.barrier()
                    hidden_states = local.view(torch.float8_e4m3fn).view(batch_size, seq, self.inner_dim)
                    return self._project_out(hidden_states, non_mm_precision, mm_out_dtype, out_gate, out_residual)
            hidden_states = native.flash_attention(q8_, k8_, vt8, 1.0, attention_mask, None, token_major_out=True,
                                                   v_rows=True)
            hidden_states = hidden_states.transpose(1, 2).reshape(batch_size, -1, heads * self.head_dim)
            if head_shard is not None:
                if gather_heads is None:
                    raise ValueError("head_shard needs a gather_heads callable on this path")
                hidden_states = gather_heads(hidden_states)
            return self._project_out(hidden_states, non_mm_precision, mm_out_dtype, out_gate, out_residual)

        query = self.to_q(hq, hs, out_dtype=mm_out_dtype)
        key = self.to_k(kq, ks, out_dtype=mm_out_dtype)
        value = self.to_v(kq, ks, out_dtype=mm_out_dtype)

        if self.qk_rms_norm:
            query = self.q_norm(query, non_mm_precision)
            key = self.k_norm(key, non_mm_precision)
        if rope_here:
            query = Q8F.rope.apply_rope(query, freqs_cis[0], freqs_cis[1], out_type=non_mm_precision)
            key = Q8F.rope.apply_rope(key, freqs_cis[0], freqs_cis[1], out_type=non_mm_precision)

        query = query.view(batch_size, -1, heads, self.head_dim).transpose(1, 2)
        key = key.view(batch_size, -1, heads, self.head_dim).transpose(1, 2)
        value = value.view(batch_size, -1, heads, self.head_dim).transpose(1, 2)
        if head_shard is not None:
            rank, world = head_shard
            per = heads // world
            sl = slice(rank * per, (rank + 1) * per)
            query, key, value = query[:, sl], key[:, sl], value[:, sl]
            heads = per

        if attn_type == "q8_kernels":
            # stored token-major, so the transpose + reshape + contiguous below is a free view
            hidden_states = Q8F.flash_attention.flash_attn_func(query, key, value, batch_mask=attention_mask,
                                                                apply_qk_hadamard=apply_qk_hadamard,
                                                                token_major_out=True)
        elif attn_type == "torch":
            query = query.to(non_mm_precision)
            key = key.to(non_mm_precision)
            value = value.to(non_mm_precision)
            if attention_mask is not None:
                positions = torch.arange(key.shape[2], device=query.device).expand(batch_size, -1)
                mask = positions < attention_mask.unsqueeze(-1)
                _attention_mask = torch.where(mask, 0.0, float("-inf"))
                attention_mask = _attention_mask.unsqueeze(1).unsqueeze(1).expand(-1, heads, -1, -1).to(query.dtype)
            hidden_states = torch.nn.functional.scaled_dot_product_attention(
                query, key, value, attn_mask=attention_mask, dropout_p=0.0, is_causal=False)
        else:
            raise ValueError(f"Invalid attention type: {attn_type}")
        hidden_states = hidden_states.transpose(1, 2).reshape(batch_size, -1, heads * self.head_dim).contiguous()
        if head_shard is not None:
            if gather_heads is None:
                raise ValueError("head_shard needs a gather_heads callable that reassembles the channel dim")
            hidden_states = gather_heads(hidden_states)

        return self._project_out(hidden_states, non_mm_precision, mm_out_dtype, out_gate, out_residual)

    def _project_out(self, hidden_states, non_mm_precision, mm_out_dtype, out_gate, out_residual):
        if out_residual is not None and mm_out_dtype == torch.bfloat16 and non_mm_precision == torch.bfloat16:
            oq, os_ = self._quantize_once(hidden_states)
            return native.mm_gate_residual(oq, self.to_out.weight.data,
                                           self.to_out.bias.data if self.to_out.bias is not None else None,
                                           os_, self.to_out.scales, out_gate, out_residual)
        hidden_states = self.to_out(hidden_states, out_dtype=mm_out_dtype)
        hidden_states = hidden_states.to(non_mm_precision)
        if out_residual is not None:
            hidden_states = (out_gate * hidden_states if out_gate is not None else hidden_states) + out_residual
        return hidden_states
