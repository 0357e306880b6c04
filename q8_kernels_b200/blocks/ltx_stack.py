"""The 28-block LTX-Video DiT stack and its 3-D RoPE table (reference:
q8_kernels/models/LTXVideo.py:86-148 for the table, :182-190 for the block loop,
:204-219 for the hyper-parameters).  The diffusers glue around the stack
(patchify, adaLN-single embedder, output head) is not part of this package; the
text states are projected by a plain bf16 linear as a stand-in for the caption
projection.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .ltx_transformer_block import LTXTransformerBlock


@dataclass
class LTXStackConfig:
    """Hyper-parameters of get_ltx_transformer() (q8_kernels/models/LTXVideo.py:204-219)."""
    num_layers: int = 28
    num_attention_heads: int = 32
    attention_head_dim: int = 64
    cross_attention_dim: int = 2048
    caption_channels: int = 4096
    bias: bool = True
    norm_elementwise_affine: bool = False
    positional_embedding_theta: float = 10000.0
    positional_embedding_max_pos: Tuple[int, int, int] = (20, 2048, 2048)
    linear: str = "int8"                  # "int8": Q8Linear blocks (the reference); "fp8": FP8Linear blocks

    @property
    def inner_dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim


def latent_grid(frames: int, height: int, width: int, device=None) -> torch.Tensor:
    """Integer (t, h, w) coordinates of a latent grid as [1, 3, frames*height*width]."""
    t, h, w = torch.meshgrid(torch.arange(frames, device=device), torch.arange(height, device=device),
                             torch.arange(width, device=device), indexing="ij")
    return torch.stack([t.flatten(), h.flatten(), w.flatten()], dim=0).unsqueeze(0).float()


def precompute_freqs_cis(indices_grid: torch.Tensor, dim: int, theta: float = 10000.0,
                         max_pos: Sequence[int] = (20, 2048, 2048)) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin tables [B, S, dim] in fp32 for the interleaved-pair RoPE ("exp"
    spacing of q8_kernels/models/LTXVideo.py:95-148): fractional positions per
    axis, dim//6 frequencies theta**linspace(0,1) * pi/2 applied to 2*pos-1, the
    three axes interleaved per frequency, every value repeated for its pair and
    the first dim % 6 channels padded with cos = 1, sin = 0."""
    frac = torch.stack([indices_grid[:, i] / max_pos[i] for i in range(3)], dim=-1)          # [B,S,3]
    idx = theta ** torch.linspace(math.log(1, theta), math.log(theta, theta), dim // 6, device=frac.device,
                                  dtype=torch.float32)
    idx = idx * math.pi / 2
    freqs = (idx * (frac.unsqueeze(-1) * 2 - 1)).transpose(-1, -2).flatten(2)
    cos = freqs.cos().repeat_interleave(2, dim=-1)
    sin = freqs.sin().repeat_interleave(2, dim=-1)
    if dim % 6 != 0:
        cos = torch.cat([torch.ones_like(cos[:, :, : dim % 6]), cos], dim=-1)
        sin = torch.cat([torch.zeros_like(sin[:, :, : dim % 6]), sin], dim=-1)
    return cos.float(), sin.float()


class LTXStack(nn.Module):
    """caption projection + ``num_layers`` LTXTransformerBlock."""

    def __init__(self, config: Optional[LTXStackConfig] = None):
        super().__init__()
        self.config = config or LTXStackConfig()
        c = self.config
        self.caption_projection = nn.Linear(c.caption_channels, c.inner_dim, bias=True)
        self.transformer_blocks = nn.ModuleList([
            LTXTransformerBlock(c.inner_dim, c.num_attention_heads, c.attention_head_dim, c.cross_attention_dim,
                                c.bias, True, c.norm_elementwise_affine, linear=c.linear)
            for _ in range(c.num_layers)])

    def freqs_cis(self, indices_grid: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        c = self.config
        return precompute_freqs_cis(indices_grid, c.inner_dim, c.positional_embedding_theta,
                                    c.positional_embedding_max_pos)

    def forward(self, hidden_states, indices_grid, encoder_hidden_states, encoder_attention_mask, timestep,
                attn_type="q8_kernels", head_shard=None, gather_heads=None, peer_buffers=None):
        """hidden_states [B,S,inner] bf16; indices_grid [1 or B,3,S]; encoder_hidden_states
        [B,T,caption_channels] bf16; encoder_attention_mask int32 [B] (valid text tokens) or None;
        timestep [B,1,6*inner] modulation values fed to every block."""
        freqs = self.freqs_cis(indices_grid)
        text = self.caption_projection(encoder_hidden_states)
        for block in self.transformer_blocks:
            hidden_states = block(hidden_states, freqs, None, text, encoder_attention_mask, timestep,
                                  attn_type=attn_type, head_shard=head_shard, gather_heads=gather_heads,
                                  peer_buffers=peer_buffers)
        return hidden_states


def random_init_(stack: nn.Module, seed: int = 0, device=None) -> nn.Module:
    """Fill every Q8Linear / FP8Linear of a stack (or block) with Hadamard-rotated 8-bit weights of
    N(0, 0.02) bf16 matrices quantised on the device, biases N(0, 0.02), norm weights ~1."""
    from ..modules.linear import FP8Linear, Q8Linear
    from .. import native
    g = torch.Generator(device="cpu").manual_seed(seed)
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    stack.to(dev)
    for mod in stack.modules():
        if isinstance(mod, (Q8Linear, FP8Linear)):
            w = (torch.randn(mod.out_features, mod.in_features, generator=g) * 0.02).to(torch.bfloat16).to(dev)
            wq, ws = native.hadamard_quant(w, 1 / math.sqrt(mod.in_features), mod.weight.dtype)
            mod.weight.data = wq
            mod.scales.data = ws
            if mod.bias is not None:
                mod.bias.data = (torch.randn(mod.out_features, generator=g) * 0.02).to(dev)
        elif isinstance(mod, nn.Linear):
            mod.weight.data = (torch.randn(mod.weight.shape, generator=g) * 0.02).to(torch.bfloat16).to(dev)
            mod.bias.data = (torch.randn(mod.bias.shape, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        elif hasattr(mod, "scale_shift_table"):
            mod.scale_shift_table.data = (torch.randn(mod.scale_shift_table.shape, generator=g)
                                          / mod.scale_shift_table.shape[1] ** 0.5).to(torch.bfloat16).to(dev)
    return stack
