"""Seeded input generators and comparators shared by the tests and the bench.

Inputs are generated on the CPU in fp32 from a ``torch.Generator`` and rounded
to bf16 there, so the CPU oracle and the GPU kernels see identical bits.
"""
from __future__ import annotations

import math
import os
import sys

import torch

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO_ROOT not in sys.path:
    sys.path.insert(0, REPO_ROOT)

E4M3 = torch.float8_e4m3fn


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def activations(rows: int, dim: int, seed: int, outliers: bool = True, dtype=torch.bfloat16) -> torch.Tensor:
    """~N(0,1) with ceil(0.1% of channels) scaled x20 (the DiT outlier-channel pattern)."""
    g = gen(seed)
    x = torch.randn(rows, dim, generator=g, dtype=torch.float32)
    if outliers:
        n_out = max(1, math.ceil(0.001 * dim))
        idx = torch.randperm(dim, generator=g)[:n_out]
        x[:, idx] *= 20.0
    return x.to(dtype)


def weights(n: int, k: int, seed: int, dtype=torch.bfloat16) -> torch.Tensor:
    return (torch.randn(n, k, generator=gen(seed), dtype=torch.float32) * 0.02).to(dtype)


def bias_vec(n: int, seed: int) -> torch.Tensor:
    return torch.randn(n, generator=gen(seed), dtype=torch.float32) * 0.02


def qkv(B: int, H: int, S: int, D: int, seed: int, outliers: bool = True):
    """q, k, v as [B,H,S,D] views of [B,S,H*D] bf16 tensors (outlier channels on q and k, drawn over H*D)."""
    hd = H * D
    out = []
    for i, has_out in enumerate((outliers, outliers, False)):
        x = activations(B * S, hd, seed + i, outliers=has_out).reshape(B, S, H, D).transpose(1, 2)
        out.append(x)
    return out


def bits(t: torch.Tensor) -> torch.Tensor:
    """Raw bit pattern for exact comparisons (NaN-safe)."""
    if t.dtype in (E4M3, torch.int8):
        return t.view(torch.uint8)
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t


def assert_bit_equal(a: torch.Tensor, b: torch.Tensor, what: str = "") -> None:
    a, b = a.cpu(), b.cpu()
    assert a.dtype == b.dtype and a.shape == b.shape, f"{what}: {a.dtype}{tuple(a.shape)} vs {b.dtype}{tuple(b.shape)}"
    ba, bb = bits(a), bits(b)
    if a.dtype == E4M3:
        # every NaN encoding is the same value; the kernels and torch may pick different signs
        fa, fb = a.float(), b.float()
        both_nan = torch.isnan(fa) & torch.isnan(fb)
        mism = (ba != bb) & ~both_nan
    else:
        mism = ba != bb
    n = int(mism.sum())
    assert n == 0, f"{what}: {n} of {a.numel()} elements differ (first at {mism.nonzero()[:3].tolist()})"


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a64, b64 = a.detach().cpu().to(torch.float64), b.detach().cpu().to(torch.float64)
    den = torch.linalg.norm(b64)
    return float(torch.linalg.norm(a64 - b64) / den) if den > 0 else float(torch.linalg.norm(a64))
