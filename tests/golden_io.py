"""Loader for the fixtures under tests/golden/ (bf16 stored as int16 bits,
e4m3 as uint8 bits)."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name: str):
    return np.load(os.path.join(GOLDEN, name))


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def e4m3(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float8_e4m3fn)


def t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))


def load_typed(name: str):
    """Fixture written with per-key dtype tags (``dtype__<key>``): key -> torch tensor of that dtype
    (or the plain numpy value for untagged entries)."""
    d = load(name)
    out = {}
    for k in d.files:
        if k.startswith("dtype__"):
            continue
        tag = f"dtype__{k}"
        if tag in d.files:
            dtype = getattr(torch, str(d[tag]).split(".")[-1])
            x = torch.from_numpy(np.ascontiguousarray(d[k]))
            out[k] = x.view(dtype) if x.dtype != dtype else x
        else:
            out[k] = d[k]
    return out
