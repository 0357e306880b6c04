"""Checkpoint conversion: a diffusers LTX-Video transformer state dict -> the 8-bit state dict the
modules of this package (and of the reference) load.

Follows q8_kernels/utils/convert_weights.py:23-78:

* inside ``transformer_blocks``: ``attn*.to_out.0.`` -> ``attn*.to_out.``, ``ff.net.0.`` ->
  ``ff.act.``, ``ff.net.2.`` -> ``ff.proj_down.``;
* attention norm weights and every bias of a block go to fp32;
* every other ``weight`` of a block is Hadamard-rotated (scale 1/sqrt(in_features)), quantised per
  output row to int8 and stored under the same key, its fp32 row scales under ``...scales``;
* ``scale_shift_table`` and everything outside the blocks pass through unchanged.

The key plan (pure Python) is separate from the arithmetic so that it can be checked without a GPU;
the arithmetic is the fused Hadamard + quantizer kernel, bit-identical to the two-kernel chain.
"""
from __future__ import annotations

import argparse
import math
import os
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

BLOCK_PREFIX = "transformer_blocks"

# what happens to one tensor of the original state dict
KEEP, TO_FP32, QUANTIZE = "keep", "fp32", "int8"


def rename_key(key: str) -> str:
    """New name of an original key (q8_kernels/utils/convert_weights.py:49-50,62-63)."""
    if BLOCK_PREFIX not in key:
        return key
    if "attn" in key:
        return key.replace("to_out.0.", "to_out.")
    if "ff" in key:
        return key.replace(".net.0.", ".act.").replace(".net.2.", ".proj_down.")
    return key


def plan_key(key: str) -> Optional[Tuple[str, str]]:
    """(new key, action) for one original key; None when the reference's converter drops the key
    (a block tensor of an attention or feed-forward layer that is neither weight nor bias)."""
    if BLOCK_PREFIX not in key:
        return key, KEEP
    is_attn, is_ff, is_table = "attn" in key, "ff" in key, "scale_shift_table" in key
    if not (is_attn or is_ff or is_table):
        raise ValueError(f"unexpected transformer block key {key!r}")
    new_key = rename_key(key)
    if is_attn:                                            # attention keys are handled first, as in the reference
        if "norm" in key and "weight" in key:
            return new_key, TO_FP32
        if "bias" in key:
            return new_key, TO_FP32
        if "weight" in key:
            return new_key, QUANTIZE
        return None
    if is_ff:
        if "bias" in key:
            return new_key, TO_FP32
        if "weight" in key:
            return new_key, QUANTIZE
        return None
    return key, KEEP


def plan_state_dict(keys) -> List[Tuple[str, str, str]]:
    """[(original key, new key, action)] for every key that survives the conversion."""
    out = []
    for k in keys:
        p = plan_key(k)
        if p is not None:
            out.append((k, p[0], p[1]))
    return out


def quantize_weight(w: torch.Tensor, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Hadamard (1/sqrt(K)) + per-row int8 quantizer of a [N, K] weight on the GPU."""
    from .. import native
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    w = w.to(dev).to(torch.bfloat16).contiguous()
    return native.hadamard_quant(w, 1 / math.sqrt(w.shape[-1]), torch.int8)


def convert_state_dict(orig_state_dict: Dict[str, torch.Tensor], device=None) -> Dict[str, torch.Tensor]:
    """The converted state dict; quantised weights and their scales live on ``device`` (default: the
    current CUDA device), everything else stays where it was."""
    new_state_dict: Dict[str, torch.Tensor] = {}
    for key, new_key, action in plan_state_dict(orig_state_dict.keys()):
        t = orig_state_dict[key]
        if action == KEEP:
            new_state_dict[new_key] = t
        elif action == TO_FP32:
            new_state_dict[new_key] = t.float()
        else:
            wq, ws = quantize_weight(t, device)
            new_state_dict[new_key] = wq
            new_state_dict[new_key.replace("weight", "scales")] = ws
    return new_state_dict


def load_unet(unet_path: Path) -> Dict[str, torch.Tensor]:
    """q8_kernels/utils/convert_weights.py:11-21: a ``.safetensors`` file, or a directory holding
    ``unet_diffusion_pytorch_model.safetensors``."""
    from safetensors.torch import load_file
    unet_path = Path(unet_path)
    if os.path.isdir(str(unet_path)):
        unet_path = unet_path / "unet_diffusion_pytorch_model.safetensors"
    if not unet_path.name.endswith(".safetensors"):
        raise ValueError(f"{unet_path} is not a .safetensors file")
    if not unet_path.exists():
        raise FileNotFoundError(str(unet_path))
    return load_file(str(unet_path))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Convert a diffusers LTX-Video transformer checkpoint to the 8-bit layout")
    ap.add_argument("--input_path", type=Path, required=True)
    ap.add_argument("--output_path", type=Path, required=True, help="output .safetensors file")
    args = ap.parse_args(argv)
    from safetensors.torch import save_file
    new_state_dict = convert_state_dict(load_unet(args.input_path))
    args.output_path.parent.mkdir(parents=True, exist_ok=True)
    save_file({k: v.detach().cpu().contiguous() for k, v in new_state_dict.items()}, str(args.output_path))
    print(f"state dict with {len(new_state_dict)} tensors saved in {args.output_path}")


if __name__ == "__main__":
    main()
