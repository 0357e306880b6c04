"""ctypes binding of the native library (``libq8k_b200.so``, C ABI declared in
``include/q8_kernels_b200.h``).

There is no CPU or eager fallback: if the library is missing, importing this
module raises, and every op raises on a non-CUDA tensor.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libq8k_b200.so")

DT_F32, DT_F16, DT_BF16, DT_E4M3, DT_I8 = 0, 1, 2, 3, 4
_TORCH_TO_DT = {
    torch.float32: DT_F32,
    torch.float16: DT_F16,
    torch.bfloat16: DT_BF16,
    torch.float8_e4m3fn: DT_E4M3,
    torch.int8: DT_I8,
}

_c_int, _c_i64, _c_f32, _c_ptr, _c_size = (ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p,
                                           ctypes.c_size_t)

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "q8k_version": (_c_int, []),
    "q8k_error_string": (ctypes.c_char_p, [_c_int]),
    "q8k_last_error_detail": (ctypes.c_char_p, []),
    "q8k_wait_selftest": (_c_int, [_c_ptr, ctypes.c_uint, _c_ptr]),
    "q8k_tokenwise_quant": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_i64, _c_ptr]),
    "q8k_fast_hadamard_transform": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_int, _c_i64, _c_int, _c_i64, _c_f32, _c_ptr]),
    "q8k_hadamard_quant": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_i64, _c_f32, _c_ptr]),
    "q8k_norm_modulate_quant": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_i64, _c_f32,
                                         _c_ptr]),
    "q8k_rms_norm": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_ptr]),
    "q8k_rope": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_int, _c_i64, _c_ptr]),
    "q8k_fma_8bit": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_i64, _c_i64,
                              _c_f32, _c_ptr]),
    "q8k_gelu_forward": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_int, _c_i64, _c_int, _c_ptr]),
    "q8k_q8_mm": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_ptr, _c_ptr]),
    "q8k_fp8_mm": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_ptr, _c_ptr]),
    "q8k_mm_gate_residual": (_c_int, [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr,
                                      _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]),
    "q8k_flash_attention": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f32,
                                     _c_ptr, _c_ptr, _c_ptr]),
    "q8k_flash_attention_strided": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                             _c_i64, _c_i64, _c_i64, _c_f32, _c_ptr, _c_ptr, _c_ptr]),
    "q8k_attention_prep": (_c_int, [_c_ptr] * 6 + [_c_int] * 4 + [_c_i64] * 9 + [_c_int, _c_f32, _c_ptr]),
    "q8k_flash_attention_multi_out": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                               _c_int, _c_i64, _c_i64, _c_i64, _c_f32, _c_ptr, _c_ptr, _c_ptr]),
    "q8k_flash_attention_v_rows": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_i64, _c_i64, _c_i64, _c_f32, _c_ptr, _c_ptr, _c_ptr]),
    "q8k_attention_cast_rows": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_ptr]),
    "q8k_ipc_export": (_c_int, [_c_ptr, _c_ptr, _c_ptr]),
    "q8k_ipc_open": (_c_int, [_c_ptr, _c_i64, _c_ptr]),
    "q8k_ipc_close": (_c_int, [_c_ptr, _c_i64]),
    "q8k_gelu_backward": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_i64, _c_int, _c_ptr]),
    "q8k_rope_backward": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_int, _c_i64, _c_ptr]),
    "q8k_rms_norm_backward": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_int, _c_ptr]),
    "q8k_qk_norm_rope_prep": (_c_int, [_c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                       _c_f32, _c_ptr]),
    "q8k_qk_norm_rope_prep_pair": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                            _c_int, _c_int, _c_int, _c_f32, _c_ptr]),
    "q8k_qkv_prep": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                              _c_int, _c_int, _c_int, _c_f32, _c_ptr]),
    "q8k_attention_prep_v": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_ptr]),
    "q8k_linear_workspace_bytes": (_c_size, [_c_int, _c_int]),
    "q8k_linear": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_ptr, _c_size, _c_ptr, _c_ptr]),
    "q8k_linear_static": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                   _c_int, _c_int, _c_int, _c_ptr, _c_ptr]),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python q8_kernels_b200/build.py` "
            "(nvcc, sm_100a).  q8_kernels_b200 has no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class Q8KernelError(RuntimeError):
    """A native entry point rejected its arguments or a CUDA call failed."""


def check(rc: int, op: str) -> None:
    if rc != 0:
        detail = lib.q8k_last_error_detail().decode()
        raise Q8KernelError(f"{op}: {lib.q8k_error_string(rc).decode()} ({rc}): {detail}")


def dt(dtype: torch.dtype) -> int:
    try:
        return _TORCH_TO_DT[dtype]
    except KeyError:
        raise Q8KernelError(f"dtype {dtype} is not supported by q8_kernels_b200") from None


def require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise Q8KernelError("q8_kernels_b200 ops need CUDA tensors; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise Q8KernelError(f"tensors on different devices: {dev} vs {t.device}")
    return dev


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# One int32 status word per device, shared by all tensor-core launches.  The
# kernels only write it when a bounded wait gives up.
_status_words = {}


def status_word(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def read_status(device: Optional[torch.device] = None) -> int:
    """Synchronise and return the device status word (0 = no kernel gave up a wait)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return int(status_word(device).item())


def check_status(device: Optional[torch.device] = None) -> None:
    code = read_status(device)
    if code != 0:
        status_word(device if device is not None else torch.device("cuda", torch.cuda.current_device())).zero_()
        raise Q8KernelError(f"a tensor-core kernel abandoned a wait: status 0x{code:x} (site {code >> 8})")
