"""Stand-ins for the reference's four pybind extension modules
(``q8_kernels_cuda.{gemm,quantizer,ops,flash_attention}._C``) and a loader that imports the
reference's own, unmodified Python layer (``q8_kernels/functional``, ``modules``, ``blocks``) on top
of them.

A *backend* is any object with the fourteen native functions under the reference's names and
positional signatures: ``oracle_backend()`` serves them from the CPU oracle, and
``q8_kernels_b200.native`` is a backend as it stands (that is the drop-in claim).  The loader needs
a checkout of KONAKONA666/q8_kernels; it never runs the reference's ``q8_kernels/__init__.py``
(which pulls in diffusers) but registers empty parent packages and loads the files one by one.

Test infrastructure: used by tests/golden/make_golden.py to produce the ``ref_*`` fixtures of the
glue layers, and by the tests when a checkout is present.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from typing import Optional

import torch

NATIVE_FUNCTIONS = {
    "gemm": ("q8_mm", "q8_mm_bias", "fp8_mm", "fp8_mm_bias"),
    "quantizer": ("tokenwise_quant",),
    "ops": ("fast_hadamard_transform", "rms_norm", "rope", "fma_8bit", "gelu_forward", "gelu_backward",
            "rms_norm_backward", "rope_backward"),
    "flash_attention": ("flash_attention",),
}


def oracle_backend() -> types.SimpleNamespace:
    """The fourteen native entry points served by oracle/q8_oracle.py with the reference's positional
    signatures (csrc/gemm/q8_gemm_api.cpp:296-302, csrc/quantizer/tokenwise_quant.cpp:114,
    csrc/ops/ops_api.cpp:20-29, csrc/flash_attention/flash_attention.cpp:53) and its argument checks:
    the Hadamard entry point takes bf16 or e4m3 rows only
    (csrc/fast_hadamard/fast_hadamard_transform.cpp:74-76)."""
    from oracle import q8_oracle as O
    E4M3 = torch.float8_e4m3fn

    def fast_hadamard_transform(x, scale, out_type=None):
        if x.dtype not in (torch.bfloat16, E4M3):
            raise RuntimeError(f"fast_hadamard_transform: input dtype {x.dtype} must be bfloat16 or float8_e4m3fn")
        return O.hadamard_transform(x, scale, out_type)

    def gemm(fn, with_bias):
        if with_bias:
            return lambda a, b, bias, sa, sb, fuse_gelu, out=None: fn(a, b, sa, sb, fuse_gelu, out or E4M3, bias=bias)
        return lambda a, b, sa, sb, fuse_gelu, out=None: fn(a, b, sa, sb, fuse_gelu, out or E4M3)

    return types.SimpleNamespace(
        tokenwise_quant=lambda x, out_type=None: list(O.tokenwise_quant(x, out_type)),
        fast_hadamard_transform=fast_hadamard_transform,
        rms_norm=lambda x, w=None, out_type=None: list(O.rms_norm(x, w, out_type)),
        rope=lambda x, c, s, out_type=None: O.rope(x, c, s, out_type),
        fma_8bit=lambda x, y, z, scale_add: O.fma_8bit(x, y, z, scale_add),
        gelu_forward=lambda x, out_type=None: O.gelu_forward(x, out_type),
        gelu_backward=lambda x, g, out_type=None: O.gelu_backward(x, g, out_type),
        rms_norm_backward=lambda xn, r, g, w=None, out_type=None: O.rms_norm_backward(xn, r, g, w, out_type),
        rope_backward=lambda g, c, s, out_type=None: O.rope_backward(g, c, s, out_type),
        q8_mm=gemm(O.q8_mm, False), q8_mm_bias=gemm(O.q8_mm, True),
        fp8_mm=gemm(O.fp8_mm, False), fp8_mm_bias=gemm(O.fp8_mm, True),
        flash_attention=lambda q, k, v, scale, mask=None: O.flash_attention(q, k, v, scale, mask, E4M3),
    )


def install(backend) -> None:
    """Register ``q8_kernels_cuda`` and its ``<module>._C`` leaves in ``sys.modules``, bound to ``backend``."""
    root = types.ModuleType("q8_kernels_cuda")
    root.__path__ = []
    sys.modules["q8_kernels_cuda"] = root
    for sub, names in NATIVE_FUNCTIONS.items():
        pkg = types.ModuleType(f"q8_kernels_cuda.{sub}")
        pkg.__path__ = []
        leaf = types.ModuleType(f"q8_kernels_cuda.{sub}._C")
        for n in names:
            setattr(leaf, n, getattr(backend, n))
        pkg._C = leaf
        setattr(root, sub, pkg)
        sys.modules[pkg.__name__] = pkg
        sys.modules[leaf.__name__] = leaf


_REF_FILES = [                                    # import order: leaves first
    "functional/quantizer.py", "functional/fast_hadamard.py", "functional/rms_norm.py", "functional/rope.py",
    "functional/fma.py", "functional/flash_attention.py", "functional/linear.py",
    "modules/rms_norm.py", "modules/linear.py", "modules/activations.py", "modules/ffn.py", "modules/attention.py",
    "blocks/ltx_transformer_block.py",
]


def load_reference(ref_root: str, backend) -> types.ModuleType:
    """Import the reference's Python layer from ``ref_root`` (the directory that holds ``q8_kernels/``)
    over ``backend`` and return the ``q8_kernels`` package object, with ``functional``, ``modules`` and
    ``blocks`` populated from the reference's own files."""
    install(backend)
    for name in [m for m in sys.modules if m == "q8_kernels" or m.startswith("q8_kernels.")]:
        del sys.modules[name]
    base = os.path.join(ref_root, "q8_kernels")
    pkg = types.ModuleType("q8_kernels")
    pkg.__path__ = [base]
    sys.modules["q8_kernels"] = pkg
    for sub in ("functional", "modules", "blocks"):
        m = types.ModuleType(f"q8_kernels.{sub}")
        m.__path__ = [os.path.join(base, sub)]
        sys.modules[m.__name__] = m
        setattr(pkg, sub, m)
    for rel in _REF_FILES:
        mod_name = "q8_kernels." + rel[:-3].replace("/", ".")
        spec = importlib.util.spec_from_file_location(mod_name, os.path.join(base, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[mod_name] = mod
        spec.loader.exec_module(mod)
        parent, leaf = mod_name.rsplit(".", 1)
        setattr(sys.modules[parent], leaf, mod)
    return pkg


def reference_root() -> Optional[str]:
    """Checkout named by $Q8_REFERENCE, if it looks like one."""
    ref = os.environ.get("Q8_REFERENCE", "")
    return ref if ref and os.path.isdir(os.path.join(ref, "q8_kernels", "functional")) else None
