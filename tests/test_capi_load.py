"""CPU checks of the drop-in boundary: the native library loads, exports every
symbol the header declares, rejects bad arguments before touching the GPU, and
the Python layer mirrors the reference's API surface."""
import inspect
import os
import re

import pytest
import torch

import helpers as Hp

HEADER = os.path.join(Hp.REPO_ROOT, "include", "q8_kernels_b200.h")


def _declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"\b(q8k_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from q8_kernels_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert _lib.lib.q8k_version() >= 100
    assert _lib.lib.q8k_error_string(-3).decode() == "workspace too small"


def test_argument_validation_without_gpu():
    """Validation happens on the host before any launch, so it is testable here."""
    from q8_kernels_b200 import _lib
    lib = _lib.lib
    buf = (torch.zeros(4096, dtype=torch.uint8).data_ptr() + 15) // 16 * 16
    # dim not a multiple of 16
    assert lib.q8k_tokenwise_quant(buf, _lib.DT_BF16, buf, _lib.DT_I8, buf, 4, 24, 24, None) == -1
    assert b"multiple of 16" in lib.q8k_last_error_detail()
    # unsupported output dtype
    assert lib.q8k_tokenwise_quant(buf, _lib.DT_BF16, buf, _lib.DT_BF16, buf, 4, 64, 64, None) == -2
    # null pointer
    assert lib.q8k_rms_norm(None, _lib.DT_BF16, None, buf, _lib.DT_BF16, None, 4, 64, None) == -1
    # Hadamard dim limit
    assert lib.q8k_fast_hadamard_transform(buf, _lib.DT_BF16, buf, _lib.DT_BF16, 1, 32768, 32768, 1.0, None) == -2
    # GEMM batch mismatch and bad N
    assert lib.q8k_q8_mm(buf, buf, None, buf, buf, buf, _lib.DT_BF16, 2, 3, 8, 16, 64, 0, None, None) == -1
    assert lib.q8k_fp8_mm(buf, buf, None, buf, buf, buf, _lib.DT_BF16, 1, 1, 8, 24, 64, 0, None, None) == -1
    # linear: workspace too small / misaligned
    need = lib.q8k_linear_workspace_bytes(128, 256)
    assert need >= 128 * 256 + 128 * 4
    ws = (buf + 255) // 256 * 256
    assert lib.q8k_linear(buf, _lib.DT_BF16, buf, _lib.DT_I8, buf, None, buf, _lib.DT_BF16, 128, 64, 256, 1, 0,
                          ws, 16, None, None) == -3
    assert lib.q8k_linear(buf, _lib.DT_BF16, buf, _lib.DT_I8, buf, None, buf, _lib.DT_BF16, 128, 64, 256, 1, 0,
                          ws + 16, need, None, None) == -1
    # zero rows is a no-op, not an error
    assert lib.q8k_tokenwise_quant(None, _lib.DT_BF16, None, _lib.DT_I8, None, 0, 64, 64, None) == 0


def test_ops_fail_loudly_on_cpu_tensors():
    import q8_kernels_b200 as q8
    x = torch.randn(4, 64).bfloat16()
    with pytest.raises(q8._lib.Q8KernelError, match="no CPU path"):
        q8.functional.quantizer.quantize(x)
    with pytest.raises(q8._lib.Q8KernelError):
        q8.functional.fast_hadamard.hadamard_transform(x)


def test_python_api_surface_matches_reference():
    import q8_kernels_b200 as q8
    F, M = q8.functional, q8.modules
    sig = lambda f: list(inspect.signature(f).parameters)  # noqa: E731
    assert sig(F.linear.q8_linear) == ["a", "b", "bias", "scale_a", "scale_b", "fuse_gelu", "out_dtype"]
    assert sig(F.linear.fp8_linear) == ["a", "b", "bias", "scale_a", "scale_b", "use_hadamard", "out_dtype"]
    assert sig(F.fast_hadamard.hadamard_transform) == ["x", "scale", "out_type"]
    assert sig(F.flash_attention.flash_attn_func)[:6] == ["q", "k", "v", "softmax_scale", "batch_mask",
                                                          "apply_qk_hadamard"]
    assert sig(F.rms_norm.rms_norm_8bit) == ["x", "weights", "out_type"]
    assert sig(F.rope.apply_rope) == ["x", "cos_freqs", "sin_freqs", "out_type"]
    assert sig(F.fma.multiply_add) == ["x", "y", "z", "scale_add"]
    assert sig(F.quantizer.quantize) == ["x"] and sig(F.quantizer.quantize_fp8) == ["x"]
    lin = M.Q8Linear(64, 32, bias=True)
    assert set(lin.state_dict()) == {"weight", "bias", "scales"}
    assert lin.weight.dtype == torch.int8 and lin.scales.dtype == torch.float32 and lin.bias.dtype == torch.float32
    f8 = M.FP8Linear(64, 32, bias=False)
    assert set(f8.state_dict()) == {"weight", "scales"} and f8.weight.dtype == torch.float8_e4m3fn
    blk = q8.blocks.LTXTransformerBlock(64, 2, 32, 64)
    keys = set(blk.state_dict())
    for k in ("scale_shift_table", "attn1.to_q.weight", "attn1.to_q.scales", "attn1.q_norm.weight",
              "attn2.to_k.bias", "attn1.to_out.weight", "ff.act.proj.weight", "ff.proj_down.scales"):
        assert k in keys, k
    assert "norm1.weight" not in keys                                      # norm_affine=False


def test_rope_table_on_cpu_matches_reference_vectors():
    """The product's RoPE table is pure torch: on the CPU it must reproduce, bit for bit, the table
    the reference's own precompute_freqs_cis produced for the golden fixture."""
    import golden_io as G
    import q8_kernels_b200 as q8
    d = G.load("ref_freqs_cis.npz")
    cos, sin = q8.blocks.precompute_freqs_cis(G.t(d["grid"]), 2048)
    Hp.assert_bit_equal(cos, G.t(d["cos"]), "cos")
    Hp.assert_bit_equal(sin, G.t(d["sin"]), "sin")
    assert torch.equal(q8.blocks.latent_grid(2, 3, 4), G.t(d["grid"]))
