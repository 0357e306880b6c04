"""The glue layers against the reference's own Python.

``tests/golden/ref_{linear_chain,flash_attn_glue,attention_module,block}.npz`` were made by importing
the reference's unmodified ``q8_kernels/functional``, ``modules`` and ``blocks`` files over a shim of
its native extension modules whose fourteen entry points are served by the CPU oracle
(tests/ref_shim.py, tests/golden/make_golden.py).  So everything that is NOT inside a native call --
which tensor gets rotated, quantised, padded, transposed or cast, in what order, with which defaults
-- is the reference's own code.

CPU tests: the oracle's restatements of those files reproduce the fixtures bit for bit (and, when a
checkout of the reference is at hand, so does a fresh run of the reference over the shim).
GPU tests: the product's mirrors (``q8_kernels_b200.functional|modules|blocks``) reproduce them
within the kernel tolerances; the only difference left is the arithmetic inside the CUDA kernels.
"""
import pytest
import torch

import golden_io as G
import helpers as Hp
import ref_shim
from oracle import q8_oracle as O
from oracle import q8_oracle_block as OB

E4M3 = torch.float8_e4m3fn
BF16 = torch.bfloat16


def _sd(d, prefix):
    return {k[len(prefix):]: v for k, v in d.items() if k.startswith(prefix)}


def _flip_fraction(a, b):
    return (Hp.bits(a.cpu()) != Hp.bits(b.cpu())).float().mean().item()


# --------------------------------------------------------------------------- CPU: oracle == reference glue

def test_oracle_linear_chains_equal_the_reference_functions():
    d = G.load_typed("ref_linear_chain.npz")
    a, w, b, a8 = d["a"], d["w"], d["bias"], d["a8"]
    cases = {
        "q8_bias_gelu_bf16": O.q8_linear(a, d["wq"], b, None, d["sw"], True, BF16),
        "q8_plain_default": O.q8_linear(a, d["wq"], None, None, d["sw"], False, None),
        "q8_from_e4m3_bf16": O.q8_linear(a8, d["wq"], b, None, d["sw"], False, BF16),
        "q8_16bit_weight_bf16": O.q8_linear(a, w, b, None, None, False, BF16),
        "fp8_bias_bf16": O.fp8_linear(a, d["wf"], b, None, d["swf"], False, BF16),
        "fp8_hadamard_bf16": O.fp8_linear(a, d["wfh"], None, None, d["swfh"], True, BF16),
        "fp8_16bit_weight_bf16": O.fp8_linear(a, w, b, None, None, False, BF16),
    }
    assert d["q8_plain_default"].dtype == E4M3            # the reference's default output type
    for name, got in cases.items():
        Hp.assert_bit_equal(got, d[name], name)


def test_oracle_linear_backward_equals_the_reference_autograd():
    """Q8LinearFunc.backward, FP8LinearFunc.backward and the LoRA linear (forward, activation gradient,
    gradients of both low-rank factors) of the reference, run through its own autograd."""
    d = G.load_typed("ref_linear_backward.npz")
    g = d["g"]
    Hp.assert_bit_equal(O.q8_linear_backward(g, d["wq"], d["sw"], BF16), d["q8_grad_a"], "q8 grad")
    Hp.assert_bit_equal(O.fp8_linear_backward(g, d["wf"], d["swf"], BF16), d["fp8_grad_a"], "fp8 grad")
    out, ga, gla, glb = O.q8_linear_lora(d["a"], d["wq"], d["bias"], d["sw"], d["lora_a"], d["lora_b"], True, BF16, g)
    Hp.assert_bit_equal(out, d["lora_out"], "lora out")
    Hp.assert_bit_equal(ga, d["lora_grad_a"], "lora grad a")
    Hp.assert_bit_equal(gla, d["lora_grad_lora_a"], "lora grad lora_a")
    Hp.assert_bit_equal(glb, d["lora_grad_lora_b"], "lora grad lora_b")


def test_oracle_flash_attn_func_equals_the_reference_function():
    d = G.load_typed("ref_flash_attn_glue.npz")
    q, k, v = d["q"], d["k"], d["v"]
    Hp.assert_bit_equal(O.flash_attn_func(q, k, v, None, None, True), d["self_hadamard"], "self_hadamard")
    Hp.assert_bit_equal(O.flash_attn_func(q, k, v, None, None, False), d["self_plain"], "self_plain")
    Hp.assert_bit_equal(O.flash_attn_func(q, k, v, 0.2, None, True), d["self_scale"], "self_scale")
    Hp.assert_bit_equal(O.flash_attn_func(q, d["kx"], d["vx"], None, d["mask"], True), d["cross_masked"], "cross_masked")
    assert d["self_hadamard"].dtype == E4M3 and tuple(d["self_hadamard"].shape) == (2, 2, 77, 64)


def test_oracle_attention_module_equals_the_reference_module():
    d = G.load_typed("ref_attention_module.npz")
    x, text, lens = d["x"], d["text"], d["lens"]
    fc = (d["cos"], d["sin"])
    kw = dict(num_heads=4, head_dim=64, non_mm_precision=BF16, mm_out_dtype=BF16)
    sd_self = {k: v for k, v in _sd(d, "self_sd__").items()}
    sd_cross = {k: v for k, v in _sd(d, "cross_sd__").items()}
    got = OB.attention_module(sd_self, "", x, fc, None, None, attn_type="torch", use_rope=True, **kw)
    Hp.assert_bit_equal(got, d["self_torch"], "self_torch")
    got = OB.attention_module(sd_self, "", x, None, text * 0 + x[:, :24], None, attn_type="q8_kernels", **kw)
    Hp.assert_bit_equal(got, d["self_q8_norope"], "self_q8_norope")
    got = OB.attention_module(sd_cross, "", x, None, text, lens, attn_type="q8_kernels", **kw)
    Hp.assert_bit_equal(got, d["cross_q8_masked"], "cross_q8_masked")
    got = OB.attention_module(sd_cross, "", x, None, text, lens, attn_type="torch", **kw)
    Hp.assert_bit_equal(got, d["cross_torch_masked"], "cross_torch_masked")


def test_reference_rejects_its_own_fp32_rope_output_on_the_fp8_path():
    """Recorded when the fixture was made: the reference's rotary embedding returns fp32 (its torch
    fallback, q8_kernels/functional/rope.py:27-41), which its Hadamard entry point does not accept, so
    self-attention with RoPE cannot take attn_type='q8_kernels' in the reference.  The product's
    apply_rope honours out_type instead."""
    d = G.load_typed("ref_attention_module.npz")
    assert str(d["self_rope_q8_outcome"]).startswith("RuntimeError")


def test_oracle_block_equals_the_reference_block():
    d = G.load_typed("ref_block.npz")
    sd = _sd(d, "sd__")
    got = OB.ltx_block(sd, d["x"], (d["cos"], d["sin"]), None, d["text"], d["lens"], d["timestep"], num_heads=4,
                       head_dim=64, attn_type="torch")
    Hp.assert_bit_equal(got, d["out"], "block")


@pytest.mark.skipif(ref_shim.reference_root() is None, reason="$Q8_REFERENCE does not name a checkout of the reference")
def test_reference_layer_over_the_oracle_shim_reproduces_the_fixtures():
    ref = ref_shim.load_reference(ref_shim.reference_root(), ref_shim.oracle_backend())
    d = G.load_typed("ref_linear_chain.npz")
    got = ref.functional.linear.q8_linear(d["a"], d["wq"], d["bias"], None, d["sw"], True, BF16)
    Hp.assert_bit_equal(got, d["q8_bias_gelu_bf16"], "q8_linear")
    f = G.load_typed("ref_flash_attn_glue.npz")
    got = ref.functional.flash_attention.flash_attn_func(f["q"], f["kx"], f["vx"], None, f["mask"], True)
    Hp.assert_bit_equal(got, f["cross_masked"], "flash_attn_func")


# --------------------------------------------------------------------------- GPU: product == reference glue

@pytest.mark.gpu
def test_product_linear_functions_against_the_reference_glue(cuda_device):
    import q8_kernels_b200.functional as Q8F
    d = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in G.load_typed("ref_linear_chain.npz").items()}
    a, w, b, a8 = d["a"], d["w"], d["bias"], d["a8"]
    L = Q8F.linear
    cases = {
        "q8_bias_gelu_bf16": L.q8_linear(a, d["wq"], b, None, d["sw"], True, BF16),
        "q8_from_e4m3_bf16": L.q8_linear(a8, d["wq"], b, None, d["sw"], False, BF16),
        "q8_16bit_weight_bf16": L.q8_linear(a, w, b, None, None, False, BF16),
        "fp8_bias_bf16": L.fp8_linear(a, d["wf"], b, None, d["swf"], False, BF16),
        "fp8_hadamard_bf16": L.fp8_linear(a, d["wfh"], None, None, d["swfh"], True, BF16),
        "fp8_16bit_weight_bf16": L.fp8_linear(a, w, b, None, None, False, BF16),
    }
    for name, got in cases.items():
        want = d[name]
        assert got.shape == want.shape and got.dtype == want.dtype, name
        err = Hp.rel_fro(got.float(), want.float())
        assert err <= 2e-3, f"{name}: rel fro {err:.3e}"
    got = L.q8_linear(a, d["wq"], None, None, d["sw"], False, None)       # default output: e4m3, saturating cast
    assert got.dtype == E4M3 and got.shape == d["q8_plain_default"].shape
    assert _flip_fraction(got, d["q8_plain_default"]) < 0.02


@pytest.mark.gpu
def test_product_linear_backward_against_the_reference_autograd(cuda_device):
    import q8_kernels_b200 as q8
    L = q8.functional.linear
    d = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in G.load_typed("ref_linear_backward.npz").items()}
    g = d["g"]
    a = d["a"].clone().requires_grad_(True)
    L.q8_linear(a, d["wq"], d["bias"], None, d["sw"], False, BF16).backward(g)
    assert Hp.rel_fro(a.grad.float(), d["q8_grad_a"].float()) <= 4e-3
    a = d["a"].clone().requires_grad_(True)
    L.fp8_linear(a, d["wf"], d["bias"], None, d["swf"], False, BF16).backward(g)
    assert Hp.rel_fro(a.grad.float(), d["fp8_grad_a"].float()) <= 4e-3
    # the LoRA module: frozen INT8 base + trainable low-rank factors
    lin = q8.modules.Q8LinearLora(256, 128, 8, bias=True, device=cuda_device)
    lin.weight.data, lin.scales.data, lin.bias.data = d["wq"], d["sw"], d["bias"]
    lin.lora_a.data, lin.lora_b.data = d["lora_a"].clone(), d["lora_b"].clone()
    a = d["a"].clone().requires_grad_(True)
    y = lin(a, fuse_gelu=True, out_dtype=BF16)
    y.backward(g)
    assert Hp.rel_fro(y.float(), d["lora_out"].float()) <= 4e-3
    assert Hp.rel_fro(a.grad.float(), d["lora_grad_a"].float()) <= 6e-3
    assert Hp.rel_fro(lin.lora_a.grad.float(), d["lora_grad_lora_a"].float()) <= 1e-2
    assert Hp.rel_fro(lin.lora_b.grad.float(), d["lora_grad_lora_b"].float()) <= 1e-2
    # without a gradient request the call takes the inference path and gives the same forward values
    with torch.no_grad():
        y2 = lin(d["a"], fuse_gelu=True, out_dtype=BF16)
    assert torch.equal(y2, y.detach())


@pytest.mark.gpu
def test_product_flash_attn_func_against_the_reference_glue(cuda_device):
    import q8_kernels_b200.functional as Q8F
    d = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in G.load_typed("ref_flash_attn_glue.npz").items()}
    F = Q8F.flash_attention.flash_attn_func
    q, k, v = d["q"], d["k"], d["v"]
    for name, got in {
        "self_hadamard": F(q, k, v, None, None, True),
        "self_plain": F(q, k, v, None, None, False),
        "self_scale": F(q, k, v, 0.2, None, True),
        "cross_masked": F(q, d["kx"], d["vx"], None, d["mask"], True),
    }.items():
        want = d[name]
        assert got.dtype == E4M3 and got.shape == want.shape, name
        # e4m3 outputs: a last-bit difference of the fp32 value before the cast flips a byte now and then
        assert _flip_fraction(got, want) < 0.02, f"{name}: {_flip_fraction(got, want):.3e} of the bytes differ"
        assert Hp.rel_fro(got.float(), want.float()) < 1e-2, name


@pytest.mark.gpu
def test_product_attention_module_against_the_reference_module(cuda_device):
    import q8_kernels_b200 as q8
    dev = cuda_device
    d = G.load_typed("ref_attention_module.npz")
    x, text, lens = d["x"].to(dev), d["text"].to(dev), d["lens"].to(dev)
    fc = (d["cos"][:1].contiguous().to(dev), d["sin"][:1].contiguous().to(dev))     # the table is the same for every batch entry
    fc_full = (d["cos"].to(dev), d["sin"].to(dev))
    self_attn = q8.modules.Attention(256, 4, 64, True, True, qk_rms_norm=True, use_rope=True).to(dev)
    cross_attn = q8.modules.Attention(256, 4, 64, True, True, qk_rms_norm=True, kv_dim=256, use_rope=False).to(dev)
    self_attn.load_state_dict({k: v.to(dev) for k, v in _sd(d, "self_sd__").items()})
    cross_attn.load_state_dict({k: v.to(dev) for k, v in _sd(d, "cross_sd__").items()})
    with torch.no_grad():
        cases = {
            "self_torch": self_attn(x, fc_full, None, None, BF16, BF16, True, "torch"),
            "self_q8_norope": self_attn(x, None, text * 0 + x[:, :24], None, BF16, BF16, True, "q8_kernels"),
            "cross_q8_masked": cross_attn(x, None, text, lens, BF16, BF16, True, "q8_kernels"),
            "cross_torch_masked": cross_attn(x, None, text, lens, BF16, BF16, True, "torch"),
        }
        # the case the reference cannot run (see the quirk test): rotary embedding + FP8 kernel; same glue, so
        # it must stay close to the SDPA result of the reference, the FP8 attention error on top
        rope_q8 = self_attn(x, fc, None, None, BF16, BF16, True, "q8_kernels")
    for name, got in cases.items():
        want = d[name].to(dev)
        err = Hp.rel_fro(got.float(), want.float())
        tol = 1.5e-2
        assert err <= tol, f"{name}: rel fro {err:.3e}"
    assert Hp.rel_fro(rope_q8.float(), d["self_torch"].to(dev).float()) < 0.1


@pytest.mark.gpu
def test_product_block_against_the_reference_block(cuda_device):
    import q8_kernels_b200 as q8
    dev = cuda_device
    d = G.load_typed("ref_block.npz")
    blk = q8.blocks.LTXTransformerBlock(256, 4, 64, 256).to(dev)
    sd = {k: v.to(dev) for k, v in _sd(d, "sd__").items()}
    missing, unexpected = blk.load_state_dict(sd, strict=True)
    assert not missing and not unexpected                     # the reference's state dict loads as it is
    blk.scale_shift_table.data = blk.scale_shift_table.data.to(BF16)   # a freshly built block holds the table in fp32
    args = (d["x"].to(dev), (d["cos"].to(dev), d["sin"].to(dev)), None, d["text"].to(dev), d["lens"].to(dev),
            d["timestep"].to(dev))
    with torch.no_grad():
        fused = blk(*args, attn_type="torch")
        plain = blk(*args, attn_type="torch", fuse=False)
    want = d["out"].to(dev)
    for name, got in (("fused", fused), ("op by op", plain)):
        err = Hp.rel_fro(got.float(), want.float())
        assert err <= 2e-2, f"{name}: rel fro {err:.3e}"
