"""GPU parity of the HBM-bound kernels (quantizer, Hadamard, fused producer,
RMSNorm, RoPE, FMA, GELU) against the CPU oracle, through the C ABI."""
import math

import pytest
import torch

import golden_io as G
import helpers as Hp
from oracle import q8_oracle as O

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def nat(cuda_device):
    from q8_kernels_b200 import native
    return native


@pytest.mark.parametrize("rows,dim", [(1, 16), (7, 64), (33, 256), (64, 2048), (19, 4096), (16, 8192), (5, 10240)])
@pytest.mark.parametrize("out_dtype", [torch.int8, E4M3])
def test_quantizer_bit_exact(nat, cuda_device, rows, dim, out_dtype):
    x = Hp.activations(rows, dim, seed=rows * 131 + dim)
    q_ref, s_ref = O.tokenwise_quant(x, out_dtype)
    q, s = nat.tokenwise_quant(x.to(cuda_device), out_dtype)
    Hp.assert_bit_equal(q, q_ref, "q")
    Hp.assert_bit_equal(s, s_ref, "scales")


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.float16, E4M3])
def test_quantizer_input_dtypes_shapes_and_zero_rows(nat, cuda_device, in_dtype):
    x = Hp.activations(24, 512, seed=77, dtype=torch.float32)
    x[5] = 0
    x = (x * 0.5).to(in_dtype) if in_dtype != E4M3 else O.c10_e4m3(x.clamp(-400, 400))
    x3 = x.reshape(2, 12, 512)
    q_ref, s_ref = O.tokenwise_quant(x3)
    q, s = nat.tokenwise_quant(x3.to(cuda_device), None)
    assert q.shape == (2, 12, 512) and s.shape == (2, 12) and q.dtype == torch.int8
    Hp.assert_bit_equal(q, q_ref, "q")
    Hp.assert_bit_equal(s, s_ref, "scales")
    assert torch.all(q.cpu().reshape(24, 512)[5] == 0) and s.cpu().reshape(24)[5] == 0


def test_quantizer_golden_fixture_strided_and_empty(nat, cuda_device):
    d = G.load("oracle_quant.npz")
    x = G.bf16(d["x"]).to(cuda_device)
    q, s = nat.tokenwise_quant(x, None)
    Hp.assert_bit_equal(q, G.t(d["q_i8"]), "golden int8")
    Hp.assert_bit_equal(s, G.t(d["s_i8"]), "golden scales")
    q, s = nat.tokenwise_quant(x, E4M3)
    Hp.assert_bit_equal(q, G.e4m3(d["q_fp8"]), "golden fp8")
    # row-strided view (every other row of a wider buffer)
    wide = torch.zeros(16, 512, dtype=torch.bfloat16, device=cuda_device)
    wide[:, :256] = x
    q2, s2 = nat.tokenwise_quant(wide[:, :256], None)
    Hp.assert_bit_equal(q2, G.t(d["q_i8"]), "strided rows")
    qe, se = nat.tokenwise_quant(torch.empty(0, 256, dtype=torch.bfloat16, device=cuda_device), None)
    assert qe.shape == (0, 256) and se.shape == (0,)


@pytest.mark.parametrize("rows,dim", [(3, 8), (50, 64), (9, 128), (40, 256), (6, 512), (12, 1024), (64, 2048),
                                      (5, 4096), (16, 8192), (2, 16384), (7, 40), (4, 1536), (3, 10240)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, E4M3])
def test_hadamard_bit_exact(nat, cuda_device, rows, dim, out_dtype):
    x = Hp.activations(rows, dim, seed=dim + rows, outliers=dim >= 1000)
    scale = 1.0 / math.sqrt(dim) if out_dtype == torch.bfloat16 else 0.0442
    ref = O.hadamard_transform(x, scale=scale, out_dtype=out_dtype)
    got = nat.fast_hadamard_transform(x.to(cuda_device), scale, out_dtype)
    Hp.assert_bit_equal(got, ref, f"hadamard {dim}")


def test_hadamard_fp8_input_golden_and_head_views(nat, cuda_device):
    d = G.load("oracle_hadamard.npz")
    for dim in (64, 2048, 40):
        x = G.bf16(d[f"x_{dim}"]).to(cuda_device)
        Hp.assert_bit_equal(nat.fast_hadamard_transform(x, 1 / math.sqrt(dim), None), G.bf16(d[f"bf16_{dim}"]),
                            f"golden bf16 {dim}")
        Hp.assert_bit_equal(nat.fast_hadamard_transform(x, 0.0442, E4M3), G.e4m3(d[f"fp8_{dim}"]),
                            f"golden fp8 {dim}")
    x8 = O.c10_e4m3(torch.randn(10, 2048, generator=Hp.gen(5)))
    ref = O.hadamard_transform(x8, out_dtype=torch.bfloat16)
    Hp.assert_bit_equal(nat.fast_hadamard_transform(x8.to(cuda_device), 1 / math.sqrt(2048), torch.bfloat16), ref)
    # non-contiguous [B,H,S,D] view of [B,S,H*D], as the attention path passes it
    q, _, _ = Hp.qkv(2, 4, 24, 64, seed=6)
    ref = O.hadamard_transform(q, scale=0.0442, out_dtype=E4M3)
    got = nat.fast_hadamard_transform(q.to(cuda_device), 0.0442, E4M3)
    assert got.shape == q.shape
    Hp.assert_bit_equal(got, ref, "head view")


@pytest.mark.parametrize("rows,dim", [(17, 64), (40, 256), (9, 512), (12, 1024), (128, 2048), (33, 8192)])
@pytest.mark.parametrize("q_dtype", [torch.int8, E4M3])
def test_fused_hadamard_quant_equals_chain(nat, cuda_device, rows, dim, q_dtype):
    x = Hp.activations(rows, dim, seed=3 * dim + rows)
    x[rows // 2] = 0
    q_ref, s_ref = O.tokenwise_quant(O.hadamard_transform(x), q_dtype)
    q, s = nat.hadamard_quant(x.to(cuda_device), 1 / math.sqrt(dim), q_dtype)
    Hp.assert_bit_equal(q, q_ref, "fused q")
    Hp.assert_bit_equal(s, s_ref, "fused scales")
    # and against the two-kernel chain on the device
    h = nat.fast_hadamard_transform(x.to(cuda_device), 1 / math.sqrt(dim), None)
    q2, s2 = nat.tokenwise_quant(h, q_dtype)
    Hp.assert_bit_equal(q, q2.cpu(), "fused vs chain q")
    Hp.assert_bit_equal(s, s2.cpu(), "fused vs chain scales")


def test_fused_hadamard_quant_e4m3_input(nat, cuda_device):
    # the e4m3 attention output feeding to_out: intermediate is rounded to e4m3 (c10 cast)
    x8 = O.c10_e4m3(torch.randn(20, 2048, generator=Hp.gen(8)) * 0.5)
    q_ref, s_ref = O.tokenwise_quant(O.hadamard_transform(x8))
    q, s = nat.hadamard_quant(x8.to(cuda_device), 1 / math.sqrt(2048), torch.int8)
    Hp.assert_bit_equal(q, q_ref)
    Hp.assert_bit_equal(s, s_ref)


@pytest.mark.parametrize("rows,dim", [(5, 64), (64, 2048), (9, 8192)])
@pytest.mark.parametrize("affine", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, E4M3])
def test_rms_norm(nat, cuda_device, rows, dim, affine, out_dtype):
    x = Hp.activations(rows, dim, seed=dim + 1)
    w = (torch.rand(dim, generator=Hp.gen(2)) + 0.5) if affine else None
    ref, r_ref = O.rms_norm(x, w, torch.float32)
    out, r = nat.rms_norm(x.to(cuda_device), None if w is None else w.to(cuda_device), out_dtype)
    assert out.dtype == out_dtype and r.shape == (rows,)
    assert torch.allclose(r.cpu(), r_ref, rtol=3e-6, atol=0)
    # fp32 summation order may move r by an ulp; allow the resulting rare 1-ulp output flips
    assert Hp.rel_fro(out.float(), ref) < (4e-3 if out_dtype == torch.bfloat16 else 4e-2)
    exact = O.cast_out(ref, out_dtype)
    flips = (Hp.bits(out.cpu()) != Hp.bits(exact)).float().mean().item()
    assert flips < 0.01, f"{flips:.4f} of outputs differ from the oracle cast"


def test_rope_bit_exact_and_reference_vectors(nat, cuda_device):
    d = G.load("ref_rope.npz")
    x, cos, sin, ref = G.bf16(d["x"]), G.t(d["cos"]), G.t(d["sin"]), G.t(d["out"])
    got = nat.rope(x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), torch.float32)
    Hp.assert_bit_equal(got, ref, "rope vs the reference's own apply_rope output")
    got16 = nat.rope(x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), torch.bfloat16)
    Hp.assert_bit_equal(got16, ref.to(torch.bfloat16), "bf16 out")
    # batch > 1 with a shared [1,S,dim] table and with a full-shape table
    xb = Hp.activations(3 * 24, 2048, seed=9).reshape(3, 24, 2048)
    refb = O.rope(xb, cos, sin, torch.bfloat16)
    Hp.assert_bit_equal(nat.rope(xb.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), torch.bfloat16), refb)
    full = nat.rope(xb.to(cuda_device), cos.expand(3, -1, -1).contiguous().to(cuda_device),
                    sin.expand(3, -1, -1).contiguous().to(cuda_device), torch.bfloat16)
    Hp.assert_bit_equal(full, refb)
    Hp.assert_bit_equal(nat.rope(xb.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), E4M3),
                        O.rope(xb, cos, sin, E4M3))


@pytest.mark.parametrize("ydt,zdt", [(torch.float32, torch.float32), (torch.float32, E4M3),
                                     (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("S,z_rows", [(12, 12), (13, 1), (8, 1), (13, 13)])
def test_fma_bit_exact(nat, cuda_device, ydt, zdt, S, z_rows):
    """z per token or broadcast like y; S = 13 makes row groups of four straddle the two batch entries and
    leaves a partial last group (the kernel widens y and z once per group when the group shares them)."""
    g = Hp.gen(10)
    x = O.c10_e4m3(torch.randn(2, S, 2048, generator=g))
    y = (torch.randn(2, 1, 2048, generator=g) * 0.3)
    z = torch.randn(2, z_rows, 2048, generator=g)
    y = y.to(ydt)
    z = O.c10_e4m3(z) if zdt == E4M3 else z.to(zdt)
    ref = O.fma_8bit(x, y, z, 1.0)
    got = nat.fma_8bit(x.to(cuda_device), y.to(cuda_device), z.to(cuda_device), 1.0)
    Hp.assert_bit_equal(got, ref, "fma")
    # a scale that pushes part of the results beyond 464: the c10 cast turns those into NaN, sign kept
    y_big = (y.float() * 900.0).to(ydt)
    ref = O.fma_8bit(x, y_big, z, 1.0)
    assert (ref.view(torch.uint8) & 0x7F == 0x7F).any()
    got = nat.fma_8bit(x.to(cuda_device), y_big.to(cuda_device), z.to(cuda_device), 1.0)
    Hp.assert_bit_equal(got, ref, "fma with overflow")


def test_gelu_forward(nat, cuda_device):
    x = Hp.activations(16, 8192, seed=11, outliers=False)
    ref = O.gelu_forward(x, torch.float32)
    got = nat.gelu_forward(x.to(cuda_device), torch.bfloat16)
    assert Hp.rel_fro(got.float(), ref) < 3e-3
    flips = (Hp.bits(got.cpu()) != Hp.bits(ref.to(torch.bfloat16))).float().mean().item()
    assert flips < 0.01


def test_dim_checks_raise(nat, cuda_device):
    from q8_kernels_b200._lib import Q8KernelError
    with pytest.raises(Q8KernelError, match="multiple of 16"):
        nat.tokenwise_quant(torch.zeros(4, 24, dtype=torch.bfloat16, device=cuda_device), None)
    with pytest.raises(Q8KernelError):
        nat.fast_hadamard_transform(torch.zeros(4, 64, dtype=torch.float32, device=cuda_device), 1.0, None)
    with pytest.raises(Q8KernelError, match="float32"):
        nat.rope(torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda_device),
                 torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda_device),
                 torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda_device), None)


# ---------------------------------------------------------------- training-side gradients
@pytest.mark.parametrize("dim", [64, 2048, 8192])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, E4M3])
def test_gelu_backward_vs_oracle(nat, cuda_device, dim, out_dtype):
    x = Hp.activations(40, dim, seed=dim + 1, outliers=False)
    g = Hp.activations(40, dim, seed=dim + 2, outliers=False)
    ref = O.gelu_backward(x, g, out_dtype)
    got = nat.gelu_backward(x.to(cuda_device), g.to(cuda_device), out_dtype).cpu()
    assert got.dtype == out_dtype
    # tanhf and FMA contraction move the fp32 value by an ulp or two: a few outputs may round the other way
    assert (Hp.bits(got) != Hp.bits(ref)).float().mean().item() < 0.01
    assert Hp.rel_fro(got.float(), ref.float()) < 2e-3


@pytest.mark.parametrize("dim", [64, 2048])
@pytest.mark.parametrize("shared", [False, True])
def test_rope_backward_bit_exact(nat, cuda_device, dim, shared):
    g = Hp.activations(2 * 24, dim, seed=dim + 5).view(2, 24, dim)
    ang = torch.rand(1 if shared else 2, 24, dim, generator=Hp.gen(7)) * 6.28
    cos, sin = ang.cos(), ang.sin()
    ref = O.rope_backward(g, cos.expand(2, 24, dim), sin.expand(2, 24, dim), torch.bfloat16)
    got = nat.rope_backward(g.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), torch.bfloat16).cpu()
    Hp.assert_bit_equal(got, ref, "rope_backward")


@pytest.mark.parametrize("dim", [256, 2048, 8192])
@pytest.mark.parametrize("affine", [False, True])
def test_rms_norm_backward_vs_oracle(nat, cuda_device, dim, affine):
    x = Hp.activations(24, dim, seed=dim + 9)
    w = (0.5 + torch.rand(dim, generator=Hp.gen(3))) if affine else None
    g = Hp.activations(24, dim, seed=dim + 10, outliers=False)
    xd = x.to(cuda_device)
    wd = w.to(cuda_device) if affine else None
    y, r = nat.rms_norm(xd, wd, torch.bfloat16)
    ref = O.rms_norm_backward(y.cpu(), r.cpu(), g, w, torch.bfloat16)
    got = nat.rms_norm_backward(y, r, g.to(cuda_device), wd, torch.bfloat16).cpu()
    assert (Hp.bits(got) != Hp.bits(ref)).float().mean().item() < 0.01
    assert Hp.rel_fro(got.float(), ref.float()) < 2e-3


def test_autograd_rules_use_the_backward_kernels(nat, cuda_device):
    import q8_kernels_b200.functional as Q8F
    dim = 2048
    x = Hp.activations(16, dim, seed=77, outliers=False).to(cuda_device).requires_grad_(True)
    w = (0.5 + torch.rand(dim, generator=Hp.gen(4))).to(cuda_device)
    g = Hp.activations(16, dim, seed=78, outliers=False).to(cuda_device)
    y = Q8F.rms_norm.rms_norm_8bit(x, w, torch.bfloat16)
    y.backward(g)
    # against torch autograd of the same function in fp32
    xf = x.detach().float().requires_grad_(True)
    yf = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True)) * w
    yf.backward(g.float())
    assert Hp.rel_fro(x.grad.float(), xf.grad) < 1e-2          # bf16 output and bf16 saved activations
    x2 = Hp.activations(16, dim, seed=79, outliers=False).view(1, 16, dim).to(cuda_device).requires_grad_(True)
    ang = torch.rand(1, 16, dim, generator=Hp.gen(8)) * 6.28
    cos, sin = ang.cos().to(cuda_device), ang.sin().to(cuda_device)
    o = Q8F.rope.apply_rope(x2, cos, sin, torch.bfloat16)
    o.backward(g.view(1, 16, dim))
    x2f = x2.detach().float().requires_grad_(True)
    t = x2f.reshape(1, 16, dim // 2, 2)
    rot = torch.stack((-t[..., 1], t[..., 0]), dim=-1).reshape(1, 16, dim)
    (x2f * cos + rot * sin).backward(g.view(1, 16, dim).float())
    assert Hp.rel_fro(x2.grad.float(), x2f.grad) < 5e-3
