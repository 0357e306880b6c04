"""GPU parity of the tcgen05 INT8 / FP8 GEMM against the CPU oracle (rel.
Frobenius <= 2e-3 on the bf16 output; the oracle is rounded to bf16 too), plus
size-independent properties at the full DiT shapes."""
import pytest
import torch

import golden_io as G
import helpers as Hp
from oracle import q8_oracle as O

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn
TOL = 2e-3


@pytest.fixture(scope="module")
def nat(cuda_device):
    from q8_kernels_b200 import native
    return native


def _operands(M, N, K, kind, seed):
    a = Hp.activations(M, K, seed)
    w = Hp.weights(N, K, seed + 1)
    qd = torch.int8 if kind == "int8" else E4M3
    aq, sa = O.tokenwise_quant(a, qd)
    wq, sw = O.tokenwise_quant(w, qd)
    return aq, sa, wq, sw, Hp.bias_vec(N, seed + 2)


def _run(nat, dev, kind, aq, sa, wq, sw, bias, gelu, out_dtype):
    mm = {"int8": (nat.q8_mm, nat.q8_mm_bias), "fp8": (nat.fp8_mm, nat.fp8_mm_bias)}[kind]
    args = [t.to(dev) for t in (aq, wq)]
    if bias is not None:
        return mm[1](args[0], args[1], bias.to(dev), sa.to(dev), sw.to(dev), gelu, out_dtype)
    return mm[0](args[0], args[1], sa.to(dev), sw.to(dev), gelu, out_dtype)


def _oracle(kind, aq, sa, wq, sw, bias, gelu, out_dtype):
    f = O.q8_mm if kind == "int8" else O.fp8_mm
    return f(aq, wq, sa, sw, gelu, out_dtype, bias=bias)


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 128, 128), (256, 512, 512), (100, 256, 256),
                                   (1, 128, 64), (300, 384, 192), (129, 640, 1024), (512, 2048, 2048),
                                   (77, 48, 80)])
def test_gemm_small_shapes(nat, cuda_device, kind, M, N, K):
    aq, sa, wq, sw, bias = _operands(M, N, K, kind, seed=M + N + K)
    got = _run(nat, cuda_device, kind, aq, sa, wq, sw, bias, False, torch.bfloat16)
    ref = _oracle(kind, aq, sa, wq, sw, bias, False, torch.bfloat16)
    assert got.shape == (1, M, N) and got.dtype == torch.bfloat16
    err = Hp.rel_fro(got.float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"
    if kind == "int8":
        # integer accumulation is exact, the epilogue differs from the oracle by at most an fma rounding
        flips = (Hp.bits(got.cpu()) != Hp.bits(ref)).float().mean().item()
        assert flips < 0.02, f"{flips:.4f} of bf16 outputs differ"


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("bias,gelu,out_dtype", [(False, False, torch.bfloat16), (True, True, torch.bfloat16),
                                                 (False, True, E4M3), (True, False, None)])
def test_gemm_epilogue_variants(nat, cuda_device, kind, bias, gelu, out_dtype):
    aq, sa, wq, sw, b = _operands(384, 512, 768, kind, seed=50)
    b = b if bias else None
    got = _run(nat, cuda_device, kind, aq, sa, wq, sw, b, gelu, out_dtype)
    ref = _oracle(kind, aq, sa, wq, sw, b, gelu, out_dtype)
    want_dtype = E4M3 if out_dtype in (None, E4M3) else out_dtype
    assert got.dtype == want_dtype                                   # default output dtype is e4m3, as in the reference
    if want_dtype == torch.bfloat16:
        assert Hp.rel_fro(got.float(), ref.float()) <= TOL
    else:
        # e4m3 output: compare as values; a 1-ulp flip is 6 %, so count flips instead of a norm
        g, r = got.float().cpu(), ref.float()
        assert not torch.isnan(g).any()
        flips = (g != r).float().mean().item()
        assert flips < 0.02, f"{flips:.4f} of e4m3 outputs differ"
        assert g.abs().max() <= 448


@pytest.mark.parametrize("kind", ["int8", "fp8"])
def test_gemm_batched_and_broadcast(nat, cuda_device, kind):
    qd = torch.int8 if kind == "int8" else E4M3
    a = Hp.activations(3 * 160, 256, seed=60).reshape(3, 160, 256)
    w = Hp.weights(3 * 128, 256, seed=61).reshape(3, 128, 256)
    aq, sa = O.tokenwise_quant(a, qd)
    wq, sw = O.tokenwise_quant(w, qd)
    f = nat.q8_mm if kind == "int8" else nat.fp8_mm
    d = cuda_device
    for (A, SA, W, SW) in [(aq, sa, wq, sw), (aq, sa, wq[0], sw[0]), (aq[1], sa[1], wq, sw)]:
        got = f(A.contiguous().to(d), W.contiguous().to(d), SA.contiguous().to(d), SW.contiguous().to(d), False,
                torch.bfloat16)
        ref = _oracle(kind, A, SA, W, SW, None, False, torch.bfloat16)
        assert got.shape == ref.shape == (3, 160, 128)
        assert Hp.rel_fro(got.float(), ref.float()) <= TOL


def test_gemm_golden_fixture(nat, cuda_device):
    d = G.load("oracle_gemm.npz")
    dev = cuda_device
    y = nat.q8_mm_bias(G.t(d["aq"]).to(dev), G.t(d["wq"]).to(dev), G.t(d["bias"]).to(dev), G.t(d["sa"]).to(dev),
                       G.t(d["sw"]).to(dev), True, torch.bfloat16)
    assert Hp.rel_fro(y.float(), G.bf16(d["y_i8"]).float()) <= TOL
    y = nat.fp8_mm_bias(G.e4m3(d["af"]).to(dev), G.e4m3(d["wf"]).to(dev), G.t(d["bias"]).to(dev),
                        G.t(d["saf"]).to(dev), G.t(d["swf"]).to(dev), True, torch.bfloat16)
    assert Hp.rel_fro(y.float(), G.bf16(d["y_f8"]).float()) <= TOL


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("K,N", [(2048, 2048), (2048, 6144), (2048, 8192), (8192, 2048)])
def test_gemm_full_dit_shapes_properties(nat, cuda_device, kind, K, N):
    """M = 6144 (one video).  The oracle is checked on a random sample of rows;
    the whole output is checked through linearity in the row scales (doubling
    sa doubles a bias-free output exactly) and a column-sum identity."""
    M = 6144
    aq, sa, wq, sw, bias = _operands(M, N, K, kind, seed=K + N)
    dev = cuda_device
    got = _run(nat, dev, kind, aq, sa, wq, sw, bias, True, torch.bfloat16)
    rows = torch.randperm(M, generator=Hp.gen(1))[:96]
    ref = _oracle(kind, aq[rows], sa[rows], wq, sw, bias, True, torch.bfloat16)
    err = Hp.rel_fro(got[0, rows.to(dev)].float(), ref[0].float())
    assert err <= TOL, f"rel fro {err:.3e}"
    plain = _run(nat, dev, kind, aq, sa, wq, sw, None, False, torch.bfloat16)
    doubled = _run(nat, dev, kind, aq, sa * 2, wq, sw, None, False, torch.bfloat16)
    assert torch.equal(doubled.float(), plain.float() * 2)              # exact: power-of-two scaling commutes with rounding
    # sum over rows of the fp32-exact product equals (sum of scaled A rows) . B^T
    a_deq = (aq.float() * sa[:, None]).to(torch.float64).sum(dim=0)
    col_ref = (wq.to(torch.float64) * sw[:, None].double()) @ a_deq
    col_got = plain[0].double().sum(dim=0).cpu()
    assert Hp.rel_fro(col_got, col_ref) < 5e-3                          # bf16 output rounding accumulates over 6144 rows


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("K,N", [(2048, 8192), (8192, 2048)])
def test_gemm_four_videos_of_tokens_sampled(nat, cuda_device, kind, K, N):
    """M = 24576 (four videos): sampled rows against the oracle, bias + tanh-GELU, bf16 out; plus exact
    power-of-two linearity of the whole bias-free output in the row scales."""
    M = 24576
    aq, sa, wq, sw, bias = _operands(M, N, K, kind, seed=3 * K + N)
    dev = cuda_device
    got = _run(nat, dev, kind, aq, sa, wq, sw, bias, True, torch.bfloat16)
    rows = torch.cat([torch.randperm(M, generator=Hp.gen(2))[:60], torch.tensor([0, 255, 256, M - 257, M - 1])])
    ref = _oracle(kind, aq[rows], sa[rows], wq, sw, bias, True, torch.bfloat16)
    err = Hp.rel_fro(got[0, rows.to(dev)].float(), ref[0].float())
    assert err <= TOL, f"rel fro {err:.3e}"
    plain = _run(nat, dev, kind, aq, sa, wq, sw, None, False, torch.bfloat16)
    halved = _run(nat, dev, kind, aq, sa * 0.5, wq, sw, None, False, torch.bfloat16)
    assert torch.equal(halved.float() * 2, plain.float())


def test_gemm_argument_errors(nat, cuda_device):
    from q8_kernels_b200._lib import Q8KernelError
    d = cuda_device
    a = torch.zeros(8, 64, dtype=torch.int8, device=d)
    w = torch.zeros(16, 64, dtype=torch.int8, device=d)
    sa = torch.ones(8, device=d)
    sw = torch.ones(16, device=d)
    with pytest.raises(Q8KernelError, match="contiguous"):
        nat.q8_mm(a.t().contiguous().t(), w, sa, sw, False, torch.bfloat16)
    with pytest.raises(Q8KernelError, match="K mismatch"):
        nat.q8_mm(a, torch.zeros(16, 32, dtype=torch.int8, device=d), sa, sw, False, torch.bfloat16)
    with pytest.raises(Q8KernelError):
        nat.fp8_mm(a, w, sa, sw, False, torch.bfloat16)                 # wrong operand dtype
    with pytest.raises(Q8KernelError, match="Batch missmatch"):
        nat.q8_mm(torch.zeros(2, 8, 64, dtype=torch.int8, device=d), torch.zeros(3, 16, 64, dtype=torch.int8, device=d),
                  torch.ones(2, 8, device=d), torch.ones(3, 16, device=d), False, torch.bfloat16)
