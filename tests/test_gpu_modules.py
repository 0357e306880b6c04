"""GPU parity of the functional / module layer (q8_linear, fp8_linear, Q8Linear,
Attention, LTXTransformerBlock) against the CPU oracle."""
import pytest
import torch
import torch.nn as nn

import helpers as Hp
from oracle import q8_oracle as O
from oracle import q8_oracle_block as OB

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn
TOL = 2e-3


@pytest.fixture(scope="module")
def q8(cuda_device):
    import q8_kernels_b200
    return q8_kernels_b200


@pytest.mark.parametrize("M,K,N", [(96, 256, 128), (300, 2048, 512), (1024, 2048, 8192)])
@pytest.mark.parametrize("gelu", [False, True])
def test_q8_linear_chain(q8, cuda_device, M, K, N, gelu):
    a = Hp.activations(M, K, seed=M + K)
    w = Hp.weights(N, K, seed=N)
    b = Hp.bias_vec(N, seed=5)
    wq, sw = O.tokenwise_quant(O.hadamard_transform(w))
    ref = O.q8_linear(a, wq, b, None, sw, gelu, torch.bfloat16)
    got = q8.functional.linear.q8_linear(a.to(cuda_device), wq.to(cuda_device), b.to(cuda_device), None,
                                         sw.to(cuda_device), gelu, torch.bfloat16)
    assert got.shape == (1, M, N)
    assert Hp.rel_fro(got.float(), ref.float()) <= TOL
    # pre-quantised activations take the plain GEMM path and must agree with the fused call
    aq, sa = O.tokenwise_quant(O.hadamard_transform(a))
    got2 = q8.functional.linear.q8_linear(aq.to(cuda_device), wq.to(cuda_device), b.to(cuda_device),
                                          sa.to(cuda_device), sw.to(cuda_device), gelu, torch.bfloat16)
    assert torch.equal(got, got2)


def test_fp8_linear_config1(q8, cuda_device):
    """The CPU-runnable linear case: X [1024,2048] ~N(0,1), W [8192,2048] ~N(0,0.02), per-token / per-channel e4m3."""
    a = Hp.activations(1024, 2048, seed=1, outliers=False)
    w = Hp.weights(8192, 2048, seed=2)
    b = Hp.bias_vec(8192, seed=3)
    ref = O.fp8_linear(a, w, b, None, None, False, torch.bfloat16)
    got = q8.functional.linear.fp8_linear(a.to(cuda_device), w.to(cuda_device), b.to(cuda_device), None, None, False,
                                          torch.bfloat16)
    assert Hp.rel_fro(got.float(), ref.float()) <= TOL


def test_q8linear_module_from_linear_and_state_dict(q8, cuda_device):
    lin = nn.Linear(512, 256, bias=True)
    with torch.no_grad():
        lin.weight.copy_(Hp.weights(256, 512, seed=7).float())
        lin.bias.copy_(Hp.bias_vec(256, seed=8))
    lin = lin.to(cuda_device).to(torch.bfloat16)
    mod = q8.modules.Q8Linear.from_linear(lin)
    wq, sw = O.tokenwise_quant(O.hadamard_transform(lin.weight.data.cpu()))
    Hp.assert_bit_equal(mod.weight.data, wq, "weight")
    Hp.assert_bit_equal(mod.scales.data, sw, "scales")
    x = Hp.activations(64, 512, seed=9).reshape(2, 32, 512)
    y = mod(x.to(cuda_device), out_dtype=torch.bfloat16)
    ref = O.q8_linear(x, wq, lin.bias.data.float().cpu(), None, sw, False, torch.bfloat16)
    assert y.shape == (2, 32, 256)
    assert Hp.rel_fro(y.float(), ref.float()) <= TOL
    mod2 = q8.modules.Q8Linear(512, 256).to(cuda_device)
    mod2.load_state_dict(mod.state_dict())
    assert torch.equal(mod2(x.to(cuda_device), out_dtype=torch.bfloat16), y)
    f8 = q8.modules.FP8Linear.from_linear(lin)
    assert f8.weight.dtype == E4M3
    y8 = f8(x.to(cuda_device))
    assert y8.dtype == torch.bfloat16 and Hp.rel_fro(y8.float(), (x.float() @ lin.weight.float().cpu().T
                                                                   + lin.bias.float().cpu())) < 0.08


def _random_block(q8, dim, heads, head_dim, kv_dim, device, seed):
    torch.manual_seed(seed)
    blk = q8.blocks.LTXTransformerBlock(dim, heads, head_dim, kv_dim)
    g = Hp.gen(seed)
    sd = {}
    for name, t in blk.state_dict().items():
        if name.endswith("weight") and t.dtype == torch.int8:
            in_f = t.shape[1]
            w = (torch.randn(t.shape, generator=g) * 0.02).to(torch.bfloat16)
            wq, sw = O.tokenwise_quant(O.hadamard_transform(w))
            sd[name] = wq
            sd[name[:-6] + "scales"] = sw
        elif name.endswith("scales"):
            continue
        elif name.endswith("bias"):
            sd[name] = torch.randn(t.shape, generator=g) * 0.02
        elif name.endswith("norm.weight"):
            sd[name] = torch.rand(t.shape, generator=g) + 0.5
        elif name == "scale_shift_table":
            sd[name] = torch.randn(t.shape, generator=g) / dim ** 0.5
        else:
            raise AssertionError(name)
    blk.load_state_dict(sd)
    return blk.to(device), sd


@pytest.mark.parametrize("attn_type", ["q8_kernels", "torch"])
def test_ltx_block_against_oracle(q8, cuda_device, attn_type):
    dim, heads, hd, S, T = 256, 4, 64, 192, 48
    blk, sd = _random_block(q8, dim, heads, hd, dim, cuda_device, seed=21)
    g = Hp.gen(22)
    x = torch.randn(2, S, dim, generator=g).to(torch.bfloat16)
    text = torch.randn(2, T, dim, generator=g).to(torch.bfloat16)
    timestep = (torch.randn(2, 1, 6 * dim, generator=g) * 0.1).to(torch.bfloat16)
    grid = torch.stack(torch.meshgrid(torch.arange(4), torch.arange(6), torch.arange(8), indexing="ij"), 0)
    cos, sin = O.precompute_freqs_cis(grid.reshape(1, 3, -1).float(), dim=dim)
    text_len = torch.tensor([17, 48], dtype=torch.int32)
    sd_t = {k: (v.to(torch.bfloat16) if k == "scale_shift_table" else v) for k, v in sd.items()}
    blk.scale_shift_table.data = blk.scale_shift_table.data.to(torch.bfloat16)
    ref = OB.ltx_block(sd_t, x, (cos, sin), None, text, text_len, timestep, num_heads=heads, head_dim=hd,
                       attn_type=attn_type)
    d = cuda_device
    got = blk(x.to(d), (cos.to(d), sin.to(d)), None, text.to(d), text_len.to(d), timestep.to(d), attn_type=attn_type)
    assert got.shape == ref.shape and got.dtype == torch.bfloat16
    # errors compound through 10 linears, two attentions and bf16 elementwise ops: bf16-level agreement
    err = Hp.rel_fro(got.float(), ref.float())
    assert err < 1.5e-2, f"rel fro {err:.3e}"


def test_freqs_cis_matches_reference_table(q8, cuda_device):
    """Product RoPE table vs the vectors produced by the reference's own precompute_freqs_cis."""
    import golden_io as G
    d = G.load("ref_freqs_cis.npz")
    grid = G.t(d["grid"]).to(cuda_device)
    cos, sin = q8.blocks.precompute_freqs_cis(grid, 2048)
    # the highest frequencies reach phases of ~1.5e4 rad, where one fp32 ulp of the frequency
    # (GPU vs CPU pow) moves the phase by ~1e-3 rad; the CPU path is checked bit for bit elsewhere
    assert torch.allclose(cos.cpu(), G.t(d["cos"]), atol=5e-3, rtol=0)
    assert torch.allclose(sin.cpu(), G.t(d["sin"]), atol=5e-3, rtol=0)
    g2 = q8.blocks.latent_grid(2, 3, 4, device=cuda_device)
    assert torch.equal(g2.cpu(), G.t(d["grid"]))


def test_ltx_stack_small_against_oracle(q8, cuda_device):
    cfg = q8.blocks.LTXStackConfig(num_layers=2, num_attention_heads=4, attention_head_dim=64,
                                   cross_attention_dim=256, caption_channels=128)
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=5, device=cuda_device)
    g = Hp.gen(31)
    S, T = 4 * 4 * 6, 40
    x = torch.randn(1, S, 256, generator=g).to(torch.bfloat16)
    text = torch.randn(1, T, 128, generator=g).to(torch.bfloat16)
    timestep = (torch.randn(1, 1, 6 * 256, generator=g) * 0.1).to(torch.bfloat16)
    grid = q8.blocks.latent_grid(4, 4, 6)
    lens = torch.tensor([29], dtype=torch.int32)
    d = cuda_device
    got = stack(x.to(d), grid.to(d), text.to(d), lens.to(d), timestep.to(d), attn_type="q8_kernels")
    # oracle: same weights, CPU
    sd = {k: v.detach().cpu() for k, v in stack.state_dict().items()}
    cos, sin = O.precompute_freqs_cis(grid, dim=256)
    proj = torch.nn.functional.linear(text.float(), sd["caption_projection.weight"].float(),
                                      sd["caption_projection.bias"].float()).to(torch.bfloat16)
    h = x
    for i in range(2):
        pre = f"transformer_blocks.{i}."
        bsd = {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}
        h = OB.ltx_block(bsd, h, (cos, sin), None, proj, lens, timestep, num_heads=4, head_dim=64)
    err = Hp.rel_fro(got.float(), h.float())
    assert got.shape == (1, S, 256) and err < 2e-2, f"rel fro {err:.3e}"


def test_norm_modulate_quant_matches_unfused_chain(q8, cuda_device):
    """Fused RMSNorm + modulation + Hadamard + quantizer vs the oracle's op-by-op chain.  Only the
    fp32 summation order of the mean square differs, so all but a few int8 codes are identical."""
    import math
    g = Hp.gen(41)
    B, S, C = 2, 96, 2048
    x = Hp.activations(B * S, C, seed=42).reshape(B, S, C)
    sc = (torch.randn(B, 1, C, generator=g) * 0.1).to(torch.bfloat16)
    sh = (torch.randn(B, 1, C, generator=g) * 0.1).to(torch.bfloat16)
    n = O.rms_norm(x, None, torch.bfloat16)[0]
    u = n * (1 + sc) + sh                                      # torch bf16 ops, as the reference block does
    q_ref, s_ref = O.tokenwise_quant(O.hadamard_transform(u))
    d = cuda_device
    q, s = q8.native.norm_modulate_quant(x.to(d), sc.to(d), sh.to(d))
    assert q.shape == (B, S, C) and s.shape == (B, S)
    diff = (q.cpu().int() - q_ref.int()).abs()
    assert diff.max().item() <= 1 and (diff != 0).float().mean().item() < 0.01
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-2)
    # against the same chain on the device the agreement is the same
    nd = q8.native.rms_norm(x.to(d), None, torch.bfloat16)[0]
    ud = nd * (1 + sc.to(d)) + sh.to(d)
    qd, sd = q8.native.hadamard_quant(ud, 1 / math.sqrt(C), torch.int8)
    assert ((q.int() - qd.int()).abs() != 0).float().mean().item() < 0.01


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("with_gate", [True, False])
@pytest.mark.parametrize("M,N,K", [(200, 512, 256), (384, 2048, 2048), (96, 128, 128), (300, 272, 192), (515, 1040, 320)])
def test_mm_gate_residual_is_bit_identical_to_separate_ops(q8, cuda_device, kind, with_gate, M, N, K):
    qd = torch.int8 if kind == "int8" else E4M3
    d = cuda_device
    B = 2
    a = Hp.activations(B * M, K, seed=M + N)
    w = Hp.weights(N, K, seed=K)
    aq, sa = O.tokenwise_quant(a, qd)
    wq, sw = O.tokenwise_quant(w, qd)
    aq, sa = aq.reshape(B, M, K).to(d), sa.reshape(B, M).to(d)
    wq, sw = wq.to(d), sw.to(d)
    bias = Hp.bias_vec(N, seed=1).to(d)
    g = Hp.gen(2)
    gate = torch.randn(B, 1, N, generator=g).to(torch.bfloat16).to(d) if with_gate else None
    resid = torch.randn(B, M, N, generator=g).to(torch.bfloat16).to(d)
    mm = q8.native.q8_mm_bias if kind == "int8" else q8.native.fp8_mm_bias
    y = mm(aq, wq, bias, sa, sw, False, torch.bfloat16)
    want = (gate * y if with_gate else y) + resid
    got = q8.native.mm_gate_residual(aq, wq, bias, sa, sw, gate, resid)
    assert got.shape == (B, M, N)
    assert torch.equal(got, want)


def test_block_fused_path_equals_op_by_op_path(q8, cuda_device):
    blk, _ = _random_block(q8, 512, 8, 64, 512, cuda_device, seed=51)
    blk.scale_shift_table.data = blk.scale_shift_table.data.to(torch.bfloat16)
    g = Hp.gen(52)
    S, T = 4 * 6 * 8, 40
    d = cuda_device
    x = torch.randn(2, S, 512, generator=g).to(torch.bfloat16).to(d)
    text = torch.randn(2, T, 512, generator=g).to(torch.bfloat16).to(d)
    ts = (torch.randn(2, 1, 6 * 512, generator=g) * 0.1).to(torch.bfloat16).to(d)
    grid = torch.stack(torch.meshgrid(torch.arange(4), torch.arange(6), torch.arange(8), indexing="ij"), 0)
    cos, sin = O.precompute_freqs_cis(grid.reshape(1, 3, -1).float(), dim=512)
    lens = torch.tensor([11, 40], dtype=torch.int32, device=d)
    a = blk(x, (cos.to(d), sin.to(d)), None, text, lens, ts, attn_type="q8_kernels", fuse=True)
    b = blk(x, (cos.to(d), sin.to(d)), None, text, lens, ts, attn_type="q8_kernels", fuse=False)
    err = Hp.rel_fro(a.float(), b.float())
    assert err < 4e-3, f"rel fro {err:.3e}"                   # only 1/rms summation order differs, amplified by int8 codes


def test_block_is_cuda_graph_capturable(q8, cuda_device):
    """No op of the block synchronises or allocates outside torch's allocator, so a whole block
    forward can be captured once and replayed (the reference does this per module with its graph.py)."""
    blk, _ = _random_block(q8, 512, 8, 64, 512, cuda_device, seed=61)
    blk.scale_shift_table.data = blk.scale_shift_table.data.to(torch.bfloat16)
    g = Hp.gen(62)
    d = cuda_device
    S, T = 4 * 4 * 8, 24
    x = torch.randn(1, S, 512, generator=g).to(torch.bfloat16).to(d)
    text = torch.randn(1, T, 512, generator=g).to(torch.bfloat16).to(d)
    ts = (torch.randn(1, 1, 6 * 512, generator=g) * 0.1).to(torch.bfloat16).to(d)
    grid = torch.stack(torch.meshgrid(torch.arange(4), torch.arange(4), torch.arange(8), indexing="ij"), 0)
    cos, sin = O.precompute_freqs_cis(grid.reshape(1, 3, -1).float(), dim=512)
    freqs = (cos.to(d), sin.to(d))
    lens = torch.tensor([17], dtype=torch.int32, device=d)
    with torch.no_grad():
        side = torch.cuda.Stream(device=d)
        side.wait_stream(torch.cuda.current_stream(d))
        with torch.cuda.stream(side):
            for _ in range(2):                                  # warm-up: first-call set-up happens outside the capture
                eager = blk(x, freqs, None, text, lens, ts, attn_type="q8_kernels")
        torch.cuda.current_stream(d).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = blk(x, freqs, None, text, lens, ts, attn_type="q8_kernels")
        x2 = torch.randn(1, S, 512, generator=g).to(torch.bfloat16).to(d)
        want = blk(x2, freqs, None, text, lens, ts, attn_type="q8_kernels").clone()
        x.copy_(x2)
        graph.replay()
        torch.cuda.synchronize(d)
    assert torch.equal(captured, want)
    assert not torch.equal(captured, eager)


@pytest.mark.parametrize("in_f,out_f", [(4096, 10240), (10240, 4096)])
@pytest.mark.parametrize("use_hadamard", [False, True])
def test_fp8_linear_from_linear_at_t5_encoder_dims(cuda_device, in_f, out_f, use_hadamard):
    """The reference builds its FP8 T5 encoder from FP8Linear.from_linear on 4096 <-> 10240 projections
    (q8_kernels/models/T5EncoderFP8.py:275-299): 10240 is not a power of two, so the Hadamard variant pads
    to 16384 and the GEMM runs with K = 10240."""
    import q8_kernels_b200 as q8
    lin = torch.nn.Linear(in_f, out_f, bias=False)
    with torch.no_grad():
        lin.weight.copy_(Hp.weights(out_f, in_f, seed=in_f % 97).float())
    lin = lin.to(torch.bfloat16)
    mod = q8.modules.FP8Linear.from_linear(lin, use_hadamard=use_hadamard)
    wsrc = O.hadamard_transform(lin.weight.data) if use_hadamard else lin.weight.data
    wq, sw = O.tokenwise_quant(wsrc, E4M3)
    Hp.assert_bit_equal(mod.weight.data, wq, "weight")
    Hp.assert_bit_equal(mod.scales.data, sw, "scales")
    x = Hp.activations(48, in_f, seed=5).reshape(1, 48, in_f)
    y = mod(x.to(cuda_device))
    ref = O.fp8_linear(x, wq, None, None, sw, use_hadamard, torch.bfloat16)
    assert y.shape == (1, 48, out_f) and y.dtype == torch.bfloat16
    assert Hp.rel_fro(y.float(), ref.float()) <= TOL


def test_fp8_linear_variant_of_the_block(q8, cuda_device):
    """The same block built from FP8Linear (Hadamard-rotated per-token e4m3 activations, e4m3
    weights): fused path against the op-by-op path, and both against the oracle block run on the
    same e4m3 weights."""
    dim, heads, S, T = 512, 8, 192, 48
    d = cuda_device
    cfg = q8.blocks.LTXStackConfig(num_layers=1, num_attention_heads=heads, attention_head_dim=64,
                                   cross_attention_dim=dim, caption_channels=64, linear="fp8")
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=41, device=d)
    blk = stack.transformer_blocks[0]
    assert blk.attn1.to_q.weight.dtype == E4M3 and blk.ff.proj_down.weight.dtype == E4M3
    g = Hp.gen(42)
    x = torch.randn(2, S, dim, generator=g).to(torch.bfloat16)
    text = torch.randn(2, T, dim, generator=g).to(torch.bfloat16)
    ts = (torch.randn(2, 1, 6 * dim, generator=g) * 0.1).to(torch.bfloat16)
    grid = torch.stack(torch.meshgrid(torch.arange(4), torch.arange(6), torch.arange(8), indexing="ij"), 0)
    cos, sin = O.precompute_freqs_cis(grid.reshape(1, 3, -1).float(), dim=dim)
    lens = torch.tensor([17, 48], dtype=torch.int32)
    args = (x.to(d), (cos.to(d), sin.to(d)), None, text.to(d), lens.to(d), ts.to(d))
    with torch.no_grad():
        fused = blk(*args)
        plain = blk(*args, fuse=False)
    sd = {k: v.detach().cpu() for k, v in blk.state_dict().items()}
    ref = OB.ltx_block(sd, x, (cos, sin), None, text, lens, ts, num_heads=heads, head_dim=64)
    assert Hp.rel_fro(fused.float(), plain.float()) < 5e-3
    for name, got in (("fused", fused), ("op by op", plain)):
        err = Hp.rel_fro(got.float(), ref.float())
        assert err < 2e-2, f"{name}: rel fro {err:.3e}"


def test_full_size_block_fused_path_equals_op_by_op_path(q8, cuda_device):
    """The block at its real size (hidden 2048, 32 x 64 heads, FFN 8192, 6144 tokens, 128 text tokens):
    the fused path (norm + modulation + Hadamard + quantizer producers, stacked QKV, fused q/k prep,
    gate/residual epilogues) against the op-by-op path of the reference.  No oracle needed: both run
    the same arithmetic, only the mean-square summation order of the q/k norm differs."""
    d = cuda_device
    cfg = q8.blocks.LTXStackConfig(num_layers=1)
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=51, device=d)
    blk = stack.transformer_blocks[0]
    g = torch.Generator(device="cpu").manual_seed(52)
    S, T = 6144, 128
    x = torch.randn(1, S, cfg.inner_dim, generator=g).to(torch.bfloat16).to(d)
    text = torch.randn(1, T, cfg.inner_dim, generator=g).to(torch.bfloat16).to(d)
    ts = (torch.randn(1, 1, 6 * cfg.inner_dim, generator=g) * 0.1).to(torch.bfloat16).to(d)
    freqs = stack.freqs_cis(q8.blocks.latent_grid(16, 16, 24, device=d))
    lens = torch.tensor([97], dtype=torch.int32, device=d)
    with torch.no_grad():
        fused = blk(x, freqs, None, text, lens, ts)
        plain = blk(x, freqs, None, text, lens, ts, fuse=False)
    assert torch.isfinite(fused.float()).all()
    err = Hp.rel_fro(fused.float(), plain.float())
    # measured 7.7e-3: a last-bit difference of 1/rms flips a few e4m3 q/k bytes, and over 6144 keys and the
    # re-quantisation of every later activation that grows to bf16-level noise; the bar of the oracle comparison
    assert err < 1.5e-2, f"rel fro {err:.3e}"


def test_full_stack_eager_equals_graph_replay(q8, cuda_device):
    """All 28 blocks on one video: finite output, and the CUDA-graph replay reproduces the eager run
    bit for bit."""
    d = cuda_device
    cfg = q8.blocks.LTXStackConfig()
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=61, device=d)
    g = torch.Generator(device="cpu").manual_seed(62)
    S, T = 6144, 128
    x = torch.randn(1, S, cfg.inner_dim, generator=g).to(torch.bfloat16).to(d)
    text = torch.randn(1, T, cfg.caption_channels, generator=g).to(torch.bfloat16).to(d)
    ts = (torch.randn(1, 1, 6 * cfg.inner_dim, generator=g) * 0.1).to(torch.bfloat16).to(d)
    grid = q8.blocks.latent_grid(16, 16, 24, device=d)
    lens = torch.tensor([97], dtype=torch.int32, device=d)
    with torch.no_grad():
        eager = stack(x, grid, text, lens, ts).clone()
        fn = q8.graph.graphed(lambda *a: stack(*a), check_status=True)
        replay1 = fn(x, grid, text, lens, ts).clone()
        replay2 = fn(x, grid, text, lens, ts)
    assert torch.isfinite(eager.float()).all()
    assert torch.equal(eager, replay1) and torch.equal(eager, replay2)


def test_gate_residual_tail_over_wide_exponent_ranges(q8, cuda_device):
    """The epilogue multiplies and adds in packed bf16; torch multiplies and adds in fp32 and rounds each result to
    bf16.  With a zero activation the linear output is the bias, so gate, bias and residual can be given any
    magnitudes: exponents spread over +-40 octaves, exact ties, cancellations, infinities."""
    d = cuda_device
    M, N, K = 256, 512, 128
    g = Hp.gen(77)
    aq = torch.zeros(1, M, K, dtype=torch.int8, device=d)
    wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(d)
    sa = torch.ones(M, device=d)
    sw = torch.ones(N, device=d)
    def spread(*shape):
        mant = 1.0 + torch.randint(0, 128, shape, generator=g).float() / 128.0
        expo = torch.randint(-40, 41, shape, generator=g).float()
        sign = torch.randint(0, 2, shape, generator=g).float() * 2 - 1
        return sign * mant * torch.exp2(expo)
    bias = spread(N).to(d)
    gate = spread(1, 1, N).to(torch.bfloat16).to(d)
    resid = spread(1, M, N).to(torch.bfloat16)
    resid[0, :, 0::7] = 0.0
    resid[0, 3, 5] = float("inf")
    resid = resid.to(d)
    y = q8.native.q8_mm_bias(aq, wq, bias, sa, sw, False, torch.bfloat16)
    # make a fifth of the residuals cancel the gated value exactly or to within a few ulps
    prod = gate * y
    resid[0, :, 1::5] = -prod[0, :, 1::5]
    resid[0, :, 2::5] = (-prod[0, :, 2::5].float() * (1 + 2.0 ** -7)).to(torch.bfloat16)
    want = gate * y + resid
    got = q8.native.mm_gate_residual(aq, wq, bias, sa, sw, gate, resid)
    assert torch.equal(Hp.bits(got), Hp.bits(want))

