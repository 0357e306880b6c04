"""GPU parity of the tcgen05 FP8 flash attention against the reference-faithful
CPU oracle (64-key blocks, last to first, e4m3 P): rel. Frobenius <= 2e-3 on the
bf16 output."""
import math

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


def _fp8_operands(B, H, M, N, seed, hadamard=True):
    q, _, _ = Hp.qkv(B, H, M, 64, seed)
    _, k, v = Hp.qkv(B, H, N, 64, seed + 7)
    scale = 64 ** -0.5
    if hadamard:
        hd = math.sqrt(1 / 64) * math.sqrt(scale)
        q8 = O.hadamard_transform(q, scale=hd, out_dtype=E4M3)
        k8 = O.hadamard_transform(k, scale=hd, out_dtype=E4M3)
        ks = 1.0
    else:
        q8, k8, ks = O.c10_e4m3(q * 0.25), O.c10_e4m3(k * 0.25), scale
    pad = (16 - N % 16) % 16
    vt = O.c10_e4m3(torch.nn.functional.pad(v.transpose(2, 3), (0, pad))).contiguous()
    return q8.contiguous(), k8.contiguous(), vt, ks


@pytest.mark.parametrize("B,H,M,N", [(1, 1, 128, 64), (1, 1, 128, 128), (1, 2, 128, 192), (2, 3, 256, 512),
                                     (1, 2, 100, 200), (1, 1, 1, 1), (1, 2, 333, 77), (1, 4, 640, 1536),
                                     (2, 2, 130, 1025)])
@pytest.mark.parametrize("hadamard", [True, False])
def test_attention_kernel_vs_oracle(nat, cuda_device, B, H, M, N, hadamard):
    q8, k8, vt, ks = _fp8_operands(B, H, M, N, seed=M + N, hadamard=hadamard)
    ref = O.flash_attention(q8, k8, vt, ks, None, torch.bfloat16)
    got = nat.flash_attention(q8.to(cuda_device), k8.to(cuda_device), vt.to(cuda_device), ks, None, torch.bfloat16)
    assert got.shape == (B, H, M, 64) and got.dtype == torch.bfloat16
    err = Hp.rel_fro(got.float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"


def test_attention_default_output_is_e4m3(nat, cuda_device):
    q8, k8, vt, ks = _fp8_operands(1, 2, 256, 320, seed=3)
    ref = O.flash_attention(q8, k8, vt, ks, None, E4M3)
    got = nat.flash_attention(q8.to(cuda_device), k8.to(cuda_device), vt.to(cuda_device), ks, None)
    assert got.dtype == E4M3
    g, r = got.float().cpu(), ref.float()
    assert (g != r).float().mean().item() < 0.02


@pytest.mark.parametrize("lens", [[16, 128], [1, 64], [65, 127], [128, 128], [0, 100]])
def test_cross_attention_key_padding_mask(nat, cuda_device, lens):
    B, H, M, N = 2, 4, 384, 128
    q8, k8, vt, ks = _fp8_operands(B, H, M, N, seed=sum(lens))
    mask = torch.tensor(lens, dtype=torch.int32)
    ref = O.flash_attention(q8, k8, vt, ks, mask, torch.bfloat16)
    got = nat.flash_attention(q8.to(cuda_device), k8.to(cuda_device), vt.to(cuda_device), ks,
                              mask.to(cuda_device), torch.bfloat16)
    err = Hp.rel_fro(got.float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"


def test_attention_golden_fixture_through_functional_api(cuda_device):
    import q8_kernels_b200.functional as Q8F
    d = G.load("oracle_attention.npz")
    q, k, v = (G.bf16(d[n]).to(cuda_device) for n in ("q", "k", "v"))
    o = Q8F.flash_attention.flash_attn_func(q, k, v, apply_qk_hadamard=True, out_dtype=torch.bfloat16)
    assert Hp.rel_fro(o.float(), G.bf16(d["o_self"]).float()) <= TOL
    o = Q8F.flash_attention.flash_attn_func(q, k, v, batch_mask=G.t(d["mask"]).to(cuda_device),
                                            apply_qk_hadamard=True, out_dtype=torch.bfloat16)
    assert Hp.rel_fro(o.float(), G.bf16(d["o_mask"]).float()) <= TOL
    assert Q8F.flash_attention.flash_attn_func(q, k, v).dtype == E4M3


@pytest.mark.parametrize("hadamard", [True, False])
def test_attention_prep_bit_exact(nat, cuda_device, hadamard):
    """The fused pre-pass equals the reference glue: Hadamard(+scale)->e4m3 or
    plain cast for Q/K, transpose + zero pad + cast for V."""
    q, k, v = Hp.qkv(2, 4, 150, 64, seed=12)                 # [B,H,S,64] views of [B,S,H*64]
    scale = 0.0442 if hadamard else 1.0
    q8, k8, vt8 = nat.attention_prep(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), hadamard, scale)
    if hadamard:
        rq = O.hadamard_transform(q, scale=scale, out_dtype=E4M3)
        rk = O.hadamard_transform(k, scale=scale, out_dtype=E4M3)
    else:
        rq, rk = O.c10_e4m3(q), O.c10_e4m3(k)
    rv = O.c10_e4m3(torch.nn.functional.pad(v.transpose(2, 3), (0, 10)))
    Hp.assert_bit_equal(q8, rq.contiguous(), "q8")
    Hp.assert_bit_equal(k8, rk.contiguous(), "k8")
    assert vt8.shape == (2, 4, 64, 160)
    Hp.assert_bit_equal(vt8, rv.contiguous(), "vt8")


def test_self_attention_dit_shape_sampled(nat, cuda_device):
    """Config-3 shape (S = 6144, D = 64) on 2 heads; the oracle is evaluated on a
    sample of query rows (every key is still visited), the full output through
    its row-sum property: with V = const the output equals that constant."""
    B, H, S = 1, 2, 6144
    q8, k8, vt, ks = _fp8_operands(B, H, S, S, seed=99)
    got = nat.flash_attention(q8.to(cuda_device), k8.to(cuda_device), vt.to(cuda_device), ks, None, torch.bfloat16)
    rows = torch.randperm(S, generator=Hp.gen(2))[:160].sort().values
    ref = O.flash_attention(q8[:, :, rows].contiguous(), k8, vt, ks, None, torch.bfloat16)
    err = Hp.rel_fro(got[:, :, rows.to(cuda_device)].float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"
    vt_const = torch.full_like(vt.float(), 0.75).to(E4M3)
    out = nat.flash_attention(q8.to(cuda_device), k8.to(cuda_device), vt_const.to(cuda_device), ks, None,
                              torch.bfloat16).float()
    # out = 0.75 * sum(e4m3(p)) / sum(p): e4m3 rounding averages out, but p below 2^-10 flushes to zero,
    # so peaky rows lose some tail mass -- never gain more than one e4m3 ulp
    assert out.max().item() <= 0.75 * (1 + 2 ** -4)
    assert (out - 0.75).abs().mean().item() < 0.03 and out.min().item() > 0.5


def test_token_major_output_is_the_same_values(nat, cuda_device):
    q8, k8, vt, ks = _fp8_operands(2, 4, 200, 333, seed=17)
    d = cuda_device
    a = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, None, torch.bfloat16)
    b = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, None, torch.bfloat16, token_major_out=True)
    assert b.shape == a.shape and not b.is_contiguous()
    assert torch.equal(a, b)
    flat = b.transpose(1, 2).reshape(2, 200, 4 * 64)
    assert flat.data_ptr() == b.data_ptr()                     # the module's reshape is a view, not a copy


@pytest.mark.parametrize("B,S,H,rope", [(2, 96, 32, True), (1, 130, 32, False), (1, 64, 4, True), (1, 33, 128, True)])
def test_fused_qk_norm_rope_prep_matches_the_op_chain(nat, cuda_device, B, S, H, rope):
    """One kernel for q_norm/k_norm + RoPE + head Hadamard + e4m3 cast against the same steps as
    separate kernels (rms_norm -> rope -> attention_prep) and against the oracle's chain.  The only
    difference allowed is the summation order of the mean square: an occasional last-bit flip."""
    C = H * 64
    x = Hp.activations(B * S, C, seed=S + H).view(B, S, C).to(cuda_device)
    w = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(5))).to(cuda_device)
    ang = torch.rand(1, S, C, generator=Hp.gen(6)) * 6.28
    cos, sin = ang.cos().to(cuda_device), ang.sin().to(cuda_device)
    scale = math.sqrt(1 / 64) * math.sqrt(64 ** -0.5)
    fc = (cos, sin) if rope else None
    got = nat.qk_norm_rope_prep(x, w, fc, H, True, scale)
    assert got.shape == (B, H, S, 64) and got.dtype == E4M3

    y = nat.rms_norm(x, w, torch.bfloat16)[0]
    if rope:
        y = nat.rope(y, cos, sin, torch.bfloat16)
    yh = y.view(B, S, H, 64).transpose(1, 2)
    want, _, _ = nat.attention_prep(yh, yh, yh, True, scale)
    mism = (Hp.bits(got) != Hp.bits(want)).float().mean().item()
    assert mism < 2e-3, f"{mism:.2e} of the bytes differ from the op chain"
    assert Hp.rel_fro(got.float(), want.float()) < 2e-3

    yo = O.rms_norm(x.cpu(), w.cpu(), torch.bfloat16)[0]
    if rope:
        yo = O.rope(yo, cos.cpu(), sin.cpu(), torch.bfloat16)
    ref = O.hadamard_transform(yo.view(B, S, H, 64).transpose(1, 2), scale=scale, out_dtype=E4M3)
    assert Hp.rel_fro(got.float().cpu(), ref.float()) < 2e-3

    # a row-strided view (e.g. a slice of a wider projection output) gives the same bytes
    wide = torch.zeros(B, S, C + 64, dtype=torch.bfloat16, device=cuda_device)
    wide[..., :C] = x
    assert torch.equal(Hp.bits(nat.qk_norm_rope_prep(wide[..., :C], w, fc, H, True, scale)), Hp.bits(got))


def test_attention_prep_v_alone_matches_attention_prep(nat, cuda_device):
    q, k, v = (t.to(cuda_device) for t in Hp.qkv(2, 3, 77, 64, seed=9))
    _, _, want = nat.attention_prep(q, k, v, False, 1.0)
    assert torch.equal(Hp.bits(nat.attention_prep_v(v)), Hp.bits(want))


def test_paired_qk_prep_is_two_single_calls(nat, cuda_device):
    """Q and K of a self-attention taken as column slices of one fused projection output."""
    B, S, H = 2, 70, 32
    C = H * 64
    qkv = Hp.activations(B * S, 3 * C, seed=21).view(B, S, 3 * C).to(cuda_device)
    wq = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(1))).to(cuda_device)
    wk = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(2))).to(cuda_device)
    ang = torch.rand(1, S, C, generator=Hp.gen(3)) * 6.28
    fc = (ang.cos().to(cuda_device), ang.sin().to(cuda_device))
    scale = 0.125 * math.sqrt(0.125)
    q8, k8 = nat.qk_norm_rope_prep_pair(qkv[..., :C], qkv[..., C:2 * C], wq, wk, fc, H, True, scale)
    assert torch.equal(Hp.bits(q8), Hp.bits(nat.qk_norm_rope_prep(qkv[..., :C], wq, fc, H, True, scale)))
    assert torch.equal(Hp.bits(k8), Hp.bits(nat.qk_norm_rope_prep(qkv[..., C:2 * C], wk, fc, H, True, scale)))


@pytest.mark.parametrize("B,H,M,N,lens,out", [(2, 32, 900, 128, [77, 128], torch.bfloat16),
                                              (2, 32, 900, 192, None, torch.bfloat16),
                                              (3, 24, 1100, 100, [0, 100, 33], None),
                                              (1, 64, 1536, 64, None, None)])
def test_short_key_sequences_with_several_query_tiles_per_cta(nat, cuda_device, B, H, M, N, lens, out):
    """With at most three key blocks and more (batch, head) pairs than a third of the device's CTA slots, a CTA
    keeps K/V and walks over several query tiles, unevenly distributed here (7, 8, 9 or 12 tiles over fewer
    CTAs, the last tile partial); every output row against the oracle, e4m3 and bf16 outputs, V both ways."""
    d = cuda_device
    q8, k8, vt, ks = _fp8_operands(B, H, M, N, seed=M + N + H)
    mask = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    ref = O.flash_attention(q8, k8, vt, ks, mask, torch.bfloat16)
    md = None if mask is None else mask.to(d)
    got = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, md, out)
    if out is None:
        assert got.dtype == E4M3
        ref8 = O.flash_attention(q8, k8, vt, ks, mask, E4M3)
        per_batch = [(Hp.bits(got[b].cpu()) != Hp.bits(ref8[b])).float().mean().item() for b in range(B)]
        assert max(per_batch) < 0.02, per_batch
    else:
        err = Hp.rel_fro(got.float(), ref.float())
        assert err <= TOL, f"rel fro {err:.3e}"
    v_rows = vt[..., :N].transpose(2, 3).contiguous()
    again = nat.flash_attention(q8.to(d), k8.to(d), v_rows.to(d), ks, md, out, v_rows=True)
    assert torch.equal(Hp.bits(again), Hp.bits(got))
    tm = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, md, out, token_major_out=True)      # stored [B,M,H,64]
    assert torch.equal(Hp.bits(tm.contiguous()), Hp.bits(got))


def test_scores_far_below_the_row_maximum(nat, cuda_device):
    """Unrotated operands with a few keys scaled up to the e4m3 range: in the blocks visited later most scores lie
    hundreds to thousands of octaves under the running maximum, which must come out as zero weight in whatever
    unit computes the exponential."""
    B, H, M, N = 1, 2, 256, 512
    g = Hp.gen(41)
    q8 = O.c10_e4m3(torch.randn(B, H, M, 64, generator=g) * 8.0)
    k = torch.randn(B, H, N, 64, generator=g) * 2.0
    k[:, :, 500] *= 100.0                                      # saturates towards +-448: one dominating key in the first-visited block
    k[:, :, 77] *= 40.0
    k8 = O.c10_e4m3(k.clamp(-440, 440))
    vt = O.c10_e4m3(torch.randn(B, H, 64, N, generator=g)).contiguous()
    ref = O.flash_attention(q8, k8, vt, 1.0, None, torch.bfloat16)
    assert torch.isfinite(ref.float()).all()
    got = nat.flash_attention(q8.to(cuda_device), k8.to(cuda_device), vt.to(cuda_device), 1.0, None, torch.bfloat16)
    err = Hp.rel_fro(got.float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"


def test_qkv_prep_adds_the_plain_cast_of_v(nat, cuda_device):
    """The three slices of a fused QKV projection in one launch: Q and K as in the paired call, V the
    unscaled e4m3 cast as rows [B,H,S,64]."""
    B, S, H = 2, 70, 32
    C = H * 64
    qkv = Hp.activations(B * S, 3 * C, seed=23).view(B, S, 3 * C).to(cuda_device)
    wq = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(1))).to(cuda_device)
    wk = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(2))).to(cuda_device)
    ang = torch.rand(1, S, C, generator=Hp.gen(3)) * 6.28
    fc = (ang.cos().to(cuda_device), ang.sin().to(cuda_device))
    scale = 0.125 * math.sqrt(0.125)
    q8, k8, v8 = nat.qk_norm_rope_prep_pair(qkv[..., :C], qkv[..., C:2 * C], wq, wk, fc, H, True, scale, xv=qkv[..., 2 * C:])
    q8b, k8b = nat.qk_norm_rope_prep_pair(qkv[..., :C], qkv[..., C:2 * C], wq, wk, fc, H, True, scale)
    assert torch.equal(Hp.bits(q8), Hp.bits(q8b)) and torch.equal(Hp.bits(k8), Hp.bits(k8b))
    want_v = qkv[..., 2 * C:].view(B, S, H, 64).transpose(1, 2).to(E4M3)          # torch's cast is the c10 one
    assert v8.shape == (B, H, S, 64) and torch.equal(Hp.bits(v8), Hp.bits(want_v.contiguous()))


def test_kv_prep_is_k_prep_plus_the_cast_of_v(nat, cuda_device):
    B, S, H = 2, 37, 32
    C = H * 64
    kv = Hp.activations(B * S, 2 * C, seed=31).view(B, S, 2 * C).to(cuda_device)
    wk = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(2))).to(cuda_device)
    scale = 0.125 * math.sqrt(0.125)
    k8, v8 = nat.kv_prep(kv[..., :C], kv[..., C:], wk, H, True, scale)
    assert torch.equal(Hp.bits(k8), Hp.bits(nat.qk_norm_rope_prep(kv[..., :C], wk, None, H, True, scale)))
    want_v = kv[..., C:].view(B, S, H, 64).transpose(1, 2).to(E4M3)
    assert torch.equal(Hp.bits(v8), Hp.bits(want_v.contiguous()))


@pytest.mark.parametrize("B,S", [(2, 70), (1, 128), (3, 33)])
def test_qk_prep_without_rotation_two_rows_per_cta(nat, cuda_device, B, S):
    """Without rotary tables an even number of rows runs two rows per CTA (B=3, S=33 is odd and takes the
    one-row kernel): both against the separate ops (RMS norm, per-head Hadamard + cast)."""
    H = 32
    C = H * 64
    x = Hp.activations(B * S, C, seed=29 + S).view(B, S, C).to(cuda_device)
    w = (1.0 + 0.1 * torch.randn(C, generator=Hp.gen(4))).to(cuda_device)
    scale = 0.125 * math.sqrt(0.125)
    got = nat.qk_norm_rope_prep(x, w, None, H, True, scale)
    normed = nat.rms_norm(x, w, None)[0]
    want = nat.fast_hadamard_transform(normed.view(B, S, H, 64).transpose(1, 2).contiguous(), scale, E4M3)
    diff = (Hp.bits(got) != Hp.bits(want)).float().mean().item()
    assert diff < 2e-3, diff                                   # the mean-square summation order is the only difference


def test_head_slices_written_into_several_full_buffers(nat, cuda_device):
    """The multi-destination output used by gather-free head sharding, on one GPU: two "ranks" each own
    half of the heads and store them into both of two full token-major buffers."""
    B, H, S = 2, 4, 200
    q, k, v = (t.to(cuda_device) for t in Hp.qkv(B, H, S, 64, seed=77))
    scale = math.sqrt(1 / 64) * math.sqrt(64 ** -0.5)
    q8, k8, vt8 = nat.attention_prep(q, k, v, True, scale)
    want = nat.flash_attention(q8, k8, vt8, 1.0, None, None, token_major_out=True).transpose(1, 2).contiguous()  # [B,S,H,64]
    bufs = [torch.zeros(B, S, H, 64, dtype=torch.uint8, device=cuda_device).view(E4M3) for _ in range(2)]
    for r in range(2):
        sl = slice(2 * r, 2 * r + 2)
        nat.flash_attention_into(q8[:, sl], k8[:, sl], vt8[:, sl], 1.0, None, E4M3, [b.data_ptr() for b in bufs], H, 2 * r)
    for b in bufs:
        assert torch.equal(Hp.bits(b), Hp.bits(want))
    with pytest.raises(Exception):
        nat.flash_attention_into(q8, k8, vt8, 1.0, None, E4M3, [bufs[0].data_ptr()], H, 2)     # heads 2..6 of 4


@pytest.mark.parametrize("N", [128, 6144])
def test_all_equal_keys_never_move_the_row_max(nat, cuda_device, N):
    """Every key identical: the row max is set by the first block visited and never moves again, so
    no step rescales O and the kernel's only reason to look at the P.V completion barrier inside
    the loop is to stay in step with it.  2 blocks (cross-attention size) and 96 blocks."""
    B, H, M = 1, 2, 256
    q8, k8, vt, ks = _fp8_operands(B, H, M, N, seed=5)
    k8 = k8[:, :, :1].expand(B, H, N, 64).contiguous()
    ref = O.flash_attention(q8, k8, vt, ks, None, torch.bfloat16)
    d = cuda_device
    for _ in range(20):
        got = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, None, torch.bfloat16)
        err = Hp.rel_fro(got.float(), ref.float())
        assert err <= TOL, f"rel fro {err:.3e}"


def test_bit_stable_under_memory_pressure(nat, cuda_device):
    """The config-3 head slice (S = 6144) launched 320 times while a second stream keeps HBM busy
    with large copies: a V tile that lands late must not change a single output byte."""
    B, H, S = 1, 8, 6144
    d = cuda_device
    q8, k8, vt, ks = (t.to(d) if isinstance(t, torch.Tensor) else t for t in _fp8_operands(B, H, S, S, seed=31))
    want = nat.flash_attention(q8, k8, vt, ks, None, torch.bfloat16)
    torch.cuda.synchronize()
    src = torch.empty(1 << 30, dtype=torch.uint8, device=d)
    dst = torch.empty_like(src)
    side = torch.cuda.Stream(device=d)
    outs = []
    bad = 0
    for it in range(320):
        if it % 4 == 0:
            with torch.cuda.stream(side):
                dst.copy_(src, non_blocking=True)
        outs.append(nat.flash_attention(q8, k8, vt, ks, None, torch.bfloat16))
        if len(outs) == 16:
            torch.cuda.synchronize()
            bad += sum(0 if torch.equal(o, want) else 1 for o in outs)
            outs.clear()
    torch.cuda.synchronize()
    bad += sum(0 if torch.equal(o, want) else 1 for o in outs)
    assert bad == 0, f"{bad} of 320 launches differ from the first"


def test_cross_attention_full_shape_sampled(nat, cuda_device):
    """Q [2,32,6144,64] x K/V [2,32,128,64] with key-padding lengths drawn from 16..128: sampled
    (batch, head, row) triples against the oracle."""
    B, H, M, N = 2, 32, 6144, 128
    q8, k8, vt, ks = _fp8_operands(B, H, M, N, seed=404)
    lens = torch.randint(16, 129, (B,), generator=Hp.gen(404), dtype=torch.int32)
    d = cuda_device
    got = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, lens.to(d), torch.bfloat16).cpu()
    heads = [0, 13, 31]
    rows = torch.randperm(M, generator=Hp.gen(7))[:192].sort().values
    ref = O.flash_attention(q8[:, heads][:, :, rows].contiguous(), k8[:, heads].contiguous(),
                            vt[:, heads].contiguous(), ks, lens, torch.bfloat16)
    err = Hp.rel_fro(got[:, heads][:, :, rows].float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"


def test_self_attention_full_shape_sampled(nat, cuda_device):
    """B = 2, H = 32, S = 6144 (the whole self-attention of one DiT block for two videos): sampled
    (head, row) pairs of both batch entries against the oracle."""
    B, H, S = 2, 32, 6144
    q8, k8, vt, ks = _fp8_operands(B, H, S, S, seed=303)
    d = cuda_device
    got = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, None, torch.bfloat16).cpu()
    heads = [3, 30]
    rows = torch.randperm(S, generator=Hp.gen(8))[:64].sort().values
    ref = O.flash_attention(q8[:, heads][:, :, rows].contiguous(), k8[:, heads].contiguous(),
                            vt[:, heads].contiguous(), ks, None, torch.bfloat16)
    err = Hp.rel_fro(got[:, heads][:, :, rows].float(), ref.float())
    assert err <= TOL, f"rel fro {err:.3e}"


def test_abandoned_wait_is_reported_and_the_context_survives(nat, cuda_device):
    """A wait that nothing satisfies runs into its limit (a warp of a self-test kernel waits on a
    barrier nobody signals): the kernel returns, the status word carries the timeout code and the
    site, launches that share the word do nothing until it is cleared, and afterwards the same
    context computes correct results again."""
    from q8_kernels_b200 import _lib
    d = cuda_device
    q8, k8, vt, ks = _fp8_operands(1, 2, 256, 320, seed=3)
    q8, k8, vt = q8.to(d), k8.to(d), vt.to(d)
    want = nat.flash_attention(q8, k8, vt, ks, None, torch.bfloat16)
    torch.cuda.synchronize()
    word = _lib.status_word(d)
    _lib.check(_lib.lib.q8k_wait_selftest(word.data_ptr(), 2000, _lib.stream_ptr(d)), "wait_selftest")
    torch.cuda.synchronize()
    assert int(word.item()) == (0x1 | (9 << 8))
    skipped = nat.flash_attention(q8, k8, vt, ks, None, torch.bfloat16)      # returns at once: status word is set
    torch.cuda.synchronize()
    with pytest.raises(_lib.Q8KernelError, match="abandoned a wait"):
        _lib.check_status(d)                                              # raises and clears the word
    assert int(word.item()) == 0
    del skipped
    again = nat.flash_attention(q8, k8, vt, ks, None, torch.bfloat16)
    assert torch.equal(again, want)


@pytest.mark.parametrize("B,H,M,N,lens", [(1, 2, 256, 320, None), (2, 3, 130, 1025, None), (2, 4, 384, 128, [65, 127]),
                                          (1, 1, 100, 77, None), (2, 2, 200, 128, [0, 100])])
def test_v_as_rows_gives_the_same_bits_as_v_transposed(nat, cuda_device, B, H, M, N, lens):
    """V handed over as [B,H,N,64] rows and read MN-major by the tensor core against the reference's
    transposed, padded layout: the same products in the same order, so identical outputs."""
    d = cuda_device
    q8, k8, vt, ks = _fp8_operands(B, H, M, N, seed=M + 3 * N)
    v_rows = vt[..., :N].transpose(2, 3).contiguous()
    mask = None if lens is None else torch.tensor(lens, dtype=torch.int32, device=d)
    a = nat.flash_attention(q8.to(d), k8.to(d), vt.to(d), ks, mask, torch.bfloat16)
    b = nat.flash_attention(q8.to(d), k8.to(d), v_rows.to(d), ks, mask, torch.bfloat16, v_rows=True)
    assert torch.equal(a, b)


def test_attention_cast_rows_is_the_unscaled_e4m3_cast(nat, cuda_device):
    _, _, v = Hp.qkv(2, 3, 77, 64, seed=9)                   # [B,H,S,64] view of [B,S,H*64]
    got = nat.attention_cast_rows(v.to(cuda_device))
    assert got.shape == (2, 3, 77, 64) and got.is_contiguous()
    Hp.assert_bit_equal(got, O.c10_e4m3(v).contiguous(), "v rows")
    # values beyond the e4m3 range, infinities and NaNs of both signs: the c10 cast gives NaN with the sign kept,
    # where the packed hardware conversion alone would saturate (the kernel patches those groups of eight)
    big = v.clone()
    flat = big.reshape(-1)
    flat[5] = 464.0; flat[6] = 465.0; flat[70] = -1000.0; flat[133] = float("inf"); flat[200] = float("-inf")
    flat[260] = float("nan"); flat[333] = -float("nan"); flat[400] = 448.0; flat[401] = -463.9
    got = nat.attention_cast_rows(big.to(cuda_device))
    Hp.assert_bit_equal(got, O.c10_e4m3(big).contiguous(), "v rows with out-of-range values")
