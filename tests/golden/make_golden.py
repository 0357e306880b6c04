"""Generate the committed fixtures under tests/golden/.

Two kinds of file:

* ``ref_*.npz`` -- produced by importing the reference's own pure-torch code
  from a checkout of KONAKONA666/q8_kernels (path in $Q8_REFERENCE):
  ``apply_rope`` (q8_kernels/functional/rope.py:25-43, the
  path the reference really runs) and ``precompute_freqs_cis``
  (q8_kernels/models/LTXVideo.py:86-148).  Their native and diffusers imports
  are replaced by inert stubs; only torch arithmetic of the reference executes.
  These pin the oracle's RoPE and RoPE-table restatements.  ``ref_convert_state_dict.npz`` is the
  reference's checkpoint converter (q8_kernels/utils/convert_weights.py:23-78) run on a miniature
  diffusers-style state dict with its Hadamard / quantizer calls served by the oracle.
* ``ref_linear_chain.npz``, ``ref_linear_backward.npz``, ``ref_flash_attn_glue.npz``, ``ref_attention_module.npz``,
  ``ref_block.npz`` -- the reference's UNMODIFIED Python layer
  (q8_kernels/functional/{linear,flash_attention}.py, modules/attention.py,
  blocks/ltx_transformer_block.py and what they import) executed on the CPU over
  tests/ref_shim.py, i.e. with the fourteen native entry points served by the oracle.
  They pin everything the glue decides -- which tensor is rotated, quantised, padded,
  transposed, cast, in what order and with which defaults -- for the oracle's own
  restatements and for the product's mirrors of those files.
* ``oracle_*.npz`` -- small seeded cases run through oracle/q8_oracle.py, kept
  so that the GPU kernels are also checked against frozen vectors and a change
  of the oracle shows up as a diff.  The reference has no tests or vectors for
  these ops, so they are NOT pinned by the reference.

Usage:  Q8_REFERENCE=<checkout of the reference> python tests/golden/make_golden.py
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import q8_oracle as O  # noqa: E402
import helpers as Hp  # noqa: E402

REF = os.environ.get("Q8_REFERENCE", "")


def _np(t: torch.Tensor) -> np.ndarray:
    """Store tensors losslessly: bf16 as int16 bits, e4m3/int8 as uint8/int8."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def _stub(name: str, **attrs) -> types.ModuleType:
    m = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


def _load(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_fixtures() -> None:
    unavailable = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("native stub"))  # noqa: E731
    _stub("q8_kernels_cuda")
    _stub("q8_kernels_cuda.ops")
    _stub("q8_kernels_cuda.ops._C", rope=unavailable, rope_backward=unavailable)
    ref_rope = _load(os.path.join(REF, "q8_kernels/functional/rope.py"), "ref_rope")

    ident = lambda f: f  # noqa: E731
    _stub("diffusers")
    _stub("diffusers.configuration_utils", ConfigMixin=object, register_to_config=ident)
    _stub("diffusers.models")
    _stub("diffusers.models.embeddings", PixArtAlphaTextProjection=object)
    _stub("diffusers.models.modeling_utils", ModelMixin=torch.nn.Module)
    _stub("diffusers.models.normalization", AdaLayerNormSingle=object)
    _stub("diffusers.utils", BaseOutput=object, is_torch_version=lambda *a: True,
          logging=types.SimpleNamespace(get_logger=lambda n: None))
    _stub("q8_kernels")
    _stub("q8_kernels.blocks")
    _stub("q8_kernels.blocks.ltx_transformer_block", LTXTransformerBlock=object)
    ref_ltx = _load(os.path.join(REF, "q8_kernels/models/LTXVideo.py"), "ref_ltx")

    # RoPE table for a 2 x 3 x 4 latent grid at the model's hyper-parameters
    cls = ref_ltx.LTXTransformer3DModel
    fake = types.SimpleNamespace(inner_dim=2048, positional_embedding_theta=10000.0,
                                 positional_embedding_max_pos=[20, 2048, 2048])
    fake.get_fractional_positions = lambda g: cls.get_fractional_positions(fake, g)
    t, h, w = torch.meshgrid(torch.arange(2), torch.arange(3), torch.arange(4), indexing="ij")
    grid = torch.stack([t.flatten(), h.flatten(), w.flatten()], dim=0).unsqueeze(0).float()     # [1,3,24]
    cos, sin = cls.precompute_freqs_cis(fake, grid)
    np.savez_compressed(os.path.join(HERE, "ref_freqs_cis.npz"), grid=grid.numpy(), cos=cos.numpy(), sin=sin.numpy())

    x = Hp.activations(24, 2048, seed=901).reshape(1, 24, 2048)
    out = ref_rope.apply_rope(x, cos, sin)
    np.savez_compressed(os.path.join(HERE, "ref_rope.npz"), x=_np(x), cos=cos.numpy(), sin=sin.numpy(),
                        out=out.numpy())
    print("reference fixtures:", tuple(cos.shape), out.dtype)


def synthetic_checkpoint(hidden: int = 64, ffn: int = 256, caption: int = 32, blocks: int = 2, seed: int = 77):
    """A diffusers-style LTX-Video transformer state dict in miniature (same key names, bf16)."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape: (torch.randn(*shape, generator=g) * 0.05).to(torch.bfloat16)  # noqa: E731
    sd = {}
    for b in range(blocks):
        pre = f"transformer_blocks.{b}."
        for attn, kv in (("attn1", hidden), ("attn2", hidden)):
            for proj, k in (("to_q", hidden), ("to_k", kv), ("to_v", kv), ("to_out.0", hidden)):
                sd[f"{pre}{attn}.{proj}.weight"] = rnd(hidden, k)
                sd[f"{pre}{attn}.{proj}.bias"] = rnd(hidden)
            sd[f"{pre}{attn}.q_norm.weight"] = 1 + rnd(hidden)
            sd[f"{pre}{attn}.k_norm.weight"] = 1 + rnd(hidden)
        sd[f"{pre}ff.net.0.proj.weight"] = rnd(ffn, hidden)
        sd[f"{pre}ff.net.0.proj.bias"] = rnd(ffn)
        sd[f"{pre}ff.net.2.weight"] = rnd(hidden, ffn)
        sd[f"{pre}ff.net.2.bias"] = rnd(hidden)
        sd[f"{pre}scale_shift_table"] = rnd(6, hidden)
    sd["patchify_proj.weight"] = rnd(hidden, 16)
    sd["patchify_proj.bias"] = rnd(hidden)
    sd["caption_projection.linear_1.weight"] = rnd(hidden, caption)
    sd["caption_projection.linear_1.bias"] = rnd(hidden)
    sd["adaln_single.linear.weight"] = rnd(6 * hidden, hidden)
    sd["scale_shift_table"] = rnd(2, hidden)
    sd["proj_out.weight"] = rnd(16, hidden)
    sd["proj_out.bias"] = rnd(16)
    return sd


def reference_convert_fixture() -> None:
    """q8_kernels/utils/convert_weights.py:23-78 run on the miniature checkpoint, with its two
    native calls (Hadamard, quantizer) served by the oracle and ``.cuda()`` made a no-op: pins the
    key renames, the dtype rules and which tensors get quantised."""
    _stub("q8_kernels.functional")
    _stub("q8_kernels.functional.quantizer", quantize=lambda x: O.tokenwise_quant(x))
    _stub("q8_kernels.functional.fast_hadamard", hadamard_transform=lambda x: O.hadamard_transform(x))
    _stub("q8_kernels.models")
    _stub("q8_kernels.models.LTXVideo", get_ltx_transformer=None)
    ref_conv = _load(os.path.join(REF, "q8_kernels/utils/convert_weights.py"), "ref_convert_weights")
    sd = synthetic_checkpoint()
    real_cuda = torch.Tensor.cuda
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        out = ref_conv.convert_state_dict(dict(sd))
    finally:
        torch.Tensor.cuda = real_cuda
    arrays = {f"in__{k}": _np(v) for k, v in sd.items()}
    arrays.update({f"out__{k}": _np(v) for k, v in out.items()})
    arrays.update({f"dtype__{k}": np.array(str(v.dtype)) for k, v in out.items()})
    np.savez_compressed(os.path.join(HERE, "ref_convert_state_dict.npz"), **arrays)
    print("reference convert_state_dict:", len(sd), "->", len(out), "tensors")


def _save(name: str, **tensors) -> None:
    """Tensors go in losslessly (see _np) with their torch dtype recorded beside them as ``dtype__<key>``."""
    arrays = {}
    for k, v in tensors.items():
        if isinstance(v, torch.Tensor):
            arrays[k] = _np(v.detach().contiguous())
            arrays[f"dtype__{k}"] = np.array(str(v.dtype))
        else:
            arrays[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name), **arrays)


def fill_q8_modules_(module: torch.nn.Module, seed: int) -> None:
    """Seeded parameters for a reference module tree: Hadamard-rotated INT8 weights of N(0,0.05)
    matrices, biases N(0,0.05), norm weights ~1, modulation table ~N(0,1/sqrt(dim))."""
    g = torch.Generator().manual_seed(seed)
    for mod in module.modules():
        if type(mod).__name__ == "Q8Linear":
            w = (torch.randn(mod.out_features, mod.in_features, generator=g) * 0.05).to(torch.bfloat16)
            wq, ws = O.tokenwise_quant(O.hadamard_transform(w))
            mod.weight.data = wq
            mod.scales.data = ws
            if mod.bias is not None:
                mod.bias.data = torch.randn(mod.out_features, generator=g) * 0.05
        elif type(mod).__name__ == "RMSNorm" and mod.weight is not None:
            mod.weight.data = 1.0 + 0.1 * torch.randn(mod.weight.shape, generator=g)
        elif hasattr(mod, "scale_shift_table"):
            t = mod.scale_shift_table
            mod.scale_shift_table.data = (torch.randn(t.shape, generator=g) / t.shape[1] ** 0.5).to(torch.bfloat16)


def reference_glue_fixtures() -> None:
    """The reference's functional / modules / blocks files, unmodified, over the oracle-backed shim."""
    import ref_shim
    ref = ref_shim.load_reference(REF, ref_shim.oracle_backend())
    RF, RM, RB = ref.functional, ref.modules, ref.blocks
    E4M3 = torch.float8_e4m3fn
    bf16 = torch.bfloat16

    # -- functional/linear.py: Q8LinearFunc.forward and FP8LinearFunc.forward
    a = Hp.activations(40, 256, seed=501).reshape(2, 20, 256)
    w = Hp.weights(128, 256, seed=502)
    b = Hp.bias_vec(128, seed=503)
    wq, sw = O.tokenwise_quant(O.hadamard_transform(w))
    a8 = O.c10_e4m3(a.float() * 0.5)                                # an e4m3 activation, as attention hands to to_out
    wf, swf = O.tokenwise_quant(w, E4M3)
    wfh, swfh = O.tokenwise_quant(O.hadamard_transform(w), E4M3)
    _save("ref_linear_chain.npz", a=a, w=w, bias=b, a8=a8, wq=wq, sw=sw, wf=wf, swf=swf, wfh=wfh, swfh=swfh,
          q8_bias_gelu_bf16=RF.linear.q8_linear(a, wq, b, None, sw, True, bf16),
          q8_plain_default=RF.linear.q8_linear(a, wq, None, None, sw, False, None),
          q8_from_e4m3_bf16=RF.linear.q8_linear(a8, wq, b, None, sw, False, bf16),
          q8_16bit_weight_bf16=RF.linear.q8_linear(a, w, b, None, None, False, bf16),
          fp8_bias_bf16=RF.linear.fp8_linear(a, wf, b, None, swf, False, bf16),
          fp8_hadamard_bf16=RF.linear.fp8_linear(a, wfh, None, None, swfh, True, bf16),
          fp8_16bit_weight_bf16=RF.linear.fp8_linear(a, w, b, None, None, False, bf16))

    # -- functional/linear.py, training side: Q8LinearFunc.backward, FP8LinearFunc.backward, Q8LinearLora
    g = (torch.randn(2, 20, 128, generator=Hp.gen(504)) * 0.1).to(bf16)
    a_q8 = a.clone().requires_grad_(True)
    RF.linear.q8_linear(a_q8, wq, b, None, sw, False, bf16).backward(g)
    a_f8 = a.clone().requires_grad_(True)
    RF.linear.fp8_linear(a_f8, wf, b, None, swf, False, bf16).backward(g)
    la = (torch.randn(8, 256, generator=Hp.gen(505)) / 8).to(bf16).requires_grad_(True)
    lb = (torch.randn(128, 8, generator=Hp.gen(506)) * 0.1).to(bf16).requires_grad_(True)
    a_lo = a.clone().requires_grad_(True)
    y_lo = RF.linear.q8_linear_lora(a_lo, wq, b, None, sw, la, lb, True, True, bf16)
    y_lo.backward(g)
    _save("ref_linear_backward.npz", a=a, bias=b, wq=wq, sw=sw, wf=wf, swf=swf, g=g, lora_a=la.detach(),
          lora_b=lb.detach(), q8_grad_a=a_q8.grad, fp8_grad_a=a_f8.grad, lora_out=y_lo.detach(),
          lora_grad_a=a_lo.grad, lora_grad_lora_a=la.grad, lora_grad_lora_b=lb.grad)

    # -- functional/flash_attention.py: FlashAttnFunc.forward
    q, k, v = Hp.qkv(2, 2, 77, 64, seed=511)                          # 77 keys: V^T is padded to 80
    _, kx, vx = Hp.qkv(2, 2, 40, 64, seed=515)
    mask = torch.tensor([13, 40], dtype=torch.int32)
    F = RF.flash_attention.flash_attn_func
    _save("ref_flash_attn_glue.npz", q=q.contiguous(), k=k.contiguous(), v=v.contiguous(), kx=kx.contiguous(),
          vx=vx.contiguous(), mask=mask,
          self_hadamard=F(q, k, v, None, None, True),
          self_plain=F(q, k, v, None, None, False),
          self_scale=F(q, k, v, 0.2, None, True),
          cross_masked=F(q, kx, vx, None, mask, True))

    # -- modules/attention.py: Attention.forward
    dim, heads = 256, 4
    S, T = 48, 24
    x = Hp.activations(2 * S, dim, seed=521).reshape(2, S, dim)
    text = Hp.activations(2 * T, dim, seed=522, outliers=False).reshape(2, T, dim)
    ang = torch.rand(1, S, dim, generator=Hp.gen(523)) * 6.28
    cos, sin = ang.cos().expand(2, S, dim).contiguous(), ang.sin().expand(2, S, dim).contiguous()
    lens = torch.tensor([9, 24], dtype=torch.int32)
    self_attn = RM.attention.Attention(dim, heads, 64, True, True, qk_rms_norm=True, use_rope=True)
    cross_attn = RM.attention.Attention(dim, heads, 64, True, True, qk_rms_norm=True, kv_dim=dim, use_rope=False)
    fill_q8_modules_(self_attn, 524)
    fill_q8_modules_(cross_attn, 525)
    with torch.no_grad():
        out = {
            # the reference's own default: torch SDPA, rotary embedding on
            "self_torch": self_attn(x, (cos, sin), None, None, bf16, bf16),
            # the FP8 kernel path; without the rotary embedding, whose fp32 result the Hadamard entry point rejects
            "self_q8_norope": self_attn(x, None, text * 0 + x[:, :T], None, bf16, bf16, True, "q8_kernels"),
            "cross_q8_masked": cross_attn(x, None, text, lens, bf16, bf16, True, "q8_kernels"),
            "cross_torch_masked": cross_attn(x, None, text, lens, bf16, bf16, True, "torch"),
        }
        try:
            self_attn(x, (cos, sin), None, None, bf16, bf16, True, "q8_kernels")
            rope_q8 = "ran"
        except Exception as exc:                                 # noqa: BLE001
            rope_q8 = f"{type(exc).__name__}: {exc}"
    _save("ref_attention_module.npz", x=x, text=text, cos=cos, sin=sin, lens=lens,
          self_rope_q8_outcome=np.array(rope_q8),
          **{f"self_sd__{k_}": v_ for k_, v_ in self_attn.state_dict().items()},
          **{f"cross_sd__{k_}": v_ for k_, v_ in cross_attn.state_dict().items()}, **out)

    # -- blocks/ltx_transformer_block.py: LTXTransformerBlock.forward (runs torch SDPA: it never forwards attn_type)
    blk = RB.ltx_transformer_block.LTXTransformerBlock(dim, heads, 64, dim)
    fill_q8_modules_(blk, 531)
    ts = (torch.randn(2, 1, 6 * dim, generator=Hp.gen(532)) * 0.1).to(bf16)
    with torch.no_grad():
        y = blk(x, (cos, sin), None, text, lens, ts)
    _save("ref_block.npz", x=x, text=text, cos=cos, sin=sin, lens=lens, timestep=ts, out=y,
          **{f"sd__{k_}": v_ for k_, v_ in blk.state_dict().items()})
    print("reference glue fixtures: linear chain, flash-attention glue, attention module (rope + q8: %s), block"
          % rope_q8.split(":")[0])


def oracle_fixtures() -> None:
    E4M3 = torch.float8_e4m3fn
    # quantizer
    x = Hp.activations(16, 256, seed=11)
    x[3] = 0                                               # all-zero row: defined edge case
    q8, s8 = O.tokenwise_quant(x)
    qf, sf = O.tokenwise_quant(x, E4M3)
    np.savez_compressed(os.path.join(HERE, "oracle_quant.npz"), x=_np(x), q_i8=_np(q8), s_i8=s8.numpy(),
                        q_fp8=_np(qf), s_fp8=sf.numpy())
    # Hadamard (power-of-two and padded dims)
    cases = {}
    for dim in (64, 2048, 40):
        xh = Hp.activations(8, dim, seed=20 + dim)
        cases[f"x_{dim}"] = _np(xh)
        cases[f"bf16_{dim}"] = _np(O.hadamard_transform(xh))
        cases[f"fp8_{dim}"] = _np(O.hadamard_transform(xh, scale=0.0442, out_dtype=E4M3))
    np.savez_compressed(os.path.join(HERE, "oracle_hadamard.npz"), **cases)
    # GEMM (int8 and fp8, bias + GELU, bf16 out)
    a = Hp.activations(96, 256, seed=31)
    w = Hp.weights(128, 256, seed=32)
    b = Hp.bias_vec(128, seed=33)
    aq, sa = O.tokenwise_quant(O.hadamard_transform(a))
    wq, sw = O.tokenwise_quant(O.hadamard_transform(w))
    y_i8 = O.q8_mm(aq, wq, sa, sw, True, torch.bfloat16, bias=b)
    af, saf = O.tokenwise_quant(a, E4M3)
    wf, swf = O.tokenwise_quant(w, E4M3)
    y_f8 = O.fp8_mm(af, wf, saf, swf, True, torch.bfloat16, bias=b)
    np.savez_compressed(os.path.join(HERE, "oracle_gemm.npz"), a=_np(a), w=_np(w), bias=b.numpy(),
                        aq=_np(aq), sa=sa.numpy(), wq=_np(wq), sw=sw.numpy(), y_i8=_np(y_i8),
                        af=_np(af), saf=saf.numpy(), wf=_np(wf), swf=swf.numpy(), y_f8=_np(y_f8))
    # attention (self, ragged length, masked)
    q, k, v = Hp.qkv(1, 2, 200, 64, seed=41)
    o_self = O.flash_attn_func(q, k, v, apply_qk_hadamard=True, out_dtype=torch.bfloat16)
    mask = torch.tensor([77], dtype=torch.int32)
    o_mask = O.flash_attn_func(q, k, v, batch_mask=mask, apply_qk_hadamard=True, out_dtype=torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "oracle_attention.npz"), q=_np(q.contiguous()), k=_np(k.contiguous()),
                        v=_np(v.contiguous()), o_self=_np(o_self), mask=mask.numpy(), o_mask=_np(o_mask))
    print("oracle fixtures written")


if __name__ == "__main__":
    if REF and os.path.isdir(REF):
        reference_fixtures()
        reference_convert_fixture()
        reference_glue_fixtures()
    else:
        print("$Q8_REFERENCE does not name a checkout of the reference: reference fixtures left untouched")
    oracle_fixtures()
