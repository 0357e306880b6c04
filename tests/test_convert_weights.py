"""Checkpoint conversion against the fixture made by running the reference's own converter
(q8_kernels/utils/convert_weights.py:23-78, see tests/golden/make_golden.py) on a miniature
diffusers-style state dict: key renames, dtype rules, which tensors are quantised -- and, on a
GPU, the quantised bytes themselves."""
import os

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
FIX = os.path.join(HERE, "golden", "ref_convert_state_dict.npz")


def _tensor(arr: np.ndarray, dtype: str) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if dtype == "torch.bfloat16":
        return t.view(torch.bfloat16)
    return t


@pytest.fixture(scope="module")
def fixture():
    z = np.load(FIX)
    ins, outs = {}, {}
    for name in z.files:
        if name.startswith("in__"):
            ins[name[4:]] = _tensor(z[name], "torch.bfloat16")
    for name in z.files:
        if name.startswith("out__"):
            key = name[5:]
            outs[key] = _tensor(z[name], str(z["dtype__" + key]))
    return ins, outs


def test_key_plan_matches_the_reference_converter(fixture):
    from q8_kernels_b200.utils import convert_weights as cw
    ins, outs = fixture
    plan = cw.plan_state_dict(ins.keys())
    produced = {}
    for key, new_key, action in plan:
        if action == cw.QUANTIZE:
            produced[new_key] = torch.int8
            produced[new_key.replace("weight", "scales")] = torch.float32
        elif action == cw.TO_FP32:
            produced[new_key] = torch.float32
        else:
            produced[new_key] = ins[key].dtype
    assert set(produced) == set(outs)
    for k, dt in produced.items():
        assert outs[k].dtype == dt, k
    # spot checks of the renames themselves
    assert "transformer_blocks.1.attn2.to_out.weight" in produced and "transformer_blocks.1.attn2.to_out.0.weight" not in produced
    assert "transformer_blocks.0.ff.act.proj.scales" in produced and "transformer_blocks.0.ff.proj_down.bias" in produced
    assert produced["transformer_blocks.0.attn1.q_norm.weight"] == torch.float32
    assert produced["caption_projection.linear_1.weight"] == torch.bfloat16          # outside the blocks: untouched


def test_unquantised_tensors_pass_through_like_the_reference(fixture):
    from q8_kernels_b200.utils import convert_weights as cw
    ins, outs = fixture
    for key, new_key, action in cw.plan_state_dict(ins.keys()):
        if action == cw.KEEP:
            assert torch.equal(ins[key].view(torch.int16), outs[new_key].view(torch.int16)), key
        elif action == cw.TO_FP32:
            assert torch.equal(ins[key].float(), outs[new_key]), key


def test_unknown_block_key_is_an_error():
    from q8_kernels_b200.utils import convert_weights as cw
    with pytest.raises(ValueError):
        cw.plan_key("transformer_blocks.0.mystery.weight")


def test_converted_block_keys_load_into_the_block_module(fixture):
    from q8_kernels_b200.blocks import LTXTransformerBlock
    _, outs = fixture
    blk = LTXTransformerBlock(64, 1, 64, 64, bias=True, use_rope=True, norm_affine=False)
    want = {k[len("transformer_blocks.0."):] for k in outs if k.startswith("transformer_blocks.0.")}
    have = set(blk.state_dict().keys())
    assert want == have
    for k in want:
        if k != "scale_shift_table":                       # passes through in the checkpoint's own dtype
            assert blk.state_dict()[k].dtype == outs["transformer_blocks.0." + k].dtype, k
        assert tuple(blk.state_dict()[k].shape) == tuple(outs["transformer_blocks.0." + k].shape), k


@pytest.mark.gpu
def test_convert_state_dict_on_gpu_is_bit_identical_to_the_fixture(fixture, cuda_device):
    from q8_kernels_b200.utils import convert_weights as cw
    ins, outs = fixture
    got = cw.convert_state_dict(ins, device=cuda_device)
    assert set(got) == set(outs)
    for k, ref in outs.items():
        g = got[k].cpu()
        assert g.dtype == ref.dtype and g.shape == ref.shape, k
        if ref.dtype == torch.bfloat16:
            assert torch.equal(g.view(torch.int16), ref.view(torch.int16)), k
        else:
            assert torch.equal(g, ref), k
    # and the converted block runs
    from q8_kernels_b200.blocks import LTXTransformerBlock
    blk = LTXTransformerBlock(64, 1, 64, 64).to(cuda_device)
    sd = {k[len("transformer_blocks.0."):]: v for k, v in got.items() if k.startswith("transformer_blocks.0.")}
    missing, unexpected = blk.load_state_dict(sd, strict=True)
    assert not missing and not unexpected
