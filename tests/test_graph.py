"""CUDA-graph wrapper (q8_kernels_b200/graph.py): argument signatures on the CPU, capture / replay
of a block on the GPU."""
import dataclasses

import pytest
import torch


def test_hash_arg_signatures():
    from q8_kernels_b200.graph import hash_arg
    a, b = torch.zeros(2, 3), torch.ones(2, 3)
    assert hash_arg(a) == hash_arg(b)                          # same device / dtype / shape
    assert hash_arg(a) != hash_arg(a.to(torch.bfloat16))
    assert hash_arg(a) != hash_arg(torch.zeros(3, 2))
    assert hash_arg(torch.tensor(3)) != hash_arg(torch.tensor(4))   # one-element CPU tensors count by value
    assert hash_arg((a, 1, "x", None)) == hash_arg([b, 1, "x", None])
    assert hash_arg({"k": a, "j": 2.0}) == hash_arg({"j": 2.0, "k": b})
    assert hash_arg(object()) is object

    @dataclasses.dataclass
    class Box:
        t: torch.Tensor
        n: int
    assert hash_arg(Box(a, 1)) == hash_arg(Box(b, 1)) != hash_arg(Box(b, 2))


def test_graphed_needs_a_cuda_tensor():
    from q8_kernels_b200.graph import graphed
    with pytest.raises(RuntimeError):
        graphed(lambda x: x + 1)(torch.zeros(4))


@pytest.mark.gpu
def test_graphed_block_replays_bit_identically_and_per_signature(cuda_device):
    import q8_kernels_b200 as q8
    from q8_kernels_b200.graph import graphed
    cfg = q8.blocks.LTXStackConfig(num_layers=1)
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=3, device=cuda_device)
    blk = stack.transformer_blocks[0]
    g = torch.Generator(device=cuda_device).manual_seed(5)

    def inputs(S):
        x = torch.randn(1, S, cfg.inner_dim, generator=g, device=cuda_device).to(torch.bfloat16)
        text = torch.randn(1, 64, cfg.inner_dim, generator=g, device=cuda_device).to(torch.bfloat16)
        ts = (torch.randn(1, 1, 6 * cfg.inner_dim, generator=g, device=cuda_device) * 0.1).to(torch.bfloat16)
        freqs = stack.freqs_cis(q8.blocks.latent_grid(S // 96, 8, 12, device=cuda_device))
        lens = torch.tensor([40], dtype=torch.int32, device=cuda_device)
        return x, freqs, None, text, lens, ts

    fn = graphed(lambda *a: blk(*a, attn_type="q8_kernels"))
    with torch.no_grad():
        for S in (192, 384, 192):
            for _ in range(2):                                 # new values, same signature: replay
                args = inputs(S)
                want = blk(*args, attn_type="q8_kernels")
                got = fn(*args)
                assert torch.equal(got, want)
    assert fn.num_graphs == 2
    q8._lib.check_status(cuda_device)


@pytest.mark.gpu
def test_apply_auto_graph_wraps_selected_modules(cuda_device):
    import q8_kernels_b200 as q8
    from q8_kernels_b200.graph import GraphedCallable, apply_auto_graph
    from q8_kernels_b200.blocks import LTXTransformerBlock
    cfg = q8.blocks.LTXStackConfig(num_layers=2)
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=4, device=cuda_device)
    g = torch.Generator(device=cuda_device).manual_seed(6)
    S = 192
    x = torch.randn(1, S, cfg.inner_dim, generator=g, device=cuda_device).to(torch.bfloat16)
    text = torch.randn(1, 32, cfg.caption_channels, generator=g, device=cuda_device).to(torch.bfloat16)
    ts = (torch.randn(1, 1, 6 * cfg.inner_dim, generator=g, device=cuda_device) * 0.1).to(torch.bfloat16)
    grid = q8.blocks.latent_grid(2, 8, 12, device=cuda_device)
    lens = torch.tensor([20], dtype=torch.int32, device=cuda_device)
    with torch.no_grad():
        want = stack(x, grid, text, lens, ts, attn_type="q8_kernels").clone()
        apply_auto_graph(stack, filter_func=lambda m: isinstance(m, LTXTransformerBlock))
        assert all(isinstance(b.forward, GraphedCallable) for b in stack.transformer_blocks)
        for _ in range(2):
            got = stack(x, grid, text, lens, ts, attn_type="q8_kernels")
            assert torch.equal(got, want)
