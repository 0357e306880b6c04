"""Two-GPU checks of the sharded paths (skipped on a single-GPU box): attention sharded by head
with an NCCL all-gather of the channel slices equals the unsharded module, and the by-video
sharding gathers the per-rank results in order.  One process per GPU, spawned from the test."""
import os
import socket

import pytest
import torch

import helpers as Hp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import q8_kernels_b200 as q8
        from q8_kernels_b200 import sharding
        cfg = q8.blocks.LTXStackConfig(num_layers=1, num_attention_heads=8, attention_head_dim=64,
                                       cross_attention_dim=512, caption_channels=64)
        stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=3, device=dev)     # same seed: replicated weights
        blk = stack.transformer_blocks[0]
        g = torch.Generator().manual_seed(5)
        S, T = 4 * 4 * 8, 32
        x = torch.randn(2, S, 512, generator=g).to(torch.bfloat16).to(dev)
        text = torch.randn(2, T, 512, generator=g).to(torch.bfloat16).to(dev)
        ts = (torch.randn(2, 1, 6 * 512, generator=g) * 0.1).to(torch.bfloat16).to(dev)
        freqs = stack.freqs_cis(q8.blocks.latent_grid(4, 4, 8, device=dev))
        lens = torch.tensor([20, 32], dtype=torch.int32, device=dev)
        with torch.no_grad():
            full = blk(x, freqs, None, text, lens, ts, attn_type="q8_kernels")
            shard = blk(x, freqs, None, text, lens, ts, attn_type="q8_kernels",
                        head_shard=sharding.head_shard(8, rank, world), gather_heads=sharding.gather_heads)
            ok_heads = torch.equal(full, shard)            # same kernels on the same heads: identical bits
            # the same with the attention kernel storing its heads straight into every rank's buffer
            peers = sharding.PeerBuffers(2 * S * 512, dev)
            for _ in range(3):                             # both halves of the buffers, and reuse
                direct = blk(x, freqs, None, text, lens, ts, attn_type="q8_kernels",
                             head_shard=sharding.head_shard(8, rank, world), peer_buffers=peers)
                ok_heads = ok_heads and torch.equal(full, direct)
            peers.close()
            # by video: each rank runs its own video, final gather restores the batch
            mine = list(sharding.video_shard(2, rank, world))
            local = blk(x[mine], freqs, None, text[mine], lens[mine], ts[mine], attn_type="q8_kernels")
            gathered = sharding.gather_videos(local, [1, 1])
            ok_video = torch.equal(gathered, full)
        q8._lib.check_status(dev)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(f"{ok_heads} {ok_video}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_head_and_video_sharding_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "True True", f"rank {r}"
