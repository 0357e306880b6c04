"""Host-side multi-GPU logic on CPU: shard maps, and gloo world_size-2 runs of the
head gather and the final video gather (spawned child processes, 127.0.0.1)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers as Hp  # noqa: F401  (sets sys.path)


def test_shard_maps_partition_exactly():
    from q8_kernels_b200 import sharding
    for n, world in [(8, 8), (8, 3), (1, 2), (5, 4), (0, 2)]:
        seen = []
        for r in range(world):
            seen += list(sharding.video_shard(n, r, world))
        assert seen == list(range(n))
    assert sharding.head_slice(32, 3, 8) == slice(12, 16)
    with pytest.raises(ValueError):
        sharding.head_shard(32, 0, 5)
    with pytest.raises(ValueError):
        sharding.video_shard(4, 2, 2)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank: int, world: int, port: int, out_path: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from q8_kernels_b200 import sharding
        B, S, H, D = 2, 12, 4, 8
        g = torch.Generator().manual_seed(7)
        q, k, v = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
        full = torch.nn.functional.scaled_dot_product_attention(q, k, v)
        full = full.transpose(1, 2).reshape(B, S, H * D)
        sl = sharding.head_slice(H, rank, world)
        local = torch.nn.functional.scaled_dot_product_attention(q[:, sl], k[:, sl], v[:, sl])
        local = local.transpose(1, 2).reshape(B, S, -1)
        got = sharding.gather_heads(local)
        ok_heads = torch.equal(got, full)
        # byte-typed gather (e4m3 activations travel as uint8)
        x8 = torch.randn(B, S, 16, generator=g).to(torch.float8_e4m3fn)
        per = 16 // world
        g8 = sharding.gather_heads(x8[..., rank * per:(rank + 1) * per])
        ok_fp8 = torch.equal(g8.view(torch.uint8), x8.view(torch.uint8))
        # by-video sharding with an uneven split
        vids = torch.arange(3 * 5, dtype=torch.float32).reshape(3, 5)
        counts = [len(sharding.video_shard(3, r, world)) for r in range(world)]
        mine = vids[list(sharding.video_shard(3, rank, world))]
        ok_vid = torch.equal(sharding.gather_videos(mine, counts), vids)
        even = torch.arange(4 * 5, dtype=torch.float32).reshape(4, 5)
        mine = even[list(sharding.video_shard(4, rank, world))]
        ok_vid = ok_vid and torch.equal(sharding.gather_videos(mine, [2, 2]), even)
        if rank == 0:
            with open(out_path, "w") as f:
                f.write(f"{ok_heads} {ok_fp8} {ok_vid}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_gloo_world2_gathers(tmp_path):
    out = str(tmp_path / "result.txt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read() == "True True True"
