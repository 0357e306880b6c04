"""Multi-GPU sharding of the DiT path: one process per GPU, ``torch.distributed``
(NCCL over NVLink on GPUs, gloo on CPU for tests).

Two ways the path shards, neither with a collective inside the hot loops:

* by video: each rank runs the whole stack on its own videos; one
  ``all_gather_into_tensor`` of the final latents at the end;
* by attention head: linears, q/k RMSNorm (it spans all heads) and RoPE run
  replicated, each rank computes attention for H/world heads and the per-rank
  channel slices are all-gathered before ``to_out`` (one collective per
  self-attention).

The reference has no multi-GPU code; this module is new host-side logic.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def video_shard(num_videos: int, rank: int, world: int) -> range:
    """Contiguous block of video indices owned by ``rank`` (sizes differ by at most one)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(num_videos, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def head_shard(num_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """(rank, world) pair accepted by ``Attention.forward(head_shard=...)`` after checking divisibility."""
    if num_heads % world != 0:
        raise ValueError(f"{num_heads} heads do not divide over {world} ranks")
    if not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world {world}")
    return rank, world


def head_slice(num_heads: int, rank: int, world: int) -> slice:
    head_shard(num_heads, rank, world)
    per = num_heads // world
    return slice(rank * per, (rank + 1) * per)


def gather_heads(x_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """[B, S, C/world] per rank -> [B, S, C] on every rank, channel blocks in rank order."""
    world = dist.get_world_size(group)
    if world == 1:
        return x_local
    x_local = x_local.contiguous()
    B, S, c = x_local.shape
    buf = torch.empty((world * B, S, c), dtype=x_local.dtype, device=x_local.device)   # rank blocks along dim 0
    if x_local.dtype == torch.float8_e4m3fn:                    # collectives move bytes
        dist.all_gather_into_tensor(buf.view(torch.uint8), x_local.view(torch.uint8), group=group)
    else:
        dist.all_gather_into_tensor(buf, x_local, group=group)
    # [world, B, S, c] -> [B, S, world, c] -> [B, S, C]
    return buf.view(world, B, S, c).permute(1, 2, 0, 3).reshape(B, S, world * c)


def gather_videos(x_local: torch.Tensor, counts: List[int], group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Final gather of the by-video sharding: per-rank [n_r, ...] -> [sum n_r, ...] on every rank."""
    world = dist.get_world_size(group)
    if world == 1:
        return x_local
    if len(set(counts)) == 1:
        out = torch.empty((sum(counts),) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=x_local.device)
        dist.all_gather_into_tensor(out, x_local.contiguous(), group=group)
        return out
    # uneven split: pad every rank to the largest share, gather once, drop the padding
    most = max(counts)
    padded = torch.zeros((most,) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=x_local.device)
    padded[: x_local.shape[0]] = x_local
    out = torch.empty((world * most,) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=x_local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * most: r * most + n] for r, n in enumerate(counts)], dim=0)


class PeerBuffers:
    """Gather-free head sharding: a device buffer on every rank that all the other ranks of the node
    can store into.

    Each rank allocates ``2 * nbytes`` bytes, exports the allocation with CUDA IPC and maps every
    other rank's into its own process (peer access over NVLink comes with the mapping).  The
    attention kernel of a rank then stores its heads of the output into the same place of EVERY
    rank's buffer (``native.flash_attention_into``), and after ``barrier()`` -- a one-element NCCL
    all-reduce on the current stream, which no rank leaves before all have entered, i.e. before all
    their attention kernels have finished -- every rank holds the complete output.  The two halves
    alternate from call to call: a rank that is already writing the next attention output cannot
    touch the half a slower peer is still reading, because it cannot get two calls ahead without that
    peer having passed the barrier in between.

    Nothing here reads from a peer, and no kernel waits on a peer: the only cross-rank wait is the
    NCCL collective, which has the process group's timeout.

    The exported buffer must be a plain ``cudaMalloc`` segment of torch's caching allocator (CUDA IPC
    cannot export ``expandable_segments`` memory; the export then fails at construction).  ``close()``
    is collective; the object is a context manager so that it also runs when the body raises.

    Checked bit-for-bit against the replicated result on 2 and on 8 GPUs in loops of 100-160 back-to-back
    calls without host synchronisation (8 GPUs: 3200 rank-calls, each comparing the whole assembled
    buffer on the device, no differing byte; repeated after every change of the kernel's epilogue).  ``MAX_WORLD`` is the number of destinations one attention
    launch can store to.
    """

    MAX_WORLD = 8

    def __init__(self, nbytes: int, device, group: Optional[dist.ProcessGroup] = None):
        import ctypes
        from ._lib import check, lib
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > self.MAX_WORLD:
            raise ValueError(f"PeerBuffers serves up to {self.MAX_WORLD} ranks of one node, got {self.world}: "
                             "use gather_heads (NCCL all-gather) instead")
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.device = torch.device(device)
        self._store = torch.empty(2 * self.nbytes, dtype=torch.uint8, device=self.device)
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._turn = 0
        self._opened = []
        self._closed = False
        handle = (ctypes.c_ubyte * 64)()
        offset = ctypes.c_int64(0)
        with torch.cuda.device(self.device):
            check(lib.q8k_ipc_export(ctypes.c_void_p(self._store.data_ptr()), ctypes.cast(handle, ctypes.c_void_p),
                                     ctypes.cast(ctypes.pointer(offset), ctypes.c_void_p)), "ipc_export")
            mine = (bytes(handle), int(offset.value))
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            self._base = []
            for r, (h, off) in enumerate(everyone):
                if r == self.rank:
                    self._base.append(self._store.data_ptr())
                    continue
                hbuf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                p = ctypes.c_void_p(0)
                check(lib.q8k_ipc_open(ctypes.cast(hbuf, ctypes.c_void_p), off,
                                       ctypes.cast(ctypes.pointer(p), ctypes.c_void_p)), "ipc_open")
                self._opened.append((p.value, off))
                self._base.append(p.value)
        dist.barrier(group=group)                               # every mapping exists before anyone stores

    def __enter__(self) -> "PeerBuffers":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        self.close()

    def next(self, nbytes: int) -> Tuple[torch.Tensor, List[int]]:
        """This call's half: (local uint8 view of ``nbytes`` bytes, its address on every rank, by rank)."""
        if self._closed:
            raise RuntimeError("PeerBuffers.next() after close()")
        if nbytes > self.nbytes:
            raise ValueError(f"peer buffers hold {self.nbytes} bytes per call, {nbytes} asked for")
        half = self._turn * self.nbytes
        self._turn ^= 1
        return self._store[half: half + nbytes], [b + half for b in self._base]

    def barrier(self) -> None:
        dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        """Collective: every rank calls it.  The local buffer stays alive until every rank has passed
        the barrier, i.e. until no peer can still store into it; use the object as a context manager so
        that this also happens on an exception."""
        from ._lib import check, lib
        import ctypes
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                          # nobody unmaps while a peer may still store
        with torch.cuda.device(self.device):
            for addr, off in self._opened:
                check(lib.q8k_ipc_close(ctypes.c_void_p(addr), off), "ipc_close")
        self._opened = []
        dist.barrier(group=self.group)                          # every mapping of this rank's buffer is gone
        self._store = None
