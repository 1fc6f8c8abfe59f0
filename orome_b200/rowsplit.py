"""Row-split of a weight matrix over the GPUs of one box, and the all-gather of its output.

Output rows of a matvec are independent, so rank r keeps rows [r*per, (r+1)*per) of every
tensor, with `per` a multiple of 32 rows (the reference's 32-row threadgroup tile,
inference/src/format.m:228-238); the last ranks may hold fewer rows, or none.  Every rank
writes its slice of y in place into a buffer of per*world floats and one in-place all-gather
completes the vector on every rank.  x is replicated (it is the previous all-gather's result).
"""
from __future__ import annotations


def rows_per_rank(n: int, world: int) -> int:
    return ((n + world - 1) // world + 31) // 32 * 32


def shard_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) of the rows rank `rank` owns."""
    per = rows_per_rank(n, world)
    lo = min(n, rank * per)
    return lo, min(n, lo + per)


def padded_rows(n: int, world: int) -> int:
    """Length of the gather buffer: equal slices for every rank, >= n."""
    return rows_per_rank(n, world) * world


def all_gather_rows(dist, buf, n: int, rank: int, world: int, group=None) -> None:
    """In-place all-gather of a row-split output vector.

    `buf` has padded_rows(n, world) elements; this rank has already written its slice
    buf[rank*per : rank*per + (hi-lo)].  After the call buf[:n] is the full vector on every rank."""
    if world == 1:
        return
    per = rows_per_rank(n, world)
    dist.all_gather_into_tensor(buf, buf[rank * per:(rank + 1) * per], group=group)


def shard_experts(n_experts: int, rank: int, world: int) -> tuple[int, int]:
    """[first, last) experts of this rank for expert-parallel MoE: contiguous blocks, expert e lives on rank
    e // ceil(n_experts / world) (16 per GPU for 128 experts on 8 GPUs)."""
    per = -(-n_experts // world)
    first = min(rank * per, n_experts)
    return first, min(first + per, n_experts)


def expert_owner(e: int, n_experts: int, world: int) -> int:
    return e // (-(-n_experts // world))


def all_reduce_sum(dist, buf, group=None) -> None:
    """Combine step of the expert-parallel FFN: every rank holds the sum over ITS experts, the layer output is the
    sum over ranks (activations and routing are replicated, so there is no dispatch step)."""
    dist.all_reduce(buf, group=group)


class _DeviceMemory:
    """Raw device memory exposed through __cuda_array_interface__ so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class PeerArena:
    """Gather arena of the fused all-gather: one allocation per rank that every other rank maps (CUDA IPC).

    Buffers are carved out at equal offsets on every rank, so a kernel that produces rows [lo, hi) of a vector can
    store them straight into the same place of every peer's arena.  `dist` (any backend, gloo is enough) is only used
    to hand the 64-byte IPC handles around."""

    def __init__(self, ctx, dist, rank: int, world: int, data_bytes: int, n_flags: int):
        import torch
        from . import format as F
        self.ctx, self.rank, self.world = ctx, rank, world
        self.data_bytes = (data_bytes + 255) // 256 * 256
        self.total = F.gather_arena_bytes(self.data_bytes, n_flags)
        self.ptr, handle = ctx.peer_alloc(self.total)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        self.ptrs = [self.ptr if r == rank else ctx.peer_open(handles[r]) for r in range(world)]
        dist.barrier()
        ctx.gather_setup(rank, world, self.ptrs, self.data_bytes, n_flags)
        self._mem = torch.as_tensor(_DeviceMemory(self.ptr, self.data_bytes), device=f"cuda:{ctx.device}")
        self._off = 0

    def floats(self, n: int):
        """A zeroed fp32 buffer of n elements inside the arena (same offset on every rank)."""
        import torch
        nbytes = (n * 4 + 255) // 256 * 256
        if self._off + nbytes > self.data_bytes:
            raise MemoryError("gather arena exhausted")
        t = self._mem[self._off:self._off + n * 4].view(torch.float32)
        self._off += nbytes
        return t
