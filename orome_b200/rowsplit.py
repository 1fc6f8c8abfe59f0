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
