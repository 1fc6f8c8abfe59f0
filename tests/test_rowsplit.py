"""Row-split + all-gather on CPU: two gloo ranks each produce their slice of y (with the
CPU oracle standing in for the kernel) and the in-place gather must reproduce the full product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from orome_b200 import rowsplit, synth


def test_shard_rows_cover_every_row_once():
    for n in (1, 31, 32, 33, 100, 1024, 4096, 151936):
        for world in (1, 2, 3, 4, 8):
            per = rowsplit.rows_per_rank(n, world)
            assert per % 32 == 0 and per * world >= n
            covered = []
            for r in range(world):
                lo, hi = rowsplit.shard_rows(n, r, world)
                assert 0 <= lo <= hi <= n and (lo % 32 == 0 or lo == n)
                covered += list(range(lo, hi))
            assert covered == list(range(n))
            assert rowsplit.padded_rows(n, world) == per * world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fmt, out_dim, in_dim, q):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        data = synth.host_tensor(fmt, out_dim, in_dim, seed=5)          # every rank derives the same full tensor
        x = synth.host_x(in_dim, seed=6)
        rb = synth.row_bytes(fmt, in_dim)
        lo, hi = rowsplit.shard_rows(out_dim, rank, world)
        buf = torch.full((rowsplit.padded_rows(out_dim, world),), float("nan"))
        if hi > lo:
            mine = oracle.matvec_f32(fmt, data[lo * rb:hi * rb], hi - lo, in_dim, x)
            buf[lo:hi] = torch.from_numpy(mine)
        rowsplit.all_gather_rows(dist, buf, out_dim, rank, world)
        full = oracle.matvec_f32(fmt, data, out_dim, in_dim, x)
        ok = bool(np.array_equal(buf[:out_dim].numpy().view(np.uint32), full.view(np.uint32)))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt,out_dim,in_dim,world", [(synth.Q8_0, 256, 512, 2), (synth.Q4_K, 100, 512, 2), (synth.Q6_K, 40, 256, 2)])
def test_two_gloo_ranks_reassemble_the_product(fmt, out_dim, in_dim, world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fmt, out_dim, in_dim, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {r: True for r in range(world)}


def test_shard_experts_covers_every_expert_once():
    from orome_b200 import rowsplit
    for n, world in ((128, 8), (128, 3), (16, 4), (5, 8), (256, 2)):
        seen = []
        for r in range(world):
            lo, hi = rowsplit.shard_experts(n, r, world)
            assert 0 <= lo <= hi <= n
            seen += list(range(lo, hi))
            assert all(rowsplit.expert_owner(e, n, world) == r for e in range(lo, hi))
        assert seen == list(range(n))
    assert rowsplit.shard_experts(128, 0, 8) == (0, 16) and rowsplit.shard_experts(128, 7, 8) == (112, 128)
