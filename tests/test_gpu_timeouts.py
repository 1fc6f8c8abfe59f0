"""Bounded device-side waits: a wait that nothing will ever satisfy must run out, leave a status code the host
can read, and leave the context usable.  The missing party is made on the host side: one process sets the gather
state up for two ranks whose arenas both live on this GPU and simply never runs the second rank, so a wait for
the second rank's data can only expire.  Nothing here faults, traps or hangs the GPU: the waits are given a
bound of a millisecond (OROME_OPT_WAIT_US) and the kernels return by themselves."""
import time

import numpy as np
import pytest

import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture()
def two_rank_ctx():
    import torch
    from orome_b200 import format as F
    ctx = F.Context(0)
    data_bytes = 64 * 1024
    total = F.gather_arena_bytes(data_bytes, 4)
    mine, _ = ctx.peer_alloc(total)
    other, _ = ctx.peer_alloc(total)                  # the arena of a rank that never runs
    ctx.gather_setup(0, 2, [mine, other], data_bytes, 4)
    ctx.set_option(F.OPT_WAIT_US, 1000)
    arena = torch.as_tensor(_Mem(mine, data_bytes), device="cuda:0").view(torch.float32)
    yield torch, F, ctx, arena
    torch.cuda.synchronize()
    ctx.set_option(F.OPT_WAIT_US, 0)
    ctx.gather_setup(0, 1, None, 0, 0)
    ctx.free(mine)
    ctx.free(other)
    ctx.close()


class _Mem:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_gather_wait_on_a_vector_nobody_publishes_expires(two_rank_ctx):
    torch, F, ctx, arena = two_rank_ctx
    fmt, n = synth.Q8_0, 256
    data = synth.host_tensor(fmt, n, n, seed=1)
    wt, xt = dev(torch, data), dev(torch, synth.host_x(n, seed=2))
    y, z = arena[:n], arena[1024:1024 + n]
    ref = F.tensor_ref(wt.data_ptr(), 0, fmt, n, n)
    # generation 1 of flag 0: this rank publishes its rows (the "peer" arena is on the same GPU and takes them too)
    ctx.gather_next(-1, 0)
    ctx.matvec(ref, xt.data_ptr(), y.data_ptr())
    torch.cuda.synchronize()
    assert ctx.status() == 0
    # nobody ever stored z under that flag: the wait can only run out
    t0 = time.perf_counter()
    ctx.gather_wait(0, z.data_ptr(), n)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    with pytest.raises(F.OromeError) as e:
        ctx.status()
    assert e.value.code == F.ETIMEOUT and "status 3" in str(e.value)
    # reported once, then the context is clean and usable again
    assert ctx.status() == 0
    ctx.gather_wait(0, y.data_ptr(), n)               # y WAS published: this wait is satisfied at once
    torch.cuda.synchronize()
    assert ctx.status() == 0
    want = oracle.matvec_f64(fmt, data, n, n, synth.host_x(n, seed=2))
    assert np.linalg.norm(y.cpu().numpy() - want) / np.linalg.norm(want) <= 2e-6


def test_chain_whose_peer_never_runs_expires_once_and_stays_usable(two_rank_ctx):
    torch, F, ctx, arena = two_rank_ctx
    fmt, n = synth.Q8_0, 256
    d1, d2 = synth.host_tensor(fmt, n // 2, n, seed=3), synth.host_tensor(fmt, n, n, seed=4)
    w1, w2, xt = dev(torch, d1), dev(torch, d2), dev(torch, synth.host_x(n, seed=5))
    y1, y2, y3 = arena[:n], arena[2048:2048 + n], arena[4096:4096 + n]
    # rank 0 of 2 holds the first half of W1's rows; the second product reads the whole vector, whose other half only
    # the absent rank could write
    ctx.chain_begin()
    ctx.matvec(F.tensor_ref(w1.data_ptr(), 0, fmt, n // 2, n), xt.data_ptr(), y1[:n // 2].data_ptr())
    ctx.matvec(F.tensor_ref(w2.data_ptr(), 0, fmt, n // 2, n), y1.data_ptr(), y2[:n // 2].data_ptr())
    ctx.matvec(F.tensor_ref(w2.data_ptr(), 0, fmt, n // 2, n), y2.data_ptr(), y3[:n // 2].data_ptr())
    ch = ctx.chain_end()
    t0 = time.perf_counter()
    ch.launch()
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    assert first < 2.0                                # every wait is bounded, and expiry is sticky inside the launch
    with pytest.raises(F.OromeError) as e:
        ctx.status()
    assert e.value.code == F.ETIMEOUT
    assert ctx.status() == 0
    # a chain without a missing party runs cleanly on the same context afterwards
    ctx.chain_begin()
    ctx.matvec(F.tensor_ref(w2.data_ptr(), 0, fmt, n, n), xt.data_ptr(), y2.data_ptr())
    ok = ctx.chain_end()
    ok.launch()
    torch.cuda.synchronize()
    assert ctx.status() == 0
    want = oracle.matvec_f64(fmt, d2, n, n, synth.host_x(n, seed=5))
    assert np.linalg.norm(y2.cpu().numpy() - want) / np.linalg.norm(want) <= 2e-6
    ch.close()
    ok.close()


def test_gather_request_is_dropped_by_calls_that_cannot_honour_it(two_rank_ctx):
    torch, F, ctx, arena = two_rank_ctx
    fmt, n = synth.Q6_K, 256
    wt = dev(torch, synth.host_tensor(fmt, n, n, seed=6))
    x8 = dev(torch, synth.host_x(n, 8, seed=7))
    y8 = torch.zeros((8, n), device="cuda")
    ref = F.tensor_ref(wt.data_ptr(), 0, fmt, n, n)
    ctx.gather_next(-1, 1)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, x8.data_ptr(), y8.data_ptr(), 3, n, n)       # batches 2-3 (one decode launch per vector) have no publish path
    assert e.value.code == F.ENOTSUP
    # the request is gone: the next batch-1 launch is a plain local one (y outside the arena would be refused if it published)
    y = torch.zeros(n, device="cuda")
    ctx.matvec(ref, x8.data_ptr(), y.data_ptr())
    torch.cuda.synchronize()
    assert ctx.status() == 0
