"""Row-split of the batched (prefill) product: each rank multiplies its rows of W by the whole X on the tensor
cores, the kernel that writes Y also stores every value into every rank's gather arena, and the next batched
product reads its X out of the arena's slots.

One GPU stands in for two ranks here: two contexts in one process, each with its own arena on this GPU and the
other's arena as its peer.  The launches are strictly ordered (both ranks publish a matrix before anybody reads
it), so no kernel ever waits for a kernel that has not run yet.  The two-process form is in test_multi_gpu.py."""
import numpy as np
import pytest

import oracle
from orome_b200 import rowsplit, synth

pytestmark = pytest.mark.gpu

TC_TOL = 5e-4          # fp16 weights and activations in the tensor-core form


class _Mem:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def rel_l2(got, want):
    want = np.asarray(want, np.float64)
    return float(np.linalg.norm(np.asarray(got, np.float64) - want) / max(np.linalg.norm(want), 1e-300))


@pytest.fixture()
def two_ranks():
    import torch
    from orome_b200 import format as F
    world, data_bytes, flags = 2, 4 << 20, 4
    total = F.gather_arena_bytes(data_bytes, flags)
    ctxs = [F.Context(0) for _ in range(world)]
    ptrs = [ctxs[r].peer_alloc(total)[0] for r in range(world)]
    for r in range(world):
        ctxs[r].gather_setup(r, world, ptrs, data_bytes, flags)
    arenas = [torch.as_tensor(_Mem(ptrs[r], data_bytes), device="cuda:0").view(torch.float32) for r in range(world)]
    yield torch, F, ctxs, arenas
    torch.cuda.synchronize()
    for r in range(world):
        assert ctxs[r].status() == 0
        ctxs[r].gather_setup(r, 1, None, 0, 0)
    for r in range(world):
        ctxs[r].free(ptrs[r])
        ctxs[r].close()


@pytest.mark.parametrize("fmt, n, m, batch", [(synth.Q8_0, 1024, 768, 8), (synth.Q4_K, 1024, 1024, 64), (synth.Q5_K, 512, 1280, 5),
                                               (synth.Q4_K, 4096, 512, 16)])
def test_two_chained_batched_products_row_split(two_ranks, fmt, n, m, batch):
    """Y1 = X W1^T (n columns -> m rows), Y2 = Y1 W2^T (m -> n rows), both row-split over two ranks; the n = 4096
    case is wide enough for the split-K form, whose reduction kernel does the publishing."""
    torch, F, ctxs, arenas = two_ranks
    world = 2
    W1, W2 = synth.host_tensor(fmt, m, n, seed=81), synth.host_tensor(fmt, n, m, seed=82)
    X = synth.host_x(n, batch, seed=83)
    xt = torch.from_numpy(np.ascontiguousarray(X)).cuda()
    mp_, np_ = rowsplit.padded_rows(m, world), rowsplit.padded_rows(n, world)
    shards = []
    for r in range(world):
        lo1, hi1 = rowsplit.shard_rows(m, r, world)
        lo2, hi2 = rowsplit.shard_rows(n, r, world)
        rb1, rb2 = synth.row_bytes(fmt, n), synth.row_bytes(fmt, m)
        shards.append((lo1, hi1, torch.from_numpy(W1[lo1 * rb1:hi1 * rb1].copy()).cuda(), lo2, hi2, torch.from_numpy(W2[lo2 * rb2:hi2 * rb2].copy()).cuda()))
    # Y1 [batch][mp_] at float offset 0 of every arena, Y2 [batch][np_] behind it
    off2 = (batch * mp_ + 63) // 64 * 64
    y1 = [arenas[r][:batch * mp_].view(batch, mp_) for r in range(world)]
    y2 = [arenas[r][off2:off2 + batch * np_].view(batch, np_) for r in range(world)]
    for rep in range(2):                                    # twice: the generations must keep pairing up
        for r in range(world):
            lo1, hi1, w1, _, _, _ = shards[r]
            ctxs[r].gather_next(-1, 0)
            ctxs[r].matvec(F.tensor_ref(w1.data_ptr(), 0, fmt, hi1 - lo1, n), xt.data_ptr(), y1[r][:, lo1:].data_ptr(), batch, n, mp_)
        torch.cuda.synchronize()
        for r in range(world):
            _, _, _, lo2, hi2, w2 = shards[r]
            ctxs[r].gather_next(0, 1)
            ctxs[r].matvec(F.tensor_ref(w2.data_ptr(), 0, fmt, hi2 - lo2, m), y1[r].data_ptr(), y2[r][:, lo2:].data_ptr(), batch, mp_, np_)
        torch.cuda.synchronize()
    for r in range(world):
        assert ctxs[r].status() == 0
        for b in range(batch):                              # complete the plain copies from the slots
            ctxs[r].gather_wait(0, y1[r][b].data_ptr(), m)
            ctxs[r].gather_wait(1, y2[r][b].data_ptr(), n)
    torch.cuda.synchronize()
    want1 = oracle.matvec_f64(fmt, W1, m, n, X)
    for r in range(world):
        got1 = y1[r][:, :m].cpu().numpy()
        assert rel_l2(got1, want1) <= TC_TOL
        want2 = oracle.matvec_f64(fmt, W2, n, m, got1)      # fed the GPU's own intermediate
        assert rel_l2(y2[r][:, :n].cpu().numpy(), want2) <= TC_TOL
    assert np.array_equal(y2[0].cpu().numpy()[:, :n], y2[1].cpu().numpy()[:, :n])       # both ranks hold the same matrix


def test_requests_the_batched_form_cannot_honour(two_ranks):
    torch, F, ctxs, arenas = two_ranks
    ctx, fmt, n = ctxs[0], synth.Q8_0, 512
    w = torch.from_numpy(synth.host_tensor(fmt, n, n, seed=91)).cuda()
    ref = F.tensor_ref(w.data_ptr(), 0, fmt, n, n)
    x = torch.zeros((80, n), device="cuda")
    outside = torch.zeros((8, n), device="cuda")
    ctx.gather_next(-1, 0)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, x.data_ptr(), outside.data_ptr(), 8, n, n)             # Y outside the arena
    assert e.value.code == F.EINVAL
    ctx.gather_next(0, -1)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, x.data_ptr(), arenas[0].data_ptr(), 8, n, n)           # X outside the arena
    assert e.value.code == F.EINVAL
    ctx.gather_next(-1, 0)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, x.data_ptr(), arenas[0].data_ptr(), 80, n, n)          # more than one launch's worth of vectors
    assert e.value.code == F.ENOTSUP
    ctx.matvec(ref, x.data_ptr(), outside.data_ptr(), 8, n, n)                 # every refusal dropped the request
    torch.cuda.synchronize()
    assert ctx.status() == 0
