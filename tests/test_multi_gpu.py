"""Row-split products with the fused peer all-gather on two and four GPUs (one process per GPU): two chained matvecs whose
intermediate vector only exists once both ranks have stored their slices into each other's arena."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from orome_b200 import rowsplit, synth

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(target, world, extra=()):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, *extra, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in results), results


def _worker(rank, world, port, fmt, n, q):
    import torch.distributed as dist
    import oracle
    from orome_b200 import format as F
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok, err = False, ""
    try:
        ctx = F.Context(rank)
        W1 = synth.host_tensor(fmt, n, n, seed=71)
        W2 = synth.host_tensor(fmt, n, n, seed=72)
        x = synth.host_x(n, seed=73)
        rb = synth.row_bytes(fmt, n)
        lo, hi = rowsplit.shard_rows(n, rank, world)
        npad = rowsplit.padded_rows(n, world)
        arena = rowsplit.PeerArena(ctx, dist, rank, world, 2 * (npad * 4 + 256), 2)
        y1, y2 = arena.floats(npad), arena.floats(npad)
        w1 = torch.from_numpy(W1[lo * rb:hi * rb].copy()).cuda()
        w2 = torch.from_numpy(W2[lo * rb:hi * rb].copy()).cuda()
        xt = torch.from_numpy(x).cuda()
        st = torch.cuda.current_stream().cuda_stream
        r1 = F.tensor_ref(w1.data_ptr(), 0, fmt, hi - lo, n)
        r2 = F.tensor_ref(w2.data_ptr(), 0, fmt, hi - lo, n)
        for rep in range(3):                                  # several rounds: the generations must keep pairing up
            ctx.gather_next(-1, 0)
            ctx.matvec(r1, xt.data_ptr(), y1[lo:hi].data_ptr(), 1, 0, 0, st)
            ctx.gather_next(0, 1)
            ctx.matvec(r2, y1.data_ptr(), y2[lo:hi].data_ptr(), 1, 0, 0, st)
            ctx.gather_wait(0, y1.data_ptr(), n, st)      # plain copies for the host-side check below
            ctx.gather_wait(1, y2.data_ptr(), n, st)
            torch.cuda.synchronize()
            dist.barrier()
        want1 = oracle.matvec_f64(fmt, W1, n, n, x)
        want2 = oracle.matvec_f64(fmt, W2, n, n, want1.astype(np.float32))
        got1, got2 = y1[:n].cpu().numpy(), y2[:n].cpu().numpy()
        e1 = np.linalg.norm(got1 - want1) / np.linalg.norm(want1)
        e2 = np.linalg.norm(got2 - want2) / np.linalg.norm(want2)
        ok = bool(e1 <= 1e-4 and e2 <= 1e-4 and ctx.status() == 0)
        err = f"e1={e1:.2e} e2={e2:.2e}"
    except Exception as ex:   # report instead of leaving the peer waiting on a barrier
        err = repr(ex)
    q.put((rank, ok, err))
    try:
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _ep_worker(rank, world, port, q):
    """Expert-parallel MoE layer: each rank holds half of the experts, computes its share, the shares are summed."""
    import torch.distributed as dist
    import oracle
    from orome_b200 import format as F
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok, err = False, ""
    try:
        ctx = F.Context(rank)
        H, M, E, K, T, dfmt = 512, 256, 16, 8, 2, synth.Q5_K
        gate = synth.host_tensor(synth.Q4_K, E * M, H, seed=81)
        up = synth.host_tensor(synth.Q4_K, E * M, H, seed=82)
        down = synth.host_tensor(dfmt, E * H, M, seed=83)
        router = synth.host_router(E, H, seed=84)
        sg, sd = synth.tensor_bytes(synth.Q4_K, M, H), synth.tensor_bytes(dfmt, H, M)
        xm = np.atleast_2d(synth.host_x(H, T, seed=85))
        e0, e1 = rowsplit.shard_experts(E, rank, world)
        n = e1 - e0
        wt = torch.from_numpy(np.concatenate([gate[e0 * sg:e1 * sg], up[e0 * sg:e1 * sg], down[e0 * sd:e1 * sd]])).cuda()
        layer = F.ExpertLayerRef(wt.data_ptr(), F.ExpertProjRef(0, sg, synth.Q4_K), F.ExpertProjRef(n * sg, sg, synth.Q4_K),
                                 F.ExpertProjRef(2 * n * sg, sd, dfmt))
        rt = torch.from_numpy(router).cuda()
        xt = torch.from_numpy(xm).cuda()
        idx = torch.zeros((T, 8), dtype=torch.int32, device="cuda")
        w = torch.zeros((T, 8), device="cuda")
        loc = torch.zeros((T, 8), dtype=torch.int32, device="cuda")
        act = torch.empty((T, K, M), device="cuda")
        out = torch.full((T, H), float("nan"), device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        # routing is replicated: every rank computes the same top-K from the same x
        ctx.moe_route(F.tensor_ref(rt.data_ptr(), 0, synth.F32, E, H), xt.data_ptr(), T, H, K, idx.data_ptr(), w.data_ptr(), 0, st)
        ctx.moe_ffn_shard(layer, 0, xt.data_ptr(), T, H, idx.data_ptr(), w.data_ptr(), K, H, M, e0, n, loc.data_ptr(), act.data_ptr(),
                          out.data_ptr(), H, st)
        torch.cuda.synchronize()
        total = out.cpu()
        rowsplit.all_reduce_sum(dist, total)
        got = total.numpy()
        worst = 0.0
        gi, gw = idx.cpu().numpy().view(np.uint32), w.cpu().numpy()      # the routing itself is covered by the single-GPU tests
        for t in range(T):
            want = oracle.moe_ffn_f64(gate, up, down, (synth.Q4_K, synth.Q4_K, dfmt), (sg, sg, sd), xm[t], H, M, gi[t], gw[t])
            worst = max(worst, float(np.linalg.norm(got[t] - want) / np.linalg.norm(want)))
        ok = bool(worst <= 1e-4 and ctx.status() == 0)
        err = f"worst={worst:.2e}"
    except Exception as ex:
        err = repr(ex)
    q.put((rank, ok, err))
    try:
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_moe(world):
    _run_ranks(_ep_worker, world)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K])
def test_fused_gather(fmt, world):
    _run_ranks(_worker, world, (fmt, 1024))


def _chain_worker(rank, world, port, q):
    """A recorded chain on row-split tensors: W1 x -> fused gate/up -> W3 act, every vector completed on both GPUs by
    the producing product's peer stores, the last one copied to its plain place inside the chain (gather_wait)."""
    import torch.distributed as dist
    import oracle
    from orome_b200 import format as F
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok, err = False, ""
    try:
        ctx = F.Context(rank)
        fmt, n, m = synth.Q8_0, 1024, 2048
        W1 = synth.host_tensor(fmt, n, n, seed=91)
        Wg, Wu = synth.host_tensor(fmt, m, n, seed=92), synth.host_tensor(fmt, m, n, seed=93)
        W3 = synth.host_tensor(fmt, n, m, seed=94)
        rbn, rbm = synth.row_bytes(fmt, n), synth.row_bytes(fmt, m)
        lo, hi = rowsplit.shard_rows(n, rank, world)
        lom, him = rowsplit.shard_rows(m, rank, world)
        npad, mpad = rowsplit.padded_rows(n, world), rowsplit.padded_rows(m, world)
        arena = rowsplit.PeerArena(ctx, dist, rank, world, 2 * (npad * 4 + 256) + (mpad * 4 + 256), 1)
        y1, act, y3 = arena.floats(npad), arena.floats(mpad), arena.floats(npad)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        w1, wg, wu, w3 = dev(W1[lo * rbn:hi * rbn]), dev(Wg[lom * rbn:him * rbn]), dev(Wu[lom * rbn:him * rbn]), dev(W3[lo * rbm:hi * rbm])
        xt = torch.zeros(n, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        ctx.chain_begin()
        ctx.matvec(F.tensor_ref(w1.data_ptr(), 0, fmt, hi - lo, n), xt.data_ptr(), y1[lo:hi].data_ptr())
        ctx.gate_up_swiglu(F.tensor_ref(wg.data_ptr(), 0, fmt, him - lom, n), F.tensor_ref(wu.data_ptr(), 0, fmt, him - lom, n),
                           y1.data_ptr(), act[lom:him].data_ptr())
        ctx.matvec(F.tensor_ref(w3.data_ptr(), 0, fmt, hi - lo, m), act.data_ptr(), y3[lo:hi].data_ptr())
        ctx.gather_wait(0, y3.data_ptr(), n)
        chain = ctx.chain_end()
        assert chain.info()["products"] == 4
        worst = 0.0
        for rep in range(3):                                  # tags of one launch must not satisfy the next
            x = synth.host_x(n, seed=95 + rep) * np.float32(20.0)
            xt.copy_(torch.from_numpy(x))
            chain.launch(st)
            torch.cuda.synchronize()
            dist.barrier()
            a1 = oracle.matvec_f64(fmt, W1, n, n, x).astype(np.float32)
            a2 = oracle.swiglu_f64(oracle.matvec_f64(fmt, Wg, m, n, a1), oracle.matvec_f64(fmt, Wu, m, n, a1)).astype(np.float32)
            want = oracle.matvec_f64(fmt, W3, n, m, a2)
            got = y3[:n].cpu().numpy()
            worst = max(worst, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
            dist.barrier()
        ok = bool(worst <= 1e-5 and ctx.status() == 0)
        err = f"worst={worst:.2e}"
        chain.close()
    except Exception as ex:   # report instead of leaving the peer waiting on a barrier
        err = repr(ex)
    q.put((rank, ok, err))
    try:
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_chain(world):
    _run_ranks(_chain_worker, world)


def _batched_worker(rank, world, port, q):
    """Two chained batched (prefill) products, both row-split: the tensor-core kernel publishes Y, the next one's
    packing kernel reads the gathered X from the arena's slots."""
    import torch.distributed as dist
    import oracle
    from orome_b200 import format as F
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok, err = False, ""
    try:
        ctx = F.Context(rank)
        errs = []
        for fmt, n, m, batch in ((synth.Q8_0, 1024, 768, 8), (synth.Q4_K, 4096, 1024, 64)):
            W1, W2 = synth.host_tensor(fmt, m, n, seed=91), synth.host_tensor(fmt, n, m, seed=92)
            X = synth.host_x(n, batch, seed=93)
            rb1, rb2 = synth.row_bytes(fmt, n), synth.row_bytes(fmt, m)
            lo1, hi1 = rowsplit.shard_rows(m, rank, world)
            lo2, hi2 = rowsplit.shard_rows(n, rank, world)
            mp_, np_ = rowsplit.padded_rows(m, world), rowsplit.padded_rows(n, world)
            arena = rowsplit.PeerArena(ctx, dist, rank, world, (batch * (mp_ + np_) * 4 + 1024), 2)
            y1, y2 = arena.floats(batch * mp_).view(batch, mp_), arena.floats(batch * np_).view(batch, np_)
            w1 = torch.from_numpy(W1[lo1 * rb1:hi1 * rb1].copy()).cuda()
            w2 = torch.from_numpy(W2[lo2 * rb2:hi2 * rb2].copy()).cuda()
            xt = torch.from_numpy(np.ascontiguousarray(X)).cuda()
            st = torch.cuda.current_stream().cuda_stream
            for rep in range(3):
                ctx.gather_next(-1, 0)
                ctx.matvec(F.tensor_ref(w1.data_ptr(), 0, fmt, hi1 - lo1, n), xt.data_ptr(), y1[:, lo1:].data_ptr(), batch, n, mp_, st)
                ctx.gather_next(0, 1)
                ctx.matvec(F.tensor_ref(w2.data_ptr(), 0, fmt, hi2 - lo2, m), y1.data_ptr(), y2[:, lo2:].data_ptr(), batch, mp_, np_, st)
                for b in range(batch):
                    ctx.gather_wait(0, y1[b].data_ptr(), m, st)
                    ctx.gather_wait(1, y2[b].data_ptr(), n, st)
                torch.cuda.synchronize()
                dist.barrier()
            want1 = oracle.matvec_f64(fmt, W1, m, n, X)
            got1 = y1[:, :m].cpu().numpy()
            want2 = oracle.matvec_f64(fmt, W2, n, m, got1)
            e1 = np.linalg.norm(got1 - want1) / np.linalg.norm(want1)
            e2 = np.linalg.norm(y2[:, :n].cpu().numpy() - want2) / np.linalg.norm(want2)
            errs.append((float(e1), float(e2)))
            ctx.gather_setup(rank, 1, None, 0, 0)
            dist.barrier()
        ok = bool(all(e1 <= 5e-4 and e2 <= 5e-4 for e1, e2 in errs) and ctx.status() == 0)
        err = repr(errs)
    except Exception as ex:   # report instead of leaving the peer waiting on a barrier
        err = repr(ex)
    q.put((rank, ok, err))
    try:
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_batched_row_split(world):
    _run_ranks(_batched_worker, world)
