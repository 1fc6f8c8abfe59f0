"""GPU parity at the shapes the benchmark configurations name (not toy row counts): whole-tensor
dequantization compared bit for bit, matvec / fused / grouped / batched products against the fp64
oracle, lm_head-sized tensors on sampled rows, the MoE layer at 128 experts.  Same pins as the
small-shape tests: tests/test_q8_0.m:27-70 style closed forms live there, here the point is the
launch geometry the timed kernels really use (148 CTAs x many row tiles, grouped tensors of 6144
rows, 151 936-row tensors, combine form at inter = 768)."""
import numpy as np
import pytest

import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-4
TC_REL_L2_TOL = 5e-4


@pytest.fixture(scope="module")
def env():
    import torch
    from orome_b200 import format as F
    ctx = F.Context(0)
    yield torch, F, ctx
    assert ctx.status() == 0
    ctx.close()


def rel_l2(got, want):
    want = np.asarray(want, np.float64)
    return float(np.linalg.norm(np.asarray(got, np.float64) - want) / max(np.linalg.norm(want), 1e-300))


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same_floats(got, want):
    got, want = np.ascontiguousarray(got, np.float32), np.ascontiguousarray(want, np.float32)
    return np.array_equal(got.view(np.uint32), want.view(np.uint32))


def whole_tensor_dequant_is_bit_exact(env, fmt, out_dim, in_dim, data, wt, variant=0, chunk=2048):
    torch, F, ctx = env
    ref = F.tensor_ref(wt.data_ptr(), 0, fmt, out_dim, in_dim, variant)
    out = torch.empty((chunk, in_dim), device="cuda")
    for r0 in range(0, out_dim, chunk):
        n = min(chunk, out_dim - r0)
        ctx.dequant_rows(ref, r0, n, out.data_ptr())
        torch.cuda.synchronize()
        want = oracle.decode_rows(fmt, data, out_dim, in_dim, row0=r0, nrows=n, layout=variant)
        assert same_floats(out[:n].cpu().numpy(), want), (fmt, r0)


def matvec(env, fmt, wt, out_dim, in_dim, x, variant=0):
    torch, F, ctx = env
    xm = np.atleast_2d(x)
    xt = dev(torch, xm)
    y = torch.full((xm.shape[0], out_dim), float("nan"), device="cuda")
    ctx.matvec(F.tensor_ref(wt.data_ptr(), 0, fmt, out_dim, in_dim, variant), xt.data_ptr(), y.data_ptr(), xm.shape[0], in_dim, out_dim)
    torch.cuda.synchronize()
    out = y.cpu().numpy()
    return out[0] if np.ndim(x) == 1 else out


# ---- configuration 1: Q8_0 4096 x 4096 ------------------------------------------------------------------
def test_cfg1_q8_0_4096x4096(env):
    torch, F, ctx = env
    fmt, n = synth.Q8_0, 4096
    data = synth.host_tensor(fmt, n, n, seed=101)
    wt = dev(torch, data)
    whole_tensor_dequant_is_bit_exact(env, fmt, n, n, data, wt)
    x = synth.host_x(n, seed=102)
    assert rel_l2(matvec(env, fmt, wt, n, n, x), oracle.matvec_f64(fmt, data, n, n, x)) <= 2e-6


def test_q8_0_matvec_on_arbitrary_bytes(env):
    """Every quant byte, -128 included (the generators above never produce it), with finite scales."""
    torch, F, ctx = env
    fmt, out_dim, in_dim = synth.Q8_0, 1000, 4096
    rng = np.random.default_rng(7)
    blocks = rng.integers(0, 256, size=(out_dim * in_dim // 32, 34), dtype=np.uint8)
    blocks[::7, 2:] = 0x80                                        # whole blocks of -128
    d = (rng.standard_normal(blocks.shape[0]) * 0.01).astype(np.float16)           # both signs
    blocks[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    data = blocks.reshape(-1)
    wt = dev(torch, data)
    x = synth.host_x(in_dim, seed=8)
    for bits in (24, 16):
        ctx.set_option(F.OPT_X_BITS, bits)
        try:
            err = rel_l2(matvec(env, fmt, wt, out_dim, in_dim, x), oracle.matvec_f64(fmt, data, out_dim, in_dim, x))
        finally:
            ctx.set_option(F.OPT_X_BITS, 24)
        assert err <= (2e-6 if bits == 24 else REL_L2_TOL), (bits, err)
    # the same tensor as one product of a chain
    xt = dev(torch, x)
    y = torch.zeros(out_dim, device="cuda")
    ctx.chain_begin()
    ctx.matvec(F.tensor_ref(wt.data_ptr(), 0, fmt, out_dim, in_dim), xt.data_ptr(), y.data_ptr())
    ch = ctx.chain_end()
    ch.launch()
    torch.cuda.synchronize()
    assert rel_l2(y.cpu().numpy(), oracle.matvec_f64(fmt, data, out_dim, in_dim, x)) <= 2e-6
    ch.close()


# ---- configuration 2: Q4_K 12288 x 4096 and 4096 x 12288, batch 1 and 64, both scale layouts --------------------
@pytest.mark.parametrize("shape", [(12288, 4096), (4096, 12288)])
def test_cfg2_q4_k_pair(env, shape):
    torch, F, ctx = env
    fmt = synth.Q4_K
    out_dim, in_dim = shape
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=synth.seed_for("cfg2", *shape))
    wt = dev(torch, data)
    whole_tensor_dequant_is_bit_exact(env, fmt, out_dim, in_dim, data, wt, variant=0)
    whole_tensor_dequant_is_bit_exact(env, fmt, out_dim, in_dim, data, wt, variant=1, chunk=4096)
    x1 = synth.host_x(in_dim, seed=3)
    x64 = synth.host_x(in_dim, 64, seed=4)
    for variant in (0, 1):
        want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x1, layout=variant)
        assert rel_l2(matvec(env, fmt, wt, out_dim, in_dim, x1, variant), want) <= 2e-6
        want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x64, layout=variant)
        got = matvec(env, fmt, wt, out_dim, in_dim, x64, variant)
        assert rel_l2(got, want) <= TC_REL_L2_TOL
        col = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
        assert col.max() <= 2 * TC_REL_L2_TOL


# ---- configuration 3: the 9B Q8_0 layer ---------------------------------------------------------------------------
def test_cfg3_layer_products(env):
    torch, F, ctx = env
    fmt, H, A, KV = synth.Q8_0, 4096, 12288, 1024
    x = synth.host_x(H, seed=11)
    xt = dev(torch, x)
    # grouped q / k / v: 6144 rows in one launch
    dims = [H, KV, KV]
    datas = [synth.host_tensor(fmt, d, H, seed=200 + i) for i, d in enumerate(dims)]
    wts = [dev(torch, d) for d in datas]
    ys = [torch.full((d,), float("nan"), device="cuda") for d in dims]
    ctx.matvec_group([F.tensor_ref(w.data_ptr(), 0, fmt, d, H) for w, d in zip(wts, dims)], xt.data_ptr(), [y.data_ptr() for y in ys])
    torch.cuda.synchronize()
    for d, data, y in zip(dims, datas, ys):
        assert rel_l2(y.cpu().numpy(), oracle.matvec_f64(fmt, data, d, H, x)) <= 2e-6
    # fused gate / up + SwiGLU, 12288 rows each
    gd, ud = synth.host_tensor(fmt, A, H, seed=210), synth.host_tensor(fmt, A, H, seed=211)
    gt, ut = dev(torch, gd), dev(torch, ud)
    xs = x * np.float32(40.0)                                      # gate values of a few units: silu outside its linear range
    xst = dev(torch, xs)
    act = torch.full((A,), float("nan"), device="cuda")
    ctx.gate_up_swiglu(F.tensor_ref(gt.data_ptr(), 0, fmt, A, H), F.tensor_ref(ut.data_ptr(), 0, fmt, A, H), xst.data_ptr(), act.data_ptr())
    torch.cuda.synchronize()
    want = oracle.swiglu_f64(oracle.matvec_f64(fmt, gd, A, H, xs), oracle.matvec_f64(fmt, ud, A, H, xs))
    assert rel_l2(act.cpu().numpy(), want) <= 1e-5
    # down: 4096 x 12288
    dd = synth.host_tensor(fmt, H, A, seed=212)
    xa = synth.host_x(A, seed=12)
    assert rel_l2(matvec(env, fmt, dev(torch, dd), H, A, xa), oracle.matvec_f64(fmt, dd, H, A, xa)) <= 2e-6
    # batch 8 of the gate tensor on the tensor-core form
    x8 = synth.host_x(H, 8, seed=13)
    assert rel_l2(matvec(env, fmt, gt, A, H, x8), oracle.matvec_f64(fmt, gd, A, H, x8)) <= TC_REL_L2_TOL


def sampled_rows_check(env, fmt, out_dim, in_dim, variant, seed, tol=2e-6, nsample=192):
    """An lm_head-sized tensor filled on the device; the product runs over all rows, the oracle over sampled ones."""
    torch, F, ctx = env
    rb = synth.row_bytes(fmt, in_dim)
    buf = torch.empty(out_dim * rb + 256, dtype=torch.uint8, device="cuda")
    synth.device_fill(buf[:out_dim * rb], fmt, out_dim, in_dim, seed=seed)
    x = synth.host_x(in_dim, seed=seed + 1)
    xt = dev(torch, x)
    y = torch.full((out_dim,), float("nan"), device="cuda")
    ctx.matvec(F.tensor_ref(buf.data_ptr(), 0, fmt, out_dim, in_dim, variant), xt.data_ptr(), y.data_ptr())
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    rng = np.random.default_rng(seed)
    sel = np.unique(np.concatenate([rng.choice(out_dim, nsample, replace=False), [0, 1, out_dim - 2, out_dim - 1],
                                    np.arange(out_dim // 2 - 20, out_dim // 2 + 20)]))
    rows = buf[:out_dim * rb].view(out_dim, rb).index_select(0, torch.as_tensor(sel, device="cuda")).cpu().numpy().reshape(-1)
    want = oracle.matvec_f64(fmt, rows, len(sel), in_dim, x, layout=variant)
    assert rel_l2(got[sel], want) <= tol
    # sampled rows decode bit for bit too
    out = torch.empty((1, in_dim), device="cuda")
    for i in (0, len(sel) // 2, len(sel) - 1):
        ctx.dequant_rows(F.tensor_ref(buf.data_ptr(), 0, fmt, out_dim, in_dim, variant), int(sel[i]), 1, out.data_ptr())
        torch.cuda.synchronize()
        assert same_floats(out.cpu().numpy(), oracle.decode_rows(fmt, rows, len(sel), in_dim, row0=i, nrows=1, layout=variant))


def test_cfg3_lm_head_q8_0_sampled_rows(env):
    sampled_rows_check(env, synth.Q8_0, 151936, 4096, 0, seed=31)


# ---- configuration 4: the 27B mixed set (llama-style kernels) --------------------------------------------------------
def test_cfg4_gate_up_q4_k_17408x5120_llama(env):
    torch, F, ctx = env
    fmt, A, H = synth.Q4_K, 17408, 5120
    gd, ud = synth.host_tensor(fmt, A, H, seed=41), synth.host_tensor(fmt, A, H, seed=42)
    gt, ut = dev(torch, gd), dev(torch, ud)
    x = synth.host_x(H, seed=43) * np.float32(0.01)                # K-quant rows have a large mean: keep gate values of a few units
    xt = dev(torch, x)
    act = torch.full((A,), float("nan"), device="cuda")
    ctx.gate_up_swiglu(F.tensor_ref(gt.data_ptr(), 0, fmt, A, H, 1), F.tensor_ref(ut.data_ptr(), 0, fmt, A, H, 1), xt.data_ptr(), act.data_ptr())
    torch.cuda.synchronize()
    want = oracle.swiglu_f64(oracle.matvec_f64(fmt, gd, A, H, x, layout=1), oracle.matvec_f64(fmt, ud, A, H, x, layout=1))
    assert rel_l2(act.cpu().numpy(), want) <= 1e-5


def test_cfg4_down_q6_k_5120x17408(env):
    torch, F, ctx = env
    fmt, H, A = synth.Q6_K, 5120, 17408
    data = synth.host_tensor(fmt, H, A, seed=44)
    wt = dev(torch, data)
    whole_tensor_dequant_is_bit_exact(env, fmt, H, A, data, wt, chunk=1024)
    x = synth.host_x(A, seed=45)
    assert rel_l2(matvec(env, fmt, wt, H, A, x), oracle.matvec_f64(fmt, data, H, A, x)) <= 2e-6


def test_cfg4_lm_head_q6_k_sampled_rows(env):
    sampled_rows_check(env, synth.Q6_K, 151936, 5120, 0, seed=46)


def test_gate_up_q5_k_llama_layout(env):
    torch, F, ctx = env
    fmt, A, H = synth.Q5_K, 3000, 2048
    gd, ud = synth.host_tensor(fmt, A, H, seed=51), synth.host_tensor(fmt, A, H, seed=52)
    gt, ut = dev(torch, gd), dev(torch, ud)
    x = synth.host_x(H, seed=53) * np.float32(0.01)
    xt = dev(torch, x)
    for variant in (0, 1):
        act = torch.full((A,), float("nan"), device="cuda")
        ctx.gate_up_swiglu(F.tensor_ref(gt.data_ptr(), 0, fmt, A, H, variant), F.tensor_ref(ut.data_ptr(), 0, fmt, A, H, variant),
                           xt.data_ptr(), act.data_ptr())
        torch.cuda.synchronize()
        want = oracle.swiglu_f64(oracle.matvec_f64(fmt, gd, A, H, x, layout=variant), oracle.matvec_f64(fmt, ud, A, H, x, layout=variant))
        assert rel_l2(act.cpu().numpy(), want) <= 1e-5, variant


# ---- configuration 5: MoE layer, 128 experts, top-8, hidden 2048, inter 768 --------------------------------------------
@pytest.fixture(scope="module")
def moe_layer(env):
    torch, F, ctx = env
    H, M, E = 2048, 768, 128
    gate = synth.host_tensor(synth.Q4_K, E * M, H, seed=61)
    up = synth.host_tensor(synth.Q4_K, E * M, H, seed=62)
    down = synth.host_tensor(synth.Q5_K, E * H, M, seed=63)
    sg, sd = synth.tensor_bytes(synth.Q4_K, M, H), synth.tensor_bytes(synth.Q5_K, H, M)
    wt = dev(torch, np.concatenate([gate, up, down]))
    layer = F.ExpertLayerRef(wt.data_ptr(), F.ExpertProjRef(0, sg, synth.Q4_K), F.ExpertProjRef(gate.size, sg, synth.Q4_K),
                             F.ExpertProjRef(gate.size + up.size, sd, synth.Q5_K))
    router = synth.host_router(E, H, seed=64)
    return dict(H=H, M=M, E=E, gate=gate, up=up, down=down, sg=sg, sd=sd, wt=wt, layer=layer, router=router)


@pytest.mark.parametrize("T", [1, 32])
def test_cfg5_moe_layer(env, moe_layer, T):
    torch, F, ctx = env
    L = moe_layer
    H, M, E, K = L["H"], L["M"], L["E"], 8
    x = np.atleast_2d(synth.host_x(H, T, seed=70 + T)) * np.float32(0.02)
    xt = dev(torch, x)
    rt = dev(torch, L["router"].view(np.uint8).reshape(-1))
    idx = torch.zeros((T, 8), device="cuda", dtype=torch.int32)
    w = torch.zeros((T, 8), device="cuda")
    logits = torch.zeros((T, E), device="cuda")
    ctx.moe_route(F.tensor_ref(rt.data_ptr(), 0, synth.F32, E, H), xt.data_ptr(), T, H, K, idx.data_ptr(), w.data_ptr(), logits.data_ptr())
    act = torch.full((T, K, M), float("nan"), device="cuda")
    out = torch.full((T, H), float("nan"), device="cuda")
    ctx.moe_ffn(L["layer"], 0, xt.data_ptr(), T, H, idx.data_ptr(), w.data_ptr(), K, H, M, act.data_ptr(), out.data_ptr(), H)
    torch.cuda.synchronize()
    lg, gi, gw, got = logits.cpu().numpy(), idx.cpu().numpy().astype(np.uint32), w.cpu().numpy(), out.cpu().numpy()
    for t in range(T):
        oi, ow = oracle.route(lg[t], K)                            # the oracle routes the logits the GPU produced
        assert np.array_equal(gi[t], oi)
        assert np.max(np.abs(gw[t] - ow)) <= 1e-6
        want = oracle.moe_ffn_f64(L["gate"], L["up"], L["down"], (synth.Q4_K, synth.Q4_K, synth.Q5_K), (L["sg"], L["sg"], L["sd"]),
                                  x[t], H, M, gi[t], gw[t])
        assert rel_l2(got[t], want) <= REL_L2_TOL, t


def test_cfg5_moe_expert_parallel_shares(env, moe_layer):
    """Eight ranks' shares (16 experts each), computed in turn on one GPU, add up to the layer."""
    from orome_b200 import rowsplit
    torch, F, ctx = env
    L = moe_layer
    H, M, E, K, T, world = L["H"], L["M"], L["E"], 8, 4, 8
    x = np.atleast_2d(synth.host_x(H, T, seed=81)) * np.float32(0.02)
    rng = np.random.default_rng(82)
    idx = np.stack([rng.permutation(E)[:8] for _ in range(T)]).astype(np.uint32)
    w = rng.random((T, 8)).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    xt, it, wtt = dev(torch, x), dev(torch, idx.view(np.int32)), dev(torch, w)
    total = np.zeros((T, H), np.float64)
    sg, sd = L["sg"], L["sd"]
    for rank in range(world):
        e0, e1 = rowsplit.shard_experts(E, rank, world)
        n = e1 - e0
        blob = np.concatenate([L["gate"][e0 * sg:e1 * sg], L["up"][e0 * sg:e1 * sg], L["down"][e0 * sd:e1 * sd]])
        wt = dev(torch, blob)
        layer = F.ExpertLayerRef(wt.data_ptr(), F.ExpertProjRef(0, sg, synth.Q4_K), F.ExpertProjRef(n * sg, sg, synth.Q4_K),
                                 F.ExpertProjRef(2 * n * sg, sd, synth.Q5_K))
        act = torch.full((T, K, M), float("nan"), device="cuda")
        out = torch.full((T, H), float("nan"), device="cuda")
        loc = torch.zeros((T, 8), dtype=torch.int32, device="cuda")
        ctx.moe_ffn_shard(layer, 0, xt.data_ptr(), T, H, it.data_ptr(), wtt.data_ptr(), K, H, M, e0, n, loc.data_ptr(), act.data_ptr(),
                          out.data_ptr(), H)
        torch.cuda.synchronize()
        total += out.cpu().numpy().astype(np.float64)
    for t in range(T):
        want = oracle.moe_ffn_f64(L["gate"], L["up"], L["down"], (synth.Q4_K, synth.Q4_K, synth.Q5_K), (sg, sg, sd), x[t], H, M, idx[t], w[t])
        assert rel_l2(total[t], want) <= REL_L2_TOL


@pytest.mark.parametrize("T", [1, 5])
def test_cfg5_moe_block_with_shared_expert(env, moe_layer, T):
    """Router + shared-gate logit in one launch, routed experts, shared expert (Q8_0 gate/up, Q4_K down), combine with
    the sigmoid gate and the residual input: the whole block of engine.m:158-340 at the 128-expert shape."""
    torch, F, ctx = env
    L = moe_layer
    H, M, E, K, S = L["H"], L["M"], L["E"], 8, 512
    sgd, sud = synth.host_tensor(synth.Q8_0, S, H, seed=91), synth.host_tensor(synth.Q8_0, S, H, seed=92)
    sdd = synth.host_tensor(synth.Q4_K, H, S, seed=93)
    sgw = (np.random.default_rng(94).standard_normal(H) / np.sqrt(H)).astype(np.float32)          # [1][H] fp32 gate row
    x = np.atleast_2d(synth.host_x(H, T, seed=95)) * np.float32(0.02)
    h_mid = np.atleast_2d(synth.host_x(H, T, seed=96))
    xt, ht = dev(torch, x), dev(torch, h_mid)
    rt, sgt = dev(torch, L["router"].view(np.uint8).reshape(-1)), dev(torch, sgw.view(np.uint8))
    tg, tu, td = dev(torch, sgd), dev(torch, sud), dev(torch, sdd)
    idx = torch.zeros((T, 8), device="cuda", dtype=torch.int32)
    w = torch.zeros((T, 8), device="cuda")
    sl = torch.full((T,), float("nan"), device="cuda")
    logits = torch.zeros((T, E + 1), device="cuda")
    ctx.moe_route_pair(F.tensor_ref(rt.data_ptr(), 0, synth.F32, E, H), F.tensor_ref(sgt.data_ptr(), 0, synth.F32, 1, H), xt.data_ptr(), T, H, K,
                       idx.data_ptr(), w.data_ptr(), sl.data_ptr(), logits.data_ptr())
    scratch = torch.empty(F.moe_block_scratch_floats(T, K, H, M, S), device="cuda")
    out = torch.full((T, H), float("nan"), device="cuda")
    shared = (F.tensor_ref(tg.data_ptr(), 0, synth.Q8_0, S, H), F.tensor_ref(tu.data_ptr(), 0, synth.Q8_0, S, H), F.tensor_ref(td.data_ptr(), 0, synth.Q4_K, H, S))
    ctx.moe_block(L["layer"], 0, shared, xt.data_ptr(), T, H, idx.data_ptr(), w.data_ptr(), sl.data_ptr(), K, H, M, ht.data_ptr(), H,
                  scratch.data_ptr(), out.data_ptr(), H)
    torch.cuda.synchronize()
    lg, gi, gw, gsl, got = logits.cpu().numpy(), idx.cpu().numpy().astype(np.uint32), w.cpu().numpy(), sl.cpu().numpy(), out.cpu().numpy()
    for t in range(T):
        # slot 8 of the reference's params: the raw logit of the gate row, which sits after the router logits
        assert gsl[t] == lg[t, E]
        assert abs(gsl[t] - float(np.dot(sgw.astype(np.float64), x[t].astype(np.float64)))) <= 1e-5
        oi, ow = oracle.route(lg[t, :E], K)
        assert np.array_equal(gi[t], oi) and np.max(np.abs(gw[t] - ow)) <= 1e-6
        want = oracle.moe_block_f64(L["gate"], L["up"], L["down"], (synth.Q4_K, synth.Q4_K, synth.Q5_K), (L["sg"], L["sg"], L["sd"]),
                                    ((synth.Q8_0, sgd, S), (synth.Q8_0, sud, S), (synth.Q4_K, sdd)), x[t], H, M, gi[t], gw[t], gsl[t], h_mid=h_mid[t])
        assert rel_l2(got[t], want) <= REL_L2_TOL, t
    # without a shared expert and without a residual input the block is the routed sum alone
    out2 = torch.full((T, H), float("nan"), device="cuda")
    ctx.moe_block(L["layer"], 0, None, xt.data_ptr(), T, H, idx.data_ptr(), w.data_ptr(), 0, K, H, M, 0, 0, scratch.data_ptr(), out2.data_ptr(), H)
    torch.cuda.synchronize()
    for t in range(T):
        want = oracle.moe_ffn_f64(L["gate"], L["up"], L["down"], (synth.Q4_K, synth.Q4_K, synth.Q5_K), (L["sg"], L["sg"], L["sd"]), x[t], H, M, gi[t], gw[t])
        assert rel_l2(out2.cpu().numpy()[t], want) <= REL_L2_TOL
