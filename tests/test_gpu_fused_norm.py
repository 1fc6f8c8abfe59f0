"""The steps either side of a product, fused into it (orome_cuda_fuse_next): the residual add + sum of squares as
the epilogue of the producing product (shaders.metal:86-124) and the RMS norm as the prologue of the products that
read the normalised vector (shaders.metal:126-149), as engine.m:625-653 strings them together.  Checked against the
numpy restatement of the two shader kernels in oracle/ and the fp64 matvec oracle."""
import ctypes as C

import numpy as np
import pytest

import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-4
EPS = 1e-6


def rel_l2(got, want):
    want = np.asarray(want, np.float64)
    return float(np.linalg.norm(np.asarray(got, np.float64) - want) / max(np.linalg.norm(want), 1e-300))


@pytest.fixture(scope="module")
def env():
    import torch
    from orome_b200 import format as F
    ctx = F.Context(0)
    yield torch, F, ctx
    assert ctx.status() == 0
    ctx.close()


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bf16_weights(n, seed):
    w = (1.0 + 0.25 * np.random.default_rng(seed).standard_normal(n)).astype(np.float32)
    return (w.view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K])
@pytest.mark.parametrize("variant", [0, 1])
def test_output_projection_then_ffn_with_the_norm_in_between(env, fmt, variant):
    torch, F, ctx = env
    if variant == 1 and fmt in (synth.Q8_0, synth.Q6_K):
        pytest.skip("one scale layout")
    H, M = 2048, 1536
    wo, wg, wu = (synth.host_tensor(fmt, r, H, seed=s) for r, s in ((H, 11), (M, 12), (M, 13)))
    attn, resid = synth.host_x(H, seed=14), synth.host_x(H, seed=15)
    resid[7], resid[100] = 7e4, -9e4                                   # beyond the clamp
    nw = bf16_weights(H, 16)
    t = {k: dev(torch, v) for k, v in dict(wo=wo, wg=wg, wu=wu, attn=attn, resid=resid, nw=nw).items()}
    parts = torch.full((F.SUM_SQ_PARTS,), float("nan"), device="cuda")
    hidden = torch.full((H,), float("nan"), device="cuda")
    act = torch.full((M,), float("nan"), device="cuda")
    ref = lambda w, rows: F.tensor_ref(w.data_ptr(), 0, fmt, rows, H, variant)

    # 1. hidden = clamp(resid + Wo attn), partial sums of hidden^2
    ctx.fuse_next(None, F.ResidualEpilogue(t["resid"].data_ptr(), parts.data_ptr()))
    ctx.matvec(ref(t["wo"], H), t["attn"].data_ptr(), hidden.data_ptr())
    torch.cuda.synchronize()
    prod = oracle.matvec_f64(fmt, wo, H, H, attn, layout=variant)
    want_hidden, want_parts = oracle.residual_add_sum_sq(resid, prod.astype(np.float32))
    got_hidden, got_parts = hidden.cpu().numpy(), parts.cpu().numpy()
    assert got_hidden[7] == np.float32(65504.0) and got_hidden[100] == np.float32(-65504.0)
    assert rel_l2(got_hidden, want_hidden) <= REL_L2_TOL
    assert np.isfinite(got_parts).all() and (got_parts >= 0).all() and np.count_nonzero(got_parts) <= 296
    assert abs(float(got_parts.astype(np.float64).sum()) / float(want_parts.astype(np.float64).sum()) - 1.0) <= 1e-5

    # 2. act = silu(Wg n) * (Wu n) with n = hidden * rsqrt(sum / H + eps) * w read on the fly
    ctx.fuse_next(F.NormPrologue(t["nw"].data_ptr(), parts.data_ptr(), EPS), None)
    ctx.gate_up_swiglu(ref(t["wg"], M), ref(t["wu"], M), hidden.data_ptr(), act.data_ptr())
    torch.cuda.synchronize()
    n = oracle.rms_norm_apply_partial(got_hidden, nw, want_parts, EPS)
    want_act = oracle.swiglu_f64(oracle.matvec_f64(fmt, wg, M, H, n, layout=variant), oracle.matvec_f64(fmt, wu, M, H, n, layout=variant))
    assert rel_l2(act.cpu().numpy(), want_act) <= REL_L2_TOL

    # 3. the same prologue on a group of tensors (q / k / v read the normalised vector too), residual added in place
    q, k = torch.full((M,), float("nan"), device="cuda"), torch.full((M,), float("nan"), device="cuda")
    ctx.fuse_next(F.NormPrologue(t["nw"].data_ptr(), parts.data_ptr(), EPS))
    ctx.matvec_group([ref(t["wg"], M), ref(t["wu"], M)], hidden.data_ptr(), [q.data_ptr(), k.data_ptr()])
    torch.cuda.synchronize()
    assert rel_l2(q.cpu().numpy(), oracle.matvec_f64(fmt, wg, M, H, n, layout=variant)) <= REL_L2_TOL
    assert rel_l2(k.cpu().numpy(), oracle.matvec_f64(fmt, wu, M, H, n, layout=variant)) <= REL_L2_TOL
    inplace = t["resid"].clone()
    ctx.fuse_next(None, F.ResidualEpilogue(inplace.data_ptr(), parts.data_ptr()))
    ctx.matvec(ref(t["wo"], H), t["attn"].data_ptr(), inplace.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(inplace.cpu().numpy(), got_hidden)
    # a plain launch afterwards is a plain launch: the request does not linger
    plain = torch.empty((H,), device="cuda")
    ctx.matvec(ref(t["wo"], H), t["attn"].data_ptr(), plain.data_ptr())
    torch.cuda.synchronize()
    assert rel_l2(plain.cpu().numpy(), prod) <= REL_L2_TOL


def test_prologue_and_epilogue_on_the_same_product(env):
    torch, F, ctx = env
    fmt, H = synth.Q8_0, 1024
    w = synth.host_tensor(fmt, H, H, seed=21)
    x, resid, nw = synth.host_x(H, seed=22), synth.host_x(H, seed=23), bf16_weights(H, 24)
    _, in_parts = oracle.residual_add_sum_sq(x, np.zeros(H, np.float32))
    pin = np.zeros(F.SUM_SQ_PARTS, np.float32)
    pin[:in_parts.size] = in_parts                                     # a caller may fill the array itself
    t = {k: dev(torch, v) for k, v in dict(w=w, x=x, resid=resid, nw=nw, pin=pin).items()}
    pout = torch.full((F.SUM_SQ_PARTS,), float("nan"), device="cuda")
    y = torch.empty((H,), device="cuda")
    ctx.fuse_next(F.NormPrologue(t["nw"].data_ptr(), t["pin"].data_ptr(), EPS), F.ResidualEpilogue(t["resid"].data_ptr(), pout.data_ptr()))
    ctx.matvec(F.tensor_ref(t["w"].data_ptr(), 0, fmt, H, H), t["x"].data_ptr(), y.data_ptr())
    torch.cuda.synchronize()
    n = oracle.rms_norm_apply_partial(x, nw, in_parts, EPS)
    want, want_parts = oracle.residual_add_sum_sq(resid, oracle.matvec_f64(fmt, w, H, H, n).astype(np.float32))
    assert rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL
    assert abs(float(pout.cpu().numpy().astype(np.float64).sum()) / float(want_parts.astype(np.float64).sum()) - 1.0) <= 1e-5


def test_calls_without_a_fused_form_drop_the_request(env):
    torch, F, ctx = env
    fmt, H = synth.Q8_0, 512
    w = dev(torch, synth.host_tensor(fmt, H, H, seed=31))
    x8, y8 = dev(torch, synth.host_x(H, 8, seed=32)), torch.zeros((8, H), device="cuda")
    nw, parts = dev(torch, bf16_weights(H, 33)), torch.zeros((F.SUM_SQ_PARTS,), device="cuda")
    ref = F.tensor_ref(w.data_ptr(), 0, fmt, H, H)
    pro = F.NormPrologue(nw.data_ptr(), parts.data_ptr(), EPS)
    epi = F.ResidualEpilogue(x8.data_ptr(), parts.data_ptr())
    ctx.fuse_next(pro)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, x8.data_ptr(), y8.data_ptr(), 8, H, H)                   # batched
    assert e.value.code == F.ENOTSUP
    ctx.fuse_next(None, epi)
    with pytest.raises(F.OromeError) as e:
        ctx.gate_up_swiglu(ref, ref, x8.data_ptr(), y8.data_ptr())               # no residual form of the fused gate/up
    assert e.value.code == F.ENOTSUP
    ctx.fuse_next(None, epi)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec_group([ref, ref], x8.data_ptr(), [y8[0].data_ptr(), y8[1].data_ptr()])     # epilogue wants one tensor
    assert e.value.code == F.ENOTSUP
    ctx.chain_begin()
    ctx.fuse_next(pro)
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, x8.data_ptr(), y8.data_ptr())                            # recordings have no fused form
    assert e.value.code == F.ENOTSUP
    ctx.matvec(ref, x8.data_ptr(), y8.data_ptr())
    ctx.chain_end().close()
    with pytest.raises(F.OromeError) as e:
        ctx.fuse_next(F.NormPrologue(nw.data_ptr() + 2, parts.data_ptr(), EPS))  # misaligned weights
    assert e.value.code == F.EINVAL
    y = torch.empty((H,), device="cuda")
    ctx.matvec(ref, x8.data_ptr(), y.data_ptr())                                 # nothing is pending any more
    torch.cuda.synchronize()
    want = oracle.matvec_f64(fmt, synth.host_tensor(fmt, H, H, seed=31), H, H, synth.host_x(H, 8, seed=32)[0])
    assert rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL
