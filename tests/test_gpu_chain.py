"""GPU parity of the chained form: a recorded sequence of products run as one resident kernel
(the reference's one command buffer per token, engine.m:453-454, 1048-1050), against the CPU
oracle applied product by product, plus the arg-max epilogue (shaders.metal:1249-1305)."""
import numpy as np
import pytest

import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu


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


class Step:
    """A decode-shaped sequence: per layer grouped q/k/v, o, fused gate/up, down; then lm_head.  Every product
    reads the output of the one before it, as in the engine (engine.m:481-1046)."""

    def __init__(self, torch, F, fmts, H, A, KV, V, layers, seed, variant=0, reuse=False):
        self.torch, self.F, self.H, self.A, self.KV, self.V, self.layers, self.variant = torch, F, H, A, KV, V, layers, variant
        self.fmts = fmts
        shapes = dict(q=(H, H), k=(KV, H), v=(KV, H), o=(H, H), gate=(A, H), up=(A, H), down=(H, A))
        self.shapes = shapes
        self.host, self.devt = [], []
        for l in range(layers):
            hl = {k: synth.host_tensor(fmts[k], *shapes[k], seed=synth.seed_for("chain", seed, l, k)) for k in shapes}
            self.host.append(hl)
            self.devt.append({k: dev(torch, v) for k, v in hl.items()})
        self.lm_host = synth.host_tensor(fmts["lm_head"], V, H, seed=synth.seed_for("chain", seed, "lm"))
        self.lm_dev = dev(torch, self.lm_host)
        nb = 1 if reuse else layers
        z = lambda n: [torch.full((n,), float("nan"), device="cuda") for _ in range(nb)]
        self.q, self.k, self.v, self.o, self.act, self.dn = z(H), z(KV), z(KV), z(H), z(A), z(H)
        self.logits = torch.full((V,), float("nan"), device="cuda")
        self.x0 = torch.zeros(H, device="cuda")
        self.tok = torch.full((1,), -1, device="cuda", dtype=torch.int32)
        self.reuse = reuse

    def ref(self, l, k):
        od, idim = self.shapes[k]
        return self.F.tensor_ref(self.devt[l][k].data_ptr(), 0, self.fmts[k], od, idim, self.variant)

    def record(self, ctx, argmax=True):
        F = self.F
        x = self.x0
        for l in range(self.layers):
            b = 0 if self.reuse else l
            ctx.matvec_group([self.ref(l, "q"), self.ref(l, "k"), self.ref(l, "v")], x.data_ptr(),
                             [self.q[b].data_ptr(), self.k[b].data_ptr(), self.v[b].data_ptr()])
            ctx.matvec(self.ref(l, "o"), self.q[b].data_ptr(), self.o[b].data_ptr())
            ctx.gate_up_swiglu(self.ref(l, "gate"), self.ref(l, "up"), self.o[b].data_ptr(), self.act[b].data_ptr())
            ctx.format_dispatch_matvec(self.ref(l, "down"), self.act[b].data_ptr(), 0, self.dn[b].data_ptr(), 0)
            x = self.dn[b]
        lm = F.tensor_ref(self.lm_dev.data_ptr(), 0, self.fmts["lm_head"], self.V, self.H, self.variant)
        ctx.matvec(lm, x.data_ptr(), self.logits.data_ptr())
        if argmax:
            ctx.argmax(self.logits.data_ptr(), self.V, self.tok.data_ptr())

    def expected(self, x0):
        """The oracle product by product; each product's fp64 result is rounded to the fp32 vector the next one reads."""
        mv = lambda fmt, data, od, idim, x: oracle.matvec_f64(fmt, data, od, idim, x, layout=self.variant)
        out = []
        x = np.asarray(x0, np.float32)
        for l in range(self.layers):
            h, f, s = self.host[l], self.fmts, self.shapes
            q = mv(f["q"], h["q"], *s["q"], x).astype(np.float32)
            k = mv(f["k"], h["k"], *s["k"], x).astype(np.float32)
            v = mv(f["v"], h["v"], *s["v"], x).astype(np.float32)
            o = mv(f["o"], h["o"], *s["o"], q).astype(np.float32)
            act = oracle.swiglu_f64(mv(f["gate"], h["gate"], *s["gate"], o), mv(f["up"], h["up"], *s["up"], o)).astype(np.float32)
            dn = mv(f["down"], h["down"], *s["down"], act).astype(np.float32)
            out.append(dict(q=q, k=k, v=v, o=o, act=act, dn=dn))
            x = dn
        logits = mv(self.fmts["lm_head"], self.lm_host, self.V, self.H, x).astype(np.float32)
        return out, logits


ALL_Q8 = {k: synth.Q8_0 for k in ("q", "k", "v", "o", "gate", "up", "down", "lm_head")}
MIXED = dict(q=synth.Q4_K, k=synth.Q4_K, v=synth.Q4_K, o=synth.Q5_K, gate=synth.Q4_K, up=synth.Q4_K, down=synth.Q6_K, lm_head=synth.Q6_K)


def run_and_check(env, st, x0, tol):
    torch, F, ctx = env
    st.x0.copy_(torch.from_numpy(x0))
    st.chain.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ctx.status() == 0
    per_layer, logits = st.expected(x0)
    worst = 0.0
    if not st.reuse:
        for l, want in enumerate(per_layer):
            for name, buf in (("q", st.q), ("k", st.k), ("v", st.v), ("o", st.o), ("act", st.act), ("dn", st.dn)):
                err = rel_l2(buf[l].cpu().numpy(), want[name])
                worst = max(worst, err)
                assert err <= tol, (l, name, err)
    got = st.logits.cpu().numpy()
    assert rel_l2(got, logits) <= tol
    # the token is the arg-max of the logits the GPU itself produced, ties as the reference's kernel resolves them
    assert int(st.tok.item()) == oracle.argmax(got)
    return worst


@pytest.mark.parametrize("x_bits", [24, 16])
def test_chain_q8_0_every_vector(env, x_bits):
    torch, F, ctx = env
    ctx.set_option(F.OPT_X_BITS, x_bits)
    try:
        st = Step(torch, F, ALL_Q8, H=512, A=1536, KV=128, V=3000, layers=3, seed=1)
        ctx.chain_begin()
        c0 = ctx.launch_count
        st.record(ctx)
        assert ctx.launch_count == c0                       # recording launches nothing
        st.chain = ctx.chain_end()
        info = st.chain.info()
        assert info["products"] == 3 * 4 + 1 and info["stages"] >= 2
        tol = 1e-5 if x_bits == 24 else 3e-4         # 16-bit x: ~3e-5 per product, carried through thirteen products
        rng = np.random.default_rng(3)
        # launch it several times with fresh inputs: tags of one launch must not satisfy the next
        for rep in range(3):
            x0 = (rng.standard_normal(512) * 30.0).astype(np.float32)
            run_and_check(env, st, x0, tol)
        assert ctx.launch_count == c0 + 3                   # one launch per step
        st.chain.close()
    finally:
        ctx.set_option(F.OPT_X_BITS, 24)


def test_chain_mixed_kquants_llama_layout(env):
    torch, F, ctx = env
    st = Step(torch, F, MIXED, H=1024, A=2048, KV=256, V=2500, layers=2, seed=2, variant=1)
    ctx.chain_begin()
    st.record(ctx)
    st.chain = ctx.chain_end()
    # K-quant blocks with random scale bytes have a large positive mean, so a vector grows by ~500x per product
    # (and squares in the SwiGLU): start small enough that two layers and the lm_head stay inside the fp32 range
    x0 = (np.random.default_rng(5).standard_normal(1024) * 1e-7).astype(np.float32)
    run_and_check(env, st, x0, 2e-5)
    st.chain.close()


def test_chain_with_reused_buffers_and_many_rows(env):
    """The benchmark's shape of use: every layer writes the same q/k/v/o/act/dn buffers (ordered by the data
    dependencies), and tensors large enough that every CTA walks several tiles and the stage ring wraps."""
    torch, F, ctx = env
    st = Step(torch, F, ALL_Q8, H=1024, A=4096, KV=256, V=40000, layers=3, seed=3, reuse=True)
    ctx.chain_begin()
    st.record(ctx)
    st.chain = ctx.chain_end()
    rng = np.random.default_rng(7)
    for rep in range(2):
        run_and_check(env, st, (rng.standard_normal(1024) * 100.0).astype(np.float32), 1e-5)
    st.chain.close()


def test_chain_agrees_with_single_launches(env):
    torch, F, ctx = env
    st = Step(torch, F, ALL_Q8, H=512, A=1024, KV=128, V=1500, layers=2, seed=4)
    x0 = (np.random.default_rng(9).standard_normal(512) * 20.0).astype(np.float32)
    st.x0.copy_(torch.from_numpy(x0))
    st.record(ctx, argmax=True)                              # not recording: the same calls launch one kernel each
    torch.cuda.synchronize()
    single = st.logits.cpu().numpy().copy()
    tok = int(st.tok.item())
    st.logits.fill_(float("nan"))
    ctx.chain_begin()
    st.record(ctx)
    st.chain = ctx.chain_end()
    st.chain.launch()
    torch.cuda.synchronize()
    assert rel_l2(st.logits.cpu().numpy(), single) <= 1e-6
    assert int(st.tok.item()) == tok
    st.chain.close()


def test_chain_rejects_unordered_overwrite_and_unsupported_calls(env):
    torch, F, ctx = env
    fmt, n = synth.Q8_0, 256
    wt = dev(torch, synth.host_tensor(fmt, n, n, seed=1))
    ref = F.tensor_ref(wt.data_ptr(), 0, fmt, n, n)
    a, b, c = (torch.zeros(n, device="cuda") for _ in range(3))
    # product 1 overwrites the vector product 0 reads, and nothing orders the two
    ctx.chain_begin()
    ctx.matvec(ref, a.data_ptr(), b.data_ptr())
    ctx.matvec(ref, c.data_ptr(), a.data_ptr())
    with pytest.raises(F.OromeError) as e:
        ctx.chain_end()
    assert e.value.code == F.ENOTSUP
    # the recording is closed by chain_end even when it fails
    ctx.matvec(ref, a.data_ptr(), b.data_ptr())
    torch.cuda.synchronize()
    # batches and unquantized tensors cannot be recorded; the recording stays open and usable
    ctx.chain_begin()
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(ref, a.data_ptr(), b.data_ptr(), 4, n, n)
    assert e.value.code == F.ENOTSUP
    ctx.matvec(ref, a.data_ptr(), b.data_ptr())
    ch = ctx.chain_end()
    assert ch.info()["products"] == 1
    ch.close()
    with pytest.raises(F.OromeError):
        ctx.chain_end()                                      # nothing open
    ctx.chain_begin()
    with pytest.raises(F.OromeError):
        ctx.chain_begin()                                    # already open
    with pytest.raises(F.OromeError):
        ctx.chain_end()                                      # empty


def test_argmax_kernel_ties_and_special_values(env):
    torch, F, ctx = env
    rng = np.random.default_rng(11)
    cases = []
    v = rng.standard_normal(5000).astype(np.float32)
    cases.append(v)
    t = v.copy(); t[[5, 1027, 2051, 3, 40, 64, 1000]] = 9.0   # equal maxima in several threads and simdgroups
    cases.append(t)
    t = v.copy(); t[[2051, 1027]] = 9.0                       # same thread: the lower index wins
    cases.append(t)
    t = v.copy(); t[10] = np.nan; t[11] = np.inf; t[2000] = np.inf
    cases.append(t)
    cases.append(np.full(3000, -np.inf, np.float32))          # no candidate: index 0
    cases.append(np.full(1500, np.nan, np.float32))
    z = np.zeros(2100, np.float32); z[1500] = -0.0
    cases.append(z)                                           # +0 and -0 are equal
    cases.append(-np.abs(v) - 1.0)
    cases.append(np.array([3.0], np.float32))
    out = torch.zeros(1, device="cuda", dtype=torch.int32)
    for c in cases:
        d = dev(torch, c)
        ctx.argmax(d.data_ptr(), c.size, out.data_ptr())
        torch.cuda.synchronize()
        assert int(out.item()) == oracle.argmax(c), c[:8]


def test_chain_argmax_with_exact_ties(env):
    """Two identical lm_head rows give bit-identical logits: the fused epilogue must pick as the reference does."""
    torch, F, ctx = env
    fmt, H, V = synth.Q8_0, 256, 4200
    rb = synth.row_bytes(fmt, H)
    w = synth.host_tensor(fmt, V, H, seed=21).reshape(V, rb).copy()
    x = synth.host_x(H, seed=22)
    y = oracle.matvec_f64(fmt, w.reshape(-1), V, H, x)
    top = int(np.argmax(y))
    for r in (7, 1031, 2055, 4100):                           # copies of the winning row at other places
        w[r] = w[top]
    wt, xt = dev(torch, w.reshape(-1)), dev(torch, x)
    logits = torch.zeros(V, device="cuda")
    tok = torch.zeros(1, device="cuda", dtype=torch.int32)
    ctx.chain_begin()
    ctx.matvec(F.tensor_ref(wt.data_ptr(), 0, fmt, V, H), xt.data_ptr(), logits.data_ptr())
    ctx.argmax(logits.data_ptr(), V, tok.data_ptr())
    ch = ctx.chain_end()
    ch.launch()
    torch.cuda.synchronize()
    got = logits.cpu().numpy()
    assert len({got[r].tobytes() for r in (top, 7, 1031, 2055, 4100)}) == 1
    assert int(tok.item()) == oracle.argmax(got)
    ch.close()
