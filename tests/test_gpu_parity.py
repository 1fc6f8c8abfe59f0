"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle and the
committed golden vectors.  Bit-exact for dequantized weights and routing indices;
rel-L2 <= 1e-4 against the fp64-accumulated oracle for matvec outputs."""
import os

import numpy as np
import pytest

import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-4          # the tolerance the path states for fp32 accumulation
TC_REL_L2_TOL = 5e-4       # tensor-core batched form: weights and x rounded to fp16 (the reference stages x as fp16 too); measured 2-3e-4
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "decode_golden.npz"))
FMTS = {"Q8_0": synth.Q8_0, "Q4_K": synth.Q4_K, "Q5_K": synth.Q5_K, "Q6_K": synth.Q6_K}
QUANT = list(FMTS.values())


@pytest.fixture(scope="module")
def env():
    import torch
    from orome_b200 import format as F
    ctx = F.Context(0)
    yield torch, F, ctx
    assert ctx.status() == 0
    ctx.close()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def assert_same_floats(got, want):
    """Bit-identical wherever the value is a number.  Where the reference yields a NaN (a NaN
    or infinite fp16 scale, which no GGUF file contains) both sides must be NaN: the bit
    pattern of an arithmetic NaN is a property of the processor, not of the algorithm (x86,
    Arm and the GPU each produce a different one)."""
    got, want = np.ascontiguousarray(got, np.float32), np.ascontiguousarray(want, np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan])


def rel_l2(got, want):
    want = np.asarray(want, np.float64)
    return float(np.linalg.norm(np.asarray(got, np.float64) - want) / max(np.linalg.norm(want), 1e-300))


def dev_bytes(torch, arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def make_ref(F, wt, fmt, out_dim, in_dim, variant=0, offset=0):
    return F.tensor_ref(wt.data_ptr(), offset, fmt, out_dim, in_dim, variant)


def gpu_matvec(env, fmt, data, out_dim, in_dim, x, variant=0):
    torch, F, ctx = env
    wt = dev_bytes(torch, data)
    xm = np.atleast_2d(x)
    xt = dev_bytes(torch, xm)
    y = torch.full((xm.shape[0], out_dim), float("nan"), device="cuda", dtype=torch.float32)
    ref = make_ref(F, wt, fmt, out_dim, in_dim, variant)
    ctx.matvec(ref, xt.data_ptr(), y.data_ptr(), xm.shape[0], in_dim, out_dim, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    out = y.cpu().numpy()
    return out[0] if np.ndim(x) == 1 else out


# ---------------------------------------------------------------- dequant ----
@pytest.mark.parametrize("name", list(FMTS))
def test_dequant_bit_exact_vs_golden(env, name):
    torch, F, ctx = env
    fmt = FMTS[name]
    rows, in_dim = (int(v) for v in GOLD[f"{name}_shape"])
    for key, nrows in ((name, rows), (f"{name}_edge", 4)):
        wt = dev_bytes(torch, GOLD[f"{key}_data"])
        out = torch.empty((nrows, in_dim), device="cuda", dtype=torch.float32)
        ctx.dequant_rows(make_ref(F, wt, fmt, nrows, in_dim), 0, nrows, out.data_ptr())
        torch.cuda.synchronize()
        assert_same_floats(out.cpu().numpy(), GOLD[f"{key}_out"])


@pytest.mark.parametrize("fmt", QUANT)
def test_dequant_bit_exact_vs_oracle_random_bytes(env, fmt):
    """Every byte pattern, including NaN / inf / subnormal fp16 scales."""
    torch, F, ctx = env
    rows, in_dim = 37, 1024
    data = np.random.default_rng(fmt).integers(0, 256, synth.tensor_bytes(fmt, rows, in_dim), dtype=np.uint8)
    wt = dev_bytes(torch, data)
    for variant in (0, 1):
        out = torch.empty((rows - 5, in_dim), device="cuda", dtype=torch.float32)
        ctx.dequant_rows(make_ref(F, wt, fmt, rows, in_dim, variant), 5, rows - 5, out.data_ptr())
        torch.cuda.synchronize()
        want = oracle.decode_rows(fmt, data, rows, in_dim, row0=5, layout=variant)
        assert_same_floats(out.cpu().numpy(), want)


def test_dequant_unquantized_formats(env):
    torch, F, ctx = env
    rng = np.random.default_rng(1)
    raw = rng.integers(0, 65536, (3, 64), dtype=np.uint16)
    for fmt in (synth.F16, synth.BF16):
        wt = dev_bytes(torch, raw.view(np.uint8).reshape(-1))
        out = torch.empty((3, 64), device="cuda", dtype=torch.float32)
        ctx.dequant_rows(make_ref(F, wt, fmt, 3, 64), 0, 3, out.data_ptr())
        torch.cuda.synchronize()
        want = oracle.decode_rows(fmt, raw.view(np.uint8).reshape(-1), 3, 64)
        assert_same_floats(out.cpu().numpy(), want)


# ----------------------------------------------------------------- matvec ----
def test_known_answer_vectors(env):
    from test_oracle import kat_f32, kat_q4_k, kat_q8_0
    data, x, expected, od, idim = kat_q8_0()
    y = gpu_matvec(env, synth.Q8_0, data, od, idim, x)
    assert np.max(np.abs(y - expected)) < 0.01                       # tests/test_q8_0.m:106
    data, x, expected, od, idim = kat_q4_k()
    y = gpu_matvec(env, synth.Q4_K, data, od, idim, x)
    assert np.all(np.abs(y - expected) / np.abs(expected) < 0.1)     # tests/test_q4k.m:93
    data, x, expected, od, idim = kat_f32()
    y = gpu_matvec(env, synth.F32, data, od, idim, x)
    assert np.max(np.abs(y - expected)) < 0.01                       # tests/test_f32.m:56


SHAPES = [(1, 256), (3, 512), (33, 1024), (64, 4096), (100, 5120), (257, 2048), (31, 768), (40, 12288), (18, 17408)]


@pytest.mark.parametrize("fmt", QUANT)
@pytest.mark.parametrize("x_bits", [24, 16])
def test_matvec_matches_oracle(env, fmt, x_bits):
    torch, F, ctx = env
    ctx.set_option(F.OPT_X_BITS, x_bits)
    try:
        for out_dim, in_dim in SHAPES:
            data = synth.host_tensor(fmt, out_dim, in_dim, seed=synth.seed_for("mv", fmt, out_dim, in_dim))
            x = synth.host_x(in_dim, seed=out_dim)
            for variant in ((0, 1) if fmt in (synth.Q4_K, synth.Q5_K) else (0,)):
                y = gpu_matvec(env, fmt, data, out_dim, in_dim, x, variant)
                want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x, layout=variant)
                if out_dim >= 16:
                    err = rel_l2(y, want)
                else:
                    # a handful of outputs can sit near zero by cancellation (the K-quant min term); measure the
                    # error against the size a row's output has without cancellation, |w_r| |x| / sqrt(in_dim)
                    w = oracle.decode_rows(fmt, data, out_dim, in_dim, layout=variant).astype(np.float64)
                    scale = np.linalg.norm(w) * np.linalg.norm(x) / np.sqrt(in_dim)
                    err = float(np.linalg.norm(y - want) / max(np.linalg.norm(want), scale))
                assert err <= REL_L2_TOL, (fmt, out_dim, in_dim, variant, err)
                if x_bits == 24:
                    assert err <= 2e-6, (fmt, out_dim, in_dim, variant, err)
    finally:
        ctx.set_option(F.OPT_X_BITS, 24)


@pytest.mark.parametrize("fmt", QUANT)
def test_generic_and_pipelined_kernels_agree(env, fmt):
    torch, F, ctx = env
    out_dim, in_dim = 129, 4096
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=77)
    x = synth.host_x(in_dim, seed=78)
    y_pipe = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
    ctx.set_option(F.OPT_FORCE_GENERIC, 1)
    try:
        y_gen = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
    finally:
        ctx.set_option(F.OPT_FORCE_GENERIC, 0)
    want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
    assert rel_l2(y_gen, want) <= 2e-6 and rel_l2(y_pipe, want) <= 2e-6


@pytest.mark.parametrize("fmt", QUANT)
@pytest.mark.parametrize("shape", [(47360, 256), (6000, 1024), (2500, 5120)])
def test_matvec_many_rows_per_cta(env, fmt, shape):
    """Shapes that give every CTA several row tiles: stage ring wrap-around, the rotation of stages over the
    consumer groups, more than one flush of the partial sums."""
    out_dim, in_dim = shape
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=synth.seed_for("rows", fmt, out_dim))
    x = synth.host_x(in_dim, seed=5)
    y = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
    assert rel_l2(y, oracle.matvec_f64(fmt, data, out_dim, in_dim, x)) <= 2e-6


@pytest.mark.parametrize("fmt", [synth.Q4_K, synth.Q5_K, synth.Q6_K])
def test_kquant_mma_and_dp4a_kernels_agree(env, fmt):
    torch, F, ctx = env
    out_dim, in_dim = 3000, 2048
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=91)
    x = synth.host_x(in_dim, seed=92)
    want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
    c0 = ctx.launch_count
    y_mma = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
    ctx.set_option(F.OPT_KQUANT_MMA, 0)
    try:
        y_dp4a = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
    finally:
        ctx.set_option(F.OPT_KQUANT_MMA, 1)
    assert ctx.launch_count == c0 + 2
    assert rel_l2(y_mma, want) <= 2e-6 and rel_l2(y_dp4a, want) <= 2e-6


def test_matvec_x_edge_cases(env):
    """Zero vector, one huge element among tiny ones, denormal-sized inputs."""
    fmt, out_dim, in_dim = synth.Q8_0, 64, 1024
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=5)
    y = gpu_matvec(env, fmt, data, out_dim, in_dim, np.zeros(in_dim, np.float32))
    assert np.all(y == 0)
    x = synth.host_x(in_dim, seed=6) * np.float32(1e-3)
    x[17] = 1e4
    want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
    assert rel_l2(gpu_matvec(env, fmt, data, out_dim, in_dim, x), want) <= REL_L2_TOL
    x = synth.host_x(in_dim, seed=7) * np.float32(1e-30)
    want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
    assert rel_l2(gpu_matvec(env, fmt, data, out_dim, in_dim, x), want) <= REL_L2_TOL


@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K, synth.Q5_K])
@pytest.mark.parametrize("shape", [(300, 4096, 64), (200, 768, 20), (128, 2048, 7)])
def test_both_forms_of_the_tensor_core_product_agree(env, fmt, shape):
    """Dequantized weights in tensor memory (default) and staged in shared memory (OROME_OPT_TC_SLABS): the same fp16
    operands and fp32 accumulation, so the two results differ only by the order of the sum over K."""
    torch, F, ctx = env
    out_dim, in_dim, batch = shape
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=synth.seed_for("forms", fmt, *shape))
    x = synth.host_x(in_dim, batch, seed=19)
    want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
    got = {}
    for slabs in (0, 1):
        ctx.set_option(F.OPT_TC_SLABS, slabs)
        try:
            got[slabs] = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
        finally:
            ctx.set_option(F.OPT_TC_SLABS, 0)
        assert rel_l2(got[slabs], want) <= TC_REL_L2_TOL, (slabs, rel_l2(got[slabs], want))
    assert rel_l2(got[0], got[1]) <= 1e-6


@pytest.mark.parametrize("fmt", QUANT + [synth.F32])
@pytest.mark.parametrize("batch", [2, 8, 13])
def test_batched_matvec(env, fmt, batch):
    out_dim, in_dim = 70, 1024
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=batch)
    x = synth.host_x(in_dim, batch, seed=3)
    y = gpu_matvec(env, fmt, data, out_dim, in_dim, x)
    want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
    on_tensor_cores = batch >= 4 and fmt in QUANT
    assert y.shape == want.shape and rel_l2(y, want) <= (TC_REL_L2_TOL if on_tensor_cores else REL_L2_TOL)


@pytest.mark.parametrize("fmt", [synth.Q4_K, synth.Q5_K])
@pytest.mark.parametrize("shape", [(300, 4096), (70, 1024), (1000, 12288), (35, 256), (2100, 5120)])
def test_two_vectors_per_launch(env, fmt, shape):
    """Batches of two and three on Q4_K / Q5_K: the mma kernel multiplies two input vectors in one pass over the weights
    (one launch for two vectors, two for three), at both x widths and both scale layouts, inside the fp32-activation bound."""
    torch, F, ctx = env
    out_dim, in_dim = shape
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=synth.seed_for("two", fmt, *shape))
    try:
        for bits in (24, 16):
            ctx.set_option(F.OPT_X_BITS, bits)
            for batch, variant in ((2, 0), (3, 1)):
                x = synth.host_x(in_dim, batch, seed=31 + batch)
                before = ctx.launch_count
                y = gpu_matvec(env, fmt, data, out_dim, in_dim, x, variant)
                assert ctx.launch_count - before == (batch + 1) // 2
                want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x, layout=variant)
                col = np.linalg.norm(y - want, axis=1) / np.linalg.norm(want, axis=1)
                assert col.max() <= REL_L2_TOL, (fmt, shape, bits, batch, col)
    finally:
        ctx.set_option(F.OPT_X_BITS, 24)


@pytest.mark.parametrize("fmt", QUANT)
@pytest.mark.parametrize("shape", [(300, 4096, 64), (128, 1024, 33), (1000, 2048, 16), (257, 12288, 48), (96, 512, 100), (131, 1280, 9)])
def test_prefill_gemm_on_tensor_cores(env, fmt, shape):
    """Ragged row tiles, split-K, padded and multi-slice batches; both scale layouts for Q4_K / Q5_K.  Q6_K rows are
    only 2-byte aligned (1280 weights: 1050 bytes a row, so rows start at every residue of 2 mod 16)."""
    torch, F, ctx = env
    out_dim, in_dim, batch = shape
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=synth.seed_for("tc", fmt, *shape))
    x = synth.host_x(in_dim, batch, seed=17)
    for variant in ((0, 1) if fmt in (synth.Q4_K, synth.Q5_K) else (0,)):
        before = ctx.launch_count
        y = gpu_matvec(env, fmt, data, out_dim, in_dim, x, variant)
        assert 2 <= ctx.launch_count - before <= 3 * ((batch + 63) // 64)                      # pack + tensor-core kernel (+ split-K reduction)
        want = oracle.matvec_f64(fmt, data, out_dim, in_dim, x, layout=variant)
        err = rel_l2(y, want)
        assert err <= TC_REL_L2_TOL, (fmt, shape, variant, err)
        # every column individually, so that a misplaced batch column cannot hide in the norm
        col = np.linalg.norm(y - want, axis=1) / np.linalg.norm(want, axis=1)
        assert col.max() <= 3 * TC_REL_L2_TOL, (fmt, shape, variant, col.max())
    # the fp32-activation kernel on the same inputs stays within the tight bound
    ctx.set_option(F.OPT_TC_MIN_BATCH, 1 << 20)
    try:
        y32 = gpu_matvec(env, fmt, data, out_dim, in_dim, x[:4], 0)
    finally:
        ctx.set_option(F.OPT_TC_MIN_BATCH, 4)
    assert rel_l2(y32, oracle.matvec_f64(fmt, data, out_dim, in_dim, x[:4])) <= REL_L2_TOL


def test_format_dispatch_matvec_offsets_and_absent_tensor(env):
    torch, F, ctx = env
    fmt, out_dim, in_dim = synth.Q4_K, 48, 512
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=1)
    blob = np.concatenate([np.zeros(64, np.uint8), data])           # tensor at byte offset 64 of its buffer
    wt = dev_bytes(torch, blob)
    x = synth.host_x(in_dim, seed=2)
    inbuf = dev_bytes(torch, np.concatenate([np.zeros(8, np.float32), x]))
    outbuf = torch.zeros(out_dim + 4, device="cuda", dtype=torch.float32)
    ref = make_ref(F, wt, fmt, out_dim, in_dim, offset=64)
    ctx.format_dispatch_matvec(ref, inbuf.data_ptr(), 32, outbuf.data_ptr(), 16)
    torch.cuda.synchronize()
    got = outbuf.cpu().numpy()
    assert np.all(got[:4] == 0)
    assert rel_l2(got[4:], oracle.matvec_f64(fmt, data, out_dim, in_dim, x)) <= 2e-6
    # a NULL buffer is a silent no-op (format.m:247-250)
    outbuf.fill_(7.0)
    ctx.format_dispatch_matvec(F.tensor_ref(0, 0, fmt, out_dim, in_dim), inbuf.data_ptr(), 32, outbuf.data_ptr(), 16)
    torch.cuda.synchronize()
    assert torch.all(outbuf == 7.0)


def test_rejected_calls_return_codes(env):
    torch, F, ctx = env
    wt = torch.zeros(4096, device="cuda", dtype=torch.uint8)
    x = torch.zeros(4096, device="cuda")
    y = torch.zeros(4096, device="cuda")
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(make_ref(F, wt, synth.Q8_0, 4, 48), x.data_ptr(), y.data_ptr())
    assert e.value.code == F.EINVAL
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(make_ref(F, wt, 9, 4, 256), x.data_ptr(), y.data_ptr())
    assert e.value.code == F.ENOTSUP
    with pytest.raises(F.OromeError) as e:
        ctx.matvec(make_ref(F, wt, synth.Q4_K, 4, 256, offset=2), x.data_ptr(), y.data_ptr())
    assert e.value.code == F.EINVAL
    with pytest.raises(F.OromeError):
        ctx.dequant_rows(make_ref(F, wt, synth.Q8_0, 4, 256), 3, 2, y.data_ptr())


def test_matvec_group_shares_x(env):
    torch, F, ctx = env
    fmt, in_dim = synth.Q8_0, 4096
    dims = [96, 24, 24]
    datas = [synth.host_tensor(fmt, d, in_dim, seed=10 + i) for i, d in enumerate(dims)]
    wts = [dev_bytes(torch, d) for d in datas]
    x = synth.host_x(in_dim, seed=4)
    xt = dev_bytes(torch, x)
    ys = [torch.full((d,), float("nan"), device="cuda") for d in dims]
    ctx.matvec_group([make_ref(F, w, fmt, d, in_dim) for w, d in zip(wts, dims)], xt.data_ptr(), [y.data_ptr() for y in ys])
    torch.cuda.synchronize()
    for d, data, y in zip(dims, datas, ys):
        assert rel_l2(y.cpu().numpy(), oracle.matvec_f64(fmt, data, d, in_dim, x)) <= 2e-6


@pytest.mark.parametrize("fmt", [synth.Q4_K, synth.Q5_K, synth.Q6_K])
def test_matvec_group_and_fused_gate_up_many_rows(env, fmt):
    """Grouped tensors whose boundaries fall inside CTAs, and the fused gate/up form with several row tiles per CTA."""
    torch, F, ctx = env
    in_dim, dims = 1024, [4000, 1000, 1000]
    datas = [synth.host_tensor(fmt, d, in_dim, seed=40 + i) for i, d in enumerate(dims)]
    wts = [dev_bytes(torch, d) for d in datas]
    x = synth.host_x(in_dim, seed=6)
    xt = dev_bytes(torch, x)
    ys = [torch.full((d,), float("nan"), device="cuda") for d in dims]
    ctx.matvec_group([make_ref(F, w, fmt, d, in_dim) for w, d in zip(wts, dims)], xt.data_ptr(), [y.data_ptr() for y in ys])
    torch.cuda.synchronize()
    for d, data, y in zip(dims, datas, ys):
        assert rel_l2(y.cpu().numpy(), oracle.matvec_f64(fmt, data, d, in_dim, x)) <= 2e-6
    out_dim = 5000
    gd, ud = synth.host_tensor(fmt, out_dim, in_dim, seed=51), synth.host_tensor(fmt, out_dim, in_dim, seed=52)
    xs = x * np.float32(8.0)
    gt, ut, xt = dev_bytes(torch, gd), dev_bytes(torch, ud), dev_bytes(torch, xs)
    out = torch.full((out_dim,), float("nan"), device="cuda")
    ctx.gate_up_swiglu(make_ref(F, gt, fmt, out_dim, in_dim), make_ref(F, ut, fmt, out_dim, in_dim), xt.data_ptr(), out.data_ptr(), 1, 0, 0)
    torch.cuda.synchronize()
    want = oracle.swiglu_f64(oracle.matvec_f64(fmt, gd, out_dim, in_dim, xs), oracle.matvec_f64(fmt, ud, out_dim, in_dim, xs))
    assert rel_l2(out.cpu().numpy(), want) <= REL_L2_TOL


@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K, synth.Q6_K])
def test_gate_up_swiglu_prefill_batch(env, fmt):
    """A batch of nine: the two products run on the tensor cores (fp16 operands), the output is a product of the two
    results, so the bound is twice the tensor-core form's."""
    torch, F, ctx = env
    out_dim, in_dim, batch = 300, 2048, 9
    gd = synth.host_tensor(fmt, out_dim, in_dim, seed=41)
    ud = synth.host_tensor(fmt, out_dim, in_dim, seed=42)
    xm = synth.host_x(in_dim, batch, seed=43)
    gt, ut, xt = dev_bytes(torch, gd), dev_bytes(torch, ud), dev_bytes(torch, xm)
    out = torch.full((batch, out_dim), float("nan"), device="cuda")
    before = ctx.launch_count
    ctx.gate_up_swiglu(make_ref(F, gt, fmt, out_dim, in_dim), make_ref(F, ut, fmt, out_dim, in_dim), xt.data_ptr(), out.data_ptr(), batch, in_dim, out_dim)
    torch.cuda.synchronize()
    assert ctx.launch_count - before >= 4                          # pack + tensor-core kernel, twice (the elementwise pass is not counted)
    want = oracle.swiglu_f64(oracle.matvec_f64(fmt, gd, out_dim, in_dim, xm), oracle.matvec_f64(fmt, ud, out_dim, in_dim, xm))
    assert rel_l2(out.cpu().numpy(), want) <= 2 * TC_REL_L2_TOL


@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K, synth.Q6_K])
@pytest.mark.parametrize("batch", [1, 3])
def test_gate_up_swiglu(env, fmt, batch):
    torch, F, ctx = env
    out_dim, in_dim = 200, 2048
    gd = synth.host_tensor(fmt, out_dim, in_dim, seed=31)
    ud = synth.host_tensor(fmt, out_dim, in_dim, seed=32)
    x = synth.host_x(in_dim, batch, seed=33) * np.float32(8.0)      # large enough that silu is not in its linear range
    xm = np.atleast_2d(x)
    gt, ut, xt = dev_bytes(torch, gd), dev_bytes(torch, ud), dev_bytes(torch, xm)
    out = torch.full((batch, out_dim), float("nan"), device="cuda")
    for variant in ((0, 1) if fmt == synth.Q4_K else (0,)):
        ctx.gate_up_swiglu(make_ref(F, gt, fmt, out_dim, in_dim, variant), make_ref(F, ut, fmt, out_dim, in_dim, variant),
                           xt.data_ptr(), out.data_ptr(), batch, in_dim, out_dim)
        torch.cuda.synchronize()
        g = oracle.matvec_f64(fmt, gd, out_dim, in_dim, xm, layout=variant)
        u = oracle.matvec_f64(fmt, ud, out_dim, in_dim, xm, layout=variant)
        want = oracle.swiglu_f64(g, u)
        assert rel_l2(out.cpu().numpy(), want) <= REL_L2_TOL


def test_matvec_host_roundtrip(env):
    torch, F, ctx = env
    fmt, out_dim, in_dim = synth.Q6_K, 96, 1024
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=8)
    wt = dev_bytes(torch, data)
    x = synth.host_x(in_dim, seed=9)
    y = np.empty(out_dim, np.float32)
    ctx.matvec_host(make_ref(F, wt, fmt, out_dim, in_dim), x, y)
    assert rel_l2(y, oracle.matvec_f64(fmt, data, out_dim, in_dim, x)) <= 2e-6


def test_upload_keeps_offsets(env):
    torch, F, ctx = env
    fmt, out_dim, in_dim = synth.Q5_K, 16, 512
    data = synth.host_tensor(fmt, out_dim, in_dim, seed=12)
    blob = np.concatenate([np.arange(96, dtype=np.uint8), data])
    base = ctx.upload(blob)
    try:
        x = synth.host_x(in_dim, seed=13)
        xt = dev_bytes(torch, x)
        y = torch.empty(out_dim, device="cuda")
        ctx.matvec(F.tensor_ref(base, 96, fmt, out_dim, in_dim), xt.data_ptr(), y.data_ptr())
        torch.cuda.synchronize()
        assert rel_l2(y.cpu().numpy(), oracle.matvec_f64(fmt, data, out_dim, in_dim, x)) <= 2e-6
    finally:
        ctx.free(base)


# -------------------------------------------------------------------- MoE ----
def test_route_matches_oracle_including_ties(env):
    torch, F, ctx = env
    n_experts, hidden, T, K = 128, 2048, 9, 8
    W = synth.host_router(n_experts, hidden, seed=2)
    W[7] = W[3]                                                      # identical rows give exact ties
    W[90] = W[3]
    x = synth.host_x(hidden, T, seed=5)
    wt, xt = dev_bytes(torch, W.view(np.uint8).reshape(-1)), dev_bytes(torch, x)
    idx = torch.zeros((T, 8), device="cuda", dtype=torch.int32)
    w = torch.zeros((T, 8), device="cuda")
    logits = torch.zeros((T, n_experts), device="cuda")
    ctx.moe_route(make_ref(F, wt, synth.F32, n_experts, hidden), xt.data_ptr(), T, hidden, K, idx.data_ptr(), w.data_ptr(),
                  logits.data_ptr())
    torch.cuda.synchronize()
    lg = logits.cpu().numpy()
    assert rel_l2(lg, oracle.matvec_f64(synth.F32, W.view(np.uint8).reshape(-1), n_experts, hidden, x)) <= 1e-5
    for t in range(T):
        oi, ow = oracle.route(lg[t], K)                              # the oracle routes the SAME logits
        assert np.array_equal(idx[t].cpu().numpy().astype(np.uint32), oi)
        assert np.max(np.abs(w[t].cpu().numpy() - ow)) <= 1e-6
    # K < 8 zero-fills, K > 8 is capped
    for K2 in (3, 12):
        ctx.moe_route(make_ref(F, wt, synth.F32, n_experts, hidden), xt.data_ptr(), 1, hidden, K2, idx.data_ptr(), w.data_ptr())
        torch.cuda.synchronize()
        oi, ow = oracle.route(lg[0], K2)
        assert np.array_equal(idx[0].cpu().numpy().astype(np.uint32), oi)
        assert np.max(np.abs(w[0].cpu().numpy() - ow)) <= 1e-6


@pytest.mark.parametrize("kquant_mma", [1, 0])
@pytest.mark.parametrize("T", [1, 5])
@pytest.mark.parametrize("down_fmt", [synth.Q5_K, synth.Q4_K, synth.Q6_K])
def test_moe_ffn_matches_oracle(env, T, down_fmt, kquant_mma):
    """Both kernels behind the entry point: the mma kernel's MoE forms (Q4_K / Q5_K; a Q6_K down projection then runs
    on the dp4a kernel after an mma gate/up) and, with OROME_OPT_KQUANT_MMA = 0, the dp4a kernel for both phases."""
    torch, F, ctx = env
    H, M, E, K = 512, 256, 16, 8
    ctx.set_option(F.OPT_KQUANT_MMA, kquant_mma)
    try:
        for bits in (24, 16):                     # the down projection follows the option, the fused gate/up always reads 24 bits
            ctx.set_option(F.OPT_X_BITS, bits)
            _moe_ffn_case(env, T, down_fmt, H, M, E, K)
    finally:
        ctx.set_option(F.OPT_KQUANT_MMA, 1)
        ctx.set_option(F.OPT_X_BITS, 24)


@pytest.mark.parametrize("shape", [(768, 256, 6, 3, 1), (256, 512, 9, 8, 37), (1024, 768, 40, 5, 2)])
def test_moe_ffn_other_shapes(env, shape):
    """Fewer than eight experts per token, a token batch larger than the grid cap, rows of one to four superblocks."""
    H, M, E, K, T = shape
    _moe_ffn_case(env, T, synth.Q5_K, H, M, E, K)


def _moe_ffn_case(env, T, down_fmt, H, M, E, K):
    torch, F, ctx = env
    gate = synth.host_tensor(synth.Q4_K, E * M, H, seed=21)
    up = synth.host_tensor(synth.Q4_K, E * M, H, seed=22)
    down = synth.host_tensor(down_fmt, E * H, M, seed=23)
    sg, sd = synth.tensor_bytes(synth.Q4_K, M, H), synth.tensor_bytes(down_fmt, H, M)
    blob = np.concatenate([gate, up, down])
    wt = dev_bytes(torch, blob)
    x = synth.host_x(H, T, seed=24)
    xm = np.atleast_2d(x)
    rng = np.random.default_rng(25)
    idx = np.zeros((T, 8), np.uint32)                # eight slots per token, the first K in use
    w = np.zeros((T, 8), np.float32)
    for t in range(T):
        idx[t, :K] = rng.permutation(E)[:K]
        w[t, :K] = rng.random(K)
    w /= w.sum(1, keepdims=True)
    layer = F.ExpertLayerRef(wt.data_ptr(), F.ExpertProjRef(0, sg, synth.Q4_K), F.ExpertProjRef(gate.size, sg, synth.Q4_K),
                             F.ExpertProjRef(gate.size + up.size, sd, down_fmt))
    xt, it, wtt = dev_bytes(torch, xm), dev_bytes(torch, idx.view(np.int32)), dev_bytes(torch, w)
    act = torch.empty((T, K, M), device="cuda")
    out = torch.full((T, H), float("nan"), device="cuda")
    ctx.moe_ffn(layer, 0, xt.data_ptr(), T, H, it.data_ptr(), wtt.data_ptr(), K, H, M, act.data_ptr(), out.data_ptr(), H)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for t in range(T):
        want = oracle.moe_ffn_f64(gate, up, down, (synth.Q4_K, synth.Q4_K, down_fmt), (sg, sg, sd), xm[t], H, M, idx[t, :K], w[t, :K])
        assert rel_l2(got[t], want) <= REL_L2_TOL, (t, rel_l2(got[t], want))


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("T", [1, 3])
def test_moe_ffn_expert_parallel_shares_add_up(env, world, T):
    """Expert-parallel form on one GPU: every rank's share (its own experts only, packed from index 0) computed in turn;
    the shares must add up to the whole layer (the all-reduce of the multi-GPU run is this sum)."""
    from orome_b200 import rowsplit
    torch, F, ctx = env
    H, M, E, K, dfmt = 512, 256, 16, 8, synth.Q5_K
    gate = synth.host_tensor(synth.Q4_K, E * M, H, seed=61)
    up = synth.host_tensor(synth.Q4_K, E * M, H, seed=62)
    down = synth.host_tensor(dfmt, E * H, M, seed=63)
    sg, sd = synth.tensor_bytes(synth.Q4_K, M, H), synth.tensor_bytes(dfmt, H, M)
    xm = np.atleast_2d(synth.host_x(H, T, seed=64))
    rng = np.random.default_rng(65)
    idx = np.stack([rng.permutation(E)[:8] for _ in range(T)]).astype(np.uint32)
    idx[0, :] = np.arange(8)                      # token 0 selects nothing from the upper half: some rank gets no work for it
    w = rng.random((T, 8)).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    xt, it, wtt = dev_bytes(torch, xm), dev_bytes(torch, idx.view(np.int32)), dev_bytes(torch, w)
    total = np.zeros((T, H), np.float64)
    for rank in range(world):
        e0, e1 = rowsplit.shard_experts(E, rank, world)
        blob = np.concatenate([gate[e0 * sg:e1 * sg], up[e0 * sg:e1 * sg], down[e0 * sd:e1 * sd]])
        wt = dev_bytes(torch, blob)
        n = e1 - e0
        layer = F.ExpertLayerRef(wt.data_ptr(), F.ExpertProjRef(0, sg, synth.Q4_K), F.ExpertProjRef(n * sg, sg, synth.Q4_K),
                                 F.ExpertProjRef(2 * n * sg, sd, dfmt))
        act = torch.full((T, K, M), float("nan"), device="cuda")
        out = torch.full((T, H), float("nan"), device="cuda")
        loc = torch.zeros((T, 8), dtype=torch.int32, device="cuda")
        ctx.moe_ffn_shard(layer, 0, xt.data_ptr(), T, H, it.data_ptr(), wtt.data_ptr(), K, H, M, e0, n, loc.data_ptr(),
                          act.data_ptr(), out.data_ptr(), H)
        torch.cuda.synchronize()
        share = out.cpu().numpy().astype(np.float64)
        assert np.all(np.isfinite(share))
        total += share
    for t in range(T):
        want = oracle.moe_ffn_f64(gate, up, down, (synth.Q4_K, synth.Q4_K, dfmt), (sg, sg, sd), xm[t], H, M, idx[t], w[t])
        assert rel_l2(total[t], want) <= REL_L2_TOL


def test_seeded_random_shapes_every_entry_point(env):
    """Sixty seeded random cases over formats, shapes (ragged row counts, narrow to wide rows), layouts, x widths,
    batches, tensor offsets inside a larger buffer and the three dense entry points, each against the fp64 oracle."""
    torch, F, ctx = env
    rng = np.random.default_rng(20240607)
    widths = {synth.Q8_0: [64, 192, 1024, 4096, 8192], synth.Q4_K: [256, 768, 2048, 5120], synth.Q5_K: [256, 1024, 4096],
              synth.Q6_K: [256, 768, 2560]}
    for case in range(60):
        fmt = QUANT[case % 4]
        in_dim = int(rng.choice(widths[fmt]))
        out_dim = int(rng.integers(1, 700))
        variant = int(rng.integers(0, 2)) if fmt in (synth.Q4_K, synth.Q5_K) else 0
        bits = int(rng.choice([16, 24]))
        kind = ["matvec", "group", "gate_up", "batched"][int(rng.integers(0, 4))]
        pad = int(rng.integers(0, 8)) * 32                                  # the tensor starts `pad` bytes into its buffer
        ctx.set_option(F.OPT_X_BITS, bits)
        try:
            tol = 1e-4
            if kind == "batched":
                batch = int(rng.integers(2, 20))
                data = synth.host_tensor(fmt, out_dim, in_dim, seed=1000 + case)
                x = synth.host_x(in_dim, batch, seed=2000 + case)
                wt = dev_bytes(torch, np.concatenate([np.zeros(pad, np.uint8), data]))
                xt, y = dev_bytes(torch, x), torch.full((batch, out_dim), float("nan"), device="cuda")
                ctx.matvec(F.tensor_ref(wt.data_ptr(), pad, fmt, out_dim, in_dim, variant), xt.data_ptr(), y.data_ptr(), batch, in_dim, out_dim)
                got, want = y, oracle.matvec_f64(fmt, data, out_dim, in_dim, x, layout=variant)
                if batch >= 4 and in_dim % 256 == 0:
                    tol = TC_REL_L2_TOL
            elif kind == "gate_up":
                gd, ud = synth.host_tensor(fmt, out_dim, in_dim, seed=1000 + case), synth.host_tensor(fmt, out_dim, in_dim, seed=3000 + case)
                x = synth.host_x(in_dim, seed=2000 + case)
                gap = (-gd.size) % 32                                      # tensors start on 32-byte boundaries, as in a GGUF file
                wt = dev_bytes(torch, np.concatenate([np.zeros(pad, np.uint8), gd, np.zeros(gap, np.uint8), ud]))
                xt, y = dev_bytes(torch, x), torch.full((out_dim,), float("nan"), device="cuda")
                ctx.gate_up_swiglu(F.tensor_ref(wt.data_ptr(), pad, fmt, out_dim, in_dim, variant),
                                   F.tensor_ref(wt.data_ptr(), pad + gd.size + gap, fmt, out_dim, in_dim, variant), xt.data_ptr(), y.data_ptr())
                got = y
                want = oracle.swiglu_f64(oracle.matvec_f64(fmt, gd, out_dim, in_dim, x, layout=variant),
                                         oracle.matvec_f64(fmt, ud, out_dim, in_dim, x, layout=variant))
            else:
                n_t = 1 if kind == "matvec" else int(rng.integers(2, 5))
                rows = [out_dim] + [int(rng.integers(1, 300)) for _ in range(n_t - 1)]
                datas = [synth.host_tensor(fmt, r, in_dim, seed=1000 + 10 * case + i) for i, r in enumerate(rows)]
                x = synth.host_x(in_dim, seed=2000 + case)
                datas_al = [np.concatenate([d, np.zeros((-d.size) % 32, np.uint8)]) for d in datas]      # 32-byte aligned starts
                wt = dev_bytes(torch, np.concatenate([np.zeros(pad, np.uint8)] + datas_al))
                xt = dev_bytes(torch, x)
                ys = [torch.full((r,), float("nan"), device="cuda") for r in rows]
                offs = np.cumsum([pad] + [d.size for d in datas_al[:-1]])
                refs = [F.tensor_ref(wt.data_ptr(), int(o), fmt, r, in_dim, variant) for o, r in zip(offs, rows)]
                if kind == "matvec":
                    ctx.matvec(refs[0], xt.data_ptr(), ys[0].data_ptr())
                else:
                    ctx.matvec_group(refs, xt.data_ptr(), [y.data_ptr() for y in ys])
                got = torch.cat(ys)
                want = np.concatenate([oracle.matvec_f64(fmt, d, r, in_dim, x, layout=variant) for d, r in zip(datas, rows)])
            torch.cuda.synchronize()
            err = rel_l2(got.cpu().numpy(), want)
            assert err <= tol, (case, kind, fmt, out_dim, in_dim, variant, bits, pad, err)
        finally:
            ctx.set_option(F.OPT_X_BITS, 24)
