"""Pin the CPU oracle: against the committed golden vectors (made by the reference's
own format.m decode), against the reference build itself when it is present, and
against the closed-form known-answer vectors of the reference's kernel tests."""
import os

import numpy as np
import pytest

import oracle
from orome_b200 import synth

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "decode_golden.npz"))
FMTS = {"Q8_0": synth.Q8_0, "Q4_K": synth.Q4_K, "Q5_K": synth.Q5_K, "Q6_K": synth.Q6_K}


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_half_to_float_all_65536_match_reference_bits():
    got = np.array([oracle.half_to_float_bits(h) for h in range(65536)], np.uint32)
    assert np.array_equal(got, GOLD["fp16_bits"])


def test_scale_layout_a_matches_reference_unpack():
    for field, pairs in zip(GOLD["scale_fields"], GOLD["scale_pairs"]):
        sc, mn = oracle.kquant_scales(field, oracle.LAYOUT_A)
        for g in range(4):
            assert [sc[2 * g], sc[2 * g + 1], mn[2 * g], mn[2 * g + 1]] == list(pairs[g])


def test_scale_layouts_agree_only_where_documented():
    rng = np.random.default_rng(3)
    diff_sc = np.zeros(8, bool)
    diff_mn = np.zeros(8, bool)
    for _ in range(200):
        f = rng.integers(0, 256, 12, dtype=np.uint8)
        sa, ma = oracle.kquant_scales(f, oracle.LAYOUT_A)
        sb, mb = oracle.kquant_scales(f, oracle.LAYOUT_B)
        diff_sc |= sa != sb
        diff_mn |= ma != mb
    assert list(np.nonzero(diff_sc)[0]) == [5, 6, 7]
    assert list(np.nonzero(diff_mn)[0]) == [4, 5, 6]


@pytest.mark.parametrize("name", list(FMTS))
def test_decode_bit_exact_vs_golden(name):
    fmt = FMTS[name]
    rows, in_dim = GOLD[f"{name}_shape"]
    got = oracle.decode_rows(fmt, GOLD[f"{name}_data"], rows, in_dim)
    assert np.array_equal(bits(got), bits(GOLD[f"{name}_out"]))
    got = oracle.decode_rows(fmt, GOLD[f"{name}_edge_data"], 4, in_dim)
    assert np.array_equal(bits(got), bits(GOLD[f"{name}_edge_out"]))


@pytest.mark.parametrize("name", list(FMTS))
def test_decode_bit_exact_vs_reference_build(name):
    if oracle.ref() is None:
        pytest.skip("reference tree not mounted; golden fixtures cover this")
    fmt = FMTS[name]
    for seed, (rows, in_dim) in enumerate([(3, 256), (17, 1024), (64, 4096)]):
        data = synth.host_tensor(fmt, rows, in_dim, seed=100 + seed)
        # arbitrary bytes everywhere (including NaN/inf scales) must decode identically too
        raw = np.random.default_rng(seed).integers(0, 256, data.size, dtype=np.uint8)
        for d in (data, raw):
            a = oracle.decode_rows(fmt, d, rows, in_dim)
            b = oracle.ref_decode_rows(fmt, d, rows, in_dim)
            assert np.array_equal(bits(a), bits(b))


def test_decode_rejects_ragged_in_dim():
    with pytest.raises(ValueError):
        oracle.decode_rows(synth.Q8_0, np.zeros(4096, np.uint8), 1, 48)
    with pytest.raises(ValueError):
        oracle.decode_rows(synth.Q4_K, np.zeros(4096, np.uint8), 1, 384)


def _trunc_half(v):
    """The truncating float->half used by the reference's tests (tests/test_q8_0.m:49-58)."""
    b = int(np.float32(v).view(np.uint32))
    sign = (b >> 31) & 1
    exp = ((b >> 23) & 0xFF) - 127 + 15
    mant = (b >> 13) & 0x3FF
    if exp <= 0:
        return 0
    if exp >= 31:
        return (sign << 15) | (31 << 10)
    return (sign << 15) | (exp << 10) | mant


def kat_q8_0():
    """tests/test_q8_0.m:27-70: 64x256, d = half(0.01*(row+1)), q = (blk*32+j)%127-63, x = 0.01*(j%10)."""
    out_dim, in_dim = 64, 256
    data = np.zeros((out_dim, in_dim // 32, 34), np.uint8)
    x = (np.float32(0.01) * (np.arange(in_dim) % 10).astype(np.float32)).astype(np.float32)
    expected = np.zeros(out_dim, np.float32)
    for r in range(out_dim):
        scale = np.float32(0.01) * np.float32(r + 1)
        h = _trunc_half(scale)
        acc = np.float32(0)
        for b in range(in_dim // 32):
            data[r, b, 0] = h & 0xFF
            data[r, b, 1] = h >> 8
            for j in range(32):
                q = (b * 32 + j) % 127 - 63
                data[r, b, 2 + j] = np.int8(q).view(np.uint8)
                acc = np.float32(acc + np.float32(np.float32(scale * np.float32(q)) * x[b * 32 + j]))
        expected[r] = acc
    return data.reshape(-1), x, expected, out_dim, in_dim


def kat_q4_k():
    """tests/test_q4k.m:19-67: 4x256, d = 0.1*(row+1), dmin = 0.01, scales 1 / mins 0 (layout A), nibbles 5, x = 0.01."""
    out_dim, in_dim = 4, 256
    data = np.zeros((out_dim, 144), np.uint8)
    expected = np.zeros(out_dim, np.float32)
    for r in range(out_dim):
        d = np.float32(0.1) * np.float32(r + 1)
        for col, v in ((0, d), (2, np.float32(0.01))):
            h = _trunc_half(v)
            data[r, col] = h & 0xFF
            data[r, col + 1] = h >> 8
        data[r, 4:8] = 1
        data[r, 12] = 0x11
        data[r, 13] = 0x11
        data[r, 16:] = 0x55
        expected[r] = np.float32(256.0) * np.float32(5.0) * d * np.float32(0.01)
    x = np.full(in_dim, 0.01, np.float32)
    return data.reshape(-1), x, expected, out_dim, in_dim


def kat_f32():
    """tests/test_f32.m:17-30: 32x64, W = 0.01*(i-j), x = 0.1*(j%5), fp32 dot."""
    out_dim, in_dim = 32, 64
    i = np.arange(out_dim)[:, None]
    j = np.arange(in_dim)[None, :]
    W = (np.float32(0.01) * (i - j).astype(np.float32)).astype(np.float32)
    x = (np.float32(0.1) * (np.arange(in_dim) % 5).astype(np.float32)).astype(np.float32)
    expected = np.zeros(out_dim, np.float32)
    for r in range(out_dim):
        acc = np.float32(0)
        for c in range(in_dim):
            acc = np.float32(acc + np.float32(W[r, c] * x[c]))
        expected[r] = acc
    return W.view(np.uint8).reshape(-1), x, expected, out_dim, in_dim


def test_known_answer_q8_0():
    data, x, expected, od, idim = kat_q8_0()
    y = oracle.matvec_f64(synth.Q8_0, data, od, idim, x)
    assert np.max(np.abs(y - expected)) < 0.01          # the reference test's tolerance (test_q8_0.m:106)
    # the scales are exactly the truncated halves
    w = oracle.decode_rows(synth.Q8_0, data, od, idim)
    d0 = np.array([_trunc_half(np.float32(0.01))], np.uint16).view(np.float16).astype(np.float32)[0]
    assert w[0, 0] == d0 * np.float32(-63)
    assert abs(w[9, 5] / np.float32(5 % 127 - 63) - 0.1) < 1e-4


def test_known_answer_q4_k_layout_a_only():
    data, x, expected, od, idim = kat_q4_k()
    y = oracle.matvec_f64(synth.Q4_K, data, od, idim, x, layout=oracle.LAYOUT_A)
    rel = np.abs(y - expected) / np.abs(expected)
    assert np.all(rel < 0.1)                             # test_q4k.m:93
    assert np.all(rel < 1e-3)                            # in fact limited only by the truncated halves
    # the same bytes under layout B give scales [1,1,1,1,1,1,0,0] and mins [0,0,0,0,1,1,0,0]
    sc, mn = oracle.kquant_scales(data[4:16], oracle.LAYOUT_B)
    assert list(sc) == [1, 1, 1, 1, 1, 1, 0, 0] and list(mn) == [0, 0, 0, 0, 1, 1, 0, 0]
    sc, mn = oracle.kquant_scales(data[4:16], oracle.LAYOUT_A)
    assert list(sc) == [1] * 8 and list(mn) == [0] * 8


def test_known_answer_f32():
    data, x, expected, od, idim = kat_f32()
    y = oracle.matvec_f32(synth.F32, data, od, idim, x)
    assert np.array_equal(bits(y), bits(expected))       # same order of fp32 operations
    y64 = oracle.matvec_f64(synth.F32, data, od, idim, x)
    assert np.max(np.abs(y64 - expected)) < 0.01         # test_f32.m:56


def test_numpy_q8_0_dequant_agrees():
    """Independent numpy Q8_0 decode as in tests/verify_gguf.py:49-59 (float16 view times int8)."""
    rows, in_dim = 7, 512
    data = synth.host_tensor(synth.Q8_0, rows, in_dim, seed=5)
    blocks = data.reshape(rows, in_dim // 32, 34)
    d = blocks[:, :, :2].copy().view(np.float16).astype(np.float32)
    q = blocks[:, :, 2:].copy().view(np.int8).astype(np.float32)
    want = (d * q).reshape(rows, in_dim)
    got = oracle.decode_rows(synth.Q8_0, data, rows, in_dim)
    assert np.array_equal(bits(got), bits(want))


def test_fused_twin_is_bit_identical():
    """a = d*sc has at most 11+6 significant bits and q at most 5, so a*q is exact in
    fp32 and `a*q - m` rounds once whether or not the compiler contracts it to an FMA:
    the contraction mode cannot change a decoded Q4_K / Q5_K weight."""
    for fmt in (synth.Q4_K, synth.Q5_K):
        data = np.random.default_rng(11).integers(0, 256, synth.tensor_bytes(fmt, 16, 1024), dtype=np.uint8)
        a = oracle.decode_rows(fmt, data, 16, 1024, fused=False)
        b = oracle.decode_rows(fmt, data, 16, 1024, fused=True)
        assert np.array_equal(bits(a), bits(b))


def test_matvec_f32_close_to_f64_and_linear():
    for fmt in (synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K):
        data = synth.host_tensor(fmt, 33, 512, seed=fmt)
        x = synth.host_x(512, 3, seed=9)
        y64 = oracle.matvec_f64(fmt, data, 33, 512, x)
        y32 = oracle.matvec_f32(fmt, data, 33, 512, x)
        assert y64.shape == (3, 33)
        assert np.linalg.norm(y32 - y64) / np.linalg.norm(y64) < 1e-5
        ysum = oracle.matvec_f64(fmt, data, 33, 512, (x[0] + x[1]).astype(np.float32))
        # linear up to the rounding of x0+x1 to fp32
        assert np.linalg.norm(ysum - (y64[0] + y64[1])) / np.linalg.norm(ysum) < 1e-6


def test_route_ties_lowest_index_and_softmax_over_selected():
    logits = np.zeros(128, np.float32)
    logits[[5, 9, 77]] = 2.0
    logits[100] = 3.0
    idx, w = oracle.route(logits, 8)
    assert list(idx[:4]) == [100, 5, 9, 77]
    assert list(idx[4:]) == [0, 1, 2, 3]                  # remaining zeros in index order
    e = np.exp(np.array([0, -1, -1, -1, -3, -3, -3, -3], np.float64))
    assert np.allclose(w, e / e.sum(), atol=1e-6)
    idx, w = oracle.route(logits, 3)                      # K < 8 zero-fills the rest
    assert list(idx) == [100, 5, 9, 0, 0, 0, 0, 0] and np.all(w[3:] == 0)
    idx, w = oracle.route(logits, 12)                     # K is capped at 8 (shaders.metal:1164)
    assert abs(w.sum() - 1) < 1e-6


def test_moe_ffn_matches_manual_composition():
    H, M, E, K = 512, 256, 6, 3
    gate = synth.host_tensor(synth.Q4_K, E * M, H, seed=21)
    up = synth.host_tensor(synth.Q4_K, E * M, H, seed=22)
    down = synth.host_tensor(synth.Q5_K, E * H, M, seed=23)
    sg = synth.tensor_bytes(synth.Q4_K, M, H)
    sd = synth.tensor_bytes(synth.Q5_K, H, M)
    x = synth.host_x(H, seed=24)
    idx = np.array([4, 0, 5], np.uint32)
    w = np.array([0.5, 0.3, 0.2], np.float32)
    got = oracle.moe_ffn_f64(gate, up, down, (synth.Q4_K, synth.Q4_K, synth.Q5_K), (sg, sg, sd), x, H, M, idx, w)
    want = np.zeros(H)
    for e, wk in zip(idx, w):
        g = oracle.matvec_f64(synth.Q4_K, gate[e * sg:(e + 1) * sg], M, H, x)
        u = oracle.matvec_f64(synth.Q4_K, up[e * sg:(e + 1) * sg], M, H, x)
        act = (g / (1 + np.exp(-g)) * u).astype(np.float32)
        want += float(wk) * oracle.matvec_f64(synth.Q5_K, down[e * sd:(e + 1) * sd], H, M, act)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)


def test_norm_restatements_known_answers():
    # shaders.metal:86-149: clamp to the fp16 range, one partial per 256 elements, weights are bf16 bit patterns
    a = np.full(600, 2.0, np.float32)
    b = np.full(600, 1.0, np.float32)
    a[3], b[3] = 65000.0, 1000.0
    a[4], b[4] = -65000.0, -1000.0
    out, parts = oracle.residual_add_sum_sq(a, b)
    assert out[3] == np.float32(65504.0) and out[4] == np.float32(-65504.0) and out[5] == np.float32(3.0)
    assert parts.size == 3 and parts[1] == np.float32(256 * 9.0) and parts[2] == np.float32(88 * 9.0)
    x = np.full(512, 3.0, np.float32)
    one, half = np.uint16(0x3F80), np.uint16(0x3F00)
    w = np.where(np.arange(512) % 2 == 0, one, half).astype(np.uint16)
    y = oracle.rms_norm_apply_partial(x, w, np.array([256 * 9.0, 256 * 9.0], np.float32), 0.0)
    assert np.allclose(y[0::2], 1.0, rtol=1e-6) and np.allclose(y[1::2], 0.5, rtol=1e-6)
