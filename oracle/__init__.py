"""CPU oracle for the quantized dequant-matvec path (ctypes over ``oracle.c``).

TEST INFRASTRUCTURE ONLY.  The shipped package (``orome_b200``) never imports this
module: it exists so that tests, the smoke check and the benchmark's CPU-baseline
leg can check or time the CUDA path against a CPU statement of the reference's
algorithm.  ``ref()`` additionally exposes the reference's own decode when it was
compiled from the reference tree (``oracle/_ref``).

Pinned against the reference's own code or vectors: the row decoders and fp16 conversion.
Parity unpinned (restated from the shader source, no reference-held vector): scale layout B,
routing, expert FFN / MoE block, arg-max tie order, residual / norm kernels.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

Q4_K, Q5_K, Q6_K, Q8_0, F16, BF16, F32 = range(7)   # inference/include/orome.h:227-235
LAYOUT_A, LAYOUT_B = 0, 1

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u32p = C.POINTER(C.c_uint32)

_lib = None
_ref = None


def _p(a, t):
    return a.ctypes.data_as(t)


def lib():
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        L = C.CDLL(path)
        L.oracle_half_to_float.restype = C.c_float
        L.oracle_half_to_float.argtypes = [C.c_uint16]
        L.oracle_row_bytes.restype = C.c_size_t
        L.oracle_row_bytes.argtypes = [C.c_int, C.c_uint32]
        L.oracle_kquant_scales.argtypes = [_u8p, C.c_int, _u8p, _u8p]
        L.oracle_decode_rows.argtypes = [C.c_int, C.c_int, C.c_int, _u8p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
        L.oracle_matvec_f64.argtypes = [C.c_int, C.c_int, _u8p, C.c_uint32, C.c_uint32, _f32p, C.c_int, C.c_int, _f64p, C.c_int]
        L.oracle_matvec_f32.argtypes = [C.c_int, C.c_int, _u8p, C.c_uint32, C.c_uint32, _f32p, C.c_int, C.c_int, _f32p, C.c_int]
        L.oracle_swiglu_f64.argtypes = [_f64p, _f64p, C.c_size_t, _f64p]
        L.oracle_route.argtypes = [_f32p, C.c_uint32, C.c_uint32, _u32p, _f32p]
        L.oracle_moe_ffn_f64.argtypes = [_u8p, C.c_size_t, C.c_int, _u8p, C.c_size_t, C.c_int, _u8p, C.c_size_t, C.c_int,
                                         C.c_int, _f32p, C.c_uint32, C.c_uint32, _u32p, _f32p, C.c_uint32, _f64p]
        L.oracle_argmax.restype = C.c_uint32
        L.oracle_argmax.argtypes = [_f32p, C.c_uint32]
        L.oracle_num_threads.restype = C.c_int
        _lib = L
    return _lib


def ref():
    """The reference's own decode (``oracle/_ref``), or None when it was never built."""
    global _ref
    if _ref is None:
        path = _build.build_ref()
        if path is None:
            return None
        L = C.CDLL(path)
        L.ref_fp16_to_f32.restype = C.c_float
        L.ref_fp16_to_f32.argtypes = [C.c_uint16]
        L.ref_unpack_scale_min_pair.argtypes = [_u8p, C.c_uint32, _f32p]
        L.ref_decode_rows.argtypes = [C.c_int, _u8p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
        L.ref_matvec_f32.argtypes = [C.c_int, _u8p, C.c_uint32, C.c_uint32, _f32p, C.c_int, C.c_int, _f32p, C.c_int]
        L.ref_num_threads.restype = C.c_int
        _ref = L
    return _ref


def row_bytes(fmt: int, in_dim: int) -> int:
    return int(lib().oracle_row_bytes(fmt, in_dim))


def half_to_float_bits(h: int) -> int:
    return int(np.float32(lib().oracle_half_to_float(h)).view(np.uint32))


def kquant_scales(packed12: np.ndarray, layout: int):
    p = np.ascontiguousarray(packed12, dtype=np.uint8)
    sc = np.zeros(8, np.uint8)
    mn = np.zeros(8, np.uint8)
    lib().oracle_kquant_scales(_p(p, _u8p), layout, _p(sc, _u8p), _p(mn, _u8p))
    return sc, mn


def _check(data: np.ndarray, fmt: int, out_dim: int, in_dim: int):
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    need = row_bytes(fmt, in_dim) * out_dim
    if data.size < need:
        raise ValueError(f"tensor needs {need} bytes, got {data.size}")
    return data


def decode_rows(fmt, data, out_dim, in_dim, row0=0, nrows=None, layout=LAYOUT_A, fused=False) -> np.ndarray:
    nrows = out_dim - row0 if nrows is None else nrows
    data = _check(data, fmt, out_dim, in_dim)
    out = np.empty((nrows, in_dim), np.float32)
    rc = lib().oracle_decode_rows(fmt, layout, int(fused), _p(data, _u8p), row0, nrows, in_dim, _p(out, _f32p))
    if rc:
        raise ValueError("decode failed (in_dim not a whole number of blocks?)")
    return out


def ref_decode_rows(fmt, data, out_dim, in_dim, row0=0, nrows=None) -> np.ndarray:
    R = ref()
    if R is None:
        raise RuntimeError("oracle/_ref was not built (reference tree absent)")
    nrows = out_dim - row0 if nrows is None else nrows
    data = _check(data, fmt, out_dim, in_dim)
    out = np.empty((nrows, in_dim), np.float32)
    rc = R.ref_decode_rows(fmt, _p(data, _u8p), row0, nrows, in_dim, _p(out, _f32p))
    if rc:
        raise ValueError("reference decode failed")
    return out


def _xmat(x, in_dim):
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    assert x.shape[1] == in_dim
    return x


def matvec_f64(fmt, data, out_dim, in_dim, x, layout=LAYOUT_A) -> np.ndarray:
    """y[b, r] in float64: decoded fp32 weights times x, accumulated in double."""
    data = _check(data, fmt, out_dim, in_dim)
    xm = _xmat(x, in_dim)
    y = np.empty((xm.shape[0], out_dim), np.float64)
    rc = lib().oracle_matvec_f64(fmt, layout, _p(data, _u8p), out_dim, in_dim, _p(xm, _f32p), xm.shape[0], in_dim,
                                 _p(y, _f64p), out_dim)
    if rc:
        raise ValueError("matvec failed")
    return y[0] if np.ndim(x) == 1 else y


def matvec_f32(fmt, data, out_dim, in_dim, x, layout=LAYOUT_A, use_ref=False) -> np.ndarray:
    """fp32-accumulated form (the CPU baseline that gets timed)."""
    data = _check(data, fmt, out_dim, in_dim)
    xm = _xmat(x, in_dim)
    y = np.empty((xm.shape[0], out_dim), np.float32)
    if use_ref:
        rc = ref().ref_matvec_f32(fmt, _p(data, _u8p), out_dim, in_dim, _p(xm, _f32p), xm.shape[0], in_dim,
                                  _p(y, _f32p), out_dim)
    else:
        rc = lib().oracle_matvec_f32(fmt, layout, _p(data, _u8p), out_dim, in_dim, _p(xm, _f32p), xm.shape[0], in_dim,
                                     _p(y, _f32p), out_dim)
    if rc:
        raise ValueError("matvec failed")
    return y[0] if np.ndim(x) == 1 else y


def swiglu_f64(gate, up) -> np.ndarray:
    g = np.ascontiguousarray(gate, np.float64)
    u = np.ascontiguousarray(up, np.float64)
    out = np.empty_like(g)
    lib().oracle_swiglu_f64(_p(g, _f64p), _p(u, _f64p), g.size, _p(out, _f64p))
    return out


def route(logits, K):
    """(idx[8] uint32, w[8] float32) for one token's router logits."""
    lg = np.ascontiguousarray(logits, np.float32)
    idx = np.zeros(8, np.uint32)
    w = np.zeros(8, np.float32)
    lib().oracle_route(_p(lg, _f32p), lg.size, K, _p(idx, _u32p), _p(w, _f32p))
    return idx, w


def moe_ffn_f64(gate, up, down, fmts, strides, x, hidden, inter, idx, w, layout=LAYOUT_A) -> np.ndarray:
    """Weighted sum over the K selected experts of down(silu(gate x) * up x), in double.

    gate/up/down are the whole 3-D expert tensors as bytes; fmts = (gate, up, down)
    formats, strides = bytes between consecutive experts of each."""
    gate = np.ascontiguousarray(gate, np.uint8).reshape(-1)
    up = np.ascontiguousarray(up, np.uint8).reshape(-1)
    down = np.ascontiguousarray(down, np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, np.float32)
    idx = np.ascontiguousarray(idx, np.uint32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty(hidden, np.float64)
    rc = lib().oracle_moe_ffn_f64(_p(gate, _u8p), strides[0], fmts[0], _p(up, _u8p), strides[1], fmts[1],
                                  _p(down, _u8p), strides[2], fmts[2], layout, _p(x, _f32p), hidden, inter,
                                  _p(idx, _u32p), _p(w, _f32p), idx.size, _p(out, _f64p))
    if rc:
        raise ValueError("moe ffn failed")
    return out


def moe_block_f64(gate, up, down, fmts, strides, shared, x, hidden, inter, idx, w, shared_logit, h_mid=None, layout=LAYOUT_A) -> np.ndarray:
    """One token through the MoE block of encode_experts_gguf (engine.m:158-340), in double:
    h_mid + sum_k w_k FFN_k(x) + sigmoid(shared_logit) * SharedFFN(x), the value moe_combine_copy_sq writes to hidden_out
    (shaders.metal:1049-1059; sigmoid as 1 / (1 + exp(-p)), line 1051).  shared: None or
    ((fmt, bytes, S), (fmt, bytes, S), (fmt, bytes)) for the shared gate, up and down tensors; the shared activation is
    rounded to fp32 before its down projection, as the buffer between the two kernels is (engine.m:263-316)."""
    out = moe_ffn_f64(gate, up, down, fmts, strides, x, hidden, inter, idx, w, layout=layout)
    if h_mid is not None:
        out = out + np.asarray(h_mid, np.float64)
    if shared is not None:
        (gf, gb, S), (uf, ub, _), (df, db) = shared
        act = swiglu_f64(matvec_f64(gf, gb, S, hidden, x, layout=layout), matvec_f64(uf, ub, S, hidden, x, layout=layout)).astype(np.float32)
        sh = matvec_f64(df, db, hidden, S, act, layout=layout)
        out = out + 1.0 / (1.0 + np.exp(-np.float64(shared_logit))) * sh
    return out


def residual_add_sum_sq(a, b, tg: int = 256):
    """residual_add_sum_sq (inference/src/shaders.metal:86-124): out = clamp(a + b, -65504, 65504) in fp32 and one
    partial sum of out^2 per threadgroup of `tg` elements (engine.m:628-638 dispatches ceil(dim / 256) groups of 256).
    Returns (out float32, parts float32); parity unpinned (restates the shader, no reference-held vector covers it)."""
    out = np.clip(np.asarray(a, np.float32) + np.asarray(b, np.float32), np.float32(-65504.0), np.float32(65504.0)).astype(np.float32)
    parts = np.array([np.sum(out[i:i + tg].astype(np.float64) ** 2) for i in range(0, out.size, tg)], np.float64)
    return out, parts.astype(np.float32)


def rms_norm_apply_partial(x, weight_bf16, parts, eps: float) -> np.ndarray:
    """rms_norm_apply_partial (shaders.metal:126-149): the partial sums added up in order in fp32, then
    x * rsqrt(total / dim + eps) * bf16 weight, fp32 products in that order.  weight_bf16: uint16 bit patterns."""
    x = np.asarray(x, np.float32)
    total = np.float32(0.0)
    for p in np.asarray(parts, np.float32):
        total = np.float32(total + p)
    rms = np.float32(1.0) / np.sqrt(np.float32(total / np.float32(x.size) + np.float32(eps)), dtype=np.float32)
    w = (np.asarray(weight_bf16, np.uint16).astype(np.uint32) << 16).view(np.float32)
    return ((x * rms).astype(np.float32) * w).astype(np.float32)


def argmax(data) -> int:
    """Index the reference's argmax_kernel returns for this vector (ties resolved as its 1024 threads do)."""
    d = np.ascontiguousarray(data, np.float32).reshape(-1)
    return int(lib().oracle_argmax(_p(d, _f32p), d.size))


def use_all_cores() -> int:
    """Make the OpenMP loops of both checkers use every host core (torchrun sets OMP_NUM_THREADS=1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(n)
    if ref() is not None:
        ref().ref_set_threads(n)
    return n


def num_threads() -> int:
    return int(lib().oracle_num_threads())
