"""Seeded synthetic GGUF block tensors (stand-ins for the Qwen3.5 GGUF files).

Block layouts follow the reference's decoders (inference/src/format.m:66-174):

* Q8_0  34 B / 32 weights : fp16 d, int8 q[32]
* Q4_K 144 B / 256 weights: fp16 d, fp16 dmin, 12 B packed 6-bit scales/mins, 128 B nibbles
* Q5_K 176 B / 256 weights: as Q4_K with 32 B of high bits before the nibbles
* Q6_K 210 B / 256 weights: 128 B low nibbles, 64 B high 2-bit pairs, int8 sc[16], fp16 d

Value distributions: d = fp16(|N(0,0.02)|/127) for Q8_0 and fp16(|N(0,0.01)|) for
the K-quants, quants and packed scale bytes uniform over every bit pattern (so
the six-bit fields are uniform under either scale layout), Q6_K sub-scales
uniform in [-32, 31].  ``host_*`` builds numpy arrays for tests; ``device_*``
fills a CUDA buffer in place with torch for benchmark-sized tensors.
"""
from __future__ import annotations

import zlib

import numpy as np

Q4_K, Q5_K, Q6_K, Q8_0, F16, BF16, F32 = range(7)   # QuantFormat order, inference/include/orome.h:227-235

BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210}
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256}
FORMAT_NAMES = {Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", Q8_0: "Q8_0", F16: "F16", BF16: "BF16", F32: "F32"}


def row_bytes(fmt: int, in_dim: int) -> int:
    if fmt == F32:
        return in_dim * 4
    if fmt in (F16, BF16):
        return in_dim * 2
    if in_dim % BLOCK_ELEMS[fmt]:
        raise ValueError(f"in_dim {in_dim} is not a multiple of {BLOCK_ELEMS[fmt]}")
    return in_dim // BLOCK_ELEMS[fmt] * BLOCK_BYTES[fmt]


def tensor_bytes(fmt: int, out_dim: int, in_dim: int) -> int:
    return out_dim * row_bytes(fmt, in_dim)


def seed_for(*parts) -> int:
    """Stable per-tensor seed from (config, tensor name, layer, ...)."""
    return zlib.crc32("/".join(str(p) for p in parts).encode())


def _put_f16(blocks: np.ndarray, col: int, vals: np.ndarray) -> None:
    blocks[:, col:col + 2] = vals.astype(np.float16).view(np.uint8).reshape(-1, 2)


def host_tensor(fmt: int, out_dim: int, in_dim: int, seed: int = 0) -> np.ndarray:
    """Packed tensor bytes, shape [out_dim * row_bytes] uint8."""
    rng = np.random.default_rng(seed)
    if fmt == F32:
        return rng.standard_normal((out_dim, in_dim), dtype=np.float32).view(np.uint8).reshape(-1)
    nblk = out_dim * (in_dim // BLOCK_ELEMS[fmt])
    bb = BLOCK_BYTES[fmt]
    blocks = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)
    if fmt == Q8_0:
        q = rng.integers(-127, 128, size=(nblk, 32), dtype=np.int8)
        blocks[:, 2:] = q.view(np.uint8)
        _put_f16(blocks, 0, np.abs(rng.normal(0.0, 0.02, nblk)) / 127.0)
    elif fmt in (Q4_K, Q5_K):
        _put_f16(blocks, 0, np.abs(rng.normal(0.0, 0.01, nblk)))
        _put_f16(blocks, 2, np.abs(rng.normal(0.0, 0.01, nblk)))
    elif fmt == Q6_K:
        sc = rng.integers(-32, 32, size=(nblk, 16), dtype=np.int8)
        blocks[:, 192:208] = sc.view(np.uint8)
        _put_f16(blocks, 208, np.abs(rng.normal(0.0, 0.01, nblk)))
    else:
        raise ValueError(f"no generator for format {fmt}")
    return blocks.reshape(-1)


def host_x(in_dim: int, batch: int = 1, seed: int = 1) -> np.ndarray:
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, in_dim), dtype=np.float32)
    return x[0] if batch == 1 else x


def host_router(n_experts: int, hidden: int, seed: int = 2) -> np.ndarray:
    """fp32 router weights ~ N(0, 1/sqrt(hidden))."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n_experts, hidden)) / np.sqrt(hidden)).astype(np.float32)


def device_fill(buf, fmt: int, out_dim: int, in_dim: int, seed: int = 0) -> None:
    """Fill ``buf`` (torch uint8 CUDA tensor of tensor_bytes) with a synthetic tensor, on the device."""
    import torch

    g = torch.Generator(device=buf.device)
    g.manual_seed(seed)
    nblk = out_dim * (in_dim // BLOCK_ELEMS[fmt])
    bb = BLOCK_BYTES[fmt]
    v = buf[: nblk * bb].view(nblk, bb)
    # uniform bytes, written in slabs to bound the int64 temporaries torch.randint may use
    step = max(1, (256 << 20) // bb)
    for s in range(0, nblk, step):
        e = min(nblk, s + step)
        v[s:e].copy_(torch.randint(0, 256, (e - s, bb), generator=g, device=buf.device, dtype=torch.uint8))

    def put_f16(col, sigma, div=1.0):
        vals = (torch.randn(nblk, generator=g, device=buf.device) * sigma).abs_() / div
        v[:, col:col + 2] = vals.to(torch.float16).view(torch.uint8).view(nblk, 2)

    if fmt == Q8_0:
        # every byte pattern except -128 (0x80): map it to -127
        q = v[:, 2:]
        q[q == 0x80] = 0x81
        put_f16(0, 0.02, 127.0)
    elif fmt in (Q4_K, Q5_K):
        put_f16(0, 0.01)
        put_f16(2, 0.01)
    elif fmt == Q6_K:
        sc = torch.randint(-32, 32, (nblk, 16), generator=g, device=buf.device, dtype=torch.int8)
        v[:, 192:208] = sc.view(torch.uint8)
        put_f16(208, 0.01)
    else:
        raise ValueError(f"no generator for format {fmt}")
