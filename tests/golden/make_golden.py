"""Generate the committed golden fixtures from the reference's own CPU decode.

Run in a container where the reference tree is mounted (oracle/_ref gets built
from it):  python tests/golden/make_golden.py

Writes tests/golden/decode_golden.npz:
  * fp16_bits        -- format_fp16_to_f32 of all 65536 halves, as uint32 bit patterns
  * scale_pairs      -- format_unpack_q4k_scale_min_pair on 64 random 12-byte fields, g = 0..3
  * <FMT>_data/_out  -- seeded packed tensors (orome_b200.synth) and the reference's
                        format_decode_*_row output for every row, for the four formats,
                        plus an "edge" tensor per format built from extreme byte patterns.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from orome_b200 import synth  # noqa: E402

SHAPES = {"Q8_0": (synth.Q8_0, 6, 512), "Q4_K": (synth.Q4_K, 5, 768), "Q5_K": (synth.Q5_K, 5, 512),
          "Q6_K": (synth.Q6_K, 5, 768)}


def edge_tensor(fmt, in_dim):
    """Rows of all-0x00, all-0xFF, alternating and large-magnitude fp16 scales (finite)."""
    rb = synth.row_bytes(fmt, in_dim)
    rows = [np.zeros(rb, np.uint8), np.full(rb, 0xFF, np.uint8),
            np.tile(np.array([0xAA, 0x55], np.uint8), rb // 2),
            np.random.default_rng(99).integers(0, 256, rb, dtype=np.uint8)]
    t = np.stack(rows)
    bb = synth.BLOCK_BYTES[fmt]
    blocks = t.reshape(len(rows), -1, bb)
    # keep the fp16 scale fields finite in the 0xFF row (0xFFFF is a NaN): use -65504 and a subnormal
    f16_cols = {synth.Q8_0: [0], synth.Q4_K: [0, 2], synth.Q5_K: [0, 2], synth.Q6_K: [208]}[fmt]
    for c in f16_cols:
        blocks[1, :, c] = 0xFF
        blocks[1, :, c + 1] = 0xFB          # 0xFBFF = -65504
        blocks[2, :, c] = 0x01
        blocks[2, :, c + 1] = 0x00          # 0x0001 = smallest subnormal
    return t.reshape(-1)


def main():
    R = oracle.ref()
    if R is None:
        raise SystemExit("reference tree not mounted: cannot build oracle/_ref")
    out = {}
    out["fp16_bits"] = np.array([np.float32(R.ref_fp16_to_f32(h)).view(np.uint32) for h in range(65536)], np.uint32)
    rng = np.random.default_rng(7)
    fields = rng.integers(0, 256, (64, 12), dtype=np.uint8)
    pairs = np.zeros((64, 4, 4), np.float32)
    import ctypes as C
    for i in range(64):
        for g in range(4):
            R.ref_unpack_scale_min_pair(fields[i].ctypes.data_as(C.POINTER(C.c_uint8)), g,
                                        pairs[i, g].ctypes.data_as(C.POINTER(C.c_float)))
    out["scale_fields"] = fields
    out["scale_pairs"] = pairs
    for name, (fmt, rows, in_dim) in SHAPES.items():
        data = synth.host_tensor(fmt, rows, in_dim, seed=synth.seed_for("golden", name))
        out[f"{name}_data"] = data
        out[f"{name}_out"] = oracle.ref_decode_rows(fmt, data, rows, in_dim)
        e = edge_tensor(fmt, in_dim)
        out[f"{name}_edge_data"] = e
        out[f"{name}_edge_out"] = oracle.ref_decode_rows(fmt, e, 4, in_dim)
        out[f"{name}_shape"] = np.array([rows, in_dim], np.int64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
