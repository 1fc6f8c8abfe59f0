"""A small GGUF writer for the tests: header, typed metadata, tensor directory, aligned data section.

Follows the published GGUF container layout (little endian): magic "GGUF", u32 version, u64 tensor count, u64
key/value count; each key/value = string key, u32 value type, value; each directory entry = string name, u32 rank,
u64 dims (fastest first), u32 ggml type, u64 offset into the data section; the data section starts at the next
multiple of general.alignment (32 when absent).  Strings are u64 length + bytes without terminator.
"""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}

# ggml type ids of the formats the path reads
GGML_F32, GGML_F16, GGML_Q8_0, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K, GGML_BF16 = 0, 1, 8, 12, 13, 14, 30


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def value(vtype: int, v) -> bytes:
    """One typed metadata value.  An array is (element type, [elements])."""
    if vtype == STR:
        return _s(v)
    if vtype == ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(value(et, x) for x in items)
    return struct.pack(_SCALAR[vtype], v)


def write(path, kvs, tensors, version: int = 3, magic: bytes = b"GGUF", alignment: int | None = None,
          truncate_to: int | None = None) -> dict:
    """kvs: [(key, value type, value)] in file order; tensors: [(name, dims fastest-first, ggml type, bytes)].
    Returns {"data_offset": ..., "offsets": {name: offset in the data section}}."""
    align = alignment or 32
    head = bytearray(magic + struct.pack("<IQQ", version, len(tensors), len(kvs) + (1 if alignment else 0)))
    if alignment:
        head += _s("general.alignment") + struct.pack("<I", U32) + value(U32, alignment)
    for key, vt, v in kvs:
        head += _s(key) + struct.pack("<I", vt) + value(vt, v)
    offsets, pos = {}, 0
    for name, dims, gtype, data in tensors:
        offsets.setdefault(name, pos)
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", gtype, pos)
        pos += (len(bytes(data)) + align - 1) // align * align
    data_offset = (len(head) + align - 1) // align * align
    body = bytearray(head) + bytes(data_offset - len(head))
    for name, dims, gtype, data in tensors:
        raw = np.ascontiguousarray(data).tobytes() if isinstance(data, np.ndarray) else bytes(data)
        body += raw + bytes((-len(raw)) % align)
    if truncate_to is not None:
        body = body[:truncate_to]
    with open(path, "wb") as f:
        f.write(body)
    return {"data_offset": data_offset, "offsets": offsets}
