"""CPU checks of the drop-in boundary: the library loads, exports every symbol the
header declares, and its pure-host helpers behave like the reference's."""
import ctypes as C
import os
import re

import pytest

from orome_b200 import format as F
from orome_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "orome_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(orome_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = F.lib()
    syms = header_symbols()
    assert len(syms) >= 19
    for s in syms:
        assert hasattr(L, s), f"{s} declared in include/orome_cuda.h but not exported"
    assert sorted(F.EXPORTS) == syms


def test_format_from_ggml_type_matches_reference_table():
    # format.m:326-337: ids 0/1/8/12/13/14/30, anything else falls back to Q4_K
    want = {8: synth.Q8_0, 12: synth.Q4_K, 13: synth.Q5_K, 14: synth.Q6_K, 1: synth.F16, 30: synth.BF16, 0: synth.F32,
            2: synth.Q4_K, 99: synth.Q4_K}
    for t, q in want.items():
        assert F.format_from_ggml_type(t) == q


def test_row_bytes_table():
    assert F.format_row_bytes(synth.Q8_0, 4096) == 4352          # 128 blocks x 34 B
    assert F.format_row_bytes(synth.Q4_K, 4096) == 2304
    assert F.format_row_bytes(synth.Q5_K, 768) == 528
    assert F.format_row_bytes(synth.Q6_K, 5120) == 4200
    assert F.format_row_bytes(synth.Q6_K, 17408) == 14280
    assert F.format_row_bytes(synth.F32, 2048) == 8192
    assert F.format_row_bytes(synth.Q8_0, 48) == 0               # ragged: not a whole number of blocks
    assert F.format_row_bytes(synth.Q4_K, 384) == 0
    for fmt in (synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K):
        assert F.format_row_bytes(fmt, 1024) == synth.row_bytes(fmt, 1024)


def test_struct_layout_matches_header():
    assert C.sizeof(F.TensorRef) == 32
    assert F.TensorRef.offset.offset == 8 and F.TensorRef.variant.offset == 16 and F.TensorRef.format.offset == 20
    assert F.TensorRef.out_dim.offset == 24 and F.TensorRef.in_dim.offset == 28
    assert C.sizeof(F.ExpertProjRef) == 24 and C.sizeof(F.ExpertLayerRef) == 80


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(F.OromeError):
        F.Context(0)


def test_integration_stub_compiles_as_c(tmp_path):
    """The reference-side stub shown in INTEGRATION.md is real C against the shipped headers."""
    import subprocess
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    block = re.search(r"```c\n(/\* format_cuda\.c.*?)```", text, flags=re.S).group(1)
    src = tmp_path / "format_cuda.c"
    src.write_text(block)
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)])
    # and the headers alone are C-clean
    hdr = tmp_path / "hdr.c"
    hdr.write_text('#include "orome_cuda.h"\n#include "orome_gguf.h"\nint main(void) { return (int)sizeof(OromeLayerTensorCache) == 0; }\n')
    subprocess.check_call(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(hdr)])
