"""Build the CPU checkers.

TEST INFRASTRUCTURE ONLY: nothing in the shipped package imports this module.

* ``liboracle.so``  -- the C restatement in ``oracle.c`` (always built).
* ``_ref/libref_format.so`` -- the reference's own CPU decode, compiled from the
  reference tree where it lies (only when that tree is mounted).  The decode
  section of ``inference/src/format.m`` (lines 17-174) is plain C; it is
  extracted by line range into ``_ref/format_core.inc`` (git-ignored, never
  committed) and compiled around ``ref_wrap.c``.  The reference's own build
  system is not run (it needs the Metal toolchain).

Both are compiled with ``-ffp-contract=off`` so that ``a*q - m`` is evaluated as
a rounded multiply followed by a rounded subtract on every host.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference tree: named by the environment, else a directory "reference" beside the repository
REF_ROOT = os.environ.get("OROME_REFERENCE_ROOT") or os.path.join(os.path.dirname(HERE), os.pardir, "reference")
REF_FORMAT = os.path.join(REF_ROOT, "inference", "src", "format.m")
REF_LINES = (17, 174)   # format_fp16_to_f32 .. end of format_decode_q6_k_row

CFLAGS = ["-std=c11", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-Wall"]


def _stale(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(s) and os.path.getmtime(s) > t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if force or _stale(out, src):
        subprocess.check_call(["gcc", *CFLAGS, "-o", out, src, "-lm"])
    return out


def build_ref(force: bool = False) -> str | None:
    """Compile the reference's decode when the reference tree is present.

    Returns the path of the library, the path of a previously built copy when
    the tree is absent, or None when neither exists."""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libref_format.so")
    if not os.path.exists(REF_FORMAT):
        return out if os.path.exists(out) else None
    os.makedirs(out_dir, exist_ok=True)
    inc = os.path.join(out_dir, "format_core.inc")
    wrap = os.path.join(HERE, "ref_wrap.c")
    if force or _stale(out, REF_FORMAT, wrap):
        with open(REF_FORMAT, "r", encoding="utf-8") as f:
            lines = f.readlines()
        with open(inc, "w", encoding="utf-8") as f:
            f.writelines(lines[REF_LINES[0] - 1:REF_LINES[1]])
        subprocess.check_call(["gcc", *CFLAGS, "-I", HERE, "-o", out, wrap, "-lm"])
    return out


def build_all(force: bool = False) -> None:
    build_oracle(force)
    build_ref(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("oracle:", build_oracle())
    print("ref   :", build_ref())
