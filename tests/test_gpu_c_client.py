"""The drop-in boundary driven from C, as the reference's own format layer would drive it: tests/c_client/format_client.c
is compiled with gcc against include/*.h and liborome_cuda.so, opens a synthetic GGUF file, uploads it, builds the tensor
cache and runs a dense FFN, the lm_head and the arg-max; the results are compared with the CPU oracle."""
import os
import subprocess

import numpy as np
import pytest

import gguf_synth as W
import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "orome_b200")


def rel_l2(got, want):
    want = np.asarray(want, np.float64)
    return float(np.linalg.norm(np.asarray(got, np.float64) - want) / max(np.linalg.norm(want), 1e-300))


def test_c_program_runs_a_layer_from_a_gguf_file(tmp_path):
    H, M, V = 1024, 2560, 4096
    gate, up = synth.host_tensor(synth.Q4_K, M, H, seed=1), synth.host_tensor(synth.Q4_K, M, H, seed=2)
    down = synth.host_tensor(synth.Q6_K, H, M, seed=3)
    embd = synth.host_tensor(synth.Q8_0, V, H, seed=4)                  # no output.weight: the head is tied to the embedding
    kv = [("general.architecture", W.STR, "qwen35"), ("qwen35.block_count", W.U32, 1), ("qwen35.embedding_length", W.U32, H),
          ("qwen35.feed_forward_length", W.U32, M), ("qwen35.attention.head_count", W.U32, 8),
          ("qwen35.attention.head_count_kv", W.U32, 2), ("qwen35.attention.key_length", W.U32, 128)]
    tensors = [("token_embd.weight", [H, V], W.GGML_Q8_0, embd), ("blk.0.ffn_gate.weight", [H, M], W.GGML_Q4_K, gate),
               ("blk.0.ffn_up.weight", [H, M], W.GGML_Q4_K, up), ("blk.0.ffn_down.weight", [M, H], W.GGML_Q6_K, down)]
    model = tmp_path / "dense.gguf"
    W.write(model, kv, tensors)
    x = synth.host_x(H, seed=5)
    x.tofile(tmp_path / "x.f32")

    exe = tmp_path / "format_client"
    subprocess.check_call(["gcc", "-std=c11", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "c_client", "format_client.c"), "-o", str(exe),
                           "-L", PKG, "-lorome_cuda", f"-Wl,-rpath,{PKG}"])
    run = subprocess.run([str(exe), str(model), str(tmp_path / "x.f32"), str(tmp_path / "out.bin"), str(H), str(M), str(V)],
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr
    out = np.fromfile(tmp_path / "out.bin", dtype=np.float32)
    assert out.size == M + H + V + 1
    act, dn, logits, token = out[:M], out[M:M + H], out[M + H:M + H + V], int(out[M + H + V:].view(np.uint32)[0])

    want_act = oracle.swiglu_f64(oracle.matvec_f64(synth.Q4_K, gate, M, H, x), oracle.matvec_f64(synth.Q4_K, up, M, H, x))
    assert rel_l2(act, want_act) <= 1e-4
    assert rel_l2(dn, oracle.matvec_f64(synth.Q6_K, down, H, M, act)) <= 1e-4
    assert rel_l2(logits, oracle.matvec_f64(synth.Q8_0, embd, V, H, dn)) <= 1e-4
    assert token == oracle.argmax(logits)
