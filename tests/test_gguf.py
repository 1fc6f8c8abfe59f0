"""CPU tests of the GGUF reader behind include/orome_gguf.h: synthetic files written by tests/gguf_synth.py are
read back through the C library.  Each case states the reference behaviour it pins (inference/src/gguf.m)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import gguf_synth as W
from orome_b200 import format as F
from orome_b200 import gguf as G
from orome_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_symbol_of_the_gguf_header():
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "orome_gguf.h")).read(), flags=re.S)
    syms = sorted(set(re.findall(r"\b(orome_[a-z0-9_]+)\s*\(", text)))
    L = G.lib()
    for s in syms:
        assert hasattr(L, s), f"{s} declared in include/orome_gguf.h but not exported"
    assert sorted(G.EXPORTS) == syms


def moe_file(tmp_path, **kw):
    H, M, E, V = 256, 512, 4, 1024
    t = [
        ("token_embd.weight", [H, V], W.GGML_Q8_0, synth.host_tensor(synth.Q8_0, V, H, seed=1)),
        ("blk.0.ffn_gate_inp.weight", [H, E], W.GGML_F32, synth.host_router(E, H, seed=2)),
        ("blk.0.ffn_gate_exps.weight", [H, M, E], W.GGML_Q4_K, synth.host_tensor(synth.Q4_K, M * E, H, seed=3)),
        ("blk.0.ffn_up_exps.weight", [H, M, E], W.GGML_Q4_K, synth.host_tensor(synth.Q4_K, M * E, H, seed=4)),
        ("blk.0.ffn_down_exps.weight", [M, H, E], W.GGML_Q6_K, synth.host_tensor(synth.Q6_K, H * E, M, seed=5)),
    ]
    kv = [
        ("general.architecture", W.STR, "qwen3moe"),
        ("general.name", W.STR, "synthetic"),
        ("qwen3moe.block_count", W.U32, 1),
        ("qwen3moe.context_length", W.U64, 4096),
        ("qwen3moe.embedding_length", W.U16, H),
        ("qwen3moe.expert_count", W.I32, E),
        ("qwen3moe.expert_used_count", W.U8, 2),
        ("qwen3moe.attention.head_count", W.I64, 8),
        ("qwen3moe.attention.head_count_kv", W.ARR, (W.I32, [2, 2])),       # an array where a scalar is expected reads as 0
        ("qwen3moe.attention.key_length", W.I16, 64),
        ("qwen3moe.attention.value_length", W.I8, 64),
        ("qwen3moe.attention.layer_norm_rms_epsilon", W.F32, 1e-6),
        ("qwen3moe.rope.freq_base", W.F64, 1e7),                             # a double reads as 0 in the reference
        ("qwen3moe.rope.dimension_count", W.U32, 64),
        ("qwen3moe.full_attention_interval", W.U32, 4),
        ("llama.block_count", W.U32, 99),                                    # another architecture's key: ignored
        ("tokenizer.ggml.tokens", W.ARR, (W.STR, ["a", "bc", "", "def"])),
        ("tokenizer.ggml.scores", W.ARR, (W.F32, [0.5, 1.5, 2.5])),
        ("tokenizer.ggml.nested", W.ARR, (W.ARR, [(W.U8, [1, 2, 3]), (W.STR, ["x"])])),
        ("tokenizer.ggml.eos_token_id", W.U32, 7),
        ("tokenizer.chat_template", W.STR, "{{ messages }}"),
        ("some.flag", W.BOOL, 1),
    ]
    path = tmp_path / "moe.gguf"
    info = W.write(path, kv, t, **kw)
    return path, info, t, (H, M, E, V)


def test_metadata_directory_and_data_round_trip(tmp_path):
    path, info, tensors, (H, M, E, V) = moe_file(tmp_path)
    with G.GGUFFile(path) as gf:
        m = gf.meta
        assert m.arch == b"qwen3moe" and m.version == 3 and m.alignment == 32
        assert (m.num_layers, m.context_length, m.hidden_dim, m.num_experts, m.num_experts_per_tok) == (1, 4096, H, E, 2)
        assert (m.num_attn_heads, m.num_kv_heads, m.attn_key_length, m.attn_value_length) == (8, 0, 64, 64)
        assert m.rms_norm_eps == pytest.approx(1e-6) and m.rope_theta == 0.0 and m.rope_dimension_count == 64
        assert m.full_attention_interval == 4
        assert (m.eos_token_id, m.padding_token_id) == (7, -1)
        assert gf.chat_template == "{{ messages }}"
        # inferred from the directory: MoE by tensor names, vocabulary from token_embd, expert width from ffn_gate_exps
        assert m.ffn_is_moe == 1 and m.vocab_size == V and m.moe_intermediate == M
        assert gf.num_tensors == len(tensors)
        assert gf.data_offset == info["data_offset"] and gf.data_offset % 32 == 0
        assert gf.file_size == os.path.getsize(path)
        base = G.lib().orome_gguf_base(gf.handle)
        for i, (name, dims, gtype, data) in enumerate(tensors):
            ti = gf.find_tensor(name)
            assert ti is not None and ti.name == name.encode() and gf.tensor(i).name == name.encode()
            assert ti.n_dims == len(dims) and list(ti.dims)[:len(dims)] == dims and ti.type == gtype
            assert ti.offset == info["offsets"][name] and ti.offset % 32 == 0
            raw = np.ascontiguousarray(data).tobytes()
            assert gf.tensor_size(ti) == len(raw)
            assert C.string_at(base + gf.data_offset + ti.offset, len(raw)) == raw
        assert gf.find_tensor("blk.1.ffn_gate_exps.weight") is None
        assert gf.tensor(len(tensors)) is None
        assert gf.tensor_size(None) == 0


def test_tensor_size_table():
    # gguf.m:64-104: weights per block and bytes per block of every ggml type the reference sizes
    want = {0: (1, 4), 1: (1, 2), 30: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),
            10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292)}
    for gtype, (weights, nbytes) in want.items():
        ti = G.TensorInfo(name=b"t", n_dims=2, dims=(C.c_uint64 * 4)(512, 6, 0, 0), type=gtype, offset=0)
        assert G.lib().orome_gguf_tensor_size(C.byref(ti)) == 512 * 6 // weights * nbytes
    unknown = G.TensorInfo(name=b"t", n_dims=1, dims=(C.c_uint64 * 4)(512, 0, 0, 0), type=77, offset=0)
    assert G.lib().orome_gguf_tensor_size(C.byref(unknown)) == 0
    three = G.TensorInfo(name=b"t", n_dims=3, dims=(C.c_uint64 * 4)(256, 8, 4, 0), type=12, offset=0)
    assert G.lib().orome_gguf_tensor_size(C.byref(three)) == 8 * 4 * 144


def test_custom_alignment_and_version_2(tmp_path):
    path, info, tensors, _ = moe_file(tmp_path, alignment=256, version=2)
    with G.GGUFFile(path) as gf:
        assert gf.meta.alignment == 256 and gf.meta.version == 2
        assert gf.data_offset == info["data_offset"] and gf.data_offset % 256 == 0
        for name, *_ in tensors:
            assert gf.find_tensor(name).offset % 256 == 0


def test_keys_before_the_architecture_are_read_as_llama(tmp_path):
    # gguf.m:345-347: the key prefix is the architecture seen so far, "llama" until then
    H = 256
    t = [("blk.0.ffn_gate.weight", [H, 768], W.GGML_Q8_0, synth.host_tensor(synth.Q8_0, 768, H, seed=1)),
         ("token_embd.weight", [H, 512], W.GGML_F16, np.zeros(512 * H, np.uint16))]
    kv = [("llama.block_count", W.U32, 3), ("llama.embedding_length", W.U32, H),
          ("general.architecture", W.STR, "qwen35"),
          ("llama.context_length", W.U32, 11), ("qwen35.context_length", W.U32, 22), ("qwen35.vocab_size", W.U32, 777)]
    path = tmp_path / "early.gguf"
    W.write(path, kv, t)
    with G.GGUFFile(path) as gf:
        m = gf.meta
        assert (m.num_layers, m.hidden_dim, m.context_length) == (3, H, 22)
        assert m.ffn_is_moe == 0 and m.moe_intermediate == 768          # dense by tensor names, width from ffn_gate
        assert m.vocab_size == 777                                      # metadata wins over the embedding's shape
        assert gf.chat_template is None


def test_ffn_kind_without_ffn_tensors_follows_expert_count(tmp_path):
    for experts, want in ((0, 0), (8, 1)):
        path = tmp_path / f"bare{experts}.gguf"
        W.write(path, [("general.architecture", W.STR, "x"), ("x.expert_count", W.U32, experts)],
                [("output_norm.weight", [64], W.GGML_F32, np.ones(64, np.float32))])
        with G.GGUFFile(path) as gf:
            assert gf.meta.ffn_is_moe == want and gf.meta.moe_intermediate == 0 and gf.meta.vocab_size == 0


def test_empty_file_directory(tmp_path):
    path = tmp_path / "empty.gguf"
    W.write(path, [], [])
    with G.GGUFFile(path) as gf:
        assert gf.num_tensors == 0 and gf.data_offset == 32 and gf.meta.arch == b""
        assert gf.find_tensor("token_embd.weight") is None


@pytest.mark.parametrize("kw, why", [
    (dict(magic=b"GGML"), "magic"),
    (dict(version=1), "version"),
    (dict(version=4), "version"),
    (dict(truncate_to=200), "exceed the file size"),
    (dict(truncate_to=700), "past the end"),
    (dict(truncate_to=20), "too short"),
    (dict(alignment=48), "power of two"),
])
def test_malformed_files_are_refused(tmp_path, kw, why):
    path, *_ = moe_file(tmp_path, **kw)
    with pytest.raises(F.OromeError) as e:
        G.GGUFFile(path)
    assert why in str(e.value)


def test_tensor_data_outside_the_file_is_refused(tmp_path):
    path, info, tensors, _ = moe_file(tmp_path)
    size = os.path.getsize(path)
    W.write(path, [], [(n, d, g, x) for n, d, g, x in tensors], truncate_to=size - 4096)
    with pytest.raises(F.OromeError) as e:
        G.GGUFFile(path)
    assert "outside the file" in str(e.value)
    with pytest.raises(F.OromeError):
        G.GGUFFile(tmp_path / "does-not-exist.gguf")
