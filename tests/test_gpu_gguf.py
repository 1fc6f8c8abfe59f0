"""From a GGUF file on disk to products on the GPU: a synthetic file is opened by the C reader, its image uploaded
by the provider, the tensor cache and the expert resolver hand out TensorRef / ExpertLayerRef handles, and every
handle is driven through the matvec entry points and checked against the CPU oracle on the bytes that were
written (inference/src/format.m:343-590)."""
import zlib

import numpy as np
import pytest

import gguf_synth as W
import oracle
from orome_b200 import synth

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-4
GGML = {synth.Q8_0: W.GGML_Q8_0, synth.Q4_K: W.GGML_Q4_K, synth.Q5_K: W.GGML_Q5_K, synth.Q6_K: W.GGML_Q6_K, synth.F32: W.GGML_F32}


def rel_l2(got, want):
    want = np.asarray(want, np.float64)
    return float(np.linalg.norm(np.asarray(got, np.float64) - want) / max(np.linalg.norm(want), 1e-300))


@pytest.fixture(scope="module")
def env():
    import torch
    from orome_b200 import format as F
    from orome_b200 import gguf as G
    ctx = F.Context(0)
    yield torch, F, G, ctx
    assert ctx.status() == 0
    ctx.close()


class Model:
    """Two layers of a hybrid MoE model: layer 0 linear attention, layer 1 gated full attention."""
    H, M, S, E, V = 512, 256, 768, 8, 2048
    heads, kv, hd = 4, 2, 64
    conv, nv, vd = 1024, 8, 64

    def __init__(self):
        H, M, S, E, V = self.H, self.M, self.S, self.E, self.V
        self.t = {}
        seed = [100]

        def add(name, fmt, out_dim, in_dim, dims=None):
            seed[0] += 1
            data = synth.host_router(out_dim, in_dim, seed=seed[0]) if fmt == synth.F32 else synth.host_tensor(fmt, out_dim, in_dim, seed=seed[0])
            self.t[name] = (dims or [in_dim, out_dim], fmt, out_dim, in_dim, data)

        add("token_embd.weight", synth.Q6_K, V, H)
        add("output.weight", synth.Q8_0, V, H)
        for i in (0, 1):
            p = f"blk.{i}."
            add(p + "ffn_gate_inp.weight", synth.F32, E, H)
            add(p + "ffn_gate_inp_shexp.weight", synth.F32, 1, H)
            add(p + "ffn_gate_shexp.weight", synth.Q4_K, S, H)
            add(p + "ffn_up_shexp.weight", synth.Q4_K, S, H)
            add(p + "ffn_down_shexp.weight", synth.Q6_K, H, S)
            add(p + "ffn_gate_exps.weight", synth.Q4_K, M * E, H, [H, M, E])
            add(p + "ffn_up_exps.weight", synth.Q4_K, M * E, H, [H, M, E])
            add(p + "ffn_down_exps.weight", synth.Q6_K, H * E, M, [M, H, E])
        tv = self.nv * self.vd
        add("blk.0.attn_qkv.weight", synth.Q5_K, self.conv, H)
        add("blk.0.attn_gate.weight", synth.Q4_K, tv, H)
        add("blk.0.ssm_alpha.weight", synth.F32, self.nv, H)
        add("blk.0.ssm_beta.weight", synth.F32, self.nv, H)
        add("blk.0.ssm_out.weight", synth.Q8_0, H, tv)
        add("blk.1.attn_q.weight", synth.Q8_0, 2 * self.heads * self.hd, H)         # query and gate rows interleaved per head
        add("blk.1.attn_k.weight", synth.Q4_K, self.kv * self.hd, H)
        add("blk.1.attn_v.weight", synth.Q6_K, self.kv * self.hd, H)
        add("blk.1.attn_output.weight", synth.Q5_K, H, self.heads * self.hd)

    def write(self, path, drop=()):
        kv = [("general.architecture", W.STR, "qwen35moe"), ("qwen35moe.block_count", W.U32, 2),
              ("qwen35moe.embedding_length", W.U32, self.H), ("qwen35moe.expert_count", W.U32, self.E),
              ("qwen35moe.expert_used_count", W.U32, 2)]
        return W.write(path, kv, [(n, d, GGML[f], data) for n, (d, f, _, _, data) in self.t.items() if n not in drop])

    def shape(self, G):
        return G.ModelShape(num_layers=2, hidden_dim=self.H, moe_intermediate=self.M, shared_intermediate=self.S,
                            num_experts=self.E, vocab_size=self.V, ffn_is_moe=1, num_attn_heads=self.heads,
                            num_kv_heads=self.kv, head_dim=self.hd, linear_conv_dim=self.conv, linear_num_v_heads=self.nv,
                            linear_value_dim=self.vd)


def run_matvec(env, ref, x):
    torch, F, G, ctx = env
    xt = torch.from_numpy(x).cuda()
    y = torch.full((ref.out_dim,), float("nan"), device="cuda")
    ctx.format_dispatch_matvec(ref, xt.data_ptr(), 0, y.data_ptr(), 0)
    torch.cuda.synchronize()
    return y.cpu().numpy()


def test_every_cached_reference_multiplies_the_bytes_in_the_file(env, tmp_path):
    torch, F, G, ctx = env
    model = Model()
    info = model.write(tmp_path / "m.gguf")
    with G.GGUFFile(tmp_path / "m.gguf") as gf:
        assert gf.meta.ffn_is_moe == 1 and gf.meta.moe_intermediate == model.M and gf.meta.vocab_size == model.V
        prov = G.Provider(ctx, gf)
        layers, glob = prov.build_tensor_cache(model.shape(G), layer_is_linear=[1, 0])
        want_names = {
            ("g", "token_embd"): "token_embd.weight", ("g", "lm_head"): "output.weight",
            (0, "lin_qkv"): "blk.0.attn_qkv.weight", (0, "lin_z"): "blk.0.attn_gate.weight", (0, "lin_a"): "blk.0.ssm_alpha.weight",
            (0, "lin_b"): "blk.0.ssm_beta.weight", (0, "lin_o"): "blk.0.ssm_out.weight",
            (1, "full_k"): "blk.1.attn_k.weight", (1, "full_v"): "blk.1.attn_v.weight", (1, "full_o"): "blk.1.attn_output.weight",
        }
        for i in (0, 1):
            for field, stem in (("routing_gate", "ffn_gate_inp"), ("shared_expert_gate", "ffn_gate_inp_shexp"), ("shared_gate", "ffn_gate_shexp"),
                                ("shared_up", "ffn_up_shexp"), ("shared_down", "ffn_down_shexp")):
                want_names[(i, field)] = f"blk.{i}.{stem}.weight"
        for (where, field), name in want_names.items():
            ref = getattr(glob if where == "g" else layers[where], field)
            dims, fmt, out_dim, in_dim, data = model.t[name]
            assert ref.buffer == prov.model_buf and ref.offset == gf.data_offset + info["offsets"][name], name
            assert (ref.format, ref.out_dim, ref.in_dim) == (fmt, out_dim, in_dim), name
            x = synth.host_x(in_dim, seed=zlib.crc32(name.encode()) % 1000)
            got = run_matvec(env, ref, x)
            want = data.reshape(out_dim, in_dim).astype(np.float64) @ x if fmt == synth.F32 else oracle.matvec_f64(fmt, data, out_dim, in_dim, x)
            assert rel_l2(got, want) <= REL_L2_TOL, name
        # tensors of the other attention kind and of a dense FFN are absent references
        for i, fields in ((0, ("full_q", "full_k", "full_v", "full_o")), (1, ("lin_qkv", "lin_z", "lin_a", "lin_b", "lin_o"))):
            for f in fields + ("dense_gate", "dense_up", "dense_down"):
                assert not getattr(layers[i], f).buffer
        assert not layers[0].owned_q
        prov.close()


def test_gated_q_rows_are_regrouped_query_rows_first(env, tmp_path):
    torch, F, G, ctx = env
    model = Model()
    model.write(tmp_path / "m.gguf")
    with G.GGUFFile(tmp_path / "m.gguf") as gf:
        prov = G.Provider(ctx, gf)
        layers, _ = prov.build_tensor_cache(model.shape(G), layer_is_linear=[1, 0])
        q = layers[1].full_q
        dims, fmt, rows, H, data = model.t["blk.1.attn_q.weight"]
        assert q.buffer == layers[1].owned_q and q.buffer != prov.model_buf and q.offset == 0
        assert (q.format, q.out_dim, q.in_dim) == (fmt, rows, H)
        # format.m:546-574: head h's query rows go to [h*hd, (h+1)*hd), its gate rows to [heads*hd + h*hd, ...)
        src = data.reshape(rows, -1)
        heads, hd = model.heads, model.hd
        order = [h * 2 * hd + r for h in range(heads) for r in range(hd)] + [h * 2 * hd + hd + r for h in range(heads) for r in range(hd)]
        regrouped = np.ascontiguousarray(src[order]).reshape(-1)
        out = torch.empty((rows, H), device="cuda")
        ctx.dequant_rows(q, 0, rows, out.data_ptr())
        torch.cuda.synchronize()
        want = oracle.decode_rows(fmt, regrouped, rows, H)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), np.ascontiguousarray(want, np.float32).view(np.uint32).reshape(rows, H))
        x = synth.host_x(H, seed=9)
        assert rel_l2(run_matvec(env, q, x), oracle.matvec_f64(fmt, regrouped, rows, H, x)) <= REL_L2_TOL
        prov.close()


def test_plain_q_tied_head_and_missing_tensors(env, tmp_path):
    torch, F, G, ctx = env
    model = Model()
    # a Q tensor with heads*hd rows is referenced in place; without output.weight the head is the embedding
    dims, fmt, rows, H, data = model.t["blk.1.attn_q.weight"]
    half = rows // 2
    model.t["blk.1.attn_q.weight"] = ([H, half], fmt, half, H, np.ascontiguousarray(data.reshape(rows, -1)[:half]).reshape(-1))
    info = model.write(tmp_path / "m.gguf", drop=("output.weight", "blk.0.ffn_up_shexp.weight", "blk.1.ffn_up_exps.weight"))
    with G.GGUFFile(tmp_path / "m.gguf") as gf:
        prov = G.Provider(ctx, gf)
        layers, glob = prov.build_tensor_cache(model.shape(G), layer_is_linear=[1, 0])
        q = layers[1].full_q
        assert not layers[1].owned_q and q.buffer == prov.model_buf and q.out_dim == half
        assert q.offset == gf.data_offset + info["offsets"]["blk.1.attn_q.weight"]
        assert (glob.lm_head.buffer, glob.lm_head.offset, glob.lm_head.format) == (glob.token_embd.buffer, glob.token_embd.offset, synth.Q6_K)
        assert not layers[0].shared_up.buffer and layers[0].shared_gate.buffer
        e = prov.resolve_expert_layer(1, model.E)
        assert e.buffer == prov.model_buf and e.up.offset == 0 and e.up.expert_stride == 0 and e.gate.expert_stride > 0
        assert not prov.resolve_expert_layer(5, model.E).gate.expert_stride
        prov.close()


def test_resolved_expert_layer_runs_the_expert_ffn(env, tmp_path):
    torch, F, G, ctx = env
    model = Model()
    info = model.write(tmp_path / "m.gguf")
    H, M, E, K = model.H, model.M, model.E, 2
    with G.GGUFFile(tmp_path / "m.gguf") as gf:
        prov = G.Provider(ctx, gf)
        for layer in (0, 1):
            e = prov.resolve_expert_layer(layer, E)
            parts = [model.t[f"blk.{layer}.ffn_{p}_exps.weight"] for p in ("gate", "up", "down")]
            for proj, name, (dims, fmt, out_dim, in_dim, data) in zip((e.gate, e.up, e.down), ("gate", "up", "down"), parts):
                assert proj.offset == gf.data_offset + info["offsets"][f"blk.{layer}.ffn_{name}_exps.weight"]
                assert proj.format == fmt and proj.expert_stride == data.size // E
            x = synth.host_x(H, seed=40 + layer)
            idx = np.array([[5, 2]], np.uint32)
            w = np.array([[0.7, 0.3]], np.float32)
            xt, it, wt = (torch.from_numpy(a).cuda() for a in (x, idx.view(np.int32), w))
            act = torch.empty((1, K, M), device="cuda")
            out = torch.full((1, H), float("nan"), device="cuda")
            ctx.moe_ffn(e, 0, xt.data_ptr(), 1, H, it.data_ptr(), wt.data_ptr(), K, H, M, act.data_ptr(), out.data_ptr(), H)
            torch.cuda.synchronize()
            fmts = tuple(p[1] for p in parts)
            strides = tuple(p[4].size // E for p in parts)
            want = oracle.moe_ffn_f64(parts[0][4], parts[1][4], parts[2][4], fmts, strides, x, H, M, idx[0], w[0])
            assert rel_l2(out.cpu().numpy()[0], want) <= REL_L2_TOL
        prov.close()
