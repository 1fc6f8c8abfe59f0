"""Qwen3.5-shape decode matvec sets on the device: the weight-bound products of one
token step, as the reference's engine issues them (inference/src/engine.m:481-1046).

Per layer: q/k/v projections (one grouped launch: the reference encodes them
back to back with no barrier, engine.m:777-784), o projection, fused gate/up +
SwiGLU (engine.m:342-387), down projection; after the last layer the lm_head.
Weights are seeded synthetic GGUF blocks; every layer has its own tensors so no
weight byte is read twice per step.  With ``world > 1`` every tensor is row-split:
rank r holds rows [r*N/world, (r+1)*N/world) and the output vector is all-gathered.
"""
from __future__ import annotations

from dataclasses import dataclass

from . import format as F
from . import synth
from .rowsplit import shard_rows

# name -> (format, out_dim, in_dim); "h" = hidden-sized input, "a" = ffn-sized input
SETS = {
    "9b_q8_0": dict(hidden=4096, ffn=12288, vocab=151936, layers=32,
                    fmt=dict(q=synth.Q8_0, k=synth.Q8_0, v=synth.Q8_0, o=synth.Q8_0, gate=synth.Q8_0, up=synth.Q8_0,
                             down=synth.Q8_0, lm_head=synth.Q8_0),
                    kv=1024, variant=F.VARIANT_DEFAULT),
    # 27B mixed set: attention and gate/up Q4_K, down and lm_head Q6_K; q/o 5120x5120 and k/v 1024x5120 by analogy
    # with the 9B set (the benchmark description gives no attention shapes); the reference routes this model to its
    # llama-style kernels (engine_qwen35_hybrid.m:86-148).
    "27b_q4_k_m": dict(hidden=5120, ffn=17408, vocab=151936, layers=64,
                       fmt=dict(q=synth.Q4_K, k=synth.Q4_K, v=synth.Q4_K, o=synth.Q4_K, gate=synth.Q4_K, up=synth.Q4_K,
                                down=synth.Q6_K, lm_head=synth.Q6_K),
                       kv=1024, variant=F.VARIANT_LLAMA),
}


@dataclass
class Tensor:
    name: str
    fmt: int
    out_dim: int      # rows held by this rank
    in_dim: int
    offset: int       # byte offset inside the arena
    nbytes: int
    full_out: int     # rows of the whole tensor


class DecodeSet:
    def __init__(self, name: str, device, rank: int = 0, world: int = 1, layers: int | None = None, seed: int = 0):
        import torch

        cfg = SETS[name]
        self.name, self.cfg, self.rank, self.world = name, cfg, rank, world
        self.layers = cfg["layers"] if layers is None else layers
        self.hidden, self.ffn, self.vocab, self.kv = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["kv"]
        self.variant = cfg["variant"]
        H, A, KV = self.hidden, self.ffn, self.kv
        shapes = dict(q=(H, H), k=(KV, H), v=(KV, H), o=(H, H), gate=(A, H), up=(A, H), down=(H, A))
        self.tensors: list[list[Tensor]] = []
        off = 0

        def add(nm, fmt, full_out, in_dim):
            nonlocal off
            lo, hi = shard_rows(full_out, rank, world)
            nb = synth.tensor_bytes(fmt, hi - lo, in_dim)
            t = Tensor(nm, fmt, hi - lo, in_dim, off, nb, full_out)
            off += (nb + 255) // 256 * 256
            return t

        for l in range(self.layers):
            self.tensors.append([add(f"blk.{l}.{k}", cfg["fmt"][k], *shapes[k]) for k in ("q", "k", "v", "o", "gate", "up", "down")])
        self.lm_head = add("lm_head", cfg["fmt"]["lm_head"], self.vocab, H)
        self.arena_bytes = off + 256
        self.arena = torch.empty(self.arena_bytes, dtype=torch.uint8, device=device)
        for lt in self.tensors:
            for t in lt:
                self._fill(t, seed)
        self._fill(self.lm_head, seed)
        self.weight_bytes = sum(t.nbytes for lt in self.tensors for t in lt) + self.lm_head.nbytes

    def _fill(self, t: Tensor, seed: int):
        if t.out_dim == 0:
            return
        synth.device_fill(self.arena[t.offset:t.offset + t.nbytes], t.fmt, t.out_dim, t.in_dim,
                          seed=synth.seed_for(self.name, t.name, self.rank, seed))

    def ref(self, t: Tensor) -> F.TensorRef:
        return F.tensor_ref(self.arena.data_ptr(), t.offset, t.fmt, t.out_dim, t.in_dim, self.variant)

    def full_weight_bytes(self) -> int:
        """Packed weight bytes of the whole (unsharded) set: the algorithmic bytes of one token step."""
        cfg, H, A, KV = self.cfg, self.hidden, self.ffn, self.kv
        shapes = dict(q=(H, H), k=(KV, H), v=(KV, H), o=(H, H), gate=(A, H), up=(A, H), down=(H, A))
        per_layer = sum(synth.tensor_bytes(cfg["fmt"][k], *shapes[k]) for k in shapes)
        return per_layer * self.layers + synth.tensor_bytes(cfg["fmt"]["lm_head"], self.vocab, H)

    def io_bytes(self) -> int:
        """fp32 activation bytes read and written by one step (x in, y out of every product)."""
        H, A, KV = self.hidden, self.ffn, self.kv
        per_layer = 4 * ((H + H + 2 * KV) + (H + H) + (H + A) + (A + H))
        return per_layer * self.layers + 4 * (H + self.vocab)
