#!/usr/bin/env python
"""Benchmark of the quantized dequant-matvec path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one decode-token pass over a Qwen3.5-shape matvec set: per layer the
grouped q/k/v projections, the o projection, the fused gate/up + SwiGLU and the down
projection, then the lm_head and the arg-max of the logits (129 products per step for
the 9B Q8_0 set).  Every product reads the output of the one before it, as in the
engine.  Every layer has its own weights (7.2 GB for the 9B set), far above the 126 MB
L2, so no weight byte is served from cache between or within steps.

Two forms of the same step.  `--mode launches` issues one kernel per product, replayed from a
CUDA graph; `--mode chain` records the step once through the C ABI and runs it as ONE resident
kernel.  The default, `--mode auto`, takes the form that measures faster for the GPU count:
launches on one GPU (the chain's hand-over between products costs more than a graph node there),
the chain on several (one launch per step instead of a launch plus a cross-GPU wait per product).

Prints ONE JSON line: metric decode_matvec_tok_s (tokens per second of the whole job),
`roofline` (algorithmic HBM bytes per step / device time against the measured copy
bandwidth), `e2e` (same steps with the input vector copied from pinned host memory and
the token read back every step), `cpu_baseline` (the reference's CPU decode + dot on
the host cores, on a bounded sample), `parity_check` (products of the timed kernel against
the CPU oracle on sampled rows) and the clocks seen during the timed region.

With N > 1 (launched by torch.distributed.run) every tensor is row-split over the
ranks and every output vector is completed on all GPUs by peer stores from the
producing kernel, so the scaling is "strong" (the same token step on more GPUs).

`--impl reference` times the reference's own CPU implementation of the path (its
format.m decode compiled into oracle/_ref, else the C restatement) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0      # used only when MEASURED_PEAKS.json is absent
NOMINAL_HBM_GBS = 8000.0


def dram_per_algorithmic(workload: str, mode: str):
    """DRAM bytes (read + write) per algorithmic byte of the dominant kernel, from the committed summary of an ncu
    capture of a small cut of the same workload (traffic grows in proportion to the rows), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return float(json.load(f)[f"{workload}/{mode}"]["dram_bytes_per_algorithmic_byte"])
    except Exception:
        return None


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period: float = 0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    NAMES = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
             0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
             0x100: "display_clock_setting"}

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.NAMES.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def finish(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU decode + dot on the host cores
# ----------------------------------------------------------------------------------------------
class CpuSteps:
    """Whole token steps on the host: the reference's CPU decode (oracle/_ref when it was compiled, else the C
    restatement) followed by an fp32 dot, OpenMP over rows on every host core.  One layer's tensors stand for all
    layers (each layer is decoded again every time: nothing is cached between products), plus the lm_head once per
    step.  Inputs are fixed vectors: on a CPU a chain of shrinking activations would end in denormal arithmetic."""

    def __init__(self, set_name: str):
        import numpy as np
        import oracle
        from orome_b200 import decode_set, synth
        self.oracle = oracle
        self.threads_requested = oracle.use_all_cores()
        cfg = decode_set.SETS[set_name]
        self.cfg, self.name = cfg, set_name
        H, A, KV, V = cfg["hidden"], cfg["ffn"], cfg["kv"], cfg["vocab"]
        self.shapes = dict(q=(H, H), k=(KV, H), v=(KV, H), o=(H, H), gate=(A, H), up=(A, H), down=(H, A))
        # the reference's CPU decode knows only its default scale layout
        self.use_ref = oracle.ref() is not None and cfg["variant"] == 0
        rng = np.random.default_rng(0)
        self.xh, self.xa = rng.standard_normal(H, dtype=np.float32), rng.standard_normal(A, dtype=np.float32)
        self.tensors = {k: synth.host_tensor(cfg["fmt"][k], *self.shapes[k], seed=synth.seed_for(set_name, "cpu", k)) for k in self.shapes}
        self.lm = synth.host_tensor(cfg["fmt"]["lm_head"], V, H, seed=synth.seed_for(set_name, "cpu", "lm_head"))
        self.layer_bytes = sum(t.size for t in self.tensors.values())
        self.step_bytes = self.layer_bytes * cfg["layers"] + self.lm.size
        self.kind = "reference" if self.use_ref else "port"
        self.cores = int(oracle.ref().ref_num_threads() if self.use_ref else oracle.num_threads())

    def step(self):
        cfg, mv = self.cfg, self.oracle.matvec_f32
        for _ in range(cfg["layers"]):
            for k, (od, idim) in self.shapes.items():
                mv(cfg["fmt"][k], self.tensors[k], od, idim, self.xa if k == "down" else self.xh, layout=cfg["variant"], use_ref=self.use_ref)
        mv(cfg["fmt"]["lm_head"], self.lm, cfg["vocab"], cfg["hidden"], self.xh, layout=cfg["variant"], use_ref=self.use_ref)

    def timed(self, steps: int, warmup: int, budget_s: float = 0.0):
        for _ in range(warmup):
            self.step()
        times, t_all = [], time.perf_counter()
        for _ in range(steps):
            t0 = time.perf_counter()
            self.step()
            times.append(time.perf_counter() - t0)
            if budget_s and time.perf_counter() - t_all > budget_s:
                break
        return times

    def sample_text(self, n: int) -> str:
        return (f"{n} whole token steps of {self.name}: {self.cfg['layers']} x one layer's tensors ({self.layer_bytes} B, decoded again "
                f"for every layer) + lm_head, {self.step_bytes} weight bytes per step, fixed input vectors")


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    cpu = CpuSteps(name)
    times = cpu.timed(max(1, args.steps), max(1, args.warmup))
    step_s = sum(times) / len(times)
    tok_s = 1.0 / step_s
    line = {
        "impl": "reference", "metric": "decode_matvec_tok_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": max(1, args.warmup), "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "batch": 1, "layers": cpu.cfg["layers"], "weight_bytes": cpu.step_bytes,
                   "l2": "inputs larger than L2: every layer has its own weights"},
        "form": "CPU: the reference's row decode + fp32 dot for every product of the step, all host threads",
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cpu.cores, "kind": cpu.kind, "sample": cpu.sample_text(len(times)),
                         "cpu_gbs": cpu.step_bytes / step_s / 1e9},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class Stepper:
    """One token step of a DecodeSet through the C ABI.  mode "chain": recorded once, one launch per step;
    mode "launches": one launch per product, replayed from a CUDA graph."""

    # flags of the gathered vectors (armed single launches on several GPUs)
    FLAG_QKV, FLAG_O, FLAG_ACT, FLAG_DN, FLAG_LOGITS = range(5)

    def __init__(self, torch, F, ctx, ds, dist=None, fused=True, mode="chain"):
        self.torch, self.F, self.ctx, self.ds, self.dist = torch, F, ctx, ds, dist
        self.mode = mode
        self.fused = fused and ds.world > 1
        dev = ds.arena.device
        H, A, KV, V = ds.hidden, ds.ffn, ds.kv, ds.vocab
        g = torch.Generator(device=dev)
        g.manual_seed(1234)
        self.x_h = torch.randn(H, device=dev, generator=g)           # the step's input vector
        from orome_b200.rowsplit import padded_rows
        w = ds.world
        # output vectors (padded to equal slices per rank when sharded); local slices are written in place
        sizes = [padded_rows(n, w) for n in (H, KV, KV, H, A, H, V)]
        if self.fused:
            from orome_b200.rowsplit import PeerArena
            self.arena = PeerArena(ctx, dist, ds.rank, w, sum((n * 4 + 255) // 256 * 256 for n in sizes), 5)
            bufs = [self.arena.floats(n) for n in sizes]
        else:
            bufs = [torch.zeros(n, device=dev) for n in sizes]
        self.q, self.k, self.v, self.o, self.act, self.dn, self.logits = bufs
        self.token = torch.full((1,), -1, device=dev, dtype=torch.int32)
        self.refs = [[ds.ref(t) for t in lt] for lt in ds.tensors]
        self.lm_ref = ds.ref(ds.lm_head)
        self.graph = self.chain = None
        self.launches_per_step = 0
        self.products_per_step = 0

    def _slice(self, full, full_out):
        from orome_b200.rowsplit import shard_rows
        lo, hi = shard_rows(full_out, self.ds.rank, self.ds.world)
        return full[lo:hi]

    def _gather(self, full, full_out):
        """All-gather of the output vector when the rows are split over ranks and the kernels do not do it themselves."""
        if self.fused or self.ds.world == 1:
            return
        from orome_b200.rowsplit import all_gather_rows
        all_gather_rows(self.dist, full, full_out, self.ds.rank, self.ds.world)

    def issue(self, stream, layers=None, recording=False):
        """The products of one step, each reading its predecessor's output (engine.m:481-1046)."""
        ctx, ds = self.ctx, self.ds
        H, A, KV, V = ds.hidden, ds.ffn, ds.kv, ds.vocab
        c0 = ctx.launch_count
        armed = self.fused and not recording                               # armed single launches say what to wait for / publish
        hint = (lambda r: None) if recording else ctx.hint_next
        gn = ctx.gather_next if armed else (lambda w, p: None)
        layer_ids = list(range(len(self.refs))) if layers is None else list(layers)
        # the parity check reads every vector on the host: on several GPUs complete their plain copies too
        unpack = (lambda flag, buf, n: ctx.gather_wait(flag, buf.data_ptr(), n, stream)) if (self.fused and layers is not None) else (lambda *a: None)
        x_in, first, nprod = self.x_h, True, 0
        for n, li in enumerate(layer_ids):
            rq, rk, rv, ro, rg, ru, rd = self.refs[li]
            nxt_q = self.refs[layer_ids[n + 1]][0] if n + 1 < len(layer_ids) else self.lm_ref
            if not (rq.out_dim and rk.out_dim and rv.out_dim and ro.out_dim and rg.out_dim and rd.out_dim):
                raise SystemExit("bench.py: a rank holds no row of some tensor; use fewer GPUs for this workload")
            hint(ro)
            gn(-1 if first else self.FLAG_DN, self.FLAG_QKV)
            ctx.matvec_group([rq, rk, rv], x_in.data_ptr(), [self._slice(self.q, H).data_ptr(), self._slice(self.k, KV).data_ptr(),
                                                            self._slice(self.v, KV).data_ptr()], stream)
            self._gather(self.q, H); self._gather(self.k, KV); self._gather(self.v, KV)
            unpack(self.FLAG_QKV, self.q, H); unpack(self.FLAG_QKV, self.k, KV); unpack(self.FLAG_QKV, self.v, KV)
            hint(rg)
            gn(self.FLAG_QKV, self.FLAG_O)
            ctx.matvec(ro, self.q.data_ptr(), self._slice(self.o, H).data_ptr(), 1, 0, 0, stream)
            self._gather(self.o, H)
            unpack(self.FLAG_O, self.o, H)
            hint(rd)
            gn(self.FLAG_O, self.FLAG_ACT)
            ctx.gate_up_swiglu(rg, ru, self.o.data_ptr(), self._slice(self.act, A).data_ptr(), 1, 0, 0, stream)
            self._gather(self.act, A)
            unpack(self.FLAG_ACT, self.act, A)
            hint(nxt_q)
            gn(self.FLAG_ACT, self.FLAG_DN)
            ctx.matvec(rd, self.act.data_ptr(), self._slice(self.dn, H).data_ptr(), 1, 0, 0, stream)
            self._gather(self.dn, H)
            unpack(self.FLAG_DN, self.dn, H)
            x_in, first, nprod = self.dn, False, nprod + 4
        hint(self.refs[layer_ids[0]][0] if layer_ids else None)            # the next token starts at the first layer again
        gn(-1 if first else self.FLAG_DN, self.FLAG_LOGITS)
        ctx.matvec(self.lm_ref, x_in.data_ptr(), self._slice(self.logits, V).data_ptr(), 1, 0, 0, stream)
        self._gather(self.logits, V)
        nprod += 1
        if self.fused:
            ctx.gather_wait(self.FLAG_LOGITS, self.logits.data_ptr(), V, stream)     # the logits are complete on this rank from here on
        if ds.world == 1 or not recording:
            ctx.argmax(self.logits.data_ptr(), V, self.token.data_ptr(), stream)     # engine.m:1036-1046
        if not recording:
            self.launches_per_step = ctx.launch_count - c0
        if layers is None:
            self.products_per_step = nprod

    def record(self, layers=None):
        """A chain over the given layers (default: all) and the lm_head."""
        self.ctx.chain_begin()
        try:
            self.issue(0, layers=layers, recording=True)
        except BaseException:
            try:
                self.ctx.chain_end().close()
            except Exception:
                pass
            raise
        return self.ctx.chain_end()

    def build(self):
        torch = self.torch
        if self.mode == "chain":
            self.chain = self.record()
            self.launches_per_step = 1 if self.ds.world == 1 else 2         # several GPUs: the arg-max of the gathered logits is its own launch
            return
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.issue(s.cuda_stream)           # warm every kernel variant before capturing
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if self.ds.world > 1 and not self.fused:
            return                              # NCCL all-gathers between the launches: issued eagerly
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            self.issue(torch.cuda.current_stream().cuda_stream)
        self.graph = g

    def step(self):
        st = self.torch.cuda.current_stream().cuda_stream
        if self.chain is not None:
            self.chain.launch(st)
            if self.ds.world > 1:
                self.ctx.argmax(self.logits.data_ptr(), self.ds.vocab, self.token.data_ptr(), st)
        elif self.graph is not None:
            self.graph.replay()
        else:
            self.issue(st)

    # ---- correctness of what was timed -------------------------------------------------------------------------
    def parity_check(self, rows_per_product=48):
        """Run the first layer and the lm_head through the timed form once more (fresh, healthy values: after a few
        layers the synthetic activations of the full step underflow) and compare sampled rows of every product with
        the CPU oracle fed the SAME input vector the GPU product read.  Returns (worst rel-L2, rows checked)."""
        import numpy as np
        import oracle
        from orome_b200 import synth
        from orome_b200.rowsplit import shard_rows
        torch, ds = self.torch, self.ds
        st = torch.cuda.current_stream().cuda_stream
        if self.mode == "chain":
            chain = self.record(layers=[0])
            chain.launch(st)
            if ds.world > 1:
                self.ctx.argmax(self.logits.data_ptr(), ds.vocab, self.token.data_ptr(), st)
        else:
            keep = self.launches_per_step
            self.issue(st, layers=[0])
            self.launches_per_step = keep
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        H, A, KV, V = ds.hidden, ds.ffn, ds.kv, ds.vocab
        host = lambda t, n: t[:n].detach().cpu().numpy().astype(np.float32)
        xh, q, k, v, o, act, dn, logits = (host(self.x_h, H), host(self.q, H), host(self.k, KV), host(self.v, KV), host(self.o, H),
                                           host(self.act, A), host(self.dn, H), host(self.logits, V))
        tq, tk, tv, to, tg, tu, td = ds.tensors[0]
        rng = np.random.default_rng(99 + ds.rank)
        worst, nrows = 0.0, 0

        def rows_of(t, sel):
            rb = synth.row_bytes(t.fmt, t.in_dim)
            idx = torch.as_tensor(sel, device=ds.arena.device, dtype=torch.int64)
            view = ds.arena[t.offset:t.offset + t.nbytes].view(t.out_dim, rb)
            return view.index_select(0, idx).cpu().numpy().reshape(-1)

        def check(t, x, got_full, t2=None):
            nonlocal worst, nrows
            lo, hi = shard_rows(t.full_out, ds.rank, ds.world)
            if hi <= lo:
                return
            sel = np.sort(rng.choice(hi - lo, size=min(rows_per_product, hi - lo), replace=False))
            want = oracle.matvec_f64(t.fmt, rows_of(t, sel), len(sel), t.in_dim, x, layout=ds.variant)
            if t2 is not None:
                want = oracle.swiglu_f64(want, oracle.matvec_f64(t2.fmt, rows_of(t2, sel), len(sel), t2.in_dim, x, layout=ds.variant))
            got = got_full[lo + sel]
            err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-300))
            worst, nrows = max(worst, err), nrows + len(sel)

        check(tq, xh, q); check(tk, xh, k); check(tv, xh, v)
        check(to, q, o)
        check(tg, o, act, t2=tu)
        check(td, act, dn)
        check(ds.lm_head, dn, logits)
        token_ok = int(self.token.item()) == oracle.argmax(logits)
        if self.dist is not None:
            t = torch.tensor([worst, float(nrows), 0.0 if token_ok else 1.0], device=ds.arena.device, dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            w2 = torch.tensor([float(nrows)], device=ds.arena.device, dtype=torch.float64)
            self.dist.all_reduce(w2, op=self.dist.ReduceOp.SUM)
            worst, nrows, token_ok = float(t[0].item()), int(w2.item()), t[2].item() == 0.0
        finite = bool(np.isfinite(logits).all())
        return {"rel_l2": worst, "rows": nrows, "token_matches_reference_argmax": bool(token_ok), "finite": finite,
                "what": "first layer + lm_head through the timed form, sampled rows of every product against the fp64 CPU oracle fed the "
                        "GPU product's own input vector; every rank checks its own rows"}


def kernel_extras(torch, F, ctx, peak, only=None, reps=3):
    """Short per-kernel passes on the other benchmark configurations (rank 0, one GPU): absolute GB/s of the
    algorithmic bytes and the fraction of the measured HBM peak, back-to-back launches over distinct weight copies,
    replayed as a CUDA graph.
    `only` restricts the run to the named cases (a small, short process for a profiler capture)."""
    from orome_b200 import synth
    dev = torch.device("cuda", ctx.device)
    st = torch.cuda.current_stream().cuda_stream
    out = {}

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / n)
        return best * 1e-3

    def graphed(fn):
        """The layers as one CUDA graph (the reference commits one command buffer per token, engine.m:1048-1050): issued
        call by call from Python, four launches of a few microseconds each are bounded by the host, not by the GPU."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn(side.cuda_stream)
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=side):
                fn(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return g

    def gemv(name, fmt, od, idim, copies, batch=1, variant=0):
        if only and name not in only:
            return
        tb = (synth.tensor_bytes(fmt, od, idim) + 255) // 256 * 256
        buf = torch.empty(tb * copies, dtype=torch.uint8, device=dev)
        for i in range(copies):
            synth.device_fill(buf[i * tb:(i + 1) * tb], fmt, od, idim, seed=synth.seed_for("extras", name, i))
        x = torch.randn(batch, idim, device=dev)
        y = torch.empty(batch, od, device=dev)
        refs = [F.tensor_ref(buf.data_ptr(), i * tb, fmt, od, idim, variant) for i in range(copies)]

        def go(stream):
            for i, r in enumerate(refs):
                if batch == 1:
                    ctx.hint_next(refs[(i + 1) % copies])
                ctx.matvec(r, x.data_ptr(), y.data_ptr(), batch, idim, od, stream)
        g = graphed(go)
        t = timed(g.replay, copies)
        nbytes = synth.tensor_bytes(fmt, od, idim) + 4 * batch * (idim + od)
        out[name] = {"us": round(t * 1e6, 2), "gbs": round(nbytes / t / 1e9, 1), "frac_of_measured_hbm": round(nbytes / t / 1e9 / peak, 3),
                     "bytes": nbytes}
        if batch > 1:
            out[name]["tflops"] = round(2.0 * od * idim * batch / t / 1e12, 1)

    gemv("q8_0_4096x4096_b1", synth.Q8_0, 4096, 4096, 24)
    gemv("q4_k_12288x4096_b1", synth.Q4_K, 12288, 4096, 12)
    gemv("q4_k_4096x12288_b1", synth.Q4_K, 4096, 12288, 12)
    gemv("q4_k_12288x4096_b2_two_vectors_per_launch", synth.Q4_K, 12288, 4096, 12, batch=2)
    gemv("q4_k_12288x4096_b3", synth.Q4_K, 12288, 4096, 12, batch=3)
    gemv("q8_0_12288x4096_b8_tcgen05", synth.Q8_0, 12288, 4096, 6, batch=8)
    gemv("q6_k_5120x17408_b8_tcgen05", synth.Q6_K, 5120, 17408, 3, batch=8)
    gemv("q6_k_5120x17408_b64_tcgen05", synth.Q6_K, 5120, 17408, 3, batch=64)
    gemv("q4_k_12288x4096_b64_tcgen05", synth.Q4_K, 12288, 4096, 6, batch=64)
    gemv("q4_k_4096x12288_b64_tcgen05", synth.Q4_K, 4096, 12288, 6, batch=64)
    gemv("q5_k_12288x4096_b1", synth.Q5_K, 12288, 4096, 10)
    gemv("q6_k_5120x17408_b1", synth.Q6_K, 5120, 17408, 6)
    gemv("q6_k_lm_head_151936x5120_b1", synth.Q6_K, 151936, 5120, 2)
    gemv("q8_0_lm_head_151936x4096_b1", synth.Q8_0, 151936, 4096, 2)
    gemv("q4_k_lm_head_151936x4096_b1", synth.Q4_K, 151936, 4096, 2)
    gemv("q5_k_lm_head_151936x4096_b1", synth.Q5_K, 151936, 4096, 2)

    if only and not ({"moe_layer_top8_of_128_t1", "moe_layer_top8_of_128_t32"} & set(only)):
        return out
    # MoE layer, one token: fp32 router 128 x 2048, top-8, gate/up Q4_K 768 x 2048, down Q5_K 2048 x 768 (6 distinct layers)
    H, M, E, K, NL = 2048, 768, 128, 8, 6
    sg, sd = synth.tensor_bytes(synth.Q4_K, M, H), synth.tensor_bytes(synth.Q5_K, H, M)
    layers = []
    for l in range(NL):
        buf = torch.empty(E * (2 * sg + sd), dtype=torch.uint8, device=dev)
        synth.device_fill(buf[:E * sg], synth.Q4_K, E * M, H, seed=3 * l)
        synth.device_fill(buf[E * sg:2 * E * sg], synth.Q4_K, E * M, H, seed=3 * l + 1)
        synth.device_fill(buf[2 * E * sg:], synth.Q5_K, E * H, M, seed=3 * l + 2)
        rw = (torch.randn(E, H, device=dev) / (H ** 0.5)).contiguous()
        layers.append((buf, rw, F.ExpertLayerRef(buf.data_ptr(), F.ExpertProjRef(0, sg, synth.Q4_K), F.ExpertProjRef(E * sg, sg, synth.Q4_K),
                                                 F.ExpertProjRef(2 * E * sg, sd, synth.Q5_K)), F.tensor_ref(rw.data_ptr(), 0, synth.F32, E, H)))
    x = torch.randn(1, H, device=dev)
    idx = torch.zeros(1, 8, dtype=torch.int32, device=dev)
    w = torch.zeros(1, 8, device=dev)
    act = torch.empty(K, M, device=dev)
    o = torch.empty(H, device=dev)
    lg = torch.empty(E, device=dev)

    def moe(stream):
        for buf, rw, layer, rref in layers:
            ctx.moe_route(rref, x.data_ptr(), 1, H, K, idx.data_ptr(), w.data_ptr(), lg.data_ptr(), stream)
            ctx.moe_ffn(layer, 0, x.data_ptr(), 1, H, idx.data_ptr(), w.data_ptr(), K, H, M, act.data_ptr(), o.data_ptr(), H, stream)
    g1 = graphed(moe)
    t = timed(g1.replay, NL)
    nbytes = K * (2 * sg + sd) + E * H * 4
    out["moe_layer_top8_of_128_t1"] = {"us": round(t * 1e6, 2), "gbs": round(nbytes / t / 1e9, 1),
                                       "frac_of_measured_hbm": round(nbytes / t / 1e9 / peak, 3), "bytes": nbytes, "launches": 4,
                                       "form": "cuda graph of 6 layers"}
    # the same layers with a batch of 32 tokens (BASELINE configuration 5): algorithmic bytes = every distinct expert
    # the batch selects, read once, plus the router
    T = 32
    xT = torch.randn(T, H, device=dev)
    idxT = torch.zeros(T, 8, dtype=torch.int32, device=dev)
    wT = torch.zeros(T, 8, device=dev)
    actT = torch.empty(T, K, M, device=dev)
    oT = torch.empty(T, H, device=dev)
    lgT = torch.empty(T, E, device=dev)

    def moe_t(stream):
        for buf, rw, layer, rref in layers:
            ctx.moe_route(rref, xT.data_ptr(), T, H, K, idxT.data_ptr(), wT.data_ptr(), lgT.data_ptr(), stream)
            ctx.moe_ffn(layer, 0, xT.data_ptr(), T, H, idxT.data_ptr(), wT.data_ptr(), K, H, M, actT.data_ptr(), oT.data_ptr(), H, stream)
    gT = graphed(moe_t)
    t = timed(gT.replay, NL)
    distinct = int(torch.unique(idxT[:, :K]).numel())               # of the last layer run; the layers differ little
    nbytes = distinct * (2 * sg + sd) + E * H * 4
    out["moe_layer_top8_of_128_t32"] = {"us": round(t * 1e6, 2), "gbs": round(nbytes / t / 1e9, 1),
                                        "frac_of_measured_hbm": round(nbytes / t / 1e9 / peak, 3), "bytes": nbytes,
                                        "distinct_experts": distinct, "launches": 4, "form": "cuda graph of 6 layers"}
    return out


def run_ours(args):
    import numpy as np
    import torch

    from orome_b200 import decode_set
    from orome_b200 import format as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    dev = torch.device("cuda", local)
    ctx = F.Context(local)
    if args.x_bits < 0:
        chained = args.mode == "chain" or (args.mode == "auto" and world > 1)
        args.x_bits = 24 if chained else 16
    if args.x_bits:
        ctx.set_option(F.OPT_X_BITS, args.x_bits)
    if args.prefetch_mb >= 0:
        ctx.set_option(F.OPT_PREFETCH_MB, args.prefetch_mb)
    if args.stage_kb > 0:
        ctx.set_option(F.OPT_STAGE_KB, args.stage_kb)
    if args.ctas_per_sm > 0:
        ctx.set_option(F.OPT_CTAS_PER_SM, args.ctas_per_sm)
    if args.grid_per_sm > 0:
        ctx.set_option(F.OPT_GRID_PER_SM, args.grid_per_sm)
    for kv in args.opt:                       # any other OROME_OPT_* by number, for experiments: --opt 15=2
        k, v = kv.split("=")
        ctx.set_option(int(k), int(v))

    if args.kernel:
        # one configuration alone, few launches: the process a profiler capture is taken from
        peak, kind = measured_peak()
        print(json.dumps({"kernels": kernel_extras(torch, F, ctx, peak, only=set(args.kernel.split(",")), reps=max(1, args.steps)),
                          "peak_gbs": peak, "peak_kind": kind}), flush=True)
        return
    ds = decode_set.DecodeSet(args.workload, dev, rank=rank, world=world, layers=args.layers)
    # auto: the chain where it measures faster (several GPUs, one weight format: 715 vs 616 tok/s at N = 2 on the Q8_0 set);
    # chains that mix formats run far slower than launches (the 27B set: 58 vs 217 tok/s on one GPU) and stay on launches
    mode = args.mode if args.mode != "auto" else ("chain" if world > 1 and args.workload == "9b_q8_0" else "launches")
    if world > 1 and args.gather != "fused":
        mode = "launches"                                  # an NCCL all-gather per product cannot be chained
    st = Stepper(torch, F, ctx, ds, dist, fused=args.gather == "fused", mode=mode)
    st.build()
    torch.cuda.synchronize()
    fallback = None
    if world > 1 and args.mode == "auto" and mode == "chain":
        # Pre-flight of the automatically chosen form: two steps and the parity check on every rank.  If any rank sees an
        # expired wait or a wrong result, every rank switches to the launch-per-product form (and the line says so).
        ok = True
        try:
            for _ in range(2):
                st.step()
            torch.cuda.synchronize()
            ok = ctx.status() == 0
            if ok:
                p = st.parity_check()
                ok = ctx.status() == 0 and p["rel_l2"] <= 1e-4 and p["token_matches_reference_argmax"] and p["finite"]
        except Exception as ex:                      # an expired wait surfaces as an error of ctx.status()
            print(f"bench.py: rank {rank}: chain pre-flight failed: {ex!r}", file=sys.stderr, flush=True)
            ok = False
        flag = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            try:
                ctx.status()
            except Exception:
                pass
            fallback = "the chain form failed its pre-flight check on this box; the launch-per-product form was timed instead"
            mode = "launches"
            st = Stepper(torch, F, ctx, ds, dist, fused=args.gather == "fused", mode=mode)
            st.build()
            torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K steps between events on the current stream; returns (device seconds max over ranks, per-step list)."""
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        barrier()
        evs[0].record()
        for i in range(steps):
            fn()
            evs[i + 1].record()
        torch.cuda.synchronize()
        barrier()
        total = evs[0].elapsed_time(evs[steps]) * 1e-3
        per = [evs[i].elapsed_time(evs[i + 1]) * 1e-3 for i in range(steps)]
        if dist is not None:
            t = torch.tensor([total], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t.item())
        return total, per

    # ---- device-resident timing ---------------------------------------------------------
    warmup = max(3, args.warmup)
    for _ in range(warmup):
        st.step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    total, per = timed(st.step, args.steps)
    launches = st.launches_per_step * args.steps
    clocks = sampler.finish()
    ms_per_step = total / args.steps * 1e3
    tok_s = args.steps / total

    # ---- end to end: x from pinned host memory, the token back to the host every step ---------
    # (the reference reads its 4-byte arg-max result after every token, engine.m:1057)
    x_pin = torch.randn(ds.hidden).pin_memory()
    tok_pin = torch.empty(1, dtype=torch.int32).pin_memory()

    def e2e_step():
        st.x_h.copy_(x_pin, non_blocking=True)
        st.step()
        tok_pin.copy_(st.token, non_blocking=True)
        torch.cuda.current_stream().synchronize()      # the host needs the token before the next one starts

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e_total, _ = timed(e2e_step, args.steps)
    wall = time.perf_counter() - t0
    e2e_tok_s = args.steps / max(e_total, 1e-12)

    if ctx.status() != 0:
        raise SystemExit("bench.py: a kernel reported an expired wait; the numbers are void")

    parity = st.parity_check()
    if ctx.status() != 0:
        raise SystemExit("bench.py: a kernel reported an expired wait during the parity check")
    if not (parity["rel_l2"] <= 1e-4 and parity["token_matches_reference_argmax"] and parity["finite"]):
        if rank == 0:
            print(json.dumps({"error": "parity check failed; the timing is void", "parity_check": parity}), flush=True)
        raise SystemExit(2)

    def leave():
        """Multi-rank exit: agree that every rank is done, then leave without tearing NCCL down
        (destroying a communicator that a captured graph still references can block)."""
        if dist is None:
            return
        sys.stdout.flush()
        sys.stderr.flush()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)

    if rank != 0:
        leave()
        return

    peak, peak_kind = measured_peak()
    w_bytes = ds.full_weight_bytes()
    alg_bytes = w_bytes + ds.io_bytes()
    achieved = alg_bytes / (total / args.steps) / 1e9
    # the dominant kernel: the resident chain kernel (one launch = one step) or the per-product GEMV launches
    dom_launches = 1 if mode == "chain" else st.products_per_step
    alg_per_launch = alg_bytes / dom_launches / world                       # bytes ONE GPU's launch moves
    ratio = dram_per_algorithmic(args.workload, mode) if world == 1 else None
    roofline = {
        "bound": "hbm", "achieved": achieved / world, "peak": peak, "unit": "GB/s", "frac": achieved / world / peak, "peak_kind": peak_kind,
        "per": "GPU: algorithmic bytes one GPU's launches move per second against one GPU's peak",
        "aggregate_gbs": achieved, "frac_of_8tbs_nominal": achieved / world / NOMINAL_HBM_GBS,
        "traffic": alg_per_launch * ratio if ratio else None,
        "traffic_note": "DRAM read + write bytes per algorithmic byte from the committed ncu capture of a short cut of this workload "
                        "(profiles/dram_traffic.json), times the algorithmic bytes of one launch",
        "kernel": "gemv_chain_kernel" if mode == "chain" else "gemv_pipe_kernel / gemv_mma_kernel",
        "algorithmic_bytes_per_step": alg_bytes, "launches_per_step": st.launches_per_step, "products_per_step": st.products_per_step,
        "avg_launch_us": ms_per_step * 1e3 / dom_launches,
        "algorithmic_bytes_per_launch": alg_per_launch,
    }

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cs = CpuSteps(args.workload)
        times = cs.timed(64, 1, budget_s=12.0)                                # about 12 s of CPU work
        step_s = sum(times) / len(times)
        cpu = {"value": 1.0 / step_s, "unit": "tok/s", "cores": cs.cores, "kind": cs.kind, "sample": cs.sample_text(len(times)),
               "cpu_gbs": cs.step_bytes / step_s / 1e9}

    line = {
        "metric": "decode_matvec_tok_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 dot products on 24-bit fixed-point x, fp32 accumulate" if ctx.get_option(F.OPT_X_BITS) == 24
        else ("int8 dot products on 16-bit fixed-point x, fp32 accumulate" if mode == "chain" else
              "int8 dot products on fixed-point x (16-bit for plain products, 24-bit for the fused gate/up), fp32 accumulate"),
        "data": "synthetic",
        # `config` names the workload only and is the same for both arms; how this arm runs it is in `form` / `parallelism`
        "config": {"workload": args.workload, "batch": 1, "layers": ds.layers, "weight_bytes": w_bytes,
                   "l2": "inputs larger than L2: every layer has its own weights"},
        "form": ("one resident kernel per token step (recorded chain), every product reads its predecessor's output" if mode == "chain"
                 else "one launch per product" + (", CUDA graph" if st.graph is not None else "")),
        "parallelism": "single GPU" if world == 1 else
        (f"row-split x{world}, y completed by tagged peer stores from the kernel epilogue (NVLink), consumers poll the data" if st.fused
         else f"row-split x{world} + all-gather (NCCL)"),
        "roofline": roofline,
        "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": ds.hidden * 4, "d2h_bytes_per_step": 4,
                "wall_tok_s": args.steps / wall},
        "parity_check": parity, **({"fallback": fallback} if fallback else {}),
        "gpu_launches": int(launches),
        "clocks": clocks,
        "step_ms_min_med_max": [min(per) * 1e3, statistics.median(per) * 1e3, max(per) * 1e3],
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if world == 1 and args.extras:
        del st, ds
        torch.cuda.empty_cache()
        line["kernels"] = kernel_extras(torch, F, ctx, peak)
    print(json.dumps(line), flush=True)
    leave()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="9b_q8_0", choices=["9b_q8_0", "27b_q4_k_m"])
    ap.add_argument("--layers", type=int, default=None, help="override the number of layers (smaller captures for profiling)")
    ap.add_argument("--x-bits", type=int, default=-1, choices=[-1, 0, 16, 24],
                    help="width of the per-group fixed-point form of x inside the kernels: 24 (the library's default: products within 2e-7 "
                         "of the oracle), 16 (plain products within about 3e-5, finer than the fp16 x of the reference's kernels; the fused "
                         "gate/up form stays at 24 bits), 0 = leave the library's default; -1 (default): 16 for the launch-per-product form "
                         "on one GPU, where the consumers' speed counts, 24 for chains (one width for all products, fused ones included)")
    ap.add_argument("--mode", default="auto", choices=["auto", "chain", "launches"],
                    help="auto: launches on one GPU, chain on several; chain: the step is recorded once and runs as one resident kernel; launches: one kernel per product (CUDA graph)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--extras", action="store_true", help="also time the other benchmark configurations kernel by kernel (adds ~20 s)")
    ap.add_argument("--kernel", default="", help="run only the named --extras case(s), comma separated, --steps timing repeats, and exit")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: complete y by peer stores from the kernel epilogue (fused) or by an NCCL all-gather per product")
    ap.add_argument("--ctas-per-sm", type=int, default=0, help="CTAs an SM is sized to hold in the decode kernels (0 = library default, 1)")
    ap.add_argument("--grid-per-sm", type=int, default=0, help="CTAs per SM a decode launch creates (0 = library default, 1)")
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE", help="set a library option by its number (OROME_OPT_*), for experiments")
    ap.add_argument("--stage-kb", type=int, default=0, help="size of one stage of the weight ring in KiB (0 = library default)")
    ap.add_argument("--prefetch-mb", type=int, default=-1, help="cap of the next-tensor L2 prefetch in MiB (0 = off, -1 = library default)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
