"""ctypes binding of ``liborome_cuda.so`` mirroring the reference's format layer.

Names follow inference/include/orome.h: ``TensorRef`` (239-246), ``ExpertProjRef`` /
``ExpertLayerRef`` (249-259), ``format_dispatch_matvec`` (319-322),
``format_from_ggml_type`` (324), ``format_decode_row_f32`` (325, here
``dequant_rows`` on the device).  Device memory is passed as integer addresses
(``tensor.data_ptr()``), streams as ``torch.cuda.current_stream().cuda_stream``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liborome_cuda.so")

VARIANT_DEFAULT, VARIANT_LLAMA = 0, 1
OPT_X_BITS, OPT_FORCE_GENERIC, OPT_STAGE_KB, OPT_CTAS_PER_SM, OPT_PDL, OPT_GRID_PER_SM, OPT_PREFETCH_MB, OPT_TC_MIN_BATCH, OPT_KQUANT_MMA, OPT_WAIT_US, OPT_CHAIN_INFLIGHT, OPT_TC_SLABS, OPT_TC_SPLIT, OPT_TC_TILES = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14

OK, EINVAL, ENOTSUP, ENOMEM, ECUDA, ETIMEOUT = 0, -22, -95, -12, -5, -110
ROUTE_STATIC_MAX_LOGITS = 64 * 256


class OromeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


class TensorRef(C.Structure):
    """orome.h:239-246 with the Metal buffer replaced by a device pointer."""
    _fields_ = [("buffer", C.c_void_p), ("offset", C.c_size_t), ("variant", C.c_uint32), ("format", C.c_int),
                ("out_dim", C.c_uint32), ("in_dim", C.c_uint32)]


class ExpertProjRef(C.Structure):
    _fields_ = [("offset", C.c_size_t), ("expert_stride", C.c_size_t), ("format", C.c_int)]


class ExpertLayerRef(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("gate", ExpertProjRef), ("up", ExpertProjRef), ("down", ExpertProjRef)]


class NormPrologue(C.Structure):
    """rms_norm_apply_partial (shaders.metal:126-149) applied while a product reads its input."""
    _fields_ = [("weight_bf16", C.c_void_p), ("sum_sq_parts", C.c_void_p), ("eps", C.c_float)]


class ResidualEpilogue(C.Structure):
    """residual_add_sum_sq (shaders.metal:86-124) applied where a product writes its output."""
    _fields_ = [("residual", C.c_void_p), ("sum_sq_parts", C.c_void_p)]


SUM_SQ_PARTS = 512


EXPORTS = [
    "orome_cuda_ctx_create", "orome_cuda_ctx_destroy", "orome_cuda_last_error", "orome_cuda_status", "orome_cuda_upload",
    "orome_cuda_free", "orome_format_from_ggml_type", "orome_format_row_bytes", "orome_format_dispatch_matvec",
    "orome_cuda_matvec", "orome_cuda_matvec_group", "orome_cuda_gate_up_swiglu", "orome_cuda_dequant_rows",
    "orome_cuda_moe_route", "orome_cuda_moe_route_static", "orome_cuda_moe_ffn", "orome_cuda_moe_ffn_shard", "orome_cuda_matvec_host", "orome_cuda_set_option",
    "orome_cuda_get_option", "orome_cuda_launch_count", "orome_cuda_hint_next", "orome_cuda_peer_alloc", "orome_cuda_peer_open", "orome_cuda_peer_close", "orome_cuda_gather_setup",
    "orome_cuda_gather_arena_bytes", "orome_cuda_gather_next", "orome_cuda_gather_wait", "orome_cuda_argmax", "orome_cuda_moe_route_pair", "orome_cuda_moe_block", "orome_cuda_moe_block_scratch_floats", "orome_cuda_chain_begin", "orome_cuda_chain_end",
    "orome_cuda_chain_launch", "orome_cuda_chain_destroy", "orome_cuda_chain_info", "orome_cuda_fuse_next", "orome_cuda_download",
]

_lib = None


def lib():
    """Load the CUDA library; fails loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m orome_b200.build` "
                          "(there is no CPU fallback for this path)")
    L = C.CDLL(LIB_PATH)
    vp, sz, u32, i32 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_int
    TR, EL = C.POINTER(TensorRef), C.POINTER(ExpertLayerRef)
    L.orome_cuda_ctx_create.argtypes = [i32, C.POINTER(vp)]
    L.orome_cuda_ctx_destroy.argtypes = [vp]
    L.orome_cuda_ctx_destroy.restype = None
    L.orome_cuda_last_error.restype = C.c_char_p
    L.orome_cuda_status.argtypes = [vp, C.POINTER(i32)]
    L.orome_cuda_upload.argtypes = [vp, vp, sz, C.POINTER(vp)]
    L.orome_cuda_free.argtypes = [vp, vp]
    L.orome_cuda_download.argtypes = [vp, vp, vp, sz]
    L.orome_format_from_ggml_type.argtypes = [u32]
    L.orome_format_row_bytes.argtypes = [i32, u32]
    L.orome_format_row_bytes.restype = sz
    L.orome_format_dispatch_matvec.argtypes = [vp, TR, vp, sz, vp, sz, vp]
    L.orome_cuda_matvec.argtypes = [vp, TR, vp, vp, i32, i32, i32, vp]
    L.orome_cuda_matvec_group.argtypes = [vp, TR, i32, vp, C.POINTER(vp), vp]
    L.orome_cuda_gate_up_swiglu.argtypes = [vp, TR, TR, vp, vp, i32, i32, i32, vp]
    L.orome_cuda_dequant_rows.argtypes = [vp, TR, u32, u32, vp, vp]
    L.orome_cuda_moe_route.argtypes = [vp, TR, vp, i32, i32, u32, vp, vp, vp, vp]
    L.orome_cuda_moe_route_static.argtypes = [vp, TR, vp, i32, i32, u32, vp, vp, vp]
    L.orome_cuda_moe_ffn.argtypes = [vp, EL, u32, vp, i32, i32, vp, vp, u32, u32, u32, vp, vp, i32, vp]
    L.orome_cuda_moe_ffn_shard.argtypes = [vp, EL, u32, vp, i32, i32, vp, vp, u32, u32, u32, u32, u32, vp, vp, vp, i32, vp]
    L.orome_cuda_matvec_host.argtypes = [vp, TR, vp, vp, i32]
    L.orome_cuda_set_option.argtypes = [vp, i32, i32]
    L.orome_cuda_get_option.argtypes = [vp, i32, C.POINTER(i32)]
    L.orome_cuda_hint_next.argtypes = [vp, TR]
    L.orome_cuda_peer_alloc.argtypes = [vp, sz, C.POINTER(vp), C.c_char_p]
    L.orome_cuda_peer_open.argtypes = [vp, C.c_char_p, C.POINTER(vp)]
    L.orome_cuda_peer_close.argtypes = [vp, vp]
    L.orome_cuda_gather_setup.argtypes = [vp, i32, i32, C.POINTER(vp), sz, i32]
    L.orome_cuda_gather_arena_bytes.argtypes = [sz, i32]
    L.orome_cuda_gather_arena_bytes.restype = sz
    L.orome_cuda_gather_next.argtypes = [vp, i32, i32]
    L.orome_cuda_gather_wait.argtypes = [vp, i32, vp, u32, vp]
    L.orome_cuda_argmax.argtypes = [vp, vp, u32, vp, vp]
    L.orome_cuda_moe_route_pair.argtypes = [vp, TR, TR, vp, i32, i32, u32, vp, vp, vp, vp, vp]
    L.orome_cuda_moe_block.argtypes = [vp, EL, u32, TR, TR, TR, vp, i32, i32, vp, vp, vp, u32, u32, u32, vp, i32, vp, vp, i32, vp]
    L.orome_cuda_moe_block_scratch_floats.argtypes = [i32, u32, u32, u32, u32]
    L.orome_cuda_moe_block_scratch_floats.restype = sz
    L.orome_cuda_chain_begin.argtypes = [vp]
    L.orome_cuda_chain_end.argtypes = [vp, C.POINTER(vp)]
    L.orome_cuda_chain_launch.argtypes = [vp, vp, vp]
    L.orome_cuda_chain_destroy.argtypes = [vp, vp]
    L.orome_cuda_chain_destroy.restype = None
    L.orome_cuda_chain_info.argtypes = [vp, C.POINTER(i32), C.POINTER(C.c_uint64), C.POINTER(i32), C.POINTER(i32)]
    L.orome_cuda_fuse_next.argtypes = [vp, C.POINTER(NormPrologue), C.POINTER(ResidualEpilogue)]
    L.orome_cuda_launch_count.argtypes = [vp]
    L.orome_cuda_launch_count.restype = C.c_uint64
    _lib = L
    return L


def _chk(rc: int):
    if rc != 0:
        raise OromeError(rc, lib().orome_cuda_last_error().decode())


def format_from_ggml_type(ggml_type: int) -> int:
    return int(lib().orome_format_from_ggml_type(ggml_type))


def format_row_bytes(fmt: int, in_dim: int) -> int:
    return int(lib().orome_format_row_bytes(fmt, in_dim))


class Context:
    """One CUDA device bound to the library (the role MetalCtx plays for this path)."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        _chk(lib().orome_cuda_ctx_create(device, C.byref(self._h)))
        self.device = device

    def close(self):
        if self._h:
            lib().orome_cuda_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- memory ---------------------------------------------------------------
    def upload(self, host_bytes) -> int:
        """Copy a bytes-like / numpy uint8 array to a new device allocation; returns the device address."""
        import numpy as np
        a = np.ascontiguousarray(np.frombuffer(host_bytes, dtype=np.uint8) if not hasattr(host_bytes, "ctypes") else host_bytes)
        out = C.c_void_p()
        _chk(lib().orome_cuda_upload(self._h, a.ctypes.data_as(C.c_void_p), a.nbytes, C.byref(out)))
        return int(out.value)

    def download(self, dev: int, nbytes: int) -> bytes:
        """Device memory as host bytes, after the device has finished (the reference reads its shared buffers directly)."""
        buf = C.create_string_buffer(nbytes)
        _chk(lib().orome_cuda_download(self._h, dev, buf, nbytes))
        return buf.raw

    def free(self, dev_base: int):
        _chk(lib().orome_cuda_free(self._h, C.c_void_p(dev_base)))

    # -- options ----------------------------------------------------------------
    def set_option(self, key: int, value: int):
        _chk(lib().orome_cuda_set_option(self._h, key, value))

    def get_option(self, key: int) -> int:
        v = C.c_int()
        _chk(lib().orome_cuda_get_option(self._h, key, C.byref(v)))
        return v.value

    def status(self) -> int:
        v = C.c_int()
        _chk(lib().orome_cuda_status(self._h, C.byref(v)))
        return v.value

    @property
    def launch_count(self) -> int:
        return int(lib().orome_cuda_launch_count(self._h))

    # -- one token step as one launch (the reference's one command buffer per token, engine.m:453-454, 1048-1050) --
    def chain_begin(self):
        """From here to chain_end the batch-1 entry points record their product instead of launching it."""
        _chk(lib().orome_cuda_chain_begin(self._h))

    def chain_end(self) -> "Chain":
        out = C.c_void_p()
        _chk(lib().orome_cuda_chain_end(self._h, C.byref(out)))
        return Chain(self, out)

    def argmax(self, data: int, count: int, result: int, stream: int = 0):
        """Index of the largest of `count` floats at `data` into the uint32 at `result` (shaders.metal:1249-1305)."""
        _chk(lib().orome_cuda_argmax(self._h, data, count, result, stream))

    # -- multi-GPU gather ----------------------------------------------------------
    def peer_alloc(self, nbytes: int):
        """(device address, 64-byte IPC handle) of a new zeroed allocation that other processes can map."""
        out = C.c_void_p()
        h = C.create_string_buffer(64)
        _chk(lib().orome_cuda_peer_alloc(self._h, nbytes, C.byref(out), h))
        return int(out.value), h.raw

    def peer_open(self, handle: bytes) -> int:
        out = C.c_void_p()
        _chk(lib().orome_cuda_peer_open(self._h, handle, C.byref(out)))
        return int(out.value)

    def peer_close(self, ptr: int):
        _chk(lib().orome_cuda_peer_close(self._h, C.c_void_p(ptr)))

    def gather_setup(self, rank: int, world: int, arenas, data_bytes: int, n_flags: int):
        arr = (C.c_void_p * world)(*arenas) if world > 1 else None
        _chk(lib().orome_cuda_gather_setup(self._h, rank, world, arr, data_bytes, n_flags))

    def gather_next(self, wait_flag: int = -1, publish_flag: int = -1):
        _chk(lib().orome_cuda_gather_next(self._h, wait_flag, publish_flag))

    def gather_wait(self, flag: int, vec_ptr: int, n: int, stream: int = 0):
        """Complete the plain copy of the gathered vector of `n` floats at `vec_ptr` (inside the arena)."""
        _chk(lib().orome_cuda_gather_wait(self._h, flag, vec_ptr, n, stream))

    def fuse_next(self, prologue: NormPrologue | None = None, epilogue: ResidualEpilogue | None = None):
        """Fuse the norm (prologue) and / or the residual add + sum of squares (epilogue) into the next batch-1 product."""
        _chk(lib().orome_cuda_fuse_next(self._h, C.byref(prologue) if prologue is not None else None,
                                        C.byref(epilogue) if epilogue is not None else None))

    def hint_next(self, ref: TensorRef | None):
        _chk(lib().orome_cuda_hint_next(self._h, C.byref(ref) if ref is not None else None))

    # -- the path ---------------------------------------------------------------
    def format_dispatch_matvec(self, ref: TensorRef, in_buf: int, in_off: int, out_buf: int, out_off: int, stream: int = 0):
        _chk(lib().orome_format_dispatch_matvec(self._h, C.byref(ref), in_buf, in_off, out_buf, out_off, stream))

    def matvec(self, ref: TensorRef, x: int, y: int, batch: int = 1, ldx: int = 0, ldy: int = 0, stream: int = 0):
        _chk(lib().orome_cuda_matvec(self._h, C.byref(ref), x, y, batch, ldx, ldy, stream))

    def matvec_group(self, refs, x: int, ys, stream: int = 0):
        arr = (TensorRef * len(refs))(*refs)
        yp = (C.c_void_p * len(ys))(*ys)
        _chk(lib().orome_cuda_matvec_group(self._h, arr, len(refs), x, yp, stream))

    def gate_up_swiglu(self, gate: TensorRef, up: TensorRef, x: int, out: int, batch: int = 1, ldx: int = 0, ldo: int = 0,
                       stream: int = 0):
        _chk(lib().orome_cuda_gate_up_swiglu(self._h, C.byref(gate), C.byref(up), x, out, batch, ldx, ldo, stream))

    def dequant_rows(self, ref: TensorRef, row0: int, nrows: int, out: int, stream: int = 0):
        _chk(lib().orome_cuda_dequant_rows(self._h, C.byref(ref), row0, nrows, out, stream))

    def moe_route(self, router: TensorRef, x: int, n_tokens: int, ldx: int, K: int, idx: int, w: int, logits: int = 0,
                  stream: int = 0):
        _chk(lib().orome_cuda_moe_route(self._h, C.byref(router), x, n_tokens, ldx, K, idx, w, logits or None, stream))

    def moe_route_static(self, router: TensorRef, x: int, n_tokens: int, ldx: int, K: int, idx: int, w: int, stream: int = 0):
        """Routing with the logits in the library's fixed scratch array: no allocation (see include/orome_cuda.h)."""
        _chk(lib().orome_cuda_moe_route_static(self._h, C.byref(router), x, n_tokens, ldx, K, idx, w, stream))

    def moe_ffn(self, layer: ExpertLayerRef, variant: int, x: int, n_tokens: int, ldx: int, idx: int, w: int, K: int,
                hidden: int, inter: int, act: int, out: int, ldo: int, stream: int = 0):
        _chk(lib().orome_cuda_moe_ffn(self._h, C.byref(layer), variant, x, n_tokens, ldx, idx, w, K, hidden, inter, act, out,
                                      ldo, stream))

    def moe_route_pair(self, router: TensorRef, shared_gate: TensorRef, x: int, n_tokens: int, ldx: int, K: int, idx: int, w: int,
                       shared_logit: int, logits: int = 0, stream: int = 0):
        """Routing plus the shared-expert gate logit in one launch (engine.m:656-679, shaders.metal:1232)."""
        _chk(lib().orome_cuda_moe_route_pair(self._h, C.byref(router), C.byref(shared_gate), x, n_tokens, ldx, K, idx, w, shared_logit,
                                             logits or None, stream))

    def moe_block(self, layer: ExpertLayerRef, variant: int, shared, x: int, n_tokens: int, ldx: int, idx: int, w: int, shared_logit: int,
                  K: int, hidden: int, inter: int, h_mid: int, ld_mid: int, scratch: int, out: int, ldo: int, stream: int = 0):
        """Routed experts + shared expert + combine (engine.m:158-340).  shared: (gate, up, down) TensorRefs or None."""
        sg, su, sd = (C.byref(r) for r in shared) if shared else (None, None, None)
        _chk(lib().orome_cuda_moe_block(self._h, C.byref(layer), variant, sg, su, sd, x, n_tokens, ldx, idx, w, shared_logit or None, K, hidden,
                                        inter, h_mid or None, ld_mid, scratch, out, ldo, stream))

    def moe_ffn_shard(self, layer_local: ExpertLayerRef, variant: int, x: int, n_tokens: int, ldx: int, idx: int, w: int, K: int,
                      hidden: int, inter: int, first_expert: int, n_local: int, idx_local: int, act: int, out: int, ldo: int,
                      stream: int = 0):
        """This GPU's share of the expert FFN: only the selected experts in [first_expert, first_expert + n_local)."""
        _chk(lib().orome_cuda_moe_ffn_shard(self._h, C.byref(layer_local), variant, x, n_tokens, ldx, idx, w, K, hidden, inter,
                                            first_expert, n_local, idx_local, act, out, ldo, stream))

    def matvec_host(self, ref: TensorRef, x_host, y_host, batch: int = 1):
        """x_host / y_host: contiguous float32 numpy arrays (host memory)."""
        _chk(lib().orome_cuda_matvec_host(self._h, C.byref(ref), x_host.ctypes.data_as(C.c_void_p),
                                          y_host.ctypes.data_as(C.c_void_p), batch))


class Chain:
    """A recorded sequence of products (orome_cuda_chain) that one launch runs."""

    def __init__(self, ctx: Context, handle):
        self.ctx, self._h = ctx, handle

    def launch(self, stream: int = 0):
        _chk(lib().orome_cuda_chain_launch(self.ctx._h, self._h, stream))
        
    def info(self) -> dict:
        n, st, sb = C.c_int(), C.c_int(), C.c_int()
        wb = C.c_uint64()
        _chk(lib().orome_cuda_chain_info(self._h, C.byref(n), C.byref(wb), C.byref(st), C.byref(sb)))
        return dict(products=n.value, weight_bytes=int(wb.value), stages=st.value, stage_bytes=sb.value)

    def close(self):
        if self._h and self.ctx._h:
            lib().orome_cuda_chain_destroy(self.ctx._h, self._h)
        self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def moe_block_scratch_floats(n_tokens: int, K: int, hidden: int, inter: int, shared_inter: int) -> int:
    return int(lib().orome_cuda_moe_block_scratch_floats(n_tokens, K, hidden, inter, shared_inter))


def gather_arena_bytes(data_bytes: int, n_flags: int) -> int:
    return int(lib().orome_cuda_gather_arena_bytes(data_bytes, n_flags))


def tensor_ref(buffer: int, offset: int, fmt: int, out_dim: int, in_dim: int, variant: int = VARIANT_DEFAULT) -> TensorRef:
    return TensorRef(buffer, offset, variant, fmt, out_dim, in_dim)
