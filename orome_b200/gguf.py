"""ctypes binding of the GGUF reader and the GGUF half of the format layer in ``liborome_cuda.so``.

Names follow the reference: ``gguf_open`` / ``gguf_find_tensor`` / ``gguf_tensor_size``
(inference/src/gguf.m:273-550), ``format_provider_open_gguf`` (inference/src/format.m:343-363),
``format_resolve_expert_layer`` (format.m:374-409) and ``build_tensor_cache_gguf`` (format.m:458-590).
The parsing is done by the C library; this module only declares the structures and wraps the handles.
"""
from __future__ import annotations

import ctypes as C

from . import format as F

EXPORTS = [
    "orome_gguf_open", "orome_gguf_close", "orome_gguf_find_tensor", "orome_gguf_tensor_size", "orome_gguf_meta",
    "orome_gguf_num_tensors", "orome_gguf_tensor", "orome_gguf_data_offset", "orome_gguf_file_size", "orome_gguf_base",
    "orome_gguf_chat_template", "orome_format_provider_open_gguf", "orome_format_provider_close",
    "orome_format_resolve_expert_layer", "orome_build_tensor_cache_gguf", "orome_free_tensor_cache",
]


class TensorInfo(C.Structure):
    """GGUFTensorInfo, orome.h:405-411."""
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("type", C.c_uint32),
                ("offset", C.c_uint64)]


class Meta(C.Structure):
    _fields_ = ([("arch", C.c_char * 32), ("ffn_is_moe", C.c_int)]
                + [(n, C.c_int) for n in (
                    "num_layers", "hidden_dim", "num_experts", "num_experts_per_tok", "num_attn_heads", "num_kv_heads",
                    "moe_intermediate", "context_length", "attn_key_length", "attn_value_length", "rope_dimension_count",
                    "ssm_conv_kernel", "ssm_state_size", "ssm_group_count", "ssm_time_step_rank", "ssm_inner_size",
                    "full_attention_interval", "eos_token_id", "padding_token_id", "vocab_size")]
                + [("rope_theta", C.c_float), ("rms_norm_eps", C.c_float), ("alignment", C.c_uint32), ("version", C.c_uint32)])


class FormatProvider(C.Structure):
    _fields_ = [("gguf", C.c_void_p), ("model_buf", C.c_void_p), ("ctx", C.c_void_p)]


class ModelShape(C.Structure):
    _fields_ = ([(n, C.c_int) for n in (
        "num_layers", "hidden_dim", "moe_intermediate", "shared_intermediate", "num_experts", "vocab_size", "ffn_is_moe",
        "num_attn_heads", "num_kv_heads", "head_dim", "linear_conv_dim", "linear_num_v_heads", "linear_value_dim")]
        + [("layer_is_linear", C.POINTER(C.c_uint8))])


_LAYER_REFS = ("routing_gate", "shared_gate", "shared_up", "shared_down", "shared_expert_gate", "dense_gate", "dense_up",
               "dense_down", "lin_qkv", "lin_z", "lin_a", "lin_b", "lin_o", "full_q", "full_k", "full_v", "full_o")


class LayerTensorCache(C.Structure):
    _fields_ = [(n, F.TensorRef) for n in _LAYER_REFS] + [("owned_q", C.c_void_p)]


class GlobalTensorCache(C.Structure):
    _fields_ = [("token_embd", F.TensorRef), ("lm_head", F.TensorRef)]


_bound = False


def lib():
    global _bound
    L = F.lib()
    if _bound:
        return L
    vp, sz, u32, i32 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_int
    TI = C.POINTER(TensorInfo)
    L.orome_gguf_open.argtypes = [C.c_char_p]
    L.orome_gguf_open.restype = vp
    L.orome_gguf_close.argtypes = [vp]
    L.orome_gguf_close.restype = None
    L.orome_gguf_find_tensor.argtypes = [vp, C.c_char_p]
    L.orome_gguf_find_tensor.restype = TI
    L.orome_gguf_tensor_size.argtypes = [TI]
    L.orome_gguf_tensor_size.restype = sz
    L.orome_gguf_meta.argtypes = [vp]
    L.orome_gguf_meta.restype = C.POINTER(Meta)
    L.orome_gguf_num_tensors.argtypes = [vp]
    L.orome_gguf_num_tensors.restype = C.c_uint64
    L.orome_gguf_tensor.argtypes = [vp, C.c_uint64]
    L.orome_gguf_tensor.restype = TI
    for f in (L.orome_gguf_data_offset, L.orome_gguf_file_size):
        f.argtypes = [vp]
        f.restype = sz
    L.orome_gguf_base.argtypes = [vp]
    L.orome_gguf_base.restype = vp
    L.orome_gguf_chat_template.argtypes = [vp]
    L.orome_gguf_chat_template.restype = C.c_char_p
    L.orome_format_provider_open_gguf.argtypes = [vp, vp, C.POINTER(FormatProvider)]
    L.orome_format_provider_close.argtypes = [C.POINTER(FormatProvider)]
    L.orome_format_provider_close.restype = None
    L.orome_format_resolve_expert_layer.argtypes = [C.POINTER(FormatProvider), i32, u32]
    L.orome_format_resolve_expert_layer.restype = F.ExpertLayerRef
    L.orome_build_tensor_cache_gguf.argtypes = [C.POINTER(FormatProvider), C.POINTER(ModelShape), u32,
                                                C.POINTER(LayerTensorCache), C.POINTER(GlobalTensorCache)]
    L.orome_free_tensor_cache.argtypes = [C.POINTER(FormatProvider), C.POINTER(LayerTensorCache), i32]
    L.orome_free_tensor_cache.restype = None
    _bound = True
    return L


class GGUFFile:
    """An opened GGUF file (gguf_open, gguf.m:273)."""

    def __init__(self, path: str):
        self._h = lib().orome_gguf_open(str(path).encode())
        if not self._h:
            raise F.OromeError(F.EINVAL, lib().orome_cuda_last_error().decode())

    def close(self):
        if self._h:
            lib().orome_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def handle(self) -> int:
        return self._h

    @property
    def meta(self) -> Meta:
        return lib().orome_gguf_meta(self._h).contents

    @property
    def num_tensors(self) -> int:
        return int(lib().orome_gguf_num_tensors(self._h))

    @property
    def data_offset(self) -> int:
        return int(lib().orome_gguf_data_offset(self._h))

    @property
    def file_size(self) -> int:
        return int(lib().orome_gguf_file_size(self._h))

    @property
    def chat_template(self):
        s = lib().orome_gguf_chat_template(self._h)
        return None if s is None else s.decode()

    def tensor(self, index: int):
        p = lib().orome_gguf_tensor(self._h, index)
        return p.contents if p else None

    def find_tensor(self, name: str):
        """gguf_find_tensor (gguf.m:531): the directory entry, or None."""
        p = lib().orome_gguf_find_tensor(self._h, name.encode())
        return p.contents if p else None

    def tensor_size(self, ti) -> int:
        """gguf_tensor_size (gguf.m:540)."""
        return int(lib().orome_gguf_tensor_size(C.byref(ti))) if ti is not None else int(lib().orome_gguf_tensor_size(None))


class Provider:
    """format_provider_open_gguf (format.m:343): the file image in device memory."""

    def __init__(self, ctx: F.Context, gf: GGUFFile):
        self.fp = FormatProvider()
        self.gf, self.ctx = gf, ctx
        F._chk(lib().orome_format_provider_open_gguf(ctx._h, gf.handle, C.byref(self.fp)))
        self._caches = []

    @property
    def model_buf(self) -> int:
        return self.fp.model_buf

    def resolve_expert_layer(self, layer_idx: int, num_experts: int) -> F.ExpertLayerRef:
        return lib().orome_format_resolve_expert_layer(C.byref(self.fp), layer_idx, num_experts)

    def build_tensor_cache(self, shape: ModelShape, variant: int = F.VARIANT_DEFAULT, layer_is_linear=None):
        """build_tensor_cache_gguf (format.m:458): (layers, globals)."""
        keep = None
        if layer_is_linear is not None:
            keep = (C.c_uint8 * shape.num_layers)(*[1 if v else 0 for v in layer_is_linear])
            shape.layer_is_linear = C.cast(keep, C.POINTER(C.c_uint8))
        layers = (LayerTensorCache * max(1, shape.num_layers))()
        glob = GlobalTensorCache()
        F._chk(lib().orome_build_tensor_cache_gguf(C.byref(self.fp), C.byref(shape), variant, layers, C.byref(glob)))
        self._caches.append((layers, shape.num_layers))
        return layers, glob

    def close(self):
        for layers, n in self._caches:
            lib().orome_free_tensor_cache(C.byref(self.fp), layers, n)
        self._caches = []
        if self.fp.model_buf:
            lib().orome_format_provider_close(C.byref(self.fp))
