// GGUF reader and the GGUF half of the format layer: from a file on disk to the TensorRef / ExpertLayerRef handles
// the matvec entry points take.  Host code only (it is a .cu file so that it is built into the same library).
//
// Follows the behaviour of Orome's inference/src/gguf.m:273-550 (container parsing, metadata extraction, shape
// inference, tensor sizes) and inference/src/format.m:343-590 (provider, expert resolver, tensor cache) -- what is
// parsed, which keys are honoured, which fall-backs apply -- with a structure of its own: a bounds-checked cursor
// that latches its first failure, a key table instead of a comparison ladder, a name index from the standard
// library, and device-side strided copies for the one tensor that is rearranged at load time.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/orome_gguf.h"
#include "ctx.h"

namespace {

// ---- the container's value types and the block geometry of the ggml tensor types ------------------------------
enum : uint32_t { VT_U8, VT_I8, VT_U16, VT_I16, VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STR, VT_ARR, VT_U64, VT_I64, VT_F64 };

struct BlockGeom { uint32_t type, weights, bytes; };
// ggml type id -> weights per block, bytes per block (gguf.m:64-104).  Types outside the table count as one
// weight per block of zero bytes, i.e. size 0, as the reference computes it.
constexpr BlockGeom kGeom[] = {
    {0, 1, 4},     {1, 1, 2},     {30, 1, 2},                                  // F32, F16, BF16
    {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},   {8, 32, 34},   {9, 32, 36},   // Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q8_1
    {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},   // Q2_K .. Q8_K
};

BlockGeom geom_of(uint32_t type)
{
    for (const BlockGeom &g : kGeom)
        if (g.type == type) return g;
    return {type, 1, 0};
}

// ---- bounds-checked little-endian cursor -------------------------------------------------------------------------
// Reading past the end yields zeros and latches `short_read`, so the parser can run to its end and report once.
struct Cursor {
    const uint8_t *base;
    size_t size, pos = 0;
    bool short_read = false;

    bool room(uint64_t n) const { return n <= size - pos; }
    template <class T> T get()
    {
        T v{};
        if (!room(sizeof(T))) { short_read = true; pos = size; return v; }
        memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    void skip(uint64_t n)
    {
        if (!room(n)) { short_read = true; pos = size; return; }
        pos += n;
    }
    // length-prefixed, not terminated in the file; strings over 1 MiB are refused like the reference does (gguf.m:165)
    bool str(std::string *out)
    {
        uint64_t len = get<uint64_t>();
        if (short_read || len > (1u << 20) || !room(len)) { short_read = true; return false; }
        out->assign(reinterpret_cast<const char *>(base + pos), len);
        pos += len;
        return true;
    }
    void skip_value(uint32_t vt, int depth = 0)
    {
        static const uint8_t width[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
        if (vt == VT_STR) { std::string s; str(&s); return; }
        if (vt == VT_ARR) {
            uint32_t et = get<uint32_t>();
            uint64_t n = get<uint64_t>();
            if (et < 13 && width[et]) { if (n > size) { short_read = true; return; } skip(n * width[et]); return; }
            if (depth > 4) { short_read = true; return; }
            for (uint64_t i = 0; i < n && !short_read; i++) skip_value(et, depth + 1);
            return;
        }
        if (vt < 13) skip(width[vt]);
        // an unknown value type consumes nothing, as in the reference (gguf.m:174-201)
    }
    // a scalar as an unsigned integer; signed types sign-extend, anything else is skipped and reads as 0 (gguf.m:204-217)
    uint64_t as_uint(uint32_t vt)
    {
        switch (vt) {
        case VT_U8: case VT_BOOL: return get<uint8_t>();
        case VT_I8:  return (uint64_t)(int64_t)get<int8_t>();
        case VT_U16: return get<uint16_t>();
        case VT_I16: return (uint64_t)(int64_t)get<int16_t>();
        case VT_U32: return get<uint32_t>();
        case VT_I32: return (uint64_t)(int64_t)get<int32_t>();
        case VT_U64: case VT_I64: return get<uint64_t>();
        default: skip_value(vt); return 0;
        }
    }
    // a scalar as a float; a double is consumed and reads as 0, which is what the reference does (gguf.m:219-223)
    float as_float(uint32_t vt)
    {
        if (vt == VT_F32) return get<float>();
        if (vt == VT_F64) { skip(8); return 0.0f; }
        return (float)as_uint(vt);
    }
};

// ---- metadata keys under "<architecture>." (gguf.m:352-393) ------------------------------------------------------
struct IntKey { const char *field; int OromeGGUFMeta::*slot; };
constexpr IntKey kIntKeys[] = {
    {"block_count", &OromeGGUFMeta::num_layers},
    {"context_length", &OromeGGUFMeta::context_length},
    {"embedding_length", &OromeGGUFMeta::hidden_dim},
    {"expert_count", &OromeGGUFMeta::num_experts},
    {"expert_used_count", &OromeGGUFMeta::num_experts_per_tok},
    {"feed_forward_length", &OromeGGUFMeta::moe_intermediate},
    {"attention.head_count", &OromeGGUFMeta::num_attn_heads},
    {"attention.head_count_kv", &OromeGGUFMeta::num_kv_heads},
    {"attention.key_length", &OromeGGUFMeta::attn_key_length},
    {"attention.value_length", &OromeGGUFMeta::attn_value_length},
    {"rope.dimension_count", &OromeGGUFMeta::rope_dimension_count},
    {"ssm.conv_kernel", &OromeGGUFMeta::ssm_conv_kernel},
    {"ssm.state_size", &OromeGGUFMeta::ssm_state_size},
    {"ssm.group_count", &OromeGGUFMeta::ssm_group_count},
    {"ssm.time_step_rank", &OromeGGUFMeta::ssm_time_step_rank},
    {"ssm.inner_size", &OromeGGUFMeta::ssm_inner_size},
    {"full_attention_interval", &OromeGGUFMeta::full_attention_interval},
    {"vocab_size", &OromeGGUFMeta::vocab_size},
};
struct FloatKey { const char *field; float OromeGGUFMeta::*slot; };
constexpr FloatKey kFloatKeys[] = {
    {"attention.layer_norm_rms_epsilon", &OromeGGUFMeta::rms_norm_eps},
    {"rope.freq_base", &OromeGGUFMeta::rope_theta},
};

bool contains(const char *hay, const char *needle) { return strstr(hay, needle) != nullptr; }

}  // namespace

struct OromeGGUFFile {
    int fd = -1;
    void *map = nullptr;
    size_t file_size = 0, data_offset = 0;
    OromeGGUFMeta meta{};
    std::vector<OromeGGUFTensorInfo> tensors;
    std::vector<std::string> names;                       // owns the bytes OromeGGUFTensorInfo.name points at
    std::unordered_map<std::string, size_t> by_name;      // first occurrence wins
    std::string chat_template;
    bool has_chat_template = false;
};

namespace {

void read_metadata(Cursor &c, uint64_t count, OromeGGUFFile *gf)
{
    OromeGGUFMeta &m = gf->meta;
    std::string key;
    for (uint64_t i = 0; i < count && !c.short_read; i++) {
        if (!c.str(&key)) break;
        uint32_t vt = c.get<uint32_t>();
        if (key == "general.architecture") {
            std::string v;
            if (vt == VT_STR && c.str(&v)) snprintf(m.arch, sizeof m.arch, "%s", v.c_str());
            else if (vt != VT_STR) c.skip_value(vt);
            continue;
        }
        if (key == "general.alignment") { m.alignment = (uint32_t)c.as_uint(vt); continue; }
        if (key == "tokenizer.ggml.eos_token_id") { m.eos_token_id = (int)c.as_uint(vt); continue; }
        if (key == "tokenizer.ggml.padding_token_id") { m.padding_token_id = (int)c.as_uint(vt); continue; }
        if (key == "tokenizer.chat_template" && vt == VT_STR) { gf->has_chat_template = c.str(&gf->chat_template); continue; }
        // architecture keys: the prefix is whatever architecture has been seen so far, "llama" before that
        std::string prefix = std::string(m.arch[0] ? m.arch : "llama") + ".";
        bool taken = false;
        if (key.compare(0, prefix.size(), prefix) == 0) {
            const char *field = key.c_str() + prefix.size();
            for (const IntKey &k : kIntKeys)
                if (!taken && strcmp(field, k.field) == 0) { m.*(k.slot) = (int)c.as_uint(vt); taken = true; }
            for (const FloatKey &k : kFloatKeys)
                if (!taken && strcmp(field, k.field) == 0) { m.*(k.slot) = c.as_float(vt); taken = true; }
        }
        if (!taken) c.skip_value(vt);
    }
}

void read_directory(Cursor &c, uint64_t count, OromeGGUFFile *gf)
{
    gf->tensors.resize(count);
    gf->names.resize(count);
    for (uint64_t i = 0; i < count && !c.short_read; i++) {
        OromeGGUFTensorInfo &t = gf->tensors[i];
        memset(&t, 0, sizeof t);
        if (!c.str(&gf->names[i])) break;
        t.n_dims = c.get<uint32_t>();
        for (uint32_t d = 0; d < t.n_dims && !c.short_read; d++) {
            uint64_t v = c.get<uint64_t>();
            if (d < 4) t.dims[d] = v;                     // further dimensions are read and dropped
        }
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
    }
    for (uint64_t i = 0; i < count; i++) {
        gf->tensors[i].name = const_cast<char *>(gf->names[i].c_str());
        gf->by_name.emplace(gf->names[i], i);
    }
}

// what the metadata leaves open is read off the tensor directory (gguf.m:439-503)
void infer_from_tensors(OromeGGUFFile *gf)
{
    OromeGGUFMeta &m = gf->meta;
    bool moe = false, dense = false;
    for (const std::string &n : gf->names) {
        const char *s = n.c_str();
        if (contains(s, "ffn_gate_exps") || contains(s, "ffn_up_exps") || contains(s, "ffn_down_exps")) moe = true;
        else if (contains(s, ".ffn_gate.weight") || contains(s, ".ffn_up.weight") || contains(s, ".ffn_down.weight")) dense = true;
    }
    m.ffn_is_moe = moe ? 1 : dense ? 0 : (m.num_experts > 0);

    if (m.vocab_size == 0) {
        auto it = gf->by_name.find("token_embd.weight");
        if (it != gf->by_name.end()) {
            const OromeGGUFTensorInfo &t = gf->tensors[it->second];
            for (uint32_t d = 0; d < t.n_dims && d < 4; d++)
                if (t.dims[d] != (uint64_t)m.hidden_dim) { m.vocab_size = (int)t.dims[d]; break; }
        }
    }
    if (m.moe_intermediate == 0) {
        for (const OromeGGUFTensorInfo &t : gf->tensors) {
            bool candidate = m.ffn_is_moe ? contains(t.name, "ffn_gate_exps")
                                          : (contains(t.name, ".ffn_gate.weight") || contains(t.name, ".ffn_up.weight"));
            if (!candidate) continue;
            for (uint32_t d = 0; d < t.n_dims && d < 4; d++) {
                uint64_t v = t.dims[d];
                bool known = v == (uint64_t)m.hidden_dim || (m.ffn_is_moe && v == (uint64_t)m.num_experts);
                if (!known) { m.moe_intermediate = (int)v; break; }
            }
            if (m.moe_intermediate) break;
        }
    }
}

OromeTensorRef ref_of(const OromeFormatProvider *fp, uint32_t variant, const char *name, uint32_t out_dim, uint32_t in_dim)
{
    OromeTensorRef r{};
    const OromeGGUFTensorInfo *t = orome_gguf_find_tensor(fp->gguf, name);
    if (!t) return r;
    r.buffer = fp->model_buf;
    r.offset = fp->gguf->data_offset + t->offset;
    r.variant = variant;
    r.format = orome_format_from_ggml_type(t->type);
    r.out_dim = out_dim;
    r.in_dim = in_dim;
    return r;
}

OromeTensorRef layer_ref(const OromeFormatProvider *fp, uint32_t variant, int layer, const char *what, int out_dim, int in_dim)
{
    char name[128];
    snprintf(name, sizeof name, "blk.%d.%s.weight", layer, what);
    return ref_of(fp, variant, name, (uint32_t)out_dim, (uint32_t)in_dim);
}

}  // namespace

extern "C" OromeGGUFFile *orome_gguf_open(const char *path)
{
    if (!path) { orome_fail(OROME_EINVAL, "gguf_open: NULL path"); return nullptr; }
    int fd = open(path, O_RDONLY);
    if (fd < 0) { orome_fail(OROME_EINVAL, "gguf_open: cannot open %s", path); return nullptr; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        orome_fail(OROME_EINVAL, "gguf_open: %s is too short to hold a GGUF header", path);
        return nullptr;
    }
    void *map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) { close(fd); orome_fail(OROME_ENOMEM, "gguf_open: mmap of %s failed", path); return nullptr; }

    Cursor c{static_cast<const uint8_t *>(map), (size_t)st.st_size};
    uint32_t magic = c.get<uint32_t>(), version = c.get<uint32_t>();
    const char *why = nullptr;
    if (magic != 0x46554747u) why = "bad magic (not \"GGUF\")";
    else if (version < 2 || version > 3) why = "unsupported version (2 and 3 are read)";
    uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    // every directory entry takes at least 24 bytes and every key/value pair at least 13
    if (!why && (n_tensors > c.size / 24 || n_kv > c.size / 13)) why = "header counts exceed the file size";
    if (why) {
        munmap(map, (size_t)st.st_size);
        close(fd);
        orome_fail(OROME_EINVAL, "gguf_open: %s: %s", path, why);
        return nullptr;
    }

    OromeGGUFFile *gf = new OromeGGUFFile;
    gf->fd = fd;
    gf->map = map;
    gf->file_size = (size_t)st.st_size;
    gf->meta.eos_token_id = gf->meta.padding_token_id = -1;
    gf->meta.alignment = 32;
    gf->meta.version = version;
    read_metadata(c, n_kv, gf);
    read_directory(c, n_tensors, gf);
    uint32_t al = gf->meta.alignment;
    if (!c.short_read && (al == 0 || (al & (al - 1)))) why = "general.alignment is not a power of two";
    if (c.short_read) why = "metadata or tensor directory runs past the end of the file";
    if (!why) {
        gf->data_offset = (c.pos + al - 1) & ~(size_t)(al - 1);
        for (const OromeGGUFTensorInfo &t : gf->tensors) {
            size_t bytes = orome_gguf_tensor_size(&t);
            if (t.offset > gf->file_size || gf->data_offset > gf->file_size - t.offset || bytes > gf->file_size - gf->data_offset - t.offset) {
                why = "a tensor's data lies outside the file";
                break;
            }
        }
    }
    if (why) {
        orome_fail(OROME_EINVAL, "gguf_open: %s: %s", path, why);
        orome_gguf_close(gf);
        return nullptr;
    }
    infer_from_tensors(gf);
    return gf;
}

extern "C" void orome_gguf_close(OromeGGUFFile *gf)
{
    if (!gf) return;
    if (gf->map) munmap(gf->map, gf->file_size);
    if (gf->fd >= 0) close(gf->fd);
    delete gf;
}

extern "C" const OromeGGUFTensorInfo *orome_gguf_find_tensor(const OromeGGUFFile *gf, const char *name)
{
    if (!gf || !name) return nullptr;
    auto it = gf->by_name.find(name);
    return it == gf->by_name.end() ? nullptr : &gf->tensors[it->second];
}

extern "C" size_t orome_gguf_tensor_size(const OromeGGUFTensorInfo *t)
{
    if (!t) return 0;
    uint64_t n = 1;
    for (uint32_t d = 0; d < t->n_dims && d < 4; d++) n *= t->dims[d];
    BlockGeom g = geom_of(t->type);
    return (size_t)(n / g.weights) * g.bytes;
}

extern "C" const OromeGGUFMeta *orome_gguf_meta(const OromeGGUFFile *gf) { return gf ? &gf->meta : nullptr; }
extern "C" uint64_t orome_gguf_num_tensors(const OromeGGUFFile *gf) { return gf ? gf->tensors.size() : 0; }
extern "C" const OromeGGUFTensorInfo *orome_gguf_tensor(const OromeGGUFFile *gf, uint64_t i)
{
    return gf && i < gf->tensors.size() ? &gf->tensors[i] : nullptr;
}
extern "C" size_t orome_gguf_data_offset(const OromeGGUFFile *gf) { return gf ? gf->data_offset : 0; }
extern "C" size_t orome_gguf_file_size(const OromeGGUFFile *gf) { return gf ? gf->file_size : 0; }
extern "C" const void *orome_gguf_base(const OromeGGUFFile *gf) { return gf ? gf->map : nullptr; }
extern "C" const char *orome_gguf_chat_template(const OromeGGUFFile *gf)
{
    return gf && gf->has_chat_template ? gf->chat_template.c_str() : nullptr;
}

// ---- provider, expert resolver, tensor cache ---------------------------------------------------------------------

extern "C" int orome_format_provider_open_gguf(orome_cuda_ctx *ctx, OromeGGUFFile *gf, OromeFormatProvider *out)
{
    if (!ctx || !gf || !out) return orome_fail(OROME_EINVAL, "format_provider_open_gguf: NULL argument");
    void *dev = nullptr;
    int rc = orome_cuda_upload(ctx, gf->map, gf->file_size, &dev);
    if (rc != OROME_OK) return rc;
    out->gguf = gf;
    out->model_buf = dev;
    out->ctx = ctx;
    return OROME_OK;
}

extern "C" void orome_format_provider_close(OromeFormatProvider *fp)
{
    if (!fp || !fp->ctx) return;
    if (fp->model_buf) orome_cuda_free(fp->ctx, fp->model_buf);
    fp->model_buf = nullptr;
    fp->gguf = nullptr;     // the file stays the caller's to close, as in the reference (format.m:365-368)
}

extern "C" OromeExpertLayerRef orome_format_resolve_expert_layer(const OromeFormatProvider *fp, int layer, uint32_t num_experts)
{
    OromeExpertLayerRef e{};
    if (!fp || !fp->gguf || num_experts == 0) return e;
    e.buffer = fp->model_buf;
    struct { const char *what; OromeExpertProjRef *proj; } parts[3] = {
        {"ffn_gate_exps", &e.gate}, {"ffn_up_exps", &e.up}, {"ffn_down_exps", &e.down}};
    for (auto &p : parts) {
        char name[128];
        snprintf(name, sizeof name, "blk.%d.%s.weight", layer, p.what);
        const OromeGGUFTensorInfo *t = orome_gguf_find_tensor(fp->gguf, name);
        if (!t) continue;
        p.proj->offset = fp->gguf->data_offset + t->offset;
        p.proj->format = orome_format_from_ggml_type(t->type);
        p.proj->expert_stride = orome_gguf_tensor_size(t) / num_experts;
    }
    return e;
}

// Query and gate rows of a gated-attention Q tensor are stored head by head: [q rows of head 0][gate rows of head 0]
// [q rows of head 1] ...  The attention kernels want all query rows first.  Two strided device-to-device copies do
// the regrouping for any block format, because it only moves whole rows.
static int regroup_q_rows(const OromeFormatProvider *fp, const OromeGGUFTensorInfo *t, int n_heads, int hd, void **out)
{
    size_t rows = (size_t)n_heads * hd * 2;
    size_t row_bytes = orome_gguf_tensor_size(t) / rows;
    size_t part = (size_t)hd * row_bytes;                 // one head's query rows, or its gate rows
    void *dst = nullptr;
    cudaError_t e = cudaMalloc(&dst, rows * row_bytes + 256);   // same zeroed slack as orome_cuda_upload leaves
    if (e != cudaSuccess) return orome_fail(OROME_ENOMEM, "tensor cache: cudaMalloc(%zu): %s", rows * row_bytes + 256, cudaGetErrorString(e));
    const uint8_t *src = static_cast<const uint8_t *>(fp->model_buf) + fp->gguf->data_offset + t->offset;
    uint8_t *d = static_cast<uint8_t *>(dst);
    cudaError_t e1 = cudaMemset(d + rows * row_bytes, 0, 256);
    cudaError_t e2 = cudaMemcpy2D(d, part, src, 2 * part, part, (size_t)n_heads, cudaMemcpyDeviceToDevice);
    cudaError_t e3 = cudaMemcpy2D(d + (size_t)n_heads * part, part, src + part, 2 * part, part, (size_t)n_heads, cudaMemcpyDeviceToDevice);
    for (cudaError_t x : {e1, e2, e3})
        if (x != cudaSuccess) {
            cudaFree(dst);
            return orome_fail(OROME_ECUDA, "tensor cache: regrouping attn_q rows: %s", cudaGetErrorString(x));
        }
    *out = dst;
    return OROME_OK;
}

extern "C" int orome_build_tensor_cache_gguf(const OromeFormatProvider *fp, const OromeModelShape *s, uint32_t variant,
                                             OromeLayerTensorCache *layers, OromeGlobalTensorCache *globals)
{
    if (!fp || !fp->gguf || !fp->model_buf || !s || (!layers && s->num_layers > 0))
        return orome_fail(OROME_EINVAL, "build_tensor_cache_gguf: NULL argument");
    const int H = s->hidden_dim, M = s->moe_intermediate;
    if (globals) {
        globals->token_embd = ref_of(fp, variant, "token_embd.weight", (uint32_t)s->vocab_size, (uint32_t)H);
        globals->lm_head = ref_of(fp, variant, "output.weight", (uint32_t)s->vocab_size, (uint32_t)H);
        if (!globals->lm_head.buffer) globals->lm_head = globals->token_embd;     // tied embeddings
    }
    for (int i = 0; i < s->num_layers; i++) {
        OromeLayerTensorCache &c = layers[i];
        memset(&c, 0, sizeof c);
        if (s->ffn_is_moe) {
            const int S = s->shared_intermediate > 0 ? s->shared_intermediate : M;
            c.routing_gate = layer_ref(fp, variant, i, "ffn_gate_inp", s->num_experts, H);
            c.shared_gate = layer_ref(fp, variant, i, "ffn_gate_shexp", S, H);
            c.shared_up = layer_ref(fp, variant, i, "ffn_up_shexp", S, H);
            c.shared_down = layer_ref(fp, variant, i, "ffn_down_shexp", H, S);
            c.shared_expert_gate = layer_ref(fp, variant, i, "ffn_gate_inp_shexp", 1, H);
        } else {
            c.dense_gate = layer_ref(fp, variant, i, "ffn_gate", M, H);
            c.dense_up = layer_ref(fp, variant, i, "ffn_up", M, H);
            c.dense_down = layer_ref(fp, variant, i, "ffn_down", H, M);
        }
        if (s->layer_is_linear && s->layer_is_linear[i]) {
            const int total_value = s->linear_num_v_heads * s->linear_value_dim;
            c.lin_qkv = layer_ref(fp, variant, i, "attn_qkv", s->linear_conv_dim, H);
            c.lin_z = layer_ref(fp, variant, i, "attn_gate", total_value, H);
            c.lin_a = layer_ref(fp, variant, i, "ssm_alpha", s->linear_num_v_heads, H);
            c.lin_b = layer_ref(fp, variant, i, "ssm_beta", s->linear_num_v_heads, H);
            c.lin_o = layer_ref(fp, variant, i, "ssm_out", H, total_value);
            continue;
        }
        const int n_heads = s->num_attn_heads, hd = s->head_dim, kv_rows = s->num_kv_heads * hd;
        char name[128];
        snprintf(name, sizeof name, "blk.%d.attn_q.weight", i);
        const OromeGGUFTensorInfo *q = orome_gguf_find_tensor(fp->gguf, name);
        const int q_rows = (q && q->n_dims >= 2) ? (int)q->dims[1] : n_heads * hd;
        c.full_q = ref_of(fp, variant, name, (uint32_t)q_rows, (uint32_t)H);
        if (q && q->n_dims >= 2 && n_heads > 0 && hd > 0 && q_rows == 2 * n_heads * hd) {
            int rc = regroup_q_rows(fp, q, n_heads, hd, &c.owned_q);
            if (rc != OROME_OK) {
                orome_free_tensor_cache(fp, layers, i);
                return rc;
            }
            c.full_q.buffer = c.owned_q;
            c.full_q.offset = 0;
        }
        c.full_k = layer_ref(fp, variant, i, "attn_k", kv_rows, H);
        c.full_v = layer_ref(fp, variant, i, "attn_v", kv_rows, H);
        c.full_o = layer_ref(fp, variant, i, "attn_output", H, n_heads * hd);
    }
    return OROME_OK;
}

extern "C" void orome_free_tensor_cache(const OromeFormatProvider *fp, OromeLayerTensorCache *layers, int num_layers)
{
    if (!fp || !layers) return;
    for (int i = 0; i < num_layers; i++)
        if (layers[i].owned_q) {
            cudaFree(layers[i].owned_q);
            layers[i].owned_q = nullptr;
            layers[i].full_q = OromeTensorRef{};
        }
}
