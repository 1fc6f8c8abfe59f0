/*
 * orome_gguf.h -- the on-disk format the quantized matvec path consumes, and the step from a
 * GGUF file to the TensorRef / ExpertLayerRef handles of orome_cuda.h.
 *
 * Host-side counterpart of Orome's GGUF reader (inference/src/gguf.m:273-550, types at
 * inference/include/orome.h:405-444) and of the GGUF half of its format layer
 * (inference/src/format.m:343-363 provider, 374-409 expert resolver, 416-590 tensor cache).
 * Paths in the comments are relative to the Orome source tree.
 *
 * What differs from the reference, and why: the reference wraps the mmap'd file as one no-copy
 * GPU buffer (unified memory); a B200 needs the bytes in HBM, so opening a provider uploads the
 * file image once (orome_cuda_upload).  Offsets stay file-relative, so a TensorRef is still
 * {model buffer, data_offset + tensor offset} exactly as format.m:422 builds it.
 */
#ifndef OROME_GGUF_H
#define OROME_GGUF_H

#include "orome_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* GGUFTensorInfo, orome.h:405-411. */
typedef struct {
    char    *name;
    uint32_t n_dims;
    uint64_t dims[4];
    uint32_t type;          /* ggml type id */
    uint64_t offset;        /* relative to the start of the data section */
} OromeGGUFTensorInfo;

/* The model description gguf_open extracts from the metadata (the scalar fields of GGUFFile,
 * orome.h:413-437), with the same inference rules: keys are read under "<architecture>."
 * ("llama." until general.architecture has been seen), the FFN kind follows the tensor names
 * (ffn_*_exps => MoE, .ffn_gate/.ffn_up/.ffn_down => dense, else by expert_count), vocab_size
 * and the FFN width are inferred from tensor shapes when the metadata has none
 * (gguf.m:455-518). */
typedef struct {
    char     arch[32];
    int      ffn_is_moe;
    int      num_layers, hidden_dim, num_experts, num_experts_per_tok;
    int      num_attn_heads, num_kv_heads, moe_intermediate;
    int      context_length, attn_key_length, attn_value_length, rope_dimension_count;
    int      ssm_conv_kernel, ssm_state_size, ssm_group_count, ssm_time_step_rank, ssm_inner_size;
    int      full_attention_interval;
    int      eos_token_id, padding_token_id;      /* -1 when absent */
    int      vocab_size;
    float    rope_theta, rms_norm_eps;
    uint32_t alignment;                           /* general.alignment, default 32 (gguf.m:323) */
    uint32_t version;
} OromeGGUFMeta;

typedef struct OromeGGUFFile OromeGGUFFile;

/* gguf_open / gguf_close (gguf.m:273-529): mmap the file, parse header, metadata and tensor
 * directory.  NULL on a missing file, bad magic, a version other than 2 or 3, or a directory
 * that runs past the end of the file; orome_cuda_last_error() has the reason. */
OromeGGUFFile *orome_gguf_open(const char *path);
void           orome_gguf_close(OromeGGUFFile *gf);

/* gguf_find_tensor (gguf.m:531-535): by exact name, NULL when absent. */
const OromeGGUFTensorInfo *orome_gguf_find_tensor(const OromeGGUFFile *gf, const char *name);
/* gguf_tensor_size (gguf.m:540-550): elements / block size * bytes per block; 0 for NULL. */
size_t orome_gguf_tensor_size(const OromeGGUFTensorInfo *ti);

const OromeGGUFMeta       *orome_gguf_meta(const OromeGGUFFile *gf);
uint64_t                   orome_gguf_num_tensors(const OromeGGUFFile *gf);
const OromeGGUFTensorInfo *orome_gguf_tensor(const OromeGGUFFile *gf, uint64_t index);
size_t                     orome_gguf_data_offset(const OromeGGUFFile *gf);   /* absolute offset of the data section */
size_t                     orome_gguf_file_size(const OromeGGUFFile *gf);
const void                *orome_gguf_base(const OromeGGUFFile *gf);          /* the mapped file */
/* tokenizer.chat_template, or NULL */
const char                *orome_gguf_chat_template(const OromeGGUFFile *gf);

/* FormatProvider (orome.h:262-265) + format_provider_open_gguf / _close (format.m:343-368): the
 * model's bytes as one device buffer.  Opening copies the whole file image to HBM. */
typedef struct {
    OromeGGUFFile  *gguf;
    void           *model_buf;      /* device copy of the file image */
    orome_cuda_ctx *ctx;
} OromeFormatProvider;

int  orome_format_provider_open_gguf(orome_cuda_ctx *ctx, OromeGGUFFile *gf, OromeFormatProvider *out);
void orome_format_provider_close(OromeFormatProvider *fp);

/* format_resolve_expert_layer (format.m:374-409): blk.<layer>.ffn_{gate,up,down}_exps.weight as
 * {offset, bytes / num_experts, format}; a projection whose tensor is absent stays zeroed. */
OromeExpertLayerRef orome_format_resolve_expert_layer(const OromeFormatProvider *fp, int layer_idx, uint32_t num_experts);

/* The shapes the cache builder needs from ModelConfig (orome.h:49-105). */
typedef struct {
    int num_layers, hidden_dim, moe_intermediate, shared_intermediate, num_experts, vocab_size;
    int ffn_is_moe;
    int num_attn_heads, num_kv_heads, head_dim;
    int linear_conv_dim, linear_num_v_heads, linear_value_dim;
    const uint8_t *layer_is_linear;      /* [num_layers]: 1 = linear-attention layer, 0 = full attention; NULL = all full */
} OromeModelShape;

/* The weight tensors of LayerTensorCache / GlobalTensorCache (orome.h:269-306) that are matvec
 * operands.  Norm weights and the recurrent-state tensors are not part of this path. */
typedef struct {
    OromeTensorRef routing_gate, shared_gate, shared_up, shared_down, shared_expert_gate;
    OromeTensorRef dense_gate, dense_up, dense_down;
    OromeTensorRef lin_qkv, lin_z, lin_a, lin_b, lin_o;
    OromeTensorRef full_q, full_k, full_v, full_o;
    void *owned_q;       /* device copy of a de-interleaved Q tensor (freed by orome_free_tensor_cache), else NULL */
} OromeLayerTensorCache;

typedef struct {
    OromeTensorRef token_embd, lm_head;
} OromeGlobalTensorCache;

/* build_tensor_cache_gguf (format.m:458-590).  Every reference is {model buffer, data_offset +
 * tensor offset, format from the ggml type (format.m:326-337), shape from `shape`}; a tensor the
 * file does not have gives a zeroed (absent) reference; output.weight falls back to
 * token_embd.weight (tied embeddings, format.m:482-485).  A full-attention Q tensor with
 * 2 * heads * head_dim rows stores query and gate rows interleaved per head; its rows are
 * regrouped at load time into all query rows followed by all gate rows (format.m:546-574) in a
 * device buffer of its own.  `layers` must hold shape->num_layers entries; `globals` may be NULL.
 * variant: the kernel family stored into every reference (OromeKernelVariant). */
int  orome_build_tensor_cache_gguf(const OromeFormatProvider *fp, const OromeModelShape *shape, uint32_t variant,
                                   OromeLayerTensorCache *layers, OromeGlobalTensorCache *globals);
void orome_free_tensor_cache(const OromeFormatProvider *fp, OromeLayerTensorCache *layers, int num_layers);

#ifdef __cplusplus
}
#endif
#endif /* OROME_GGUF_H */
