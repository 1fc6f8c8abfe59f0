/*
 * orome_cuda.h -- C ABI of the B200 (sm_100a) implementation of Orome's
 * quantized dequant-matvec path.
 *
 * The library replaces, for an NVIDIA B200, the part of Orome's "format" layer
 * through which the engine issues every weight-bound product of a decode step:
 * the GGUF block-quantized matvec (Q8_0 / Q4_K / Q5_K / Q6_K), the fused
 * gate/up + SwiGLU forms, the batched (prefill) form and the MoE top-k expert
 * gather-matvec.  Each declaration cites the reference interface it replaces
 * (paths are relative to the Orome source tree).
 *
 * Conventions
 *   - Plain C types only: pointers, sizes, enums.  `stream` arguments are a
 *     cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Every compute entry point only ENQUEUES work on the given stream and never
 *     synchronises, like the reference's encoder-style dispatch
 *     (format.m:240-303 returns after dispatchThreadgroups).  Ordering between
 *     dependent calls is stream order; that replaces the reference's explicit
 *     memoryBarrierWithScope calls (engine.m:564, 594, 624, ...).
 *   - Return value: 0 on success, a negative errno-style code on a rejected
 *     call (OROME_EINVAL, OROME_ENOTSUP, OROME_ECUDA ...), and
 *     orome_cuda_last_error() gives the message.  The reference returns void and
 *     prints to stderr (format.m:260-264); a NULL weight buffer is a silent
 *     no-op returning 0, which keeps the reference's optional-tensor convention
 *     (format.m:247-250).
 *   - A context is not thread-safe (neither is the reference's MetalCtx).
 *   - All device pointers must belong to the context's device.  Weight tensors
 *     must start on a 16-byte boundary (GGUF aligns tensor data to 32 bytes,
 *     gguf.m:323) and activations / outputs on a 16-byte boundary.
 */
#ifndef OROME_CUDA_H
#define OROME_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define OROME_OK        0
#define OROME_EINVAL   (-22)   /* bad dimensions, NULL where not allowed, misaligned pointer */
#define OROME_ENOTSUP  (-95)   /* format / variant combination without a kernel               */
#define OROME_ENOMEM   (-12)   /* device allocation failed                                   */
#define OROME_ECUDA    (-5)    /* a CUDA runtime call failed (message has the CUDA error)     */
#define OROME_ETIMEOUT (-110)  /* a bounded device-side wait gave up (see orome_cuda_status)   */

/* ---- types mirrored from inference/include/orome.h ---------------------- */

/* QuantFormat, orome.h:227-235 -- same enumerators in the same order. */
typedef enum {
    OROME_QFMT_GGUF_Q4_K = 0,   /* 256 weights in a 144-byte superblock */
    OROME_QFMT_GGUF_Q5_K = 1,   /* 256 weights in a 176-byte superblock */
    OROME_QFMT_GGUF_Q6_K = 2,   /* 256 weights in a 210-byte superblock */
    OROME_QFMT_GGUF_Q8_0 = 3,   /* 32 int8 weights + fp16 scale, 34 bytes */
    OROME_QFMT_F16       = 4,
    OROME_QFMT_BF16      = 5,
    OROME_QFMT_F32       = 6
} OromeQuantFormat;

/* Kernel family, the role `pipeline` plays in the reference's TensorRef.
 * DEFAULT reads the six-bit K-quant scales the way the reference's CPU decode
 * and default kernels do (format.m:41-64, shaders.metal:1413-1436).  LLAMA reads
 * them the way the reference's `_llama` kernels do (shaders.metal:1575-1578,
 * 2053-2056), which is what engine_qwen35_hybrid.m:86-148 selects for the 27B
 * model.  The two differ on sub-blocks 4..7; all other arithmetic is shared. */
typedef enum {
    OROME_VARIANT_DEFAULT = 0,
    OROME_VARIANT_LLAMA   = 1
} OromeKernelVariant;

/* TensorRef, orome.h:239-246.  `buffer` is a device pointer instead of an
 * id<MTLBuffer>; `variant` stands where the reference keeps the pipeline. */
typedef struct {
    void            *buffer;     /* device allocation holding the tensor (NULL = absent tensor) */
    size_t           offset;     /* byte offset of the tensor inside `buffer`                   */
    uint32_t         variant;    /* OromeKernelVariant                                          */
    OromeQuantFormat format;
    uint32_t         out_dim;    /* rows                                                        */
    uint32_t         in_dim;     /* columns (weights per row)                                   */
} OromeTensorRef;

/* ExpertProjRef / ExpertLayerRef, orome.h:249-259: expert e of a projection
 * starts at buffer + offset + e * expert_stride (format.m:381-406). */
typedef struct {
    size_t           offset;
    size_t           expert_stride;
    OromeQuantFormat format;
} OromeExpertProjRef;

typedef struct {
    void              *buffer;
    OromeExpertProjRef gate, up, down;
} OromeExpertLayerRef;

typedef struct orome_cuda_ctx orome_cuda_ctx;

/* ---- context, memory, errors ------------------------------------------- */

/* Replaces metal_setup / metal_free (orome.h:219-221, metal.m:41) for this path:
 * binds a CUDA device, allocates the context's status word.  No scratch is sized
 * from a model config; the path's kernels need none beyond their outputs. */
int  orome_cuda_ctx_create(int device, orome_cuda_ctx **out);
void orome_cuda_ctx_destroy(orome_cuda_ctx *ctx);

/* Message of the last failed call on this thread ("" if none). */
const char *orome_cuda_last_error(void);

/* Device-side status word: 0, or the code left by a kernel whose bounded wait ran out
 * (1, 2: a stage of its own copy pipeline; 3: an input element that a peer GPU or an
 * earlier product of a chain should have written; 4: the tensor-core form's pipeline).
 * Synchronises the context's device, returns OROME_ETIMEOUT when the word is set and then
 * clears it, so the condition is reported once.  While the word is set, chain launches and
 * gather waits do not wait at all (their results are void until the word is cleared). */
int  orome_cuda_status(orome_cuda_ctx *ctx, int *status_out);

/* Replaces format_provider_open_gguf (format.m:343-363).  The reference wraps
 * the mmap'd file as one no-copy buffer (unified memory); a discrete GPU needs
 * the bytes in HBM, so this copies `bytes` bytes to a new 256-byte aligned
 * device allocation.  Offsets relative to `host` stay valid relative to
 * `*dev_base`, so TensorRef.offset = data_offset + tensor offset is unchanged
 * (format.m:422). */
int  orome_cuda_upload(orome_cuda_ctx *ctx, const void *host, size_t bytes, void **dev_base);
int  orome_cuda_free(orome_cuda_ctx *ctx, void *dev_base);

/* Copy `bytes` bytes of device memory to the host after everything queued on the device has finished.  The
 * reference reads results straight out of its shared (unified-memory) buffers, e.g. the arg-max token at
 * engine.m:1057; on a discrete GPU that read is this call. */
int  orome_cuda_download(orome_cuda_ctx *ctx, const void *dev, void *host, size_t bytes);

/* ---- format helpers ------------------------------------------------------ */

/* format_from_ggml_type, format.m:326-337 (unknown ids map to Q4_K, line 335). */
OromeQuantFormat orome_format_from_ggml_type(uint32_t ggml_type);

/* Bytes of one row; 0 if in_dim is not a whole number of blocks
 * (row strides of format.m:198, 203, 208, 213). */
size_t orome_format_row_bytes(OromeQuantFormat format, uint32_t in_dim);

/* ---- the hot path -------------------------------------------------------- */

/* format_dispatch_matvec, format.m:240-303 / orome.h:319-322.
 * y[out_dim] = W[out_dim][in_dim] . x[in_dim], x and y fp32.  in_buf/in_off and
 * out_buf/out_off are a device buffer and a byte offset, exactly the reference's
 * (buffer, offset) pairs. */
int  orome_format_dispatch_matvec(orome_cuda_ctx *ctx, const OromeTensorRef *ref,
                                  const void *in_buf, size_t in_off,
                                  void *out_buf, size_t out_off, void *stream);

/* Batched form of the same product: y[b][r] = sum_c W[r][c] x[b][c] for
 * b < batch, x row stride ldx, y row stride ldy (in floats).  batch == 1 is the
 * decode matvec; larger batches are the prefill form, which the reference runs
 * as one matvec per token (main.m:745-747).  Batches of OROME_OPT_TC_MIN_BATCH (default 4)
 * and more on Q8_0 / Q4_K / Q5_K / Q6_K tensors whose in_dim is a multiple of 256 run on the tensor
 * cores (tcgen05) with weights and x rounded to fp16 and fp32 accumulation: rel-L2 <= 5e-4
 * against an exact evaluation, the class of rounding the reference's own kernels apply to x
 * (shaders.metal:1470).  The first such call allocates scratch inside the context: make it
 * before any stream capture.  Smaller batches keep fp32 activations (rel-L2 <= 1e-4): one decode
 * launch per vector, or, on Q4_K / Q5_K, one per pair of vectors (the weights are read once per pair).
 * Range of the fp16 operands: a weight is formed as (q - bias) * half(d * sc) + half(-dmin * mn),
 * so |d * sc| and |dmin * mn| (Q8_0: |d|; Q6_K: |d * sc| only) must stay below 65504 and lose precision below 6e-5;
 * GGUF scales of real models are orders of magnitude inside that range, and x is expected within
 * the fp16 range as in the reference (shaders.metal:1470).  Tensors outside it: set
 * OROME_OPT_TC_MIN_BATCH above the batch and use the fp32-activation kernels.
 * With a multi-GPU gather request armed (orome_cuda_gather_next) the batch-1 quantized form and
 * this tensor-core form (4 <= batch <= 64, one launch) are available: Y goes to every rank's
 * arena from the kernel that writes it, a gathered X is read from its slots.  Any other call
 * drops the request and returns OROME_ENOTSUP. */
int  orome_cuda_matvec(orome_cuda_ctx *ctx, const OromeTensorRef *ref,
                       const float *x_dev, float *y_dev, int batch, int ldx, int ldy, void *stream);

/* Several tensors that share one input vector in a single launch (the
 * reference encodes q/k/v projections back to back with no barrier between
 * them, engine.m:554-563, 777-784, so they run concurrently).  y_dev[i] receives
 * refs[i].out_dim floats.  All refs must share format, variant and in_dim. */
int  orome_cuda_matvec_group(orome_cuda_ctx *ctx, const OromeTensorRef *refs, int n_refs,
                             const float *x_dev, float *const *y_dev, void *stream);

/* Fused gate/up + SwiGLU: out[b][r] = silu(Wg x_b)[r] * (Wu x_b)[r], silu(g) = g / (1 + exp(-g)).
 * Replaces shared_gate_up_swiglu_q4k / _q8_0 and fused_gate_up_swiglu_q4k_llama
 * (shaders.metal:2316-2445, 2451-2584) as dispatched by encode_dense_ffn
 * (engine.m:342-392).  gate and up must have identical shape and format.
 * batch > 1 is two batched products (orome_cuda_matvec: its dispatch, scratch and precision class;
 * from OROME_OPT_TC_MIN_BATCH vectors on that is the fp16 tensor-core form) and an elementwise pass,
 * the reference's unfused branch (engine.m:388-404). */
int  orome_cuda_gate_up_swiglu(orome_cuda_ctx *ctx, const OromeTensorRef *gate, const OromeTensorRef *up,
                               const float *x_dev, float *out_dev, int batch, int ldx, int ldo, void *stream);

/* Device counterpart of format_decode_row_f32 (format.m:176-218, orome.h:325):
 * decodes rows [row0, row0 + nrows) to out_dev[nrows][in_dim], bit-identical to
 * the reference's CPU decode (also the embedding lookup of engine.m:122-141). */
int  orome_cuda_dequant_rows(orome_cuda_ctx *ctx, const OromeTensorRef *ref,
                             uint32_t row0, uint32_t nrows, float *out_dev, void *stream);

/* argmax_kernel (shaders.metal:1249-1305) as dispatched after the lm_head (engine.m:1036-1046):
 * *result_dev = index of the largest of `count` floats, so that a token costs the host a 4-byte
 * read (engine.m:1057) instead of the logits.  Equal values resolve exactly as the reference's kernel resolves them
 * (its 1024 threads stride over the vector, then two shuffle-down trees pick among threads; the
 * smallest index wins only among elements of the same thread); NaN and -inf never win; no
 * candidate gives index 0.
 * While a chain is being recorded, the call must name the whole output of the product
 * recorded last: the reduction then runs inside that product's epilogue (single GPU). */
int  orome_cuda_argmax(orome_cuda_ctx *ctx, const float *data_dev, uint32_t count, uint32_t *result_dev, void *stream);

/* MoE routing: logits = Wr x per token (matvec_f32 / matvec_f32_pair,
 * shaders.metal:1342-1392, engine.m:656-684) followed by softmax_topk_route
 * (shaders.metal:1141-1234): K rounds of arg-max, ties to the lowest index,
 * softmax over the selected logits only, K capped at 8, n_experts <= 256.
 * idx_dev[t][8] and w_dev[t][8] (slots >= K zero-filled) per token t.
 * `router` must be an F32 tensor [n_experts][hidden]. */
int  orome_cuda_moe_route(orome_cuda_ctx *ctx, const OromeTensorRef *router,
                          const float *x_dev, int n_tokens, int ldx, uint32_t K,
                          uint32_t *idx_dev, float *w_dev, float *logits_dev /* optional [t][n_experts] */,
                          void *stream);

/* The same routing with the shared-expert gate computed in the router launch: matvec_f32_pair
 * (shaders.metal:1368-1392) as dispatched at engine.m:656-679 puts the logit of the [1][hidden]
 * fp32 gate tensor after the router logits, and softmax_topk_route copies it to out_params[8]
 * (shaders.metal:1232) for the combine kernel.  idx_dev / w_dev as above; shared_logit_dev[t]
 * receives that raw logit (the reference keeps it in slot 8 of the same 9-float params buffer;
 * here it is its own array so that the [t][8] weight layout of the expert kernels is
 * unchanged).  shared_gate may be an absent tensor (buffer NULL): the logit is then 0.
 * logits_dev (optional) must hold n_experts + 1 floats per token. */
int  orome_cuda_moe_route_pair(orome_cuda_ctx *ctx, const OromeTensorRef *router, const OromeTensorRef *shared_gate,
                               const float *x_dev, int n_tokens, int ldx, uint32_t K,
                               uint32_t *idx_dev, float *w_dev, float *shared_logit_dev,
                               float *logits_dev /* optional [t][n_experts + 1] */, void *stream);

/* Routing for callers that must not allocate.  No counterpart in the reference (its
 * Metal context sizes every scratch buffer once, at start-up, metal.m:155-251).
 *
 * Same result as orome_cuda_moe_route called without a logits buffer, but the router
 * logits go to a fixed array that is part of the library image (device memory of
 * OROME_ROUTE_STATIC_MAX_LOGITS floats, 64 KiB, held by every GPU that loads the library
 * until the process exits) instead of context scratch obtained with cudaMalloc.  It is
 * meant for the per-token loop of an engine that, like the reference, reserves all device
 * memory up front and then forbids allocation - cudaMalloc synchronises the whole device
 * and can fail once the model has filled HBM - and for hosts whose device memory belongs
 * entirely to another allocator.  The call itself performs no cudaMalloc / cudaFree and
 * calls no allocating library routine.
 *
 *   - n_tokens * n_experts must not exceed OROME_ROUTE_STATIC_MAX_LOGITS, else OROME_EINVAL.
 *   - The first call on a device looks up the array's device address (once per device,
 *     with that device current); make that first call before any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's logits.
 *     Nothing in it has to start at zero (every entry that is read is written first by the
 *     same call), but two calls whose kernels overlap on the GPU - different streams, or
 *     different contexts on the same device - race on it: keep them in one stream. */
#define OROME_ROUTE_STATIC_MAX_LOGITS (64 * 256)
int  orome_cuda_moe_route_static(orome_cuda_ctx *ctx, const OromeTensorRef *router,
                                 const float *x_dev, int n_tokens, int ldx, uint32_t K,
                                 uint32_t *idx_dev, float *w_dev, void *stream);

/* Routed-expert FFN with the weighted combine, replacing
 * batch_expert_gate_up_swiglu_q4k_dyn, batch_expert_down_q4k_dyn / _q5k_dyn and
 * the expert term of moe_combine_copy_sq (shaders.metal:2232-2310, 2590-2760,
 * 1049-1055) as sequenced by encode_experts_gguf (engine.m:158-340):
 *   out[t][h] = sum_{k<K} w[t][k] * ( Wd[e] ( silu(Wg[e] x_t) * (Wu[e] x_t) ) )[h],  e = idx[t][k].
 * idx/w use the [t][8] layout written by orome_cuda_moe_route.  act_dev is
 * caller-provided scratch of n_tokens * K * inter floats (the reference's
 * buf_batch_expert_act, orome.h:189).  The shared-expert term and the residual
 * add of the reference's combine kernel are outside this entry point. */
int  orome_cuda_moe_ffn(orome_cuda_ctx *ctx, const OromeExpertLayerRef *layer, uint32_t variant,
                        const float *x_dev, int n_tokens, int ldx,
                        const uint32_t *idx_dev, const float *w_dev, uint32_t K,
                        uint32_t hidden, uint32_t inter, float *act_dev, float *out_dev, int ldo,
                        void *stream);

/* The whole MoE block of encode_experts_gguf (engine.m:158-340) after routing:
 *   out[t] = h_mid[t] + sum_k w[t][k] FFN_{e_k}(x_t) + sigmoid(shared_logit[t]) * SharedFFN(x_t)
 * i.e. the routed experts (as orome_cuda_moe_ffn), the shared expert (fused gate/up + SwiGLU,
 * engine.m:263-275; its down projection, engine.m:314-316) and the value the combine kernels write
 * to hidden_out (moe_combine_copy_sq / _k8, shaders.metal:1049-1059, 1100-1120; sigmoid written as
 * 1 / (1 + exp(-p)) like there).  The residual copy and the sum of squares those kernels also
 * produce belong to the normalisation that follows and are not part of this path.
 * The three shared-expert tensors may be absent (NULL pointers or NULL buffers): no shared term.
 * h_mid_dev may be NULL (no residual input).  scratch_dev: caller-provided,
 * orome_cuda_moe_block_scratch_floats(...) floats, 16-byte aligned. */
int  orome_cuda_moe_block(orome_cuda_ctx *ctx, const OromeExpertLayerRef *layer, uint32_t variant,
                          const OromeTensorRef *shared_gate_proj, const OromeTensorRef *shared_up_proj,
                          const OromeTensorRef *shared_down_proj, const float *x_dev, int n_tokens, int ldx,
                          const uint32_t *idx_dev, const float *w_dev, const float *shared_logit_dev,
                          uint32_t K, uint32_t hidden, uint32_t inter, const float *h_mid_dev, int ld_mid,
                          float *scratch_dev, float *out_dev, int ldo, void *stream);
size_t orome_cuda_moe_block_scratch_floats(int n_tokens, uint32_t K, uint32_t hidden, uint32_t inter, uint32_t shared_inter);

/* Expert-parallel share of the same operation -- no counterpart in the reference (one GPU).  This GPU holds the
 * experts [first_expert, first_expert + n_local) of the layer, packed from index 0 in layer_local; the call adds
 * up only those of each token's K selected experts that live here (out = 0 where none does), so the layer's
 * output is the SUM of the ranks' outputs (one all-reduce of n_tokens x hidden floats, done by the caller).
 * The activations x and the routing result are replicated on every rank, as they are after a row-split product,
 * so no token dispatch is needed.  idx_local_dev: scratch of n_tokens * 8 indices.  A selected expert that lives
 * elsewhere costs this GPU no weight traffic. */
int  orome_cuda_moe_ffn_shard(orome_cuda_ctx *ctx, const OromeExpertLayerRef *layer_local, uint32_t variant,
                              const float *x_dev, int n_tokens, int ldx, const uint32_t *idx_dev, const float *w_dev,
                              uint32_t K, uint32_t hidden, uint32_t inter, uint32_t first_expert, uint32_t n_local,
                              uint32_t *idx_local_dev, float *act_dev, float *out_dev, int ldo, void *stream);

/* Optional hint: the tensor the NEXT matvec / group / gate-up call on this context will read.
 * The launch issued in between pulls the first bytes of that tensor into L2 once its own rows
 * are requested, so HBM keeps streaming across the launch boundary (a decode step is a fixed
 * sequence of products, engine.m:481-1046, so the caller always knows the next tensor).  The hint
 * is consumed by the next launch and then cleared; passing NULL clears it.  Purely a
 * performance hint: results do not depend on it. */
int  orome_cuda_hint_next(orome_cuda_ctx *ctx, const OromeTensorRef *next);

/* ---- the steps either side of a product, fused into it ---------------------------------
 *
 * The reference runs three small kernels between the attention output projection and the FFN
 * products (engine.m:625-653): residual_add_sum_sq (shaders.metal:86-124: out = clamp(a + b,
 * +-65504) and one partial sum of out^2 per threadgroup), then rms_norm_apply_partial
 * (shaders.metal:126-149: x * rsqrt(sum(parts) / dim + eps) * bf16 weight).  Here the first is
 * the epilogue of the product that makes b, the second the prologue of every product that reads
 * the normalised vector, so neither the un-normalised nor the normalised intermediate costs a
 * launch of its own:
 *
 *   orome_cuda_fuse_next(ctx, NULL, &epi);  orome_cuda_matvec(ctx, &o_proj, attn, hidden, ...);
 *       hidden[r] = clamp(epi.residual[r] + (W attn)[r]);  epi.sum_sq_parts = partial sums of hidden^2
 *   orome_cuda_fuse_next(ctx, &pro, NULL);  orome_cuda_gate_up_swiglu(ctx, &gate, &up, hidden, act, ...);
 *       the product reads hidden[c] * rsqrt(sum(pro.sum_sq_parts) / in_dim + pro.eps) * bf16(pro.weight_bf16[c])
 *
 * A request applies to the NEXT batch-1 launch of orome_cuda_matvec / orome_format_dispatch_matvec /
 * orome_cuda_matvec_group (prologue; epilogue for a single tensor only) or orome_cuda_gate_up_swiglu
 * (prologue only) and is consumed by it.  A call that cannot honour it (batch > 1, F16/BF16/F32 tensors,
 * shapes outside the decode kernels, a chain recording, a multi-GPU gather request on the same launch)
 * drops it and returns OROME_ENOTSUP.  residual may equal the product's y (in-place add, as the
 * reference does with buf_moe_hidden, engine.m:629).  A partials array holds OROME_SUM_SQ_PARTS floats
 * of device memory; the epilogue writes all of them (one per CTA, zeros behind), the prologue adds all
 * of them up, so the array needs no clearing and the two sides need not agree on a grid size. */
#define OROME_SUM_SQ_PARTS 512
typedef struct {
    const void  *weight_bf16;    /* [in_dim] bf16 norm weights, 8-byte aligned (the BF16 copies format.m:437-452 makes of F32 norm tensors) */
    const float *sum_sq_parts;   /* [OROME_SUM_SQ_PARTS], written by an epilogue (or by the caller: total in [0], zeros behind) */
    float        eps;
} OromeNormPrologue;
typedef struct {
    const float *residual;       /* [out_dim] */
    float       *sum_sq_parts;   /* [OROME_SUM_SQ_PARTS] */
} OromeResidualEpilogue;
int  orome_cuda_fuse_next(orome_cuda_ctx *ctx, const OromeNormPrologue *prologue, const OromeResidualEpilogue *epilogue);

/* ---- one token step as ONE launch ---------------------------------------------------------
 *
 * The reference encodes every product of a token into one command buffer and commits it once
 * (engine.m:453-454 open the buffer and its encoder, format_dispatch_matvec and the fused
 * gate/up dispatch only encode, engine.m:1048-1050 commit and wait).  The same shape here:
 * between orome_cuda_chain_begin and orome_cuda_chain_end, orome_format_dispatch_matvec,
 * orome_cuda_matvec (batch 1), orome_cuda_matvec_group, orome_cuda_gate_up_swiglu,
 * orome_cuda_argmax and orome_cuda_gather_wait RECORD their operation instead of launching it;
 * orome_cuda_chain_launch then runs the recorded sequence as a single resident kernel (one CTA
 * per SM) in which the weights of the next product stream into shared memory while the current
 * one is still being consumed.  A chain is reusable: pointers and shapes are fixed at record
 * time, the vectors' contents are read at launch time.
 *
 * Ordering.  A product whose input vector is (inside) the output of an earlier recorded product
 * waits for it element by element; inputs that no recorded product writes are read as they are
 * at launch.  A product may overwrite a vector an earlier product reads or writes only if a
 * chain of such data dependencies orders the two (true for a decode step, where each product
 * consumes its predecessor's output); otherwise chain_end returns OROME_ENOTSUP.  Outputs are
 * complete for other readers when the launch has completed in stream order.
 *
 * Quantized tensors only (Q8_0 with in_dim a multiple of 64; Q4_K / Q5_K / Q6_K with in_dim a
 * multiple of 256), batch 1, at most 4 tensors per grouped product.  chain_end allocates (device
 * table, {value, tag} slots of every output); chain_launch allocates nothing.  All CTAs of the
 * launch must be resident at once, so it is issued as a cooperative launch: it fails with
 * OROME_ECUDA rather than hang when the device cannot hold one CTA per SM.
 *
 * Several GPUs (after orome_cuda_gather_setup): products whose outputs lie in the gather arena
 * publish them to every peer from their epilogue, exactly like an armed single launch; a
 * product that reads such a vector polls the peers' elements too.  Every rank records the same
 * sequence and launches it the same number of times; gather_next is not needed inside a
 * recording.  orome_cuda_gather_wait inside a recording copies a gathered vector to its plain
 * place as part of the chain.  The chains of one context share a tag counter: launch them one at a
 * time (stream order on one stream is enough). */
typedef struct orome_cuda_chain orome_cuda_chain;
int  orome_cuda_chain_begin(orome_cuda_ctx *ctx);
int  orome_cuda_chain_end(orome_cuda_ctx *ctx, orome_cuda_chain **out);     /* always closes the recording */
int  orome_cuda_chain_launch(orome_cuda_ctx *ctx, orome_cuda_chain *chain, void *stream);
void orome_cuda_chain_destroy(orome_cuda_ctx *ctx, orome_cuda_chain *chain);
/* What was recorded: products, packed weight bytes they read, ring stages and bytes per stage. */
int  orome_cuda_chain_info(orome_cuda_chain *chain, int *n_products, uint64_t *weight_bytes, int *stages, int *stage_bytes);

/* ---- multi-GPU: row-split products, output vector completed on every GPU ---------------
 *
 * No counterpart in the reference (single GPU, unified memory).  Output rows of a matvec are
 * independent, so rank r of `world` GPUs in one box keeps a slice of the rows of every tensor
 * and the full y must reach every GPU before the next product.  Instead of a collective after
 * the kernel, the kernel that produces a slice stores every value, together with a generation
 * tag in the same 8-byte store, into the same slot of its own and of each peer's "gather
 * arena" over NVLink (plain peer stores).  The launch that consumes the vector reads x from
 * those slots and polls each element until it carries the generation expected (bounded: after
 * about a second it records status 3, see orome_cuda_status, and carries on).  No fence, no
 * separate flag, no collective call.
 *
 * Set-up: every process allocates an arena of orome_cuda_gather_arena_bytes(data_bytes, n_flags)
 * bytes with orome_cuda_peer_alloc, exchanges the 64-byte handles by any host channel, opens the
 * others with orome_cuda_peer_open and passes all `world` pointers (its own included, at index
 * rank) to orome_cuda_gather_setup.  The first data_bytes of the arena hold the gathered vectors
 * as plain floats (the caller places them), the rest their slots.  n_flags (<= 64) is the number
 * of vectors in flight the caller tells apart ("flags"; each has a generation counter).
 * Before a matvec / group / gate-up launch, orome_cuda_gather_next(ctx, wait_flag, publish_flag)
 * says that the launch's x is the gathered vector published under wait_flag (-1: x is a plain
 * vector) and that its y rows are to be published under publish_flag (-1: y stays local); it
 * applies to the next launch only.  A waiting launch must take x from the local arena, a
 * publishing launch must write y into it.  Every rank must run the same sequence of publishing
 * launches per flag (so every rank must hold at least one row of every published tensor), and a
 * flag may be published again only after every rank has consumed its previous generation.  orome_cuda_gather_wait(ctx, flag, vec, n, stream) completes the plain
 * copy of a gathered vector (n floats at vec, inside the arena) for readers other than this
 * library's kernels. */
int  orome_cuda_peer_alloc(orome_cuda_ctx *ctx, size_t bytes, void **dev_ptr, unsigned char handle_out[64]);
int  orome_cuda_peer_open(orome_cuda_ctx *ctx, const unsigned char handle[64], void **dev_ptr);
int  orome_cuda_peer_close(orome_cuda_ctx *ctx, void *dev_ptr);
int  orome_cuda_gather_setup(orome_cuda_ctx *ctx, int rank, int world, void *const *arenas, size_t data_bytes, int n_flags);
size_t orome_cuda_gather_arena_bytes(size_t data_bytes, int n_flags);
int  orome_cuda_gather_next(orome_cuda_ctx *ctx, int wait_flag, int publish_flag);
/* Enqueue a wait for one round of `flag` with nothing else attached (e.g. before copying the
 * gathered logits to the host). */
int  orome_cuda_gather_wait(orome_cuda_ctx *ctx, int flag, float *vec_dev, uint32_t n, void *stream);

/* ---- host-buffer convenience (end-to-end form) --------------------------- */

/* Same product as orome_cuda_matvec with HOST x and y: copies x to the device,
 * runs the kernel, copies y back and waits.  Staging buffers are owned by the
 * context and grow on demand. */
int  orome_cuda_matvec_host(orome_cuda_ctx *ctx, const OromeTensorRef *ref,
                            const float *x_host, float *y_host, int batch);

/* ---- tuning knobs -------------------------------------------------------- */

/* Integer options; unknown keys return OROME_EINVAL.
 *   OROME_OPT_X_BITS      16 or 24: fixed-point width used for x inside the
 *                         quantized matvec kernels (default 24: products within 2e-6 of an
 *                         exact evaluation).  16 makes plain products about 3 % faster on
 *                         Q8_0 at about 3e-5 (finer than the fp16 x of the reference's kernels,
 *                         inside the path's 1e-4).  The fused gate/up form reads x at 24 bits
 *                         whatever the option says: its output is a product of two results
 *                         and reached 1e-4 at 16 bits.  A recorded chain uses one width for all
 *                         of its products: the option's.
 *   OROME_OPT_FORCE_GENERIC  1 = always use the plain (non-pipelined) kernels. */
#define OROME_OPT_X_BITS         1
#define OROME_OPT_FORCE_GENERIC  2
#define OROME_OPT_STAGE_KB       3
#define OROME_OPT_CTAS_PER_SM    4
#define OROME_OPT_PDL            5
#define OROME_OPT_GRID_PER_SM    6
#define OROME_OPT_PREFETCH_MB     7   /* cap on the L2 prefetch of orome_cuda_hint_next, MiB (default 8; 0 = off) */
#define OROME_OPT_TC_MIN_BATCH    8   /* batches from this size on use the tensor-core kernel (default 4); smaller ones run one decode launch per vector */
#define OROME_OPT_KQUANT_MMA      9   /* 1 (default): Q4_K / Q5_K batch-1 products run on the mma.sync kernel; 0: on the dp4a kernel */
#define OROME_OPT_CHAIN_INFLIGHT 11   /* stages a chain's weight stream keeps outstanding at most (0, default: what fits 136 KiB, two at least; at most the ring); read at chain_end */
#define OROME_OPT_TC_SLABS       12   /* batched tensor-core form: 0 (default) keeps the dequantized weights in tensor memory, 1 stages them in shared memory */
#define OROME_OPT_TC_SPLIT       13   /* batched tensor-core form: K parts per row tile, 1..12; 0 (default): chosen by a cost model */
#define OROME_OPT_TC_TILES       14   /* batched tensor-core form (tensor-memory variant): row tiles a CTA works on side by side, 1, 2 or 4; 0 (default): cost model */
#define OROME_OPT_WAIT_US        10   /* bound of one device-side wait (peer data, chain inputs, chain stages) in microseconds; 0 (default): about a second */
int  orome_cuda_set_option(orome_cuda_ctx *ctx, int key, int value);
int  orome_cuda_get_option(orome_cuda_ctx *ctx, int key, int *value);

/* Number of kernel launches issued through this context since creation. */
uint64_t orome_cuda_launch_count(orome_cuda_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* OROME_CUDA_H */
