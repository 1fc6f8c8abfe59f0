// ctx.h -- the context object and the small host helpers shared by the library's translation units.
#pragma once
#include "../../include/orome_cuda.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <tuple>
#include <vector>

struct orome_cuda_chain;

struct MapKey {
    const uint8_t *w;
    uint32_t unit, units, rows, kb;
    bool operator<(const MapKey &o) const { return std::tie(w, unit, units, rows, kb) < std::tie(o.w, o.unit, o.units, o.rows, o.kb); }
};

struct orome_cuda_ctx {
    std::map<MapKey, CUtensorMap> maps;   // tensor maps of the mma kernel's tensors
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    int *status_dev = nullptr;
    unsigned int *chain_gen_dev = nullptr;   // generation base of chain tags: one counter per context, so chains that share vectors never reuse a tag
    uint64_t launches = 0;
    // options
    int x_bits = 24;
    int force_generic = 0;
    int stage_kb = 0;        // 0 = automatic
    int ctas_per_sm = 1;     // CTAs an SM is sized to hold (1 or 2); measured best with one large CTA
    int grid_per_sm = 1;     // CTAs per SM a launch creates; 1 with ctas_per_sm 2 leaves room for the next kernel's CTA
    int pdl = 1;
    int prefetch_mb = 8;     // at most this many MiB of the next tensor are pulled into L2 by the current launch (measured on the 9B set
                             // once x is requested before the weights: 3 MiB 655, 6 658.6, 8 656.5, 12 657, 24 649-650, 40 649 tok/s; 27B set 217.6 at 8, 213-216 at 24)
    const uint8_t *hint_ptr = nullptr;   // set by orome_cuda_hint_next, consumed by the next pipelined launch
    uint64_t hint_bytes = 0;
    // multi-GPU gather state (orome_cuda_gather_setup)
    int g_rank = 0, g_world = 1, g_nflags = 0;
    uint8_t *g_arena[8] = {nullptr};          // every rank's arena as mapped in this process
    size_t g_data_bytes = 0;
    unsigned int *g_local = nullptr;          // [n_flags] generation of each gathered vector, then the publish arrival counter
    int g_wait = -1, g_publish = -1;          // request for the next pipelined launch
    // fused neighbours requested for the next batch-1 product (orome_cuda_fuse_next)
    const void *fuse_norm_w = nullptr;
    const float *fuse_norm_parts = nullptr;
    float fuse_norm_eps = 0.0f;
    const float *fuse_res_in = nullptr;
    float *fuse_res_parts = nullptr;
    unsigned long long *trace_dev = nullptr;   // diagnostics buffer [trace_cap][sm_count][8]
    int trace_cap = 0, trace_next = 0;
    // staging for the host-buffer entry point
    float *stage_x_host = nullptr, *stage_y_host = nullptr, *stage_x_dev = nullptr, *stage_y_dev = nullptr;
    size_t stage_x_cap = 0, stage_y_cap = 0;
    cudaStream_t own_stream = nullptr;
    // scratch for routing logits when the caller passes none
    float *logits_dev = nullptr;
    size_t logits_cap = 0;
    // scratch for the unfused gate/up fallback
    float *gu_dev = nullptr;
    size_t gu_cap = 0;
    // scratch of the tensor-core batched form: packed fp16 X and split-K partial sums
    float *tc_xp = nullptr, *tc_part = nullptr;
    size_t tc_xp_cap = 0, tc_part_cap = 0;
    int tc_min_batch = 4;    // batches from this size on use the tensor-core kernel (smaller ones: one decode launch per vector)
    int tc_slabs = 0;        // batched form: 1 = dequantized weights staged in shared memory (the earlier form), 0 = in tensor memory
    int tc_tiles = 0;        // batched form in tensor memory: row tiles per CTA (0: chosen by the cost model)
    int tc_split = 0;        // batched form: K parts per row tile (0: chosen by the cost model)
    int kquant_mma = 1;      // Q4_K / Q5_K batch-1 products on the mma.sync kernel (0: dp4a kernel)
    int chain_inflight = 0;  // stages a chain's producer keeps outstanding at most (0: what fits 136 KiB, two at least)
    int wait_us = 0;         // bound of every device-side wait in microseconds of SM clock (0: about one second)
    // chain recording (orome_cuda_chain_begin .. _end): while set, the batch-1 entry points record instead of launching
    struct ChainRecording *rec = nullptr;
};

// Records the message of a failed call (returned by orome_cuda_last_error) and hands `code` back.
int orome_fail(int code, const char *fmt, ...);

#define CU(call)                                                                                         \
    do {                                                                                                 \
        cudaError_t e_ = (call);                                                                         \
        if (e_ != cudaSuccess) return orome_fail(OROME_ECUDA, "%s: %s", #call, cudaGetErrorString(e_));  \
    } while (0)

// ---- helpers shared by the translation units (defined in orome_cuda.cu) --------------------------------------
int orome_check_ref(const char *who, const OromeTensorRef *r, const uint8_t **data);
uint32_t orome_pipe_group_threads(int fmt, uint32_t in_dim);
bool orome_pipe_supported(int fmt, uint32_t in_dim);
long long orome_wait_cycles(const orome_cuda_ctx *c);

// ---- chain recording (defined in chain.cu) --------------------------------------------------------------------
// Called by the batch-1 entry points, after their own validation, while a recording is open.
int orome_chain_record_group(orome_cuda_ctx *c, const OromeTensorRef *refs, int n_refs, const float *x, float *const *y);
int orome_chain_record_gate_up(orome_cuda_ctx *c, const OromeTensorRef *gate, const OromeTensorRef *up, const float *x, float *out);
int orome_chain_record_unpack(orome_cuda_ctx *c, float *vec, uint32_t n);
int orome_chain_record_argmax(orome_cuda_ctx *c, const float *data, uint32_t count, uint32_t *result);
void orome_chain_abandon(orome_cuda_ctx *c);

// ---- diagnostics builds only (-DOROME_DIAGNOSTICS); not part of the public header ------------------------------------
#ifdef OROME_DIAGNOSTICS
extern "C" {
// The next `launches` pipelined launches record eight %globaltimer stamps per CTA; trace_read synchronises and
// copies launches * sm_count * 8 values out.
int orome_cuda_trace_begin(orome_cuda_ctx *ctx, int launches);
int orome_cuda_trace_read(orome_cuda_ctx *ctx, unsigned long long *out, size_t n_values);
}
#endif
