// orome_cuda.cu -- C ABI (include/orome_cuda.h) and host-side dispatch for the
// B200 quantized dequant-matvec path.  The host logic here is the counterpart
// of the reference's format layer (inference/src/format.m:224-337): validate the
// TensorRef, pick the kernel from its format/variant, size the launch.
#include "ctx.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <tuple>

#include "decode.cuh"
#include "gemv_generic.cuh"
#include "gemv_pipe.cuh"
#include "gemv_mma.cuh"
#include "moe.cuh"
#include "gemm_tc.cuh"

using namespace orome;

static thread_local std::string g_err;

int orome_fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}
#define fail orome_fail

extern "C" const char *orome_cuda_last_error(void) { return g_err.c_str(); }

extern "C" int orome_cuda_ctx_create(int device, orome_cuda_ctx **out)
{
    if (!out) return fail(OROME_EINVAL, "ctx_create: out is NULL");
    int n = 0;
    CU(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n) return fail(OROME_EINVAL, "ctx_create: device %d of %d", device, n);
    CU(cudaSetDevice(device));
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10) return fail(OROME_ENOTSUP, "ctx_create: device is sm_%d%d, the kernels are built for sm_100a", prop.major, prop.minor);
    auto *c = new orome_cuda_ctx;
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = (int)prop.sharedMemPerBlockOptin;
    CU(cudaMalloc(&c->status_dev, 256));          // the status word, and (64 bytes on) the tag generation shared by the context's chains
    CU(cudaMemset(c->status_dev, 0, 256));
    c->chain_gen_dev = reinterpret_cast<unsigned int *>(c->status_dev) + 16;
    CU(cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking));
    *out = c;
    return OROME_OK;
}

extern "C" void orome_cuda_ctx_destroy(orome_cuda_ctx *c)
{
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->rec) orome_chain_abandon(c);
    cudaFree(c->status_dev);
    cudaFree(c->stage_x_dev);
    cudaFree(c->stage_y_dev);
    cudaFree(c->logits_dev);
    cudaFree(c->gu_dev);
    cudaFree(c->tc_xp);
    cudaFree(c->tc_part);
    cudaFree(c->trace_dev);
    cudaFree(c->g_local);
    cudaFreeHost(c->stage_x_host);
    cudaFreeHost(c->stage_y_host);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
}

extern "C" int orome_cuda_status(orome_cuda_ctx *c, int *status_out)
{
    if (!c || !status_out) return fail(OROME_EINVAL, "status: NULL argument");
    CU(cudaSetDevice(c->device));
    CU(cudaDeviceSynchronize());
    CU(cudaMemcpy(status_out, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_out) CU(cudaMemset(c->status_dev, 0, sizeof(int)));      // reported once; later launches wait again
    return *status_out ? fail(OROME_ETIMEOUT, "a kernel's bounded wait expired (status %d)", *status_out) : OROME_OK;
}

extern "C" int orome_cuda_upload(orome_cuda_ctx *c, const void *host, size_t bytes, void **dev_base)
{
    if (!c || !dev_base || (!host && bytes)) return fail(OROME_EINVAL, "upload: NULL argument");
    CU(cudaSetDevice(c->device));
    void *p = nullptr;
    // 256 bytes of zeroed slack after the data keep 16-byte granular reads of a ragged tensor end inside the allocation
    cudaError_t e = cudaMalloc(&p, bytes + 256);
    if (e != cudaSuccess) return fail(OROME_ENOMEM, "upload: cudaMalloc(%zu): %s", bytes + 256, cudaGetErrorString(e));
    CU(cudaMemset(static_cast<uint8_t *>(p) + bytes, 0, 256));
    if (bytes) CU(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice));
    *dev_base = p;
    return OROME_OK;
}

extern "C" int orome_cuda_download(orome_cuda_ctx *c, const void *dev, void *host, size_t bytes)
{
    if (!c || (bytes && (!dev || !host))) return fail(OROME_EINVAL, "download: NULL argument");
    CU(cudaSetDevice(c->device));
    CU(cudaDeviceSynchronize());
    if (bytes) CU(cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost));
    return OROME_OK;
}

extern "C" int orome_cuda_free(orome_cuda_ctx *c, void *dev_base)
{
    if (!c) return fail(OROME_EINVAL, "free: NULL ctx");
    CU(cudaSetDevice(c->device));
    CU(cudaFree(dev_base));
    return OROME_OK;
}

extern "C" OromeQuantFormat orome_format_from_ggml_type(uint32_t t)
{
    switch (t) {
    case 8: return OROME_QFMT_GGUF_Q8_0;
    case 12: return OROME_QFMT_GGUF_Q4_K;
    case 13: return OROME_QFMT_GGUF_Q5_K;
    case 14: return OROME_QFMT_GGUF_Q6_K;
    case 1: return OROME_QFMT_F16;
    case 30: return OROME_QFMT_BF16;
    case 0: return OROME_QFMT_F32;
    default: return OROME_QFMT_GGUF_Q4_K;   // the reference's fallback (format.m:335)
    }
}

extern "C" size_t orome_format_row_bytes(OromeQuantFormat f, uint32_t in_dim)
{
    int fmt = (int)f;
    if (fmt < 0 || fmt > FMT_F32) return 0;
    if (fmt <= FMT_Q8_0 && in_dim % block_elems(fmt)) return 0;
    return row_bytes_of(fmt, in_dim);
}

extern "C" int orome_cuda_set_option(orome_cuda_ctx *c, int key, int value)
{
    if (!c) return fail(OROME_EINVAL, "set_option: NULL ctx");
    switch (key) {
    case OROME_OPT_X_BITS:
        if (value != 16 && value != 24) return fail(OROME_EINVAL, "X_BITS must be 16 or 24");
        c->x_bits = value; return OROME_OK;
    case OROME_OPT_FORCE_GENERIC: c->force_generic = value != 0; return OROME_OK;
    case OROME_OPT_STAGE_KB:
        if (value < 0 || value > 200) return fail(OROME_EINVAL, "STAGE_KB out of range");
        c->stage_kb = value; return OROME_OK;
    case OROME_OPT_CTAS_PER_SM:
        if (value < 1 || value > 4) return fail(OROME_EINVAL, "CTAS_PER_SM must be 1..4");
        c->ctas_per_sm = value; return OROME_OK;
    case OROME_OPT_PDL: c->pdl = value != 0; return OROME_OK;
    case OROME_OPT_TC_SLABS: c->tc_slabs = value != 0; return OROME_OK;
    case OROME_OPT_TC_SPLIT:
        if (value < 0 || value > 12) return fail(OROME_EINVAL, "TC_SPLIT must be 0 (automatic) .. 12");
        c->tc_split = value; return OROME_OK;
    case OROME_OPT_TC_TILES:
        if (value != 0 && value != 1 && value != 2 && value != 4) return fail(OROME_EINVAL, "TC_TILES must be 0 (automatic), 1, 2 or 4");
        c->tc_tiles = value; return OROME_OK;
    case OROME_OPT_GRID_PER_SM:
        if (value < 1 || value > 2) return fail(OROME_EINVAL, "GRID_PER_SM must be 1 or 2");
        c->grid_per_sm = value; return OROME_OK;
    case OROME_OPT_KQUANT_MMA: c->kquant_mma = value != 0; return OROME_OK;
    case OROME_OPT_TC_MIN_BATCH:
        if (value < 2) return fail(OROME_EINVAL, "TC_MIN_BATCH must be at least 2");
        c->tc_min_batch = value; return OROME_OK;
    case OROME_OPT_PREFETCH_MB:
        if (value < 0 || value > 96) return fail(OROME_EINVAL, "PREFETCH_MB must be 0..96");
        c->prefetch_mb = value; return OROME_OK;
    case OROME_OPT_WAIT_US:
        if (value < 0 || value > 10000000) return fail(OROME_EINVAL, "WAIT_US must be 0..10000000");
        c->wait_us = value; return OROME_OK;
    case OROME_OPT_CHAIN_INFLIGHT:
        if (value < 0 || value > PIPE_MAX_STAGES) return fail(OROME_EINVAL, "CHAIN_INFLIGHT must be 0..%d", PIPE_MAX_STAGES);
        c->chain_inflight = value; return OROME_OK;
    }
    return fail(OROME_EINVAL, "set_option: unknown key %d", key);
}

extern "C" int orome_cuda_get_option(orome_cuda_ctx *c, int key, int *value)
{
    if (!c || !value) return fail(OROME_EINVAL, "get_option: NULL argument");
    switch (key) {
    case OROME_OPT_X_BITS: *value = c->x_bits; return OROME_OK;
    case OROME_OPT_FORCE_GENERIC: *value = c->force_generic; return OROME_OK;
    case OROME_OPT_STAGE_KB: *value = c->stage_kb; return OROME_OK;
    case OROME_OPT_TC_SLABS: *value = c->tc_slabs; return OROME_OK;
    case OROME_OPT_TC_SPLIT: *value = c->tc_split; return OROME_OK;
    case OROME_OPT_TC_TILES: *value = c->tc_tiles; return OROME_OK;
    case OROME_OPT_CTAS_PER_SM: *value = c->ctas_per_sm; return OROME_OK;
    case OROME_OPT_PDL: *value = c->pdl; return OROME_OK;
    case OROME_OPT_GRID_PER_SM: *value = c->grid_per_sm; return OROME_OK;
    case OROME_OPT_PREFETCH_MB: *value = c->prefetch_mb; return OROME_OK;
    case OROME_OPT_TC_MIN_BATCH: *value = c->tc_min_batch; return OROME_OK;
    case OROME_OPT_KQUANT_MMA: *value = c->kquant_mma; return OROME_OK;
    case OROME_OPT_WAIT_US: *value = c->wait_us; return OROME_OK;
    case OROME_OPT_CHAIN_INFLIGHT: *value = c->chain_inflight; return OROME_OK;
    }
    return fail(OROME_EINVAL, "get_option: unknown key %d", key);
}

#ifdef OROME_DIAGNOSTICS
// Per-CTA timeline stamps of the pipelined kernels; compiled only into diagnostics builds (-DOROME_DIAGNOSTICS).
extern "C" int orome_cuda_trace_begin(orome_cuda_ctx *c, int launches)
{
    if (!c || launches < 0) return fail(OROME_EINVAL, "trace_begin: bad argument");
    CU(cudaSetDevice(c->device));
    if (c->trace_dev) cudaFree(c->trace_dev);
    c->trace_dev = nullptr;
    c->trace_cap = c->trace_next = 0;
    if (launches == 0) return OROME_OK;
    size_t bytes = (size_t)launches * c->sm_count * 8 * sizeof(unsigned long long);
    CU(cudaMalloc(&c->trace_dev, bytes));
    CU(cudaMemset(c->trace_dev, 0, bytes));
    c->trace_cap = launches;
    return OROME_OK;
}

extern "C" int orome_cuda_trace_read(orome_cuda_ctx *c, unsigned long long *out, size_t n_values)
{
    if (!c || !out || !c->trace_dev) return fail(OROME_EINVAL, "trace_read: no trace");
    CU(cudaSetDevice(c->device));
    CU(cudaDeviceSynchronize());
    size_t have = (size_t)c->trace_cap * c->sm_count * 8;
    CU(cudaMemcpy(out, c->trace_dev, std::min(have, n_values) * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return OROME_OK;
}

#endif

extern "C" uint64_t orome_cuda_launch_count(orome_cuda_ctx *c) { return c ? c->launches : 0; }

// ---------------------------------------------------------------------------
// validation shared by the entry points
// ---------------------------------------------------------------------------
int orome_check_ref(const char *who, const OromeTensorRef *r, const uint8_t **data)
{
    if (!r) return fail(OROME_EINVAL, "%s: NULL TensorRef", who);
    int fmt = (int)r->format;
    if (fmt < 0 || fmt > FMT_F32) return fail(OROME_ENOTSUP, "%s: unknown format %d", who, fmt);
    if (r->variant > OROME_VARIANT_LLAMA) return fail(OROME_ENOTSUP, "%s: unknown kernel variant %u", who, r->variant);
    if (r->out_dim == 0 || r->in_dim == 0) return fail(OROME_EINVAL, "%s: empty tensor (%u x %u)", who, r->out_dim, r->in_dim);
    if (fmt <= FMT_Q8_0 && r->in_dim % block_elems(fmt))
        return fail(OROME_EINVAL, "%s: in_dim %u is not a multiple of %d", who, r->in_dim, block_elems(fmt));
    const uint8_t *p = static_cast<const uint8_t *>(r->buffer) + r->offset;
    if (reinterpret_cast<uintptr_t>(p) & 15) return fail(OROME_EINVAL, "%s: tensor data is not 16-byte aligned", who);
    *data = p;
    return OROME_OK;
}

// Bound of one device-side wait in SM cycles (the SM clock is about 2 GHz).
long long orome_wait_cycles(const orome_cuda_ctx *c) { return c->wait_us > 0 ? (long long)c->wait_us * 2000ll : PIPE_WAIT_CYCLES; }

static int post_launch(orome_cuda_ctx *c, const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(OROME_ECUDA, "%s launch: %s", what, cudaGetErrorString(e));
    ++c->launches;
    return OROME_OK;
}

// Launch with programmatic stream serialization, so the kernel's launch overlaps the tail of its predecessor
// (the kernel itself starts with griddepcontrol.wait).
template <typename... KArgs, typename... Args>
static int launch_pdl_smem(orome_cuda_ctx *c, const char *what, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args);

template <typename... KArgs, typename... Args>
static int launch_pdl(orome_cuda_ctx *c, const char *what, void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args)
{
    return launch_pdl_smem(c, what, kern, grid, block, 0, st, args...);
}

template <typename... KArgs, typename... Args>
static int launch_pdl_smem(orome_cuda_ctx *c, const char *what, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return fail(OROME_ECUDA, "%s launch: %s", what, cudaGetErrorString(e));
    ++c->launches;
    return OROME_OK;
}

static int launch_generic(orome_cuda_ctx *c, int fmt, const uint8_t *data, uint32_t out_dim, uint32_t in_dim, int layout,
                          const float *x, int batch, int ldx, float *y, int ldy, cudaStream_t st);

// shared_gate: the single-row fp32 tensor of the shared-expert gate, or NULL.  With it the logits have ne + 1 entries per
// token and shared_logit[t] receives the last one.
static int launch_router(orome_cuda_ctx *c, const uint8_t *data, uint32_t ne, uint32_t in_dim, const float *x, int n_tokens, int ldx,
                         float *logits, uint32_t K, uint32_t *idx, float *w, cudaStream_t st, const uint8_t *shared_gate = nullptr,
                         float *shared_logit = nullptr)
{
    int rc;
    const uint32_t rows = ne + (shared_gate ? 1u : 0u);
    if (in_dim % 4 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) && (n_tokens == 1 || ldx % 4 == 0))
        rc = launch_pdl(c, "gemv_f32", gemv_f32_kernel, dim3(rows, (unsigned)(n_tokens + 3) / 4), dim3(128), st, reinterpret_cast<const float *>(data), ne, in_dim,
                        x, n_tokens, ldx, logits, (int)rows, reinterpret_cast<const float *>(shared_gate));
    else {
        rc = launch_generic(c, FMT_F32, data, ne, in_dim, 0, x, n_tokens, ldx, logits, (int)rows, st);
        if (!rc && shared_gate) rc = launch_generic(c, FMT_F32, shared_gate, 1, in_dim, 0, x, n_tokens, ldx, logits + ne, (int)rows, st);
    }
    if (rc) return rc;
    return launch_pdl(c, "route_topk", route_topk_kernel, dim3(n_tokens), dim3(256), st, (const float *)logits, (int)rows, ne, K, idx, w,
                      shared_gate ? shared_logit : (float *)nullptr);
}

// ---------------------------------------------------------------------------
// generic kernels
// ---------------------------------------------------------------------------
template <int FMT>
static int launch_generic_fmt(orome_cuda_ctx *c, const uint8_t *data, uint32_t out_dim, uint32_t in_dim, int layout,
                              const float *x, int batch, int ldx, float *y, int ldy, cudaStream_t st)
{
    size_t rb = row_bytes_of(FMT, in_dim);
    dim3 grid((out_dim + 7) / 8), block(256);
    if (batch == 1) gemv_generic_kernel<FMT, 1><<<grid, block, 0, st>>>(data, rb, out_dim, in_dim, layout, x, batch, ldx, y, ldy);
    else if (batch <= 4) gemv_generic_kernel<FMT, 4><<<grid, block, 0, st>>>(data, rb, out_dim, in_dim, layout, x, batch, ldx, y, ldy);
    else gemv_generic_kernel<FMT, 8><<<grid, block, 0, st>>>(data, rb, out_dim, in_dim, layout, x, batch, ldx, y, ldy);
    return post_launch(c, "gemv_generic");
}

static int launch_generic(orome_cuda_ctx *c, int fmt, const uint8_t *data, uint32_t out_dim, uint32_t in_dim, int layout,
                          const float *x, int batch, int ldx, float *y, int ldy, cudaStream_t st)
{
    switch (fmt) {
    case FMT_Q4_K: return launch_generic_fmt<FMT_Q4_K>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    case FMT_Q5_K: return launch_generic_fmt<FMT_Q5_K>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    case FMT_Q6_K: return launch_generic_fmt<FMT_Q6_K>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    case FMT_Q8_0: return launch_generic_fmt<FMT_Q8_0>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    case FMT_F16: return launch_generic_fmt<FMT_F16>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    case FMT_BF16: return launch_generic_fmt<FMT_BF16>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    case FMT_F32: return launch_generic_fmt<FMT_F32>(c, data, out_dim, in_dim, layout, x, batch, ldx, y, ldy, st);
    }
    return fail(OROME_ENOTSUP, "no kernel for format %d", fmt);
}

// ---------------------------------------------------------------------------
// pipelined decode kernel: planning and launch
// ---------------------------------------------------------------------------
struct PipePlan {
    PipeArgs args;
    int threads;
    int grid;
    int minb;       // CTAs per SM the kernel instance is compiled for
    size_t smem;
    int tokens;     // token batch of the MoE forms (grid.y); 0 or 1: a single-token launch
};

uint32_t orome_pipe_group_threads(int fmt, uint32_t in_dim)
{
    const uint32_t slots = fmt == FMT_Q8_0 ? in_dim / 64 : in_dim / 256 * 4;
    return (slots + 31) / 32 * 32;
}

bool orome_pipe_supported(int fmt, uint32_t in_dim)
{
    if (fmt == FMT_Q8_0) return in_dim % 64 == 0 && orome_pipe_group_threads(fmt, in_dim) <= PIPE_MAX_CONSUMERS;
    if (fmt == FMT_Q4_K || fmt == FMT_Q5_K || fmt == FMT_Q6_K)
        return in_dim % 256 == 0 && orome_pipe_group_threads(fmt, in_dim) <= PIPE_MAX_CONSUMERS;
    return false;
}

// Multi-GPU: turn the request left by orome_cuda_gather_next into the launch's publish / wait fields.
template <typename Args>
static int arm_gather(orome_cuda_ctx *c, Args &a, uint32_t in_dim)
{
    a.npeers = 0;
    a.x_ll = nullptr;
    if (c->g_world > 1) {
        uint8_t *mine = c->g_arena[c->g_rank];
        a.arena_base = mine;
        a.ll_origin = mine + c->g_data_bytes;
        if (c->g_publish >= 0) {
            int n = 0;
            for (int r = 0; r < c->g_world; ++r) {
                if (r == c->g_rank) continue;
                a.peer_delta[n++] = (long long)(c->g_arena[r] - mine);
            }
            a.npeers = n;
            a.pub_gen = c->g_local + c->g_publish;
            a.pub_arrived = c->g_local + c->g_nflags;
        }
        if (c->g_wait >= 0) {
            const uint8_t *xb = reinterpret_cast<const uint8_t *>(a.x);
            if (xb < mine || xb + (size_t)in_dim * 4 > mine + c->g_data_bytes || ((xb - mine) & 15)) {
                c->g_wait = c->g_publish = -1;
                return fail(OROME_EINVAL, "a launch that waits for a gathered vector must read x from the gather arena (16-byte aligned)");
            }
            a.x_ll = reinterpret_cast<const uint2 *>(a.ll_origin + 2 * (size_t)(xb - mine));
            a.wait_gen = c->g_local + c->g_wait;
        }
        c->g_wait = c->g_publish = -1;
    }
    return OROME_OK;
}

// Fill everything of the plan except the segments' pointers.
static int plan_pipe(orome_cuda_ctx *c, int fmt, uint32_t in_dim, uint32_t total_rows, int mode, PipePlan &p)
{
    const bool swiglu = mode == 1, combine = mode == 2;   // combine: total_rows = rows of one segment, args.nseg input vectors
    PipeArgs &a = p.args;
    a.in_dim = in_dim;
    a.row_bytes = (uint32_t)row_bytes_of(fmt, in_dim);
    a.units = fmt == FMT_Q8_0 ? in_dim / 64 : in_dim / 256;
    a.group_threads = orome_pipe_group_threads(fmt, in_dim);
    a.total_rows = total_rows;
    p.minb = c->ctas_per_sm >= 2 && a.group_threads <= PIPE_CONSUMERS_2CTA && !combine ? 2 : 1;
    if (fmt == FMT_Q6_K && swiglu) p.minb = 1;   // the fused form reads x at 24 bits: more than the 96 registers of the two-CTA build
    const uint32_t max_consumers = p.minb == 2 ? PIPE_CONSUMERS_2CTA : PIPE_MAX_CONSUMERS;
    a.rows_par = std::max(1u, std::min((uint32_t)PIPE_MAX_ROWS_PAR, max_consumers / a.group_threads));
    a.rows_par = std::min(a.rows_par, std::max(1u, total_rows));
    const uint32_t consumers = a.group_threads * a.rows_par, gw = a.group_threads / 32;
    p.threads = (int)consumers + 32;

    p.grid = (int)std::min<uint64_t>((uint64_t)c->sm_count * std::min(p.minb, c->grid_per_sm), (total_rows + a.rows_par - 1) / a.rows_par);
    // a token batch spreads about two waves of CTAs over the tokens (grid.y), each token's rows over grid.x CTAs
    // (measured at 32 tokens: one wave 408 us per layer, two 380, three or four 412, six 461)
    if (p.tokens > 1) p.grid = std::min(p.grid, std::max(1, 2 * c->sm_count / p.tokens));
    p.grid = std::max(p.grid, 1);
    const uint32_t share = (total_rows + p.grid - 1) / p.grid;            // rows of the busiest CTA

    const uint32_t per_row = a.row_bytes * (swiglu ? 2 : 1);
    // plain Q8_0 products pair rows inside a tile (two rows per group in flight), which needs tiles of two rows per group
    const uint32_t want = (c->stage_kb ? (uint32_t)c->stage_kb : (fmt == FMT_Q8_0 && mode == 0 ? 64u : 16u)) * 1024u;
    a.iters = std::max(1u, std::min((uint32_t)PIPE_MAX_ITERS, want / (per_row * a.rows_par)));
    a.iters = std::min(a.iters, (share + a.rows_par - 1) / a.rows_par);

    // shared memory of one SM is 228 KiB; every resident CTA also reserves 1 KiB
    const size_t sm_total = 228 * 1024;
    size_t budget = sm_total / p.minb - 1024 - 256;
    budget = std::min(budget, (size_t)c->smem_optin - 256);
    a.red_base = 2 * 8 * PIPE_MAX_STAGES;
    // partial-sum buffers: a whole CTA share when it is small, else batches of 256 rows (at most 16 KiB per buffer)
    a.red_rows = std::min<uint32_t>(std::max<uint32_t>(share, a.rows_par * PIPE_MAX_ITERS), 256u);
    a.red_rows = std::max<uint32_t>(std::min<uint32_t>(a.red_rows, 4096u / gw), a.rows_par * PIPE_MAX_ITERS);
    if (combine) a.red_rows = std::max<uint32_t>(a.red_rows, (share * a.rows_par + 1) / 2);   // one slot per row, group and warp fits the two buffers
    const size_t red_bytes = (size_t)2 * a.red_rows * gw * (swiglu ? 2 : 1) * sizeof(float);
    a.xs_base = (uint32_t)((a.red_base + red_bytes + 127) / 128 * 128);
    // quantized x: one byte plane per 8 bits of x, a scale per group (16 for Q6_K, else 32), a sum per 32 elements
    // the fused gate/up form always reads x at 24 bits: its output is a product of two results, which at 16 bits can
    // leave the 1e-4 bound (measured: 5e-5 typical, 1.1e-4 on small row sets); plain products follow the option
    const size_t np = (c->x_bits == 24 || swiglu) ? 3 : 2;
    const size_t xq_vec = (np * in_dim + (size_t)in_dim / (fmt == FMT_Q6_K ? 16 : 32) * 4 + (size_t)in_dim / 32 * 4 + 15) / 16 * 16;
    a.xq_vec_bytes = (uint32_t)xq_vec;
    const size_t xq_bytes = xq_vec * (combine ? std::max(a.nseg, 1) : 1);
    a.acc_base = (uint32_t)((a.xs_base + xq_bytes + 15) / 16 * 16);
    a.stage_base = (uint32_t)((a.acc_base + (combine ? (size_t)(share + 1) * sizeof(float) : 0) + 127) / 128 * 128);
    for (;;) {
        a.half_stride = (a.rows_par * a.iters * a.row_bytes + 48 + 127) / 128 * 128;
        a.stage_stride = a.half_stride * (swiglu ? 2 : 1);
        const size_t room = budget > a.stage_base ? budget - a.stage_base : 0;
        uint32_t ns = (uint32_t)std::min<size_t>(PIPE_MAX_STAGES, room / a.stage_stride);
        if (ns >= 3 || a.iters == 1) {
            if (ns < 1) return fail(OROME_ENOTSUP, "pipe plan: a stage of %u bytes does not fit shared memory", a.stage_stride);
            // the combine form walks the CTA's row range once per segment
            const uint32_t tiles = ((share + a.rows_par * a.iters - 1) / (a.rows_par * a.iters)) * (combine ? (uint32_t)std::max(a.nseg, 1) : 1u) + 1;
            a.nstages = std::min(ns, tiles);
            break;
        }
        --a.iters;
    }
    p.smem = a.stage_base + (size_t)a.stage_stride * a.nstages;
    a.status = c->status_dev;
    a.wait_cycles = orome_wait_cycles(c);
    a.trace = nullptr;
    if (c->trace_dev && c->trace_next < c->trace_cap) a.trace = c->trace_dev + (size_t)(c->trace_next++) * c->sm_count * 8;
    {
        int rc = arm_gather(c, a, in_dim);
        if (rc) return rc;
    }
    a.pf_ptr = c->hint_ptr;
    a.pf_bytes = c->hint_bytes;
    c->hint_ptr = nullptr;
    c->hint_bytes = 0;
    // fused norm prologue / residual epilogue (the entry points have checked that this launch can take them)
    a.norm_w = static_cast<const uint16_t *>(c->fuse_norm_w);
    a.norm_parts = c->fuse_norm_parts;
    a.norm_eps = c->fuse_norm_eps;
    a.res_in = c->fuse_res_in;
    a.res_parts = c->fuse_res_parts;
    c->fuse_norm_w = nullptr; c->fuse_norm_parts = nullptr; c->fuse_res_in = nullptr; c->fuse_res_parts = nullptr;
    if (a.res_parts && p.grid > PIPE_SUM_SQ_PARTS) return fail(OROME_ENOTSUP, "pipe plan: more CTAs than entries in a partials array");
    return OROME_OK;
}

template <int FMT, int NP, int MODE, int MINB, bool EXT>
static int launch_pipe_ext(orome_cuda_ctx *c, const PipePlan &p, cudaStream_t st)
{
    auto kern = gemv_pipe_kernel<FMT, NP, MODE, MINB, EXT>;
    static size_t configured[64] = {0};   // per device: dynamic shared memory opted in so far
    if (configured[c->device] < p.smem) {
        cudaFuncAttributes fa;
        CU(cudaFuncGetAttributes(&fa, kern));
        const int max_dyn = c->smem_optin - (int)fa.sharedSizeBytes;   // the opt-in limit covers static + dynamic
        if ((size_t)max_dyn < p.smem) return fail(OROME_ENOTSUP, "pipe launch: %zu bytes of shared memory exceed the limit %d", p.smem, max_dyn);
        CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dyn));
        configured[c->device] = (size_t)max_dyn;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid, std::max(p.tokens, 1));
    cfg.blockDim = dim3(p.threads);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->pdl ? 1 : 0;
    CU(cudaLaunchKernelEx(&cfg, kern, p.args));
    ++c->launches;
    return OROME_OK;
}

template <int FMT, int NP, int MODE, int MINB>
static int launch_pipe_inst(orome_cuda_ctx *c, const PipePlan &p, cudaStream_t st)
{
    const bool ext = p.args.seg_expert || p.args.npeers > 0 || p.args.x_ll || p.args.norm_w || p.args.res_in || p.tokens > 1;
    if constexpr (MODE == 2) return launch_pipe_ext<FMT, NP, MODE, MINB, true>(c, p, st);
    else return ext ? launch_pipe_ext<FMT, NP, MODE, MINB, true>(c, p, st) : launch_pipe_ext<FMT, NP, MODE, MINB, false>(c, p, st);
}

template <int FMT, int NP>
static int launch_pipe_np(orome_cuda_ctx *c, const PipePlan &p, int mode, cudaStream_t st)
{
    if (mode == 2) return launch_pipe_inst<FMT, NP, 2, 1>(c, p, st);
    if (p.minb == 2) return mode == 1 ? launch_pipe_inst<FMT, NP, 1, 2>(c, p, st) : launch_pipe_inst<FMT, NP, 0, 2>(c, p, st);
    return mode == 1 ? launch_pipe_inst<FMT, NP, 1, 1>(c, p, st) : launch_pipe_inst<FMT, NP, 0, 1>(c, p, st);
}

template <int FMT>
static int launch_pipe_fmt(orome_cuda_ctx *c, const PipePlan &p, int mode, cudaStream_t st)
{
    return (c->x_bits == 24 || mode == 1) ? launch_pipe_np<FMT, 3>(c, p, mode, st) : launch_pipe_np<FMT, 2>(c, p, mode, st);
}

static int launch_pipe(orome_cuda_ctx *c, int fmt, const PipePlan &p, int mode, cudaStream_t st)
{
    switch (fmt) {
    case FMT_Q4_K: return launch_pipe_fmt<FMT_Q4_K>(c, p, mode, st);
    case FMT_Q5_K: return launch_pipe_fmt<FMT_Q5_K>(c, p, mode, st);
    case FMT_Q6_K: return launch_pipe_fmt<FMT_Q6_K>(c, p, mode, st);
    case FMT_Q8_0: return launch_pipe_fmt<FMT_Q8_0>(c, p, mode, st);
    }
    return fail(OROME_ENOTSUP, "no pipelined kernel for format %d", fmt);
}

// ---------------------------------------------------------------------------
// Q4_K / Q5_K batch-1 kernel on mma.sync: planning and launch
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn();

struct MmaPlan {
    MmaArgs args;
    int threads, grid;
    int tokens;        // MoE forms: grid rows (one per token)
    size_t smem;
};

// Dense single-GPU launches only: every tensor 16-byte aligned (rows are then 16-byte aligned too, as the row length
// is a multiple of 16 bytes), no expert indirection, no peers.
static bool mma_supported(const orome_cuda_ctx *c, int fmt, uint32_t in_dim, bool swiglu)
{
    const bool fmt_ok = fmt == FMT_Q4_K || fmt == FMT_Q5_K || (fmt == FMT_Q6_K && !swiglu);
    return c->kquant_mma && !c->force_generic && fmt_ok && in_dim % 256 == 0 && in_dim >= 256;
}

// nvec > 1: the combine form of the MoE down projection -- a row is the sum over nvec experts of a product with that
// expert's own input vector (in_dim wide each, one behind the other); a stage then holds one expert's whole rows.
// grid_cap > 0 (MoE forms): at most that many CTAs, each with the same whole number of row tiles where that divides.
// two: the form that multiplies two input vectors at once (plain Q4_K / Q5_K): wider quantized x, two result planes.
static int plan_mma(orome_cuda_ctx *c, int fmt, uint32_t in_dim, uint32_t total_rows, bool swiglu, MmaPlan &p, uint32_t nvec = 0, uint32_t grid_cap = 0,
                    bool two = false)
{
    MmaArgs &a = p.args;
    const uint32_t unit = fmt == FMT_Q4_K ? 144u : fmt == FMT_Q5_K ? 176u : 210u;
    const uint32_t units_row = in_dim / 256;
    a.in_dim = in_dim;
    a.units = units_row * std::max(1u, nvec);
    a.row_bytes = units_row * unit;
    a.total_rows = total_rows;
    // a stage of about stage_kb (default 40) KiB: 16 rows (x2 in the fused form) of kc superblocks
    const uint32_t want = (c->stage_kb ? (uint32_t)c->stage_kb : 40u) * 1024u;
    const uint32_t kc_max = std::max(1u, std::min(units_row, want / (MMA_TILE_ROWS * unit * (swiglu ? 2u : 1u))));
    if (nvec > 0) {
        if (units_row > kc_max) return fail(OROME_ENOTSUP, "mma plan: combine form with rows of %u superblocks", units_row);
        a.nchunks = nvec;
        a.kc = units_row;
    } else {
        a.nchunks = (a.units + kc_max - 1) / kc_max;
        a.kc = (a.units + a.nchunks - 1) / a.nchunks;
    }
    const uint32_t rounds = (a.kc + MMA_MAX_WARPS - 1) / MMA_MAX_WARPS;
    a.nwarps = (a.kc + rounds - 1) / rounds;
    p.grid = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)c->sm_count, (total_rows + MMA_TILE_ROWS - 1) / MMA_TILE_ROWS));
    if (grid_cap) {
        const uint32_t tiles = (total_rows + MMA_TILE_ROWS - 1) / MMA_TILE_ROWS, cap = std::max(1u, std::min(grid_cap, tiles));
        const uint32_t per = (tiles + cap - 1) / cap;
        p.grid = (int)((tiles + per - 1) / per);
    }
    const uint32_t share = (total_rows + p.grid - 1) / p.grid;
    // stages (row tiles x chunks) go round the groups: as many groups as the warp budget and the CTA's stage count allow
    const uint32_t cta_stages = (share + MMA_TILE_ROWS - 1) / MMA_TILE_ROWS * a.nchunks;
    a.ngroups = std::max(1u, std::min(std::min<uint32_t>(MMA_MAX_GROUPS, MMA_MAX_CONSUMER_WARPS / a.nwarps), cta_stages));
    p.threads = (int)(a.nwarps * a.ngroups + (fmt == FMT_Q6_K ? 2 : 1)) * 32;
    // box width in superblocks: the smallest kb >= kc with kb = 2 (mod 4), which makes the row pitch 32 or 96 (mod 128)
    const uint32_t kb = a.kc + ((6 - a.kc % 4) % 4);
    a.pitch = kb * unit;
    if (fmt == FMT_Q6_K) {
        // rows arrive by their own copies, widened to 16-byte boundaries (up to 15 bytes before and after the chunk)
        a.pitch = (a.kc * unit + 30 + 15) / 16 * 16;
        while (a.pitch % 128 != 16) a.pitch += 16;      // the quads of the eight rows of a load then read eight different four-bank groups
    }
    a.box_bytes = MMA_TILE_ROWS * a.pitch;
    a.half_stride = MMA_TILE_ROWS * a.pitch;
    a.stage_stride = a.half_stride * (swiglu ? 2 : 1);
    a.red_base = 2 * 8 * PIPE_MAX_STAGES;
    a.red_rows = std::max<uint32_t>(MMA_TILE_ROWS, std::min<uint32_t>((share + MMA_TILE_ROWS - 1) / MMA_TILE_ROWS * MMA_TILE_ROWS, 128u));
    const size_t red_bytes = (size_t)2 * a.red_rows * a.nwarps * a.ngroups * (swiglu || two ? 2 : 1) * sizeof(float);
    a.xs_base = (uint32_t)((a.red_base + red_bytes + 127) / 128 * 128);
    const size_t xq_sb = !two ? MMA_XQ_SB : (c->x_bits == 24 ? mma_xq_sb<3, 2>() : mma_xq_sb<2, 2>());
    const size_t xq_bytes = (size_t)a.units * xq_sb + (size_t)a.units * 8 * (two ? 2 : 1) + 768;   // planes and sums, two scales per superblock and vector, a block of zeros
    a.stage_base = (uint32_t)((a.xs_base + xq_bytes + 127) / 128 * 128);
    const size_t budget = std::min<size_t>(228 * 1024 - 1024 - 256, (size_t)c->smem_optin - 256);
    if (budget < a.stage_base + a.stage_stride) return fail(OROME_ENOTSUP, "mma plan: in_dim %u does not fit shared memory", in_dim);
    const uint32_t tiles = ((share + MMA_TILE_ROWS - 1) / MMA_TILE_ROWS + 1) * a.nchunks;
    a.nstages = (uint32_t)std::min<size_t>(std::min<size_t>(PIPE_MAX_STAGES, tiles), (budget - a.stage_base) / a.stage_stride);
    p.smem = a.stage_base + (size_t)a.stage_stride * a.nstages;
#ifdef OROME_MMA_TILE_TRACE
    a.dbg_tile = OROME_MMA_TILE_TRACE;      // diagnostics build: first row tile whose per-warp timeline is recorded
#endif
    a.status = c->status_dev;
    a.trace = nullptr;
    if (c->trace_dev && c->trace_next < c->trace_cap) a.trace = c->trace_dev + (size_t)(c->trace_next++) * c->sm_count * 8;
    a.pf_ptr = c->hint_ptr;
    a.pf_bytes = c->hint_bytes;
    c->hint_ptr = nullptr;
    c->hint_bytes = 0;
    return arm_gather(c, a, in_dim);
}

// Tensor map of one K-quant tensor for the boxes above: {words of a superblock, superblocks of a row, rows}.
// Encoding costs the host about a microsecond, so maps are kept per (address, shape, box).
static int mma_tensor_map(orome_cuda_ctx *c, const uint8_t *w, uint32_t unit, uint32_t units, uint32_t rows, uint32_t kb, CUtensorMap *out)
{
    const MapKey key{w, unit, units, rows, kb};
    auto it = c->maps.find(key);
    if (it == c->maps.end()) {
        EncodeTiledFn enc = encode_tiled_fn();
        if (!enc) return fail(OROME_ECUDA, "mma plan: cuTensorMapEncodeTiled is not available");
        CUtensorMap m;
        const cuuint64_t dims[3] = {unit / 4, units, rows};
        const cuuint64_t strides[2] = {unit, (cuuint64_t)unit * units};
        const cuuint32_t box[3] = {unit / 4, kb, (cuuint32_t)MMA_TILE_ROWS}, estr[3] = {1, 1, 1};
        CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t *>(w), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(OROME_ECUDA, "mma plan: cuTensorMapEncodeTiled failed (%d)", (int)r);
        if (c->maps.size() >= 4096) c->maps.clear();
        it = c->maps.emplace(key, m).first;
    }
    *out = it->second;
    return OROME_OK;
}

static int mma_encode_maps(orome_cuda_ctx *c, int fmt, MmaPlan &p, bool swiglu)
{
    MmaArgs &a = p.args;
    if (fmt == FMT_Q6_K) return OROME_OK;        // no tensor map: 210-byte superblocks move by plain bulk copies
    const uint32_t unit = fmt == FMT_Q4_K ? 144u : 176u, kb = a.pitch / unit;
    for (int i = 0; i < a.nseg; ++i) {
        int rc = mma_tensor_map(c, a.seg[i].w, unit, a.units, a.seg[i].rows, kb, &a.map[i][0]);
        if (rc) return rc;
        if (swiglu) { rc = mma_tensor_map(c, a.seg[i].w2, unit, a.units, a.seg[i].rows, kb, &a.map[i][1]); if (rc) return rc; }
    }
    return OROME_OK;
}

template <int FMT, int NP, bool SWIGLU, bool EXT, int MOE = 0, int NTOK = 1>
static int launch_mma_ext(orome_cuda_ctx *c, const MmaPlan &p, cudaStream_t st)
{
    auto kern = gemv_mma_kernel<FMT, NP, SWIGLU, EXT, MOE, NTOK>;
    static size_t configured[64] = {0};   // per device: dynamic shared memory opted in so far
    if (configured[c->device] < p.smem) {
        cudaFuncAttributes fa;
        CU(cudaFuncGetAttributes(&fa, kern));
        const int max_dyn = c->smem_optin - (int)fa.sharedSizeBytes;
        if ((size_t)max_dyn < p.smem) return fail(OROME_ENOTSUP, "mma launch: %zu bytes of shared memory exceed the limit %d", p.smem, max_dyn);
        CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dyn));
        configured[c->device] = (size_t)max_dyn;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid, MOE != 0 ? p.tokens : 1);
    cfg.blockDim = dim3(p.threads);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->pdl ? 1 : 0;
    CU(cudaLaunchKernelEx(&cfg, kern, p.args));
    ++c->launches;
    return OROME_OK;
}

// Two input vectors in one pass over the weights (plain Q4_K / Q5_K): x at the context's width.
static int launch_mma_two(orome_cuda_ctx *c, int fmt, MmaPlan &p, cudaStream_t st)
{
    int rc = mma_encode_maps(c, fmt, p, false);
    if (rc) return rc;
    const bool b24 = c->x_bits == 24;
    if (fmt == FMT_Q4_K) return b24 ? launch_mma_ext<FMT_Q4_K, 3, false, false, 0, 2>(c, p, st) : launch_mma_ext<FMT_Q4_K, 2, false, false, 0, 2>(c, p, st);
    return b24 ? launch_mma_ext<FMT_Q5_K, 3, false, false, 0, 2>(c, p, st) : launch_mma_ext<FMT_Q5_K, 2, false, false, 0, 2>(c, p, st);
}

// The MoE forms of the mma kernel (Q4_K / Q5_K): fused gate/up over device-chosen experts, down + weighted combine.
static int launch_mma_moe(orome_cuda_ctx *c, int fmt, MmaPlan &p, bool gate_up, cudaStream_t st)
{
    const bool b24 = c->x_bits == 24;
    if (gate_up)      // the fused form always reads x at 24 bits
        return fmt == FMT_Q4_K ? launch_mma_ext<FMT_Q4_K, 3, true, false, 1>(c, p, st) : launch_mma_ext<FMT_Q5_K, 3, true, false, 1>(c, p, st);
    if (fmt == FMT_Q4_K) return b24 ? launch_mma_ext<FMT_Q4_K, 3, false, false, 2>(c, p, st) : launch_mma_ext<FMT_Q4_K, 2, false, false, 2>(c, p, st);
    return b24 ? launch_mma_ext<FMT_Q5_K, 3, false, false, 2>(c, p, st) : launch_mma_ext<FMT_Q5_K, 2, false, false, 2>(c, p, st);
}

template <int FMT, int NP, bool SWIGLU>
static int launch_mma_inst(orome_cuda_ctx *c, const MmaPlan &p, cudaStream_t st)
{
    return p.args.npeers > 0 || p.args.x_ll ? launch_mma_ext<FMT, NP, SWIGLU, true>(c, p, st) : launch_mma_ext<FMT, NP, SWIGLU, false>(c, p, st);
}

static int launch_mma(orome_cuda_ctx *c, int fmt, MmaPlan &p, bool swiglu, cudaStream_t st)
{
    int rc = mma_encode_maps(c, fmt, p, swiglu);
    if (rc) return rc;
    const bool b24 = c->x_bits == 24;
    // the fused form always reads x at 24 bits (see plan_pipe)
    if (fmt == FMT_Q4_K) {
        if (swiglu) return launch_mma_inst<FMT_Q4_K, 3, true>(c, p, st);
        return b24 ? launch_mma_inst<FMT_Q4_K, 3, false>(c, p, st) : launch_mma_inst<FMT_Q4_K, 2, false>(c, p, st);
    }
    if (fmt == FMT_Q6_K) return b24 ? launch_mma_inst<FMT_Q6_K, 3, false>(c, p, st) : launch_mma_inst<FMT_Q6_K, 2, false>(c, p, st);
    if (swiglu) return launch_mma_inst<FMT_Q5_K, 3, true>(c, p, st);
    return b24 ? launch_mma_inst<FMT_Q5_K, 3, false>(c, p, st) : launch_mma_inst<FMT_Q5_K, 2, false>(c, p, st);
}

extern "C" int orome_cuda_hint_next(orome_cuda_ctx *c, const OromeTensorRef *next)
{
    if (!c) return fail(OROME_EINVAL, "hint_next: NULL ctx");
    c->hint_ptr = nullptr;
    c->hint_bytes = 0;
    if (!next || !next->buffer || c->prefetch_mb <= 0) return OROME_OK;
    const int fmt = (int)next->format;
    if (fmt < 0 || fmt > FMT_F32) return OROME_OK;
    if (fmt <= FMT_Q8_0 && next->in_dim % block_elems(fmt)) return OROME_OK;
    const uint8_t *p = static_cast<const uint8_t *>(next->buffer) + next->offset;
    if (reinterpret_cast<uintptr_t>(p) & 15) return OROME_OK;
    const uint64_t total = (uint64_t)row_bytes_of(fmt, next->in_dim) * next->out_dim;
    c->hint_ptr = p;
    c->hint_bytes = std::min<uint64_t>(total, (uint64_t)c->prefetch_mb << 20) & ~(uint64_t)15;
    return OROME_OK;
}

// ---------------------------------------------------------------------------
// multi-GPU gather
// ---------------------------------------------------------------------------
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the ABI passes IPC handles as 64 bytes");

extern "C" size_t orome_cuda_gather_arena_bytes(size_t data_bytes, int n_flags)
{
    (void)n_flags;     // the generations live in local device memory, not in the arena
    return 3 * ((data_bytes + 255) / 256 * 256) + 256;   // the vectors as plain floats, then their {value, tag} slots
}

extern "C" int orome_cuda_peer_alloc(orome_cuda_ctx *c, size_t bytes, void **dev_ptr, unsigned char handle_out[64])
{
    if (!c || !dev_ptr || !handle_out || !bytes) return fail(OROME_EINVAL, "peer_alloc: bad argument");
    CU(cudaSetDevice(c->device));
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(OROME_ENOMEM, "peer_alloc: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    CU(cudaMemset(p, 0, bytes));
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return fail(OROME_ECUDA, "peer_alloc: cudaIpcGetMemHandle: %s", cudaGetErrorString(e)); }
    memcpy(handle_out, &h, 64);
    CU(cudaDeviceSynchronize());
    *dev_ptr = p;
    return OROME_OK;
}

extern "C" int orome_cuda_peer_open(orome_cuda_ctx *c, const unsigned char handle[64], void **dev_ptr)
{
    if (!c || !handle || !dev_ptr) return fail(OROME_EINVAL, "peer_open: NULL argument");
    CU(cudaSetDevice(c->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(OROME_ECUDA, "peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    *dev_ptr = p;
    return OROME_OK;
}

extern "C" int orome_cuda_peer_close(orome_cuda_ctx *c, void *dev_ptr)
{
    if (!c || !dev_ptr) return fail(OROME_EINVAL, "peer_close: NULL argument");
    CU(cudaSetDevice(c->device));
    CU(cudaIpcCloseMemHandle(dev_ptr));
    return OROME_OK;
}

extern "C" int orome_cuda_gather_setup(orome_cuda_ctx *c, int rank, int world, void *const *arenas, size_t data_bytes, int n_flags)
{
    if (!c) return fail(OROME_EINVAL, "gather_setup: NULL ctx");
    if (world == 1 || !arenas) {   // back to single-GPU behaviour
        c->g_world = 1; c->g_rank = 0; c->g_wait = c->g_publish = -1;
        return OROME_OK;
    }
    if (world < 2 || world > PIPE_MAX_PEERS + 1 || rank < 0 || rank >= world) return fail(OROME_EINVAL, "gather_setup: rank %d of %d (at most %d GPUs)", rank, world, PIPE_MAX_PEERS + 1);
    if (n_flags < 1 || n_flags > 64) return fail(OROME_EINVAL, "gather_setup: n_flags %d (1..64)", n_flags);
    if (data_bytes % 256) return fail(OROME_EINVAL, "gather_setup: data_bytes must be a multiple of 256");
    for (int r = 0; r < world; ++r)
        if (!arenas[r] || (reinterpret_cast<uintptr_t>(arenas[r]) & 255)) return fail(OROME_EINVAL, "gather_setup: arena %d is NULL or not 256-byte aligned", r);
    CU(cudaSetDevice(c->device));
    cudaFree(c->g_local);
    c->g_local = nullptr;
    CU(cudaMalloc(&c->g_local, (size_t)(n_flags + 2) * sizeof(unsigned int)));
    CU(cudaMemset(c->g_local, 0, (size_t)(n_flags + 2) * sizeof(unsigned int)));
    for (int r = 0; r < world; ++r) c->g_arena[r] = static_cast<uint8_t *>(arenas[r]);
    c->g_rank = rank; c->g_world = world; c->g_nflags = n_flags; c->g_data_bytes = data_bytes;
    c->g_wait = c->g_publish = -1;
    return OROME_OK;
}

extern "C" int orome_cuda_gather_next(orome_cuda_ctx *c, int wait_flag, int publish_flag)
{
    if (!c) return fail(OROME_EINVAL, "gather_next: NULL ctx");
    if (c->g_world < 2 || c->rec) { c->g_wait = c->g_publish = -1; return OROME_OK; }   // single GPU, or a chain (which orders its products by their addresses)
    if (wait_flag >= c->g_nflags || publish_flag >= c->g_nflags) return fail(OROME_EINVAL, "gather_next: flag out of range (%d flags)", c->g_nflags);
    c->g_wait = wait_flag < 0 ? -1 : wait_flag;
    c->g_publish = publish_flag < 0 ? -1 : publish_flag;
    return OROME_OK;
}

// Copies a gathered vector from its {value, tag} slots to its plain place in the arena, polling every element
// (bounded) for the generation this rank published last under the flag.
__global__ void __launch_bounds__(256) gather_unpack_kernel(const uint2 *slots, float *dst, uint32_t n4, const unsigned int *gen, int *status,
                                                            long long wait_cycles)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned int tag = *reinterpret_cast<const volatile unsigned int *>(gen);
    bool ok = *reinterpret_cast<const volatile int *>(status) == 0;      // an earlier expiry: copy what is there, wait for nothing
    const bool was_ok = ok;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x)
        reinterpret_cast<float4 *>(dst)[i] = ld_gathered4(slots + 4 * (size_t)i, tag, &ok, wait_cycles, status);
    if (!ok && was_ok) atomicExch(status, 3);
}

extern "C" int orome_cuda_gather_wait(orome_cuda_ctx *c, int flag, float *vec_dev, uint32_t n, void *stream)
{
    if (!c) return fail(OROME_EINVAL, "gather_wait: NULL ctx");
    if (c->g_world < 2) return OROME_OK;
    if (flag < 0 || flag >= c->g_nflags) return fail(OROME_EINVAL, "gather_wait: flag %d of %d", flag, c->g_nflags);
    uint8_t *mine = c->g_arena[c->g_rank], *v = reinterpret_cast<uint8_t *>(vec_dev);
    if (!vec_dev || n % 4 || v < mine || v + (size_t)n * 4 > mine + c->g_data_bytes || ((v - mine) & 15))
        return fail(OROME_EINVAL, "gather_wait: the vector must lie in the gather arena, 16-byte aligned, a multiple of 4 long");
    if (c->rec) return orome_chain_record_unpack(c, vec_dev, n);
    CU(cudaSetDevice(c->device));
    const uint2 *slots = reinterpret_cast<const uint2 *>(mine + c->g_data_bytes + 2 * (size_t)(v - mine));
    const unsigned blocks = std::max(1u, std::min((n / 4 + 255) / 256, (unsigned)c->sm_count));
    return launch_pdl(c, "gather_unpack", gather_unpack_kernel, dim3(blocks), dim3(256), static_cast<cudaStream_t>(stream), slots, vec_dev,
                      n / 4, (const unsigned int *)(c->g_local + flag), c->status_dev, orome_wait_cycles(c));
}

#ifdef OROME_DIAGNOSTICS
// Diagnostics builds only: the SM-cycle stamps CTA 0 of the last tensor-core launch left (8 kinds x 80 entries).
extern "C" int orome_cuda_tc_trace_read(long long *host)
{
    CU(cudaDeviceSynchronize());
    CU(cudaMemcpyFromSymbol(host, g_tc_trace, sizeof(long long) * 8 * 80));
    return OROME_OK;
}
#endif

// ---------------------------------------------------------------------------
// fused neighbours of a product
// ---------------------------------------------------------------------------
static_assert(OROME_SUM_SQ_PARTS == PIPE_SUM_SQ_PARTS, "the header and the kernel must agree on the partials array");

static void drop_fuse(orome_cuda_ctx *c)
{
    c->fuse_norm_w = nullptr; c->fuse_norm_parts = nullptr; c->fuse_res_in = nullptr; c->fuse_res_parts = nullptr;
}
static bool fuse_pending(const orome_cuda_ctx *c) { return c->fuse_norm_w || c->fuse_res_in; }
// A fuse request on a path without the fused form: dropped, with an error, like a gather request.
static int refuse_fuse(orome_cuda_ctx *c, const char *who)
{
    drop_fuse(c);
    c->g_wait = c->g_publish = -1;
    return fail(OROME_ENOTSUP, "%s: this call has no fused norm / residual form (the request was dropped)", who);
}

extern "C" int orome_cuda_fuse_next(orome_cuda_ctx *c, const OromeNormPrologue *pro, const OromeResidualEpilogue *epi)
{
    if (!c) return fail(OROME_EINVAL, "fuse_next: NULL ctx");
    drop_fuse(c);
    if (pro) {
        if (!pro->weight_bf16 || !pro->sum_sq_parts || (reinterpret_cast<uintptr_t>(pro->weight_bf16) & 7) || !(pro->eps >= 0.0f))
            return fail(OROME_EINVAL, "fuse_next: the prologue needs 8-byte aligned bf16 weights, a partials array and eps >= 0");
        c->fuse_norm_w = pro->weight_bf16;
        c->fuse_norm_parts = pro->sum_sq_parts;
        c->fuse_norm_eps = pro->eps;
    }
    if (epi) {
        if (!epi->residual || !epi->sum_sq_parts) { drop_fuse(c); return fail(OROME_EINVAL, "fuse_next: the epilogue needs a residual vector and a partials array"); }
        c->fuse_res_in = epi->residual;
        c->fuse_res_parts = epi->sum_sq_parts;
    }
    return OROME_OK;
}

// ---------------------------------------------------------------------------
// matvec entry points
// ---------------------------------------------------------------------------
extern "C" int orome_cuda_matvec_group(orome_cuda_ctx *c, const OromeTensorRef *refs, int n_refs, const float *x_dev,
                                       float *const *y_dev, void *stream)
{
    if (!c || !refs || !y_dev || n_refs < 1) return fail(OROME_EINVAL, "matvec_group: NULL or empty argument");
    if (n_refs > PIPE_MAX_SEG) return fail(OROME_EINVAL, "matvec_group: at most %d tensors per launch", PIPE_MAX_SEG);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CU(cudaSetDevice(c->device));
    const uint8_t *data[PIPE_MAX_SEG];
    for (int i = 0; i < n_refs; ++i) {
        if (!refs[i].buffer) return fail(OROME_EINVAL, "matvec_group: tensor %d is absent", i);
        int rc = orome_check_ref("matvec_group", &refs[i], &data[i]);
        if (rc) return rc;
        if (refs[i].format != refs[0].format || refs[i].variant != refs[0].variant || refs[i].in_dim != refs[0].in_dim)
            return fail(OROME_EINVAL, "matvec_group: tensors must share format, variant and in_dim");
        if (!y_dev[i]) return fail(OROME_EINVAL, "matvec_group: y_dev[%d] is NULL", i);
    }
    if (!x_dev || (reinterpret_cast<uintptr_t>(x_dev) & 15)) return fail(OROME_EINVAL, "matvec_group: x must be a 16-byte aligned device pointer");
    const int fmt = (int)refs[0].format, layout = (int)refs[0].variant;
    if (c->g_world > 1 && c->g_publish >= 0) {
        const uint8_t *lo = c->g_arena[c->g_rank], *hi = lo + c->g_data_bytes;
        for (int i = 0; i < n_refs; ++i) {
            const uint8_t *y0 = reinterpret_cast<const uint8_t *>(y_dev[i]);
            if (y0 < lo || y0 + (size_t)refs[i].out_dim * 4 > hi) { c->g_wait = c->g_publish = -1; return fail(OROME_EINVAL, "matvec_group: a published y must lie inside the gather arena"); }
        }
    }
    const bool fused = fuse_pending(c);
    if (fused && (c->rec || c->force_generic || !orome_pipe_supported(fmt, refs[0].in_dim) || (c->fuse_res_in && n_refs != 1) ||
                  (c->g_world > 1 && (c->g_publish >= 0 || c->g_wait >= 0))))
        return refuse_fuse(c, "matvec_group");
    if (c->rec) return orome_chain_record_group(c, refs, n_refs, x_dev, y_dev);
    if (c->force_generic || !orome_pipe_supported(fmt, refs[0].in_dim)) {
        if (c->g_world > 1 && (c->g_publish >= 0 || c->g_wait >= 0)) { c->g_wait = c->g_publish = -1; return fail(OROME_ENOTSUP, "matvec_group: this shape has no multi-GPU form"); }
        for (int i = 0; i < n_refs; ++i) {
            int rc = launch_generic(c, fmt, data[i], refs[i].out_dim, refs[i].in_dim, layout, x_dev, 1, 0, y_dev[i], 0, st);
            if (rc) return rc;
        }
        return OROME_OK;
    }
    bool aligned16 = true;
    for (int i = 0; i < n_refs; ++i) aligned16 = aligned16 && !(reinterpret_cast<uintptr_t>(data[i]) & 15);
    if (!fused && (aligned16 || fmt == FMT_Q6_K) && mma_supported(c, fmt, refs[0].in_dim, false)) {   // the fused forms live in the dp4a kernel
        MmaPlan m;
        memset(&m, 0, sizeof m);
        uint32_t rows = 0;
        for (int i = 0; i < n_refs; ++i) {
            m.args.seg[i] = PipeSeg{data[i], nullptr, y_dev[i], refs[i].out_dim, rows};
            rows += refs[i].out_dim;
        }
        m.args.nseg = n_refs;
        m.args.x = x_dev;
        m.args.layout = layout;
        int rc = plan_mma(c, fmt, refs[0].in_dim, rows, false, m);
        if (rc == OROME_OK) return launch_mma(c, fmt, m, false, st);
        if (rc != OROME_ENOTSUP) return rc;      // too wide for this kernel's shared memory: the dp4a kernel takes it
    }
    PipePlan p;
    memset(&p, 0, sizeof p);
    uint32_t total = 0;
    for (int i = 0; i < n_refs; ++i) {
        p.args.seg[i].w = data[i];
        p.args.seg[i].w2 = nullptr;
        p.args.seg[i].y = y_dev[i];
        p.args.seg[i].rows = refs[i].out_dim;
        p.args.seg[i].vstart = total;
        total += refs[i].out_dim;
    }
    p.args.nseg = n_refs;
    p.args.x = x_dev;
    p.args.layout = layout;
    int rc = plan_pipe(c, fmt, refs[0].in_dim, total, 0, p);
    if (rc) return rc;
    return launch_pipe(c, fmt, p, 0, st);
}

// ---------------------------------------------------------------------------
// batched form on the tensor cores
// ---------------------------------------------------------------------------
// Q6_K (rows only 2-byte aligned, no tensor map possible) exists in the tensor-memory form only.
static bool tc_supported(const orome_cuda_ctx *c, int fmt, uint32_t in_dim)
{
    if (in_dim % TC_KC != 0) return false;
    return fmt == FMT_Q8_0 || fmt == FMT_Q4_K || fmt == FMT_Q5_K || (fmt == FMT_Q6_K && !c->tc_slabs);
}

template <int FMT>
static int launch_tca_fmt(orome_cuda_ctx *c, const TcArgs &a, int grid, size_t smem, cudaStream_t st)
{
    auto kern = gemm_tca_kernel<FMT>;
    static bool configured[64] = {false};
    if (!configured[c->device]) {
        cudaFuncAttributes fa;
        CU(cudaFuncGetAttributes(&fa, kern));
        CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, c->smem_optin - (int)fa.sharedSizeBytes));
        configured[c->device] = true;
    }
    return launch_pdl_smem(c, "gemm_tca", kern, dim3(grid), dim3(TCA_THREADS), smem, st, a);
}

template <int FMT>
static int launch_tc_fmt(orome_cuda_ctx *c, const TcArgs &a, int grid, size_t smem, cudaStream_t st)
{
    auto kern = gemm_tc_kernel<FMT>;
    static bool configured[64] = {false};
    if (!configured[c->device]) {
        cudaFuncAttributes fa;
        CU(cudaFuncGetAttributes(&fa, kern));
        CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, c->smem_optin - (int)fa.sharedSizeBytes));
        configured[c->device] = true;
    }
    return launch_pdl_smem(c, "gemm_tc", kern, dim3(grid), dim3(TC_THREADS), smem, st, a);
}

static int ensure(float **p, size_t *cap, size_t floats);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Y[b][r] for b < batch (<= TC_MAX_N per launch; larger batches are cut into slices that each re-read the weights).
// pub / x_ll / wait_gen: the row-split form on several GPUs (batch <= TC_MAX_N, one launch): Y is published to every
// rank's arena by the kernel that writes it, a gathered X is read from its slots by the packing kernel.
static int launch_tc(orome_cuda_ctx *c, int fmt, const uint8_t *data, uint32_t out_dim, uint32_t in_dim, int layout, const float *x,
                     int batch, int ldx, float *y, int ldy, cudaStream_t st, const TcPub *pub = nullptr, const uint2 *x_ll = nullptr,
                     const unsigned int *wait_gen = nullptr)
{
    TcPub no_pub;
    memset(&no_pub, 0, sizeof no_pub);
    if (!pub) pub = &no_pub;
    const uint32_t chunk_bytes = fmt == FMT_Q8_0 ? 272u : fmt == FMT_Q4_K ? 144u : fmt == FMT_Q5_K ? 176u : 210u;
    const uint32_t chunks = in_dim / TC_KC, tiles = (out_dim + TC_M - 1) / TC_M;
    // Split K so that the SMs stay busy: a CTA costs about one time unit per chunk plus about five to set up (TMEM,
    // barriers, pipeline fill -- measured: three parts in two waves were slower than one part on 96 of 148 SMs), the
    // grid runs in waves of sm_count CTAs, a split adds a reduction pass.  Parts may be uneven.
    // Split K so that the SMs stay busy: a CTA costs about one time unit per chunk plus about five to set up (TMEM,
    // barriers, pipeline fill -- measured: three parts in two waves were slower than one part on 96 of 148 SMs), the
    // grid runs in waves of sm_count CTAs, a split adds a reduction pass.  Parts may be uneven.
    // Row tiles per CTA (tensor-memory form): one.  Two or four tiles sharing each X tile were measured slower at every
    // split (12288 x 4096, batch 64: 29 us with one tile, 37-48 us with two): the MMA issue, not the X traffic, is what a
    // CTA waits for.  OROME_OPT_TC_TILES keeps the choice open for experiments.
    uint32_t split = 1;
    const uint32_t tt = c->tc_slabs ? 1u : (c->tc_tiles ? std::min<uint32_t>((uint32_t)c->tc_tiles, tiles) : 1u);
    double best = 1e30;
    for (uint32_t s = c->tc_split ? (uint32_t)c->tc_split : 1u; s <= (c->tc_split ? (uint32_t)c->tc_split : 12u) && s <= chunks; ++s) {
        const uint32_t ctas = (tiles + tt - 1) / tt * s, waves = (ctas + c->sm_count - 1) / c->sm_count;
        const double cost = (double)waves * ((double)((chunks + s - 1) / s) * tt + 5.0) + (s > 1 ? 1.0 + 0.25 * s : 0.0);
        if (cost < best) { best = cost; split = s; }
    }
    for (int b0 = 0; b0 < batch; b0 += TC_MAX_N) {
        const int nb = std::min(batch - b0, TC_MAX_N);
        const uint32_t npad = (uint32_t)(nb + 15) / 16 * 16;
        int rc = ensure(&c->tc_xp, &c->tc_xp_cap, (size_t)in_dim * npad / 2 + 64);
        if (rc) return rc;
        if (split > 1) { rc = ensure(&c->tc_part, &c->tc_part_cap, (size_t)split * nb * out_dim); if (rc) return rc; }
        __half *xp = reinterpret_cast<__half *>(c->tc_xp);
        const size_t pieces = (size_t)(in_dim / TC_SLAB_K) * npad * 8;
        rc = launch_pdl(c, "pack_x_f16", pack_x_f16_kernel, dim3((unsigned)std::min<size_t>((pieces + 255) / 256, 1184)), dim3(256), st,
                        x + (size_t)b0 * ldx, nb, ldx, in_dim, npad, xp, x_ll, wait_gen, orome_wait_cycles(c), c->status_dev);
        if (rc) return rc;
        TcArgs a;
        memset(&a, 0, sizeof a);
        if (c->tc_slabs) {      // the staged form fetches its packed weights with tensor copies
            EncodeTiledFn enc = encode_tiled_fn();
            if (!enc) return fail(OROME_ECUDA, "gemm_tc: cuTensorMapEncodeTiled is not available");
            const cuuint64_t dims[2] = {(cuuint64_t)row_bytes_of(fmt, in_dim) / 4, out_dim};
            const cuuint64_t strides[1] = {(cuuint64_t)row_bytes_of(fmt, in_dim)};
            const cuuint32_t box[2] = {chunk_bytes / 4, (cuuint32_t)TC_M}, estr[2] = {1, 1};
            CUresult r = enc(&a.wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(data), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(OROME_ECUDA, "gemm_tc: cuTensorMapEncodeTiled failed (%d)", (int)r);
        }
        a.w = data; a.xp = xp; a.y = split == 1 ? y + (size_t)b0 * ldy : c->tc_part;
        a.rows = out_dim; a.in_dim = in_dim; a.row_bytes = (uint32_t)row_bytes_of(fmt, in_dim); a.chunk_bytes = chunk_bytes;
        a.batch = (uint32_t)nb; a.npad = npad; a.ldy = (uint32_t)ldy; a.split = split; a.chunks = chunks; a.tiles_per_cta = tt;
        a.layout = layout; a.status = c->status_dev;
        a.pub = *pub;
        // Shared memory: one chunk's worth of fp16 slab buffers, two X tile stages, two packed-weight stages (169 KB for
        // Q4_K at batch 64).  Measured on Q4_K 12288x4096, batch 64: deeper rings (seven slab buffers, a third X stage, up
        // to six packed-weight stages, sized at run time) made the launch slower (35-41 us against 34 us), and removing
        // the dequant arithmetic altogether only brings it to 31 us: ring depth is not what bounds this kernel, and
        // run-time ring sizes put integer divisions on the hand-off path of every slab.
        const size_t pk_stage = (TC_M * chunk_bytes + 127) & ~127u, b_tile = (size_t)npad * 128 * TC_SLABS;
        const int grid = (int)((tiles + tt - 1) / tt * split);
        if (!c->tc_slabs) {
            // dequantized weights in tensor memory: shared memory holds X tiles and packed stages only; at least half an
            // SM's worth is requested so that two CTAs (each wants all 512 columns of tensor memory) never share an SM
            size_t smem = 1024 + (size_t)TCA_B_STAGES * b_tile + 512;
            smem = std::max<size_t>(smem, 120 * 1024);
            if (smem > (size_t)c->smem_optin - 1024) return fail(OROME_ENOTSUP, "gemm_tca: batch %d does not fit shared memory", nb);
            switch (fmt) {
            case FMT_Q8_0: rc = launch_tca_fmt<FMT_Q8_0>(c, a, grid, smem, st); break;
            case FMT_Q4_K: rc = launch_tca_fmt<FMT_Q4_K>(c, a, grid, smem, st); break;
            case FMT_Q5_K: rc = launch_tca_fmt<FMT_Q5_K>(c, a, grid, smem, st); break;
            default: rc = launch_tca_fmt<FMT_Q6_K>(c, a, grid, smem, st); break;
            }
        } else {
            const size_t smem = 1024 + (size_t)TC_MAX_RING * 16384 + (size_t)TC_B_STAGES * b_tile + 512 + (size_t)tc_pk_stages(fmt) * pk_stage;
            if (smem > (size_t)c->smem_optin - 1024) return fail(OROME_ENOTSUP, "gemm_tc: batch %d does not fit shared memory", nb);
            switch (fmt) {
            case FMT_Q8_0: rc = launch_tc_fmt<FMT_Q8_0>(c, a, grid, smem, st); break;
            case FMT_Q4_K: rc = launch_tc_fmt<FMT_Q4_K>(c, a, grid, smem, st); break;
            default: rc = launch_tc_fmt<FMT_Q5_K>(c, a, grid, smem, st); break;
            }
        }
        if (rc) return rc;
        if (split > 1) {
            const size_t n = (size_t)nb * out_dim;
            rc = launch_pdl(c, "splitk_reduce", splitk_reduce_kernel, dim3((unsigned)std::min<size_t>((n + 255) / 256, 1184)), dim3(256), st,
                            (const float *)c->tc_part, split, (uint32_t)nb, out_dim, y + (size_t)b0 * ldy, (uint32_t)ldy, *pub);
            if (rc) return rc;
        }
    }
    return OROME_OK;
}

extern "C" int orome_cuda_matvec(orome_cuda_ctx *c, const OromeTensorRef *ref, const float *x_dev, float *y_dev, int batch,
                                 int ldx, int ldy, void *stream)
{
    if (!c || !ref) return fail(OROME_EINVAL, "matvec: NULL argument");
    if (!ref->buffer) return OROME_OK;   // absent optional tensor: silent no-op (format.m:247-250)
    if (batch < 1) return fail(OROME_EINVAL, "matvec: batch %d", batch);
    if (!x_dev || !y_dev) return fail(OROME_EINVAL, "matvec: NULL x or y");
    if (batch == 1 && (int)ref->format <= FMT_Q8_0) {
        float *ys[1] = {y_dev};
        return orome_cuda_matvec_group(c, ref, 1, x_dev, ys, stream);
    }
    if (fuse_pending(c)) return refuse_fuse(c, "matvec");
    if (c->rec) return fail(OROME_ENOTSUP, "matvec: only batch-1 products of quantized tensors can be recorded into a chain");
    if (batch > 1 && (ldx < (int)ref->in_dim || ldy < (int)ref->out_dim))
        return fail(OROME_EINVAL, "matvec: ldx/ldy smaller than the row length");
    const uint8_t *data;
    int rc = orome_check_ref("matvec", ref, &data);
    if (rc) { c->g_wait = c->g_publish = -1; return rc; }
    CU(cudaSetDevice(c->device));
    const bool x_ok = ldx % 4 == 0 && !(reinterpret_cast<uintptr_t>(x_dev) & 15);
    const bool tc_ok = batch >= c->tc_min_batch && !c->force_generic && tc_supported(c, (int)ref->format, ref->in_dim) && x_ok;
    if (c->g_world > 1 && (c->g_wait >= 0 || c->g_publish >= 0)) {
        // Row-split batched product: only the tensor-core form has a publish / wait path, and only as one launch.  Any
        // other call drops the request and says so, rather than leave it armed for an unrelated later launch.
        const int wait = c->g_wait, publish = c->g_publish;
        c->g_wait = c->g_publish = -1;
        if (!tc_ok || batch > TC_MAX_N)
            return fail(OROME_ENOTSUP, "matvec: this batch / format has no multi-GPU form (the gather request was dropped)");
        uint8_t *mine = c->g_arena[c->g_rank];
        const uint8_t *end = mine + c->g_data_bytes;
        TcPub pub;
        memset(&pub, 0, sizeof pub);
        pub.arena_base = mine;
        pub.ll_origin = mine + c->g_data_bytes;
        const uint2 *x_ll = nullptr;
        const unsigned int *wait_gen = nullptr;
        if (publish >= 0) {
            const uint8_t *y0 = reinterpret_cast<const uint8_t *>(y_dev);
            if (y0 < mine || y0 + ((size_t)(batch - 1) * ldy + ref->out_dim) * 4 > end)
                return fail(OROME_EINVAL, "matvec: a published Y must lie inside the gather arena");
            for (int r = 0; r < c->g_world; ++r)
                if (r != c->g_rank) pub.peer_delta[pub.npeers++] = (long long)(c->g_arena[r] - mine);
            pub.pub_gen = c->g_local + publish;
            pub.pub_arrived = c->g_local + c->g_nflags;
        }
        if (wait >= 0) {
            const uint8_t *xb = reinterpret_cast<const uint8_t *>(x_dev);
            if (xb < mine || xb + ((size_t)(batch - 1) * ldx + ref->in_dim) * 4 > end)
                return fail(OROME_EINVAL, "matvec: a launch that waits for a gathered X must read it from the gather arena");
            x_ll = reinterpret_cast<const uint2 *>(pub.ll_origin + 2 * (size_t)(xb - mine));
            wait_gen = c->g_local + wait;
        }
        return launch_tc(c, (int)ref->format, data, ref->out_dim, ref->in_dim, (int)ref->variant, x_dev, batch, ldx, y_dev, ldy,
                         static_cast<cudaStream_t>(stream), &pub, x_ll, wait_gen);
    }
    if (tc_ok)
        return launch_tc(c, (int)ref->format, data, ref->out_dim, ref->in_dim, (int)ref->variant, x_dev, batch, ldx, y_dev, ldy,
                         static_cast<cudaStream_t>(stream));
    // Small batches, and formats the tensor-core form does not take (Q6_K): one batch-1 launch per input vector.  The
    // weights are read once per vector, but the decode kernels run near the memory rate while the shape-agnostic
    // kernel below needs ~190 us per vector for a 12288 x 4096 tensor (measured: batch 8 in 1.5 ms).
    if (!c->force_generic && x_ok && (int)ref->format <= FMT_Q8_0 && c->g_world == 1 &&
        (orome_pipe_supported((int)ref->format, ref->in_dim) || mma_supported(c, (int)ref->format, ref->in_dim, false))) {
        // Q4_K / Q5_K: two vectors per launch in the mma kernel (the second one's byte planes ride in columns of the B
        // operand that a single vector leaves empty), so a batch of two or three reads the weights once or twice
        const int fmt = (int)ref->format;
        const bool pairs = (fmt == FMT_Q4_K || fmt == FMT_Q5_K) && mma_supported(c, fmt, ref->in_dim, false) && !(reinterpret_cast<uintptr_t>(data) & 15);
        int b = 0;
        for (; pairs && b + 1 < batch; b += 2) {
            MmaPlan m;
            memset(&m, 0, sizeof m);
            m.args.seg[0] = PipeSeg{data, nullptr, y_dev + (size_t)b * ldy, ref->out_dim, 0};
            m.args.nseg = 1;
            m.args.x = x_dev + (size_t)b * ldx;
            m.args.layout = (int)ref->variant;
            rc = plan_mma(c, fmt, ref->in_dim, ref->out_dim, false, m, 0, 0, true);
            if (rc == OROME_ENOTSUP) break;      // too wide for the two-vector layout: one vector per launch
            if (rc) return rc;
            m.args.tok_x_stride = (uint32_t)ldx;
            m.args.tok_y_stride = (uint32_t)ldy;
            rc = launch_mma_two(c, fmt, m, static_cast<cudaStream_t>(stream));
            if (rc) return rc;
        }
        for (; b < batch; ++b) {
            float *ys[1] = {y_dev + (size_t)b * ldy};
            rc = orome_cuda_matvec_group(c, ref, 1, x_dev + (size_t)b * ldx, ys, stream);
            if (rc) return rc;
        }
        return OROME_OK;
    }
    return launch_generic(c, (int)ref->format, data, ref->out_dim, ref->in_dim, (int)ref->variant, x_dev, batch, ldx, y_dev, ldy,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int orome_format_dispatch_matvec(orome_cuda_ctx *c, const OromeTensorRef *ref, const void *in_buf, size_t in_off,
                                            void *out_buf, size_t out_off, void *stream)
{
    if (!c || !ref) return fail(OROME_EINVAL, "format_dispatch_matvec: NULL argument");
    if (!ref->buffer) return OROME_OK;
    if (!in_buf || !out_buf) return fail(OROME_EINVAL, "format_dispatch_matvec: NULL buffer");
    if ((in_off | out_off) & 3) return fail(OROME_EINVAL, "format_dispatch_matvec: offsets must be multiples of 4");
    const float *x = reinterpret_cast<const float *>(static_cast<const uint8_t *>(in_buf) + in_off);
    float *y = reinterpret_cast<float *>(static_cast<uint8_t *>(out_buf) + out_off);
    return orome_cuda_matvec(c, ref, x, y, 1, 0, 0, stream);
}

static int ensure(float **p, size_t *cap, size_t floats)
{
    if (*cap >= floats) return OROME_OK;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    cudaError_t e = cudaMalloc(p, floats * sizeof(float));
    if (e != cudaSuccess) return fail(OROME_ENOMEM, "scratch of %zu floats: %s", floats, cudaGetErrorString(e));
    *cap = floats;
    return OROME_OK;
}

extern "C" int orome_cuda_gate_up_swiglu(orome_cuda_ctx *c, const OromeTensorRef *gate, const OromeTensorRef *up,
                                         const float *x_dev, float *out_dev, int batch, int ldx, int ldo, void *stream)
{
    if (!c || !gate || !up) return fail(OROME_EINVAL, "gate_up_swiglu: NULL argument");
    if (!gate->buffer || !up->buffer) return OROME_OK;
    if (batch < 1 || !x_dev || !out_dev) return fail(OROME_EINVAL, "gate_up_swiglu: bad x/out/batch");
    const uint8_t *gd, *ud;
    int rc = orome_check_ref("gate_up_swiglu(gate)", gate, &gd);
    if (rc) return rc;
    rc = orome_check_ref("gate_up_swiglu(up)", up, &ud);
    if (rc) return rc;
    if (gate->format != up->format || gate->variant != up->variant || gate->out_dim != up->out_dim || gate->in_dim != up->in_dim)
        return fail(OROME_EINVAL, "gate_up_swiglu: gate and up must have the same shape, format and variant");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CU(cudaSetDevice(c->device));
    const int fmt = (int)gate->format, layout = (int)gate->variant;
    if (c->g_world > 1 && c->g_publish >= 0) {
        const uint8_t *lo = c->g_arena[c->g_rank], *hi = lo + c->g_data_bytes, *y0 = reinterpret_cast<const uint8_t *>(out_dev);
        if (y0 < lo || y0 + (size_t)gate->out_dim * 4 > hi) { c->g_wait = c->g_publish = -1; return fail(OROME_EINVAL, "gate_up_swiglu: a published output must lie inside the gather arena"); }
    }
    const bool fused = fuse_pending(c);
    if (fused && (c->rec || c->fuse_res_in || batch != 1 || c->force_generic || !orome_pipe_supported(fmt, gate->in_dim) ||
                  (c->g_world > 1 && (c->g_publish >= 0 || c->g_wait >= 0))))
        return refuse_fuse(c, "gate_up_swiglu");
    if (c->rec) {
        if (batch != 1) return fail(OROME_ENOTSUP, "gate_up_swiglu: only batch-1 products can be recorded into a chain");
        return orome_chain_record_gate_up(c, gate, up, x_dev, out_dev);
    }
    if (c->g_world > 1 && (c->g_publish >= 0 || c->g_wait >= 0) && !(batch == 1 && !c->force_generic && orome_pipe_supported(fmt, gate->in_dim))) {
        c->g_wait = c->g_publish = -1;
        return fail(OROME_ENOTSUP, "gate_up_swiglu: this shape has no multi-GPU form");
    }
    if (batch == 1 && !c->force_generic && orome_pipe_supported(fmt, gate->in_dim)) {
        if (reinterpret_cast<uintptr_t>(x_dev) & 15) return fail(OROME_EINVAL, "gate_up_swiglu: x must be 16-byte aligned");
        if (!fused && !((reinterpret_cast<uintptr_t>(gd) | reinterpret_cast<uintptr_t>(ud)) & 15) && mma_supported(c, fmt, gate->in_dim, true)) {
            MmaPlan m;
            memset(&m, 0, sizeof m);
            m.args.seg[0] = PipeSeg{gd, ud, out_dev, gate->out_dim, 0};
            m.args.nseg = 1;
            m.args.x = x_dev;
            m.args.layout = layout;
            rc = plan_mma(c, fmt, gate->in_dim, gate->out_dim, true, m);
            if (rc == OROME_OK) return launch_mma(c, fmt, m, true, st);
            if (rc != OROME_ENOTSUP) return rc;
        }
        PipePlan p;
        memset(&p, 0, sizeof p);
        p.args.seg[0] = PipeSeg{gd, ud, out_dev, gate->out_dim, 0};
        p.args.nseg = 1;
        p.args.x = x_dev;
        p.args.layout = layout;
        rc = plan_pipe(c, fmt, gate->in_dim, gate->out_dim, 1, p);
        if (rc) return rc;
        return launch_pipe(c, fmt, p, 1, st);
    }
    // two matvecs into context scratch, then the elementwise epilogue (the reference's unfused branch, engine.m:388-404)
    if (batch > 1 && (ldx < (int)gate->in_dim || ldo < (int)gate->out_dim))
        return fail(OROME_EINVAL, "gate_up_swiglu: ldx/ldo smaller than the row length");
    const size_t n = (size_t)gate->out_dim;
    rc = ensure(&c->gu_dev, &c->gu_cap, 2 * n * batch);
    if (rc) return rc;
    float *g = c->gu_dev, *u = c->gu_dev + n * batch;
    if (batch > 1) {
        // the batched product's own dispatch: tensor cores from OROME_OPT_TC_MIN_BATCH vectors on, decode launches below
        rc = orome_cuda_matvec(c, gate, x_dev, g, batch, ldx, (int)n, stream);
        if (rc) return rc;
        rc = orome_cuda_matvec(c, up, x_dev, u, batch, ldx, (int)n, stream);
        if (rc) return rc;
    } else {
        rc = launch_generic(c, fmt, gd, gate->out_dim, gate->in_dim, layout, x_dev, batch, ldx, g, (int)n, st);
        if (rc) return rc;
        rc = launch_generic(c, fmt, ud, up->out_dim, up->in_dim, layout, x_dev, batch, ldx, u, (int)n, st);
        if (rc) return rc;
    }
    size_t tot = n * batch;
    swiglu_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(g, u, out_dev, (uint32_t)n, batch, (int)n, batch == 1 ? (int)n : ldo);
    return post_launch(c, "swiglu");
}

extern "C" int orome_cuda_dequant_rows(orome_cuda_ctx *c, const OromeTensorRef *ref, uint32_t row0, uint32_t nrows,
                                       float *out_dev, void *stream)
{
    if (!c || !ref || !out_dev) return fail(OROME_EINVAL, "dequant_rows: NULL argument");
    if (!ref->buffer) return fail(OROME_EINVAL, "dequant_rows: tensor is absent");   // the reference returns false (format.m:177)
    const uint8_t *data;
    int rc = orome_check_ref("dequant_rows", ref, &data);
    if (rc) return rc;
    if (row0 >= ref->out_dim || nrows > ref->out_dim - row0) return fail(OROME_EINVAL, "dequant_rows: rows [%u, %u) of %u", row0, row0 + nrows, ref->out_dim);
    if (nrows == 0) return OROME_OK;
    if (ref->in_dim % 32) return fail(OROME_EINVAL, "dequant_rows: in_dim %u is not a multiple of 32", ref->in_dim);
    if (reinterpret_cast<uintptr_t>(out_dev) & 15) return fail(OROME_EINVAL, "dequant_rows: out must be 16-byte aligned");
    CU(cudaSetDevice(c->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int fmt = (int)ref->format, layout = (int)ref->variant;
    size_t rb = row_bytes_of(fmt, ref->in_dim);
    size_t groups = (size_t)nrows * (ref->in_dim / 32);
    unsigned grid = (unsigned)((groups + 127) / 128);
#define DQ(F) dequant_rows_kernel<F><<<grid, 128, 0, st>>>(data, rb, row0, nrows, ref->in_dim, layout, out_dev)
    switch (fmt) {
    case FMT_Q4_K: DQ(FMT_Q4_K); break;
    case FMT_Q5_K: DQ(FMT_Q5_K); break;
    case FMT_Q6_K: DQ(FMT_Q6_K); break;
    case FMT_Q8_0: DQ(FMT_Q8_0); break;
    case FMT_F16: DQ(FMT_F16); break;
    case FMT_BF16: DQ(FMT_BF16); break;
    case FMT_F32: DQ(FMT_F32); break;
    }
#undef DQ
    return post_launch(c, "dequant_rows");
}

extern "C" int orome_cuda_argmax(orome_cuda_ctx *c, const float *data_dev, uint32_t count, uint32_t *result_dev, void *stream)
{
    if (!c || !data_dev || !result_dev || count == 0) return fail(OROME_EINVAL, "argmax: NULL or empty argument");
    if (c->rec) return orome_chain_record_argmax(c, data_dev, count, result_dev);
    CU(cudaSetDevice(c->device));
    const unsigned blocks = std::max(1u, std::min((count + 1023) / 1024, (unsigned)c->sm_count));
    // reduction state: two 64-bit words of the context's status block (128 bytes in), left zero by every call
    unsigned long long *state = reinterpret_cast<unsigned long long *>(c->status_dev) + 16;
    return launch_pdl(c, "argmax", argmax_kernel, dim3(blocks), dim3(256), static_cast<cudaStream_t>(stream), data_dev, count, result_dev, state);
}

// ---------------------------------------------------------------------------
// MoE
// ---------------------------------------------------------------------------
extern "C" int orome_cuda_moe_route(orome_cuda_ctx *c, const OromeTensorRef *router, const float *x_dev, int n_tokens, int ldx,
                                    uint32_t K, uint32_t *idx_dev, float *w_dev, float *logits_dev, void *stream)
{
    if (!c || !router || !x_dev || !idx_dev || !w_dev) return fail(OROME_EINVAL, "moe_route: NULL argument");
    if (!router->buffer) return fail(OROME_EINVAL, "moe_route: router tensor is absent");
    const uint8_t *data;
    int rc = orome_check_ref("moe_route", router, &data);
    if (rc) return rc;
    if (router->format != OROME_QFMT_F32) return fail(OROME_ENOTSUP, "moe_route: the router must be an F32 tensor");
    if (router->out_dim > 256) return fail(OROME_EINVAL, "moe_route: %u experts (the routing kernel takes at most 256)", router->out_dim);
    if (n_tokens < 1 || (n_tokens > 1 && ldx < (int)router->in_dim)) return fail(OROME_EINVAL, "moe_route: bad n_tokens/ldx");
    if (K < 1) return fail(OROME_EINVAL, "moe_route: K must be at least 1");
    CU(cudaSetDevice(c->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t ne = router->out_dim;
    if (!logits_dev) {
        rc = ensure(&c->logits_dev, &c->logits_cap, (size_t)ne * n_tokens);
        if (rc) return rc;
        logits_dev = c->logits_dev;
    }
    return launch_router(c, data, ne, router->in_dim, x_dev, n_tokens, ldx, logits_dev, K, idx_dev, w_dev, st);
}

extern "C" int orome_cuda_moe_route_pair(orome_cuda_ctx *c, const OromeTensorRef *router, const OromeTensorRef *shared_gate,
                                         const float *x_dev, int n_tokens, int ldx, uint32_t K, uint32_t *idx_dev, float *w_dev,
                                         float *shared_logit_dev, float *logits_dev, void *stream)
{
    if (!c || !router || !shared_gate || !x_dev || !idx_dev || !w_dev || !shared_logit_dev) return fail(OROME_EINVAL, "moe_route_pair: NULL argument");
    if (!router->buffer) return fail(OROME_EINVAL, "moe_route_pair: router tensor is absent");
    const uint8_t *data, *sg = nullptr;
    int rc = orome_check_ref("moe_route_pair", router, &data);
    if (rc) return rc;
    if (router->format != OROME_QFMT_F32) return fail(OROME_ENOTSUP, "moe_route_pair: the router must be an F32 tensor");
    if (router->out_dim > 255) return fail(OROME_EINVAL, "moe_route_pair: %u experts (at most 255 beside the gate row)", router->out_dim);
    if (n_tokens < 1 || (n_tokens > 1 && ldx < (int)router->in_dim)) return fail(OROME_EINVAL, "moe_route_pair: bad n_tokens/ldx");
    if (K < 1) return fail(OROME_EINVAL, "moe_route_pair: K must be at least 1");
    CU(cudaSetDevice(c->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t ne = router->out_dim;
    if (shared_gate->buffer) {
        rc = orome_check_ref("moe_route_pair(shared gate)", shared_gate, &sg);
        if (rc) return rc;
        // the reference fuses the two only for this shape (engine.m:660-666); anything else is not a shared-expert gate
        if (shared_gate->format != OROME_QFMT_F32 || shared_gate->out_dim != 1 || shared_gate->in_dim != router->in_dim)
            return fail(OROME_EINVAL, "moe_route_pair: the shared-expert gate must be an F32 tensor [1][%u]", router->in_dim);
    } else {
        CU(cudaMemsetAsync(shared_logit_dev, 0, (size_t)n_tokens * sizeof(float), st));      // absent gate: logit 0
    }
    if (!logits_dev) {
        rc = ensure(&c->logits_dev, &c->logits_cap, (size_t)(ne + 1) * n_tokens);
        if (rc) return rc;
        logits_dev = c->logits_dev;
    }
    return launch_router(c, data, ne, router->in_dim, x_dev, n_tokens, ldx, logits_dev, K, idx_dev, w_dev, st, sg, shared_logit_dev);
}

// ---------------------------------------------------------------------------
// routing without any allocation
// ---------------------------------------------------------------------------
// Scratch for the router logits of orome_cuda_moe_route_static.  The array lives in the library image: every
// device that loads the library holds its 64 KiB until the process exits.  In host code this name is only a
// stand-in for the symbol, not a device address; the address a kernel may use comes from cudaGetSymbolAddress,
// looked up once per device with that device current.
static __device__ __align__(256) float g_route_logits_static[OROME_ROUTE_STATIC_MAX_LOGITS];
static float *g_route_logits_addr[64];   // per device ordinal, filled on first use

extern "C" int orome_cuda_moe_route_static(orome_cuda_ctx *c, const OromeTensorRef *router, const float *x_dev, int n_tokens,
                                           int ldx, uint32_t K, uint32_t *idx_dev, float *w_dev, void *stream)
{
    if (!c || !router || !x_dev || !idx_dev || !w_dev) return fail(OROME_EINVAL, "moe_route_static: NULL argument");
    if (!router->buffer) return fail(OROME_EINVAL, "moe_route_static: router tensor is absent");
    const uint8_t *data;
    int rc = orome_check_ref("moe_route_static", router, &data);
    if (rc) return rc;
    if (router->format != OROME_QFMT_F32) return fail(OROME_ENOTSUP, "moe_route_static: the router must be an F32 tensor");
    if (router->out_dim > 256) return fail(OROME_EINVAL, "moe_route_static: %u experts (the routing kernel takes at most 256)", router->out_dim);
    if (n_tokens < 1 || (n_tokens > 1 && ldx < (int)router->in_dim)) return fail(OROME_EINVAL, "moe_route_static: bad n_tokens/ldx");
    if (K < 1) return fail(OROME_EINVAL, "moe_route_static: K must be at least 1");
    const uint32_t ne = router->out_dim;
    if ((size_t)n_tokens * ne > (size_t)OROME_ROUTE_STATIC_MAX_LOGITS)
        return fail(OROME_EINVAL, "moe_route_static: %d tokens x %u experts = %zu logits exceed the fixed scratch of %d floats; "
                    "use orome_cuda_moe_route with a caller buffer", n_tokens, ne, (size_t)n_tokens * ne, OROME_ROUTE_STATIC_MAX_LOGITS);
    if (c->device < 0 || c->device >= 64) return fail(OROME_EINVAL, "moe_route_static: device ordinal %d out of range", c->device);
    CU(cudaSetDevice(c->device));
    if (!g_route_logits_addr[c->device]) {   // set-up: once per device, with that device current
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_route_logits_static);
        if (e != cudaSuccess || !p) return fail(OROME_ECUDA, "moe_route_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_route_logits_addr[c->device] = static_cast<float *>(p);
    }
    float *logits = g_route_logits_addr[c->device];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return launch_router(c, data, ne, router->in_dim, x_dev, n_tokens, ldx, logits, K, idx_dev, w_dev, st);
}

// Set by orome_cuda_moe_ffn_shard around its call: the index list may hold "no expert here" entries, which only the
// dp4a kernel steps over.
static thread_local bool g_moe_may_skip = false;
// Row extent given to the tensor map of an expert stack (the number of experts is not part of an ExpertLayerRef; row
// tiles never leave an expert's rows, so the extent only has to cover every expert).
constexpr uint32_t MOE_STACK_ROWS = 1u << 24;

extern "C" int orome_cuda_moe_ffn(orome_cuda_ctx *c, const OromeExpertLayerRef *L, uint32_t variant, const float *x_dev,
                                  int n_tokens, int ldx, const uint32_t *idx_dev, const float *w_dev, uint32_t K, uint32_t hidden,
                                  uint32_t inter, float *act_dev, float *out_dev, int ldo, void *stream)
{
    if (!c || !L || !x_dev || !idx_dev || !w_dev || !act_dev || !out_dev) return fail(OROME_EINVAL, "moe_ffn: NULL argument");
    if (fuse_pending(c)) return refuse_fuse(c, "moe_ffn");
    if (!L->buffer) return OROME_OK;
    if (K < 1 || K > 8) return fail(OROME_EINVAL, "moe_ffn: K = %u (1..8; the reference's routing caps K at 8)", K);
    if (variant > OROME_VARIANT_LLAMA) return fail(OROME_ENOTSUP, "moe_ffn: unknown kernel variant %u", variant);
    if (n_tokens < 1 || (n_tokens > 1 && (ldx < (int)hidden || ldo < (int)hidden))) return fail(OROME_EINVAL, "moe_ffn: bad n_tokens/ldx/ldo");
    if (L->gate.format != L->up.format) return fail(OROME_ENOTSUP, "moe_ffn: gate and up must share a format");
    const int gfmt = (int)L->gate.format, dfmt = (int)L->down.format;
    if (gfmt < 0 || gfmt > FMT_Q8_0 || dfmt < 0 || dfmt > FMT_Q8_0) return fail(OROME_ENOTSUP, "moe_ffn: expert tensors must be quantized (Q4_K/Q5_K/Q6_K/Q8_0)");
    if (hidden % block_elems(gfmt) || inter % block_elems(dfmt)) return fail(OROME_EINVAL, "moe_ffn: hidden/inter not a whole number of blocks");
    const uint8_t *base = static_cast<const uint8_t *>(L->buffer);
    const uint8_t *gate = base + L->gate.offset, *up = base + L->up.offset, *down = base + L->down.offset;
    if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(down) | L->gate.expert_stride |
         L->up.expert_stride | L->down.expert_stride) & 15)
        return fail(OROME_EINVAL, "moe_ffn: expert tensors and strides must be 16-byte aligned");
    CU(cudaSetDevice(c->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t grb = row_bytes_of(gfmt, hidden), drb = row_bytes_of(dfmt, inter);
    // Q4_K / Q5_K experts stacked without gaps: the mma kernel's MoE forms (the indices must all be real experts).
    auto mma_moe_ok = [&](int fmt, uint32_t in_dim, uint32_t rows, size_t stride, size_t rb) {
        return c->kquant_mma && !c->force_generic && !g_moe_may_skip && (fmt == FMT_Q4_K || fmt == FMT_Q5_K) && in_dim % 256 == 0 &&
               rows % MMA_TILE_ROWS == 0 && stride == (size_t)rows * rb;
    };
    const uint32_t moe_grid_cap = n_tokens == 1 ? (uint32_t)c->sm_count : std::max(1u, 2u * (uint32_t)c->sm_count / (uint32_t)n_tokens);
    const bool x_ok16 = !((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(act_dev)) & 15) && (ldx % 4 == 0 || n_tokens == 1);
    const size_t out_ld_m = n_tokens == 1 ? hidden : (size_t)ldo;
    const bool sizes_ok = (size_t)n_tokens * K * inter <= 0xFFFFFFFFull && out_ld_m * (size_t)n_tokens <= 0xFFFFFFFFull;
    bool gate_up_done = false;
    if (x_ok16 && sizes_ok && mma_moe_ok(gfmt, hidden, inter, L->gate.expert_stride, grb) && L->up.expert_stride == L->gate.expert_stride) {
        MmaPlan m;
        memset(&m, 0, sizeof m);
        for (uint32_t k = 0; k < K; ++k) m.args.seg[k] = PipeSeg{gate, up, act_dev + (size_t)k * inter, inter, k * inter};
        m.args.nseg = (int)K;
        m.args.x = x_dev;
        m.args.layout = (int)variant;
        int rc = plan_mma(c, gfmt, hidden, K * inter, true, m, 0, moe_grid_cap);
        if (rc == OROME_OK) {
            const uint32_t unit = gfmt == FMT_Q4_K ? 144u : 176u, kb = m.args.pitch / unit;
            rc = mma_tensor_map(c, gate, unit, hidden / 256, MOE_STACK_ROWS, kb, &m.args.map[0][0]);
            if (rc == OROME_OK) rc = mma_tensor_map(c, up, unit, hidden / 256, MOE_STACK_ROWS, kb, &m.args.map[0][1]);
            if (rc) return rc;
            m.args.seg_expert = idx_dev;
            m.args.expert_rows = inter;
            m.args.tok_x_stride = n_tokens == 1 ? 0u : (uint32_t)ldx;
            m.args.tok_y_stride = K * inter;
            m.args.tok_sel_stride = 8;
            m.tokens = n_tokens;
            rc = launch_mma_moe(c, gfmt, m, true, st);
            if (rc) return rc;
            gate_up_done = true;
        } else if (rc != OROME_ENOTSUP) return rc;
    }
    auto down_mma = [&]() -> int {      // OROME_ENOTSUP: not this form
        if (!(x_ok16 && sizes_ok && mma_moe_ok(dfmt, inter, hidden, L->down.expert_stride, drb))) return OROME_ENOTSUP;
        MmaPlan m;
        memset(&m, 0, sizeof m);
        m.args.seg[0] = PipeSeg{down, nullptr, out_dev, hidden, 0};
        m.args.nseg = 1;
        m.args.x = act_dev;
        m.args.layout = (int)variant;
        int rc = plan_mma(c, dfmt, inter, hidden, false, m, K, moe_grid_cap);
        if (rc) return rc;
        const uint32_t unit = dfmt == FMT_Q4_K ? 144u : 176u, kb = m.args.pitch / unit;
        rc = mma_tensor_map(c, down, unit, inter / 256, MOE_STACK_ROWS, kb, &m.args.map[0][0]);
        if (rc) return rc;
        m.args.seg_expert = idx_dev;
        m.args.seg_weight = w_dev;
        m.args.expert_rows = hidden;
        m.args.tok_x_stride = K * inter;
        m.args.tok_y_stride = (uint32_t)out_ld_m;
        m.args.tok_sel_stride = 8;
        m.tokens = n_tokens;
        return launch_mma_moe(c, dfmt, m, false, st);
    };
    if (gate_up_done) {
        const int rc = down_mma();
        if (rc != OROME_ENOTSUP) return rc;
    }
    if (!c->force_generic && orome_pipe_supported(gfmt, hidden) && orome_pipe_supported(dfmt, inter) && K <= (uint32_t)PIPE_MAX_SEG &&
        !((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(act_dev)) & 15) && (ldx % 4 == 0 || n_tokens == 1) && inter % 4 == 0) {
        // One fused gate/up launch over the K selected experts of every token (device-side expert indices; grid.y =
        // token), then one down launch that gives every (token, expert) its own input vector and adds a token's K
        // results with its routing weights.
        const size_t out_ld = n_tokens == 1 ? hidden : (size_t)ldo;
        if ((size_t)n_tokens * K * inter > 0xFFFFFFFFull || out_ld * (size_t)n_tokens > 0xFFFFFFFFull)
            return fail(OROME_EINVAL, "moe_ffn: token batch too large");
        PipePlan p;
        int rc;
        if (!gate_up_done) {
            memset(&p, 0, sizeof p);
            for (uint32_t k = 0; k < K; ++k)
                p.args.seg[k] = PipeSeg{gate, up, act_dev + (size_t)k * inter, inter, k * inter};
            p.args.nseg = (int)K;
            p.args.x = x_dev;
            p.args.layout = (int)variant;
            p.tokens = n_tokens;
            rc = plan_pipe(c, gfmt, hidden, K * inter, 1, p);
            if (rc) return rc;
            p.args.seg_expert = idx_dev;
            p.args.w_stride = L->gate.expert_stride;
            p.args.w2_stride = L->up.expert_stride;
            p.args.tok_x_stride = n_tokens == 1 ? 0u : (uint32_t)ldx;
            p.args.tok_y_stride = K * inter;
            p.args.tok_sel_stride = 8;
            rc = launch_pipe(c, gfmt, p, 1, st);
            if (rc) return rc;
            rc = down_mma();
            if (rc != OROME_ENOTSUP) return rc;
        }

        memset(&p, 0, sizeof p);
        for (uint32_t k = 0; k < K; ++k) p.args.seg[k] = PipeSeg{down, nullptr, out_dev, hidden, 0};
        p.args.nseg = (int)K;
        p.args.x = act_dev;
        p.args.layout = (int)variant;
        p.tokens = n_tokens;
        rc = plan_pipe(c, dfmt, inter, hidden, 2, p);
        if (rc) return rc;
        p.args.seg_expert = idx_dev;
        p.args.w_stride = L->down.expert_stride;
        p.args.x_stride = inter;
        p.args.seg_weight = w_dev;
        p.args.tok_x_stride = K * inter;
        p.args.tok_y_stride = (uint32_t)out_ld;
        p.args.tok_sel_stride = 8;
        return launch_pipe(c, dfmt, p, 2, st);
    }
    dim3 g1((inter + 7) / 8, (unsigned)n_tokens * K), g2((hidden + 7) / 8, (unsigned)n_tokens);
#define GU(F) moe_gate_up_kernel<F><<<g1, 256, 0, st>>>(gate, L->gate.expert_stride, up, L->up.expert_stride, grb, inter, hidden, (int)variant, x_dev, ldx, idx_dev, K, act_dev)
    switch (gfmt) {
    case FMT_Q4_K: GU(FMT_Q4_K); break;
    case FMT_Q5_K: GU(FMT_Q5_K); break;
    case FMT_Q6_K: GU(FMT_Q6_K); break;
    case FMT_Q8_0: GU(FMT_Q8_0); break;
    }
#undef GU
    int rc = post_launch(c, "moe_gate_up");
    if (rc) return rc;
#define DN(F) moe_down_kernel<F><<<g2, 256, 0, st>>>(down, L->down.expert_stride, drb, hidden, inter, (int)variant, act_dev, idx_dev, w_dev, K, out_dev, n_tokens == 1 ? (int)hidden : ldo)
    switch (dfmt) {
    case FMT_Q4_K: DN(FMT_Q4_K); break;
    case FMT_Q5_K: DN(FMT_Q5_K); break;
    case FMT_Q6_K: DN(FMT_Q6_K); break;
    case FMT_Q8_0: DN(FMT_Q8_0); break;
    }
#undef DN
    return post_launch(c, "moe_down");
}

extern "C" int orome_cuda_moe_block(orome_cuda_ctx *c, const OromeExpertLayerRef *L, uint32_t variant, const OromeTensorRef *shared_gate_proj,
                                    const OromeTensorRef *shared_up_proj, const OromeTensorRef *shared_down_proj, const float *x_dev,
                                    int n_tokens, int ldx, const uint32_t *idx_dev, const float *w_dev, const float *shared_logit_dev,
                                    uint32_t K, uint32_t hidden, uint32_t inter, const float *h_mid_dev, int ld_mid, float *scratch_dev,
                                    float *out_dev, int ldo, void *stream)
{
    if (!c || !L || !x_dev || !idx_dev || !w_dev || !scratch_dev || !out_dev) return fail(OROME_EINVAL, "moe_block: NULL argument");
    if (fuse_pending(c)) return refuse_fuse(c, "moe_block");
    if (n_tokens < 1 || (n_tokens > 1 && (ldx < (int)hidden || ldo < (int)hidden))) return fail(OROME_EINVAL, "moe_block: bad n_tokens/ldx/ldo");
    if (h_mid_dev && n_tokens > 1 && ld_mid < (int)hidden) return fail(OROME_EINVAL, "moe_block: bad ld_mid");
    const bool shared = shared_gate_proj && shared_up_proj && shared_down_proj && shared_gate_proj->buffer && shared_up_proj->buffer &&
                        shared_down_proj->buffer;
    uint32_t S = 0;
    if (shared) {
        S = shared_gate_proj->out_dim;
        if (!shared_logit_dev) return fail(OROME_EINVAL, "moe_block: a shared expert needs its gate logit (orome_cuda_moe_route_pair)");
        if (shared_gate_proj->in_dim != hidden || shared_up_proj->in_dim != hidden || shared_up_proj->out_dim != S ||
            shared_down_proj->in_dim != S || shared_down_proj->out_dim != hidden)
            return fail(OROME_EINVAL, "moe_block: shared expert shapes must be [S][hidden], [S][hidden], [hidden][S]");
    }
    // scratch: routed activations [T][K][inter], weighted expert sum [T][hidden], shared activations [T][S], shared output [T][hidden]
    const size_t T = (size_t)n_tokens;
    float *act = scratch_dev, *moe = act + T * K * inter, *sact = moe + T * hidden, *sout = sact + T * S;
    if (reinterpret_cast<uintptr_t>(scratch_dev) & 15 || (K * inter) % 4 || hidden % 4 || S % 4)
        return fail(OROME_EINVAL, "moe_block: scratch must be 16-byte aligned and the dimensions multiples of 4");
    int rc = orome_cuda_moe_ffn(c, L, variant, x_dev, n_tokens, ldx, idx_dev, w_dev, K, hidden, inter, act, moe, (int)hidden, stream);
    if (rc) return rc;
    if (!L->buffer) {       // no routed experts in this layer: their sum is zero
        CU(cudaMemsetAsync(moe, 0, T * hidden * sizeof(float), static_cast<cudaStream_t>(stream)));
    }
    if (shared) {
        // the shared expert is independent of the routing result (engine.m:261-283): fused gate/up, then its down projection
        rc = orome_cuda_gate_up_swiglu(c, shared_gate_proj, shared_up_proj, x_dev, sact, n_tokens, ldx, (int)S, stream);
        if (rc) return rc;
        rc = orome_cuda_matvec(c, shared_down_proj, sact, sout, n_tokens, (int)S, (int)hidden, stream);
        if (rc) return rc;
    }
    CU(cudaSetDevice(c->device));
    return launch_pdl(c, "moe_combine", moe_combine_kernel, dim3((hidden + 255) / 256, (unsigned)n_tokens), dim3(256), static_cast<cudaStream_t>(stream),
                      h_mid_dev, n_tokens == 1 ? (int)hidden : ld_mid, (const float *)moe, (int)hidden, shared ? (const float *)sout : (const float *)nullptr,
                      (int)hidden, shared_logit_dev, hidden, out_dev, n_tokens == 1 ? (int)hidden : ldo);
}

extern "C" size_t orome_cuda_moe_block_scratch_floats(int n_tokens, uint32_t K, uint32_t hidden, uint32_t inter, uint32_t shared_inter)
{
    return (size_t)n_tokens * ((size_t)K * inter + 2 * (size_t)hidden + shared_inter);
}

extern "C" int orome_cuda_moe_ffn_shard(orome_cuda_ctx *c, const OromeExpertLayerRef *L_local, uint32_t variant, const float *x_dev,
                                        int n_tokens, int ldx, const uint32_t *idx_dev, const float *w_dev, uint32_t K, uint32_t hidden,
                                        uint32_t inter, uint32_t first_expert, uint32_t n_local, uint32_t *idx_local_dev, float *act_dev,
                                        float *out_dev, int ldo, void *stream)
{
    if (!c || !idx_dev || !idx_local_dev) return fail(OROME_EINVAL, "moe_ffn_shard: NULL argument");
    if (fuse_pending(c)) return refuse_fuse(c, "moe_ffn_shard");
    if (n_tokens < 1) return fail(OROME_EINVAL, "moe_ffn_shard: n_tokens %d", n_tokens);
    if (L_local && !L_local->buffer) {      // this GPU holds no expert of the layer: its share of the sum is zero
        CU(cudaSetDevice(c->device));
        for (int t = 0; t < n_tokens; ++t)
            CU(cudaMemsetAsync(out_dev + (size_t)t * (n_tokens == 1 ? hidden : ldo), 0, (size_t)hidden * 4, static_cast<cudaStream_t>(stream)));
        return OROME_OK;
    }
    CU(cudaSetDevice(c->device));
    const uint32_t n = (uint32_t)n_tokens * 8;
    int rc = launch_pdl(c, "moe_localize", moe_localize_kernel, dim3((n + 127) / 128), dim3(128), static_cast<cudaStream_t>(stream), idx_dev, n,
                        first_expert, n_local, idx_local_dev);
    if (rc) return rc;
    g_moe_may_skip = true;
    rc = orome_cuda_moe_ffn(c, L_local, variant, x_dev, n_tokens, ldx, idx_local_dev, w_dev, K, hidden, inter, act_dev, out_dev, ldo, stream);
    g_moe_may_skip = false;
    return rc;
}

// ---------------------------------------------------------------------------
// host-buffer form
// ---------------------------------------------------------------------------
extern "C" int orome_cuda_matvec_host(orome_cuda_ctx *c, const OromeTensorRef *ref, const float *x_host, float *y_host, int batch)
{
    if (!c || !ref || !x_host || !y_host) return fail(OROME_EINVAL, "matvec_host: NULL argument");
    if (!ref->buffer) return OROME_OK;
    if (batch < 1) return fail(OROME_EINVAL, "matvec_host: batch %d", batch);
    CU(cudaSetDevice(c->device));
    const size_t nx = (size_t)ref->in_dim * batch, ny = (size_t)ref->out_dim * batch;
    if (c->stage_x_cap < nx) {
        cudaFreeHost(c->stage_x_host); cudaFree(c->stage_x_dev);
        c->stage_x_host = c->stage_x_dev = nullptr; c->stage_x_cap = 0;
        CU(cudaMallocHost(&c->stage_x_host, nx * sizeof(float)));
        CU(cudaMalloc(&c->stage_x_dev, nx * sizeof(float)));
        c->stage_x_cap = nx;
    }
    if (c->stage_y_cap < ny) {
        cudaFreeHost(c->stage_y_host); cudaFree(c->stage_y_dev);
        c->stage_y_host = c->stage_y_dev = nullptr; c->stage_y_cap = 0;
        CU(cudaMallocHost(&c->stage_y_host, ny * sizeof(float)));
        CU(cudaMalloc(&c->stage_y_dev, ny * sizeof(float)));
        c->stage_y_cap = ny;
    }
    memcpy(c->stage_x_host, x_host, nx * sizeof(float));
    CU(cudaMemcpyAsync(c->stage_x_dev, c->stage_x_host, nx * sizeof(float), cudaMemcpyHostToDevice, c->own_stream));
    int rc = orome_cuda_matvec(c, ref, c->stage_x_dev, c->stage_y_dev, batch, (int)ref->in_dim, (int)ref->out_dim, c->own_stream);
    if (rc) return rc;
    CU(cudaMemcpyAsync(c->stage_y_host, c->stage_y_dev, ny * sizeof(float), cudaMemcpyDeviceToHost, c->own_stream));
    CU(cudaStreamSynchronize(c->own_stream));
    memcpy(y_host, c->stage_y_host, ny * sizeof(float));
    return OROME_OK;
}
