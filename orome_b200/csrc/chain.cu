// chain.cu -- recording a token step's products and running them as one resident kernel (gemv_chain.cuh).
//
// Counterpart of the reference's one-command-buffer-per-token dispatch (inference/src/engine.m:453-454 open the
// command buffer and its encoder, every format_dispatch_matvec / fused gate-up call only encodes into it,
// engine.m:1048-1050 commit once): between orome_cuda_chain_begin and orome_cuda_chain_end the batch-1 entry points
// record their product instead of launching it; orome_cuda_chain_launch runs the recorded sequence.
#include "ctx.h"

#include <algorithm>
#include <cstring>
#include <vector>

#include "gemv_chain.cuh"

using namespace orome;

#define fail orome_fail

struct ChainRec {
    uint32_t mode = CHAIN_MODE_PLAIN;
    int nseg = 0;
    const uint8_t *w[CHAIN_MAX_SEG] = {nullptr}, *w2[CHAIN_MAX_SEG] = {nullptr};
    float *y[CHAIN_MAX_SEG] = {nullptr};
    uint32_t rows[CHAIN_MAX_SEG] = {0};
    const float *x = nullptr;
    uint32_t in_dim = 0;
    int fmt = 0, layout = 0;
    bool argmax = false;
};

struct ChainRecording {
    std::vector<ChainRec> recs;
    uint32_t *argmax_out = nullptr;
};

struct orome_cuda_chain {
    orome_cuda_ctx *ctx = nullptr;
    std::vector<ChainProd> prods;
    ChainProd *prods_dev = nullptr;
    uint8_t *slots_dev = nullptr;
    unsigned int *words_dev = nullptr;            // arrival counter of a launch
    unsigned long long *argmax_part = nullptr;
    ChainArgs args;
    int grid = 0, np = 3, fmts = 0;
    size_t smem = 0;
    uint64_t weight_bytes = 0;
};

static bool overlaps(const void *a, size_t an, const void *b, size_t bn)
{
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + bn && b0 < a0 + an;
}
static bool contains(const void *outer, size_t on, const void *inner, size_t in)
{
    const uintptr_t o0 = reinterpret_cast<uintptr_t>(outer), i0 = reinterpret_cast<uintptr_t>(inner);
    return i0 >= o0 && i0 + in <= o0 + on;
}

extern "C" int orome_cuda_chain_begin(orome_cuda_ctx *c)
{
    if (!c) return fail(OROME_EINVAL, "chain_begin: NULL ctx");
    if (c->rec) return fail(OROME_EINVAL, "chain_begin: a recording is already open on this context");
    c->rec = new ChainRecording;
    return OROME_OK;
}

void orome_chain_abandon(orome_cuda_ctx *c)
{
    delete c->rec;
    c->rec = nullptr;
}

int orome_chain_record_group(orome_cuda_ctx *c, const OromeTensorRef *refs, int n_refs, const float *x, float *const *y)
{
    if (n_refs > CHAIN_MAX_SEG) return fail(OROME_ENOTSUP, "chain: at most %d tensors per grouped product", CHAIN_MAX_SEG);
    const int fmt = (int)refs[0].format;
    if (!orome_pipe_supported(fmt, refs[0].in_dim) || orome_pipe_group_threads(fmt, refs[0].in_dim) > (uint32_t)CHAIN_CONSUMERS)
        return fail(OROME_ENOTSUP, "chain: format %d with in_dim %u has no chained form (Q8_0: in_dim a multiple of 64, K-quants: of 256)", fmt, refs[0].in_dim);
    ChainRec r;
    r.mode = CHAIN_MODE_PLAIN;
    r.nseg = n_refs;
    for (int i = 0; i < n_refs; ++i) {
        r.w[i] = static_cast<const uint8_t *>(refs[i].buffer) + refs[i].offset;
        r.y[i] = y[i];
        r.rows[i] = refs[i].out_dim;
        if (reinterpret_cast<uintptr_t>(y[i]) & 15) return fail(OROME_EINVAL, "chain: y must be 16-byte aligned");
    }
    r.x = x;
    r.in_dim = refs[0].in_dim;
    r.fmt = fmt;
    r.layout = (int)refs[0].variant;
    c->rec->recs.push_back(r);
    return OROME_OK;
}

int orome_chain_record_gate_up(orome_cuda_ctx *c, const OromeTensorRef *gate, const OromeTensorRef *up, const float *x, float *out)
{
    const int fmt = (int)gate->format;
    if (!orome_pipe_supported(fmt, gate->in_dim) || orome_pipe_group_threads(fmt, gate->in_dim) > (uint32_t)CHAIN_CONSUMERS)
        return fail(OROME_ENOTSUP, "chain: format %d with in_dim %u has no chained form", fmt, gate->in_dim);
    if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) & 15) return fail(OROME_EINVAL, "chain: x and out must be 16-byte aligned");
    ChainRec r;
    r.mode = CHAIN_MODE_SWIGLU;
    r.nseg = 1;
    r.w[0] = static_cast<const uint8_t *>(gate->buffer) + gate->offset;
    r.w2[0] = static_cast<const uint8_t *>(up->buffer) + up->offset;
    r.y[0] = out;
    r.rows[0] = gate->out_dim;
    r.x = x;
    r.in_dim = gate->in_dim;
    r.fmt = fmt;
    r.layout = (int)gate->variant;
    c->rec->recs.push_back(r);
    return OROME_OK;
}

int orome_chain_record_unpack(orome_cuda_ctx *c, float *vec, uint32_t n)
{
    ChainRec r;
    r.mode = CHAIN_MODE_UNPACK;
    r.nseg = 1;
    r.y[0] = vec;
    r.x = vec;
    r.in_dim = n;
    r.rows[0] = 0;
    c->rec->recs.push_back(r);
    return OROME_OK;
}

int orome_chain_record_argmax(orome_cuda_ctx *c, const float *data, uint32_t count, uint32_t *result)
{
    if (c->g_world > 1) return fail(OROME_ENOTSUP, "chain: the arg-max epilogue is single-GPU (row-split logits end on different GPUs)");
    if (c->rec->argmax_out) return fail(OROME_ENOTSUP, "chain: one arg-max per chain");
    for (auto it = c->rec->recs.rbegin(); it != c->rec->recs.rend(); ++it) {
        if (it->mode == CHAIN_MODE_UNPACK) continue;
        uint32_t total = 0;
        for (int i = 0; i < it->nseg; ++i) total += it->rows[i];
        if (it->nseg == 1 && it->y[0] == data && total == count) {
            it->argmax = true;
            c->rec->argmax_out = result;
            return OROME_OK;
        }
        break;
    }
    return fail(OROME_ENOTSUP, "chain: arg-max must follow the product whose whole output it reduces");
}

template <int NP, int FMTS>
static int chain_configure(const orome_cuda_ctx *c, size_t *static_smem)
{
    auto kern = gemv_chain_kernel<NP, FMTS>;
    cudaFuncAttributes fa;
    CU(cudaFuncGetAttributes(&fa, kern));
    CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, c->smem_optin - (int)fa.sharedSizeBytes));
    *static_smem = fa.sharedSizeBytes;
    return OROME_OK;
}

template <int NP, int FMTS>
static int chain_launch_inst(orome_cuda_chain *ch, cudaStream_t st)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ch->grid);
    cfg.blockDim = dim3(CHAIN_THREADS);
    cfg.dynamicSmemBytes = ch->smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // every CTA resident at once, or the launch fails: the CTAs wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU(cudaLaunchKernelEx(&cfg, gemv_chain_kernel<NP, FMTS>, ch->args));
    ++ch->ctx->launches;
    return OROME_OK;
}

constexpr int FMTS_Q8 = 1 << FMT_Q8_0;
constexpr int FMTS_ALL = (1 << FMT_Q8_0) | (1 << FMT_Q4_K) | (1 << FMT_Q5_K) | (1 << FMT_Q6_K);

extern "C" void orome_cuda_chain_destroy(orome_cuda_ctx *c, orome_cuda_chain *ch)
{
    if (!ch) return;
    if (c) cudaSetDevice(c->device);
    cudaFree(ch->prods_dev);
    cudaFree(ch->slots_dev);
    cudaFree(ch->words_dev);
    cudaFree(ch->argmax_part);
    delete ch;
}

extern "C" int orome_cuda_chain_end(orome_cuda_ctx *c, orome_cuda_chain **out)
{
    if (!c || !out) return fail(OROME_EINVAL, "chain_end: NULL argument");
    if (!c->rec) return fail(OROME_EINVAL, "chain_end: no recording is open");
    std::vector<ChainRec> recs;
    recs.swap(c->rec->recs);
    uint32_t *argmax_out = c->rec->argmax_out;
    orome_chain_abandon(c);
    const size_t n = recs.size();
    if (n == 0) return fail(OROME_EINVAL, "chain_end: nothing was recorded");
    CU(cudaSetDevice(c->device));

    orome_cuda_chain *ch = new orome_cuda_chain;
    ch->ctx = c;
    ch->np = c->x_bits == 24 ? 3 : 2;
    ch->grid = c->sm_count;
    ch->prods.resize(n);
    int rc = OROME_OK;
    auto bail = [&](int code) { orome_cuda_chain_destroy(c, ch); return code; };

    // ---- geometry of every product -----------------------------------------------------------------------------
    const uint32_t G = (uint32_t)ch->grid;
    uint32_t stage_min = 0;        // smallest stage that holds one tile (rows_par rows of one tensor) of every product
    size_t xq_max = 0;
    for (size_t p = 0; p < n; ++p) {
        const ChainRec &r = recs[p];
        ChainProd &P = ch->prods[p];
        memset(&P, 0, sizeof P);
        P.mode = r.mode;
        P.in_dim = r.in_dim;
        P.x = r.x;
        P.y_tag = (uint32_t)p + 1;
        if (r.mode == CHAIN_MODE_UNPACK) {
            P.nseg = 1; P.seg[0].y = r.y[0];
            P.rows_q = r.in_dim / 4 / (uint32_t)ch->grid; P.rows_r = r.in_dim / 4 % (uint32_t)ch->grid;
            continue;
        }
        ch->fmts |= 1 << r.fmt;
        P.fmt = (uint8_t)r.fmt;
        P.layout = (uint8_t)r.layout;
        P.nseg = (uint8_t)r.nseg;
        P.argmax = r.argmax;
        uint32_t total = 0;
        for (int i = 0; i < r.nseg; ++i) {
            P.seg[i].w = r.w[i]; P.seg[i].w2 = r.w2[i]; P.seg[i].y = r.y[i]; P.seg[i].rows = r.rows[i]; P.seg[i].vstart = total;
            total += r.rows[i];
            ch->weight_bytes += (uint64_t)r.rows[i] * row_bytes_of(r.fmt, r.in_dim) * (r.mode == CHAIN_MODE_SWIGLU ? 2 : 1);
        }
        P.total_rows = total;
        P.rows_q = total / G; P.rows_r = total % G;
        P.row_bytes = (uint32_t)row_bytes_of(r.fmt, r.in_dim);
        P.units = r.fmt == FMT_Q8_0 ? r.in_dim / 64 : r.in_dim / 256;
        P.group_threads = orome_pipe_group_threads(r.fmt, r.in_dim);
        P.gt_magic = (uint32_t)((0x100000000ull + P.group_threads - 1) / P.group_threads);      // exact for dividends below 2^16
        P.u_magic = (uint32_t)((0x100000000ull + P.units - 1) / P.units);
        P.rows_par = std::max(1u, std::min((uint32_t)PIPE_MAX_ROWS_PAR, (uint32_t)CHAIN_CONSUMERS / P.group_threads));
        // a stage has two halves of rows_par rows each (gate and up rows in the fused form, else two passes over the groups)
        stage_min = std::max(stage_min, 2 * ((P.rows_par * P.row_bytes + 48 + 127) / 128 * 128));
        // quantized x: one byte plane per 8 bits, a scale per group (16 elements for Q6_K, else 32), K-quant sums per 32
        const size_t grp = r.fmt == FMT_Q6_K ? 16 : 32, sums = (r.fmt == FMT_Q4_K || r.fmt == FMT_Q5_K) ? (size_t)r.in_dim / 32 * 4 : 0;
        xq_max = std::max(xq_max, ((size_t)ch->np * r.in_dim + r.in_dim / grp * 4 + sums + 15) / 16 * 16);
    }
    if (ch->fmts == 0) return bail(fail(OROME_EINVAL, "chain_end: the chain holds no product"));

    size_t static_smem = 0;
    const bool q8_only = ch->fmts == FMTS_Q8;
#ifdef OROME_CHAIN_Q8_ONLY      // compile-time experiment builds: only the Q8_0 instances
    if (!q8_only) return bail(fail(OROME_ENOTSUP, "chain_end: this build holds only the Q8_0 chain kernel"));
    rc = ch->np == 3 ? chain_configure<3, FMTS_Q8>(c, &static_smem) : chain_configure<2, FMTS_Q8>(c, &static_smem);
#else
    if (ch->np == 3) rc = q8_only ? chain_configure<3, FMTS_Q8>(c, &static_smem) : chain_configure<3, FMTS_ALL>(c, &static_smem);
    else rc = q8_only ? chain_configure<2, FMTS_Q8>(c, &static_smem) : chain_configure<2, FMTS_ALL>(c, &static_smem);
#endif
    if (rc) return bail(rc);

    // ---- shared memory: barriers, three descriptors, partial sums, quantized x, then the ring ---------------------
    // A stage holds two halves of rows_par rows: about 61 KB for 4096-wide Q8_0 rows, three stages deep.
    ChainArgs &a = ch->args;
    memset(&a, 0, sizeof a);
    const size_t budget = std::min<size_t>(228 * 1024 - 1024, (size_t)c->smem_optin) - static_smem - 128;
    const size_t red_bytes = 8 * 1024;
    a.desc_base = 2 * 8 * PIPE_MAX_STAGES;
    a.red_base = a.desc_base + 3 * (uint32_t)sizeof(ChainProd);
    a.xs_base = (uint32_t)((a.red_base + red_bytes + 127) / 128 * 128);
    a.stage_base = (uint32_t)((a.xs_base + xq_max + 127) / 128 * 128);
    if (budget < a.stage_base + 2 * (size_t)stage_min)
        return bail(fail(OROME_ENOTSUP, "chain_end: two stages of %u bytes do not fit shared memory beside %zu bytes of quantized x", stage_min, xq_max));
    const size_t room = budget - a.stage_base;
    uint32_t stride = std::max(stage_min, c->stage_kb ? (uint32_t)c->stage_kb * 1024u : 0u);
    stride = (stride + 127) / 128 * 128;
    if (room / stride < 2) stride = stage_min;
    const uint32_t ns = (uint32_t)std::min<size_t>(PIPE_MAX_STAGES, room / stride);
    a.nstages = ns;
    a.stage_stride = stride;
    // Two stages outstanding by default: what is on its way to the SM queues in front of the loads with which the consumers
    // fetch the next input vector.  Measured on the 9B set, whole ring (three stages) against two: 598 -> 616 tok/s on one
    // GPU, 754 -> 787 on two, 884 -> 895 on four; one stage: 765 on two.
    // (The default is what fits 136 KiB, i.e. two of the 60-68 KiB stages of a Q8_0 chain; chains of small stages keep more.)
    a.inflight = c->chain_inflight > 0 ? std::min<uint32_t>((uint32_t)c->chain_inflight, ns)
                                       : std::min<uint32_t>(std::max<uint32_t>(2u, (uint32_t)((136u * 1024u) / stride)), ns);
    ch->smem = a.stage_base + (size_t)stride * ns;

    for (size_t p = 0; p < n; ++p) {
        ChainProd &P = ch->prods[p];
        if (P.mode == CHAIN_MODE_UNPACK) continue;
        const uint32_t sw = P.mode == CHAIN_MODE_SWIGLU ? 2u : 1u, gw = P.group_threads / 32;
        const uint32_t share = (P.total_rows + G - 1) / G;
        P.half_stride = stride / 2 / 128 * 128;
        // rows per group and tile: the fused form fills a half with each tensor's rows, the plain form the whole stage
        uint32_t iters = sw == 2 ? (P.half_stride - 48) / (P.rows_par * P.row_bytes) : (stride - 48) / (P.rows_par * P.row_bytes);
        iters = std::max(1u, std::min((uint32_t)PIPE_MAX_ITERS, iters));
        iters = std::min(iters, std::max(1u, (share + P.rows_par - 1) / P.rows_par));
        // two partial-sum buffers of red_rows rows must fit the space set aside for them
        const uint32_t red_cap = (uint32_t)(red_bytes / (2 * sizeof(float) * gw * sw));
        while (iters > 1 && P.rows_par * iters > red_cap) --iters;
        if (P.rows_par * iters > red_cap) return bail(fail(OROME_ENOTSUP, "chain_end: product %zu needs %u partial sums per tile", p, P.rows_par * gw * sw));
        P.iters = (uint8_t)iters;
        P.red_rows = std::min(red_cap, std::max(std::min(share, 256u), P.rows_par * iters));
    }

    // ---- inputs produced inside the chain, hazards -----------------------------------------------------------------
    // sync[p]: the product whose completion on every CTA (and GPU) product p waits for by polling its input.
    const bool multi = c->g_world > 1;
    const uint8_t *arena = multi ? c->g_arena[c->g_rank] : nullptr;
    auto in_arena = [&](const void *ptr, size_t bytes) { return multi && contains(arena, c->g_data_bytes, ptr, bytes); };
    std::vector<long> sync(n, -1), slot_off(n * CHAIN_MAX_SEG, -1);
    size_t slot_bytes = 0;
    for (size_t p = 0; p < n; ++p) {
        ChainProd &P = ch->prods[p];
        if (P.mode == CHAIN_MODE_UNPACK) continue;
        for (uint32_t i = 0; i < P.nseg; ++i) {
            if (in_arena(P.seg[i].y, (size_t)P.seg[i].rows * 4)) { P.publish = 1; continue; }
            slot_off[p * CHAIN_MAX_SEG + i] = (long)slot_bytes;
            slot_bytes += ((size_t)P.seg[i].rows * 8 + 255) / 256 * 256;
        }
        if (P.publish)
            for (uint32_t i = 0; i < P.nseg; ++i)
                if (!in_arena(P.seg[i].y, (size_t)P.seg[i].rows * 4))
                    return bail(fail(OROME_EINVAL, "chain_end: product %zu writes some outputs inside the gather arena and some outside", p));
    }
    if (slot_bytes) {
        cudaError_t e = cudaMalloc(&ch->slots_dev, slot_bytes);
        if (e != cudaSuccess) return bail(fail(OROME_ENOMEM, "chain_end: %zu bytes of output slots: %s", slot_bytes, cudaGetErrorString(e)));
        CU(cudaMemset(ch->slots_dev, 0, slot_bytes));
    }
    auto arena_slots = [&](const void *ptr) {
        return reinterpret_cast<uint2 *>(const_cast<uint8_t *>(arena) + c->g_data_bytes + 2 * (size_t)(static_cast<const uint8_t *>(ptr) - arena));
    };
    for (size_t p = 0; p < n; ++p) {
        ChainProd &P = ch->prods[p];
        if (P.mode != CHAIN_MODE_UNPACK)
            for (uint32_t i = 0; i < P.nseg; ++i)
                P.seg[i].ys = P.publish ? arena_slots(P.seg[i].y) : reinterpret_cast<uint2 *>(ch->slots_dev + slot_off[p * CHAIN_MAX_SEG + i]);
        // the latest earlier product that writes any part of this product's input
        const size_t xbytes = (size_t)P.in_dim * 4;
        for (long q = (long)p - 1; q >= 0 && sync[p] < 0; --q) {
            const ChainProd &Q = ch->prods[q];
            if (Q.mode == CHAIN_MODE_UNPACK) continue;
            for (uint32_t i = 0; i < Q.nseg; ++i) {
                const size_t ybytes = (size_t)Q.seg[i].rows * 4;
                if (!overlaps(P.x, xbytes, Q.seg[i].y, ybytes)) continue;
                if (Q.publish) {
                    // a row-split vector: this GPU wrote a slice of it, the peers the rest, all under the same tag
                    if (!in_arena(P.x, xbytes) || ((reinterpret_cast<const uint8_t *>(P.x) - arena) & 15))
                        return bail(fail(OROME_EINVAL, "chain_end: product %zu reads a gathered vector that is not inside the arena (16-byte aligned)", p));
                    P.xs = arena_slots(P.x);
                } else {
                    if (!contains(Q.seg[i].y, ybytes, P.x, xbytes))
                        return bail(fail(OROME_ENOTSUP, "chain_end: the input of product %zu overlaps the output of product %ld without lying inside it", p, q));
                    P.xs = Q.seg[i].ys + (P.x - Q.seg[i].y);
                    if (reinterpret_cast<uintptr_t>(P.xs) & 15) return bail(fail(OROME_EINVAL, "chain_end: the input of product %zu is not 16-byte aligned inside its producer's output", p));
                }
                P.x_tag = Q.y_tag;
                P.dep_peers = Q.publish;
                sync[p] = q;
                break;
            }
        }
        if (P.mode == CHAIN_MODE_UNPACK && sync[p] < 0)
            return bail(fail(OROME_EINVAL, "chain_end: gather_wait names a vector that no recorded product writes"));
    }
    // A CTA runs its products in order and starts product p only when all of sync[p] is complete everywhere, so
    // "every CTA has finished every product up to F[p]" holds when any CTA writes outputs of p, F[p] = max sync[0..p].
    // A product that overwrites what an earlier one reads or writes must have that earlier one within F.
    {
        long F = -1;
        for (size_t p = 0; p < n; ++p) {
            F = std::max(F, sync[p]);
            const ChainProd &P = ch->prods[p];
            if (P.mode == CHAIN_MODE_UNPACK) continue;
            for (long r = (long)p - 1; r > F; --r) {
                const ChainProd &Q = ch->prods[r];
                for (uint32_t i = 0; i < P.nseg; ++i) {
                    const size_t ybytes = (size_t)P.seg[i].rows * 4;
                    bool clash = overlaps(P.seg[i].y, ybytes, Q.x, (size_t)Q.in_dim * 4);
                    if (Q.mode != CHAIN_MODE_UNPACK)
                        for (uint32_t k = 0; k < Q.nseg; ++k) clash = clash || overlaps(P.seg[i].y, ybytes, Q.seg[k].y, (size_t)Q.seg[k].rows * 4);
                    if (clash)
                        return bail(fail(OROME_ENOTSUP, "chain_end: product %zu overwrites a vector that product %ld reads or writes, and no data dependency "
                                         "orders them; split the chain there", p, r));
                }
            }
        }
        // Several GPUs: the next launch's first products run while a slower peer may still be in this launch, past
        // the last product anyone waited for.  What those first products publish must not be read back there.
        if (multi) {
            size_t first_sync = n;
            for (size_t p = 0; p < n; ++p) if (sync[p] >= 0) { first_sync = p; break; }
            for (size_t p = 0; p < first_sync && p < n; ++p) {
                const ChainProd &P = ch->prods[p];
                if (P.mode == CHAIN_MODE_UNPACK || !P.publish) continue;
                for (size_t r = (size_t)(F + 1); r < n; ++r) {       // a peer has finished product F: it is somewhere after it
                    const ChainProd &Q = ch->prods[r];
                    for (uint32_t i = 0; i < P.nseg; ++i)
                        if (Q.xs && overlaps(P.seg[i].y, (size_t)P.seg[i].rows * 4, Q.x, (size_t)Q.in_dim * 4))
                            return bail(fail(OROME_ENOTSUP, "chain_end: product %zu of the next launch would overwrite the input of product %zu of a launch a peer "
                                             "may still be running", p, r));
                }
            }
        }
    }

    // ---- device copies ---------------------------------------------------------------------------------------------
    CU(cudaMalloc(&ch->prods_dev, n * sizeof(ChainProd)));
    CU(cudaMemcpy(ch->prods_dev, ch->prods.data(), n * sizeof(ChainProd), cudaMemcpyHostToDevice));
    CU(cudaMalloc(&ch->words_dev, 16 * sizeof(unsigned int)));       // [0] arrivals of a launch
    CU(cudaMemset(ch->words_dev, 0, 16 * sizeof(unsigned int)));
    a.prods = ch->prods_dev;
    a.nprods = (uint32_t)n;
    a.status = c->status_dev;
    a.gen = c->chain_gen_dev;
    a.arrived = ch->words_dev;
    a.rank = 0;
    if (argmax_out) {
        CU(cudaMalloc(&ch->argmax_part, (size_t)ch->grid * sizeof(unsigned long long)));
        a.argmax_part = ch->argmax_part;
        a.argmax_out = argmax_out;
    }
    if (multi) {
        int np = 0;
        for (int r = 0; r < c->g_world; ++r)
            if (r != c->g_rank) a.peer_delta[np++] = (long long)(c->g_arena[r] - arena);
        a.npeers = np;
        a.rank = c->g_rank;
    }
    *out = ch;
    return OROME_OK;
}

extern "C" int orome_cuda_chain_launch(orome_cuda_ctx *c, orome_cuda_chain *ch, void *stream)
{
    if (!c || !ch || ch->ctx != c) return fail(OROME_EINVAL, "chain_launch: NULL or foreign chain");
    if (c->rec) return fail(OROME_EINVAL, "chain_launch: a recording is open");
    CU(cudaSetDevice(c->device));
    ch->args.wait_cycles = orome_wait_cycles(c);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool q8_only = ch->fmts == FMTS_Q8;
#ifdef OROME_CHAIN_Q8_ONLY
    return ch->np == 3 ? chain_launch_inst<3, FMTS_Q8>(ch, st) : chain_launch_inst<2, FMTS_Q8>(ch, st);
#else
    if (ch->np == 3) return q8_only ? chain_launch_inst<3, FMTS_Q8>(ch, st) : chain_launch_inst<3, FMTS_ALL>(ch, st);
    return q8_only ? chain_launch_inst<2, FMTS_Q8>(ch, st) : chain_launch_inst<2, FMTS_ALL>(ch, st);
#endif
}

extern "C" int orome_cuda_chain_info(orome_cuda_chain *ch, int *n_products, uint64_t *weight_bytes, int *stages, int *stage_bytes)
{
    if (!ch) return fail(OROME_EINVAL, "chain_info: NULL chain");
    if (n_products) *n_products = (int)ch->prods.size();
    if (weight_bytes) *weight_bytes = ch->weight_bytes;
    if (stages) *stages = (int)ch->args.nstages;
    if (stage_bytes) *stage_bytes = (int)ch->args.stage_stride;
    return OROME_OK;
}

#ifdef OROME_DIAGNOSTICS
// Diagnostics builds: the next launches of `ch` stamp their timeline into trace_dev ([grid][products][8] uint64), NULL stops it.
extern "C" int orome_cuda_chain_trace(orome_cuda_chain *ch, unsigned long long *trace_dev)
{
    if (!ch) return fail(OROME_EINVAL, "chain_trace: NULL chain");
    ch->args.trace = trace_dev;
    return OROME_OK;
}
#endif
