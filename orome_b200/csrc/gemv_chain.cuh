// gemv_chain.cuh -- a whole token step's matvecs as ONE resident kernel.
//
// The reference encodes every product of a token into one command buffer and commits it once
// (inference/src/engine.m:453-454, 1048-1050).  Launching each product as its own kernel costs this GPU a
// launch-to-launch dependency chain of about 4 us per product (grid drain, launch, x load, first tile), which is
// as long as the product itself for a 17 MB tensor.  Here one CTA per SM stays resident and walks a table of
// products in device memory:
//
//   * The producer warp streams the CTA's rows of product after product into one ring of shared-memory stages
//     (1-D bulk copies completing on mbarriers).  Weights never depend on activations, so the ring keeps
//     filling while the consumers wait for an input vector: HBM does not idle at a product boundary.
//   * A product's output is written twice: as plain floats (for readers outside the chain) and as 8-byte
//     {value, tag} slots.  A later product of the chain whose input is that vector reads the slots and polls
//     every element until it carries the tag of the producing product and launch -- value and tag arrive in one
//     store, so no fence, no flag and no grid-wide barrier are involved.  On several GPUs (row-split tensors)
//     the same store also goes to the same slot of each peer over NVLink, which completes the vector everywhere.
//   * Consumers (15 warps) are the pipelined kernel's: x as per-group fixed point in byte planes, dp4a against
//     the packed weights as they lie, per-row partial sums flushed in batches.  The thread mapping (threads per
//     row, rows side by side) is per product and comes from the table.
//   * Nothing announces a finished product: a reader goes straight to the slots, takes what carries the tag and polls
//     (bounded) for what does not yet.  Completion counters per product, watched by one lane per warp before anyone
//     touched the slots, and progress words stored into the peers, were built to keep 71 000 threads from re-reading
//     the same 32 KB; measured, they only delayed the readers (9B Q8_0 set: N = 1 552 -> 604 tok/s without them,
//     N = 2 695 -> 768, N = 4 728 -> 982) and were removed.
//   * Every wait is bounded (wait_cycles); expiry sets the status word, is sticky for the rest of the launch, and
//     a launch that finds the status word set does not wait at all.
//
// All CTAs must be resident together (they wait on one another's outputs): the host launches the kernel
// cooperatively with at most one CTA per SM.
#pragma once
#include "gemv_pipe.cuh"

namespace orome {

constexpr int CHAIN_MAX_SEG = 4;
constexpr int CHAIN_CONSUMERS = 448;                      // 14 warps: seven 64-thread or two 192-thread row groups; leaves 136 registers per thread
constexpr int CHAIN_THREADS = CHAIN_CONSUMERS + 32;       // + the producer warp
constexpr uint32_t CHAIN_TAG = 0x80000000u;               // chain tags have the top bit set; armed single launches count from 1

enum : uint32_t { CHAIN_MODE_PLAIN = 0, CHAIN_MODE_SWIGLU = 1, CHAIN_MODE_UNPACK = 2 };

struct ChainSeg {
    const uint8_t *w, *w2;      // tensor (gate and up tensors in the fused form)
    float *y;                   // output rows as plain floats
    uint2 *ys;                  // the same rows as {value, tag} slots in this GPU's memory
    uint32_t rows, vstart;      // rows of the segment, its first virtual row (segments are concatenated)
};

struct alignas(16) ChainProd {
    ChainSeg seg[CHAIN_MAX_SEG];
    const float *x;             // input vector as plain floats (read when xs is NULL)
    const uint2 *xs;            // its slots when a product of the chain (here or on a peer) writes it
    uint32_t x_tag, y_tag;      // tag offsets: the input must carry base + x_tag, the outputs get base + y_tag
    uint8_t nseg, mode, layout, fmt;
    uint8_t publish;            // outputs also go to the peers' slots
    uint8_t argmax;             // the launch also reduces this product's outputs to the index of their maximum
    uint8_t dep_peers;          // the product that writes the input is row-split over the GPUs (kept for diagnostics)
    uint8_t iters;              // rows per group and tile
    uint32_t in_dim, row_bytes, units, group_threads;
    uint32_t rows_par, half_stride, total_rows, red_rows;
    // Division-free row split: CTA b owns rows [b * rows_q + min(b, rows_r), ...) -- rows_q or rows_q + 1 of them (for the
    // unpack pseudo-product the "rows" are four-float pieces); gt_magic / u_magic = ceil(2^32 / d) turn the two
    // divisions of the thread mapping into a multiply-high.
    uint32_t rows_q, rows_r, gt_magic, u_magic;
    uint32_t pad[4];
};
static_assert(sizeof(ChainProd) == 256, "descriptors are copied as sixteen 16-byte pieces");

struct ChainArgs {
    const ChainProd *prods;
    uint32_t nprods;
    uint32_t nstages, stage_stride, stage_base, red_base, xs_base, desc_base;
    uint32_t inflight;          // stages the producer keeps outstanding at most
    int *status;
    unsigned int *gen;          // generation base of the chain's tags, advanced by nprods when a launch ends
    unsigned int *arrived;      // CTAs that finished the launch
    int rank;
    long long wait_cycles;
    unsigned long long *argmax_part;   // [grid] per-CTA candidates of the arg-max epilogue
    uint32_t *argmax_out;              // index of the largest output of the product marked `argmax`
    int npeers;
    long long peer_delta[PIPE_MAX_PEERS];
    unsigned long long *trace;  // diagnostics builds: [grid][nprods][12] %globaltimer stamps, else NULL
};

// Diagnostics builds (-DOROME_DIAGNOSTICS) stamp, per CTA and product: 0 consumers enter, 1 input reported complete,
// 2 input quantized, 3 first tile landed, 4 last tile consumed, 5 outputs stored; 6 / 7 producer issued first / last tile;
// 8 thread 0 has quantized its own pieces, 9 the last thread of the CTA has (both before the barrier that precedes 2).
#ifdef OROME_DIAGNOSTICS
#define CHAIN_STAMP(a, p, k)                                                                                                  \
    do {                                                                                                                      \
        if ((a).trace) (a).trace[((size_t)blockIdx.x * (a).nprods + (p)) * 12 + (k)] = global_ns();                            \
    } while (0)
#else
#define CHAIN_STAMP(a, p, k) do { } while (0)
#endif

__device__ __forceinline__ unsigned int chain_tag(unsigned int base, uint32_t off) { return CHAIN_TAG | ((base + off) & 0x7FFFFFFFu); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct ChainTile { uint32_t seg, row0, n; };
struct ChainWalk { uint32_t cur, hi, seg; };

// Next run of rows of this CTA's range [cur, hi) of the concatenated rows that lies inside one segment.
template <typename Prod>
__device__ __forceinline__ bool chain_next_tile(const Prod &P, uint32_t nseg, uint32_t cap, ChainWalk &w, ChainTile &t)
{
    if (w.cur >= w.hi) return false;
    uint32_t s = w.seg;
    while (s + 1 < nseg && w.cur >= P.seg[s + 1].vstart) ++s;
    w.seg = s;
    const uint32_t seg_end = P.seg[s].vstart + P.seg[s].rows;
    const uint32_t lim = w.hi < seg_end ? w.hi : seg_end;
    uint32_t n = lim - w.cur;
    if (n > cap) n = cap;
    t.seg = s; t.row0 = w.cur - P.seg[s].vstart; t.n = n;
    w.cur += n;
    return true;
}

// One product on the consumer side.  `s` / `parity`: position in the stage ring, carried from product to product.
// A tile of the fused gate/up form takes two consecutive stages (gate rows, then up rows), any other tile one.
// The fused form is a run-time flag, not a second instance: two inlined instances in one loop made the compiler
// spill the x slice in the row loop.
template <int FMT, int NP>
__device__ __forceinline__ void chain_product(const ChainArgs &a, const ChainProd &P, uint8_t *smem, uint64_t *full, uint64_t *empty,
                                              uint32_t lo, uint32_t hi, uint32_t &s, uint32_t &parity, unsigned int base,
                                              volatile int *s_abort, unsigned long long *best_slot, uint32_t p)
{
    const bool SWIGLU = P.mode == CHAIN_MODE_SWIGLU;
    using SlotT = Slot<FMT, NP>;
    constexpr int PARTS = SlotT::PARTS;
    constexpr int C = CHAIN_CONSUMERS;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint32_t GT = P.group_threads, GW = GT >> 5, U = P.units, RP = P.rows_par;
    const uint32_t group = __umulhi(tid, P.gt_magic), j = tid - group * GT, wig = j >> 5;
    const bool in_group = group < RP;
    const uint32_t part = __umulhi(j, P.u_magic), unit = j - part * U;
    const bool active = in_group && j < (uint32_t)PARTS * U;

    // ---- the input vector: read from its slots when the chain produces it (every element checked for its tag),
    // quantized once per CTA; every CTA starts at a different place of the vector
    uint8_t *xq = smem + a.xs_base;
    {
        const unsigned int want = chain_tag(base, P.x_tag);
        uint32_t rot = blockIdx.x * 32u;                      // start pieces: a warp's worth (1 KiB of slots) apart per CTA
        while (rot >= P.in_dim / 4) rot -= P.in_dim / 4;
        const bool ok = P.xs && !*s_abort
            ? quantize_slots_to_smem<NP, SlotT::GROUP, SlotT::SUMS>(P.xs, want, P.in_dim, xq, tid, (uint32_t)C, a.wait_cycles, a.status, rot,
                                                                    a.trace && tid == 0 ? a.trace + ((size_t)blockIdx.x * a.nprods + p) * 12 + 10 : nullptr)
            : quantize_x_to_smem<NP, SlotT::GROUP, SlotT::SUMS>(P.x, P.in_dim, 1u, 0u, xq, 0u, tid, (uint32_t)C, nullptr, 0u, a.wait_cycles, a.status, rot);
        if (!ok) { *s_abort = 1; atomicExch(a.status, 3); }
    }
    if (tid == 0) CHAIN_STAMP(a, p, 8);
    if (tid == C - 1) CHAIN_STAMP(a, p, 9);
    cp_async_wait_all();                       // the next product's descriptor (issued by the caller) has landed
    named_bar_sync(PIPE_BAR_CONSUMERS, C);
    if (tid == 0) CHAIN_STAMP(a, p, 2);
    SlotT slot;
    if (active) slot.load(make_xq_view<NP, SlotT::GROUP>(xq, P.in_dim), unit, (int)part);

    // ---- tiles.  The walk below must visit tiles exactly as the producer issues them: the CTA's rows in order, cut at
    // segment ends and every `cap` rows, one stage per tile.  A stage has two halves: gate rows and up rows in the
    // fused form, else the rows of the first and of the second pass over the row groups.  A group works on one row
    // of each half at a time, so two independent dot products and reductions are in flight per warp.
    const uint32_t S = SWIGLU ? 2u : 1u;
    const uint32_t CAP = P.red_rows, PLANE = CAP * GW;
    float *pbuf = reinterpret_cast<float *>(smem + a.red_base);
    uint32_t which = 0, buf_n = 0, buf_row0 = 0, buf_seg = 0, seg = 0;
    const uint32_t stages_s = smem_u32(smem + a.stage_base);
    const uint32_t rb = P.row_bytes, nstages = a.nstages, stride = a.stage_stride;
    const uint32_t lane_off = unit * SlotT::UNIT_BYTES + group * rb;      // this thread's unit inside the group's first row of a half
    const bool rows16 = (rb & 15u) == 0;     // then every row of a segment starts at the same offset inside its 16-byte piece
    const uint32_t cap = RP * P.iters, nseg = P.nseg, layout = P.layout, half_stride = P.half_stride;
    uint32_t cur = lo, seg_start = P.seg[0].vstart, seg_end = seg_start + P.seg[0].rows;
    uint32_t delta = 0, delta2 = 0;
    bool fresh_seg = true;
    for (;;) {
        const bool more = cur < hi;
        uint32_t n = 0;
        bool new_seg = false;
        if (more) {
            while (cur >= seg_end && seg + 1 < nseg) { ++seg; seg_start = P.seg[seg].vstart; seg_end = seg_start + P.seg[seg].rows; new_seg = fresh_seg = true; }
            const uint32_t lim = hi < seg_end ? hi : seg_end;
            n = lim - cur < cap ? lim - cur : cap;
        }
        // one flush site: the batch is full, the segment (and with it the output vector) changes, or the rows are done
        if (buf_n && (!more || new_seg || buf_n + n > CAP)) {
            named_bar_sync(PIPE_BAR_CONSUMERS, C);
            const unsigned int y_tag = chain_tag(base, P.y_tag);
            const float *src = pbuf + (size_t)which * PLANE * S;
            const ChainSeg &sg = P.seg[buf_seg];
            unsigned long long fbest = 0ull;
            for (uint32_t r = tid; r < buf_n; r += C) {
                float g = 0.0f, u = 0.0f;
                for (uint32_t w = 0; w < GW; ++w) {
                    g += src[r * GW + w];
                    if (SWIGLU) u += src[PLANE + r * GW + w];
                }
                const float val = SWIGLU ? silu_mul(g, u) : g;
                const uint32_t row = buf_row0 + r;
                sg.y[row] = val;
                uint2 *sl = sg.ys + row;
                st_slot(sl, val, y_tag);
                if (P.publish)
                    for (int q = 0; q < a.npeers; ++q) st_slot(reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(sl) + a.peer_delta[q]), val, y_tag);
                if (P.argmax && val > -INFINITY) {      // as in the reference: NaN and -inf never replace the running maximum
                    const unsigned long long cand = ((unsigned long long)float_key(val) << 32) | (uint32_t)~argmax_rank(sg.vstart + row);
                    if (cand > fbest) fbest = cand;
                }
            }
            if (P.argmax) {                             // the warp's best candidate of this batch into the warp's running best
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, fbest, o);
                    if (other > fbest) fbest = other;
                }
                if (lane == 0 && fbest > *best_slot) *best_slot = fbest;
            }
            which ^= 1u;
            buf_n = 0;
        }
        if (!more) break;
        if (buf_n == 0) { buf_row0 = cur - seg_start; buf_seg = seg; }
        if (fresh_seg || !rows16) {             // offset of the tile's first byte inside its 16-byte piece, per tensor
            fresh_seg = false;
            const uint32_t off = (cur - seg_start) * rb;
            delta = ((uint32_t)reinterpret_cast<uintptr_t>(P.seg[seg].w) + off) & 15u;
            if (SWIGLU) delta2 = ((uint32_t)reinterpret_cast<uintptr_t>(P.seg[seg].w2) + off) & 15u;
        }
        if (!*s_abort && !mbar_wait_bounded(smem_u32(full + s), parity, a.wait_cycles)) {
            *s_abort = 1;
            atomicExch(a.status, 1);
        }
        if (tid == 0 && cur == lo) CHAIN_STAMP(a, p, 3);
        if (in_group) {
            // first half: rows group, group + 2 RP, ... (fused: every gate row); second half: the rows RP further on
            // (fused: the up rows, at half_stride)
            const uint32_t sbase = stages_s + s * stride + lane_off;
            uint32_t bA = sbase + delta;
            uint32_t bB = SWIGLU ? sbase + half_stride + delta2 : bA + RP * rb;
            float *dA = pbuf + (size_t)which * PLANE * S + (size_t)(buf_n + group) * GW + wig;
            float *dB = SWIGLU ? dA + PLANE : dA + RP * GW;
            const uint32_t rstep = SWIGLU ? RP : 2u * RP;
            const uint32_t step_b = rstep * rb, step_d = rstep * GW;
#pragma unroll 1
            for (uint32_t r = group; r < n; r += rstep) {
                const bool two = SWIGLU || r + RP < n;
                float vA = 0.0f, vB = 0.0f;
#ifdef OROME_CHAIN_FAKE_DOT      // experiment builds: an (almost) free consumer, to see what the rest of the kernel costs
                if (active) { vA = __uint_as_float(lds32<0>(bA)) + slot.s0; if (two) vB = __uint_as_float(lds32<0>(bB)); }
#else
                if (active) {
                    vA = slot.dot(bA, (int)part, (int)layout);
                    if (two) vB = slot.dot(bB, (int)part, (int)layout);
                }
#endif
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    vA += __shfl_xor_sync(0xffffffffu, vA, o);
                    vB += __shfl_xor_sync(0xffffffffu, vB, o);
                }
                if (lane == 0) {
                    *dA = vA;
                    if (two) *dB = vB;
                }
                bA += step_b; bB += step_b;
                dA += step_d; dB += step_d;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + s));     // this warp is done with the stage (warps without rows too)
        if (++s == nstages) { s = 0; parity ^= 1u; }
        buf_n += n;
        cur += n;
    }
    if (tid == 0) CHAIN_STAMP(a, p, 4);
}


// A vector completed by the peers, copied from its slots to its plain place (for readers outside the chain).
template <int C>      // consumer threads of the calling kernel
__device__ __forceinline__ void chain_unpack(const ChainArgs &a, const ChainProd &P, uint32_t lo4, uint32_t hi4, unsigned int base,
                                             volatile int *s_abort)
{
    bool ok = !*s_abort;
    const unsigned int want = chain_tag(base, P.x_tag);
    float4 *dst = reinterpret_cast<float4 *>(P.seg[0].y);
    for (uint32_t i = lo4 + threadIdx.x; i < hi4; i += C) dst[i] = ld_gathered4(P.xs + 4 * (size_t)i, want, &ok, a.wait_cycles, a.status);
    if (!ok && !*s_abort) { *s_abort = 1; atomicExch(a.status, 3); }
    cp_async_wait_all();
    named_bar_sync(PIPE_BAR_CONSUMERS, C);
}

// Chains that mix formats: one out-of-line instance per format, each with its own register allocation (several
// formats inlined into one loop body made the compiler spill the x slice in the row loop).  The ring position goes in
// and comes back by value.
template <int FMT, int NP>
__device__ __noinline__ uint32_t chain_product_call(const ChainArgs *a, const ChainProd *P, uint8_t *smem, uint32_t lo, uint32_t hi, uint32_t ring,
                                                    unsigned int base, volatile int *s_abort, unsigned long long *best, uint32_t p)
{
    uint32_t s = ring >> 1, parity = ring & 1u;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    chain_product<FMT, NP>(*a, *P, smem, full, full + PIPE_MAX_STAGES, lo, hi, s, parity, base, s_abort, best, p);
    return (s << 1) | parity;
}

template <int NP>
__device__ __forceinline__ void chain_dispatch(const ChainArgs &a, const ChainProd &P, uint8_t *smem, uint64_t *full, uint64_t *empty,
                                               uint32_t lo, uint32_t hi, uint32_t &s, uint32_t &parity, unsigned int base,
                                               volatile int *s_abort, unsigned long long *best, uint32_t p)
{
    uint32_t ring = (s << 1) | parity;
    switch (P.fmt) {
    case FMT_Q8_0: ring = chain_product_call<FMT_Q8_0, NP>(&a, &P, smem, lo, hi, ring, base, s_abort, best, p); break;
    case FMT_Q4_K: ring = chain_product_call<FMT_Q4_K, NP>(&a, &P, smem, lo, hi, ring, base, s_abort, best, p); break;
    case FMT_Q5_K: ring = chain_product_call<FMT_Q5_K, NP>(&a, &P, smem, lo, hi, ring, base, s_abort, best, p); break;
    default: ring = chain_product_call<FMT_Q6_K, NP>(&a, &P, smem, lo, hi, ring, base, s_abort, best, p); break;
    }
    s = ring >> 1; parity = ring & 1u;
}

// FMTS: bit f set = the chain may hold products of format f (instances carry only the formats they need).
template <int NP, int FMTS>
__global__ void __launch_bounds__(CHAIN_THREADS, 1)
gemv_chain_kernel(const __grid_constant__ ChainArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + PIPE_MAX_STAGES;
    ChainProd *desc = reinterpret_cast<ChainProd *>(smem + a.desc_base);      // three buffers: product p sits in p % 3
    __shared__ volatile int s_abort;
    __shared__ unsigned long long s_best[CHAIN_CONSUMERS / 32];      // per warp: its best arg-max candidate so far
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint32_t G = gridDim.x, B = blockIdx.x;

    if (tid == 0) {
        s_abort = *reinterpret_cast<const volatile int *>(a.status) != 0;   // an earlier launch gave up: wait for nothing
        for (uint32_t s = 0; s < a.nstages; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), CHAIN_CONSUMERS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid < 64) reinterpret_cast<uint32_t *>(desc)[tid] = __ldg(reinterpret_cast<const uint32_t *>(a.prods) + tid);
    __syncthreads();
    const unsigned int base = *reinterpret_cast<const volatile unsigned int *>(a.gen);

    if (tid >= CHAIN_CONSUMERS) {
        // ---- producer: this CTA's rows of every product, in order, into the ring
        if (lane == 0) {
            uint32_t s = 0, k = 0, issued = 0;
            bool stop = false;
            const uint64_t stream_policy = l2_policy_evict_first();
            for (uint32_t p = 0; p < a.nprods && !stop; ++p) {
                const ChainProd &P = a.prods[p];
                const uint32_t mode = P.mode;
                if (mode == CHAIN_MODE_UNPACK) continue;
                const uint32_t nseg = P.nseg, rb = __ldg(&P.row_bytes);
                const uint32_t cap = __ldg(&P.rows_par) * P.iters;
                const uint32_t rq = __ldg(&P.rows_q), rr = __ldg(&P.rows_r);
                ChainWalk w{B * rq + (B < rr ? B : rr), (B + 1) * rq + (B + 1 < rr ? B + 1 : rr), 0};
                ChainTile t;
                bool first_tile = true;
                const bool two = mode == CHAIN_MODE_SWIGLU;
                const uint32_t hs = __ldg(&P.half_stride);
                while (chain_next_tile(P, nseg, cap, w, t)) {
                    if (k > 0) {
                        if (s_abort || !mbar_wait_bounded(smem_u32(empty + s), (k - 1) & 1u, a.wait_cycles)) {
                            if (!s_abort) { s_abort = 1; atomicExch(a.status, 2); }
                            stop = true;
                            break;
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    if (issued >= a.inflight) {
                        // Keep at most `inflight` stages on their way: everything outstanding queues in front of the loads
                        // with which the consumers fetch a product's input vector.
                        const uint32_t old = issued - a.inflight, os = old % a.nstages;
                        if (!s_abort && !mbar_wait_bounded(smem_u32(full + os), (old / a.nstages) & 1u, a.wait_cycles)) {
                            s_abort = 1; atomicExch(a.status, 2);
                            stop = true;
                            break;
                        }
                    }
                    uint8_t *stage = smem + a.stage_base + (size_t)s * a.stage_stride;
                    const uint32_t bar = smem_u32(full + s);
                    // a tensor's bytes of the tile from the 16-byte boundary at or before the first to the one at or before the
                    // end; bytes past that boundary come by plain loads, so that no copy reads beyond the tensor
                    auto span = [&](const uint8_t *wb, uint8_t *dst, uintptr_t &from, uint32_t &bytes) {
                        const uintptr_t src = reinterpret_cast<uintptr_t>(wb) + (size_t)t.row0 * rb, end = src + (size_t)t.n * rb;
                        from = src & ~(uintptr_t)15;
                        const uintptr_t upto = end & ~(uintptr_t)15;
                        for (uintptr_t q = upto; q < end; q += 2)
                            *reinterpret_cast<uint16_t *>(dst + (q - from)) = *reinterpret_cast<const uint16_t *>(q);
                        bytes = (uint32_t)(upto - from);
                    };
                    uintptr_t f0 = 0, f1 = 0;
                    uint32_t n0 = 0, n1 = 0;
                    span(P.seg[t.seg].w, stage, f0, n0);
                    if (two) span(P.seg[t.seg].w2, stage + hs, f1, n1);
                    mbar_expect_tx(bar, n0 + n1);
                    bulk_g2s_hint(smem_u32(stage), reinterpret_cast<const void *>(f0), n0, bar, stream_policy);
                    if (two) bulk_g2s_hint(smem_u32(stage + hs), reinterpret_cast<const void *>(f1), n1, bar, stream_policy);
                    ++issued;
                    if (first_tile) { CHAIN_STAMP(a, p, 6); first_tile = false; }
                    if (++s == a.nstages) { s = 0; ++k; }
                }
                CHAIN_STAMP(a, p, 7);
            }
            if (s_abort) {   // give copies still in flight a bounded time to land before this warp leaves
                for (uint32_t q = 0; q < a.nstages && q < issued; ++q) {
                    const uint32_t last = ((issued - 1 - q) / a.nstages) * a.nstages + q;   // newest tile issued into stage q
                    mbar_wait_bounded(smem_u32(full + q), (last / a.nstages) & 1u, a.wait_cycles);
                }
            }
        }
        return;
    }

    // ---- consumers
    uint32_t s = 0, parity = 0;
    unsigned long long *best = s_best + (tid >> 5);
    if (lane == 0) *best = 0ull;
    for (uint32_t p = 0; p < a.nprods; ++p) {
        const ChainProd &P = desc[p % 3];
        // the next product's descriptor goes into the buffer that held product p - 2, which every thread has left
        if (p + 1 < a.nprods && tid < 16) cp_async16(smem_u32(&desc[(p + 1) % 3]) + 16 * tid, reinterpret_cast<const uint8_t *>(&a.prods[p + 1]) + 16 * tid);
        const bool unpack = P.mode == CHAIN_MODE_UNPACK;
        const uint32_t lo = B * P.rows_q + (B < P.rows_r ? B : P.rows_r), hi = (B + 1) * P.rows_q + (B + 1 < P.rows_r ? B + 1 : P.rows_r);
        if (lo >= hi) {          // no row of this product here: nothing to wait for, nothing to write
            cp_async_wait_all();
            named_bar_sync(PIPE_BAR_CONSUMERS, CHAIN_CONSUMERS);
            continue;
        }
        if (tid == 0) CHAIN_STAMP(a, p, 0);
        if (tid == 0) CHAIN_STAMP(a, p, 1);
        if (unpack) {
            chain_unpack<CHAIN_CONSUMERS>(a, P, lo, hi, base, &s_abort);
            continue;
        }
        if constexpr (FMTS == (1 << FMT_Q8_0)) {
            chain_product<FMT_Q8_0, NP>(a, P, smem, full, empty, lo, hi, s, parity, base, &s_abort, best, p);
        } else {
            chain_dispatch<NP>(a, P, smem, full, empty, lo, hi, s, parity, base, &s_abort, best, p);
        }
        named_bar_sync(PIPE_BAR_CONSUMERS, CHAIN_CONSUMERS);      // every thread has issued its stores of this product
        if (tid == 0) CHAIN_STAMP(a, p, 5);
    }

    // ---- arg-max epilogue: the CTA's best candidate, then the last CTA to arrive reduces all of them
    if (a.argmax_out) {
        named_bar_sync(PIPE_BAR_CONSUMERS, CHAIN_CONSUMERS);
        if (tid < 32) {
            unsigned long long m = tid < CHAIN_CONSUMERS / 32 ? s_best[tid] : 0ull;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, m, o);
                if (other > m) m = other;
            }
            if (tid == 0) *reinterpret_cast<volatile unsigned long long *>(a.argmax_part + B) = m;
        }
    }
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.arrived, 1u) == G - 1) {
            __threadfence();
            if (a.argmax_out) {
                unsigned long long m = 0ull;
                for (uint32_t b = 0; b < G; ++b) {
                    const unsigned long long c = *reinterpret_cast<const volatile unsigned long long *>(a.argmax_part + b);
                    if (c > m) m = c;
                }
                *a.argmax_out = m ? argmax_unrank(~(uint32_t)m) : 0u;     // no candidate at all: index 0, like the reference
            }
            *reinterpret_cast<volatile unsigned int *>(a.arrived) = 0;
            *reinterpret_cast<volatile unsigned int *>(a.gen) = base + a.nprods;
        }
    }
}

}  // namespace orome
