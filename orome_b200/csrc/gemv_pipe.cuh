// gemv_pipe.cuh -- the decode matvec kernel for sm_100a.
//
// Design (HBM-bound byte work, no tensor cores):
//   * The packed rows a CTA owns are one contiguous byte range of the tensor.
//     A producer warp streams that range into a ring of shared-memory stages
//     with 1-D bulk async copies (cp.async.bulk ... mbarrier::complete_tx), several
//     stages deep, so tens of KB per SM are in flight without spending registers.
//     Consumer warps hand a stage back through a second ("empty") barrier; there
//     is no block-wide synchronisation in the main loop.
//   * Consumer threads are arranged in row groups: a group of warps covers the
//     columns of one row, rows_par groups work on different rows side by side.
//     Every thread owns a fixed 64-weight column slot ("unit" x "part") and keeps
//     its slice of x in registers for the whole kernel, as per-group fixed point:
//     x_i ~= s * X_i with X_i a 16- or 24-bit integer split into bytes (top byte
//     signed, lower bytes unsigned).  The packed weights are multiplied against
//     those bytes with dp4a, so the integer dot products are exact and the only
//     approximation is the fixed-point rounding of x (2^-23 or 2^-15 of the
//     group's max).  x is quantized once per CTA, cooperatively and with
//     coalesced loads, into shared memory; each thread then picks up its slice.
//   * A row's partial sums are added inside each warp by shuffles; the per-warp
//     sums of a batch of rows wait in shared memory and all consumer threads add
//     them up together, one barrier per batch, writing y (or silu(g)*u for the
//     fused gate/up form) with coalesced stores.
//   * The producer starts its copies before griddepcontrol.wait, so under
//     programmatic dependent launch they overlap the previous kernel's tail; only
//     x (the previous kernel's output) is read after the wait.  CTAs are sized so
//     that two fit on an SM, which lets the next kernel's CTA become resident
//     beside a running one.
//   * Every wait on a copy barrier is bounded by a timer; on expiry the kernel
//     records a code in the status word, stops waiting and runs to completion.
#pragma once
#include "decode.cuh"

namespace orome {

constexpr int PIPE_MAX_SEG = 8;
constexpr int PIPE_MAX_PEERS = 7;
constexpr int PIPE_MAX_STAGES = 16;
constexpr int PIPE_MAX_CONSUMERS = 480;          // 15 consumer warps + the producer warp = 512 threads
constexpr int PIPE_MAX_THREADS = PIPE_MAX_CONSUMERS + 32;
constexpr int PIPE_CONSUMERS_2CTA = 288;           // consumer threads of a CTA meant to share an SM with another
constexpr int PIPE_THREADS_2CTA = PIPE_CONSUMERS_2CTA + 32;
constexpr int PIPE_MAX_ITERS = 8;               // rows a group handles per tile
constexpr int PIPE_MAX_ROWS_PAR = 15;           // row groups side by side (one warp each for the narrowest rows)
constexpr int PIPE_BAR_CONSUMERS = 9;           // named barrier over all consumer threads
constexpr long long PIPE_WAIT_CYCLES = 2000000000ll;   // per wait: about one second of SM clock

struct PipeSeg {
    const uint8_t *w;     // tensor (gate tensor in the fused form)
    const uint8_t *w2;    // up tensor in the fused form, else unused
    float *y;             // output rows of this segment
    uint32_t rows;
    uint32_t vstart;      // first virtual row (segments are concatenated)
};

struct PipeArgs {
    PipeSeg seg[PIPE_MAX_SEG];
    int nseg;
    const float *x;
    uint32_t in_dim, row_bytes;
    uint32_t units;            // column units per row (64 weights for Q8_0, one superblock for K-quants)
    uint32_t group_threads;    // consumer threads per row group: parts*units rounded up to a warp multiple
    uint32_t rows_par;         // row groups working side by side
    uint32_t iters;            // rows per group per tile; a tile is rows_par*iters rows
    uint32_t nstages;
    uint32_t stage_stride;     // bytes between stages
    uint32_t half_stride;      // offset of the second tensor's rows inside a stage (fused form)
    uint32_t stage_base;       // offset of stage 0 in dynamic shared memory
    uint32_t red_base;         // offset of the per-row partial-sum buffers
    uint32_t red_rows;         // rows one partial-sum buffer holds before it is flushed
    uint32_t xs_base;          // offset of the quantized copy of x (byte planes, scales, sums)
    uint32_t total_rows;
    int layout;
    int *status;
    const uint8_t *pf_ptr;     // weights of the launch that follows (16-byte aligned), or NULL
    uint64_t pf_bytes;         // how many of its leading bytes to pull into L2
    unsigned long long *trace; // diagnostics: 8 %globaltimer stamps per CTA, or NULL
    // MoE forms.  seg_expert: segment s reads expert seg_expert[s] of a 3-D expert tensor, i.e. its weights start
    // at seg[s].w + seg_expert[s] * w_stride (w2_stride for the second tensor); NULL = plain tensors.
    const uint32_t *seg_expert;
    uint64_t w_stride, w2_stride;
    // Combine form (expert down projection): every segment has its own input vector x + s * x_stride, every CTA
    // owns the same row range of all segments and writes y[r] = sum_s seg_weight[s] * (W_s x_s)[r] to seg[0].y.
    uint32_t x_stride;         // floats between the segments' input vectors
    const float *seg_weight;   // [nseg]
    uint32_t acc_base;         // offset of the fp32 accumulators of the CTA's rows
    // Token batches of the MoE forms: blockIdx.y = token.  Token t reads x + t * tok_x_stride, selects its experts and
    // weights at seg_expert / seg_weight + t * tok_sel_stride and writes every segment's output tok_y_stride floats
    // behind token 0's.  All zero for single-token launches.
    uint32_t tok_x_stride, tok_y_stride, tok_sel_stride;
    uint32_t xq_vec_bytes;     // bytes of one quantized input vector in shared memory
    // Multi-GPU (row-split) forms.  A gathered vector lives in every rank's gather arena as 8-byte slots
    // {value, tag}: slot of the float at arena address A = ll_origin + 2 * (A - arena_base).  Publishing: every y
    // value goes, with tag = *pub_gen + 1, into the local slot and into the same slot of each peer (peer address =
    // local address + peer_delta[p]); the last CTA of the grid then stores the tag to *pub_gen.  Value and tag
    // travel in one 8-byte store, so no fence and no separate flag are needed.  Waiting: x is read from its slots
    // (x_ll) and every element is polled until its tag equals *wait_gen -- this rank published its own slice of
    // that vector with the same tag in an earlier launch of the stream.  The generation words live in device
    // memory, so a captured graph can be replayed.
    int npeers;
    long long peer_delta[PIPE_MAX_PEERS];
    const uint8_t *arena_base;                // this rank's arena
    uint8_t *ll_origin;                       // its slot region
    unsigned int *pub_gen;                    // generation of the vector being published
    unsigned int *pub_arrived;                // CTAs of this launch that finished publishing
    const uint2 *x_ll;                        // slots of x, or NULL when x is a plain vector
    const unsigned int *wait_gen;             // generation x must carry
    long long wait_cycles;                    // bound of the polls of a gathered x
    // Fused neighbours of the product (single-tensor plain form).  Prologue: x is normalised while it is read,
    // x[c] * rsqrt(sum(norm_parts) / in_dim + norm_eps) * bf16(norm_w[c]).  Epilogue: y[r] = clamp(res_in[r] + (W x)[r])
    // and every CTA leaves the sum of squares of its y values in res_parts[blockIdx.x] (entries past the grid are zeroed).
    const uint16_t *norm_w;
    const float *norm_parts;
    float norm_eps;
    const float *res_in;
    float *res_parts;
};
constexpr int PIPE_SUM_SQ_PARTS = 512;          // length of a sum-of-squares partials array

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// The same copy with an L2 eviction policy.  Weights are read exactly once per step: marked evict-first they do not
// push the small vectors that the products hand to one another out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void stamp(unsigned long long *trace, int k)
{
    if (trace) trace[(size_t)blockIdx.x * 8 + k] = global_ns();
}
// Two {value, tag} slots in one 16-byte load that is not served from L1 (the peers write these slots).
__device__ __forceinline__ uint4 ld_slots2(const uint2 *p)
{
    uint4 v;
#if OROME_SLOT_LD == 1
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
#elif OROME_SLOT_LD == 2
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
#else
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
#endif
    return v;
}
__device__ __forceinline__ void st_slot(uint2 *p, float v, unsigned int tag)
{
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
// Four consecutive floats of a gathered vector from their slots, polled until all four carry `tag`
// (at most PIPE_WAIT_CYCLES; *ok is cleared on expiry and whatever is there is returned).
// Expiry is sticky: once *ok is false this thread polls no more, and every so often the poll looks at the
// context's status word, so one lost peer costs a launch one wait, not one wait per element.
__device__ __forceinline__ float4 ld_gathered4(const uint2 *slots, unsigned int tag, bool *ok, long long limit = PIPE_WAIT_CYCLES,
                                               const int *status = nullptr)
{
    uint4 a = ld_slots2(slots), b = ld_slots2(slots + 2);
    if ((a.y != tag || a.w != tag || b.y != tag || b.w != tag) && *ok) {
        const long long t0 = clock64();
        for (uint32_t it = 0;; ++it) {
            a = ld_slots2(slots); b = ld_slots2(slots + 2);
            if (a.y == tag && a.w == tag && b.y == tag && b.w == tag) break;
            if (clock64() - t0 > limit) { *ok = false; break; }
            if (status && (it & 255u) == 255u && *reinterpret_cast<const volatile int *>(status) != 0) { *ok = false; break; }
        }
    }
    return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Wait for a phase of a copy barrier, at most PIPE_WAIT_CYCLES.  Returns false on expiry.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit = PIPE_WAIT_CYCLES)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) return false;
    }
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c)
{
    int d; asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c)
{
    int d; asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c)
{
    uint32_t d; asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"((uint32_t)c)); return (int)d;
}

// Shared-memory loads by 32-bit shared-space address with a compile-time byte offset: one instruction each,
// no generic-address arithmetic.  volatile keeps them behind the barrier wait that publishes the stage.
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds16(uint32_t a)
{
    uint32_t v;
    asm volatile("{\n .reg .u16 t;\n ld.shared.u16 t, [%1+%2];\n cvt.u32.u16 %0, t;\n}\n" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
    return v;
}

// Quantized x in shared memory: NP byte planes of in_dim bytes (plane p holds byte p of every X_i), then one
// fp32 scale per group of G elements, then (Q4_K/Q5_K) one fp32 sum of x per 32 elements.
struct XqView {
    const uint8_t *planes;   // plane p at planes + p * in_dim
    const float *scales;     // [in_dim / G]
    const float *sums;       // [in_dim / 32] (K-quants with a min term)
    uint32_t in_dim;
};

// 16-byte pieces of a plane are permuted inside each aligned group of eight (128 bytes) so that threads
// whose slices start 64 or 256 bytes apart read different banks: piece c lives at plane_swz(c).
__device__ __forceinline__ uint32_t plane_swz(uint32_t c) { return (c & ~7u) | ((c ^ (c >> 3) ^ (c >> 4)) & 7u); }

// ---- x as per-group fixed point -------------------------------------------
// pc[p][k]: byte p of X_{4k..4k+3}, packed little-endian; piece NP-1 is the signed top byte.
template <int NP, int N>
struct XGroup {
    uint32_t pc[NP][N / 4];
    float scale;
};

template <int NP, int G>
__device__ __forceinline__ XqView make_xq_view(const uint8_t *xq, uint32_t in_dim)
{
    XqView xv;
    xv.planes = xq;
    xv.scales = reinterpret_cast<const float *>(xq + (size_t)NP * in_dim);
    xv.sums = xv.scales + in_dim / G;
    xv.in_dim = in_dim;
    return xv;
}

// N/4 words of every plane for N consecutive elements starting at element e0 (multiple of 16)
template <int NP, int N>
__device__ __forceinline__ void load_group(const XqView &xv, uint32_t e0, uint32_t scale_idx, XGroup<NP, N> &g)
{
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        const uint4 *plane = reinterpret_cast<const uint4 *>(xv.planes + (size_t)p * xv.in_dim);
#pragma unroll
        for (int k = 0; k < N / 16; ++k) {
            const uint4 w = plane[plane_swz(e0 / 16 + k)];
            g.pc[p][4 * k] = w.x; g.pc[p][4 * k + 1] = w.y; g.pc[p][4 * k + 2] = w.z; g.pc[p][4 * k + 3] = w.w;
        }
    }
    g.scale = xv.scales[scale_idx];
}

// sum_i q_i X_i from per-byte partial dot products I[p] = sum_i q_i * byte_p(X_i)
template <int NP>
__device__ __forceinline__ float combine(const int (&I)[NP])
{
    if constexpr (NP == 3) return fmaf((float)I[2], 65536.0f, (float)(I[1] * 256 + I[0]));
    else return (float)(I[1] * 256 + I[0]);
}

// unsigned weight bytes against the pieces of one word of x
template <int NP, int N>
__device__ __forceinline__ void dot_u(uint32_t q, const XGroup<NP, N> &g, int k, int (&I)[NP])
{
#pragma unroll
    for (int p = 0; p < NP; ++p) I[p] = (p == NP - 1) ? dp4a_us(q, g.pc[p][k], I[p]) : dp4a_uu(q, g.pc[p][k], I[p]);
}
// signed weight bytes
template <int NP, int N>
__device__ __forceinline__ void dot_s(uint32_t q, const XGroup<NP, N> &g, int k, int (&I)[NP])
{
#pragma unroll
    for (int p = 0; p < NP; ++p) I[p] = (p == NP - 1) ? dp4a_ss(q, g.pc[p][k], I[p]) : dp4a_su(q, g.pc[p][k], I[p]);
}

// ---- x in shared memory, quantized once per CTA --------------------------------------------
// Layout at xq: NP byte planes of in_dim bytes (plane p holds byte p of every X_i), then one fp32
// scale per group of G elements, then (Q4_K/Q5_K only) one fp32 sum of x per 32 elements.

// Cooperative pass over x by `nthreads` consumer threads (whole warps): every lane owns 4
// consecutive floats, a group of G elements is G/4 adjacent lanes.
// `nvec` vectors of in_dim floats, x_stride floats apart, are quantized in one pass (all loads of a batch are in
// flight together); vector v goes to xq + v * vec_bytes.  in_dim is a multiple of 32, so groups never straddle vectors.
// With `slots` set, x is a gathered vector: its elements come from {value, tag} slots and are polled for `tag`;
// the return value is false when a poll expired.
// One four-float piece (piece number f of its vector) into the quantized copy at xq: the lanes of a group agree on the
// group's scale by shuffles, so whole warps must call this together (`valid` false for lanes past the end).
template <int NP, int G, bool SUMS>
__device__ __forceinline__ void quantize_piece(const float4 v, uint32_t f, bool valid, uint32_t lane, uint8_t *xq, uint32_t in_dim)
{
    constexpr float QMAX = NP == 3 ? 8388607.0f : 32767.0f;
    const uint32_t n4 = in_dim / 4;
    uint32_t *planes = reinterpret_cast<uint32_t *>(xq);
    float *scales = reinterpret_cast<float *>(xq + (size_t)NP * in_dim);
    float *sums = scales + in_dim / G;
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 1; o < G / 4; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float inv = amax > 0.0f ? QMAX / amax : 0.0f;
    int X[4];
    X[0] = __float2int_rn(v.x * inv); X[1] = __float2int_rn(v.y * inv);
    X[2] = __float2int_rn(v.z * inv); X[3] = __float2int_rn(v.w * inv);
#pragma unroll
    for (int j = 0; j < 4; ++j) X[j] = max(-(int)QMAX, min((int)QMAX, X[j]));
    float sum = 0.0f;
    if constexpr (SUMS) {
        sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    if (valid) {
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            const uint32_t sel = (uint32_t)p | ((uint32_t)(4 + p) << 4);
            const uint32_t lo = __byte_perm((uint32_t)X[0], (uint32_t)X[1], sel);
            const uint32_t hi = __byte_perm((uint32_t)X[2], (uint32_t)X[3], sel);
            planes[(size_t)p * n4 + 4 * plane_swz(f >> 2) + (f & 3u)] = __byte_perm(lo, hi, 0x5410);
        }
        if ((lane & (G / 4 - 1)) == 0) scales[f / (G / 4)] = amax / QMAX;
        if constexpr (SUMS)
            if ((lane & 7u) == 0) sums[f / 8] = sum;
    }
}

template <int NP, int G, bool SUMS>
__device__ __forceinline__ bool quantize_x_to_smem(const float *__restrict__ x, uint32_t in_dim, uint32_t nvec, uint32_t x_stride,
                                                   uint8_t *xq0, uint32_t vec_bytes, uint32_t tid, uint32_t nthreads,
                                                   const uint2 *slots = nullptr, unsigned int tag = 0,
                                                   long long limit = PIPE_WAIT_CYCLES, const int *status = nullptr, uint32_t rot = 0,
                                                   const uint16_t *norm_w = nullptr, float rms = 1.0f, uint32_t issued_bar = 0)
{
    // issued_bar: shared address of an mbarrier on which every warp arrives once the loads of its first batch are on
    // their way (0: none).  The weight producer holds its copies back until then, see the kernel.
    // rot (single vector only; a multiple of 32 four-float pieces): this CTA walks the vector starting rot pieces in and
    // wraps around.  When every CTA of a grid reads the same vector at the same moment, different rot values keep them
    // on different cache lines (L2 slices) at any one time instead of all queueing on the same line.
    bool ok = true;
    constexpr int BATCH = 8;
    const uint32_t n4 = in_dim / 4, n4_all = n4 * nvec, lane = tid & 31u;
    if (issued_bar && slots) {      // a gathered x is polled until the peers have written it: nothing to order the copies behind
        __syncwarp();
        if (lane == 0) mbar_arrive(issued_bar);
        issued_bar = 0;
    }
    for (uint32_t base = tid - lane; base < n4_all; base += nthreads * BATCH) {
        float4 v[BATCH];
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const uint32_t fa = base + b * nthreads + lane;
            const uint32_t vec = nvec == 1 ? 0u : fa / n4;      // no division on the single-vector path
            uint32_t fl = fa - vec * n4;
            if (nvec == 1) { fl += rot; if (fl >= n4) fl -= n4; }
            if (slots) v[b] = fa < n4_all ? ld_gathered4(slots + 4 * (size_t)fl, tag, &ok, limit, status) : make_float4(0.f, 0.f, 0.f, 0.f);
            else v[b] = fa < n4_all ? __ldcg(reinterpret_cast<const float4 *>(x + (size_t)vec * x_stride) + fl) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (norm_w && fa < n4_all) {      // the RMS-norm scale and the bf16 norm weights, applied in the reference's order
                const uint2 w = __ldg(reinterpret_cast<const uint2 *>(norm_w) + fl);
                v[b].x = v[b].x * rms * __uint_as_float(w.x << 16);
                v[b].y = v[b].y * rms * __uint_as_float(w.x & 0xffff0000u);
                v[b].z = v[b].z * rms * __uint_as_float(w.y << 16);
                v[b].w = v[b].w * rms * __uint_as_float(w.y & 0xffff0000u);
            }
        }
        if (issued_bar && base == tid - lane) {
            __syncwarp();
            if (lane == 0) mbar_arrive(issued_bar);
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const uint32_t fb = base + b * nthreads;       // warp-uniform
            if (fb >= n4_all) break;
            const uint32_t fa = fb + lane;
            const uint32_t vec = nvec == 1 ? 0u : fa / n4;
            uint32_t f = fa - vec * n4;
            if (nvec == 1) { f += rot; if (f >= n4) f -= n4; }
            quantize_piece<NP, G, SUMS>(v[b], f, fa < n4_all, lane, xq0 + (size_t)vec * vec_bytes, in_dim);
        }
    }
    if (issued_bar && tid - lane >= n4_all) {      // a warp without a piece of x arrives all the same
        __syncwarp();
        if (lane == 0) mbar_arrive(issued_bar);
    }
    return ok;
}

// The same pass for one vector whose elements come from {value, tag} slots: the loads of a batch are issued together
// (one round trip instead of one per piece), then the tags are checked and only a piece whose tag is not there yet is
// polled (bounded; *ok false on expiry).  rot as above.
template <int NP, int G, bool SUMS>
__device__ __forceinline__ bool quantize_slots_to_smem(const uint2 *slots, unsigned int tag, uint32_t in_dim, uint8_t *xq, uint32_t tid,
                                                       uint32_t nthreads, long long limit, const int *status, uint32_t rot,
                                                       unsigned long long *stamps = nullptr)
{
    bool ok = true;
    constexpr int BATCH = 4;
    const uint32_t n4 = in_dim / 4, lane = tid & 31u;
    for (uint32_t base = tid - lane; base < n4; base += nthreads * BATCH) {
        uint4 lo[BATCH], hi[BATCH];
        if (stamps && base == tid) stamps[0] = global_ns();
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const uint32_t fa = base + b * nthreads + lane;
            uint32_t fl = fa + rot;
            if (fl >= n4) fl -= n4;
            lo[b] = hi[b] = make_uint4(0u, tag, 0u, tag);
            if (fa < n4) { lo[b] = ld_slots2(slots + 4 * (size_t)fl); hi[b] = ld_slots2(slots + 4 * (size_t)fl + 2); }
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const uint32_t fb = base + b * nthreads;       // warp-uniform
            if (fb >= n4) break;
            const uint32_t fa = fb + lane;
            uint32_t f = fa + rot;
            if (f >= n4) f -= n4;
            float4 v = make_float4(__uint_as_float(lo[b].x), __uint_as_float(lo[b].z), __uint_as_float(hi[b].x), __uint_as_float(hi[b].z));
            if (lo[b].y != tag || lo[b].w != tag || hi[b].y != tag || hi[b].w != tag) v = ld_gathered4(slots + 4 * (size_t)f, tag, &ok, limit, status);
            if (stamps && b == 0 && base == tid) stamps[1] = global_ns();
            quantize_piece<NP, G, SUMS>(v, f, fa < n4, lane, xq, in_dim);
        }
    }
    return ok;
}

// 16 (8) bytes from a shared address that is only 2-byte aligned: aligned words around it, fixed up with prmt.
__device__ __forceinline__ void lds16_a2(uint32_t a, uint32_t (&o)[4])
{
    const uint32_t q = a & ~3u, sel = (a & 2u) ? 0x5432u : 0x3210u;
    const uint32_t v0 = lds32<0>(q), v1 = lds32<4>(q), v2 = lds32<8>(q), v3 = lds32<12>(q), v4 = lds32<16>(q);
    o[0] = __byte_perm(v0, v1, sel); o[1] = __byte_perm(v1, v2, sel);
    o[2] = __byte_perm(v2, v3, sel); o[3] = __byte_perm(v3, v4, sel);
}
__device__ __forceinline__ void lds8_a2(uint32_t a, uint32_t (&o)[2])
{
    const uint32_t q = a & ~3u, sel = (a & 2u) ? 0x5432u : 0x3210u;
    const uint32_t v0 = lds32<0>(q), v1 = lds32<4>(q), v2 = lds32<8>(q);
    o[0] = __byte_perm(v0, v1, sel); o[1] = __byte_perm(v1, v2, sel);
}

// Six-bit scales/mins of the sub-block pair (2g, 2g+1) from the three packed words
// (bytes 0-3, 4-7, 8-11).  Layout A: format.m:41-64; layout B: shaders.metal:1575-1578.
__device__ __forceinline__ void pair_scales(uint32_t w0, uint32_t w1, uint32_t w2, int layout, int g,
                                            uint32_t &scA, uint32_t &scB, uint32_t &mnA, uint32_t &mnB)
{
    int u = g & 1, sh = 16 * u;
    if (g < 2) {
        scA = (w0 >> sh) & 63u; scB = (w0 >> (sh + 8)) & 63u;
        mnA = (w1 >> sh) & 63u; mnB = (w1 >> (sh + 8)) & 63u;
    } else {
        uint32_t tA = ((w0 >> (sh + 6)) & 3u) << 4, tB = ((w0 >> (sh + 14)) & 3u) << 4;
        uint32_t uA = ((w1 >> (sh + 6)) & 3u) << 4, uB = ((w1 >> (sh + 14)) & 3u) << 4;
        if (layout == LAYOUT_A) {
            uint32_t sp = (w2 >> (8 * u)) & 255u, mp = (w2 >> (16 + 8 * u)) & 255u;
            scA = (sp & 15u) | tA; scB = (sp >> 4) | tB;
            mnA = (mp & 15u) | uA; mnB = (mp >> 4) | uB;
        } else {
            scA = ((w2 >> sh) & 15u) | tA;        mnA = ((w2 >> (sh + 4)) & 15u) | uA;
            scB = ((w2 >> (sh + 8)) & 15u) | tB;  mnB = ((w2 >> (sh + 12)) & 15u) | uB;
        }
    }
}

// ---- per-format column slots ----------------------------------------------
template <int FMT, int NP> struct Slot;

// Q8_0: unit = two blocks (68 bytes, 4-byte aligned), one part.  The first block's quants sit
// two bytes into their words (after the fp16 scale), so the thread keeps that block's x bytes
// shifted the same way, with zero bytes facing the scale bytes: nine dp4a per byte plane cover
// the unit's first nine words as they are, no realignment of the weights needed.
template <int NP>
struct Slot<FMT_Q8_0, NP> {
    static constexpr int PARTS = 1, UNIT_ELEMS = 64;
    static constexpr int GROUP = 32;
    static constexpr bool SUMS = false;
    uint32_t x0[NP][9];       // block 0, shifted by two bytes
    XGroup<NP, 32> g1;        // block 1, word aligned
    float s0;
    __device__ __forceinline__ void load(const XqView &xv, uint32_t unit, int)
    {
        XGroup<NP, 32> g0;
        load_group<NP, 32>(xv, unit * 64, unit * 2, g0);
        load_group<NP, 32>(xv, unit * 64 + 32, unit * 2 + 1, g1);
        s0 = g0.scale;
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            x0[p][0] = g0.pc[p][0] << 16;
#pragma unroll
            for (int j = 1; j < 8; ++j) x0[p][j] = __byte_perm(g0.pc[p][j - 1], g0.pc[p][j], 0x5432);
            x0[p][8] = g0.pc[p][7] >> 16;
        }
    }
    static constexpr uint32_t UNIT_BYTES = 68;
    // `u` = shared-space address of this thread's unit inside the row
    __device__ __forceinline__ float dot(uint32_t u, int, int) const
    {
        uint32_t v[17];
        v[0] = lds32<0>(u);   v[1] = lds32<4>(u);   v[2] = lds32<8>(u);   v[3] = lds32<12>(u);  v[4] = lds32<16>(u);
        v[5] = lds32<20>(u);  v[6] = lds32<24>(u);  v[7] = lds32<28>(u);  v[8] = lds32<32>(u);  v[9] = lds32<36>(u);
        v[10] = lds32<40>(u); v[11] = lds32<44>(u); v[12] = lds32<48>(u); v[13] = lds32<52>(u); v[14] = lds32<56>(u);
        v[15] = lds32<60>(u); v[16] = lds32<64>(u);
        int I0[NP], I1[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) { I0[p] = 0; I1[p] = 0; }
#pragma unroll
        for (int j = 0; j < 9; ++j) {
#pragma unroll
            for (int p = 0; p < NP; ++p)
                I0[p] = (p == NP - 1) ? dp4a_ss(v[j], x0[p][j], I0[p]) : dp4a_su(v[j], x0[p][j], I0[p]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) dot_s<NP, 32>(v[9 + j], g1, j, I1);
        float d0 = __half2float(__ushort_as_half((unsigned short)(v[0] & 0xffffu)));
        float d1 = __half2float(__ushort_as_half((unsigned short)(v[8] >> 16)));
        return fmaf(d0 * s0, combine<NP>(I0), d1 * g1.scale * combine<NP>(I1));
    }
};

// Q4_K / Q5_K: unit = superblock, part g = the 64 weights of sub-blocks 2g, 2g+1.
template <int FMT, int NP>
struct SlotK45 {
    static constexpr int PARTS = 4, UNIT_ELEMS = 256;
    XGroup<NP, 32> a, b;
    float sumA, sumB;
    static constexpr int GROUP = 32;
    static constexpr bool SUMS = true;
    __device__ __forceinline__ void load(const XqView &xv, uint32_t unit, int g)
    {
        const uint32_t e0 = unit * 256 + 64 * g;
        load_group<NP, 32>(xv, e0, e0 / 32, a);
        load_group<NP, 32>(xv, e0 + 32, e0 / 32 + 1, b);
        sumA = xv.sums[e0 / 32];
        sumB = xv.sums[e0 / 32 + 1];
    }
    static constexpr uint32_t UNIT_BYTES = FMT == FMT_Q4_K ? 144 : 176;
    // `sb` = shared-space address of this thread's superblock inside the row
    __device__ __forceinline__ float dot(uint32_t sb, int g, int layout) const
    {
        constexpr int QOFF = FMT == FMT_Q4_K ? 16 : 48;
        const uint4 h = lds128<0>(sb);
        const uint32_t qa = sb + 32u * (uint32_t)g;
        const uint4 q0 = lds128<QOFF>(qa), q1 = lds128<QOFF + 16>(qa);
        uint32_t ql[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t qh[8];
        if constexpr (FMT == FMT_Q5_K) {
            const uint4 h0 = lds128<16>(sb), h1 = lds128<32>(sb);
            qh[0] = h0.x; qh[1] = h0.y; qh[2] = h0.z; qh[3] = h0.w;
            qh[4] = h1.x; qh[5] = h1.y; qh[6] = h1.z; qh[7] = h1.w;
        }
        int IA[NP], IB[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) { IA[p] = 0; IB[p] = 0; }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t lo = ql[k] & 0x0F0F0F0Fu, hi = (ql[k] >> 4) & 0x0F0F0F0Fu;
            if constexpr (FMT == FMT_Q5_K) {
                uint32_t t = qh[k] >> (2 * g);
                lo |= (t & 0x01010101u) << 4;
                hi |= (t & 0x02020202u) << 3;
            }
            dot_u<NP, 32>(lo, a, k, IA);
            dot_u<NP, 32>(hi, b, k, IB);
        }
        uint32_t scA, scB, mnA, mnB;
        pair_scales(h.y, h.z, h.w, layout, g, scA, scB, mnA, mnB);
        float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        float pos = fmaf((float)scA * a.scale, combine<NP>(IA), (float)scB * b.scale * combine<NP>(IB));
        float neg = fmaf((float)mnA, sumA, (float)mnB * sumB);
        return fmaf(d, pos, -dmin * neg);
    }
};
template <int NP> struct Slot<FMT_Q4_K, NP> : SlotK45<FMT_Q4_K, NP> {};
template <int NP> struct Slot<FMT_Q5_K, NP> : SlotK45<FMT_Q5_K, NP> {};

// Q6_K: unit = superblock (210 bytes, 2-byte aligned), part = (half, lh): the 64 weights
// at positions 128*half + 32*t + 16*lh + (0..15), t = 0..3, each 16-group with its own scale.
template <int NP>
struct Slot<FMT_Q6_K, NP> {
    static constexpr int PARTS = 4, UNIT_ELEMS = 256;
    XGroup<NP, 16> g[4];
    int sx[4][NP];   // sum of the piece bytes, for the -32 offset of the 6-bit quants
    static constexpr int GROUP = 16;
    static constexpr bool SUMS = false;
    __device__ __forceinline__ void load(const XqView &xv, uint32_t unit, int part)
    {
        const uint32_t e0 = unit * 256 + 128 * (part >> 1) + 16 * (part & 1);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            load_group<NP, 16>(xv, e0 + 32 * t, (e0 + 32 * t) / 16, g[t]);
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                int s = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    s = (p == NP - 1) ? dp4a_us(0x01010101u, g[t].pc[p][k], s) : dp4a_uu(0x01010101u, g[t].pc[p][k], s);
                sx[t][p] = s;
            }
        }
    }
    static constexpr uint32_t UNIT_BYTES = 210;
    __device__ __forceinline__ float dot(uint32_t sb, int part, int) const
    {
        int half = part >> 1, lh = part & 1;
        uint32_t qa[4], qb[4], qh[4], scw[2];
        lds16_a2(sb + 64 * half + 16 * lh, qa);
        lds16_a2(sb + 64 * half + 32 + 16 * lh, qb);
        lds16_a2(sb + 128 + 32 * half + 16 * lh, qh);
        lds8_a2(sb + 192 + 8 * half, scw);   // this half's 8 sub-scales; group t uses byte lh + 2t
        int I[4][NP];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int p = 0; p < NP; ++p) I[t][p] = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint32_t h = qh[k];
            dot_u<NP, 16>((qa[k] & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u), g[0], k, I[0]);
            dot_u<NP, 16>((qb[k] & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u), g[1], k, I[1]);
            dot_u<NP, 16>(((qa[k] >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u), g[2], k, I[2]);
            dot_u<NP, 16>(((qb[k] >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u), g[3], k, I[3]);
        }
        float d = __half2float(__ushort_as_half((unsigned short)lds16<208>(sb)));
        float acc = 0.0f;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            int J[NP];
#pragma unroll
            for (int p = 0; p < NP; ++p) J[p] = I[t][p] - 32 * sx[t][p];
            int sc = (int)(scw[t >> 1] << (24 - 8 * (lh + 2 * (t & 1)))) >> 24;   // sign-extended int8
            acc = fmaf((float)sc * g[t].scale, combine<NP>(J), acc);
        }
        return d * acc;
    }
};

// ---- tile walk -------------------------------------------------------------
struct PipeTile { int seg; uint32_t row0, n; };
struct PipeWalk { uint32_t cur, lo, hi; int seg; };

// Rows of this CTA.  Plain forms: a contiguous range of the concatenated (virtual) rows, walked once.
// Combine form: the same range of segment-local rows, walked once per segment.
template <bool COMBINE>
__device__ __forceinline__ void walk_init(const PipeArgs &a, PipeWalk &w)
{
    const uint32_t R = COMBINE ? a.seg[0].rows : a.total_rows;
    w.lo = (uint32_t)((uint64_t)blockIdx.x * R / gridDim.x);
    w.hi = (uint32_t)((uint64_t)(blockIdx.x + 1) * R / gridDim.x);
    w.cur = w.lo;
    w.seg = 0;
}

// Expert-parallel MoE: a segment whose device-side expert index is PIPE_NO_EXPERT belongs to another GPU and is
// stepped over by producer and consumers alike (no copy, no arithmetic, its rows are left unwritten).
constexpr uint32_t PIPE_NO_EXPERT = 0xFFFFFFFFu;
template <bool EXT>
__device__ __forceinline__ bool seg_skipped(const PipeArgs &a, int s)
{
    if constexpr (EXT) return a.seg_expert && a.seg_expert[blockIdx.y * a.tok_sel_stride + s] == PIPE_NO_EXPERT;
    else return false;
}

template <bool COMBINE, bool EXT = false>
__device__ __forceinline__ bool next_tile(const PipeArgs &a, PipeWalk &w, PipeTile &t)
{
    const uint32_t cap = a.rows_par * a.iters;
    if constexpr (COMBINE) {
        if (w.lo >= w.hi) return false;
        if (w.cur >= w.hi) { ++w.seg; w.cur = w.lo; }
        while (w.seg < a.nseg && seg_skipped<EXT>(a, w.seg)) ++w.seg;
        if (w.seg >= a.nseg) return false;
        uint32_t n = w.hi - w.cur;
        if (n > cap) n = cap;
        t.seg = w.seg; t.row0 = w.cur; t.n = n;
        w.cur += n;
        return true;
    } else {
        if (a.nseg == 1) {   // one tensor: no segment search, no segment clipping
            if (w.cur >= w.hi) return false;
            uint32_t n = w.hi - w.cur;
            if (n > cap) n = cap;
            t.seg = 0; t.row0 = w.cur; t.n = n;
            w.cur += n;
            return true;
        }
        for (;;) {
            if (w.cur >= w.hi) return false;
            int s = w.seg;
            while (s + 1 < a.nseg && w.cur >= a.seg[s + 1].vstart) ++s;
            w.seg = s;
            const uint32_t seg_end = a.seg[s].vstart + a.seg[s].rows;
            const uint32_t lim = w.hi < seg_end ? w.hi : seg_end;
            if (seg_skipped<EXT>(a, s)) { w.cur = lim; continue; }
            uint32_t n = lim - w.cur;
            if (n > cap) n = cap;
            t.seg = s; t.row0 = w.cur - a.seg[s].vstart; t.n = n;
            w.cur += n;
            return true;
        }
    }
}

template <bool EXT>
__device__ __forceinline__ const uint8_t *seg_w(const PipeArgs &a, int s)
{
    const uint8_t *p = a.seg[s].w;
    if constexpr (EXT) { if (a.seg_expert) p += (uint64_t)a.seg_expert[blockIdx.y * a.tok_sel_stride + s] * a.w_stride; }
    return p;
}
template <bool EXT>
__device__ __forceinline__ const uint8_t *seg_w2(const PipeArgs &a, int s)
{
    const uint8_t *p = a.seg[s].w2;
    if constexpr (EXT) { if (a.seg_expert) p += (uint64_t)a.seg_expert[blockIdx.y * a.tok_sel_stride + s] * a.w2_stride; }
    return p;
}

template <bool SWIGLU, bool EXT>
__device__ __forceinline__ void issue_tile(const PipeArgs &a, const PipeTile &t, uint8_t *stage, uint32_t bar)
{
    uint32_t tx = 0;
    uintptr_t a0[2], e1[2];
#pragma unroll
    for (int h = 0; h < (SWIGLU ? 2 : 1); ++h) {
        const uint8_t *base = h ? seg_w2<EXT>(a, t.seg) : seg_w<EXT>(a, t.seg);
        uintptr_t src = reinterpret_cast<uintptr_t>(base) + (size_t)t.row0 * a.row_bytes;
        uintptr_t end = src + (size_t)t.n * a.row_bytes;
        a0[h] = src & ~(uintptr_t)15;
        e1[h] = end & ~(uintptr_t)15;
        uint8_t *dst = stage + h * a.half_stride;
        // bytes past the last 16-byte boundary are fetched with plain loads so no copy reads beyond the tensor
        for (uintptr_t p = e1[h]; p < end; p += 2)
            *reinterpret_cast<uint16_t *>(dst + (p - a0[h])) = *reinterpret_cast<const uint16_t *>(p);
        tx += (uint32_t)(e1[h] - a0[h]);
    }
    mbar_expect_tx(bar, tx);
#pragma unroll
    for (int h = 0; h < (SWIGLU ? 2 : 1); ++h)
        bulk_g2s(smem_u32(stage + h * a.half_stride), reinterpret_cast<const void *>(a0[h]), (uint32_t)(e1[h] - a0[h]), bar);
}

// MODE 0: y = W x.  MODE 1: fused gate/up, y = silu(Wg x) * (Wu x).  MODE 2: combine, y = sum_s weight_s * (W_s x_s).
// EXT compiles in the expert indirection and the multi-GPU publish / wait paths; dense single-GPU launches use the
// EXT = false instance, which carries none of that code.
template <int FMT, int NP, int MODE, int MINB, bool EXT>
__global__ void __launch_bounds__(MINB == 2 ? PIPE_THREADS_2CTA : PIPE_MAX_THREADS, MINB)
gemv_pipe_kernel(const __grid_constant__ PipeArgs a)
{
    constexpr bool SWIGLU = MODE == 1, COMBINE = MODE == 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + PIPE_MAX_STAGES;
    float *red = reinterpret_cast<float *>(smem + a.red_base);
    uint8_t *stages = smem + a.stage_base;
    __shared__ volatile int s_abort;
    // x before weights: when this kernel's weights already sit in L2 (the previous launch prefetched them), a full ring
    // of copies requested at entry keeps the SM's inbound path busy for microseconds, and the loads of x -- which the
    // consumers can only issue once the previous kernel has finished -- queue behind all of it.  So the producer
    // requests its first tile at once and the rest only after every consumer warp has its loads of x on their way.
    __shared__ uint64_t s_x_issued;

    using SlotT = Slot<FMT, NP>;
    constexpr int P = SlotT::PARTS;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint32_t GT = a.group_threads, C = GT * a.rows_par, GW = GT >> 5;
    const uint32_t U = a.units;
    const bool producer = tid >= C;


    if (tid == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < a.nstages; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), C >> 5);
        }
        mbar_init(smem_u32(&s_x_issued), C >> 5);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    if (tid == 0) stamp(a.trace, 0);

    if (producer) {
        // The weight copies do not depend on the previous kernel: no griddepcontrol.wait on this path.
        if (lane == 0) {
            if constexpr (EXT) { if (a.seg_expert) pdl_wait(); }   // the expert indices are the previous kernel's output
            PipeWalk w;
            walk_init<COMBINE>(a, w);
            uint32_t i = 0, s = 0, k = 0;       // tile index, its stage and how many times the ring has wrapped
            PipeTile t;
            while (next_tile<COMBINE, EXT>(a, w, t)) {
                if (k > 0) {
                    if (s_abort || !mbar_wait_bounded(smem_u32(empty + s), (k - 1) & 1u)) {
                        if (!s_abort) { s_abort = 1; atomicExch(a.status, 2); }
                        break;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                issue_tile<SWIGLU, EXT>(a, t, stages + (size_t)s * a.stage_stride, smem_u32(full + s));
                ++i;
                if (++s == a.nstages) { s = 0; ++k; }
                if (i == 1) mbar_wait_bounded(smem_u32(&s_x_issued), 0);      // x first (see above); an expired wait only loses the ordering
            }
            stamp(a.trace, 1);
            // All of this CTA's rows are requested.  Pull the head of the next launch's weights into L2 so that HBM
            // keeps streaming while this grid drains and the next one starts.
            if (a.pf_ptr && !s_abort && blockIdx.y == 0) {
                const uint64_t per = (a.pf_bytes / gridDim.x) & ~(uint64_t)15;
                const uint8_t *p = a.pf_ptr + (uint64_t)blockIdx.x * per;
                for (uint64_t off = 0; off < per; off += 32768) {
                    const uint64_t n = per - off < 32768 ? per - off : 32768;
                    bulk_prefetch_l2(p + off, (uint32_t)n);
                }
            }
            if (s_abort) {   // give copies still in flight a bounded time to land before this warp leaves
                for (uint32_t s = 0; s < a.nstages && s < i; ++s) {
                    const uint32_t last = ((i - 1 - s) / a.nstages) * a.nstages + s;   // newest tile issued into stage s
                    mbar_wait_bounded(smem_u32(full + s), (last / a.nstages) & 1u);
                }
            }
        }
        return;
    }

    // ---- consumers ------------------------------------------------------------------------
    const uint32_t group = tid / GT, j = tid % GT, wig = j >> 5;
    const bool active = j < (uint32_t)P * U;
    const int part = (int)(j / U);
    const uint32_t unit = j % U;

    pdl_wait();   // x is the previous kernel's output
    if (tid == 0) stamp(a.trace, 2);

    SlotT slot;
    {
        uint8_t *xq = smem + a.xs_base;
        // a gathered x: every element is polled for the generation this rank gave its own slice (visible after the wait above)
        const uint2 *slots = EXT ? a.x_ll : nullptr;
        const unsigned int want = EXT && a.x_ll ? *reinterpret_cast<const volatile unsigned int *>(a.wait_gen) : 0u;
        const uint16_t *norm_w = EXT ? a.norm_w : nullptr;
        float rms = 1.0f;
        if (norm_w) {                         // every warp adds up the partial sums of squares for itself
            float t = 0.0f;
            for (uint32_t i = lane; i < (uint32_t)PIPE_SUM_SQ_PARTS; i += 32) t += __ldcg(a.norm_parts + i);
            rms = rsqrtf(warp_sum(t) / (float)a.in_dim + a.norm_eps);
        }
        if (!quantize_x_to_smem<NP, SlotT::GROUP, SlotT::SUMS>(a.x + (EXT ? (size_t)blockIdx.y * a.tok_x_stride : 0), a.in_dim, COMBINE ? (uint32_t)a.nseg : 1u, a.x_stride, xq, a.xq_vec_bytes, tid, C,
                                                               slots, want, a.wait_cycles, a.status,
                                                               COMBINE ? 0u : (uint32_t)((uint64_t)blockIdx.x * (a.in_dim / 4) / gridDim.x) & ~31u,
                                                               norm_w, rms, smem_u32(&s_x_issued))) {
            s_abort = 1;
            atomicExch(a.status, 3);
        }
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
        if (tid == 0) stamp(a.trace, 3);
        if constexpr (!COMBINE) {
            if (active) slot.load(make_xq_view<NP, SlotT::GROUP>(xq, a.in_dim), unit, part);
        }
        if (tid == 0) stamp(a.trace, 4);
    }

    // Per-row partial sums (one per warp of the row's group) collect in shared memory and are added up, a whole
    // batch of rows at a time, by all consumer threads: one consumer-wide barrier per batch, coalesced stores of y.
    // Two buffers alternate, so the barrier that opens a flush also protects the buffer written two flushes ago.
    const unsigned int pub_tag = EXT && a.npeers > 0 ? *reinterpret_cast<const volatile unsigned int *>(a.pub_gen) + 1u : 0u;
    const uint32_t CAP = a.red_rows, PLANE = CAP * GW;                 // floats per buffer (per tensor)
    PipeWalk wk;
    walk_init<COMBINE>(a, wk);
    float *accbuf = reinterpret_cast<float *>(smem + a.acc_base);
    if constexpr (COMBINE) {
        for (uint32_t r = tid; r < wk.hi - wk.lo; r += C) accbuf[r] = 0.0f;   // ordered before its first use by the first flush's barrier
    }
    float *pbuf = red;
    // Combine form with the CTA's rows fitting one buffer: every segment adds weight * partial sum into the same
    // slots (a slot always belongs to the same lane), so there is one flush at the end instead of one barrier and
    // flush per segment.
    // and the row groups split the SEGMENTS among them (group g takes segments g, g + rows_par, ...; all rows of a
    // segment's tile), each with its own slots: the eight experts of a token advance side by side.
    const uint32_t SL = COMBINE ? GW * a.rows_par : GW;                 // partial sums per row
    // (single-token launches only: a token batch gives every CTA hundreds of rows per segment, which all row groups share)
    const bool comb_acc = COMBINE && gridDim.y == 1 && (wk.hi - wk.lo) * SL <= 2 * PLANE;
    if (comb_acc) {
        for (uint32_t r = tid; r < (wk.hi - wk.lo) * SL; r += C) pbuf[r] = 0.0f;
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
    }
    uint32_t which = 0, buf_n = 0, buf_row0 = 0;
    int buf_seg = 0;
    float sq = 0.0f;                          // this thread's share of the sum of squares of the outputs (residual epilogue)
    auto flush = [&]() {
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
        const float *src = pbuf + (size_t)which * PLANE * (SWIGLU ? 2 : 1);
        float *y = a.seg[buf_seg].y + buf_row0 + (EXT ? (size_t)blockIdx.y * a.tok_y_stride : 0);
        for (uint32_t r = tid; r < buf_n; r += C) {
            float g = 0.0f, u = 0.0f;
            const uint32_t nsl = comb_acc ? SL : GW;
            for (uint32_t w = 0; w < nsl; ++w) {
                g += src[r * nsl + w];
                if constexpr (SWIGLU) u += src[PLANE + r * GW + w];
            }
            if constexpr (COMBINE) accbuf[buf_row0 - wk.lo + r] += (comb_acc ? 1.0f : a.seg_weight[blockIdx.y * a.tok_sel_stride + buf_seg]) * g;   // one owner per row and flush
            else {
                float val = SWIGLU ? silu_mul(g, u) : g;
                if constexpr (EXT && MODE == 0) {
                    if (a.res_in) {           // residual add, clamped to the fp16 range as the reference's kernel does
                        val = fminf(fmaxf(a.res_in[buf_row0 + r] + val, -65504.0f), 65504.0f);
                        sq = fmaf(val, val, sq);
                    }
                }
                y[r] = val;
                if constexpr (EXT) {
                    if (a.npeers > 0) {
                        uint8_t *slot = a.ll_origin + 2 * (reinterpret_cast<const uint8_t *>(y + r) - a.arena_base);
                        st_slot(reinterpret_cast<uint2 *>(slot), val, pub_tag);
                        for (int p = 0; p < a.npeers; ++p) st_slot(reinterpret_cast<uint2 *>(slot + a.peer_delta[p]), val, pub_tag);
                    }
                }
            }
        }
        which ^= 1u;
        buf_n = 0;
    };

    const uint32_t stages_s = smem_u32(stages);
    const uint32_t unit_off = unit * SlotT::UNIT_BYTES;
    uint32_t i = 0, s = 0, parity = 0;
    int slot_seg = -1, delta_seg = -1;
    uint32_t delta = 0, delta2 = 0;
    const bool rows16 = (a.row_bytes & 15u) == 0;     // then every row starts at the same offset inside its 16-byte piece
    PipeTile t;
    while (next_tile<COMBINE, EXT>(a, wk, t)) {
        if (!comb_acc && buf_n && (t.seg != buf_seg || buf_n + t.n > CAP)) flush();
        if (!comb_acc && buf_n == 0) { buf_seg = t.seg; buf_row0 = t.row0; }
        const bool mine = !comb_acc || (uint32_t)t.seg % a.rows_par == group;    // segment-parallel combine: one group per segment
        if constexpr (COMBINE) {
            if (mine && t.seg != slot_seg) {   // this segment's own input vector
                slot_seg = t.seg;
                if (active) slot.load(make_xq_view<NP, SlotT::GROUP>(smem + a.xs_base + (size_t)t.seg * a.xq_vec_bytes, a.in_dim), unit, part);
            }
            if (!mine) {                       // another group's segment: hand the stage on untouched (after its data
                                               // has landed, so that no warp gets a whole ring ahead of the barriers' phases)
                if (!s_abort && !mbar_wait_bounded(smem_u32(full + s), parity)) {
                    s_abort = 1;
                    atomicExch(a.status, 1);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(empty + s));
                buf_n = wk.hi - wk.lo; buf_seg = 0; buf_row0 = wk.lo;
                ++i;
                if (++s == a.nstages) { s = 0; parity ^= 1u; }
                continue;
            }
        }
        if (!s_abort && !mbar_wait_bounded(smem_u32(full + s), parity)) {
            s_abort = 1;
            atomicExch(a.status, 1);
        }
        if (i == 0 && tid == 0) stamp(a.trace, 5);
        if (!rows16 || t.seg != delta_seg) {   // offset of the tile's first byte inside its 16-byte piece
            delta_seg = t.seg;
            delta = ((uint32_t)reinterpret_cast<uintptr_t>(seg_w<EXT>(a, t.seg)) + t.row0 * a.row_bytes) & 15u;
            if constexpr (SWIGLU) delta2 = ((uint32_t)reinterpret_cast<uintptr_t>(seg_w2<EXT>(a, t.seg)) + t.row0 * a.row_bytes) & 15u;
        }
        const uint32_t base = stages_s + s * a.stage_stride + delta + unit_off;
        uint32_t base2 = 0;
        if constexpr (SWIGLU) base2 = stages_s + s * a.stage_stride + a.half_stride + unit_off + delta2;
        float *dst = comb_acc ? pbuf + (size_t)(t.row0 - wk.lo) * SL + group * GW + wig
                              : pbuf + (size_t)which * PLANE * (SWIGLU ? 2 : 1) + (size_t)buf_n * GW + wig;
        const float segw = comb_acc ? a.seg_weight[blockIdx.y * a.tok_sel_stride + t.seg] : 0.0f;
        const uint32_t rstride = comb_acc ? SL : GW;
        // Plain Q8_0 products keep two rows of a group in flight when a tile holds more than one row per group (this
        // row and the one rows_par further on): two independent dot products and reductions per warp hide each
        // other's shared-memory and shuffle latency, as the gate and up rows of the fused form do.
        constexpr bool PAIR = MODE == 0 && FMT == FMT_Q8_0;
        const uint32_t rstep = comb_acc ? 1u : (PAIR ? 2u * a.rows_par : a.rows_par);
#pragma unroll 1
        for (uint32_t r = comb_acc ? 0u : group; r < t.n; r += rstep) {
            float v = 0.0f, v2 = 0.0f;
            const bool second = PAIR && r + a.rows_par < t.n;
            if (active) {
                v = slot.dot(base + r * a.row_bytes, part, a.layout);
                if constexpr (SWIGLU) v2 = slot.dot(base2 + r * a.row_bytes, part, a.layout);
                if constexpr (PAIR) { if (second) v2 = slot.dot(base + (r + a.rows_par) * a.row_bytes, part, a.layout); }
            }
            if constexpr (SWIGLU || PAIR) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    v += __shfl_xor_sync(0xffffffffu, v, o);
                    v2 += __shfl_xor_sync(0xffffffffu, v2, o);
                }
            } else {
                v = warp_sum(v);
            }
            if (lane == 0) {
                if (comb_acc) dst[r * rstride] = fmaf(segw, v, dst[r * rstride]);
                else dst[r * GW] = v;
                if constexpr (SWIGLU) dst[PLANE + r * GW] = v2;
                if constexpr (PAIR) { if (second) dst[(r + a.rows_par) * GW] = v2; }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + s));   // this warp is done reading the stage
        if (comb_acc) { buf_n = wk.hi - wk.lo; buf_seg = 0; buf_row0 = wk.lo; }
        else buf_n += t.n;
        ++i;
        if (++s == a.nstages) { s = 0; parity ^= 1u; }
    }
    if (tid == 0) stamp(a.trace, 6);
    if (buf_n) flush();
    if constexpr (COMBINE) {
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
        for (uint32_t r = tid; r < wk.hi - wk.lo; r += C) {
            float *dst = a.seg[0].y + wk.lo + r + (EXT ? (size_t)blockIdx.y * a.tok_y_stride : 0);
            *dst = accbuf[r];
            if constexpr (EXT) {
                if (a.npeers > 0) {
                    uint8_t *slot = a.ll_origin + 2 * (reinterpret_cast<const uint8_t *>(dst) - a.arena_base);
                    st_slot(reinterpret_cast<uint2 *>(slot), accbuf[r], pub_tag);
                    for (int p = 0; p < a.npeers; ++p) st_slot(reinterpret_cast<uint2 *>(slot + a.peer_delta[p]), accbuf[r], pub_tag);
                }
            }
        }
    }
    if constexpr (EXT && MODE == 0) {
        if (a.res_parts) {
            __shared__ float s_sq[PIPE_MAX_CONSUMERS / 32];
            sq = warp_sum(sq);
            if (lane == 0) s_sq[tid >> 5] = sq;
            named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
            if (tid == 0) {
                float t = 0.0f;
                for (uint32_t w = 0; w < (C >> 5); ++w) t += s_sq[w];
                a.res_parts[blockIdx.x] = t;
            }
            for (uint32_t i = gridDim.x + blockIdx.x * C + tid; i < (uint32_t)PIPE_SUM_SQ_PARTS; i += gridDim.x * C) a.res_parts[i] = 0.0f;
        }
    }
    if (EXT && a.npeers > 0) {
        // the last CTA to get here makes the new generation this rank's current one; a launch that consumes the
        // vector reads it after its griddepcontrol.wait, i.e. after this grid has completed
        if (tid == 0 && atomicAdd(a.pub_arrived, 1u) == gridDim.x - 1) {
            *reinterpret_cast<volatile unsigned int *>(a.pub_arrived) = 0;
            *reinterpret_cast<volatile unsigned int *>(a.pub_gen) = pub_tag;
        }
    }
    if (tid == 0) stamp(a.trace, 7);
}

}  // namespace orome
