// gemv_mma.cuh -- batch-1 matvec for Q4_K / Q5_K with the integer dot products on mma.sync (int8).
//
// Why: with dp4a a warp spends ~270 instructions per 2048 Q4_K weights (nibble masks, one dp4a per four
// weights and byte plane, a shuffle reduction per row) and the ALU pipe, not HBM, sets the pace.  Here a warp
// takes a 16-row x 256-weight piece at a time: the unpacked nibbles of 16 rows are the A operand of
// m16n8k32 (u8), the byte planes of the fixed-point x are columns of the B operand (s8), so one instruction
// replaces 128 dp4a and the per-row shuffle reduction disappears (the k-sum happens inside the instruction).
// What is left per piece is unpacking (two logic ops per word), eight mma, the six-bit scales as integer
// multiply-adds, and a handful of float operations per superblock.
//
// x is held as fixed point per SUPERBLOCK of 256 elements: x_i ~= xs[u] * X_i, X_i = X2*65536 + X1*256 + X0 with
// balanced digits in [-128, 127] (all planes signed, as the B operand has one type).  The per-sub-block sums of
// x that the "min" term needs are fixed point too (sx_j ~= sxs[u] * S_j), so that term is one more small mma
// (m16n8k16: the eight 6-bit mins of a row against the eight sums).  Integer sums are exact; the only
// approximation is the rounding of x and of the sums (2^-23 of the superblock's max with three planes).
//
// Data movement: a producer warp streams 16-row x kc-superblock boxes into a ring of shared-memory stages, one
// 3-D TMA tensor copy per box (dimensions: 36 or 44 words of a superblock, superblocks of a row, rows), completing
// on mbarriers; bounded waits, programmatic dependent launch and the L2 prefetch of the next tensor are the
// pipelined kernel's.  One instruction per box matters: a bulk copy per row costs the issuing warp ~100 cycles
// each, which capped the ring at ~27 GB/s per SM.  The box is kb superblocks wide with kb = 2 (mod 4), so the row
// pitch kb * 144 (176) is 32 or 96 (mod 128) and the 8-byte fragment loads of rows g..g+3 fall into different
// banks; superblocks past the row's end arrive as zeros.
#pragma once
#include <cuda.h>
#include "gemv_pipe.cuh"

namespace orome {

constexpr int MMA_TILE_ROWS = 16;
constexpr int MMA_MAX_WARPS = 8;                  // consumer warps of a group
constexpr int MMA_MAX_GROUPS = 2;
constexpr int MMA_MAX_THREADS = (MMA_MAX_WARPS * MMA_MAX_GROUPS + 1) * 32;   // one more warp produces
constexpr uint32_t MMA_XQ_SB = 800;               // quantized x per superblock: 8 sub-blocks x 3 planes x 32 B, 3 x 8 sum bytes, pad

struct MmaArgs {
    alignas(64) CUtensorMap map[PIPE_MAX_SEG][2];   // per segment: its tensor (and the up tensor in the fused form)
    PipeSeg seg[PIPE_MAX_SEG];
    int nseg;
    const float *x;
    uint32_t in_dim, row_bytes;
    uint32_t units;            // superblocks per row
    uint32_t nwarps;           // consumer warps of one group: a group covers the kc superblocks of a stage
    uint32_t ngroups;          // groups; row tile i belongs to group i % ngroups
    uint32_t kc;               // superblocks per stage
    uint32_t nchunks;          // stages per row tile = ceil(units / kc)
    uint32_t dbg_tile;         // diagnostics build: first row tile whose per-warp timeline is recorded
    uint32_t pitch;            // bytes between rows inside a stage = box width in superblocks * superblock bytes
    uint32_t box_bytes;        // bytes one tensor copy delivers (16 rows * pitch)
    uint32_t nstages, stage_stride, half_stride, stage_base;
    uint32_t red_base, red_rows, xs_base;
    uint32_t total_rows;
    int layout;
    int *status;
    const uint8_t *pf_ptr;
    uint64_t pf_bytes;
    unsigned long long *trace;
};

template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF));
    return v;
}

// D = A(16x32, u8) * B(32x8, s8), int32.  Thread (g = lane / 4, t = lane % 4): a = {row g k 4t.., row g+8 k 4t..,
// row g k 16+4t.., row g+8 k 16+4t..}, b = {k 4t.. col g, k 16+4t.. col g}, d = {row g cols 2t, 2t+1, row g+8 cols 2t, 2t+1}.
__device__ __forceinline__ void mma_u8s8_k32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
// D = A(16x16, u8) * B(16x8, s8): a = {row g k 4t.., row g+8 k 4t..}, b = {k 4t.. col g}
__device__ __forceinline__ void mma_u8s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// The eight 6-bit scales and mins of a superblock as four words of four bytes each (sub-blocks 0-3, 4-7).
// Layout A: format.m:41-64; layout B: shaders.metal:1575-1578.
__device__ __forceinline__ void unpack_scales4(uint32_t w0, uint32_t w1, uint32_t w2, int layout,
                                               uint32_t &scl, uint32_t &sch, uint32_t &mnl, uint32_t &mnh)
{
    scl = w0 & 0x3F3F3F3Fu;
    mnl = w1 & 0x3F3F3F3Fu;
    const uint32_t hs = (w0 >> 2) & 0x30303030u, hm = (w1 >> 2) & 0x30303030u;
    if (layout == LAYOUT_A) {
        const uint32_t w2s = w2 >> 4;
        sch = (__byte_perm(w2, w2s, 0x5140) & 0x0F0F0F0Fu) | hs;
        mnh = (__byte_perm(w2, w2s, 0x7362) & 0x0F0F0F0Fu) | hm;
    } else {
        sch = (w2 & 0x0F0F0F0Fu) | hs;
        mnh = ((w2 >> 4) & 0x0F0F0F0Fu) | hm;
    }
}

template <int K>
__device__ __forceinline__ int byte_of(uint32_t lo, uint32_t hi)   // byte K (0..7) of the pair as an int
{
    return (int)__byte_perm(K < 4 ? lo : hi, 0u, 0x4440u + (K & 3));
}

// One superblock of rows g and g+8 against the superblock's x: y0 += (W x)[row g], y1 += (W x)[row g + 8],
// each thread carrying the columns (byte planes) 2t and 2t+1 of the products; the quad adds them up later.
//   s0, s1: shared addresses of the two rows' superblocks, already advanced by 8t;  h0, h1: without the 8t
//   B[j]: this thread's x bytes of sub-block j (plane g);  bsx: x-sum bytes of its plane, elements 4(t&1)..
template <int FMT, int SB>
__device__ __forceinline__ void mma_pair(uint2 w0, uint2 w1, const uint2 (&B)[8], uint2 qh0, uint2 qh1,
                                         uint32_t scl0, uint32_t sch0, uint32_t scl1, uint32_t sch1, int (&acc)[4], int (&accH)[4])
{
    uint32_t alo[4], ahi[4];
    if constexpr (FMT == FMT_Q4_K) {
        // high nibbles stay where they are (16 x value): their products go to accH and are scaled back at the end
        alo[0] = w0.x & 0x0F0F0F0Fu; alo[1] = w1.x & 0x0F0F0F0Fu; alo[2] = w0.y & 0x0F0F0F0Fu; alo[3] = w1.y & 0x0F0F0F0Fu;
        ahi[0] = w0.x & 0xF0F0F0F0u; ahi[1] = w1.x & 0xF0F0F0F0u; ahi[2] = w0.y & 0xF0F0F0F0u; ahi[3] = w1.y & 0xF0F0F0F0u;
    } else {
        // fifth bit of sub-block j is bit j of the qh byte of the element
        auto lo5 = [](uint32_t q, uint32_t h) { return (q & 0x0F0F0F0Fu) | (((h >> (2 * SB)) & 0x01010101u) << 4); };
        auto hi5 = [](uint32_t q, uint32_t h) { return ((q >> 4) & 0x0F0F0F0Fu) | (((h >> (2 * SB + 1)) & 0x01010101u) << 4); };
        alo[0] = lo5(w0.x, qh0.x); alo[1] = lo5(w1.x, qh1.x); alo[2] = lo5(w0.y, qh0.y); alo[3] = lo5(w1.y, qh1.y);
        ahi[0] = hi5(w0.x, qh0.x); ahi[1] = hi5(w1.x, qh1.x); ahi[2] = hi5(w0.y, qh0.y); ahi[3] = hi5(w1.y, qh1.y);
    }
    int c[4], ch[4];
    mma_u8s8_k32(c, alo, B[2 * SB].x, B[2 * SB].y);
    mma_u8s8_k32(ch, ahi, B[2 * SB + 1].x, B[2 * SB + 1].y);
    const int sa0 = byte_of<2 * SB>(scl0, sch0), sb0 = byte_of<2 * SB + 1>(scl0, sch0);
    const int sa1 = byte_of<2 * SB>(scl1, sch1), sb1 = byte_of<2 * SB + 1>(scl1, sch1);
    acc[0] += sa0 * c[0]; acc[1] += sa0 * c[1]; acc[2] += sa1 * c[2]; acc[3] += sa1 * c[3];
    if constexpr (FMT == FMT_Q4_K) {
        accH[0] += sb0 * ch[0]; accH[1] += sb0 * ch[1]; accH[2] += sb1 * ch[2]; accH[3] += sb1 * ch[3];
    } else {
        acc[0] += sb0 * ch[0]; acc[1] += sb0 * ch[1]; acc[2] += sb1 * ch[2]; acc[3] += sb1 * ch[3];
    }
}

template <int FMT>
__device__ __forceinline__ void mma_superblock(uint32_t h0, uint32_t h1, uint32_t t, const uint2 (&B)[8], uint32_t bsx,
                                               float xs, float sxs, float cw0, float cw1, int layout, float &y0, float &y1)
{
    // every load of the piece first, so that their latencies overlap
    constexpr int QOFF = FMT == FMT_Q4_K ? 16 : 48;
    const uint32_t s0 = h0 + 8u * t, s1 = h1 + 8u * t;
    const uint4 hd0 = lds128<0>(h0), hd1 = lds128<0>(h1);
    const uint2 wa0 = lds64<QOFF>(s0), wa1 = lds64<QOFF>(s1), wb0 = lds64<QOFF + 32>(s0), wb1 = lds64<QOFF + 32>(s1);
    const uint2 wc0 = lds64<QOFF + 64>(s0), wc1 = lds64<QOFF + 64>(s1), wd0 = lds64<QOFF + 96>(s0), wd1 = lds64<QOFF + 96>(s1);
    uint2 qh0 = make_uint2(0u, 0u), qh1 = make_uint2(0u, 0u);
    if constexpr (FMT == FMT_Q5_K) { qh0 = lds64<16>(s0); qh1 = lds64<16>(s1); }
    const uint32_t bs = lds32<0>(bsx);
    uint32_t scl0, sch0, mnl0, mnh0, scl1, sch1, mnl1, mnh1;
    unpack_scales4(hd0.y, hd0.z, hd0.w, layout, scl0, sch0, mnl0, mnh0);
    unpack_scales4(hd1.y, hd1.z, hd1.w, layout, scl1, sch1, mnl1, mnh1);
    int acc[4] = {0, 0, 0, 0}, accH[4] = {0, 0, 0, 0};
    mma_pair<FMT, 0>(wa0, wa1, B, qh0, qh1, scl0, sch0, scl1, sch1, acc, accH);
    mma_pair<FMT, 1>(wb0, wb1, B, qh0, qh1, scl0, sch0, scl1, sch1, acc, accH);
    mma_pair<FMT, 2>(wc0, wc1, B, qh0, qh1, scl0, sch0, scl1, sch1, acc, accH);
    mma_pair<FMT, 3>(wd0, wd1, B, qh0, qh1, scl0, sch0, scl1, sch1, acc, accH);
    // mins: k = sub-block; threads t = 0, 1 hold sub-blocks 0-3, 4-7 of their rows, the others contribute zeros
    int m[4];
    mma_u8s8_k16(m, t == 0 ? mnl0 : (t == 1 ? mnh0 : 0u), t == 0 ? mnl1 : (t == 1 ? mnh1 : 0u), bs);
    float f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = FMT == FMT_Q4_K ? fmaf((float)accH[i], 0.0625f, (float)acc[i]) : (float)acc[i];
    const float d0 = __half2float(__ushort_as_half((unsigned short)(hd0.x & 0xffffu))) * xs;
    const float d1 = __half2float(__ushort_as_half((unsigned short)(hd1.x & 0xffffu))) * xs;
    const float n0 = __half2float(__ushort_as_half((unsigned short)(hd0.x >> 16))) * sxs;
    const float n1 = __half2float(__ushort_as_half((unsigned short)(hd1.x >> 16))) * sxs;
    y0 = fmaf(d0, fmaf(cw1, f[1], cw0 * f[0]), y0);
    y0 = fmaf(-n0, fmaf(cw1, (float)m[1], cw0 * (float)m[0]), y0);
    y1 = fmaf(d1, fmaf(cw1, f[3], cw0 * f[2]), y1);
    y1 = fmaf(-n1, fmaf(cw1, (float)m[3], cw0 * (float)m[2]), y1);
}

// Balanced base-256 digits, all elements at once: for |v| <= 0x7F7F7F (0x7F7F) the bytes of v + 0x808080 (0x8080) are
// the digits plus 128, so a plane word is three byte permutes and one xor with 0x80808080.
template <int NP> __device__ __forceinline__ uint32_t digit_bias() { return NP == 3 ? 0x00808080u : 0x00008080u; }
__device__ __forceinline__ uint32_t plane_word(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t u3, int p)
{
    const uint32_t sel = (uint32_t)p | ((uint32_t)(4 + p) << 4);
    return __byte_perm(__byte_perm(u0, u1, sel), __byte_perm(u2, u3, sel), 0x5410) ^ 0x80808080u;
}

// x -> shared memory, one warp per superblock: lane l owns elements 8l..8l+7 (sub-block l / 4, bytes 8 (l % 4)..).
// Layout per superblock u at xq + u * MMA_XQ_SB: [sub-block j][plane p][32 bytes], then at +768 [plane p][8 sum bytes];
// xs[u], sxs[u] after all superblocks.  A warp takes up to four superblocks at a time: their loads are issued together
// and their shuffle reductions interleave.
template <int NP>
__device__ __forceinline__ void quantize_x_mma(const float *__restrict__ x, uint32_t units, uint8_t *xq, uint32_t warp, uint32_t lane,
                                               uint32_t nwarps)
{
    constexpr int QMAXI = NP == 3 ? 127 * 65536 + 127 * 256 + 127 : 127 * 256 + 127;
    constexpr float QMAX = (float)QMAXI;
    constexpr int XB = 4;
    float *xs = reinterpret_cast<float *>(xq + (size_t)units * MMA_XQ_SB), *sxs = xs + units;
    for (uint32_t ub = warp; ub < units; ub += nwarps * XB) {
        float4 v0[XB], v1[XB];
#pragma unroll
        for (int b = 0; b < XB; ++b) {
            const uint32_t u = ub + b * nwarps;
            const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)u * 256) + 2 * lane;
            v0[b] = u < units ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
            v1[b] = u < units ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float amax[XB], sum[XB], smax[XB];
#pragma unroll
        for (int b = 0; b < XB; ++b) {
            amax[b] = fmaxf(fmaxf(fmaxf(fabsf(v0[b].x), fabsf(v0[b].y)), fmaxf(fabsf(v0[b].z), fabsf(v0[b].w))),
                            fmaxf(fmaxf(fabsf(v1[b].x), fabsf(v1[b].y)), fmaxf(fabsf(v1[b].z), fabsf(v1[b].w))));
            sum[b] = ((v0[b].x + v0[b].y) + (v0[b].z + v0[b].w)) + ((v1[b].x + v1[b].y) + (v1[b].z + v1[b].w));
        }
#pragma unroll
        for (int o = 1; o < 4; o <<= 1) {
#pragma unroll
            for (int b = 0; b < XB; ++b) {
                amax[b] = fmaxf(amax[b], __shfl_xor_sync(0xffffffffu, amax[b], o));
                sum[b] += __shfl_xor_sync(0xffffffffu, sum[b], o);      // ends as the sum of x over the lane's sub-block
            }
        }
#pragma unroll
        for (int b = 0; b < XB; ++b) smax[b] = fabsf(sum[b]);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
#pragma unroll
            for (int b = 0; b < XB; ++b) {
                amax[b] = fmaxf(amax[b], __shfl_xor_sync(0xffffffffu, amax[b], o));
                smax[b] = fmaxf(smax[b], __shfl_xor_sync(0xffffffffu, smax[b], o));
            }
        }
#pragma unroll
        for (int b = 0; b < XB; ++b) {
            const uint32_t u = ub + b * nwarps;
            if (u >= units) break;
            const float inv = amax[b] > 0.0f ? QMAX / amax[b] : 0.0f, sinv = smax[b] > 0.0f ? QMAX / smax[b] : 0.0f;
            const float v[8] = {v0[b].x, v0[b].y, v0[b].z, v0[b].w, v1[b].x, v1[b].y, v1[b].z, v1[b].w};
            uint32_t uq[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) uq[i] = (uint32_t)max(-QMAXI, min(QMAXI, __float2int_rn(v[i] * inv))) + digit_bias<NP>();
            uint8_t *sb = xq + (size_t)u * MMA_XQ_SB;
#pragma unroll
            for (int p = 0; p < NP; ++p)
                *reinterpret_cast<uint2 *>(sb + (lane >> 2) * 96 + p * 32 + (lane & 3u) * 8) =
                    make_uint2(plane_word(uq[0], uq[1], uq[2], uq[3], p), plane_word(uq[4], uq[5], uq[6], uq[7], p));
            const uint32_t us = (uint32_t)max(-QMAXI, min(QMAXI, __float2int_rn(sum[b] * sinv))) + digit_bias<NP>();
            if ((lane & 3u) == 0) {
#pragma unroll
                for (int p = 0; p < NP; ++p) sb[768 + p * 8 + (lane >> 2)] = (uint8_t)(((us >> (8 * p)) & 255u) ^ 0x80u);
            }
            if (lane == 0) { xs[u] = amax[b] / QMAX; sxs[u] = smax[b] / QMAX; }
        }
    }
}

// One box: words 0.. of superblocks sb0.. of rows row0..row0+15 (coordinates in elements of the tensor map).
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap *map, uint32_t sb0, uint32_t row0, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(0), "r"(sb0), "r"(row0), "r"(bar) : "memory");
}

struct MmaTile { int seg; uint32_t row0, n; };

// Diagnostics build only (-DOROME_MMA_TILE_TRACE): CTA 0 records, for eight row tiles from OROME_DBG_TILE on, when each
// consumer warp starts waiting for the tile, gets it and is done with it, into the trace area of ten launches later.
#ifdef OROME_MMA_TILE_TRACE
#define MMA_TILE_STAMP(a, tile, warp, k)                                                                                      \
    do {                                                                                                                      \
        if ((a).trace && blockIdx.x == 0 && (threadIdx.x & 31u) == 0 && (tile) >= (a).dbg_tile && (tile) < (a).dbg_tile + 8)    \
            (a).trace[(size_t)gridDim.x * 80 + 3 * (((tile) - (a).dbg_tile) * 16 + (warp)) + (k)] = global_ns();             \
    } while (0)
#else
#define MMA_TILE_STAMP(a, tile, warp, k) do { } while (0)
#endif

// Tiles of at most 16 rows over this CTA's range of the concatenated rows; a tile never crosses a segment.
__device__ __forceinline__ bool mma_next_tile(const MmaArgs &a, uint32_t &cur, uint32_t hi, int &seg, MmaTile &t)
{
    if (cur >= hi) return false;
    int s = seg;
    while (s + 1 < a.nseg && cur >= a.seg[s + 1].vstart) ++s;
    seg = s;
    const uint32_t seg_end = a.seg[s].vstart + a.seg[s].rows;
    const uint32_t lim = hi < seg_end ? hi : seg_end;
    uint32_t n = lim - cur;
    if (n > (uint32_t)MMA_TILE_ROWS) n = MMA_TILE_ROWS;
    t.seg = s; t.row0 = cur - a.seg[s].vstart; t.n = n;
    cur += n;
    return true;
}

template <int FMT, int NP, bool SWIGLU>
__global__ void __launch_bounds__(MMA_MAX_THREADS, 1)
gemv_mma_kernel(const __grid_constant__ MmaArgs a)
{
    constexpr uint32_t UNIT = FMT == FMT_Q4_K ? 144 : 176;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + PIPE_MAX_STAGES;
    float *red = reinterpret_cast<float *>(smem + a.red_base);
    uint8_t *stages = smem + a.stage_base;
    __shared__ volatile int s_abort;

    // the warp index goes through a shuffle so that the compiler treats it (and every loop bound and address derived
    // from it) as warp-uniform: no convergence barriers around the mma instructions, uniform-datapath address math
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t NW = a.nwarps, NG = a.ngroups, CW = NW * NG, C = CW * 32, U = a.units;
    const bool producer = warp >= CW;

    if (tid == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < a.nstages; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), NW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    if (tid == 0) stamp(a.trace, 0);

    const uint32_t lo = (uint32_t)((uint64_t)blockIdx.x * a.total_rows / gridDim.x);
    const uint32_t hi = (uint32_t)((uint64_t)(blockIdx.x + 1) * a.total_rows / gridDim.x);

    if (producer) {
        // The weight copies do not depend on the previous kernel: no griddepcontrol.wait on this path.
        uint32_t cur = lo, s = 0, k = 0, issued = 0;
        int seg = 0;
        bool ok = true;
        MmaTile t;
        while (ok && mma_next_tile(a, cur, hi, seg, t)) {
            for (uint32_t c = 0; c < a.nchunks && ok; ++c) {
                if (k > 0) {
                    int good = 1;
                    if (lane == 0) {
                        good = !s_abort && mbar_wait_bounded(smem_u32(empty + s), (k - 1) & 1u);
                        if (!good && !s_abort) { s_abort = 1; atomicExch(a.status, 2); }
                    }
                    good = __shfl_sync(0xffffffffu, good, 0);
                    if (!good) { ok = false; break; }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                const uint32_t bar = smem_u32(full + s);
                if (lane == 0) {
                    const uint32_t dst = smem_u32(stages + (size_t)s * a.stage_stride);
                    mbar_expect_tx(bar, a.box_bytes * (SWIGLU ? 2u : 1u));   // a box is always whole: what lies outside the tensor arrives as zeros
                    tma_box(dst, &a.map[t.seg][0], c * a.kc, t.row0, bar);
                    if constexpr (SWIGLU) tma_box(dst + a.half_stride, &a.map[t.seg][1], c * a.kc, t.row0, bar);
                }
                ++issued;
                if (++s == a.nstages) { s = 0; ++k; }
            }
        }
        if (lane == 0) stamp(a.trace, 1);
        // All of this CTA's rows are requested: pull the head of the next launch's weights into L2.
        if (a.pf_ptr && ok) {
            const uint64_t per = (a.pf_bytes / gridDim.x) & ~(uint64_t)15;
            const uint8_t *p = a.pf_ptr + (uint64_t)blockIdx.x * per;
            for (uint64_t off = (uint64_t)lane * 32768; off < per; off += 32 * 32768) {
                const uint64_t n = per - off < 32768 ? per - off : 32768;
                bulk_prefetch_l2(p + off, (uint32_t)n);
            }
        }
        if (!ok && lane == 0) {   // give copies still in flight a bounded time to land before this warp leaves
            for (uint32_t q = 0; q < a.nstages && q < issued; ++q) {
                const uint32_t last = ((issued - 1 - q) / a.nstages) * a.nstages + q;   // newest copy set issued into stage q
                mbar_wait_bounded(smem_u32(full + q), (last / a.nstages) & 1u);
            }
        }
        return;
    }

    // ---- consumers ------------------------------------------------------------------------
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    pdl_wait();   // x is the previous kernel's output
    if (tid == 0) stamp(a.trace, 2);
    uint8_t *xq = smem + a.xs_base;
    quantize_x_mma<NP>(a.x, U, xq, warp, lane, CW);
    named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
    if (tid == 0) stamp(a.trace, 3);
    const uint32_t xs_s = smem_u32(xq) + U * MMA_XQ_SB;                // xs[U], then sxs[U]
    const uint32_t plane = g < (uint32_t)NP ? g : 0u;                  // columns past the planes repeat plane 0 and are weighted 0
    const uint32_t xq_s = smem_u32(xq) + plane * 32u + t4 * 8u;       // this thread's x bytes of sub-block 0, superblock 0
    const uint32_t sx_s = smem_u32(xq) + 768u + plane * 8u + (t4 & 1u) * 4u;
    // columns 2t, 2t+1 of the products are byte planes 2t, 2t+1
    const float cw0 = t4 == 0 ? 1.0f : (t4 == 1 && NP == 3 ? 65536.0f : 0.0f), cw1 = t4 == 0 ? 256.0f : 0.0f;

    const uint32_t CAP = a.red_rows, PLANE = CAP * NW;
    uint32_t which = 0, buf_n = 0, buf_row0 = 0;
    int buf_seg = 0;
    auto flush = [&]() {
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
        const float *src = red + (size_t)which * PLANE * (SWIGLU ? 2 : 1);
        float *y = a.seg[buf_seg].y + buf_row0;
        for (uint32_t r = tid; r < buf_n; r += C) {
            float gsum = 0.0f, usum = 0.0f;
            for (uint32_t w = 0; w < NW; ++w) {
                gsum += src[r * NW + w];
                if constexpr (SWIGLU) usum += src[PLANE + r * NW + w];
            }
            y[r] = SWIGLU ? silu_mul(gsum, usum) : gsum;
        }
        which ^= 1u;
        buf_n = 0;
    };

    const uint32_t stages_s = smem_u32(stages);
    const uint32_t group = warp / NW, wig = warp - group * NW;
    uint32_t cur = lo, s = 0, parity = 0, i = 0, turn = 0, tile_no = 0;
    int seg = 0;
    MmaTile t;
    for (; mma_next_tile(a, cur, hi, seg, t); ++tile_no) {
        if (buf_n && (t.seg != buf_seg || buf_n + t.n > CAP)) flush();
        if (buf_n == 0) { buf_seg = t.seg; buf_row0 = t.row0; }
        if (turn != group) {     // another group's tile: step over its stages
            if (++turn == NG) turn = 0;
            s += a.nchunks;
            while (s >= a.nstages) { s -= a.nstages; parity ^= 1u; }
            buf_n += t.n;
            continue;
        }
        if (++turn == NG) turn = 0;
        float yg0 = 0.0f, yg1 = 0.0f, yu0 = 0.0f, yu1 = 0.0f;
        for (uint32_t c = 0; c < a.nchunks; ++c) {
            if (c == 0) MMA_TILE_STAMP(a, tile_no, warp, 0);
            if (!s_abort && !mbar_wait_bounded(smem_u32(full + s), parity)) {
                s_abort = 1;
                atomicExch(a.status, 1);
            }
            if (c == 0) MMA_TILE_STAMP(a, tile_no, warp, 1);
            if (i == 0 && tid == 0) stamp(a.trace, 5);
            const uint32_t u0 = c * a.kc, kn = U - u0 < a.kc ? U - u0 : a.kc;
            const uint32_t row_s = stages_s + s * a.stage_stride + g * a.pitch;
            for (uint32_t u = wig; u < kn; u += NW) {
                const uint32_t ug = u0 + u;
                uint2 B[8];
                const uint32_t xa = xq_s + ug * MMA_XQ_SB;
                B[0] = lds64<0>(xa);   B[1] = lds64<96>(xa);  B[2] = lds64<192>(xa); B[3] = lds64<288>(xa);
                B[4] = lds64<384>(xa); B[5] = lds64<480>(xa); B[6] = lds64<576>(xa); B[7] = lds64<672>(xa);
                const float xsu = __uint_as_float(lds32<0>(xs_s + 4u * ug)), sxsu = __uint_as_float(lds32<0>(xs_s + 4u * (U + ug)));
                const uint32_t h0 = row_s + u * UNIT, h1 = h0 + 8u * a.pitch;
                mma_superblock<FMT>(h0, h1, t4, B, sx_s + ug * MMA_XQ_SB, xsu, sxsu, cw0, cw1, a.layout, yg0, yg1);
                if constexpr (SWIGLU)
                    mma_superblock<FMT>(h0 + a.half_stride, h1 + a.half_stride, t4, B, sx_s + ug * MMA_XQ_SB, xsu, sxsu, cw0, cw1, a.layout, yu0, yu1);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(empty + s));   // this warp is done reading the stage
            ++i;
            if (++s == a.nstages) { s = 0; parity ^= 1u; }
        }
        // add the byte planes (quad) and leave this warp's share of rows g, g+8 for the flush
        yg0 += __shfl_xor_sync(0xffffffffu, yg0, 1); yg1 += __shfl_xor_sync(0xffffffffu, yg1, 1);
        yg0 += __shfl_xor_sync(0xffffffffu, yg0, 2); yg1 += __shfl_xor_sync(0xffffffffu, yg1, 2);
        if constexpr (SWIGLU) {
            yu0 += __shfl_xor_sync(0xffffffffu, yu0, 1); yu1 += __shfl_xor_sync(0xffffffffu, yu1, 1);
            yu0 += __shfl_xor_sync(0xffffffffu, yu0, 2); yu1 += __shfl_xor_sync(0xffffffffu, yu1, 2);
        }
        if (t4 == 0) {
            float *dst = red + (size_t)which * PLANE * (SWIGLU ? 2 : 1) + (size_t)buf_n * NW + wig;
            if (g < t.n) { dst[g * NW] = yg0; if constexpr (SWIGLU) dst[PLANE + g * NW] = yu0; }
            if (g + 8 < t.n) { dst[(g + 8) * NW] = yg1; if constexpr (SWIGLU) dst[PLANE + (g + 8) * NW] = yu1; }
        }
        buf_n += t.n;
        MMA_TILE_STAMP(a, tile_no, warp, 2);
    }
    if (tid == 0) stamp(a.trace, 6);
    if (buf_n) flush();
    if (tid == 0) stamp(a.trace, 7);
}

}  // namespace orome
