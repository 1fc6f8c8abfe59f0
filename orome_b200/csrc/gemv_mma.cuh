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
constexpr int MMA_MAX_GROUPS = 5;
constexpr int MMA_MAX_CONSUMER_WARPS = 16;        // groups * warps per group
constexpr int MMA_MAX_PRODUCERS = 2;              // producer warps (two where every row is its own copy)
constexpr int MMA_MAX_THREADS = (MMA_MAX_CONSUMER_WARPS + MMA_MAX_PRODUCERS) * 32;
constexpr uint32_t MMA_XQ_SB = 864;               // quantized x per superblock: 8 groups x 3 planes x 32 B, then the sums (<= 96 B)
// Two input vectors at once (NTOK = 2; Q4_K / Q5_K plain products): the mma's B operand has eight columns of which one
// vector's byte planes fill two or three, so the planes of a second vector ride in the next columns and both products come
// out of the same instructions -- the weights are read, unpacked and multiplied once for the two.  Column c = vector c / NP,
// plane c % NP.  Quantized x per superblock: [sub-block][column][32 B], then [column][8 sum bytes]; two scales per vector.
template <int NP, int NTOK> __host__ __device__ constexpr uint32_t mma_xq_js() { return NTOK == 1 ? 96u : (uint32_t)(NTOK * NP) * 32u; }
template <int NP, int NTOK> __host__ __device__ constexpr uint32_t mma_xq_sums() { return NTOK == 1 ? 768u : 8u * mma_xq_js<NP, NTOK>(); }
template <int NP, int NTOK> __host__ __device__ constexpr uint32_t mma_xq_sb()
{
    return NTOK == 1 ? MMA_XQ_SB : (mma_xq_sums<NP, NTOK>() + (uint32_t)(NTOK * NP) * 8u + 15u) / 16u * 16u;
}

struct MmaArgs {
    alignas(64) CUtensorMap map[PIPE_MAX_SEG][2];   // per segment: its tensor (and the up tensor in the fused form)
    PipeSeg seg[PIPE_MAX_SEG];
    int nseg;
    const float *x;
    uint32_t in_dim, row_bytes;
    uint32_t units;            // superblocks per row
    uint32_t nwarps;           // consumer warps of one group: a group covers the kc superblocks of a stage
    uint32_t ngroups;          // groups; stage i (counted over row tiles and their chunks) belongs to group i % ngroups
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
    // multi-GPU forms, as in PipeArgs: tagged {value, tag} slots in the gather arenas
    int npeers;
    long long peer_delta[PIPE_MAX_PEERS];
    const uint8_t *arena_base;
    uint8_t *ll_origin;
    unsigned int *pub_gen, *pub_arrived;
    const uint2 *x_ll;
    const unsigned int *wait_gen;
    // MoE forms (template parameter MOE): the experts of a projection are one stacked tensor (expert e = rows
    // e * expert_rows .. of the tensor that map[0] describes), the chosen experts are read on the device.
    //   MOE 1, fused gate/up: segment s = expert seg_expert[s], all segments share x.
    //   MOE 2, down + combine: y[r] = sum_s seg_weight[s] * (W_{seg_expert[s]}[r] . x_s); the x_s lie one behind the
    //          other (units = nchunks * kc superblocks), chunk s of a row tile is expert s, the weight is folded
    //          into the scales of x_s.
    // blockIdx.y = token: x, y, indices and weights advance by their strides.
    const uint32_t *seg_expert;
    const float *seg_weight;
    uint32_t expert_rows;
    uint32_t tok_x_stride, tok_y_stride, tok_sel_stride;
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

// The integer part of one superblock of rows g, g+8: f[0..1] / f[2..3] = the scaled dot products of row g / g+8 in this thread's
// two columns, m[..] the same for the mins term; hx0 / hx1 = the rows' (d, dmin) words.
template <int FMT>
__device__ __forceinline__ void mma_superblock_core(uint32_t h0, uint32_t h1, uint32_t t, const uint2 (&B)[8], uint32_t bsx, int layout,
                                                    float (&f)[4], int (&m)[4], uint32_t &hx0, uint32_t &hx1)
{
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
    mma_u8s8_k16(m, t == 0 ? mnl0 : (t == 1 ? mnh0 : 0u), t == 0 ? mnl1 : (t == 1 ? mnh1 : 0u), bs);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = FMT == FMT_Q4_K ? fmaf((float)accH[i], 0.0625f, (float)acc[i]) : (float)acc[i];
    hx0 = hd0.x;
    hx1 = hd1.x;
}

// Two input vectors (A, B): this thread's two columns belong to A and / or B with the weights cwA*, cwB* (0 where a column is
// not the vector's).
template <int FMT>
__device__ __forceinline__ void mma_superblock2(uint32_t h0, uint32_t h1, uint32_t t, const uint2 (&B)[8], uint32_t bsx, float xsA, float sxsA,
                                                float xsB, float sxsB, float cwA0, float cwA1, float cwB0, float cwB1, int layout,
                                                float &yA0, float &yA1, float &yB0, float &yB1)
{
    float f[4];
    int m[4];
    uint32_t hx0, hx1;
    mma_superblock_core<FMT>(h0, h1, t, B, bsx, layout, f, m, hx0, hx1);
    const float d0 = __half2float(__ushort_as_half((unsigned short)(hx0 & 0xffffu))), d1 = __half2float(__ushort_as_half((unsigned short)(hx1 & 0xffffu)));
    const float n0 = __half2float(__ushort_as_half((unsigned short)(hx0 >> 16))), n1 = __half2float(__ushort_as_half((unsigned short)(hx1 >> 16)));
    const float m0 = (float)m[0], m1 = (float)m[1], m2 = (float)m[2], m3 = (float)m[3];
    yA0 = fmaf(d0 * xsA, fmaf(cwA1, f[1], cwA0 * f[0]), yA0);
    yA0 = fmaf(-n0 * sxsA, fmaf(cwA1, m1, cwA0 * m0), yA0);
    yB0 = fmaf(d0 * xsB, fmaf(cwB1, f[1], cwB0 * f[0]), yB0);
    yB0 = fmaf(-n0 * sxsB, fmaf(cwB1, m1, cwB0 * m0), yB0);
    yA1 = fmaf(d1 * xsA, fmaf(cwA1, f[3], cwA0 * f[2]), yA1);
    yA1 = fmaf(-n1 * sxsA, fmaf(cwA1, m3, cwA0 * m2), yA1);
    yB1 = fmaf(d1 * xsB, fmaf(cwB1, f[3], cwB0 * f[2]), yB1);
    yB1 = fmaf(-n1 * sxsB, fmaf(cwB1, m3, cwB0 * m2), yB1);
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


// ---- Q6_K -----------------------------------------------------------------
// Superblock = 210 bytes, only 2-byte aligned: ql[128] low nibbles, qh[64] two high bits, 16 int8 scales (one per 16
// weights), fp16 d.  Group (h, j) = weights 128h + 32j .. +31, with scales 8h + 2j (first 16) and 8h + 2j + 1.
// One m16n8k32 per group: the B columns are the x planes of the group's first 16 elements (columns 0..2, zero in the
// other 16 k-slots) and of its second 16 (columns 3..5), so the two scale groups come out in separate columns.
// The quants stay unsigned (0..63); their -32 offset is one more small mma per superblock: the row's 16 scales
// against the 16 per-group sums of the x digits.

// prmt in its generic form: a selector nibble with bit 3 set yields the sign of the chosen byte in all eight bits
// (the __byte_perm intrinsic documents only the three index bits)
__device__ __forceinline__ int prmt_sext(uint32_t x, uint32_t sel)
{
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(0u), "r"(sel));
    return r;
}
// D = A(16x16, s8) * B(16x8, s8)
__device__ __forceinline__ void mma_s8s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// Per-thread constants of the Q6_K step.  Thread t of a quad holds product columns 2t, 2t+1:
// t = 0: (first 16, plane 0), (first 16, plane 1); t = 1: (first 16, plane 2), (second 16, plane 0);
// t = 2: (second 16, plane 1), (second 16, plane 2); t = 3: unused columns.
struct Q6Lane {
    uint32_t sel[2][2];   // [scale byte pair 0/1 or 2/3 of a word][column c0 / c1]: permute selector, sign-extending
    float cw0, cw1, cwm;  // weights of the two columns' planes, and of the offset term's plane
};
template <int NP>
__device__ __forceinline__ Q6Lane q6_lane(uint32_t t)
{
    auto sext = [](uint32_t b) { return b | ((8u | b) << 4) | ((8u | b) << 8) | ((8u | b) << 12); };
    Q6Lane L;
    const uint32_t s0 = t <= 1 ? 0u : 1u, s1 = t == 0 ? 0u : 1u;   // which of the group's two scales column c0 / c1 takes
    L.sel[0][0] = sext(s0);     L.sel[0][1] = sext(s1);
    L.sel[1][0] = sext(2 + s0); L.sel[1][1] = sext(2 + s1);
    constexpr float W0 = 1.0f, W1 = 256.0f, W2 = NP == 3 ? 65536.0f : 0.0f;
    L.cw0 = t == 0 ? W0 : t == 1 ? W2 : t == 2 ? W1 : 0.0f;
    L.cw1 = t == 0 ? W1 : t == 1 ? W0 : t == 2 ? W2 : 0.0f;
    L.cwm = t == 0 ? W0 : t == 1 ? W1 : t == 2 ? W2 : 0.0f;
    return L;
}

// Four bytes from a shared address: aligned form, or two aligned words realigned by a byte permute when the address
// is only 2-byte aligned (sel = 0x5432 for addresses 2 mod 4, 0x3210 else).
template <bool ALIGNED>
__device__ __forceinline__ uint32_t q6_word(uint32_t a, uint32_t sel)
{
    if constexpr (ALIGNED) return lds32<0>(a);
    else {
        const uint32_t q = a & ~3u;
        return __byte_perm(lds32<0>(q), lds32<4>(q), sel);
    }
}

// Group (H, J) of rows g, g+8.  ql*/qh*: this thread's words of the half's ql (J even: bytes 0..31, J odd: 32..63) and
// qh, index 0 = elements 4t..4t+3, 1 = elements 16+4t..16+4t+3; suffix 0 / 1 = row g / g+8.
template <int H, int J>
__device__ __forceinline__ void q6_group(const uint32_t (&ql0)[2], const uint32_t (&ql1)[2], const uint32_t (&qh0)[2], const uint32_t (&qh1)[2],
                                         uint32_t b0, uint32_t b1, const uint32_t (&sc0)[4], const uint32_t (&sc1)[4], const Q6Lane &L, int (&acc)[4])
{
    auto unpack = [](uint32_t ql, uint32_t qh) {
        const uint32_t lo = J < 2 ? (ql & 0x0F0F0F0Fu) : ((ql >> 4) & 0x0F0F0F0Fu);
        const uint32_t hi = J == 0 ? (qh << 4) : J == 1 ? (qh << 2) : J == 2 ? qh : (qh >> 2);
        return lo | (hi & 0x30303030u);
    };
    const uint32_t av[4] = {unpack(ql0[0], qh0[0]), unpack(ql1[0], qh1[0]), unpack(ql0[1], qh0[1]), unpack(ql1[1], qh1[1])};
    int c[4];
    mma_u8s8_k32(c, av, b0, b1);
    constexpr int W = 2 * H + J / 2, P = J & 1;      // scale word and byte pair of this group
    acc[0] += prmt_sext(sc0[W], L.sel[P][0]) * c[0];
    acc[1] += prmt_sext(sc0[W], L.sel[P][1]) * c[1];
    acc[2] += prmt_sext(sc1[W], L.sel[P][0]) * c[2];
    acc[3] += prmt_sext(sc1[W], L.sel[P][1]) * c[3];
}

// One Q6_K superblock of rows g and g+8.  s0, s1: shared addresses of the rows' superblocks (2-byte aligned);
// bx: this thread's x word of group 0 (plane of its column; first or second 16 elements); first: the column covers
// the first 16 elements of a group (the word is operand b0 and b1 is zero) or the second 16 (b0 zero);
// bsx: the digit sums of its column.  Thread t owns elements 4t..4t+3 and 16+4t..16+4t+3 of every group, so the
// quad reads four consecutive words per row and the eight rows of a load fall into different banks.
template <bool ALIGNED>
__device__ __forceinline__ void mma_superblock_q6(uint32_t s0, uint32_t s1, uint32_t t, uint32_t bx, bool first, uint32_t bsx, float xs,
                                                  const Q6Lane &L, float &y0, float &y1)
{
    const uint32_t o = 4u * t;
    const uint32_t sel0 = (s0 & 2u) ? 0x5432u : 0x3210u, sel1 = (s1 & 2u) ? 0x5432u : 0x3210u;
    uint32_t xb[8];
    xb[0] = lds32<0>(bx);   xb[1] = lds32<96>(bx);  xb[2] = lds32<192>(bx); xb[3] = lds32<288>(bx);
    xb[4] = lds32<384>(bx); xb[5] = lds32<480>(bx); xb[6] = lds32<576>(bx); xb[7] = lds32<672>(bx);
    const uint32_t bs = lds32<0>(bsx);
    uint32_t sc0[4], sc1[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { sc0[k] = q6_word<ALIGNED>(s0 + 192 + 4 * k, sel0); sc1[k] = q6_word<ALIGNED>(s1 + 192 + 4 * k, sel1); }
    const uint32_t d0h = lds16<208>(s0), d1h = lds16<208>(s1);
    int acc[4] = {0, 0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t qa0[2], qa1[2], qb0[2], qb1[2], h0[2], h1[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            qa0[k] = q6_word<ALIGNED>(s0 + 64 * h + 16 * k + o, sel0);       qa1[k] = q6_word<ALIGNED>(s1 + 64 * h + 16 * k + o, sel1);
            qb0[k] = q6_word<ALIGNED>(s0 + 64 * h + 32 + 16 * k + o, sel0);  qb1[k] = q6_word<ALIGNED>(s1 + 64 * h + 32 + 16 * k + o, sel1);
            h0[k] = q6_word<ALIGNED>(s0 + 128 + 32 * h + 16 * k + o, sel0);  h1[k] = q6_word<ALIGNED>(s1 + 128 + 32 * h + 16 * k + o, sel1);
        }
        if (h == 0) {
            q6_group<0, 0>(qa0, qa1, h0, h1, first ? xb[0] : 0u, first ? 0u : xb[0], sc0, sc1, L, acc);
            q6_group<0, 1>(qb0, qb1, h0, h1, first ? xb[1] : 0u, first ? 0u : xb[1], sc0, sc1, L, acc);
            q6_group<0, 2>(qa0, qa1, h0, h1, first ? xb[2] : 0u, first ? 0u : xb[2], sc0, sc1, L, acc);
            q6_group<0, 3>(qb0, qb1, h0, h1, first ? xb[3] : 0u, first ? 0u : xb[3], sc0, sc1, L, acc);
        } else {
            q6_group<1, 0>(qa0, qa1, h0, h1, first ? xb[4] : 0u, first ? 0u : xb[4], sc0, sc1, L, acc);
            q6_group<1, 1>(qb0, qb1, h0, h1, first ? xb[5] : 0u, first ? 0u : xb[5], sc0, sc1, L, acc);
            q6_group<1, 2>(qa0, qa1, h0, h1, first ? xb[6] : 0u, first ? 0u : xb[6], sc0, sc1, L, acc);
            q6_group<1, 3>(qb0, qb1, h0, h1, first ? xb[7] : 0u, first ? 0u : xb[7], sc0, sc1, L, acc);
        }
    }
    // offset: sum over the 16 groups of scale * (sum of the x digits), columns (plane, low / high byte of the sum)
    int m[4];
    mma_s8s8_k16(m, t == 0 ? sc0[0] : t == 1 ? sc0[1] : t == 2 ? sc0[2] : sc0[3], t == 0 ? sc1[0] : t == 1 ? sc1[1] : t == 2 ? sc1[2] : sc1[3], bs);
    const float d0 = __half2float(__ushort_as_half((unsigned short)d0h)) * xs, d1 = __half2float(__ushort_as_half((unsigned short)d1h)) * xs;
    const float off0 = fmaf((float)m[1], 256.0f, (float)m[0]) * (32.0f * L.cwm), off1 = fmaf((float)m[3], 256.0f, (float)m[2]) * (32.0f * L.cwm);
    y0 = fmaf(d0, fmaf(L.cw1, (float)acc[1], fmaf(L.cw0, (float)acc[0], -off0)), y0);
    y1 = fmaf(d1, fmaf(L.cw1, (float)acc[3], fmaf(L.cw0, (float)acc[2], -off1)), y1);
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
// Q6 form: instead of the float sums, the sums of the signed digits over every 16 elements, as two balanced bytes:
// at +768 [plane p][low / high byte][16 groups].
// With `slots` set x is a gathered vector read from its {value, tag} slots (polled for `tag`); false = a poll expired.
// NTOK = 2: vector `b` (0 or 1) of two, into its columns of the wider layout (see mma_xq_sb).
template <int NP, bool Q6, int NTOK = 1>
__device__ __forceinline__ bool quantize_x_mma(const float *__restrict__ x, uint32_t units, uint8_t *xq, uint32_t warp, uint32_t lane,
                                               uint32_t nwarps, const uint2 *slots = nullptr, unsigned int tag = 0, uint32_t b_tok = 0)
{
    static_assert(NTOK == 1 || !Q6, "two vectors at once: Q4_K / Q5_K only");
    constexpr uint32_t XQSB = mma_xq_sb<NP, NTOK>(), JS = mma_xq_js<NP, NTOK>(), SUMS = mma_xq_sums<NP, NTOK>();
    const uint32_t col0 = NTOK == 1 ? 0u : b_tok * NP;
    bool ok = true;
    constexpr int QMAXI = NP == 3 ? 127 * 65536 + 127 * 256 + 127 : 127 * 256 + 127;
    constexpr float QMAX = (float)QMAXI;
    constexpr int XB = 4;
    float *xs = reinterpret_cast<float *>(xq + (size_t)units * XQSB), *sxs = xs + units * NTOK;
    for (uint32_t ub = warp; ub < units; ub += nwarps * XB) {
        float4 v0[XB], v1[XB];
#pragma unroll
        for (int b = 0; b < XB; ++b) {
            const uint32_t u = ub + b * nwarps;
            const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)u * 256) + 2 * lane;
            if (slots) {
                const uint2 *sl = slots + (size_t)u * 256 + 8 * lane;
                v0[b] = u < units ? ld_gathered4(sl, tag, &ok) : make_float4(0.f, 0.f, 0.f, 0.f);
                v1[b] = u < units ? ld_gathered4(sl + 4, tag, &ok) : make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                v0[b] = u < units ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                v1[b] = u < units ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
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
            uint8_t *sb = xq + (size_t)u * XQSB;
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                const uint2 pw = make_uint2(plane_word(uq[0], uq[1], uq[2], uq[3], p), plane_word(uq[4], uq[5], uq[6], uq[7], p));
                *reinterpret_cast<uint2 *>(sb + (lane >> 2) * JS + (col0 + p) * 32 + (lane & 3u) * 8) = pw;
                if constexpr (Q6) {
                    int sd = __dp4a((int)pw.x, 0x01010101, __dp4a((int)pw.y, 0x01010101, 0));
                    sd += __shfl_xor_sync(0xffffffffu, sd, 1);                    // 16 elements = two lanes
                    const int lo8 = (int)(signed char)(sd & 0xFF);
                    if ((lane & 1u) == 0) {
                        sb[768 + (2 * p) * 16 + (lane >> 1)] = (uint8_t)(lo8 & 255);
                        sb[768 + (2 * p + 1) * 16 + (lane >> 1)] = (uint8_t)(((sd - lo8) >> 8) & 255);
                    }
                }
            }
            if constexpr (!Q6) {
                const uint32_t us = (uint32_t)max(-QMAXI, min(QMAXI, __float2int_rn(sum[b] * sinv))) + digit_bias<NP>();
                if ((lane & 3u) == 0) {
#pragma unroll
                    for (int p = 0; p < NP; ++p) sb[SUMS + (col0 + p) * 8 + (lane >> 2)] = (uint8_t)(((us >> (8 * p)) & 255u) ^ 0x80u);
                }
            }
            if (lane == 0) { xs[u * NTOK + (NTOK == 1 ? 0u : b_tok)] = amax[b] / QMAX; sxs[u * NTOK + (NTOK == 1 ? 0u : b_tok)] = smax[b] / QMAX; }
        }
    }
    return ok;
}

// One box: words 0.. of superblocks sb0.. of rows row0..row0+15 (coordinates in elements of the tensor map).
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap *map, uint32_t sb0, uint32_t row0, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(0), "r"(sb0), "r"(row0), "r"(bar) : "memory");
}

struct MmaTile { int seg; uint32_t row0, n; };

// Diagnostics build only (-DOROME_MMA_TILE_TRACE): CTA 0 records, for eight row tiles from tile number OROME_MMA_TILE_TRACE on, when each
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

template <int FMT, int NP, bool SWIGLU, bool EXT, int MOE = 0, int NTOK = 1>
__global__ void __launch_bounds__(MMA_MAX_THREADS, 1)
gemv_mma_kernel(const __grid_constant__ MmaArgs a)
{
    static_assert(MOE == 0 || (FMT != FMT_Q6_K && !EXT), "the MoE forms are built for Q4_K / Q5_K on one GPU");
    static_assert(NTOK == 1 || (NTOK == 2 && FMT != FMT_Q6_K && !SWIGLU && !EXT && MOE == 0), "two vectors at once: plain Q4_K / Q5_K products on one GPU");
    constexpr bool TWO = NTOK == 2;
    constexpr uint32_t XQSB = mma_xq_sb<NP, NTOK>(), XJS = mma_xq_js<NP, NTOK>(), XSUMS = mma_xq_sums<NP, NTOK>();
    static_assert(MOE != 1 || SWIGLU, "MOE 1 is the fused gate/up form");
    static_assert(MOE != 2 || !SWIGLU, "MOE 2 is the down + combine form");
    __shared__ uint32_t s_expert[PIPE_MAX_SEG];
    constexpr uint32_t UNIT = FMT == FMT_Q4_K ? 144 : FMT == FMT_Q5_K ? 176 : 210;
    constexpr bool Q6 = FMT == FMT_Q6_K;
    static_assert(!(Q6 && SWIGLU), "the fused gate/up form is built for Q4_K and Q5_K only");
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + PIPE_MAX_STAGES;
    float *red = reinterpret_cast<float *>(smem + a.red_base);
    uint8_t *stages = smem + a.stage_base;
    __shared__ volatile int s_abort;

    // the warp index goes through a shuffle so that the compiler treats it (and every loop bound and address derived
    // from it) as warp-uniform: no convergence barriers around the mma instructions, uniform-datapath address math
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    constexpr uint32_t NPROD = Q6 ? 2u : 1u;
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

    // MoE forms: whole row tiles per CTA (row counts are multiples of 16 there), so that no box reaches past the rows
    // of the last expert of the stack
    const uint32_t split_units = MOE != 0 ? a.total_rows / MMA_TILE_ROWS : a.total_rows, split_mul = MOE != 0 ? MMA_TILE_ROWS : 1u;
    const uint32_t lo = (uint32_t)((uint64_t)blockIdx.x * split_units / gridDim.x) * split_mul;
    const uint32_t hi = (uint32_t)((uint64_t)(blockIdx.x + 1) * split_units / gridDim.x) * split_mul;

    if (producer) {
        // The weight copies do not depend on the previous kernel: no griddepcontrol.wait on this path.
        // With two producer warps, warp p issues the stages i with i % 2 == p.
        const uint32_t pw = warp - CW;
        if constexpr (MOE != 0) {      // the expert indices are the previous kernel's output
            pdl_wait();
            const uint32_t nsel = MOE == 1 ? (uint32_t)a.nseg : a.nchunks;
            if (lane < (uint32_t)PIPE_MAX_SEG) s_expert[lane] = lane < nsel ? a.seg_expert[blockIdx.y * a.tok_sel_stride + lane] : 0u;
            __syncwarp();
        }
        uint32_t cur = lo, s = 0, k = 0, issued = 0, used_mask = 0, par_mask = 0;
        int seg = 0;
        bool ok = true;
        MmaTile t;
        while (ok && mma_next_tile(a, cur, hi, seg, t)) {
            for (uint32_t c = 0; c < a.nchunks && ok; ++c, ++issued) {
                const uint32_t sc = s, kc_ = k;
                if (++s == a.nstages) { s = 0; ++k; }
                if (NPROD > 1 && issued % NPROD != pw) continue;
                if (kc_ > 0) {
                    int good = 1;
                    if (lane == 0) {
                        good = !s_abort && mbar_wait_bounded(smem_u32(empty + sc), (kc_ - 1) & 1u);
                        if (!good && !s_abort) { s_abort = 1; atomicExch(a.status, 2); }
                    }
                    good = __shfl_sync(0xffffffffu, good, 0);
                    if (!good) { ok = false; break; }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                used_mask |= 1u << sc;
                par_mask = (par_mask & ~(1u << sc)) | ((kc_ & 1u) << sc);
                const uint32_t bar = smem_u32(full + sc);
                if constexpr (Q6) {
                    // 210-byte superblocks rule out a tensor map (strides must be multiples of 16 bytes): one bulk copy per
                    // row, each widened to 16-byte boundaries; the consumers add the row's offset inside its first piece
                    const uint32_t u0 = c * a.kc, kn = U - u0 < a.kc ? U - u0 : a.kc;
                    uint32_t bytes = 0, dst = 0;
                    uintptr_t a0 = 0;
                    if (lane < t.n) {
                        const uintptr_t base = reinterpret_cast<uintptr_t>(a.seg[t.seg].w);
                        const uintptr_t src = base + (size_t)(t.row0 + lane) * a.row_bytes + (size_t)u0 * UNIT, end = src + (size_t)kn * UNIT;
                        const uintptr_t lim = base + (size_t)a.seg[t.seg].rows * a.row_bytes;
                        uint8_t *drow = stages + (size_t)sc * a.stage_stride + (size_t)lane * a.pitch;
                        a0 = src & ~(uintptr_t)15;
                        uintptr_t e1 = (end + 15) & ~(uintptr_t)15;
                        if (e1 > lim) {   // the tensor's last bytes: the copy stops at the last boundary, plain loads fetch the rest
                            e1 = end & ~(uintptr_t)15;
                            for (uintptr_t q = e1; q < end; q += 2)
                                *reinterpret_cast<uint16_t *>(drow + (q - a0)) = *reinterpret_cast<const uint16_t *>(q);
                        }
                        bytes = (uint32_t)(e1 - a0);
                        dst = smem_u32(drow);
                    }
                    const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
                    __syncwarp();
                    if (lane == 0) mbar_expect_tx(bar, total);
                    __syncwarp();
                    if (bytes) bulk_g2s(dst, reinterpret_cast<const void *>(a0), bytes, bar);
                } else if (lane == 0) {
                    const uint32_t dst = smem_u32(stages + (size_t)sc * a.stage_stride);
                    mbar_expect_tx(bar, a.box_bytes * (SWIGLU ? 2u : 1u));   // a box is always whole: what lies outside the tensor arrives as zeros
                    const int ms = MOE == 0 ? t.seg : 0;
                    uint32_t sb0 = c * a.kc, row0 = t.row0;
                    if constexpr (MOE == 1) row0 += s_expert[t.seg] * a.expert_rows;
                    if constexpr (MOE == 2) { row0 += s_expert[c] * a.expert_rows; sb0 = 0; }
                    tma_box(dst, &a.map[ms][0], sb0, row0, bar);
                    if constexpr (SWIGLU) tma_box(dst + a.half_stride, &a.map[ms][1], sb0, row0, bar);
                }
            }
        }
        if (lane == 0 && pw == 0) stamp(a.trace, 1);
        // All of this CTA's rows are requested: pull the head of the next launch's weights into L2.
        if (a.pf_ptr && ok && pw == 0) {
            const uint64_t per = (a.pf_bytes / gridDim.x) & ~(uint64_t)15;
            const uint8_t *p = a.pf_ptr + (uint64_t)blockIdx.x * per;
            for (uint64_t off = (uint64_t)lane * 32768; off < per; off += 32 * 32768) {
                const uint64_t n = per - off < 32768 ? per - off : 32768;
                bulk_prefetch_l2(p + off, (uint32_t)n);
            }
        }
        if (!ok && lane == 0) {   // give this warp's copies still in flight a bounded time to land before it leaves
            for (uint32_t q = 0; q < a.nstages; ++q)
                if (used_mask >> q & 1u) mbar_wait_bounded(smem_u32(full + q), par_mask >> q & 1u);
        }
        return;
    }

    // ---- consumers ------------------------------------------------------------------------
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    pdl_wait();   // x is the previous kernel's output
    if (tid == 0) stamp(a.trace, 2);
    uint8_t *xq = smem + a.xs_base;
    float moe_wgt = 1.0f;      // MoE form 2: the routing weight of the expert whose input this thread's superblock belongs to
    if constexpr (MOE == 2) { if (tid < U) moe_wgt = a.seg_weight[blockIdx.y * a.tok_sel_stride + tid / a.kc]; }
    {
        const uint2 *slots = EXT ? a.x_ll : nullptr;
        const unsigned int want = EXT && a.x_ll ? *reinterpret_cast<const volatile unsigned int *>(a.wait_gen) : 0u;
        if (!quantize_x_mma<NP, Q6, NTOK>(a.x + (MOE != 0 ? (size_t)blockIdx.y * a.tok_x_stride : 0), U, xq, warp, lane, CW, slots, want, 0u)) {
            s_abort = 1;
            atomicExch(a.status, 3);
        }
        if constexpr (TWO) quantize_x_mma<NP, Q6, NTOK>(a.x + a.tok_x_stride, U, xq, warp, lane, CW, nullptr, 0u, 1u);
    }
    const unsigned int pub_tag = EXT && a.npeers > 0 ? *reinterpret_cast<const volatile unsigned int *>(a.pub_gen) + 1u : 0u;
    if constexpr (Q6) {   // a block of zeros for lanes whose product column is empty
        for (uint32_t z = tid; z < 768 / 4; z += C) reinterpret_cast<uint32_t *>(xq + (size_t)U * MMA_XQ_SB + 8 * U)[z] = 0u;
    }
    named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
    if constexpr (MOE == 2) {      // the routing weight of an expert goes into the scales of its input vector
        float *xsf = reinterpret_cast<float *>(xq + (size_t)U * MMA_XQ_SB);
        for (uint32_t u = tid; u < U; u += C) {
            const float wgt = u == tid ? moe_wgt : a.seg_weight[blockIdx.y * a.tok_sel_stride + u / a.kc];   // loaded before the quantization above
            xsf[u] *= wgt;
            xsf[U + u] *= wgt;
        }
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
    }
    if (tid == 0) stamp(a.trace, 3);
    const uint32_t xs_s = smem_u32(xq) + U * XQSB;                     // xs[U * NTOK], then sxs[U * NTOK]
    const uint32_t plane = g < (uint32_t)(NP * NTOK) ? g : 0u;         // columns past the planes repeat column 0 and are weighted 0
    const uint32_t xq_s = smem_u32(xq) + plane * 32u + t4 * 8u;       // this thread's x bytes of sub-block 0, superblock 0
    const uint32_t sx_s = smem_u32(xq) + XSUMS + plane * 8u + (t4 & 1u) * 4u;
    // columns 2t, 2t+1 of the products are byte planes 2t, 2t+1
    const float cw0 = t4 == 0 ? 1.0f : (t4 == 1 && NP == 3 ? 65536.0f : 0.0f), cw1 = t4 == 0 ? 256.0f : 0.0f;
    // two vectors: column c is plane c % NP of vector c / NP; this thread's columns 2t, 2t+1 count for vector A and / or B
    auto col_w = [](uint32_t c, uint32_t vec) {
        const uint32_t pl = c % NP;
        const float w = pl == 0 ? 1.0f : (pl == 1 ? 256.0f : 65536.0f);
        return c < (uint32_t)(2 * NP) && c / NP == vec ? w : 0.0f;
    };
    const float cwA0 = col_w(2 * t4, 0), cwA1 = col_w(2 * t4 + 1, 0), cwB0 = col_w(2 * t4, 1), cwB1 = col_w(2 * t4 + 1, 1);

    // Q6_K: column g = (first / second 16 elements of a group, plane g % 3); lanes of unused columns read a block of zeros
    const uint32_t q6_plane = g % 3u;
    const bool q6_col = Q6 && g < 6u && q6_plane < (uint32_t)NP;
    const uint32_t q6_bx = q6_col ? smem_u32(xq) + q6_plane * 32u + (g < 3u ? 0u : 16u) + t4 * 4u : xs_s + 8u * U;
    const uint32_t q6_bstride = q6_col ? MMA_XQ_SB : 0u;
    const uint32_t q6_sx = smem_u32(xq) + 768u + (g < 6u ? g : 0u) * 16u + t4 * 4u;
    const Q6Lane q6l = q6_lane<NP>(t4);

    const uint32_t CAP = a.red_rows, SLOTS = NW * NG, PLANE = CAP * SLOTS;   // every warp of every group leaves one partial sum per row
    uint32_t which = 0, buf_n = 0, buf_row0 = 0;
    int buf_seg = 0;
    auto flush = [&]() {
        named_bar_sync(PIPE_BAR_CONSUMERS, (int)C);
        const float *src = red + (size_t)which * PLANE * (SWIGLU || TWO ? 2 : 1);
        float *y = a.seg[buf_seg].y + buf_row0 + (MOE != 0 ? (size_t)blockIdx.y * a.tok_y_stride : 0);
        for (uint32_t r = tid; r < buf_n; r += C) {
            float gsum = 0.0f, usum = 0.0f;
            for (uint32_t w = 0; w < SLOTS; ++w) {
                gsum += src[r * SLOTS + w];
                if constexpr (SWIGLU || TWO) usum += src[PLANE + r * SLOTS + w];
            }
            const float val = SWIGLU ? silu_mul(gsum, usum) : gsum;
            y[r] = val;
            if constexpr (TWO) y[a.tok_y_stride + r] = usum;      // the second vector's product
            if constexpr (EXT) {
                if (a.npeers > 0) {
                    uint8_t *slot = a.ll_origin + 2 * (reinterpret_cast<const uint8_t *>(y + r) - a.arena_base);
                    st_slot(reinterpret_cast<uint2 *>(slot), val, pub_tag);
                    for (int p = 0; p < a.npeers; ++p) st_slot(reinterpret_cast<uint2 *>(slot + a.peer_delta[p]), val, pub_tag);
                }
            }
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
        float yg0 = 0.0f, yg1 = 0.0f, yu0 = 0.0f, yu1 = 0.0f;
        for (uint32_t c = 0; c < a.nchunks; ++c) {
            const bool mine = turn == group;        // stages go round the groups
            if (++turn == NG) turn = 0;
            if (!mine) {
                if (++s == a.nstages) { s = 0; parity ^= 1u; }
                continue;
            }
            if (c == 0) MMA_TILE_STAMP(a, tile_no, warp, 0);
            if (!s_abort && !mbar_wait_bounded(smem_u32(full + s), parity)) {
                s_abort = 1;
                atomicExch(a.status, 1);
            }
            if (c == 0) MMA_TILE_STAMP(a, tile_no, warp, 1);
            if (i == 0 && tid == 0) stamp(a.trace, 5);
            const uint32_t u0 = c * a.kc, kn = U - u0 < a.kc ? U - u0 : a.kc;
            const uint32_t row_s = stages_s + s * a.stage_stride + g * a.pitch;
            if constexpr (Q6) {
                // where the two rows start inside their first 16-byte piece (the copies were widened to 16-byte boundaries)
                const uint32_t wlo = (uint32_t)reinterpret_cast<uintptr_t>(a.seg[t.seg].w) + u0 * UNIT;
                const uint32_t r0 = row_s + ((wlo + (t.row0 + g) * a.row_bytes) & 15u);
                const uint32_t r1 = row_s + 8u * a.pitch + ((wlo + (t.row0 + g + 8u) * a.row_bytes) & 15u);
                for (uint32_t u = wig; u < kn; u += NW) {
                    const uint32_t ug = u0 + u;
                    const float xsu = __uint_as_float(lds32<0>(xs_s + 4u * ug));
                    const uint32_t sa = r0 + u * UNIT, sb = r1 + u * UNIT;
                    if (__all_sync(0xffffffffu, ((sa | sb) & 2u) == 0u))
                        mma_superblock_q6<true>(sa, sb, t4, q6_bx + ug * q6_bstride, g < 3u, q6_sx + ug * MMA_XQ_SB, xsu, q6l, yg0, yg1);
                    else
                        mma_superblock_q6<false>(sa, sb, t4, q6_bx + ug * q6_bstride, g < 3u, q6_sx + ug * MMA_XQ_SB, xsu, q6l, yg0, yg1);
                }
            } else {
                for (uint32_t u = wig; u < kn; u += NW) {
                    const uint32_t ug = u0 + u;
                    uint2 B[8];
                    const uint32_t xa = xq_s + ug * XQSB;
                    B[0] = lds64<0>(xa);       B[1] = lds64<XJS>(xa);     B[2] = lds64<2 * XJS>(xa); B[3] = lds64<3 * XJS>(xa);
                    B[4] = lds64<4 * XJS>(xa); B[5] = lds64<5 * XJS>(xa); B[6] = lds64<6 * XJS>(xa); B[7] = lds64<7 * XJS>(xa);
                    const uint32_t h0 = row_s + u * UNIT, h1 = h0 + 8u * a.pitch;
                    if constexpr (TWO) {
                        const float xsA = __uint_as_float(lds32<0>(xs_s + 8u * ug)), xsB = __uint_as_float(lds32<4>(xs_s + 8u * ug));
                        const float sxsA = __uint_as_float(lds32<0>(xs_s + 8u * (U + ug))), sxsB = __uint_as_float(lds32<4>(xs_s + 8u * (U + ug)));
                        mma_superblock2<FMT>(h0, h1, t4, B, sx_s + ug * XQSB, xsA, sxsA, xsB, sxsB, cwA0, cwA1, cwB0, cwB1, a.layout, yg0, yg1, yu0, yu1);
                    } else {
                        const float xsu = __uint_as_float(lds32<0>(xs_s + 4u * ug)), sxsu = __uint_as_float(lds32<0>(xs_s + 4u * (U + ug)));
                        mma_superblock<FMT>(h0, h1, t4, B, sx_s + ug * XQSB, xsu, sxsu, cw0, cw1, a.layout, yg0, yg1);
                        if constexpr (SWIGLU)
                            mma_superblock<FMT>(h0 + a.half_stride, h1 + a.half_stride, t4, B, sx_s + ug * XQSB, xsu, sxsu, cw0, cw1, a.layout, yu0, yu1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(empty + s));   // this warp is done reading the stage
            ++i;
            if (++s == a.nstages) { s = 0; parity ^= 1u; }
        }
        // add the byte planes (quad) and leave this warp's share of rows g, g+8 for the flush
        yg0 += __shfl_xor_sync(0xffffffffu, yg0, 1); yg1 += __shfl_xor_sync(0xffffffffu, yg1, 1);
        yg0 += __shfl_xor_sync(0xffffffffu, yg0, 2); yg1 += __shfl_xor_sync(0xffffffffu, yg1, 2);
        if constexpr (SWIGLU || TWO) {
            yu0 += __shfl_xor_sync(0xffffffffu, yu0, 1); yu1 += __shfl_xor_sync(0xffffffffu, yu1, 1);
            yu0 += __shfl_xor_sync(0xffffffffu, yu0, 2); yu1 += __shfl_xor_sync(0xffffffffu, yu1, 2);
        }
        if (t4 == 0) {
            float *dst = red + (size_t)which * PLANE * (SWIGLU || TWO ? 2 : 1) + (size_t)buf_n * SLOTS + warp;
            if (g < t.n) { dst[g * SLOTS] = yg0; if constexpr (SWIGLU || TWO) dst[PLANE + g * SLOTS] = yu0; }
            if (g + 8 < t.n) { dst[(g + 8) * SLOTS] = yg1; if constexpr (SWIGLU || TWO) dst[PLANE + (g + 8) * SLOTS] = yu1; }
        }
        buf_n += t.n;
        MMA_TILE_STAMP(a, tile_no, warp, 2);
    }
    if (tid == 0) stamp(a.trace, 6);
    if (buf_n) flush();
    if (EXT && a.npeers > 0) {
        if (tid == 0 && atomicAdd(a.pub_arrived, 1u) == gridDim.x - 1) {   // last CTA: the new generation becomes current
            *reinterpret_cast<volatile unsigned int *>(a.pub_arrived) = 0;
            *reinterpret_cast<volatile unsigned int *>(a.pub_gen) = pub_tag;
        }
    }
    if (tid == 0) stamp(a.trace, 7);
}

}  // namespace orome
