// gemm_tc.cuh -- the batched (prefill) form on the 5th-generation tensor cores.
//
//   Y[b][r] = sum_c W[r][c] * X[b][c],   b < batch (16..128 after padding), W block-quantized.
//
// With tens of input vectors the product is a real contraction (about 2*batch flop per weight
// byte), so the weights are dequantized once into fp16 tiles and multiplied with tcgen05.mma:
//
//   producer warp   one 2-D TMA tensor copy per stage (128 packed rows x one 256-weight chunk; rows past the
//                   tensor are zero-filled) and one bulk copy of the matching pre-packed fp16 tile of X
//   16 dequant warps packed stage -> fp16 A slabs (two groups of 8 warps take alternate slabs) of 128 rows x 64 k in the K-major 128-byte-swizzle
//                   layout the tensor core reads (row = 128 bytes, 16-byte pieces XORed with row % 8)
//   MMA warp        one thread issues 4 x tcgen05.mma (M128 x N x K16) per slab, accumulator in TMEM;
//                   tcgen05.commit hands slabs and X tiles back
//   epilogue        warps 0-3 read the accumulator with tcgen05.ld (lane = row) and store Y (or a
//                   split-K partial)
//
// Operand precision: weights and x are rounded to fp16 once (the accumulator is fp32), the same
// class of rounding the reference's kernels apply to x (shaders.metal:1470); measured rel-L2 against
// the fp64 oracle is a few 1e-4.  X is packed to fp16 tiles by pack_x_f16_kernel beforehand, so no
// CTA converts it again.  Every barrier wait is bounded (status code 4 on expiry).
#pragma once
#include <cuda.h>

#include "decode.cuh"
#include "gemv_pipe.cuh"

namespace orome {

constexpr int TC_M = 128;            // rows per CTA tile
constexpr int TC_KC = 256;           // weights per packed chunk (8 Q8_0 blocks / one K-quant superblock)
constexpr int TC_SLAB_K = 64;        // k per A slab = one 128-byte swizzle row of fp16
constexpr int TC_SLABS = 4;          // fp16 slabs per 256-weight chunk
#ifndef OROME_TC_RING
#define OROME_TC_RING 4
#endif
#ifndef OROME_TC_PK
#define OROME_TC_PK 2
#endif
#ifndef OROME_TC_BS
#define OROME_TC_BS 2
#endif
constexpr int TC_MAX_RING = OROME_TC_RING;   // fp16 slab buffers
constexpr int TC_PK_MAX_STAGES = 8;
// packed-weight stages in flight: what hides the latency of the weight stream (a Q8_0 stage is 34 KB, a Q4_K one 18 KB)
constexpr int tc_pk_stages(int fmt) { return fmt == FMT_Q8_0 ? (OROME_TC_PK < 3 ? OROME_TC_PK : 3) : OROME_TC_PK; }
constexpr int TC_MAX_N = 64;         // input vectors per launch (padded to a multiple of 16)
constexpr int TC_B_STAGES = OROME_TC_BS;     // X tile stages (one chunk each)
constexpr int TC_B_MAX_STAGES = 4;
constexpr int TC_DEQ_WARPS = 16;     // two groups of 8 warps take alternate slabs
constexpr int TC_SLAB_WARPS = 8;     // warps that fill one slab
constexpr int TC_THREADS = (TC_DEQ_WARPS + 3) * 32;     // + weight producer, MMA issuer, X producer

// Row-split form on several GPUs (the batched counterpart of the publish fields of PipeArgs): every Y value also
// goes, as a {value, tag} slot, into this rank's and every peer's copy of the gather arena.
struct TcPub {
    int npeers;                               // 0: single GPU, nothing is published
    long long peer_delta[PIPE_MAX_PEERS];
    const uint8_t *arena_base;
    uint8_t *ll_origin;
    unsigned int *pub_gen, *pub_arrived;
};
__device__ __forceinline__ void tc_publish(const TcPub &g, const float *addr, float val, unsigned int tag)
{
    uint8_t *slot = g.ll_origin + 2 * (reinterpret_cast<const uint8_t *>(addr) - g.arena_base);
    st_slot(reinterpret_cast<uint2 *>(slot), val, tag);
    for (int p = 0; p < g.npeers; ++p) st_slot(reinterpret_cast<uint2 *>(slot + g.peer_delta[p]), val, tag);
}
// One thread per CTA, after the CTA's stores: the last CTA of the grid makes the new generation this rank's current one.
__device__ __forceinline__ void tc_publish_done(const TcPub &g, unsigned int tag)
{
    if (atomicAdd(g.pub_arrived, 1u) == gridDim.x - 1) {
        *reinterpret_cast<volatile unsigned int *>(g.pub_arrived) = 0;
        *reinterpret_cast<volatile unsigned int *>(g.pub_gen) = tag;
    }
}

// Diagnostics builds only: SM-cycle stamps of CTA 0's pipeline (kind, index), read back by a test-bench helper.
#ifdef OROME_DIAGNOSTICS
__device__ long long g_tc_trace[8][80];
#define TC_STAMP(kind, idx) do { if (blockIdx.x == 0 && (idx) < 80) g_tc_trace[kind][idx] = clock64(); } while (0)
#else
#define TC_STAMP(kind, idx) do { } while (0)
#endif

struct TcArgs {
    alignas(64) CUtensorMap wmap;   // the tensor as a 2-D array of 32-bit words [rows][row_bytes / 4], box = 128 rows x one chunk
    const uint8_t *w;          // tensor
    const __half *xp;          // packed X: [k_slab][npad rows][64] fp16, swizzled (pack_x_f16_kernel)
    float *y;                  // Y [batch][ldy] when split == 1, else partials [split][batch][rows]
    uint32_t rows, in_dim, row_bytes, chunk_bytes;   // chunk_bytes = packed bytes of 256 weights of one row
    uint32_t batch, npad, ldy;
    uint32_t split, chunks;       // split-K parts and 256-weight chunks per row: part p takes chunks [p*chunks/split, (p+1)*chunks/split)
    uint32_t tiles_per_cta;       // tensor-memory form: row tiles a CTA works on side by side (1, 2 or 4)
    int layout;
    int *status;
    TcPub pub;                 // split == 1 only: with split-K the reduction kernel publishes
};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// K-major, 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t saddr)
{
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// Byte offset of 16-byte piece `c` (0..7) of row `r` inside a K-major SW128 tile.
__device__ __forceinline__ uint32_t sw128_off(uint32_t r, uint32_t c) { return (r >> 3) * 1024u + (r & 7u) * 128u + ((c ^ (r & 7u)) << 4); }

// X fp32 [batch][ldx] -> fp16 tiles [k_slab][npad][64] in the same swizzled layout; rows >= batch are zero.
// x_ll: X is a gathered matrix in the arena, read from its slots (every element polled, bounded, for the generation
// *wait_gen); NULL: a plain matrix.
__global__ void pack_x_f16_kernel(const float *__restrict__ x, int batch, int ldx, uint32_t in_dim, uint32_t npad, __half *__restrict__ xp,
                                  const uint2 *x_ll, const unsigned int *wait_gen, long long wait_cycles, int *status)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned int want = x_ll ? *reinterpret_cast<const volatile unsigned int *>(wait_gen) : 0u;
    bool ok = true;
    const uint32_t slabs = in_dim / TC_SLAB_K;
    const size_t total = (size_t)slabs * npad * 8;   // one thread per 16-byte piece
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(i & 7), n = (uint32_t)((i >> 3) % npad), ks = (uint32_t)(i / ((size_t)npad * 8));
        __half2 h[4];
        if ((int)n < batch) {
            const size_t off = (size_t)n * ldx + (size_t)ks * TC_SLAB_K + c * 8;
            const float4 *src = reinterpret_cast<const float4 *>(x + off);
            const float4 a = x_ll ? ld_gathered4(x_ll + off, want, &ok, wait_cycles, status) : src[0];
            const float4 b = x_ll ? ld_gathered4(x_ll + off + 4, want, &ok, wait_cycles, status) : src[1];
            h[0] = __floats2half2_rn(a.x, a.y); h[1] = __floats2half2_rn(a.z, a.w);
            h[2] = __floats2half2_rn(b.x, b.y); h[3] = __floats2half2_rn(b.z, b.w);
        } else {
            h[0] = h[1] = h[2] = h[3] = __floats2half2_rn(0.f, 0.f);
        }
        uint8_t *dst = reinterpret_cast<uint8_t *>(xp) + (size_t)ks * npad * 128 + sw128_off(n, c);
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(h);
    }
    if (!ok) atomicExch(status, 3);
}

// 8 consecutive weights of one row as fp16 -> one 16-byte piece.
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }

// Two byte lanes of `w` (selected by `sel`) -> fp16 pair (byte - bias) * scale + addend.  0x6400 | byte is the
// fp16 number 1024 + byte exactly, so the bias comes off exactly before the one rounded multiply-add.
__device__ __forceinline__ __half2 two_weights(uint32_t w, uint32_t sel, __half2 bias, __half2 scale, __half2 addend)
{
    const uint32_t bits = __byte_perm(w, 0x64646464u, sel);
    return __hfma2(__hsub2(*reinterpret_cast<const __half2 *>(&bits), bias), scale, addend);
}

// 32 consecutive weights of one row (a Q8_0 block / a K-quant sub-block) -> four 16-byte fp16 pieces.
// `g32` is the index of the 32-group inside the 256-weight chunk (0..7).
template <int FMT>
__device__ __forceinline__ void dequant_group32(const uint8_t *pk_row, uint32_t g32, int layout, uint4 (&out)[4])
{
    uint32_t w[8];          // the 32 quants as bytes, in element order
    __half2 scale, bias, addend;
    if constexpr (FMT == FMT_Q8_0) {
        const uint32_t a = smem_u32(pk_row) + g32 * 34u;                   // 2-byte aligned block
        const uint32_t base = a & ~3u;
        uint32_t v[10];
        v[0] = lds32<0>(base); v[1] = lds32<4>(base); v[2] = lds32<8>(base); v[3] = lds32<12>(base); v[4] = lds32<16>(base);
        v[5] = lds32<20>(base); v[6] = lds32<24>(base); v[7] = lds32<28>(base); v[8] = lds32<32>(base); v[9] = lds32<36>(base);
        const bool odd = (a & 2u) != 0;                                    // block starts in the upper half of v[0]
        const uint32_t dbits = odd ? (v[0] >> 16) : (v[0] & 0xffffu);
        const uint32_t sel = odd ? 0x3210u : 0x5432u;                      // quants start 2 bytes after the scale
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (odd ? __byte_perm(v[i + 1], v[i + 2], sel) : __byte_perm(v[i], v[i + 1], sel)) ^ 0x80808080u;
        const float d = __half2float(__ushort_as_half((unsigned short)dbits));
        scale = __float2half2_rn(d); bias = __float2half2_rn(1152.0f); addend = __float2half2_rn(0.0f);   // bytes are q + 128
    } else {
        constexpr int QOFF = FMT == FMT_Q4_K ? 16 : 48;
        const uint32_t sb = smem_u32(pk_row);
        const uint4 h = lds128<0>(sb);
        uint32_t scA, scB, mnA, mnB;
        pair_scales(h.y, h.z, h.w, layout, (int)(g32 >> 1), scA, scB, mnA, mnB);
        const uint32_t sc = (g32 & 1u) ? scB : scA, mn = (g32 & 1u) ? mnB : mnA;
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        const uint32_t qa = sb + 32u * (g32 >> 1);
        const uint4 q0 = lds128<QOFF>(qa), q1 = lds128<QOFF + 16>(qa);
        w[0] = q0.x; w[1] = q0.y; w[2] = q0.z; w[3] = q0.w; w[4] = q1.x; w[5] = q1.y; w[6] = q1.z; w[7] = q1.w;
        const uint32_t shift = (g32 & 1u) * 4u;
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (w[i] >> shift) & 0x0F0F0F0Fu;
        if constexpr (FMT == FMT_Q5_K) {
            const uint4 h0 = lds128<16>(sb), h1 = lds128<32>(sb);
            const uint32_t hb[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] |= ((hb[i] >> g32) & 0x01010101u) << 4;
        }
        scale = __float2half2_rn(d * (float)sc); bias = __float2half2_rn(1024.0f); addend = __float2half2_rn(-(dmin * (float)mn));
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        out[p].x = h2_bits(two_weights(w[2 * p], 0x5140u, bias, scale, addend));
        out[p].y = h2_bits(two_weights(w[2 * p], 0x7362u, bias, scale, addend));
        out[p].z = h2_bits(two_weights(w[2 * p + 1], 0x5140u, bias, scale, addend));
        out[p].w = h2_bits(two_weights(w[2 * p + 1], 0x7362u, bias, scale, addend));
    }
}

template <int FMT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ TcArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles must start on 1024-byte boundaries: align the base by hand (the launch adds 1 KiB of slack)
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // layout: [A slabs 4 x 16 KiB][X tiles 2 x npad*512][packed stages 2 x 128*chunk_bytes][barriers]
    uint8_t *a_slabs = smem;
    const uint32_t b_tile_bytes = a.npad * 128u * TC_SLABS;
    constexpr uint32_t RING = TC_MAX_RING;   // compile-time ring sizes: the divisions below sit on the hand-off path of every slab
    uint8_t *b_tiles = a_slabs + RING * 16384;
    const uint32_t pk_stage_bytes = (TC_M * a.chunk_bytes + 127u) & ~127u;
    constexpr uint32_t BS = TC_B_STAGES;
    uint8_t *pk = b_tiles + BS * b_tile_bytes;
    constexpr uint32_t PKS = tc_pk_stages(FMT);
    uint64_t *bars = reinterpret_cast<uint64_t *>(pk + PKS * pk_stage_bytes);
    uint64_t *pk_full = bars, *pk_empty = bars + TC_PK_MAX_STAGES, *b_full = pk_empty + TC_PK_MAX_STAGES, *b_empty = b_full + TC_B_MAX_STAGES;
    uint64_t *a_full = b_empty + TC_B_MAX_STAGES, *a_empty = a_full + TC_MAX_RING, *acc_done = a_empty + TC_MAX_RING;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_done + 1);
    __shared__ volatile int s_abort;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t tile = blockIdx.x / a.split, sp = blockIdx.x % a.split;
    const uint32_t row0 = tile * TC_M, nrows = min((uint32_t)TC_M, a.rows - row0);
    const uint32_t chunk0 = sp * a.chunks / a.split, nchunks = (sp + 1) * a.chunks / a.split - chunk0;
    uint32_t ncols = 32;
    while (ncols < a.npad) ncols <<= 1;
    // Every CTA walks its chunks of K from a different starting point (and wraps): at any one time the CTAs then read
    // different tiles of the packed X, instead of all of them fetching the same 32 KB from the same few L2 slices at
    // the same moment (measured: 3700 cycles for one X tile in lockstep).  The sum over K does not care about order.
    const uint32_t rot = (tile * 5u + sp * 3u) % nchunks;

    if (tid == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < PKS; ++s) { mbar_init(smem_u32(pk_full + s), 1); mbar_init(smem_u32(pk_empty + s), TC_DEQ_WARPS); }
        for (uint32_t s = 0; s < BS; ++s) { mbar_init(smem_u32(b_full + s), 1); mbar_init(smem_u32(b_empty + s), 1); }
        for (uint32_t s = 0; s < RING; ++s) { mbar_init(smem_u32(a_full + s), TC_SLAB_WARPS); mbar_init(smem_u32(a_empty + s), 1); }
        mbar_init(smem_u32(acc_done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {   // TMEM allocation: one warp, power-of-two columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    pdl_launch_dependents();

    auto wait = [&](uint64_t *bar, uint32_t parity) {
        if (!s_abort && !mbar_wait_bounded(smem_u32(bar), parity)) { s_abort = 1; atomicExch(a.status, 4); }
    };

    if (warp == TC_DEQ_WARPS) {
        // ---- weight producer: packed stages, independent of the previous kernel ----
        if (lane == 0) {
            const uint32_t words = a.chunk_bytes / 4;
            for (uint32_t c = 0; c < nchunks && !s_abort; ++c) {
                const uint32_t s = c % PKS, k = c / PKS;
                if (k > 0) { wait(pk_empty + s, (k - 1) & 1u); asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
                mbar_expect_tx(smem_u32(pk_full + s), TC_M * a.chunk_bytes);   // the box is always full: out-of-range rows arrive as zeros
                // x coordinate in 32-bit words: (chunk index) * chunk_bytes / 4, a multiple of 16 bytes for every format
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(smem_u32(pk + (size_t)s * pk_stage_bytes)), "l"(&a.wmap), "r"((chunk0 + (c + rot < nchunks ? c + rot : c + rot - nchunks)) * words), "r"(row0),
                               "r"(smem_u32(pk_full + s)) : "memory");
                TC_STAMP(0, c);
            }
        }
    } else if (warp == TC_DEQ_WARPS + 2) {
        // ---- X producer: the matching pre-packed fp16 tiles (the previous kernel's output) ----
        if (lane == 0) {
            pdl_wait();
            for (uint32_t c = 0; c < nchunks && !s_abort; ++c) {
                const uint32_t sb = c % BS, kb = c / BS;
                if (kb > 0) { wait(b_empty + sb, (kb - 1) & 1u); asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
                mbar_expect_tx(smem_u32(b_full + sb), b_tile_bytes);
                bulk_g2s(smem_u32(b_tiles + (size_t)sb * b_tile_bytes),
                         reinterpret_cast<const uint8_t *>(a.xp) + (size_t)(chunk0 + (c + rot < nchunks ? c + rot : c + rot - nchunks)) * b_tile_bytes,
                         b_tile_bytes, smem_u32(b_full + sb));
                TC_STAMP(6, c);
            }
        }
    } else if (warp == TC_DEQ_WARPS + 1) {
        // ---- MMA issue: one thread ----
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((a.npad >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);   // fp32 accumulate, fp16 x fp16, K-major both
            uint32_t slab_i = 0;
            for (uint32_t c = 0; c < nchunks && !s_abort; ++c) {
                const uint32_t sb = c % BS;
                wait(b_full + sb, (c / BS) & 1u);
                TC_STAMP(7, c);
                for (uint32_t j = 0; j < TC_SLABS; ++j, ++slab_i) {
                    const uint32_t sa = slab_i % RING;
                    wait(a_full + sa, (slab_i / RING) & 1u);
                    TC_STAMP(4, slab_i);
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(a_slabs + sa * 16384), b_addr = smem_u32(b_tiles + (size_t)sb * b_tile_bytes + (size_t)j * a.npad * 128);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < 4; ++k16)
                        tc_mma_f16(tmem_acc, tc_desc_sw128(a_addr + k16 * 32), tc_desc_sw128(b_addr + k16 * 32), idesc, (slab_i | k16) ? 1u : 0u);
                    tc_commit(smem_u32(a_empty + sa));     // slab free once these MMAs have read it
                    TC_STAMP(5, slab_i);
                }
                tc_commit(smem_u32(b_empty + sb));
            }
            tc_commit(smem_u32(acc_done));
        }
    } else {
        // ---- dequant warps: packed stage -> fp16 slabs ----
        // Two groups of eight warps fill alternate slabs, one (row, 32-weight group) per thread.  (One thread per row and
        // sub-block pair, which shares the header and scale unpacking, measured 10 % slower: the slab's latency counts.)
        const uint32_t dt = tid & 255u, grp = warp / TC_SLAB_WARPS;
        uint32_t slab_i = 0;
        for (uint32_t c = 0; c < nchunks; ++c) {
            const uint32_t s = c % PKS;
            wait(pk_full + s, (c / PKS) & 1u);
            if (tid == 0) TC_STAMP(1, c);
            const uint8_t *stage = pk + (size_t)s * pk_stage_bytes;
            for (uint32_t j = 0; j < TC_SLABS; ++j, ++slab_i) {
                if ((slab_i & 1u) != grp) continue;
                const uint32_t sa = slab_i % RING, ka = slab_i / RING;
                if (ka > 0) wait(a_empty + sa, (ka - 1) & 1u);
                if ((tid & 255u) == 0) TC_STAMP(2, slab_i);
                tc_fence_after();
                uint8_t *slab = a_slabs + sa * 16384;
                // a slab is 128 rows x two 32-weight groups: one (row, group) per thread, four 16-byte pieces each
                {
                    const uint32_t r = dt >> 1, half = dt & 1u;
                    uint4 v[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                    if (r < nrows) dequant_group32<FMT>(stage + (size_t)r * a.chunk_bytes, j * 2 + half, a.layout, v);
#pragma unroll
                    for (uint32_t p = 0; p < 4; ++p) *reinterpret_cast<uint4 *>(slab + sw128_off(r, half * 4 + p)) = v[p];
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(a_full + sa));
                if ((tid & 255u) == 0) TC_STAMP(3, slab_i);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(pk_empty + s));
        }
        // ---- epilogue: warps 0-3, lane = row ----
        if (warp < 4) {
            wait(acc_done, 0);
            tc_fence_after();
            const uint32_t r = warp * 32 + lane;
            float *ybase = a.split == 1 ? a.y : a.y + (size_t)sp * a.batch * a.rows;
            const uint32_t ld = a.split == 1 ? a.ldy : a.rows;
            const bool publish = a.split == 1 && a.pub.npeers > 0;
            const unsigned int pub_tag = publish ? *reinterpret_cast<const volatile unsigned int *>(a.pub.pub_gen) + 1u : 0u;
            for (uint32_t n0 = 0; n0 < a.npad; n0 += 16) {
                uint32_t v[16];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                               "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                             : "r"(tmem_acc + ((warp * 32u) << 16) + n0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < nrows && !s_abort) {
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i)
                        if (n0 + i < a.batch) {
                            float *dst = ybase + (size_t)(n0 + i) * ld + row0 + r;
                            *dst = __uint_as_float(v[i]);
                            if (publish) tc_publish(a.pub, dst, __uint_as_float(v[i]), pub_tag);
                        }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(ncols) : "memory");
    }
    if (threadIdx.x == 0 && a.split == 1 && a.pub.npeers > 0)
        tc_publish_done(a.pub, *reinterpret_cast<const volatile unsigned int *>(a.pub.pub_gen) + 1u);
}


// ---- the same product with the dequantized weights in TENSOR MEMORY --------------------------------------------------
// Two findings from cycle-stamping the form above drive this one.
// (1) A 256-weight chunk of a 128-row tile costs 64 KB of shared-memory stores (the fp16 slabs) and 64 KB of operand
//     reads by the tensor core next to 18 KB of packed weights; its MMAs took ~100 cycles each instead of ~34.  Here
//     the dequant warps write the fp16 weights straight into tensor memory (tcgen05.st: lane = row, two weights per
//     32-bit column) and the MMA takes its A operand from there.
// (2) The copy engine, not memory, set the pace after that: a tensor copy of 128 rows x 144 bytes took ~2100 cycles
//     whether the tensor sat in HBM or in L2, and everything else queued behind it (an X tile: 4000-8000 cycles).
//     Here the dequant threads read their packed weights with plain 16-byte loads straight into registers, one unit
//     ahead of the one they convert; the copy engine carries only the X tiles.
// A CTA works on `tiles_per_cta` (TT) row tiles side by side: every X tile is fetched once and multiplied with the
// chunk of each of its row tiles, each with its own accumulator; K is split over more CTAs (args.split) instead.
//   tensor memory (512 columns): A stages of 128 columns (one chunk of one row tile: 128 rows x 256 fp16) from column
//   0; TT accumulators of 64 columns at the top (TT = 1, 2: three A stages; TT = 4: two).
//   dequant warp w: rows 32 * (w % 4) + lane (the lanes of tensor memory a warp may touch), weights
//   64 * (w / 4) .. + 63 of the chunk; every warp works on every (chunk, tile) unit.
constexpr int TCA_B_STAGES = 4;
constexpr int TCA_MAX_TT = 4;
constexpr int TCA_THREADS = (TC_DEQ_WARPS + 2) * 32;     // + MMA issuer, X producer
constexpr uint32_t tca_a_stages(uint32_t tt) { return (512u - 64u * tt) / 128u; }

__device__ __forceinline__ void tc_mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint4 (&v)[4])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w),
                   "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z), "r"(v[3].w) : "memory");
}

// The packed bytes one dequant thread needs for its 64 weights (sub-blocks 2kq, 2kq+1 of a K-quant superblock, blocks
// 2kq, 2kq+1 of a Q8_0 chunk) of one row, as 16-byte pieces.
//   Q4_K: header (d, dmin, 12 scale bytes), 32 quant bytes (low nibbles = sub-block 2kq, high = 2kq+1).
//   Q5_K: the same plus the 32 bytes of fifth bits (all eight sub-blocks share them).
//   Q8_0: the 80 bytes from the 16-byte boundary at or below byte 68*kq of the chunk; the thread's 68 bytes start kq words in.
//   Q6_K (210-byte superblocks, 2-byte aligned): thread kq takes half n = kq / 2 of the superblock and the elements
//   l = 16 (kq % 2) .. + 15 of that half's four 32-groups (weights 128 n + 32 j + l, j = 0..3): 16 bytes of ql[l],
//   16 of ql[32 + l], 16 of qh[l], the half's eight scale bytes and d.  (Taking 64 consecutive weights instead would
//   need all 64 ql bytes for one of their nibbles each.)
template <int FMT> struct TcPacked { uint4 p[FMT == FMT_Q4_K ? 3 : 5]; };
template <> struct TcPacked<FMT_Q6_K> { uint32_t qa[4], qb[4], qh[4], sc[2], d; };

// N consecutive 32-bit words from a 2-byte aligned address: aligned word loads, one more and a funnel shift when the
// address is 2 (mod 4).  Reads at most two bytes before p and never a whole word past p + 4 N.
template <int N>
__device__ __forceinline__ void ldg_words_a2(const uint8_t *p, uint32_t (&out)[N])
{
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
    const bool odd = (a & 2u) != 0;
    uint32_t w[N + 1];
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __ldg(q + i);
    w[N] = odd ? __ldg(q + N) : 0u;
    const uint32_t sh = odd ? 16u : 0u;
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
}

template <int FMT>
__device__ __forceinline__ void tc_load_packed(const uint8_t *chunk, uint32_t kq, bool live, TcPacked<FMT> &d)
{
    if constexpr (FMT == FMT_Q6_K) {
        if (!live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) d.qa[i] = d.qb[i] = d.qh[i] = 0u;
            d.sc[0] = d.sc[1] = d.d = 0u;
            return;
        }
        const uint32_t n = kq >> 1, l0 = 16u * (kq & 1u);
        ldg_words_a2<4>(chunk + 64u * n + l0, d.qa);
        ldg_words_a2<4>(chunk + 64u * n + 32u + l0, d.qb);
        ldg_words_a2<4>(chunk + 128u + 32u * n + l0, d.qh);
        ldg_words_a2<2>(chunk + 192u + 8u * n, d.sc);
        d.d = __ldg(reinterpret_cast<const unsigned short *>(chunk + 208));
        return;
    } else {
    constexpr int N = FMT == FMT_Q4_K ? 3 : 5;
    if (!live) {
#pragma unroll
        for (int i = 0; i < N; ++i) d.p[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    if constexpr (FMT == FMT_Q8_0) {
        const uint4 *src = reinterpret_cast<const uint4 *>(chunk + ((kq * 68u) & ~15u));
#pragma unroll
        for (int i = 0; i < 5; ++i) d.p[i] = __ldg(src + i);
    } else {
        d.p[0] = __ldg(reinterpret_cast<const uint4 *>(chunk));
        constexpr uint32_t QOFF = FMT == FMT_Q4_K ? 16u : 48u;
        const uint4 *q = reinterpret_cast<const uint4 *>(chunk + QOFF + 32u * kq);
        d.p[1] = __ldg(q);
        d.p[2] = __ldg(q + 1);
        if constexpr (FMT == FMT_Q5_K) {
            d.p[3] = __ldg(reinterpret_cast<const uint4 *>(chunk + 16));
            d.p[4] = __ldg(reinterpret_cast<const uint4 *>(chunk + 32));
        }
    }
    }
}

// 32 weights (half h of the thread's 64) from the packed pieces -> four 16-byte fp16 pieces, element order.
template <int FMT, int KQ>
__device__ __forceinline__ void tc_dequant_half(const TcPacked<FMT> &d, uint32_t h, int layout, uint4 (&out)[4])
{
    uint32_t w[8];
    __half2 scale, bias, addend;
    if constexpr (FMT == FMT_Q8_0) {
        // words KQ .. KQ+16 of the 20 loaded: block A = fp16 scale in the low half of word KQ, quants from its upper half
        // on; block B = scale in the upper half of word KQ+8, quants = words KQ+9 .. KQ+16
        const uint32_t v[20] = {d.p[0].x, d.p[0].y, d.p[0].z, d.p[0].w, d.p[1].x, d.p[1].y, d.p[1].z, d.p[1].w, d.p[2].x, d.p[2].y,
                                d.p[2].z, d.p[2].w, d.p[3].x, d.p[3].y, d.p[3].z, d.p[3].w, d.p[4].x, d.p[4].y, d.p[4].z, d.p[4].w};
        uint32_t dbits;
        if (h == 0) {
            dbits = v[KQ] & 0xffffu;
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = __byte_perm(v[KQ + i], v[KQ + i + 1], 0x5432u) ^ 0x80808080u;
        } else {
            dbits = v[KQ + 8] >> 16;
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = v[KQ + 9 + i] ^ 0x80808080u;
        }
        const float dd = __half2float(__ushort_as_half((unsigned short)dbits));
        scale = __float2half2_rn(dd); bias = __float2half2_rn(1152.0f); addend = __float2half2_rn(0.0f);   // bytes are q + 128
    } else {
        const uint4 hd = d.p[0];
        uint32_t scA, scB, mnA, mnB;
        pair_scales(hd.y, hd.z, hd.w, layout, KQ, scA, scB, mnA, mnB);
        const uint32_t sc = h ? scB : scA, mn = h ? mnB : mnA;
        const float dd = __half2float(__ushort_as_half((unsigned short)(hd.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hd.x >> 16)));
        w[0] = d.p[1].x; w[1] = d.p[1].y; w[2] = d.p[1].z; w[3] = d.p[1].w; w[4] = d.p[2].x; w[5] = d.p[2].y; w[6] = d.p[2].z; w[7] = d.p[2].w;
        const uint32_t shift = h * 4u;
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (w[i] >> shift) & 0x0F0F0F0Fu;
        if constexpr (FMT == FMT_Q5_K) {
            const uint32_t hb[8] = {d.p[3].x, d.p[3].y, d.p[3].z, d.p[3].w, d.p[4].x, d.p[4].y, d.p[4].z, d.p[4].w};
            const uint32_t g32 = 2u * KQ + h;
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] |= ((hb[i] >> g32) & 0x01010101u) << 4;
        }
        scale = __float2half2_rn(dd * (float)sc); bias = __float2half2_rn(1024.0f); addend = __float2half2_rn(-(dmin * (float)mn));
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        out[p].x = h2_bits(two_weights(w[2 * p], 0x5140u, bias, scale, addend));
        out[p].y = h2_bits(two_weights(w[2 * p], 0x7362u, bias, scale, addend));
        out[p].z = h2_bits(two_weights(w[2 * p + 1], 0x5140u, bias, scale, addend));
        out[p].w = h2_bits(two_weights(w[2 * p + 1], 0x7362u, bias, scale, addend));
    }
}

__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t (&v)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

// Q6_K, 32-group J of the thread's half: its 16 weights (q - 32) * d * scale as fp16, two per word (format.m:131-174:
// ql nibble | two qh bits << 4, scale 8 n + 2 J + l / 16).
template <int KQ, int J>
__device__ __forceinline__ void tc_dequant_q6_group(const TcPacked<FMT_Q6_K> &d, uint32_t (&out)[8])
{
    constexpr int SI = (KQ & 1) + 2 * J;             // scale byte inside the half's eight
    const int sc = (int)(signed char)((d.sc[SI >> 2] >> (8 * (SI & 3))) & 0xffu);
    const float dd = __half2float(__ushort_as_half((unsigned short)d.d));
    const __half2 scale = __float2half2_rn(dd * (float)sc), bias = __float2half2_rn(1056.0f), addend = __float2half2_rn(0.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t ql = (J & 1) ? d.qb[i] : d.qa[i];
        const uint32_t lo = (J < 2 ? ql : ql >> 4) & 0x0F0F0F0Fu;
        const uint32_t w = lo | (((d.qh[i] >> (2 * J)) & 0x03030303u) << 4);
        out[2 * i] = h2_bits(two_weights(w, 0x5140u, bias, scale, addend));
        out[2 * i + 1] = h2_bits(two_weights(w, 0x7362u, bias, scale, addend));
    }
}

// taddr: the thread's lane and the stage's column 32 * KQ (two weights per column).
template <int FMT, int KQ>
__device__ __forceinline__ void tc_convert_unit(const TcPacked<FMT> &d, int layout, uint32_t taddr)
{
    if constexpr (FMT == FMT_Q6_K) {
        // group J, elements 16 (KQ % 2) ..: weights 128 (KQ / 2) + 32 J + 16 (KQ % 2) .., i.e. column 64 (KQ / 2) + 16 J + 8 (KQ % 2)
        const uint32_t col = taddr - 24u * (KQ & 1);
        uint32_t v[8];
        tc_dequant_q6_group<KQ, 0>(d, v); tc_st8(col, v);
        tc_dequant_q6_group<KQ, 1>(d, v); tc_st8(col + 16u, v);
        tc_dequant_q6_group<KQ, 2>(d, v); tc_st8(col + 32u, v);
        tc_dequant_q6_group<KQ, 3>(d, v); tc_st8(col + 48u, v);
    } else {
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) {
            uint4 v[4];
            tc_dequant_half<FMT, KQ>(d, h, layout, v);
            tc_st16(taddr + h * 16u, v);
        }
    }
}

template <int FMT>
__global__ void __launch_bounds__(TCA_THREADS, 1)
gemm_tca_kernel(const __grid_constant__ TcArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // layout: [X tiles BS x npad*512][barriers]
    constexpr uint32_t BS = TCA_B_STAGES, MAX_AS = 3;
    const uint32_t TT = a.tiles_per_cta, AS = tca_a_stages(TT);
    const uint32_t b_tile_bytes = a.npad * 128u * TC_SLABS;
    uint8_t *b_tiles = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(b_tiles + BS * b_tile_bytes);
    uint64_t *b_full = bars, *b_empty = b_full + BS;
    uint64_t *a_full = b_empty + BS, *a_empty = a_full + MAX_AS, *acc_done = a_empty + MAX_AS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_done + 1);
    __shared__ volatile int s_abort;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t tgroup = blockIdx.x / a.split, sp = blockIdx.x % a.split;
    const uint32_t tile0 = tgroup * TT;                          // this CTA's row tiles: tile0 .. tile0 + TT - 1 (those inside the tensor)
    const uint32_t chunk0 = sp * a.chunks / a.split, nchunks = (sp + 1) * a.chunks / a.split - chunk0;
    const uint32_t rot = (tgroup * 5u + sp * 3u) % nchunks;      // CTAs start their walk over K at different chunks
    const uint32_t nunits = nchunks * TT;                        // unit u = (chunk u / TT, tile u % TT)
    const uint32_t acc_col0 = 512u - 64u * TT;

    if (tid == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < BS; ++s) { mbar_init(smem_u32(b_full + s), 1); mbar_init(smem_u32(b_empty + s), 1); }
        for (uint32_t s = 0; s < MAX_AS; ++s) { mbar_init(smem_u32(a_full + s), TC_DEQ_WARPS); mbar_init(smem_u32(a_empty + s), 1); }
        mbar_init(smem_u32(acc_done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {   // all 512 columns: one CTA per SM (its shared memory request sees to that)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    pdl_launch_dependents();

    auto wait = [&](uint64_t *bar, uint32_t parity) {
        if (!s_abort && !mbar_wait_bounded(smem_u32(bar), parity)) { s_abort = 1; atomicExch(a.status, 4); }
    };
    auto chunk_of = [&](uint32_t c) { return chunk0 + (c + rot < nchunks ? c + rot : c + rot - nchunks); };

    if (warp == TC_DEQ_WARPS + 1) {
        // ---- X producer: the pre-packed fp16 tiles (the previous kernel's output), one per chunk ----
        if (lane == 0) {
            pdl_wait();
            for (uint32_t c = 0; c < nchunks && !s_abort; ++c) {
                const uint32_t sb = c % BS, kb = c / BS;
                if (kb > 0) { wait(b_empty + sb, (kb - 1) & 1u); asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
                mbar_expect_tx(smem_u32(b_full + sb), b_tile_bytes);
                bulk_g2s(smem_u32(b_tiles + (size_t)sb * b_tile_bytes), reinterpret_cast<const uint8_t *>(a.xp) + (size_t)chunk_of(c) * b_tile_bytes,
                         b_tile_bytes, smem_u32(b_full + sb));
                TC_STAMP(6, c);
            }
        }
    } else if (warp == TC_DEQ_WARPS) {
        // ---- MMA issue: one thread; 16 x (M128 x N x K16) per unit, A from tensor memory, B = the chunk's X tile ----
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((a.npad >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);   // fp32 accumulate, fp16 x fp16, K-major both
            uint32_t sa = 0, ka = 0, u = 0;
            for (uint32_t c = 0; c < nchunks && !s_abort; ++c) {
                const uint32_t sb = c % BS;
                wait(b_full + sb, (c / BS) & 1u);
                TC_STAMP(7, c);
                const uint32_t b_addr = smem_u32(b_tiles + (size_t)sb * b_tile_bytes);
                for (uint32_t t = 0; t < TT; ++t, ++u) {
                    wait(a_full + sa, ka & 1u);
                    TC_STAMP(4, u);
                    tc_fence_after();
                    const uint32_t a_col = tmem_base + sa * 128u, d_col = tmem_base + acc_col0 + t * 64u;
#pragma unroll
                    for (uint32_t k16 = 0; k16 < 16; ++k16)
                        tc_mma_f16_ta(d_col, a_col + k16 * 8u, tc_desc_sw128(b_addr + (k16 >> 2) * a.npad * 128u + (k16 & 3u) * 32u), idesc,
                                      (c | k16) ? 1u : 0u);
                    tc_commit(smem_u32(a_empty + sa));     // the A stage is free once these MMAs have read it
                    TC_STAMP(5, u);
                    if (++sa == AS) { sa = 0; ++ka; }
                }
                tc_commit(smem_u32(b_empty + sb));         // and the X tile after the chunk's last row tile
            }
            tc_commit(smem_u32(acc_done));
        }
    } else {
        // ---- dequant warps: packed weights (global -> registers, one unit ahead) -> fp16 weights in tensor memory ----
        const uint32_t quad = warp & 3u, kq = warp >> 2, r = quad * 32u + lane;
        const uint32_t lane_addr = (quad * 32u) << 16;
        uint32_t sa = 0, ka = 0, t = 0, c = 0;
        auto unit_ptr = [&](uint32_t cc, uint32_t tt, bool &live) {
            const uint32_t grow = (tile0 + tt) * TC_M + r;
            live = grow < a.rows;
            return a.w + (size_t)grow * a.row_bytes + (size_t)chunk_of(cc) * a.chunk_bytes;
        };
        TcPacked<FMT> cur, nxt;
        {
            bool live;
            const uint8_t *p = unit_ptr(0, 0, live);
            tc_load_packed<FMT>(p, kq, live, cur);
        }
        for (uint32_t u = 0; u < nunits; ++u) {
            uint32_t tn = t + 1, cn = c;
            if (tn == TT) { tn = 0; ++cn; }
            if (u + 1 < nunits) {                 // the next unit's bytes are on their way while this one is converted
                bool live;
                const uint8_t *p = unit_ptr(cn, tn, live);
                tc_load_packed<FMT>(p, kq, live, nxt);
            }
            if (tid == 0) TC_STAMP(1, u);
            if (ka > 0) wait(a_empty + sa, (ka - 1) & 1u);
            if (tid == 0) TC_STAMP(2, u);
            tc_fence_after();
            const uint32_t taddr = tmem_base + lane_addr + sa * 128u + kq * 32u;
            switch (kq) {                         // warp-uniform; the sub-block index is a compile-time constant inside
            case 0: tc_convert_unit<FMT, 0>(cur, a.layout, taddr); break;
            case 1: tc_convert_unit<FMT, 1>(cur, a.layout, taddr); break;
            case 2: tc_convert_unit<FMT, 2>(cur, a.layout, taddr); break;
            default: tc_convert_unit<FMT, 3>(cur, a.layout, taddr); break;
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(a_full + sa));
                if (tid == 0) TC_STAMP(3, u);
            }
            cur = nxt;
            if (++sa == AS) { sa = 0; ++ka; }
            t = tn; c = cn;
        }
        // ---- epilogue: warps 0-3, lane = row, one accumulator per row tile ----
        if (warp < 4) {
            wait(acc_done, 0);
            tc_fence_after();
            float *ybase = a.split == 1 ? a.y : a.y + (size_t)sp * a.batch * a.rows;
            const uint32_t ld = a.split == 1 ? a.ldy : a.rows;
            const bool publish = a.split == 1 && a.pub.npeers > 0;
            const unsigned int pub_tag = publish ? *reinterpret_cast<const volatile unsigned int *>(a.pub.pub_gen) + 1u : 0u;
            for (uint32_t tt = 0; tt < TT; ++tt) {
                const uint32_t grow = (tile0 + tt) * TC_M + warp * 32 + lane;
                for (uint32_t n0 = 0; n0 < a.npad; n0 += 16) {
                    uint32_t v[16];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                                 : "r"(tmem_base + ((warp * 32u) << 16) + acc_col0 + tt * 64u + n0));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (grow < a.rows && !s_abort) {
#pragma unroll
                        for (uint32_t i = 0; i < 16; ++i)
                            if (n0 + i < a.batch) {
                                float *dst = ybase + (size_t)(n0 + i) * ld + grow;
                                *dst = __uint_as_float(v[i]);
                                if (publish) tc_publish(a.pub, dst, __uint_as_float(v[i]), pub_tag);
                            }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if (threadIdx.x == 0 && a.split == 1 && a.pub.npeers > 0)
        tc_publish_done(a.pub, *reinterpret_cast<const volatile unsigned int *>(a.pub.pub_gen) + 1u);
}

// Y[b][r] = sum over splits of partial[s][b][r]
__global__ void splitk_reduce_kernel(const float *__restrict__ part, uint32_t split, uint32_t batch, uint32_t rows, float *__restrict__ y, uint32_t ldy,
                                     const TcPub pub)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned int pub_tag = pub.npeers > 0 ? *reinterpret_cast<const volatile unsigned int *>(pub.pub_gen) + 1u : 0u;
    const size_t n = (size_t)batch * rows;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (uint32_t s = 0; s < split; ++s) acc += part[(size_t)s * n + i];
        float *dst = y + (i / rows) * ldy + (i % rows);
        *dst = acc;
        if (pub.npeers > 0) tc_publish(pub, dst, acc, pub_tag);
    }
    if (pub.npeers > 0) {
        __syncthreads();
        if (threadIdx.x == 0) tc_publish_done(pub, pub_tag);
    }
}

}  // namespace orome
