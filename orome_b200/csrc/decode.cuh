// decode.cuh -- device-side block decoders shared by every kernel of the path.
//
// Bit-exact contract: decode32() reproduces the reference's CPU decode
// (inference/src/format.m:17-174) for 32 consecutive weights of a row, using
// explicitly rounded multiplies / subtracts (no reliance on -fmad).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace orome {

enum : int { FMT_Q4_K = 0, FMT_Q5_K = 1, FMT_Q6_K = 2, FMT_Q8_0 = 3, FMT_F16 = 4, FMT_BF16 = 5, FMT_F32 = 6 };
enum : int { LAYOUT_A = 0, LAYOUT_B = 1 };

__host__ __device__ constexpr int block_bytes(int fmt)
{
    return fmt == FMT_Q8_0 ? 34 : fmt == FMT_Q4_K ? 144 : fmt == FMT_Q5_K ? 176 : fmt == FMT_Q6_K ? 210 : 0;
}
__host__ __device__ constexpr int block_elems(int fmt) { return fmt == FMT_Q8_0 ? 32 : 256; }

// IEEE half bits -> float with the reference's conventions (format.m:17-32):
// every finite value and infinity exactly; any NaN becomes the positive quiet NaN.
__device__ __forceinline__ float half_bits_to_float(uint32_t h)
{
    float f = __half2float(__ushort_as_half((unsigned short)h));
    if ((h & 0x7C00u) == 0x7C00u && (h & 0x3FFu)) f = __uint_as_float(0x7FC00000u);
    return f;
}

__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }

// Six-bit scale and min of sub-block `sub` (0..7) from the 12 packed bytes.
// Layout A: format.m:41-64.  Layout B: shaders.metal:1575-1578.
__device__ __forceinline__ void kq_scale_min(const uint8_t *p, int layout, int sub, uint32_t &sc, uint32_t &mn)
{
    if (sub < 4) {
        sc = p[sub] & 63u;
        mn = p[sub + 4] & 63u;
    } else if (layout == LAYOUT_A) {
        int u = (sub - 4) >> 1, hi = sub & 1;
        uint32_t sp = p[8 + u], mp = p[10 + u];
        sc = (hi ? (sp >> 4) : (sp & 15u)) | ((uint32_t)(p[2 * u + hi] >> 6) << 4);
        mn = (hi ? (mp >> 4) : (mp & 15u)) | ((uint32_t)(p[2 * u + 4 + hi] >> 6) << 4);
    } else {
        sc = (p[sub + 4] & 15u) | ((uint32_t)(p[sub - 4] >> 6) << 4);
        mn = (uint32_t)(p[sub + 4] >> 4) | ((uint32_t)(p[sub] >> 6) << 4);
    }
}

// Decode weights [32*b32, 32*b32 + 32) of the row starting at `row`.
template <int FMT>
__device__ __forceinline__ void decode32(const uint8_t *__restrict__ row, uint32_t b32, int layout, float (&w)[32])
{
    if constexpr (FMT == FMT_Q8_0) {
        const uint8_t *blk = row + (size_t)b32 * 34;
        float d = half_bits_to_float(ld16(blk));
        const int8_t *q = reinterpret_cast<const int8_t *>(blk + 2);
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = __fmul_rn(d, (float)q[j]);
    } else if constexpr (FMT == FMT_Q4_K || FMT == FMT_Q5_K) {
        constexpr int BB = FMT == FMT_Q4_K ? 144 : 176;
        const uint8_t *sb = row + (size_t)(b32 >> 3) * BB;
        int sub = b32 & 7;
        float d = half_bits_to_float(ld16(sb)), dmin = half_bits_to_float(ld16(sb + 2));
        uint32_t sc, mn;
        kq_scale_min(sb + 4, layout, sub, sc, mn);
        float a = __fmul_rn(d, (float)sc), m = __fmul_rn(dmin, (float)mn);
        const uint8_t *qs = sb + (FMT == FMT_Q4_K ? 16 : 48) + 32 * (sub >> 1);
        int shift = (sub & 1) * 4;
#pragma unroll
        for (int l = 0; l < 32; ++l) {
            uint32_t q = (qs[l] >> shift) & 15u;
            if constexpr (FMT == FMT_Q5_K) q |= ((uint32_t)(sb[16 + l] >> sub) & 1u) << 4;
            w[l] = __fsub_rn(__fmul_rn(a, (float)q), m);
        }
    } else if constexpr (FMT == FMT_Q6_K) {
        const uint8_t *sb = row + (size_t)(b32 >> 3) * 210;
        int half = (b32 >> 2) & 1, t = b32 & 3;
        const uint8_t *ql = sb + 64 * half + 32 * (t & 1), *qh = sb + 128 + 32 * half;
        const int8_t *sc = reinterpret_cast<const int8_t *>(sb + 192 + 8 * half + 2 * t);
        float d = half_bits_to_float(ld16(sb + 208));
#pragma unroll
        for (int l = 0; l < 32; ++l) {
            int lo = (ql[l] >> (4 * (t >> 1))) & 15, hi = (qh[l] >> (2 * t)) & 3;
            int q = (lo | (hi << 4)) - 32;
            w[l] = __fmul_rn(__fmul_rn(d, (float)sc[l >> 4]), (float)q);
        }
    } else if constexpr (FMT == FMT_F16) {
        const uint8_t *p = row + (size_t)b32 * 64;
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = half_bits_to_float(ld16(p + 2 * j));
    } else if constexpr (FMT == FMT_BF16) {
        const uint8_t *p = row + (size_t)b32 * 64;
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = __uint_as_float(ld16(p + 2 * j) << 16);
    } else {
        const float *p = reinterpret_cast<const float *>(row) + (size_t)b32 * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = p[j];
    }
}

__host__ __device__ inline size_t row_bytes_of(int fmt, uint32_t in_dim)
{
    switch (fmt) {
    case FMT_Q8_0: return (size_t)(in_dim / 32) * 34;
    case FMT_Q4_K: return (size_t)(in_dim / 256) * 144;
    case FMT_Q5_K: return (size_t)(in_dim / 256) * 176;
    case FMT_Q6_K: return (size_t)(in_dim / 256) * 210;
    case FMT_F16: case FMT_BF16: return (size_t)in_dim * 2;
    case FMT_F32: return (size_t)in_dim * 4;
    }
    return 0;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// Order-preserving key of a float (larger float, larger key), so that {key, ~index} packed in 64 bits orders
// candidates by value first and by LOWER index second.
__device__ __forceinline__ uint32_t float_key(float v)
{
    const uint32_t b = __float_as_uint(v + 0.0f);      // -0 and +0 compare equal, so they share a key
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Tie order of the reference's argmax_kernel (shaders.metal:1249-1305).  Its 1024 threads stride over the vector and
// each keeps its FIRST maximum; a shuffle-down tree (offsets 16, 8, 4, 2, 1; the lower lane keeps its pair unless the
// other value is strictly greater) reduces the 32 lanes of a simdgroup, and the same tree reduces the 32 simdgroups.
// In such a tree lane 0 ends up preferring, among equal values, the lane whose 5-bit number read backwards is
// smallest (the last step decides between even and odd lanes, the one before between lanes = 0 and 2 mod 4, ...).
// So among equal values the winner has the smallest bit-reversed simdgroup, then the smallest bit-reversed lane,
// then the smallest index: argmax_rank() packs exactly that order.
__device__ __host__ __forceinline__ uint32_t brev5(uint32_t v) { return ((v & 1u) << 4) | ((v & 2u) << 2) | (v & 4u) | ((v & 8u) >> 2) | ((v & 16u) >> 4); }
__device__ __host__ __forceinline__ uint32_t argmax_rank(uint32_t i) { return (brev5((i >> 5) & 31u) << 27) | (brev5(i & 31u) << 22) | (i >> 10); }
__device__ __host__ __forceinline__ uint32_t argmax_unrank(uint32_t r) { return ((r & 0x3FFFFFu) << 10) | (brev5(r >> 27) << 5) | brev5((r >> 22) & 31u); }

}  // namespace orome
