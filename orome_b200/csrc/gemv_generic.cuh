// gemv_generic.cuh -- shape-agnostic kernels: row decode, warp-per-row matvec for
// any format / batch, SwiGLU epilogue.  They take every shape the formats allow;
// the pipelined kernels in gemv_pipe.cuh take over for the decode-sized ones.
#pragma once
#include "decode.cuh"

namespace orome {

// One thread per 32-weight group: out[(r - row0) * in_dim + 32*b .. +32].
// Device counterpart of format_decode_row_f32 (format.m:176-218).
template <int FMT>
__global__ void dequant_rows_kernel(const uint8_t *__restrict__ data, size_t row_bytes, uint32_t row0, uint32_t nrows,
                                    uint32_t in_dim, int layout, float *__restrict__ out)
{
    uint32_t groups = in_dim / 32;
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (size_t)nrows * groups) return;
    uint32_t r = (uint32_t)(gid / groups), b = (uint32_t)(gid % groups);
    float w[32];
    decode32<FMT>(data + (size_t)(row0 + r) * row_bytes, b, layout, w);
    float4 *o = reinterpret_cast<float4 *>(out + (size_t)r * in_dim + (size_t)b * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = make_float4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

// Tail of an unquantized row whose length is not a multiple of 32 (F32/F16/BF16 only).
template <int FMT>
__device__ __forceinline__ float plain_elem(const uint8_t *row, uint32_t c)
{
    if constexpr (FMT == FMT_F32) return reinterpret_cast<const float *>(row)[c];
    else if constexpr (FMT == FMT_F16) return half_bits_to_float(ld16(row + 2 * (size_t)c));
    else return __uint_as_float(ld16(row + 2 * (size_t)c) << 16);
}

// y[b][r] = sum_c W[r][c] x[b][c]; one warp per row, lanes stride over 32-weight
// groups, NB batch columns per pass (the weights are decoded once per pass).
template <int FMT, int NB>
__global__ void __launch_bounds__(256)
gemv_generic_kernel(const uint8_t *__restrict__ data, size_t row_bytes, uint32_t out_dim, uint32_t in_dim, int layout,
                    const float *__restrict__ x, int batch, int ldx, float *__restrict__ y, int ldy)
{
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    uint32_t lane = threadIdx.x & 31;
    if (row >= out_dim) return;
    const uint8_t *rp = data + (size_t)row * row_bytes;
    uint32_t groups = in_dim / 32;
    for (int b0 = 0; b0 < batch; b0 += NB) {
        float acc[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) acc[i] = 0.0f;
        for (uint32_t g = lane; g < groups; g += 32) {
            float w[32];
            decode32<FMT>(rp, g, layout, w);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                if (b0 + i < batch) {
                    const float *xb = x + (size_t)(b0 + i) * ldx + (size_t)g * 32;
                    float a = 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) a = fmaf(w[j], xb[j], a);
                    acc[i] += a;
                }
            }
        }
        if constexpr (FMT == FMT_F32 || FMT == FMT_F16 || FMT == FMT_BF16) {
            for (uint32_t c = groups * 32 + lane; c < in_dim; c += 32) {
                float wv = plain_elem<FMT>(rp, c);
#pragma unroll
                for (int i = 0; i < NB; ++i)
                    if (b0 + i < batch) acc[i] = fmaf(wv, x[(size_t)(b0 + i) * ldx + c], acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            float s = warp_sum(acc[i]);
            if (lane == 0 && b0 + i < batch) y[(size_t)(b0 + i) * ldy + row] = s;
        }
    }
}

// fp32 weights (the MoE router, shaders.metal:1342-1366): one warp per row, lanes take consecutive float4s so every
// load is coalesced; up to 4 input vectors per pass.  Waits for the previous kernel first (it may produce x).
// With W1 set, one more output row (index out_dim) comes from that single-row tensor: the router logits and the
// shared-expert gate logit in one launch, as matvec_f32_pair does (shaders.metal:1368-1392).
__global__ void __launch_bounds__(128)
gemv_f32_kernel(const float *__restrict__ W, uint32_t out_dim, uint32_t in_dim, const float *__restrict__ x, int batch, int ldx,
                float *__restrict__ y, int ldy, const float *__restrict__ W1 = nullptr)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may set itself up; it waits for this one's results itself
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // One CTA of four warps per row: a 2048-wide row is then one round of four 16-byte loads per thread, all in flight
    // together (a warp per row needed four dependent rounds, and a 128-row router matrix kept only 33 CTAs busy).
    const uint32_t row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float4 *w4 = reinterpret_cast<const float4 *>(row < out_dim ? W + (size_t)row * in_dim : W1);
    const uint32_t n4 = in_dim / 4;
    // grid.y cuts the batch into groups of four vectors
    const int b0 = (int)blockIdx.y * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t c0 = tid; c0 < n4; c0 += 512) {
        float4 w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) w[u] = c0 + 128 * u < n4 ? __ldg(w4 + c0 + 128 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (b0 + i < batch) {
                const float4 *x4 = reinterpret_cast<const float4 *>(x + (size_t)(b0 + i) * ldx);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (c0 + 128 * u < n4) {
                        const float4 xv = x4[c0 + 128 * u];
                        acc[i] = fmaf(w[u].x, xv.x, fmaf(w[u].y, xv.y, fmaf(w[u].z, xv.z, fmaf(w[u].w, xv.w, acc[i]))));
                    }
                }
            }
        }
    }
    __shared__ float red[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float s = warp_sum(acc[i]);
        if (lane == 0) red[warp][i] = s;
    }
    __syncthreads();
    if (tid < 4 && b0 + (int)tid < batch) y[(size_t)(b0 + tid) * ldy + row] = (red[0][tid] + red[1][tid]) + (red[2][tid] + red[3][tid]);
}

// out = silu(gate) * up, elementwise (shaders.metal:1018-1030); used after two
// generic matvecs when the fused kernel does not take the shape.
__global__ void swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ out,
                              uint32_t n, int batch, int ldg, int ldo)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n * batch) return;
    uint32_t b = (uint32_t)(i / n), c = (uint32_t)(i % n);
    out[(size_t)b * ldo + c] = silu_mul(gate[(size_t)b * ldg + c], up[(size_t)b * ldg + c]);
}

// Index of the largest element: argmax_kernel (shaders.metal:1249-1305), dispatched after the lm_head at
// engine.m:1036-1046 so that a token costs the host a 4-byte read.  The reference runs one threadgroup of 1024
// threads; one CTA reading 600 KB takes tens of microseconds here, so the vector is cut over up to 148 CTAs.
// Candidates are compared as {value key, ~tie rank} (argmax_rank), a total order in which equal values resolve
// exactly as the reference's strided scan and shuffle-down trees do, so the cut changes nothing; NaN and -inf never
// win, an input without candidates gives index 0.  state[0]: running best (atomicMax), state[1]: CTAs done; the last
// CTA writes the result and clears both for the next call.
__global__ void __launch_bounds__(256)
argmax_kernel(const float *__restrict__ data, uint32_t count, uint32_t *__restrict__ result, unsigned long long *__restrict__ state)
{
    __shared__ unsigned long long s_best[8];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    unsigned long long best = 0ull;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
        const float v = __ldcg(data + i);
        if (v > -INFINITY) {
            const unsigned long long cand = ((unsigned long long)float_key(v) << 32) | (uint32_t)~argmax_rank(i);
            if (cand > best) best = cand;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        if (other > best) best = other;
    }
    if ((threadIdx.x & 31u) == 0) s_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) if (s_best[w] > best) best = s_best[w];
        if (best) atomicMax(state, best);
        __threadfence();
        if (atomicAdd(state + 1, 1ull) == gridDim.x - 1) {
            __threadfence();
            const unsigned long long m = atomicExch(state, 0ull);
            *result = m ? argmax_unrank(~(uint32_t)m) : 0u;
            atomicExch(state + 1, 0ull);
        }
    }
}

}  // namespace orome
