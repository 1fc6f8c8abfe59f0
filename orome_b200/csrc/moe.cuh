// moe.cuh -- MoE routing and routed-expert kernels.
#pragma once
#include "decode.cuh"

namespace orome {

// softmax_topk_route (shaders.metal:1141-1234), one CTA of 256 threads per token.
// K rounds of arg-max over <= 256 logits; a candidate replaces the current best
// only when strictly greater, and candidates are visited in index order, so the
// lowest index wins ties.  Softmax over the selected logits only.
__global__ void __launch_bounds__(256)
route_topk_kernel(const float *__restrict__ logits, int ld_logits, uint32_t n_experts, uint32_t K,
                  uint32_t *__restrict__ idx_out, float *__restrict__ w_out, float *__restrict__ shared_logit_out = nullptr)
{
    // Per round one barrier: the warps' candidates go to one of two buffers in turn, and EVERY warp then reduces the eight
    // candidates for itself (same operations in the same order, so the same winner), which saves the second barrier
    // and the trip of the winner through shared memory.  Lanes 8..31 of that second reduction hold -inf, so its
    // steps 16 and 8 can never change lanes 0..7 and are left out.
    __shared__ float s_val[2][8];
    __shared__ uint32_t s_idx[2][8];
    __shared__ float f_val[8];
    __shared__ uint32_t f_idx[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may set itself up; it waits for this one's results itself
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the logits are the previous kernel's output
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float *lg = logits + (size_t)blockIdx.x * ld_logits;
    float my = tid < n_experts ? lg[tid] : -INFINITY;
    const uint32_t limit = K < 8 ? K : 8;
    for (uint32_t round = 0; round < limit; ++round) {
        const uint32_t buf = round & 1u;
        float v = my;
        uint32_t id = tid;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_down_sync(0xffffffffu, v, o);
            uint32_t oi = __shfl_down_sync(0xffffffffu, id, o);
            if (ov > v) { v = ov; id = oi; }
        }
        if (lane == 0) { s_val[buf][warp] = v; s_idx[buf][warp] = id; }
        __syncthreads();
        float v2 = lane < 8 ? s_val[buf][lane] : -INFINITY;
        uint32_t i2 = lane < 8 ? s_idx[buf][lane] : 0u;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            float ov = __shfl_down_sync(0xffffffffu, v2, o);
            uint32_t oi = __shfl_down_sync(0xffffffffu, i2, o);
            if (ov > v2) { v2 = ov; i2 = oi; }
        }
        v2 = __shfl_sync(0xffffffffu, v2, 0);
        i2 = __shfl_sync(0xffffffffu, i2, 0);
        if (tid == 0) { f_val[round] = v2; f_idx[round] = i2; }
        if (tid == i2) my = -INFINITY;
    }
    if (tid == 0) {
        float w[8], sum = 0.0f, mx = limit ? f_val[0] : 0.0f;
        for (uint32_t k = 0; k < limit; ++k) { w[k] = expf(f_val[k] - mx); sum += w[k]; }
        float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        uint32_t *io = idx_out + (size_t)blockIdx.x * 8;
        float *wo = w_out + (size_t)blockIdx.x * 8;
        for (uint32_t k = 0; k < 8; ++k) {
            io[k] = k < limit ? f_idx[k] : 0u;
            wo[k] = k < limit ? w[k] * inv : 0.0f;
        }
        // the raw logit of the shared-expert gate, which sits after the router logits (out_params[8], shaders.metal:1232)
        if (shared_logit_out) shared_logit_out[blockIdx.x] = lg[n_experts];
    }
}

// hidden = h_mid + moe + sigmoid(shared gate logit) * shared_out: the value the reference's combine kernels compute
// (moe_combine_copy_sq / _k8, shaders.metal:1049-1059, 1100-1120) with the weighted expert sum already formed by the
// down-projection launch.  sigmoid as the reference writes it, 1 / (1 + exp(-p)).  h_mid and shared_out may be NULL.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float *__restrict__ h_mid, int ld_mid, const float *__restrict__ moe, int ld_moe, const float *__restrict__ shared_out,
                   int ld_shared, const float *__restrict__ shared_logit, uint32_t hidden, float *__restrict__ out, int ldo)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t t = blockIdx.y, h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= hidden) return;
    float v = moe[(size_t)t * ld_moe + h];
    if (h_mid) v = h_mid[(size_t)t * ld_mid + h] + v;
    if (shared_out) {
        const float gate = 1.0f / (1.0f + expf(-shared_logit[t]));
        v += gate * shared_out[(size_t)t * ld_shared + h];
    }
    out[(size_t)t * ldo + h] = v;
}

// Expert-parallel form: indices of the experts [first, first + count) become local (0..count-1), all others the
// "not here" mark that the expert kernels step over.
__global__ void moe_localize_kernel(const uint32_t *__restrict__ idx, uint32_t n, uint32_t first, uint32_t count, uint32_t *__restrict__ out)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the indices are the routing kernel's output
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const uint32_t e = idx[i] - first;
        out[i] = e < count ? e : 0xFFFFFFFFu;
    }
}

// act[t][k][m] = silu(Wg[e] x_t)[m] * (Wu[e] x_t)[m], e = idx[t][k]; one warp per (t, k, m).
template <int FMT>
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(const uint8_t *__restrict__ gate, size_t gate_stride, const uint8_t *__restrict__ up, size_t up_stride,
                   size_t row_bytes, uint32_t inter, uint32_t hidden, int layout, const float *__restrict__ x, int ldx,
                   const uint32_t *__restrict__ idx, uint32_t K, float *__restrict__ act)
{
    const uint32_t tk = blockIdx.y, t = tk / K, k = tk % K;
    const uint32_t m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (m >= inter) return;
    const size_t e = idx[(size_t)t * 8 + k];
    if (e == 0xFFFFFFFFu) return;                 // expert of another GPU (expert-parallel form)
    const uint8_t *gr = gate + e * gate_stride + (size_t)m * row_bytes;
    const uint8_t *ur = up + e * up_stride + (size_t)m * row_bytes;
    const float *xt = x + (size_t)t * ldx;
    float ag = 0.0f, au = 0.0f;
    for (uint32_t g = lane; g < hidden / 32; g += 32) {
        float w[32];
        const float *xb = xt + (size_t)g * 32;
        decode32<FMT>(gr, g, layout, w);
#pragma unroll
        for (int j = 0; j < 32; ++j) ag = fmaf(w[j], xb[j], ag);
        decode32<FMT>(ur, g, layout, w);
#pragma unroll
        for (int j = 0; j < 32; ++j) au = fmaf(w[j], xb[j], au);
    }
    ag = warp_sum(ag);
    au = warp_sum(au);
    if (lane == 0) act[((size_t)t * K + k) * inter + m] = silu_mul(ag, au);
}

// out[t][h] = sum_k w[t][k] * (Wd[e_k] act[t][k])[h]; one warp per (t, h), experts added in slot order.
template <int FMT>
__global__ void __launch_bounds__(256)
moe_down_kernel(const uint8_t *__restrict__ down, size_t down_stride, size_t row_bytes, uint32_t hidden, uint32_t inter,
                int layout, const float *__restrict__ act, const uint32_t *__restrict__ idx, const float *__restrict__ wts,
                uint32_t K, float *__restrict__ out, int ldo)
{
    const uint32_t t = blockIdx.y;
    const uint32_t h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (h >= hidden) return;
    float total = 0.0f;
    for (uint32_t k = 0; k < K; ++k) {
        const size_t e = idx[(size_t)t * 8 + k];
        if (e == 0xFFFFFFFFu) continue;           // expert of another GPU
        const uint8_t *row = down + e * down_stride + (size_t)h * row_bytes;
        const float *a = act + ((size_t)t * K + k) * inter;
        float acc = 0.0f;
        for (uint32_t g = lane; g < inter / 32; g += 32) {
            float w[32];
            decode32<FMT>(row, g, layout, w);
            const float *ab = a + (size_t)g * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) acc = fmaf(w[j], ab[j], acc);
        }
        acc = warp_sum(acc);
        total = fmaf(wts[(size_t)t * 8 + k], acc, total);
    }
    if (lane == 0) out[(size_t)t * ldo + h] = total;
}

}  // namespace orome
