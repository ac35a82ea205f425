// Router logits and top-k routing (softmax and sigmoid + selection bias families).
// Replaces router_k / topk_k / topk_warp_k (src/experts/moe.cu:17-166,237-267) and route_k (src/experts/moe_common.cu:18-70).
// Selection rule everywhere: larger key first, lower index on ties (src/experts/moe.cpp:75-78); weights come from
// the unbiased probabilities (src/experts/moe.cpp:85-86); the renormalising sum is clamped at 6.103515625e-5
// (src/experts/moe.hpp:38) and accumulated in selection order like the host reference (src/experts/moe.cpp:103-108).
#include <math_constants.h>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int ROUTER_TOK = 8;   // tokens one warp carries per pass over a weight row

// One warp per router row (row `experts` = the shared-gate vector), ROUTER_TOK tokens at a time, fp32 accumulation.
template <int DT>
__global__ void router_k(const float * __restrict__ w, const float * __restrict__ shared, const typename Elem<DT>::type * __restrict__ x,
                         float * __restrict__ logits, int ld, int h, int e, int rows, int n) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float * wr = row == e ? shared : w + size_t(row) * h;
    for (int t0 = blockIdx.y * ROUTER_TOK; t0 < n; t0 += gridDim.y * ROUTER_TOK) {
        float acc[ROUTER_TOK];
#pragma unroll
        for (int c = 0; c < ROUTER_TOK; ++c) acc[c] = 0.f;
        for (int j = lane * 4; j < h; j += 128) {
            const float4 wv = *reinterpret_cast<const float4 *>(wr + j);
#pragma unroll
            for (int c = 0; c < ROUTER_TOK; ++c) {
                if (t0 + c < n) {
                    const typename Elem<DT>::type * xr = x + size_t(t0 + c) * h + j;
                    acc[c] += wv.x * Elem<DT>::to_f(xr[0]) + wv.y * Elem<DT>::to_f(xr[1]) + wv.z * Elem<DT>::to_f(xr[2]) +
                              wv.w * Elem<DT>::to_f(xr[3]);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < ROUTER_TOK; ++c) {
            float s = acc[c];
            for (int d = 16; d; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
            if (lane == 0 && t0 + c < n) logits[size_t(t0 + c) * ld + row] = s;
        }
    }
}

__device__ __forceinline__ void argmax_merge(float & v, int & i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// One warp per token. p[] = unbiased probabilities, key[] = selection keys (p, or p + bias), both in shared memory.
template <int GATING>
__global__ void route_k(const float * __restrict__ logits, int ld, const float * __restrict__ bias, int * __restrict__ ids,
                        float * __restrict__ weights, float * __restrict__ shared_weights, int e, int k, int norm, float scale, int n) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int token = blockIdx.x * warps + warp;
    if (token >= n) return;
    float * p = smem + size_t(warp) * 2 * e;
    float * key = p + e;
    const float * x = logits + size_t(token) * ld;
    if (GATING == B2MOE_SOFTMAX) {
        float m = -CUDART_INF_F;
        for (int j = lane; j < e; j += 32) m = fmaxf(m, x[j]);
        for (int d = 16; d; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        float sum = 0.f;
        for (int j = lane; j < e; j += 32) { const float v = expf(x[j] - m); p[j] = v; sum += v; }
        for (int d = 16; d; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        for (int j = lane; j < e; j += 32) { const float v = p[j] / sum; p[j] = v; key[j] = v; }
    } else {
        for (int j = lane; j < e; j += 32) {
            const float v = 1.f / (1.f + expf(-x[j]));
            p[j] = v;
            key[j] = bias ? v + bias[j] : v;
        }
    }
    __syncwarp();
    float sel_sum = 0.f;
    for (int r = 0; r < k; ++r) {
        float bv = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int j = lane; j < e; j += 32) {
            const float v = key[j];                  // taken entries hold NaN and never compare true
            if (v > bv || (bi == 0x7fffffff && v == v)) { bv = v; bi = j; }   // ascending j: the lowest index keeps a tie
        }
        for (int d = 16; d; d >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, d), __shfl_xor_sync(0xffffffffu, bi, d));
        if (bi == 0x7fffffff) bi = 0;              // only when the logits themselves hold NaN
        if (lane == 0) {
            const float pv = p[bi];
            ids[size_t(token) * k + r] = bi;
            weights[size_t(token) * k + r] = pv;
            sel_sum += pv;
            key[bi] = CUDART_NAN_F;
        }
        __syncwarp();
    }
    if (lane == 0) {
        float * w = weights + size_t(token) * k;
        if (norm) {
            const float total = fmaxf(sel_sum, 6.103515625e-5f);
            for (int r = 0; r < k; ++r) w[r] = w[r] / total;
        }
        if (scale != 0.f && scale != 1.f) for (int r = 0; r < k; ++r) w[r] *= scale;
        if (shared_weights) shared_weights[token] = 1.f / (1.f + expf(-x[e]));
    }
}

template <int GATING>
int32_t route_launch(const float * logits, int ld, const float * bias, int * ids, float * weights, float * shared_weights, int e,
                     int k, int norm, float scale, int n, cudaStream_t s) {
    const int warps = e <= 1024 ? 4 : 1;
    const size_t smem = size_t(warps) * 2 * e * sizeof(float);
    route_k<GATING><<<ceil_div(n, warps), warps * 32, smem, s>>>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, n);
    return launch_status();
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API int32_t b2moe_router(const float * router_w, const float * shared_gate, const void * x, int32_t x_dtype, float * logits,
                                int32_t ld, int32_t hidden, int32_t experts, int32_t n, b2moe_stream stream) {
    if (hidden <= 0 || experts <= 0 || n <= 0 || hidden % 8 || ld < experts + (shared_gate ? 1 : 0)) return B2MOE_ERR_SHAPE;
    if (!router_w || !x || !logits) return B2MOE_ERR_NULL;
    if (!valid_dtype(x_dtype)) return B2MOE_ERR_SHAPE;
    if (!aligned16(router_w) || !aligned16(x) || (shared_gate && !aligned16(shared_gate))) return B2MOE_ERR_ALIGN;
    const int rows = experts + (shared_gate ? 1 : 0);
    const dim3 grid(ceil_div(rows, 8), std::min(ceil_div(n, ROUTER_TOK), 64));
    cudaStream_t s = as_stream(stream);
    if (x_dtype == B2MOE_F32)
        router_k<B2MOE_F32><<<grid, 256, 0, s>>>(router_w, shared_gate, static_cast<const float *>(x), logits, ld, hidden, experts, rows, n);
    else if (x_dtype == B2MOE_BF16)
        router_k<B2MOE_BF16><<<grid, 256, 0, s>>>(router_w, shared_gate, static_cast<const __nv_bfloat16 *>(x), logits, ld, hidden, experts, rows, n);
    else
        router_k<B2MOE_F16><<<grid, 256, 0, s>>>(router_w, shared_gate, static_cast<const __half *>(x), logits, ld, hidden, experts, rows, n);
    return launch_status();
}

extern "C" B2MOE_API int32_t b2moe_topk_softmax(const float * logits, int32_t ld, int32_t * ids, float * weights, float * shared_weights,
                                      int32_t experts, int32_t topk, int32_t n, float scale, b2moe_stream stream) {
    if (experts <= 0 || experts > 4096 || topk <= 0 || topk > experts || n <= 0 || ld < experts + (shared_weights ? 1 : 0))
        return B2MOE_ERR_SHAPE;
    if (!logits || !ids || !weights) return B2MOE_ERR_NULL;
    return route_launch<B2MOE_SOFTMAX>(logits, ld, nullptr, ids, weights, shared_weights, experts, topk, 1, scale, n, as_stream(stream));
}

extern "C" B2MOE_API int32_t b2moe_route_sigmoid(const float * logits, int32_t ld, const float * bias, int32_t * ids, float * weights,
                                       int32_t experts, int32_t topk, int32_t norm, float scale, int32_t n, b2moe_stream stream) {
    if (experts <= 0 || experts > 4096 || topk <= 0 || topk > experts || n <= 0 || ld < experts) return B2MOE_ERR_SHAPE;
    if (!logits || !ids || !weights) return B2MOE_ERR_NULL;
    return route_launch<B2MOE_SIGMOID>(logits, ld, bias, ids, weights, nullptr, experts, topk, norm, scale, n, as_stream(stream));
}
