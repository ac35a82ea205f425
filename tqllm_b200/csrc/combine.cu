// Weighted scatter-combine: out[t] = sum_s w[t][s] * y[t*topk + s] (slot order) + shared weight * y[n*topk + t].
// Replaces sum_k / moe_sum_k / fn_moe_combine_k (src/experts/moe.cu:223-234, src/experts/moe_common.cu:186-194,
// src/models/qwen/qwen4exp/qwen4exp.cu:846-851); fp32 accumulation in the order of moe_combine (src/experts/moe.cpp:157-163).
#include "common.cuh"

namespace b2 {
namespace {

// residual (may be null): rows [n][h] of the output's type added to the sum: the layer's skip connection in the same pass
template <int DT>
__global__ void combine_k(const float * __restrict__ y, const int * __restrict__ ids, const float * __restrict__ w,
                          const float * __restrict__ sw, int n, int k, int h, int shared_tokens, const typename Elem<DT>::type * residual,
                          typename Elem<DT>::type * out) {                 // residual may be out: no __restrict__ on the two
    const int t = blockIdx.x;                     // tokens on gridDim.x: any batch size
    const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    grid_release();
    grid_wait();
    if (j >= h) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < k; ++s) {
        if (ids && ids[size_t(t) * k + s] < 0) continue;
        const float ws = w[size_t(t) * k + s];
        const float4 v = *reinterpret_cast<const float4 *>(y + (size_t(t) * k + s) * h + j);
        acc.x += ws * v.x; acc.y += ws * v.y; acc.z += ws * v.z; acc.w += ws * v.w;
    }
    if (shared_tokens) {
        const float ws = sw ? sw[t] : 1.f;
        const float4 v = *reinterpret_cast<const float4 *>(y + (size_t(n) * k + t) * h + j);
        acc.x += ws * v.x; acc.y += ws * v.y; acc.z += ws * v.z; acc.w += ws * v.w;
    }
    if (residual) {
        const typename Elem<DT>::type * r = residual + size_t(t) * h + j;
        acc.x += Elem<DT>::to_f(r[0]); acc.y += Elem<DT>::to_f(r[1]); acc.z += Elem<DT>::to_f(r[2]); acc.w += Elem<DT>::to_f(r[3]);
    }
    typename Elem<DT>::type * o = out + size_t(t) * h + j;
    if (DT == B2MOE_F32) {
        *reinterpret_cast<float4 *>(o) = acc;
    } else {
        store_act(o, DT, 0, acc.x); store_act(o, DT, 1, acc.y); store_act(o, DT, 2, acc.z); store_act(o, DT, 3, acc.w);
    }
}

}  // namespace
}  // namespace b2

using namespace b2;

static int32_t combine_any(const float * y, const int32_t * ids, const float * weights, const float * shared_weights, const void * residual, int32_t n,
                           int32_t topk, int32_t hidden, int32_t shared_tokens, void * out, int32_t out_dtype, b2moe_stream stream) {
    if (n <= 0 || topk <= 0 || hidden <= 0 || hidden % 4 || (shared_tokens != 0 && shared_tokens != n)) return B2MOE_ERR_SHAPE;
    if (!valid_dtype(out_dtype)) return B2MOE_ERR_SHAPE;
    if (!y || !weights || !out) return B2MOE_ERR_NULL;
    if (!aligned16(y) || !aligned16(out)) return B2MOE_ERR_ALIGN;
    const dim3 grid(n, ceil_div(hidden / 4, 128));
    cudaStream_t s = as_stream(stream);
    if (out_dtype == B2MOE_F32)
        launch_overlapped(combine_k<B2MOE_F32>, grid, dim3(128), 0, s, y, ids, weights, shared_weights, n, topk, hidden, shared_tokens,
                          static_cast<const float *>(residual), static_cast<float *>(out));
    else if (out_dtype == B2MOE_BF16)
        launch_overlapped(combine_k<B2MOE_BF16>, grid, dim3(128), 0, s, y, ids, weights, shared_weights, n, topk, hidden, shared_tokens,
                          static_cast<const __nv_bfloat16 *>(residual), static_cast<__nv_bfloat16 *>(out));
    else
        launch_overlapped(combine_k<B2MOE_F16>, grid, dim3(128), 0, s, y, ids, weights, shared_weights, n, topk, hidden, shared_tokens,
                          static_cast<const __half *>(residual), static_cast<__half *>(out));
    return launch_status();
}

extern "C" B2MOE_API int32_t b2moe_combine(const float * y, const int32_t * ids, const float * weights, const float * shared_weights, int32_t n,
                                 int32_t topk, int32_t hidden, int32_t shared_tokens, void * out, int32_t out_dtype,
                                 b2moe_stream stream) {
    return combine_any(y, ids, weights, shared_weights, nullptr, n, topk, hidden, shared_tokens, out, out_dtype, stream);
}

// The same with the layer's skip connection added in the same pass: out[t] = residual[t] + the weighted sum. residual has
// the output's type and may be the output buffer itself (each element is read before it is written, by the same thread).
extern "C" B2MOE_API int32_t b2moe_combine_residual(const float * y, const int32_t * ids, const float * weights, const float * shared_weights,
                                          const void * residual, int32_t n, int32_t topk, int32_t hidden, int32_t shared_tokens, void * out,
                                          int32_t out_dtype, b2moe_stream stream) {
    if (!residual) return B2MOE_ERR_NULL;
    if (!aligned16(residual)) return B2MOE_ERR_ALIGN;
    return combine_any(y, ids, weights, shared_weights, residual, n, topk, hidden, shared_tokens, out, out_dtype, stream);
}
