// Expert-parallel helpers: rank r of G owns the contiguous experts [first, first + count); tokens stay data-parallel.
// A rank sees every rank's tokens and routed ids, computes the assignments of its own experts, and returns per-token
// partial sums to the tokens' home ranks. Replaces the reference's two-rank ownership kernels ep_local_ids / ep_gather /
// ep_scatter (src/experts/moe.cu:496-541) for any number of ranks; the exchange itself is NCCL, driven by the host.
#include "common.cuh"

namespace b2 {
namespace {

// local[i] = ids[i] - first when the expert is this rank's, else -1 (every grouped kernel skips -1)
__global__ void ep_local_ids_k(const int * __restrict__ ids, int * __restrict__ local, int count, int first, int experts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        const int v = ids[i] - first;
        local[i] = (v >= 0 && v < experts) ? v : -1;
    }
}

// out[t] = sum over source ranks r (ascending: the same bits on every run) of parts[r][t] + shared weight * shared_y[t]
template <int DT>
__global__ void ep_reduce_k(const float * __restrict__ parts, int ranks, const float * __restrict__ shared_y,
                            const float * __restrict__ shared_w, int n, int h, typename Elem<DT>::type * __restrict__ out) {
    const int t = blockIdx.y, j = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (j >= h) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < ranks; ++r) {
        const float4 v = *reinterpret_cast<const float4 *>(parts + (size_t(r) * n + t) * h + j);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (shared_y) {
        const float w = shared_w ? shared_w[t] : 1.f;
        const float4 v = *reinterpret_cast<const float4 *>(shared_y + size_t(t) * h + j);
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    typename Elem<DT>::type * o = out + size_t(t) * h + j;
    if (DT == B2MOE_F32) *reinterpret_cast<float4 *>(o) = acc;
    else { store_act(o, DT, 0, acc.x); store_act(o, DT, 1, acc.y); store_act(o, DT, 2, acc.z); store_act(o, DT, 3, acc.w); }
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API int32_t b2moe_ep_local_ids(const int32_t * ids, int32_t * local_ids, int32_t count, int32_t first_expert,
                                                int32_t local_experts, b2moe_stream stream) {
    if (count <= 0 || first_expert < 0 || local_experts <= 0) return B2MOE_ERR_SHAPE;
    if (!ids || !local_ids) return B2MOE_ERR_NULL;
    ep_local_ids_k<<<ceil_div(count, 256), 256, 0, as_stream(stream)>>>(ids, local_ids, count, first_expert, local_experts);
    return launch_status();
}

extern "C" B2MOE_API int32_t b2moe_ep_reduce(const float * parts, int32_t ranks, const float * shared_y, const float * shared_weights,
                                             int32_t n, int32_t hidden, void * out, int32_t out_dtype, b2moe_stream stream) {
    if (ranks <= 0 || n <= 0 || n > 65535 || hidden <= 0 || hidden % 4 || !valid_dtype(out_dtype)) return B2MOE_ERR_SHAPE;
    if (!parts || !out) return B2MOE_ERR_NULL;
    if (!aligned16(parts) || !aligned16(out) || (shared_y && !aligned16(shared_y))) return B2MOE_ERR_ALIGN;
    const dim3 grid(ceil_div(hidden / 4, 128), n);
    cudaStream_t s = as_stream(stream);
    if (out_dtype == B2MOE_F32) ep_reduce_k<B2MOE_F32><<<grid, 128, 0, s>>>(parts, ranks, shared_y, shared_weights, n, hidden, static_cast<float *>(out));
    else if (out_dtype == B2MOE_BF16) ep_reduce_k<B2MOE_BF16><<<grid, 128, 0, s>>>(parts, ranks, shared_y, shared_weights, n, hidden, static_cast<__nv_bfloat16 *>(out));
    else ep_reduce_k<B2MOE_F16><<<grid, 128, 0, s>>>(parts, ranks, shared_y, shared_weights, n, hidden, static_cast<__half *>(out));
    return launch_status();
}
