// Expert-parallel helpers: rank r of G owns the contiguous experts [first, first + count); tokens stay data-parallel.
// A rank sees every rank's tokens and routed ids, computes the assignments of its own experts, and returns per-token
// partial sums to the tokens' home ranks. Replaces the reference's two-rank ownership kernels ep_local_ids / ep_gather /
// ep_scatter (src/experts/moe.cu:496-541) for any number of ranks; the exchange itself is NCCL, driven by the host.
#include "common.cuh"

namespace b2 {
namespace {

// routing histogram, added up over calls (count_k, src/experts/moe.cu:183-186); ids outside [0, experts) are skipped
__global__ void count_ids_k(const int * __restrict__ ids, unsigned long long * __restrict__ counts, int count, int experts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) { const int e = ids[i]; if (e >= 0 && e < experts) atomicAdd(counts + e, 1ull); }
}


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
    const int t = blockIdx.x, j = (blockIdx.y * blockDim.x + threadIdx.x) * 4;      // tokens on gridDim.x: any batch size
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
    if (ranks <= 0 || n <= 0 || hidden <= 0 || hidden % 4 || !valid_dtype(out_dtype)) return B2MOE_ERR_SHAPE;
    if (!parts || !out) return B2MOE_ERR_NULL;
    if (!aligned16(parts) || !aligned16(out) || (shared_y && !aligned16(shared_y))) return B2MOE_ERR_ALIGN;
    const dim3 grid(n, ceil_div(hidden / 4, 128));
    cudaStream_t s = as_stream(stream);
    if (out_dtype == B2MOE_F32) ep_reduce_k<B2MOE_F32><<<grid, 128, 0, s>>>(parts, ranks, shared_y, shared_weights, n, hidden, static_cast<float *>(out));
    else if (out_dtype == B2MOE_BF16) ep_reduce_k<B2MOE_BF16><<<grid, 128, 0, s>>>(parts, ranks, shared_y, shared_weights, n, hidden, static_cast<__nv_bfloat16 *>(out));
    else ep_reduce_k<B2MOE_F16><<<grid, 128, 0, s>>>(parts, ranks, shared_y, shared_weights, n, hidden, static_cast<__half *>(out));
    return launch_status();
}

// ---- all-to-all dispatch (batches where gathering every token on every rank is too much) ------------------------
// A rank sends a token only to the ranks that own one of its routed experts (src/models/qwen/qwen4exp/fn_layer_forward.cpp:475-503
// exchanges result rows the same way between two ranks), and always to itself, so that the shared expert finds every own
// token in the local batch. Records travel as bytes: the activation row, the k routed ids, the k routing weights.
namespace b2 {
namespace {

// One block per peer p: tokens with an expert in [bounds[p], bounds[p + 1]) (every token for p = self), in ascending
// order: pos[p][t] = its position in p's list or -1, list[p][pos] = t, counts[p] = list length.
__global__ void ep_peer_lists_k(const int * __restrict__ ids, int n, int topk, const int * __restrict__ bounds, int self,
                                int * __restrict__ counts, int * __restrict__ pos, int * __restrict__ list) {
    __shared__ int warp_sum[32];
    __shared__ int base;
    const int p = blockIdx.x, lo = bounds[p], hi = bounds[p + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int t0 = 0; t0 < n; t0 += blockDim.x) {
        const int t = t0 + threadIdx.x;
        bool f = false;
        if (t < n) {
            f = p == self;
            for (int s = 0; s < topk && !f; ++s) { const int e = ids[size_t(t) * topk + s]; f = e >= lo && e < hi; }
        }
        const unsigned m = __ballot_sync(0xffffffffu, f);
        if (lane == 0) warp_sum[warp] = __popc(m);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += warp_sum[w];
        const int my = before + __popc(m & ((1u << lane) - 1u));
        if (t < n) {
            pos[size_t(p) * n + t] = f ? my : -1;
            if (f) list[size_t(p) * n + my] = t;
        }
        __syncthreads();
        if (threadIdx.x == 0) { int tot = 0; for (int w = 0; w < warps; ++w) tot += warp_sum[w]; base += tot; }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[p] = base;
}
// record j of the send buffer (peer segments back to back, segment p at offsets[p]): token list[p][j - offsets[p]]
__global__ void ep_pack_k(const uint8_t * __restrict__ x, int xbytes, const int * __restrict__ ids, const float * __restrict__ w, int topk, int n,
                          const int * __restrict__ list, const int * __restrict__ offsets, int peers, uint8_t * __restrict__ out) {
    const int j = blockIdx.x;
    int p = 0;
    while (p + 1 < peers && j >= offsets[p + 1]) ++p;
    const int t = list[size_t(p) * n + (j - offsets[p])];
    const int rec = xbytes + 8 * topk;
    uint8_t * o = out + size_t(j) * rec;
    for (int b = threadIdx.x * 16; b < xbytes; b += blockDim.x * 16)
        *reinterpret_cast<uint4 *>(o + b) = *reinterpret_cast<const uint4 *>(x + size_t(t) * xbytes + b);
    for (int s = threadIdx.x; s < topk; s += blockDim.x) {
        reinterpret_cast<int *>(o + xbytes)[s] = ids[size_t(t) * topk + s];
        reinterpret_cast<float *>(o + xbytes + 4 * topk)[s] = w[size_t(t) * topk + s];
    }
}
// received records -> x [m][xbytes], ids [m][topk] (only this rank's experts kept, as local ids; others -1), w [m][topk]
__global__ void ep_unpack_k(const uint8_t * __restrict__ rec_in, int xbytes, int topk, int first, int local, uint8_t * __restrict__ x,
                            int * __restrict__ ids, float * __restrict__ w) {
    const int j = blockIdx.x, rec = xbytes + 8 * topk;
    const uint8_t * r = rec_in + size_t(j) * rec;
    for (int b = threadIdx.x * 16; b < xbytes; b += blockDim.x * 16)
        *reinterpret_cast<uint4 *>(x + size_t(j) * xbytes + b) = *reinterpret_cast<const uint4 *>(r + b);
    for (int s = threadIdx.x; s < topk; s += blockDim.x) {
        const int v = reinterpret_cast<const int *>(r + xbytes)[s] - first;
        ids[size_t(j) * topk + s] = (v >= 0 && v < local) ? v : -1;
        w[size_t(j) * topk + s] = reinterpret_cast<const float *>(r + xbytes + 4 * topk)[s];
    }
}
// out[t] = sum over peers p (ascending: the same bits on every run) of back[offsets[p] + pos[p][t]] where pos >= 0,
//          + shared weight * shared_y[t]
template <int DT>
__global__ void ep_return_reduce_k(const float * __restrict__ back, const int * __restrict__ pos, const int * __restrict__ offsets, int peers,
                                   const float * __restrict__ shared_y, const float * __restrict__ shared_w, int n, int h,
                                   typename Elem<DT>::type * __restrict__ out) {
    const int t = blockIdx.x;
    for (int j = threadIdx.x * 4; j < h; j += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < peers; ++p) {
            const int q = pos[size_t(p) * n + t];
            if (q < 0) continue;
            const float4 v = *reinterpret_cast<const float4 *>(back + (size_t(offsets[p]) + q) * h + j);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (shared_y) {
            const float sw = shared_w ? shared_w[t] : 1.f;
            const float4 v = *reinterpret_cast<const float4 *>(shared_y + size_t(t) * h + j);
            acc.x += sw * v.x; acc.y += sw * v.y; acc.z += sw * v.z; acc.w += sw * v.w;
        }
        typename Elem<DT>::type * o = out + size_t(t) * h + j;
        if (DT == B2MOE_F32) *reinterpret_cast<float4 *>(o) = acc;
        else { store_act(o, DT, 0, acc.x); store_act(o, DT, 1, acc.y); store_act(o, DT, 2, acc.z); store_act(o, DT, 3, acc.w); }
    }
}

}  // namespace
}  // namespace b2

extern "C" B2MOE_API int32_t b2moe_ep_peer_lists(const int32_t * ids, int32_t n, int32_t topk, const int32_t * bounds, int32_t peers, int32_t self,
                                                 int32_t * counts, int32_t * pos, int32_t * list, b2moe_stream stream) {
    if (n <= 0 || topk <= 0 || peers <= 0 || self < 0 || self >= peers) return B2MOE_ERR_SHAPE;
    if (!ids || !bounds || !counts || !pos || !list) return B2MOE_ERR_NULL;
    ep_peer_lists_k<<<peers, 1024, 0, as_stream(stream)>>>(ids, n, topk, bounds, self, counts, pos, list);
    return launch_status();
}
extern "C" B2MOE_API int32_t b2moe_ep_pack(const void * x, int32_t x_row_bytes, const int32_t * ids, const float * weights, int32_t topk, int32_t n,
                                           const int32_t * list, const int32_t * offsets, int32_t peers, int32_t records, void * out,
                                           b2moe_stream stream) {
    if (x_row_bytes <= 0 || x_row_bytes % 16 || topk <= 0 || n <= 0 || peers <= 0 || records < 0) return B2MOE_ERR_SHAPE;
    if (!x || !ids || !weights || !list || !offsets || !out) return B2MOE_ERR_NULL;
    if (!aligned16(x) || !aligned16(out) || (8 * topk) % 16) return B2MOE_ERR_ALIGN;
    if (records == 0) return B2MOE_OK;
    ep_pack_k<<<records, 128, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(x), x_row_bytes, ids, weights, topk, n, list, offsets, peers,
                                                      static_cast<uint8_t *>(out));
    return launch_status();
}
extern "C" B2MOE_API int32_t b2moe_ep_unpack(const void * records_in, int32_t records, int32_t x_row_bytes, int32_t topk, int32_t first_expert,
                                             int32_t local_experts, void * x, int32_t * local_ids, float * weights, b2moe_stream stream) {
    if (x_row_bytes <= 0 || x_row_bytes % 16 || topk <= 0 || records < 0 || first_expert < 0 || local_experts <= 0) return B2MOE_ERR_SHAPE;
    if (!records_in || !x || !local_ids || !weights) return B2MOE_ERR_NULL;
    if (!aligned16(records_in) || !aligned16(x) || (8 * topk) % 16) return B2MOE_ERR_ALIGN;
    if (records == 0) return B2MOE_OK;
    ep_unpack_k<<<records, 128, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(records_in), x_row_bytes, topk, first_expert, local_experts,
                                                        static_cast<uint8_t *>(x), local_ids, weights);
    return launch_status();
}
extern "C" B2MOE_API int32_t b2moe_ep_return_reduce(const float * back, const int32_t * pos, const int32_t * offsets, int32_t peers,
                                                    const float * shared_y, const float * shared_weights, int32_t n, int32_t hidden, void * out,
                                                    int32_t out_dtype, b2moe_stream stream) {
    if (peers <= 0 || n <= 0 || hidden <= 0 || hidden % 4 || !valid_dtype(out_dtype)) return B2MOE_ERR_SHAPE;
    if (!back || !pos || !offsets || !out) return B2MOE_ERR_NULL;
    if (!aligned16(back) || !aligned16(out) || (shared_y && !aligned16(shared_y))) return B2MOE_ERR_ALIGN;
    cudaStream_t s = as_stream(stream);
    if (out_dtype == B2MOE_F32) ep_return_reduce_k<B2MOE_F32><<<n, 256, 0, s>>>(back, pos, offsets, peers, shared_y, shared_weights, n, hidden, static_cast<float *>(out));
    else if (out_dtype == B2MOE_BF16) ep_return_reduce_k<B2MOE_BF16><<<n, 256, 0, s>>>(back, pos, offsets, peers, shared_y, shared_weights, n, hidden, static_cast<__nv_bfloat16 *>(out));
    else ep_return_reduce_k<B2MOE_F16><<<n, 256, 0, s>>>(back, pos, offsets, peers, shared_y, shared_weights, n, hidden, static_cast<__half *>(out));
    return launch_status();
}

extern "C" B2MOE_API int32_t b2moe_count(const int32_t * ids, uint64_t * counts, int32_t count, int32_t experts, b2moe_stream stream) {
    if (count <= 0 || experts <= 0) return B2MOE_ERR_SHAPE;
    if (!ids || !counts) return B2MOE_ERR_NULL;
    count_ids_k<<<ceil_div(count, 256), 256, 0, as_stream(stream)>>>(ids, reinterpret_cast<unsigned long long *>(counts), count, experts);
    return launch_status();
}

// Load-aware placement (host): experts in descending order of their counts, each to the rank with the smallest load so far
// that still has a free slot (every rank holds exactly experts / ranks: the banks stay equal in size). order[] lists the
// experts rank by rank: rank r owns order[r * per .. (r + 1) * per), so a loader that stacks router rows, selection bias
// and banks in this order keeps the library's contiguous-block ownership. Ties: lower expert id first, lower rank first.
extern "C" B2MOE_API int32_t b2moe_place_experts(const uint64_t * counts, int32_t experts, int32_t ranks, int32_t * order, uint64_t * rank_load) {
    if (experts <= 0 || ranks <= 0 || experts % ranks) return B2MOE_ERR_SHAPE;
    if (!counts || !order) return B2MOE_ERR_NULL;
    const int per = experts / ranks;
    int * by_count = new int[experts];
    for (int e = 0; e < experts; ++e) by_count[e] = e;
    // insertion sort by (count descending, id ascending): a few thousand experts at most, run once per placement
    for (int i = 1; i < experts; ++i) {
        const int e = by_count[i];
        int j = i - 1;
        while (j >= 0 && (counts[by_count[j]] < counts[e])) { by_count[j + 1] = by_count[j]; --j; }
        by_count[j + 1] = e;
    }
    uint64_t * load = new uint64_t[ranks]();
    int * filled = new int[ranks]();
    for (int i = 0; i < experts; ++i) {
        const int e = by_count[i];
        int best = -1;
        for (int r = 0; r < ranks; ++r)
            if (filled[r] < per && (best < 0 || load[r] < load[best])) best = r;
        order[best * per + filled[best]++] = e;
        load[best] += counts[e];
    }
    if (rank_load) for (int r = 0; r < ranks; ++r) rank_load[r] = load[r];
    delete[] by_count; delete[] load; delete[] filled;
    return B2MOE_OK;
}
