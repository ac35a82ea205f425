// Token -> expert dispatch on the device: per-expert histogram, exclusive prefix sum, stable permutation.
// The permutation lists, expert by expert, the assignment indices in ascending order: the order the reference's
// host builder fill_pass_lists (src/models/qwen/qwen4exp/prefill_plan.hpp:62-76) and its single-block
// dedup_maps_k (src/experts/moe.cu:453-483) produce, without the O(A^2) walk of the latter or the atomics of group_k
// (src/experts/moe.cu:168-176), whose list order is not deterministic.
//
// Method: the assignments are cut into chunks that one warp walks 32 at a time. __match_any_sync groups the lanes
// holding the same expert, so each distinct expert of a step has one leader lane that bumps the chunk's private
// counter by the group size (no atomics); an exclusive scan over (expert, chunk) turns the counters into each
// chunk's first output slot per expert; a second walk in the same order hands every assignment
// base + (number of lower lanes with the same expert), which keeps ascending order inside an expert.
#include "common.cuh"
#include "dispatch.cuh"

namespace b2 {
namespace {

constexpr int CHUNK = 256;   // assignments per warp-chunk on the multi-block path

__global__ void dispatch_small_k(const int * __restrict__ ids, int A, int e, int shared_first, int shared_tokens, int * __restrict__ plan) {
    extern __shared__ unsigned short hist[];       // [32 warps][e]
    grid_release();
    grid_wait();
    dispatch_small_body(ids, A, e, shared_first, shared_tokens, plan, hist);
}

// ---- multi-block path: chunk counters in global scratch [chunks][e] ----
__global__ void dispatch_hist_k(const int * __restrict__ ids, int A, int e, int * __restrict__ hist) {
    const int lane = threadIdx.x & 31, chunk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int a0 = chunk * CHUNK;
    if (a0 >= A) return;
    int * h = hist + size_t(chunk) * e;
    for (int a = a0 + lane; a - lane < min(A, a0 + CHUNK); a += 32) {
        const int id = valid_id(ids, a, A, e);
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        if (id >= 0 && lane == __ffs(peers) - 1) h[id] += __popc(peers);
        __syncwarp();
    }
}
__global__ void dispatch_scan_k(int * __restrict__ hist, int chunks, int e, int A, int shared_tokens, int * __restrict__ plan) {
    const int e1 = e + 1;
    int * counts = plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1;
    for (int x = threadIdx.x; x < e; x += blockDim.x) {
        int run = 0;
        // eight chunk counters at a time: the loads of a batch are independent of its stores (one load per store would wait
        // for the store before it, since both go to the same array)
        for (int c0 = 0; c0 < chunks; c0 += 8) {
            int v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = c0 + i < chunks ? hist[size_t(c0 + i) * e + x] : 0;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c0 + i < chunks) { hist[size_t(c0 + i) * e + x] = run; run += v[i]; }
        }
        counts[x] = run;
    }
    if (threadIdx.x == 0) counts[e] = shared_tokens;
    __syncthreads();
    if (threadIdx.x < 32) finish_plan(plan, counts, offsets, active, offsets, active, active + e1 + A + shared_tokens, e1, threadIdx.x);
}
__global__ void dispatch_scatter_k(const int * __restrict__ ids, int A, int e, int shared_first, int shared_tokens, int * __restrict__ hist,
                                   int * __restrict__ plan) {
    const int e1 = e + 1;
    const int * offsets = plan + PLAN_HDR + e1;
    int * perm = plan + PLAN_HDR + e1 + e1 + 1 + e1;
    const int lane = threadIdx.x & 31, chunk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int a0 = chunk * CHUNK;
    if (blockIdx.x == 0)
        for (int t = threadIdx.x; t < shared_tokens; t += blockDim.x) perm[offsets[e] + t] = A + shared_first + t;
    if (a0 >= A) return;
    int * h = hist + size_t(chunk) * e;
    for (int a = a0 + lane; a - lane < min(A, a0 + CHUNK); a += 32) {
        const int id = valid_id(ids, a, A, e);
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        if (id >= 0) perm[offsets[id] + h[id] + __popc(peers & ((1u << lane) - 1u))] = a;
        __syncwarp();
        if (id >= 0 && lane == __ffs(peers) - 1) h[id] += __popc(peers);
        __syncwarp();
    }
}

__global__ void plan_to_groups_k(const int * __restrict__ plan, int n, int e, int * __restrict__ counts, int * __restrict__ groups) {
    const int e1 = e + 1;
    const int * pc = plan + PLAN_HDR, * offsets = pc + e1, * perm = offsets + e1 + 1 + e1;
    const int x = blockIdx.x;
    if (threadIdx.x == 0) counts[x] = pc[x];
    for (int j = threadIdx.x; j < pc[x]; j += blockDim.x) groups[size_t(x) * n + j] = perm[offsets[x] + j];
}

inline bool small_path(int e, int A) { return dispatch_small_path(e, A); }

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API int64_t b2moe_plan_ints(int32_t experts, int32_t assignments, int32_t shared_tokens) {
    if (experts <= 0 || assignments < 0 || shared_tokens < 0) return 0;
    const int64_t e1 = int64_t(experts) + 1;
    return PLAN_HDR + e1 + (e1 + 1) + e1 + assignments + shared_tokens + (e1 + 1);
}
extern "C" B2MOE_API void b2moe_plan_view_of(int32_t experts, int32_t assignments, int32_t shared_tokens, b2moe_plan_view * v) {
    const int64_t e1 = int64_t(experts) + 1;
    v->counts = PLAN_HDR;
    v->offsets = v->counts + e1;
    v->active = v->offsets + e1 + 1;
    v->perm = v->active + e1;
    v->passes = v->perm + assignments + shared_tokens;
    v->total = v->passes + e1 + 1;
}
extern "C" B2MOE_API size_t b2moe_dispatch_workspace_bytes(int32_t experts, int32_t assignments) {
    if (experts <= 0 || assignments < 0) return 0;
    if (small_path(experts, assignments)) return 16;
    return align_up(size_t(ceil_div(assignments, CHUNK)) * experts * sizeof(int), 16);
}

extern "C" B2MOE_API int32_t b2moe_dispatch_range(const int32_t * ids, int32_t n, int32_t topk, int32_t experts, int32_t shared_first,
                                        int32_t shared_count, int32_t * plan, void * workspace, size_t workspace_bytes,
                                        b2moe_stream stream) {
    if (n <= 0 || topk <= 0 || experts <= 0 || shared_first < 0 || shared_count < 0 || shared_first + shared_count > n) return B2MOE_ERR_SHAPE;
    if ((long long)n * topk > 0x3fffffffLL) return B2MOE_ERR_SHAPE;
    if (!ids || !plan) return B2MOE_ERR_NULL;
    const int A = n * topk;
    cudaStream_t s = as_stream(stream);
    if (small_path(experts, A)) {
        launch_overlapped(dispatch_small_k, dim3(1), dim3(1024), dispatch_small_smem(32, experts), s, ids, A, experts, shared_first, shared_count, plan);
        return launch_status();
    }
    const size_t need = b2moe_dispatch_workspace_bytes(experts, A);
    if (!workspace) return B2MOE_ERR_NULL;
    if (workspace_bytes < need) return B2MOE_ERR_WORKSPACE;
    int * hist = static_cast<int *>(workspace);
    const int chunks = ceil_div(A, CHUNK);
    if (cudaMemsetAsync(hist, 0, size_t(chunks) * experts * sizeof(int), s) != cudaSuccess) return B2MOE_ERR_CUDA;
    dispatch_hist_k<<<ceil_div(chunks, 8), 256, 0, s>>>(ids, A, experts, hist);
    dispatch_scan_k<<<1, 1024, 0, s>>>(hist, chunks, experts, A, shared_count, plan);
    dispatch_scatter_k<<<ceil_div(chunks, 8), 256, 0, s>>>(ids, A, experts, shared_first, shared_count, hist, plan);
    return launch_status();
}

extern "C" B2MOE_API int32_t b2moe_dispatch(const int32_t * ids, int32_t n, int32_t topk, int32_t experts, int32_t shared_tokens,
                                  int32_t * plan, void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    if (shared_tokens != 0 && shared_tokens != n) return B2MOE_ERR_SHAPE;
    return b2moe_dispatch_range(ids, n, topk, experts, 0, shared_tokens, plan, workspace, workspace_bytes, stream);
}

extern "C" B2MOE_API int32_t b2moe_plan_to_groups(const int32_t * plan, int32_t n, int32_t topk, int32_t experts, int32_t * counts,
                                        int32_t * groups, b2moe_stream stream) {
    if (n <= 0 || topk <= 0 || experts <= 0) return B2MOE_ERR_SHAPE;
    if (!plan || !counts || !groups) return B2MOE_ERR_NULL;
    plan_to_groups_k<<<experts, 128, 0, as_stream(stream)>>>(plan, n, experts, counts, groups);
    return launch_status();
}
