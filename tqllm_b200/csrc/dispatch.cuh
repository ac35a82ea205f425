// Device code of the token -> expert dispatch shared by the stand-alone kernels (dispatch.cu) and the fused
// top-k + dispatch kernel (route.cu). See dispatch.cu for the method.
#pragma once
#include "common.cuh"

namespace b2 {

__device__ __forceinline__ int valid_id(const int * ids, int a, int A, int e) {
    if (a >= A) return -1;
    const int v = ids[a];
    return (v >= 0 && v < e) ? v : -1;
}

// counts[0..e1) -> offsets[0..e1], active list and the header words; one warp, each lane a contiguous span. The arrays it reads
// back (counts, active, offsets) are shared-memory copies (cs, as, os): the chains of dependent loads of the pass list would
// otherwise each cross to L2; every result is also written to the plan in global memory.
__device__ inline void finish_plan(int * plan, const int * cs, int * os, int * as, int * offsets, int * active, int * passes, int e1, int lane) {
    const int span = (e1 + 31) / 32, lo = lane * span, hi = min(e1, lo + span);
    int sum = 0, act = 0;
    for (int i = lo; i < hi; ++i) { sum += cs[i]; act += cs[i] > 0; }
    int ps = sum, pa = act;
    for (int d = 1; d < 32; d <<= 1) {
        const int o1 = __shfl_up_sync(0xffffffffu, ps, d), oa = __shfl_up_sync(0xffffffffu, pa, d);
        if (lane >= d) { ps += o1; pa += oa; }
    }
    int run = ps - sum, ra = pa - act;
    for (int i = lo; i < hi; ++i) {
        offsets[i] = run; os[i] = run;
        if (cs[i] > 0) { active[ra] = i; as[ra] = i; ++ra; }
        run += cs[i];
    }
    if (lane == 31) { offsets[e1] = ps; os[e1] = ps; plan[PLAN_NGROUPED] = ps; plan[PLAN_NACTIVE] = pa; plan[PLAN_STATUS] = 0; }
    // pass list: active experts from the last (the shared expert, the heaviest) to the first, cut into passes of
    // PASS_TOKENS tokens; passes[i] = number of passes before the i-th expert of that order
    const int na = __shfl_sync(0xffffffffu, pa, 31);
    __syncwarp();
    const int sp = (na + 31) / 32, l2 = lane * sp, h2 = min(na, l2 + sp);
    int mine = 0;
    for (int i = l2; i < h2; ++i) mine += (cs[as[na - 1 - i]] + PASS_TOKENS - 1) / PASS_TOKENS;
    int pp = mine;
    for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, pp, d);
        if (lane >= d) pp += o;
    }
    int rp = pp - mine;
    for (int i = l2; i < h2; ++i) { passes[i] = rp; rp += (cs[as[na - 1 - i]] + PASS_TOKENS - 1) / PASS_TOKENS; }
    if (lane == 31) { passes[na] = pp; plan[PLAN_NPASS] = pp; }
}

// shared memory of dispatch_small_body for a block of `warps` warps: hist [warps][e] (16-bit) + three int arrays of e + 2
__host__ __device__ inline size_t dispatch_small_smem(int warps, int e) { return (size_t(warps) * e * 2 + 15) / 16 * 16 + size_t(3) * (e + 2) * 4; }

// ---- single block (up to 32 warps): every phase in shared memory (decode-sized batches); hist = [warps][e] ----
__device__ __forceinline__ void dispatch_small_body(const int * __restrict__ ids, int A, int e, int shared_first, int shared_tokens,
                                                    int * __restrict__ plan, unsigned short * hist) {
    const int e1 = e + 1;
    int * counts = plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int * cs = reinterpret_cast<int *>(reinterpret_cast<unsigned char *>(hist) + (size_t(nw) * e * 2 + 15) / 16 * 16), * os = cs + e + 2, * as = os + e + 2;
    const int chunk = ((A + nw - 1) / nw + 31) / 32 * 32;   // per warp, a multiple of 32
    for (int i = threadIdx.x; i < nw * e; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int a0 = warp * chunk;
    for (int a = a0 + lane; a - lane < min(A, a0 + chunk); a += 32) {
        const int id = valid_id(ids, a, A, e);
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        if (id >= 0 && lane == __ffs(peers) - 1) hist[warp * e + id] += (unsigned short)__popc(peers);
        __syncwarp();                 // the leader's update is in place before the next step's leaders read the counter
    }
    __syncthreads();
    for (int x = threadIdx.x; x < e; x += blockDim.x) {
        int run = 0;
        for (int w = 0; w < nw; ++w) { const int c = hist[w * e + x]; hist[w * e + x] = (unsigned short)run; run += c; }
        counts[x] = run; cs[x] = run;
    }
    if (threadIdx.x == 0) { counts[e] = shared_tokens; cs[e] = shared_tokens; }
    __syncthreads();
    if (warp == 0) finish_plan(plan, cs, os, as, offsets, active, perm + A + shared_tokens, e1, lane);
    __syncthreads();
    for (int a = a0 + lane; a - lane < min(A, a0 + chunk); a += 32) {
        const int id = valid_id(ids, a, A, e);
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        if (id >= 0) {
            const int base = hist[warp * e + id];
            perm[os[id] + base + __popc(peers & ((1u << lane) - 1u))] = a;
        }
        __syncwarp();
        if (id >= 0 && lane == __ffs(peers) - 1) hist[warp * e + id] += (unsigned short)__popc(peers);
        __syncwarp();
    }
    for (int t = threadIdx.x; t < shared_tokens; t += blockDim.x) perm[os[e] + t] = A + shared_first + t;
}


inline bool dispatch_small_path(int e, int A) { return A <= 32 * 2048 / 8 && dispatch_small_smem(32, e) <= 46 * 1024; }

}  // namespace b2
