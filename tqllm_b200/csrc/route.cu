// Router logits and top-k routing (softmax and sigmoid + selection bias families).
// Replaces router_k / topk_k / topk_warp_k (src/experts/moe.cu:17-166,237-267) and route_k (src/experts/moe_common.cu:18-70).
// Selection rule everywhere: larger key first, lower index on ties (src/experts/moe.cpp:75-78); weights come from
// the unbiased probabilities (src/experts/moe.cpp:85-86); the renormalising sum is clamped at 6.103515625e-5
// (src/experts/moe.hpp:38) and accumulated in selection order like the host reference (src/experts/moe.cpp:103-108).
#include <cooperative_groups.h>
#include <math_constants.h>

#include "common.cuh"
#include "dec4_stage.cuh"
#include "dispatch.cuh"

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

// ---- tensor-core router for bf16 activations ----
// logits = W x with W fp32 split exactly into three bf16 terms (hi + mid + lo = 24 significant bits) and x bf16 as it
// is: every product is exact in fp32 and the sums are fp32, so the result is fp32-accurate (within 3e-6 of an fp64
// dot) at a fraction of the instructions of the scalar loop. One block = 16 router rows x 64 tokens; its 8 warps
// split the hidden dimension and add their partial tiles in shared memory in warp order.
constexpr int RM_WARPS = 16, RM_PART = 8;   // warps per block (each takes a slice of the columns); partial-sum slots in shared memory
__device__ __forceinline__ void split3(float2 w, uint32_t & hi, uint32_t & mid, uint32_t & lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(w.x), h1 = __float2bfloat16_rn(w.y);
    const float r0 = w.x - __bfloat162float(h0), r1 = w.y - __bfloat162float(h1);
    const __nv_bfloat16 m0 = __float2bfloat16_rn(r0), m1 = __float2bfloat16_rn(r1);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(r0 - __bfloat162float(m0)), l1 = __float2bfloat16_rn(r1 - __bfloat162float(m1));
    hi = uint32_t(__bfloat16_as_ushort(h0)) | (uint32_t(__bfloat16_as_ushort(h1)) << 16);
    mid = uint32_t(__bfloat16_as_ushort(m0)) | (uint32_t(__bfloat16_as_ushort(m1)) << 16);
    lo = uint32_t(__bfloat16_as_ushort(l0)) | (uint32_t(__bfloat16_as_ushort(l1)) << 16);
}
__device__ __forceinline__ void mma_bf16_acc(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__global__ void __launch_bounds__(RM_WARPS * 32) router_mma_k(const float * __restrict__ w, const float * __restrict__ shared,
                                                                const __nv_bfloat16 * __restrict__ x, float * __restrict__ logits, int ld,
                                                                int h, int e, int rows, int n) {
    __shared__ float part[RM_PART][16][65];
    __shared__ float tile[16][65];                                      // this block's sums over its slice of the columns
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();                    // the gridDim.z blocks that split the hidden dimension
    grid_release();
    grid_wait();                                                       // x may be the output of the launch before this one
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * 16, t0 = blockIdx.y * 64;
    const int ra = min(r0 + g, rows - 1), rb = min(r0 + g + 8, rows - 1);
    const float * wa = ra == e ? shared : w + size_t(ra) * h, * wb = rb == e ? shared : w + size_t(rb) * h;
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const int hs = h / int(gridDim.z), h_lo = int(blockIdx.z) * hs;     // this block's columns (a multiple of 16)
    const int kper = (hs / 16 + RM_WARPS - 1) / RM_WARPS * 16;          // columns per warp, a multiple of 16
    const int k_lo = h_lo + warp * kper, k_hi = min(h_lo + hs, k_lo + kper);
#pragma unroll 4
    for (int k0 = k_lo; k0 < k_hi; k0 += 16) {
        uint32_t hi[4], mid[4], lo[4];
        split3(*reinterpret_cast<const float2 *>(wa + k0 + 2 * t), hi[0], mid[0], lo[0]);
        split3(*reinterpret_cast<const float2 *>(wb + k0 + 2 * t), hi[1], mid[1], lo[1]);
        split3(*reinterpret_cast<const float2 *>(wa + k0 + 2 * t + 8), hi[2], mid[2], lo[2]);
        split3(*reinterpret_cast<const float2 *>(wb + k0 + 2 * t + 8), hi[3], mid[3], lo[3]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int tok = min(t0 + 8 * j + g, n - 1);
            const uint32_t * xr = reinterpret_cast<const uint32_t *>(x + size_t(tok) * h + k0 + 2 * t);
            const uint32_t b0 = xr[0], b1 = xr[4];
            mma_bf16_acc(acc[j], lo, b0, b1);                            // smallest terms first
            mma_bf16_acc(acc[j], mid, b0, b1);
            mma_bf16_acc(acc[j], hi, b0, b1);
        }
    }
    // warps 8..15 park their sums, warps 0..7 add theirs on top (always in this order: the same bits every run)
    if (warp >= RM_PART) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            part[warp - RM_PART][g][8 * j + 2 * t] = acc[j][0]; part[warp - RM_PART][g][8 * j + 2 * t + 1] = acc[j][1];
            part[warp - RM_PART][g + 8][8 * j + 2 * t] = acc[j][2]; part[warp - RM_PART][g + 8][8 * j + 2 * t + 1] = acc[j][3];
        }
    }
    __syncthreads();
    if (warp < RM_PART) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            part[warp][g][8 * j + 2 * t] += acc[j][0]; part[warp][g][8 * j + 2 * t + 1] += acc[j][1];
            part[warp][g + 8][8 * j + 2 * t] += acc[j][2]; part[warp][g + 8][8 * j + 2 * t + 1] += acc[j][3];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * 64; i += blockDim.x) {
        const int r = i & 15, c = i >> 4;
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < RM_PART; ++q) s += part[q][r][c];
        tile[r][c] = s;
    }
    // the blocks of the cluster hold the sums of their column slices: block 0 adds them in block order through
    // distributed shared memory (the same bits every run) and writes the logits
    cluster.sync();
    if (blockIdx.z == 0) {
        for (int i = threadIdx.x; i < 16 * 64; i += blockDim.x) {
            const int r = i & 15, c = i >> 4;
            if (r0 + r < rows && t0 + c < n) {
                float s = tile[r][c];
                for (unsigned z = 1; z < gridDim.z; ++z) s += cluster.map_shared_rank(&tile[0][0], z)[r * 65 + c];
                logits[size_t(t0 + c) * ld + r0 + r] = s;
            }
        }
    }
    cluster.sync();                                                     // the other blocks' tiles stay alive until block 0 has read them
}

// ---- the same product for many tokens (prefill): shared-memory tiles ----
// One block = 64 router rows x 128 tokens, 8 warps of 32 x 32 outputs, 32 columns per stage: the weights are split into
// their three bf16 terms once per block and stage (not once per 64 tokens and warp as above) and both operands reach the
// MMAs through ldmatrix, so a stage costs a warp 16 shared loads for its 48 MMAs. Every output is summed by one warp over
// the whole hidden dimension in ascending column order (terms lo, mid, hi per 16 columns; 256 columns per partial sum): the
// same bits every run.
constexpr int RT_ROWS = 64, RT_TOK = 128, RT_K = 32, RT_THREADS = 256, RT_LD = RT_K + 8;   // row stride in shared memory: 80 bytes, conflict-free for ldmatrix
constexpr int RT_W_STAGE = 3 * RT_ROWS * RT_LD * 2, RT_X_STAGE = RT_TOK * RT_LD * 2, RT_SMEM = 2 * (RT_W_STAGE + RT_X_STAGE);
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// (w.x, w.y) -> bf16x2 terms hi, mid, lo with hi + mid + lo = w exactly (24 significant bits); same values as split3
__device__ __forceinline__ void split3_pair(float2 w, uint32_t & hi, uint32_t & mid, uint32_t & lo) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(w.y), "f"(w.x));
    const float r0 = w.x - __uint_as_float(hi << 16), r1 = w.y - __uint_as_float(hi & 0xffff0000u);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(mid) : "f"(r1), "f"(r0));
    const float q0 = r0 - __uint_as_float(mid << 16), q1 = r1 - __uint_as_float(mid & 0xffff0000u);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(q1), "f"(q0));
}
__global__ void __launch_bounds__(RT_THREADS) router_tile_k(const float * __restrict__ w, const float * __restrict__ shared,
                                                             const __nv_bfloat16 * __restrict__ x, float * __restrict__ logits, int ld, int h,
                                                             int e, int rows, int n) {
    extern __shared__ __align__(128) uint8_t rt_smem[];
    uint8_t * w_sm = rt_smem;                                          // [2 stages][3 terms][64 rows][RT_LD] bf16
    uint8_t * x_sm = rt_smem + 2 * RT_W_STAGE;                         // [2 stages][128 tokens][RT_LD] bf16
    grid_release();
    grid_wait();                                                       // x may be the output of the launch before this one
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * RT_ROWS, t0 = blockIdx.y * RT_TOK;
    const int wr = warp >> 2, wc = warp & 3;                            // the warp's 32 rows x 32 tokens
    // this thread's four float2 of a weight stage: row f / 16, columns 2 (f % 16), f = tid + 256 j
    const float * wsrc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int f = tid + RT_THREADS * j, row = min(r0 + (f >> 4), rows - 1);
        wsrc[j] = (row == e ? shared : w + size_t(row) * h) + 2 * (f & 15);
    }
    // this thread's two 16-byte pieces of an activation stage: token p / 4, piece p % 4, p = tid + 256 j
    const __nv_bfloat16 * xsrc[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int p = tid + RT_THREADS * j;
        xsrc[j] = x + size_t(min(t0 + (p >> 2), n - 1)) * h + 8 * (p & 3);
    }
    auto load_x = [&](int stage, int k0) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int p = tid + RT_THREADS * j;
            const uint32_t dst = uint32_t(__cvta_generic_to_shared(x_sm + stage * RT_X_STAGE + ((p >> 2) * RT_LD + 8 * (p & 3)) * 2));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(__cvta_generic_to_global(xsrc[j] + k0)) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float2 wreg[4];
    auto load_w = [&](int k0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) wreg[j] = *reinterpret_cast<const float2 *>(wsrc[j] + k0);
    };
    auto store_w = [&](int stage) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = tid + RT_THREADS * j;
            uint32_t hi, mid, lo;
            split3_pair(wreg[j], hi, mid, lo);
            uint32_t * dst = reinterpret_cast<uint32_t *>(w_sm + stage * RT_W_STAGE + ((f >> 4) * RT_LD + 2 * (f & 15)) * 2);
            dst[0] = hi;
            dst[RT_ROWS * RT_LD / 2] = mid;
            dst[2 * RT_ROWS * RT_LD / 2] = lo;
        }
    };
    // acc sums 256 columns at a time and is then added to tot: the rounding error of a long fp32 chain grows with its
    // length, and the router's tolerance against an fp64 dot (3e-6) leaves no room for a 2048-term chain
    float acc[2][4][4], tot[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][b][c] = tot[a][b][c] = 0.f;
    // ldmatrix addresses of this lane inside a stage: A rows 32 wr + 16 rt + (lane % 16), columns 8 (lane / 16);
    // B tokens 32 wc + 16 pr + (lane % 8) + 8 (lane / 16), columns 8 ((lane / 8) % 2)
    const uint32_t w_base = uint32_t(__cvta_generic_to_shared(w_sm)) + ((32 * wr + (lane & 15)) * RT_LD + 8 * (lane >> 4)) * 2;
    const uint32_t x_base = uint32_t(__cvta_generic_to_shared(x_sm)) + ((32 * wc + (lane & 7) + 8 * (lane >> 4)) * RT_LD + 8 * ((lane >> 3) & 1)) * 2;
    const int stages = h / RT_K;
    load_x(0, 0);
    load_w(0);
    for (int s = 0; s < stages; ++s) {
        const int buf = s & 1;
        store_w(buf);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                               // stage s is complete; every warp is done with stage s - 1
        if (s + 1 < stages) { load_x(buf ^ 1, (s + 1) * RT_K); load_w((s + 1) * RT_K); }
#pragma unroll
        for (int kk = 0; kk < RT_K / 16; ++kk) {
            uint32_t b[2][4];                                          // token tiles (0, 1) and (2, 3): b0, b1 of each
#pragma unroll
            for (int pr = 0; pr < 2; ++pr) ldmatrix4(b[pr], x_base + buf * RT_X_STAGE + (16 * pr * RT_LD + 16 * kk) * 2);
#pragma unroll
            for (int term = 2; term >= 0; --term) {                    // smallest terms first
#pragma unroll
                for (int rt = 0; rt < 2; ++rt) {
                    uint32_t a[4];
                    ldmatrix4(a, w_base + buf * RT_W_STAGE + ((term * RT_ROWS + 16 * rt) * RT_LD + 16 * kk) * 2);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) mma_bf16_acc(acc[rt][nt], a, b[nt >> 1][2 * (nt & 1)], b[nt >> 1][2 * (nt & 1) + 1]);
                }
            }
        }
        if ((s & 7) == 7 || s + 1 == stages) {
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int c = 0; c < 4; ++c) { tot[a][b][c] += acc[a][b][c]; acc[a][b][c] = 0.f; }
        }
    }
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int row = r0 + 32 * wr + 16 * rt + g + 8 * (c >> 1), tok = t0 + 32 * wc + 8 * nt + 2 * t + (c & 1);
                if (row < rows && tok < n) logits[size_t(tok) * ld + row] = tot[rt][nt][c];
            }
}

__device__ __forceinline__ void argmax_merge(float & v, int & i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// ---- register-resident routing of one token by one warp (experts <= 32 R) ----
// Lane l keeps experts l, l + 32, ... in registers; a round is a local scan, one warp-wide max of an order-preserving
// integer image of the key and one warp-wide min over the indices that hold it (ties -> lowest index), so the ten
// rounds of a top-10 cost about a microsecond instead of a chain of shared-memory scans and shuffle ladders.
__device__ __forceinline__ uint32_t ordered_bits(float v) {          // monotonic float -> uint (taken entries use 0)
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
template <int GATING, int R>
__device__ __forceinline__ void route_token_regs(const float * __restrict__ logits, int ld, const float * __restrict__ bias,
                                                 int * __restrict__ ids, float * __restrict__ weights, float * __restrict__ shared_weights,
                                                 int e, int k, int norm, float scale, int token, int lane) {
    const float * x = logits + size_t(token) * ld;
    float p[R];
    uint32_t key[R];
#pragma unroll
    for (int r = 0; r < R; ++r) p[r] = lane + 32 * r < e ? x[lane + 32 * r] : -CUDART_INF_F;
    if (GATING == B2MOE_SOFTMAX) {
        float m = -CUDART_INF_F;
#pragma unroll
        for (int r = 0; r < R; ++r) m = fmaxf(m, p[r]);
        for (int d = 16; d; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        float sum = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) if (lane + 32 * r < e) { p[r] = expf(p[r] - m); sum += p[r]; }
        for (int d = 16; d; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
#pragma unroll
        for (int r = 0; r < R; ++r) { p[r] = p[r] / sum; key[r] = lane + 32 * r < e ? ordered_bits(p[r]) : 0u; }
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const bool in = lane + 32 * r < e;
            p[r] = 1.f / (1.f + expf(-p[r]));
            key[r] = in ? ordered_bits(bias ? p[r] + bias[lane + 32 * r] : p[r]) : 0u;
        }
    }
    // lane q keeps the q-th selection (k <= 32 on this path): one coalesced store of ids and weights at the end instead of a
    // store per round and a read-modify-write pass of lane 0 over global memory
    float sel_sum = 0.f, my_p = 0.f;
    int my_idx = 0;
    for (int q = 0; q < k; ++q) {
        uint32_t best = 0;
        int br = 0;
#pragma unroll
        for (int r = 0; r < R; ++r) if (key[r] > best) { best = key[r]; br = r; }     // ascending r: the lowest index keeps a tie
        const uint32_t top = __reduce_max_sync(0xffffffffu, best);
        const int idx = int(__reduce_min_sync(0xffffffffu, (best == top && best != 0u) ? uint32_t(lane + 32 * br) : 0x7fffffffu));
        const int owner = idx & 31, orow = idx >> 5;
        float pv = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) if (r == orow) { pv = p[r]; if (lane == owner) key[r] = 0u; }
        pv = __shfl_sync(0xffffffffu, pv, owner);
        if (lane == q) { my_idx = idx == 0x7fffffff ? 0 : idx; my_p = pv; }
        sel_sum += pv;
    }
    if (lane < k) {
        float w = my_p;
        if (norm) w = w / fmaxf(sel_sum, 6.103515625e-5f);
        if (scale != 0.f && scale != 1.f) w *= scale;
        ids[size_t(token) * k + lane] = my_idx;
        weights[size_t(token) * k + lane] = w;
    }
    if (lane == 0 && shared_weights) shared_weights[token] = 1.f / (1.f + expf(-x[e]));
}

// One warp per token. p[] = unbiased probabilities, key[] = selection keys (p, or p + bias), both in shared memory.
// routes one token with one warp; p / key: e floats each of shared memory owned by the warp
template <int GATING>
__device__ __forceinline__ void route_token(const float * __restrict__ logits, int ld, const float * __restrict__ bias, int * __restrict__ ids,
                                            float * __restrict__ weights, float * __restrict__ shared_weights, int e, int k, int norm,
                                            float scale, int token, int lane, float * p, float * key) {
    if (k <= 32 && e <= 128) return route_token_regs<GATING, 4>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, token, lane);
    if (k <= 32 && e <= 256) return route_token_regs<GATING, 8>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, token, lane);
    if (k <= 32 && e <= 512) return route_token_regs<GATING, 16>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, token, lane);
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
__global__ void route_k(const float * __restrict__ logits, int ld, const float * __restrict__ bias, int * __restrict__ ids,
                        float * __restrict__ weights, float * __restrict__ shared_weights, int e, int k, int norm, float scale, int n) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int token = blockIdx.x * warps + warp;
    grid_release();
    grid_wait();
    if (token >= n) return;
    float * p = smem + size_t(warp) * 2 * e;
    route_token<GATING>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, token, lane, p, p + e);
}

// Two routings in one launch (blockIdx.y picks the set): this layer's logits and the next layer's predicted ones
// (topk_warp2_k, src/experts/moe.cu:160-166). Each token's selection is route_k's.
struct RouteSet { const float * logits; int * ids; float * weights; float * shared_weights; };
template <int GATING>
__global__ void route2_k(const RouteSet a, const RouteSet b, int ld, const float * __restrict__ bias, int e, int k, int norm, float scale, int n) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int token = blockIdx.x * warps + warp;
    const RouteSet & t = blockIdx.y ? b : a;
    grid_release();
    grid_wait();
    if (token >= n) return;
    float * p = smem + size_t(warp) * 2 * e;
    route_token<GATING>(t.logits, ld, bias, t.ids, t.weights, t.shared_weights, e, k, norm, scale, token, lane, p, p + e);
}

// Top-k routing and dispatch in one launch for decode-sized batches: the block's 16 warps route the tokens (round
// robin), then the same block builds the plan from the ids it just wrote. Saves a launch and a device-wide drain.
// 512 threads: the register-resident top-k keeps 32 values per lane, which a 1024-thread block's 64 registers would spill.
constexpr int RD_THREADS = 512;
template <int GATING>
__global__ void __launch_bounds__(RD_THREADS) route_dispatch_k(const float * __restrict__ logits, int ld, const float * __restrict__ bias,
                                                         int * __restrict__ ids, float * __restrict__ weights,
                                                         float * __restrict__ shared_weights, int e, int k, int norm, float scale, int n,
                                                         int shared_first, int shared_count, int * __restrict__ plan) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float * p = smem + size_t(warp) * 2 * e;
    grid_release();
    grid_wait();
    for (int token = warp; token < n; token += RD_THREADS / 32) {
        route_token<GATING>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, token, lane, p, p + e);
        __syncwarp();
    }
    __syncthreads();                              // the ids are written and the routing scratch is dead
    dispatch_small_body(ids, n * k, e, shared_first, shared_count, plan, reinterpret_cast<unsigned short *>(smem));
}

// The same for up to RC_BLOCKS * RD_THREADS / 32 tokens, as one thread-block cluster: every block routes its share of the tokens
// (a warp per token), the cluster meets once, block 0 builds the plan from the ids and the other blocks meanwhile bring the
// layer's activation rows into the staged form of the 4-bit decode kernels (dec4_stage.cuh), which depends on the rows
// alone. One launch instead of three (top-k, dispatch, staging) on the critical path of a decode-sized layer call.
constexpr int RC_BLOCKS = 8;
struct StageJob { const void * x; int dtype, k, bits; uint8_t * rows; float * inv_scale; };     // x = nullptr: nothing to stage
template <int GATING>
__global__ void __launch_bounds__(RD_THREADS) route_cluster_k(const float * __restrict__ logits, int ld, const float * __restrict__ bias,
                                                        int * __restrict__ ids, float * __restrict__ weights,
                                                        float * __restrict__ shared_weights, int e, int k, int norm, float scale, int n,
                                                        int shared_first, int shared_count, int * __restrict__ plan, const StageJob st) {
    extern __shared__ float smem[];
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rank = int(cluster.block_rank()), nb = int(cluster.num_blocks());
    float * p = smem + size_t(warp) * 2 * e;
    grid_release();
    grid_wait();
    for (int token = rank + nb * warp; token < n; token += nb * (RD_THREADS / 32)) {
        route_token<GATING>(logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, token, lane, p, p + e);
        __syncwarp();
    }
    __threadfence();
    cluster.sync();                               // every block's ids are written and visible
    if (rank == 0) {
        dispatch_small_body(ids, n * k, e, shared_first, shared_count, plan, reinterpret_cast<unsigned short *>(smem));
    } else if (st.x) {
        for (int row = (rank - 1) + (nb - 1) * warp; row < n; row += (nb - 1) * (RD_THREADS / 32))
            stage_row_warp(st.x, st.dtype, row, st.k, st.bits, st.rows, st.inv_scale, lane);
    }
}

template <int GATING>
int32_t route_launch(const float * logits, int ld, const float * bias, int * ids, float * weights, float * shared_weights, int e,
                     int k, int norm, float scale, int n, cudaStream_t s) {
    const int warps = e <= 1024 ? 4 : 1;
    const size_t smem = size_t(warps) * 2 * e * sizeof(float);
    launch_overlapped(route_k<GATING>, dim3(ceil_div(n, warps)), dim3(warps * 32), smem, s, logits, ld, bias, ids, weights, shared_weights, e, k, norm, scale, n);
    return launch_status();
}

}  // namespace

// true when the one-cluster routing launch takes this shape: a warp per token, the plan built by one block
bool route_cluster_fits(int experts, int topk, int n) {
    return n >= 1 && n <= RC_BLOCKS * (RD_THREADS / 32) && dispatch_small_path(experts, n * topk) &&
           size_t(RD_THREADS / 32) * 2 * experts * sizeof(float) <= 160 * 1024;
}
// Top-k + dispatch (+ staging of the n activation rows x[n][k] for the 4-bit decode kernels when x is given) as one cluster
// launch. *took = false and B2MOE_OK when the shape does not fit: the caller takes the separate launches.
int32_t route_plan_stage(int gating, const float * logits, int ld, const float * bias, int * ids, float * weights, float * shared_weights,
                         int experts, int topk, int norm, float scale, int n, int shared_first, int shared_count, int * plan, const void * x,
                         int x_dtype, int k, int bits, uint8_t * staged_rows, float * inv_scale, cudaStream_t s, bool * took) {
    *took = false;
    if (!route_cluster_fits(experts, topk, n)) return B2MOE_OK;
    const size_t smem = size_t(RD_THREADS / 32) * 2 * experts * sizeof(float);
    const StageJob st{x, x_dtype, k, bits, staged_rows, inv_scale};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(RC_BLOCKS);
    cfg.blockDim = dim3(RD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = RC_BLOCKS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_overlap ? 2 : 1;
    if (gating == B2MOE_SOFTMAX) {
        if (cudaFuncSetAttribute(route_cluster_k<B2MOE_SOFTMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
        cudaLaunchKernelEx(&cfg, route_cluster_k<B2MOE_SOFTMAX>, logits, ld, (const float *)nullptr, ids, weights, shared_weights, experts, topk, 1, scale, n,
                           shared_first, shared_count, plan, st);
    } else {
        if (cudaFuncSetAttribute(route_cluster_k<B2MOE_SIGMOID>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
        cudaLaunchKernelEx(&cfg, route_cluster_k<B2MOE_SIGMOID>, logits, ld, bias, ids, weights, (float *)nullptr, experts, topk, norm, scale, n,
                           shared_first, shared_count, plan, st);
    }
    *took = true;
    return launch_status();
}
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
    else if (x_dtype == B2MOE_BF16 && hidden % RT_K == 0 && n >= 2 * RT_TOK) {
        if (cudaFuncSetAttribute(router_tile_k, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM) != cudaSuccess) return B2MOE_ERR_CUDA;
        launch_overlapped(router_tile_k, dim3(ceil_div(rows, RT_ROWS), ceil_div(n, RT_TOK)), dim3(RT_THREADS), size_t(RT_SMEM), s, router_w, shared_gate,
                          static_cast<const __nv_bfloat16 *>(x), logits, ld, hidden, experts, rows, n);
    }
    else if (x_dtype == B2MOE_BF16 && hidden % 16 == 0)
    {
        // split the hidden dimension over a cluster of up to 4 blocks while every block keeps at least 256 columns
        int ks = 1;
        while (ks < 4 && hidden % (32 * ks) == 0 && hidden / (2 * ks) >= 256) ks *= 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ceil_div(rows, 16), ceil_div(n, 64), ks);
        cfg.blockDim = dim3(RM_WARPS * 32);
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = ks;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_overlap ? 2 : 1;
        if (cudaLaunchKernelEx(&cfg, router_mma_k, router_w, shared_gate, static_cast<const __nv_bfloat16 *>(x), logits, ld, hidden, experts,
                               rows, n) != cudaSuccess) return B2MOE_ERR_CUDA;
    }
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

extern "C" B2MOE_API int32_t b2moe_topk_softmax2(const float * logits, int32_t * ids, float * weights, float * shared_weights, const float * logits2,
                                                 int32_t * ids2, float * weights2, float * shared_weights2, int32_t ld, int32_t experts, int32_t topk,
                                                 int32_t n, float scale, b2moe_stream stream) {
    if (experts <= 0 || experts > 4096 || topk <= 0 || topk > experts || n <= 0 || ld < experts + ((shared_weights || shared_weights2) ? 1 : 0))
        return B2MOE_ERR_SHAPE;
    if (!logits || !ids || !weights || !logits2 || !ids2 || !weights2) return B2MOE_ERR_NULL;
    const int warps = experts <= 1024 ? 4 : 1;
    const size_t smem = size_t(warps) * 2 * experts * sizeof(float);
    const RouteSet a{logits, ids, weights, shared_weights}, b{logits2, ids2, weights2, shared_weights2};
    launch_overlapped(route2_k<B2MOE_SOFTMAX>, dim3(ceil_div(n, warps), 2), dim3(warps * 32), smem, as_stream(stream), a, b, ld, (const float *)nullptr,
                      experts, topk, 1, scale, n);
    return launch_status();
}

extern "C" B2MOE_API int32_t b2moe_route_sigmoid(const float * logits, int32_t ld, const float * bias, int32_t * ids, float * weights,
                                       int32_t experts, int32_t topk, int32_t norm, float scale, int32_t n, b2moe_stream stream) {
    if (experts <= 0 || experts > 4096 || topk <= 0 || topk > experts || n <= 0 || ld < experts) return B2MOE_ERR_SHAPE;
    if (!logits || !ids || !weights) return B2MOE_ERR_NULL;
    return route_launch<B2MOE_SIGMOID>(logits, ld, bias, ids, weights, nullptr, experts, topk, norm, scale, n, as_stream(stream));
}

// b2moe_topk_softmax / b2moe_route_sigmoid followed by b2moe_dispatch_range, as one launch when the batch is
// decode-sized (otherwise the separate launches); same outputs, same bits.
extern "C" B2MOE_API int32_t b2moe_route_dispatch(int32_t gating, const float * logits, int32_t ld, const float * bias, int32_t * ids,
                                                  float * weights, float * shared_weights, int32_t experts, int32_t topk, int32_t norm,
                                                  float scale, int32_t n, int32_t shared_first, int32_t shared_count, int32_t * plan,
                                                  void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    if (gating != B2MOE_SOFTMAX && gating != B2MOE_SIGMOID) return B2MOE_ERR_SHAPE;
    if (experts <= 0 || experts > 4096 || topk <= 0 || topk > experts || n <= 0 || ld < experts + (shared_weights ? 1 : 0)) return B2MOE_ERR_SHAPE;
    if (shared_first < 0 || shared_count < 0 || shared_first + shared_count > n || (long long)n * topk > 0x3fffffffLL) return B2MOE_ERR_SHAPE;
    if (!logits || !ids || !weights || !plan) return B2MOE_ERR_NULL;
    const size_t smem = size_t(RD_THREADS / 32) * 2 * experts * sizeof(float);
    // one launch only while every token has a warp of its own: the single block routes its tokens RD_THREADS / 32 at a time,
    // and a token's ten selection rounds are a dependent chain of about ten microseconds (measured: 64 tokens, 512 experts:
    // 53 us fused against 12 + 10 us as two launches)
    if (n <= RD_THREADS / 32 && dispatch_small_path(experts, n * topk) && smem <= 160 * 1024) {
        cudaStream_t s = as_stream(stream);
        if (gating == B2MOE_SOFTMAX) {
            if (cudaFuncSetAttribute(route_dispatch_k<B2MOE_SOFTMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
            launch_overlapped(route_dispatch_k<B2MOE_SOFTMAX>, dim3(1), dim3(RD_THREADS), smem, s, logits, ld, nullptr, ids, weights, shared_weights, experts,
                              topk, 1, scale, n, shared_first, shared_count, plan);
        } else {
            if (cudaFuncSetAttribute(route_dispatch_k<B2MOE_SIGMOID>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
            launch_overlapped(route_dispatch_k<B2MOE_SIGMOID>, dim3(1), dim3(RD_THREADS), smem, s, logits, ld, bias, ids, weights, nullptr, experts, topk,
                              norm, scale, n, shared_first, shared_count, plan);
        }
        return launch_status();
    }
    if (route_cluster_fits(experts, topk, n)) {
        bool took = false;
        const int32_t rc = route_plan_stage(gating, logits, ld, bias, ids, weights, shared_weights, experts, topk, norm, scale, n, shared_first,
                                            shared_count, plan, nullptr, 0, 0, 0, nullptr, nullptr, as_stream(stream), &took);
        if (rc || took) return rc;
    }
    if (int32_t rc = gating == B2MOE_SOFTMAX ? b2moe_topk_softmax(logits, ld, ids, weights, shared_weights, experts, topk, n, scale, stream)
                                             : b2moe_route_sigmoid(logits, ld, bias, ids, weights, experts, topk, norm, scale, n, stream)) return rc;
    return b2moe_dispatch_range(ids, n, topk, experts, shared_first, shared_count, plan, workspace, workspace_bytes, stream);
}
