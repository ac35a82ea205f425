// Grouped expert products for IQ3_S banks: the bandwidth-bound decode kernels.
// Replaces u4h_matvec_k<..., FMT = 4, GROUPED> with its paired gate/up and dedup variants
// (src/formats/weight/quant_u4h.inc:424-604, launchers src/formats/weight/quant.cu:69-233) and the separate SwiGLU pass
// (src/experts/moe.cu:188-195).
//
// Every expert's weights are read once per launch, by the tokens the dispatch plan grouped on it. The arithmetic
// runs on the tensor cores in fp8 without losing anything:
//   * an IQ3_S weight is  d * (1 + 2 s) * (+-m)  with m an odd magnitude 1..15 from the 512-entry grid: +-m is exact
//     in E4M3, so a grid entry (four magnitudes) re-encoded as four E4M3 bytes IS one A-fragment register of
//     mma.m16n8k32, and the four signs are one shift + one xor away (bank layout, formats.cuh);
//   * an activation x is split exactly into E4M3 terms x * 2^e = h0 + h1 / 16 + h2 / 256 + ... (each term the E4M3
//     rounding of the remainder), two terms for bf16 inputs, four for fp32; the terms of one token are adjacent
//     columns of the B fragment, recombined in fp32 after the loop;
//   * one MMA covers one 32-weight sub-block, so its fp32 result is scaled by that sub-block's d (1 + 2 s) with one
//     FFMA per accumulator: sums stay fp32, as in the host reference (src/experts/moe.cpp:115-155).
// Lane L = 4 g + t of a warp owns rows g, g + 8 of a 16-row tile and grid entries 2t, 2t + 1 of every sub-block.
#include <cuda_fp8.h>

#include "common.cuh"
#include "formats.cuh"

namespace b2 {
namespace {

constexpr int TILE = 1760;          // bytes of one 16 x 256 IQ3_S tile

// ---------------------------------------------------------------------------------------------------------------
// Activation split: rows [R][K] -> E4M3 terms [R][K / 32][NTERM][32 bytes] (natural k order) + 1 / scale per row.
// One warp per row. scale = 2^e puts the row's largest magnitude in [128, 256), inside E4M3's finite range (448).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}
__device__ __forceinline__ void e4m3x4_to_float(uint32_t v, float (&f)[4]) {
    const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffffu), __NV_E4M3);
    const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3);
    const float2 fa = __half22float2(__half2(a)), fb = __half22float2(__half2(b));
    f[0] = fa.x; f[1] = fa.y; f[2] = fb.x; f[3] = fb.y;
}

template <int NTERM>
__global__ void act_split_k(const void * __restrict__ x, int dtype, int rows, int k, uint8_t * __restrict__ terms,
                            float * __restrict__ inv_scale) {
    const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float mx = 0.f;
    for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(load_act(x, dtype, size_t(row) * k + j)));
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    int ex = int((__float_as_uint(mx) >> 23) & 255u) - 127;            // floor(log2(mx)) for normal mx
    ex = mx > 0.f ? max(-100, min(100, ex)) : 7;
    const float scale = __uint_as_float(uint32_t(127 + 7 - ex) << 23);   // 2^(7 - ex)
    if (lane == 0) inv_scale[row] = __uint_as_float(uint32_t(127 - 7 + ex) << 23);
    uint32_t * out = reinterpret_cast<uint32_t *>(terms + size_t(row) * (k / 32) * NTERM * 32);
    for (int q = lane; q < k / 4; q += 32) {                             // four consecutive k per step
        float r[4], f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = load_act(x, dtype, size_t(row) * k + 4 * q + i) * scale;
        const int blk = q >> 3, w = q & 7;
#pragma unroll
        for (int term = 0; term < NTERM; ++term) {
            const uint32_t v = e4m3x4(r[0], r[1], r[2], r[3]);
            out[(blk * NTERM + term) * 8 + w] = v;
            e4m3x4_to_float(v, f);
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = (r[i] - f[i]) * 16.f;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// tile registers of one lane and the per-sub-block decode
// ---------------------------------------------------------------------------------------------------------------
struct TileRegs {
    uint32_t w[13];     // 9 words of 9-bit grid indices + 4 sign words (formats.cuh, Fmt<T_IQ3_S>)
    uint32_t sc0, sc8;  // eight 4-bit sub-block scales of rows g, g + 8
    float d0, d8;       // block scales of rows g, g + 8
};

__device__ __forceinline__ void load_tile(TileRegs & r, const uint8_t * tile, int lane) {
    const uint4 p0 = __ldcs(reinterpret_cast<const uint4 *>(tile) + lane);
    const uint4 p1 = __ldcs(reinterpret_cast<const uint4 *>(tile + 512) + lane);
    const uint4 p2 = __ldcs(reinterpret_cast<const uint4 *>(tile + 1024) + lane);
    r.w[12] = __ldcs(reinterpret_cast<const uint32_t *>(tile + 1536) + lane);
    const int g = lane >> 2;
    r.sc0 = __ldg(reinterpret_cast<const uint32_t *>(tile + 1664) + g);
    r.sc8 = __ldg(reinterpret_cast<const uint32_t *>(tile + 1664) + g + 8);
    r.d0 = __half2float(__ldg(reinterpret_cast<const __half *>(tile + 1728) + g));
    r.d8 = __half2float(__ldg(reinterpret_cast<const __half *>(tile + 1728) + g + 8));
    r.w[0] = p0.x; r.w[1] = p0.y; r.w[2] = p0.z; r.w[3] = p0.w;
    r.w[4] = p1.x; r.w[5] = p1.y; r.w[6] = p1.z; r.w[7] = p1.w;
    r.w[8] = p2.x; r.w[9] = p2.y; r.w[10] = p2.z; r.w[11] = p2.w;
}

// grid index n of the lane's stream (bits [9n, 9n + 9)); n is a compile-time constant after unrolling
__device__ __forceinline__ uint32_t grid_index(const TileRegs & r, int n) {
    const int bit = 9 * n, q = bit >> 5, sh = bit & 31;
    const uint32_t v = sh <= 23 ? r.w[q] >> sh : __funnelshift_r(r.w[q], r.w[q + 1], sh);
    return v & 511u;
}
// d * (1 + 2 s) without an int -> float conversion: 0x4B000001 | 2 s is the float 2^23 + 1 + 2 s
__device__ __forceinline__ float sub_scale(uint32_t sc, float d, float dneg, int ib) {
    const uint32_t two_s = (ib ? sc >> (4 * ib - 1) : sc << 1) & 0x1Eu;
    return fmaf(d, __uint_as_float(two_s | 0x4B000001u), dneg);
}
__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f), "f"(0.f), "f"(0.f));
}

// ---------------------------------------------------------------------------------------------------------------
// Bulk-copy ring: each warp owns STAGES tile slots in shared memory and one mbarrier per slot. Lane 0 posts the
// expected byte count and issues one cp.async.bulk (the 1-D bulk copy of the tensor memory accelerator, no
// multicast) per 1760-byte tile; the warp waits on the slot's mbarrier phase, copies its 17 words to registers and
// hands the slot straight back. Every wait is bounded: a warp that gives up writes PLAN_STATUS and stops.
// ---------------------------------------------------------------------------------------------------------------
constexpr int STAGES = 4;
constexpr int CTA_WARPS = 16;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void * p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait on one phase; false = gave up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}

// tile words of this lane from a shared-memory tile slot
__device__ __forceinline__ void read_tile(TileRegs & r, const uint8_t * tile, int lane) {
    const uint4 p0 = reinterpret_cast<const uint4 *>(tile)[lane];
    const uint4 p1 = reinterpret_cast<const uint4 *>(tile + 512)[lane];
    const uint4 p2 = reinterpret_cast<const uint4 *>(tile + 1024)[lane];
    r.w[12] = reinterpret_cast<const uint32_t *>(tile + 1536)[lane];
    const int g = lane >> 2;
    r.sc0 = reinterpret_cast<const uint32_t *>(tile + 1664)[g];
    r.sc8 = reinterpret_cast<const uint32_t *>(tile + 1664)[g + 8];
    r.d0 = __half2float(reinterpret_cast<const __half *>(tile + 1728)[g]);
    r.d8 = __half2float(reinterpret_cast<const __half *>(tile + 1728)[g + 8]);
    r.w[0] = p0.x; r.w[1] = p0.y; r.w[2] = p0.z; r.w[3] = p0.w;
    r.w[4] = p1.x; r.w[5] = p1.y; r.w[6] = p1.z; r.w[7] = p1.w;
    r.w[8] = p2.x; r.w[9] = p2.y; r.w[10] = p2.z; r.w[11] = p2.w;
}

// ---------------------------------------------------------------------------------------------------------------
// The grouped kernel: one resident block of 16 warps per SM. A work item = (pass, 16-row tile): a pass is up to 8
// tokens of one active expert (the plan's pass list, heaviest expert first); the warp streams every column tile of
// its row tile (gate and up tiles alternating when MODE = 0) through its ring and issues NCH MMAs per decoded
// sub-block (NCH * 8 / NTERM = 8 tokens). Items are dealt round-robin over all warps of the grid.
// The grid lives in shared memory 32 times, copy L in bank L, so the 32 lanes' random lookups never conflict.
// MODE 0: out = act[a][row] = silu(gate . x) * (up . x);   MODE 1: out = y[a][row] = down . act[a]
// ---------------------------------------------------------------------------------------------------------------
struct Iq3sArgs {
    const uint8_t * w0, * w1, * s0, * s1;   // stacked banks (gate, up | down, -) and the shared expert's
    size_t bank_bytes;
    const uint8_t * terms;                   // E4M3 activation terms [rows_x][k / 32][NTERM][32]
    const float * inv_scale;                 // [rows_x]
    int * plan;
    float * out;                             // [A + shared][rows]
    int rows, k_tiles, experts, topk, A;
};

constexpr size_t IQ3S_SMEM = 512 * 32 * 4 + size_t(CTA_WARPS) * STAGES * TILE + CTA_WARPS * STAGES * 8;

template <int MODE, int NTERM>
__global__ void __launch_bounds__(CTA_WARPS * 32, 1) iq3s_grouped_k(Iq3sArgs p) {
    constexpr int NMAT = MODE == 0 ? 2 : 1, NCH = NTERM, TPM = 8 / NTERM;
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t * grid32 = reinterpret_cast<uint32_t *>(smem);                    // [512][32]: entry i of lane L at i * 32 + L
    uint8_t * ring = smem + 512 * 32 * 4;                                       // [warp][stage][TILE]
    uint64_t * bars = reinterpret_cast<uint64_t *>(ring + size_t(CTA_WARPS) * STAGES * TILE);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int e1 = p.experts + 1;
    const int * counts = p.plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    const int * passes = perm + p.A + counts[p.experts];
    const int na = p.plan[PLAN_NACTIVE], row_tiles = (p.rows + 15) >> 4;
    const int n_items = p.plan[PLAN_NPASS] * row_tiles;

    for (int j = 0; j < 32; ++j) {
        const int i = (threadIdx.x >> 5) + CTA_WARPS * j;
        const uint32_t m = c_iq3s_grid[i];   // odd magnitudes 1..15 -> E4M3 codes 0x38 0x44 0x4A 0x4E 0x51 0x53 0x55 0x57
        uint32_t v = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) v |= uint32_t((0x575553514E4A4438ull >> (8 * (((m >> (8 * b)) & 15u) >> 1))) & 255u) << (8 * b);
        grid32[i * 32 + lane] = v;
    }
    uint8_t * my_ring = ring + size_t(warp) * STAGES * TILE;
    const uint32_t bar0 = smem_addr(bars + warp * STAGES), ring0 = smem_addr(my_ring);
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t * my_grid = grid32 + lane;
    const size_t row_bytes = size_t(p.k_tiles) * 8 * NTERM * 32;
    const int ntiles = p.k_tiles * NMAT;
    uint32_t filled = 0, drained = 0;      // tiles issued into / taken out of this warp's ring since launch
    bool alive = true;

    for (int it = warp * gridDim.x + blockIdx.x; it < n_items && alive; it += CTA_WARPS * gridDim.x) {
        const int w = it / row_tiles, rt = it - w * row_tiles;
        int lo = 0, hi = na - 1;             // largest i with passes[i] <= w
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (passes[mid] <= w) lo = mid; else hi = mid - 1; }
        const int e = active[na - 1 - lo], cnt = counts[e], off = offsets[e], c0 = (w - passes[lo]) * PASS_TOKENS;
        const bool shared = e == p.experts;
        const uint8_t * base0 = (shared ? p.s0 : p.w0 + size_t(e) * p.bank_bytes) + size_t(rt) * p.k_tiles * TILE;
        const uint8_t * base1 = NMAT == 2 ? (shared ? p.s1 : p.w1 + size_t(e) * p.bank_bytes) + size_t(rt) * p.k_tiles * TILE : base0;
        auto issue = [&](int j) {            // tile j of this item -> the next ring slot (lane 0 only)
            const uint32_t s = filled % STAGES;
            const uint8_t * src = ((NMAT == 2 && (j & 1)) ? base1 : base0) + size_t(NMAT == 2 ? j >> 1 : j) * TILE;
            mbar_expect_tx(bar0 + 8 * s, TILE);
            bulk_g2s(ring0 + s * TILE, src, TILE, bar0 + 8 * s);
        };
        for (int j = 0; j < STAGES && j < ntiles; ++j) { if (lane == 0) issue(j); ++filled; }

        const uint8_t * bptr[NCH];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {      // column g of chunk c = (token slot g / NTERM, term g % NTERM)
            const int a = perm[off + min(c0 + c * TPM + g / NTERM, cnt - 1)];
            const int xr = MODE == 0 ? (a < p.A ? a / p.topk : a - p.A) : a;
            bptr[c] = p.terms + size_t(xr) * row_bytes + (g % NTERM) * 32 + t * 8;
        }
        const int nch = min(NCH, (cnt - c0 + TPM - 1) / TPM);
        float acc[NMAT][NCH][4];
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[m][c][i] = 0.f;

        for (int kt = 0; kt < p.k_tiles && alive; ++kt) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint32_t s = drained % STAGES;
                if (!__all_sync(0xffffffffu, mbar_wait(bar0 + 8 * s, (drained / STAGES) & 1u))) { alive = false; break; }
                TileRegs cur;
                read_tile(cur, my_ring + s * TILE, lane);
                ++drained;
                __syncwarp();                 // every lane has its words: the slot can be refilled
                const int jn = kt * NMAT + m + STAGES;
                if (jn < ntiles) { if (lane == 0) issue(jn); ++filled; }
                const float dn0 = cur.d0 * -8388608.f, dn8 = cur.d8 * -8388608.f;
#pragma unroll
                for (int ib = 0; ib < 8; ++ib) {
                    const uint32_t s0 = cur.w[9 + (ib >> 2)], s8 = cur.w[11 + (ib >> 2)];
                    const int R = 2 * (ib & 3);
                    const uint32_t a0 = my_grid[grid_index(cur, 2 * ib) * 32] ^ ((s0 << (7 - R)) & 0x80808080u);
                    const uint32_t a2 = my_grid[grid_index(cur, 2 * ib + 1) * 32] ^ ((s0 << (6 - R)) & 0x80808080u);
                    const uint32_t a1 = my_grid[grid_index(cur, 16 + 2 * ib) * 32] ^ ((s8 << (7 - R)) & 0x80808080u);
                    const uint32_t a3 = my_grid[grid_index(cur, 17 + 2 * ib) * 32] ^ ((s8 << (6 - R)) & 0x80808080u);
                    const float db0 = sub_scale(cur.sc0, cur.d0, dn0, ib), db8 = sub_scale(cur.sc8, cur.d8, dn8, ib);
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        if (c < nch) {
                            const uint2 b = __ldg(reinterpret_cast<const uint2 *>(bptr[c] + size_t(kt * 8 + ib) * NTERM * 32));
                            float r[4];
                            mma_e4m3(r, a0, a1, a2, a3, b.x, b.y);
                            acc[m][c][0] = fmaf(db0, r[0], acc[m][c][0]); acc[m][c][1] = fmaf(db0, r[1], acc[m][c][1]);
                            acc[m][c][2] = fmaf(db8, r[2], acc[m][c][2]); acc[m][c][3] = fmaf(db8, r[3], acc[m][c][3]);
                        }
                    }
                }
            }
        }
        if (!alive) break;
        // epilogue: the lane holds rows g, g + 8 x columns 2t, 2t + 1 of every chunk; recombine the terms of a token
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            float v[NMAT][2];                 // [matrix][row g / row g + 8]
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                float lo0 = acc[m][c][0] + acc[m][c][1] * 0.0625f, lo8 = acc[m][c][2] + acc[m][c][3] * 0.0625f;
                if (NTERM == 4) {             // a token's columns 4s..4s+3 sit in lanes t = 2s (terms 0, 1) and 2s + 1 (terms 2, 3)
                    const float o0 = __shfl_xor_sync(0xffffffffu, lo0, 1), o8 = __shfl_xor_sync(0xffffffffu, lo8, 1);
                    lo0 = (t & 1) ? o0 + lo0 * 0.00390625f : lo0 + o0 * 0.00390625f;
                    lo8 = (t & 1) ? o8 + lo8 * 0.00390625f : lo8 + o8 * 0.00390625f;
                }
                v[m][0] = lo0; v[m][1] = lo8;
            }
            const int slot = c0 + c * TPM + (NTERM == 2 ? t : t >> 1);
            const bool writer = slot < cnt && (NTERM == 2 || (t & 1) == 0) && c < nch;
            const int a = perm[off + min(slot, cnt - 1)];          // the token of this lane's OUTPUT columns
            const float is = p.inv_scale[MODE == 0 ? (a < p.A ? a / p.topk : a - p.A) : a];
            if (writer) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = 16 * rt + g + 8 * h;
                    if (row < p.rows) {
                        float o;
                        if (MODE == 0) {
                            const float gv = v[0][h] * is, uv = v[NMAT - 1][h] * is;
                            o = (gv / (1.f + expf(-gv))) * uv;
                        } else {
                            o = v[0][h] * is;
                        }
                        p.out[size_t(a) * p.rows + row] = o;
                    }
                }
            }
        }
    }
    if (!alive) {                             // a wait ran out: report it and let the copies in flight land before leaving
        if (lane == 0) atomicExch(p.plan + PLAN_STATUS, 1);
        for (; drained < filled; ++drained) mbar_wait(bar0 + 8 * (drained % STAGES), (drained / STAGES) & 1u);
    }
}

inline int nterm_of(int dtype) { return dtype == B2MOE_BF16 ? 2 : 4; }

int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

// max_items: an upper bound of passes * row tiles (the true count is read from the plan on the device)
template <int MODE, int NTERM>
int32_t launch_grouped(const Iq3sArgs & a, long long max_items, cudaStream_t s) {
    const int sms = sm_count();
    if (sms <= 0) return B2MOE_ERR_CUDA;
    if (cudaFuncSetAttribute(iq3s_grouped_k<MODE, NTERM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(IQ3S_SMEM)) != cudaSuccess)
        return B2MOE_ERR_CUDA;
    const int blocks = int(std::min<long long>(sms, std::max<long long>(1, max_items)));
    iq3s_grouped_k<MODE, NTERM><<<blocks, CTA_WARPS * 32, IQ3S_SMEM, s>>>(a);
    return launch_status();
}

int32_t split(const void * x, int dtype, int rows, int k, uint8_t * terms, float * inv_scale, int nterm, cudaStream_t s) {
    const dim3 grid(ceil_div(rows, 4));
    if (nterm == 2) act_split_k<2><<<grid, 128, 0, s>>>(x, dtype, rows, k, terms, inv_scale);
    else act_split_k<4><<<grid, 128, 0, s>>>(x, dtype, rows, k, terms, inv_scale);
    return launch_status();
}

}  // namespace

// scratch of the IQ3_S kernels: the E4M3 terms of `rows_x` activation rows of length k, and one float per row
size_t iq3s_workspace_bytes(int rows_x, int k, int dtype) {
    return align_up(size_t(rows_x) * k * nterm_of(dtype), 256) + align_up(size_t(rows_x) * sizeof(float), 256);
}

int32_t iq3s_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x,
                    int x_dtype, const int * plan, int n, int topk, int shared_tokens, float * act, void * ws, int max_active,
                    cudaStream_t s) {
    const int nterm = nterm_of(x_dtype), k = gate->cols;
    uint8_t * terms = static_cast<uint8_t *>(ws);
    float * inv = reinterpret_cast<float *>(terms + align_up(size_t(n) * k * nterm, 256));
    if (int32_t rc = split(x, x_dtype, n, k, terms, inv, nterm, s)) return rc;
    Iq3sArgs a{};
    a.w0 = static_cast<const uint8_t *>(gate->data); a.w1 = static_cast<const uint8_t *>(up->data);
    if (shared_tokens) { a.s0 = static_cast<const uint8_t *>(sg->data); a.s1 = static_cast<const uint8_t *>(su->data); }
    a.bank_bytes = b2moe_bank_bytes(gate->type, gate->rows, gate->cols);
    a.terms = terms; a.inv_scale = inv; a.plan = const_cast<int *>(plan); a.out = act;
    a.rows = gate->rows; a.k_tiles = k / 256; a.experts = gate->experts; a.topk = topk; a.A = n * topk;
    const long long items = (long long)(max_active + (n * topk + shared_tokens) / PASS_TOKENS) * ceil_div(gate->rows, 16);
    return nterm == 2 ? launch_grouped<0, 2>(a, items, s) : launch_grouped<0, 4>(a, items, s);
}

int32_t iq3s_down(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk,
                  int shared_tokens, float * y, void * ws, int max_active, cudaStream_t s) {
    const int rows_x = n * topk + shared_tokens, k = down->cols;
    uint8_t * terms = static_cast<uint8_t *>(ws);
    float * inv = reinterpret_cast<float *>(terms + align_up(size_t(rows_x) * k * 4, 256));
    if (int32_t rc = split(act, B2MOE_F32, rows_x, k, terms, inv, 4, s)) return rc;
    Iq3sArgs a{};
    a.w0 = static_cast<const uint8_t *>(down->data);
    if (shared_tokens) a.s0 = static_cast<const uint8_t *>(sd->data);
    a.bank_bytes = b2moe_bank_bytes(down->type, down->rows, down->cols);
    a.terms = terms; a.inv_scale = inv; a.plan = const_cast<int *>(plan); a.out = y;
    a.rows = down->rows; a.k_tiles = k / 256; a.experts = down->experts; a.topk = topk; a.A = n * topk;
    return launch_grouped<1, 4>(a, (long long)(max_active + rows_x / PASS_TOKENS) * ceil_div(down->rows, 16), s);
}

}  // namespace b2
