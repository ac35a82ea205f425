// Grouped expert products for IQ3_S banks: the bandwidth-bound decode kernels.
// Replaces u4h_matvec_k<..., FMT = 4, GROUPED> with its paired gate/up and dedup variants
// (src/formats/weight/quant_u4h.inc:424-604, launchers src/formats/weight/quant.cu:69-233) and the separate SwiGLU pass
// (src/experts/moe.cu:188-195).
//
// Every expert's weights are read once per pass of up to 8 of its tokens. The arithmetic runs on the tensor cores
// (mma.m16n8k16 -> fp32):
//   * an IQ3_S weight is  d * (1 + 2 s) * (+-m)  with m an odd magnitude 1..15 from the 512-entry grid; +-m is exact
//     in bf16 and in fp16, so a grid entry re-encoded as four 16-bit floats IS two A-fragment registers, fetched with
//     one 8-byte shared-memory load, and its signs are one shift + one xor per register (bank layout, formats.cuh);
//   * bf16 activations are the B fragment as they are (bf16 x bf16, nothing lost); fp32 / fp16 activations (the down
//     product's inputs among them) become one fp16 term per value after a per-row power-of-two scale (fp16 x fp16,
//     relative rounding 2^-12 per activation: 1e-4 of the output RMS; two bf16 terms were exact to 2^-17 but doubled
//     the MMAs, the scaling FMAs and the activation loads of the down product);
//   * the two MMAs of one 32-weight sub-block start from zero and their fp32 result is scaled by that sub-block's
//     d (1 + 2 s) with one FFMA per accumulator: sums stay fp32, as in the host reference (src/experts/moe.cpp:115-155).
// Lane L = 4 g + t of a warp owns rows g, g + 8 of a 16-row tile and grid entries 2t, 2t + 1 of every sub-block,
// i.e. weights 8t .. 8t + 7 of the sub-block; its B operand is the same 8 activations of token column g (16 bytes).
#include "common.cuh"
#include "formats.cuh"

namespace b2 {
namespace {

constexpr int TILE = 1760;           // bytes of one 16 x 256 IQ3_S tile
constexpr int STAGES = 3;            // tile slots per warp
constexpr int CTA_WARPS = 16;
constexpr int XPAD = 64;             // bytes added to an activation row in shared memory (bank spread)
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// ---------------------------------------------------------------------------------------------------------------
// fp32 / fp16 rows [R][K] -> one fp16 term [R][K], the row multiplied by 2^e so that its largest magnitude lies in
// [2^14, 2^15) (relative rounding error 2^-12 per element, no overflow whatever the input range), + 2^-e per row.
// One warp per row.
__global__ void act_f16_k(const void * __restrict__ x, int dtype, int rows, int k, __half * __restrict__ out, float * __restrict__ inv_scale) {
    const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float mx = 0.f;
    for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(load_act(x, dtype, size_t(row) * k + j)));
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    int ex = int((__float_as_uint(mx) >> 23) & 255u) - 127;              // floor(log2(mx)) for a normal mx
    ex = (mx > 0.f && mx < 3e38f) ? max(-100, min(100, ex)) : 14;
    const float scale = __uint_as_float(uint32_t(127 + 14 - ex) << 23);  // 2^(14 - ex)
    if (lane == 0) inv_scale[row] = __uint_as_float(uint32_t(127 - 14 + ex) << 23);
    for (int j = lane; j < k; j += 32) out[size_t(row) * k + j] = __float2half_rn(load_act(x, dtype, size_t(row) * k + j) * scale);
}

// ---------------------------------------------------------------------------------------------------------------
// mbarrier + bulk copy (the tensor memory accelerator's 1-D copy, no multicast). Every wait is bounded.
// ---------------------------------------------------------------------------------------------------------------
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {   // false = gave up
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}

// ---------------------------------------------------------------------------------------------------------------
// tile registers of one lane and the per-sub-block decode
// ---------------------------------------------------------------------------------------------------------------
struct TileRegs {
    uint32_t w[13];     // 9 words of 9-bit grid indices + 4 sign words (formats.cuh, Fmt<T_IQ3_S>)
    uint32_t sc0, sc8;  // eight 4-bit sub-block scales of rows g, g + 8
    float d0, d8;       // block scales of rows g, g + 8
};
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
// byte offset (index * 128) of grid entry n of the lane's 9-bit stream; n is a compile-time constant after unrolling
__device__ __forceinline__ uint32_t grid_offset(const TileRegs & r, int n) {
    const int bit = 9 * n, q = bit >> 5, sh = bit & 31;
    uint32_t v;
    if (sh >= 7 && sh <= 23) v = r.w[q] >> (sh - 7);
    else if (sh < 7) v = r.w[q] << (7 - sh);
    else v = __funnelshift_r(r.w[q], r.w[q + 1], sh - 7);
    return v & (511u << 7);
}
// d * (1 + 2 s) without an int -> float conversion: 0x4B000001 | 2 s is the float 2^23 + 1 + 2 s
__device__ __forceinline__ float sub_scale(uint32_t sc, float d, float dneg, int ib) {
    const uint32_t two_s = (ib ? sc >> (4 * ib - 1) : sc << 1) & 0x1Eu;
    return fmaf(d, __uint_as_float(two_s | 0x4B000001u), dneg);
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_bf16_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// ---------------------------------------------------------------------------------------------------------------
// The grouped kernel: one resident block of 16 warps per SM.
//   item  = (pass, group of 16 * rpw row tiles); a pass is up to 8 tokens of one active expert (the plan's pass list,
//           the heaviest expert first). Items are dealt round-robin over the blocks.
//   block : stages the pass's activation rows in shared memory with bulk copies (double-buffered when it fits), one
//           barrier per item.
//   warp  : streams the column tiles of its row tile(s) through its own ring of STAGES tile slots (gate and up tiles
//           alternating when MODE = 0): lane 0 posts the byte count on the slot's mbarrier and issues one bulk copy
//           per 1760-byte tile; the warp waits on the phase, copies its 17 words to registers, hands the slot back.
// The grid sits in shared memory as bf16 quadruples, 16 copies, copy c in banks 2c, 2c + 1: the 16 lanes of a
// half-warp (one wavefront of an 8-byte load) never collide.
// MODE 0: out = act[a][row] = silu(gate . x) * (up . x);   MODE 1: out = y[a][row] = down . act[a]
// NTERM terms per activation value ([rows_x][NTERM][k]; the launchers use one). OP 0: bf16 operands (bf16 activations as
// they are); OP 1: fp16 operands (fp32 / fp16 activations as one scaled fp16 term, the sums multiplied by the row's 2^-e).
// ---------------------------------------------------------------------------------------------------------------
struct Iq3sArgs {
    const uint8_t * w0, * w1, * s0, * s1;   // stacked banks (gate, up | down, -) and the shared expert's
    size_t bank_bytes;
    const __nv_bfloat16 * x;                 // 16-bit activation terms: bf16 (OP 0) or scaled fp16 (OP 1)
    const float * inv_scale;                 // OP 1: 2^-e of every activation row
    int * plan;
    float * out;                             // [A + shared][rows]
    int rows, k_tiles, experts, topk, A, rpw, nbuf;
};

constexpr size_t TABLE_BYTES = 512 * 16 * 8, RING_BYTES = size_t(CTA_WARPS) * STAGES * TILE, BAR_BYTES = (CTA_WARPS * STAGES + 2) * 8 + 16;   // the ring barriers, two activation barriers, the block's abort flag
inline size_t xs_bytes(int k, int nterm, int nbuf) { return size_t(nbuf) * 8 * nterm * (size_t(k) * 2 + XPAD); }

template <int MODE, int NTERM, int OP>
__global__ void __launch_bounds__(CTA_WARPS * 32, 1) iq3s_grouped_k(Iq3sArgs p) {
    constexpr int NMAT = MODE == 0 ? 2 : 1, NCH = NTERM;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * table = smem;                                       // entry i, copy c at i * 128 + c * 8
    uint8_t * ring = smem + TABLE_BYTES;                          // [warp][stage][TILE]
    uint64_t * bars = reinterpret_cast<uint64_t *>(ring + RING_BYTES);
    uint8_t * xs = reinterpret_cast<uint8_t *>(bars) + BAR_BYTES; // [buf][8 * NTERM rows][2 k + XPAD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int e1 = p.experts + 1, K = p.k_tiles * 256;
    const int * counts = p.plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    const int * passes = perm + p.A + counts[p.experts];
    const int na = p.plan[PLAN_NACTIVE], row_tiles = (p.rows + 15) >> 4;
    const int groups = (row_tiles + CTA_WARPS * p.rpw - 1) / (CTA_WARPS * p.rpw);
    const int n_items = p.plan[PLAN_NPASS] * groups;
    const uint32_t xrow = uint32_t(K) * 2 + XPAD, xbuf = 8 * NTERM * xrow;

    for (int j = 0; j < 16; ++j) {                                // 512 entries x 16 copies = 8192 slots, 16 per thread
        const int slot = threadIdx.x + CTA_WARPS * 32 * j, i = slot >> 4, c = slot & 15;
        const uint32_t m = c_iq3s_grid[i];                        // four odd magnitudes 1..15 -> bf16 bits (exact)
        uint32_t h[4];
#pragma unroll
        for (int b = 0; b < 4; ++b)
            h[b] = OP == 0 ? __float_as_uint(float((m >> (8 * b)) & 255u)) >> 16 : uint32_t(__half_as_ushort(__float2half_rn(float((m >> (8 * b)) & 255u))));
        *reinterpret_cast<uint2 *>(table + i * 128 + c * 8) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    }
    uint8_t * my_ring = ring + size_t(warp) * STAGES * TILE;
    const uint32_t bar0 = smem_addr(bars + warp * STAGES), ring0 = smem_addr(my_ring);
    const uint32_t xbar = smem_addr(bars + CTA_WARPS * STAGES), xs0 = smem_addr(xs);
    if (lane == 0) for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
    volatile int * abort_flag = reinterpret_cast<volatile int *>(bars + CTA_WARPS * STAGES + 2);   // set by a warp whose bounded wait ran out
    if (threadIdx.x == 0) { mbar_init(xbar, 1); mbar_init(xbar + 8, 1); *abort_flag = 0; }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // pass w -> (expert, first token slot); the pass list runs over the active experts from the last to the first
    auto locate = [&](int w, int & e, int & c0) {
        int lo = 0, hi = na - 1;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (passes[mid] <= w) lo = mid; else hi = mid - 1; }
        e = active[na - 1 - lo];
        c0 = (w - passes[lo]) * PASS_TOKENS;
    };
    // activation rows of item `it` -> buffer b (one thread): one bulk copy per (token, term)
    auto stage_x = [&](int it, int b) {
        int e, c0;
        locate(it / groups, e, c0);
        const int nv = min(PASS_TOKENS, counts[e] - c0);
        mbar_expect_tx(xbar + 8 * b, uint32_t(nv) * NTERM * K * 2);
        for (int s = 0; s < nv; ++s) {
            const int a = perm[offsets[e] + c0 + s];
            const size_t row = MODE == 0 ? size_t(a < p.A ? a / p.topk : a - p.A) : size_t(a);
            for (int term = 0; term < NTERM; ++term)
                bulk_g2s(xs0 + b * xbuf + (s * NTERM + term) * xrow, p.x + (row * NTERM + term) * K, uint32_t(K) * 2, xbar + 8 * b);
        }
    };

    const uint8_t * tab = table + (lane & 15) * 8;
    const int ntiles = p.k_tiles * NMAT;
    uint32_t filled = 0, drained = 0;      // tiles issued into / taken out of this warp's ring since launch
    bool alive = true;
    uint32_t xissued = 0;                  // thread 0: activation stagings issued (their copies must land before the block leaves)
    if (threadIdx.x == 0 && int(blockIdx.x) < n_items) { stage_x(blockIdx.x, 0); ++xissued; }

    int iter = 0;
    for (int it = blockIdx.x; it < n_items; it += gridDim.x, ++iter) {
        const int b = p.nbuf == 2 ? (iter & 1) : 0;
        __syncthreads();                     // every warp is done with the previous item's activation buffer
        if (*abort_flag) break;              // uniform over the block after the barrier: nobody stages or multiplies any more
        if (threadIdx.x == 0) {
            if (p.nbuf == 2) { if (it + int(gridDim.x) < n_items) { stage_x(it + gridDim.x, b ^ 1); ++xissued; } }
            else if (iter > 0) { stage_x(it, 0); ++xissued; }
        }
        if (!alive) continue;
        if (!__all_sync(0xffffffffu, mbar_wait(xbar + 8 * b, (p.nbuf == 2 ? iter >> 1 : iter) & 1u))) { alive = false; *abort_flag = 1; continue; }
        int e, c0;
        locate(it / groups, e, c0);
        const int grp = it % groups, cnt = counts[e], off = offsets[e], nv = min(PASS_TOKENS, cnt - c0);
        const bool shared = e == p.experts;
        const uint8_t * xw = xs + b * xbuf + t * 16;              // + column row * xrow + sub-block * 64

        for (int jr = 0; jr < p.rpw && alive; ++jr) {
            const int rt = (grp * p.rpw + jr) * CTA_WARPS + warp;
            if (rt >= row_tiles) break;
            const uint8_t * base0 = (shared ? p.s0 : p.w0 + size_t(e) * p.bank_bytes) + size_t(rt) * p.k_tiles * TILE;
            const uint8_t * base1 = NMAT == 2 ? (shared ? p.s1 : p.w1 + size_t(e) * p.bank_bytes) + size_t(rt) * p.k_tiles * TILE : base0;
            auto issue = [&](int j) {        // tile j of this row tile -> the next ring slot (lane 0 only)
                const uint32_t s = filled % STAGES;
                const uint8_t * src = ((NMAT == 2 && (j & 1)) ? base1 : base0) + size_t(NMAT == 2 ? j >> 1 : j) * TILE;
                mbar_expect_tx(bar0 + 8 * s, TILE);
                bulk_g2s(ring0 + s * TILE, src, TILE, bar0 + 8 * s);
            };
            for (int j = 0; j < STAGES && j < ntiles; ++j) { if (lane == 0) issue(j); ++filled; }
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
                    if (!__all_sync(0xffffffffu, mbar_wait(bar0 + 8 * s, (drained / STAGES) & 1u))) { alive = false; *abort_flag = 1; break; }
                    TileRegs cur;
                    read_tile(cur, my_ring + s * TILE, lane);
                    ++drained;
                    __syncwarp();             // every lane has its words: the slot can be refilled
                    const int jn = kt * NMAT + m + STAGES;
                    if (jn < ntiles) { if (lane == 0) issue(jn); ++filled; }
                    const float dn0 = cur.d0 * -8388608.f, dn8 = cur.d8 * -8388608.f;
#pragma unroll
                    for (int ib = 0; ib < 8; ++ib) {
                        const uint32_t s0 = cur.w[9 + (ib >> 2)], s8 = cur.w[11 + (ib >> 2)];
                        const int R = 2 * (ib & 3);
                        const uint2 e0 = *reinterpret_cast<const uint2 *>(tab + grid_offset(cur, 2 * ib));
                        const uint2 e1 = *reinterpret_cast<const uint2 *>(tab + grid_offset(cur, 16 + 2 * ib));
                        const uint2 e2 = *reinterpret_cast<const uint2 *>(tab + grid_offset(cur, 2 * ib + 1));
                        const uint2 e3 = *reinterpret_cast<const uint2 *>(tab + grid_offset(cur, 17 + 2 * ib));
                        // first MMA: grid entry 2t (weights 8t .. 8t+3); second: entry 2t + 1 (weights 8t+4 .. 8t+7)
                        const uint32_t a0 = e0.x ^ ((s0 << (15 - R)) & 0x80008000u), a2 = e0.y ^ ((s0 << (7 - R)) & 0x80008000u);
                        const uint32_t a1 = e1.x ^ ((s8 << (15 - R)) & 0x80008000u), a3 = e1.y ^ ((s8 << (7 - R)) & 0x80008000u);
                        const uint32_t c0r = e2.x ^ ((s0 << (14 - R)) & 0x80008000u), c2r = e2.y ^ ((s0 << (6 - R)) & 0x80008000u);
                        const uint32_t c1r = e3.x ^ ((s8 << (14 - R)) & 0x80008000u), c3r = e3.y ^ ((s8 << (6 - R)) & 0x80008000u);
                        const float db0 = sub_scale(cur.sc0, cur.d0, dn0, ib), db8 = sub_scale(cur.sc8, cur.d8, dn8, ib);
#pragma unroll
                        for (int c = 0; c < NCH; ++c) {
                            const uint4 xv = *reinterpret_cast<const uint4 *>(xw + (8 * c + g) * xrow + (kt * 8 + ib) * 64);
                            float r[4];
                            if (OP == 0) { mma_bf16_zero(r, a0, a1, a2, a3, xv.x, xv.y); mma_bf16(r, c0r, c1r, c2r, c3r, xv.z, xv.w); }
                            else { mma_f16_zero(r, a0, a1, a2, a3, xv.x, xv.y); mma_f16(r, c0r, c1r, c2r, c3r, xv.z, xv.w); }
                            acc[m][c][0] = fmaf(db0, r[0], acc[m][c][0]); acc[m][c][1] = fmaf(db0, r[1], acc[m][c][1]);
                            acc[m][c][2] = fmaf(db8, r[2], acc[m][c][2]); acc[m][c][3] = fmaf(db8, r[3], acc[m][c][3]);
                        }
                    }
                }
            }
            if (!alive) break;
            // epilogue: the lane holds rows g, g + 8 x columns 2t, 2t + 1 of every chunk
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
#pragma unroll
                for (int q = 0; q < (NTERM == 1 ? 2 : 1); ++q) {
                    // NTERM 1: columns 2t, 2t + 1 are two tokens; NTERM 2: they are the hi and lo terms of token 4c + t
                    const int slot = NTERM == 1 ? 2 * t + q : 4 * c + t;
                    if (slot >= nv) continue;
                    const int a = perm[off + c0 + slot];
                    const float is = OP == 0 ? 1.f : p.inv_scale[MODE == 0 ? (a < p.A ? a / p.topk : a - p.A) : a];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = 16 * rt + g + 8 * h;
                        if (row >= p.rows) continue;
                        float v[NMAT];
#pragma unroll
                        for (int m = 0; m < NMAT; ++m)
                            v[m] = (NTERM == 1 ? acc[m][c][2 * h + q] : acc[m][c][2 * h] + acc[m][c][2 * h + 1]) * is;
                        p.out[size_t(a) * p.rows + row] = MODE == 0 ? (v[0] / (1.f + expf(-v[0]))) * v[NMAT - 1] : v[0];
                    }
                }
            }
        }
    }
    if (!alive) {                             // a wait ran out: report it and let the copies in flight land before leaving
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.plan + PLAN_STATUS, 1);
        for (; drained < filled; ++drained) mbar_wait(bar0 + 8 * (drained % STAGES), (drained / STAGES) & 1u);
    }
    if (threadIdx.x == 0 && *abort_flag) {    // the last staging into each activation buffer (bounded waits; after a clean run they were consumed)
        const uint32_t nb = uint32_t(p.nbuf);
        for (uint32_t i = xissued > nb ? xissued - nb : 0; i < xissued; ++i) mbar_wait(xbar + 8 * (nb == 2 ? (i & 1u) : 0u), (nb == 2 ? i >> 1 : i) & 1u);
    }
    __syncthreads();                          // nobody leaves while a copy into the block's shared memory may be in flight
}

int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}
constexpr size_t SMEM_LIMIT = 232448 - 1024;

// max_items: an upper bound of passes * groups (the true count is read from the plan on the device)
template <int MODE, int NTERM, int OP>
int32_t launch_grouped(Iq3sArgs a, long long max_items, cudaStream_t s) {
    const int sms = sm_count(), k = a.k_tiles * 256;
    if (sms <= 0) return B2MOE_ERR_CUDA;
    const size_t fixed = TABLE_BYTES + RING_BYTES + BAR_BYTES;
    a.nbuf = fixed + xs_bytes(k, NTERM, 2) <= SMEM_LIMIT ? 2 : 1;
    const size_t smem = fixed + xs_bytes(k, NTERM, a.nbuf);
    if (smem > SMEM_LIMIT) return B2MOE_ERR_SHAPE;
    if (cudaFuncSetAttribute(iq3s_grouped_k<MODE, NTERM, OP>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
        return B2MOE_ERR_CUDA;
    const int blocks = int(std::min<long long>(sms, std::max<long long>(1, max_items)));
    iq3s_grouped_k<MODE, NTERM, OP><<<blocks, CTA_WARPS * 32, smem, s>>>(a);
    return launch_status();
}

// bf16 activations are exact bf16 operands; fp32 / fp16 activations become one scaled fp16 term
inline bool f16_path(int dtype) { return dtype != B2MOE_BF16; }
// row tiles per warp of one work item: as many as keep at least two items per SM (an item = a pass of <= 8 tokens x
// CTA_WARPS * rpw row tiles), so that a handful of tokens still spreads over the SMs; at most row_tiles / 32
inline int rpw_of(int rows, long long est_passes) {
    const int row_tiles = ceil_div(rows, 16), sms = std::max(1, sm_count());
    int rpw = std::max(1, row_tiles / (2 * CTA_WARPS));
    while (rpw > 1 && est_passes * ceil_div(row_tiles, CTA_WARPS * rpw) < 2LL * sms) rpw >>= 1;
    return rpw;
}
inline size_t f16_terms_bytes(int rows_x, int k) { return align_up(size_t(rows_x) * k * sizeof(__half), 256); }
// x -> scaled fp16 rows + inverse scales in the workspace; fills a.x / a.inv_scale
int32_t stage_f16(Iq3sArgs & a, const void * x, int dtype, int rows_x, int k, void * ws, cudaStream_t s) {
    __half * terms = static_cast<__half *>(ws);
    float * inv = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + f16_terms_bytes(rows_x, k));
    act_f16_k<<<ceil_div(rows_x, 8), 256, 0, s>>>(x, dtype, rows_x, k, terms, inv);
    a.x = reinterpret_cast<const __nv_bfloat16 *>(terms);
    a.inv_scale = inv;
    return launch_status();
}

}  // namespace

// true when the IQ3_S kernels take an activation row of length k in `dtype` (it must fit their shared-memory staging)
bool iq3s_supported(int k, int dtype) {
    (void)dtype;
    return k % 256 == 0 && TABLE_BYTES + RING_BYTES + BAR_BYTES + xs_bytes(k, 1, 1) <= SMEM_LIMIT;
}
// scratch: the scaled fp16 copy of `rows_x` activation rows of length k + one float per row (nothing for bf16 activations)
size_t iq3s_workspace_bytes(int rows_x, int k, int dtype) {
    return f16_path(dtype) ? f16_terms_bytes(rows_x, k) + align_up(size_t(rows_x) * sizeof(float), 256) : 0;
}

int32_t iq3s_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x,
                    int x_dtype, const int * plan, int n, int topk, int shared_tokens, float * act, void * ws, int max_active,
                    cudaStream_t s) {
    const int k = gate->cols;
    Iq3sArgs a{};
    a.x = static_cast<const __nv_bfloat16 *>(x);
    if (f16_path(x_dtype))
        if (int32_t rc = stage_f16(a, x, x_dtype, n, k, ws, s)) return rc;
    a.w0 = static_cast<const uint8_t *>(gate->data); a.w1 = static_cast<const uint8_t *>(up->data);
    if (shared_tokens) { a.s0 = static_cast<const uint8_t *>(sg->data); a.s1 = static_cast<const uint8_t *>(su->data); }
    a.bank_bytes = b2moe_bank_bytes(gate->type, gate->rows, gate->cols);
    a.plan = const_cast<int *>(plan); a.out = act;
    a.rows = gate->rows; a.k_tiles = k / 256; a.experts = gate->experts; a.topk = topk; a.A = n * topk;
    const long long est = (long long)max_active + (n * topk + shared_tokens) / PASS_TOKENS;
    a.rpw = rpw_of(gate->rows, est);
    const long long items = est * ceil_div(ceil_div(gate->rows, 16), CTA_WARPS * a.rpw);
    return f16_path(x_dtype) ? launch_grouped<0, 1, 1>(a, items, s) : launch_grouped<0, 1, 0>(a, items, s);
}

int32_t iq3s_down(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk,
                  int shared_tokens, float * y, void * ws, int max_active, cudaStream_t s) {
    const int rows_x = n * topk + shared_tokens, k = down->cols;
    Iq3sArgs a{};
    if (int32_t rc = stage_f16(a, act, B2MOE_F32, rows_x, k, ws, s)) return rc;
    a.w0 = static_cast<const uint8_t *>(down->data);
    if (shared_tokens) a.s0 = static_cast<const uint8_t *>(sd->data);
    a.bank_bytes = b2moe_bank_bytes(down->type, down->rows, down->cols);
    a.plan = const_cast<int *>(plan); a.out = y;
    a.rows = down->rows; a.k_tiles = k / 256; a.experts = down->experts; a.topk = topk; a.A = n * topk;
    const long long est = (long long)max_active + rows_x / PASS_TOKENS;
    a.rpw = rpw_of(down->rows, est);
    const long long items = est * ceil_div(ceil_div(down->rows, 16), CTA_WARPS * a.rpw);
    return launch_grouped<1, 1, 1>(a, items, s);
}

}  // namespace b2
