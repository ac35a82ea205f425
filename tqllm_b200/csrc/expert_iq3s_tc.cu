// Grouped expert products for IQ3_S banks on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory): the decode kernels for batches where every expert sees a few tokens.
// Replaces u4h_matvec_k<..., FMT = 4, GROUPED> with its paired gate/up and dedup variants
// (src/formats/weight/quant_u4h.inc:424-604, launchers src/formats/weight/quant.cu:69-233) and the SwiGLU pass
// (src/experts/moe.cu:188-195).
//
// Why tcgen05 for a bandwidth-bound product: with mma.sync the CUDA cores must build every A fragment in registers,
// and the legacy fp8 MMA is not native on sm_100a, so an IQ3_S weight costs about four issued instructions and the
// kernel is issue-bound at a third of the HBM rate. Here the CUDA cores only turn grid indices + sign bits into E4M3
// bytes in shared memory (exact: +-m, m odd <= 15); one thread issues tcgen05.mma kind::f8f6f4 (M 128 x N 16/32 x
// K 32 = one 32-weight sub-block of 128 rows), and the per-sub-block scale d (1 + 2 s) is applied when the fp32
// result is read back from tensor memory. Activations are split exactly into E4M3 terms (x 2^e = h0 + h1/16 + ...),
// the terms of a token being adjacent columns of the B operand.
//
// Block = 18 warps, one block per SM, persistent over items (pass of <= 8 tokens of one expert, 128-row block):
//   warp 17      lane 0 streams the raw 1760-byte tiles of the next steps into a ring with cp.async.bulk + mbarrier;
//   warps 0..15  decode: warps w and w + 8 turn row tile w of the step (16 rows x 256 columns, four sub-blocks each)
//                into the A operand (canonical K-major core-matrix layout, no swizzle), then — one step later — read
//                the step's fp32 results from tensor memory and accumulate them, scaled, in registers (thread = row,
//                two of the eight sub-blocks);
//   warp 16      lane 0 issues the eight MMAs of a step when all decode warps have arrived, and commits them to the
//                mbarrier the read-back waits on.
// Every wait is bounded; a wait that runs out sets the plan's status word and the block drains and leaves.
#include <cuda_fp8.h>

#include <type_traits>

#include "common.cuh"
#include "formats.cuh"

namespace b2 {
namespace {

constexpr int TILE = 1760;                  // bytes of one 16 x 256 IQ3_S tile
constexpr int ROWS = 128;                   // rows of one item = M of the MMA
constexpr int RAW_SLOTS = 3;                // ring of raw steps (8 tiles each)
constexpr int RAW_SLOT_BYTES = 8 * TILE;
constexpr int A_LBO = 2048 + 64;            // bytes between the two 16-byte k cores of a sub-block (+64: bank spread)
constexpr int A_IB = 2 * A_LBO;             // bytes of one sub-block operand (128 rows x 32 k)
constexpr int A_BUF = 8 * A_IB;             // one step's A operand (128 rows x 256 k)
constexpr int DEC_WARPS = 16;                // decode / read-back warps: two per row tile (four sub-blocks each)
constexpr int MMA_WARP = DEC_WARPS, TMA_WARP = DEC_WARPS + 1;
constexpr int TC_THREADS = (DEC_WARPS + 2) * 32;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 18;

__device__ __forceinline__ uint32_t saddr(const void * p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar) : "memory");
}
// waits on one phase with the hardware's suspending try_wait (up to about a microsecond per try); false = gave up
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory matrix descriptor: K-major, no swizzle; lbo = bytes between the k cores, sbo = between 8-row groups
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(lbo >> 4) << 16) | (uint64_t(sbo >> 4) << 32) | (uint64_t(1) << 46);
}
// D (tensor memory, fp32) = A (128 x 32 E4M3) * B (N x 32 E4M3)^T, overwriting D
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// Activation split: rows [R][K] -> E4M3 terms [R][K / 16][NTERM][16 bytes] + 1 / scale per row. One warp per row.
// scale = 2^e puts the row's largest magnitude in [128, 256) (E4M3 is finite up to 448); term j is the E4M3
// rounding of the remainder times 16^j. Inside every group of four columns the bytes sit in the order 0, 2, 1, 3:
// the order of the weights inside an A-operand word (see decode below).
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
__global__ void act_split_e4m3_k(const void * __restrict__ x, int dtype, int rows, int k, uint8_t * __restrict__ terms,
                                 float * __restrict__ inv_scale) {
    const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float mx = 0.f;
    for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(load_act(x, dtype, size_t(row) * k + j)));
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    int ex = int((__float_as_uint(mx) >> 23) & 255u) - 127;              // floor(log2(mx)) for a normal mx
    ex = (mx > 0.f && mx < 3e38f) ? max(-100, min(100, ex)) : 7;
    const float scale = __uint_as_float(uint32_t(127 + 7 - ex) << 23);   // 2^(7 - ex)
    if (lane == 0) inv_scale[row] = __uint_as_float(uint32_t(127 - 7 + ex) << 23);
    uint32_t * out = reinterpret_cast<uint32_t *>(terms + size_t(row) * k * NTERM);
    for (int q = lane; q < k / 4; q += 32) {                             // four consecutive columns per step
        float r[4], f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = load_act(x, dtype, size_t(row) * k + 4 * q + i) * scale;
        const int core = q >> 2, word = q & 3;
#pragma unroll
        for (int term = 0; term < NTERM; ++term) {
            const uint32_t v = e4m3x4(r[0], r[2], r[1], r[3]);           // byte order 0, 2, 1, 3
            out[(core * NTERM + term) * 4 + word] = v;
            e4m3x4_to_float(v, f);
            r[0] = (r[0] - f[0]) * 16.f; r[2] = (r[2] - f[1]) * 16.f; r[1] = (r[1] - f[2]) * 16.f; r[3] = (r[3] - f[3]) * 16.f;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// the grouped kernel
// ---------------------------------------------------------------------------------------------------------------
struct TcArgs {
    const uint8_t * w0, * w1, * s0, * s1;   // stacked banks (gate, up | down, -) and the shared expert's
    size_t bank_bytes;
    const uint8_t * terms;                   // E4M3 activation terms [rows_x][k / 16][NTERM][16]
    const float * inv_scale;                 // [rows_x]
    int * plan;
    float * out;                             // [A + shared][rows]
    int rows, k_tiles, experts, topk, A;
};

struct TileRegs {
    uint32_t w[13];     // 9 words of 9-bit grid indices + 4 sign words (formats.cuh, Fmt<T_IQ3_S>)
    uint32_t sc0, sc8;  // eight 4-bit sub-block scales of rows g, g + 8
    uint32_t d0, d8;    // block scales of rows g, g + 8 (fp32 bits)
};
__device__ __forceinline__ void read_tile(TileRegs & r, const uint8_t * tile, int lane) {
    const uint4 p0 = reinterpret_cast<const uint4 *>(tile)[lane];
    const uint4 p1 = reinterpret_cast<const uint4 *>(tile + 512)[lane];
    const uint4 p2 = reinterpret_cast<const uint4 *>(tile + 1024)[lane];
    r.w[12] = reinterpret_cast<const uint32_t *>(tile + 1536)[lane];
    const int g = lane >> 2;
    r.sc0 = reinterpret_cast<const uint32_t *>(tile + 1664)[g];
    r.sc8 = reinterpret_cast<const uint32_t *>(tile + 1664)[g + 8];
    r.d0 = __float_as_uint(__half2float(reinterpret_cast<const __half *>(tile + 1728)[g]));
    r.d8 = __float_as_uint(__half2float(reinterpret_cast<const __half *>(tile + 1728)[g + 8]));
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
// one grid entry as four E4M3 bytes with the signs applied. The A-operand word holds the entry's weights in the
// order 0, 2, 1, 3, and so do the sign bits of sign register R of the bank's sign word (bits R, R + 8, R + 16, R + 24).
__device__ __forceinline__ uint32_t entry_e4m3(const uint8_t * tab, const TileRegs & r, int n, uint32_t signs, int R) {
    const uint32_t e = *reinterpret_cast<const uint32_t *>(tab + grid_offset(r, n));
    return e ^ ((signs << (7 - R)) & 0x80808080u);
}

constexpr size_t TC_TABLE = 512 * 32 * 4, TC_RING = size_t(RAW_SLOTS) * RAW_SLOT_BYTES, TC_AOP = 2 * size_t(A_BUF), TC_SCALES = 4 * ROWS * 8;
__host__ __device__ inline size_t tc_b_bytes(int k, int ncol) { return size_t(k) * ncol; }          // k / 32 sub-blocks x (2 cores x ncol x 16 bytes)
__host__ __device__ inline size_t tc_b_area(int k, int ncol, int) { return tc_b_bytes(k, ncol) < 1024 ? 1024 : tc_b_bytes(k, ncol); }
inline size_t tc_smem_bytes(int k, int ncol, int nmat) { return TC_TABLE + TC_RING + TC_AOP + TC_SCALES + tc_b_area(k, ncol, nmat) + 256; }

template <int MODE, int NTERM>
__global__ void __launch_bounds__(TC_THREADS, 1) iq3s_tc_k(TcArgs p) {
    constexpr int NMAT = MODE == 0 ? 2 : 1, NCOL = 8 * NTERM, B_IB = 32 * NCOL, TMEM_COLS = 2 * 8 * NCOL;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t * table = smem;                                   // E4M3 grid: entry i, copy L at i * 128 + L * 4
    uint8_t * ring = table + TC_TABLE;                        // [RAW_SLOTS][8 tiles][TILE]
    uint8_t * aop = ring + TC_RING;                           // [2][8 sub-blocks][2 k cores][16 row groups][8][16]
    uint2 * scales = reinterpret_cast<uint2 *>(aop + TC_AOP); // [4][128] (sub-block scale nibbles, d as fp32 bits), step & 3
    uint8_t * bop = reinterpret_cast<uint8_t *>(scales) + TC_SCALES;   // [k / 32][2 k cores][NCOL / 8][8][16]; also the exchange area
    const int K = p.k_tiles * 256;
    uint64_t * bars = reinterpret_cast<uint64_t *>(bop + tc_b_area(K, NCOL, NMAT));
    // bars: raw_full[3], raw_empty[3], op_full[2], mma_done[2]; then tmem base and the abort flag
    uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
    volatile int * abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t raw_full = saddr(bars), raw_empty = saddr(bars + 3), op_full = saddr(bars + 6), mma_done = saddr(bars + 8);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e1 = p.experts + 1;
    const int * counts = p.plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    const int * passes = perm + p.A + counts[p.experts];
    const int na = p.plan[PLAN_NACTIVE], row_tiles = (p.rows + 15) >> 4, row_blocks = (row_tiles + 7) >> 3;
    const int n_items = p.plan[PLAN_NPASS] * row_blocks, nsteps = p.k_tiles * NMAT;

    for (int i = threadIdx.x; i < 512 * 32; i += TC_THREADS) {
        const uint32_t m = c_iq3s_grid[i >> 5];               // odd magnitudes 1..15 -> E4M3 codes 0x38 0x44 0x4A 0x4E 0x51 0x53 0x55 0x57
        uint32_t b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = uint32_t((0x575553514E4A4438ull >> (8 * (((m >> (8 * j)) & 15u) >> 1))) & 255u);
        reinterpret_cast<uint32_t *>(table)[i] = b[0] | (b[2] << 8) | (b[1] << 16) | (b[3] << 24);   // weights 0, 2, 1, 3
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < 3; ++s) { bar_init(raw_full + 8 * s, 1); bar_init(raw_empty + 8 * s, DEC_WARPS); }
        for (int s = 0; s < 2; ++s) { bar_init(op_full + 8 * s, DEC_WARPS); bar_init(mma_done + 8 * s, 1); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // pass w -> (expert, first token slot); the pass list runs over the active experts from the last to the first
    auto locate = [&](int w, int & e, int & c0) {
        int lo = 0, hi = na - 1;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (passes[mid] <= w) lo = mid; else hi = mid - 1; }
        e = active[na - 1 - lo];
        c0 = (w - passes[lo]) * PASS_TOKENS;
    };
    auto give_up = [&]() { *abort_flag = 1; atomicExch(p.plan + PLAN_STATUS, 2); };

    if (warp == TMA_WARP) {
        // ---- producer: raw tiles of every step, RAW_SLOTS steps ahead ----
        uint32_t gs = 0;
        for (int it = blockIdx.x; it < n_items && !*abort_flag; it += gridDim.x) {
            int e, c0;
            locate(it / row_blocks, e, c0);
            const int rt0 = (it % row_blocks) * 8, nt = min(8, row_tiles - rt0);
            const bool shared = e == p.experts;
            const uint8_t * base0 = (shared ? p.s0 : p.w0 + size_t(e) * p.bank_bytes) + size_t(rt0) * p.k_tiles * TILE;
            const uint8_t * base1 = NMAT == 2 ? (shared ? p.s1 : p.w1 + size_t(e) * p.bank_bytes) + size_t(rt0) * p.k_tiles * TILE : base0;
            for (int s = 0; s < nsteps; ++s, ++gs) {
                const uint32_t slot = gs % RAW_SLOTS, n = gs / RAW_SLOTS;
                if (lane == 0) {
                    if (n > 0 && !bar_wait(raw_empty + 8 * slot, (n - 1) & 1u)) give_up();
                    if (!*abort_flag) {
                        const uint8_t * src = ((NMAT == 2 && (s & 1)) ? base1 : base0) + size_t(NMAT == 2 ? s >> 1 : s) * TILE;
                        bar_expect_tx(raw_full + 8 * slot, uint32_t(nt) * TILE);
                        for (int j = 0; j < nt; ++j)
                            bulk_copy(saddr(ring) + slot * RAW_SLOT_BYTES + j * TILE, src + size_t(j) * p.k_tiles * TILE, TILE, raw_full + 8 * slot);
                    }
                }
                __syncwarp();
                if (*abort_flag) break;
            }
        }
    } else if (warp == MMA_WARP) {
        // ---- MMA issuer ----
        const uint32_t idesc = (1u << 4) | (uint32_t(NCOL >> 3) << 17) | (8u << 24);   // fp32 D, E4M3 x E4M3, K-major, N, M = 128
        uint32_t gs = 0;
        for (int it = blockIdx.x; it < n_items && !*abort_flag; it += gridDim.x) {
            for (int s = 0; s < nsteps; ++s, ++gs) {
                const uint32_t buf = gs & 1u;
                if (lane == 0) {
                    if (!bar_wait(op_full + 8 * buf, (gs >> 1) & 1u)) give_up();
                    if (!*abort_flag) {
                        tc_fence_after();
                        const int kt = NMAT == 2 ? s >> 1 : s;
#pragma unroll
                        for (int ib = 0; ib < 8; ++ib)
                            mma_f8(tmem + buf * 8 * NCOL + ib * NCOL, smem_desc(saddr(aop) + buf * A_BUF + ib * A_IB, A_LBO, 128),
                                   smem_desc(saddr(bop) + (kt * 8 + ib) * B_IB, NCOL * 16, 128), idesc);
                        mma_commit(mma_done + 8 * buf);
                    }
                }
                __syncwarp();
                if (*abort_flag) break;
            }
        }
    } else {
        // ---- decode + read-back warps: warps w and w + 8 share row tile w & 7 (sub-blocks 0..3 / 4..7) ----
        const int g = lane >> 2, t = lane & 3, w = warp, tw = w & 7, half = w >> 3;
        const uint8_t * tab = table + lane * 4;
        const int my_row = 32 * (w & 3) + lane, ib0 = (w >> 2) * 2;          // read-back: this thread's row and its two sub-blocks
        const int tid = threadIdx.x;                                          // 0..511
        uint32_t gs = 0;
        bool alive = true;

        // scaled accumulation of step `g_step`'s results (matrix m): acc[m][c] += d (1 + 2 s) * D[row][c]
        float acc[NMAT][NCOL];
        int ncols = NCOL;                     // valid B columns of the current pass (tokens x terms)
        auto read_back = [&](uint32_t g_step, auto mtag) {
            constexpr int m = decltype(mtag)::value;
            const uint32_t buf = g_step & 1u;
            if (!__all_sync(0xffffffffu, bar_wait(mma_done + 8 * buf, (g_step >> 1) & 1u))) { alive = false; return; }
            tc_fence_after();
            const uint2 sd = scales[(g_step & 3u) * ROWS + my_row];
            const float d = __uint_as_float(sd.y), dneg = d * -8388608.f;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int ib = ib0 + q;
                // d * (1 + 2 s): 0x4B000001 | 2 s is the float 2^23 + 1 + 2 s
                const float db = fmaf(d, __uint_as_float(((sd.x >> (4 * ib) << 1) & 0x1Eu) | 0x4B000001u), dneg);
                const uint32_t taddr = tmem + (uint32_t(32 * (w & 3)) << 16) + buf * 8 * NCOL + ib * NCOL;
                uint32_t r[16];
                if (ncols <= 4) {                 // one or two tokens: the common pass when few tokens share an expert
                    tmem_ld4(taddr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[m][c] = fmaf(db, __uint_as_float(r[c]), acc[m][c]);
                } else if (ncols <= 8) {
                    tmem_ld8(taddr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 8; ++c) acc[m][c] = fmaf(db, __uint_as_float(r[c]), acc[m][c]);
                } else {
#pragma unroll
                    for (int h = 0; h < NCOL / 16; ++h) {
                        if (16 * h < ncols) {
                            tmem_ld16(taddr + 16 * h, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 16; ++c) acc[m][16 * h + c] = fmaf(db, __uint_as_float(r[c]), acc[m][16 * h + c]);
                        }
                    }
                }
            }
            tc_fence_before();
        };

        for (int it = blockIdx.x; it < n_items && alive && !*abort_flag; it += gridDim.x) {
            int e, c0;
            locate(it / row_blocks, e, c0);
            const int rb = it % row_blocks, rt0 = rb * 8, nt = min(8, row_tiles - rt0);
            const int cnt = counts[e], off = offsets[e], nv = min(PASS_TOKENS, cnt - c0);
            ncols = nv * NTERM;
            // stage the B operand: 16-byte pieces of the pass's token rows into core-matrix order
            {
                const int cores = K / 16, per_slot = cores * NTERM;
                for (int pi = tid; pi < nv * per_slot; pi += DEC_WARPS * 32) {
                    const int slot = pi / per_slot, rem = pi - slot * per_slot, c = rem / NTERM, term = rem - c * NTERM;
                    const int a = perm[off + c0 + slot];
                    const size_t row = MODE == 0 ? size_t(a < p.A ? a / p.topk : a - p.A) : size_t(a);
                    const int n = slot * NTERM + term;
                    const uint4 v = *reinterpret_cast<const uint4 *>(p.terms + (row * cores + c) * NTERM * 16 + term * 16);
                    *reinterpret_cast<uint4 *>(bop + (c >> 1) * B_IB + (c & 1) * (NCOL * 16) + (n >> 3) * 128 + (n & 7) * 16) = v;
                }
            }
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int c = 0; c < NCOL; ++c) acc[m][c] = 0.f;

            auto step = [&](int kt, auto mtag) {
                    constexpr int m = decltype(mtag)::value;
                    if (!alive) return;
                    const uint32_t buf = gs & 1u, slot = gs % RAW_SLOTS;
                    if (!__all_sync(0xffffffffu, bar_wait(raw_full + 8 * slot, (gs / RAW_SLOTS) & 1u))) { alive = false; return; }
                    if (tw < nt) {
                        TileRegs cur;
                        read_tile(cur, ring + slot * RAW_SLOT_BYTES + tw * TILE, lane);
                        uint8_t * dst = aop + buf * A_BUF + (t >> 1) * A_LBO + (2 * tw) * 128 + g * 16 + (t & 1) * 8;
                        auto decode_half = [&](auto htag) {
                            constexpr int H = decltype(htag)::value;
                            const uint32_t s0 = cur.w[9 + H], s8 = cur.w[11 + H];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                constexpr int dummy = 0; (void)dummy;
                                const int ib = 4 * H + q, R = 2 * q;
                                uint2 lo, hi;
                                lo.x = entry_e4m3(tab, cur, 2 * ib, s0, R);       lo.y = entry_e4m3(tab, cur, 2 * ib + 1, s0, R + 1);
                                hi.x = entry_e4m3(tab, cur, 16 + 2 * ib, s8, R);  hi.y = entry_e4m3(tab, cur, 17 + 2 * ib, s8, R + 1);
                                *reinterpret_cast<uint2 *>(dst + ib * A_IB) = lo;          // row g
                                *reinterpret_cast<uint2 *>(dst + ib * A_IB + 128) = hi;    // row g + 8
                            }
                        };
                        if (half == 0) {
                            decode_half(std::integral_constant<int, 0>{});
                            if (t == 0) {
                                scales[(gs & 3u) * ROWS + 16 * tw + g] = make_uint2(cur.sc0, cur.d0);
                                scales[(gs & 3u) * ROWS + 16 * tw + g + 8] = make_uint2(cur.sc8, cur.d8);
                            }
                        } else {
                            decode_half(std::integral_constant<int, 1>{});
                        }
                    }
                    fence_async_smem();       // the operand bytes (and the B pieces) must be visible to the tensor core
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { bar_arrive(op_full + 8 * buf); bar_arrive(raw_empty + 8 * slot); }
                    // results of the previous step (the other matrix when there are two)
                    if (kt > 0 || m > 0) read_back(gs - 1, std::integral_constant<int, (m + NMAT - 1) % NMAT>{});
                    ++gs;
            };
            for (int kt = 0; kt < p.k_tiles && alive; ++kt) {
                step(kt, std::integral_constant<int, 0>{});
                if (NMAT == 2) step(kt, std::integral_constant<int, NMAT - 1>{});
            }
            if (alive) read_back(gs - 1, std::integral_constant<int, NMAT - 1>{});
            if (!alive && lane == 0) give_up();

            // four warps hold different sub-blocks of the same rows: three park their sums in shared memory (the A operand
            // area: every MMA of the item has completed), the fourth adds them and finishes the rows
            float * exch = reinterpret_cast<float *>(aop);
            const int grp = w >> 2;
            if (grp > 0) {
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
#pragma unroll
                    for (int c = 0; c < NCOL; ++c) exch[(((grp - 1) * NMAT + m) * NCOL + c) * ROWS + my_row] = acc[m][c];
            }
            asm volatile("bar.sync 1, 512;" ::: "memory");
            if (grp == 0) {
                const int row = rb * ROWS + my_row;
#pragma unroll
                for (int slot = 0; slot < PASS_TOKENS; ++slot) {
                    if (alive && slot < nv && row < p.rows) {
                        const int a = perm[off + c0 + slot];
                        const float is = p.inv_scale[MODE == 0 ? (a < p.A ? a / p.topk : a - p.A) : a];
                        float v[NMAT];
#pragma unroll
                        for (int m = 0; m < NMAT; ++m) {
                            float sum = 0.f, wgt = 1.f;
#pragma unroll
                            for (int term = 0; term < NTERM; ++term) {
                                const int c = slot * NTERM + term;
                                float part = acc[m][c];
#pragma unroll
                                for (int q = 0; q < 3; ++q) part += exch[((q * NMAT + m) * NCOL + c) * ROWS + my_row];
                                sum = fmaf(part, wgt, sum);
                                wgt *= 0.0625f;
                            }
                            v[m] = sum * is;
                        }
                        p.out[size_t(a) * p.rows + row] = MODE == 0 ? (v[0] / (1.f + expf(-v[0]))) * v[NMAT - 1] : v[0];
                    }
                }
            }
            asm volatile("bar.sync 1, 512;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

constexpr size_t TC_SMEM_LIMIT = 232448 - 1024;
int tc_sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}
inline int tc_nterm(int dtype) { return dtype == B2MOE_BF16 ? 2 : 4; }   // bf16 is exact in two E4M3 terms; fp32 / fp16 get four

template <int NTERM>
int32_t tc_split(const void * x, int dtype, int rows, int k, uint8_t * terms, float * inv, cudaStream_t s) {
    act_split_e4m3_k<NTERM><<<ceil_div(rows, 4), 128, 0, s>>>(x, dtype, rows, k, terms, inv);
    return launch_status();
}
template <int MODE, int NTERM>
int32_t tc_launch(const TcArgs & a, long long max_items, cudaStream_t s) {
    const int sms = tc_sm_count();
    if (sms <= 0) return B2MOE_ERR_CUDA;
    const size_t smem = tc_smem_bytes(a.k_tiles * 256, 8 * NTERM, MODE == 0 ? 2 : 1);
    if (smem > TC_SMEM_LIMIT) return B2MOE_ERR_SHAPE;
    if (cudaFuncSetAttribute(iq3s_tc_k<MODE, NTERM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
    const int blocks = int(std::min<long long>(sms, std::max<long long>(1, max_items)));
    iq3s_tc_k<MODE, NTERM><<<blocks, TC_THREADS, smem, s>>>(a);
    return launch_status();
}

}  // namespace

// true when the tcgen05 kernels take activation rows of length k in `dtype` for a product over nmat matrices (2 = gate/up,
// 1 = down): the operands must fit shared memory
bool iq3s_tc_supported(int k, int dtype, int nmat) {
    if (nmat == 2 && tc_nterm(dtype) == 4) return false;      // 64 accumulators per thread do not fit 18 warps' registers
    return k % 256 == 0 && tc_smem_bytes(k, 8 * tc_nterm(dtype), nmat) <= TC_SMEM_LIMIT;
}
// scratch: the E4M3 terms of `rows_x` activation rows of length k and one float per row
size_t iq3s_tc_workspace_bytes(int rows_x, int k, int dtype) {
    return align_up(size_t(rows_x) * k * tc_nterm(dtype), 256) + align_up(size_t(rows_x) * sizeof(float), 256);
}

int32_t iq3s_tc_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x,
                       int x_dtype, const int * plan, int n, int topk, int shared_tokens, float * act, void * ws, int max_active,
                       cudaStream_t s) {
    const int nterm = tc_nterm(x_dtype), k = gate->cols;
    uint8_t * terms = static_cast<uint8_t *>(ws);
    float * inv = reinterpret_cast<float *>(terms + align_up(size_t(n) * k * nterm, 256));
    if (int32_t rc = nterm == 2 ? tc_split<2>(x, x_dtype, n, k, terms, inv, s) : tc_split<4>(x, x_dtype, n, k, terms, inv, s)) return rc;
    TcArgs a{};
    a.w0 = static_cast<const uint8_t *>(gate->data); a.w1 = static_cast<const uint8_t *>(up->data);
    if (shared_tokens) { a.s0 = static_cast<const uint8_t *>(sg->data); a.s1 = static_cast<const uint8_t *>(su->data); }
    a.bank_bytes = b2moe_bank_bytes(gate->type, gate->rows, gate->cols);
    a.terms = terms; a.inv_scale = inv; a.plan = const_cast<int *>(plan); a.out = act;
    a.rows = gate->rows; a.k_tiles = k / 256; a.experts = gate->experts; a.topk = topk; a.A = n * topk;
    const long long items = (long long)(max_active + (n * topk + shared_tokens) / PASS_TOKENS) * ceil_div(gate->rows, ROWS);
    return nterm == 2 ? tc_launch<0, 2>(a, items, s) : tc_launch<0, 4>(a, items, s);
}

int32_t iq3s_tc_down(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk,
                     int shared_tokens, float * y, void * ws, int max_active, cudaStream_t s) {
    const int rows_x = n * topk + shared_tokens, k = down->cols;
    uint8_t * terms = static_cast<uint8_t *>(ws);
    float * inv = reinterpret_cast<float *>(terms + align_up(size_t(rows_x) * k * 4, 256));
    if (int32_t rc = tc_split<4>(act, B2MOE_F32, rows_x, k, terms, inv, s)) return rc;
    TcArgs a{};
    a.w0 = static_cast<const uint8_t *>(down->data);
    if (shared_tokens) a.s0 = static_cast<const uint8_t *>(sd->data);
    a.bank_bytes = b2moe_bank_bytes(down->type, down->rows, down->cols);
    a.terms = terms; a.inv_scale = inv; a.plan = const_cast<int *>(plan); a.out = y;
    a.rows = down->rows; a.k_tiles = k / 256; a.experts = down->experts; a.topk = topk; a.A = n * topk;
    const long long items = (long long)(max_active + rows_x / PASS_TOKENS) * ceil_div(down->rows, ROWS);
    return tc_launch<1, 4>(a, items, s);
}

}  // namespace b2
