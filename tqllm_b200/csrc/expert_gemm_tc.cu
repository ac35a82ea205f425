// Grouped expert GEMM on the 5th-generation tensor cores for every bank format: the path for batches where an expert
// sees many tokens (prefill) and the tensor-core path of the formats that have no hand-tuned decode kernel.
// Replaces the grouped prefill kernels u4h_gemm_k / k_expert_gemm / k_expert_gemm_gateup
// (src/formats/weight/quant_u4h.inc:609-774, src/formats/weight/quant.cu:286-405) with their fused SwiGLU epilogue
// (quant_u4h.inc:756-759): per expert Y_e = W_e . X_e^T over the expert's gathered token rows.
//
// One persistent block per SM; an item is (expert, tile of <= 128 of its tokens, two blocks of 128 weight rows): the same
// 128 rows of the gate and of the up matrix, or two consecutive row blocks of the down matrix. Per row block
//   D[128 rows][N tokens] (fp32, tensor memory) = sum over K of A[128][K] (fp16) . B[N][K] (fp16)
//   A: the weight rows, decoded from the bank's block format to fp16 in shared memory by the CUDA cores, 64 columns per
//      step (canonical K-major core-matrix layout, no swizzle); the raw blocks arrive through a per-warp ring of bulk
//      copies (cp.async.bulk + mbarrier), 256 columns per copy;
//   B: the tokens' activation rows (fp16, each row scaled by a power of two), gathered through the dispatch permutation with 16-byte cp.async;
//   the two row blocks of an item share B (one gathered copy of the token rows serves 256 weight rows) and have an
//   accumulator each; two accumulator sets alternate between items, so the epilogue of one item (SwiGLU, stores) overlaps
//   the products of the next.
// Warps: 0 issues tcgen05.mma (one lane); 1..4 epilogue (tcgen05.ld, one TMEM lane quarter each); 5..6 load B;
// 7..22 decode A (two warps per row tile of the block: rows g and rows g + 8 of the lane-major tile). Every wait is bounded; a wait that runs out sets the plan's
// status word, and the block drains and leaves.
//
// Numerics: weights are rounded to fp16 after the exact fp32 decode (relative error <= 2^-11 per weight; bf16 operands
// gave 3e-2 of the output RMS as the largest error, fp16 stays below the layer tolerance). An activation row is
// multiplied by 2^e so that its largest magnitude lies in [2^14, 2^15) and rounded to fp16: exact for bf16 inputs down
// to 2^-29 of the row maximum; the epilogue multiplies the sums (fp32) by 2^-e.
#include <type_traits>

#include "common.cuh"
#include "formats.cuh"
#include "gemm_decode.cuh"
#include "tc_ptx.cuh"

namespace b2 {
namespace {
using namespace tc;

constexpr int G_ROWS = 128;                 // weight rows per item = M
// tokens per item: template parameter NT = 128 (two accumulator sets, four B stages; the default) or 256 (one accumulator
// set in the gate/up product, two B stages; opt-in)
constexpr int G_KS = 64;                    // columns per pipeline step (four MMAs of K = 16 per matrix)
constexpr int NMAT = 2;                     // row blocks per item: (gate, up) or two consecutive blocks of the down matrix
constexpr int A_STAGES = 2;                 // stages of decoded A operand (two row blocks each)
constexpr int MAX_A_STAGES = A_STAGES, RAW_SLOTS = 2, MAX_B_STAGES = 4;
constexpr uint32_t DEC_BACKOFF = 60;       // ns between tries of a decode warp's waits
constexpr int A_LBO = gdec::A_LBO;          // bytes between k cores of A
constexpr int A_MAT = 8 * A_LBO;            // one matrix of one A stage: 128 rows x 64 columns
#ifndef B2_LOAD_WARPS
#define B2_LOAD_WARPS 2
#endif
constexpr int MMA_WARP = 0, LOAD_WARP0 = 5, LOAD_WARPS = B2_LOAD_WARPS, LOAD_THREADS = 32 * LOAD_WARPS, DEC_WARP0 = LOAD_WARP0 + LOAD_WARPS, DEC_WARPS = 16;   // warps 1..4: epilogue
constexpr int G_THREADS = (DEC_WARP0 + DEC_WARPS) * 32;
constexpr int N_BARS = 2 * 8 * RAW_SLOTS + 2 * MAX_A_STAGES + 2 * MAX_B_STAGES + 4;

struct GemmArgs {
    const uint8_t * w0, * w1;               // stacked banks (gate, up) or (down, -)
    const uint8_t * s0, * s1;               // the shared expert's banks (may be null)
    const float * aux0, * aux1, * saux0, * saux1;
    size_t bank_bytes;
    const __half * xb;                      // activation rows, fp16, row stride k, row r scaled by 1 / inv_scale[r]
    const float * inv_scale;
    int * plan;
    float * out;
    int rows, k, experts, topk, A;
};

template <uint32_t T> constexpr int chunk_tiles() { return 256 / Fmt<T>::KT; }
template <uint32_t T> constexpr int chunk_bytes() { return chunk_tiles<T>() * Fmt<T>::TILE; }

template <uint32_t T, int NT>
constexpr size_t gemm_smem(int experts) {
    return size_t(A_STAGES) * NMAT * A_MAT + size_t(NT == 128 ? 4 : 2) * (8 * NT * 16) + size_t(8) * RAW_SLOTS * NMAT * chunk_bytes<T>() +
           gdec::Dec<T>::TAB_BYTES + size_t(experts + 3) * 4 + 16 + size_t(N_BARS) * 8 + 16;
}

// any activation dtype -> fp16 rows scaled by a power of two per row (one warp per row) + the inverse scales; inside every
// 64-column step the columns are stored in the order of the format's A operand (gdec::colmap). Two passes over the row:
// its largest magnitude with 16-byte loads, then (from the cache) two source columns per lane and step into one half2
template <uint32_t T, int DT>
__global__ void rows_to_f16_k(const typename Elem<DT>::type * __restrict__ x, int rows, int k, bool wide_loads, __half * __restrict__ out,
                              float * __restrict__ inv_scale) {
    using E = typename Elem<DT>::type;
    constexpr int V = 16 / int(sizeof(E));                              // elements per 16-byte load
    const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const E * xr = x + size_t(row) * k;
    float mx = 0.f;
    if (wide_loads) {                                                  // rows start on 16-byte boundaries (k is a multiple of 64)
#pragma unroll 4
        for (int j = lane * V; j < k; j += 32 * V) {
            const uint4 q = *reinterpret_cast<const uint4 *>(xr + j);
            const E * e = reinterpret_cast<const E *>(&q);
#pragma unroll
            for (int i = 0; i < V; ++i) mx = fmaxf(mx, fabsf(Elem<DT>::to_f(e[i])));
        }
    } else {
        for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(Elem<DT>::to_f(xr[j])));
    }
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    int ex = int((__float_as_uint(mx) >> 23) & 255u) - 127;              // floor(log2(mx)) for a normal mx
    ex = (mx > 0.f && mx < 3e38f) ? max(-100, min(100, ex)) : 14;
    const float scale = __uint_as_float(uint32_t(127 + 14 - ex) << 23);  // 2^(14 - ex)
    if (lane == 0) inv_scale[row] = __uint_as_float(uint32_t(127 - 14 + ex) << 23);
    const int c0 = gdec::colmap<T>(2 * lane), c1 = gdec::colmap<T>(2 * lane + 1);       // source columns of this lane's two positions
    __half2 * orow = reinterpret_cast<__half2 *>(out + size_t(row) * k) + lane;
#pragma unroll 4
    for (int gb = 0; gb < k; gb += 64)
        orow[gb >> 1] = __floats2half2_rn(Elem<DT>::to_f(xr[gb + c0]) * scale, Elem<DT>::to_f(xr[gb + c1]) * scale);
}

// MODE 0: act[a][r] = silu(gate_r . x_tok(a)) * (up_r . x_tok(a));  MODE 1: y[a][r] = down_r . act[a]
template <uint32_t T, int MODE, int NT>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_tc_k(const GemmArgs p) {
    constexpr int G_NT = NT, B_LBO = NT * 16, B_STAGE = 8 * B_LBO;      // B: bytes between k cores; NT tokens x 64 columns
    constexpr int B_STAGES = NT == 128 ? 4 : 2, B_LAG = NT == 128 ? 2 : 1;
    constexpr uint32_t ACC_SETS = NMAT * NT * 2 <= 512 ? 2 : 1;        // accumulator sets that fit the 512 tensor-memory columns
    constexpr int KT = Fmt<T>::KT, TILE = Fmt<T>::TILE, CT = chunk_tiles<T>(), CB = chunk_bytes<T>();
    constexpr uint32_t TMEM_COLS = 512;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * a_st = smem;                                            // [A_STAGES][NMAT][A_MAT]
    uint8_t * b_st = a_st + A_STAGES * NMAT * A_MAT;                  // [B_STAGES][B_STAGE]
    uint8_t * raw = b_st + B_STAGES * B_STAGE;                        // [8 warps][RAW_SLOTS][NMAT][CB]
    uint8_t * dec_tab = raw + 8 * RAW_SLOTS * NMAT * CB;             // the decoder's lookup table
    int * cum = reinterpret_cast<int *>(dec_tab + gdec::Dec<T>::TAB_BYTES);                                   // [na + 1]
    uint64_t * bars = reinterpret_cast<uint64_t *>((reinterpret_cast<uintptr_t>(cum + p.experts + 3) + 15) & ~uintptr_t(15));
    uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(bars + N_BARS);
    volatile int * abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t raw_full = saddr(bars), raw_empty = raw_full + 8 * 8 * RAW_SLOTS, a_full = raw_empty + 8 * 8 * RAW_SLOTS, a_empty = a_full + 8 * MAX_A_STAGES,
                   b_full = a_empty + 8 * MAX_A_STAGES, b_empty = b_full + 8 * MAX_B_STAGES, acc_full = b_empty + 8 * MAX_B_STAGES,
                   acc_empty = acc_full + 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e1 = p.experts + 1;
    const int * counts = p.plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    constexpr int ITEM_TILES = MODE == 0 ? 8 : 16;                     // row tiles of one matrix that an item covers
    const int na = p.plan[PLAN_NACTIVE], row_tiles = (p.rows + 15) >> 4, row_blocks = (row_tiles + ITEM_TILES - 1) / ITEM_TILES;
    const int k_tiles = p.k / KT, ksteps = p.k / G_KS, nchunks = (k_tiles + CT - 1) / CT;

    gdec::Dec<T>::init(dec_tab, threadIdx.x, G_THREADS);
    if (warp == 1) {                                                  // items before active expert i: cum[i]
        int carry = 0;
        for (int base = 0; base < na; base += 32) {
            const int i = base + lane;
            int v = i < na ? ((counts[active[i]] + G_NT - 1) / G_NT) * row_blocks : 0;
            for (int d = 1; d < 32; d <<= 1) { const int o = __shfl_up_sync(0xffffffffu, v, d); if (lane >= d) v += o; }
            if (i < na) cum[i + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) cum[0] = 0;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8 * RAW_SLOTS; ++i) { bar_init(raw_full + 8 * i, 1); bar_init(raw_empty + 8 * i, 2); }
        for (int i = 0; i < A_STAGES; ++i) { bar_init(a_full + 8 * i, DEC_WARPS); bar_init(a_empty + 8 * i, 1); }
        for (int i = 0; i < MAX_B_STAGES; ++i) { bar_init(b_full + 8 * i, LOAD_WARPS); bar_init(b_empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { bar_init(acc_full + 8 * i, 1); bar_init(acc_empty + 8 * i, 4); }
        *abort_flag = 0;
        bar_init_fence();
    }
    if (warp == MMA_WARP) tmem_alloc(saddr(tmem_slot), TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const int n_items = cum[na];

    // item -> expert, first token slot, token count, row block
    struct Item { int e, off, c0, nv, rb; };
    auto locate = [&](int it) {
        int lo = 0, hi = na - 1;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (cum[mid] <= it) lo = mid; else hi = mid - 1; }
        Item r;
        r.e = active[lo];
        const int cnt = counts[r.e], nt = (cnt + G_NT - 1) / G_NT, local = it - cum[lo];
        r.off = offsets[r.e];
        r.rb = local / nt;
        r.c0 = (local - r.rb * nt) * G_NT;
        r.nv = min(G_NT, cnt - r.c0);
        return r;
    };
    auto give_up = [&]() { *abort_flag = 1; atomicExch(p.plan + PLAN_STATUS, 2); };

    if (warp == MMA_WARP) {
        // ---- MMA issuer ----
        uint32_t gk = 0, ic = 0;
        // descriptor halves: low = address / 16 | (bytes between k cores / 16) << 16; high = (128 / 16) | the format's fixed bit 46
        const uint32_t a_lo0 = ((saddr(a_st) & 0x3FFFFu) >> 4) | (uint32_t(A_LBO >> 4) << 16);
        const uint32_t b_lo0 = ((saddr(b_st) & 0x3FFFFu) >> 4) | (uint32_t(B_LBO >> 4) << 16);
        const uint32_t a_hi = (128u >> 4) | (1u << 14), b_hi = a_hi;
        for (int it = blockIdx.x; it < n_items && !*abort_flag; it += gridDim.x, ++ic) {
            const Item im = locate(it);
            const uint32_t npad = uint32_t(im.nv + 15) & ~15u, id = idesc(G_ROWS, npad, 0), ab = ic % ACC_SETS;
            if (lane == 0) {
                if (ic >= ACC_SETS && !bar_wait(acc_empty + 8 * ab, ((ic / ACC_SETS) - 1) & 1u, 100)) give_up();
                fence_after();
                for (int ks = 0; ks < ksteps && !*abort_flag; ++ks, ++gk) {
                    const uint32_t sa = gk % A_STAGES, sb = gk % B_STAGES;
                    if (!bar_wait(a_full + 8 * sa, (gk / A_STAGES) & 1u, 40)) { give_up(); break; }
                    if (!bar_wait(b_full + 8 * sb, (gk / B_STAGES) & 1u, 40)) { give_up(); break; }
                    fence_after();
                    const uint32_t a_lo = a_lo0 + sa * uint32_t((NMAT * A_MAT) >> 4), b_lo = b_lo0 + sb * uint32_t(B_STAGE >> 4);
                    const uint32_t d0 = tmem + ab * (NMAT * G_NT);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                        for (int m = 0; m < NMAT; ++m)
                            mma_f16_lohi(d0 + m * G_NT, a_lo + uint32_t((m * A_MAT + 2 * kk * A_LBO) >> 4), a_hi,
                                         b_lo + uint32_t((2 * kk * B_LBO) >> 4), b_hi, id, (ks | kk) != 0);
                    }
                    mma_commit(a_empty + 8 * sa);
                    mma_commit(b_empty + 8 * sb);
                }
                mma_commit(acc_full + 8 * ab);
            }
            __syncwarp();
        }
    } else if (warp < LOAD_WARP0) {
        // ---- epilogue: warp q reads TMEM lanes [32 q, 32 q + 32) = rows of the block ----
        const int q = warp & 3;
        uint32_t ic = 0;
        for (int it = blockIdx.x; it < n_items && !*abort_flag; it += gridDim.x, ++ic) {
            const Item im = locate(it);
            const uint32_t ab = ic % ACC_SETS;
            if (!__all_sync(0xffffffffu, bar_wait(acc_full + 8 * ab, (ic / ACC_SETS) & 1u, 1000))) { if (lane == 0) give_up(); break; }
            fence_after();
            // this thread's weight row in accumulator 0 and in accumulator 1 (the up matrix's same row, or the next row block)
            const int row = im.rb * (ITEM_TILES * 16) + 32 * q + lane, row1 = MODE == 0 ? row : row + G_ROWS;
            float rs[NMAT];                                            // fp32 row scales of the bank (NVFP4G), else 1
            {
                const bool shared = im.e == p.experts;
                const size_t ai = size_t(shared ? 0 : im.e) * row_tiles * 16;
                const float * a0 = shared ? p.saux0 : p.aux0, * a1 = MODE == 0 ? (shared ? p.saux1 : p.aux1) : a0;
                rs[0] = (a0 && row < p.rows) ? a0[ai + row] : 1.f;
                rs[1] = (a1 && row1 < p.rows) ? a1[ai + row1] : 1.f;
            }
            const uint32_t taddr = tmem + (uint32_t(32 * q) << 16) + ab * (NMAT * G_NT);
            // the item's assignments and their activation scales, 32 per round in registers: the stores below may alias any
            // global array as far as the compiler knows, so loads inside the token loop would each wait for the one before
            int a_of[G_NT / 32];
            float is_of[G_NT / 32];
#pragma unroll
            for (int i = 0; i < G_NT / 32; ++i) {
                const int idx = 32 * i + lane;
                a_of[i] = idx < im.nv ? perm[im.off + im.c0 + idx] : -1;
                is_of[i] = a_of[i] >= 0 ? p.inv_scale[MODE == 0 ? (a_of[i] < p.A ? a_of[i] / p.topk : a_of[i] - p.A) : a_of[i]] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < G_NT / 32; ++i) {
                if (32 * i >= im.nv) break;
#pragma unroll
                for (int c2 = 0; c2 < 32; c2 += 16) {
                    const int c = 32 * i + c2;
                    if (c >= im.nv) break;
                    uint32_t g[16], u[16];
                    tmem_ld16(taddr + c, g);
                    tmem_ld16(taddr + G_NT + c, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int a = __shfl_sync(0xffffffffu, a_of[i], c2 + j);
                        const float is = __shfl_sync(0xffffffffu, is_of[i], c2 + j);
                        if (a >= 0 && row < p.rows) {
                            const float gv = __uint_as_float(g[j]) * (is * rs[0]), uv = __uint_as_float(u[j]) * (is * rs[1]);
                            p.out[size_t(a) * p.rows + row] = MODE == 0 ? __fdividef(gv, 1.f + __expf(-gv)) * uv : gv;      // fast exp and divide: relative error about 2^-21
                            if (MODE == 1 && row1 < p.rows) p.out[size_t(a) * p.rows + row1] = uv;
                        }
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) bar_arrive(acc_empty + 8 * ab);
        }
    } else if (warp < DEC_WARP0) {
        // ---- B loader: thread n copies the 128 bytes of token rows n, n + 64, ... of every step, B_LAG steps in flight ----
        const int n = threadIdx.x - LOAD_WARP0 * 32;
        uint32_t gk = 0, arrived = 0;
        bool ok = true;
        auto arrive_next = [&]() {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) bar_arrive(b_full + 8 * (arrived % B_STAGES));
            ++arrived;
        };
        for (int it = blockIdx.x; it < n_items && ok && !*abort_flag; it += gridDim.x) {
            const Item im = locate(it);
            const int npad = (im.nv + 15) & ~15;
            constexpr int RPT = NT / LOAD_THREADS;                      // token rows per loader thread
            const __half * src[RPT];
            uint32_t src_bytes[RPT];
#pragma unroll
            for (int h = 0; h < RPT; ++h) {
                src[h] = p.xb;
                src_bytes[h] = 0;
                if (n + LOAD_THREADS * h < im.nv) {
                    const int a = perm[im.off + im.c0 + n + LOAD_THREADS * h];
                    src[h] = p.xb + size_t(MODE == 0 ? (a < p.A ? a / p.topk : a - p.A) : a) * p.k;
                    src_bytes[h] = 16;
                }
            }
            const uint32_t dst0 = saddr(b_st) + (n >> 3) * 128 + (n & 7) * 16;
            for (int ks = 0; ks < ksteps; ++ks, ++gk) {
                const uint32_t sb = gk % B_STAGES;
                if (gk >= B_STAGES && !__all_sync(0xffffffffu, bar_wait(b_empty + 8 * sb, ((gk / B_STAGES) - 1) & 1u, 200))) { ok = false; break; }
#pragma unroll
                for (int h = 0; h < RPT; ++h) {
                    if (n + LOAD_THREADS * h < npad) {
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            cp_async16(dst0 + sb * B_STAGE + c * B_LBO + h * (LOAD_THREADS * 16), src[h] + (src_bytes[h] ? ks * G_KS + c * 8 : 0), src_bytes[h]);
                    }
                }
                cp_async_commit();
                if (gk - arrived >= B_LAG) { cp_async_wait<B_LAG>(); arrive_next(); }
            }
        }
        cp_async_wait<0>();
        while (arrived < gk) arrive_next();
        if (!ok && lane == 0) give_up();
    } else {
        // ---- A decoder: warps tw and tw + 8 own row tile tw of the block (rows g / rows g + 8 of the tile): raw chunks
        // (256 columns) -> fp16 operand, 64 columns a step; the first warp of the pair streams the chunks ----
        const int dwi = warp - DEC_WARP0, tw = dwi & 7, half = dwi >> 3;
        uint8_t * my_raw = raw + tw * RAW_SLOTS * NMAT * CB;
        const uint32_t my_full = raw_full + 8 * tw * RAW_SLOTS, my_empty = raw_empty + 8 * tw * RAW_SLOTS;
        uint32_t gk = 0, gc = 0;
        bool ok = true;
        for (int it = blockIdx.x; it < n_items && ok && !*abort_flag; it += gridDim.x) {
            const Item im = locate(it);
            // row tile of accumulator 0 and of accumulator 1: the same tile of the gate and the up matrix, or tiles tw and tw + 8 of the item's 16
            const int rt = im.rb * ITEM_TILES + tw, rt1 = MODE == 0 ? rt : rt + 8;
            const bool live = rt < row_tiles, live1 = rt1 < row_tiles, shared = im.e == p.experts;      // live1 implies live
            const uint8_t * bank0 = shared ? p.s0 : p.w0 + size_t(im.e) * p.bank_bytes;
            const uint8_t * bank1 = MODE == 0 ? (shared ? p.s1 : p.w1 + size_t(im.e) * p.bank_bytes) : bank0;
            const uint8_t * base[NMAT] = {bank0 + size_t(rt) * k_tiles * TILE, bank1 + size_t(rt1) * k_tiles * TILE};
            // chunk c of this row tile -> the ring slot of use number u (lane 0 of the pair's first warp); false = gave up
            auto issue = [&](int c, uint32_t u) {
                const uint32_t slot = u % RAW_SLOTS;
                if (u >= RAW_SLOTS && !bar_wait(my_empty + 8 * slot, ((u / RAW_SLOTS) - 1) & 1u)) return false;   // both warps are done with it
                const int tiles = min(CT, k_tiles - c * CT);
                const uint32_t bytes = uint32_t(tiles) * TILE, bar = my_full + 8 * slot;
                bar_expect_tx(bar, live1 ? 2 * bytes : bytes);
                bulk_copy(saddr(my_raw) + (slot * NMAT + 0) * CB, base[0] + size_t(c) * CT * TILE, bytes, bar);
                if (live1) bulk_copy(saddr(my_raw) + (slot * NMAT + 1) * CB, base[1] + size_t(c) * CT * TILE, bytes, bar);
                return true;
            };
            if (live && half == 0 && lane == 0)
                for (int c = 0; c < RAW_SLOTS && c < nchunks; ++c)
                    if (!issue(c, gc + c)) { give_up(); break; }
            for (int c = 0; c < nchunks && ok; ++c, gc += live ? 1u : 0u) {     // a dead row tile (past the last row) uses no slot
                const uint32_t slot = gc % RAW_SLOTS;
                if (live && !__all_sync(0xffffffffu, bar_wait(my_full + 8 * slot, (gc / RAW_SLOTS) & 1u, DEC_BACKOFF))) { ok = false; break; }
                const int steps = min(4, ksteps - 4 * c);
                typename gdec::Dec<T>::Pre pre[NMAT];                  // per-chunk constants of the decoder
                const uint8_t * chunk0 = my_raw + (slot * NMAT + 0) * CB, * chunk1 = my_raw + (slot * NMAT + 1) * CB;
                typename gdec::Dec<T>::Raw rw[NMAT];                   // the raw words of the step that comes next
                if (live) { pre[0] = gdec::Dec<T>::prep(chunk0, lane, half); rw[0] = gdec::Dec<T>::template load<0>(chunk0, lane, half); }
                if (live1) { pre[1] = gdec::Dec<T>::prep(chunk1, lane, half); rw[1] = gdec::Dec<T>::template load<0>(chunk1, lane, half); }
                // the (up to) four 64-column steps of the chunk, written out so that every step is straight-line code with its
                // column offset a constant and the lane's row / table / scale addresses computed once per chunk
                auto one_step = [&](auto J) {
                    constexpr int j = decltype(J)::value;
                    if (j >= steps || !ok) return;
                    const uint32_t sa = gk % A_STAGES;
                    if (gk >= A_STAGES && !__all_sync(0xffffffffu, bar_wait(a_empty + 8 * sa, ((gk / A_STAGES) - 1) & 1u, DEC_BACKOFF))) { ok = false; return; }
                    const int row16 = (lane >> 2) + 8 * half, tq = lane & 3;
                    if (live) {
                        uint4 o[2];
                        gdec::Dec<T>::template compute<j>(rw[0], chunk0, lane, dec_tab, half, pre[0], o);
                        uint8_t * dst = a_st + (sa * NMAT + 0) * A_MAT + 2 * tw * 128;
                        *gdec::core_row(dst, tq, row16) = o[0];
                        *gdec::core_row(dst, tq + 4, row16) = o[1];
                    }
                    if (live1) {
                        uint4 o[2];
                        gdec::Dec<T>::template compute<j>(rw[1], chunk1, lane, dec_tab, half, pre[1], o);
                        uint8_t * dst = a_st + (sa * NMAT + 1) * A_MAT + 2 * tw * 128;
                        *gdec::core_row(dst, tq, row16) = o[0];
                        *gdec::core_row(dst, tq + 4, row16) = o[1];
                    }
                    if (j + 1 < 4 && j + 1 < steps) {                  // the next step's raw words, in flight across the hand-off and the next wait
                        if (live) rw[0] = gdec::Dec<T>::template load<(j + 1) & 3>(chunk0, lane, half);
                        if (live1) rw[1] = gdec::Dec<T>::template load<(j + 1) & 3>(chunk1, lane, half);
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) bar_arrive(a_full + 8 * sa);
                    ++gk;
                };
                one_step(std::integral_constant<int, 0>{});
                one_step(std::integral_constant<int, 1>{});
                one_step(std::integral_constant<int, 2>{});
                one_step(std::integral_constant<int, 3>{});
                if (!ok) break;
                __syncwarp();                                          // every lane is done with the slot
                if (live && lane == 0) {
                    bar_arrive(my_empty + 8 * slot);
                    if (half == 0 && c + RAW_SLOTS < nchunks && !issue(c + RAW_SLOTS, gc + RAW_SLOTS)) { give_up(); ok = false; }
                }
                ok = __all_sync(0xffffffffu, ok);
            }
        }
        if (!ok && lane == 0) give_up();
    }
    fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_free(tmem, TMEM_COLS);
}

int gemm_sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}
constexpr size_t GEMM_SMEM_LIMIT = 232448 - 1024;

template <uint32_t T, int MODE, int NT>
int32_t gemm_launch_nt(const GemmArgs & a, int sms, cudaStream_t s) {
    const size_t smem = gemm_smem<T, NT>(a.experts);
    if (smem > GEMM_SMEM_LIMIT) return B2MOE_ERR_SHAPE;
    if (cudaFuncSetAttribute(gemm_tc_k<T, MODE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
    gemm_tc_k<T, MODE, NT><<<sms, G_THREADS, smem, s>>>(a);
    return launch_status();
}
// 128-token items. The 256-token variant (weights decoded once per 256 tokens, but one accumulator set and two B stages) is
// correct and slower where it was measured (c5, 512 tokens per expert: 261 against 395 TFLOP/s: the gathered B loads with one
// step of lookahead become the limit); b2moe_harness_select(.., 256) selects it for measurements
int g_item_tokens = 128;
template <uint32_t T, int MODE>
int32_t gemm_launch_t(const GemmArgs & a, cudaStream_t s) {
    const int sms = gemm_sm_count();
    if (sms <= 0) return B2MOE_ERR_CUDA;
    const bool wide = g_item_tokens == 256;
    if (wide && gemm_smem<T, 256>(a.experts) <= GEMM_SMEM_LIMIT) return gemm_launch_nt<T, MODE, 256>(a, sms, s);
    return gemm_launch_nt<T, MODE, 128>(a, sms, s);
}
template <int MODE>
int32_t gemm_launch(uint32_t type, const GemmArgs & a, cudaStream_t s) {
    switch (type) {
        case T_Q4_K: return gemm_launch_t<T_Q4_K, MODE>(a, s);
        case T_IQ3_S: return gemm_launch_t<T_IQ3_S, MODE>(a, s);
        case T_IQ3S4: return gemm_launch_t<T_IQ3S4, MODE>(a, s);
        case T_IQ4_XS: return gemm_launch_t<T_IQ4_XS, MODE>(a, s);
        case T_IQ4_NL: return gemm_launch_t<T_IQ4_NL, MODE>(a, s);
        case T_NVFP4G: return gemm_launch_t<T_NVFP4G, MODE>(a, s);
    }
    return B2MOE_ERR_FORMAT;
}
size_t gemm_smem_of(uint32_t type, int experts) {
    switch (type) {
        case T_Q4_K: return gemm_smem<T_Q4_K, 128>(experts);
        case T_IQ3_S: return gemm_smem<T_IQ3_S, 128>(experts);
        case T_IQ3S4: return gemm_smem<T_IQ3S4, 128>(experts);
        case T_IQ4_XS: return gemm_smem<T_IQ4_XS, 128>(experts);
        case T_IQ4_NL: return gemm_smem<T_IQ4_NL, 128>(experts);
        case T_NVFP4G: return gemm_smem<T_NVFP4G, 128>(experts);
    }
    return ~size_t(0);
}
template <uint32_t T>
int32_t convert_rows_t(const void * x, int dtype, int rows, int k, __half * out, float * inv, cudaStream_t s) {
    const int blocks = ceil_div(rows, 8);
    const bool wide = aligned16(x);
    switch (dtype) {
        case B2MOE_F32: rows_to_f16_k<T, B2MOE_F32><<<blocks, 256, 0, s>>>(static_cast<const float *>(x), rows, k, wide, out, inv); break;
        case B2MOE_F16: rows_to_f16_k<T, B2MOE_F16><<<blocks, 256, 0, s>>>(static_cast<const __half *>(x), rows, k, wide, out, inv); break;
        case B2MOE_BF16: rows_to_f16_k<T, B2MOE_BF16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(x), rows, k, wide, out, inv); break;
        default: return B2MOE_ERR_SHAPE;
    }
    return launch_status();
}
int32_t convert_rows(uint32_t type, const void * x, int dtype, int rows, int k, __half * out, float * inv, cudaStream_t s) {
    switch (type) {
        case T_Q4_K: return convert_rows_t<T_Q4_K>(x, dtype, rows, k, out, inv, s);
        case T_IQ3_S: return convert_rows_t<T_IQ3_S>(x, dtype, rows, k, out, inv, s);
        case T_IQ3S4: return convert_rows_t<T_IQ3S4>(x, dtype, rows, k, out, inv, s);
        case T_IQ4_XS: return convert_rows_t<T_IQ4_XS>(x, dtype, rows, k, out, inv, s);
        case T_IQ4_NL: return convert_rows_t<T_IQ4_NL>(x, dtype, rows, k, out, inv, s);
        case T_NVFP4G: return convert_rows_t<T_NVFP4G>(x, dtype, rows, k, out, inv, s);
    }
    return B2MOE_ERR_FORMAT;
}

}  // namespace

void gemm_tc_item_tokens(int tokens) { g_item_tokens = tokens == 256 ? 256 : 128; }
// true when the tensor-core GEMM takes banks of this type with rows of length k (nmat: 2 = gate/up, 1 = down)
bool gemm_tc_supported(uint32_t type, int k, int nmat, int experts) {
    (void)nmat;                                                       // both products stage two row blocks per item
    return k >= G_KS && k % G_KS == 0 && gemm_smem_of(type, experts) <= GEMM_SMEM_LIMIT;
}
// scratch: the scaled fp16 copy of `rows_x` activation rows of length k and one float per row
size_t gemm_tc_workspace_bytes(int rows_x, int k) {
    return align_up(size_t(rows_x) * k * 2, 256) + align_up(size_t(rows_x) * sizeof(float), 256);
}

int32_t gemm_tc_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x,
                       int x_dtype, const int * plan, int n, int topk, int shared_tokens, float * act, void * ws, cudaStream_t s) {
    const int k = gate->cols;
    __half * xb = static_cast<__half *>(ws);
    float * inv = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + align_up(size_t(n) * k * 2, 256));
    if (int32_t rc = convert_rows(gate->type, x, x_dtype, n, k, xb, inv, s)) return rc;
    GemmArgs a{};
    a.w0 = static_cast<const uint8_t *>(gate->data); a.w1 = static_cast<const uint8_t *>(up->data);
    a.aux0 = static_cast<const float *>(gate->aux); a.aux1 = static_cast<const float *>(up->aux);
    if (shared_tokens) {
        a.s0 = static_cast<const uint8_t *>(sg->data); a.s1 = static_cast<const uint8_t *>(su->data);
        a.saux0 = static_cast<const float *>(sg->aux); a.saux1 = static_cast<const float *>(su->aux);
    }
    a.bank_bytes = b2moe_bank_bytes(gate->type, gate->rows, gate->cols);
    a.xb = xb; a.inv_scale = inv; a.plan = const_cast<int *>(plan); a.out = act;
    a.rows = gate->rows; a.k = k; a.experts = gate->experts; a.topk = topk; a.A = n * topk;
    return gemm_launch<0>(gate->type, a, s);
}

int32_t gemm_tc_down(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk,
                     int shared_tokens, float * y, void * ws, cudaStream_t s) {
    const int rows_x = n * topk + shared_tokens, k = down->cols;
    __half * xb = static_cast<__half *>(ws);
    float * inv = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + align_up(size_t(rows_x) * k * 2, 256));
    if (int32_t rc = convert_rows(down->type, act, B2MOE_F32, rows_x, k, xb, inv, s)) return rc;
    GemmArgs a{};
    a.w0 = static_cast<const uint8_t *>(down->data);
    a.aux0 = static_cast<const float *>(down->aux);
    if (shared_tokens) { a.s0 = static_cast<const uint8_t *>(sd->data); a.saux0 = static_cast<const float *>(sd->aux); }
    a.bank_bytes = b2moe_bank_bytes(down->type, down->rows, down->cols);
    a.xb = xb; a.inv_scale = inv; a.plan = const_cast<int *>(plan); a.out = y;
    a.rows = down->rows; a.k = k; a.experts = down->experts; a.topk = topk; a.A = n * topk;
    return gemm_launch<1>(down->type, a, s);
}

}  // namespace b2
