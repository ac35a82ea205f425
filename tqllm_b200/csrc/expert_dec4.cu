// Grouped expert products for banks of 4-bit codes when every expert sees only a few tokens: the bandwidth-bound
// decode kernels of Q4_K and of IQ3_S held as 4-bit codes (formats.cuh, Fmt<T_IQ3S4>).
// Replaces u4h_matvec_k<..., GROUPED> with its paired gate/up and dedup variants
// (src/formats/weight/quant_u4h.inc:424-604, launchers src/formats/weight/quant.cu:69-233) and the separate SwiGLU
// pass (src/experts/moe.cu:188-195).
//
// Arithmetic. A weight of a 32-weight sub-block is an affine function of its 4-bit code n with constants of the (row,
// sub-block): Q4_K  d sc n - dmin m;  IQ3_S  d (1 + 2 s) (2 n - 15). The activations are brought to 16-bit fixed point
// per row (a power-of-two scale; 14 or 15 significant bits) and split into a signed high and an unsigned low byte, so
// that  sum_k n_k x_k  is two integer tensor-core products per sub-block (mma.m16n8k32, u8 x s8 and u8 x u8 -> s32: the
// masked code words ARE the A fragment, no conversion) and every sum up to the end of a 256-column tile is an exact
// integer: the 6-bit / 4-bit sub-block scales multiply as integers, and the offset terms (- dmin m, - 15 d (1 + 2 s))
// times the activation sum of each sub-block, which the staging kernel takes once per activation row, are one more
// small MMA per tile (fp16 operands that hold the integer factors and the sums exactly). Two fp32 multiply-adds per
// tile and accumulator apply d / dmin. The only rounding that matters is that of the activations to fixed point
// (absolute error <= 2^-15 of the row's largest magnitude).
//
// Work. One resident block per SM: 16 consumer warps and one producer warp. A job = (pass of up to 8 tokens of one active
// expert, 16-row tile); the pass-major list of all jobs of the launch is cut into one contiguous share per block, equal
// to within a job, which the block walks as segments (runs of row tiles of one pass). Consumer warp w multiplies every
// 16th row tile of a segment; lane w of the producer warp is its feeder: it streams the tiles warp w will read, in
// order, over the whole share, through that warp's own ring of bulk copies (cp.async.bulk + mbarrier, no multicast;
// a full and an empty barrier per slot), so the ring never drains between jobs or segments. Lanes 16 .. 23 of the
// producer copy the staged activation rows of a segment's tokens into one of two shared buffers, one segment ahead, and
// leave each token column's assignment index and inverse scale beside them (the consumers' loop touches no global
// memory but its stores); the consumers hand a buffer back through a barrier of their own, so no block-wide barrier
// sits in the loop.
// Small launches (a few row jobs per block, known from the call's shape): 2 or 4 consumer warps share a row job, each
// taking a part of its columns, and meet in shared memory where the first of them adds the parts in a fixed order; the
// down product then also has one more warp that stages its fp32 activation rows itself (no staging launch).
// Every wait is bounded; a wait that runs out sets the plan's status word and a block-wide flag, every warp stops at
// its next wait or item, the producer lets the copies in flight land, and the block leaves.
#include "common.cuh"
#include "dec4_stage.cuh"
#include "formats.cuh"

namespace b2 {
namespace {

constexpr int CTA_WARPS = 16;
constexpr int XPAD = 64;             // bytes added to an activation row in shared memory (bank spread)
constexpr int MAX_STAGES = 4;
constexpr int MAX_SLOT_TILES = 2;    // consecutive column tiles of one matrix per ring slot and bulk copy (1 or 2): an SM sustains its share of
                                     // the HBM bandwidth with a few dozen large copies in flight, and loses half of it beyond about 64 copies
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// try_wait suspends the thread for a hardware-chosen time while the phase is pending: the fast path of every wait
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint32_t h2u(__half2 v) { return *reinterpret_cast<const uint32_t *>(&v); }
__device__ __forceinline__ __half2 u2h(uint32_t v) { return *reinterpret_cast<const __half2 *>(&v); }
// m16n8k16 fp16 MMA from zero (the offset-correction product of a tile)
__device__ __forceinline__ void mma_f16_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// m16n8k32 integer MMA, A unsigned bytes, B signed (SB = 1) or unsigned (SB = 0) bytes, C = 0
template <int SB>
__device__ __forceinline__ void mma_i8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (SB)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// Activation staging (layout and row code: dec4_stage.cuh): a warp per row, four rows per block.
constexpr int STAGE_WARPS = 4;
__global__ void __launch_bounds__(STAGE_WARPS * 32) dec4_stage_k(const void * __restrict__ x, int dtype, int rows, int k, int bits,
                                                                 uint8_t * __restrict__ out, float * __restrict__ inv_scale) {
    const int lane = threadIdx.x & 31, row = blockIdx.x * STAGE_WARPS + (threadIdx.x >> 5);
    grid_release();
    grid_wait();
    if (row < rows) stage_row_warp(x, dtype, row, k, bits, out, inv_scale, lane);
}

// ---------------------------------------------------------------------------------------------------------------
// Per-format pieces. A lane L = 4 g + t owns rows g, g + 8; of plane p (sub-blocks 2p, 2p + 1) it holds the words
// {row g: wa, wb; row g + 8: wa, wb}: wa = codes of weights 4t .. 4t + 3, wb = of weights 16 + 4t .. 16 + 4t + 3, low
// nibbles sub-block 2p, high nibbles sub-block 2p + 1: masked, the four words ARE the A fragment of the m16n8k32 MMA.
// A weight is (per row and sub-block)  Q4_K: d (sc n) - dmin (m);  IQ3_S codes: d (1 + 2 s) (2 n - 15). With integer
// activations the tile's sums stay integers:  main = sum_sb isc_sb * sum_k n_k x_k  and  corr = sum_sb ico_sb * S_sb
// (isc = sc | 1 + 2 s, ico = m | 1 + 2 s, S_sb = sum_k x_k), then one fp32 step per tile:
// acc += f_main * main + f_corr * corr  with (f_main, f_corr) = (d, -dmin) | (2 d, -15 d).
// Hdr::isc[r][h]: the integer scales of row g + 8 r, byte q = sub-block 2 q + h. Hdr::ico[r]: the correction factors of
// sub-block t in rows g / g + 8 and of sub-block t + 4 as fp16 pairs (ico, ico): the A fragment of the correction MMA (Hdr4::ca).
// BITS: width of the fixed-point activations, chosen so that `main` cannot overflow 32 bits (32 * 15 * 2^(BITS-1) *
// max isc * 8 sub-blocks < 2^31).
// ---------------------------------------------------------------------------------------------------------------
template <uint32_t T> struct D4;
struct Hdr4 { uint32_t isc[2][2], ca[4]; float f_main[2], f_corr[2]; };
// the byte of `word` that `sel` names, as the fp16 pair (v, v): 0x64 above a byte is the fp16 1024 + byte
__device__ __forceinline__ uint32_t byte_h2(uint32_t word, uint32_t sel) {
    return h2u(__hsub2(u2h(__byte_perm(word, 0x64646464u, sel)), __float2half2_rn(1024.f)));
}

template <> struct D4<T_Q4_K> {
    static constexpr int TILE = 2304, BITS = 15, FLUSH_AT = 1;   // scales up to 63: two halves of a tile stay inside 32 bits
    __device__ __forceinline__ static void load(Hdr4 & h, const uint8_t * tile, int lane) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 q = *reinterpret_cast<const uint4 *>(tile + 2048 + 16 * (g + 8 * r));   // d, dmin | scales[12]
            h.f_main[r] = __half2float(__ushort_as_half((unsigned short)(q.x & 0xffffu)));
            h.f_corr[r] = -64.f * __half2float(__ushort_as_half((unsigned short)(q.x >> 16)));   // the correction product carries S / 64
            // the 6-bit fields of sub-blocks 0..3 and 4..7 as bytes (src/formats/weight/dequant.cpp:56-64), four at a time
            const uint32_t sc03 = q.y & 0x3F3F3F3Fu, mn03 = q.z & 0x3F3F3F3Fu;
            const uint32_t sc47 = (q.w & 0x0F0F0F0Fu) | ((q.y >> 2) & 0x30303030u), mn47 = ((q.w >> 4) & 0x0F0F0F0Fu) | ((q.z >> 2) & 0x30303030u);
            h.isc[r][0] = __byte_perm(sc03, sc47, 0x6420);    // sub-blocks 0, 2, 4, 6
            h.isc[r][1] = __byte_perm(sc03, sc47, 0x7531);    // sub-blocks 1, 3, 5, 7
            const uint32_t sel = 0x4040u | (uint32_t(t) * 0x0101u);           // byte t twice, 0x64 above each
            h.ca[r] = byte_h2(mn03, sel);                     // min of sub-block t
            h.ca[2 + r] = byte_h2(mn47, sel);                 // of sub-block t + 4
        }
    }
};

template <> struct D4<T_IQ3S4> {
    static constexpr int TILE = 2144, BITS = 15, FLUSH_AT = -1;  // scales up to 31: a whole tile stays inside 32 bits
    __device__ __forceinline__ static void load(Hdr4 & h, const uint8_t * tile, int lane) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t sc = *reinterpret_cast<const uint32_t *>(tile + 2048 + 4 * (g + 8 * r));
            const float d = __half2float(*reinterpret_cast<const __half *>(tile + 2112 + 2 * (g + 8 * r)));
            h.f_main[r] = 2.f * d;
            h.f_corr[r] = -960.f * d;                                         // -15 d, and the correction product carries S / 64
            h.isc[r][0] = ((sc & 0x0F0F0F0Fu) << 1) | 0x01010101u;          // 1 + 2 s of sub-blocks 0, 2, 4, 6
            h.isc[r][1] = ((sc >> 3) & 0x1E1E1E1Eu) | 0x01010101u;          // of sub-blocks 1, 3, 5, 7
            const uint32_t word = (t & 1) ? h.isc[r][1] : h.isc[r][0], sel = 0x4040u | (uint32_t(t >> 1) * 0x0101u);   // sub-block t: byte t / 2 of its word
            h.ca[r] = byte_h2(word, sel);
            h.ca[2 + r] = byte_h2(word, sel + 0x0202u);                       // sub-block t + 4: two bytes on
        }
    }
};

struct Dec4Args {
    const uint8_t * w0, * w1, * s0, * s1;   // stacked banks (gate, up | down, -) and the shared expert's
    size_t bank_bytes;
    const uint8_t * x;                       // MODE 0: staged activation rows [rows_x][staged_row_bytes(k)]
    const float * x_raw;                     // MODE 1: the fp32 activation rows [A + shared][k], staged inside the kernel
    const float * inv_scale;                 // [rows_x]
    int * plan;
    float * out;                             // [A + shared][rows]
    int rows, k_tiles, experts, topk, A, nbuf, stages, slot_tiles;
    int passes_bound;                        // host: an upper bound of the plan's pass count, from the call's shape
    int ksplit;                              // consumer warps that share one row job, each taking 1 / ksplit of its columns (1, 2 or 4)
    uint32_t wait_limit;
    int drop_tile;                           // test hook: the copy into ring slot use number drop_tile (per warp, counted from 0) is never issued; -1 = none
};

// bytes of one activation row in shared memory: the staged row, padded so that consecutive rows start 64 bytes apart
// modulo 128 (the 16-byte loads of two token columns then share no bank)
__host__ __device__ inline uint32_t xrow_bytes(int k) { return uint32_t((staged_row_bytes(k) + 127) / 128 * 128 + XPAD); }
__host__ __device__ inline size_t xs_bytes(int k, int nbuf) { return size_t(nbuf) * 8 * xrow_bytes(k); }
// what the consumers need to know about a segment's tokens, written by the producer beside the activation rows it copies:
// per token column the assignment index (-1 = no token) and the inverse activation scale
struct SegMeta { int col_a[PASS_TOKENS]; float col_is[PASS_TOKENS]; };
// barriers: full[warp][stage], empty[warp][stage], xfull[2], xempty[2]; then the abort flag; then SegMeta[2]; then the
// barriers of the split-column reduction: red_full[8], red_free[8] (one pair per group of warps that share a row job)
constexpr size_t BAR_BYTES = (2 * CTA_WARPS * MAX_STAGES + 4) * 8 + 16 + 2 * sizeof(SegMeta) + 16 * 8;
constexpr size_t RED_BYTES = size_t(CTA_WARPS) * 8 * 32 * sizeof(float);     // partial sums of every warp: [warp][8 accumulators][lane]
// 16 consumer warps + the producer warp; the STAGER instance of the down product (small launches) has one more warp that brings
// its activation rows (fp32, the gate/up product's output) into the staged form inside the kernel, a segment ahead of the
// consumers: no staging launch between the two products. A scheduler partition holds 16 K registers, so its five warps may take 96 each: the launch bound is given
// as 640 threads to make the compiler stay at 96 (65536 / 640 rounds down to it), whatever the block really has.
template <bool STAGER> constexpr int threads_of() { return (CTA_WARPS + (STAGER ? 2 : 1)) * 32; }
template <bool STAGER> constexpr int bound_threads() { return STAGER ? 640 : threads_of<false>(); }

// MODE 0: out = act[a][row] = silu(gate . x) * (up . x);   MODE 1: out = y[a][row] = down . act[a]
template <uint32_t T, int MODE, bool STAGER>
__global__ void __launch_bounds__(bound_threads<STAGER>(), 1) dec4_k(const Dec4Args p) {
    using F = D4<T>;
    constexpr int NMAT = MODE == 0 ? 2 : 1, TILE = F::TILE;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t * bars = reinterpret_cast<uint64_t *>(smem);
    volatile int * abort_flag = reinterpret_cast<volatile int *>(smem + (2 * CTA_WARPS * MAX_STAGES + 4) * 8);
    SegMeta * meta = reinterpret_cast<SegMeta *>(smem + (2 * CTA_WARPS * MAX_STAGES + 4) * 8 + 16);
    const uint32_t red_full = smem_addr(meta + 2), red_free = red_full + 64;
    const int SLOT_TILES = p.slot_tiles, SLOT = SLOT_TILES * TILE;
    uint8_t * ring = smem + BAR_BYTES;                                        // [warp][stage][SLOT]
    uint8_t * xs = ring + size_t(CTA_WARPS) * p.stages * SLOT;               // [buf][8 rows][xrow]
    float * red = reinterpret_cast<float *>(xs + xs_bytes(p.k_tiles * 256, p.nbuf));   // [warp][8][32], only when ksplit > 1
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = p.k_tiles * 256;
    const int e1 = p.experts + 1;
    const uint32_t xrow = xrow_bytes(K), xbuf = 8 * xrow, xglob = uint32_t(staged_row_bytes(K));
    const int S = p.stages, kslots = (p.k_tiles + SLOT_TILES - 1) / SLOT_TILES;                            // column slots of one row job
    // ksplit warps share a row job: warp w takes part w % ksplit of its column slots (ksplit divides kslots); JW jobs run side by side
    const int KSP = p.ksplit, JW = CTA_WARPS / KSP, kpart = kslots / KSP, nslots = kpart * NMAT;           // slots of one warp's part of a job
    const uint32_t full0 = smem_addr(bars), empty0 = full0 + 8 * CTA_WARPS * MAX_STAGES, xfull = empty0 + 8 * CTA_WARPS * MAX_STAGES,
                   xempty = xfull + 16, xs0 = smem_addr(xs);

    if (threadIdx.x < CTA_WARPS * MAX_STAGES) { mbar_init(full0 + 8 * threadIdx.x, 1); mbar_init(empty0 + 8 * threadIdx.x, 1); }
    if (threadIdx.x == 0) {
        mbar_init(xfull, 1); mbar_init(xfull + 8, 1);
        mbar_init(xempty, CTA_WARPS); mbar_init(xempty + 8, CTA_WARPS);
        for (int i = 0; i < 8; ++i) { mbar_init(red_full + 8 * i, uint32_t(p.ksplit)); mbar_init(red_free + 8 * i, 1); }
        *abort_flag = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    grid_wait();              // the plan and the staged rows come from the launches before this one: no global access above this line
    __syncthreads();

    const int * counts = p.plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    const int * passes = perm + p.A + counts[p.experts];     // the plan's own count of always-on rows (a range of the tokens under expert parallelism)
    const int na = p.plan[PLAN_NACTIVE], row_tiles = (p.rows + 15) >> 4;
    // the block's share of the launch: jobs [u_begin, u_end) of the pass-major list of (pass, row tile) jobs; it walks the
    // share as segments = runs of row tiles [r0, r1) of one pass
    const long long n_jobs = (long long)p.plan[PLAN_NPASS] * row_tiles;
    const long long u_begin = n_jobs * blockIdx.x / gridDim.x, u_end = n_jobs * (blockIdx.x + 1) / gridDim.x;
    auto segment = [&](long long u, int & pass, int & r0, int & r1) {
        pass = int(u / row_tiles);
        r0 = int(u - (long long)pass * row_tiles);
        r1 = int(min((long long)row_tiles, r0 + (u_end - u)));
    };

    // pass w -> (expert, first token slot); the pass list runs over the active experts from the last to the first. Called by
    // all lanes of the producer warp together: two rounds of 32 probes instead of a ten-step chain of dependent loads.
    auto locate = [&](int w, int & e, int & c0) {
        const int stride = (na + 31) >> 5;                                         // first round: every stride-th entry
        const int i1 = min(lane * stride, na - 1);
        const unsigned m1 = __ballot_sync(0xffffffffu, lane * stride < na && passes[i1] <= w);
        const int base = (31 - __clz(int(m1 | 1u))) * stride;                      // passes[0] = 0 <= w always
        int lo = base;
        for (int o = 0; o < stride; o += 32) {                                     // second round: the entries of that stretch
            const int i2 = base + o + lane;
            const unsigned m2 = __ballot_sync(0xffffffffu, i2 < min(na, base + stride) && passes[min(i2, na - 1)] <= w);
            if (m2) lo = base + o + 31 - __clz(int(m2));
        }
        e = active[na - 1 - lo];
        c0 = (w - passes[lo]) * PASS_TOKENS;
    };
    constexpr bool in_kernel = STAGER;                             // the down product stages its rows itself (small launches)
    auto x_row = [&](int a) { return MODE == 0 ? size_t(a < p.A ? a / p.topk : a - p.A) : size_t(a); };
    // a bounded wait that also gives up when another warp of the block has
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (mbar_try(bar, parity)) return true;
        for (uint32_t i = 0; i < p.wait_limit; ++i) {
            if (mbar_try(bar, parity)) return true;
            if ((i & 63) == 63 && *abort_flag) return false;
        }
        return false;
    };

    if (warp == CTA_WARPS) {
        // ---- producer: lane w < 16 feeds consumer warp w (its ring, its barriers); lanes 16 .. 23 copy the activation rows ----
        const int w = lane & (CTA_WARPS - 1);
        const uint32_t my_full = full0 + 8 * w * MAX_STAGES, my_empty = empty0 + 8 * w * MAX_STAGES, my_ring = smem_addr(ring) + uint32_t(w) * S * SLOT;
        uint32_t slot = 0, issued = 0, xissued = 0;
        bool ok = true;
        // known = the caller has already located this pass (e_in, c0_in)
        auto stage_x = [&](int pass, uint32_t idx, bool known = false, int e_in = 0, int c0_in = 0) {       // rows of the item with running index idx -> buffer idx % nbuf
            const uint32_t b = p.nbuf == 2 ? (idx & 1u) : 0u, use = p.nbuf == 2 ? idx >> 1 : idx;
            if (use > 0 && !wait(xempty + 8 * b, (use - 1) & 1u)) ok = false;     // the consumers are done with the buffer's previous rows
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            int e = e_in, c0 = c0_in;
            if (!known) locate(pass, e, c0);
            const int nv = min(PASS_TOKENS, counts[e] - c0);
            const int col = lane - 16;                                        // lanes 16 .. 23: one token column each
            int a = -1;
            if (col >= 0 && col < PASS_TOKENS) {
                if (col < nv) a = perm[offsets[e] + c0 + col];
                // the row's copy leaves first; its bytes count against the phase that lane 16's arrival below opens (the
                // transaction count may run ahead of the expectation; the phase cannot complete before that arrival)
                if (a >= 0) bulk_g2s(xs0 + b * xbuf + col * xrow, p.x + x_row(a) * xglob, xglob, xfull + 8 * b);
                meta[b].col_a[col] = a;
                meta[b].col_is[col] = a >= 0 ? p.inv_scale[x_row(a)] : 0.f;
            }
            __syncwarp();                                                     // the columns are written before lane 16's arrival publishes them
            if (lane == 16) mbar_expect_tx(xfull + 8 * b, uint32_t(nv) * xglob);
            ++xissued;
        };
        int pass, r0, r1;
        uint32_t idx = 0;
        bool first_staged = false;                         // the first segment's rows are asked for right after its first weight copies
        for (long long u = u_begin; u < u_end && ok; u += r1 - r0, ++idx) {
            segment(u, pass, r0, r1);
            int e, c0;
            locate(pass, e, c0);
            const bool shared = e == p.experts;
            const long long u_next = u + (r1 - r0);
            int npass = 0, nr0, nr1;
            if (u_next < u_end) segment(u_next, npass, nr0, nr1);
            bool next_staged = p.nbuf != 2 || u_next >= u_end;
            int in_seg = 0;
            for (int rb = r0; rb < r1 && ok; rb += JW) {                  // JW row tiles at a time, warp w its part of its own
                const int rt = rb + w / KSP, k_first = (w % KSP) * kpart;
                const bool mine = lane < CTA_WARPS && rt < r1;
                const uint8_t * b0 = (shared ? p.s0 : p.w0 + size_t(e) * p.bank_bytes) + size_t(rt) * p.k_tiles * TILE;
                const uint8_t * b1 = NMAT == 2 ? (shared ? p.s1 : p.w1 + size_t(e) * p.bank_bytes) + size_t(rt) * p.k_tiles * TILE : b0;
                for (int j = 0; j < nslots && ok; ++j, ++in_seg) {
                    if (mine) {
                        if (issued >= uint32_t(S) && !wait(my_empty + 8 * slot, ((issued / S) - 1) & 1u)) ok = false;
                        else if (int(issued) != p.drop_tile) {
                            const int ks = k_first + (NMAT == 2 ? j >> 1 : j);                       // slot of column tiles of the job
                            const uint8_t * src = ((NMAT == 2 && (j & 1)) ? b1 : b0) + size_t(ks) * SLOT;
                            const uint32_t bytes = uint32_t(min(SLOT_TILES, p.k_tiles - ks * SLOT_TILES)) * TILE;
                            mbar_expect_tx(my_full + 8 * slot, bytes);
                            bulk_g2s(my_ring + slot * SLOT, src, bytes, my_full + 8 * slot);
                        }
                        ++issued;
                        slot = slot + 1 == uint32_t(S) ? 0 : slot + 1;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!in_kernel && !first_staged) { stage_x(pass, 0, true, e, c0); first_staged = true; }
                    // once every consumer is S slots into this segment, the previous segment's buffer is free: bring the next one's rows
                    if (!in_kernel && !next_staged && in_seg == S) { stage_x(npass, idx + 1); next_staged = true; }
                }
            }
            if (!in_kernel && !next_staged && ok) stage_x(npass, idx + 1);
            if (!in_kernel && p.nbuf == 1 && u_next < u_end && ok) stage_x(npass, idx + 1);
        }
        if (!ok) { *abort_flag = 1; if (lane == 0) atomicExch(p.plan + PLAN_STATUS, 3); }
        // before leaving, every copy this lane issued must have landed: the last S slots of its ring (earlier ones were
        // consumed, or their slot could not have been reused) and the last activation buffers. After a clean run these
        // waits return at once.
        if (lane < CTA_WARPS) {
            const uint32_t first = issued > uint32_t(S) ? issued - S : 0;
            for (uint32_t i = first; i < issued; ++i)
                if (int(i) != p.drop_tile) wait(my_full + 8 * (i % S), (i / S) & 1u);
        }
        if (!in_kernel && lane == 16)       // the last copy into each activation buffer (an earlier phase of a barrier can no longer be waited for)
            for (uint32_t i = xissued > uint32_t(p.nbuf) ? xissued - p.nbuf : 0; i < xissued; ++i)
                wait(xfull + 8 * (p.nbuf == 2 ? (i & 1u) : 0u), (p.nbuf == 2 ? i >> 1 : i) & 1u);
    } else if (STAGER && warp == CTA_WARPS + 1) {
        {
        // ---- stager (down product): segment q's activation rows, fp32 in global memory -> staged form in buffer q % nbuf ----
        const int pass_first = u_begin < u_end ? int(u_begin / row_tiles) : 0;
        const int nseg = u_begin < u_end ? int((u_end - 1) / row_tiles) - pass_first + 1 : 0;
        bool ok = true;
        for (int q = 0; q < nseg && ok; ++q) {
            const uint32_t b = p.nbuf == 2 ? (uint32_t(q) & 1u) : 0u, use = p.nbuf == 2 ? uint32_t(q) >> 1 : uint32_t(q);
            if (use > 0 && !__all_sync(0xffffffffu, wait(xempty + 8 * b, (use - 1) & 1u))) { ok = false; break; }   // the consumers are done with the buffer
            int e, c0;
            locate(pass_first + q, e, c0);
            const int nv = min(PASS_TOKENS, counts[e] - c0);
            const int mine = lane < nv ? perm[offsets[e] + c0 + lane] : -1;
            for (int col = 0; col < PASS_TOKENS; ++col) {
                const int a = __shfl_sync(0xffffffffu, mine, col);
                float inv = 0.f;
                if (a >= 0) inv = stage_row_lanes<B2MOE_F32>(p.x_raw, size_t(a) * K, K, F::BITS, xs + b * xbuf + col * xrow, lane);
                if (lane == 0) { meta[b].col_a[col] = a; meta[b].col_is[col] = inv; }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(xfull + 8 * b);
        }
        if (!ok) { *abort_flag = 1; if (lane == 0) atomicExch(p.plan + PLAN_STATUS, 3); }
        }
    } else {
        // ---- consumers ----
        const int g = lane >> 2, t = lane & 3;
        const uint8_t * my_ring = ring + size_t(warp) * S * SLOT;
        const uint32_t my_full = full0 + 8 * warp * MAX_STAGES, my_empty = empty0 + 8 * warp * MAX_STAGES;
        uint32_t c_slot = 0, c_phase = 0, red_use = 0;
        bool alive = true;
        int pass, r0, r1;
        uint32_t idx = 0;
        for (long long u = u_begin; u < u_end && alive; u += r1 - r0, ++idx) {
            segment(u, pass, r0, r1);
            const uint32_t b = p.nbuf == 2 ? (idx & 1u) : 0u, use = p.nbuf == 2 ? idx >> 1 : idx;
            if (*abort_flag) break;
            if (!__all_sync(0xffffffffu, wait(xfull + 8 * b, use & 1u))) { alive = false; break; }
            const uint8_t * xw = xs + b * xbuf + g * xrow + t * 16;          // + sub-block * 64
            const uint8_t * rec = xs + b * xbuf + g * xrow + size_t(K) * 2 + t * 8;   // + tile * 32
            // the lane's two token columns (2t, 2t + 1): assignment index and inverse activation scale, as the producer left them
            int col_a[2];
            float col_is[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) { col_a[q] = meta[b].col_a[2 * t + q]; col_is[q] = meta[b].col_is[2 * t + q]; }

            const int grp = warp / KSP, part = warp % KSP;                  // row-job slot of this warp and its part of the columns
            for (int rt = r0 + grp; rt < r1 && alive; rt += JW) {
                float acc[NMAT][4];
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;

                for (int ks = part * kpart; ks < (part + 1) * kpart && alive; ++ks) {
                    const int nt = min(SLOT_TILES, p.k_tiles - ks * SLOT_TILES);
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        if (!__all_sync(0xffffffffu, wait(my_full + 8 * c_slot, c_phase))) { alive = false; break; }
                        for (int kk = 0; kk < nt; ++kk) {
                            const int kt = ks * SLOT_TILES + kk;
                            const uint8_t * tile = my_ring + c_slot * SLOT + kk * TILE;
                            // the sub-block sums of this tile's columns: B fragment of the correction MMA
                            const uint2 sp = *reinterpret_cast<const uint2 *>(rec + kt * 32);
                            const uint4 * xk = reinterpret_cast<const uint4 *>(xw + kt * 512);
                            Hdr4 hdr;
                            F::load(hdr, tile, lane);
                            int main_[4] = {0, 0, 0, 0};
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const uint4 pl = reinterpret_cast<const uint4 *>(tile + 512 * q)[lane];
#pragma unroll
                                for (int half = 0; half < 2; ++half) {                     // sub-block 2q (low nibbles), 2q + 1 (high nibbles)
                                    const uint32_t a0 = (half ? pl.x >> 4 : pl.x) & 0x0F0F0F0Fu, a2 = (half ? pl.y >> 4 : pl.y) & 0x0F0F0F0Fu;
                                    const uint32_t a1 = (half ? pl.z >> 4 : pl.z) & 0x0F0F0F0Fu, a3 = (half ? pl.w >> 4 : pl.w) & 0x0F0F0F0Fu;
                                    const uint4 xv = xk[(2 * q + half) * 4];             // dead token columns read stale rows: they feed dead C columns only
                                    int rh[4], rl[4];
                                    mma_i8<1>(rh, a0, a1, a2, a3, xv.x, xv.y);             // high bytes of the activations (signed)
                                    mma_i8<0>(rl, a0, a1, a2, a3, xv.z, xv.w);             // low bytes (unsigned)
                                    const int s0 = int(__byte_perm(hdr.isc[0][half], 0u, 0x4440 + q)), s8 = int(__byte_perm(hdr.isc[1][half], 0u, 0x4440 + q));
                                    main_[0] += s0 * (rh[0] * 256 + rl[0]); main_[1] += s0 * (rh[1] * 256 + rl[1]);
                                    main_[2] += s8 * (rh[2] * 256 + rl[2]); main_[3] += s8 * (rh[3] * 256 + rl[3]);
                                }
                                if (F::FLUSH_AT == q) {      // keep `main` inside 32 bits: hand the first half of the tile over now
#pragma unroll
                                    for (int i = 0; i < 4; ++i) { acc[m][i] = fmaf(hdr.f_main[i >> 1], float(main_[i]), acc[m][i]); main_[i] = 0; }
                                }
                            }
                            float corr[4];
                            mma_f16_zero(corr, hdr.ca[0], hdr.ca[1], hdr.ca[2], hdr.ca[3], sp.x, sp.y);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                acc[m][i] = fmaf(hdr.f_main[i >> 1], float(main_[i]), fmaf(hdr.f_corr[i >> 1], corr[i], acc[m][i]));
                        }
                        __syncwarp();             // every lane has read its words: the slot can be refilled
                        if (lane == 0) mbar_arrive(my_empty + 8 * c_slot);
                        c_slot = c_slot + 1 == uint32_t(S) ? 0 : c_slot + 1;
                        c_phase ^= c_slot == 0 ? 1u : 0u;
                    }
                }
                if (!alive) break;
                if (KSP > 1) {
                    // the parts of the row job meet in shared memory: every warp leaves its sums, part 0 adds them in part order
                    // (the same bits every run) and carries on alone. red_use counts this group's jobs of the whole launch.
                    float * mine = red + size_t(warp) * 8 * 32;
                    if (part != 0) {
                        if (red_use > 0 && !__all_sync(0xffffffffu, wait(red_free + 8 * grp, (red_use - 1) & 1u))) { alive = false; break; }
#pragma unroll
                        for (int m = 0; m < NMAT; ++m)
#pragma unroll
                            for (int i = 0; i < 4; ++i) mine[(m * 4 + i) * 32 + lane] = acc[m][i];
                        __syncwarp();
                        if (lane == 0) mbar_arrive(red_full + 8 * grp);
                        ++red_use;
                        continue;
                    }
                    if (lane == 0) mbar_arrive(red_full + 8 * grp);
                    if (!__all_sync(0xffffffffu, wait(red_full + 8 * grp, red_use & 1u))) { alive = false; break; }
                    for (int o = 1; o < KSP; ++o)
#pragma unroll
                        for (int m = 0; m < NMAT; ++m)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[m][i] += red[size_t(warp + o) * 8 * 32 + (m * 4 + i) * 32 + lane];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(red_free + 8 * grp);
                    ++red_use;
                }
                // epilogue: the lane holds rows g, g + 8 x token columns 2t, 2t + 1
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int a = col_a[q];
                    if (a < 0) continue;
                    const float is = col_is[q];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = 16 * rt + g + 8 * h;
                        if (row >= p.rows) continue;
                        const float v0 = acc[0][2 * h + q] * is, v1 = acc[NMAT - 1][2 * h + q] * is;
                        p.out[size_t(a) * p.rows + row] = MODE == 0 ? (v0 / (1.f + expf(-v0))) * v1 : v0;
                    }
                }
            }
            if (!alive) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(xempty + 8 * b);      // this warp is done with the item's activation rows
        }
        if (!alive) { *abort_flag = 1; if (lane == 0) atomicExch(p.plan + PLAN_STATUS, 3); }
    }
    grid_release();           // only now: a launch that became resident earlier would share this SM's issue slots for the whole kernel
    __syncthreads();          // nobody leaves while a copy into the block's shared memory may be in flight
}

int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}
constexpr size_t SMEM_LIMIT = 232448 - 1024;

template <uint32_t T> size_t dec4_smem(int k, int nbuf, int stages, int slot_tiles) {
    return BAR_BYTES + size_t(CTA_WARPS) * stages * slot_tiles * D4<T>::TILE + xs_bytes(k, nbuf);
}
// (activation buffers, ring stages, tiles per slot) in order of preference, the first that fits: large copies first (measured:
// two-tile slots with one activation buffer beat one-tile slots with two), then two activation buffers (the next segment's
// rows arrive while this one is multiplied), then a deeper ring
int g_ring[3] = {0, 0, 0};            // test hook: (activation buffers, stages, tiles per slot) forced, 0 = the first that fits
template <uint32_t T> bool dec4_fit(int k, int & nbuf, int & stages, int & slot_tiles) {
    if (g_ring[0] >= 1 && g_ring[0] <= 2 && g_ring[1] >= 2 && g_ring[1] <= MAX_STAGES && g_ring[2] >= 1 && g_ring[2] <= MAX_SLOT_TILES &&
        dec4_smem<T>(k, g_ring[0], g_ring[1], g_ring[2]) <= SMEM_LIMIT) {
        nbuf = g_ring[0]; stages = g_ring[1]; slot_tiles = g_ring[2];
        return true;
    }
    const int opts[6][3] = {{2, 3, 2}, {2, 2, 2}, {1, 3, 2}, {1, 2, 2}, {2, 3, 1}, {1, 3, 1}};
    for (const auto & o : opts)
        if (dec4_smem<T>(k, o[0], o[1], o[2]) <= SMEM_LIMIT) { nbuf = o[0]; stages = o[1]; slot_tiles = o[2]; return true; }
    return false;
}

int g_ksplit_max = 4;                 // test hook: 1 switches the column split of small launches off
int g_drop_tile = -1;                 // test hooks (b2moe_harness_wait_probe, b2moe_harness_skip_staging)
bool g_skip_stage = false;
uint32_t g_wait_limit = WAIT_LIMIT;

template <uint32_t T, int MODE, bool STAGER = false>
int32_t launch_dec4(Dec4Args a, cudaStream_t s) {
    const int sms = sm_count(), k = a.k_tiles * 256;
    if (sms <= 0) return B2MOE_ERR_CUDA;
    if (!dec4_fit<T>(k, a.nbuf, a.stages, a.slot_tiles)) return B2MOE_ERR_SHAPE;
    // When the launch cannot have more than a few row jobs per block (a handful of tokens), 2 or 4 warps share a job, each
    // taking a part of its columns: a job is then a chain of kslots / ksplit copies instead of kslots. The bound comes from
    // the call's shape (every pass holds at least one assignment), never from the plan, so a captured launch keeps it.
    const int kslots = (a.k_tiles + a.slot_tiles - 1) / a.slot_tiles;
    const long long jobs_bound = (long long)a.passes_bound * ((a.rows + 15) / 16), per_block = (jobs_bound + sms - 1) / sms;
    a.ksplit = 1;
    for (int ks = 4; ks >= 2; ks >>= 1)
        if (per_block <= CTA_WARPS / ks && kslots % ks == 0 && g_ksplit_max >= ks &&
            dec4_smem<T>(k, a.nbuf, a.stages, a.slot_tiles) + RED_BYTES <= SMEM_LIMIT) { a.ksplit = ks; break; }
    const size_t smem = dec4_smem<T>(k, a.nbuf, a.stages, a.slot_tiles) + (a.ksplit > 1 ? RED_BYTES : 0);
    if (cudaFuncSetAttribute(dec4_k<T, MODE, STAGER>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return B2MOE_ERR_CUDA;
    a.wait_limit = g_wait_limit;
    a.drop_tile = g_drop_tile;
    launch_overlapped(dec4_k<T, MODE, STAGER>, dim3(sms), dim3(threads_of<STAGER>()), smem, s, a);       // every block takes an equal share of the (pass, row tile) jobs
    return launch_status();
}

template <uint32_t T>
int32_t stage(Dec4Args & a, const void * x, int dtype, int rows_x, int k, void * ws, cudaStream_t s, bool already = false) {
    uint8_t * w = static_cast<uint8_t *>(ws);
    float * inv = reinterpret_cast<float *>(w + staged_bytes(rows_x, k));
    a.x = w; a.inv_scale = inv;
    if (already) return B2MOE_OK;            // an earlier launch of the caller wrote the staged rows (route_plan_stage)
    if (g_skip_stage) return B2MOE_OK;       // the workspace still holds the staged rows of the previous call (benchmarks: the product alone)
    launch_overlapped(dec4_stage_k, dim3((rows_x + STAGE_WARPS - 1) / STAGE_WARPS), dim3(STAGE_WARPS * 32), 0, s, x, dtype, rows_x, k, int(D4<T>::BITS), w, inv);
    return launch_status();
}

template <uint32_t T>
int32_t gateup_t(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x, int x_dtype,
                 const int * plan, int n, int topk, int shared_tokens, float * act, void * ws, int max_active, cudaStream_t s, bool x_staged) {
    const int k = gate->cols;
    Dec4Args a{};
    if (int32_t rc = stage<T>(a, x, x_dtype, n, k, ws, s, x_staged)) return rc;
    a.w0 = static_cast<const uint8_t *>(gate->data); a.w1 = static_cast<const uint8_t *>(up->data);
    if (shared_tokens) { a.s0 = static_cast<const uint8_t *>(sg->data); a.s1 = static_cast<const uint8_t *>(su->data); }
    a.bank_bytes = b2moe_bank_bytes(gate->type, gate->rows, gate->cols);
    a.plan = const_cast<int *>(plan); a.out = act;
    a.rows = gate->rows; a.k_tiles = k / 256; a.experts = gate->experts; a.topk = topk; a.A = n * topk;
    a.passes_bound = n * topk + (shared_tokens + PASS_TOKENS - 1) / PASS_TOKENS;
    return launch_dec4<T, 0>(a, s);
}
template <uint32_t T>
int32_t down_t(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk, int shared_tokens,
               float * y, void * ws, int max_active, cudaStream_t s) {
    const int rows_x = n * topk + shared_tokens, k = down->cols;
    Dec4Args a{};
    // A launch of a few jobs per block is a chain of latencies: its rows are staged inside the kernel by a warp of their own
    // (one launch less). A full launch keeps the staging kernel: measured at 64 tokens the in-kernel staging costs 11 us more
    // than the launch it saves (the staging warp shares a scheduler with five busy warps).
    const long long jobs_bound = (long long)(n * topk + (shared_tokens + PASS_TOKENS - 1) / PASS_TOKENS) * ((down->rows + 15) / 16);
    const int sms = sm_count();
    const bool in_kernel = sms > 0 && jobs_bound <= 24LL * sms && !g_skip_stage;
    if (in_kernel) a.x_raw = act;
    else if (int32_t rc = stage<T>(a, act, B2MOE_F32, rows_x, k, ws, s)) return rc;
    a.w0 = static_cast<const uint8_t *>(down->data);
    if (shared_tokens) a.s0 = static_cast<const uint8_t *>(sd->data);
    a.bank_bytes = b2moe_bank_bytes(down->type, down->rows, down->cols);
    a.plan = const_cast<int *>(plan); a.out = y;
    a.rows = down->rows; a.k_tiles = k / 256; a.experts = down->experts; a.topk = topk; a.A = n * topk;
    a.passes_bound = n * topk + (shared_tokens + PASS_TOKENS - 1) / PASS_TOKENS;
    return in_kernel ? launch_dec4<T, 1, true>(a, s) : launch_dec4<T, 1>(a, s);
}

}  // namespace

// true when the 4-bit decode kernels take banks of this type with rows of length k
bool dec4_supported(uint32_t type, int k) {
    int nbuf, stages, st;
    if (k <= 0 || k % 256) return false;
    if (type == T_Q4_K) return dec4_fit<T_Q4_K>(k, nbuf, stages, st);
    if (type == T_IQ3S4) return dec4_fit<T_IQ3S4>(k, nbuf, stages, st);
    return false;
}
// scratch: the staged form of `rows_x` activation rows of length k and one float per row
size_t dec4_workspace_bytes(int rows_x, int k) {
    return staged_bytes(rows_x, k) + align_up(size_t(rows_x) * sizeof(float), 256);
}
int32_t dec4_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x,
                    int x_dtype, const int * plan, int n, int topk, int shared_tokens, float * act, void * ws, int max_active,
                    cudaStream_t s, bool x_staged) {
    if (gate->type == T_Q4_K) return gateup_t<T_Q4_K>(gate, up, sg, su, x, x_dtype, plan, n, topk, shared_tokens, act, ws, max_active, s, x_staged);
    if (gate->type == T_IQ3S4) return gateup_t<T_IQ3S4>(gate, up, sg, su, x, x_dtype, plan, n, topk, shared_tokens, act, ws, max_active, s, x_staged);
    return B2MOE_ERR_FORMAT;
}
int32_t dec4_down(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk,
                  int shared_tokens, float * y, void * ws, int max_active, cudaStream_t s) {
    if (down->type == T_Q4_K) return down_t<T_Q4_K>(down, sd, act, plan, n, topk, shared_tokens, y, ws, max_active, s);
    if (down->type == T_IQ3S4) return down_t<T_IQ3S4>(down, sd, act, plan, n, topk, shared_tokens, y, ws, max_active, s);
    return B2MOE_ERR_FORMAT;
}
void dec4_skip_staging(bool on) { g_skip_stage = on; }
void dec4_ring(int nbuf, int stages, int slot_tiles) { g_ring[0] = nbuf; g_ring[1] = stages; g_ring[2] = slot_tiles; }
void dec4_ksplit_max(int ks) { g_ksplit_max = ks < 1 ? 1 : ks; }
// where dec4_gateup expects the staged form of n activation rows of length k inside its workspace, and with how many bits
void dec4_stage_target(uint32_t type, void * ws, int n, int k, uint8_t ** rows, float ** inv_scale, int * bits) {
    *rows = static_cast<uint8_t *>(ws);
    *inv_scale = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + staged_bytes(n, k));
    *bits = type == T_Q4_K ? D4<T_Q4_K>::BITS : D4<T_IQ3S4>::BITS;
}
void dec4_debug(int drop_tile, uint32_t wait_limit) {
    g_drop_tile = drop_tile;
    g_wait_limit = wait_limit ? wait_limit : WAIT_LIMIT;
}

}  // namespace b2
