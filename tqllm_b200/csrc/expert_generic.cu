// Grouped expert products, format-generic path: every format and every shape, fp32 weights decoded exactly as the
// host reference decodes them (formats.cuh) and fp32 sums taken in ascending column order like moe_expert_ffn
// (src/experts/moe.cpp:115-155). It is the correctness floor under the tuned per-format kernels and serves the
// shapes those do not cover. One block owns (active expert, 16-row tile), walks the expert's tokens 16 at a time
// and the columns one bank tile at a time: decode tile(s) -> shared memory, stage the token rows, multiply.
#include "common.cuh"
#include "formats.cuh"

namespace b2 {
int32_t check_bank(const b2moe_bank * b);

namespace {

constexpr int NT = 16;   // tokens per pass

struct GroupArgs {
    const uint8_t * w0, * w1;        // stacked banks (gate, up) or (down, -)
    const uint8_t * s0, * s1;        // the shared expert's banks (may be null)
    const float * aux0, * aux1, * saux0, * saux1;
    size_t bank_bytes;               // bytes of one expert's matrix
    int rows, cols, experts, topk, A;
    int k_tiles, units;
};

// MODE 0: act[a][r] = silu(gate_r . x_tok(a)) * (up_r . x_tok(a));  MODE 1: y[a][r] = down_r . act[a]
template <uint32_t T, int MODE>
__global__ void __launch_bounds__(256) expert_generic_k(GroupArgs g, const void * __restrict__ x, int x_dtype,
                                                        const int * __restrict__ plan, float * __restrict__ out) {
    constexpr int KT = Fmt<T>::KT, LDX = KT + 1;
    extern __shared__ float sm[];
    float * w0 = sm, * w1 = w0 + 16 * KT, * xs = w0 + (MODE == 0 ? 2 : 1) * 16 * KT;
    __shared__ float aux[2][16];
    __shared__ int toks[NT];
    const int e1 = g.experts + 1;
    const int * counts = plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    if (int(blockIdx.y) >= plan[PLAN_NACTIVE]) return;
    const int e = active[blockIdx.y], cnt = counts[e], off = offsets[e], rt = blockIdx.x;
    const bool shared = e == g.experts;
    const int row_tiles = gridDim.x;
    const uint8_t * b0 = (shared ? g.s0 : g.w0 + size_t(e) * g.bank_bytes) + size_t(rt) * g.k_tiles * Fmt<T>::TILE;
    const uint8_t * b1 = MODE == 0 ? (shared ? g.s1 : g.w1 + size_t(e) * g.bank_bytes) + size_t(rt) * g.k_tiles * Fmt<T>::TILE : nullptr;
    if (threadIdx.x < 32) {
        const int which = threadIdx.x >> 4, r = threadIdx.x & 15;
        const float * a = which ? (shared ? g.saux1 : g.aux1) : (shared ? g.saux0 : g.aux0);
        aux[which][r] = a ? a[(size_t(shared ? 0 : e) * row_tiles + rt) * 16 + r] : 0.f;
    }
    const int r = threadIdx.x >> 4, c = threadIdx.x & 15;
    for (int c0 = 0; c0 < cnt; c0 += NT) {
        __syncthreads();
        if (threadIdx.x < NT) toks[threadIdx.x] = c0 + threadIdx.x < cnt ? perm[off + c0 + threadIdx.x] : -1;
        float acc0 = 0.f, acc1 = 0.f;
        for (int kt = 0; kt < g.k_tiles; ++kt) {
            __syncthreads();
            decode_tile<T>(b0 + size_t(kt) * Fmt<T>::TILE, aux[0], w0, KT, threadIdx.x, blockDim.x, g.units);
            if (MODE == 0) decode_tile<T>(b1 + size_t(kt) * Fmt<T>::TILE, aux[1], w1, KT, threadIdx.x, blockDim.x, g.units);
            for (int i = threadIdx.x; i < NT * KT; i += blockDim.x) {
                const int tc = i / KT, k = i % KT, a = toks[tc];
                float v = 0.f;
                if (a >= 0) {
                    if (MODE == 0) v = load_act(x, x_dtype, size_t(a < g.A ? a / g.topk : a - g.A) * g.cols + size_t(kt) * KT + k);
                    else v = static_cast<const float *>(x)[size_t(a) * g.cols + size_t(kt) * KT + k];
                }
                xs[tc * LDX + k] = v;
            }
            __syncthreads();
            const float * wr0 = w0 + r * KT, * wr1 = w1 + r * KT, * xr = xs + c * LDX;
#pragma unroll 8
            for (int k = 0; k < KT; ++k) {
                acc0 += wr0[k] * xr[k];
                if (MODE == 0) acc1 += wr1[k] * xr[k];
            }
        }
        const int a = toks[c], row = 16 * rt + r;
        if (a >= 0 && row < g.rows)
            out[size_t(a) * g.rows + row] = MODE == 0 ? (acc0 / (1.f + expf(-acc0))) * acc1 : acc0;
    }
}

template <uint32_t T, int MODE>
int32_t launch_t(const GroupArgs & g, const void * x, int x_dtype, const int * plan, float * out, int max_active, cudaStream_t s) {
    const size_t smem = (size_t(MODE == 0 ? 2 : 1) * 16 * Fmt<T>::KT + size_t(NT) * (Fmt<T>::KT + 1)) * sizeof(float);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(expert_generic_k<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
        return B2MOE_ERR_CUDA;
    const dim3 grid(ceil_div(g.rows, 16), max_active);
    expert_generic_k<T, MODE><<<grid, 256, smem, s>>>(g, x, x_dtype, plan, out);
    return launch_status();
}

template <int MODE>
int32_t launch(uint32_t type, const GroupArgs & g, const void * x, int x_dtype, const int * plan, float * out, int max_active,
               cudaStream_t s) {
    switch (type) {
        case T_Q4_K: return launch_t<T_Q4_K, MODE>(g, x, x_dtype, plan, out, max_active, s);
        case T_IQ3_S: return launch_t<T_IQ3_S, MODE>(g, x, x_dtype, plan, out, max_active, s);
        case T_IQ3S4: return launch_t<T_IQ3S4, MODE>(g, x, x_dtype, plan, out, max_active, s);
        case T_IQ4_XS: return launch_t<T_IQ4_XS, MODE>(g, x, x_dtype, plan, out, max_active, s);
        case T_IQ4_NL: return launch_t<T_IQ4_NL, MODE>(g, x, x_dtype, plan, out, max_active, s);
        case T_NVFP4G: return launch_t<T_NVFP4G, MODE>(g, x, x_dtype, plan, out, max_active, s);
    }
    return B2MOE_ERR_FORMAT;
}

}  // namespace

// the number of (expert) work slots a launch must cover: experts that can be active, plus the shared one
static inline int max_active_of_generic(int experts, int n, int topk, int shared_tokens) {
    const long long a = (long long)n * topk;
    return int(a < experts ? a : experts) + (shared_tokens ? 1 : 0);
}

int32_t generic_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * sg, const b2moe_bank * su, const void * x,
                       int x_dtype, const int * plan, int n, int topk, int shared_tokens, float * act, cudaStream_t s) {
    FmtInfo f;
    fmt_info(gate->type, f);
    GroupArgs g{};
    g.w0 = static_cast<const uint8_t *>(gate->data); g.w1 = static_cast<const uint8_t *>(up->data);
    g.aux0 = static_cast<const float *>(gate->aux); g.aux1 = static_cast<const float *>(up->aux);
    if (shared_tokens) {
        g.s0 = static_cast<const uint8_t *>(sg->data); g.s1 = static_cast<const uint8_t *>(su->data);
        g.saux0 = static_cast<const float *>(sg->aux); g.saux1 = static_cast<const float *>(su->aux);
    }
    g.bank_bytes = b2moe_bank_bytes(gate->type, gate->rows, gate->cols);
    g.rows = gate->rows; g.cols = gate->cols; g.experts = gate->experts; g.topk = topk; g.A = n * topk;
    g.k_tiles = gate->cols / f.kt; g.units = f.units;
    return launch<0>(gate->type, g, x, x_dtype, plan, act, max_active_of_generic(gate->experts, n, topk, shared_tokens), s);
}

int32_t generic_down(const b2moe_bank * down, const b2moe_bank * sd, const float * act, const int * plan, int n, int topk,
                     int shared_tokens, float * y, cudaStream_t s) {
    FmtInfo f;
    fmt_info(down->type, f);
    GroupArgs g{};
    g.w0 = static_cast<const uint8_t *>(down->data);
    g.aux0 = static_cast<const float *>(down->aux);
    if (shared_tokens) { g.s0 = static_cast<const uint8_t *>(sd->data); g.saux0 = static_cast<const float *>(sd->aux); }
    g.bank_bytes = b2moe_bank_bytes(down->type, down->rows, down->cols);
    g.rows = down->rows; g.cols = down->cols; g.experts = down->experts; g.topk = topk; g.A = n * topk;
    g.k_tiles = down->cols / f.kt; g.units = f.units;
    return launch<1>(down->type, g, act, B2MOE_F32, plan, y, max_active_of_generic(down->experts, n, topk, shared_tokens), s);
}

}  // namespace b2
