// Entry points with the argument shapes of the reference's per-matrix expert calls, for the WeightFormat adapter:
// device ids or moe_group's (counts, groups) in, bf16 / fp16 per-assignment rows out. They are thin compositions of the
// dispatch and the grouped products of this library (an engine that adopts b2moe_layer_forward does not need them):
//   WeightFormat::expert_matvec      (src/formats/weight/weight_format.hpp:62-63)  -> b2moe_expert_matvec
//   WeightFormat::expert_gemm        (weight_format.hpp:51-53)                     -> b2moe_expert_gemm
//   WeightFormat::expert_gemm_gateup (weight_format.hpp:58-59)                     -> b2moe_expert_gemm_gateup
// Scratch comes from the caller's workspace, carved here: the plan, the dispatch scratch, the fp32 input / output rows
// of the product and the product's own scratch.
#include "common.cuh"
#include "dispatch.cuh"
#include "formats.cuh"

namespace b2 {
int32_t check_bank(const b2moe_bank * b);

namespace {

// counts / groups of moe_group (src/experts/moe_kernels.cuh:29: groups [experts][capacity], counts [experts]) -> the plan's
// counts, offsets, active list and pass list (one block), then the permutation (grid): expert x's list is copied as it is
__global__ void groups_head_k(const int * __restrict__ counts_in, int experts, int capacity, int * __restrict__ plan, int assignments) {
    const int e1 = experts + 1;
    int * counts = plan + PLAN_HDR, * offsets = counts + e1, * active = offsets + e1 + 1, * perm = active + e1;
    for (int x = threadIdx.x; x < experts; x += blockDim.x) counts[x] = max(0, min(counts_in[x], capacity));
    if (threadIdx.x == 0) counts[experts] = 0;
    __syncthreads();
    if (threadIdx.x < 32) finish_plan(plan, counts, offsets, active, offsets, active, perm + assignments, e1, threadIdx.x);
}
__global__ void groups_perm_k(const int * __restrict__ groups, int experts, int capacity, int * __restrict__ plan) {
    const int e1 = experts + 1;
    const int * counts = plan + PLAN_HDR, * offsets = counts + e1;
    int * perm = plan + PLAN_HDR + e1 + e1 + 1 + e1;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)experts * capacity) return;
    const int x = int(i / capacity), j = int(i % capacity);
    if (j < counts[x]) perm[offsets[x] + j] = groups[i];
}
// x [n or A][cols] of any dtype -> fp32 [A][cols]: assignment a reads row a (per_assignment) or row a / topk
__global__ void rows_expand_k(const void * __restrict__ x, int dtype, int A, int cols, int topk, int per_assignment, float * __restrict__ out) {
    const int a = blockIdx.x;
    const size_t src = size_t(per_assignment ? a : a / topk) * cols;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) out[size_t(a) * cols + j] = load_act(x, dtype, src + j);
}
// rows of the grouped assignments only (the others stay untouched, as in the reference): y[a] = convert(y32[a])
__global__ void rows_convert_k(const float * __restrict__ y32, const int * __restrict__ plan, int experts, int rows, void * __restrict__ y, int dtype) {
    const int e1 = experts + 1;
    const int * perm = plan + PLAN_HDR + e1 + e1 + 1 + e1;
    if (int(blockIdx.x) >= plan[PLAN_NGROUPED]) return;
    const int a = perm[blockIdx.x];
    for (int j = threadIdx.x; j < rows; j += blockDim.x) store_act(y, dtype, size_t(a) * rows + j, y32[size_t(a) * rows + j]);
}

// out[t] = sum_s w[t][s] routed[t * topk + s] + sw[t] (1 when null) * shared[t]: typed per-assignment rows in, typed rows out
__global__ void sum_rows_k(const void * __restrict__ routed, int rdt, const void * __restrict__ shared, const float * __restrict__ w,
                           const float * __restrict__ sw, int hidden, int topk, void * __restrict__ out, int odt) {
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < topk; ++s) acc += w[size_t(t) * topk + s] * load_act(routed, rdt, (size_t(t) * topk + s) * hidden + j);
        if (shared) acc += (sw ? sw[t] : 1.f) * load_act(shared, rdt, size_t(t) * hidden + j);
        store_act(out, odt, size_t(t) * hidden + j, acc);
    }
}
__global__ void swiglu_k(const void * __restrict__ g, const void * __restrict__ u, int idt, void * __restrict__ act, int adt, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float gv = load_act(g, idt, size_t(i)), uv = load_act(u, idt, size_t(i));
    store_act(act, adt, size_t(i), gv / (1.f + expf(-gv)) * uv);
}
__global__ void rows_to_dtype_k(const float * __restrict__ in, long long count, void * __restrict__ out, int dt) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) store_act(out, dt, size_t(i), in[i]);
}

struct Carve {
    char * base; size_t at = 0, cap;
    Carve(void * p, size_t bytes) : base(static_cast<char *>(p)), cap(bytes) {}
    void * take(size_t bytes) { const size_t o = at; at = align_up(at + bytes, 256); return base ? base + o : nullptr; }
    bool fits() const { return at <= cap; }
};
struct Parts { int32_t * plan; void * dws; size_t dws_bytes; float * x32, * y32; void * ews; size_t ews_bytes; size_t total; };
// rows_x: rows of the product's fp32 input copy (0: the product reads the caller's x directly); out_cols: row length of the fp32 output
Parts carve(void * ws, size_t bytes, const b2moe_bank * b, int A, int rows_x, int out_cols, size_t ews_bytes) {
    Carve c(ws, bytes);
    Parts p{};
    p.plan = static_cast<int32_t *>(c.take(size_t(b2moe_plan_ints(b->experts, A, 0)) * sizeof(int32_t)));
    p.dws_bytes = b2moe_dispatch_workspace_bytes(b->experts, A);
    p.dws = c.take(p.dws_bytes);
    p.x32 = static_cast<float *>(c.take(size_t(rows_x) * b->cols * sizeof(float)));
    p.y32 = static_cast<float *>(c.take(size_t(A) * out_cols * sizeof(float)));
    p.ews_bytes = ews_bytes;
    p.ews = c.take(ews_bytes);
    p.total = c.at;
    return p;
}
int32_t plan_from_groups(const int32_t * counts, const int32_t * groups, int capacity, int experts, int A, int32_t * plan, cudaStream_t s) {
    groups_head_k<<<1, 1024, 0, s>>>(counts, experts, capacity, plan, A);
    if (int32_t rc = launch_status()) return rc;
    const long long cells = (long long)experts * capacity;
    groups_perm_k<<<unsigned((cells + 255) / 256), 256, 0, s>>>(groups, experts, capacity, plan);
    return launch_status();
}
// the single-matrix product over a ready plan: fp32 copy of the input rows, product, typed output rows
int32_t single_product(const b2moe_bank * m, const void * x, int x_dtype, void * y, int y_dtype, const Parts & p, int n, int topk,
                       int per_expert_input, cudaStream_t s) {
    const int A = n * topk;
    rows_expand_k<<<A, 128, 0, s>>>(x, x_dtype, A, m->cols, topk, per_expert_input, p.x32);
    if (int32_t rc = launch_status()) return rc;
    if (int32_t rc = b2moe_expert_down(m, nullptr, p.x32, p.plan, n, topk, 0, p.y32, p.ews, p.ews_bytes, s)) return rc;
    rows_convert_k<<<A, 128, 0, s>>>(p.y32, p.plan, m->experts, m->rows, y, y_dtype);
    return launch_status();
}
int32_t check_common(const b2moe_bank * m, int n, int topk, int x_dtype, int y_dtype) {
    if (int32_t rc = check_bank(m)) return rc;
    if (n <= 0 || topk <= 0 || (long long)n * topk > 0x3fffffffLL || !valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return B2MOE_ERR_SHAPE;
    return B2MOE_OK;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API size_t b2moe_expert_matvec_workspace_bytes(const b2moe_bank * m, int32_t n, int32_t topk) {
    if (!m || n <= 0 || topk <= 0) return 0;
    const int A = n * topk;
    return carve(nullptr, 0, m, A, A, m->rows, b2moe_expert_workspace_bytes(m->type, A, m->cols, B2MOE_F32)).total;
}
extern "C" B2MOE_API size_t b2moe_expert_gemm_gateup_workspace_bytes(const b2moe_bank * gate, int32_t n, int32_t topk, int32_t x_dtype) {
    if (!gate || n <= 0 || topk <= 0 || !valid_dtype(x_dtype)) return 0;
    return carve(nullptr, 0, gate, n * topk, 0, gate->rows, b2moe_expert_workspace_bytes(gate->type, n, gate->cols, x_dtype)).total;
}

extern "C" B2MOE_API int32_t b2moe_plan_from_groups(const int32_t * counts, const int32_t * groups, int32_t capacity, int32_t experts,
                                                    int32_t assignments, int32_t * plan, b2moe_stream stream) {
    if (capacity <= 0 || experts <= 0 || assignments <= 0) return B2MOE_ERR_SHAPE;
    if (!counts || !groups || !plan) return B2MOE_ERR_NULL;
    return plan_from_groups(counts, groups, capacity, experts, assignments, plan, as_stream(stream));
}

extern "C" B2MOE_API int32_t b2moe_expert_matvec(const b2moe_bank * m, const void * x, int32_t x_dtype, void * y, int32_t y_dtype,
                                                 const int32_t * ids, int32_t n, int32_t topk, int32_t per_expert_input, void * workspace,
                                                 size_t workspace_bytes, b2moe_stream stream) {
    if (int32_t rc = check_common(m, n, topk, x_dtype, y_dtype)) return rc;
    if (!x || !y || !ids || !workspace) return B2MOE_ERR_NULL;
    if (!aligned16(x) || !aligned16(y) || !aligned16(workspace)) return B2MOE_ERR_ALIGN;
    const int A = n * topk;
    const Parts p = carve(workspace, workspace_bytes, m, A, A, m->rows, b2moe_expert_workspace_bytes(m->type, A, m->cols, B2MOE_F32));
    if (p.total > workspace_bytes) return B2MOE_ERR_WORKSPACE;
    if (int32_t rc = b2moe_dispatch(ids, n, topk, m->experts, 0, p.plan, p.dws, p.dws_bytes, stream)) return rc;
    return single_product(m, x, x_dtype, y, y_dtype, p, n, topk, per_expert_input, as_stream(stream));
}

extern "C" B2MOE_API int32_t b2moe_expert_gemm(const b2moe_bank * m, const void * x, int32_t x_dtype, void * y, int32_t y_dtype,
                                               const int32_t * counts, const int32_t * groups, int32_t capacity, int32_t topk,
                                               int32_t per_expert_input, void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    const int n = capacity;                      // moe_group's lists hold one assignment per expert per token: capacity = tokens
    if (int32_t rc = check_common(m, n, topk, x_dtype, y_dtype)) return rc;
    if (!x || !y || !counts || !groups || !workspace) return B2MOE_ERR_NULL;
    if (!aligned16(x) || !aligned16(y) || !aligned16(workspace)) return B2MOE_ERR_ALIGN;
    const int A = n * topk;
    const Parts p = carve(workspace, workspace_bytes, m, A, A, m->rows, b2moe_expert_workspace_bytes(m->type, A, m->cols, B2MOE_F32));
    if (p.total > workspace_bytes) return B2MOE_ERR_WORKSPACE;
    if (int32_t rc = plan_from_groups(counts, groups, capacity, m->experts, A, p.plan, as_stream(stream))) return rc;
    return single_product(m, x, x_dtype, y, y_dtype, p, n, topk, per_expert_input, as_stream(stream));
}

extern "C" B2MOE_API int32_t b2moe_expert_gemm_gateup(const b2moe_bank * gate, const b2moe_bank * up, const void * x, int32_t x_dtype, void * act,
                                                      int32_t act_dtype, const int32_t * counts, const int32_t * groups, int32_t capacity,
                                                      int32_t topk, void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    const int n = capacity;
    if (int32_t rc = check_common(gate, n, topk, x_dtype, act_dtype)) return rc;
    if (int32_t rc = check_bank(up)) return rc;
    if (!x || !act || !counts || !groups || !workspace) return B2MOE_ERR_NULL;
    if (!aligned16(x) || !aligned16(act) || !aligned16(workspace)) return B2MOE_ERR_ALIGN;
    const int A = n * topk;
    const Parts p = carve(workspace, workspace_bytes, gate, A, 0, gate->rows, b2moe_expert_workspace_bytes(gate->type, n, gate->cols, x_dtype));
    if (p.total > workspace_bytes) return B2MOE_ERR_WORKSPACE;
    cudaStream_t s = as_stream(stream);
    if (int32_t rc = plan_from_groups(counts, groups, capacity, gate->experts, A, p.plan, s)) return rc;
    if (int32_t rc = b2moe_expert_gateup_swiglu(gate, up, nullptr, nullptr, x, x_dtype, p.plan, n, topk, 0, p.y32, p.ews, p.ews_bytes, stream)) return rc;
    rows_convert_k<<<A, 128, 0, s>>>(p.y32, p.plan, gate->experts, gate->rows, act, act_dtype);
    return launch_status();
}

// moe_sum with the reference's row types (src/experts/moe_kernels.cuh:73-74): per-assignment rows and shared rows of
// `in_dtype` (bf16 there), fp32 weights, out [n][hidden] of out_dtype. shared / shared_weights may be null.
extern "C" B2MOE_API int32_t b2moe_sum_rows(const void * routed, const void * shared, int32_t in_dtype, const float * weights,
                                            const float * shared_weights, void * out, int32_t out_dtype, int32_t hidden, int32_t topk, int32_t n,
                                            b2moe_stream stream) {
    if (hidden <= 0 || topk <= 0 || n <= 0 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype)) return B2MOE_ERR_SHAPE;
    if (!routed || !weights || !out) return B2MOE_ERR_NULL;
    sum_rows_k<<<n, 256, 0, as_stream(stream)>>>(routed, in_dtype, shared, weights, shared_weights, hidden, topk, out, out_dtype);
    return launch_status();
}
// moe_swiglu (src/experts/moe_kernels.cuh:71-72): act[i] = silu(gate[i]) * up[i] over `count` values
extern "C" B2MOE_API int32_t b2moe_swiglu(const void * gate, const void * up, int32_t in_dtype, void * act, int32_t act_dtype, int64_t count,
                                          b2moe_stream stream) {
    if (count <= 0 || !valid_dtype(in_dtype) || !valid_dtype(act_dtype)) return B2MOE_ERR_SHAPE;
    if (!gate || !up || !act) return B2MOE_ERR_NULL;
    swiglu_k<<<unsigned((count + 255) / 256), 256, 0, as_stream(stream)>>>(gate, up, in_dtype, act, act_dtype, count);
    return launch_status();
}
// the exact dequantisation of b2moe_dequant_dump rounded once to out_dtype (WeightFormat::dequant_h,
// src/formats/weight/weight_format.hpp:78); workspace: experts * rows * cols floats
extern "C" B2MOE_API int32_t b2moe_dequant_dump_as(const b2moe_bank * bank, void * out, int32_t out_dtype, void * workspace, size_t workspace_bytes,
                                                   b2moe_stream stream) {
    if (int32_t rc = check_bank(bank)) return rc;
    if (!valid_dtype(out_dtype)) return B2MOE_ERR_SHAPE;
    if (!out || !workspace) return B2MOE_ERR_NULL;
    const long long count = (long long)bank->experts * bank->rows * bank->cols;
    if (workspace_bytes < size_t(count) * sizeof(float)) return B2MOE_ERR_WORKSPACE;
    if (int32_t rc = b2moe_dequant_dump(bank, static_cast<float *>(workspace), stream)) return rc;
    rows_to_dtype_k<<<unsigned((count + 255) / 256), 256, 0, as_stream(stream)>>>(static_cast<const float *>(workspace), count, out, out_dtype);
    return launch_status();
}
