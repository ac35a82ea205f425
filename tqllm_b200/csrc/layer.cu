// C entry points of the expert products and the whole-layer sequence (router -> top-k -> dispatch -> gate/up + SwiGLU
// -> down -> combine): the launch order of qwen35_forward.cpp:1121-1252 / fn_layer_forward.cpp:311-336,504-522 /
// minimax.cpp:1083-1131 with every step stream-ordered on the device and no host read-back of the routing.
#include "common.cuh"
#include "formats.cuh"

namespace b2 {
int32_t check_bank(const b2moe_bank * b);
int32_t generic_gateup(const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const void *, int, const int *, int,
                       int, int, float *, cudaStream_t);
int32_t generic_down(const b2moe_bank *, const b2moe_bank *, const float *, const int *, int, int, int, float *, cudaStream_t);
size_t iq3s_workspace_bytes(int rows_x, int k, int dtype);
bool iq3s_supported(int k, int dtype);
int32_t iq3s_gateup(const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const void *, int, const int *, int,
                    int, int, float *, void *, int, cudaStream_t);
int32_t iq3s_down(const b2moe_bank *, const b2moe_bank *, const float *, const int *, int, int, int, float *, void *, int, cudaStream_t);
bool dec4_supported(uint32_t type, int k);
size_t dec4_workspace_bytes(int rows_x, int k);
int32_t dec4_gateup(const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const void *, int, const int *, int,
                    int, int, float *, void *, int, cudaStream_t, bool x_staged);
void dec4_stage_target(uint32_t type, void * ws, int n, int k, uint8_t ** rows, float ** inv_scale, int * bits);
bool route_cluster_fits(int experts, int topk, int n);
int32_t route_plan_stage(int gating, const float * logits, int ld, const float * bias, int * ids, float * weights, float * shared_weights,
                         int experts, int topk, int norm, float scale, int n, int shared_first, int shared_count, int * plan, const void * x,
                         int x_dtype, int k, int bits, uint8_t * staged_rows, float * inv_scale, cudaStream_t s, bool * took);
int32_t dec4_down(const b2moe_bank *, const b2moe_bank *, const float *, const int *, int, int, int, float *, void *, int, cudaStream_t);
void dec4_debug(int drop_tile, uint32_t wait_limit);
void dec4_skip_staging(bool on);
void dec4_ring(int nbuf, int stages, int slot_tiles);
void dec4_ksplit_max(int ks);
unsigned long long g_launch_count = 0;
bool g_overlap = true;
bool gemm_tc_supported(uint32_t type, int k, int nmat, int experts);
size_t gemm_tc_workspace_bytes(int rows_x, int k);
int32_t gemm_tc_gateup(const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const b2moe_bank *, const void *, int, const int *, int,
                       int, int, float *, void *, cudaStream_t);
int32_t gemm_tc_down(const b2moe_bank *, const b2moe_bank *, const float *, const int *, int, int, int, float *, void *, cudaStream_t);
void gemm_tc_item_tokens(int tokens);

namespace {
int32_t same_shape(const b2moe_bank * a, const b2moe_bank * b, bool same_experts) {
    if (a->type != b->type) return B2MOE_ERR_FORMAT;
    if (a->rows != b->rows || a->cols != b->cols || (same_experts && a->experts != b->experts)) return B2MOE_ERR_SHAPE;
    return B2MOE_OK;
}
// experts that can be active in one launch, plus the shared one: the grid's second dimension
int max_active_of(int experts, int n, int topk, int shared_tokens) {
    const long long a = (long long)n * topk;
    return int(a < experts ? a : experts) + (shared_tokens ? 1 : 0);
}
// The decode kernel of a bank type: DEC_IQ3S for IQ3_S in its GGUF-sized layout (grid lookup in the kernel), DEC_4BIT for
// banks of 4-bit codes (Q4_K, IQ3_S held as codes), DEC_NONE otherwise.
enum { DEC_NONE = 0, DEC_IQ3S = 1, DEC_4BIT = 2 };
int decode_kernel(uint32_t type, int k, int dtype) {
    if (type == T_IQ3_S && iq3s_supported(k, dtype)) return DEC_IQ3S;
    if (dec4_supported(type, k)) return DEC_4BIT;
    return DEC_NONE;
}
// The kernel family of one expert product.
//   decode   every expert sees a few tokens, the product is bound by streaming the weights;
//   GEMM     the tcgen05 grouped GEMM (all formats): the weights of an expert are decoded once per 128 tokens;
//   generic  exact fp32 CUDA-core path: every shape, the floor under the other two.
// Default: a type with a decode kernel takes it while the batch averages fewer than GEMM_MIN_PER assignments per expert
// or the bank has fewer than GEMM_MIN_EXPERTS experts (too few 128-row x 128-token items to fill the SMs), everything
// else the GEMM. b2moe_harness_select forces a family where it supports the shape (tests and benchmarks).
constexpr int GEMM_MIN_PER = 32, GEMM_MIN_EXPERTS = 128;   // measured on the c2 shape: below either, the decode kernels' finer work items win
int g_family = B2MOE_FAMILY_AUTO;
int expert_path(uint32_t type, int k, int dtype, int nmat, int experts, long long assignments) {
    if (g_family == B2MOE_FAMILY_GENERIC) return B2MOE_FAMILY_GENERIC;
    const bool dec = decode_kernel(type, k, dtype) != DEC_NONE, gemm = gemm_tc_supported(type, k, nmat, experts);
    if (g_family == B2MOE_FAMILY_DECODE) return dec ? B2MOE_FAMILY_DECODE : B2MOE_FAMILY_GENERIC;
    if (g_family == B2MOE_FAMILY_GEMM) return gemm ? B2MOE_FAMILY_GEMM : dec ? B2MOE_FAMILY_DECODE : B2MOE_FAMILY_GENERIC;
    if (dec && (!gemm || assignments < (long long)GEMM_MIN_PER * experts || experts < GEMM_MIN_EXPERTS)) return B2MOE_FAMILY_DECODE;
    return gemm ? B2MOE_FAMILY_GEMM : B2MOE_FAMILY_GENERIC;
}
}  // namespace
// true when b2moe_expert_down would take the format-generic kernels (which use no scratch) for this call
bool expert_down_is_generic(const b2moe_bank * down, int n, int topk) {
    return expert_path(down->type, down->cols, B2MOE_F32, 1, down->experts, (long long)n * topk) == B2MOE_FAMILY_GENERIC;
}
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API const char * b2moe_status_string(int32_t status) {
    switch (status) {
        case B2MOE_OK: return "ok";
        case B2MOE_ERR_SHAPE: return "invalid shape";
        case B2MOE_ERR_ALIGN: return "pointer is not 16-byte aligned";
        case B2MOE_ERR_FORMAT: return "unsupported or mismatched block format";
        case B2MOE_ERR_NULL: return "null pointer";
        case B2MOE_ERR_WORKSPACE: return "workspace too small";
        case B2MOE_ERR_CUDA: return "CUDA call failed";
        case B2MOE_ERR_CAPACITY: return "capacity exceeded";
    }
    return "unknown status";
}
extern "C" B2MOE_API int32_t b2moe_abi_version(void) { return B2MOE_ABI_VERSION; }
extern "C" B2MOE_API void b2moe_codebooks(uint32_t * grid, int8_t * kv) {
    if (grid) for (int i = 0; i < 512; ++i) grid[i] = h_iq3s_grid[i];
    if (kv) for (int i = 0; i < 16; ++i) kv[i] = h_kvalues_iq4nl[i];
}

extern "C" B2MOE_API void b2moe_harness_select(int32_t family, int32_t gemm_item_tokens) {
    g_family = family >= B2MOE_FAMILY_AUTO && family <= B2MOE_FAMILY_GEMM ? family : B2MOE_FAMILY_AUTO;
    gemm_tc_item_tokens(gemm_item_tokens);
}
extern "C" B2MOE_API void b2moe_harness_wait_probe(int32_t drop_tile, uint32_t wait_limit) { dec4_debug(drop_tile, wait_limit); }
extern "C" B2MOE_API void b2moe_harness_skip_staging(int32_t on) { dec4_skip_staging(on != 0); }
extern "C" B2MOE_API void b2moe_harness_ring(int32_t nbuf, int32_t stages, int32_t slot_tiles) { dec4_ring(nbuf, stages, slot_tiles); }
extern "C" B2MOE_API void b2moe_harness_column_split(int32_t max_warps_per_job) { dec4_ksplit_max(max_warps_per_job); }
extern "C" B2MOE_API void b2moe_harness_overlap(int32_t on) { g_overlap = on != 0; }
extern "C" B2MOE_API uint64_t b2moe_harness_launches(void) { return g_launch_count; }

extern "C" B2MOE_API size_t b2moe_expert_workspace_bytes(uint32_t type, int32_t rows_x, int32_t k, int32_t x_dtype) {
    if (rows_x <= 0 || k <= 0 || !valid_dtype(x_dtype)) return 0;
    FmtInfo f;
    if (!fmt_info(type, f)) return 0;
    // the largest of what the families that can serve this type would take (the family is chosen per call)
    const int dk = decode_kernel(type, k, x_dtype);
    size_t need = dk == DEC_IQ3S ? iq3s_workspace_bytes(rows_x, k, x_dtype) : dk == DEC_4BIT ? dec4_workspace_bytes(rows_x, k) : 0;
    const size_t g = gemm_tc_workspace_bytes(rows_x, k);
    return g > need ? g : need;
}

// x_staged: the caller has already written the staged form of x where the 4-bit decode kernels expect it (b2moe_layer_forward)
static int32_t expert_gateup(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * shared_gate, const b2moe_bank * shared_up,
                             const void * x, int32_t x_dtype, const int32_t * plan, int32_t n, int32_t topk, int32_t shared_tokens, float * act,
                             void * workspace, size_t workspace_bytes, b2moe_stream stream, bool x_staged, long long live = -1) {
    if (int32_t rc = check_bank(gate)) return rc;
    if (int32_t rc = check_bank(up)) return rc;
    if (int32_t rc = same_shape(gate, up, true)) return rc;
    if (n <= 0 || topk <= 0 || (shared_tokens != 0 && shared_tokens != n) || !valid_dtype(x_dtype)) return B2MOE_ERR_SHAPE;
    if (shared_tokens) {
        if (int32_t rc = check_bank(shared_gate)) return rc;
        if (int32_t rc = check_bank(shared_up)) return rc;
        if (int32_t rc = same_shape(gate, shared_gate, false)) return rc;
        if (int32_t rc = same_shape(gate, shared_up, false)) return rc;
    }
    if (!x || !plan || !act) return B2MOE_ERR_NULL;
    if (!aligned16(x) || !aligned16(act)) return B2MOE_ERR_ALIGN;
    const int path = expert_path(gate->type, gate->cols, x_dtype, 2, gate->experts, live >= 0 ? live : (long long)n * topk);
    if (path != B2MOE_FAMILY_GENERIC) {
        const size_t need = b2moe_expert_workspace_bytes(gate->type, n, gate->cols, x_dtype);
        if (need && !workspace) return B2MOE_ERR_NULL;
        if (need && !aligned16(workspace)) return B2MOE_ERR_ALIGN;
        if (workspace_bytes < need) return B2MOE_ERR_WORKSPACE;
        if (path == B2MOE_FAMILY_GEMM)
            return gemm_tc_gateup(gate, up, shared_gate, shared_up, x, x_dtype, plan, n, topk, shared_tokens, act, workspace, as_stream(stream));
        const int ma = max_active_of(gate->experts, n, topk, shared_tokens);
        if (decode_kernel(gate->type, gate->cols, x_dtype) == DEC_4BIT)
            return dec4_gateup(gate, up, shared_gate, shared_up, x, x_dtype, plan, n, topk, shared_tokens, act, workspace, ma, as_stream(stream), x_staged);
        return iq3s_gateup(gate, up, shared_gate, shared_up, x, x_dtype, plan, n, topk, shared_tokens, act, workspace, ma, as_stream(stream));
    }
    return generic_gateup(gate, up, shared_gate, shared_up, x, x_dtype, plan, n, topk, shared_tokens, act, as_stream(stream));
}

extern "C" B2MOE_API int32_t b2moe_expert_gateup_swiglu(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * shared_gate,
                                              const b2moe_bank * shared_up, const void * x, int32_t x_dtype, const int32_t * plan,
                                              int32_t n, int32_t topk, int32_t shared_tokens, float * act, void * workspace,
                                              size_t workspace_bytes, b2moe_stream stream) {
    return expert_gateup(gate, up, shared_gate, shared_up, x, x_dtype, plan, n, topk, shared_tokens, act, workspace, workspace_bytes, stream, false);
}

static int32_t expert_down(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act, const int32_t * plan, int32_t n, int32_t topk,
                           int32_t shared_tokens, float * y, void * workspace, size_t workspace_bytes, b2moe_stream stream, long long live) {
    if (int32_t rc = check_bank(down)) return rc;
    if (n <= 0 || topk <= 0 || (shared_tokens != 0 && shared_tokens != n)) return B2MOE_ERR_SHAPE;
    if (shared_tokens) {
        if (int32_t rc = check_bank(shared_down)) return rc;
        if (int32_t rc = same_shape(down, shared_down, false)) return rc;
    }
    if (!act || !plan || !y) return B2MOE_ERR_NULL;
    if (!aligned16(act) || !aligned16(y)) return B2MOE_ERR_ALIGN;
    const int path = expert_path(down->type, down->cols, B2MOE_F32, 1, down->experts, live >= 0 ? live : (long long)n * topk);
    if (path != B2MOE_FAMILY_GENERIC) {
        const int rows_x = n * topk + shared_tokens;
        if (!workspace) return B2MOE_ERR_NULL;
        if (!aligned16(workspace)) return B2MOE_ERR_ALIGN;
        if (workspace_bytes < b2moe_expert_workspace_bytes(down->type, rows_x, down->cols, B2MOE_F32)) return B2MOE_ERR_WORKSPACE;
        if (path == B2MOE_FAMILY_GEMM)
            return gemm_tc_down(down, shared_down, act, plan, n, topk, shared_tokens, y, workspace, as_stream(stream));
        const int ma = max_active_of(down->experts, n, topk, shared_tokens);
        if (decode_kernel(down->type, down->cols, B2MOE_F32) == DEC_4BIT)
            return dec4_down(down, shared_down, act, plan, n, topk, shared_tokens, y, workspace, ma, as_stream(stream));
        return iq3s_down(down, shared_down, act, plan, n, topk, shared_tokens, y, workspace, ma, as_stream(stream));
    }
    return generic_down(down, shared_down, act, plan, n, topk, shared_tokens, y, as_stream(stream));
}

extern "C" B2MOE_API int32_t b2moe_expert_down(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act, const int32_t * plan,
                                     int32_t n, int32_t topk, int32_t shared_tokens, float * y, void * workspace,
                                     size_t workspace_bytes, b2moe_stream stream) {
    return expert_down(down, shared_down, act, plan, n, topk, shared_tokens, y, workspace, workspace_bytes, stream, -1);
}
// The two products for a caller that knows how many of the n * topk assignments are live (id >= 0): under expert parallelism a
// rank sees every token but owns 1 / G of the experts, and the kernel family is chosen by tokens per expert.
extern "C" B2MOE_API int32_t b2moe_expert_gateup_swiglu_sparse(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * shared_gate,
                                                     const b2moe_bank * shared_up, const void * x, int32_t x_dtype, const int32_t * plan, int32_t n,
                                                     int32_t topk, int32_t shared_tokens, int64_t live_assignments, float * act, void * workspace,
                                                     size_t workspace_bytes, b2moe_stream stream) {
    if (live_assignments < 0 || live_assignments > (long long)n * topk) return B2MOE_ERR_SHAPE;
    return expert_gateup(gate, up, shared_gate, shared_up, x, x_dtype, plan, n, topk, shared_tokens, act, workspace, workspace_bytes, stream, false,
                         live_assignments);
}
extern "C" B2MOE_API int32_t b2moe_expert_down_sparse(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act, const int32_t * plan,
                                            int32_t n, int32_t topk, int32_t shared_tokens, int64_t live_assignments, float * y, void * workspace,
                                            size_t workspace_bytes, b2moe_stream stream) {
    if (live_assignments < 0 || live_assignments > (long long)n * topk) return B2MOE_ERR_SHAPE;
    return expert_down(down, shared_down, act, plan, n, topk, shared_tokens, y, workspace, workspace_bytes, stream, live_assignments);
}

extern "C" B2MOE_API int32_t b2moe_layer_workspace(const b2moe_layer * L, int32_t n, b2moe_layer_ws * ws) {
    if (!L || !ws) return B2MOE_ERR_NULL;
    if (n <= 0 || L->hidden <= 0 || L->experts <= 0 || L->topk <= 0 || L->topk > L->experts || L->ff <= 0) return B2MOE_ERR_SHAPE;
    if ((long long)n * L->topk > 0x3fffffffLL) return B2MOE_ERR_SHAPE;
    const size_t A = size_t(n) * L->topk, At = A + (L->has_shared ? n : 0);
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t o = at; at = align_up(at + bytes, 256); return o; };
    ws->logits = take(size_t(n) * (L->experts + 1) * sizeof(float));
    ws->ids = take(A * sizeof(int32_t));
    ws->weights = take(A * sizeof(float));
    ws->shared_weights = take(size_t(n) * sizeof(float));
    ws->plan = take(size_t(b2moe_plan_ints(L->experts, int32_t(A), L->has_shared ? n : 0)) * sizeof(int32_t));
    ws->act = take(At * L->ff * sizeof(float));
    ws->y = take(At * L->hidden * sizeof(float));
    ws->scratch = take(b2moe_dispatch_workspace_bytes(L->experts, int32_t(A)));
    const size_t eg = b2moe_expert_workspace_bytes(L->gate.type, n, L->hidden, B2MOE_F32);
    const size_t ed = b2moe_expert_workspace_bytes(L->down.type, int32_t(At), L->ff, B2MOE_F32);
    ws->expert_scratch = take(eg > ed ? eg : ed);
    ws->total = at;
    return B2MOE_OK;
}

static int32_t layer_forward(const b2moe_layer * L, const void * x, int32_t x_dtype, int32_t n, const void * residual, void * out,
                             int32_t out_dtype, void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    b2moe_layer_ws ws;
    if (int32_t rc = b2moe_layer_workspace(L, n, &ws)) return rc;
    if (!x || !out || !workspace || !L->router_w) return B2MOE_ERR_NULL;
    if (workspace_bytes < ws.total) return B2MOE_ERR_WORKSPACE;
    if (!aligned16(workspace)) return B2MOE_ERR_ALIGN;
    if (L->gating != B2MOE_SOFTMAX && L->gating != B2MOE_SIGMOID) return B2MOE_ERR_SHAPE;
    if (L->gate.rows != L->ff || L->gate.cols != L->hidden || L->down.rows != L->hidden || L->down.cols != L->ff ||
        L->gate.experts != L->experts || L->down.experts != L->experts) return B2MOE_ERR_SHAPE;
    char * base = static_cast<char *>(workspace);
    float * logits = reinterpret_cast<float *>(base + ws.logits);
    int32_t * ids = reinterpret_cast<int32_t *>(base + ws.ids);
    float * weights = reinterpret_cast<float *>(base + ws.weights);
    float * shw = reinterpret_cast<float *>(base + ws.shared_weights);
    int32_t * plan = reinterpret_cast<int32_t *>(base + ws.plan);
    float * act = reinterpret_cast<float *>(base + ws.act);
    float * y = reinterpret_cast<float *>(base + ws.y);
    const int ld = L->experts + 1, sh = L->has_shared ? n : 0;
    const bool gated_shared = L->has_shared && L->shared_gate_vec;

    if (int32_t rc = b2moe_router(L->router_w, gated_shared ? L->shared_gate_vec : nullptr, x, x_dtype, logits, ld, L->hidden, L->experts,
                                  n, stream)) return rc;
    if (L->gating == B2MOE_SIGMOID && gated_shared) return B2MOE_ERR_SHAPE;   // the sigmoid family adds its shared expert unscaled (moe_common.cu:191)
    void * es = base + ws.expert_scratch;
    const size_t es_bytes = ws.total - ws.expert_scratch;
    // decode-sized call on the 4-bit decode kernels: top-k, dispatch and the staging of x in one cluster launch
    bool x_staged = false;
    if (route_cluster_fits(L->experts, L->topk, n) && es_bytes >= b2moe_expert_workspace_bytes(L->gate.type, n, L->gate.cols, x_dtype) &&
        expert_path(L->gate.type, L->gate.cols, x_dtype, 2, L->gate.experts, (long long)n * L->topk) == B2MOE_FAMILY_DECODE &&
        decode_kernel(L->gate.type, L->gate.cols, x_dtype) == DEC_4BIT && valid_dtype(x_dtype)) {
        uint8_t * rows;
        float * inv;
        int bits;
        dec4_stage_target(L->gate.type, es, n, L->gate.cols, &rows, &inv, &bits);
        if (int32_t rc = route_plan_stage(L->gating, logits, ld, L->sel_bias, ids, weights, gated_shared ? shw : nullptr, L->experts, L->topk, L->norm,
                                          L->scale, n, 0, sh, plan, x, x_dtype, L->gate.cols, bits, rows, inv, as_stream(stream), &x_staged)) return rc;
    }
    if (!x_staged)
        if (int32_t rc = b2moe_route_dispatch(L->gating, logits, ld, L->sel_bias, ids, weights, gated_shared ? shw : nullptr, L->experts, L->topk,
                                              L->norm, L->scale, n, 0, sh, plan, base + ws.scratch, ws.expert_scratch - ws.scratch, stream))
            return rc;
    if (int32_t rc = expert_gateup(&L->gate, &L->up, &L->sh_gate, &L->sh_up, x, x_dtype, plan, n, L->topk, sh, act, es, es_bytes, stream, x_staged))
        return rc;
    if (int32_t rc = b2moe_expert_down(&L->down, &L->sh_down, act, plan, n, L->topk, sh, y, es, es_bytes, stream)) return rc;
    if (residual) return b2moe_combine_residual(y, nullptr, weights, gated_shared ? shw : nullptr, residual, n, L->topk, L->hidden, sh, out, out_dtype, stream);
    return b2moe_combine(y, nullptr, weights, gated_shared ? shw : nullptr, n, L->topk, L->hidden, sh, out, out_dtype, stream);
}

extern "C" B2MOE_API int32_t b2moe_layer_forward(const b2moe_layer * L, const void * x, int32_t x_dtype, int32_t n, void * out,
                                       int32_t out_dtype, void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    return layer_forward(L, x, x_dtype, n, nullptr, out, out_dtype, workspace, workspace_bytes, stream);
}
// the layer with its skip connection: out = residual + MoE(x); residual [n][hidden] of out_dtype, may be the out buffer
extern "C" B2MOE_API int32_t b2moe_layer_forward_residual(const b2moe_layer * L, const void * x, int32_t x_dtype, int32_t n, const void * residual,
                                                void * out, int32_t out_dtype, void * workspace, size_t workspace_bytes, b2moe_stream stream) {
    if (!residual) return B2MOE_ERR_NULL;
    return layer_forward(L, x, x_dtype, n, residual, out, out_dtype, workspace, workspace_bytes, stream);
}
