/* b2moe — C ABI of the B200 (sm_100a) mixture-of-experts layer path.
 *
 * Drop-in boundary for tqLLM's expert-layer interface. tqLLM calls this path through the C++ virtual
 * tqllm::WeightFormat (src/formats/weight/weight_format.hpp:33-110) and the free functions of namespace tqllm_cuda
 * (src/experts/moe_kernels.cuh:7-82, src/experts/moe_common.cuh:11-22); its C plugin ABI (include/tqllm/plugin.h:36-75)
 * carries only dequant and dense matvec and forwards every expert_* call to the built-in, so the seam is this C ABI
 * plus the C++ adapter in tqllm_b200/adapter/ that implements the reference's virtuals on top of it.
 *
 * Conventions (identical to the reference's, src/experts/moe_kernels.cuh:29, src/formats/weight/quant_u4h.inc:445,658):
 *   - every pointer is DEVICE memory unless a parameter says "host"; the caller owns all of it;
 *   - stacked expert weights are [experts * rows][cols]; ids are [n][topk] int32, id -1 = skip the assignment;
 *   - assignment a = token * topk + slot; per-assignment outputs are [n * topk][rows];
 *   - every entry point is stream-ordered, does no host synchronisation and allocates nothing: scratch comes from a
 *     caller-provided workspace, and the library keeps no mutable state between calls (re-entrant across streams).
 *     Exceptions, each stated where it is declared: b2moe_expert_down_static keeps its scratch in one array inside the
 *     library; the b2moe_harness_* hooks set process-wide switches for tests and benchmarks; b2moe_peer_alloc /
 *     b2moe_peer_open (set-up of the multi-GPU exchange, called once, outside any step) allocate and map device memory
 *     and synchronise with the device, and b2moe_gguf_* is host code that maps a file;
 *   - return value: 0 = ok, otherwise a b2moe_status code (b2moe_status_string gives the text). Nothing is launched
 *     when the arguments are rejected. There is no CPU fallback: without a CUDA device every compute entry point
 *     returns B2MOE_ERR_CUDA.
 */
#ifndef B2MOE_H
#define B2MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2MOE_ABI_VERSION 1

#if defined(__GNUC__)
#define B2MOE_API __attribute__((visibility("default")))
#else
#define B2MOE_API
#endif

typedef void * b2moe_stream; /* cudaStream_t */

enum b2moe_status {
    B2MOE_OK = 0,
    B2MOE_ERR_SHAPE = 1,     /* a dimension is out of range for the kernel (reference: std::invalid_argument) */
    B2MOE_ERR_ALIGN = 2,     /* a pointer is not 16-byte aligned */
    B2MOE_ERR_FORMAT = 3,    /* GGUF type id is not one of the five block formats of this path */
    B2MOE_ERR_NULL = 4,      /* a required pointer is null */
    B2MOE_ERR_WORKSPACE = 5, /* the workspace is smaller than b2moe_*_workspace_bytes says */
    B2MOE_ERR_CUDA = 6,      /* a CUDA call or launch failed (reference: std::runtime_error) */
    B2MOE_ERR_CAPACITY = 7   /* a per-expert or per-peer capacity was exceeded */
};

/* GGUF type ids of the block formats (src/core/gguf.hpp:18-37) */
enum b2moe_type {
    B2MOE_Q4_K = 12, B2MOE_IQ4_NL = 20, B2MOE_IQ3_S = 21, B2MOE_IQ4_XS = 23, B2MOE_NVFP4G = 323,
    /* Not a GGUF type: a second bank layout for IQ3_S blocks. b2moe_bank_load takes the same raw IQ3_S blocks and
     * stores every weight as a 4-bit code (grid lookup and sign applied once, at load time): 134 bytes per 256 weights
     * in HBM instead of 110, the same fp32 values bit for bit, and decode kernels that need no codebook lookup. The
     * layout to choose when HBM capacity allows (21.8 % more bytes per expert); B2MOE_IQ3_S keeps the GGUF size. */
    B2MOE_IQ3_S_X4 = 0x1015
};
enum b2moe_dtype { B2MOE_F32 = 0, B2MOE_F16 = 1, B2MOE_BF16 = 2 };
/* MoeGating values, src/experts/moe.hpp:20-26 (the two the device path implements) */
enum b2moe_gating { B2MOE_SOFTMAX = 1, B2MOE_SIGMOID = 2 };

B2MOE_API const char * b2moe_status_string(int32_t status);
B2MOE_API int32_t b2moe_abi_version(void);
/* The 512-entry IQ3_S grid and the 16 IQ4_NL values the library was built with (host memory, for test harnesses). */
B2MOE_API void b2moe_codebooks(uint32_t * iq3s_grid_512, int8_t * kvalues_iq4nl_16);

/* ---- expert banks ---------------------------------------------------------------------------------------------
 * A bank is one stacked expert matrix repacked from GGUF block bytes into 16-row tiles whose bytes sit in the order
 * the kernels' lanes consume them. Replaces the loaders Q4_K::load / IQ3_S::load / IQ4_XS::load / IQ4_NL::load /
 * NVFP4G::load (src/formats/weight/q4.cpp:807-825, 300-318, 582-600, 537-568, 500-523). */
typedef struct b2moe_bank {
    const void * data; /* tiles: [experts][ceil(rows/16)][cols / k_tile][tile bytes] */
    const void * aux;  /* NVFP4G: f32 tensor scale per padded row [experts][16*ceil(rows/16)]; NULL otherwise */
    uint32_t type;     /* b2moe_type */
    int32_t experts, rows, cols;
} b2moe_bank;

/* bytes of `rows` x `cols` in GGUF block form (host arithmetic; 0 when the type or shape is invalid; B2MOE_IQ3_S_X4
 * loads from IQ3_S blocks and reports their size) */
B2MOE_API size_t b2moe_raw_bytes(uint32_t type, int32_t rows, int32_t cols);
/* bytes of one expert's matrix in bank form, and of its aux array (0 when the type has none) */
B2MOE_API size_t b2moe_bank_bytes(uint32_t type, int32_t rows, int32_t cols);
B2MOE_API size_t b2moe_bank_aux_bytes(uint32_t type, int32_t rows, int32_t cols);
/* raw GGUF blocks (device, [experts*rows] rows) -> bank. `data`/`aux` are the caller's buffers of experts * the sizes above. */
B2MOE_API int32_t b2moe_bank_load(uint32_t type, const void * raw, int32_t experts, int32_t rows, int32_t cols, void * data,
                        void * aux, b2moe_stream stream);
/* The same bank built on the host: raw, data and aux are HOST memory and no CUDA call is made (a loader that uploads
 * finished banks through the engine's own upload callback, or packs expert files offline). */
B2MOE_API int32_t b2moe_bank_pack_host(uint32_t type, const void * raw, int32_t experts, int32_t rows, int32_t cols, void * data, void * aux);
/* bank -> fp32 [experts*rows][cols], bit-identical to dequantize_host (src/formats/weight/dequant.cpp:393-606) */
B2MOE_API int32_t b2moe_dequant_dump(const b2moe_bank * bank, float * out, b2moe_stream stream);

/* ---- routing --------------------------------------------------------------------------------------------------
 * b2moe_router replaces moe_router / moe_router_f32 (src/experts/moe.cu:17-33,237-247): logits[t][r] = W[r] . x[t] for
 * r < experts, and column `experts` = shared_gate . x[t] when shared_gate is given. ld = row stride of logits
 * (the reference uses experts + 1). x is [n][hidden] of x_dtype. */
B2MOE_API int32_t b2moe_router(const float * router_w, const float * shared_gate, const void * x, int32_t x_dtype, float * logits,
                     int32_t ld, int32_t hidden, int32_t experts, int32_t n, b2moe_stream stream);
/* replaces moe_topk (src/experts/moe.cu:35-166,248-267): softmax over experts, top-k (larger value, then lower index),
 * weights = p / max(sum of selected p, 6.103515625e-5) * (scale == 0 ? 1 : scale); shared_weights[t] =
 * sigmoid(logits[t][experts]) when shared_weights is given. experts <= 4096. */
B2MOE_API int32_t b2moe_topk_softmax(const float * logits, int32_t ld, int32_t * ids, float * weights, float * shared_weights,
                           int32_t experts, int32_t topk, int32_t n, float scale, b2moe_stream stream);
/* replaces moe_topk2 (src/experts/moe.cu:160-166,255-267, src/experts/moe_kernels.cuh:24-25): b2moe_topk_softmax on two
 * routings of the same n tokens in one launch (this layer's logits and the next layer's predicted ones); both logit
 * arrays have row stride ld; outputs and bits are those of two separate calls. */
B2MOE_API int32_t b2moe_topk_softmax2(const float * logits, int32_t * ids, float * weights, float * shared_weights, const float * logits2,
                            int32_t * ids2, float * weights2, float * shared_weights2, int32_t ld, int32_t experts, int32_t topk,
                            int32_t n, float scale, b2moe_stream stream);
/* replaces moe_common::route (src/experts/moe_common.cu:18-70,197-203): p = sigmoid(logits); select top-k of p + bias
 * (bias may be null); weights = p[selected], divided by their clamped sum when norm, times scale unless 0 or 1. */
B2MOE_API int32_t b2moe_route_sigmoid(const float * logits, int32_t ld, const float * bias, int32_t * ids, float * weights,
                            int32_t experts, int32_t topk, int32_t norm, float scale, int32_t n, b2moe_stream stream);

/* ---- dispatch -------------------------------------------------------------------------------------------------
 * Token -> expert dispatch: per-expert histogram, exclusive prefix sum, stable permutation (assignment indices in
 * ascending order inside each expert). Replaces moe_group (src/experts/moe.cu:168-176,268-273, whose list order is
 * non-deterministic), the host builder fill_pass_lists (src/models/qwen/qwen4exp/prefill_plan.hpp:62-76) and
 * moe_dedup_maps (src/experts/moe.cu:453-483). With shared_tokens = n the always-on expert is appended as expert
 * `experts` holding the virtual assignments n*topk .. n*topk + n - 1 (token = a - n*topk), the device form of
 * moe_extend_ids (src/experts/moe.cu:209-222).
 *
 * The plan is one int32 device array of b2moe_plan_ints(experts, n * topk, shared_tokens) entries:
 *   [0] number of active experts   [1] number of grouped assignments   [2] number of passes   [3] kernel status word
 *   then counts[E1], offsets[E1 + 1], active[E1] (ids of experts with count > 0, ascending), perm[A + shared_tokens],
 *   passes[E1 + 1] (work list of the decode kernels: the active experts taken from the last to the first, each cut
 *   into passes of 8 tokens; passes[i] = passes before the i-th expert of that order)
 * with E1 = experts + 1. b2moe_plan_view gives the element offsets of the arrays (host arithmetic). Word [3] stays 0
 * unless a kernel gave up a bounded wait (it then holds a nonzero code and that launch's outputs are invalid). */
typedef struct b2moe_plan_view { int64_t counts, offsets, active, perm, passes, total; } b2moe_plan_view;
B2MOE_API int64_t b2moe_plan_ints(int32_t experts, int32_t assignments, int32_t shared_tokens);
B2MOE_API void b2moe_plan_view_of(int32_t experts, int32_t assignments, int32_t shared_tokens, b2moe_plan_view * view);
/* workspace: b2moe_dispatch_workspace_bytes(experts, assignments) bytes, 16-byte aligned */
B2MOE_API size_t b2moe_dispatch_workspace_bytes(int32_t experts, int32_t assignments);
B2MOE_API int32_t b2moe_dispatch(const int32_t * ids, int32_t n, int32_t topk, int32_t experts, int32_t shared_tokens, int32_t * plan,
                       void * workspace, size_t workspace_bytes, b2moe_stream stream);
/* The same with the always-on expert evaluated for the token range [shared_first, shared_first + shared_count) only
 * (expert parallelism: a rank routes every rank's tokens but owns the shared expert of its own). The plan is sized
 * with shared_tokens = shared_count; the shared rows of act / y still sit at n*topk + token. */
B2MOE_API int32_t b2moe_dispatch_range(const int32_t * ids, int32_t n, int32_t topk, int32_t experts, int32_t shared_first,
                             int32_t shared_count, int32_t * plan, void * workspace, size_t workspace_bytes,
                             b2moe_stream stream);
/* Routing and dispatch together (b2moe_topk_softmax or b2moe_route_sigmoid, then b2moe_dispatch_range): one launch for
 * decode-sized batches, the separate launches otherwise; outputs and bits are those of the separate calls. gating is a
 * b2moe_gating value; bias / norm apply to the sigmoid family, shared_weights to the softmax family. */
B2MOE_API int32_t b2moe_route_dispatch(int32_t gating, const float * logits, int32_t ld, const float * bias, int32_t * ids,
                             float * weights, float * shared_weights, int32_t experts, int32_t topk, int32_t norm, float scale,
                             int32_t n, int32_t shared_first, int32_t shared_count, int32_t * plan, void * workspace,
                             size_t workspace_bytes, b2moe_stream stream);
/* moe_group-compatible view of a plan (src/experts/moe_kernels.cuh:29): counts [experts], groups [experts][n] */
B2MOE_API int32_t b2moe_plan_to_groups(const int32_t * plan, int32_t n, int32_t topk, int32_t experts, int32_t * counts,
                             int32_t * groups, b2moe_stream stream);

/* ---- expert products ------------------------------------------------------------------------------------------
 * Scratch: the tensor-core kernels first bring the activation rows into operand form (one fp16 term per value, the row
 * scaled by a power of two, + that scale) inside a caller-provided workspace of b2moe_expert_workspace_bytes(type, rows_x, k, x_dtype) bytes (16-byte aligned), where
 * rows_x = n for the gate/up product (k = hidden) and n*topk + shared_tokens for the down product (k = ff, x_dtype
 * B2MOE_F32). The workspace may be NULL only where the size is 0. */
B2MOE_API size_t b2moe_expert_workspace_bytes(uint32_t type, int32_t rows_x, int32_t k, int32_t x_dtype);
/* act[a][f] = silu(gate_e(a)[f] . x[token(a)]) * (up_e(a)[f] . x[token(a)]) for every grouped assignment a: the
 * paired gate/up product with the SwiGLU fused (replaces expert_matvec2 / expert_matvec_dedup2 / expert_gemm_gateup +
 * moe_swiglu: src/formats/weight/weight_format.hpp:58-73, src/formats/weight/quant.cu:167-233,384-405,
 * src/experts/moe.cu:188-195). shared_* may be null when the plan has no shared expert. act is fp32
 * [n*topk + shared_tokens][ff]; rows of skipped assignments are left untouched. */
B2MOE_API int32_t b2moe_expert_gateup_swiglu(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * shared_gate,
                                   const b2moe_bank * shared_up, const void * x, int32_t x_dtype, const int32_t * plan,
                                   int32_t n, int32_t topk, int32_t shared_tokens, float * act, void * workspace,
                                   size_t workspace_bytes, b2moe_stream stream);
/* y[a][h] = down_e(a)[h] . act[a]   (replaces expert_matvec / expert_matvec_dedup / expert_gemm with
 * per_expert_input: src/formats/weight/weight_format.hpp:51-63, src/formats/weight/quant.cu:69-143,286-317). y fp32. */
B2MOE_API int32_t b2moe_expert_down(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act, const int32_t * plan,
                          int32_t n, int32_t topk, int32_t shared_tokens, float * y, void * workspace, size_t workspace_bytes,
                          b2moe_stream stream);
/* The two products for a caller that knows how many of the n * topk assignments are live (id >= 0). Under expert parallelism a
 * rank sees every gathered token but owns 1 / G of the experts (the other ids are -1, src/experts/moe.cu:496-503
 * ep_local_ids); the kernel family is chosen by live assignments per expert, which the plain entry points take as n * topk.
 * live_assignments is an estimate used for that choice only (0 <= live_assignments <= n * topk); results do not depend on it
 * beyond the family's rounding. */
B2MOE_API int32_t b2moe_expert_gateup_swiglu_sparse(const b2moe_bank * gate, const b2moe_bank * up, const b2moe_bank * shared_gate,
                                          const b2moe_bank * shared_up, const void * x, int32_t x_dtype, const int32_t * plan, int32_t n,
                                          int32_t topk, int32_t shared_tokens, int64_t live_assignments, float * act, void * workspace,
                                          size_t workspace_bytes, b2moe_stream stream);
B2MOE_API int32_t b2moe_expert_down_sparse(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act, const int32_t * plan,
                                 int32_t n, int32_t topk, int32_t shared_tokens, int64_t live_assignments, float * y, void * workspace,
                                 size_t workspace_bytes, b2moe_stream stream);
/* The down product without a workspace argument and without any allocation, for callers that cannot provide
 * scratch (an engine plugin that owns no device memory; code inside a stream capture or another region where
 * cudaMalloc is not allowed). It has no counterpart in the reference. The scratch b2moe_expert_down would take from
 * the caller lives in a fixed B2MOE_STATIC_SCRATCH_BYTES array inside the library's device image: every GPU that
 * loads the library holds that array until the process exits. Limits: the operand form of the activation rows,
 * b2moe_expert_workspace_bytes(type, n*topk + shared_tokens, cols, B2MOE_F32) bytes (about 2 bytes per value), must fit the array, else B2MOE_ERR_CAPACITY and nothing is launched;
 * all calls on a device share the array, so calls that overlap on the GPU (different streams) race on it. The first
 * call on each device looks the array's device address up (with that device current) and should come before any
 * stream capture; later calls only launch (the cached address does not survive a cudaDeviceReset). A call that
 * resolves to the format-generic kernels uses no scratch and is not limited. Results are those of b2moe_expert_down. */
#define B2MOE_STATIC_SCRATCH_BYTES (16u << 20)
B2MOE_API size_t b2moe_static_scratch_bytes(void);
B2MOE_API int32_t b2moe_expert_down_static(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act,
                                 const int32_t * plan, int32_t n, int32_t topk, int32_t shared_tokens, float * y,
                                 b2moe_stream stream);
/* ---- the reference's per-matrix expert calls ------------------------------------------------------------------
 * The same products with the argument shapes of tqllm::WeightFormat's expert virtuals, for an adapter that implements
 * them (tqllm_b200/adapter/b200_expert_format.cpp): device ids or moe_group's (counts, groups) in, bf16 / fp16 rows per
 * assignment out, no plan to keep. Each call dispatches, multiplies and converts inside the caller's workspace.
 * b2moe_expert_matvec replaces WeightFormat::expert_matvec (src/formats/weight/weight_format.hpp:62-63):
 *   y[a][r] = W_ids[a][r] . x[per_expert_input ? a : a / topk] for every a with ids[a] >= 0; other rows stay untouched.
 * b2moe_expert_gemm replaces WeightFormat::expert_gemm (weight_format.hpp:51-53): the same over groups [experts][capacity]
 *   and counts [experts] as moe_group leaves them (src/experts/moe_kernels.cuh:29; capacity = tokens).
 * b2moe_expert_gemm_gateup replaces WeightFormat::expert_gemm_gateup (weight_format.hpp:58-59): act[a] = silu(gate . x) * (up . x).
 * b2moe_plan_from_groups turns moe_group's lists into a plan (no shared expert) for the plan-driven entry points.
 * Workspace: b2moe_expert_matvec_workspace_bytes(bank, n, topk) serves the first two,
 * b2moe_expert_gemm_gateup_workspace_bytes(gate, n, topk, x_dtype) the third; 16-byte aligned. */
B2MOE_API size_t b2moe_expert_matvec_workspace_bytes(const b2moe_bank * bank, int32_t n, int32_t topk);
B2MOE_API size_t b2moe_expert_gemm_gateup_workspace_bytes(const b2moe_bank * gate, int32_t n, int32_t topk, int32_t x_dtype);
B2MOE_API int32_t b2moe_plan_from_groups(const int32_t * counts, const int32_t * groups, int32_t capacity, int32_t experts,
                               int32_t assignments, int32_t * plan, b2moe_stream stream);
B2MOE_API int32_t b2moe_expert_matvec(const b2moe_bank * bank, const void * x, int32_t x_dtype, void * y, int32_t y_dtype, const int32_t * ids,
                            int32_t n, int32_t topk, int32_t per_expert_input, void * workspace, size_t workspace_bytes,
                            b2moe_stream stream);
B2MOE_API int32_t b2moe_expert_gemm(const b2moe_bank * bank, const void * x, int32_t x_dtype, void * y, int32_t y_dtype, const int32_t * counts,
                          const int32_t * groups, int32_t capacity, int32_t topk, int32_t per_expert_input, void * workspace,
                          size_t workspace_bytes, b2moe_stream stream);
B2MOE_API int32_t b2moe_expert_gemm_gateup(const b2moe_bank * gate, const b2moe_bank * up, const void * x, int32_t x_dtype, void * act,
                                 int32_t act_dtype, const int32_t * counts, const int32_t * groups, int32_t capacity, int32_t topk,
                                 void * workspace, size_t workspace_bytes, b2moe_stream stream);
/* moe_sum (src/experts/moe_kernels.cuh:73-74) and moe_swiglu (:71-72) on the reference's row types, and
 * WeightFormat::dequant_h (weight_format.hpp:78; workspace: experts * rows * cols floats). */
B2MOE_API int32_t b2moe_sum_rows(const void * routed, const void * shared, int32_t in_dtype, const float * weights, const float * shared_weights,
                       void * out, int32_t out_dtype, int32_t hidden, int32_t topk, int32_t n, b2moe_stream stream);
B2MOE_API int32_t b2moe_swiglu(const void * gate, const void * up, int32_t in_dtype, void * act, int32_t act_dtype, int64_t count,
                     b2moe_stream stream);
B2MOE_API int32_t b2moe_dequant_dump_as(const b2moe_bank * bank, void * out, int32_t out_dtype, void * workspace, size_t workspace_bytes,
                              b2moe_stream stream);

/* out[t] = sum_s weights[t][s] * y[t*topk + s] (slot order, skipped where ids[t][s] < 0 when ids is given)
 *          + shared_weights[t] (1 when null) * y[n*topk + t] when shared_tokens = n.
 * Replaces moe_sum / moe_common::moe_sum / fn_moe_combine (src/experts/moe.cu:223-234, src/experts/moe_common.cu:186-194,
 * src/models/qwen/qwen4exp/qwen4exp.cu:846-851). out is [n][hidden] of out_dtype. */
B2MOE_API int32_t b2moe_combine(const float * y, const int32_t * ids, const float * weights, const float * shared_weights, int32_t n,
                      int32_t topk, int32_t hidden, int32_t shared_tokens, void * out, int32_t out_dtype,
                      b2moe_stream stream);

/* The combine with the layer's skip connection fused (the residual add the engines do right after the MoE block,
 * src/models/qwen/qwen35/qwen35_forward.cpp:1113 add_sumsq, src/models/qwen/qwen4exp/fn_prefill.cpp:279-285): out[t] =
 * residual[t] + the weighted sum. residual is [n][hidden] of out_dtype and may be the out buffer itself. */
B2MOE_API int32_t b2moe_combine_residual(const float * y, const int32_t * ids, const float * weights, const float * shared_weights,
                               const void * residual, int32_t n, int32_t topk, int32_t hidden, int32_t shared_tokens, void * out,
                               int32_t out_dtype, b2moe_stream stream);

/* ---- expert parallelism --------------------------------------------------------------------------------------
 * Rank r of G owns the contiguous experts [first_expert, first_expert + local_experts); tokens are data-parallel and
 * router weights replicated. Per layer: all ranks exchange their activation rows and routed ids (NCCL, host-driven),
 * each rank maps the ids onto its own experts (b2moe_ep_local_ids: others become -1 and are skipped), runs dispatch /
 * gate-up / down on them, forms per-token partial sums with b2moe_combine (ids = the local ids), returns them to the
 * tokens' home ranks (NCCL all-to-all) and the home rank adds the partial sums in ascending rank order plus its own
 * shared expert (b2moe_ep_reduce). Generalises the reference's two-rank ep_local_ids / ep_gather / ep_scatter
 * (src/experts/moe.cu:496-541, src/experts/moe_kernels.cuh:40-50) to G ranks without a result cap. */
B2MOE_API int32_t b2moe_ep_local_ids(const int32_t * ids, int32_t * local_ids, int32_t count, int32_t first_expert,
                           int32_t local_experts, b2moe_stream stream);
/* parts: fp32 [ranks][n][hidden] (slice r = rank r's partial sums for this rank's n tokens); shared_y fp32 [n][hidden]
 * and shared_weights [n] may be NULL (no shared expert / weight 1). out [n][hidden] of out_dtype. */
B2MOE_API int32_t b2moe_ep_reduce(const float * parts, int32_t ranks, const float * shared_y, const float * shared_weights,
                        int32_t n, int32_t hidden, void * out, int32_t out_dtype, b2moe_stream stream);

/* All-to-all dispatch, for batches where gathering every token on every rank is too much: a rank sends a token only to the
 * ranks that own one of its routed experts, and always to itself (the shared expert then finds every own token in the local
 * batch). The exchange itself is two variable-size all-to-alls driven by the host (NCCL), preceded by a count exchange.
 * b2moe_ep_peer_lists: bounds [peers + 1] = first expert of every rank's block (device). For peer p, ascending token order:
 *   list[p][j] = j-th token sent to p, pos[p][t] = position of token t in p's list or -1, counts[p] = list length
 *   (pos, list: [peers][n] ints).
 * b2moe_ep_pack: records = sum of counts; offsets [peers + 1] = prefix sums of counts (device). A record is the activation
 *   row (x_row_bytes, a multiple of 16), topk int32 routed ids, topk fp32 weights; 8 * topk must be a multiple of 16.
 * b2moe_ep_unpack: received records -> x rows, local ids (ids outside [first_expert, first_expert + local_experts) become -1)
 *   and weights, ready for b2moe_dispatch_range and the expert products.
 * b2moe_ep_return_reduce: back = the partial sums that came home, in the order the records were sent;
 *   out[t] = sum over peers in ascending order of back[offsets[p] + pos[p][t]] + shared_weights[t] * shared_y[t]. */
B2MOE_API int32_t b2moe_ep_peer_lists(const int32_t * ids, int32_t n, int32_t topk, const int32_t * bounds, int32_t peers, int32_t self,
                            int32_t * counts, int32_t * pos, int32_t * list, b2moe_stream stream);
B2MOE_API int32_t b2moe_ep_pack(const void * x, int32_t x_row_bytes, const int32_t * ids, const float * weights, int32_t topk, int32_t n,
                      const int32_t * list, const int32_t * offsets, int32_t peers, int32_t records, void * out, b2moe_stream stream);
B2MOE_API int32_t b2moe_ep_unpack(const void * records_in, int32_t records, int32_t x_row_bytes, int32_t topk, int32_t first_expert,
                        int32_t local_experts, void * x, int32_t * local_ids, float * weights, b2moe_stream stream);
B2MOE_API int32_t b2moe_ep_return_reduce(const float * back, const int32_t * pos, const int32_t * offsets, int32_t peers, const float * shared_y,
                               const float * shared_weights, int32_t n, int32_t hidden, void * out, int32_t out_dtype,
                               b2moe_stream stream);

/* Exchanges over peer memory for the small messages of decode batches (one process per GPU on one NVLink / NVSwitch node),
 * in place of the library collectives between the compute phases: the reference sends and receives with grouped
 * ncclSend / ncclRecv (src/models/qwen/qwen4exp/fn_layer_forward.cpp:475-503). Only plain peer loads and stores cross the
 * link; no multicast object is bound.
 * b2moe_peer_alloc: a zeroed device allocation of `bytes` and its 64-byte inter-process handle; b2moe_peer_open maps a
 *   peer's allocation from its handle (same node, another process) and enables peer access; b2moe_peer_close /
 *   b2moe_peer_free undo them. An inbox is an allocation with one slot per sender; a counter row is one int32 per sender.
 * b2moe_peer_put: for every peer p, `bytes` (a multiple of 16) from src + p * src_stride (stride 0: the same block to
 *   everyone) are stored to dst[p] (this sender's slot in p's inbox; device array of `peers` pointers) and then, after a
 *   system-wide fence, `seq` is stored to flags[p] (this sender's counter at p). tickets: `peers` + 2 zeroed int32 of local
 *   scratch. seq <= 0: the launch numbers the exchange itself (one more than the last, kept in tickets[peers + 1]), so
 *   that the same launch can be replayed from a CUDA graph.
 * b2moe_peer_wait: returns (on the stream) once each of the `peers` local counters has reached `seq` (seq <= 0: one more
 *   than at the last wait, kept in counters[peers]: the row needs peers + 1 words); a counter that has
 *   not after two to three seconds sets *status (device int32, 0 before) to 1 + its index and the kernel returns: it never
 *   spins without a bound. A slot may be written again only after its reader has finished with it; the order of an
 *   expert-parallel layer gives that (a rank sends exchange s + 1 only after it has received all of exchange s). */
B2MOE_API int32_t b2moe_peer_alloc(size_t bytes, void ** ptr, uint8_t handle[64]);
B2MOE_API int32_t b2moe_peer_open(const uint8_t handle[64], void ** ptr);
B2MOE_API int32_t b2moe_peer_close(void * ptr);
B2MOE_API int32_t b2moe_peer_free(void * ptr);
B2MOE_API int32_t b2moe_peer_put(const void * src, size_t src_stride, size_t bytes, void * const * dst, int32_t * const * flags,
                       int32_t * tickets, int32_t peers, int32_t seq, b2moe_stream stream);
B2MOE_API int32_t b2moe_peer_wait(int32_t * counters, int32_t peers, int32_t seq, int32_t * status, b2moe_stream stream);

/* ---- GGUF expert reader and bank packer (host code, host pointers; no CUDA call) ------------------------------------
 * Replaces the expert-serving part of the reference's reader: gguf_expert_count / gguf_expert_slice
 * (src/core/gguf.hpp:77-91, src/core/gguf.cpp:174-213) with the block table of the five expert formats (gguf.cpp:116-152),
 * and the loaders' device repack: the packed result is a finished bank, like the reference's packed expert file
 * (src/experts/packed_experts.hpp:2-5). The file (GGUF version 2 or 3) is mapped read-only by b2moe_gguf_open; a file whose
 * header, alignment or byte ranges are inconsistent is refused with B2MOE_ERR_FORMAT.
 * b2moe_gguf_tensor: type, dims {cols, rows, experts} (1 beyond the rank), offset in the file and byte count (0 when the
 *   block format is not one of the five) of a tensor by name; B2MOE_ERR_SHAPE when there is no such tensor.
 * b2moe_gguf_expert_slice: experts [first, first + count) of a 3-D expert tensor as a pointer into the mapping (raw GGUF
 *   rows, expert-major): one expert or a rank's block without reading the others. A 2-D tensor (a shared expert's matrix)
 *   counts as one expert.
 * b2moe_gguf_expert_bank: the same experts packed into the bank layout of bank_type (the tensor's type, or
 *   B2MOE_IQ3_S_X4 for an IQ3_S tensor): data / aux sized by b2moe_bank_bytes / b2moe_bank_aux_bytes(bank_type, count *
 *   rows, cols); rows must be a multiple of 16. */
B2MOE_API int32_t b2moe_gguf_open(const char * path, void ** handle);
B2MOE_API void b2moe_gguf_close(void * handle);
B2MOE_API int32_t b2moe_gguf_tensor_count(const void * handle);
B2MOE_API int32_t b2moe_gguf_tensor_name(const void * handle, int32_t index, char * name, int32_t name_bytes);
B2MOE_API int32_t b2moe_gguf_tensor(const void * handle, const char * name, uint32_t * type, int64_t dims[3], uint64_t * offset, uint64_t * bytes);
B2MOE_API int32_t b2moe_gguf_expert_slice(const void * handle, const char * name, int32_t first, int32_t count, uint32_t * type, int32_t * rows,
                                int32_t * cols, const void ** raw, uint64_t * raw_bytes);
B2MOE_API int32_t b2moe_gguf_expert_bank(const void * handle, const char * name, int32_t first, int32_t count, uint32_t bank_type, void * data,
                               void * aux);

/* Skew handling. b2moe_count replaces moe_count (src/experts/moe.cu:183-186, src/experts/moe_kernels.cuh:54): counts[e] += the
 * number of ids equal to e, accumulated over calls into a device array of `experts` 64-bit counters the caller zeroed
 * (ids outside [0, experts) are skipped). b2moe_place_experts (host code, host pointers) turns such a histogram into a
 * load-aware placement for `ranks` GPUs: greedy longest-first bin packing under the constraint that every rank holds
 * experts / ranks experts. order[r * per + i] = the expert in slot i of rank r; a loader that stacks the router rows, the
 * selection bias and the three banks in this order keeps the contiguous-block ownership the other calls assume (the layer's
 * result does not depend on the order). rank_load (may be null) receives the summed counts per rank. */
B2MOE_API int32_t b2moe_count(const int32_t * ids, uint64_t * counts, int32_t count, int32_t experts, b2moe_stream stream);
B2MOE_API int32_t b2moe_place_experts(const uint64_t * counts, int32_t experts, int32_t ranks, int32_t * order, uint64_t * rank_load);

/* ---- harness hooks ---------------------------------------------------------------------------------------------
 * For tests and benchmarks, not for engines: process-wide switches, not thread-safe, to be set while no call of this
 * library is running. They have no counterpart in the reference.
 * b2moe_harness_select: family = the kernel family every later expert product takes where it supports the shape
 * (AUTO = the library's own choice by tokens per expert, the default); gemm_item_tokens = 128 (default; 0 means the
 * same) or 256 tokens per work item of the grouped GEMM.
 * b2moe_harness_wait_probe: the 4-bit decode kernels skip the copy of weight tile number drop_tile of every warp
 * (-1 = none, the default) and bound each wait by wait_limit polls (0 = default), so that a test can watch a bounded
 * wait run out: the launch then sets plan word [3] and returns, its outputs invalid.
 * b2moe_harness_skip_staging: while on, the 4-bit decode kernels skip their activation staging launch and read the
 * staged rows the previous call left in the same workspace (a benchmark times the product kernel alone this way).
 * b2moe_harness_overlap: on (the default), the launches of a layer call are chained by programmatic dependent launch: a
 * kernel may become resident and set up its shared memory while the one before it drains, and waits on the device for
 * that one's completion before it touches global memory; off = plain stream order (for A/B timing).
 * b2moe_harness_ring: forces the shared-memory configuration of the 4-bit decode kernels (activation buffers 1-2, ring
 * stages 2-4, tiles per slot 1-2) where it fits; zeros = the library's own order of preference.
 * b2moe_harness_column_split: the most warps (1, 2 or 4; default 4) that the 4-bit decode kernels let share one row job
 * when a launch has only a few jobs per block; 1 switches the split off.
 * b2moe_harness_launches: kernel launches the library has made in this process so far. */
enum b2moe_family { B2MOE_FAMILY_AUTO = 0, B2MOE_FAMILY_GENERIC = 1, B2MOE_FAMILY_DECODE = 2, B2MOE_FAMILY_GEMM = 3 };
B2MOE_API void b2moe_harness_select(int32_t family, int32_t gemm_item_tokens);
B2MOE_API void b2moe_harness_wait_probe(int32_t drop_tile, uint32_t wait_limit);
B2MOE_API void b2moe_harness_skip_staging(int32_t on);
B2MOE_API void b2moe_harness_overlap(int32_t on);
B2MOE_API void b2moe_harness_ring(int32_t activation_buffers, int32_t stages, int32_t slot_tiles);
B2MOE_API void b2moe_harness_column_split(int32_t max_warps_per_job);
B2MOE_API uint64_t b2moe_harness_launches(void);

/* ---- whole layer ----------------------------------------------------------------------------------------------
 * router -> top-k -> dispatch -> gate/up + SwiGLU -> down -> combine, the sequence of qwen35_forward.cpp:1121-1252,
 * fn_layer_forward.cpp:311-336,504-522 and minimax.cpp:1083-1131, as stream-ordered launches with no host round trip. */
typedef struct b2moe_layer {
    int32_t hidden, experts, topk, ff;
    int32_t gating;                /* b2moe_gating */
    int32_t norm;                  /* sigmoid gating: normalise the selected weights (softmax gating always does) */
    float scale;                   /* 0 and 1 both mean "no scaling" (src/experts/moe.hpp:33) */
    int32_t has_shared;            /* 1: an always-on expert is evaluated for every token */
    const float * router_w;        /* f32 [experts][hidden] */
    const float * sel_bias;        /* f32 [experts] selection-only bias (sigmoid gating) or NULL */
    const float * shared_gate_vec; /* f32 [hidden]: shared weight = sigmoid(vec . x); NULL = weight 1 */
    b2moe_bank gate, up, down;     /* experts stacked */
    b2moe_bank sh_gate, sh_up, sh_down; /* experts = 1; ignored unless has_shared */
} b2moe_layer;

/* byte offsets of the intermediates inside a layer workspace (so a harness can read the routing artefacts back) */
typedef struct b2moe_layer_ws {
    size_t logits;         /* f32 [n][experts + 1] */
    size_t ids;            /* i32 [n][topk] */
    size_t weights;        /* f32 [n][topk] */
    size_t shared_weights; /* f32 [n] */
    size_t plan;           /* i32 [b2moe_plan_ints] */
    size_t act;            /* f32 [n*topk + shared][ff] */
    size_t y;              /* f32 [n*topk + shared][hidden] */
    size_t scratch;        /* dispatch scratch */
    size_t expert_scratch; /* scratch of the expert products */
    size_t total;          /* workspace bytes needed */
} b2moe_layer_ws;
B2MOE_API int32_t b2moe_layer_workspace(const b2moe_layer * layer, int32_t n, b2moe_layer_ws * ws);
B2MOE_API int32_t b2moe_layer_forward(const b2moe_layer * layer, const void * x, int32_t x_dtype, int32_t n, void * out,
                            int32_t out_dtype, void * workspace, size_t workspace_bytes, b2moe_stream stream);
/* b2moe_layer_forward with the skip connection: out = residual + layer(x) (b2moe_combine_residual as its last launch). */
B2MOE_API int32_t b2moe_layer_forward_residual(const b2moe_layer * layer, const void * x, int32_t x_dtype, int32_t n, const void * residual,
                                     void * out, int32_t out_dtype, void * workspace, size_t workspace_bytes, b2moe_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* B2MOE_H */
