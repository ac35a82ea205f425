// Reference-side shims: tqLLM's free functions of the expert path (namespace tqllm_cuda, src/experts/moe_kernels.cuh:7-82,
// src/experts/moe_common.cuh:11-22) expressed through the C ABI of include/b2moe.h. A tqLLM build links this file and
// libb2moe.so instead of src/experts/moe.cu / moe_common.cu. Same argument order and meaning as the reference; errors
// become the reference's exceptions (std::invalid_argument for shapes, std::runtime_error for launch failures,
// src/experts/moe.cu:239,250, src/experts/moe_common.cu:10-13). Compile check: tests/test_adapter_compiles.py.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "b2moe.h"

namespace tqllm_cuda {

static void b2_check(int32_t rc, const char * what) {
    if (rc == B2MOE_ERR_CUDA) throw std::runtime_error(std::string(what) + ": " + b2moe_status_string(rc));
    if (rc != B2MOE_OK) throw std::invalid_argument(std::string(what) + ": " + b2moe_status_string(rc));
}

// moe_kernels.cuh:8-9: logits [n][experts + 1] = router . x (+ the shared gate row); fp16 activations
void moe_router(const float * router, const float * shared_gate, const __half * x, float * logits, int hidden, int experts, int n,
                cudaStream_t s) {
    b2_check(b2moe_router(router, shared_gate, x, B2MOE_F16, logits, experts + 1, hidden, experts, n, s), "moe_router");
}

// moe_kernels.cuh:19-20: softmax top-k, renormalised weights, sigmoid of the shared logit
void moe_topk(const float * logits, int * ids, float * weights, float * shared_weights, int experts, int topk, int n, float scale,
              cudaStream_t s) {
    b2_check(b2moe_topk_softmax(logits, experts + 1, ids, weights, shared_weights, experts, topk, n, scale, s), "moe_topk");
}

namespace moe_common {
// moe_common.cuh:11-12: sigmoid scores, bias only in the selection, optional renormalisation, scale
void route(const float * logits, const float * bias, int * ids, float * w, int experts, int k, bool norm, float scale, cudaStream_t s,
           int n) {
    b2_check(b2moe_route_sigmoid(logits, experts, bias, ids, w, experts, k, norm ? 1 : 0, scale, n, s), "route");
}
}  // namespace moe_common

// moe_kernels.cuh:29: counts [experts], groups [experts][n]. `plan` and `scratch` come from the engine's per-layer arena
// (b2moe_plan_ints, b2moe_dispatch_workspace_bytes). Unlike the reference's atomics the lists come out in ascending
// assignment order every time.
void moe_group(const int * ids, int * counts, int * groups, int experts, int n, int topk, cudaStream_t s, int32_t * plan, void * scratch,
               size_t scratch_bytes) {
    b2_check(b2moe_dispatch(ids, n, topk, experts, 0, plan, scratch, scratch_bytes, s), "moe_group");
    b2_check(b2moe_plan_to_groups(plan, n, topk, experts, counts, groups, s), "moe_group");
}

// moe_kernels.cuh:71-72 (moe_sum): out[t] = sum over the token's slots of weights[t][s] * y[t * topk + s] (+ the shared
// expert's row times its weight); per-assignment rows are fp32 here, the output bf16 as in the reference
void moe_sum(const float * y, const float * weights, const float * shared_weights, int n, int topk, int hidden, int shared_tokens,
             void * out_bf16, cudaStream_t s) {
    b2_check(b2moe_combine(y, nullptr, weights, shared_weights, n, topk, hidden, shared_tokens, out_bf16, B2MOE_BF16, s), "moe_sum");
}

// The gate/up product with the SwiGLU fused and the down product, over a plan built by moe_group / b2moe_dispatch: what
// WeightFormat::expert_matvec2 + moe_swiglu and WeightFormat::expert_matvec(per_expert_input) compute
// (src/formats/weight/weight_format.hpp:62-73), for an adapter class to forward to.
void expert_gateup_swiglu(const b2moe_bank & gate, const b2moe_bank & up, const __half * x, const int32_t * plan, int n, int topk, float * act,
                          void * workspace, size_t workspace_bytes, cudaStream_t s) {
    b2_check(b2moe_expert_gateup_swiglu(&gate, &up, nullptr, nullptr, x, B2MOE_F16, plan, n, topk, 0, act, workspace, workspace_bytes, s),
             "expert_gateup_swiglu");
}
void expert_down(const b2moe_bank & down, const float * act, const int32_t * plan, int n, int topk, float * y, void * workspace,
                 size_t workspace_bytes, cudaStream_t s) {
    b2_check(b2moe_expert_down(&down, nullptr, act, plan, n, topk, 0, y, workspace, workspace_bytes, s), "expert_down");
}

}  // namespace tqllm_cuda
