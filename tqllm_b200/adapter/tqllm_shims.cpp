// Reference-side shims: tqLLM's free functions of the expert path (namespace tqllm_cuda, src/experts/moe_kernels.cuh:7-82,
// src/experts/moe_common.cuh:11-22) expressed through the C ABI of include/b2moe.h. A tqLLM build links this file and
// libb2moe.so instead of src/experts/moe.cu / moe_common.cu. Same argument order and meaning as the reference; errors
// become the reference's exceptions (std::invalid_argument for shapes, std::runtime_error for launch failures,
// src/experts/moe.cu:239,250, src/experts/moe_common.cu:10-13). Compile check: tests/test_adapter_compiles.py.
#include <cuda_bf16.h>
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

// moe_kernels.cuh:24-25: moe_topk on two routings in one launch (this layer's and the next layer's prediction); e <= 1024
void moe_topk2(const float * logits, int * ids, float * weights, float * shared_weights, const float * logits2, int * ids2, float * weights2,
               float * shared_weights2, int e, int k, int n, float scale, cudaStream_t s) {
    if (e > 1024) throw std::invalid_argument("moe_topk2: invalid shape");
    b2_check(b2moe_topk_softmax2(logits, ids, weights, shared_weights, logits2, ids2, weights2, shared_weights2, e + 1, e, k, n, scale, s), "moe_topk2");
}

namespace moe_common {
// moe_common.cuh:11-12: sigmoid scores, bias only in the selection, optional renormalisation, scale
void route(const float * logits, const float * bias, int * ids, float * w, int experts, int k, bool norm, float scale, cudaStream_t s,
           int n) {
    b2_check(b2moe_route_sigmoid(logits, experts, bias, ids, w, experts, k, norm ? 1 : 0, scale, n, s), "route");
}
}  // namespace moe_common

// Device scratch of the shims that need one (moe_group): owned by the engine, set once per engine thread.
static thread_local struct { void * p = nullptr; size_t bytes = 0; } g_scratch;
void b200_set_shim_scratch(void * device_ptr, size_t bytes) { g_scratch.p = device_ptr; g_scratch.bytes = bytes; }
size_t b200_shim_scratch_bytes(int experts, int n, int topk) {
    return size_t(b2moe_plan_ints(experts, n * topk, 0)) * sizeof(int32_t) + 256 + b2moe_dispatch_workspace_bytes(experts, n * topk);
}

// moe_kernels.cuh:29: counts [experts], groups [experts][n]; negative ids are skipped. Unlike the reference's atomics the
// lists come out in ascending assignment order every time. The plan and the dispatch scratch live in the shim scratch.
void moe_group(const int * ids, int * counts, int * groups, int experts, int n, int topk, cudaStream_t s) {
    const size_t plan_bytes = (size_t(b2moe_plan_ints(experts, n * topk, 0)) * sizeof(int32_t) + 255) / 256 * 256;
    if (!g_scratch.p || g_scratch.bytes < b200_shim_scratch_bytes(experts, n, topk)) throw std::invalid_argument("moe_group: shim scratch missing or too small");
    int32_t * plan = static_cast<int32_t *>(g_scratch.p);
    b2_check(b2moe_dispatch(ids, n, topk, experts, 0, plan, static_cast<char *>(g_scratch.p) + plan_bytes, g_scratch.bytes - plan_bytes, s), "moe_group");
    b2_check(b2moe_plan_to_groups(plan, n, topk, experts, counts, groups, s), "moe_group");
}

// moe_kernels.cuh:71-72: act = silu(gate) * up over `count` values, bf16 in, fp16 out
void moe_swiglu(const __nv_bfloat16 * gate, const __nv_bfloat16 * up, __half * act, int count, cudaStream_t s) {
    b2_check(b2moe_swiglu(gate, up, B2MOE_BF16, act, B2MOE_F16, count, s), "moe_swiglu");
}

// moe_kernels.cuh:73-74: out[t] = sum_s weights[t][s] * routed[t * topk + s] + shared_weights[t] * shared[t]; bf16 rows
void moe_sum(const __nv_bfloat16 * routed, const __nv_bfloat16 * shared, const float * weights, const float * shared_weights,
             __nv_bfloat16 * out, int hidden, int topk, int n, cudaStream_t s) {
    b2_check(b2moe_sum_rows(routed, shared, B2MOE_BF16, weights, shared_weights, out, B2MOE_BF16, hidden, topk, n, s), "moe_sum");
}

}  // namespace tqllm_cuda
