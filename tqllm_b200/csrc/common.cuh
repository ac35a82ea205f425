// Shared host-side helpers of the C ABI: status codes, argument checks, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b2moe.h"

namespace b2 {

// every kernel launch of the library is followed by launch_status(): it also counts them (b2moe_harness_launches)
extern unsigned long long g_launch_count;
inline int32_t launch_status() {
    ++g_launch_count;
    return cudaGetLastError() == cudaSuccess ? B2MOE_OK : B2MOE_ERR_CUDA;
}
// Programmatic dependent launch for the chain of small launches of one layer call: a kernel launched through launch_overlapped
// may become resident while the launch before it on the stream is still running; it runs its prologue (barrier and shared-
// memory setup, no global access) and then every thread calls grid_wait(), which returns once the earlier launches have
// completed and their writes are visible. grid_release() lets the launch after this one do the same. A kernel that is
// launched this way must call grid_wait() in every thread before its first global access and before any early return,
// so that completion stays transitive along the chain. g_overlap = false (b2moe_harness_overlap) falls back to plain launches.
extern bool g_overlap;
__device__ __forceinline__ void grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = g_overlap ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);       // the error, if any, is read by launch_status()
}
inline bool aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline cudaStream_t as_stream(b2moe_stream s) { return static_cast<cudaStream_t>(s); }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// activation element -> float
template <int DT> struct Elem;
template <> struct Elem<B2MOE_F32> { using type = float; __device__ static float to_f(float v) { return v; } };
template <> struct Elem<B2MOE_F16> { using type = __half; __device__ static float to_f(__half v) { return __half2float(v); } };
template <> struct Elem<B2MOE_BF16> { using type = __nv_bfloat16; __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); } };

__device__ __forceinline__ float load_act(const void * x, int dtype, size_t i) {
    if (dtype == B2MOE_F32) return static_cast<const float *>(x)[i];
    if (dtype == B2MOE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(x)[i]);
    return __half2float(static_cast<const __half *>(x)[i]);
}
__device__ __forceinline__ void store_act(void * x, int dtype, size_t i, float v) {
    if (dtype == B2MOE_F32) static_cast<float *>(x)[i] = v;
    else if (dtype == B2MOE_BF16) static_cast<__nv_bfloat16 *>(x)[i] = __float2bfloat16_rn(v);
    else static_cast<__half *>(x)[i] = __float2half_rn(v);
}
inline bool valid_dtype(int dt) { return dt == B2MOE_F32 || dt == B2MOE_F16 || dt == B2MOE_BF16; }
inline size_t dtype_bytes(int dt) { return dt == B2MOE_F32 ? 4 : 2; }

// plan header slots
enum { PLAN_NACTIVE = 0, PLAN_NGROUPED = 1, PLAN_NPASS = 2, PLAN_STATUS = 3, PLAN_HDR = 4 };
// tokens of one expert that one pass of the decode kernels takes; the plan's pass list is cut in these units
constexpr int PASS_TOKENS = 8;

}  // namespace b2
