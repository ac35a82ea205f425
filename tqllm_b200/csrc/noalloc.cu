// b2moe_expert_down_static: the down product for callers that have no way to hand the library scratch memory.
//
// Some hosts of this library cannot allocate device memory themselves: a plugin loaded into an engine whose memory
// is fully owned and pre-partitioned by that engine (the engine hands the plugin input and output pointers and
// nothing else), or code running inside a region where cudaMalloc is forbidden, such as a stream capture or a
// callback on a latency-critical serving thread. b2moe_expert_down needs scratch for the tensor-core operand form of the
// activation rows when the bank has a tensor-core kernel; this entry point keeps that scratch in a fixed array inside
// the library's own device image instead, so the call allocates nothing and takes no workspace argument.
//
// Cost and limits: every GPU that loads the library carries the B2MOE_STATIC_SCRATCH_BYTES array until the process
// exits. Calls whose split does not fit are rejected with B2MOE_ERR_CAPACITY. All calls on one device share the one
// array: two calls that overlap on the GPU (different streams) race on it; calls on one stream are safe. The array
// keeps whatever the previous call left; the kernels overwrite every row they read, so nothing needs clearing.
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "formats.cuh"

namespace b2 {
int32_t check_bank(const b2moe_bank * b);
bool expert_down_is_generic(const b2moe_bank * down, int n, int topk);

namespace {

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[B2MOE_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_mutex;
void * g_scratch_of[MAX_DEVICES] = {};          // device address of the array, per device ordinal (null = not yet asked)

// Device address of the scratch array on the current device. The first call on a device asks the runtime for it
// (with that device current); later calls read the cached pointer.
int32_t static_scratch(void ** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return B2MOE_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_of[dev]) {
        void * p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return B2MOE_ERR_CUDA;
        g_scratch_of[dev] = p;
    }
    *out = g_scratch_of[dev];
    return B2MOE_OK;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API size_t b2moe_static_scratch_bytes(void) { return B2MOE_STATIC_SCRATCH_BYTES; }

extern "C" B2MOE_API int32_t b2moe_expert_down_static(const b2moe_bank * down, const b2moe_bank * shared_down, const float * act,
                                                      const int32_t * plan, int32_t n, int32_t topk, int32_t shared_tokens, float * y,
                                                      b2moe_stream stream) {
    if (int32_t rc = check_bank(down)) return rc;
    if (n <= 0 || topk <= 0 || (shared_tokens != 0 && shared_tokens != n) || (long long)n * topk > 0x3fffffffLL) return B2MOE_ERR_SHAPE;
    if (shared_tokens) {
        if (int32_t rc = check_bank(shared_down)) return rc;
        if (shared_down->type != down->type) return B2MOE_ERR_FORMAT;
        if (shared_down->rows != down->rows || shared_down->cols != down->cols) return B2MOE_ERR_SHAPE;
    }
    if (!act || !plan || !y) return B2MOE_ERR_NULL;
    if (!aligned16(act) || !aligned16(y)) return B2MOE_ERR_ALIGN;
    // the same kernels as b2moe_expert_down, with the library's own array as their workspace
    // (a call that takes the format-generic kernels uses no scratch: b2moe_expert_down ignores the workspace then)
    const size_t need = expert_down_is_generic(down, n, topk) ? 0
                                                              : b2moe_expert_workspace_bytes(down->type, n * topk + shared_tokens, down->cols, B2MOE_F32);
    if (need > B2MOE_STATIC_SCRATCH_BYTES) return B2MOE_ERR_CAPACITY;
    void * scratch = nullptr;
    if (need) {
        if (int32_t rc = static_scratch(&scratch)) return rc;
    }
    return b2moe_expert_down(down, shared_down, act, plan, n, topk, shared_tokens, y, scratch, need ? B2MOE_STATIC_SCRATCH_BYTES : 0, stream);
}
