// Expert-parallel exchanges over peer memory (NVLink / NVSwitch, one process per GPU): every rank owns an inbox with one
// slot per sender and a row of arrival counters; a sender's kernel stores its block straight into the receivers' inboxes
// and then raises their counters, the receiver's kernel waits (bounded) until every sender's counter has reached the
// exchange's sequence number. Replaces the library collectives between the compute phases of an expert-parallel layer (the
// reference sends and receives with grouped ncclSend / ncclRecv, src/models/qwen/qwen4exp/fn_layer_forward.cpp:475-503) for
// the small messages of decode batches, where a collective's latency is several times the transfer time.
//
// Memory: inboxes and counters are plain cudaMalloc allocations exported with cudaIpcGetMemHandle and opened by the peers
// (cudaIpcOpenMemHandle enables peer access); only ordinary loads and stores cross the link: no multicast object is bound.
// Order: a sender's data stores, a system-wide fence, then the counter store; the receiver polls the counter with
// volatile loads and its later kernels read the inbox (a kernel boundary). A slot is reused only after its reader has
// finished, which the layer's own order gives: a rank sends exchange s + 1 after it has received everything of exchange s.
#include <cstring>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int PUT_THREADS = 256;
constexpr uint32_t PEER_WAIT_TRIES = 1u << 24;     // polls of 100 to 200 ns: the wait gives up after two to three seconds

struct PutArgs {
    const uint8_t * src;        // the sender's data
    size_t src_stride;          // bytes between the blocks for consecutive peers (0: the same block goes to everyone)
    size_t bytes;               // bytes per peer, a multiple of 16
    void * const * dst;         // [peers] device array: this sender's slot in every peer's inbox
    int * const * flag;         // [peers] device array: this sender's counter in every peer's counter row
    int * tickets;              // [peers + 2] local scratch: a ticket per peer and one for the launch (zero between launches), the sequence counter
    int peers, blocks_per_peer, seq;   // seq <= 0: the number of this exchange is tickets[peers + 1] + 1, and the launch advances it
};

// grid = peers x blocks_per_peer; the last block of a peer's group to finish raises that peer's counter
__global__ void __launch_bounds__(PUT_THREADS) peer_put_k(const PutArgs a) {
    const int peer = blockIdx.x / a.blocks_per_peer, part = blockIdx.x % a.blocks_per_peer;
    // the counter is advanced by the last block of the launch to finish, after every block has read it (below)
    const int seq = a.seq > 0 ? a.seq : *reinterpret_cast<volatile int *>(a.tickets + a.peers + 1) + 1;
    const uint4 * src = reinterpret_cast<const uint4 *>(a.src + size_t(peer) * a.src_stride);
    uint4 * dst = static_cast<uint4 *>(a.dst[peer]);
    const size_t n16 = a.bytes >> 4;
    for (size_t i = size_t(part) * PUT_THREADS + threadIdx.x; i < n16; i += size_t(a.blocks_per_peer) * PUT_THREADS) dst[i] = src[i];
    __threadfence_system();                                            // this thread's stores are visible to the peer before the counter
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(a.tickets + peer, 1);
        if (ticket == a.blocks_per_peer - 1) {
            a.tickets[peer] = 0;                                        // ready for the next launch (stream order)
            __threadfence_system();
            *reinterpret_cast<volatile int *>(a.flag[peer]) = seq;
        }
        if (a.seq <= 0 && atomicAdd(a.tickets + a.peers, 1) == int(gridDim.x) - 1) {       // every block has its seq by now
            a.tickets[a.peers] = 0;
            a.tickets[a.peers + 1] = seq;
        }
    }
}

// one block; thread p waits for sender p's counter. status: 0 = all arrived, otherwise 1 + the first sender that did not.
// seq_in <= 0: the number of this exchange is counters[peers] + 1 (a word of the row that no sender writes), advanced here
__global__ void peer_wait_k(int * counters, int peers, int seq_in, int * status) {
    const int p = threadIdx.x;
    const int seq = seq_in > 0 ? seq_in : *reinterpret_cast<volatile int *>(counters + peers) + 1;
    __syncthreads();                                                   // everyone has read the number before thread 0 advances it
    if (seq_in <= 0 && p == 0) counters[peers] = seq;
    bool ok = true;
    if (p < peers) {
        const volatile int * c = counters + p;
        ok = false;
        for (uint32_t i = 0; i < PEER_WAIT_TRIES; ++i) {
            if (*c - seq >= 0) { ok = true; break; }
            __nanosleep(100);
        }
    }
    __threadfence_system();
    if (!ok) atomicCAS(status, 0, 1 + p);
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API int32_t b2moe_peer_alloc(size_t bytes, void ** ptr, uint8_t handle[64]) {
    if (!ptr || !handle) return B2MOE_ERR_NULL;
    if (bytes == 0) return B2MOE_ERR_SHAPE;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the exported handle is 64 bytes");
    void * p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return B2MOE_ERR_CUDA;
    cudaIpcMemHandle_t h;
    // the zeroing must have finished before any peer can write here: wait for it (set-up time, never inside a capture)
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaStreamSynchronize(nullptr) != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaFree(p);
        cudaGetLastError();
        return B2MOE_ERR_CUDA;
    }
    std::memcpy(handle, &h, 64);
    *ptr = p;
    return B2MOE_OK;
}
extern "C" B2MOE_API int32_t b2moe_peer_open(const uint8_t handle[64], void ** ptr) {
    if (!ptr || !handle) return B2MOE_ERR_NULL;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return B2MOE_ERR_CUDA; }
    return B2MOE_OK;
}
extern "C" B2MOE_API int32_t b2moe_peer_close(void * ptr) {
    if (!ptr) return B2MOE_ERR_NULL;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? B2MOE_OK : B2MOE_ERR_CUDA;
}
extern "C" B2MOE_API int32_t b2moe_peer_free(void * ptr) {
    if (!ptr) return B2MOE_ERR_NULL;
    return cudaFree(ptr) == cudaSuccess ? B2MOE_OK : B2MOE_ERR_CUDA;
}

extern "C" B2MOE_API int32_t b2moe_peer_put(const void * src, size_t src_stride, size_t bytes, void * const * dst, int32_t * const * flags,
                                            int32_t * tickets, int32_t peers, int32_t seq, b2moe_stream stream) {
    if (!src || !dst || !flags || !tickets) return B2MOE_ERR_NULL;
    if (peers <= 0 || peers > 1024 || bytes == 0 || bytes % 16 || src_stride % 16) return B2MOE_ERR_SHAPE;
    if (!aligned16(src)) return B2MOE_ERR_ALIGN;
    PutArgs a{};
    a.src = static_cast<const uint8_t *>(src); a.src_stride = src_stride; a.bytes = bytes; a.dst = dst; a.flag = flags; a.tickets = tickets;
    a.peers = peers; a.seq = seq;
    a.blocks_per_peer = int(std::min<size_t>(16, std::max<size_t>(1, (bytes >> 4) / (4 * PUT_THREADS))));   // at least four 16-byte stores per thread
    peer_put_k<<<peers * a.blocks_per_peer, PUT_THREADS, 0, as_stream(stream)>>>(a);
    return launch_status();
}
extern "C" B2MOE_API int32_t b2moe_peer_wait(int32_t * counters, int32_t peers, int32_t seq, int32_t * status, b2moe_stream stream) {
    if (!counters || !status) return B2MOE_ERR_NULL;
    if (peers <= 0 || peers > 1024) return B2MOE_ERR_SHAPE;
    peer_wait_k<<<1, (peers + 31) / 32 * 32, 0, as_stream(stream)>>>(counters, peers, seq, status);
    return launch_status();
}
