// B200ExpertFormat: the reference's WeightFormat virtuals of the expert path (src/formats/weight/weight_format.hpp:33-110)
// on top of the C ABI of include/b2moe.h. Same argument meaning as the reference's built-in formats: stacked weights
// [experts * rows][cols], device ids [n][topk] with -1 = skip, outputs [n * topk][rows] in bf16 (fp16 for the fused
// gate/up + SwiGLU), errors as std::invalid_argument / std::runtime_error, `false` from the expert_gemm* calls = "not
// supported, the caller falls back" (weight_format.hpp:51-53).
#include "b200_expert_format.hpp"

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "b2moe.h"

namespace b2adapter {
namespace {

struct Workspace { void * p = nullptr; size_t bytes = 0; };
thread_local Workspace g_ws;

void check(int32_t rc, const char * what) {
    if (rc == B2MOE_ERR_CUDA) throw std::runtime_error(std::string(what) + ": " + b2moe_status_string(rc));
    if (rc != B2MOE_OK) throw std::invalid_argument(std::string(what) + ": " + b2moe_status_string(rc));
}
size_t up256(size_t v) { return (v + 255) / 256 * 256; }

class B200ExpertFormat final : public tqllm::WeightFormat {
public:
    B200ExpertFormat(uint32_t gguf_type, bool codes) : gguf_(gguf_type), bank_type_(gguf_type == B2MOE_IQ3_S && codes ? uint32_t(B2MOE_IQ3_S_X4) : gguf_type) {}
    const char * name() const override { return "b200-expert"; }
    tqllm::Basis basis() const override { return tqllm::Basis::Plain; }

    // GGUF rows -> bank, packed on the host and uploaded through the engine's own callback (one resident copy). Stacked
    // experts keep the layout of a single matrix as long as an expert's row count is a multiple of 16 (checked at the calls).
    tqllm::Mat load(const std::vector<char> & raw, int rows, int cols, const tqllm::Upload & up, cudaStream_t) const override {
        if (b2moe_raw_bytes(bank_type_, rows, cols) != raw.size() || raw.empty()) throw std::invalid_argument("b200-expert load: byte count does not match rows x cols");
        std::vector<char> data(b2moe_bank_bytes(bank_type_, rows, cols)), aux(b2moe_bank_aux_bytes(bank_type_, rows, cols));
        check(b2moe_bank_pack_host(bank_type_, raw.data(), 1, rows, cols, data.data(), aux.empty() ? nullptr : aux.data()), "b200-expert load");
        tqllm::Mat m;
        m.p = up(data.data(), data.size());
        m.aux = aux.empty() ? nullptr : up(aux.data(), aux.size());
        m.type = bank_type_; m.rows = rows; m.cols = cols; m.fmt = this;
        return m;
    }

    // dense y[n][rows] = W x[n]: the matrix as a bank of one expert, every token routed to it
    void matvec(const tqllm::Mat & m, const __half * x, __nv_bfloat16 * y, int n, cudaStream_t s) const override {
        const b2moe_bank b = bank(m, m.rows, 1);
        const size_t idb = up256(size_t(n) * sizeof(int32_t));
        need(idb + b2moe_expert_matvec_workspace_bytes(&b, n, 1), "matvec");
        if (cudaMemsetAsync(g_ws.p, 0, size_t(n) * sizeof(int32_t), s) != cudaSuccess) throw std::runtime_error("b200-expert matvec: memset failed");
        check(b2moe_expert_matvec(&b, x, B2MOE_F16, y, B2MOE_BF16, static_cast<const int32_t *>(g_ws.p), n, 1, 1,
                                  static_cast<char *>(g_ws.p) + idb, g_ws.bytes - idb, s), "b200-expert matvec");
    }
    void dequant_h(const tqllm::Mat & m, __half * out, cudaStream_t s) const override {
        const b2moe_bank b = bank(m, m.rows, 1);
        need(size_t(m.rows) * m.cols * sizeof(float), "dequant_h");
        check(b2moe_dequant_dump_as(&b, out, B2MOE_F16, g_ws.p, g_ws.bytes, s), "b200-expert dequant_h");
    }

    bool has_expert_matvec() const override { return true; }
    void expert_matvec(const tqllm::Mat & m, const __half * x, __nv_bfloat16 * y, int rows, const int * ids, int n, int topk,
                       bool per_expert_input, cudaStream_t s) const override {
        const b2moe_bank b = stacked(m, rows, "expert_matvec");
        need(b2moe_expert_matvec_workspace_bytes(&b, n, topk), "expert_matvec");
        check(b2moe_expert_matvec(&b, x, B2MOE_F16, y, B2MOE_BF16, ids, n, topk, per_expert_input ? 1 : 0, g_ws.p, g_ws.bytes, s),
              "b200-expert expert_matvec");
    }
    // gate and up over the same ids, unfused as the reference defines it (the engine applies moe_swiglu to yg, yu afterwards)
    void expert_matvec2(const tqllm::Mat & g, const tqllm::Mat & u, const __half * x, __nv_bfloat16 * yg, __nv_bfloat16 * yu, int rows,
                        const int * ids, int n, int topk, cudaStream_t s) const override {
        expert_matvec(g, x, yg, rows, ids, n, topk, false, s);
        expert_matvec(u, x, yu, rows, ids, n, topk, false, s);
    }
    bool expert_gemm(const tqllm::Mat & m, const __half * x, __nv_bfloat16 * y, int rows, const int * counts, const int * groups, int capacity,
                     int experts, int topk, bool per_expert_input, cudaStream_t s) const override {
        if (rows <= 0 || rows % 16 || m.rows != experts * rows) return false;
        const b2moe_bank b = bank(m, rows, experts);
        if (b2moe_expert_matvec_workspace_bytes(&b, capacity, topk) > g_ws.bytes) return false;
        check(b2moe_expert_gemm(&b, x, B2MOE_F16, y, B2MOE_BF16, counts, groups, capacity, topk, per_expert_input ? 1 : 0, g_ws.p, g_ws.bytes, s),
              "b200-expert expert_gemm");
        return true;
    }
    bool expert_gemm_gateup(const tqllm::Mat & g, const tqllm::Mat & u, const __half * x, __half * y, int rows, const int * counts,
                            const int * groups, int capacity, int experts, int topk, cudaStream_t s) const override {
        if (rows <= 0 || rows % 16 || g.rows != experts * rows || u.rows != g.rows || u.type != g.type) return false;
        const b2moe_bank bg = bank(g, rows, experts), bu = bank(u, rows, experts);
        if (b2moe_expert_gemm_gateup_workspace_bytes(&bg, capacity, topk, B2MOE_F16) > g_ws.bytes) return false;
        check(b2moe_expert_gemm_gateup(&bg, &bu, x, B2MOE_F16, y, B2MOE_F16, counts, groups, capacity, topk, g_ws.p, g_ws.bytes, s),
              "b200-expert expert_gemm_gateup");
        return true;
    }
    // device bytes of one row: a row range that starts on a multiple of 16 rows (every expert does) is a Mat of its own
    size_t row_bytes(int cols) const override { return b2moe_bank_bytes(bank_type_, 16, cols) / 16; }
    size_t aux_row_bytes(int cols) const override { return b2moe_bank_aux_bytes(bank_type_, 16, cols) / 16; }

private:
    static b2moe_bank bank(const tqllm::Mat & m, int rows, int experts) {
        b2moe_bank b;
        b.data = m.p; b.aux = m.aux; b.type = m.type; b.experts = experts; b.rows = rows; b.cols = m.cols;
        return b;
    }
    static b2moe_bank stacked(const tqllm::Mat & m, int rows, const char * what) {
        if (rows <= 0 || rows % 16 || m.rows % rows) throw std::invalid_argument(std::string("b200-expert ") + what + ": rows per expert must be a multiple of 16 that divides the stacked rows");
        return bank(m, rows, m.rows / rows);
    }
    static void need(size_t bytes, const char * what) {
        if (!g_ws.p || g_ws.bytes < bytes) throw std::invalid_argument(std::string("b200-expert ") + what + ": workspace missing or too small (b200_set_workspace)");
    }
    uint32_t gguf_, bank_type_;
};

}  // namespace

void b200_set_workspace(void * device_ptr, size_t bytes) { g_ws.p = device_ptr; g_ws.bytes = bytes; }

size_t b200_workspace_bytes(uint32_t bank_type, int experts, int rows, int cols, int n, int topk) {
    b2moe_bank b{};
    b.type = bank_type; b.experts = experts; b.rows = rows; b.cols = cols;
    const size_t a = b2moe_expert_matvec_workspace_bytes(&b, n, topk), g = b2moe_expert_gemm_gateup_workspace_bytes(&b, n, topk, B2MOE_F16);
    return (a > g ? a : g) + up256(size_t(n) * topk * sizeof(int32_t));
}

std::unique_ptr<tqllm::WeightFormat> make_b200_expert_format(uint32_t gguf_type, bool iq3s_as_codes) {
    if (b2moe_raw_bytes(gguf_type, 16, 256) == 0) throw std::invalid_argument("b200-expert: not one of the five expert block formats");
    return std::make_unique<B200ExpertFormat>(gguf_type, iq3s_as_codes);
}
void register_b200_expert_formats(bool iq3s_as_codes) {
    for (uint32_t t : {12u, 20u, 21u, 23u, 323u}) tqllm::register_weight_format(t, make_b200_expert_format(t, iq3s_as_codes));
}

}  // namespace b2adapter
