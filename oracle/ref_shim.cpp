// C entry points over the reference's own CPU sources (tqLLM src/experts/moe.cpp and src/formats/weight/dequant.cpp),
// which oracle/build.py compiles where they lie in the reference checkout into oracle/_ref/libtqref.so.
// TEST INFRASTRUCTURE ONLY: used to validate oracle/oracle.cpp bit for bit and as the "reference" CPU baseline.
// This file contains no reference code; it only calls the reference's public functions.
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "dequant.hpp"   // reference: src/formats/weight/dequant.hpp
#include "moe.hpp"       // reference: src/experts/moe.hpp

namespace {
template <class F> void parallel_for(int n, int threads, F && fn) {
    threads = std::max(1, std::min(threads, n));
    if (threads == 1) { for (int i = 0; i < n; ++i) fn(i); return; }
    std::atomic<int> next{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) pool.emplace_back([&] { for (int i; (i = next.fetch_add(1)) < n;) fn(i); });
    for (auto & th : pool) th.join();
}
struct Blk { int elems, bytes; };
bool blk(uint32_t type, Blk & b) {
    switch (type) {
        case 12: b = {256, 144}; return true;
        case 21: b = {256, 110}; return true;
        case 23: b = {256, 136}; return true;
        case 20: b = {32, 18}; return true;
        case 323: b = {128, 76}; return true;
        default: return false;
    }
}
tqllm::MoeConfig make_cfg(int gating, int n_expert, int n_used, int norm, float scale) {
    tqllm::MoeConfig c;
    c.n_expert = n_expert; c.n_expert_used = n_used; c.gating = tqllm::MoeGating(gating);
    c.norm_weights = norm != 0; c.weight_scale = scale;
    return c;
}
}  // namespace

extern "C" {

float ref_half_to_float(uint16_t h) { return tqllm::half_to_float(h); }
float ref_e4m3_to_float(uint8_t b) { return tqllm::e4m3_to_float(b); }

int ref_dequant(uint32_t type, const void * src, float * dst, int64_t n) {
    try { tqllm::dequantize_host(type, src, dst, n); } catch (...) { return 1; }
    return 0;
}

int ref_route(int gating, int n_expert, int n_used, int norm, float scale, const float * logits, const float * sel_bias,
              int * ids, float * weights) {
    try {
        const auto sel = tqllm::moe_route(make_cfg(gating, n_expert, n_used, norm, scale), logits, sel_bias);
        std::copy(sel.ids.begin(), sel.ids.end(), ids);
        std::copy(sel.weights.begin(), sel.weights.end(), weights);
    } catch (...) { return 1; }
    return 0;
}

void ref_expert_ffn(const float * x, int hidden, const float * wg, const float * wu, const float * wd, int ff, float clamp,
                    int clamp_gate, float * out) {
    tqllm::moe_expert_ffn(x, hidden, wg, wu, wd, ff, clamp, clamp_gate != 0, out);
}

void ref_combine(const int * ids, const float * weights, int n_used, const float * expert_outs, int hidden, float * out) {
    tqllm::MoeSelection s;
    s.ids.assign(ids, ids + n_used);
    s.weights.assign(weights, weights + n_used);
    tqllm::moe_combine(s, expert_outs, hidden, out);
}

// The same composition as orc_moe_layer (oracle/oracle.cpp), built from the reference's functions: dequantize_host,
// moe_route, moe_expert_ffn, moe_combine. Routing reads logits_in [tokens][ld_logits] (required here).
int ref_moe_layer(int tokens, int hidden, int experts, int topk, int ff, int gating, int norm, float scale,
                  const float * sel_bias, const float * x,
                  uint32_t type_gate, const void * gate, uint32_t type_up, const void * up, uint32_t type_down, const void * down,
                  int has_shared, const void * sh_gate, const void * sh_up, const void * sh_down, const float * shared_gate_vec,
                  const float * logits_in, int ld_logits, int * ids, float * weights, float * out, int threads) {
    Blk bg, bu, bd;
    if (!logits_in || !blk(type_gate, bg) || !blk(type_up, bu) || !blk(type_down, bd)) return 1;
    const auto cfg = make_cfg(gating, experts, topk, norm, scale);
    const int A = tokens * topk;
    try {
        for (int t = 0; t < tokens; ++t) {
            const auto sel = tqllm::moe_route(cfg, logits_in + size_t(t) * ld_logits, sel_bias);
            std::copy(sel.ids.begin(), sel.ids.end(), ids + size_t(t) * topk);
            std::copy(sel.weights.begin(), sel.weights.end(), weights + size_t(t) * topk);
        }
        std::vector<std::vector<int>> lists(experts);
        for (int a = 0; a < A; ++a) lists[ids[a]].push_back(a);
        std::vector<float> eo(size_t(A + (has_shared ? tokens : 0)) * hidden);
        const size_t gb = size_t(ff) * (hidden / bg.elems) * bg.bytes, ub = size_t(ff) * (hidden / bu.elems) * bu.bytes;
        const size_t db = size_t(hidden) * (ff / bd.elems) * bd.bytes;
        parallel_for(experts + (has_shared ? 1 : 0), threads, [&](int e) {
            const bool shared = e == experts;
            const int n = shared ? tokens : int(lists[e].size());
            if (!n) return;
            std::vector<float> wg(size_t(ff) * hidden), wu(size_t(ff) * hidden), wd(size_t(hidden) * ff);
            const auto * pg = static_cast<const uint8_t *>(shared ? sh_gate : gate) + (shared ? 0 : e * gb);
            const auto * pu = static_cast<const uint8_t *>(shared ? sh_up : up) + (shared ? 0 : e * ub);
            const auto * pd = static_cast<const uint8_t *>(shared ? sh_down : down) + (shared ? 0 : e * db);
            tqllm::dequantize_host(type_gate, pg, wg.data(), int64_t(ff) * hidden);
            tqllm::dequantize_host(type_up, pu, wu.data(), int64_t(ff) * hidden);
            tqllm::dequantize_host(type_down, pd, wd.data(), int64_t(hidden) * ff);
            for (int j = 0; j < n; ++j) {
                const int a = shared ? A + j : lists[e][j];
                const int t = shared ? j : a / topk;
                tqllm::moe_expert_ffn(x + size_t(t) * hidden, hidden, wg.data(), wu.data(), wd.data(), ff, 0.f, false,
                                      &eo[size_t(a) * hidden]);
            }
        });
        parallel_for(tokens, threads, [&](int t) {
            float * o = out + size_t(t) * hidden;
            std::fill(o, o + hidden, 0.f);
            tqllm::MoeSelection s;
            s.ids.assign(ids + size_t(t) * topk, ids + size_t(t + 1) * topk);
            s.weights.assign(weights + size_t(t) * topk, weights + size_t(t + 1) * topk);
            tqllm::moe_combine(s, &eo[size_t(t) * topk * hidden], hidden, o);
            if (has_shared) {
                float sw = 1.f;
                if (shared_gate_vec) {
                    float d = 0.f;
                    for (int j = 0; j < hidden; ++j) d += shared_gate_vec[j] * x[size_t(t) * hidden + j];
                    sw = tqllm::moe_sigmoid(d);
                }
                tqllm::MoeSelection one;
                one.ids = {0}; one.weights = {sw};
                tqllm::moe_combine(one, &eo[size_t(A + t) * hidden], hidden, o);
            }
        });
    } catch (...) { return 1; }
    return 0;
}

}  // extern "C"
