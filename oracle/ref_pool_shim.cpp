// C entry points over the reference's production CPU expert path: CpuMissPool (tqLLM
// src/models/qwen/qwen4exp/fn_cpu_experts.hpp:345-554: int8 AVX2 dots for the IQ3_S gate / up rows, dequantise + fp32 dot
// for IQ3_S down rows, bf16 / fp16 rounding like the GPU path), which oracle/build.py compiles where it lies in the
// reference checkout into oracle/_ref/libtqrefpool.so together with src/formats/weight/dequant.cpp.
// TEST AND BENCHMARK INFRASTRUCTURE ONLY: this is the CPU arm bench.py times; it is never used for parity (the pool's
// numerics are the reference's int8 / bf16 ones, not fp32). This file contains no reference code; it only builds the
// job list the reference's engine builds (one job per expert and group of up to 8 token columns) and calls the pool.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "fn_cpu_experts.hpp"   // reference: src/models/qwen/qwen4exp/fn_cpu_experts.hpp

namespace {
CpuMissPool * g_pool = nullptr;      // never destroyed: its destructor prints statistics to stdout
int g_threads = 0, g_hidden = 0, g_ff = 0;
size_t row_bytes_of(uint32_t type, int cols) {
    switch (type) {
        case 12: return size_t(cols / 256) * 144;
        case 21: return size_t(cols / 256) * 110;
        case 23: return size_t(cols / 256) * 136;
        case 20: return size_t(cols / 32) * 18;
        default: return 0;
    }
}
}  // namespace

extern "C" {

// threads worker threads pinned to CPUs 1 .. threads, the caller to CPU 0 (the pool's own policy)
int refpool_create(int threads, int hidden, int ff) {
    if (g_pool && (threads != g_threads || hidden != g_hidden || ff != g_ff)) return 1;
    if (!g_pool) {
        try { g_pool = new CpuMissPool(threads, hidden, ff); } catch (...) { return 2; }
        g_threads = threads; g_hidden = hidden; g_ff = ff;
    }
    return 0;
}

// One layer's expert products and combine through the pool. ids / weights: the routing ([tokens][topk], id < 0 = skip).
// gate / up / down: stacked GGUF rows of the routed experts; sh_*: the always-on expert's (weight 1) when has_shared.
// out: fp32 [tokens][hidden] = sum of weight * the pool's bf16 expert outputs, in slot order.
int refpool_layer(int tokens, int hidden, int experts, int topk, int ff, const float * x, const int * ids, const float * weights,
                  const uint32_t * types, const char * gate, const char * up, const char * down, int has_shared, const char * sh_gate,
                  const char * sh_up, const char * sh_down, float * out) {
    if (!g_pool || hidden != g_hidden || ff != g_ff) return 1;
    const size_t rb[3] = {row_bytes_of(types[0], hidden), row_bytes_of(types[1], hidden), row_bytes_of(types[2], ff)};
    if (!rb[0] || !rb[1] || !rb[2]) return 2;
    const size_t mat[3] = {rb[0] * ff, rb[1] * ff, rb[2] * hidden};
    // assignments of every expert in ascending order (the stable dispatch), cut into jobs of up to 8 token columns
    std::vector<std::vector<int>> lists(size_t(experts) + 1);
    for (int a = 0; a < tokens * topk; ++a) if (ids[a] >= 0 && ids[a] < experts) lists[size_t(ids[a])].push_back(a);
    if (has_shared) for (int t = 0; t < tokens; ++t) lists[size_t(experts)].push_back(tokens * topk + t);
    std::vector<CpuMissPool::Job> jobs;
    std::vector<int> col_assignment;
    for (int e = 0; e <= experts; ++e) {
        const auto & l = lists[size_t(e)];
        for (size_t c0 = 0; c0 < l.size(); c0 += 8) {
            CpuMissPool::Job j;
            const bool sh = e == experts;
            const char * base[3] = {sh ? sh_gate : gate + size_t(e) * mat[0], sh ? sh_up : up + size_t(e) * mat[1], sh ? sh_down : down + size_t(e) * mat[2]};
            for (int m = 0; m < 3; ++m) { j.w[m] = base[m]; j.type[m] = types[m]; j.row_bytes[m] = rb[m]; }
            for (size_t c = c0; c < std::min(l.size(), c0 + 8); ++c) {
                const int a = l[c];
                j.cols_t[j.ncols++] = a < tokens * topk ? a / topk : a - tokens * topk;
                col_assignment.push_back(a);
            }
            jobs.push_back(j);
        }
    }
    std::vector<__nv_bfloat16> rows(col_assignment.size() * size_t(hidden));
    try {
        g_pool->start(x, tokens, std::move(jobs), rows.data());
        g_pool->wait();
    } catch (...) { return 3; }
    std::vector<int> col_of(size_t(tokens) * topk + (has_shared ? tokens : 0), -1);
    for (size_t c = 0; c < col_assignment.size(); ++c) col_of[size_t(col_assignment[c])] = int(c);
    for (int t = 0; t < tokens; ++t) {
        float * o = out + size_t(t) * hidden;
        std::fill(o, o + hidden, 0.f);
        for (int s = 0; s <= topk; ++s) {
            if (s == topk && !has_shared) break;
            const int a = s < topk ? t * topk + s : tokens * topk + t;
            const int c = col_of[size_t(a)];
            if (c < 0) continue;
            const float w = s < topk ? weights[a] : 1.f;
            const __nv_bfloat16 * r = rows.data() + size_t(c) * hidden;
            for (int h = 0; h < hidden; ++h) o[h] += w * __bfloat162float(r[h]);
        }
    }
    return 0;
}

}  // extern "C"
