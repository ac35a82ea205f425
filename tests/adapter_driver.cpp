// Drives the WeightFormat adapter (tqllm_b200/adapter/) the way the reference drives its built-in formats in
// tests/moe_device.cu:117-219: through the reference's own declarations (weight_format.hpp, moe_kernels.cuh), so a
// signature that differs from the reference's fails to link. Reads one case from a file, writes every result to another;
// tests/test_gpu_adapter.py makes the case and checks the results against the oracle. Test code.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <stdexcept>
#include <vector>

#include "b200_expert_format.hpp"
#include "b2moe.h"
#include "moe_kernels.cuh"     // reference: src/experts/moe_kernels.cuh
#include "weight_format.hpp"   // reference: src/formats/weight/weight_format.hpp

namespace tqllm_cuda {         // the shims' own scratch hooks (tqllm_shims.cpp)
void b200_set_shim_scratch(void * device_ptr, size_t bytes);
size_t b200_shim_scratch_bytes(int experts, int n, int topk);
}

#define CK(x) do { if ((x) != cudaSuccess) { std::fprintf(stderr, "CUDA error at %s:%d\n", __FILE__, __LINE__); std::exit(2); } } while (0)

template <class T> std::vector<T> rd(FILE * f, size_t n) {
    std::vector<T> v(n);
    if (n && std::fread(v.data(), sizeof(T), n, f) != n) { std::fprintf(stderr, "short read\n"); std::exit(3); }
    return v;
}
template <class T> T * to_dev(const std::vector<T> & v) {
    T * p = nullptr;
    CK(cudaMalloc(&p, std::max<size_t>(v.size() * sizeof(T), 16)));
    CK(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return p;
}
template <class T> void wr(FILE * f, const T * dev, size_t n) {
    std::vector<T> v(n);
    CK(cudaMemcpy(v.data(), dev, n * sizeof(T), cudaMemcpyDeviceToHost));
    std::fwrite(v.data(), sizeof(T), n, f);
}
template <class T> T * dev_buf(size_t n, int fill = 0) {
    T * p = nullptr;
    CK(cudaMalloc(&p, std::max<size_t>(n * sizeof(T), 16)));
    CK(cudaMemset(p, fill, n * sizeof(T)));
    return p;
}

int main(int argc, char ** argv) {
    if (argc < 3) return 1;
    FILE * in = std::fopen(argv[1], "rb"), * out = std::fopen(argv[2], "wb");
    if (!in || !out) return 1;
    const auto hdr = rd<int>(in, 8);
    const int type = hdr[0], experts = hdr[1], rows = hdr[2], cols = hdr[3], n = hdr[4], topk = hdr[5], codes = hdr[6];
    const size_t raw_bytes = b2moe_raw_bytes(uint32_t(type), experts * rows, cols);
    const auto raw_g = rd<char>(in, raw_bytes), raw_u = rd<char>(in, raw_bytes);
    const int A = n * topk;
    const auto x = rd<__half>(in, size_t(n) * cols), xa = rd<__half>(in, size_t(A) * cols);
    const auto ids = rd<int>(in, A);
    const auto w = rd<float>(in, A);
    try {
        auto fmt = b2adapter::make_b200_expert_format(uint32_t(type), codes != 0);
        const tqllm::Upload up = [](const void * host, size_t bytes) -> const void * {
            void * p = nullptr;
            CK(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
            CK(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice));
            return p;
        };
        const tqllm::Mat g = fmt->load(raw_g, experts * rows, cols, up, nullptr), u = fmt->load(raw_u, experts * rows, cols, up, nullptr);
        const size_t ws_bytes = b2adapter::b200_workspace_bytes(g.type, experts, rows, cols, n, topk) + size_t(experts) * rows * cols * 4;
        b2adapter::b200_set_workspace(dev_buf<char>(ws_bytes), ws_bytes);
        const size_t sb = tqllm_cuda::b200_shim_scratch_bytes(experts, n, topk);
        tqllm_cuda::b200_set_shim_scratch(dev_buf<char>(sb), sb);
        const __half * dx = to_dev(x), * dxa = to_dev(xa);
        const int * dids = to_dev(ids);
        const float * dw = to_dev(w);
        cudaStream_t s = nullptr;
        // 1. expert_matvec over the tokens' rows, and with one input row per assignment
        __nv_bfloat16 * y_tok = dev_buf<__nv_bfloat16>(size_t(A) * rows, 0x7f), * y_pei = dev_buf<__nv_bfloat16>(size_t(A) * rows, 0x7f);
        fmt->expert_matvec(g, dx, y_tok, rows, dids, n, topk, false, s);
        fmt->expert_matvec(u, dxa, y_pei, rows, dids, n, topk, true, s);
        // 2. expert_matvec2 + the reference's moe_swiglu
        __nv_bfloat16 * yg = dev_buf<__nv_bfloat16>(size_t(A) * rows), * yu = dev_buf<__nv_bfloat16>(size_t(A) * rows);
        __half * act2 = dev_buf<__half>(size_t(A) * rows);
        fmt->expert_matvec2(g, u, dx, yg, yu, rows, dids, n, topk, s);
        tqllm_cuda::moe_swiglu(yg, yu, act2, A * rows, s);
        // 3. moe_group + expert_gemm / expert_gemm_gateup
        int * counts = dev_buf<int>(experts), * groups = dev_buf<int>(size_t(experts) * n, 0xff);
        tqllm_cuda::moe_group(dids, counts, groups, experts, n, topk, s);
        __nv_bfloat16 * y_gemm = dev_buf<__nv_bfloat16>(size_t(A) * rows);
        __half * act_f = dev_buf<__half>(size_t(A) * rows);
        const bool ok1 = fmt->expert_gemm(g, dx, y_gemm, rows, counts, groups, n, experts, topk, false, s);
        const bool ok2 = fmt->expert_gemm_gateup(g, u, dx, act_f, rows, counts, groups, n, experts, topk, s);
        // 4. moe_sum over the per-assignment rows (hidden = rows here)
        __nv_bfloat16 * sum = dev_buf<__nv_bfloat16>(size_t(n) * rows);
        tqllm_cuda::moe_sum(y_tok, nullptr, dw, nullptr, sum, rows, topk, n, s);
        // 5. expert 0's rows as a matrix of its own (row_bytes / aux_row_bytes): dense matvec over every token
        tqllm::Mat e1 = g;
        const int pick = experts > 1 ? 1 : 0;
        e1.p = static_cast<const char *>(g.p) + size_t(pick) * rows * fmt->row_bytes(cols);
        e1.aux = g.aux ? static_cast<const char *>(g.aux) + size_t(pick) * rows * fmt->aux_row_bytes(cols) : nullptr;
        e1.rows = rows;
        __nv_bfloat16 * y_dense = dev_buf<__nv_bfloat16>(size_t(n) * rows);
        fmt->matvec(e1, dx, y_dense, n, s);
        __half * deq = dev_buf<__half>(size_t(rows) * cols);
        fmt->dequant_h(e1, deq, s);
        // 6. moe_topk2 through the reference's declaration: two routings in one launch equal two moe_topk calls
        const int tk = std::min(topk, experts);
        std::vector<float> la(size_t(n) * (experts + 1)), lb(la.size());
        for (size_t i = 0; i < la.size(); ++i) { la[i] = 3.f * std::sin(0.37f * float(i) + 0.11f * float(i % 7)); lb[i] = 3.f * std::cos(0.23f * float(i) + 1.f); }
        const float * dla = to_dev(la), * dlb = to_dev(lb);
        int * i1 = dev_buf<int>(size_t(n) * tk), * i2 = dev_buf<int>(size_t(n) * tk), * j1 = dev_buf<int>(size_t(n) * tk), * j2 = dev_buf<int>(size_t(n) * tk);
        float * w1 = dev_buf<float>(size_t(n) * tk), * w2 = dev_buf<float>(size_t(n) * tk), * v1 = dev_buf<float>(size_t(n) * tk), * v2 = dev_buf<float>(size_t(n) * tk);
        float * s1 = dev_buf<float>(n), * s2 = dev_buf<float>(n), * r1 = dev_buf<float>(n), * r2 = dev_buf<float>(n);
        tqllm_cuda::moe_topk2(dla, i1, w1, s1, dlb, i2, w2, s2, experts, tk, n, 1.f, s);
        tqllm_cuda::moe_topk(dla, j1, v1, r1, experts, tk, n, 1.f, s);
        tqllm_cuda::moe_topk(dlb, j2, v2, r2, experts, tk, n, 1.f, s);
        CK(cudaDeviceSynchronize());
        auto same = [&](const void * a, const void * b, size_t bytes) {
            std::vector<char> ha(bytes), hb(bytes);
            CK(cudaMemcpy(ha.data(), a, bytes, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(hb.data(), b, bytes, cudaMemcpyDeviceToHost));
            return std::memcmp(ha.data(), hb.data(), bytes) == 0;
        };
        const size_t ib = size_t(n) * tk * 4;
        const bool topk2_ok = same(i1, j1, ib) && same(i2, j2, ib) && same(w1, v1, ib) && same(w2, v2, ib) && same(s1, r1, size_t(n) * 4) && same(s2, r2, size_t(n) * 4);
        const int flags[4] = {ok1 ? 1 : 0, ok2 ? 1 : 0, pick, topk2_ok ? 1 : 0};
        std::fwrite(flags, sizeof(int), 4, out);
        wr(out, y_tok, size_t(A) * rows); wr(out, y_pei, size_t(A) * rows); wr(out, yg, size_t(A) * rows); wr(out, yu, size_t(A) * rows);
        wr(out, act2, size_t(A) * rows); wr(out, y_gemm, size_t(A) * rows); wr(out, act_f, size_t(A) * rows); wr(out, sum, size_t(n) * rows);
        wr(out, y_dense, size_t(n) * rows); wr(out, deq, size_t(rows) * cols);
        // 7. errors reach the caller as the reference's exceptions: a row count that is not a multiple of 16
        int threw = 0;
        try { fmt->expert_matvec(g, dx, y_tok, rows - 1, dids, n, topk, false, s); } catch (const std::invalid_argument &) { threw = 1; }
        std::fwrite(&threw, sizeof(int), 1, out);
    } catch (const std::exception & e) {
        std::fprintf(stderr, "adapter_driver: %s\n", e.what());
        return 4;
    }
    std::fclose(out);
    return 0;
}
