// Test-only stand-ins for the out-of-line members of tqllm::WeightFormat and the registry, which a real tqLLM build takes
// from src/formats/weight/registry.cpp and q4.cpp: they let the adapter link on its own (--no-undefined). They are the
// base-class defaults ("not supported"); the adapter overrides what the expert path uses.
#include <map>
#include <stdexcept>

#include "weight_format.hpp"

namespace tqllm {
void WeightFormat::matvec_f32(const Mat &, const __half *, float *, int, cudaStream_t) const { throw std::runtime_error("matvec_f32: not supported"); }
bool WeightFormat::expert_gemm_i8(const Mat &, const int8_t *, const float *, const int16_t *, __nv_bfloat16 *, int, const int *, const int *, int, int,
                                  int, bool, cudaStream_t, int) const { return false; }
bool WeightFormat::expert_gemm_gateup(const Mat &, const Mat &, const __half *, __half *, int, const int *, const int *, int, int, int,
                                      cudaStream_t) const { return false; }
void WeightFormat::expert_matvec(const Mat &, const __half *, __nv_bfloat16 *, int, const int *, int, int, bool, cudaStream_t) const {
    throw std::runtime_error("expert_matvec: not supported");
}
void WeightFormat::expert_matvec_dedup(const Mat &, const __half *, __nv_bfloat16 *, int, const int *, int, cudaStream_t) const {
    throw std::runtime_error("expert_matvec_dedup: not supported");
}
void WeightFormat::expert_matvec_dedup2(const Mat &, const Mat &, const __half *, __nv_bfloat16 *, __nv_bfloat16 *, int, const int *, int,
                                        cudaStream_t) const { throw std::runtime_error("expert_matvec_dedup2: not supported"); }
void WeightFormat::expert_matvec2(const Mat &, const Mat &, const __half *, __nv_bfloat16 *, __nv_bfloat16 *, int, const int *, int, int,
                                  cudaStream_t) const { throw std::runtime_error("expert_matvec2: not supported"); }
static std::map<uint32_t, std::unique_ptr<WeightFormat>> & reg() { static std::map<uint32_t, std::unique_ptr<WeightFormat>> r; return r; }
const WeightFormat * weight_format(uint32_t t) { auto it = reg().find(t); return it == reg().end() ? nullptr : it->second.get(); }
void register_weight_format(uint32_t t, std::unique_ptr<WeightFormat> f) { reg()[t] = std::move(f); }
}  // namespace tqllm
