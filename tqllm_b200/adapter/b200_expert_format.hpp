// B200ExpertFormat: tqLLM's weight-format strategy (tqllm::WeightFormat, src/formats/weight/weight_format.hpp:33-110) for
// expert banks served by libb2moe.so. A tqLLM build compiles b200_expert_format.cpp and tqllm_shims.cpp, links
// libb2moe.so and registers the formats before any model loads (register_b200_expert_formats below calls
// tqllm::register_weight_format, src/formats/weight/registry.cpp:77-87).
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>

#include "weight_format.hpp"   // the reference's header

namespace b2adapter {

// Device scratch the adapter's calls carve their plans, fp32 rows and kernel scratch from: owned by the engine (its
// per-step arena), set once per engine thread before the first call; the calls are stream-ordered on the caller's stream
// and use it one at a time. b200_workspace_bytes gives the size one layer call of the stated shape needs.
void b200_set_workspace(void * device_ptr, size_t bytes);
size_t b200_workspace_bytes(uint32_t bank_type, int experts, int rows, int cols, int n, int topk);

// One instance per GGUF expert type: 12 (Q4_K), 20 (IQ4_NL), 21 (IQ3_S), 23 (IQ4_XS), 323 (NVFP4G). `iq3s_as_codes`
// loads IQ3_S blocks into the 4-bit-code bank layout (B2MOE_IQ3_S_X4).
std::unique_ptr<tqllm::WeightFormat> make_b200_expert_format(uint32_t gguf_type, bool iq3s_as_codes = true);
// registers the five formats with the reference's registry
void register_b200_expert_formats(bool iq3s_as_codes = true);

}  // namespace b2adapter
