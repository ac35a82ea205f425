// Host build of the bank layout functions of tqllm_b200/csrc/formats.cuh (pack_word + decode_unit are
// __host__ __device__): packs GGUF blocks into bank tiles and decodes them back on the CPU, so the layout arithmetic
// is checked against the oracle without a GPU. Test code only; the library itself has no CPU path.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../tqllm_b200/csrc/formats.cuh"

using namespace b2;

template <uint32_t T>
static void run(const uint8_t * raw, int rows, int cols, uint8_t * bank, float * out) {
    FmtInfo f;
    fmt_info(T, f);
    const int row_tiles = (rows + 15) / 16, k_tiles = cols / f.kt;
    std::vector<float> w(16 * f.kt);
    for (int rt = 0; rt < row_tiles; ++rt)
        for (int kt = 0; kt < k_tiles; ++kt) {
            uint8_t * tile = bank + (size_t(rt) * k_tiles + kt) * f.tile;
            for (int wi = 0; wi < f.tile / 4; ++wi) {
                const uint32_t v = Fmt<T>::pack_word(raw, rows, k_tiles, rt, kt, wi);
                std::memcpy(tile + 4 * wi, &v, 4);
            }
            float aux16[16];
            for (int r = 0; r < 16; ++r) {
                const int row = 16 * rt + r;
                aux16[r] = 0.f;
                if (T == T_NVFP4G && row < rows) std::memcpy(&aux16[r], raw + size_t(row) * k_tiles * 76, 4);
            }
            for (int u = 0; u < f.units; ++u) decode_unit<T>(tile, aux16, u, w.data(), f.kt);
            for (int r = 0; r < 16 && 16 * rt + r < rows; ++r)
                std::memcpy(out + size_t(16 * rt + r) * cols + size_t(kt) * f.kt, &w[size_t(r) * f.kt], sizeof(float) * f.kt);
        }
}

// raw: one matrix [rows][cols] of GGUF blocks; bank: rows_pad/16 * cols/kt * tile bytes; out: fp32 [rows][cols]
extern "C" int host_pack_decode(uint32_t type, const uint8_t * raw, int rows, int cols, uint8_t * bank, float * out) {
    switch (type) {
        case T_Q4_K: run<T_Q4_K>(raw, rows, cols, bank, out); return 0;
        case T_IQ3_S: run<T_IQ3_S>(raw, rows, cols, bank, out); return 0;
        case T_IQ3S4: run<T_IQ3S4>(raw, rows, cols, bank, out); return 0;
        case T_IQ4_XS: run<T_IQ4_XS>(raw, rows, cols, bank, out); return 0;
        case T_IQ4_NL: run<T_IQ4_NL>(raw, rows, cols, bank, out); return 0;
        case T_NVFP4G: run<T_NVFP4G>(raw, rows, cols, bank, out); return 0;
    }
    return 1;
}
