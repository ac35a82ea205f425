// Bank loaders (GGUF block bytes -> tiled bank, on the device) and the exact fp32 dump used by the parity tests.
// Replaces the host repackers of src/formats/weight/q4.cpp:295-325,495-607,802-832 and pins the decoders of
// formats.cuh against dequantize_host (src/formats/weight/dequant.cpp:393-606).
#include "common.cuh"
#include "formats.cuh"

namespace b2 {
namespace {

template <uint32_t T>
__global__ void bank_pack_k(const uint8_t * __restrict__ raw, uint32_t * __restrict__ data, int rows, int row_tiles, int k_tiles) {
    const int tile = blockIdx.x;                       // ((expert * row_tiles) + rt) * k_tiles + kt
    const int kt = tile % k_tiles, rt = (tile / k_tiles) % row_tiles, e = tile / (k_tiles * row_tiles);
    const uint8_t * src = raw + size_t(e) * rows * k_tiles * Fmt<T>::RAW;
    uint32_t * dst = data + size_t(tile) * (Fmt<T>::TILE / 4);
    for (int wi = threadIdx.x; wi < Fmt<T>::TILE / 4; wi += blockDim.x) dst[wi] = Fmt<T>::pack_word(src, rows, k_tiles, rt, kt, wi);
}

// NVFP4G: the fp32 tensor scale of each row (bytes 0..3 of the row's first block), one float per padded row
__global__ void nvfp4_aux_k(const uint8_t * __restrict__ raw, float * __restrict__ aux, int rows, int rows_pad, int nblk, int total) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int e = i / rows_pad, r = i % rows_pad;
    aux[i] = r < rows ? __uint_as_float(ld_u32_bytes(raw + (size_t(e) * rows + r) * nblk * 76)) : 0.f;
}

template <uint32_t T>
__global__ void bank_dump_k(const uint8_t * __restrict__ data, const float * __restrict__ aux, float * __restrict__ out, int rows,
                            int cols, int row_tiles, int k_tiles, int units) {
    constexpr int KT = Fmt<T>::KT;
    __shared__ float w[16 * KT];
    __shared__ float aux16[16];
    const int tile = blockIdx.x;
    const int kt = tile % k_tiles, rt = (tile / k_tiles) % row_tiles, e = tile / (k_tiles * row_tiles);
    if (threadIdx.x < 16) aux16[threadIdx.x] = aux ? aux[(size_t(e) * row_tiles + rt) * 16 + threadIdx.x] : 0.f;
    __syncthreads();
    decode_tile<T>(data + size_t(tile) * Fmt<T>::TILE, aux16, w, KT, threadIdx.x, blockDim.x, units);
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * KT; i += blockDim.x) {
        const int r = i / KT, k = i % KT, row = 16 * rt + r;
        if (row < rows) out[(size_t(e) * rows + row) * cols + size_t(kt) * KT + k] = w[i];
    }
}

template <uint32_t T>
int32_t load_t(const void * raw, int experts, int rows, int cols, void * data, cudaStream_t s) {
    const int row_tiles = ceil_div(rows, 16), k_tiles = cols / Fmt<T>::KT;
    const long long tiles = (long long)experts * row_tiles * k_tiles;
    if (tiles > 0x7fffffffLL) return B2MOE_ERR_SHAPE;
    bank_pack_k<T><<<unsigned(tiles), 128, 0, s>>>(static_cast<const uint8_t *>(raw), static_cast<uint32_t *>(data), rows, row_tiles, k_tiles);
    return launch_status();
}
template <uint32_t T>
int32_t dump_t(const b2moe_bank & b, float * out, cudaStream_t s) {
    FmtInfo f;
    fmt_info(T, f);
    const int row_tiles = ceil_div(b.rows, 16), k_tiles = b.cols / Fmt<T>::KT;
    const long long tiles = (long long)b.experts * row_tiles * k_tiles;
    if (tiles > 0x7fffffffLL) return B2MOE_ERR_SHAPE;
    bank_dump_k<T><<<unsigned(tiles), 256, 0, s>>>(static_cast<const uint8_t *>(b.data), static_cast<const float *>(b.aux), out, b.rows,
                                                     b.cols, row_tiles, k_tiles, f.units);
    return launch_status();
}

}  // namespace

int32_t check_bank(const b2moe_bank * b) {
    FmtInfo f;
    if (!b) return B2MOE_ERR_NULL;
    if (!fmt_info(b->type, f)) return B2MOE_ERR_FORMAT;
    if (b->experts <= 0 || b->rows <= 0 || b->cols <= 0 || b->cols % f.kt) return B2MOE_ERR_SHAPE;
    if (!b->data || (f.aux && !b->aux)) return B2MOE_ERR_NULL;
    if (!aligned16(b->data)) return B2MOE_ERR_ALIGN;
    return B2MOE_OK;
}

}  // namespace b2

using namespace b2;

extern "C" B2MOE_API size_t b2moe_raw_bytes(uint32_t type, int32_t rows, int32_t cols) {
    FmtInfo f;
    if (!fmt_info(type, f) || rows <= 0 || cols <= 0 || cols % f.raw_elems) return 0;
    return size_t(rows) * (cols / f.raw_elems) * f.raw_bytes;
}
extern "C" B2MOE_API size_t b2moe_bank_bytes(uint32_t type, int32_t rows, int32_t cols) {
    FmtInfo f;
    if (!fmt_info(type, f) || rows <= 0 || cols <= 0 || cols % f.kt) return 0;
    return size_t(ceil_div(rows, 16)) * (cols / f.kt) * f.tile;
}
extern "C" B2MOE_API size_t b2moe_bank_aux_bytes(uint32_t type, int32_t rows, int32_t cols) {
    FmtInfo f;
    if (!fmt_info(type, f) || rows <= 0 || cols <= 0 || cols % f.kt || !f.aux) return 0;
    return size_t(ceil_div(rows, 16)) * 16 * sizeof(float);
}

extern "C" B2MOE_API int32_t b2moe_bank_load(uint32_t type, const void * raw, int32_t experts, int32_t rows, int32_t cols, void * data,
                                   void * aux, b2moe_stream stream) {
    FmtInfo f;
    if (!fmt_info(type, f)) return B2MOE_ERR_FORMAT;
    if (experts <= 0 || rows <= 0 || cols <= 0 || cols % f.kt) return B2MOE_ERR_SHAPE;
    if (!raw || !data || (f.aux && !aux)) return B2MOE_ERR_NULL;
    if (!aligned16(data)) return B2MOE_ERR_ALIGN;
    cudaStream_t s = as_stream(stream);
    switch (type) {
        case T_Q4_K: return load_t<T_Q4_K>(raw, experts, rows, cols, data, s);
        case T_IQ3_S: return load_t<T_IQ3_S>(raw, experts, rows, cols, data, s);
        case T_IQ3S4: return load_t<T_IQ3S4>(raw, experts, rows, cols, data, s);
        case T_IQ4_XS: return load_t<T_IQ4_XS>(raw, experts, rows, cols, data, s);
        case T_IQ4_NL: return load_t<T_IQ4_NL>(raw, experts, rows, cols, data, s);
        case T_NVFP4G: {
            const int rows_pad = 16 * ceil_div(rows, 16);
            const long long total = (long long)experts * rows_pad;
            if (total > 0x7fffffffLL) return B2MOE_ERR_SHAPE;
            nvfp4_aux_k<<<unsigned((total + 255) / 256), 256, 0, s>>>(static_cast<const uint8_t *>(raw), static_cast<float *>(aux), rows,
                                                                      rows_pad, cols / 128, int(total));
            if (launch_status()) return B2MOE_ERR_CUDA;
            return load_t<T_NVFP4G>(raw, experts, rows, cols, data, s);
        }
    }
    return B2MOE_ERR_FORMAT;
}

namespace b2 {
namespace {
template <uint32_t T>
void pack_host_t(const uint8_t * raw, int experts, int rows, int cols, uint8_t * data) {
    const int row_tiles = ceil_div(rows, 16), k_tiles = cols / Fmt<T>::KT;
    for (int e = 0; e < experts; ++e)
        for (int rt = 0; rt < row_tiles; ++rt)
            for (int kt = 0; kt < k_tiles; ++kt) {
                uint32_t * dst = reinterpret_cast<uint32_t *>(data + ((size_t(e) * row_tiles + rt) * k_tiles + kt) * Fmt<T>::TILE);
                const uint8_t * src = raw + size_t(e) * rows * k_tiles * Fmt<T>::RAW;
                for (int wi = 0; wi < Fmt<T>::TILE / 4; ++wi) dst[wi] = Fmt<T>::pack_word(src, rows, k_tiles, rt, kt, wi);
            }
}
}  // namespace
}  // namespace b2

// The bank of b2moe_bank_load built on the host (all pointers host memory): the same bytes, for a loader that uploads
// finished banks through the engine's own upload path (WeightFormat::load, src/formats/weight/weight_format.hpp:39) and
// for packing expert files offline. No CUDA call is made.
extern "C" B2MOE_API int32_t b2moe_bank_pack_host(uint32_t type, const void * raw, int32_t experts, int32_t rows, int32_t cols, void * data,
                                                  void * aux) {
    FmtInfo f;
    if (!fmt_info(type, f)) return B2MOE_ERR_FORMAT;
    if (experts <= 0 || rows <= 0 || cols <= 0 || cols % f.kt) return B2MOE_ERR_SHAPE;
    if (!raw || !data || (f.aux && !aux)) return B2MOE_ERR_NULL;
    const uint8_t * r = static_cast<const uint8_t *>(raw);
    uint8_t * d = static_cast<uint8_t *>(data);
    switch (type) {
        case T_Q4_K: pack_host_t<T_Q4_K>(r, experts, rows, cols, d); break;
        case T_IQ3_S: pack_host_t<T_IQ3_S>(r, experts, rows, cols, d); break;
        case T_IQ3S4: pack_host_t<T_IQ3S4>(r, experts, rows, cols, d); break;
        case T_IQ4_XS: pack_host_t<T_IQ4_XS>(r, experts, rows, cols, d); break;
        case T_IQ4_NL: pack_host_t<T_IQ4_NL>(r, experts, rows, cols, d); break;
        case T_NVFP4G: {
            const int rows_pad = 16 * ceil_div(rows, 16), nblk = cols / 128;
            float * a = static_cast<float *>(aux);
            for (int e = 0; e < experts; ++e)
                for (int rr = 0; rr < rows_pad; ++rr)
                    a[size_t(e) * rows_pad + rr] = rr < rows ? bits_to_float(ld_u32_bytes(r + (size_t(e) * rows + rr) * nblk * 76)) : 0.f;
            pack_host_t<T_NVFP4G>(r, experts, rows, cols, d);
            break;
        }
        default: return B2MOE_ERR_FORMAT;
    }
    return B2MOE_OK;
}

extern "C" B2MOE_API int32_t b2moe_dequant_dump(const b2moe_bank * bank, float * out, b2moe_stream stream) {
    if (const int32_t rc = check_bank(bank)) return rc;
    if (!out) return B2MOE_ERR_NULL;
    cudaStream_t s = as_stream(stream);
    switch (bank->type) {
        case T_Q4_K: return dump_t<T_Q4_K>(*bank, out, s);
        case T_IQ3_S: return dump_t<T_IQ3_S>(*bank, out, s);
        case T_IQ3S4: return dump_t<T_IQ3S4>(*bank, out, s);
        case T_IQ4_XS: return dump_t<T_IQ4_XS>(*bank, out, s);
        case T_IQ4_NL: return dump_t<T_IQ4_NL>(*bank, out, s);
        case T_NVFP4G: return dump_t<T_NVFP4G>(*bank, out, s);
    }
    return B2MOE_ERR_FORMAT;
}
