// Bank layouts of the five block formats and their exact fp32 decoders.
//
// A bank stores a stacked expert matrix as tiles of 16 rows x KT columns; inside a tile the code bytes are
// "lane-major": lane L = 4*g + t of a warp (g = L >> 2, t = L & 3) owns rows g and g + 8 and, of every 32-weight
// sub-block, the quarter whose codes the tensor-core A fragment of that lane needs, so one coalesced 16-byte load
// per lane per plane brings exactly the lane's own operands. Scales and block headers follow the planes.
// No byte is added to the GGUF block size: tile bytes = 16 * (KT / block elements) * block bytes.
//
// Every decoder reproduces the fp32 arithmetic of the reference's host decoder dequantize_host
// (src/formats/weight/dequant.cpp): q4k :80-99, iq3s :137-150, iq4xs :177-192, iq4nl :352-360, NVFP4G :397-409,
// half_to_float :32-54, e4m3_to_float :387-391, scale_min_k4 :56-64 — same operand order, one rounding per product.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>
#include <string.h>

#include "_gen/ggml_tables.h"

namespace b2 {

enum : uint32_t { T_Q4_K = 12, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ4_XS = 23, T_NVFP4G = 323,
                  // IQ3_S blocks held as 4-bit codes (no grid lookup on the read side): a bank layout of this library, not a GGUF type
                  T_IQ3S4 = 0x1015 };

struct FmtInfo {
    int kt;         // columns per tile
    int tile;       // bytes per 16-row tile
    int raw_elems;  // weights per GGUF block
    int raw_bytes;  // bytes per GGUF block
    int units;      // decode units per tile (see decode_unit)
    int unit_elems; // weights one unit decodes
    bool aux;       // has a per-row fp32 aux array
};

__host__ __device__ inline bool fmt_info(uint32_t type, FmtInfo & f) {
    switch (type) {
        case T_Q4_K: f = {256, 2304, 256, 144, 512, 8, false}; return true;
        case T_IQ3_S: f = {256, 1760, 256, 110, 1024, 4, false}; return true;
        case T_IQ3S4: f = {256, 2144, 256, 110, 512, 8, false}; return true;
        case T_IQ4_XS: f = {256, 2176, 256, 136, 512, 8, false}; return true;
        case T_IQ4_NL: f = {32, 288, 32, 18, 64, 8, false}; return true;
        case T_NVFP4G: f = {128, 1152, 128, 76, 256, 8, true}; return true;
        default: return false;
    }
}

static __device__ __constant__ uint32_t c_iq3s_grid[512] = B2_IQ3S_GRID_INIT;
static __device__ __constant__ int8_t c_kvalues_iq4nl[16] = B2_KVALUES_IQ4NL_INIT;
// host copies: the layout functions below also compile for the host so the CPU test suite can check them
static const uint32_t h_iq3s_grid[512] = B2_IQ3S_GRID_INIT;
static const int8_t h_kvalues_iq4nl[16] = B2_KVALUES_IQ4NL_INIT;
#ifdef __CUDA_ARCH__
#define B2_GRID(i) c_iq3s_grid[i]
#define B2_KV(i) c_kvalues_iq4nl[i]
#else
#define B2_GRID(i) h_iq3s_grid[i]
#define B2_KV(i) h_kvalues_iq4nl[i]
#endif

__host__ __device__ __forceinline__ uint32_t ld_u32_bytes(const uint8_t * p) {
    return uint32_t(p[0]) | (uint32_t(p[1]) << 8) | (uint32_t(p[2]) << 16) | (uint32_t(p[3]) << 24);
}
__host__ __device__ __forceinline__ uint32_t ld_u16_bytes(const uint8_t * p) { return uint32_t(p[0]) | (uint32_t(p[1]) << 8); }
__host__ __device__ __forceinline__ float bits_to_float(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}
__host__ __device__ __forceinline__ float half_bits_to_float(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// OCP E4M3 byte -> float; 0x7F / 0xFF = NaN (src/formats/weight/dequant.cpp:387-391)
__host__ __device__ __forceinline__ float e4m3_to_float(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float v;
    if (e == 15u && m == 7u) v = bits_to_float(0x7FC00000u);
    else if (e == 0u) v = float(m) * 0.001953125f;                     // m / 8 * 2^-6
    else v = bits_to_float(((e + 120u) << 23) | (m << 20));           // (1 + m/8) * 2^(e-7)
    return (b & 0x80u) ? -v : v;
}

// Q4_K / Q5_K 6-bit scale and min of sub-block j from the 12 packed bytes (src/formats/weight/dequant.cpp:56-64)
__host__ __device__ __forceinline__ void k4_scale_min(int j, const uint8_t * s, int & sc, int & mn) {
    if (j < 4) { sc = s[j] & 63; mn = s[j + 4] & 63; }
    else { sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4); mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

// ---------------------------------------------------------------------------------------------------------------
// pack_word: value of 32-bit word `wi` of the tile (row tile rt, column tile kt) of one expert's matrix, gathered from
// the GGUF blocks `raw` of that expert ([rows][nblk][raw_bytes]). Rows >= rows decode to zero weights.
// unit_vals: unit u of a tile -> its weights as fp32: v[0..3] are columns k0.. of row `row`, v[4..7] columns k1.. (k1 < 0: the
// unit has four weights). step_unit enumerates the units of one 64-column step for the tensor-core GEMM path.
// ---------------------------------------------------------------------------------------------------------------
template <uint32_t T> struct Fmt;

template <> struct Fmt<T_Q4_K> {
    // planes p = 0..3 (64-weight pair p) at 512 p + 16 L: {row g: qs word t, word t + 4; row g + 8: the same};
    // qs word m of pair p = raw qs bytes [32 p + 4 m, +4): low nibbles = sub-block 2p, high nibbles = sub-block 2p + 1.
    // 2048 + 16 row: the raw 16-byte header (d, dmin, scales[12]).
    static constexpr int KT = 256, TILE = 2304, RAW = 144;
    __host__ __device__ static uint32_t pack_word(const uint8_t * raw, int rows, int nblk, int rt, int kt, int wi) {
        int row, off;
        if (wi < 512) {
            const int p = wi >> 7, L = (wi >> 2) & 31, c = wi & 3;
            row = 16 * rt + (L >> 2) + 8 * (c >> 1);
            off = 16 + 32 * p + 4 * ((L & 3) + 4 * (c & 1));
        } else {
            row = 16 * rt + ((wi - 512) >> 2);
            off = 4 * ((wi - 512) & 3);
        }
        if (row >= rows) return 0u;
        return ld_u32_bytes(raw + (size_t(row) * nblk + kt) * RAW + off);
    }
    __host__ __device__ static void unit_vals(const uint8_t * tile, const float *, int u, float (&v)[8], int & row, int & k0, int & k1,
                                              const uint32_t * = nullptr) {
        row = u >> 5;
        const int p = (u >> 3) & 3, m = u & 7;
        const int L = 4 * (row & 7) + (m & 3);
        const uint32_t w = *reinterpret_cast<const uint32_t *>(tile + 512 * p + 16 * L + 8 * (row >> 3) + 4 * (m >> 2));
        const uint8_t * h = tile + 2048 + 16 * row;
        const float d = half_bits_to_float(ld_u16_bytes(h)), dmin = half_bits_to_float(ld_u16_bytes(h + 2));
        int sc, mn;
        k4_scale_min(2 * p, h + 4, sc, mn);
        const float d1 = d * float(sc), m1 = dmin * float(mn);
        k4_scale_min(2 * p + 1, h + 4, sc, mn);
        const float d2 = d * float(sc), m2 = dmin * float(mn);
        k0 = 64 * p + 4 * m;
        k1 = k0 + 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = d1 * float((w >> (8 * i)) & 15u) - m1;
            v[4 + i] = d2 * float((w >> (8 * i + 4)) & 15u) - m2;
        }
    }
    // unit i (of STEP_UNITS) of the 64 columns [64 j, 64 j + 64) of a 256-column chunk: tile inside the chunk, unit id
    static constexpr int STEP_UNITS = 128;
    __host__ __device__ static void step_unit(int j, int i, int & tl, int & u) { tl = 0; u = (i >> 3) * 32 + j * 8 + (i & 7); }
};

template <> struct Fmt<T_IQ3_S> {
    // Per lane 13 words. Words 0..8: thirty-two 9-bit grid indices, entry n = 16 r + 2 ib + j at bits [9n, 9n + 9)
    // (r = 0: row g, 1: row g + 8; sub-block ib; j selects grid entry w = 2 t + j of the sub-block's eight).
    // Words 9..12: sign bits, word 9 + 2 r + (ib >> 2) covers sub-blocks 4 (ib >> 2) .. +3 of row g + 8 r. The signs of
    // grid entry 2 t + j of sub-block ib (R = 2 (ib & 3) + j) sit at bits R (weight 0), R + 8 (weight 2), R + 16
    // (weight 1), R + 24 (weight 3): one shift gives the sign mask of either tensor-core operand form —
    // (word << (7 - R)) & 0x80808080 for the entry as four E4M3 bytes in the order 0, 2, 1, 3, and
    // (word << (15 - R)) & 0x80008000 / (word << (7 - R)) & 0x80008000 for the bf16 pairs (0, 1) / (2, 3).
    // Words 4q'..4q'+3 (q' = 0..2) form plane q' at 512 q' + 16 L; word 12 at 1536 + 4 L.
    // 1664 + 4 row: the four scale bytes (nibble ib = 4-bit sub-block scale); 1728 + 2 row: d (fp16).
    static constexpr int KT = 256, TILE = 1760, RAW = 110;
    __host__ __device__ static uint32_t grid_index(const uint8_t * blk, int ib, int w) {
        return uint32_t(blk[2 + 8 * ib + w]) | (((uint32_t(blk[66 + ib]) >> w) & 1u) << 8);
    }
    __host__ __device__ static uint32_t pack_word(const uint8_t * raw, int rows, int nblk, int rt, int kt, int wi) {
        if (wi < 416) {
            int L, q;
            if (wi < 384) { L = (wi >> 2) & 31; q = 4 * (wi >> 7) + (wi & 3); }
            else { L = wi - 384; q = 12; }
            const int g = L >> 2, t = L & 3;
            if (q < 9) {
                uint32_t v = 0;
                for (int n = (32 * q) / 9; n <= (32 * q + 31) / 9 && n < 32; ++n) {
                    const int row = 16 * rt + g + 8 * (n >> 4), ib = (n >> 1) & 7, w = 2 * t + (n & 1);
                    if (row >= rows) continue;
                    const uint64_t idx = grid_index(raw + (size_t(row) * nblk + kt) * RAW, ib, w);
                    const int sh = 9 * n - 32 * q;
                    v |= sh >= 0 ? uint32_t(idx << sh) : uint32_t(idx >> -sh);
                }
                return v;
            }
            const int row = 16 * rt + g + 8 * ((q - 9) >> 1), half = (q - 9) & 1;
            if (row >= rows) return 0u;
            const uint8_t * blk = raw + (size_t(row) * nblk + kt) * RAW;
            uint32_t v = 0;
            for (int b = 0; b < 4; ++b) {
                const uint32_t sb = blk[74 + 4 * (4 * half + b) + t];      // raw sign byte: bit 4 j + i = weight i of entry 2t + j
                for (int j = 0; j < 2; ++j)
                    for (int i = 0; i < 4; ++i) v |= ((sb >> (4 * j + i)) & 1u) << (2 * b + j + 8 * ((i >> 1) + 2 * (i & 1)));
            }
            return v;
        }
        if (wi < 432) {
            const int row = 16 * rt + (wi - 416);
            return row < rows ? ld_u32_bytes(raw + (size_t(row) * nblk + kt) * RAW + 106) : 0u;
        }
        uint32_t v = 0;
        for (int i = 0; i < 2; ++i) {
            const int row = 16 * rt + 2 * (wi - 432) + i;
            if (row < rows) v |= ld_u16_bytes(raw + (size_t(row) * nblk + kt) * RAW) << (16 * i);
        }
        return v;
    }
    __host__ __device__ __forceinline__ static uint32_t lane_word(const uint8_t * tile, int L, int q) {
        return *reinterpret_cast<const uint32_t *>(q < 12 ? tile + 512 * (q >> 2) + 16 * L + 4 * (q & 3) : tile + 1536 + 4 * L);
    }
    __host__ __device__ static void unit_vals(const uint8_t * tile, const float *, int u, float (&v)[8], int & row, int & k0, int & k1,
                                              const uint32_t * grid_tab = nullptr) {
        row = u >> 6;
        const int ib = (u >> 3) & 7, w = u & 7;
        const int g = row & 7, r = row >> 3, t = w >> 1, j = w & 1, L = 4 * g + t;
        const int bit = 9 * (16 * r + 2 * ib + j), q = bit >> 5, sh = bit & 31;
        uint64_t two = lane_word(tile, L, q);
        if (sh > 23) two |= uint64_t(lane_word(tile, L, q + 1)) << 32;
        const uint32_t idx = uint32_t(two >> sh) & 511u;
        const uint32_t sg = lane_word(tile, L, 9 + 2 * r + (ib >> 2)) >> (2 * (ib & 3) + j);   // weight i at bit 8 ((i >> 1) + 2 (i & 1))
        const uint32_t sc = *reinterpret_cast<const uint32_t *>(tile + 1664 + 4 * row);
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tile + 1728 + 2 * row));
        const float db = d * float(1 + 2 * int((sc >> (4 * ib)) & 15u));
        const uint32_t grid = grid_tab ? grid_tab[idx] : B2_GRID(idx);
        k0 = 32 * ib + 4 * w;
        k1 = -1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float mag = db * float((grid >> (8 * i)) & 255u);
            v[i] = ((sg >> (8 * ((i >> 1) + 2 * (i & 1)))) & 1u) ? -mag : mag;
            v[4 + i] = 0.f;
        }
    }
    static constexpr int STEP_UNITS = 256;
    __host__ __device__ static void step_unit(int j, int i, int & tl, int & u) { tl = 0; u = (i >> 4) * 64 + (2 * j + ((i >> 3) & 1)) * 8 + (i & 7); }
};

template <> struct Fmt<T_IQ3S4> {
    // IQ3_S blocks with the grid lookup and the sign already applied when the bank is packed: an IQ3_S weight is
    // d (1 + 2 s) (+-m), m an odd magnitude 1..15, so +-m = 2 n - 15 with a 4-bit code n = (15 +- m) / 2. The tile has the
    // shape of the Q4_K tile: planes p = 0..3 (sub-blocks 2p, 2p + 1) at 512 p + 16 L: {row g: word t, word t + 4;
    // row g + 8: the same}; byte i of word m holds the codes of weight 4 m + i of sub-block 2p (low nibble) and of
    // sub-block 2p + 1 (high nibble). 2048 + 4 row: the raw scale bytes (nibble ib = 4-bit scale of sub-block ib);
    // 2112 + 2 row: d (fp16). 134 bytes per 256 weights against the 110 of the GGUF block.
    static constexpr int KT = 256, TILE = 2144, RAW = 110;
    __host__ __device__ static uint32_t code(const uint8_t * blk, int ib, int j) {
        const int w = j >> 2, i = j & 3;
        const uint32_t idx = Fmt<T_IQ3_S>::grid_index(blk, ib, w);
        const uint32_t mag = (B2_GRID(idx) >> (8 * i)) & 255u;
        const uint32_t neg = (uint32_t(blk[74 + 4 * ib + (w >> 1)]) >> (4 * (w & 1) + i)) & 1u;
        return neg ? (15u - mag) >> 1 : (15u + mag) >> 1;
    }
    __host__ __device__ static uint32_t pack_word(const uint8_t * raw, int rows, int nblk, int rt, int kt, int wi) {
        if (wi < 512) {
            const int p = wi >> 7, L = (wi >> 2) & 31, c = wi & 3;
            const int row = 16 * rt + (L >> 2) + 8 * (c >> 1), m = (L & 3) + 4 * (c & 1);
            if (row >= rows) return 0u;
            const uint8_t * blk = raw + (size_t(row) * nblk + kt) * RAW;
            uint32_t v = 0;
            for (int i = 0; i < 4; ++i) v |= (code(blk, 2 * p, 4 * m + i) | (code(blk, 2 * p + 1, 4 * m + i) << 4)) << (8 * i);
            return v;
        }
        if (wi < 528) {
            const int row = 16 * rt + (wi - 512);
            return row < rows ? ld_u32_bytes(raw + (size_t(row) * nblk + kt) * RAW + 106) : 0u;
        }
        uint32_t v = 0;
        for (int i = 0; i < 2; ++i) {
            const int row = 16 * rt + 2 * (wi - 528) + i;
            if (row < rows) v |= ld_u16_bytes(raw + (size_t(row) * nblk + kt) * RAW) << (16 * i);
        }
        return v;
    }
    __host__ __device__ static void unit_vals(const uint8_t * tile, const float *, int u, float (&v)[8], int & row, int & k0, int & k1,
                                              const uint32_t * = nullptr) {
        row = u >> 5;
        const int p = (u >> 3) & 3, m = u & 7;
        const int L = 4 * (row & 7) + (m & 3);
        const uint32_t w = *reinterpret_cast<const uint32_t *>(tile + 512 * p + 16 * L + 8 * (row >> 3) + 4 * (m >> 2));
        const uint32_t sc = *reinterpret_cast<const uint32_t *>(tile + 2048 + 4 * row);
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tile + 2112 + 2 * row));
        const float db1 = d * float(1 + 2 * int((sc >> (8 * p)) & 15u)), db2 = d * float(1 + 2 * int((sc >> (8 * p + 4)) & 15u));
        k0 = 64 * p + 4 * m;
        k1 = k0 + 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = db1 * float(2 * int((w >> (8 * i)) & 15u) - 15);          // exact: the host decoder's db * magnitude, negated
            v[4 + i] = db2 * float(2 * int((w >> (8 * i + 4)) & 15u) - 15);
        }
    }
    static constexpr int STEP_UNITS = 128;
    __host__ __device__ static void step_unit(int j, int i, int & tl, int & u) { tl = 0; u = (i >> 3) * 32 + j * 8 + (i & 7); }
};

template <> struct Fmt<T_IQ4_XS> {
    // planes p = 0..3 at 512 p + 16 L: {row g: sub-block 2p word t, sub-block 2p + 1 word t; row g + 8: the same};
    // word m of sub-block ib = raw qs bytes [16 ib + 4 m, +4): low nibble of byte j = weight j, high = weight j + 16.
    // 2048 + 8 row: the raw 8-byte header (d, scales_h, scales_l[4]).
    static constexpr int KT = 256, TILE = 2176, RAW = 136;
    __host__ __device__ static uint32_t pack_word(const uint8_t * raw, int rows, int nblk, int rt, int kt, int wi) {
        int row, off;
        if (wi < 512) {
            const int p = wi >> 7, L = (wi >> 2) & 31, c = wi & 3;
            row = 16 * rt + (L >> 2) + 8 * (c >> 1);
            off = 8 + 16 * (2 * p + (c & 1)) + 4 * (L & 3);
        } else {
            row = 16 * rt + ((wi - 512) >> 1);
            off = 4 * ((wi - 512) & 1);
        }
        if (row >= rows) return 0u;
        return ld_u32_bytes(raw + (size_t(row) * nblk + kt) * RAW + off);
    }
    __host__ __device__ static void unit_vals(const uint8_t * tile, const float *, int u, float (&v)[8], int & row, int & k0, int & k1,
                                              const uint32_t * = nullptr) {
        row = u >> 5;
        const int ib = (u >> 2) & 7, m = u & 3;
        const int L = 4 * (row & 7) + m;
        const uint32_t w = *reinterpret_cast<const uint32_t *>(tile + 512 * (ib >> 1) + 16 * L + 8 * (row >> 3) + 4 * (ib & 1));
        const uint8_t * h = tile + 2048 + 8 * row;
        const float d = half_bits_to_float(ld_u16_bytes(h));
        const uint32_t sh = ld_u16_bytes(h + 2);
        const int ls = int((h[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15) | int(((sh >> (2 * ib)) & 3u) << 4);
        const float dl = d * float(ls - 32);
        k0 = 32 * ib + 4 * m;
        k1 = k0 + 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = dl * float(B2_KV((w >> (8 * i)) & 15u));
            v[4 + i] = dl * float(B2_KV((w >> (8 * i + 4)) & 15u));
        }
    }
    static constexpr int STEP_UNITS = 128;
    __host__ __device__ static void step_unit(int j, int i, int & tl, int & u) { tl = 0; u = (i >> 3) * 32 + (2 * j + ((i >> 2) & 1)) * 4 + (i & 3); }
};

template <> struct Fmt<T_IQ4_NL> {
    // 8 L: {row g word t, row g + 8 word t} of the block's 16 code bytes; 256 + 2 row: d (fp16).
    static constexpr int KT = 32, TILE = 288, RAW = 18;
    __host__ __device__ static uint32_t pack_word(const uint8_t * raw, int rows, int nblk, int rt, int kt, int wi) {
        if (wi < 64) {
            const int L = wi >> 1, row = 16 * rt + (L >> 2) + 8 * (wi & 1);
            return row < rows ? ld_u32_bytes(raw + (size_t(row) * nblk + kt) * RAW + 2 + 4 * (L & 3)) : 0u;
        }
        uint32_t v = 0;
        for (int i = 0; i < 2; ++i) {
            const int row = 16 * rt + 2 * (wi - 64) + i;
            if (row < rows) v |= ld_u16_bytes(raw + (size_t(row) * nblk + kt) * RAW) << (16 * i);
        }
        return v;
    }
    __host__ __device__ static void unit_vals(const uint8_t * tile, const float *, int u, float (&v)[8], int & row, int & k0, int & k1,
                                              const uint32_t * = nullptr) {
        row = u >> 2;
        const int m = u & 3, L = 4 * (row & 7) + m;
        const uint32_t w = *reinterpret_cast<const uint32_t *>(tile + 8 * L + 4 * (row >> 3));
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tile + 256 + 2 * row));
        k0 = 4 * m;
        k1 = k0 + 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = d * float(B2_KV((w >> (8 * i)) & 15u));
            v[4 + i] = d * float(B2_KV((w >> (8 * i + 4)) & 15u));
        }
    }
    static constexpr int STEP_UNITS = 128;
    __host__ __device__ static void step_unit(int j, int i, int & tl, int & u) { tl = 2 * j + (i >> 6); u = i & 63; }
};

template <> struct Fmt<T_NVFP4G> {
    // planes p = 0..1 at 512 p + 16 L: {row g: sub-block 2p word t, sub-block 2p + 1 word t; row g + 8: the same};
    // word m of 32-weight sub-block s = raw code bytes [16 s + 4 m, +4): byte i holds weights 2i (low) and 2i + 1.
    // 1024 + 8 row: the eight E4M3 group scales. aux[row]: the fp32 tensor scale of that row.
    static constexpr int KT = 128, TILE = 1152, RAW = 76;
    __host__ __device__ static uint32_t pack_word(const uint8_t * raw, int rows, int nblk, int rt, int kt, int wi) {
        int row, off;
        if (wi < 256) {
            const int p = wi >> 7, L = (wi >> 2) & 31, c = wi & 3;
            row = 16 * rt + (L >> 2) + 8 * (c >> 1);
            off = 12 + 16 * (2 * p + (c & 1)) + 4 * (L & 3);
        } else {
            row = 16 * rt + ((wi - 256) >> 1);
            off = 4 + 4 * ((wi - 256) & 1);
        }
        if (row >= rows) return 0u;
        return ld_u32_bytes(raw + (size_t(row) * nblk + kt) * RAW + off);
    }
    __host__ __device__ static void unit_vals(const uint8_t * tile, const float * aux16, int u, float (&v)[8], int & row, int & k0, int & k1,
                                              const uint32_t * = nullptr) {
        const float lut[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
        row = u >> 4;
        const int s = (u >> 2) & 3, m = u & 3, L = 4 * (row & 7) + m;
        const uint32_t w = *reinterpret_cast<const uint32_t *>(tile + 512 * (s >> 1) + 16 * L + 8 * (row >> 3) + 4 * (s & 1));
        const float d = e4m3_to_float(tile[1024 + 8 * row + 2 * s + (m >> 1)]) * aux16[row];
        k0 = 32 * s + 8 * m;
        k1 = k0 + 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = lut[(w >> (8 * i)) & 15u] * d;
            v[2 * i + 1] = lut[(w >> (8 * i + 4)) & 15u] * d;
        }
    }
    static constexpr int STEP_UNITS = 128;
    __host__ __device__ static void step_unit(int j, int i, int & tl, int & u) { tl = j >> 1; u = (i >> 3) * 16 + (2 * (j & 1) + ((i >> 2) & 1)) * 4 + (i & 3); }
};

// unit u of a tile -> out[row * ld + k]
template <uint32_t T>
__host__ __device__ __forceinline__ void decode_unit(const uint8_t * tile, const float * aux16, int u, float * out, int ld) {
    float v[8];
    int row, k0, k1;
    Fmt<T>::unit_vals(tile, aux16, u, v, row, k0, k1);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[row * ld + k0 + i] = v[i];
    if (k1 >= 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[row * ld + k1 + i] = v[4 + i];
    }
}

// decode a whole tile (16 x KT fp32, row stride ld) with the calling block's threads
template <uint32_t T>
__host__ __device__ __forceinline__ void decode_tile(const uint8_t * tile, const float * aux16, float * out, int ld, int tid, int nthreads,
                                            int units) {
    for (int u = tid; u < units; u += nthreads) decode_unit<T>(tile, aux16, u, out, ld);
}

}  // namespace b2
