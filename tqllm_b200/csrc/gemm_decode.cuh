// Weight decoders of the tensor-core grouped GEMM: one 64-column step of one 16-row bank tile -> fp16 A operand.
//
// Two warps own a row tile (warp half r decodes rows g + 8 r); lane L = 4 g + t holds, in the bank's lane-major
// layout, the code words of rows g and g + 8 (formats.cuh). Every code word (or pair of IQ3_S grid entries) decodes to eight fp16 values = one 16-byte row of one
// core matrix, so a lane writes whole core-matrix rows with 16-byte stores: per step the rows of cores t and t + 4.
// A decoder is two halves: load<J> reads the lane's raw words of step J into registers, compute<J> turns them into the
// two 16-byte rows; the kernel issues the loads of the next step before it hands the current one over, so that their
// latency passes during the hand-off and the next wait (the compiler cannot move them itself: it cannot prove that the
// operand stores and the raw loads do not alias, and the waits are barriers to it). Which eight columns a word covers depends
// on the format (a Q4_K byte holds column c of two different sub-blocks, an IQ4 byte columns c and c + 16, ...): rather
// than shuffling values between lanes, the GEMM permutes the 64 columns of a step — colmap<T>(pos) is the column stored
// at operand position pos — and the activation rows are written in the same order (the sum over K does not care).
//
// Values: the formula of the format's host decoder (dequantize_host, src/formats/weight/dequant.cpp:80-99,137-150,
// 177-192,352-360,397-409) in fp16 arithmetic on two weights per instruction, arranged so that every intermediate but the
// last is exact: IQ3_S (odd magnitude x (1 + 2 s)) exact, then x d; the 4-bit IQ3_S codes the same; IQ4_NL kvalue x d;
// NVFP4 e2m1 x e4m3 exact (the fp32 row scale is applied to the accumulator in the epilogue): one rounding each. Q4_K:
// sc q exact, x d - the leading fp16 term of dmin m (one rounding), + the rest of dmin m (a second rounding, which removes
// the error the 32 weights of a sub-block would otherwise share). IQ4_XS multiplies the kvalue by
// fp16(d (ls - 32)): that factor's rounding (relative 2^-12, the same for the 32 weights of a sub-block) comes on top.
#pragma once
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "formats.cuh"

namespace b2 {
namespace gdec {

constexpr int A_LBO = 2048 + 32;            // bytes between the k cores of the A operand (+32: conflict-free 16-byte stores)

// column (0..63, inside the step) held at operand position pos (0..63)
template <uint32_t T> __host__ __device__ inline int colmap(int pos) {
    const int c = pos >> 3, q = pos & 7;                               // core, position inside the 16-byte row
    // word c: low nibbles = sub-block 0, high nibbles = sub-block 1; inside each the decoder emits bytes 0, 2, 1, 3 (nibble pairs 16 bits apart)
    if (T == T_Q4_K || T == T_IQ3S4) return (q < 4 ? 0 : 32) + 4 * c + ((q & 1) << 1) + ((q >> 1) & 1);
    if (T == T_IQ4_XS || T == T_IQ4_NL) return 32 * (c >> 2) + 4 * (c & 3) + (q >> 1) + 16 * (q & 1);   // byte i: columns i, i + 16
    return pos;                                                        // IQ3_S, NVFP4G: eight consecutive columns per word
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<const uint32_t *>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<const __half2 *>(&v); }
// the 16-byte row of core matrix `core` for row r16 (0..15) of the warp's tile; base = the warp's first row group
__device__ __forceinline__ uint4 * core_row(uint8_t * base, int core, int r16) {
    return reinterpret_cast<uint4 *>(base + core * A_LBO + (r16 >> 3) * 128 + (r16 & 7) * 16);
}

// 256-entry table byte -> half2(value of the low nibble, value of the high nibble), sixteen interleaved copies
// (entry b of copy c at word 16 b + c) so that the lanes of a warp spread over the banks
constexpr int LUT_COPIES = 16, LUT_BYTES = 256 * LUT_COPIES * 4;      // 16 KB: two lanes share a copy (8 copies: c5 gate/up 3.65 ms, 16: 3.47)
template <uint32_t T> __device__ inline void build_lut(uint32_t * lut, int tid, int nthreads) {
    for (int i = tid; i < 256 * LUT_COPIES; i += nthreads) {
        const int b = i / LUT_COPIES;
        float lo, hi;
        lo = float(c_kvalues_iq4nl[b & 15]);
        hi = float(c_kvalues_iq4nl[b >> 4]);
        lut[i] = pack_h2(lo, hi);
    }
}
// the four bytes of a code word -> eight values times `scale`, in byte order (low, high, low, high, ...)
__device__ __forceinline__ uint4 lut_word(const uint32_t * lut_lane, uint32_t w, __half2 scale) {
    uint4 o;
    o.x = h2_bits(__hmul2(bits_h2(lut_lane[(w & 255u) * LUT_COPIES]), scale));
    o.y = h2_bits(__hmul2(bits_h2(lut_lane[((w >> 8) & 255u) * LUT_COPIES]), scale));
    o.z = h2_bits(__hmul2(bits_h2(lut_lane[((w >> 16) & 255u) * LUT_COPIES]), scale));
    o.w = h2_bits(__hmul2(bits_h2(lut_lane[(w >> 24) * LUT_COPIES]), scale));
    return o;
}

template <uint32_t T> struct Dec;

// ---------------------------------------------------------------------------------------------------------------
template <> struct Dec<T_Q4_K> {
    static constexpr int TAB_BYTES = 0;
    __device__ static void init(void *, int, int) {}
    // The nibbles at bits POS and POS + 16 of w as the half2 (1 + q / 16, 1 + q' / 16): one shift and one logic operation for
    // two weights (the nibble lands in the top four mantissa bits under the exponent of 1.0).
    template <int POS> __device__ __forceinline__ static __half2 pair(uint32_t w) {
        const uint32_t s = POS <= 6 ? w << (6 - POS) : w >> (POS - 6);
        return bits_h2((s & 0x03C003C0u) | 0x3C003C00u);
    }
    // d sc q - dmin m on two weights per instruction: t = (1 + q / 16) (16 sc) - 16 sc = sc q (an integer below 1024:
    // exact), then t d + MH (exact product, one rounding of the weight) and + ML, where MH + ML = -dmin m split into two fp16
    // terms. Rounding the sub-block's d sc or dmin m to one fp16 constant would be cheaper, but that error is shared by the
    // 32 weights of the sub-block and adds up along a row, and rounding t d before the subtraction loses the bits that
    // cancel (both measured: 2.5 to 3 times the output error of this form).
    __device__ __forceinline__ static uint32_t two(__half2 pr, __half2 SC, __half2 NSC, __half2 MH, __half2 ML, __half2 D) {
        return h2_bits(__hadd2(__hfma2(__hfma2(pr, SC, NSC), D, MH), ML));
    }
    struct Sub { __half2 SC, MH, ML; };                              // constants of one sub-block
    __device__ __forceinline__ static uint4 word(uint32_t w, const Sub & s1, const Sub & s2, __half2 D) {
        const __half2 NSC1 = __hneg2(s1.SC), NSC2 = __hneg2(s2.SC);
        uint4 o;
        o.x = two(pair<0>(w), s1.SC, NSC1, s1.MH, s1.ML, D);            // bytes 0 and 2, low nibbles
        o.y = two(pair<8>(w), s1.SC, NSC1, s1.MH, s1.ML, D);            // bytes 1 and 3, low nibbles
        o.z = two(pair<4>(w), s2.SC, NSC2, s2.MH, s2.ML, D);            // bytes 0 and 2, high nibbles
        o.w = two(pair<12>(w), s2.SC, NSC2, s2.MH, s2.ML, D);           // bytes 1 and 3, high nibbles
        return o;
    }
    // Once per 256-column chunk: every lane keeps its row's (d, d); lane t of a row's four lanes turns the header into 16 sc
    // and the two terms of -dmin m of sub-blocks 2 t and 2 t + 1 (both halves of a half2); a step fetches the pair it needs
    // from lane J with shuffles.
    struct Pre { uint32_t SC[2], MH[2], ML[2], D; };
    __device__ __forceinline__ static Pre prep(const uint8_t * chunk, int lane, int r) {
        const int g = lane >> 2, t = lane & 3;
        const uint4 h = *reinterpret_cast<const uint4 *>(chunk + 2048 + 16 * (g + 8 * r));
        // bytes of the 12-byte scale field: s[i] = byte i of (h.y, h.z, h.w)
        const uint32_t hi = h.w;
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        Pre p;
        p.D = (h.x & 0xffffu) * 0x10001u;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int jj = 2 * t + b;
            uint32_t sc, mn;
            if (t < 2) {                                               // jj < 4: sc = s[jj] & 63, mn = s[jj + 4] & 63
                sc = (h.y >> (8 * jj)) & 63u;
                mn = (h.z >> (8 * jj)) & 63u;
            } else {                                                   // jj >= 4: high bits from s[jj - 4] / s[jj], low nibbles from s[jj + 4]
                const uint32_t q = (hi >> (8 * (jj - 4))) & 255u;
                sc = (q & 15u) | ((((h.y >> (8 * (jj - 4))) & 255u) >> 6) << 4);
                mn = (q >> 4) | ((((h.z >> (8 * (jj - 4))) & 255u) >> 6) << 4);
            }
            p.SC[b] = h2_bits(__float2half2_rn(float(16u * sc)));
            const float m = -(dmin * float(mn));                        // exact in fp32 (11 x 6 bits)
            const __half mh = __float2half_rn(m);
            p.MH[b] = h2_bits(__half2half2(mh));
            p.ML[b] = h2_bits(__float2half2_rn(m - __half2float(mh)));
        }
        return p;
    }
    struct Raw { uint2 w; };                                          // the code words of cores t and t + 4 of this warp's row (g + 8 r)
    template <int J> __device__ __forceinline__ static Raw load(const uint8_t * chunk, int lane, int r) {
        return Raw{*reinterpret_cast<const uint2 *>(chunk + 512 * J + 16 * lane + 8 * r)};
    }
    template <int J> __device__ __forceinline__ static void compute(const Raw & raw, const uint8_t *, int lane, const void *, int, const Pre & pre, uint4 (&o)[2]) {
        const int src = (lane & ~3) | J;
        Sub s1, s2;
        s1.SC = bits_h2(__shfl_sync(0xffffffffu, pre.SC[0], src)); s2.SC = bits_h2(__shfl_sync(0xffffffffu, pre.SC[1], src));
        s1.MH = bits_h2(__shfl_sync(0xffffffffu, pre.MH[0], src)); s2.MH = bits_h2(__shfl_sync(0xffffffffu, pre.MH[1], src));
        s1.ML = bits_h2(__shfl_sync(0xffffffffu, pre.ML[0], src)); s2.ML = bits_h2(__shfl_sync(0xffffffffu, pre.ML[1], src));
        o[0] = word(raw.w.x, s1, s2, bits_h2(pre.D));
        o[1] = word(raw.w.y, s1, s2, bits_h2(pre.D));
    }
};

// IQ3_S held as 4-bit codes (formats.cuh, Fmt<T_IQ3S4>): the tile has the Q4_K shape and a weight is d (1 + 2 s) (2 n - 15):
// t = (1 + n / 16) (32 (1 + 2 s)) - 47 (1 + 2 s) = (1 + 2 s) (2 n - 15), an integer below 512 from exact constants, then t d
// (one rounding)
template <> struct Dec<T_IQ3S4> {
    static constexpr int TAB_BYTES = 0;
    __device__ static void init(void *, int, int) {}
    struct Pre { uint32_t SC[2], C[2], D; };
    __device__ __forceinline__ static Pre prep(const uint8_t * chunk, int lane, int r) {
        const int g = lane >> 2, t = lane & 3, row = g + 8 * r;
        const uint32_t sc = *reinterpret_cast<const uint32_t *>(chunk + 2048 + 4 * row);
        Pre p;
        p.D = uint32_t(*reinterpret_cast<const unsigned short *>(chunk + 2112 + 2 * row)) * 0x10001u;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const float s1 = float(1 + 2 * int((sc >> (4 * (2 * t + b))) & 15u));
            p.SC[b] = h2_bits(__float2half2_rn(32.f * s1));
            p.C[b] = h2_bits(__float2half2_rn(-47.f * s1));
        }
        return p;
    }
    __device__ __forceinline__ static uint4 word(uint32_t w, __half2 SC1, __half2 C1, __half2 SC2, __half2 C2, __half2 D) {
        using Q = Dec<T_Q4_K>;
        uint4 o;
        o.x = h2_bits(__hmul2(__hfma2(Q::pair<0>(w), SC1, C1), D));
        o.y = h2_bits(__hmul2(__hfma2(Q::pair<8>(w), SC1, C1), D));
        o.z = h2_bits(__hmul2(__hfma2(Q::pair<4>(w), SC2, C2), D));
        o.w = h2_bits(__hmul2(__hfma2(Q::pair<12>(w), SC2, C2), D));
        return o;
    }
    using Raw = Dec<T_Q4_K>::Raw;
    template <int J> __device__ __forceinline__ static Raw load(const uint8_t * chunk, int lane, int r) { return Dec<T_Q4_K>::load<J>(chunk, lane, r); }
    template <int J> __device__ __forceinline__ static void compute(const Raw & raw, const uint8_t *, int lane, const void *, int, const Pre & pre, uint4 (&o)[2]) {
        const int src = (lane & ~3) | J;
        const __half2 SC1 = bits_h2(__shfl_sync(0xffffffffu, pre.SC[0], src)), C1 = bits_h2(__shfl_sync(0xffffffffu, pre.C[0], src));
        const __half2 SC2 = bits_h2(__shfl_sync(0xffffffffu, pre.SC[1], src)), C2 = bits_h2(__shfl_sync(0xffffffffu, pre.C[1], src));
        o[0] = word(raw.w.x, SC1, C1, SC2, C2, bits_h2(pre.D));
        o[1] = word(raw.w.y, SC1, C1, SC2, C2, bits_h2(pre.D));
    }
};

// ---------------------------------------------------------------------------------------------------------------
template <> struct Dec<T_IQ4_XS> {
    static constexpr int TAB_BYTES = LUT_BYTES;
    __device__ static void init(void * tab, int tid, int n) { build_lut<T_IQ4_XS>(static_cast<uint32_t *>(tab), tid, n); }
    // once per chunk: lane t holds fp16(d (ls - 32)) of sub-blocks 2 t and 2 t + 1 of its row
    struct Pre { uint32_t dl[2]; };
    __device__ __forceinline__ static Pre prep(const uint8_t * chunk, int lane, int r) {
        const int g = lane >> 2, t = lane & 3;
        const uint2 h = *reinterpret_cast<const uint2 *>(chunk + 2048 + 8 * (g + 8 * r));       // d, scales_h | scales_l[4]
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const uint32_t sh = h.x >> 16;
        Pre p;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int ib = 2 * t + b;
            const int ls = int((h.y >> (4 * ib)) & 15u) | int(((sh >> (2 * ib)) & 3u) << 4);
            p.dl[b] = h2_bits(__float2half2_rn(d * float(ls - 32)));
        }
        return p;
    }
    using Raw = Dec<T_Q4_K>::Raw;
    template <int J> __device__ __forceinline__ static Raw load(const uint8_t * chunk, int lane, int r) { return Dec<T_Q4_K>::load<J>(chunk, lane, r); }
    template <int J> __device__ __forceinline__ static void compute(const Raw & raw, const uint8_t *, int lane, const void * tab, int, const Pre & pre, uint4 (&o)[2]) {
        const int src = (lane & ~3) | J;
        const uint32_t * lut = static_cast<const uint32_t *>(tab) + (lane & (LUT_COPIES - 1));
        const uint32_t d0 = __shfl_sync(0xffffffffu, pre.dl[0], src), d1 = __shfl_sync(0xffffffffu, pre.dl[1], src);
        o[0] = lut_word(lut, raw.w.x, bits_h2(d0));
        o[1] = lut_word(lut, raw.w.y, bits_h2(d1));
    }
};

template <> struct Dec<T_IQ4_NL> {
    struct Pre {};
    __device__ __forceinline__ static Pre prep(const uint8_t *, int, int) { return Pre{}; }
    static constexpr int TAB_BYTES = LUT_BYTES;
    __device__ static void init(void * tab, int tid, int n) { build_lut<T_IQ4_NL>(static_cast<uint32_t *>(tab), tid, n); }
    struct Raw { uint32_t w[2]; unsigned short d[2]; };                // per 32-column tile of the step: the row's code word and its fp16 scale
    template <int J> __device__ __forceinline__ static Raw load(const uint8_t * chunk, int lane, int r) {
        const int g = lane >> 2;
        Raw raw;
#pragma unroll
        for (int b = 0; b < 2; ++b) {                                   // the step's two 32-column tiles
            const uint8_t * tile = chunk + (2 * J + b) * Fmt<T_IQ4_NL>::TILE;
            raw.w[b] = *reinterpret_cast<const uint32_t *>(tile + 8 * lane + 4 * r);
            raw.d[b] = *reinterpret_cast<const unsigned short *>(tile + 256 + 2 * (g + 8 * r));
        }
        return raw;
    }
    template <int J> __device__ __forceinline__ static void compute(const Raw & raw, const uint8_t *, int lane, const void * tab, int, const Pre &, uint4 (&o)[2]) {
        const uint32_t * lut = static_cast<const uint32_t *>(tab) + (lane & (LUT_COPIES - 1));
#pragma unroll
        for (int b = 0; b < 2; ++b) o[b] = lut_word(lut, raw.w[b], __half2half2(__ushort_as_half(raw.d[b])));
    }
};

// ---------------------------------------------------------------------------------------------------------------
template <> struct Dec<T_NVFP4G> {
    struct Pre {};
    __device__ __forceinline__ static Pre prep(const uint8_t *, int, int) { return Pre{}; }
    static constexpr int TAB_BYTES = 0;
    __device__ static void init(void *, int, int) {}
    // the eight e2m1 codes of a word -> eight fp16 values (the hardware conversion, two codes per instruction: low nibble
    // first) times `scale`; every product of an e2m1 and an e4m3 value is exact in fp16
    __device__ __forceinline__ static uint4 word(uint32_t w, __half2 scale) {
        uint32_t v0, v1, v2, v3;
        asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
            " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(w));
        uint4 o;
        o.x = h2_bits(__hmul2(bits_h2(v0), scale));
        o.y = h2_bits(__hmul2(bits_h2(v1), scale));
        o.z = h2_bits(__hmul2(bits_h2(v2), scale));
        o.w = h2_bits(__hmul2(bits_h2(v3), scale));
        return o;
    }
    struct Raw { uint2 w; uint32_t scw; };                            // the row's two code words of the step and its four E4M3 group scales
    template <int J> __device__ __forceinline__ static Raw load(const uint8_t * chunk, int lane, int r) {
        const int g = lane >> 2;
        const uint8_t * tile = chunk + (J >> 1) * Fmt<T_NVFP4G>::TILE;
        constexpr int P = J & 1;                                         // plane = sub-blocks 2 P, 2 P + 1 of the 128-column tile
        Raw raw;
        raw.w = *reinterpret_cast<const uint2 *>(tile + 512 * P + 16 * lane + 8 * r);           // this warp's row: g + 8 r
        raw.scw = *reinterpret_cast<const uint32_t *>(tile + 1024 + 8 * (g + 8 * r) + 4 * P);   // scales of sub-blocks 2 P (bytes 0, 1), 2 P + 1 (bytes 2, 3)
        return raw;
    }
    template <int J> __device__ __forceinline__ static void compute(const Raw & raw, const uint8_t *, int lane, const void *, int, const Pre &, uint4 (&o)[2]) {
        const int t = lane & 3;
        const uint32_t wr[2] = {raw.w.x, raw.w.y};
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const uint32_t sbyte = (raw.scw >> (16 * b + 8 * (t >> 1))) & 255u;       // the 16-weight group of word t
            const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(sbyte | (sbyte << 8)), __NV_E4M3);
            o[b] = word(wr[b], __half2(hr));
        }
    }
};

// ---------------------------------------------------------------------------------------------------------------
template <> struct Dec<T_IQ3_S> {
    struct Pre {};
    __device__ __forceinline__ static Pre prep(const uint8_t *, int, int) { return Pre{}; }
    // table: grid entry -> its four odd magnitudes as fp16 (8 bytes)
    static constexpr int TAB_BYTES = 512 * 8;
    __device__ static void init(void * tab, int tid, int n) {
        uint2 * t2 = static_cast<uint2 *>(tab);
        for (int i = tid; i < 512; i += n) {
            const uint32_t m = c_iq3s_grid[i];
            t2[i] = make_uint2(pack_h2(float(m & 255u), float((m >> 8) & 255u)), pack_h2(float((m >> 16) & 255u), float(m >> 24)));
        }
    }
    struct Raw {};                                                     // 13 words a lane: read inside compute
    template <int J> __device__ __forceinline__ static Raw load(const uint8_t *, int, int) { return Raw{}; }
    template <int J> __device__ __forceinline__ static void compute(const Raw &, const uint8_t * chunk, int lane, const void * tab, int r, const Pre &, uint4 (&out)[2]) {
        const int g = lane >> 2;
        const uint2 * mags = static_cast<const uint2 *>(tab);
        uint32_t w[13];
        {
            const uint4 p0 = reinterpret_cast<const uint4 *>(chunk)[lane], p1 = reinterpret_cast<const uint4 *>(chunk + 512)[lane],
                        p2 = reinterpret_cast<const uint4 *>(chunk + 1024)[lane];
            w[0] = p0.x; w[1] = p0.y; w[2] = p0.z; w[3] = p0.w; w[4] = p1.x; w[5] = p1.y; w[6] = p1.z; w[7] = p1.w;
            w[8] = p2.x; w[9] = p2.y; w[10] = p2.z; w[11] = p2.w;
            w[12] = reinterpret_cast<const uint32_t *>(chunk + 1536)[lane];
        }
        {
            const int row = g + 8 * r;
            const uint32_t scales = *reinterpret_cast<const uint32_t *>(chunk + 1664 + 4 * row);
            const __half2 d2 = __half2half2(__ushort_as_half(*reinterpret_cast<const unsigned short *>(chunk + 1728 + 2 * row)));
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                constexpr int dummy = 0; (void)dummy;
                const int ib = 2 * J + b;
                const __half2 s2 = __float2half2_rn(float(1 + 2 * int((scales >> (4 * ib)) & 15u)));      // 1 + 2 s: exact
                const uint32_t sg = r ? w[11 + (ib >> 2)] : w[9 + (ib >> 2)];
                uint32_t o[4];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    // entry n = 16 r + 2 ib + jj of the lane's 9-bit stream; r = 1 starts at bit 144 = word 4, bit 16
                    const int n0 = 2 * ib + jj;
                    const int bitA = 9 * n0, bitB = 9 * (16 + n0);
                    const uint32_t ia = (((bitA & 31) > 23 ? __funnelshift_r(w[bitA >> 5], w[(bitA >> 5) + 1], bitA & 31) : w[bitA >> 5] >> (bitA & 31))) & 511u;
                    const uint32_t ibx = (((bitB & 31) > 23 ? __funnelshift_r(w[bitB >> 5], w[(bitB >> 5) + 1 > 8 ? 8 : (bitB >> 5) + 1], bitB & 31) : w[bitB >> 5] >> (bitB & 31))) & 511u;
                    const uint32_t idx = r ? ibx : ia;
                    const uint2 m = mags[idx];
                    const int R = 2 * (ib & 3) + jj;
                    // (mag x (1 + 2 s)) exact (<= 465), x d: one rounding; then the sign bits of the pairs (0, 1) and (2, 3)
                    o[2 * jj] = h2_bits(__hmul2(__hmul2(bits_h2(m.x), s2), d2)) ^ ((sg << (15 - R)) & 0x80008000u);
                    o[2 * jj + 1] = h2_bits(__hmul2(__hmul2(bits_h2(m.y), s2), d2)) ^ ((R <= 7 ? sg << (7 - R) : sg >> (R - 7)) & 0x80008000u);
                }
                out[b] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
};

}  // namespace gdec
}  // namespace b2
