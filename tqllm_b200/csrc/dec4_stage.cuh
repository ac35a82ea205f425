// Staged activation rows of the 4-bit decode kernels (expert_dec4.cu): layout and the device code that writes one row.
// Rows [R][K] of any dtype -> 16-bit fixed point, the row scaled by a power of two so that the largest magnitude lies
// in [2^(bits-2), 2^(bits-1)), split into a signed high byte and an unsigned low byte (x16 = 256 hi + lo).
// One staged row = K / 32 sub-blocks of 64 bytes + K / 256 records of 32 bytes:
//   sub-block: for t = 0..3 the 16 bytes {hi of columns 4t..4t+3, hi of 16+4t..16+4t+3, lo of 4t.., lo of 16+4t..}: the
//              B fragments of the lane with that t for the high-byte and the low-byte MMA;
//   record of 8 sub-blocks: their sums S = sum of x16 over the sub-block, each as the fp16 pair (16 (S >> 10), (S & 1023) / 64)
//              (both exact; together S / 64), in the order 0, 4, 1, 5, 2, 6, 3, 7: the B fragment of the offset-correction
//              MMA of a tile (m16n8k16: k = 2 sub-block + term).
// inv_scale[R] = the inverse of the row's power of two.
#pragma once
#include "common.cuh"

namespace b2 {

__host__ __device__ inline size_t staged_row_bytes(int k) { return size_t(k) * 2 + size_t(k / 256) * 32; }
inline size_t staged_bytes(int rows_x, int k) { return align_up(size_t(rows_x) * staged_row_bytes(k), 256); }

// the row's power-of-two scale from its largest magnitude
__device__ __forceinline__ float stage_scale(float mx, int bits, float & inv) {
    int ex = int((__float_as_uint(mx) >> 23) & 255u) - 127;              // floor(log2(mx)) for a normal mx
    ex = (mx > 0.f && mx < 3e38f) ? max(-100, min(100, ex)) : bits - 2;
    inv = __uint_as_float(uint32_t(127 - (bits - 2) + ex) << 23);
    return __uint_as_float(uint32_t(127 + bits - 2 - ex) << 23);         // 2^(bits - 2 - ex)
}
// One row by one warp, a lane per sub-block (32 consecutive columns each): no cross-lane step except the row maximum, so a
// warp that shares its scheduler with busy warps still stages a row in about a microsecond. Rows must start on 16 bytes.
template <int DT> struct RowLoad;
template <> struct RowLoad<B2MOE_F32> {      // eight columns from two 16-byte loads
    __device__ static void eight(const void * x, size_t first, int i, float (&v)[8]) {
        const float4 * p = reinterpret_cast<const float4 *>(static_cast<const float *>(x) + first) + 2 * i;
        const float4 a = p[0], b = p[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct RowLoad<B2MOE_BF16> {
    __device__ static void eight(const void * x, size_t first, int i, float (&v)[8]) {
        const uint4 q = (reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(x) + first))[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
    }
};
template <> struct RowLoad<B2MOE_F16> {
    __device__ static void eight(const void * x, size_t first, int i, float (&v)[8]) {
        const uint4 q = (reinterpret_cast<const uint4 *>(static_cast<const __half *>(x) + first))[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
            v[2 * j] = f.x; v[2 * j + 1] = f.y;
        }
    }
};
template <int DT>
__device__ inline float stage_row_lanes(const void * __restrict__ x, size_t first, int k, int bits, uint8_t * orow, int lane) {
    float mx = 0.f;
    for (int i = lane; i < (k >> 3); i += 32) {
        float v[8];
        RowLoad<DT>::eight(x, first, i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(v[j]));
    }
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float inv;
    const float scale = stage_scale(mx, bits, inv);
    uint8_t * recs = orow + size_t(k) * 2;
    for (int b = lane; b < (k >> 5); b += 32) {
        uint32_t hi[8], lo[8];                      // bytes of columns 4 i .. 4 i + 3
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v[8];
            RowLoad<DT>::eight(x, first, b * 4 + i, v);
            int q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { q[j] = __float2int_rn(v[j] * scale); sum += q[j]; }
            // byte 1 (high) and byte 0 (low) of four values, in column order
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t a = uint32_t(q[4 * h]), c = uint32_t(q[4 * h + 1]), d = uint32_t(q[4 * h + 2]), e = uint32_t(q[4 * h + 3]);
                hi[2 * i + h] = __byte_perm(__byte_perm(a, c, 0x0051), __byte_perm(d, e, 0x0051), 0x5410);
                lo[2 * i + h] = __byte_perm(__byte_perm(a, c, 0x0040), __byte_perm(d, e, 0x0040), 0x5410);
            }
        }
        uint4 * sb = reinterpret_cast<uint4 *>(orow + size_t(b) * 64);
#pragma unroll
        for (int t = 0; t < 4; ++t) sb[t] = make_uint4(hi[t], hi[4 + t], lo[t], lo[4 + t]);
        const int bb = b & 7;
        reinterpret_cast<__half2 *>(recs + size_t(b >> 3) * 32)[2 * (bb & 3) + (bb >> 2)] =
            __floats2half2_rn(float((sum >> 10) * 16), float(sum & 1023) * 0.015625f);
    }
    return inv;
}
__device__ inline float stage_row_lanes(const void * x, int dtype, size_t first, int k, int bits, uint8_t * orow, int lane) {
    if (dtype == B2MOE_F32) return stage_row_lanes<B2MOE_F32>(x, first, k, bits, orow, lane);
    if (dtype == B2MOE_BF16) return stage_row_lanes<B2MOE_BF16>(x, first, k, bits, orow, lane);
    return stage_row_lanes<B2MOE_F16>(x, first, k, bits, orow, lane);
}
// row `row` of x[.][k] into the array of staged rows `out`, its inverse scale into inv_scale[row]
__device__ inline void stage_row_warp(const void * x, int dtype, int row, int k, int bits, uint8_t * out, float * inv_scale, int lane) {
    const float inv = stage_row_lanes(x, dtype, size_t(row) * k, k, bits, out + size_t(row) * staged_row_bytes(k), lane);
    if (lane == 0) inv_scale[row] = inv;
}

}  // namespace b2
