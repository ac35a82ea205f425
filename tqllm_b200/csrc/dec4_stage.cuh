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
// sub-block b of a row: one lane per column; every lane of the warp calls it. orow / recs: the row's staged bytes and records
// (global or shared memory)
__device__ __forceinline__ void stage_sub_block(const void * x, int dtype, size_t row_first, int b, float scale, uint8_t * orow, uint8_t * recs, int lane) {
    const int t = (lane & 15) >> 2, j = lane & 3, h = lane >> 4;
    const int v = __float2int_rn(load_act(x, dtype, row_first + 32 * b + lane) * scale);
    uint8_t * sb = orow + size_t(b) * 64 + t * 16 + h * 4 + j;
    sb[0] = uint8_t(v >> 8);
    sb[8] = uint8_t(v & 255);
    int sum = v;
    for (int d = 16; d; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane == 0) {
        const int bb = b & 7;
        reinterpret_cast<__half2 *>(recs + size_t(b >> 3) * 32)[2 * (bb & 3) + (bb >> 2)] =
            __floats2half2_rn(float((sum >> 10) * 16), float(sum & 1023) * 0.015625f);
    }
}
// one whole row (elements [first, first + k) of x) by one warp into `orow`; returns the row's inverse scale
__device__ inline float stage_row_to(const void * x, int dtype, size_t first, int k, int bits, uint8_t * orow, int lane) {
    float mx = 0.f;
    for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(load_act(x, dtype, first + j)));
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float inv;
    const float scale = stage_scale(mx, bits, inv);
    uint8_t * recs = orow + size_t(k) * 2;
#pragma unroll 4
    for (int b = 0; b < (k >> 5); ++b) stage_sub_block(x, dtype, first, b, scale, orow, recs, lane);
    return inv;
}
// The same row with a lane per sub-block (32 consecutive columns each): no cross-lane step except the row maximum, for the
// warp that stages rows inside the down product while the consumer warps take most issue slots. fp32 rows, k a multiple of 32.
__device__ inline float stage_row_f32_lanes(const float * __restrict__ x, size_t first, int k, int bits, uint8_t * orow, int lane) {
    const float4 * row4 = reinterpret_cast<const float4 *>(x + first);
    float mx = 0.f;
    for (int j = lane; j < (k >> 2); j += 32) {
        const float4 v = row4[j];
        mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float inv;
    const float scale = stage_scale(mx, bits, inv);
    uint8_t * recs = orow + size_t(k) * 2;
    for (int b = lane; b < (k >> 5); b += 32) {
        uint32_t hi[8], lo[8];                      // bytes of columns 4 i .. 4 i + 3
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = row4[b * 8 + i];
            const int a = __float2int_rn(v.x * scale), c = __float2int_rn(v.y * scale), d = __float2int_rn(v.z * scale), e = __float2int_rn(v.w * scale);
            sum += a + c + d + e;
            // byte 1 (high) and byte 0 (low) of the four values, in column order
            hi[i] = __byte_perm(__byte_perm(uint32_t(a), uint32_t(c), 0x0051), __byte_perm(uint32_t(d), uint32_t(e), 0x0051), 0x5410);
            lo[i] = __byte_perm(__byte_perm(uint32_t(a), uint32_t(c), 0x0040), __byte_perm(uint32_t(d), uint32_t(e), 0x0040), 0x5410);
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
// row `row` of x[.][k] into the array of staged rows `out`, its inverse scale into inv_scale[row]
__device__ inline void stage_row_warp(const void * x, int dtype, int row, int k, int bits, uint8_t * out, float * inv_scale, int lane) {
    const float inv = stage_row_to(x, dtype, size_t(row) * k, k, bits, out + size_t(row) * staged_row_bytes(k), lane);
    if (lane == 0) inv_scale[row] = inv;
}

}  // namespace b2
