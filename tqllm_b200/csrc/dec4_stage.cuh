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
// sub-block b of a row: one lane per column; every lane of the warp calls it
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
// one whole row by one warp
__device__ inline void stage_row_warp(const void * x, int dtype, int row, int k, int bits, uint8_t * out, float * inv_scale, int lane) {
    const size_t first = size_t(row) * k;
    float mx = 0.f;
    for (int j = lane; j < k; j += 32) mx = fmaxf(mx, fabsf(load_act(x, dtype, first + j)));
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float inv;
    const float scale = stage_scale(mx, bits, inv);
    if (lane == 0) inv_scale[row] = inv;
    uint8_t * orow = out + size_t(row) * staged_row_bytes(k);
    uint8_t * recs = orow + size_t(k) * 2;
    for (int b = 0; b < (k >> 5); ++b) stage_sub_block(x, dtype, first, b, scale, orow, recs, lane);
}

}  // namespace b2
