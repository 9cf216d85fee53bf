// MXFP8 operand planes of the triangle multiplication: e4m3 values, one e8m0 scale (a power of
// two) per 32 consecutive elements along the contraction index k.
//
// Values: byte planes [channel][row][pitch], pitch a multiple of 16 bytes.
// Scales: blocks of 512 bytes, one per (channel, group of 4 k-blocks = 128 k, block of 128 rows),
//   block index = (channel * kgroups + kgroup) * row_blocks + row / 128,
//   byte inside = (row % 32) * 16 + ((row % 128) / 32) * 4 + k_block % 4.
// This is the order tcgen05.cp (32x128b.warpx4) wants: lane i of tensor memory receives 16 bytes =
// 4 columns, column g holding the 4 k-block scales of row 32 g + i, which is how a block-scaled
// tcgen05.mma looks its scales up.  row_blocks is even so that the two blocks a 256-row B tile
// needs are adjacent.  Scale bytes of rows that do not exist stay 0 (= 2^-127, harmless against
// the zero values TMA fills in for those rows).
//
// Scale rule: the smallest power of two with amax / scale <= 448 (the largest e4m3 value), so no
// element saturates; blocks of zeros get scale byte 0.
#pragma once
#include <cuda_fp8.h>
#include <stdint.h>

namespace b200pf {
namespace mx {

constexpr int BLOCK = 32;          // elements per scale
constexpr int SF_BLOCK_BYTES = 512;

__host__ __device__ inline int kgroups(int cols) { return (cols + 127) / 128; }
__host__ __device__ inline int row_blocks(int rows) { return 2 * ((rows + 255) / 256); }
__host__ __device__ inline long long scale_bytes(int rows, int cols, int channels) {
    return (long long)channels * kgroups(cols) * row_blocks(rows) * SF_BLOCK_BYTES;
}
__host__ __device__ inline long long scale_offset(int d, int row, int kblock, int kgroups_, int row_blocks_) {
    return (((long long)d * kgroups_ + (kblock >> 2)) * row_blocks_ + (row >> 7)) * SF_BLOCK_BYTES +
           (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kblock & 3);
}

// e8m0 byte of the scale for a block whose largest magnitude is amax (finite, >= 0).
__device__ __forceinline__ uint32_t scale_byte(float amax) {
    const uint32_t bits = __float_as_uint(amax * (1.0f / 448.0f));
    uint32_t e = (bits >> 23) + ((bits & 0x7FFFFFu) ? 1u : 0u);
    return e > 253u ? 253u : e;
}
// 2^(127 - e): what a value is multiplied by before rounding to e4m3.
__device__ __forceinline__ float inv_scale(uint32_t e) { return __uint_as_float((254u - e) << 23); }
// 2^(e - 127) for e >= 1; e == 0 only occurs for all-zero blocks, where any finite value will do.
__device__ __forceinline__ float scale_value(uint32_t e) { return __uint_as_float((e ? e : 1u) << 23); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

}  // namespace mx
}  // namespace b200pf
