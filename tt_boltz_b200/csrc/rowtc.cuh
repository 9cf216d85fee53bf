// Building blocks of the tcgen05 "row-tile" kernels: a CTA owns tiles of 128 pair positions,
// loader warps normalise them into a bf16 A operand in shared memory (K-major, 128-byte swizzle:
// the layout TMA would produce), one thread issues tcgen05.mma against weight matrices kept in
// shared memory in the same layout, epilogue warps read the fp32 result from TMEM.
#pragma once

#include "sm100.cuh"

namespace b200pf {
namespace rtc {

constexpr int TM = 128;                     // positions per tile
constexpr int KC = 128;                     // channels
constexpr int A_KB_BYTES = TM * 128;        // one 64-channel k-block of the A tile
constexpr int A_TILE_BYTES = 2 * A_KB_BYTES;

// Byte offset of the 16-byte chunk `chunk` (8 channels) of row `row` inside one k-block.
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
    return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// Copy W[rows][128] (bf16, row-major in global memory) into shared memory as two k-blocks of
// [rows][128 bytes] with the 128-byte swizzle.  All `nthreads` threads take part.
__device__ __forceinline__ void load_weights_sw128(uint8_t* dst, const __nv_bfloat16* src, int rows, int tid, int nthreads) {
    for (int i = tid; i < rows * 16; i += nthreads) {
        int r = i >> 4, c16 = i & 15;
        uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (long long)r * KC) + c16);
        *reinterpret_cast<uint4*>(dst + (c16 >> 3) * (rows * 128) + sw128(r, c16 & 7)) = v;
    }
}

// LayerNorm (no affine) of 16 rows into the A tile; called by one warp.  Lane layout: 8 lanes per
// row, 4 rows per pass; lane (sub, j) owns channels (j*8 + sub)*4 .. +3.  `xh` receives the
// normalised fp32 values of the last processed pass only when KEEP is set (used for the extra
// head projections), via the callback `per_row(row_in_tile, v[4] normalised float4s)`.
template <class RowPtr, class PerRow>
__device__ __forceinline__ void ln_rows16_to_sw128(RowPtr rowptr, uint8_t* a_tile, int row0, int lane, PerRow per_row) {
    const int sub = lane & 7, rq = lane >> 3;
    float4 v[4][4];
    const float4* ptrs[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        ptrs[it] = reinterpret_cast<const float4*>(rowptr(row0 + it * 4 + rq));
#pragma unroll
        for (int j = 0; j < 4; ++j)
            v[it][j] = ptrs[it] ? __ldg(ptrs[it] + j * 8 + sub) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int row = row0 + it * 4 + rq;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) s += (v[it][j].x + v[it][j].y) + (v[it][j].z + v[it][j].w);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        const float mean = s * (1.f / KC);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[it][j].x -= mean; v[it][j].y -= mean; v[it][j].z -= mean; v[it][j].w -= mean;
            ss += (v[it][j].x * v[it][j].x + v[it][j].y * v[it][j].y) + (v[it][j].z * v[it][j].z + v[it][j].w * v[it][j].w);
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        const float rstd = rsqrtf(ss * (1.f / KC) + LN_EPS);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[it][j].x *= rstd; v[it][j].y *= rstd; v[it][j].z *= rstd; v[it][j].w *= rstd;
            uint2 o;
            o.x = pack_bf16x2(v[it][j].x, v[it][j].y);
            o.y = pack_bf16x2(v[it][j].z, v[it][j].w);
            const int chunk = (j & 1) * 4 + (sub >> 1);
            *reinterpret_cast<uint2*>(a_tile + (j >> 1) * A_KB_BYTES + sw128(row, chunk) + (sub & 1) * 8) = o;
        }
        per_row(row, v[it]);
    }
}

// D[tmem] = A(128 x 128, smem) * W(rows n0 .. n0 + n_cols of a [w_rows][128] matrix, smem)^T: 8 k-steps.
__device__ __forceinline__ void issue_gemm_k128(uint32_t tmem_d, uint32_t a_addr, uint32_t w_addr, int w_rows, int n0,
                                                uint32_t idesc) {
    using namespace sm100;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int kb = ks >> 2, kk = ks & 3;
        uint64_t da = make_desc_k_sw128(a_addr + kb * A_KB_BYTES + kk * 32);
        uint64_t db = make_desc_k_sw128(w_addr + kb * (w_rows * 128) + n0 * 128 + kk * 32);
        umma_bf16(tmem_d, da, db, idesc, ks ? 1u : 0u);
    }
}

__device__ __forceinline__ float sigmoid_tanh(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}

}  // namespace rtc
}  // namespace b200pf
