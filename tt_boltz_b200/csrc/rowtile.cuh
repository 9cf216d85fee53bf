// Building blocks of the "row-tile" kernels: every warp owns units of 32 pair positions
// (32 rows x 128 channels), normalises them into a private bf16 operand tile in shared memory
// and multiplies that tile with weight matrices that the whole CTA keeps in shared memory.
// LayerNorm gains are folded into the weights and offsets into an fp32 bias vector by the host
// packer, so the device only computes (x - mean) * rstd.
#pragma once

#include "mma.cuh"

namespace b200pf {

constexpr int UNIT = 32;                         // pair positions per warp unit
constexpr int WARPS = 8;                         // warps per CTA in the row-tile kernels
constexpr int A_TILE_BYTES = UNIT * APITCH * 2;  // 8704

// Normalise 32 rows of 128 fp32 channels (no affine) into `tile` ([32][APITCH] bf16).
// rowptr(l) returns the address of row l or nullptr (row of zeros).
// Lane layout: 8 lanes per row, 4 rows per pass; lane holds float4 #(j*8 + sub), j = 0..3.
template <class RowPtr>
__device__ __forceinline__ void ln_rows_to_tile(RowPtr rowptr, __nv_bfloat16* tile, int lane) {
    const int sub = lane & 7, rq = lane >> 3;
#pragma unroll 2
    for (int it = 0; it < 8; ++it) {
        int row = it * 4 + rq;
        const float4* p = reinterpret_cast<const float4*>(rowptr(row));
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = p ? __ldg(p + j * 8 + sub) : make_float4(0.f, 0.f, 0.f, 0.f);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        float mean = s * (1.f / KC);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
            ss += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        float rstd = rsqrtf(ss * (1.f / KC) + LN_EPS);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint2 o;
            o.x = pack_bf16x2(v[j].x * rstd, v[j].y * rstd);
            o.y = pack_bf16x2(v[j].z * rstd, v[j].w * rstd);
            *reinterpret_cast<uint2*>(tile + row * APITCH + (j * 8 + sub) * 4) = o;
        }
    }
}

// All A fragments of a 32 x 128 tile: frag[mi][ks][4].
__device__ __forceinline__ void load_a_all(uint32_t tile_addr, int lane, uint32_t (&a)[2][8][4]) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) load_a_frag(tile_addr, APITCH, mi * 16, ks * 16, lane, a[mi][ks]);
}

// acc[mi][nt] += A(32 x 128, fragments in registers) * W[n0 + 8*nt ...][0..128)^T
template <int NT>
__device__ __forceinline__ void warp_gemm_regA(const uint32_t (&a)[2][8][4], uint32_t w_addr, int w_pitch, int n0,
                                               int lane, float (&acc)[2][NT][4]) {
    static_assert(NT % 2 == 0, "n-tiles come in pairs");
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            load_b_frag2(w_addr, w_pitch, n0 + np * 16, ks * 16, lane, b);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                mma_bf16(acc[mi][np * 2], a[mi][ks], b[0], b[1]);
                mma_bf16(acc[mi][np * 2 + 1], a[mi][ks], b[2], b[3]);
            }
        }
    }
}

// Same with the A fragments re-read from shared memory for every k step (saves 64 registers).
template <int NT>
__device__ __forceinline__ void warp_gemm_smemA(uint32_t a_addr, uint32_t w_addr, int w_pitch, int n0, int lane,
                                                float (&acc)[2][NT][4]) {
    static_assert(NT % 2 == 0, "n-tiles come in pairs");
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[2][4];
        load_a_frag(a_addr, APITCH, 0, ks * 16, lane, a[0]);
        load_a_frag(a_addr, APITCH, 16, ks * 16, lane, a[1]);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            load_b_frag2(w_addr, w_pitch, n0 + np * 16, ks * 16, lane, b);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                mma_bf16(acc[mi][np * 2], a[mi], b[0], b[1]);
                mma_bf16(acc[mi][np * 2 + 1], a[mi], b[2], b[3]);
            }
        }
    }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[2][NT][4]) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mi][nt][e] = 0.f;
}

// Copy a [rows][128] bf16 weight matrix from global memory into shared memory with row pitch
// APITCH; all threads of the CTA take part.  Caller synchronises.
__device__ __forceinline__ void load_weights_k128(__nv_bfloat16* dst, const __nv_bfloat16* src, int rows) {
    for (int i = threadIdx.x; i < rows * 16; i += blockDim.x) {
        int r = i >> 4, c = i & 15;
        *reinterpret_cast<uint4*>(dst + r * APITCH + c * 8) = __ldg(reinterpret_cast<const uint4*>(src + r * KC + c * 8));
    }
}

}  // namespace b200pf
