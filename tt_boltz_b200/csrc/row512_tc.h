// Host-side interface of the tcgen05 "128 -> 512" producer kernels (row512_tc.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200pf {
namespace r512 {

struct Args {
    const float* z;
    const __nv_bfloat16* z_bf16;       // when set, the pair tensor is read from here (bf16, same [rows][n][128] view) instead of z
    const float* ln_gamma;             // [128] LayerNorm gain, applied by the loader warps
    const float* ln_beta;              // [128] LayerNorm offset
    const uint8_t* mask;               // triangle multiplication: [rows][n]
    const __nv_bfloat16* w;            // [512][128] weights (layout per mode, see row512_tc.cu)
    // triangle-multiplication outputs
    __nv_bfloat16* planes[2];
    long long plane_stride[2], group_stride[2];
    int row_group[2];
    int pitch;
    // MXFP8 planes (launch_trimul_mx): `planes` are byte planes, pitch / plane_stride in bytes
    uint8_t* scales[2];
    int sf_kgroups, sf_row_blocks;
    // triangle-attention outputs
    __nv_bfloat16 *q, *k, *v, *g, *tri_bias;
    const float* w_bias_f32;           // [4][128] triangle-bias rows (already times log2 e)
    long long bias_hs, bias_qs;
    int vt_pitch;
    // geometry: z viewed as [rows][n][128]; transposed != 0 walks columns (incoming / ending)
    int rows, n, transposed;
};

int launch_trimul(const Args& a, cudaStream_t st);
int launch_trimul_mx(const Args& a, cudaStream_t st);
int launch_triatt(const Args& a, cudaStream_t st);

}  // namespace r512
}  // namespace b200pf
