// Outer-product mean (MSA stack -> pair tensor): the stages around its two GEMMs.
//
//   z[i][j][:] += W_o * vec( sum_s a[s][i][:] (x) b[s][j][:] ) / max(1, sum_s mask[s][i] mask[s][j]) + bias
//   a = mask * (LN(m) W_a^T),  b = mask * (LN(m) W_b^T)            (m: [S][N][64], 32 channels each)
//
// The sum over the S sequences is one K-major GEMM with rows (i, c) and columns (j, d)
// (b200pf_opm_outer: the triangle-multiplication contraction kernel writing each pair's 32 x 32 block
// contiguously), the projection a second one over the 1024 (c, d) products (b200pf_trimul_contract with one
// channel).  This file holds what feeds and drains them:
//   opm_producer_kernel : LayerNorm + both projections + mask, written TRANSPOSED (sequence index contiguous) as
//                         the GEMM's K-major operands; one thread per (sequence, token) row, weights broadcast from
//                         shared memory, fp32 throughout, bf16 on store.
//   opm_mask_bits_kernel: the MSA mask as one bit per sequence, 32 sequences per word and token.
//   opm_finalize_kernel : pair counts by popcount of the two tokens' words, then y / count + bias added into (or
//                         written over) the fp32 pair rows.
#include "common.cuh"

namespace b200pf {
namespace opm {

constexpr int CM = 64;            // MSA channels
constexpr int CH = 32;            // projected channels per side
constexpr int PROD_THREADS = 128;
constexpr int FIN_THREADS = 256, FIN_J = 64;
constexpr int MAX_WORDS = 512;    // sequences / 32 the finalize kernel keeps in shared memory (S <= 16384)

__global__ void __launch_bounds__(PROD_THREADS)
opm_producer_kernel(const float* __restrict__ m, const uint8_t* __restrict__ mask, const float* __restrict__ gamma,
                    const float* __restrict__ beta, const float* __restrict__ w_ab, __nv_bfloat16* __restrict__ a_t,
                    __nv_bfloat16* __restrict__ b_t, int s_len, int n, int pitch) {
    __shared__ __align__(16) float w_s[2 * CH * CM];
    __shared__ float gb_s[2 * CM];
    for (int i = threadIdx.x; i < 2 * CH * CM; i += PROD_THREADS) w_s[i] = w_ab[i];
    if (threadIdx.x < CM) { gb_s[threadIdx.x] = gamma[threadIdx.x]; gb_s[CM + threadIdx.x] = beta[threadIdx.x]; }
    __syncthreads();
    const int tok = blockIdx.y;
    const int s = blockIdx.x * PROD_THREADS + threadIdx.x;
    if (s >= s_len) return;
    const float4* src = reinterpret_cast<const float4*>(m + ((long long)s * n + tok) * CM);
    float x[CM];
#pragma unroll
    for (int j = 0; j < CM / 4; ++j) {
        const float4 v = __ldg(src + j);
        x[4 * j] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
    }
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < CM; ++k) sum += x[k];
    const float mean = sum * (1.f / CM);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < CM; ++k) { x[k] -= mean; ss = fmaf(x[k], x[k], ss); }
    const float rstd = rsqrtf(ss * (1.f / CM) + LN_EPS);
#pragma unroll
    for (int k = 0; k < CM; ++k) x[k] = fmaf(x[k] * rstd, gb_s[k], gb_s[CM + k]);
    const float keep = mask[(long long)s * n + tok] ? 1.f : 0.f;
    __nv_bfloat16* a_row = a_t + (long long)tok * CH * pitch + s;
    __nv_bfloat16* b_row = b_t + (long long)tok * CH * pitch + s;
#pragma unroll 4
    for (int o = 0; o < 2 * CH; ++o) {
        const float4* wr = reinterpret_cast<const float4*>(w_s + o * CM);
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int k4 = 0; k4 < CM / 4; k4 += 2) {
            const float4 w0 = wr[k4], w1 = wr[k4 + 1];
            acc0 = fmaf(w0.x, x[4 * k4], fmaf(w0.y, x[4 * k4 + 1], fmaf(w0.z, x[4 * k4 + 2], fmaf(w0.w, x[4 * k4 + 3], acc0))));
            acc1 = fmaf(w1.x, x[4 * k4 + 4], fmaf(w1.y, x[4 * k4 + 5], fmaf(w1.z, x[4 * k4 + 6], fmaf(w1.w, x[4 * k4 + 7], acc1))));
        }
        const __nv_bfloat16 r = __float2bfloat16((acc0 + acc1) * keep);
        if (o < CH) a_row[(long long)o * pitch] = r;
        else b_row[(long long)(o - CH) * pitch] = r;
    }
}

__global__ void opm_mask_bits_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ bits, int s_len, int n, int words) {
    const int tok = blockIdx.x * blockDim.x + threadIdx.x, w = blockIdx.y;
    if (tok >= n) return;
    uint32_t v = 0;
    for (int b = 0; b < 32; ++b) {
        const int s = w * 32 + b;
        if (s < s_len && mask[(long long)s * n + tok]) v |= 1u << b;
    }
    bits[(long long)tok * words + w] = v;
}

__global__ void __launch_bounds__(FIN_THREADS)
opm_finalize_kernel(const __nv_bfloat16* __restrict__ y, const uint32_t* __restrict__ bits, const float* __restrict__ bias,
                    float* __restrict__ z, int i0, int n, int words, int accumulate) {
    __shared__ uint32_t bi_s[MAX_WORDS];
    __shared__ float inv_s[FIN_J];
    const int il = blockIdx.y, i = i0 + il, j0 = blockIdx.x * FIN_J;
    for (int w = threadIdx.x; w < words; w += FIN_THREADS) bi_s[w] = bits[(long long)i * words + w];
    __syncthreads();
    if (threadIdx.x < FIN_J) {
        const int j = j0 + threadIdx.x;
        int cnt = 0;
        if (j < n) {
            const uint32_t* bj = bits + (long long)j * words;
            for (int w = 0; w < words; ++w) cnt += __popc(bi_s[w] & __ldg(bj + w));
        }
        inv_s[threadIdx.x] = 1.f / (float)(cnt > 0 ? cnt : 1);
    }
    __syncthreads();
    const int c4 = threadIdx.x & 31;                                  // four channels
    const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias) + c4);
    for (int jl = threadIdx.x >> 5; jl < FIN_J; jl += FIN_THREADS / 32) {
        const int j = j0 + jl;
        if (j >= n) break;
        const long long row = (long long)il * n + j;
        const uint2 yv = __ldg(reinterpret_cast<const uint2*>(y + row * 128) + c4);
        const float inv = inv_s[jl];
        float4 o;
        o.x = fmaf(bf16_lo(yv.x), inv, b4.x);
        o.y = fmaf(bf16_hi(yv.x), inv, b4.y);
        o.z = fmaf(bf16_lo(yv.y), inv, b4.z);
        o.w = fmaf(bf16_hi(yv.y), inv, b4.w);
        float4* zp = reinterpret_cast<float4*>(z + row * 128) + c4;
        if (accumulate) {
            const float4 old = *zp;
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        *zp = o;
    }
}

}  // namespace opm
}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_opm_producer(const float* m, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                                   const float* w_ab, b200pf_bf16* a_t, b200pf_bf16* b_t, int s_len, int n, int pitch,
                                   void* stream) {
    using namespace opm;
    B200PF_REQUIRE(m && mask && ln_gamma && ln_beta && w_ab && a_t && b_t, B200PF_ERR_INVALID, "opm_producer: null pointer");
    B200PF_REQUIRE(aligned16(m) && aligned16(w_ab), B200PF_ERR_INVALID, "opm_producer: m and w_ab must be 16-byte aligned");
    B200PF_REQUIRE(s_len > 0 && n > 0 && n <= 65535 && pitch >= s_len, B200PF_ERR_INVALID, "opm_producer: bad sizes");
    dim3 grid((unsigned)((s_len + PROD_THREADS - 1) / PROD_THREADS), (unsigned)n);
    opm_producer_kernel<<<grid, PROD_THREADS, 0, (cudaStream_t)stream>>>(m, mask, ln_gamma, ln_beta, w_ab, (__nv_bfloat16*)a_t,
                                                                          (__nv_bfloat16*)b_t, s_len, n, pitch);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_opm_mask_bits(const uint8_t* mask, uint32_t* bits, int s_len, int n, void* stream) {
    using namespace opm;
    B200PF_REQUIRE(mask && bits && s_len > 0 && n > 0, B200PF_ERR_INVALID, "opm_mask_bits: bad arguments");
    const int words = (s_len + 31) / 32;
    B200PF_REQUIRE(words <= 65535, B200PF_ERR_UNSUPPORTED, "opm_mask_bits: too many sequences");
    dim3 grid((unsigned)((n + 127) / 128), (unsigned)words);
    opm_mask_bits_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(mask, bits, s_len, n, words);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_opm_finalize(const b200pf_bf16* y, const uint32_t* bits, const float* bias, float* z, int s_len,
                                   int i0, int n_i, int n, int accumulate, void* stream) {
    using namespace opm;
    B200PF_REQUIRE(y && bits && bias && z && aligned16(y) && aligned16(z) && aligned16(bias), B200PF_ERR_INVALID,
                   "opm_finalize: null or misaligned pointer");
    const int words = (s_len + 31) / 32;
    B200PF_REQUIRE(s_len > 0 && words <= MAX_WORDS, B200PF_ERR_UNSUPPORTED, "opm_finalize: at most %d sequences", MAX_WORDS * 32);
    B200PF_REQUIRE(n > 0 && i0 >= 0 && n_i > 0 && i0 + n_i <= n && n_i <= 65535, B200PF_ERR_INVALID, "opm_finalize: bad sizes");
    dim3 grid((unsigned)((n + FIN_J - 1) / FIN_J), (unsigned)n_i);
    opm_finalize_kernel<<<grid, FIN_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y, bits, bias, z, i0, n, words, accumulate);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
