// Row kernels of the MSA stack (64-channel MSA activations m[S][N][64]) around the GEMMs that the
// triangle-multiplication contraction kernel runs for it:
//   pair-weighted averaging  m += W_o (sigmoid(W_g LN(m)) * sum_j softmax_j(W_z LN(z) + mask)[i][j] (W_m LN(m))[j])
//   MSA transition           m += W_3 (silu(W_1 LN(m)) * W_2 LN(m))
// Every GEMM operand is bf16 and K-major; the token axis is padded to a multiple of 8 (`np`) so that rows of
// every operand start 16-byte aligned, with zero rows for the padding tokens (the pair-weighted averaging pads to
// 32: its projected rows are written in groups of np columns).
#include "common.cuh"

namespace b200pf {
namespace msa {

constexpr int CM = 64;

// LayerNorm over the 64 channels of every (sequence, token) row -> bf16 [S][np][64]; rows of padding tokens are zero.
// Sixteen lanes per row (one float4 each), two rows per warp and step.
__global__ void __launch_bounds__(256)
ln_rows_bf16_kernel(const float* __restrict__ m, const float* __restrict__ gamma, const float* __restrict__ beta,
                    __nv_bfloat16* __restrict__ out, int s_len, int n, int np) {
    const int lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
    const long long rows = (long long)s_len * np;
    const float4 g4 = __ldg(reinterpret_cast<const float4*>(gamma) + sub), b4 = __ldg(reinterpret_cast<const float4*>(beta) + sub);
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const uint32_t members = 0xffffu << (half * 16);              // the 16 lanes that share this row
    for (long long r = warp0 * 2 + half; r < rows; r += nwarps * 2) {
        const int s = (int)(r / np), tok = (int)(r % np);
        const bool valid = tok < n;                                 // uniform over the row's lanes
        float4 v = valid ? __ldg(reinterpret_cast<const float4*>(m + ((long long)s * n + tok) * CM) + sub) : make_float4(0.f, 0.f, 0.f, 0.f);
        float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int k = 1; k < 16; k <<= 1) sum += __shfl_xor_sync(members, sum, k, 16);
        const float mean = sum * (1.f / CM);
        v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
        float ss = (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
#pragma unroll
        for (int k = 1; k < 16; k <<= 1) ss += __shfl_xor_sync(members, ss, k, 16);
        const float rstd = rsqrtf(ss * (1.f / CM) + LN_EPS);
        uint2 o = make_uint2(0u, 0u);
        if (valid) {
            o.x = pack_bf16x2(fmaf(v.x * rstd, g4.x, b4.x), fmaf(v.y * rstd, g4.y, b4.y));
            o.y = pack_bf16x2(fmaf(v.z * rstd, g4.z, b4.z), fmaf(v.w * rstd, g4.w, b4.w));
        }
        reinterpret_cast<uint2*>(out + r * CM)[sub] = o;
    }
}

// w[h][i][j] = softmax_j(logit[h][i][j] - inf * (1 - mask[i][j])) as bf16 rows of `pitch` elements (zero beyond n).
// One warp per (head, i).
__global__ void __launch_bounds__(256)
pwa_softmax_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ mask, __nv_bfloat16* __restrict__ w,
                   int n, int pitch, int heads, float inf_value) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (long long)heads * n) return;
    const int i = (int)(row % n);
    const float* src = logits + row * n;
    const uint8_t* mk = mask + (long long)i * n;
    __nv_bfloat16* dst = w + row * pitch;
    float mx = -INFINITY;
    for (int j = lane; j < n; j += 32) mx = fmaxf(mx, src[j] - (mk[j] ? 0.f : inf_value));
#pragma unroll
    for (int k = 16; k; k >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, k));
    float sum = 0.f;
    for (int j = lane; j < n; j += 32) sum += __expf(src[j] - (mk[j] ? 0.f : inf_value) - mx);
#pragma unroll
    for (int k = 16; k; k >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, k);
    const float inv = 1.f / sum;
    for (int j = lane; j < pitch; j += 32)
        dst[j] = __float2bfloat16(j < n ? __expf(src[j] - (mk[j] ? 0.f : inf_value) - mx) * inv : 0.f);
}

// val[(s, tok)][c] = o * sigmoid(g) for the 256 channels c = (head, d): the gated average turned K-major for the
// output projection's GEMM.  o and g are [8 heads][S][32][np] (token contiguous), which is how the GEMMs before
// leave them.  A CTA takes 64 tokens of one sequence.  Eight lanes read the 128 bytes of one channel (four channels
// per warp and step, every load a full line); the tile is transposed through shared memory, whose 16-byte chunks
// are XOR-swizzled with the token group so that neither side has bank conflicts, and leaves as full 512-byte rows.
constexpr int GT_POS = 64;
__global__ void __launch_bounds__(256)
pwa_gate_transpose_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ g,
                          __nv_bfloat16* __restrict__ val, int s_len, int np) {
    __shared__ __align__(16) __nv_bfloat16 tile[GT_POS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = lane & 7, csub = lane >> 3;
    const int s = blockIdx.y, t0 = blockIdx.x * GT_POS;
    const bool in_range = t0 + q * 8 < np;                                  // np is a multiple of 8
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int c = warp * 32 + it * 4 + csub, head = c >> 5, d = c & 31;
        if (!in_range) continue;
        const long long row = (((long long)head * s_len + s) * 32 + d) * np + t0;
        const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o + row) + q);
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(g + row) + q);
        const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
        const int cs = c ^ (q << 3);                                        // chunk (c >> 3) ^ token group
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            tile[q * 8 + 2 * k][cs] = __float2bfloat16(bf16_lo(ow[k]) / (1.f + __expf(-bf16_lo(gw[k]))));
            tile[q * 8 + 2 * k + 1][cs] = __float2bfloat16(bf16_hi(ow[k]) / (1.f + __expf(-bf16_hi(gw[k]))));
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GT_POS * 32; idx += 256) {          // 32 chunks of 8 channels per token row
        const int pl = idx >> 5, c8 = idx & 31;
        if (t0 + pl >= np) break;
        reinterpret_cast<uint4*>(val + ((long long)s * np + t0 + pl) * 256)[c8] =
            *reinterpret_cast<const uint4*>(&tile[pl][(c8 ^ (pl >> 3)) * 8]);
    }
}

// hsw[r][c] = silu(h[r][c]) * h[r][256 + c] for rows of 512 bf16 -> rows of 256 bf16; eight values per thread.
__global__ void __launch_bounds__(256)
swiglu_rows_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out, long long rows) {
    const long long total = rows * 32;                            // groups of 8 output values
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx >> 5;
        const int c8 = (int)(idx & 31);
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(h + r * 512) + c8);
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(h + r * 512 + 256) + c8);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a0 = bf16_lo(aw[k]), a1 = bf16_hi(aw[k]);
            ow[k] = pack_bf16x2(a0 / (1.f + __expf(-a0)) * bf16_lo(bw[k]), a1 / (1.f + __expf(-a1)) * bf16_hi(bw[k]));
        }
        reinterpret_cast<uint4*>(out + r * 256)[c8] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// m[s][i][:] += t[s * np + i][:] (bf16 rows of 64); four values per thread.
__global__ void __launch_bounds__(256)
add_rows_kernel(float* __restrict__ m, const __nv_bfloat16* __restrict__ t, int s_len, int n, int np) {
    const long long total = (long long)s_len * n * 16;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx >> 4;
        const int c4 = (int)(idx & 15);
        const int s = (int)(row / n), tok = (int)(row % n);
        const uint2 tv = __ldg(reinterpret_cast<const uint2*>(t + ((long long)s * np + tok) * CM) + c4);
        float4* mp = reinterpret_cast<float4*>(m + row * CM) + c4;
        float4 v = *mp;
        v.x += bf16_lo(tv.x); v.y += bf16_hi(tv.x); v.z += bf16_lo(tv.y); v.w += bf16_hi(tv.y);
        *mp = v;
    }
}

// m[s][i][:] += e[i][:] (fp32 rows of 64): the single representation's projection added to every sequence's embedding.
__global__ void __launch_bounds__(256)
add_token_rows_kernel(float* __restrict__ m, const float* __restrict__ e, int s_len, int n) {
    const long long per_seq = (long long)n * 16, total = per_seq * s_len;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const float4 ev = __ldg(reinterpret_cast<const float4*>(e) + idx % per_seq);
        float4* mp = reinterpret_cast<float4*>(m) + idx;
        float4 v = *mp;
        v.x += ev.x; v.y += ev.y; v.z += ev.z; v.w += ev.w;
        *mp = v;
    }
}

static unsigned grid_for(long long items, int per_block) {
    long long b = (items + per_block - 1) / per_block;
    const long long cap = 148LL * 32;
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace msa
}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_msa_ln_bf16(const float* m, const float* gamma, const float* beta, b200pf_bf16* out, int s_len, int n,
                                  int np, void* stream) {
    B200PF_REQUIRE(m && gamma && beta && out && aligned16(m) && aligned16(gamma) && aligned16(beta) && aligned16(out),
                   B200PF_ERR_INVALID, "msa_ln_bf16: null or misaligned pointer");
    B200PF_REQUIRE(s_len > 0 && n > 0 && np >= n && np % 8 == 0, B200PF_ERR_INVALID, "msa_ln_bf16: bad sizes");
    msa::ln_rows_bf16_kernel<<<msa::grid_for((long long)s_len * np, 16), 256, 0, (cudaStream_t)stream>>>(
        m, gamma, beta, (__nv_bfloat16*)out, s_len, n, np);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_pwa_softmax(const float* logits, const uint8_t* mask, b200pf_bf16* w, int n, int pitch, int heads,
                                  float inf_value, void* stream) {
    B200PF_REQUIRE(logits && mask && w && n > 0 && pitch >= n && heads > 0, B200PF_ERR_INVALID, "pwa_softmax: bad arguments");
    const long long rows = (long long)heads * n;
    msa::pwa_softmax_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(logits, mask, (__nv_bfloat16*)w, n, pitch,
                                                                                          heads, inf_value);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_pwa_gate_transpose(const b200pf_bf16* o, const b200pf_bf16* g, b200pf_bf16* val, int s_len, int np,
                                         void* stream) {
    using namespace msa;
    B200PF_REQUIRE(o && g && val && aligned16(o) && aligned16(g) && aligned16(val), B200PF_ERR_INVALID,
                   "pwa_gate_transpose: null or misaligned pointer");
    B200PF_REQUIRE(s_len > 0 && s_len <= 65535 && np > 0 && np % 8 == 0, B200PF_ERR_INVALID,
                   "pwa_gate_transpose: np must be a positive multiple of 8, at most 65535 sequences per call");
    dim3 grid((unsigned)((np + GT_POS - 1) / GT_POS), (unsigned)s_len);
    pwa_gate_transpose_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)g,
                                                                      (__nv_bfloat16*)val, s_len, np);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_msa_swiglu(const b200pf_bf16* h, b200pf_bf16* out, long long rows, void* stream) {
    B200PF_REQUIRE(h && out && aligned16(h) && aligned16(out) && rows > 0, B200PF_ERR_INVALID, "msa_swiglu: bad arguments");
    msa::swiglu_rows_kernel<<<msa::grid_for(rows * 32, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)h,
                                                                                              (__nv_bfloat16*)out, rows);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_msa_add_rows(float* m, const b200pf_bf16* t, int s_len, int n, int np, void* stream) {
    B200PF_REQUIRE(m && t && aligned16(m) && aligned16(t) && s_len > 0 && n > 0 && np >= n, B200PF_ERR_INVALID,
                   "msa_add_rows: bad arguments");
    msa::add_rows_kernel<<<msa::grid_for((long long)s_len * n * 16, 256), 256, 0, (cudaStream_t)stream>>>(
        m, (const __nv_bfloat16*)t, s_len, n, np);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_msa_add_token_rows(float* m, const float* e, int s_len, int n, void* stream) {
    B200PF_REQUIRE(m && e && aligned16(m) && aligned16(e) && s_len > 0 && n > 0, B200PF_ERR_INVALID, "msa_add_token_rows: bad arguments");
    msa::add_token_rows_kernel<<<msa::grid_for((long long)s_len * n * 16, 256), 256, 0, (cudaStream_t)stream>>>(m, e, s_len, n);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
