// fp32 validation tier: plain SIMT kernels, fp32 arithmetic end to end.
// These exist so that the 1e-4-per-layer tier can be met on the GPU (tensor cores have no
// fp32 mode) and they double as the single-track path, which the reference keeps in fp32
// (tt_bio/reference.py:906-912).  Speed is secondary here; clarity and exactness come first.
#include "common.cuh"

namespace b200pf {

// ------------------------------------------------------------------------------------------
// LayerNorm: one warp per row, two-pass mean / variance.
// ------------------------------------------------------------------------------------------
__global__ void f32_layernorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, float* __restrict__ y,
                                     long long rows, int c) {
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    const float* xr = x + row * c;
    float s = 0.f;
    for (int i = lane; i < c; i += 32) s += xr[i];
    float mean = warp_sum(s) / c;
    float v = 0.f;
    for (int i = lane; i < c; i += 32) { float d = xr[i] - mean; v += d * d; }
    float rstd = rsqrtf(warp_sum(v) / c + LN_EPS);
    float* yr = y + row * c;
    for (int i = lane; i < c; i += 32) yr[i] = (xr[i] - mean) * rstd * gamma[i] + beta[i];
}

// ------------------------------------------------------------------------------------------
// Linear: y[M][N] (+)= x[M][K] w[N][K]^T (+ bias).  64x64 tile, BK = 16, 4x4 per thread.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
f32_linear_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                  float* __restrict__ y, long long m, int k, int n, int accumulate) {
    __shared__ float xs[16][64 + 4];
    __shared__ float ws[16][64 + 4];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    long long m0 = (long long)blockIdx.x * 64;
    int n0 = blockIdx.y * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += 16) {
        // each thread loads 4 x-values and 4 w-values: element (row = t/4 .. , kk = (t%4)*4..)
        int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int kk = k0 + lk + e;
            long long r = m0 + lr;
            xs[lk + e][lr] = (r < m && kk < k) ? x[r * k + kk] : 0.f;
            int c = n0 + lr;
            ws[lk + e][lr] = (c < n && kk < k) ? w[(long long)c * k + kk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        long long r = m0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int c = n0 + tx * 4 + j;
            if (c >= n) continue;
            float v = acc[i][j] + (bias ? bias[c] : 0.f);
            long long idx = r * n + c;
            y[idx] = accumulate ? y[idx] + v : v;
        }
    }
}

// ------------------------------------------------------------------------------------------
// Element-wise gates.
// ------------------------------------------------------------------------------------------
__global__ void f32_gate_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                const uint8_t* __restrict__ row_mask, float* __restrict__ y,
                                long long total, int c, int mode) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        float av = a[i], bv = b[i];
        if (mode == 0) {
            float mk = row_mask ? (float)row_mask[i / c] : 1.f;
            y[i] = av * sigmoid_precise(bv) * mk;
        } else if (mode == 1) {
            y[i] = av * sigmoid_precise(av) * bv;
        } else {
            y[i] += av * sigmoid_precise(bv);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Triangle contraction, fp32: block = 8 x 8 (i, j) positions x all channels, thread = channel.
// Element (row, kk) of an operand sits at ptr[(row*s_row + kk*s_k) * pitch + c].
// ------------------------------------------------------------------------------------------
__global__ void f32_trimul_contract_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                           float* __restrict__ t, int n, int d, int pitch,
                                           long long s_row, long long s_k) {
    int c = blockIdx.z * blockDim.x + threadIdx.x;
    if (c >= d) return;
    int i0 = blockIdx.y * 8, j0 = blockIdx.x * 8;
    float acc[8][8] = {};
    for (int kk = 0; kk < n; ++kk) {
        float av[8], bv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            int i = min(i0 + u, n - 1), j = min(j0 + u, n - 1);
            av[u] = a[(i * s_row + kk * s_k) * pitch + c];
            bv[u] = b[(j * s_row + kk * s_k) * pitch + c];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int v = 0; v < 8; ++v) acc[u][v] = fmaf(av[u], bv[v], acc[u][v]);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int v = 0; v < 8; ++v)
            if (i0 + u < n && j0 + v < n) t[((long long)(i0 + u) * n + (j0 + v)) * d + c] = acc[u][v];
}

// ------------------------------------------------------------------------------------------
// Attention, fp32: one warp per (batch row r, head h, query q); logits staged in shared memory.
// ------------------------------------------------------------------------------------------
struct AttnArgs {
    const float *q, *k, *v, *bias;
    float* o;
    const uint8_t* mask;
    long long bias_hs, bias_qs, bias_ks, mask_rs, mask_ks, rs, ps;
    int batch, n_q, n_k, heads, hd, order;
    float scale, inf_value;
};

__global__ void f32_attention_kernel(AttnArgs p) {
    extern __shared__ float smem[];
    int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    float* logit = smem + (size_t)wid * p.n_k;
    long long total = (long long)p.batch * p.heads * p.n_q;
    for (long long w = (long long)blockIdx.x * nw + wid; w < total; w += (long long)gridDim.x * nw) {
        int qi = (int)(w % p.n_q);
        int h = (int)((w / p.n_q) % p.heads);
        long long r = w / ((long long)p.n_q * p.heads);
        const float* qp = p.q + r * p.rs + (long long)qi * p.ps + h * p.hd;
        float mx = -INFINITY;
        for (int kk = lane; kk < p.n_k; kk += 32) {
            const float* kp = p.k + r * p.rs + (long long)kk * p.ps + h * p.hd;
            float dot = 0.f;
            for (int e = 0; e < p.hd; ++e) dot = fmaf(qp[e] * p.scale, kp[e], dot);
            float mterm = 0.f;
            if (p.mask) mterm = -p.inf_value * (1.f - (float)p.mask[r * p.mask_rs + kk * p.mask_ks]);
            float bterm = p.bias ? p.bias[h * p.bias_hs + qi * p.bias_qs + kk * p.bias_ks] : 0.f;
            float l = p.order == 0 ? (dot + mterm) + bterm : (dot + bterm) + mterm;
            logit[kk] = l;
            mx = fmaxf(mx, l);
        }
        mx = warp_max(mx);
        float sum = 0.f;
        for (int kk = lane; kk < p.n_k; kk += 32) {
            float e = expf(logit[kk] - mx);
            logit[kk] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        __syncwarp();
        float inv = 1.f / sum;
        for (int e = lane; e < p.hd; e += 32) {
            float acc = 0.f;
            const float* vp = p.v + r * p.rs + h * p.hd + e;
            for (int kk = 0; kk < p.n_k; ++kk) acc = fmaf(logit[kk], vp[(long long)kk * p.ps], acc);
            p.o[r * p.rs + (long long)qi * p.ps + h * p.hd + e] = acc * inv;
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------
// dst[j][i][:] (+)= src[i][j][:]
// ------------------------------------------------------------------------------------------
__global__ void f32_transpose01_kernel(const float* __restrict__ src, float* __restrict__ dst, int n, int c,
                                       int accumulate) {
    long long pos = blockIdx.x;            // pos = i*n + j
    int i = (int)(pos / n), j = (int)(pos % n);
    const float* s = src + pos * c;
    float* d = dst + ((long long)j * n + i) * c;
    for (int e = threadIdx.x; e < c; e += blockDim.x) d[e] = accumulate ? d[e] + s[e] : s[e];
}

// ------------------------------------------------------------------------------------------
// LayerNorm + projection to a few heads; a warp walks 32 consecutive rows and keeps row l's
// results in lane l so that the stores are coalesced along the row index.
// ------------------------------------------------------------------------------------------
template <int HEADS>
__global__ void __launch_bounds__(256)
ln_proj_heads_kernel(const float* __restrict__ z, const float* __restrict__ gamma, const float* __restrict__ beta,
                     const float* __restrict__ w, float* __restrict__ out, long long out_hs, long long rows) {
    constexpr int C = 128;
    __shared__ float ws[HEADS][C];
    __shared__ float cs[HEADS];            // sum_c beta[c]*w[h][c]
    for (int i = threadIdx.x; i < HEADS * C; i += blockDim.x) ws[i / C][i % C] = w[i] * gamma[i % C];
    __syncthreads();
    if (threadIdx.x < HEADS) {
        float s = 0.f;
        for (int c = 0; c < C; ++c) s += w[threadIdx.x * C + c] * beta[c];
        cs[threadIdx.x] = s;
    }
    __syncthreads();
    int lane = threadIdx.x & 31;
    long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long base = warp * 32; base < rows; base += nwarps * 32) {
        float res[HEADS];
#pragma unroll
        for (int h = 0; h < HEADS; ++h) res[h] = 0.f;
        int cnt = (int)min((long long)32, rows - base);
        for (int rr = 0; rr < cnt; ++rr) {
            float4 xv = reinterpret_cast<const float4*>(z + (base + rr) * C)[lane];
            float mean = warp_sum(xv.x + xv.y + xv.z + xv.w) * (1.f / C);
            float d0 = xv.x - mean, d1 = xv.y - mean, d2 = xv.z - mean, d3 = xv.w - mean;
            float rstd = rsqrtf(warp_sum(d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3) * (1.f / C) + LN_EPS);
            d0 *= rstd; d1 *= rstd; d2 *= rstd; d3 *= rstd;
#pragma unroll
            for (int h = 0; h < HEADS; ++h) {
                const float* wr = &ws[h][lane * 4];
                float pth = d0 * wr[0] + d1 * wr[1] + d2 * wr[2] + d3 * wr[3];
                pth = warp_sum(pth) + cs[h];
                if (lane == rr) res[h] = pth;
            }
        }
        if (lane < cnt) {
#pragma unroll
            for (int h = 0; h < HEADS; ++h) out[h * out_hs + base + lane] = res[h];
        }
    }
}

}  // namespace b200pf

using namespace b200pf;

extern "C" {

int b200pf_f32_layernorm(const float* x, const float* gamma, const float* beta, float* y,
                         long long rows, int c, void* stream) {
    B200PF_REQUIRE(x && gamma && beta && y && rows >= 0 && c > 0, B200PF_ERR_INVALID, "f32_layernorm: bad argument");
    if (rows == 0) return B200PF_OK;
    unsigned blocks = (unsigned)((rows + 7) / 8);
    f32_layernorm_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, gamma, beta, y, rows, c);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_linear(const float* x, const float* w, const float* bias, float* y,
                      long long rows, int k, int n_out, int accumulate, void* stream) {
    B200PF_REQUIRE(x && w && y && rows >= 0 && k > 0 && n_out > 0, B200PF_ERR_INVALID, "f32_linear: bad argument");
    if (rows == 0) return B200PF_OK;
    dim3 grid((unsigned)((rows + 63) / 64), (unsigned)((n_out + 63) / 64));
    f32_linear_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, w, bias, y, rows, k, n_out, accumulate);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_gate(const float* a, const float* b, const uint8_t* row_mask, float* y,
                    long long rows, int c, int mode, void* stream) {
    B200PF_REQUIRE(a && b && y && rows >= 0 && c > 0 && mode >= 0 && mode <= 2, B200PF_ERR_INVALID,
                   "f32_gate: bad argument");
    long long total = rows * c;
    if (total == 0) return B200PF_OK;
    unsigned blocks = (unsigned)min((long long)148 * 16, (total + 255) / 256);
    f32_gate_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a, b, row_mask, y, total, c, mode);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_trimul_contract(const float* a, const float* b, float* t, int n, int d,
                               int in_pitch, int incoming, void* stream) {
    B200PF_REQUIRE(a && b && t && n > 0 && d > 0 && in_pitch >= d, B200PF_ERR_INVALID,
                   "f32_trimul_contract: bad argument");
    int threads = d < 128 ? d : 128;
    B200PF_REQUIRE(d % threads == 0, B200PF_ERR_UNSUPPORTED, "f32_trimul_contract: d must be <=128 or a multiple of 128");
    dim3 grid((n + 7) / 8, (n + 7) / 8, d / threads);
    long long s_row = incoming ? 1 : n, s_k = incoming ? n : 1;
    f32_trimul_contract_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(a, b, t, n, d, in_pitch, s_row, s_k);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_attention(const float* q, const float* k, const float* v, float* o,
                         const float* bias, long long bias_hs, long long bias_qs, long long bias_ks,
                         const uint8_t* mask, long long mask_rs, long long mask_ks,
                         int batch, int n_q, int n_k, int heads, int hd,
                         long long rs, long long ps, float scale, float inf_value, int order,
                         void* stream) {
    B200PF_REQUIRE(q && k && v && o && batch > 0 && n_q > 0 && n_k > 0 && heads > 0 && hd > 0,
                   B200PF_ERR_INVALID, "f32_attention: bad argument");
    AttnArgs p{q, k, v, bias, o, mask, bias_hs, bias_qs, bias_ks, mask_rs, mask_ks, rs, ps,
               batch, n_q, n_k, heads, hd, order, scale, inf_value};
    int warps = 8;
    size_t smem = (size_t)warps * n_k * sizeof(float);
    B200PF_REQUIRE(smem <= 200 * 1024, B200PF_ERR_UNSUPPORTED, "f32_attention: n_k too large (%d)", n_k);
    if (smem > 48 * 1024)
        B200PF_CUDA(cudaFuncSetAttribute(f32_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    long long total = (long long)batch * heads * n_q;
    unsigned blocks = (unsigned)min((long long)148 * 8, (total + warps - 1) / warps);
    f32_attention_kernel<<<blocks, warps * 32, smem, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_transpose01(const float* src, float* dst, int n, int c, int accumulate, void* stream) {
    B200PF_REQUIRE(src && dst && n > 0 && c > 0 && src != dst, B200PF_ERR_INVALID, "f32_transpose01: bad argument");
    f32_transpose01_kernel<<<(unsigned)((long long)n * n), c < 128 ? 32 : 128, 0, (cudaStream_t)stream>>>(src, dst, n, c, accumulate);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_ln_proj_heads(const float* z, const float* gamma, const float* beta, const float* w,
                         float* out, long long out_hs, long long rows, int c, int heads, void* stream) {
    B200PF_REQUIRE(z && gamma && beta && w && out && rows >= 0, B200PF_ERR_INVALID, "ln_proj_heads: bad argument");
    B200PF_REQUIRE(c == 128 && (heads == 4 || heads == 16), B200PF_ERR_UNSUPPORTED,
                   "ln_proj_heads: built for c = 128 and 4 or 16 heads (got c=%d heads=%d)", c, heads);
    B200PF_REQUIRE(aligned16(z), B200PF_ERR_INVALID, "ln_proj_heads: z must be 16-byte aligned");
    if (rows == 0) return B200PF_OK;
    unsigned blocks = (unsigned)min((long long)148 * 4, (rows + 255) / 256);
    if (heads == 4)
        ln_proj_heads_kernel<4><<<blocks, 256, 0, (cudaStream_t)stream>>>(z, gamma, beta, w, out, out_hs, rows);
    else
        ln_proj_heads_kernel<16><<<blocks, 256, 0, (cudaStream_t)stream>>>(z, gamma, beta, w, out, out_hs, rows);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

}  // extern "C"
