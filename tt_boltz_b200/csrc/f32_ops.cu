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
                  float* __restrict__ y, long long m, int k, int n, int accumulate, long long yt_pitch) {
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
            long long idx = yt_pitch > 0 ? (long long)c * yt_pitch + r : r * n + c;      // transposed: y^T[c][r]
            y[idx] = accumulate ? y[idx] + v : v;
        }
    }
}

// ------------------------------------------------------------------------------------------
// Element-wise gates.
// ------------------------------------------------------------------------------------------
__global__ void f32_gate_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                const uint8_t* __restrict__ row_mask, float* __restrict__ y,
                                long long total, int c, int mode, long long pa, long long pb, long long py) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long r = i / c;
        int col = (int)(i - r * c);
        float av = a[r * pa + col], bv = b[r * pb + col];
        float* yp = y + r * py + col;
        if (mode == 0) {
            float mk = row_mask ? (float)row_mask[r] : 1.f;
            *yp = av * sigmoid_precise(bv) * mk;
        } else if (mode == 1) {
            *yp = av * sigmoid_precise(av) * bv;
        } else {
            *yp += av * sigmoid_precise(bv);
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

template <int HD>
__global__ void f32_attention_kernel(AttnArgs p) {
    // One warp per (batch row r, head h, query q).  Lanes split the keys in all three passes:
    // logits -> shared memory, exponentials, then each lane accumulates its keys' share of the
    // output vector in registers and the warp reduces the HD partial sums with shuffles.
    extern __shared__ float smem[];
    int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    float* logit = smem + (size_t)wid * p.n_k;
    long long total = (long long)p.batch * p.heads * p.n_q;
    for (long long w = (long long)blockIdx.x * nw + wid; w < total; w += (long long)gridDim.x * nw) {
        int qi = (int)(w % p.n_q);
        int h = (int)((w / p.n_q) % p.heads);
        long long r = w / ((long long)p.n_q * p.heads);
        const float* qp = p.q + r * p.rs + (long long)qi * p.ps + h * HD;
        float qv[HD];
#pragma unroll
        for (int e = 0; e < HD; ++e) qv[e] = qp[e] * p.scale;
        float mx = -INFINITY;
        for (int kk = lane; kk < p.n_k; kk += 32) {
            const float4* kp = reinterpret_cast<const float4*>(p.k + r * p.rs + (long long)kk * p.ps + h * HD);
            float dot = 0.f;
#pragma unroll
            for (int e4 = 0; e4 < HD / 4; ++e4) {
                float4 kv = kp[e4];
                dot = fmaf(qv[e4 * 4], kv.x, dot);
                dot = fmaf(qv[e4 * 4 + 1], kv.y, dot);
                dot = fmaf(qv[e4 * 4 + 2], kv.z, dot);
                dot = fmaf(qv[e4 * 4 + 3], kv.w, dot);
            }
            float mterm = 0.f;
            if (p.mask) mterm = -p.inf_value * (1.f - (float)p.mask[r * p.mask_rs + kk * p.mask_ks]);
            float bterm = p.bias ? p.bias[h * p.bias_hs + qi * p.bias_qs + kk * p.bias_ks] : 0.f;
            float l = p.order == 0 ? (dot + mterm) + bterm : (dot + bterm) + mterm;
            logit[kk] = l;
            mx = fmaxf(mx, l);
        }
        mx = warp_max(mx);
        float sum = 0.f;
        float acc[HD];
#pragma unroll
        for (int e = 0; e < HD; ++e) acc[e] = 0.f;
        for (int kk = lane; kk < p.n_k; kk += 32) {
            float pe = expf(logit[kk] - mx);
            sum += pe;
            const float4* vp = reinterpret_cast<const float4*>(p.v + r * p.rs + (long long)kk * p.ps + h * HD);
#pragma unroll
            for (int e4 = 0; e4 < HD / 4; ++e4) {
                float4 vv = vp[e4];
                acc[e4 * 4] = fmaf(pe, vv.x, acc[e4 * 4]);
                acc[e4 * 4 + 1] = fmaf(pe, vv.y, acc[e4 * 4 + 1]);
                acc[e4 * 4 + 2] = fmaf(pe, vv.z, acc[e4 * 4 + 2]);
                acc[e4 * 4 + 3] = fmaf(pe, vv.w, acc[e4 * 4 + 3]);
            }
        }
        float inv = 1.f / warp_sum(sum);
        float mine = 0.f;
#pragma unroll
        for (int e = 0; e < HD; ++e) {
            float tot = warp_sum(acc[e]);
            if (lane == e) mine = tot;
        }
        if (lane < HD) p.o[r * p.rs + (long long)qi * p.ps + h * HD + lane] = mine * inv;
    }
}

// ------------------------------------------------------------------------------------------
// Single-track attention, fp32, with K and V given transposed ([head*HD + e][key], keys contiguous):
// a block owns one head and 32 queries (8 warps x 4 queries), lanes split the keys, so every
// K / V load is one coalesced line shared by four queries.  Two passes over the keys: row
// maxima first, then exponentials, the P V partial sums and the row sums; the gate
// sigmoid(g) is applied before the store.
// ------------------------------------------------------------------------------------------
struct SAttnArgs {
    const float *q, *g, *kt, *vt, *bias;
    float* o;
    const uint8_t* mask;
    long long q_pitch, g_pitch, o_pitch, kt_pitch, bias_hs, bias_qs;
    int n_q, n_k, heads;
    float scale, inf_value;
};

template <int HD>
__global__ void __launch_bounds__(256) f32_sattention_kernel(SAttnArgs p) {
    constexpr int QB = 4;
    __shared__ float qs[8][HD][QB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qblocks = (p.n_q + 31) / 32;
    const int h = blockIdx.x / qblocks, q0 = (blockIdx.x % qblocks) * 32 + warp * QB;
    if (q0 >= p.n_q) return;
    for (int i = lane; i < HD * QB; i += 32) {
        int e = i / QB, qb = i % QB;
        int qi = min(q0 + qb, p.n_q - 1);
        qs[warp][e][qb] = p.q[(long long)qi * p.q_pitch + h * HD + e] * p.scale;
    }
    __syncwarp();
    const float* kt = p.kt + (long long)h * HD * p.kt_pitch;
    const float* vt = p.vt + (long long)h * HD * p.kt_pitch;
    auto logits = [&](int kk, float (&l)[QB]) {
#pragma unroll
        for (int qb = 0; qb < QB; ++qb) l[qb] = 0.f;
#pragma unroll
        for (int e = 0; e < HD; ++e) {
            const float kv = kt[(long long)e * p.kt_pitch + kk];
            const float4 qv = *reinterpret_cast<const float4*>(&qs[warp][e][0]);
            l[0] = fmaf(qv.x, kv, l[0]); l[1] = fmaf(qv.y, kv, l[1]); l[2] = fmaf(qv.z, kv, l[2]); l[3] = fmaf(qv.w, kv, l[3]);
        }
        const float mterm = p.mask ? -p.inf_value * (1.f - (float)p.mask[kk]) : 0.f;
#pragma unroll
        for (int qb = 0; qb < QB; ++qb) {
            int qi = min(q0 + qb, p.n_q - 1);
            l[qb] = (l[qb] + p.bias[h * p.bias_hs + qi * p.bias_qs + kk]) + mterm;
        }
    };
    float mx[QB];
#pragma unroll
    for (int qb = 0; qb < QB; ++qb) mx[qb] = -INFINITY;
    for (int kk = lane; kk < p.n_k; kk += 32) {
        float l[QB];
        logits(kk, l);
#pragma unroll
        for (int qb = 0; qb < QB; ++qb) mx[qb] = fmaxf(mx[qb], l[qb]);
    }
#pragma unroll
    for (int qb = 0; qb < QB; ++qb) mx[qb] = warp_max(mx[qb]);
    float sum[QB], acc[QB][HD];
#pragma unroll
    for (int qb = 0; qb < QB; ++qb) {
        sum[qb] = 0.f;
#pragma unroll
        for (int e = 0; e < HD; ++e) acc[qb][e] = 0.f;
    }
    for (int kk = lane; kk < p.n_k; kk += 32) {
        float l[QB];
        logits(kk, l);
#pragma unroll
        for (int qb = 0; qb < QB; ++qb) { l[qb] = expf(l[qb] - mx[qb]); sum[qb] += l[qb]; }
#pragma unroll
        for (int e = 0; e < HD; ++e) {
            const float vv = vt[(long long)e * p.kt_pitch + kk];
#pragma unroll
            for (int qb = 0; qb < QB; ++qb) acc[qb][e] = fmaf(l[qb], vv, acc[qb][e]);
        }
    }
#pragma unroll
    for (int qb = 0; qb < QB; ++qb) {
        const float inv = 1.f / warp_sum(sum[qb]);
        float mine = 0.f;
#pragma unroll
        for (int e = 0; e < HD; ++e) {
            float tot = warp_sum(acc[qb][e]);
            if (lane == e) mine = tot;
        }
        const int qi = q0 + qb;
        if (qi < p.n_q && lane < HD) {
            float gate = p.g ? sigmoid_precise(p.g[(long long)qi * p.g_pitch + h * HD + lane]) : 1.f;
            p.o[(long long)qi * p.o_pitch + h * HD + lane] = mine * inv * gate;
        }
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
    // 8 lanes per row (16 channels each), 4 rows per pass, 32 rows per warp unit.  Head sums are
    // reduced over the 8 lanes with a halving butterfly (HEADS -> HEADS/8 values per lane), staged
    // in shared memory as [head][row] and written as 128-byte runs along the row index.
    constexpr int C = 128;
    constexpr int PER = HEADS >= 8 ? HEADS / 8 : 1;      // heads a lane ends up owning
    __shared__ float ws[HEADS][C + 4];
    __shared__ float cs[HEADS];
    __shared__ float stage[8][HEADS][32 + 1];
    for (int i = threadIdx.x; i < HEADS * C; i += blockDim.x) ws[i / C][i % C] = w[i] * gamma[i % C];
    if (threadIdx.x < HEADS) {
        float sacc = 0.f;
        for (int c = 0; c < C; ++c) sacc += w[threadIdx.x * C + c] * beta[c];
        cs[threadIdx.x] = sacc;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, sub = lane & 7, rq = lane >> 3;
    long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + wid;
    long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long base = warp * 32; base < rows; base += nwarps * 32) {
#pragma unroll 2
        for (int it = 0; it < 8; ++it) {
            long long row = base + it * 4 + rq;
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                v[j] = row < rows ? __ldg(reinterpret_cast<const float4*>(z + row * C) + j * 8 + sub) : make_float4(0.f, 0.f, 0.f, 0.f);
            float sm = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) sm += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            sm += __shfl_xor_sync(0xffffffffu, sm, 1);
            sm += __shfl_xor_sync(0xffffffffu, sm, 2);
            sm += __shfl_xor_sync(0xffffffffu, sm, 4);
            float mean = sm * (1.f / C), ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
                ss += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
            }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            float rstd = rsqrtf(ss * (1.f / C) + LN_EPS);
            float part[HEADS];
#pragma unroll
            for (int h = 0; h < HEADS; ++h) {
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float* wr = &ws[h][(j * 8 + sub) * 4];
                    a += v[j].x * wr[0] + v[j].y * wr[1] + v[j].z * wr[2] + v[j].w * wr[3];
                }
                part[h] = a * rstd;
            }
            if (HEADS >= 8) {
                // butterfly over lane bits 2, 1, 0: keep the half of the heads selected by the lane bit
#pragma unroll
                for (int step = 0; step < 3; ++step) {
                    const int bit = 4 >> step, half = HEADS >> (step + 1);
                    const bool upper = (sub & bit) != 0;
#pragma unroll
                    for (int h = 0; h < half; ++h) {
                        float keep = upper ? part[h + half] : part[h];
                        float send = upper ? part[h] : part[h + half];
                        part[h] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                    }
                }
                // lane `sub` now owns heads: bits of sub select halves: head index = sub_bits-weighted
                int hbase = ((sub >> 2) & 1) * (HEADS / 2) + ((sub >> 1) & 1) * (HEADS / 4) + (sub & 1) * (HEADS / 8);
#pragma unroll
                for (int h = 0; h < PER; ++h) stage[wid][hbase + h][it * 4 + rq] = part[h] + cs[hbase + h];
            } else {
#pragma unroll
                for (int h = 0; h < HEADS; ++h) {
                    float tsum = part[h];
                    tsum += __shfl_xor_sync(0xffffffffu, tsum, 1);
                    tsum += __shfl_xor_sync(0xffffffffu, tsum, 2);
                    tsum += __shfl_xor_sync(0xffffffffu, tsum, 4);
                    if (sub == h) stage[wid][h][it * 4 + rq] = tsum + cs[h];
                }
            }
        }
        __syncwarp();
        for (int h = 0; h < HEADS; ++h)
            if (base + lane < rows) out[h * out_hs + base + lane] = stage[wid][h][lane];
        __syncwarp();
    }
}

// The same for 16 heads on the tensor cores, still at fp32 accuracy: mma.sync m16n8k8 with the
// 3xTF32 split (x = hi + lo in tf32; hi*hi + lo*hi + hi*lo, fp32 accumulation: error ~2^-19 per
// product).  A warp takes 16 rows per step: lane (g, t) = (lane / 4, lane % 4) holds channels
// 16 j + 4 t .. + 3 (j = 0 .. 7) of rows g and g + 8, so the four lanes of a row read 64 contiguous bytes
// per load instruction.  K step ks uses the lane's values 2 ks and 2 ks + 1, i.e. channels
// 16 (ks / 2) + 4 t + 2 (ks % 2) (+1): the k <-> channel map the weights are laid out with in shared memory.
// Round to tf32 (nearest, ties away from zero: what cvt.rna.tf32.f32 returns for every finite value that does not
// overflow) with two integer instructions on the bit pattern.  The cvt instruction itself runs at a few lanes per
// clock: with two of them per operand element the 3xTF32 kernels below were bound by the conversions, at a
// quarter of the rate of the MMAs they feed.
__device__ __forceinline__ uint32_t to_tf32(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256)
ln_proj_heads16_mma_kernel(const float* __restrict__ z, const float* __restrict__ gamma, const float* __restrict__ beta,
                           const float* __restrict__ w, float* __restrict__ out, long long out_hs, long long rows) {
    constexpr int C = 128, HEADS = 16;
    __shared__ uint2 w_hi[16][2][32], w_lo[16][2][32];       // [k step][n tile][lane] -> (b0, b1)
    __shared__ float cs[HEADS];
    for (int i = threadIdx.x; i < 16 * 2 * 32; i += blockDim.x) {
        const int ln = i & 31, nt = (i >> 5) & 1, ks = i >> 6;
        const int g = ln >> 2, t = ln & 3, h = nt * 8 + g, c0 = 16 * (ks >> 1) + 4 * t + 2 * (ks & 1);
        const float v0 = w[h * C + c0] * gamma[c0], v1 = w[h * C + c0 + 1] * gamma[c0 + 1];
        const uint32_t h0 = to_tf32(v0), h1 = to_tf32(v1);
        w_hi[ks][nt][ln] = make_uint2(h0, h1);
        w_lo[ks][nt][ln] = make_uint2(to_tf32(v0 - __uint_as_float(h0)), to_tf32(v1 - __uint_as_float(h1)));
    }
    {   // LayerNorm offset carried through the weights, cs[h] = sum_c w[h][c] beta[c]: 16 threads per head (one
        // thread per head walked 128 dependent steps while the rest of the CTA waited at the barrier)
        const int h = threadIdx.x >> 4, sub = threadIdx.x & 15;
        float sacc = 0.f;
#pragma unroll
        for (int j = 0; j < C / 16; ++j) sacc += w[h * C + sub + 16 * j] * beta[sub + 16 * j];
#pragma unroll
        for (int st = 1; st < 16; st <<= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, st);
        if (sub == 0) cs[h] = sacc;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long base = warp * 16; base < rows; base += nwarps * 16) {
        float x[2][32];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const long long row = base + g + 8 * r;
            const float4* src = reinterpret_cast<const float4*>(z + (row < rows ? row : 0) * C) + t;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 v = row < rows ? __ldg(src + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
                x[r][4 * q] = v.x; x[r][4 * q + 1] = v.y; x[r][4 * q + 2] = v.z; x[r][4 * q + 3] = v.w;
            }
        }
        float sm[2], ss[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float a = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e) a += x[r][e];
            sm[r] = a;
        }
#pragma unroll
        for (int st = 1; st < 4; st <<= 1)
#pragma unroll
            for (int r = 0; r < 2; ++r) sm[r] += __shfl_xor_sync(0xffffffffu, sm[r], st);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float mean = sm[r] * (1.f / C);
            float a = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e) { x[r][e] -= mean; a = fmaf(x[r][e], x[r][e], a); }
            ss[r] = a;
        }
#pragma unroll
        for (int st = 1; st < 4; st <<= 1)
#pragma unroll
            for (int r = 0; r < 2; ++r) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], st);
        const float rstd0 = rsqrtf(ss[0] * (1.f / C) + LN_EPS), rstd1 = rsqrtf(ss[1] * (1.f / C) + LN_EPS);
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
            const float v0 = x[0][2 * ks] * rstd0, v1 = x[1][2 * ks] * rstd1, v2 = x[0][2 * ks + 1] * rstd0, v3 = x[1][2 * ks + 1] * rstd1;
            const uint32_t a0 = to_tf32(v0), a1 = to_tf32(v1), a2 = to_tf32(v2), a3 = to_tf32(v3);
            const uint32_t l0 = to_tf32(v0 - __uint_as_float(a0)), l1 = to_tf32(v1 - __uint_as_float(a1));
            const uint32_t l2 = to_tf32(v2 - __uint_as_float(a2)), l3 = to_tf32(v3 - __uint_as_float(a3));
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const uint2 bh = w_hi[ks][nt][lane], bl = w_lo[ks][nt][lane];
                mma_tf32(acc[nt], l0, l1, l2, l3, bh.x, bh.y);
                mma_tf32(acc[nt], a0, a1, a2, a3, bl.x, bl.y);
                mma_tf32(acc[nt], a0, a1, a2, a3, bh.x, bh.y);
            }
        }
        // c0: (row g, head 2t), c1: (row g, head 2t + 1), c2 / c3: the same for row g + 8
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const long long row = base + g + 8 * (e >> 1);
                const int h = nt * 8 + 2 * t + (e & 1);
                if (row < rows) out[h * out_hs + row] = acc[nt][e] + cs[h];
            }
    }
}

// ------------------------------------------------------------------------------------------
// The single track's attention on the tensor cores at fp32 accuracy (3xTF32, see above).  One CTA = one head x 64
// queries, 4 warps of 16 queries; keys walked in tiles of 64 with K^T, V^T, the 64 bias rows and the mask terms of a
// tile staged in shared memory (cp.async, two stages).  Per tile and warp: S = Q K^T as m16n8k8 products (Q
// pre-scaled and split once), + bias + mask term in the accumulator layout, one-pass softmax with a running row
// maximum (rows g and g + 8 of a thread, reduced over the four lanes of a quad), then O += P V with P taken straight
// from the accumulators: an accumulator holds columns 2t, 2t + 1 of an 8-key block where the A operand wants k slots
// t, t + 4, so slot t stands for key 2t and slot t + 4 for key 2t + 1, and the V fragment is read in that order (a
// sum over keys does not care).  Row pitch 72 floats: every fragment read is bank-conflict free.
// Needs 16-byte aligned kt / vt / bias and pitches that are multiples of 4 floats.
// ------------------------------------------------------------------------------------------
namespace satc {
constexpr int KT = 64, QT = 64, LD = KT + 8, STAGES = 2;
template <int HD> __host__ __device__ constexpr int stage_floats() { return (2 * HD + QT) * LD + KT; }
template <int HD> __host__ __device__ constexpr int smem_bytes() { return STAGES * stage_floats<HD>() * 4; }

__device__ __forceinline__ void cp_async16(float* dst, const float* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
    hi = to_tf32(v);
    lo = to_tf32(v - __uint_as_float(hi));
}
}  // namespace satc

template <int HD>
__global__ void __launch_bounds__(128) f32_sattention_mma_kernel(SAttnArgs p) {
    using namespace satc;
    static_assert(HD % 8 == 0, "head dim in k steps of 8");
    constexpr int KS = HD / 8, NB = KT / 8;
    extern __shared__ __align__(16) float satc_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int qblocks = (p.n_q + QT - 1) / QT;
    const int h = blockIdx.x / qblocks, q0 = (blockIdx.x % qblocks) * QT, qw = q0 + warp * 16;
    const bool active = qw < p.n_q;                                     // idle warps still help to load
    const float* kt = p.kt + (long long)h * HD * p.kt_pitch;
    const float* vt = p.vt + (long long)h * HD * p.kt_pitch;
    const int ntiles = (p.n_k + KT - 1) / KT;
    const int qr0 = min(qw + g, p.n_q - 1), qr1 = min(qw + g + 8, p.n_q - 1);

    auto load_tile = [&](int tile) {
        float* st = satc_smem + (tile & 1) * stage_floats<HD>();
        const int k0 = tile * KT;
        constexpr int CH = KT / 4;                                      // 16-byte chunks per row
        for (int i = tid; i < HD * CH; i += 128) {
            const int e = i / CH, c4 = (i % CH) * 4, kk = k0 + c4;
            const int bytes = max(0, min(16, (p.n_k - kk) * 4));
            const long long off = (long long)e * p.kt_pitch + (bytes ? kk : 0);
            cp_async16(st + e * LD + c4, kt + off, bytes);
            cp_async16(st + (HD + e) * LD + c4, vt + off, bytes);
        }
        for (int i = tid; i < QT * CH; i += 128) {
            const int r = i / CH, c4 = (i % CH) * 4, kk = k0 + c4;
            const int qi = min(q0 + r, p.n_q - 1);
            const int bytes = max(0, min(16, (p.n_k - kk) * 4));
            cp_async16(st + (2 * HD + r) * LD + c4, p.bias + h * p.bias_hs + qi * p.bias_qs + (bytes ? kk : 0), bytes);
        }
        if (tid < KT) {                                                 // keys past the end never count
            const int kk = k0 + tid;
            st[(2 * HD + QT) * LD + tid] = kk < p.n_k ? (p.mask ? -p.inf_value * (1.f - (float)p.mask[kk]) : 0.f) : -INFINITY;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // this warp's queries as A fragments, scaled, split once
    uint32_t qh[KS][4], ql[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const float* r0 = p.q + (long long)qr0 * p.q_pitch + h * HD + 8 * ks;
        const float* r1 = p.q + (long long)qr1 * p.q_pitch + h * HD + 8 * ks;
        split_tf32(r0[t] * p.scale, qh[ks][0], ql[ks][0]);
        split_tf32(r1[t] * p.scale, qh[ks][1], ql[ks][1]);
        split_tf32(r0[t + 4] * p.scale, qh[ks][2], ql[ks][2]);
        split_tf32(r1[t + 4] * p.scale, qh[ks][3], ql[ks][3]);
    }
    float o[KS][4];
#pragma unroll
    for (int ei = 0; ei < KS; ++ei) { o[ei][0] = o[ei][1] = o[ei][2] = o[ei][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    load_tile(0);
#pragma unroll 1
    for (int tile = 0; tile < ntiles; ++tile) {
        if (tile + 1 < ntiles) {
            load_tile(tile + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* st = satc_smem + (tile & 1) * stage_floats<HD>();
        if (active) {
            float s[NB][4];
#pragma unroll
            for (int ni = 0; ni < NB; ++ni) { s[ni][0] = s[ni][1] = s[ni][2] = s[ni][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int ni = 0; ni < NB; ++ni) {
                    uint32_t bh0, bl0, bh1, bl1;                        // B[k = e][n = key]: K^T[e][key]
                    split_tf32(st[(8 * ks + t) * LD + 8 * ni + g], bh0, bl0);
                    split_tf32(st[(8 * ks + t + 4) * LD + 8 * ni + g], bh1, bl1);
                    mma_tf32(s[ni], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], bh0, bh1);
                    mma_tf32(s[ni], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], bl0, bl1);
                    mma_tf32(s[ni], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], bh0, bh1);
                }
            }
            // + bias + mask term (in that order), row maxima
            const float* brow0 = st + (2 * HD + warp * 16 + g) * LD + 2 * t;
            const float* brow1 = brow0 + 8 * LD;
            const float* mrow = st + (2 * HD + QT) * LD + 2 * t;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int ni = 0; ni < NB; ++ni) {
                const float2 b0 = *reinterpret_cast<const float2*>(brow0 + 8 * ni);
                const float2 b1 = *reinterpret_cast<const float2*>(brow1 + 8 * ni);
                const float2 mt = *reinterpret_cast<const float2*>(mrow + 8 * ni);
                s[ni][0] = (s[ni][0] + b0.x) + mt.x; s[ni][1] = (s[ni][1] + b0.y) + mt.y;
                s[ni][2] = (s[ni][2] + b1.x) + mt.x; s[ni][3] = (s[ni][3] + b1.y) + mt.y;
                mx0 = fmaxf(mx0, fmaxf(s[ni][0], s[ni][1]));
                mx1 = fmaxf(mx1, fmaxf(s[ni][2], s[ni][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // every tile holds at least one key inside n_k, whose logit is finite: the new maxima are finite
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
            const float a0 = expf(m0 - n0), a1 = expf(m1 - n1);        // 0 on the first tile
            m0 = n0; m1 = n1;
            l0 *= a0; l1 *= a1;
#pragma unroll
            for (int ei = 0; ei < KS; ++ei) { o[ei][0] *= a0; o[ei][1] *= a0; o[ei][2] *= a1; o[ei][3] *= a1; }
#pragma unroll
            for (int ni = 0; ni < NB; ++ni) {
                // ex2.approx of the scaled difference: relative error ~1e-6 for the differences that still count
                const float p0 = __expf(s[ni][0] - n0), p1 = __expf(s[ni][1] - n0);
                const float p2 = __expf(s[ni][2] - n1), p3 = __expf(s[ni][3] - n1);
                l0 += p0 + p1; l1 += p2 + p3;
                // A fragment of P: a0 (row g, slot t) = key 2t, a1 (row g + 8, slot t), a2 / a3 (slot t + 4) = key 2t + 1
                uint32_t ph[4], pl[4];
                split_tf32(p0, ph[0], pl[0]); split_tf32(p2, ph[1], pl[1]);
                split_tf32(p1, ph[2], pl[2]); split_tf32(p3, ph[3], pl[3]);
#pragma unroll
                for (int ei = 0; ei < KS; ++ei) {
                    // B[k slot][n = e]: V^T[e = 8 ei + g][keys 8 ni + 2t, 8 ni + 2t + 1]
                    const float2 v = *reinterpret_cast<const float2*>(st + (HD + 8 * ei + g) * LD + 8 * ni + 2 * t);
                    uint32_t vh0, vl0, vh1, vl1;
                    split_tf32(v.x, vh0, vl0); split_tf32(v.y, vh1, vl1);
                    mma_tf32(o[ei], pl[0], pl[1], pl[2], pl[3], vh0, vh1);
                    mma_tf32(o[ei], ph[0], ph[1], ph[2], ph[3], vl0, vl1);
                    mma_tf32(o[ei], ph[0], ph[1], ph[2], ph[3], vh0, vh1);
                }
            }
        }
        __syncthreads();                                                // the stage is refilled two tiles later
    }
    if (!active) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int ei = 0; ei < KS; ++ei) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int qi = qw + g + 8 * (c >> 1), e = 8 * ei + 2 * t + (c & 1);
            if (qi >= p.n_q) continue;
            const float gate = p.g ? sigmoid_precise(p.g[(long long)qi * p.g_pitch + h * HD + e]) : 1.f;
            p.o[(long long)qi * p.o_pitch + h * HD + e] = o[ei][c] * ((c >> 1) ? inv1 : inv0) * gate;
        }
    }
}

// Linear on the tensor cores at fp32 accuracy (3xTF32, see above): y[M][N] (+)= x[M][K] w[N][K]^T (+ bias), or the
// transposed result y^T[N][yt_pitch].  64 x 64 tile per CTA of KQ warp quartets: four warps cover the tile (32 x 32
// each) and the quartets split every 64-wide K step between them (8 / KQ k steps of 8 each); their partial sums meet in
// shared memory at the end, in a fixed order.  With one quartet per CTA the single track's launches (72 to 192 CTAs)
// ran about one warp per scheduler and were bound by instruction latency.  The launches use KQ = 2 (256 threads, two
// CTAs per SM): a CTA of four quartets holds an SM's whole register file, which on a side stream leaves it waiting
// for an empty SM.  The next K step's global loads are in flight while the current one is multiplied.
// Needs K % 4 == 0 and 16-byte rows.
template <int KQ>
__global__ void __launch_bounds__(128 * KQ, KQ == 4 ? 1 : 2)
f32_linear_mma_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                      float* __restrict__ y, long long m, int k, int n, int accumulate, long long yt_pitch) {
    static_assert(KQ == 2 || KQ == 4, "two or four warp quartets");
    constexpr int BM = 64, BN = 64, BK = 64, LD = BK + 4, RL = 8 * KQ, LE = 64 / RL, KS = 8 / KQ;
    __shared__ __align__(16) float lin_smem[(BM + BN) * LD];            // x tile | w tile; the partial sums afterwards
    static_assert((BM + BN) * LD >= 8 * 32 * 32, "the tile buffer also holds eight warps' partial sums");
    float (*xs)[LD] = reinterpret_cast<float (*)[LD]>(lin_smem);
    float (*ws)[LD] = reinterpret_cast<float (*)[LD]>(lin_smem + BM * LD);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int kq = warp >> 2, wq = warp & 3;                    // K quarter of every step; position in the tile
    const int wm = (wq >> 1) * 32, wn = (wq & 1) * 32;
    const long long m0 = (long long)blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    const int lr = tid >> 4, lk = (tid & 15) * 4;               // this thread's load slot: rows lr + RL e, k offset lk
    float4 px[LE], pw[LE];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int e = 0; e < LE; ++e) {
            const long long r = m0 + lr + RL * e;
            const int c = n0 + lr + RL * e;
            const bool kin = k0 + lk < k;
            px[e] = (r < m && kin) ? __ldg(reinterpret_cast<const float4*>(x + r * k + k0 + lk)) : make_float4(0.f, 0.f, 0.f, 0.f);
            pw[e] = (c < n && kin) ? __ldg(reinterpret_cast<const float4*>(w + (long long)c * k + k0 + lk)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    float acc[2][4][4] = {};
    fetch(0);
    for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
        for (int e = 0; e < LE; ++e) {
            *reinterpret_cast<float4*>(&xs[lr + RL * e][lk]) = px[e];
            *reinterpret_cast<float4*>(&ws[lr + RL * e][lk]) = pw[e];
        }
        __syncthreads();
        if (k0 + BK < k) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            const int k8 = (kq * KS + kk) * 8;
            uint32_t ah[2][4], al[2][4], bh[4][2], bl[4][2];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                const float v[4] = {xs[wm + 16 * mi + g][k8 + t], xs[wm + 16 * mi + g + 8][k8 + t],
                                    xs[wm + 16 * mi + g][k8 + t + 4], xs[wm + 16 * mi + g + 8][k8 + t + 4]};
#pragma unroll
                for (int q = 0; q < 4; ++q) { ah[mi][q] = to_tf32(v[q]); al[mi][q] = to_tf32(v[q] - __uint_as_float(ah[mi][q])); }
            }
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                const float v[2] = {ws[wn + 8 * ni + g][k8 + t], ws[wn + 8 * ni + g][k8 + t + 4]};
#pragma unroll
                for (int q = 0; q < 2; ++q) { bh[ni][q] = to_tf32(v[q]); bl[ni][q] = to_tf32(v[q] - __uint_as_float(bh[ni][q])); }
            }
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    mma_tf32(acc[mi][ni], al[mi][0], al[mi][1], al[mi][2], al[mi][3], bh[ni][0], bh[ni][1]);
                    mma_tf32(acc[mi][ni], ah[mi][0], ah[mi][1], ah[mi][2], ah[mi][3], bl[ni][0], bl[ni][1]);
                    mma_tf32(acc[mi][ni], ah[mi][0], ah[mi][1], ah[mi][2], ah[mi][3], bh[ni][0], bh[ni][1]);
                }
        }
        __syncthreads();
    }
    // (quartet 0 + quartet 2) + (quartet 1 + quartet 3): partial sums laid out [warp slot][value][lane]
    float* red = lin_smem;
    auto put = [&](int slot) {
#pragma unroll
        for (int i = 0; i < 32; ++i) red[(slot * 32 + i) * 32 + lane] = acc[i >> 4][(i >> 2) & 3][i & 3];
    };
    auto add = [&](int slot) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i >> 4][(i >> 2) & 3][i & 3] += red[(slot * 32 + i) * 32 + lane];
    };
    if (KQ == 4) {
        if (kq >= 2) put(warp - 8);
        __syncthreads();
        if (kq < 2) add(warp);
        __syncthreads();
    }
    if (kq == 1) put(warp - 4);
    __syncthreads();
    if (kq != 0) return;
    add(warp);
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const long long r = m0 + wm + 16 * mi + g + 8 * (e >> 1);
                const int c = n0 + wn + 8 * ni + 2 * t + (e & 1);
                if (r >= m || c >= n) continue;
                const float v = acc[mi][ni][e] + (bias ? bias[c] : 0.f);
                const long long idx = yt_pitch > 0 ? (long long)c * yt_pitch + r : r * n + c;      // transposed: y^T[c][r]
                y[idx] = accumulate ? y[idx] + v : v;
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
    if (k % 4 == 0 && aligned16(x) && aligned16(w)) {
        f32_linear_mma_kernel<2><<<grid, 256, 0, (cudaStream_t)stream>>>(x, w, bias, y, rows, k, n_out, accumulate, 0);
    } else
        f32_linear_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, w, bias, y, rows, k, n_out, accumulate, 0);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_linear_t(const float* x, const float* w, const float* bias, float* yt, long long yt_pitch,
                        long long rows, int k, int n_out, void* stream) {
    B200PF_REQUIRE(x && w && yt && rows >= 0 && k > 0 && n_out > 0 && yt_pitch >= rows, B200PF_ERR_INVALID,
                   "f32_linear_t: bad argument");
    if (rows == 0) return B200PF_OK;
    dim3 grid((unsigned)((rows + 63) / 64), (unsigned)((n_out + 63) / 64));
    if (k % 4 == 0 && aligned16(x) && aligned16(w)) {
        f32_linear_mma_kernel<2><<<grid, 256, 0, (cudaStream_t)stream>>>(x, w, bias, yt, rows, k, n_out, 0, yt_pitch);
    } else
        f32_linear_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, w, bias, yt, rows, k, n_out, 0, yt_pitch);
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
    f32_gate_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a, b, row_mask, y, total, c, mode, c, c, c);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_gate_strided(const float* a, long long a_pitch, const float* b, long long b_pitch, float* y, long long y_pitch,
                            long long rows, int c, int mode, void* stream) {
    B200PF_REQUIRE(a && b && y && rows >= 0 && c > 0 && mode >= 0 && mode <= 2 && a_pitch >= c && b_pitch >= c && y_pitch >= c,
                   B200PF_ERR_INVALID, "f32_gate_strided: bad argument");
    long long total = rows * c;
    if (total == 0) return B200PF_OK;
    unsigned blocks = (unsigned)min((long long)148 * 16, (total + 255) / 256);
    f32_gate_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a, b, nullptr, y, total, c, mode, a_pitch, b_pitch, y_pitch);
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
    B200PF_REQUIRE(hd == 24 || hd == 32, B200PF_ERR_UNSUPPORTED, "f32_attention: head dim must be 24 or 32 (got %d)", hd);
    B200PF_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && rs % 4 == 0 && ps % 4 == 0, B200PF_ERR_INVALID,
                   "f32_attention: q/k/v must be 16-byte aligned with strides that are multiples of 4");
    auto kern = hd == 24 ? f32_attention_kernel<24> : f32_attention_kernel<32>;
    if (smem > 48 * 1024)
        B200PF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    long long total = (long long)batch * heads * n_q;
    unsigned blocks = (unsigned)min((long long)148 * 8, (total + warps - 1) / warps);
    kern<<<blocks, warps * 32, smem, (cudaStream_t)stream>>>(p);
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
        ln_proj_heads16_mma_kernel<<<(unsigned)min((long long)148 * 2, (rows + 127) / 128), 256, 0, (cudaStream_t)stream>>>(
            z, gamma, beta, w, out, out_hs, rows);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int b200pf_f32_sattention(const float* q, long long q_pitch, const float* g, long long g_pitch,
                          const float* kt, const float* vt, long long kt_pitch, float* o, long long o_pitch,
                          const float* bias, long long bias_hs, long long bias_qs, const uint8_t* mask,
                          int n_q, int n_k, int heads, int hd, float scale, float inf_value, void* stream) {
    B200PF_REQUIRE(q && kt && vt && o && bias && n_q > 0 && n_k > 0 && heads > 0, B200PF_ERR_INVALID, "f32_sattention: bad argument");
    B200PF_REQUIRE(hd == 24, B200PF_ERR_UNSUPPORTED, "f32_sattention: built for head dim 24 (got %d)", hd);
    B200PF_REQUIRE(kt_pitch >= n_k, B200PF_ERR_INVALID, "f32_sattention: kt_pitch must cover the keys");
    SAttnArgs p{q, g, kt, vt, bias, o, mask, q_pitch, g_pitch, o_pitch, kt_pitch, bias_hs, bias_qs, n_q, n_k, heads, scale, inf_value};
    const bool staged = aligned16(kt) && aligned16(vt) && aligned16(bias) && kt_pitch % 4 == 0 && bias_hs % 4 == 0 && bias_qs % 4 == 0;
    if (staged) {
        B200PF_SMEM_ATTR_ONCE(f32_sattention_mma_kernel<24>, satc::smem_bytes<24>());
        f32_sattention_mma_kernel<24><<<(unsigned)(heads * ((n_q + satc::QT - 1) / satc::QT)), 128, satc::smem_bytes<24>(), (cudaStream_t)stream>>>(p);
    } else {
        f32_sattention_kernel<24><<<(unsigned)(heads * ((n_q + 31) / 32)), 256, 0, (cudaStream_t)stream>>>(p);
    }
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

}  // extern "C"
