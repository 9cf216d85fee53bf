// Triangle attention, the two row-local stages around the fused attention core.
//
//   producer : z -> LN -> [q | k | v | g] projection (128 -> 512) + 4-head triangle bias;
//              q, k, v written per (line, head) as [pos][32]; sigmoid(g) in z layout; bias [h][q][k]
//   epilogue : z += (o * g) W_o^T
//
// Host packing (tt_boltz_b200/weights.py): w_qkvg [528][128] = q (scaled by log2(e)/sqrt(32)),
// k, v, g rows, then the 4 bias rows (scaled by log2(e)) and 12 zero rows, LN gain folded in;
// bias_qkvg [528] = the matching LN-offset terms.
#include "row512_tc.h"
#include "rowtile.cuh"

namespace b200pf {

constexpr int QKVG_ROWS = 528;
constexpr int HDIM = 32;
constexpr int ST_PITCH = 72;     // staging: 64 columns + 8 pad (bf16 elements)

struct AttProducerArgs {
    const float* z;
    const __nv_bfloat16* w;
    const float* wbias;
    __nv_bfloat16 *q, *k, *v, *g, *tri_bias;
    long long bias_hs, bias_qs;
    int vt_pitch;                     // > 0: v is written transposed, [line][head][32][vt_pitch]
    int rows, n, ending;              // z viewed as [rows][n][128]
};

__global__ void __launch_bounds__(WARPS * 32, 1) triatt_producer_kernel(AttProducerArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __nv_bfloat16* w_s = reinterpret_cast<__nv_bfloat16*>(smem);
    float* bias_s = reinterpret_cast<float*>(smem + QKVG_ROWS * APITCH * 2);
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem + QKVG_ROWS * APITCH * 2 + 528 * 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __nv_bfloat16* tile = tiles + warp * (UNIT * APITCH);
    load_weights_k128(w_s, p.w, QKVG_ROWS);
    for (int i = threadIdx.x; i < QKVG_ROWS; i += blockDim.x) bias_s[i] = p.wbias[i];
    __syncthreads();
    const uint32_t w_addr = smem_u32(w_s), tile_addr = smem_u32(tile);
    const int n = p.n;
    const int span = p.ending ? p.rows : n;          // positions along a line
    const int upl = (span + UNIT - 1) / UNIT;
    const long long units = (long long)(p.ending ? n : p.rows) * upl;
    const int g = lane >> 2, t = lane & 3;

    for (long long u = (long long)blockIdx.x * WARPS + warp; u < units; u += (long long)gridDim.x * WARPS) {
        const int line = (int)(u / upl), pos0 = (int)(u % upl) * UNIT;
        auto flat = [&](int l) -> long long {
            int pos = pos0 + l;
            if (pos >= span) return -1;
            return p.ending ? (long long)pos * n + line : (long long)line * n + pos;
        };
        ln_rows_to_tile([&](int l) -> const float* { long long f = flat(l); return f < 0 ? nullptr : p.z + f * KC; },
                        tile, lane);
        __syncwarp();
        uint32_t afrag[2][8][4];
        load_a_all(tile_addr, lane, afrag);
        __syncwarp();
        __nv_bfloat16* stage = tile;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
            float acc[2][8][4];
            zero_acc(acc);
            warp_gemm_regA<8>(afrag, w_addr, APITCH, c * 64, lane, acc);
            const bool gate = c >= 6;
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        int col = nt * 8 + 2 * t;
                        float v0 = acc[mi][nt][hh * 2] + bias_s[c * 64 + col];
                        float v1 = acc[mi][nt][hh * 2 + 1] + bias_s[c * 64 + col + 1];
                        if (gate) { v0 = sigmoidf_(v0); v1 = sigmoidf_(v1); }
                        *reinterpret_cast<uint32_t*>(stage + (mi * 16 + g + hh * 8) * ST_PITCH + col) = pack_bf16x2(v0, v1);
                    }
            __syncwarp();
            if (p.vt_pitch > 0 && (c == 4 || c == 5)) {
                // V transposed: for each (head, d) the unit's 32 positions are 64 contiguous bytes
#pragma unroll
                for (int pass = 0; pass < 8; ++pass) {
                    int col = pass * 8 + (lane >> 2), piece = lane & 3;          // col = head_local*32 + d
                    uint32_t w4[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        int l0 = piece * 8 + e * 2;
                        uint32_t lo = *reinterpret_cast<const uint16_t*>(stage + l0 * ST_PITCH + col);
                        uint32_t hi = *reinterpret_cast<const uint16_t*>(stage + (l0 + 1) * ST_PITCH + col);
                        w4[e] = lo | (hi << 16);
                    }
                    int head = (c & 1) * 2 + (col >> 5), dd = col & 31;
                    int pos = pos0 + piece * 8;
                    if (pos + 8 <= p.vt_pitch)
                        *reinterpret_cast<uint4*>(p.v + (((long long)line * 4 + head) * HDIM + dd) * p.vt_pitch + pos) =
                            make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
                __syncwarp();
                continue;
            }
#pragma unroll
            for (int pass = 0; pass < 8; ++pass) {
                int l = pass * 4 + (lane >> 3), piece = lane & 7;
                long long f = flat(l);
                if (f < 0) continue;
                uint4 v = *reinterpret_cast<const uint4*>(stage + l * ST_PITCH + piece * 8);
                if (gate) {
                    *reinterpret_cast<uint4*>(p.g + f * KC + (c - 6) * 64 + piece * 8) = v;
                } else {
                    __nv_bfloat16* dst = c < 2 ? p.q : (c < 4 ? p.k : p.v);
                    int head = (c & 1) * 2 + (piece >> 2);
                    *reinterpret_cast<uint4*>(dst + (((long long)line * 4 + head) * span + pos0 + l) * 32 + (piece & 3) * 8) = v;
                }
            }
            __syncwarp();
        }
        // ---- triangle bias: 4 heads in one extra n-tile pair (rows 512..519 of the packed weights) ----
        {
            float acc[2][2][4];
            zero_acc(acc);
            warp_gemm_regA<2>(afrag, w_addr, APITCH, 512, lane, acc);
            if (t < 2) {
#pragma unroll
                for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        int l = mi * 16 + g + hh * 8;
                        if (pos0 + l >= span) continue;
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            int h = 2 * t + e;
                            p.tri_bias[h * p.bias_hs + (long long)line * p.bias_qs + pos0 + l] =
                                __float2bfloat16(acc[mi][0][hh * 2 + e] + bias_s[512 + h]);
                        }
                    }
            }
        }
        __syncwarp();
    }
}

struct AttEpilogueArgs {
    float* z;
    const __nv_bfloat16 *o, *g, *w_o;
    long long rows_flat;
};

__global__ void __launch_bounds__(WARPS * 32, 1) triatt_epilogue_kernel(AttEpilogueArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __nv_bfloat16* w_s = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* tiles = w_s + 128 * APITCH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __nv_bfloat16* tile = tiles + warp * (UNIT * APITCH);
    load_weights_k128(w_s, p.w_o, 128);
    __syncthreads();
    const uint32_t w_addr = smem_u32(w_s), tile_addr = smem_u32(tile);
    const long long units = (p.rows_flat + UNIT - 1) / UNIT;
    const int g = lane >> 2, t = lane & 3;
    for (long long u = (long long)blockIdx.x * WARPS + warp; u < units; u += (long long)gridDim.x * WARPS) {
        const long long base = u * UNIT;
        // gather o * g into the operand tile: 8 lanes per row, 16 channels per lane
#pragma unroll 2
        for (int it = 0; it < 8; ++it) {
            int l = it * 4 + (lane >> 3), sub = lane & 7;
            long long f = base + l;
            uint4 ov[2], gv[2];
            if (f < p.rows_flat) {
                const uint4* op = reinterpret_cast<const uint4*>(p.o + f * KC) + sub * 2;
                const uint4* gp = reinterpret_cast<const uint4*>(p.g + f * KC) + sub * 2;
                ov[0] = __ldg(op); ov[1] = __ldg(op + 1); gv[0] = __ldg(gp); gv[1] = __ldg(gp + 1);
            } else {
                ov[0] = ov[1] = gv[0] = gv[1] = make_uint4(0, 0, 0, 0);
            }
            uint4 r[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const uint32_t* a = reinterpret_cast<const uint32_t*>(&ov[h2]);
                const uint32_t* b = reinterpret_cast<const uint32_t*>(&gv[h2]);
                uint32_t* d = reinterpret_cast<uint32_t*>(&r[h2]);
#pragma unroll
                for (int e = 0; e < 4; ++e) d[e] = pack_bf16x2(bf16_lo(a[e]) * bf16_lo(b[e]), bf16_hi(a[e]) * bf16_hi(b[e]));
            }
            uint4* dst = reinterpret_cast<uint4*>(tile + l * APITCH + sub * 16);
            dst[0] = r[0];
            dst[1] = r[1];
        }
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            float acc[2][8][4];
            zero_acc(acc);
            warp_gemm_smemA<8>(tile_addr, w_addr, APITCH, c * 64, lane, acc);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    long long f = base + mi * 16 + g + hh * 8;
                    if (f >= p.rows_flat) continue;
                    float* zr = p.z + f * KC + c * 64 + 2 * t;
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt)      // residual add done by L2 (no load to wait for)
                        asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(zr + nt * 8), "f"(acc[mi][nt][hh * 2]),
                                     "f"(acc[mi][nt][hh * 2 + 1]) : "memory");
                }
        }
        __syncwarp();
    }
}

constexpr int ATT_PRODUCER_SMEM = 528 * APITCH * 2 + 528 * 4 + WARPS * A_TILE_BYTES;   // 215,360
constexpr int ATT_EPILOGUE_SMEM = 128 * APITCH * 2 + WARPS * A_TILE_BYTES;             // 104,448

static int grid_for_units(long long units, int ctas_per_sm) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long ctas = (units + WARPS - 1) / WARPS;
    long long cap = (long long)sms * ctas_per_sm;
    return (int)(ctas < cap ? ctas : cap);
}

}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_triatt_producer(const float* z, const float* ln_gamma, const float* ln_beta, const float* w_bias_f32,
                                      const b200pf_bf16* w_qkvg, const float* bias_qkvg,
                                      b200pf_bf16* q, b200pf_bf16* k, b200pf_bf16* v, b200pf_bf16* g,
                                      b200pf_bf16* tri_bias, long long bias_hs, long long bias_qs,
                                      int vt_pitch, int rows, int n, int ending, int impl, void* stream) {
    B200PF_REQUIRE(z && w_qkvg && q && k && v && g && tri_bias, B200PF_ERR_INVALID, "triatt_producer: null pointer");
    B200PF_REQUIRE(impl == 0 ? (ln_gamma && ln_beta && w_bias_f32 && vt_pitch > 0) : (bias_qkvg != nullptr), B200PF_ERR_INVALID,
                   "triatt_producer: impl 0 needs ln_gamma / ln_beta / w_bias_f32 and vt_pitch > 0, impl 1 needs bias_qkvg");
    B200PF_REQUIRE(rows > 0 && n > 0, B200PF_ERR_INVALID, "triatt_producer: bad rows/n");
    B200PF_REQUIRE(bias_hs > 0 && bias_qs > 0, B200PF_ERR_INVALID, "triatt_producer: bad bias strides");
    B200PF_REQUIRE(vt_pitch == 0 || (vt_pitch % 8 == 0 && vt_pitch >= (ending ? rows : n)), B200PF_ERR_INVALID,
                   "triatt_producer: vt_pitch must be 0 or a multiple of 8 covering the positions of a line");
    B200PF_REQUIRE(aligned16(z) && aligned16(w_qkvg) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g),
                   B200PF_ERR_INVALID, "triatt_producer: pointers must be 16-byte aligned");
    AttProducerArgs p{z, (const __nv_bfloat16*)w_qkvg, bias_qkvg, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                      (__nv_bfloat16*)v, (__nv_bfloat16*)g, (__nv_bfloat16*)tri_bias, bias_hs, bias_qs, vt_pitch, rows, n, ending};
    B200PF_REQUIRE(impl == 0 || impl == 1, B200PF_ERR_INVALID, "triatt_producer: impl must be 0 (tcgen05) or 1 (mma.sync)");
    if (impl == 0) {
        r512::Args a{};
        a.z = z; a.w = (const __nv_bfloat16*)w_qkvg; a.ln_gamma = ln_gamma; a.ln_beta = ln_beta; a.w_bias_f32 = w_bias_f32;
        a.q = (__nv_bfloat16*)q; a.k = (__nv_bfloat16*)k; a.v = (__nv_bfloat16*)v; a.g = (__nv_bfloat16*)g;
        a.tri_bias = (__nv_bfloat16*)tri_bias;
        a.bias_hs = bias_hs; a.bias_qs = bias_qs; a.vt_pitch = vt_pitch;
        a.rows = rows; a.n = n; a.transposed = ending;
        return r512::launch_triatt(a, (cudaStream_t)stream);
    }
    B200PF_SMEM_ATTR_ONCE(triatt_producer_kernel, ATT_PRODUCER_SMEM);
    int span = ending ? rows : n;
    long long units = (long long)(ending ? n : rows) * ((span + UNIT - 1) / UNIT);
    triatt_producer_kernel<<<grid_for_units(units, 1), WARPS * 32, ATT_PRODUCER_SMEM, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_triatt_epilogue(float* z, const b200pf_bf16* o, const b200pf_bf16* g,
                                      const b200pf_bf16* w_o, long long n_rows_flat, void* stream) {
    B200PF_REQUIRE(z && o && g && w_o && n_rows_flat > 0, B200PF_ERR_INVALID, "triatt_epilogue: bad argument");
    B200PF_REQUIRE(aligned16(z) && aligned16(o) && aligned16(g) && aligned16(w_o), B200PF_ERR_INVALID,
                   "triatt_epilogue: pointers must be 16-byte aligned");
    AttEpilogueArgs p{z, (const __nv_bfloat16*)o, (const __nv_bfloat16*)g, (const __nv_bfloat16*)w_o, n_rows_flat};
    B200PF_SMEM_ATTR_ONCE(triatt_epilogue_kernel, ATT_EPILOGUE_SMEM);
    long long units = (n_rows_flat + UNIT - 1) / UNIT;
    triatt_epilogue_kernel<<<grid_for_units(units, 2), WARPS * 32, ATT_EPILOGUE_SMEM, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
