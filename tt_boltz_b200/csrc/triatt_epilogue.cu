// Triangle attention, the two row-local stages around the fused attention core.
//
//   producer : z -> LN -> [q | k | g | v] projection (128 -> 512) + 4-head triangle bias; the kernel is
//              row512_kernel<1> in row512_tc.cu, this file holds its entry point
//   epilogue : z += (o * g) W_o^T   (mma.sync; the residual is added by red.global.add, so z is not read)
#include "row512_tc.h"
#include "rowtile.cuh"

namespace b200pf {

struct AttEpilogueArgs {
    float* z;                       // residual stream to add into, or
    __nv_bfloat16* upd;             // (z == nullptr) where to store the update itself, bf16, same layout
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
                    if (p.z) {
                        float* zr = p.z + f * KC + c * 64 + 2 * t;
#pragma unroll
                        for (int nt = 0; nt < 8; ++nt)      // residual add done by L2 (no load to wait for)
                            asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(zr + nt * 8), "f"(acc[mi][nt][hh * 2]),
                                         "f"(acc[mi][nt][hh * 2 + 1]) : "memory");
                    } else {
                        uint32_t* ur = reinterpret_cast<uint32_t*>(p.upd + f * KC + c * 64 + 2 * t);
#pragma unroll
                        for (int nt = 0; nt < 8; ++nt) ur[nt * 4] = pack_bf16x2(acc[mi][nt][hh * 2], acc[mi][nt][hh * 2 + 1]);
                    }
                }
        }
        __syncwarp();
    }
}

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

static int triatt_producer(const float* z, const b200pf_bf16* z_bf16, const float* ln_gamma, const float* ln_beta,
                           const float* w_bias_f32, const b200pf_bf16* w_qkgv,
                           b200pf_bf16* q, b200pf_bf16* k, b200pf_bf16* v, b200pf_bf16* g,
                           b200pf_bf16* tri_bias, long long bias_hs, long long bias_qs,
                           int vt_pitch, int rows, int n, int ending, void* stream) {
    B200PF_REQUIRE((z || z_bf16) && ln_gamma && ln_beta && w_bias_f32 && w_qkgv && q && k && v && g && tri_bias, B200PF_ERR_INVALID,
                   "triatt_producer: null pointer");
    B200PF_REQUIRE(rows > 0 && n > 0, B200PF_ERR_INVALID, "triatt_producer: bad rows/n");
    B200PF_REQUIRE(bias_hs > 0 && bias_qs > 0, B200PF_ERR_INVALID, "triatt_producer: bad bias strides");
    B200PF_REQUIRE(vt_pitch > 0 && vt_pitch % 8 == 0 && vt_pitch >= (ending ? rows : n), B200PF_ERR_INVALID,
                   "triatt_producer: vt_pitch must be a multiple of 8 covering the positions of a line");
    B200PF_REQUIRE(aligned16(z) && aligned16(z_bf16) && aligned16(w_qkgv) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g),
                   B200PF_ERR_INVALID, "triatt_producer: pointers must be 16-byte aligned");
    r512::Args a{};
    a.z = z; a.z_bf16 = (const __nv_bfloat16*)z_bf16;
    a.w = (const __nv_bfloat16*)w_qkgv; a.ln_gamma = ln_gamma; a.ln_beta = ln_beta; a.w_bias_f32 = w_bias_f32;
    a.q = (__nv_bfloat16*)q; a.k = (__nv_bfloat16*)k; a.v = (__nv_bfloat16*)v; a.g = (__nv_bfloat16*)g;
    a.tri_bias = (__nv_bfloat16*)tri_bias;
    a.bias_hs = bias_hs; a.bias_qs = bias_qs; a.vt_pitch = vt_pitch;
    a.rows = rows; a.n = n; a.transposed = ending;
    return r512::launch_triatt(a, (cudaStream_t)stream);
}

extern "C" int b200pf_triatt_producer(const float* z, const float* ln_gamma, const float* ln_beta, const float* w_bias_f32,
                                      const b200pf_bf16* w_qkgv,
                                      b200pf_bf16* q, b200pf_bf16* k, b200pf_bf16* v, b200pf_bf16* g,
                                      b200pf_bf16* tri_bias, long long bias_hs, long long bias_qs,
                                      int vt_pitch, int rows, int n, int ending, void* stream) {
    B200PF_REQUIRE(z, B200PF_ERR_INVALID, "triatt_producer: null pointer");
    return triatt_producer(z, nullptr, ln_gamma, ln_beta, w_bias_f32, w_qkgv, q, k, v, g, tri_bias, bias_hs, bias_qs, vt_pitch,
                           rows, n, ending, stream);
}

extern "C" int b200pf_triatt_producer_bf16z(const b200pf_bf16* z, const float* ln_gamma, const float* ln_beta, const float* w_bias_f32,
                                            const b200pf_bf16* w_qkgv,
                                            b200pf_bf16* q, b200pf_bf16* k, b200pf_bf16* v, b200pf_bf16* g,
                                            b200pf_bf16* tri_bias, long long bias_hs, long long bias_qs,
                                            int vt_pitch, int rows, int n, int ending, void* stream) {
    B200PF_REQUIRE(z, B200PF_ERR_INVALID, "triatt_producer_bf16z: null pointer");
    return triatt_producer(nullptr, z, ln_gamma, ln_beta, w_bias_f32, w_qkgv, q, k, v, g, tri_bias, bias_hs, bias_qs, vt_pitch,
                           rows, n, ending, stream);
}

static int triatt_epilogue(float* z, b200pf_bf16* upd, const b200pf_bf16* o, const b200pf_bf16* g,
                           const b200pf_bf16* w_o, long long n_rows_flat, void* stream) {
    B200PF_REQUIRE((z || upd) && o && g && w_o && n_rows_flat > 0, B200PF_ERR_INVALID, "triatt_epilogue: bad argument");
    B200PF_REQUIRE(aligned16(z) && aligned16(upd) && aligned16(o) && aligned16(g) && aligned16(w_o), B200PF_ERR_INVALID,
                   "triatt_epilogue: pointers must be 16-byte aligned");
    AttEpilogueArgs p{z, (__nv_bfloat16*)upd, (const __nv_bfloat16*)o, (const __nv_bfloat16*)g, (const __nv_bfloat16*)w_o, n_rows_flat};
    B200PF_SMEM_ATTR_ONCE(triatt_epilogue_kernel, ATT_EPILOGUE_SMEM);
    long long units = (n_rows_flat + UNIT - 1) / UNIT;
    triatt_epilogue_kernel<<<grid_for_units(units, 2), WARPS * 32, ATT_EPILOGUE_SMEM, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_triatt_epilogue(float* z, const b200pf_bf16* o, const b200pf_bf16* g,
                                      const b200pf_bf16* w_o, long long n_rows_flat, void* stream) {
    B200PF_REQUIRE(z, B200PF_ERR_INVALID, "triatt_epilogue: bad argument");
    return triatt_epilogue(z, nullptr, o, g, w_o, n_rows_flat, stream);
}

extern "C" int b200pf_triatt_epilogue_update(b200pf_bf16* upd, const b200pf_bf16* o, const b200pf_bf16* g,
                                             const b200pf_bf16* w_o, long long n_rows_flat, void* stream) {
    B200PF_REQUIRE(upd, B200PF_ERR_INVALID, "triatt_epilogue_update: bad argument");
    return triatt_epilogue(nullptr, upd, o, g, w_o, n_rows_flat, stream);
}
