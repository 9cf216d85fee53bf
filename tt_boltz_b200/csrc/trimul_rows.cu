// Triangle multiplication, the two row-local stages around the contraction.
//
//   producer : z -> LN -> [p | g] projection (128 -> 512) -> p * sigmoid(g) * mask -> a / b planes
//   epilogue : x planes -> LN over channels -> p_out ; LN(z) -> g_out ; z += p_out * sigmoid(g_out)
//
// Weight packing done by the host (tt_boltz_b200/weights.py):
//   w_pg  [512][128]: 8 chunks of 64 rows; chunk q holds, for channels 32*(q%4) .. +31 of operand
//         a (q < 4) or b (q >= 4), the 32 p_in rows followed by the 32 g_in rows, LN gain folded in;
//   bias_pg [512]   : the matching LN-offset term (W beta), fp32, same order.
#include "row512_tc.h"
#include "rowtile.cuh"

namespace b200pf {

constexpr int STAGE_PITCH = 40;   // bf16 elements per staged channel row (32 positions + pad)

struct ProducerArgs {
    const float* z;
    const uint8_t* mask;
    const __nv_bfloat16* w_pg;
    const float* bias_pg;
    __nv_bfloat16* planes[2];        // a, b
    long long plane_stride[2];       // elements between channels
    long long group_stride[2];       // elements between groups of plane rows
    int row_group[2];                // plane rows per group (>= plane rows when ungrouped)
    int pitch, rows, n, incoming;
};

__global__ void __launch_bounds__(WARPS * 32, 1) trimul_producer_kernel(ProducerArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __nv_bfloat16* w_s = reinterpret_cast<__nv_bfloat16*>(smem);                        // [512][APITCH]
    float* bias_s = reinterpret_cast<float*>(smem + 512 * APITCH * 2);                  // [512]
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem + 512 * APITCH * 2 + 512 * 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __nv_bfloat16* tile = tiles + warp * (UNIT * APITCH);
    load_weights_k128(w_s, p.w_pg, 512);
    for (int i = threadIdx.x; i < 512; i += blockDim.x) bias_s[i] = p.bias_pg[i];
    __syncthreads();
    const uint32_t w_addr = smem_u32(w_s), tile_addr = smem_u32(tile);

    // unit -> (line, first position): outgoing walks a z row, incoming walks a z column.
    const int span = p.incoming ? p.rows : p.n;              // positions along a unit's line
    const int upl = (span + UNIT - 1) / UNIT;
    const long long units = (long long)(p.incoming ? p.n : p.rows) * upl;
    const int g = lane >> 2, t = lane & 3;

    for (long long u = (long long)blockIdx.x * WARPS + warp; u < units; u += (long long)gridDim.x * WARPS) {
        const int line = (int)(u / upl), pos0 = (int)(u % upl) * UNIT;
        auto flat = [&](int l) -> long long {   // flat (r * n + c) index of position l, or -1
            int pos = pos0 + l;
            if (pos >= span) return -1;
            return p.incoming ? (long long)pos * p.n + line : (long long)line * p.n + pos;
        };
        ln_rows_to_tile([&](int l) -> const float* { long long f = flat(l); return f < 0 ? nullptr : p.z + f * KC; },
                        tile, lane);
        __syncwarp();
        uint32_t afrag[2][8][4];
        load_a_all(tile_addr, lane, afrag);
        float mk[2][2];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                long long f = flat(mi * 16 + g + hh * 8);
                mk[mi][hh] = f < 0 ? 0.f : (float)p.mask[f];
            }
        __syncwarp();                                   // tile is now free: reuse it as staging
        __nv_bfloat16* stage = tile;
#pragma unroll 1
        for (int q = 0; q < 8; ++q) {
            float acc[2][8][4];
            zero_acc(acc);
            warp_gemm_regA<8>(afrag, w_addr, APITCH, q * 64, lane, acc);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        int col = nt * 8 + 2 * t + (e & 1);
                        float pv = acc[mi][nt][e] + bias_s[q * 64 + col];
                        float gv = acc[mi][nt + 4][e] + bias_s[q * 64 + 32 + col];
                        float uv = pv * sigmoidf_(gv) * mk[mi][e >> 1];
                        stage[col * STAGE_PITCH + mi * 16 + g + (e >> 1) * 8] = __float2bfloat16(uv);
                    }
            __syncwarp();
            const int op = q >> 2;
            const long long ps = p.plane_stride[op];
            __nv_bfloat16* planes = p.planes[op] + (long long)((q & 3) * 32) * ps +
                                    (long long)(line / p.row_group[op]) * p.group_stride[op] +
                                    (long long)(line % p.row_group[op]) * p.pitch;
#pragma unroll
            for (int pass = 0; pass < 4; ++pass) {
                int ch = pass * 8 + (lane >> 2), piece = lane & 3;
                int col = pos0 + piece * 8;
                if (col + 8 <= p.pitch) {
                    uint4 v = *reinterpret_cast<const uint4*>(stage + ch * STAGE_PITCH + piece * 8);
                    *reinterpret_cast<uint4*>(planes + ch * ps + col) = v;
                }
            }
            __syncwarp();
        }
    }
}

struct EpilogueArgs {
    float* z;
    const __nv_bfloat16* x;
    long long x_plane_stride;
    int x_pitch;
    const __nv_bfloat16* w_pout;   // [128][128], LN_out gain folded
    const __nv_bfloat16* w_gout;   // [128][128], LN_in gain folded
    const float* bias_pout;        // [128]
    const float* bias_gout;        // [128]
    int rows, n;
};

__global__ void __launch_bounds__(WARPS * 32, 1) trimul_epilogue_kernel(EpilogueArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __nv_bfloat16* wp_s = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* wg_s = wp_s + 128 * APITCH;
    float* bias_s = reinterpret_cast<float*>(wg_s + 128 * APITCH);     // [256]: p_out then g_out
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(bias_s + 256);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __nv_bfloat16* tile_x = tiles + warp * (2 * UNIT * APITCH);
    __nv_bfloat16* tile_z = tile_x + UNIT * APITCH;
    load_weights_k128(wp_s, p.w_pout, 128);
    load_weights_k128(wg_s, p.w_gout, 128);
    for (int i = threadIdx.x; i < 128; i += blockDim.x) { bias_s[i] = p.bias_pout[i]; bias_s[128 + i] = p.bias_gout[i]; }
    __syncthreads();
    const uint32_t wp_addr = smem_u32(wp_s), wg_addr = smem_u32(wg_s);
    const uint32_t tx_addr = smem_u32(tile_x), tz_addr = smem_u32(tile_z);
    const int upl = (p.n + UNIT - 1) / UNIT;
    const long long units = (long long)p.rows * upl;
    const int g = lane >> 2, t = lane & 3;

    for (long long u = (long long)blockIdx.x * WARPS + warp; u < units; u += (long long)gridDim.x * WARPS) {
        const int r = (int)(u / upl), c0 = (int)(u % upl) * UNIT;
        // ---- x planes -> LayerNorm over channels -> tile_x[position][channel] ----
        {
            const int piece = lane & 3, dsub = lane >> 2;
            const bool in_pitch = c0 + piece * 8 + 8 <= p.x_pitch;
            const __nv_bfloat16* xp = p.x + (long long)r * p.x_pitch + c0 + piece * 8;
            uint4 xv[16];
            float s[8], ss[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) { s[e] = 0.f; ss[e] = 0.f; }
#pragma unroll
            for (int pass = 0; pass < 16; ++pass) {
                int d = pass * 8 + dsub;
                xv[pass] = in_pitch ? __ldg(reinterpret_cast<const uint4*>(xp + d * p.x_plane_stride)) : make_uint4(0, 0, 0, 0);
                const uint32_t* w = reinterpret_cast<const uint32_t*>(&xv[pass]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float lo = bf16_lo(w[e]), hi = bf16_hi(w[e]);
                    s[2 * e] += lo; ss[2 * e] += lo * lo;
                    s[2 * e + 1] += hi; ss[2 * e + 1] += hi * hi;
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
#pragma unroll
                for (int o = 4; o <= 16; o <<= 1) {
                    s[e] += __shfl_xor_sync(0xffffffffu, s[e], o);
                    ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], o);
                }
                float mean = s[e] * (1.f / KC);
                float var = fmaxf(ss[e] * (1.f / KC) - mean * mean, 0.f);
                s[e] = mean;
                ss[e] = rsqrtf(var + LN_EPS);
            }
#pragma unroll
            for (int pass = 0; pass < 16; ++pass) {
                int d = pass * 8 + dsub;
                const uint32_t* w = reinterpret_cast<const uint32_t*>(&xv[pass]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float lo = (bf16_lo(w[e]) - s[2 * e]) * ss[2 * e];
                    float hi = (bf16_hi(w[e]) - s[2 * e + 1]) * ss[2 * e + 1];
                    tile_x[(piece * 8 + 2 * e) * APITCH + d] = __float2bfloat16(lo);
                    tile_x[(piece * 8 + 2 * e + 1) * APITCH + d] = __float2bfloat16(hi);
                }
            }
        }
        // ---- LN_in(z) rows -> tile_z ----
        ln_rows_to_tile([&](int l) -> const float* {
            return c0 + l < p.n ? p.z + ((long long)r * p.n + c0 + l) * KC : nullptr; }, tile_z, lane);
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            float acc_p[2][8][4], acc_g[2][8][4];
            zero_acc(acc_p);
            zero_acc(acc_g);
            warp_gemm_smemA<8>(tx_addr, wp_addr, APITCH, c * 64, lane, acc_p);
            warp_gemm_smemA<8>(tz_addr, wg_addr, APITCH, c * 64, lane, acc_g);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    int l = mi * 16 + g + hh * 8;
                    if (c0 + l >= p.n) continue;
                    float* zr = p.z + ((long long)r * p.n + c0 + l) * KC + c * 64 + 2 * t;
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt) {
                        int col = c * 64 + nt * 8 + 2 * t;
                        float2 zv = *reinterpret_cast<float2*>(zr + nt * 8);
                        zv.x += (acc_p[mi][nt][hh * 2] + bias_s[col]) * sigmoidf_(acc_g[mi][nt][hh * 2] + bias_s[128 + col]);
                        zv.y += (acc_p[mi][nt][hh * 2 + 1] + bias_s[col + 1]) * sigmoidf_(acc_g[mi][nt][hh * 2 + 1] + bias_s[128 + col + 1]);
                        *reinterpret_cast<float2*>(zr + nt * 8) = zv;
                    }
                }
        }
        __syncwarp();
    }
}

constexpr int PRODUCER_SMEM = 512 * APITCH * 2 + 512 * 4 + WARPS * A_TILE_BYTES;          // 210,944
constexpr int EPILOGUE_SMEM = 2 * 128 * APITCH * 2 + 256 * 4 + WARPS * 2 * A_TILE_BYTES;  // 209,920

static int grid_for(long long units) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long ctas = (units + WARPS - 1) / WARPS;
    return (int)(ctas < sms ? ctas : sms);
}

}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_trimul_producer(const float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                                      const float* bias_pg, const b200pf_bf16* w_pg, const b200pf_plane_out* a_out,
                                      const b200pf_plane_out* b_out, int pitch, int rows, int n, int incoming,
                                      int value_mode, int impl, void* stream) {
    B200PF_REQUIRE(z && mask && w_pg && a_out && b_out && a_out->ptr && b_out->ptr, B200PF_ERR_INVALID,
                   "trimul_producer: null pointer");
    B200PF_REQUIRE(impl == 0 ? (ln_gamma && ln_beta) : (bias_pg != nullptr), B200PF_ERR_INVALID,
                   "trimul_producer: impl 0 needs ln_gamma / ln_beta, impl 1 needs bias_pg");
    B200PF_REQUIRE(rows > 0 && n > 0 && rows <= n, B200PF_ERR_INVALID, "trimul_producer: bad rows/n");
    B200PF_REQUIRE(value_mode == 0, B200PF_ERR_UNSUPPORTED, "trimul_producer: value mode %d is not built", value_mode);
    int cols = incoming ? rows : n, prow = incoming ? n : rows;
    B200PF_REQUIRE(pitch % 8 == 0 && pitch >= cols, B200PF_ERR_INVALID, "trimul_producer: bad pitch");
    ProducerArgs p;
    p.z = z; p.mask = mask; p.w_pg = (const __nv_bfloat16*)w_pg; p.bias_pg = bias_pg;
    const b200pf_plane_out* outs[2] = {a_out, b_out};
    for (int i = 0; i < 2; ++i) {
        const b200pf_plane_out* o = outs[i];
        int rg = o->row_group > 0 ? o->row_group : prow;
        B200PF_REQUIRE(o->plane_stride % 8 == 0 && o->plane_stride >= (long long)pitch * (rg < prow ? rg : prow),
                       B200PF_ERR_INVALID, "trimul_producer: bad plane stride");
        B200PF_REQUIRE(rg >= prow || (o->group_stride % 8 == 0 && o->group_stride > 0), B200PF_ERR_INVALID,
                       "trimul_producer: bad group stride");
        B200PF_REQUIRE(aligned16(o->ptr), B200PF_ERR_INVALID, "trimul_producer: planes must be 16-byte aligned");
        p.planes[i] = (__nv_bfloat16*)o->ptr; p.plane_stride[i] = o->plane_stride;
        p.group_stride[i] = o->group_stride; p.row_group[i] = rg;
    }
    B200PF_REQUIRE(aligned16(z) && aligned16(w_pg), B200PF_ERR_INVALID, "trimul_producer: pointers must be 16-byte aligned");
    p.pitch = pitch; p.rows = rows; p.n = n; p.incoming = incoming;
    B200PF_REQUIRE(impl == 0 || impl == 1, B200PF_ERR_INVALID, "trimul_producer: impl must be 0 (tcgen05) or 1 (mma.sync)");
    if (impl == 0) {
        r512::Args a{};
        a.z = z; a.mask = mask; a.w = p.w_pg; a.ln_gamma = ln_gamma; a.ln_beta = ln_beta;
        for (int i = 0; i < 2; ++i) {
            a.planes[i] = p.planes[i]; a.plane_stride[i] = p.plane_stride[i];
            a.group_stride[i] = p.group_stride[i]; a.row_group[i] = p.row_group[i];
        }
        a.pitch = pitch; a.rows = rows; a.n = n; a.transposed = incoming;
        return r512::launch_trimul(a, (cudaStream_t)stream);
    }
    B200PF_SMEM_ATTR_ONCE(trimul_producer_kernel, PRODUCER_SMEM);
    int span = incoming ? rows : n;
    long long units = (long long)(incoming ? n : rows) * ((span + UNIT - 1) / UNIT);
    trimul_producer_kernel<<<grid_for(units), WARPS * 32, PRODUCER_SMEM, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_trimul_producer_mx(const float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                                         const b200pf_bf16* w_pg, uint8_t* a_out, uint8_t* b_out, uint8_t* a_scales,
                                         uint8_t* b_scales, long long plane_stride, int pitch, int rows, int n, int incoming,
                                         void* stream) {
    B200PF_REQUIRE(z && mask && ln_gamma && ln_beta && w_pg && a_out && b_out && a_scales && b_scales, B200PF_ERR_INVALID,
                   "trimul_producer_mx: null pointer");
    B200PF_REQUIRE(rows > 0 && n > 0 && rows <= n, B200PF_ERR_INVALID, "trimul_producer_mx: bad rows/n");
    const int cols = incoming ? rows : n, prow = incoming ? n : rows;
    B200PF_REQUIRE(pitch % 16 == 0 && pitch >= cols && plane_stride % 16 == 0 && plane_stride >= (long long)pitch * prow,
                   B200PF_ERR_INVALID, "trimul_producer_mx: pitch / plane stride must be multiples of 16 bytes and large enough");
    B200PF_REQUIRE(aligned16(z) && aligned16(w_pg) && aligned16(a_out) && aligned16(b_out) && aligned16(a_scales) &&
                       aligned16(b_scales), B200PF_ERR_INVALID, "trimul_producer_mx: pointers must be 16-byte aligned");
    r512::Args a{};
    a.z = z; a.mask = mask; a.w = (const __nv_bfloat16*)w_pg; a.ln_gamma = ln_gamma; a.ln_beta = ln_beta;
    a.planes[0] = reinterpret_cast<__nv_bfloat16*>(a_out); a.planes[1] = reinterpret_cast<__nv_bfloat16*>(b_out);
    a.scales[0] = a_scales; a.scales[1] = b_scales;
    for (int i = 0; i < 2; ++i) { a.plane_stride[i] = plane_stride; a.group_stride[i] = 0; a.row_group[i] = prow; }
    a.sf_kgroups = (cols + 127) / 128;
    a.sf_row_blocks = 2 * ((prow + 255) / 256);
    a.pitch = pitch; a.rows = rows; a.n = n; a.transposed = incoming;
    return r512::launch_trimul_mx(a, (cudaStream_t)stream);
}

extern "C" int b200pf_trimul_epilogue(float* z, const b200pf_bf16* x, long long x_plane_stride, int x_pitch,
                                      const b200pf_bf16* w_pout, const b200pf_bf16* w_gout,
                                      const float* bias_pout, const float* bias_gout,
                                      int rows, int n, void* stream) {
    B200PF_REQUIRE(z && x && w_pout && w_gout && bias_pout && bias_gout, B200PF_ERR_INVALID, "trimul_epilogue: null pointer");
    B200PF_REQUIRE(rows > 0 && n > 0 && x_pitch % 8 == 0 && x_pitch >= n && x_plane_stride % 8 == 0,
                   B200PF_ERR_INVALID, "trimul_epilogue: bad sizes");
    B200PF_REQUIRE(aligned16(z) && aligned16(x) && aligned16(w_pout) && aligned16(w_gout), B200PF_ERR_INVALID,
                   "trimul_epilogue: pointers must be 16-byte aligned");
    EpilogueArgs p{z, (const __nv_bfloat16*)x, x_plane_stride, x_pitch, (const __nv_bfloat16*)w_pout,
                   (const __nv_bfloat16*)w_gout, bias_pout, bias_gout, rows, n};
    B200PF_SMEM_ATTR_ONCE(trimul_epilogue_kernel, EPILOGUE_SMEM);
    long long units = (long long)rows * ((n + UNIT - 1) / UNIT);
    trimul_epilogue_kernel<<<grid_for(units), WARPS * 32, EPILOGUE_SMEM, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
