// Entry points of the triangle-multiplication producer (the kernels are row512_kernel<0> / <2> in row512_tc.cu):
//   z -> LayerNorm -> [p_a | g_a | p_b | g_b] projection (128 -> 512) -> p * sigmoid(g) * mask -> a / b planes
// as bf16 planes, or as MXFP8 planes (e4m3 values + e8m0 scale blocks).
#include "common.cuh"
#include "row512_tc.h"

using namespace b200pf;

extern "C" int b200pf_trimul_producer(const float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                                      const b200pf_bf16* w_pg, const b200pf_plane_out* a_out, const b200pf_plane_out* b_out,
                                      int pitch, int rows, int n, int incoming, void* stream) {
    B200PF_REQUIRE(z && mask && ln_gamma && ln_beta && w_pg && a_out && b_out && a_out->ptr && b_out->ptr, B200PF_ERR_INVALID,
                   "trimul_producer: null pointer");
    B200PF_REQUIRE(rows > 0 && n > 0 && rows <= n, B200PF_ERR_INVALID, "trimul_producer: bad rows/n");
    const int cols = incoming ? rows : n, prow = incoming ? n : rows;
    B200PF_REQUIRE(pitch % 8 == 0 && pitch >= cols, B200PF_ERR_INVALID, "trimul_producer: bad pitch");
    B200PF_REQUIRE(aligned16(z) && aligned16(w_pg), B200PF_ERR_INVALID, "trimul_producer: pointers must be 16-byte aligned");
    r512::Args a{};
    a.z = z; a.mask = mask; a.w = (const __nv_bfloat16*)w_pg; a.ln_gamma = ln_gamma; a.ln_beta = ln_beta;
    const b200pf_plane_out* outs[2] = {a_out, b_out};
    for (int i = 0; i < 2; ++i) {
        const b200pf_plane_out* o = outs[i];
        const int rg = o->row_group > 0 ? o->row_group : prow;
        B200PF_REQUIRE(o->plane_stride % 8 == 0 && o->plane_stride >= (long long)pitch * (rg < prow ? rg : prow),
                       B200PF_ERR_INVALID, "trimul_producer: bad plane stride");
        B200PF_REQUIRE(rg >= prow || (o->group_stride % 8 == 0 && o->group_stride > 0), B200PF_ERR_INVALID,
                       "trimul_producer: bad group stride");
        B200PF_REQUIRE(aligned16(o->ptr), B200PF_ERR_INVALID, "trimul_producer: planes must be 16-byte aligned");
        a.planes[i] = (__nv_bfloat16*)o->ptr; a.plane_stride[i] = o->plane_stride;
        a.group_stride[i] = o->group_stride; a.row_group[i] = rg;
    }
    a.pitch = pitch; a.rows = rows; a.n = n; a.transposed = incoming;
    return r512::launch_trimul(a, (cudaStream_t)stream);
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
