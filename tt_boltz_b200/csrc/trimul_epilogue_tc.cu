// Triangle-multiplication epilogue on tcgen05:
//   z += (LN_out(x) W_pout^T) * sigmoid(LN_in(z) W_gout^T)        per tile of 128 positions of one row.
//
// x arrives as channel-major planes x[d][row][pos].  A TMA load brings the [128 d][128 pos] block in
// as it lies (d rows, positions contiguous), which is exactly an MN-major A operand, so the first
// GEMM runs on the RAW x with W' = 0.5 * W_pout * gamma_out and the LayerNorm over d is applied
// afterwards per position:  p' = rstd * (acc - mean * wsum[c]) + wb[c],  wsum[c] = sum_d W'[c][d],
// wb = 0.5 * W_pout beta_out.  mean / rstd over d are taken from the same tile in shared memory.
// The gate GEMM uses LN_in(z) (affine applied by the loader warps) against 0.5 * W_gout, so that
// p * sigmoid(g) = p' + p' * tanh(g').  The fp32 update leaves through TMA reduce-add straight
// into z: the kernel never reads z for the residual.
// Roles (416 threads): warps 0-3 loaders (LN of z rows, x statistics, TMA issue), warp 4 MMA issuer,
// warps 5-12 epilogue.
#include "rowtc.cuh"
#include "tmap.cuh"

namespace b200pf {
namespace tme {

using namespace rtc;

constexpr int LOAD_WARPS = 4, MMA_WARP = 4, EPI_WARP0 = 5, EPI_WARPS = 8, THREADS = 13 * 32;
constexpr int W_TILE = 128 * 128 * 2;                    // 32 KB: two k-blocks of [128][128 B]
constexpr int OFF_WP = 0, OFF_WG = W_TILE;
constexpr int OFF_AZ = 2 * W_TILE;                       // 2 stages
constexpr int OFF_XT = OFF_AZ + 2 * A_TILE_BYTES;        // 1 stage: 2 boxes of [128 d][64 pos]
constexpr int XT_BOX = 128 * 128;
constexpr int OFF_STG = OFF_XT + 2 * XT_BOX;             // staging: 2 boxes of [128 pos][32 fp32], 128-byte swizzle
constexpr int STG_BOX = 128 * 128, STG_BUF = 2 * STG_BOX;
constexpr int OFF_CONST = OFF_STG + STG_BUF;             // wsum[128], wb[128] fp32
constexpr int OFF_STATS = OFF_CONST + 1024;              // [2][128] float2 (mean, rstd)
constexpr int OFF_BAR = OFF_STATS + 2048;
constexpr int SMEM_BYTES = OFF_BAR + 128;                // 199,808; the dynamic window must start 1024-byte aligned
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr int EPI_BAR_ID = 1;

struct Args {
    const float* z;                 // read for LN_in; the residual is added by TMA reduce
    const float* ln_in_gamma;
    const float* ln_in_beta;
    const __nv_bfloat16* w_pout;    // [128][128] = 0.5 * W_pout * gamma_out
    const __nv_bfloat16* w_gout;    // [128][128] = 0.5 * W_gout
    const float* wsum;              // [128] row sums of w_pout (as stored in bf16)
    const float* wb;                // [128] 0.5 * W_pout beta_out
    int rows, n;
};

struct Bars {
    uint64_t x_full, x_empty, in_full[2], in_empty[2], acc_full[2], acc_empty[2];
    uint32_t tmem_slot;
    int abort_flag;
};

// MN-major A operand: rows of the tile are K (d), 64 positions (128 bytes) per row, 128-byte swizzle;
// the two 64-position boxes are XT_BOX bytes apart (leading offset), 8-row K groups 1024 bytes (stride offset).
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(XT_BOX >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ float tanh_approx(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}

__global__ void __launch_bounds__(THREADS, 1)
trimul_epilogue_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_z, Args p,
                          unsigned int* status) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicOr(status, DEV_STATUS_BAD_INDEX);
        return;
    }
    Bars* B = reinterpret_cast<Bars*>(smem + OFF_BAR);
    volatile int* abort_flag = &B->abort_flag;
    float* wsum_s = reinterpret_cast<float*>(smem + OFF_CONST);
    float* wb_s = wsum_s + 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int tpl = (p.n + TM - 1) / TM;
    const long long tiles = (long long)p.rows * tpl;

    if (tid == 0) {
        mbar_init(&B->x_full, 1);
        mbar_init(&B->x_empty, 1 + EPI_WARPS);      // the MMAs and the epilogue warps' statistics pass both read the x tile
        for (int i = 0; i < 2; ++i) {
            mbar_init(&B->in_full[i], LOAD_WARPS); mbar_init(&B->in_empty[i], 1);
            mbar_init(&B->acc_full[i], 1); mbar_init(&B->acc_empty[i], EPI_WARPS);
        }
        B->abort_flag = 0;
        fence_barrier_init();
    }
    load_weights_sw128(smem + OFF_WP, p.w_pout, 128, tid, THREADS);
    load_weights_sw128(smem + OFF_WG, p.w_gout, 128, tid, THREADS);
    if (tid < 128) { wsum_s[tid] = p.wsum[tid]; wb_s[tid] = p.wb[tid]; }
    fence_proxy_async();
    if (warp == MMA_WARP) { tmem_alloc(&B->tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = B->tmem_slot;

    if (warp < LOAD_WARPS) {
        // ---------------------------- loaders ----------------------------
        const int sub = lane & 7, rq = lane >> 3;
        float4 gam[4], bet[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            gam[j] = __ldg(reinterpret_cast<const float4*>(p.ln_in_gamma) + j * 8 + sub);
            bet[j] = __ldg(reinterpret_cast<const float4*>(p.ln_in_beta) + j * 8 + sub);
        }
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const int r = (int)(t / tpl), pos0 = (int)(t % tpl) * TM;
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait(&B->in_empty[stage], ph ^ 1, abort_flag) && mbar_wait(&B->acc_empty[stage], ph ^ 1, abort_flag);
            if (!ok) break;
            uint8_t* a_tile = smem + OFF_AZ + stage * A_TILE_BYTES;
            {   // ask L2 for this warp's 32 rows of the NEXT tile (one lane per row, four 128-byte lines)
                const long long tn = t + gridDim.x;
                const int posn = (int)(tn % tpl) * TM + warp * 32 + lane;
                if (tn < tiles && posn < p.n) {
                    const char* rowp = reinterpret_cast<const char*>(p.z + ((tn / tpl) * p.n + posn) * KC);
#pragma unroll
                    for (int j = 0; j < 4; ++j) asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + j * 128));
                }
            }
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
                const int row0 = warp * 32 + pass * 16;
                float4 v[4][4];
                bool valid[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int pos = pos0 + row0 + i * 4 + rq;
                    valid[i] = pos < p.n;
                    const float4* src = reinterpret_cast<const float4*>(p.z + ((long long)r * p.n + (valid[i] ? pos : 0)) * KC);
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[i][j] = valid[i] ? __ldg(src + j * 8 + sub) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                if (pass == 0 && warp == 0 && lane == 0) {
                    // x tile of this tile: the buffer is free once the MMAs of the previous tile are done
                    ok = mbar_wait(&B->x_empty, (it & 1) ^ 1, abort_flag);
                    if (ok) {
                        mbar_arrive_expect_tx(&B->x_full, 2 * XT_BOX);
                        tma_load_4d(smem + OFF_XT, &map_x, &B->x_full, pos0, r, 0, 0);
                        tma_load_4d(smem + OFF_XT + XT_BOX, &map_x, &B->x_full, pos0 + 64, r, 0, 0);
                    }
                }
                // the four rows of a pass stage by stage (sums, shuffles, variance, ...): instruction-level parallelism
                // for a warp that has its scheduler almost to itself
                float s4[4], ss4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) s += (v[i][j].x + v[i][j].y) + (v[i][j].z + v[i][j].w);
                    s4[i] = s;
                }
#pragma unroll
                for (int step = 1; step < 8; step <<= 1)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s4[i] += __shfl_xor_sync(0xffffffffu, s4[i], step);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float mean = s4[i] * (1.f / KC);
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[i][j].x -= mean; v[i][j].y -= mean; v[i][j].z -= mean; v[i][j].w -= mean;
                        ss += (v[i][j].x * v[i][j].x + v[i][j].y * v[i][j].y) + (v[i][j].z * v[i][j].z + v[i][j].w * v[i][j].w);
                    }
                    ss4[i] = ss;
                }
#pragma unroll
                for (int step = 1; step < 8; step <<= 1)
#pragma unroll
                    for (int i = 0; i < 4; ++i) ss4[i] += __shfl_xor_sync(0xffffffffu, ss4[i], step);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = row0 + i * 4 + rq;
                    const float rstd = rsqrtf(ss4[i] * (1.f / KC) + LN_EPS);
                    const float kz = valid[i] ? 1.f : 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint2 o;
                        o.x = pack_bf16x2(fmaf(v[i][j].x * rstd, gam[j].x, bet[j].x) * kz, fmaf(v[i][j].y * rstd, gam[j].y, bet[j].y) * kz);
                        o.y = pack_bf16x2(fmaf(v[i][j].z * rstd, gam[j].z, bet[j].z) * kz, fmaf(v[i][j].w * rstd, gam[j].w, bet[j].w) * kz);
                        const int chunk = (j & 1) * 4 + (sub >> 1);
                        *reinterpret_cast<uint2*>(a_tile + (j >> 1) * A_KB_BYTES + sw128(row, chunk) + (sub & 1) * 8) = o;
                    }
                }
            }
            if (warp == 0) ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;     // lane 0 waited for the x buffer
            if (!ok) break;
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->in_full[stage]);
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else if (warp == MMA_WARP) {
        // ---------------------------- MMA issuer ----------------------------
        // The whole warp runs the loop and waits; one elected lane issues (see sm100::elect_one).
        constexpr uint32_t idesc_g = make_idesc_bf16(TM, 128);
        constexpr uint32_t idesc_p = make_idesc_bf16(TM, 128) | (1u << 15);      // A operand MN-major
        const uint32_t wp_addr = smem_u32(smem + OFF_WP), wg_addr = smem_u32(smem + OFF_WG), xt_addr = smem_u32(smem + OFF_XT);
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait_warp(&B->in_full[stage], ph, abort_flag) && mbar_wait_warp(&B->x_full, it & 1, abort_flag) &&
                 mbar_wait_warp(&B->acc_empty[stage], ph ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t az_addr = smem_u32(smem + OFF_AZ + stage * A_TILE_BYTES);
                const uint32_t d = tmem_base + stage * 256;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)      // D_p = x^T-tile (MN-major, 16 d rows per step) * W_pout'^T
                    umma_bf16(d, desc_mn_sw128(xt_addr + ks * 2048), make_desc_k_sw128(wp_addr + (ks >> 2) * (128 * 128) + (ks & 3) * 32),
                              idesc_p, ks ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)      // D_g = LN_in(z) tile * W_gout'^T
                    umma_bf16(d + 128, make_desc_k_sw128(az_addr + (ks >> 2) * A_KB_BYTES + (ks & 3) * 32),
                              make_desc_k_sw128(wg_addr + (ks >> 2) * (128 * 128) + (ks & 3) * 32), idesc_g, ks ? 1u : 0u);
                umma_commit(&B->in_empty[stage]);
                umma_commit(&B->x_empty);
                umma_commit(&B->acc_full[stage]);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else {
        // ---------------------------- epilogue ----------------------------
        const int quarter = warp & 3, chalf = (warp - EPI_WARP0) >> 2;
        const int epi_tid = threadIdx.x - EPI_WARP0 * 32;
        const int lrow = quarter * 32 + lane;                     // position inside the tile
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        uint32_t it = 0, round = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const int r = (int)(t / tpl), pos0 = (int)(t % tpl) * TM;
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            // LayerNorm statistics over the 128 channels of the raw x tile for this thread's position (both warps of a
            // lane quarter compute them; it is cheaper here than on the four loader warps, which bound the kernel)
            ok = mbar_wait(&B->x_full, it & 1, abort_flag);
            if (!ok) break;
            float2 st;
            {
                const uint8_t* col = smem + OFF_XT + (lrow >> 6) * XT_BOX + (lrow & 7) * 2;
                const int pchunk = (lrow & 63) >> 3;
                float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll 8
                for (int d = 0; d < 128; d += 2) {
                    const float xa = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(col + d * 128 + ((pchunk ^ (d & 7)) << 4)));
                    const float xb = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(col + (d + 1) * 128 + ((pchunk ^ ((d + 1) & 7)) << 4)));
                    s0 += xa; q0 = fmaf(xa, xa, q0);
                    s1 += xb; q1 = fmaf(xb, xb, q1);
                }
                const float mean = (s0 + s1) * (1.f / KC);
                const float var = fmaxf((q0 + q1) * (1.f / KC) - mean * mean, 0.f);
                st = make_float2(mean, rsqrtf(var + LN_EPS));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->x_empty);
            ok = mbar_wait(&B->acc_full[stage], ph, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tbase = tmem_base + lane_off + stage * 256;
#pragma unroll 1
            for (int rd = 0; rd < 2; ++rd, ++round) {
                const int c0 = rd * 64 + chalf * 32;
                uint32_t pr[32], gr[32];
                tmem_ld_32x32(tbase + c0, pr);
                tmem_ld_32x32(tbase + 128 + c0, gr);
                tmem_ld_wait();
                float4 o[8];
                float* of = reinterpret_cast<float*>(o);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    float ph2 = fmaf(st.y, fmaf(-st.x, wsum_s[c0 + e], __uint_as_float(pr[e])), wb_s[c0 + e]);
                    of[e] = fmaf(ph2, tanh_approx(__uint_as_float(gr[e])), ph2);
                }
                uint8_t* stg = smem + OFF_STG;
                if (epi_tid == 0) bulk_wait_read0();               // the previous round's reduce has read the staging tile
                named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
#pragma unroll
                for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(stg + chalf * STG_BOX + sw128(lrow, j)) = o[j];
                fence_proxy_async();
                named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
                if (epi_tid == 0) {
                    tma_reduce_add_4d(&map_z, stg, rd * 64, pos0, r, 0);
                    tma_reduce_add_4d(&map_z, stg + STG_BOX, rd * 64 + 32, pos0, r, 0);
                    bulk_commit();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->acc_empty[stage]);
        }
        if (epi_tid == 0) bulk_wait0();
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace tme
}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_trimul_epilogue_tc(float* z, const b200pf_bf16* x, long long x_plane_stride, int x_pitch,
                                         const float* ln_in_gamma, const float* ln_in_beta,
                                         const b200pf_bf16* w_pout, const b200pf_bf16* w_gout,
                                         const float* wsum, const float* wb, int rows, int n, void* stream) {
    using namespace tme;
    B200PF_REQUIRE(z && x && ln_in_gamma && ln_in_beta && w_pout && w_gout && wsum && wb, B200PF_ERR_INVALID,
                   "trimul_epilogue_tc: null pointer");
    B200PF_REQUIRE(rows > 0 && n > 0 && x_pitch % 8 == 0 && x_pitch >= n && x_plane_stride % 8 == 0 &&
                   x_plane_stride >= (long long)x_pitch * rows, B200PF_ERR_INVALID, "trimul_epilogue_tc: bad sizes");
    B200PF_REQUIRE(aligned16(z) && aligned16(x) && aligned16(w_pout) && aligned16(w_gout) && aligned16(ln_in_gamma) &&
                   aligned16(ln_in_beta), B200PF_ERR_INVALID, "trimul_epilogue_tc: pointers must be 16-byte aligned");
    CUtensorMap mx, mz;
    int rc;
    {
        cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)rows, 128, 1};
        cuuint64_t str[3] = {(cuuint64_t)x_pitch * 2, (cuuint64_t)x_plane_stride * 2, (cuuint64_t)x_plane_stride * 2 * 128};
        cuuint32_t box[4] = {64, 1, 128, 1};
        if ((rc = tmap_encode(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "x")) != B200PF_OK) return rc;
    }
    {
        cuuint64_t dims[4] = {128, (cuuint64_t)n, (cuuint64_t)rows, 1};
        cuuint64_t str[3] = {512, (cuuint64_t)n * 512, (cuuint64_t)n * 512 * rows};
        cuuint32_t box[4] = {32, 128, 1, 1};
        if ((rc = tmap_encode(&mz, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, z, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "z")) != B200PF_OK) return rc;
    }
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "trimul_epilogue_tc: no device status word");
    B200PF_SMEM_ATTR_ONCE(trimul_epilogue_tc_kernel, SMEM_BYTES);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long tiles = (long long)rows * ((n + TM - 1) / TM);
    Args a{z, ln_in_gamma, ln_in_beta, (const __nv_bfloat16*)w_pout, (const __nv_bfloat16*)w_gout, wsum, wb, rows, n};
    trimul_epilogue_tc_kernel<<<(unsigned)(tiles < sms ? tiles : sms), THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(mx, mz, a, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
