// Pair transition on tcgen05:  z += W3( silu(W1 LN(z)) * (W2 LN(z)) )  per tile of 128 positions.
//
// The 512-wide hidden layer is walked in 8 chunks of 64 channels.  Per chunk c:
//   GEMM1  D1[c&1] (128 x 128 fp32, TMEM) = A (LN(z) tile, smem) x [fc1 rows | fc2 rows of the chunk]^T
//   epilogue-1 (8 warps, thread = position)  h = silu(f1) * f2 -> packed bf16 pairs -> TMEM (tcgen05.st)
//   GEMM2  D2 (128 x 128 fp32, TMEM) += h (A operand read from TMEM) x W3[:, chunk]^T
// D1 is double buffered, so GEMM1 of chunk c+1 runs while epilogue-1 works on chunk c; the hidden
// activations never leave the SM (they do not even touch shared memory).  After the last chunk the
// update leaves through TMA reduce-add into z.  silu uses one MUFU: the host halves fc1, so with
// a = f1/2:  silu(f1) = a + a*tanh(a).
// Weights (384 KB bf16) do not fit in shared memory: a dedicated warp streams the chunk pair
// (32 KB + 16 KB) from L2 with TMA through a three-stage ring.
// Roles (448 threads): warps 0-3 LayerNorm loaders, warp 4 MMA issuer, warp 5 weight TMA, warps 6-13 epilogue.
#include "rowtc.cuh"
#include "tmap.cuh"

namespace b200pf {
namespace trz {

using namespace rtc;

constexpr int LOAD_WARPS = 4, MMA_WARP = 4, TMA_WARP = 5, EPI_WARP0 = 6, EPI_WARPS = 8, THREADS = 14 * 32;
constexpr int CHUNKS = 8;
constexpr int W12_BYTES = 128 * 128 * 2;                  // [128 rows][128 K]: two k-blocks of 16 KB
constexpr int W3_BYTES = 128 * 64 * 2;                    // [128 out][64 hidden]
constexpr int WSTAGE = W12_BYTES + W3_BYTES;              // 49,152
constexpr int OFF_W = 0;                                  // 2 stages
constexpr int WSTAGES = 3;                                // the weight stream comes from L2 for every tile: the MMA
                                                          // issuer waited ~6.4 k clocks per tile on it with 2 stages
constexpr int OFF_A = WSTAGES * WSTAGE;                   // 2 stages x 32 KB
constexpr int OFF_STG = OFF_A + 2 * A_TILE_BYTES;         // staging: one box of [128 pos][32 fp32]
constexpr int STG_BOX = 128 * 128;
constexpr int OFF_BAR = OFF_STG + STG_BOX;
constexpr int SMEM_BYTES = OFF_BAR + 256;                 // 229,632
constexpr int EPI_BAR_ID = 1;
// TMEM columns
constexpr uint32_t COL_D1 = 0, COL_D2 = 256, COL_H = 384;

struct Args {
    const float* z;
    const float* ln_gamma;
    const float* ln_beta;
    long long rows_flat;
};

struct Bars {
    uint64_t w_full[WSTAGES], w_empty[WSTAGES], a_full[2], a_empty[2], d1_full[2], h_full[2], d2_full, d2_empty;
    uint32_t tmem_slot;
    int abort_flag;
};

__device__ __forceinline__ float tanh_approx(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
transition_tc_kernel(const __grid_constant__ CUtensorMap map_w12, const __grid_constant__ CUtensorMap map_w3,
                     const __grid_constant__ CUtensorMap map_z, Args p, unsigned int* status) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicOr(status, DEV_STATUS_BAD_INDEX);
        return;
    }
    Bars* B = reinterpret_cast<Bars*>(smem + OFF_BAR);
    volatile int* abort_flag = &B->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const long long tiles = (p.rows_flat + TM - 1) / TM;

    if (tid == 0) {
        for (int i = 0; i < WSTAGES; ++i) { mbar_init(&B->w_full[i], 1); mbar_init(&B->w_empty[i], 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&B->a_full[i], LOAD_WARPS); mbar_init(&B->a_empty[i], 1);
            mbar_init(&B->d1_full[i], 1); mbar_init(&B->h_full[i], EPI_WARPS);
        }
        mbar_init(&B->d2_full, 1);
        mbar_init(&B->d2_empty, EPI_WARPS);
        B->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == MMA_WARP) { tmem_alloc(&B->tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = B->tmem_slot;

    if (warp < LOAD_WARPS) {
        // ---------------------------- LayerNorm loaders ----------------------------
        const int sub = lane & 7, rq = lane >> 3;
        float4 gam[4], bet[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            gam[j] = __ldg(reinterpret_cast<const float4*>(p.ln_gamma) + j * 8 + sub);
            bet[j] = __ldg(reinterpret_cast<const float4*>(p.ln_beta) + j * 8 + sub);
        }
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const long long base = t * TM;
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait(&B->a_empty[stage], ph ^ 1, abort_flag);
            if (!ok) break;
            uint8_t* a_tile = smem + OFF_A + stage * A_TILE_BYTES;
            {   // ask L2 for this warp's 32 rows of the NEXT tile (one lane per row, four 128-byte lines)
                const long long fn = (t + gridDim.x) * TM + warp * 32 + lane;
                if (t + gridDim.x < tiles && fn < p.rows_flat) {
                    const char* rowp = reinterpret_cast<const char*>(p.z + fn * KC);
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
                    const long long f = base + row0 + i * 4 + rq;
                    valid[i] = f < p.rows_flat;
                    const float4* src = reinterpret_cast<const float4*>(p.z + (valid[i] ? f : 0) * KC);
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[i][j] = valid[i] ? __ldg(src + j * 8 + sub) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = row0 + i * 4 + rq;
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) s += (v[i][j].x + v[i][j].y) + (v[i][j].z + v[i][j].w);
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    const float mean = s * (1.f / KC);
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[i][j].x -= mean; v[i][j].y -= mean; v[i][j].z -= mean; v[i][j].w -= mean;
                        ss += (v[i][j].x * v[i][j].x + v[i][j].y * v[i][j].y) + (v[i][j].z * v[i][j].z + v[i][j].w * v[i][j].w);
                    }
                    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                    const float rstd = rsqrtf(ss * (1.f / KC) + LN_EPS);
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
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->a_full[stage]);
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else if (warp == TMA_WARP) {
        if (lane == 0) {
            // ---------------------------- weight TMA ----------------------------
            uint32_t g = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                for (int c = 0; c < CHUNKS; ++c, ++g) {
                    const uint32_t stage = g % WSTAGES, ph = (g / WSTAGES) & 1;
                    ok = mbar_wait(&B->w_empty[stage], ph ^ 1, abort_flag);
                    if (!ok) break;
                    uint8_t* ws = smem + OFF_W + stage * WSTAGE;
                    mbar_arrive_expect_tx(&B->w_full[stage], WSTAGE);
                    tma_load_3d(ws, &map_w12, &B->w_full[stage], 0, 0, c);
                    tma_load_3d(ws + 128 * 128, &map_w12, &B->w_full[stage], 64, 0, c);
                    tma_load_3d(ws + W12_BYTES, &map_w3, &B->w_full[stage], 0, 0, c);
                }
            }
            if (!ok) {
                atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
                uint64_t t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------------------- MMA issuer ----------------------------
        // The whole warp runs the loop and waits; one elected lane issues (see sm100::elect_one).
        constexpr uint32_t idesc = make_idesc_bf16(TM, 128);
        uint32_t it = 0, g = 0, h_cnt[2] = {0, 0};
        bool ok = true;
        // descriptors are a precomputed base plus constants (the address field counts 16-byte units)
        const uint64_t d_a0 = make_desc_k_sw128(smem_u32(smem + OFF_A));
        const uint64_t d_w0 = make_desc_k_sw128(smem_u32(smem + OFF_W));
        const uint64_t d_w3_0 = make_desc_k_sw128(smem_u32(smem + OFF_W + W12_BYTES));
        auto gemm1 = [&](uint32_t a_stage, uint32_t w_stage, uint32_t buf, bool release_a) {
            if (elect_one()) {
                const uint64_t da = d_a0 + a_stage * (uint64_t)(A_TILE_BYTES >> 4), dw = d_w0 + w_stage * (uint64_t)(WSTAGE >> 4);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_bf16(tmem_base + COL_D1 + buf * 128, da + (ks >> 2) * (A_KB_BYTES >> 4) + (ks & 3) * 2,
                              dw + (ks >> 2) * ((128 * 128) >> 4) + (ks & 3) * 2, idesc, ks ? 1u : 0u);
                umma_commit(&B->d1_full[buf]);
                if (release_a) umma_commit(&B->a_empty[a_stage]);    // all GEMM1 of this tile issued: the A tile is free once they finish
            }
            __syncwarp();
        };
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait_warp(&B->a_full[stage], ph, abort_flag) && mbar_wait_warp(&B->w_full[g % WSTAGES], (g / WSTAGES) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            gemm1(stage, g % WSTAGES, 0, CHUNKS == 1);
            for (int c = 0; c < CHUNKS && ok; ++c, ++g) {
                const uint32_t buf = c & 1, ws = g % WSTAGES;
                if (c + 1 < CHUNKS) {
                    const uint32_t g1 = g + 1;
                    ok = mbar_wait_warp(&B->w_full[g1 % WSTAGES], (g1 / WSTAGES) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    gemm1(stage, g1 % WSTAGES, buf ^ 1, c + 2 == CHUNKS);
                }
                ok = mbar_wait_warp(&B->h_full[buf], h_cnt[buf] & 1, abort_flag);
                if (!ok) break;
                ++h_cnt[buf];
                if (c == 0) {                                // D2 of the previous tile has been read out
                    ok = mbar_wait_warp(&B->d2_empty, (it & 1) ^ 1, abort_flag);
                    if (!ok) break;
                }
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t dw3 = d_w3_0 + ws * (uint64_t)(WSTAGE >> 4);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)               // 64 hidden = 4 k-steps; h: 8 TMEM columns per step
                        umma_bf16_ts(tmem_base + COL_D2, tmem_base + COL_H + buf * 32 + kk * 8, dw3 + kk * 2, idesc, (c | kk) ? 1u : 0u);
                    umma_commit(&B->w_empty[ws]);
                    if (c + 1 == CHUNKS) umma_commit(&B->d2_full);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else {
        // ---------------------------- epilogue ----------------------------
        const int quarter = warp & 3, eh = (warp - EPI_WARP0) >> 2;
        const int epi_tid = threadIdx.x - EPI_WARP0 * 32;
        const int lrow = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        uint32_t it = 0, d1_cnt[2] = {0, 0};
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            for (int c = 0; c < CHUNKS && ok; ++c) {
                const uint32_t buf = c & 1;
                ok = mbar_wait(&B->d1_full[buf], d1_cnt[buf] & 1, abort_flag);
                if (!ok) break;
                ++d1_cnt[buf];
                tc_fence_after();
                // this warp: hidden channels 32*eh .. +31 of the chunk: f1 at columns [32 eh, +32), f2 at [64 + 32 eh, +32)
                uint32_t f1[32], f2[32];
                tmem_ld_32x32(tmem_base + lane_off + COL_D1 + buf * 128 + eh * 32, f1);
                tmem_ld_32x32(tmem_base + lane_off + COL_D1 + buf * 128 + 64 + eh * 32, f2);
                tmem_ld_wait();
                uint32_t hw[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float a0 = __uint_as_float(f1[2 * e]), a1 = __uint_as_float(f1[2 * e + 1]);
                    float h0 = fmaf(a0, tanh_approx(a0), a0) * __uint_as_float(f2[2 * e]);
                    float h1 = fmaf(a1, tanh_approx(a1), a1) * __uint_as_float(f2[2 * e + 1]);
                    hw[e] = pack_bf16x2(h0, h1);
                }
                tmem_st_x16(tmem_base + lane_off + COL_H + buf * 32 + eh * 16, hw);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B->h_full[buf]);
            }
            if (!ok) break;
            // update: D2 -> fp32 staging -> TMA reduce-add into z; this warp: output channels 64*eh .. +63
            ok = mbar_wait(&B->d2_full, it & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t d[2][32];
            tmem_ld_32x32(tmem_base + lane_off + COL_D2 + eh * 64, d[0]);
            tmem_ld_32x32(tmem_base + lane_off + COL_D2 + eh * 64 + 32, d[1]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->d2_empty);
            const long long base = t * TM;
#pragma unroll
            for (int rd = 0; rd < 4; ++rd) {
                // round rd stores channels [32 rd, +32): they are held by the warps with eh == rd / 2 (register half rd % 2)
                if (epi_tid == 0) bulk_wait_read0();
                named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
                if (eh == (rd >> 1)) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 v = make_uint4(d[rd & 1][4 * j], d[rd & 1][4 * j + 1], d[rd & 1][4 * j + 2], d[rd & 1][4 * j + 3]);
                        *reinterpret_cast<uint4*>(smem + OFF_STG + sw128(lrow, j)) = v;
                    }
                }
                fence_proxy_async();
                named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
                if (epi_tid == 0) {
                    tma_reduce_add_4d(&map_z, smem + OFF_STG, rd * 32, (int)(base & 0x7fffffff), 0, 0);
                    bulk_commit();
                }
            }
        }
        if (epi_tid == 0) bulk_wait0();
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace trz
}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_transition_z_tc(float* z, const float* ln_gamma, const float* ln_beta,
                                      const b200pf_bf16* w12, const b200pf_bf16* w3, long long n_rows_flat, void* stream) {
    using namespace trz;
    B200PF_REQUIRE(z && ln_gamma && ln_beta && w12 && w3 && n_rows_flat > 0, B200PF_ERR_INVALID, "transition_z_tc: bad argument");
    B200PF_REQUIRE(n_rows_flat < (1ll << 31), B200PF_ERR_UNSUPPORTED, "transition_z_tc: too many rows");
    B200PF_REQUIRE(aligned16(z) && aligned16(w12) && aligned16(w3) && aligned16(ln_gamma) && aligned16(ln_beta),
                   B200PF_ERR_INVALID, "transition_z_tc: pointers must be 16-byte aligned");
    CUtensorMap m12, m3, mz;
    int rc;
    {
        cuuint64_t dims[3] = {128, 128, CHUNKS};
        cuuint64_t str[2] = {256, 128 * 256};
        cuuint32_t box[3] = {64, 128, 1};
        if ((rc = tmap_encode(&m12, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, w12, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "w12")) != B200PF_OK) return rc;
    }
    {
        cuuint64_t dims[3] = {64, 128, CHUNKS};
        cuuint64_t str[2] = {128, 128 * 128};
        cuuint32_t box[3] = {64, 128, 1};
        if ((rc = tmap_encode(&m3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, w3, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "w3")) != B200PF_OK) return rc;
    }
    {
        cuuint64_t dims[4] = {128, (cuuint64_t)n_rows_flat, 1, 1};
        cuuint64_t str[3] = {512, (cuuint64_t)n_rows_flat * 512, (cuuint64_t)n_rows_flat * 512};
        cuuint32_t box[4] = {32, 128, 1, 1};
        if ((rc = tmap_encode(&mz, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, z, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "z")) != B200PF_OK) return rc;
    }
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "transition_z_tc: no device status word");
    B200PF_SMEM_ATTR_ONCE(transition_tc_kernel, SMEM_BYTES);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long tiles = (n_rows_flat + TM - 1) / TM;
    Args a{z, ln_gamma, ln_beta, n_rows_flat};
    transition_tc_kernel<<<(unsigned)(tiles < sms ? tiles : sms), THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(m12, m3, mz, a, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
