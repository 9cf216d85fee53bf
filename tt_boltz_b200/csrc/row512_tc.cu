// The two "128 -> 512" producers on tcgen05: LayerNorm (with its affine) -> GEMMs of one tile of 128
// pair positions against 512 weight rows kept in shared memory -> thin epilogue out of TMEM.
//
// The orientation of each GEMM is chosen so that the epilogue thread already holds the values
// in the order they are stored, and nothing is transposed through shared memory:
//   MODE_TRIMUL : D[channel][position] = W x^T for the four groups p_a, g_a, p_b, g_b (M = 128
//                 channels, N = 128 positions): thread = channel, 32 consecutive positions per
//                 tcgen05.ld = 64 contiguous bytes of a plane row.  u = p*sigmoid(g) costs one
//                 MUFU and one FMA per element: the host halves W_p and W_g, so with
//                 p' = p/2, t = tanh(g/2):  p*sigmoid(g) = p' + p'*t.  Masked / out-of-range
//                 positions are zero rows of x, which makes p' (and u) exactly zero.
//   MODE_TRIATT : D[position][q|k] = x W^T and D[position][g] = x W_g^T (thread = position:
//                 64-byte head rows and z-layout gate rows), D[v-channel][position] = W_v x^T
//                 (thread = channel: rows of the transposed V).  The 4 triangle-bias heads are
//                 dotted by the epilogue warps (fp32 weights and accumulation) from the normalised
//                 bf16 rows of the A tile: on the loader warps, one per scheduler, the same work
//                 doubled the time of the whole kernel.
// Output goes TMEM -> registers -> a swizzled staging tile -> TMA stores, so that global memory
// only ever sees full, contiguous lines (thread-per-row 16-byte stores were 3x slower).
// Roles (416 threads): warps 0-3 LayerNorm loaders (32 rows each), warp 4 MMA issuer, warps 5-12
// epilogue (two warps per TMEM lane quarter, each taking half of the columns).  TMEM is used as
// two halves of 256 columns so the epilogue of one half overlaps the MMAs of the next, and the x
// tile is double buffered so the loaders run a tile ahead.
#include "mxfp8.cuh"
#include "row512_tc.h"
#include "rowtc.cuh"
#include "tmap.cuh"

namespace b200pf {
namespace r512 {

using namespace rtc;

constexpr int MODE_TRIMUL = 0, MODE_TRIATT = 1, MODE_TRIMUL_MX = 2;   // MX: e4m3 planes + e8m0 scales (mxfp8.cuh)
constexpr int LOAD_WARPS = 4, MMA_WARP = 4, EPI_WARP0 = 5, EPI_WARPS = 8, THREADS = 13 * 32;
constexpr int W_BYTES = 512 * 128 * 2;                 // two k-blocks of [512][128 B]
constexpr int W_KB = 512 * 128;
constexpr int OFF_A = W_BYTES;                          // 2 stages x 32 KB
constexpr int OFF_STG = OFF_A + 2 * A_TILE_BYTES;       // output staging: 2 boxes of [128 rows][128 B], 128-byte swizzle
constexpr int STG_BOX = 128 * 128;
constexpr int OFF_WB = OFF_STG + 2 * STG_BOX;           // triangle-bias rows [4][128] fp32
constexpr int OFF_BAR = OFF_WB + 4 * 128 * 4;
constexpr int SMEM_BYTES = OFF_BAR + 128;               // 231,552: the dynamic window must start 1024-byte aligned
constexpr int EPI_BAR_ID = 1;

struct Bars {
    uint64_t a_full[2], a_empty[2], acc_full[2], acc_empty[2];
    uint32_t tmem_slot;
    int abort_flag;
};

// D[tmem] = A (M = 128 rows) * B^T over K = 128: two k-blocks of 64, each four K = 16 steps.  Operands are given as
// ready descriptors of their first k-block (address field in 16-byte units) plus the k-block distance in the same
// units: the issuing thread must not spend longer per instruction than the ~64 cycles it occupies the tensor pipe.
__device__ __forceinline__ void gemm_k128(uint32_t tmem_d, uint64_t da, uint32_t a_kb16, uint64_t db, uint32_t b_kb16, uint32_t idesc) {
    using namespace sm100;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint32_t kb = ks >> 2, kk = ks & 3;
        umma_bf16(tmem_d, da + kb * a_kb16 + kk * 2, db + kb * b_kb16 + kk * 2, idesc, ks ? 1u : 0u);
    }
}

__device__ __forceinline__ float tanh_approx(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
row512_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
              const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3, Args p, unsigned int* status) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {       // swizzled tiles need 1024-byte alignment; there is no slack to fix it up
        if (threadIdx.x == 0) atomicOr(status, DEV_STATUS_BAD_INDEX);
        return;
    }
    Bars* B = reinterpret_cast<Bars*>(smem + OFF_BAR);
    volatile int* abort_flag = &B->abort_flag;
    float* wb_s = reinterpret_cast<float*>(smem + OFF_WB);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

    const int span = p.transposed ? p.rows : p.n;                 // positions along a line
    const int n_lines = p.transposed ? p.n : p.rows;
    const int tpl = (span + TM - 1) / TM;
    const long long tiles = (long long)n_lines * tpl;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&B->a_full[i], LOAD_WARPS); mbar_init(&B->a_empty[i], MODE == MODE_TRIATT ? 1 + EPI_WARPS : 1);
            mbar_init(&B->acc_full[i], 1); mbar_init(&B->acc_empty[i], EPI_WARPS);
        }
        B->abort_flag = 0;
        fence_barrier_init();
    }
    load_weights_sw128(smem, p.w, 512, tid, THREADS);
    if (MODE == MODE_TRIATT)
        for (int i = tid; i < 4 * 128; i += THREADS) wb_s[i] = p.w_bias_f32[i];
    fence_proxy_async();
    if (warp == MMA_WARP) { tmem_alloc(&B->tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = B->tmem_slot;

    auto flat_of = [&](int line, int pos) -> long long {   // flat (r * n + c) index, or -1 outside
        if (pos >= span) return -1;
        return p.transposed ? (long long)pos * p.n + line : (long long)line * p.n + pos;
    };

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
            const int line = (int)(t / tpl), pos0 = (int)(t % tpl) * TM;
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait(&B->a_empty[stage], ph ^ 1, abort_flag);
            if (!ok) break;
            uint8_t* a_tile = smem + OFF_A + stage * A_TILE_BYTES;
            // this warp's 32 rows of the NEXT tile: one lane per row asks L2 for its four 128-byte lines, so the
            // loads of the next round find them there instead of paying the DRAM latency with only 4 warps in flight
            {
                const long long tn = t + gridDim.x;
                if (tn < tiles) {
                    const long long f = flat_of((int)(tn / tpl), (int)(tn % tpl) * TM + warp * 32 + lane);
                    if (f >= 0) {
                        if (p.z_bf16) {
                            const char* rowp = reinterpret_cast<const char*>(p.z_bf16 + f * KC);
#pragma unroll
                            for (int j = 0; j < 2; ++j) asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + j * 128));
                        } else {
                            const char* rowp = reinterpret_cast<const char*>(p.z + f * KC);
#pragma unroll
                            for (int j = 0; j < 4; ++j) asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + j * 128));
                        }
                    }
                }
            }
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
                const int row0 = warp * 32 + pass * 16;
                float4 v[4][4];
                long long fl[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    fl[i] = flat_of(line, pos0 + row0 + i * 4 + rq);
                    if (p.z_bf16) {          // warp-uniform: four bf16 channels per lane and j, widened on the fly
                        const uint2* src = reinterpret_cast<const uint2*>(p.z_bf16 + (fl[i] < 0 ? 0 : fl[i]) * KC);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint2 w = fl[i] < 0 ? make_uint2(0u, 0u) : __ldg(src + j * 8 + sub);
                            v[i][j] = make_float4(bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y));
                        }
                    } else {
                        const float4* src = reinterpret_cast<const float4*>(p.z + (fl[i] < 0 ? 0 : fl[i]) * KC);
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[i][j] = fl[i] < 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : __ldg(src + j * 8 + sub);
                    }
                }
                // The four rows of a pass are worked on stage by stage (all sums, then all shuffles, ...), not row by
                // row: one loader warp per scheduler has nothing else to hide a dependent chain behind.
                float kz[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    bool keep = fl[i] >= 0;
                    if (MODE != MODE_TRIATT) keep = keep && __ldg(p.mask + (fl[i] < 0 ? 0 : fl[i])) != 0;
                    kz[i] = keep ? 1.f : 0.f;
                }
                float s4[4];
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
                float ss4[4];
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
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[i][j].x = fmaf(v[i][j].x * rstd, gam[j].x, bet[j].x) * kz[i];
                        v[i][j].y = fmaf(v[i][j].y * rstd, gam[j].y, bet[j].y) * kz[i];
                        v[i][j].z = fmaf(v[i][j].z * rstd, gam[j].z, bet[j].z) * kz[i];
                        v[i][j].w = fmaf(v[i][j].w * rstd, gam[j].w, bet[j].w) * kz[i];
                        uint2 o;
                        o.x = pack_bf16x2(v[i][j].x, v[i][j].y);
                        o.y = pack_bf16x2(v[i][j].z, v[i][j].w);
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
    } else if (warp == MMA_WARP) {
        // ---------------------------- MMA issuer ----------------------------
        // The whole warp runs the loop and waits; one elected lane issues (see sm100::elect_one).
        constexpr uint32_t idesc128 = make_idesc_bf16(TM, 128), idesc256 = make_idesc_bf16(TM, 256);
        const uint64_t d_w = make_desc_k_sw128(smem_u32(smem));            // weight row r starts 8 r units further
        const uint64_t d_x0 = make_desc_k_sw128(smem_u32(smem + OFF_A));
        constexpr uint32_t W_KB16 = W_KB >> 4, A_KB16 = A_KB_BYTES >> 4;
        uint32_t it = 0, acc_cnt[2] = {0, 0};
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait_warp(&B->a_full[stage], ph, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t d_x = d_x0 + stage * (uint64_t)(A_TILE_BYTES >> 4);
            for (int half = 0; half < 2 && ok; ++half) {
                ok = mbar_wait_warp(&B->acc_empty[half], (acc_cnt[half] & 1) ^ 1, abort_flag);
                if (!ok) break;
                ++acc_cnt[half];
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t d = tmem_base + half * 256;
                    if (MODE != MODE_TRIATT) {
                        // channels on the lanes: A = 128 weight rows, B = the x tile (positions)
                        gemm_k128(d, d_w + (half * 256) * 8, W_KB16, d_x, A_KB16, idesc128);
                        gemm_k128(d + 128, d_w + (half * 256 + 128) * 8, W_KB16, d_x, A_KB16, idesc128);
                    } else if (half == 0) {
                        gemm_k128(d, d_x, A_KB16, d_w, W_KB16, idesc256);                          // [q | k]
                    } else {
                        gemm_k128(d, d_x, A_KB16, d_w + 256 * 8, W_KB16, idesc128);                // g
                        gemm_k128(d + 128, d_w + 384 * 8, W_KB16, d_x, A_KB16, idesc128);          // v^T
                    }
                    umma_commit(&B->acc_full[half]);
                    if (half == 1) umma_commit(&B->a_empty[stage]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else {
        // ---------------------------- epilogue ----------------------------
        // Each round moves one [128 x 128] bf16 block out: TMEM -> registers -> swizzled staging tile
        // -> two TMA stores of [128 rows x 64 elements], so global memory only sees full lines.
        const int quarter = warp & 3, chalf = (warp - EPI_WARP0) >> 2;
        const int epi_tid = threadIdx.x - EPI_WARP0 * 32;
        const int lrow = quarter * 32 + lane;                     // TMEM lane of this thread = staging row
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        uint8_t* stg = smem + OFF_STG;
        uint32_t acc_cnt = 0;
        bool ok = true;
        // tanh_mode: 0 = copy, 1 = p' + p' * tanh(g')  (gate columns at +128), 2 = 0.5 + 0.5 * tanh(x)
        auto load64 = [&](uint32_t taddr, int tanh_mode, uint4 (&o)[8]) {
            uint32_t r[2][32];
            tmem_ld_32x32(taddr, r[0]);
            tmem_ld_32x32(taddr + 32, r[1]);
            uint32_t gq[2][32];
            if (tanh_mode == 1) {
                tmem_ld_32x32(taddr + 128, gq[0]);
                tmem_ld_32x32(taddr + 160, gq[1]);
            }
            tmem_ld_wait();
            uint32_t* w = reinterpret_cast<uint32_t*>(o);
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                float v0 = __uint_as_float(r[e >> 4][(2 * e) & 31]), v1 = __uint_as_float(r[e >> 4][(2 * e + 1) & 31]);
                if (tanh_mode == 1) {
                    v0 = fmaf(v0, tanh_approx(__uint_as_float(gq[e >> 4][(2 * e) & 31])), v0);
                    v1 = fmaf(v1, tanh_approx(__uint_as_float(gq[e >> 4][(2 * e + 1) & 31])), v1);
                } else if (tanh_mode == 2) {
                    v0 = fmaf(0.5f, tanh_approx(v0), 0.5f);
                    v1 = fmaf(0.5f, tanh_approx(v1), 0.5f);
                }
                w[e] = pack_bf16x2(v0, v1);
            }
        };
        auto store_round = [&](const uint4 (&o)[8], const CUtensorMap* map, int c0, int c1, int c2, int c3) {
            if (epi_tid == 0) bulk_wait_read0();               // the previous round's stores have read the staging tile
            named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(stg + chalf * STG_BOX + sw128(lrow, j)) = o[j];
            fence_proxy_async();
            named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
            if (epi_tid == 0) {
                tma_store_4d(map, stg, c0, c1, c2, c3);
                tma_store_4d(map, stg + STG_BOX, c0 + 64, c1, c2, c3);
                bulk_commit();
            }
        };
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++acc_cnt) {
            const int line = (int)(t / tpl), pos0 = (int)(t % tpl) * TM;
            for (int half = 0; half < 2 && ok; ++half) {
                ok = mbar_wait(&B->acc_full[half], acc_cnt & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tbase = tmem_base + lane_off + half * 256;
                uint4 o[8];
                if (MODE == MODE_TRIMUL_MX) {
                    // lane = channel of operand `half`; this warp's 64 positions are two scale blocks
                    uint32_t sc = 0;
#pragma unroll
                    for (int blk = 0; blk < 2; ++blk) {
                        uint32_t pr[32], gr[32];
                        tmem_ld_32x32(tbase + chalf * 64 + blk * 32, pr);
                        tmem_ld_32x32(tbase + 128 + chalf * 64 + blk * 32, gr);
                        tmem_ld_wait();
                        float amax = 0.f;
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const float pv = __uint_as_float(pr[e]);
                            const float u = fmaf(pv, tanh_approx(__uint_as_float(gr[e])), pv);
                            pr[e] = __float_as_uint(u);
                            amax = fmaxf(amax, fabsf(u));
                        }
                        const uint32_t eb = mx::scale_byte(amax);
                        const float inv = mx::inv_scale(eb);
                        sc |= eb << (8 * blk);
                        uint32_t* w = reinterpret_cast<uint32_t*>(&o[blk * 2]);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            w[e] = mx::pack_e4m3x4(__uint_as_float(pr[4 * e]) * inv, __uint_as_float(pr[4 * e + 1]) * inv,
                                                   __uint_as_float(pr[4 * e + 2]) * inv, __uint_as_float(pr[4 * e + 3]) * inv);
                    }
                    *reinterpret_cast<uint16_t*>(p.scales[half] + mx::scale_offset(lrow, line, (pos0 >> 5) + chalf * 2,
                                                                                   p.sf_kgroups, p.sf_row_blocks)) = (uint16_t)sc;
                    if (epi_tid == 0) bulk_wait_read0();
                    named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
#pragma unroll
                    for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(stg + sw128(lrow, chalf * 4 + j)) = o[j];
                    fence_proxy_async();
                    named_bar_sync(EPI_BAR_ID, EPI_WARPS * 32);
                    if (epi_tid == 0) {
                        tma_store_4d(half == 0 ? &map0 : &map1, stg, pos0, line, 0, 0);
                        bulk_commit();
                    }
                } else if (MODE == MODE_TRIMUL) {
                    // lane = channel of operand `half`, columns = positions; this warp's 64 positions = box `chalf`
                    load64(tbase + chalf * 64, 1, o);
                    const int rg = p.row_group[half];
                    store_round(o, half == 0 ? &map0 : &map1, pos0, line % rg, 0, line / rg);
                } else if (half == 0) {
                    {   // The 4 triangle-bias heads of this tile, from the normalised bf16 rows still in the A tile (the
                        // accumulator being ready means the loaders' writes are visible): thread = position `lrow`,
                        // this warp's two heads 2 chalf, 2 chalf + 1; fp32 weights, fp32 accumulation.
                        const uint32_t stage = acc_cnt & 1;
                        const uint8_t* a_row = smem + OFF_A + stage * A_TILE_BYTES + lrow * 128;
                        const float* w0 = wb_s + (2 * chalf) * 128;
                        float b0 = 0.f, b1 = 0.f;
#pragma unroll
                        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                const uint4 xv = *reinterpret_cast<const uint4*>(a_row + kb * A_KB_BYTES + ((c ^ (lrow & 7)) << 4));
                                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    const float4 wa = *reinterpret_cast<const float4*>(w0 + kb * 64 + c * 8 + q * 4);
                                    const float4 wc = *reinterpret_cast<const float4*>(w0 + 128 + kb * 64 + c * 8 + q * 4);
                                    const float x0 = __uint_as_float(xw[2 * q] << 16), x1 = __uint_as_float(xw[2 * q] & 0xffff0000u);
                                    const float x2 = __uint_as_float(xw[2 * q + 1] << 16), x3 = __uint_as_float(xw[2 * q + 1] & 0xffff0000u);
                                    b0 = fmaf(x0, wa.x, fmaf(x1, wa.y, fmaf(x2, wa.z, fmaf(x3, wa.w, b0))));
                                    b1 = fmaf(x0, wc.x, fmaf(x1, wc.y, fmaf(x2, wc.z, fmaf(x3, wc.w, b1))));
                                }
                            }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&B->a_empty[stage]);          // the A tile may be overwritten
                        if (pos0 + lrow < span) {
                            __nv_bfloat16* bp = p.tri_bias + (long long)line * p.bias_qs + pos0 + lrow;
                            bp[(2 * chalf) * p.bias_hs] = __float2bfloat16(b0);
                            bp[(2 * chalf + 1) * p.bias_hs] = __float2bfloat16(b1);
                        }
                    }
                    // lane = position, columns = channels of q then k; box `chalf` = channels 64*chalf ..
                    load64(tbase + chalf * 64, 0, o);
                    store_round(o, &map0, 0, pos0, line, 0);
                    load64(tbase + 128 + chalf * 64, 0, o);
                    store_round(o, &map1, 0, pos0, line, 0);
                } else {
                    load64(tbase + chalf * 64, 2, o);                       // gate: sigmoid
                    if (p.transposed) store_round(o, &map2, 0, line, pos0, 0);
                    else store_round(o, &map2, 0, pos0, line, 0);
                    load64(tbase + 128 + chalf * 64, 0, o);                 // v^T: lane = v channel, columns = positions
                    store_round(o, &map3, pos0, 0, line, 0);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B->acc_empty[half]);
            }
        }
        if (epi_tid == 0) bulk_wait0();
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

static int make_maps(int mode, const Args& a, CUtensorMap (&m)[4]) {
    const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int span = a.transposed ? a.rows : a.n, lines = a.transposed ? a.n : a.rows;
    int rc;
    if (mode == MODE_TRIMUL_MX) {
        for (int i = 0; i < 2; ++i) {     // byte planes [d][line][pitch]
            cuuint64_t dims[4] = {(cuuint64_t)a.pitch, (cuuint64_t)lines, 128, 1};
            cuuint64_t str[3] = {(cuuint64_t)a.pitch, (cuuint64_t)a.plane_stride[i], (cuuint64_t)a.plane_stride[i] * 128};
            cuuint32_t box[4] = {128, 1, 128, 1};
            if ((rc = tmap_encode(&m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, a.planes[i], 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                  "mx planes")) != B200PF_OK) return rc;
        }
        m[2] = m[0];
        m[3] = m[0];
        return B200PF_OK;
    }
    if (mode == MODE_TRIMUL) {
        for (int i = 0; i < 2; ++i) {
            const int rg = a.row_group[i], groups = (lines + rg - 1) / rg;
            cuuint64_t dims[4] = {(cuuint64_t)a.pitch, (cuuint64_t)(rg < lines ? rg : lines), 128, (cuuint64_t)groups};
            cuuint64_t str[3] = {(cuuint64_t)a.pitch * 2, (cuuint64_t)a.plane_stride[i] * 2,
                                 (cuuint64_t)(groups > 1 ? a.group_stride[i] : a.plane_stride[i] * 128) * 2};
            cuuint32_t box[4] = {64, 1, 128, 1};
            if ((rc = tmap_encode(&m[i], bf, a.planes[i], 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "planes")) != B200PF_OK) return rc;
        }
        m[2] = m[0];
        m[3] = m[0];
        return B200PF_OK;
    }
    {   // q, k: [line][pos][128]
        cuuint64_t dims[4] = {128, (cuuint64_t)span, (cuuint64_t)lines, 1};
        cuuint64_t str[3] = {256, (cuuint64_t)span * 256, (cuuint64_t)span * 256 * lines};
        cuuint32_t box[4] = {64, 128, 1, 1};
        if ((rc = tmap_encode(&m[0], bf, a.q, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "q")) != B200PF_OK) return rc;
        if ((rc = tmap_encode(&m[1], bf, a.k, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "k")) != B200PF_OK) return rc;
    }
    {   // g in the layout of the z view [rows][n][128]
        cuuint64_t dims[4] = {128, (cuuint64_t)a.n, (cuuint64_t)a.rows, 1};
        cuuint64_t str[3] = {256, (cuuint64_t)a.n * 256, (cuuint64_t)a.n * 256 * a.rows};
        cuuint32_t box_rows[4] = {64, 128, 1, 1}, box_cols[4] = {64, 1, 128, 1};
        if ((rc = tmap_encode(&m[2], bf, a.g, 4, dims, str, a.transposed ? box_cols : box_rows, CU_TENSOR_MAP_SWIZZLE_128B, "g")) != B200PF_OK) return rc;
    }
    {   // v transposed: [line][head*32 + d][vt_pitch]
        cuuint64_t dims[4] = {(cuuint64_t)a.vt_pitch, 128, (cuuint64_t)lines, 1};
        cuuint64_t str[3] = {(cuuint64_t)a.vt_pitch * 2, (cuuint64_t)a.vt_pitch * 256, (cuuint64_t)a.vt_pitch * 256 * lines};
        cuuint32_t box[4] = {64, 128, 1, 1};
        if ((rc = tmap_encode(&m[3], bf, a.v, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "vt")) != B200PF_OK) return rc;
    }
    return B200PF_OK;
}

template <int MODE>
static int launch(const Args& a, cudaStream_t st) {
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "row512: no device status word");
    B200PF_REQUIRE(a.ln_gamma && a.ln_beta && aligned16(a.ln_gamma) && aligned16(a.ln_beta), B200PF_ERR_INVALID,
                   "row512: LayerNorm gain / offset must be given and 16-byte aligned");
    B200PF_SMEM_ATTR_ONCE(row512_kernel<MODE>, SMEM_BYTES);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int span = a.transposed ? a.rows : a.n, lines = a.transposed ? a.n : a.rows;
    long long tiles = (long long)lines * ((span + TM - 1) / TM);
    CUtensorMap m[4];
    int rc = make_maps(MODE, a, m);
    if (rc != B200PF_OK) return rc;
    row512_kernel<MODE><<<(unsigned)(tiles < sms ? tiles : sms), THREADS, SMEM_BYTES, st>>>(m[0], m[1], m[2], m[3], a, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int launch_trimul(const Args& a, cudaStream_t st) { return launch<MODE_TRIMUL>(a, st); }
int launch_trimul_mx(const Args& a, cudaStream_t st) { return launch<MODE_TRIMUL_MX>(a, st); }
int launch_triatt(const Args& a, cudaStream_t st) { return launch<MODE_TRIATT>(a, st); }

}  // namespace r512
}  // namespace b200pf
