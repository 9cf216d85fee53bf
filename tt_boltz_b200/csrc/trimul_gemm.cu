// Triangle-multiplication contraction: x[d][i][j] = sum_k A[d][i][k] * B[d][j][k].
//
// One batched K-major GEMM over the 128 channels.  Persistent, warp-specialised kernel:
//   warp 0   : TMA producer (one lane) - 128x64 bf16 boxes, 128-byte swizzle, 4-stage ring
//   warp 1   : TMEM owner + MMA issuer (one lane) - tcgen05.mma 128x256x16, fp32 accumulators
//   warps 2-5: epilogue - tcgen05.ld the finished 128x256 accumulator, round to bf16, store
// Two accumulators (2 x 256 TMEM columns) let the epilogue of tile t overlap the MMAs of t+1.
// Ragged sizes need no padding: TMA zero-fills out-of-range rows / columns, stores are guarded.
#include <cstdlib>

#include "sm100.cuh"

namespace b200pf {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct GemmShape {
    int m_rows;          // rows of A (output rows)
    int n_rows;          // rows of B over all row segments (output columns)
    int k_total;         // contraction length over all k segments
    int a_kseg_cols;     // columns per k segment of A (== k_total when unsegmented)
    int b_kseg_cols;
    int a_rowseg_rows;   // rows per row segment of A (> m_rows when unsegmented)
    int b_rowseg_rows;   // rows per row segment of B (> n_rows when unsegmented)
    int channels;
    int x_pitch;
    long long x_plane_stride;
    int x_row_group;     // output rows per group (> m_rows when the output is plain planes)
    long long x_group_stride;
    int x_cols;          // columns written (whole 8-column vectors below this bound)
    int x_col_group;     // > 0: output columns in groups of this many (a multiple of 32), x_colgroup_stride elements apart
    long long x_colgroup_stride;
};
// Output element (d, row, col) lives at (row / x_row_group) * x_group_stride + d * x_plane_stride + (row % x_row_group) * x_pitch + col.
__device__ __forceinline__ long long x_row_offset(const GemmShape& s, int d, int row) {
    const int grp = row / s.x_row_group;
    return (long long)grp * s.x_group_stride + (long long)d * s.x_plane_stride + (long long)(row - grp * s.x_row_group) * s.x_pitch;
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
trimul_contract_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          __nv_bfloat16* __restrict__ x, GemmShape s, unsigned int* status) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                    // [STAGES]
    uint64_t* empty = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = (s.m_rows + BM - 1) / BM, nt = (s.n_rows + BN - 1) / BN;
    const int kb_total = (s.k_total + BK - 1) / BK;
    const long long tiles = (long long)s.channels * mt * nt;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            int d = (int)(t / (mt * nt));
            int rem = (int)(t % (mt * nt));
            int m0 = (rem / nt) * BM, n0 = (rem % nt) * BN;
            for (int kb = 0; kb < kb_total; ++kb) {
                ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag);
                if (!ok) break;
                uint8_t* sa = smem + stage * STAGE_BYTES;
                uint8_t* sb = sa + A_BYTES;
                mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
                int k0 = kb * BK;
                tma_load_4d(sa, &map_a, &full[stage], k0 % s.a_kseg_cols, m0 % s.a_rowseg_rows, d, m0 / s.a_rowseg_rows + k0 / s.a_kseg_cols);
                int kseg_b = k0 / s.b_kseg_cols, kin_b = k0 % s.b_kseg_cols;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    int j = n0 + half * 128;
                    int rseg = j / s.b_rowseg_rows, rin = j % s.b_rowseg_rows;
                    tma_load_4d(sb + half * (128 * BK * 2), &map_b, &full[stage], kin_b, rin, d, rseg + kseg_b);
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok) {   // give copies in flight time to land before the CTA's shared memory goes away
            atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
            uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop and waits; one elected lane issues (see sm100::elect_one).
        constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
        const uint64_t d_a0 = make_desc_k_sw128(smem_u32(smem)), d_b0 = make_desc_k_sw128(smem_u32(smem + A_BYTES));
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        long long it = 0;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            uint32_t ab = (uint32_t)(it & 1), aphase = (uint32_t)((it >> 1) & 1);
            ok = mbar_wait_warp(&acc_empty[ab], aphase ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t tmem_d = tmem_base + ab * BN;
            for (int kb = 0; kb < kb_total; ++kb) {
                ok = mbar_wait_warp(&full[stage], phase, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t so = stage * (uint64_t)(STAGE_BYTES >> 4);      // descriptors: precomputed base + 16-byte units
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) umma_bf16(tmem_d, d_a0 + so + kk * 2, d_b0 + so + kk * 2, idesc, (kb | kk) ? 1u : 0u);
                    umma_commit(&empty[stage]);
                    if (kb + 1 == kb_total) umma_commit(&acc_full[ab]);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;                 // TMEM lanes this warp may touch: 32*quarter ..
        bool ok = true;
        long long it = 0;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            uint32_t ab = (uint32_t)(it & 1), aphase = (uint32_t)((it >> 1) & 1);
            int d = (int)(t / (mt * nt));
            int rem = (int)(t % (mt * nt));
            int m0 = (rem / nt) * BM, n0 = (rem % nt) * BN;
            ok = mbar_wait(&acc_full[ab], aphase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            int row = m0 + quarter * 32 + lane;
            __nv_bfloat16* xrow = x + x_row_offset(s, d, row < s.m_rows ? row : 0);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                int col = n0 + c * 32;
                if (col >= s.x_cols) break;           // warp-uniform
                __nv_bfloat16* xdst = s.x_col_group > 0
                                          ? xrow + (long long)(col / s.x_col_group) * s.x_colgroup_stride + (col % s.x_col_group)
                                          : xrow + col;
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * BN + c * 32, r);
                tmem_ld_wait();
                if (row < s.m_rows) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        if (col + v * 8 + 8 <= s.x_cols) {
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                            *reinterpret_cast<uint4*>(xdst + v * 8) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---- the same GEMM on CTA pairs ------------------------------------------------------------------
// Two CTAs of a cluster (the two SMs of a TPC) share one 256 x 256 output tile: each stages its 128 rows of A and
// its 128 rows of B (32 KB per k-block instead of the 48 KB a lone CTA needs for 128 x 256: the lone kernel is bound
// by the 96 bytes per clock it has to pull from L2), the even CTA issues tcgen05.mma.cta_group::2 over both halves,
// and each CTA drains its own 128 accumulator rows.  Loads land in the loading CTA's own shared memory (never a
// multicast); their bytes are counted on the even CTA's barrier.  Every role of both CTAs always reaches the two
// cluster barriers, also after a wait ran out.
constexpr int P_STAGES = 6, P_STAGE_BYTES = 2 * (128 * BK * 2);
constexpr int PAIR_SMEM = P_STAGES * P_STAGE_BYTES + 1024 + 256;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
trimul_contract_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            __nv_bfloat16* __restrict__ x, GemmShape s, unsigned int* status) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
    uint64_t* full = bars;                      // [P_STAGES]  used in the even CTA: both CTAs' loads
    uint64_t* empty = bars + P_STAGES;          // [P_STAGES]  one per CTA
    uint64_t* acc_full = bars + 2 * P_STAGES;   // [2]         one per CTA
    uint64_t* acc_empty = acc_full + 2;         // [2]         used in the even CTA: both CTAs' epilogue warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                     // 0: issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int mt = (s.m_rows + 255) / 256, nt = (s.n_rows + BN - 1) / BN;
    const int kb_total = (s.k_total + BK - 1) / BK;
    const long long tiles = (long long)s.channels * mt * nt;

    if (threadIdx.x == 0) {
        for (int i = 0; i < P_STAGES; ++i) { mbar_init(&full[i], 2); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                              // the other CTA's barriers and tensor memory are ready
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer: this CTA's half of A and of B ----------------
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        const uint32_t full0 = map_to_cta(&full[0], 0);            // the even CTA's barriers, 8 bytes apart
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (long long t = pair; t < tiles && ok; t += pairs) {
            const int d = (int)(t / (mt * nt));
            const int rem = (int)(t % (mt * nt));
            const int m0 = (rem / nt) * 256 + (int)rank * 128, n0 = (rem % nt) * BN + (int)rank * 128;
            // row coordinates once per tile; the k coordinates advance by BK (a k segment is a multiple of BK long)
            const int a_row = m0 % s.a_rowseg_rows, a_seg0 = m0 / s.a_rowseg_rows;
            const int b_row = n0 % s.b_rowseg_rows, b_seg0 = n0 / s.b_rowseg_rows;
            int a_k = 0, a_ks = 0, b_k = 0, b_ks = 0;
            for (int kb = 0; kb < kb_total; ++kb) {
                ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag);
                if (!ok) break;
                uint8_t* sa = smem + stage * P_STAGE_BYTES;
                const uint32_t fb = full0 + stage * 8;
                if (rank == 0) mbar_arrive_expect_tx(&full[stage], P_STAGE_BYTES);
                else mbar_arrive_expect_tx_cluster(fb, P_STAGE_BYTES);
                tma_load_4d_pair(sa, &map_a, fb, a_k, a_row, d, a_seg0 + a_ks);
                tma_load_4d_pair(sa + 128 * BK * 2, &map_b, fb, b_k, b_row, d, b_seg0 + b_ks);
                a_k += BK; if (a_k >= s.a_kseg_cols) { a_k = 0; ++a_ks; }
                b_k += BK; if (b_k >= s.b_kseg_cols) { b_k = 0; ++b_ks; }
                if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok) {   // give copies in flight time to land before the CTA's shared memory goes away
            atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
            uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
    } else if (warp == 1 && rank == 0) {
        // ---------------- MMA issuer (even CTA only) ----------------
        constexpr uint32_t idesc = make_idesc_bf16(256, BN);
        const uint64_t d_a0 = make_desc_k_sw128(smem_u32(smem)), d_b0 = make_desc_k_sw128(smem_u32(smem + 128 * BK * 2));
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        long long it = 0;
        for (long long t = pair; t < tiles && ok; t += pairs, ++it) {
            uint32_t ab = (uint32_t)(it & 1), aphase = (uint32_t)((it >> 1) & 1);
            ok = mbar_wait_warp(&acc_empty[ab], aphase ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t tmem_d = tmem_base + ab * BN;
            for (int kb = 0; kb < kb_total; ++kb) {
                ok = mbar_wait_warp(&full[stage], phase, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t so = stage * (uint64_t)(P_STAGE_BYTES >> 4);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) umma_bf16_pair(tmem_d, d_a0 + so + kk * 2, d_b0 + so + kk * 2, idesc, (kb | kk) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&empty[stage]));
                    umma_commit_pair(map_to_cta(&empty[stage], 1));
                    if (kb + 1 == kb_total) {
                        umma_commit_pair(smem_u32(&acc_full[ab]));
                        umma_commit_pair(map_to_cta(&acc_full[ab], 1));
                    }
                }
                __syncwarp();
                if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else if (warp >= 2) {
        // ---------------- epilogue: this CTA's 128 rows of the tile ----------------
        const int quarter = warp & 3;
        bool ok = true;
        long long it = 0;
        for (long long t = pair; t < tiles && ok; t += pairs, ++it) {
            uint32_t ab = (uint32_t)(it & 1), aphase = (uint32_t)((it >> 1) & 1);
            int d = (int)(t / (mt * nt));
            int rem = (int)(t % (mt * nt));
            int m0 = (rem / nt) * 256 + (int)rank * 128, n0 = (rem % nt) * BN;
            ok = mbar_wait(&acc_full[ab], aphase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            int row = m0 + quarter * 32 + lane;
            __nv_bfloat16* xrow = x + x_row_offset(s, d, row < s.m_rows ? row : 0);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                int col = n0 + c * 32;
                if (col >= s.x_cols) break;           // warp-uniform
                __nv_bfloat16* xdst = s.x_col_group > 0
                                          ? xrow + (long long)(col / s.x_col_group) * s.x_colgroup_stride + (col % s.x_col_group)
                                          : xrow + col;
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * BN + c * 32, r);
                tmem_ld_wait();
                if (row < s.m_rows) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        if (col + v * 8 + 8 <= s.x_cols) {
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                            *reinterpret_cast<uint4*>(xdst + v * 8) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[ab], 0));
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                              // nobody signals or reads the other CTA after this
    if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, 512); }
}

// ---- host: tensor maps -----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static int make_plane_map(CUtensorMap* map, const b200pf_planes* p, int channels, const char* what) {
    EncodeTiledFn fn = encode_fn();
    B200PF_REQUIRE(fn != nullptr, B200PF_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
    long long seg_stride = p->nseg > 1 ? p->seg_stride : p->plane_stride * channels;
    cuuint64_t dims[4] = {(cuuint64_t)p->cols, (cuuint64_t)p->rows, (cuuint64_t)channels, (cuuint64_t)p->nseg};
    cuuint64_t strides[3] = {(cuuint64_t)p->pitch * 2, (cuuint64_t)p->plane_stride * 2, (cuuint64_t)seg_stride * 2};
    cuuint32_t box[4] = {(cuuint32_t)BK, 128u, 1u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(p->ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200PF_REQUIRE(r == CUDA_SUCCESS, B200PF_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return B200PF_OK;
}

static int check_planes(const b200pf_planes* p, const char* what) {
    B200PF_REQUIRE(p && p->ptr, B200PF_ERR_INVALID, "trimul_contract: %s is null", what);
    B200PF_REQUIRE(aligned16(p->ptr), B200PF_ERR_INVALID, "trimul_contract: %s not 16-byte aligned", what);
    B200PF_REQUIRE(p->rows > 0 && p->cols > 0 && p->nseg >= 1, B200PF_ERR_INVALID, "trimul_contract: %s has empty extent", what);
    B200PF_REQUIRE(p->pitch >= p->cols && p->pitch % 8 == 0, B200PF_ERR_INVALID,
                   "trimul_contract: %s pitch %d must be >= cols %d and a multiple of 8", what, p->pitch, p->cols);
    B200PF_REQUIRE(p->plane_stride % 8 == 0 && p->plane_stride >= (long long)p->pitch * p->rows, B200PF_ERR_INVALID,
                   "trimul_contract: %s plane stride too small or not a multiple of 8", what);
    if (p->nseg > 1) {
        B200PF_REQUIRE(p->seg_stride % 8 == 0 && p->seg_stride > 0, B200PF_ERR_INVALID, "trimul_contract: %s bad segment stride", what);
        if (p->seg_is_k)
            B200PF_REQUIRE(p->cols % BK == 0, B200PF_ERR_UNSUPPORTED,
                           "trimul_contract: %s k segments must be multiples of %d columns", what, BK);
        else
            B200PF_REQUIRE(p->rows % 128 == 0, B200PF_ERR_UNSUPPORTED,
                           "trimul_contract: %s row segments must be multiples of 128 rows", what);
    }
    return B200PF_OK;
}

// B200PF_CONTRACT_PAIR=0 keeps every GEMM on the one-CTA kernel (read once).
static bool use_pair_kernel() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200PF_CONTRACT_PAIR");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}
static bool pair_attr_set[64] = {false};

static int launch_contract_tc(const b200pf_planes* a, const b200pf_planes* b, b200pf_bf16* x, const GemmShape& s, cudaStream_t st) {
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "trimul_contract: no device status word");
    CUtensorMap map_a, map_b;
    int rc;
    if ((rc = make_plane_map(&map_a, a, s.channels, "A")) != B200PF_OK) return rc;
    if ((rc = make_plane_map(&map_b, b, s.channels, "B")) != B200PF_OK) return rc;
    static bool attr_set[64] = {false};
    int dev = 0;
    B200PF_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        B200PF_CUDA(cudaFuncSetAttribute(trimul_contract_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM));
        attr_set[dev] = true;
    }
    int sms = 0;
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (use_pair_kernel() && s.m_rows > BM) {
        if (dev >= 0 && dev < 64 && !pair_attr_set[dev]) {
            B200PF_CUDA(cudaFuncSetAttribute(trimul_contract_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM));
            pair_attr_set[dev] = true;
        }
        long long tiles = (long long)s.channels * ((s.m_rows + 255) / 256) * ((s.n_rows + BN - 1) / BN);
        // A persistent grid must be resident at once: a pair that only starts when another has finished would
        // double the time.  Not every SM can be half of a pair, so ask how many pairs fit.
        static int resident_pairs[64] = {0};
        if (dev >= 0 && dev < 64 && resident_pairs[dev] == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
            cfg.blockDim = dim3(GEMM_THREADS);
            cfg.dynamicSmemBytes = PAIR_SMEM;
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2;
            attr.val.clusterDim.y = 1;
            attr.val.clusterDim.z = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            int n = 0;
            B200PF_CUDA(cudaOccupancyMaxActiveClusters(&n, trimul_contract_pair_kernel, &cfg));
            B200PF_REQUIRE(n > 0, B200PF_ERR_CUDA, "trimul_contract: no CTA pair fits on this device");
            resident_pairs[dev] = n < sms / 2 ? n : sms / 2;
        }
        long long pairs = (dev >= 0 && dev < 64) ? resident_pairs[dev] : sms / 2;
        unsigned grid = 2u * (unsigned)(tiles < pairs ? tiles : pairs);
        trimul_contract_pair_kernel<<<grid, GEMM_THREADS, PAIR_SMEM, st>>>(map_a, map_b, (__nv_bfloat16*)x, s, status);
        B200PF_LAUNCH_CHECK();
        return B200PF_OK;
    }
    long long tiles = (long long)s.channels * ((s.m_rows + BM - 1) / BM) * ((s.n_rows + BN - 1) / BN);
    unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    trimul_contract_tc_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(map_a, map_b, (__nv_bfloat16*)x, s, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

namespace gemm_mx {   // block-scaled fp8 kernel, trimul_gemm_mx.cu
int launch_contract(const b200pf_planes* a, const b200pf_planes* b, const void* a_scales, const void* b_scales,
                    b200pf_bf16* x, long long x_plane_stride, int x_pitch, int x_row_group, long long x_group_stride,
                    int channels, cudaStream_t st);
}

}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_trimul_contract(const b200pf_planes* a, const b200pf_planes* b,
                                      const void* a_scales, const void* b_scales,
                                      b200pf_bf16* x, long long x_plane_stride, int x_pitch,
                                      int x_row_group, long long x_group_stride,
                                      int channels, int variant, void* stream) {
    if (variant == 2) {
        return gemm_mx::launch_contract(a, b, a_scales, b_scales, x, x_plane_stride, x_pitch, x_row_group, x_group_stride, channels,
                                        static_cast<cudaStream_t>(stream));
    }
    int rc;
    if ((rc = check_planes(a, "A")) != B200PF_OK) return rc;
    if ((rc = check_planes(b, "B")) != B200PF_OK) return rc;
    B200PF_REQUIRE(x && aligned16(x) && channels > 0, B200PF_ERR_INVALID, "trimul_contract: bad output");
    GemmShape s;
    s.m_rows = (a->nseg > 1 && !a->seg_is_k) ? a->rows * a->nseg : a->rows;
    s.n_rows = (b->nseg > 1 && !b->seg_is_k) ? b->rows * b->nseg : b->rows;
    int ka = (a->nseg > 1 && a->seg_is_k) ? a->cols * a->nseg : a->cols;
    int kb = (b->nseg > 1 && b->seg_is_k) ? b->cols * b->nseg : b->cols;
    B200PF_REQUIRE(ka == kb, B200PF_ERR_INVALID, "trimul_contract: contraction lengths differ (%d vs %d)", ka, kb);
    s.k_total = ka;
    s.a_kseg_cols = (a->nseg > 1 && a->seg_is_k) ? a->cols : (ka + BK);          // never reached by k0 when unsegmented
    s.a_rowseg_rows = (a->nseg > 1 && !a->seg_is_k) ? a->rows : (s.m_rows + BM);
    s.b_kseg_cols = (b->nseg > 1 && b->seg_is_k) ? b->cols : (kb + BK);
    s.b_rowseg_rows = (b->nseg > 1 && !b->seg_is_k) ? b->rows : (s.n_rows + BN);
    s.channels = channels;
    s.x_pitch = x_pitch;
    s.x_plane_stride = x_plane_stride;
    const bool grouped = x_row_group > 0 && x_row_group < s.m_rows;
    s.x_row_group = grouped ? x_row_group : s.m_rows + BM;
    s.x_group_stride = grouped ? x_group_stride : 0;
    s.x_cols = x_pitch;
    s.x_col_group = 0;
    s.x_colgroup_stride = 0;
    B200PF_REQUIRE(x_pitch % 8 == 0 && x_pitch >= s.n_rows &&
                       x_plane_stride >= (long long)x_pitch * (grouped ? x_row_group : s.m_rows) && x_plane_stride % 8 == 0,
                   B200PF_ERR_INVALID, "trimul_contract: bad x pitch / plane stride");
    B200PF_REQUIRE(!grouped || (x_group_stride % 8 == 0 && x_group_stride >= x_plane_stride * channels), B200PF_ERR_INVALID,
                   "trimul_contract: bad x group stride");
    B200PF_REQUIRE(variant == 0, B200PF_ERR_UNSUPPORTED, "trimul_contract: variant %d is not built", variant);
    return launch_contract_tc(a, b, x, s, static_cast<cudaStream_t>(stream));
}

/* The same GEMM with both output indices regrouped: element (d, row, col) is written to
 *   (row / x_row_group) * x_group_stride + d * x_plane_stride + (row % x_row_group) * x_pitch
 *   + (col / x_col_group) * x_colgroup_stride + col % x_col_group
 * (x_row_group <= 0: rows not grouped; x_col_group a multiple of 32).  Operands as for b200pf_trimul_contract, bf16 only. */
extern "C" int b200pf_gemm_grouped(const b200pf_planes* a, const b200pf_planes* b, b200pf_bf16* x, long long x_plane_stride,
                                   int x_pitch, int x_row_group, long long x_group_stride, int x_col_group,
                                   long long x_colgroup_stride, int channels, void* stream) {
    int rc;
    if ((rc = check_planes(a, "A")) != B200PF_OK) return rc;
    if ((rc = check_planes(b, "B")) != B200PF_OK) return rc;
    B200PF_REQUIRE(x && aligned16(x) && channels > 0, B200PF_ERR_INVALID, "gemm_grouped: bad output");
    B200PF_REQUIRE(a->nseg == 1 && b->nseg == 1 && a->cols == b->cols, B200PF_ERR_INVALID,
                   "gemm_grouped: unsegmented operands of equal contraction length only");
    B200PF_REQUIRE(x_col_group > 0 && x_col_group % 32 == 0 && x_colgroup_stride % 8 == 0 && x_pitch % 8 == 0 &&
                       x_pitch >= x_col_group && x_plane_stride % 8 == 0 && x_group_stride % 8 == 0,
                   B200PF_ERR_INVALID, "gemm_grouped: column groups must be multiples of 32 and every stride a multiple of 8");
    GemmShape s;
    s.m_rows = a->rows;
    s.n_rows = b->rows;
    s.k_total = a->cols;
    s.a_kseg_cols = a->cols + BK;
    s.b_kseg_cols = b->cols + BK;
    s.a_rowseg_rows = s.m_rows + BM;
    s.b_rowseg_rows = s.n_rows + BN;
    s.channels = channels;
    s.x_pitch = x_pitch;
    s.x_plane_stride = x_plane_stride;
    const bool grouped = x_row_group > 0 && x_row_group < s.m_rows;
    s.x_row_group = grouped ? x_row_group : s.m_rows + BM;
    s.x_group_stride = grouped ? x_group_stride : 0;
    s.x_cols = (s.n_rows + 7) / 8 * 8;
    s.x_col_group = x_col_group;
    s.x_colgroup_stride = x_colgroup_stride;
    return launch_contract_tc(a, b, x, s, static_cast<cudaStream_t>(stream));
}

/* Outer product of the outer-product-mean: x2[i][j][c][d] = sum_s a_t[(i, c)][s] * b_t[(j, d)][s], the same kernel with
 * its output rows (i, c) and columns (j, d) regrouped so that the 32 x 32 block of a token pair is contiguous. */
extern "C" int b200pf_opm_outer(const b200pf_bf16* a_t, const b200pf_bf16* b_t, b200pf_bf16* x2,
                                int s_len, int n_i, int n_j, int pitch, void* stream) {
    B200PF_REQUIRE(a_t && b_t && x2 && aligned16(a_t) && aligned16(b_t) && aligned16(x2), B200PF_ERR_INVALID,
                   "opm_outer: null or misaligned pointer");
    B200PF_REQUIRE(s_len > 0 && n_i > 0 && n_j > 0 && pitch >= s_len && pitch % 8 == 0, B200PF_ERR_INVALID, "opm_outer: bad sizes");
    B200PF_REQUIRE((long long)n_j * 32 <= 0x7fffffffLL / 2 && (long long)n_i * 32 <= 0x7fffffffLL / 2, B200PF_ERR_UNSUPPORTED,
                   "opm_outer: too many tokens");
    b200pf_planes a{a_t, (long long)pitch * n_i * 32, 0, pitch, n_i * 32, s_len, 1, 0};
    b200pf_planes b{b_t, (long long)pitch * n_j * 32, 0, pitch, n_j * 32, s_len, 1, 0};
    GemmShape s;
    s.m_rows = n_i * 32;
    s.n_rows = n_j * 32;
    s.k_total = s_len;
    s.a_kseg_cols = s_len + BK;
    s.b_kseg_cols = s_len + BK;
    s.a_rowseg_rows = s.m_rows + BM;
    s.b_rowseg_rows = s.n_rows + BN;
    s.channels = 1;
    s.x_pitch = 32;                                   // row (i, c): c * 32 inside the pair's block
    s.x_plane_stride = 0;
    s.x_row_group = 32;
    s.x_group_stride = (long long)n_j * 1024;         // next i
    s.x_cols = s.n_rows;
    s.x_col_group = 32;
    s.x_colgroup_stride = 1024;                       // next j
    return launch_contract_tc(&a, &b, x2, s, static_cast<cudaStream_t>(stream));
}
