// Triangle-multiplication contraction on MXFP8 operands:
//   x[d][i][j] = sum_k (A[d][i][k] * 2^sa[d][i][k/32]) * (B[d][j][k] * 2^sb[d][j][k/32])
// with the block-scaled tensor-core instruction (tcgen05.mma.kind::mxf8f6f4.block_scale): e4m3
// values come from shared memory, the e8m0 scales from tensor memory.
//
// Same roles as the bf16 kernel (warp 0 TMA, warp 1 MMA issuer, warps 2-5 epilogue), but:
//   * a stage is 128 k (= 128 bytes per row, one 128-byte swizzle atom): A 128 rows, B 256 rows,
//     plus their scale blocks (512 B for A, 2 x 512 B for B; layout in mxfp8.cuh) fetched with
//     untiled bulk copies onto the same mbarrier;
//   * per stage the issuer copies the three scale blocks into tensor memory (tcgen05.cp, 4 columns
//     each) and then issues four K = 32 MMAs, each selecting its scale byte through the
//     instruction descriptor.  tcgen05.cp and tcgen05.mma of one thread execute in issue order, so
//     the scale columns are single-buffered;
//   * the 12 scale columns leave room for only one 256-column accumulator, so the epilogue of a
//     tile does not overlap the MMAs of the next (TMA still runs ahead through the 4-stage ring).
#include "mxfp8.cuh"
#include "sm100.cuh"
#include "tmap.cuh"

namespace b200pf {
namespace gemm_mx {

constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, DATA_BYTES = A_BYTES + B_BYTES;       // 48 KB
constexpr int SF_BYTES = 3 * mx::SF_BLOCK_BYTES;                                            // A, B lo, B hi
constexpr int OFF_SF = STAGES * DATA_BYTES, OFF_BAR = OFF_SF + STAGES * SF_BYTES;
constexpr int THREADS = 192;
constexpr int SMEM = OFF_BAR + 256 + 1024 /*alignment slack*/;
constexpr uint32_t COL_SFA = 256, COL_SFB = 264;

// Operands may arrive in segments (the sharded trunk: one per source rank), either blocks of ROWS or blocks of the
// contraction index; a segment holds [channels][rows][pitch] values and, packed right behind each other in the
// same order, [channels][kgroups][row_blocks] scale blocks.  Unsegmented operands set the segment extents beyond
// the tensor, so the quotients below are 0.
struct Shape {
    int m_rows, n_rows, k_total, channels, x_pitch;
    long long x_plane_stride;
    int a_kgroups, a_row_blocks, b_kgroups, b_row_blocks;      // per segment
    int a_kseg_cols, a_rowseg_rows, b_kseg_cols, b_rowseg_rows;
    long long a_sf_seg, b_sf_seg;                              // bytes between the scale buffers of two segments
    int x_row_group;                                           // output rows per group (> m_rows: plain planes)
    long long x_group_stride;
};
__device__ __forceinline__ long long sf_block_offset(int d, int k0, int row0, int kseg_cols, int rowseg_rows, int kgroups_, int row_blocks_,
                                                     long long seg_stride) {
    const int kseg = k0 / kseg_cols, kin = k0 - kseg * kseg_cols;
    const int rseg = row0 / rowseg_rows, rin = row0 - rseg * rowseg_rows;
    return (long long)(kseg + rseg) * seg_stride +
           (((long long)d * kgroups_ + (kin >> 7)) * row_blocks_ + (rin >> 7)) * mx::SF_BLOCK_BYTES;
}

__global__ void __launch_bounds__(THREADS, 1)
trimul_contract_mx_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb,
                          __nv_bfloat16* __restrict__ x, Shape s, unsigned int* status) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* full = bars;                    // [STAGES]
    uint64_t* empty = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = (s.m_rows + BM - 1) / BM, nt = (s.n_rows + BN - 1) / BN;
    const int kb_total = (s.k_total + BK - 1) / BK;
    const long long tiles = (long long)s.channels * mt * nt;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
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
            const int d = (int)(t / (mt * nt)), rem = (int)(t % (mt * nt));
            const int m0 = (rem / nt) * BM, n0 = (rem % nt) * BN;
            for (int kb = 0; kb < kb_total; ++kb) {
                ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag);
                if (!ok) break;
                uint8_t* sa = smem + stage * DATA_BYTES;
                uint8_t* sb = sa + A_BYTES;
                uint8_t* sf = smem + OFF_SF + stage * SF_BYTES;
                mbar_arrive_expect_tx(&full[stage], DATA_BYTES + SF_BYTES);
                const int k0 = kb * BK;
                tma_load_4d(sa, &map_a, &full[stage], k0 % s.a_kseg_cols, m0 % s.a_rowseg_rows, d, m0 / s.a_rowseg_rows + k0 / s.a_kseg_cols);
                bulk_load_1d(sf, sfa + sf_block_offset(d, k0, m0, s.a_kseg_cols, s.a_rowseg_rows, s.a_kgroups, s.a_row_blocks, s.a_sf_seg),
                             mx::SF_BLOCK_BYTES, &full[stage]);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int j = n0 + half * 128;
                    tma_load_4d(sb + half * (128 * BK), &map_b, &full[stage], k0 % s.b_kseg_cols, j % s.b_rowseg_rows, d,
                                j / s.b_rowseg_rows + k0 / s.b_kseg_cols);          // rows past the end: zero fill
                    const int js = j < s.n_rows ? j : n0;                           // their scales: any block that exists
                    bulk_load_1d(sf + (1 + half) * mx::SF_BLOCK_BYTES,
                                 sfb + sf_block_offset(d, k0, js, s.b_kseg_cols, s.b_rowseg_rows, s.b_kgroups, s.b_row_blocks, s.b_sf_seg),
                                 mx::SF_BLOCK_BYTES, &full[stage]);
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
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        long long it = 0;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            ok = mbar_wait_warp(acc_empty, (uint32_t)(it & 1) ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            for (int kb = 0; kb < kb_total; ++kb) {
                ok = mbar_wait_warp(&full[stage], phase, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t sa = smem_u32(smem + stage * DATA_BYTES), sb = sa + A_BYTES;
                    const uint32_t sf = smem_u32(smem + OFF_SF + stage * SF_BYTES);
                    tmem_cp_scale_block(tmem_base + COL_SFA, make_desc_scale_block(sf));
                    tmem_cp_scale_block(tmem_base + COL_SFB, make_desc_scale_block(sf + mx::SF_BLOCK_BYTES));
                    tmem_cp_scale_block(tmem_base + COL_SFB + 4, make_desc_scale_block(sf + 2 * mx::SF_BLOCK_BYTES));
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk) {
                        umma_mxf8(tmem_base, make_desc_k_sw128(sa + kk * 32), make_desc_k_sw128(sb + kk * 32),
                                  make_idesc_mxf8(BM, BN, kk, kk), (tmem_base + COL_SFA) | (kk << 30),
                                  (tmem_base + COL_SFB) | (kk << 30), (kb | (int)kk) ? 1u : 0u);
                    }
                    umma_commit(&empty[stage]);
                    if (kb + 1 == kb_total) umma_commit(acc_full);
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
            const int d = (int)(t / (mt * nt)), rem = (int)(t % (mt * nt));
            const int m0 = (rem / nt) * BM, n0 = (rem % nt) * BN;
            ok = mbar_wait(acc_full, (uint32_t)(it & 1), abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const int rsafe = row < s.m_rows ? row : 0, grp = rsafe / s.x_row_group;
            __nv_bfloat16* xrow = x + (long long)grp * s.x_group_stride + (long long)d * s.x_plane_stride +
                                  (long long)(rsafe - grp * s.x_row_group) * s.x_pitch;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col = n0 + c * 32;
                if (col >= s.x_pitch) break;          // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 32, r);
                tmem_ld_wait();
                if (row < s.m_rows) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        if (col + v * 8 + 8 <= s.x_pitch) {
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                            *reinterpret_cast<uint4*>(xrow + col + v * 8) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// Expand MXFP8 planes into bf16 planes (exact: e4m3 x 2^e fits in bf16).  Used as the cross-check
// of the block-scaled GEMM and wherever a consumer wants plain bf16 operands.
__global__ void __launch_bounds__(256)
mx_dequant_kernel(const uint8_t* __restrict__ planes, const uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                  long long plane_stride, int pitch, long long out_plane_stride, int out_pitch, int rows, int cols, int channels,
                  int kgroups_, int row_blocks_) {
    const int chunks = (cols + 15) / 16;                         // 16 values per thread
    const long long total = (long long)channels * rows * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ch = (int)(i % chunks);
        const long long dr = i / chunks;
        const int row = (int)(dr % rows), d = (int)(dr / rows);
        const int k0 = ch * 16;
        const uint4 raw = *reinterpret_cast<const uint4*>(planes + d * plane_stride + (long long)row * pitch + k0);
        const uint32_t e = scales[mx::scale_offset(d, row, k0 >> 5, kgroups_, row_blocks_)];
        const float sc = mx::scale_value(e);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        __nv_bfloat16* dst = out + d * out_plane_stride + (long long)row * out_pitch + k0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const __nv_fp8_storage_t b = (__nv_fp8_storage_t)((w[j >> 2] >> (8 * (j & 3))) & 0xFF);
            const float v = __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3))) * sc;
            if (k0 + j < out_pitch) dst[j] = __float2bfloat16(k0 + j < cols ? v : 0.f);
        }
    }
}

static int check_mx_planes(const b200pf_planes* p, const void* scales, const char* what) {
    B200PF_REQUIRE(p && p->ptr && scales, B200PF_ERR_INVALID, "mx: %s planes / scales are null", what);
    B200PF_REQUIRE(aligned16(p->ptr) && aligned16(scales), B200PF_ERR_INVALID, "mx: %s not 16-byte aligned", what);
    B200PF_REQUIRE(p->rows > 0 && p->cols > 0 && p->nseg >= 1 && p->pitch >= p->cols && p->pitch % 16 == 0, B200PF_ERR_INVALID,
                   "mx: %s pitch %d must be >= cols %d and a multiple of 16 bytes", what, p->pitch, p->cols);
    B200PF_REQUIRE(p->plane_stride % 16 == 0 && p->plane_stride >= (long long)p->pitch * p->rows, B200PF_ERR_INVALID,
                   "mx: %s plane stride too small or not a multiple of 16", what);
    if (p->nseg > 1) {
        B200PF_REQUIRE(p->seg_stride % 16 == 0 && p->seg_stride > 0, B200PF_ERR_INVALID, "mx: %s bad segment stride", what);
        if (p->seg_is_k)
            B200PF_REQUIRE(p->cols % BK == 0, B200PF_ERR_UNSUPPORTED, "mx: %s k segments must be multiples of %d columns", what, BK);
        else
            B200PF_REQUIRE(p->rows % 128 == 0, B200PF_ERR_UNSUPPORTED, "mx: %s row segments must be multiples of 128 rows", what);
    }
    return B200PF_OK;
}

int launch_contract(const b200pf_planes* a, const b200pf_planes* b, const void* a_scales, const void* b_scales,
                    b200pf_bf16* x, long long x_plane_stride, int x_pitch, int x_row_group, long long x_group_stride,
                    int channels, cudaStream_t st) {
    int rc;
    if ((rc = check_mx_planes(a, a_scales, "A")) != B200PF_OK) return rc;
    if ((rc = check_mx_planes(b, b_scales, "B")) != B200PF_OK) return rc;
    Shape s;
    s.m_rows = (a->nseg > 1 && !a->seg_is_k) ? a->rows * a->nseg : a->rows;
    s.n_rows = (b->nseg > 1 && !b->seg_is_k) ? b->rows * b->nseg : b->rows;
    const int ka = (a->nseg > 1 && a->seg_is_k) ? a->cols * a->nseg : a->cols;
    const int kb = (b->nseg > 1 && b->seg_is_k) ? b->cols * b->nseg : b->cols;
    B200PF_REQUIRE(ka == kb, B200PF_ERR_INVALID, "mx contract: contraction lengths differ (%d vs %d)", ka, kb);
    s.k_total = ka; s.channels = channels;
    s.a_kseg_cols = (a->nseg > 1 && a->seg_is_k) ? a->cols : (ka + BK);           // never reached by k0 when unsegmented
    s.a_rowseg_rows = (a->nseg > 1 && !a->seg_is_k) ? a->rows : (s.m_rows + BM);
    s.b_kseg_cols = (b->nseg > 1 && b->seg_is_k) ? b->cols : (kb + BK);
    s.b_rowseg_rows = (b->nseg > 1 && !b->seg_is_k) ? b->rows : (s.n_rows + BN);
    const bool grouped = x_row_group > 0 && x_row_group < s.m_rows;
    s.x_row_group = grouped ? x_row_group : s.m_rows + BM;
    s.x_group_stride = grouped ? x_group_stride : 0;
    B200PF_REQUIRE(x && aligned16(x) && channels > 0 && x_pitch % 8 == 0 && x_pitch >= s.n_rows && x_plane_stride % 8 == 0 &&
                       x_plane_stride >= (long long)x_pitch * (grouped ? x_row_group : s.m_rows),
                   B200PF_ERR_INVALID, "mx contract: bad output");
    B200PF_REQUIRE(!grouped || (x_group_stride % 8 == 0 && x_group_stride >= x_plane_stride * channels), B200PF_ERR_INVALID,
                   "mx contract: bad x group stride");
    s.x_pitch = x_pitch; s.x_plane_stride = x_plane_stride;
    s.a_kgroups = mx::kgroups(a->cols); s.a_row_blocks = mx::row_blocks(a->rows);
    s.b_kgroups = mx::kgroups(b->cols); s.b_row_blocks = mx::row_blocks(b->rows);
    s.a_sf_seg = mx::scale_bytes(a->rows, a->cols, channels);
    s.b_sf_seg = mx::scale_bytes(b->rows, b->cols, channels);
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "mx contract: no device status word");
    CUtensorMap maps[2];
    const b200pf_planes* ops[2] = {a, b};
    for (int i = 0; i < 2; ++i) {
        const long long seg_stride = ops[i]->nseg > 1 ? ops[i]->seg_stride : ops[i]->plane_stride * channels;
        cuuint64_t dims[4] = {(cuuint64_t)ops[i]->cols, (cuuint64_t)ops[i]->rows, (cuuint64_t)channels, (cuuint64_t)ops[i]->nseg};
        cuuint64_t str[3] = {(cuuint64_t)ops[i]->pitch, (cuuint64_t)ops[i]->plane_stride, (cuuint64_t)seg_stride};
        cuuint32_t box[4] = {(cuuint32_t)BK, 128u, 1u, 1u};
        if ((rc = tmap_encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, const_cast<void*>(ops[i]->ptr), 4, dims, str, box,
                              CU_TENSOR_MAP_SWIZZLE_128B, i ? "mx B" : "mx A")) != B200PF_OK) return rc;
    }
    B200PF_SMEM_ATTR_ONCE(trimul_contract_mx_kernel, SMEM);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long tiles = (long long)channels * ((s.m_rows + BM - 1) / BM) * ((s.n_rows + BN - 1) / BN);
    trimul_contract_mx_kernel<<<(unsigned)(tiles < sms ? tiles : sms), THREADS, SMEM, st>>>(
        maps[0], maps[1], static_cast<const uint8_t*>(a_scales), static_cast<const uint8_t*>(b_scales), (__nv_bfloat16*)x, s, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

}  // namespace gemm_mx
}  // namespace b200pf

using namespace b200pf;

extern "C" long long b200pf_mx_scale_bytes(int rows, int cols, int channels) {
    if (rows <= 0 || cols <= 0 || channels <= 0) return 0;
    return mx::scale_bytes(rows, cols, channels);
}

extern "C" int b200pf_mx_dequant(const uint8_t* planes, const uint8_t* scales, b200pf_bf16* out, long long plane_stride,
                                 int pitch, long long out_plane_stride, int out_pitch, int rows, int cols, int channels,
                                 void* stream) {
    B200PF_REQUIRE(planes && scales && out, B200PF_ERR_INVALID, "mx_dequant: null pointer");
    B200PF_REQUIRE(rows > 0 && cols > 0 && channels > 0 && pitch % 16 == 0 && pitch >= cols && plane_stride % 16 == 0 &&
                       out_pitch % 8 == 0 && out_pitch >= cols && aligned16(planes) && aligned16(out),
                   B200PF_ERR_INVALID, "mx_dequant: bad sizes or alignment");
    const long long total = (long long)channels * rows * ((cols + 15) / 16);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    gemm_mx::mx_dequant_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        planes, scales, (__nv_bfloat16*)out, plane_stride, pitch, out_plane_stride, out_pitch, rows, cols, channels,
        mx::kgroups(cols), mx::row_blocks(rows));
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
