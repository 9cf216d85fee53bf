// Fused triangle attention on tcgen05 / TMEM (the production attention core).
//
// One CTA works on (head, 128-query tile, a PAIR of lines) at a time and walks the keys in tiles
// of 64.  Roles (352 threads):
//   warps 0-3  softmax group 0  -> line l        (thread = query row = TMEM lane)
//   warps 4-7  softmax group 1  -> line l + 1
//   warp  8    TMA producer     (bias tile shared by both lines, K and V^T tiles per line)
//   warps 9,10 MMA issuers      (one per group: S = Q K^T + bias into TMEM, then O_tile = P V)
// Per key tile and group:  S (128 x 64 fp32, TMEM) (the bf16 bias tile, fetched once for both lines, is added inside the same
// MMA chain by multiplying it with an identity tile) -> mask -> running max -> p = exp2(s - m) (fp32 ex2.approx, packed to bf16)
// -> packed bf16 pairs written back to TENSOR memory (tcgen05.st) and used from there as the A
// operand of tcgen05.mma with V^T: the probabilities never touch shared memory, whose bandwidth
// is the scarce resource of this kernel (Q, K, V^T and the bias tile are re-read every tile).
// V^T carries an extra row of ones, so column 32 of the PV result is the row sum of exactly the
// bf16 probabilities that were multiplied: no separate summation.  The running output stays in
// registers (32 fp32 per thread) and is rescaled when the maximum moves.
// Scores are in the log2 domain (host folds log2(e)/sqrt(32) into W_q and log2(e) into the bias).
// Every wait is bounded; a wait that runs out raises the status word and the CTA unwinds.
#include <stdlib.h>

#include "sm100.cuh"

namespace b200pf {
namespace atc {

constexpr int AQ = 128, AK = 64, HD = 32, PV_N = 48, ST = 4;
constexpr int BIAS_BYTES = AQ * AK * 2;          // 16384, SW128
constexpr int K_BYTES = AK * HD * 2;             // 4096,  SW64
constexpr int VT_BYTES = PV_N * AK * 2;          // 6144,  SW128 (rows 32.. are the constant rows)
constexpr int VT_TMA_BYTES = HD * AK * 2;        // 4096
constexpr int STAGE_BYTES = BIAS_BYTES + 2 * K_BYTES + 2 * VT_BYTES;     // 36864
constexpr int Q_BYTES = AQ * HD * 2;             // 8192 per line, SW64
constexpr int P_BYTES = AQ * AK * 2;             // 16384 per group, SW128
constexpr int OFF_Q = ST * STAGE_BYTES;
constexpr int OFF_IDENT = OFF_Q + 4 * Q_BYTES;     // [64 keys][64] bf16 identity, SW128: adds the bias tile inside the MMA
constexpr int IDENT_BYTES = AK * AK * 2;
constexpr int OFF_BAR = OFF_IDENT + IDENT_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
constexpr int THREADS = 352;
constexpr uint32_t TX_STAGE = BIAS_BYTES + 2 * K_BYTES + 2 * VT_TMA_BYTES;
constexpr float MASKED_SCORE = -1.0e9f * 1.4426950408889634f;

struct Args {
    const uint8_t* mask;        // [lines][mask_pitch], 1 = attend
    __nv_bfloat16* o;
    long long o_ls, o_ps;
    int mask_pitch, lines, n;
    int debug;                  // non-zero: accumulate cycle counters (profiling aid)
};

// Cycle counters of softmax group 0 / warp 0 / lane 0 of CTA 0 (profiling aid, read by b200pf_debug_counters).
__device__ long long g_att_cycles[16];

struct Bars {
    uint64_t kv_full[ST], kv_empty[ST];
    uint64_t s_full[2][2], s_empty[2][2];
    uint64_t p_full[2], pv_full[2];
    uint64_t q_full[2], q_empty[2];
    uint64_t turn[2];            // exp-phase hand-off between the two softmax groups (ping-pong)
    uint32_t tmem_slot;
    int abort_flag;
};

__device__ __forceinline__ uint64_t desc_sw64(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;     // 8 rows of 64 bytes
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;              // 64-byte swizzle
    return d;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x1(uint32_t taddr, uint32_t& r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
}
__device__ __forceinline__ float ex2_f32(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two probabilities as packed bf16.  The exponential is taken in fp32: rounding the argument to
// bf16 first (the packed ex2 form) would put up to 1 % error on each probability.
__device__ __forceinline__ uint32_t ex2_bf16x2(float lo, float hi) {
    return pack_bf16x2(ex2_f32(lo), ex2_f32(hi));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float m;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
    return m;
}

__global__ void __launch_bounds__(THREADS, 1)
triatt_core_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_vt, const __grid_constant__ CUtensorMap map_bias,
                      Args p, unsigned int* status) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Bars* B = reinterpret_cast<Bars*>(smem + OFF_BAR);
    volatile int* abort_flag = &B->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n = p.n;
    const int qtiles = (n + AQ - 1) / AQ, T = (n + AK - 1) / AK;
    const int pairs = (p.lines + 1) / 2;
    const long long items = (long long)pairs * 4 * qtiles;

    if (tid == 0) {
        for (int i = 0; i < ST; ++i) { mbar_init(&B->kv_full[i], 1); mbar_init(&B->kv_empty[i], 2); }
        for (int w = 0; w < 2; ++w) {
            for (int b = 0; b < 2; ++b) { mbar_init(&B->s_full[w][b], 1); mbar_init(&B->s_empty[w][b], 4); }
            mbar_init(&B->p_full[w], 4);
            mbar_init(&B->pv_full[w], 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(&B->q_full[i], 1); mbar_init(&B->q_empty[i], 2); }
        mbar_init(&B->turn[0], 4);
        mbar_init(&B->turn[1], 4);
        B->abort_flag = 0;
        fence_barrier_init();
    }
    // constant rows of every V^T tile: row 32 = ones (row-sum column), rows 33..47 = zeros
    for (int i = tid; i < ST * 2 * (PV_N - HD) * (AK * 2 / 16); i += THREADS) {
        int chunk = i % 8, row = (i / 8) % (PV_N - HD), tile = i / (8 * (PV_N - HD));
        uint8_t* base = smem + (tile >> 1) * STAGE_BYTES + BIAS_BYTES + 2 * K_BYTES + (tile & 1) * VT_BYTES;
        uint32_t v = row == 0 ? 0x3F803F80u : 0u;       // bf16 1.0 pairs
        *reinterpret_cast<uint4*>(base + (HD + row) * 128 + chunk * 16) = make_uint4(v, v, v, v);
    }
    // identity tile I[n][k] = (n == k): S += bias_tile * I^T adds bias[q][key] exactly (bf16 x 1, fp32 accumulate)
    for (int i = tid; i < AK * 8; i += THREADS) {
        int row = i >> 3, chunk = i & 7;
        uint32_t w4[4] = {0u, 0u, 0u, 0u};
        if ((row >> 3) == chunk) w4[(row & 7) >> 1] = (row & 1) ? 0x3F800000u : 0x00003F80u;
        *reinterpret_cast<uint4*>(smem + OFF_IDENT + row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    fence_proxy_async();
    if (warp == 9) { tmem_alloc(&B->tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = B->tmem_slot;

    auto decode = [&](long long it, int& qt, int& h, int& line0) {
        qt = (int)(it % qtiles);
        h = (int)((it / qtiles) & 3);
        line0 = (int)(it / (qtiles * 4)) * 2;
    };
    auto clamp_line = [&](int l) { return l < p.lines ? l : p.lines - 1; };

    if (warp == 8) {
        if (lane == 0) {
            // ------------------------------ TMA producer ------------------------------
            uint32_t g = 0, qn = 0;
            bool ok = true;
            for (long long it = blockIdx.x; it < items && ok; it += gridDim.x, ++qn) {
                int qt, h, line0;
                decode(it, qt, h, line0);
                const uint32_t qb = qn & 1, qph = (qn >> 1) & 1;           // Q tiles are double buffered across items
                ok = mbar_wait(&B->q_empty[qb], qph ^ 1, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(&B->q_full[qb], 2 * Q_BYTES);
                for (int w = 0; w < 2; ++w)
                    tma_load_4d(smem + OFF_Q + (qb * 2 + w) * Q_BYTES, &map_q, &B->q_full[qb], 0, h, qt * AQ, clamp_line(line0 + w));
                for (int j = 0; j < T; ++j, ++g) {
                    uint32_t stage = g % ST, phase = (g / ST) & 1;
                    ok = mbar_wait(&B->kv_empty[stage], phase ^ 1, abort_flag);
                    if (!ok) break;
                    uint8_t* st = smem + stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(&B->kv_full[stage], TX_STAGE);
                    tma_load_3d(st, &map_bias, &B->kv_full[stage], j * AK, h, qt * AQ);
                    for (int w = 0; w < 2; ++w) {
                        int line = clamp_line(line0 + w);
                        tma_load_4d(st + BIAS_BYTES + w * K_BYTES, &map_k, &B->kv_full[stage], 0, h, j * AK, line);
                        tma_load_4d(st + BIAS_BYTES + 2 * K_BYTES + w * VT_BYTES, &map_vt, &B->kv_full[stage], j * AK, 0, h, line);
                    }
                }
            }
            if (!ok) {
                atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
                uint64_t t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (warp == 9 || warp == 10) {
        if (lane == 0) {
            // ------------------------------ MMA issuer of softmax group w ------------------------------
            // One issuing thread per group: S of the next key tile goes out a full iteration ahead of
            // the group that consumes it, and the two groups do not wait on each other's P tiles.
            const int w = warp - 9;
            constexpr uint32_t idesc_s = make_idesc_bf16(AQ, AK);
            constexpr uint32_t idesc_pv = make_idesc_bf16(AQ, PV_N);
            const uint32_t ident_addr = smem_u32(smem + OFF_IDENT);
            uint32_t g = 0, qn = 0, s_cnt = 0, p_cnt = 0;
            bool ok = true;
            auto issue_s = [&](uint32_t stage, uint32_t q_addr) -> bool {
                uint32_t b = s_cnt & 1, ph = (s_cnt >> 1) & 1;
                if (!mbar_wait(&B->s_empty[w][b], ph ^ 1, abort_flag)) return false;
                tc_fence_after();
                uint32_t bias_addr = smem_u32(smem + stage * STAGE_BYTES);
                uint32_t k_addr = bias_addr + BIAS_BYTES + w * K_BYTES;
                uint32_t d = tmem_base + (uint32_t)((w * 2 + b) * AK);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    umma_bf16(d, desc_sw64(q_addr + kk * 32), desc_sw64(k_addr + kk * 32), idesc_s, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < AK / 16; ++kk)
                    umma_bf16(d, make_desc_k_sw128(bias_addr + kk * 32), make_desc_k_sw128(ident_addr + kk * 32), idesc_s, 1u);
                umma_commit(&B->s_full[w][b]);
                ++s_cnt;
                return true;
            };
            for (long long it = blockIdx.x; it < items && ok; it += gridDim.x, ++qn) {
                const uint32_t qb = qn & 1, qph = (qn >> 1) & 1;
                const uint32_t q_addr = smem_u32(smem + OFF_Q + (qb * 2 + w) * Q_BYTES);
                ok = mbar_wait(&B->q_full[qb], qph, abort_flag) && mbar_wait(&B->kv_full[g % ST], (g / ST) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                ok = issue_s(g % ST, q_addr);
                if (ok && T == 1) umma_commit(&B->q_empty[qb]);
                for (int j = 0; j < T && ok; ++j, ++g) {
                    const uint32_t stage = g % ST;
                    if (j + 1 < T) {
                        const uint32_t g1 = g + 1;
                        ok = mbar_wait(&B->kv_full[g1 % ST], (g1 / ST) & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        ok = issue_s(g1 % ST, q_addr);
                        if (!ok) break;
                        if (j + 2 == T) umma_commit(&B->q_empty[qb]);
                    }
                    ok = mbar_wait(&B->p_full[w], p_cnt & 1, abort_flag);
                    if (!ok) break;
                    ++p_cnt;
                    tc_fence_after();
                    const uint32_t vt_addr = smem_u32(smem + stage * STAGE_BYTES + BIAS_BYTES + 2 * K_BYTES + w * VT_BYTES);
                    const uint32_t d = tmem_base + 256u + (uint32_t)(w * 64);
#pragma unroll
                    for (int kk = 0; kk < AK / 16; ++kk)
                        umma_bf16_ts(d, tmem_base + 384u + (uint32_t)(w * 32 + kk * 8), make_desc_k_sw128(vt_addr + kk * 32),
                                     idesc_pv, kk ? 1u : 0u);
                    umma_commit(&B->pv_full[w]);
                    umma_commit(&B->kv_empty[stage]);
                }
            }
            if (!ok) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
        }
    } else {
        // ------------------------------ softmax groups ------------------------------
        const int w = warp >> 2, quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        uint32_t g = 0, s_cnt = 0, pv_cnt = 0, turn_cnt = 0;
        bool ok = true;
        for (long long it = blockIdx.x; it < items && ok; it += gridDim.x) {
            int qt, h, line0;
            decode(it, qt, h, line0);
            const int line = line0 + w;
            const uint8_t* mrow = p.mask + (long long)clamp_line(line) * p.mask_pitch;
            float o_acc[HD];
#pragma unroll
            for (int e = 0; e < HD; ++e) o_acc[e] = 0.f;
            float m_run = -INFINITY, l_run = 0.f;
            for (int j = 0; j < T && ok; ++j, ++g) {
                const uint32_t stage = g % ST;
                long long c0 = clock64();
                // mask bytes of this key tile (same for every thread of the group)
                uint32_t mw[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 v = __ldg(reinterpret_cast<const uint4*>(mrow + j * AK) + c);
                    mw[c * 4] = v.x; mw[c * 4 + 1] = v.y; mw[c * 4 + 2] = v.z; mw[c * 4 + 3] = v.w;
                }
                uint32_t all = 0x01010101u;
#pragma unroll
                for (int c = 0; c < 16; ++c) all &= mw[c];
                const bool fast = (all == 0x01010101u) && (j * AK + AK <= n);
                // scores
                uint32_t b = s_cnt & 1, ph = (s_cnt >> 1) & 1;
                long long c1 = clock64();
                ok = mbar_wait(&B->s_full[w][b], ph, abort_flag);
                if (!ok) break;
                ++s_cnt;
                tc_fence_after();
                long long c2 = clock64();
                uint32_t sr[2][32];
                tmem_ld_32x32(tmem_base + lane_off + (uint32_t)((w * 2 + b) * AK), sr[0]);
                tmem_ld_32x32(tmem_base + lane_off + (uint32_t)((w * 2 + b) * AK + 32), sr[1]);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B->s_empty[w][b]);
                long long c3 = clock64();
                float s[64];
#pragma unroll
                for (int e = 0; e < 64; ++e) s[e] = __uint_as_float(sr[e >> 5][e & 31]);
                float mx = m_run;
                if (fast) {
                    float m4[4] = {mx, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int e = 0; e < 64; e += 8) {
                        m4[0] = max3(m4[0], s[e], s[e + 1]);
                        m4[1] = max3(m4[1], s[e + 2], s[e + 3]);
                        m4[2] = max3(m4[2], s[e + 4], s[e + 5]);
                        m4[3] = max3(m4[3], s[e + 6], s[e + 7]);
                    }
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                } else {
#pragma unroll
                    for (int e = 0; e < 64; ++e) {
                        uint32_t mbyte = (mw[e >> 2] >> ((e & 3) * 8)) & 0xffu;
                        float v = (j * AK + e >= n) ? -INFINITY : (mbyte ? s[e] : MASKED_SCORE);
                        s[e] = v;
                        mx = fmaxf(mx, v);
                    }
                }
                const float scale = ex2_f32(m_run - mx);                // first tile: exp2(-inf) = 0
                m_run = mx;
                long long c4 = clock64(), c5 = c4, c6 = c4;
                // fold in the previous tile's P V (computed with the previous maximum), then rescale
                if (j > 0) {
                    ok = mbar_wait(&B->pv_full[w], pv_cnt & 1, abort_flag);
                    if (!ok) break;
                    ++pv_cnt;
                    tc_fence_after();
                    c5 = clock64();
                    uint32_t pv[32], ps;
                    tmem_ld_32x32(tmem_base + lane_off + 256u + (uint32_t)(w * 64), pv);
                    tmem_ld_x1(tmem_base + lane_off + 256u + (uint32_t)(w * 64 + HD), ps);
                    tmem_ld_wait();
                    tc_fence_before();
#pragma unroll
                    for (int e = 0; e < HD; ++e) o_acc[e] = (o_acc[e] + __uint_as_float(pv[e])) * scale;
                    l_run = (l_run + __uint_as_float(ps)) * scale;
                    c6 = clock64();
                }
                // probabilities -> packed bf16 pairs in tensor memory: the A operand of the P V product
                long long c7 = clock64();
                {
                    uint32_t pw[32];
#pragma unroll
                    for (int e = 0; e < 32; ++e) pw[e] = ex2_bf16x2(s[2 * e] - mx, s[2 * e + 1] - mx);
                    tmem_st_32x32(tmem_base + lane_off + 384u + (uint32_t)(w * 32), pw);
                    tmem_st_wait();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B->p_full[w]);
                if (p.debug && blockIdx.x == 0 && warp == 0 && lane == 0) {
                    long long c8 = clock64();
                    g_att_cycles[0] += c1 - c0;   // mask loads
                    g_att_cycles[1] += c2 - c1;   // wait S
                    g_att_cycles[2] += c3 - c2;   // tcgen05.ld S
                    g_att_cycles[3] += c4 - c3;   // max + scale
                    g_att_cycles[4] += c5 - c4;   // wait PV
                    g_att_cycles[5] += c6 - c5;   // ld PV + O update
                    g_att_cycles[6] += c7 - c6;   // wait turn
                    g_att_cycles[7] += c8 - c7;   // exp + P store + fences
                    g_att_cycles[8] += 1;
                }
            }
            if (!ok) break;
            // last tile's P V, normalise, store
            ok = mbar_wait(&B->pv_full[w], pv_cnt & 1, abort_flag);
            if (!ok) break;
            ++pv_cnt;
            tc_fence_after();
            {
                uint32_t pv[32], ps;
                tmem_ld_32x32(tmem_base + lane_off + 256u + (uint32_t)(w * 64), pv);
                tmem_ld_x1(tmem_base + lane_off + 256u + (uint32_t)(w * 64 + HD), ps);
                tmem_ld_wait();
                tc_fence_before();
#pragma unroll
                for (int e = 0; e < HD; ++e) o_acc[e] += __uint_as_float(pv[e]);
                l_run += __uint_as_float(ps);
            }
            const int qi = qt * AQ + row;
            if (line < p.lines && qi < n) {
                const float inv = 1.f / l_run;
                __nv_bfloat16* dst = p.o + (long long)line * p.o_ls + (long long)qi * p.o_ps + h * HD;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 v;
                    v.x = pack_bf16x2(o_acc[c * 8 + 0] * inv, o_acc[c * 8 + 1] * inv);
                    v.y = pack_bf16x2(o_acc[c * 8 + 2] * inv, o_acc[c * 8 + 3] * inv);
                    v.z = pack_bf16x2(o_acc[c * 8 + 4] * inv, o_acc[c * 8 + 5] * inv);
                    v.w = pack_bf16x2(o_acc[c * 8 + 6] * inv, o_acc[c * 8 + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + c * 8) = v;
                }
            }
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}
static int encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box, CUtensorMapSwizzle sw, const char* what) {
    EncodeTiledFn fn = encode_fn();
    B200PF_REQUIRE(fn != nullptr, B200PF_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200PF_REQUIRE(r == CUDA_SUCCESS, B200PF_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return B200PF_OK;
}

}  // namespace atc
}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_triatt_core_tc(const b200pf_bf16* q, const b200pf_bf16* k, const b200pf_bf16* vt, int vt_pitch,
                                     const b200pf_bf16* bias, long long bias_hs, long long bias_qs,
                                     const uint8_t* mask_lines, int mask_pitch,
                                     b200pf_bf16* o, long long o_line_stride, long long o_pos_stride,
                                     int lines, int n, void* stream) {
    using namespace atc;
    B200PF_REQUIRE(q && k && vt && bias && mask_lines && o && lines > 0 && n > 0, B200PF_ERR_INVALID, "triatt_core_tc: bad argument");
    B200PF_REQUIRE(aligned16(q) && aligned16(k) && aligned16(vt) && aligned16(bias) && aligned16(o) && aligned16(mask_lines),
                   B200PF_ERR_INVALID, "triatt_core_tc: pointers must be 16-byte aligned");
    B200PF_REQUIRE(vt_pitch % 8 == 0 && vt_pitch >= n && bias_hs % 8 == 0 && bias_qs % 8 == 0 && bias_hs >= n,
                   B200PF_ERR_INVALID, "triatt_core_tc: pitches / strides must be multiples of 8 elements and >= n");
    B200PF_REQUIRE(mask_pitch % 16 == 0 && mask_pitch >= (n + AK - 1) / AK * AK, B200PF_ERR_INVALID,
                   "triatt_core_tc: mask pitch must be a multiple of 16 and cover n rounded up to 64");
    B200PF_REQUIRE(o_line_stride % 8 == 0 && o_pos_stride % 8 == 0, B200PF_ERR_INVALID, "triatt_core_tc: bad o strides");
    CUtensorMap mq, mk, mvt, mb;
    int rc;
    {   // q, k: [line][pos][head][32]; coordinates (d, head, pos, line)
        cuuint64_t dims[4] = {(cuuint64_t)HD, 4, (cuuint64_t)n, (cuuint64_t)lines};
        cuuint64_t str[3] = {(cuuint64_t)HD * 2, (cuuint64_t)4 * HD * 2, (cuuint64_t)n * 4 * HD * 2};
        cuuint32_t boxq[4] = {HD, 1, AQ, 1}, boxk[4] = {HD, 1, AK, 1};
        if ((rc = encode(&mq, q, 4, dims, str, boxq, CU_TENSOR_MAP_SWIZZLE_64B, "q")) != B200PF_OK) return rc;
        if ((rc = encode(&mk, k, 4, dims, str, boxk, CU_TENSOR_MAP_SWIZZLE_64B, "k")) != B200PF_OK) return rc;
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)HD, 4, (cuuint64_t)lines};
        cuuint64_t str[3] = {(cuuint64_t)vt_pitch * 2, (cuuint64_t)HD * vt_pitch * 2, (cuuint64_t)4 * HD * vt_pitch * 2};
        cuuint32_t box[4] = {AK, HD, 1, 1};
        if ((rc = encode(&mvt, vt, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "vt")) != B200PF_OK) return rc;
    }
    {
        cuuint64_t dims[3] = {(cuuint64_t)n, 4, (cuuint64_t)n};
        cuuint64_t str[2] = {(cuuint64_t)bias_hs * 2, (cuuint64_t)bias_qs * 2};
        cuuint32_t box[3] = {AK, 1, AQ};
        if ((rc = encode(&mb, bias, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "bias")) != B200PF_OK) return rc;
    }
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "triatt_core_tc: no device status word");
    B200PF_SMEM_ATTR_ONCE(triatt_core_tc_kernel, SMEM_BYTES);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long items = (long long)((lines + 1) / 2) * 4 * ((n + AQ - 1) / AQ);
    Args a{mask_lines, (__nv_bfloat16*)o, o_line_stride, o_pos_stride, mask_pitch, lines, n, getenv("B200PF_ATT_DEBUG") != nullptr};
    triatt_core_tc_kernel<<<(unsigned)(items < sms ? items : sms), THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(mq, mk, mvt, mb, a, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

// Profiling aid: copies (and clears) the attention kernel's cycle counters; synchronises the device.
extern "C" int b200pf_debug_counters(long long* host_out, int n) {
    B200PF_REQUIRE(host_out && n > 0 && n <= 16, B200PF_ERR_INVALID, "debug_counters: bad argument");
    long long tmp[16] = {0};
    B200PF_CUDA(cudaDeviceSynchronize());
    B200PF_CUDA(cudaMemcpyFromSymbol(tmp, atc::g_att_cycles, sizeof(tmp)));
    for (int i = 0; i < n; ++i) host_out[i] = tmp[i];
    long long zero[16] = {0};
    B200PF_CUDA(cudaMemcpyToSymbol(atc::g_att_cycles, zero, sizeof(zero)));
    return B200PF_OK;
}
