// Fused triangle attention on tcgen05 / TMEM, four lines per CTA.
//
// One CTA works on (head, 128-query tile, four consecutive lines that share the bias tile).  Roles (608 threads):
//   warps 0-15  softmax group g = warp / 4 -> line l + g   (thread = query row = TMEM lane); four groups, i.e.
//               four warps per scheduler, so that one group's exponentials run in the latency gaps of the others
//   warp  16    TMA producer   (bias tile shared by the four lines; K and V^T tiles per line)
//   warps 17,18 MMA issuers    (one per pair of groups; a polling state machine over both groups' next scores and
//                               P V products, so a group that is not ready never holds up the other.  The whole warp
//                               runs it and one elected lane issues.)
// Per key tile of 64 and group: S_g (128 x 64 fp32, TMEM) = bias_tile x I^T (the bf16 bias lands in the score columns
// exactly), then S_g += Q_g K_g^T.  (Producing the scores of a pair's two groups together, one bias product for
// both, made each group wait for the other to release its columns: 2 % slower.)  The softmax thread reads its row
// in two halves, applies the key mask and computes p = exp2(s - m) in ONE pass with the reference m of the tiles
// before (scaling by a stale reference is exact in floating point; a check keeps it far from overflow and hands the
// rare tile that fails it, like the first tile of a line, to a two-pass path).  p goes back to TENSOR memory as
// packed bf16, the A operand of O_g += P_g V_g^T.  The running output stays in tensor memory and is rescaled only
// when a row maximum has grown by more than 2^8; row sums are kept in fp32 registers.
// TMEM columns: S 4 x 64 | P 4 x 32 | O 4 x 32 = 512.  S and P are single-buffered; S is released as soon as its
// second half is in registers, so the next tile's products run under this tile's exponentials.
// What bounds it (measured by leaving parts out): with no softmax arithmetic at all the MMA / barrier skeleton takes
// 1.08 ms at N = 1024 (every tcgen05.mma costs its issuing thread ~40 clocks and every tcgen05.commit ~75, and the
// bias product alone 0.22 ms); with the softmax arithmetic and only the Q K^T products 1.36 ms; together 1.45 ms
// (1.43 ms since the groups of a pair get their scores independently).
// Scores are in the log2 domain (host folds log2(e)/sqrt(32) into W_q and log2(e) into the bias).
// Every wait is bounded; a wait that runs out raises the status word and the CTA unwinds.
#include "sm100.cuh"
#include "tmap.cuh"

namespace b200pf {
namespace atc4 {

constexpr int AQ = 128, AK = 64, HD = 32, ST = 3, NG = 4;
constexpr int BIAS_BYTES = AQ * AK * 2;          // 16384, SW128
constexpr int K_BYTES = AK * HD * 2;             // 4096,  SW64
constexpr int VT_BYTES = HD * AK * 2;            // 4096,  SW128
constexpr int STAGE_BYTES = BIAS_BYTES + NG * (K_BYTES + VT_BYTES);      // 49152
constexpr int Q_BYTES = AQ * HD * 2;             // 8192 per line, SW64
constexpr int OFF_Q = ST * STAGE_BYTES;          // 2 buffers x 4 lines
constexpr int OFF_IDENT = OFF_Q + 2 * NG * Q_BYTES;   // [128 n][64 k] bf16, SW128: I stacked twice
constexpr int IDENT_BYTES = 2 * AK * AK * 2;
constexpr int OFF_BAR = OFF_IDENT + IDENT_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 512;        // 229,888: the dynamic window must start 1024-byte aligned
constexpr int THREADS = 19 * 32;
constexpr int TMA_WARP = 16, MMA_WARP0 = 17;
constexpr uint32_t COL_S = 0, COL_P = 256, COL_O = 384;
constexpr float MASKED_SCORE = -1.0e9f * 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;
constexpr float ONE_PASS_HEADROOM = 64.f;        // a one-pass tile may exceed its reference by 2^64 at most

struct Args {
    const uint8_t* mask;        // [lines][mask_pitch], 1 = attend
    __nv_bfloat16* o;
    long long o_ls, o_ps;
    int mask_pitch, lines, n;
};

struct Bars {
    uint64_t kv_full[ST], kv_empty[ST];
    uint64_t s_full[NG], s_empty[NG], p_full[NG], pv_done[NG];
    uint64_t q_full[2], q_empty[2];
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
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ float ex2_f32(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float m;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
    return m;
}
// Two fp32 values in one 64-bit register for the packed add (one instruction, two results).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// Masked keys of a full tile get the score the reference's fp32 sum rounds to.  `even` / `odd` hold one bit per
// key pair (bit l: key 2l / 2l+1 attends); they are uniform over the warp, so every test is a uniform branch and a
// tile (or a group of 8 keys) without masked keys costs one compare.
template <int HF>
__device__ __forceinline__ void mask_half(uint32_t (&sr)[32], uint32_t even, uint32_t odd) {
    const uint32_t e16 = (even >> (HF * 16)) & 0xffffu, o16 = (odd >> (HF * 16)) & 0xffffu, b16 = e16 & o16;
    if (b16 == 0xffffu) return;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (((b16 >> (4 * q)) & 0xfu) == 0xfu) continue;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int pe = 4 * q + t;
            if (!((e16 >> pe) & 1u)) sr[2 * pe] = __float_as_uint(MASKED_SCORE);
            if (!((o16 >> pe) & 1u)) sr[2 * pe + 1] = __float_as_uint(MASKED_SCORE);
        }
    }
}
// The same for any tile: keys at or beyond n (tile padding) are excluded altogether.
__device__ __forceinline__ void mask_half_general(uint32_t (&sr)[32], uint32_t even, uint32_t odd, int hf, int key0, int n) {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
        const int pe = hf * 16 + (e >> 1);
        const uint32_t bit = (((e & 1) ? odd : even) >> pe) & 1u;
        const int key = key0 + hf * 32 + e;
        sr[e] = (key >= n) ? __float_as_uint(-INFINITY) : (bit ? sr[e] : __float_as_uint(MASKED_SCORE));
    }
}
__device__ __forceinline__ void max_half(const uint32_t (&sr)[32], float (&m4)[4]) {
#pragma unroll
    for (int e = 0; e < 32; e += 8) {
        m4[0] = max3(m4[0], __uint_as_float(sr[e]), __uint_as_float(sr[e + 1]));
        m4[1] = max3(m4[1], __uint_as_float(sr[e + 2]), __uint_as_float(sr[e + 3]));
        m4[2] = max3(m4[2], __uint_as_float(sr[e + 4]), __uint_as_float(sr[e + 5]));
        m4[3] = max3(m4[3], __uint_as_float(sr[e + 6]), __uint_as_float(sr[e + 7]));
    }
}
// p = exp2(s - m) for 32 scores -> 16 packed bf16 pairs; the subtraction and the row sums use the packed fp32 add.
__device__ __forceinline__ void exp_half(const uint32_t (&sr)[32], uint32_t (&pw)[16], uint64_t negm2, uint64_t& l2a, uint64_t& l2b) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        float x0, x1;
        f2_unpack(f2_add(f2_pack(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1])), negm2), x0, x1);
        const float p0 = ex2_f32(x0), p1 = ex2_f32(x1);
        if (e & 1) l2b = f2_add(l2b, f2_pack(p0, p1));
        else l2a = f2_add(l2a, f2_pack(p0, p1));
        pw[e] = pack_bf16x2(p0, p1);
    }
}
// Gives up (false) after ~2 s without progress or when another thread of the CTA has aborted.
struct IdleGuard {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    __device__ __forceinline__ bool keep_waiting(volatile int* abort_flag) {
        if ((++spins & 1023u) != 0) return true;
        if (*abort_flag) return false;
        const uint64_t now = sm100::global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > sm100::WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
        return true;
    }
    __device__ __forceinline__ void reset() { spins = 0; t0 = 0; }
};

__global__ void __launch_bounds__(THREADS, 1)
triatt_core_tc4_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_vt, const __grid_constant__ CUtensorMap map_bias,
                       Args p, unsigned int* status) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {       // swizzled tiles need 1024-byte alignment; there is no slack to fix it up
        if (threadIdx.x == 0) atomicOr(status, DEV_STATUS_BAD_INDEX);
        return;
    }
    Bars* B = reinterpret_cast<Bars*>(smem + OFF_BAR);
    volatile int* abort_flag = &B->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n = p.n;
    const int qtiles = (n + AQ - 1) / AQ, T = (n + AK - 1) / AK;
    const int quads = (p.lines + NG - 1) / NG;
    const long long items = (long long)quads * 4 * qtiles;
    const uint32_t my_items = blockIdx.x < items ? (uint32_t)((items - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0u;
    const uint32_t total_tiles = my_items * (uint32_t)T;

    if (tid == 0) {
        for (int i = 0; i < ST; ++i) { mbar_init(&B->kv_full[i], 1); mbar_init(&B->kv_empty[i], 2); }
        for (int g = 0; g < NG; ++g) {
            mbar_init(&B->s_full[g], 1); mbar_init(&B->s_empty[g], 4);
            mbar_init(&B->p_full[g], 4); mbar_init(&B->pv_done[g], 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(&B->q_full[i], 1); mbar_init(&B->q_empty[i], 2); }
        B->abort_flag = 0;
        fence_barrier_init();
    }
    // 64 x 64 identity as the B operand: bias_tile x I^T puts bias[q][k] into score column k (bf16 x 1 with fp32
    // accumulation: exact)
    for (int i = tid; i < AK * 8; i += THREADS) {
        const int row = i >> 3, chunk = i & 7, k = row & (AK - 1);
        uint32_t w4[4] = {0u, 0u, 0u, 0u};
        if ((k >> 3) == chunk) w4[(k & 7) >> 1] = (k & 1) ? 0x3F800000u : 0x00003F80u;
        *reinterpret_cast<uint4*>(smem + OFF_IDENT + row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    fence_proxy_async();
    if (warp == MMA_WARP0) { tmem_alloc(&B->tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = B->tmem_slot;

    auto decode = [&](long long it, int& qt, int& h, int& line0) {
        qt = (int)(it % qtiles);
        h = (int)((it / qtiles) & 3);
        line0 = (int)(it / (qtiles * 4)) * NG;
    };
    auto clamp_line = [&](int l) { return l < p.lines ? l : p.lines - 1; };

    if (warp == TMA_WARP) {
        if (lane == 0) {
            // ------------------------------ TMA producer ------------------------------
            uint32_t G = 0, k = 0;
            bool ok = true;
            for (long long it = blockIdx.x; it < items && ok; it += gridDim.x, ++k) {
                int qt, h, line0;
                decode(it, qt, h, line0);
                const uint32_t qb = k & 1;
                ok = mbar_wait(&B->q_empty[qb], ((k >> 1) & 1) ^ 1, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(&B->q_full[qb], NG * Q_BYTES);
                for (int g = 0; g < NG; ++g)
                    tma_load_4d(smem + OFF_Q + (qb * NG + g) * Q_BYTES, &map_q, &B->q_full[qb], 0, h, qt * AQ, clamp_line(line0 + g));
                for (int j = 0; j < T; ++j, ++G) {
                    const uint32_t stage = G % ST;
                    ok = mbar_wait(&B->kv_empty[stage], ((G / ST) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    uint8_t* st = smem + stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(&B->kv_full[stage], STAGE_BYTES);
                    tma_load_3d(st, &map_bias, &B->kv_full[stage], j * AK, h, qt * AQ);
                    for (int g = 0; g < NG; ++g) {
                        const int line = clamp_line(line0 + g);
                        tma_load_4d(st + BIAS_BYTES + g * K_BYTES, &map_k, &B->kv_full[stage], 0, h, j * AK, line);
                        tma_load_4d(st + BIAS_BYTES + NG * K_BYTES + g * VT_BYTES, &map_vt, &B->kv_full[stage], j * AK, 0, h, line);
                    }
                }
            }
            if (!ok) {
                atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
                uint64_t t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (warp >= MMA_WARP0) {
        // ------------------------------ MMA issuer of the group pair pr ------------------------------
        // Run by the WHOLE warp with warp-uniform state; one elected lane issues, so that descriptors and
        // barrier addresses stay in uniform registers (issued from a divergent `lane == 0` branch, every
        // tcgen05 instruction cost the thread ~100 clocks instead of ~40, measured with clock64).  Polls with
        // the non-blocking test_wait what is ready instead of blocking on one barrier: the next S of the
        // pair, and the P V product of either group.  Tiles are counted over all items of this CTA.
        const int pr = __shfl_sync(0xffffffffu, warp - MMA_WARP0, 0), g0 = 2 * pr;
        constexpr uint32_t idesc_s = make_idesc_bf16(AQ, AK), idesc_bias = idesc_s;
        constexpr uint32_t idesc_pv = make_idesc_bf16(AQ, HD);
        // every descriptor is a precomputed base plus a small constant (the address field counts 16-byte
        // units; a K step of 16 bf16 is 32 bytes = 2)
        constexpr uint64_t STAGE_STEP = STAGE_BYTES >> 4, Q_STEP = (NG * Q_BYTES) >> 4;
        const uint64_t d_ident = make_desc_k_sw128(smem_u32(smem + OFF_IDENT));
        const uint64_t d_bias0 = make_desc_k_sw128(smem_u32(smem));
        const uint64_t d_k0[2] = {desc_sw64(smem_u32(smem + BIAS_BYTES + g0 * K_BYTES)),
                                  desc_sw64(smem_u32(smem + BIAS_BYTES + (g0 + 1) * K_BYTES))};
        const uint64_t d_vt0[2] = {make_desc_k_sw128(smem_u32(smem + BIAS_BYTES + NG * K_BYTES + g0 * VT_BYTES)),
                                   make_desc_k_sw128(smem_u32(smem + BIAS_BYTES + NG * K_BYTES + (g0 + 1) * VT_BYTES))};
        const uint64_t d_q0[2] = {desc_sw64(smem_u32(smem + OFF_Q + g0 * Q_BYTES)), desc_sw64(smem_u32(smem + OFF_Q + (g0 + 1) * Q_BYTES))};
        const uint32_t t_s = tmem_base + COL_S + (uint32_t)(g0 * AK);
        const uint32_t t_p = tmem_base + COL_P + (uint32_t)(g0 * (AK / 2));
        const uint32_t t_o = tmem_base + COL_O + (uint32_t)(g0 * HD);
        uint32_t Gs[2] = {0u, 0u}, Gp[2] = {0u, 0u};
        uint32_t js[2] = {0u, 0u}, ks[2] = {0u, 0u}, stage_s[2] = {0u, 0u}, phase_s[2] = {0u, 0u};   // per group: the next S
        uint32_t jp[2] = {0u, 0u}, stage_p[2] = {0u, 0u};
        IdleGuard guard;
        bool ok = true;
        while (ok && (Gp[0] < total_tiles || Gp[1] < total_tiles)) {
            bool progress = false;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (Gs[i] < total_tiles) {
                    const uint32_t qb = ks[i] & 1;
                    if (mbar_test_wait(&B->kv_full[stage_s[i]], phase_s[i]) && mbar_test_wait(&B->s_empty[g0 + i], (Gs[i] & 1) ^ 1) &&
                        (js[i] != 0 || mbar_test_wait(&B->q_full[qb], (ks[i] >> 1) & 1))) {
                        tc_fence_after();
                        if (elect_one()) {
                            const uint64_t so = stage_s[i] * STAGE_STEP;
                            const uint32_t ts = t_s + (uint32_t)(i * AK);
#pragma unroll
                            for (int kk = 0; kk < AK / 16; ++kk)
                                umma_bf16(ts, d_bias0 + so + 2 * kk, d_ident + 2 * kk, idesc_bias, kk ? 1u : 0u);
#pragma unroll
                            for (int kk = 0; kk < HD / 16; ++kk)
                                umma_bf16(ts, d_q0[i] + qb * Q_STEP + 2 * kk, d_k0[i] + so + 2 * kk, idesc_s, 1u);
                            umma_commit(&B->s_full[g0 + i]);
                            // the later of the pair's two groups to issue the item's last scores frees the Q tiles
                            if (js[i] == (uint32_t)T - 1 && Gs[1 - i] > Gs[i]) umma_commit(&B->q_empty[qb]);
                        }
                        __syncwarp();
                        ++Gs[i];
                        if (++js[i] == (uint32_t)T) { js[i] = 0; ++ks[i]; }
                        if (++stage_s[i] == ST) { stage_s[i] = 0; phase_s[i] ^= 1; }
                        progress = true;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t G = Gp[i];
                if (G < Gs[i] && mbar_test_wait(&B->p_full[g0 + i], G & 1)) {
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t dv = d_vt0[i] + stage_p[i] * STAGE_STEP;
                        const uint32_t d = t_o + (uint32_t)(i * HD), a = t_p + (uint32_t)(i * (AK / 2));
                        if (jp[i] == 0) umma_bf16_ts(d, a, dv, idesc_pv, 0u);
                        else umma_bf16_ts(d, a, dv, idesc_pv, 1u);
#pragma unroll
                        for (int kk = 1; kk < AK / 16; ++kk) umma_bf16_ts(d, a + (uint32_t)(kk * 8), dv + 2 * kk, idesc_pv, 1u);
                        umma_commit(&B->pv_done[g0 + i]);
                        if (Gp[1 - i] > G) umma_commit(&B->kv_empty[stage_p[i]]);     // both groups of the pair are through this stage
                    }
                    __syncwarp();
                    Gp[i] = G + 1;
                    if (++jp[i] == (uint32_t)T) jp[i] = 0;
                    if (++stage_p[i] == ST) stage_p[i] = 0;
                    progress = true;
                }
            }
            if (progress) guard.reset();
            else ok = __all_sync(0xffffffffu, guard.keep_waiting(abort_flag));
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else {
        // ------------------------------ softmax groups ------------------------------
        const int g = warp >> 2, quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_off + COL_S + (uint32_t)(g * AK);
        const uint32_t p_addr = tmem_base + lane_off + COL_P + (uint32_t)(g * (AK / 2));
        const uint32_t o_addr = tmem_base + lane_off + COL_O + (uint32_t)(g * HD);
        uint32_t G = 0;
        bool ok = true;
        // The key mask of a line is the same for every query row, i.e. uniform over the warp: lane l fetches the
        // mask bytes of keys 2l and 2l+1 of the NEXT tile, and two ballots turn them into one bit per key.
        auto mask_fetch = [&](const uint8_t* mrow, int j) -> uint32_t {
            return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(mrow + j * AK) + lane);
        };
        for (long long it = blockIdx.x; it < items && ok; it += gridDim.x) {
            int qt, h, line0;
            decode(it, qt, h, line0);
            const int line = line0 + g;
            const uint8_t* mrow = p.mask + (long long)clamp_line(line) * p.mask_pitch;
            // m_used: the reference the stored probabilities and the running output are scaled by; m_seen: the
            // largest score met so far.  They differ by at most RESCALE_STEP after a rescale, and by whatever one
            // tile of the one-pass path has added since (bounded by ONE_PASS_HEADROOM).
            float m_used = 0.f, m_seen = 0.f, l_run = 0.f;
            bool pending = false;                       // warp-uniform: some row is due for a rescale
            uint32_t vnext = mask_fetch(mrow, 0);
            for (int j = 0; j < T && ok; ++j, ++G) {
                const uint32_t even = __ballot_sync(0xffffffffu, (vnext & 0x00ffu) != 0);    // bit l: key 2l attends
                const uint32_t odd = __ballot_sync(0xffffffffu, (vnext & 0xff00u) != 0);     // bit l: key 2l+1 attends
                const bool full_tile = (j * AK + AK <= n);
                if (j + 1 < T) vnext = mask_fetch(mrow, j + 1);
                ok = mbar_wait(&B->s_full[g], G & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                bool done = false;
                if (j > 0 && full_tile && !pending) {
                    // ---- one pass: p = exp2(s - m_used) with the reference of the tiles before, no maximum first.
                    // Scaling by a stale reference is exact in floating point; it only has to stay far from
                    // overflow, which the check before the scores are released guarantees (otherwise the tile is
                    // redone by the two-pass path below, the scores being still in tensor memory).
                    const uint64_t negm2 = f2_pack(-m_used, -m_used);
                    uint64_t l2a = f2_pack(0.f, 0.f), l2b = l2a;
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    uint32_t sr[32], pw[16];
                    tmem_ld_32x32(s_addr, sr);
                    tmem_ld_wait();
                    mask_half<0>(sr, even, odd);
                    max_half(sr, m4);
                    exp_half(sr, pw, negm2, l2a, l2b);
                    // the previous P V product of this group must have read its P operand before it is overwritten
                    ok = mbar_wait(&B->pv_done[g], (G & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    tmem_st_32x16(p_addr, pw);
                    tmem_ld_32x32(s_addr + 32, sr);
                    tmem_ld_wait();
                    mask_half<1>(sr, even, odd);
                    max_half(sr, m4);
                    const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                    if (!__any_sync(0xffffffffu, mx > m_used + ONE_PASS_HEADROOM)) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&B->s_empty[g]);          // S may be overwritten by the next tile
                        exp_half(sr, pw, negm2, l2a, l2b);
                        tmem_st_32x16(p_addr + 16, pw);
                        float a0, a1, b0, b1;
                        f2_unpack(l2a, a0, a1);
                        f2_unpack(l2b, b0, b1);
                        l_run += (a0 + a1) + (b0 + b1);
                        m_seen = fmaxf(m_seen, mx);
                        pending = __any_sync(0xffffffffu, m_seen > m_used + RESCALE_STEP);
                        done = true;
                    }
                }
                if (!done) {
                    // ---- two passes (first tile of a line, ragged last tile, a rescale that is due, or a tile the
                    // one-pass path gave back): row maximum first, then the exponentials
                    const bool plain = full_tile && (even & odd) == 0xffffffffu;
                    float mx;
                    {
                        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            uint32_t sr[32];
                            tmem_ld_32x32(s_addr + hf * 32, sr);
                            tmem_ld_wait();
                            if (!plain) mask_half_general(sr, even, odd, hf, j * AK, n);
                            max_half(sr, m4);
                        }
                        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                    }
                    // The previous P V product of this group has to be complete before its P operand is overwritten
                    // and before the running output is rescaled.
                    ok = mbar_wait(&B->pv_done[g], (G & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if (j == 0) {
                        m_used = m_seen = mx;
                    } else {
                        m_seen = fmaxf(m_seen, mx);
                        const bool grow = m_seen > m_used + RESCALE_STEP;
                        if (__any_sync(0xffffffffu, grow)) {
                            const float f = grow ? ex2_f32(m_used - m_seen) : 1.f;
                            if (grow) m_used = m_seen;
                            uint32_t ov[32];
                            tmem_ld_32x32(o_addr, ov);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < HD; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * f);
                            tmem_st_32x32(o_addr, ov);
                            l_run *= f;
                        }
                    }
                    pending = false;
                    const uint64_t negm2 = f2_pack(-m_used, -m_used);
                    uint64_t l2a = f2_pack(0.f, 0.f), l2b = l2a;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        uint32_t sr[32], pw[16];
                        tmem_ld_32x32(s_addr + hf * 32, sr);
                        tmem_ld_wait();
                        if (hf == 1) {               // every score is in registers or consumed: S may be overwritten
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&B->s_empty[g]);
                        }
                        if (!plain) mask_half_general(sr, even, odd, hf, j * AK, n);
                        exp_half(sr, pw, negm2, l2a, l2b);
                        tmem_st_32x16(p_addr + hf * 16, pw);
                    }
                    float a0, a1, b0, b1;
                    f2_unpack(l2a, a0, a1);
                    f2_unpack(l2b, b0, b1);
                    l_run += (a0 + a1) + (b0 + b1);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B->p_full[g]);
            }
            if (!ok) break;
            // the last P V of this item, normalise, store
            ok = mbar_wait(&B->pv_done[g], (G & 1) ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t ov[32];
            tmem_ld_32x32(o_addr, ov);
            tmem_ld_wait();
            tc_fence_before();
            const int qi = qt * AQ + row;
            if (line < p.lines && qi < n) {
                const float inv = 1.f / l_run;
                __nv_bfloat16* dst = p.o + (long long)line * p.o_ls + (long long)qi * p.o_ps + h * HD;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 v;
                    v.x = pack_bf16x2(__uint_as_float(ov[c * 8 + 0]) * inv, __uint_as_float(ov[c * 8 + 1]) * inv);
                    v.y = pack_bf16x2(__uint_as_float(ov[c * 8 + 2]) * inv, __uint_as_float(ov[c * 8 + 3]) * inv);
                    v.z = pack_bf16x2(__uint_as_float(ov[c * 8 + 4]) * inv, __uint_as_float(ov[c * 8 + 5]) * inv);
                    v.w = pack_bf16x2(__uint_as_float(ov[c * 8 + 6]) * inv, __uint_as_float(ov[c * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(dst + c * 8) = v;
                }
            }
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP0) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace atc4
}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_triatt_core_tc4(const b200pf_bf16* q, const b200pf_bf16* k, const b200pf_bf16* vt, int vt_pitch,
                                      const b200pf_bf16* bias, long long bias_hs, long long bias_qs,
                                      const uint8_t* mask_lines, int mask_pitch,
                                      b200pf_bf16* o, long long o_line_stride, long long o_pos_stride,
                                      int lines, int n, void* stream) {
    using namespace atc4;
    B200PF_REQUIRE(q && k && vt && bias && mask_lines && o && lines > 0 && n > 0, B200PF_ERR_INVALID, "triatt_core_tc4: bad argument");
    B200PF_REQUIRE(aligned16(q) && aligned16(k) && aligned16(vt) && aligned16(bias) && aligned16(o) && aligned16(mask_lines),
                   B200PF_ERR_INVALID, "triatt_core_tc4: pointers must be 16-byte aligned");
    B200PF_REQUIRE(vt_pitch % 8 == 0 && vt_pitch >= n && bias_hs % 8 == 0 && bias_qs % 8 == 0 && bias_hs >= n,
                   B200PF_ERR_INVALID, "triatt_core_tc4: pitches / strides must be multiples of 8 elements and >= n");
    B200PF_REQUIRE(mask_pitch % 16 == 0 && mask_pitch >= (n + AK - 1) / AK * AK, B200PF_ERR_INVALID,
                   "triatt_core_tc4: mask pitch must be a multiple of 16 and cover n rounded up to 64");
    B200PF_REQUIRE(o_line_stride % 8 == 0 && o_pos_stride % 8 == 0, B200PF_ERR_INVALID, "triatt_core_tc4: bad o strides");
    const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap mq, mk, mvt, mb;
    int rc;
    {   // q, k: [line][pos][head][32]; coordinates (d, head, pos, line)
        cuuint64_t dims[4] = {(cuuint64_t)HD, 4, (cuuint64_t)n, (cuuint64_t)lines};
        cuuint64_t str[3] = {(cuuint64_t)HD * 2, (cuuint64_t)4 * HD * 2, (cuuint64_t)n * 4 * HD * 2};
        cuuint32_t boxq[4] = {HD, 1, AQ, 1}, boxk[4] = {HD, 1, AK, 1};
        if ((rc = tmap_encode(&mq, bf, q, 4, dims, str, boxq, CU_TENSOR_MAP_SWIZZLE_64B, "q")) != B200PF_OK) return rc;
        if ((rc = tmap_encode(&mk, bf, k, 4, dims, str, boxk, CU_TENSOR_MAP_SWIZZLE_64B, "k")) != B200PF_OK) return rc;
    }
    {   // v transposed: [line][head][32][vt_pitch]; coordinates (key, d, head, line)
        cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)HD, 4, (cuuint64_t)lines};
        cuuint64_t str[3] = {(cuuint64_t)vt_pitch * 2, (cuuint64_t)HD * vt_pitch * 2, (cuuint64_t)4 * HD * vt_pitch * 2};
        cuuint32_t box[4] = {AK, HD, 1, 1};
        if ((rc = tmap_encode(&mvt, bf, vt, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "vt")) != B200PF_OK) return rc;
    }
    {   // bias: [query][head][key]
        cuuint64_t dims[3] = {(cuuint64_t)n, 4, (cuuint64_t)n};
        cuuint64_t str[2] = {(cuuint64_t)bias_hs * 2, (cuuint64_t)bias_qs * 2};
        cuuint32_t box[3] = {AK, 1, AQ};
        if ((rc = tmap_encode(&mb, bf, bias, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "bias")) != B200PF_OK) return rc;
    }
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "triatt_core_tc4: no device status word");
    B200PF_SMEM_ATTR_ONCE(triatt_core_tc4_kernel, SMEM_BYTES);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long items = (long long)((lines + NG - 1) / NG) * 4 * ((n + AQ - 1) / AQ);
    Args a{mask_lines, (__nv_bfloat16*)o, o_line_stride, o_pos_stride, mask_pitch, lines, n};
    triatt_core_tc4_kernel<<<(unsigned)(items < sms ? items : sms), THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(mq, mk, mvt, mb, a, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

