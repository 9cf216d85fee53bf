// Fused triangle attention core (flash style): for every line (row i for the starting node,
// column j for the ending node) and head, O = softmax(Q K^T + mask + bias) V with an online
// softmax; logits and probabilities never leave the SM.
//
// CTA = 8 warps x 16 queries = 128 queries of one head, for LINES consecutive lines at once:
// the [128 x 64] tile of the triangle bias, which does not depend on the line, is fetched once
// per key tile and re-used for all LINES lines; only the small K / V tiles are per line.
// Scores are kept in the log2 domain: the host folds log2(e)/sqrt(32) into W_q and log2(e)
// into the bias projection, so p = exp2(s - m).
//   masked key (mask byte 0)  -> score = -1e9 * log2(e) for every query, as in fp32 where
//                                 qk + (-1e9) + bias rounds to -1e9; a fully masked line thus
//                                 gives the uniform average of V exactly like the reference;
//   key index >= n (padding)  -> excluded (probability exactly 0).
#include "mma.cuh"

namespace b200pf {

constexpr int AQ = 128;       // queries per CTA
constexpr int AK = 64;        // keys per tile
constexpr int HD = 32;        // head dim
constexpr float MASKED_SCORE = -1.0e9f * 1.4426950408889634f;

struct AttCoreArgs {
    const __nv_bfloat16 *q, *k, *v, *bias;
    const uint8_t* mask;
    __nv_bfloat16* o;
    long long mask_ls, mask_ks, o_ls, o_ps, bias_hs, bias_qs;
    int bias_cols, lines, n;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t kv_off(int row, int chunk) {          // [rows][32] bf16, 64-byte rows
    return (uint32_t)(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
}
__device__ __forceinline__ uint32_t bias_off(int row, int chunk) {        // [128][64] bf16, 128-byte rows
    return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int LINES>
struct AttSmem {
    static constexpr int BIAS_BYTES = AQ * AK * 2;                  // 16 KB
    static constexpr int KV_BYTES = AK * HD * 2;                    // 4 KB per line and operand
    static constexpr int MASK_BYTES = ((LINES * AK + 15) / 16) * 16;
    static constexpr int STAGE = BIAS_BYTES + 2 * LINES * KV_BYTES + MASK_BYTES;
    static constexpr int Q_BYTES = LINES * AQ * HD * 2;
    static constexpr int TOTAL = 2 * STAGE + Q_BYTES;
};

template <int LINES>
__global__ void __launch_bounds__(256) triatt_core_kernel(AttCoreArgs p) {
    using S = AttSmem<LINES>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* q_s = smem + 2 * S::STAGE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int g = lane >> 2, t = lane & 3;
    const int n = p.n;
    const int qtiles = (n + AQ - 1) / AQ;
    const int qt = blockIdx.x % qtiles;
    const int h = (blockIdx.x / qtiles) & 3;
    const int line0 = (blockIdx.x / (qtiles * 4)) * LINES;
    const int q0 = qt * AQ;
    const int nkt = (n + AK - 1) / AK;

    auto line_of = [&](int ln) { int l = line0 + ln; return l < p.lines ? l : p.lines - 1; };

    auto issue_tile = [&](int kt) {
        uint8_t* st = smem + (kt & 1) * S::STAGE;
        const int k0 = kt * AK;
        // bias tile: 128 rows x 8 chunks
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int idx = tid + i * 256, row = idx >> 3, c = idx & 7;
            int qrow = q0 + row, col = k0 + c * 8;
            bool ok = qrow < n && col + 8 <= p.bias_cols;
            const __nv_bfloat16* src = p.bias + h * p.bias_hs + (long long)(ok ? qrow : 0) * p.bias_qs + (ok ? col : 0);
            cp_async16_zfill(st + bias_off(row, c), src, ok);
        }
        // K and V tiles: 64 rows x 4 chunks per line = one chunk per thread per operand
        {
            int row = tid >> 2, c = tid & 3;
            bool ok = k0 + row < n;
#pragma unroll
            for (int ln = 0; ln < LINES; ++ln) {
                long long base = (((long long)line_of(ln) * 4 + h) * n + (ok ? k0 + row : 0)) * HD + c * 8;
                cp_async16_zfill(st + S::BIAS_BYTES + ln * S::KV_BYTES + kv_off(row, c), p.k + base, ok);
                cp_async16_zfill(st + S::BIAS_BYTES + (LINES + ln) * S::KV_BYTES + kv_off(row, c), p.v + base, ok);
            }
        }
        // mask codes: 0 = attend, 1 = masked, 2 = beyond n
        uint8_t* mk = st + S::BIAS_BYTES + 2 * LINES * S::KV_BYTES;
        for (int i = tid; i < LINES * AK; i += 256) {
            int ln = i / AK, key = k0 + (i % AK);
            uint8_t code = 2;
            if (key < n) code = p.mask[line_of(ln) * p.mask_ls + key * p.mask_ks] ? 0 : 1;
            mk[i] = code;
        }
    };

    // ---- prologue: Q tile for all lines + first key tile ----
    for (int i = tid; i < LINES * AQ * 4; i += 256) {
        int ln = i / (AQ * 4), row = (i / 4) % AQ, c = i & 3;
        bool ok = q0 + row < n;
        long long base = (((long long)line_of(ln) * 4 + h) * n + (ok ? q0 + row : 0)) * HD + c * 8;
        cp_async16_zfill(q_s + ln * (AQ * HD * 2) + kv_off(row, c), p.q + base, ok);
    }
    issue_tile(0);
    cp_async_commit();

    uint32_t qf[LINES][2][4];
    float o_acc[LINES][4][4];
    float m_run[LINES][2], l_run[LINES][2];
#pragma unroll
    for (int ln = 0; ln < LINES; ++ln) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o_acc[ln][nt][e] = 0.f;
        m_run[ln][0] = m_run[ln][1] = -INFINITY;
        l_run[ln][0] = l_run[ln][1] = 0.f;
    }

    for (int kt = 0; kt < nkt; ++kt) {
        if (kt + 1 < nkt) {
            issue_tile(kt + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kt == 0) {
#pragma unroll
            for (int ln = 0; ln < LINES; ++ln)
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    uint32_t addr = smem_u32(q_s + ln * (AQ * HD * 2)) + kv_off(warp * 16 + (lane & 15), ks * 2 + (lane >> 4));
                    ldsm_x4(addr, qf[ln][ks][0], qf[ln][ks][1], qf[ln][ks][2], qf[ln][ks][3]);
                }
        }
        const uint8_t* st = smem + (kt & 1) * S::STAGE;
        const uint32_t st_addr = smem_u32(st);
        // bias fragment for this warp's 16 queries: rows g / g+8, key columns 8*nt + 2t, +1
        uint32_t bfr[8][2];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            bfr[nt][0] = *reinterpret_cast<const uint32_t*>(st + bias_off(warp * 16 + g, nt) + t * 4);
            bfr[nt][1] = *reinterpret_cast<const uint32_t*>(st + bias_off(warp * 16 + g + 8, nt) + t * 4);
        }
        const uint8_t* mk = st + S::BIAS_BYTES + 2 * LINES * S::KV_BYTES;
#pragma unroll
        for (int ln = 0; ln < LINES; ++ln) {
            const uint32_t k_addr = st_addr + S::BIAS_BYTES + ln * S::KV_BYTES;
            const uint32_t v_addr = st_addr + S::BIAS_BYTES + (LINES + ln) * S::KV_BYTES;
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldsm_x4(k_addr + kv_off(key, ks * 2 + ((lane >> 3) & 1)), b[0], b[1], b[2], b[3]);
                    mma_bf16(s[np * 2], qf[ln][ks], b[0], b[1]);
                    mma_bf16(s[np * 2 + 1], qf[ln][ks], b[2], b[3]);
                }
            // bias, mask, running max
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint16_t codes = *reinterpret_cast<const uint16_t*>(mk + ln * AK + nt * 8 + 2 * t);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint32_t bw = bfr[nt][e >> 1];
                    float bv = (e & 1) ? bf16_hi(bw) : bf16_lo(bw);
                    uint32_t code = (codes >> ((e & 1) * 8)) & 0xff;
                    float sv = s[nt][e] + bv;
                    sv = code == 0 ? sv : (code == 1 ? MASKED_SCORE : -INFINITY);
                    s[nt][e] = sv;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sv);
                }
            }
            float scale[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                float m_new = fmaxf(m_run[ln][r], mx[r]);
                scale[r] = fast_exp2(m_run[ln][r] - m_new);        // first tile: exp2(-inf) = 0
                m_run[ln][r] = m_new;
            }
            float rs[2] = {0.f, 0.f};
            uint32_t pf[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float p0 = fast_exp2(s[nt][0] - m_run[ln][0]);
                float p1 = fast_exp2(s[nt][1] - m_run[ln][0]);
                float p2 = fast_exp2(s[nt][2] - m_run[ln][1]);
                float p3 = fast_exp2(s[nt][3] - m_run[ln][1]);
                rs[0] += p0 + p1;
                rs[1] += p2 + p3;
                pf[nt >> 1][(nt & 1) * 2] = pack_bf16x2(p0, p1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[ln][r] = l_run[ln][r] * scale[r] + rs[r];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                o_acc[ln][nt][0] *= scale[0]; o_acc[ln][nt][1] *= scale[0];
                o_acc[ln][nt][2] *= scale[1]; o_acc[ln][nt][3] *= scale[1];
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    uint32_t b[4];
                    int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldsm_x4_trans(v_addr + kv_off(key, np * 2 + (lane >> 4)), b[0], b[1], b[2], b[3]);
                    mma_bf16(o_acc[ln][np * 2], pf[kk], b[0], b[1]);
                    mma_bf16(o_acc[ln][np * 2 + 1], pf[kk], b[2], b[3]);
                }
        }
        __syncthreads();
    }

    // ---- epilogue: normalise, stage per warp, 16-byte stores ----
    uint8_t* ostage = q_s + warp * (16 * 64);       // 16 rows x 64 bytes, inside this warp's Q rows of line 0
#pragma unroll
    for (int ln = 0; ln < LINES; ++ln) {
        float inv[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float l = l_run[ln][r];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            inv[r] = 1.f / l;
        }
        __syncwarp();
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            *reinterpret_cast<uint32_t*>(ostage + g * 64 + nt * 16 + t * 4) = pack_bf16x2(o_acc[ln][nt][0] * inv[0], o_acc[ln][nt][1] * inv[0]);
            *reinterpret_cast<uint32_t*>(ostage + (g + 8) * 64 + nt * 16 + t * 4) = pack_bf16x2(o_acc[ln][nt][2] * inv[1], o_acc[ln][nt][3] * inv[1]);
        }
        __syncwarp();
        if (line0 + ln < p.lines) {
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                int row = pass * 8 + (lane >> 2), piece = lane & 3;
                int qi = q0 + warp * 16 + row;
                if (qi < n) {
                    uint4 v = *reinterpret_cast<const uint4*>(ostage + row * 64 + piece * 16);
                    *reinterpret_cast<uint4*>(p.o + (long long)(line0 + ln) * p.o_ls + (long long)qi * p.o_ps + h * HD + piece * 8) = v;
                }
            }
        }
    }
}

template <int LINES>
static int launch_core(const AttCoreArgs& p, cudaStream_t st) {
    using S = AttSmem<LINES>;
    B200PF_SMEM_ATTR_ONCE(triatt_core_kernel<LINES>, S::TOTAL);
    int qtiles = (p.n + AQ - 1) / AQ;
    long long blocks = (long long)qtiles * 4 * ((p.lines + LINES - 1) / LINES);
    B200PF_REQUIRE(blocks < (1ll << 31), B200PF_ERR_UNSUPPORTED, "triatt_core: grid too large");
    triatt_core_kernel<LINES><<<(unsigned)blocks, 256, S::TOTAL, st>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_triatt_core(const b200pf_bf16* q, const b200pf_bf16* k, const b200pf_bf16* v,
                                  const b200pf_bf16* bias, long long bias_hs, long long bias_qs, int bias_cols,
                                  const uint8_t* mask, long long mask_ls, long long mask_ks,
                                  b200pf_bf16* o, long long o_line_stride, long long o_pos_stride,
                                  int lines, int n, int lines_per_cta, void* stream) {
    B200PF_REQUIRE(q && k && v && bias && mask && o && lines > 0 && n > 0, B200PF_ERR_INVALID, "triatt_core: bad argument");
    B200PF_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(bias) && aligned16(o), B200PF_ERR_INVALID,
                   "triatt_core: pointers must be 16-byte aligned");
    B200PF_REQUIRE(bias_cols % 8 == 0 && bias_cols >= n && bias_hs % 8 == 0 && bias_qs % 8 == 0 && o_line_stride % 8 == 0 && o_pos_stride % 8 == 0,
                   B200PF_ERR_INVALID, "triatt_core: strides must be multiples of 8 elements");
    AttCoreArgs p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)bias,
                  mask, (__nv_bfloat16*)o, mask_ls, mask_ks, o_line_stride, o_pos_stride, bias_hs, bias_qs, bias_cols, lines, n};
    cudaStream_t st = (cudaStream_t)stream;
    switch (lines_per_cta) {
        case 1: return launch_core<1>(p, st);
        case 0:
        case 2: return launch_core<2>(p, st);
        case 4: return launch_core<4>(p, st);
        default: B200PF_REQUIRE(false, B200PF_ERR_UNSUPPORTED, "triatt_core: lines_per_cta must be 0, 1, 2 or 4");
    }
    return B200PF_OK;
}
