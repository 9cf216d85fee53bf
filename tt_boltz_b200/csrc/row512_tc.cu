// The two "128 -> 512" producers on tcgen05: LayerNorm -> one [128 x 128] x [128 x 512] GEMM per tile
// of 128 pair positions -> element-wise epilogue straight out of TMEM.
//
//   MODE_TRIMUL : [p_a | g_a] [p_b | g_b] -> p * sigmoid(g) * mask -> a / b planes (channel-major)
//   MODE_TRIATT : [q | k] [v | g]          -> q, k rows per head, v transposed, sigmoid(g) in z layout;
//                 the 4 triangle-bias heads are dotted on the CUDA cores by the loader warps (fp32)
//
// Roles (416 threads): warps 0-7 LayerNorm loaders (16 rows each), warp 8 MMA issuer, warps 9-12
// epilogue (thread = row = TMEM lane).  The 512 output columns are two halves of 256 that live in
// the two halves of TMEM, so the epilogue of one half overlaps the MMAs of the next; the A tile is
// double buffered so the loaders run a tile ahead.  Weights stay in shared memory (128 KB).
#include "row512_tc.h"
#include "rowtc.cuh"

namespace b200pf {
namespace r512 {

using namespace rtc;

constexpr int MODE_TRIMUL = 0, MODE_TRIATT = 1;
constexpr int LOAD_WARPS = 8, EPI_WARP0 = 9, THREADS = 13 * 32;
constexpr int W_BYTES = 512 * 128 * 2;                 // 131072 (two k-blocks of [512][128 B])
constexpr int OFF_A = W_BYTES;                          // 2 stages x 32 KB
constexpr int OFF_STAGE = OFF_A + 2 * A_TILE_BYTES;     // per epilogue warp: [32][40] bf16 = 2560 B
constexpr int STG_PITCH = 40;
constexpr int OFF_BIAS = OFF_STAGE + 4 * 32 * STG_PITCH * 2;   // 512 fp32
constexpr int OFF_WB = OFF_BIAS + 512 * 4;              // triangle-bias rows [4][128] fp32 + 4 offsets
constexpr int OFF_BAR = OFF_WB + (4 * 128 + 4) * 4;
constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024;

struct Bars {
    uint64_t a_full[2], a_empty[2], acc_full[2], acc_empty[2];
    uint32_t tmem_slot;
    int abort_flag;
};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) row512_kernel(Args p, unsigned int* status) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Bars* B = reinterpret_cast<Bars*>(smem + OFF_BAR);
    volatile int* abort_flag = &B->abort_flag;
    float* bias_s = reinterpret_cast<float*>(smem + OFF_BIAS);
    float* wb_s = reinterpret_cast<float*>(smem + OFF_WB);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

    const int span = p.transposed ? p.rows : p.n;                 // positions along a line
    const int n_lines = p.transposed ? p.n : p.rows;
    const int tpl = (span + TM - 1) / TM;
    const long long tiles = (long long)n_lines * tpl;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&B->a_full[i], LOAD_WARPS); mbar_init(&B->a_empty[i], 1);
            mbar_init(&B->acc_full[i], 1); mbar_init(&B->acc_empty[i], 4);
        }
        B->abort_flag = 0;
        fence_barrier_init();
    }
    load_weights_sw128(smem, p.w, 512, tid, THREADS);
    for (int i = tid; i < 512; i += THREADS) bias_s[i] = p.wbias[i];
    if (MODE == MODE_TRIATT) {
        for (int i = tid; i < 4 * 128; i += THREADS) wb_s[i] = __bfloat162float(p.w_bias_rows[i]);
        if (tid < 4) wb_s[512 + tid] = p.wbias[512 + tid];
    }
    fence_proxy_async();
    if (warp == 8) { tmem_alloc(&B->tmem_slot, 512); tmem_relinquish(); }
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
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
            const int line = (int)(t / tpl), pos0 = (int)(t % tpl) * TM;
            const uint32_t stage = it & 1, ph = (it >> 1) & 1;
            ok = mbar_wait(&B->a_empty[stage], ph ^ 1, abort_flag);
            if (!ok) break;
            uint8_t* a_tile = smem + OFF_A + stage * A_TILE_BYTES;
            ln_rows16_to_sw128(
                [&](int r) -> const float* { long long f = flat_of(line, pos0 + r); return f < 0 ? nullptr : p.z + f * KC; },
                a_tile, warp * 16, lane,
                [&](int r, const float4 (&v)[4]) {
                    if (MODE == MODE_TRIATT) {
                        float acc[4];
#pragma unroll
                        for (int h = 0; h < 4; ++h) {
                            float a = 0.f;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float4 wv = *reinterpret_cast<const float4*>(wb_s + h * 128 + (j * 8 + (lane & 7)) * 4);
                                a += v[j].x * wv.x + v[j].y * wv.y + v[j].z * wv.z + v[j].w * wv.w;
                            }
                            a += __shfl_xor_sync(0xffffffffu, a, 1);
                            a += __shfl_xor_sync(0xffffffffu, a, 2);
                            a += __shfl_xor_sync(0xffffffffu, a, 4);
                            acc[h] = a;
                        }
                        const int sub = lane & 7;
                        if (sub < 4 && pos0 + r < span) {
                            float val = sub == 0 ? acc[0] : (sub == 1 ? acc[1] : (sub == 2 ? acc[2] : acc[3]));
                            p.tri_bias[sub * p.bias_hs + (long long)line * p.bias_qs + pos0 + r] = __float2bfloat16(val + wb_s[512 + sub]);
                        }
                    }
                });
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->a_full[stage]);
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    } else if (warp == 8) {
        if (lane == 0) {
            // ---------------------------- MMA issuer ----------------------------
            constexpr uint32_t idesc = make_idesc_bf16(TM, 256);
            const uint32_t w_addr = smem_u32(smem);
            uint32_t it = 0, acc_cnt[2] = {0, 0};
            bool ok = true;
            for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
                const uint32_t stage = it & 1, ph = (it >> 1) & 1;
                ok = mbar_wait(&B->a_full[stage], ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + OFF_A + stage * A_TILE_BYTES);
                for (int half = 0; half < 2 && ok; ++half) {
                    ok = mbar_wait(&B->acc_empty[half], (acc_cnt[half] & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    ++acc_cnt[half];
                    tc_fence_after();
                    issue_gemm_k128(tmem_base + half * 256, a_addr, w_addr, 512, half * 256, idesc);
                    umma_commit(&B->acc_full[half]);
                }
                if (ok) umma_commit(&B->a_empty[stage]);
            }
            if (!ok) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
        }
    } else {
        // ---------------------------- epilogue ----------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + OFF_STAGE) + (warp - EPI_WARP0) * 32 * STG_PITCH;
        uint32_t acc_cnt = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            const int line = (int)(t / tpl), pos0 = (int)(t % tpl) * TM;
            const long long flat = flat_of(line, pos0 + row);
            float mk = 1.f;
            if (MODE == MODE_TRIMUL) mk = flat < 0 ? 0.f : (float)p.mask[flat];
            for (int half = 0; half < 2 && ok; ++half) {
                ok = mbar_wait(&B->acc_full[half], acc_cnt & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tbase = tmem_base + lane_off + half * 256;
                if (MODE == MODE_TRIMUL) {
                    // columns [0,128) = p, [128,256) = g of operand `half`; 32 channels per step
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t pr[32], gr[32];
                        tmem_ld_32x32(tbase + c * 32, pr);
                        tmem_ld_32x32(tbase + 128 + c * 32, gr);
                        tmem_ld_wait();
                        const float* bp = bias_s + half * 256 + c * 32;
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            float u = (__uint_as_float(pr[e]) + bp[e]) * sigmoid_tanh(__uint_as_float(gr[e]) + bp[128 + e]) * mk;
                            stg[e * STG_PITCH + lane] = __float2bfloat16(u);
                        }
                        __syncwarp();
                        const long long ps = p.plane_stride[half];
                        __nv_bfloat16* planes = p.planes[half] + (long long)(c * 32) * ps +
                                                (long long)(line / p.row_group[half]) * p.group_stride[half] +
                                                (long long)(line % p.row_group[half]) * p.pitch;
#pragma unroll
                        for (int pass = 0; pass < 4; ++pass) {
                            int ch = pass * 8 + (lane >> 2), piece = lane & 3;
                            int col = pos0 + quarter * 32 + piece * 8;
                            if (col + 8 <= p.pitch)
                                *reinterpret_cast<uint4*>(planes + ch * ps + col) =
                                    *reinterpret_cast<const uint4*>(stg + ch * STG_PITCH + piece * 8);
                        }
                        __syncwarp();
                    }
                } else {
                    // half 0: [q | k], half 1: [v | g]; 32 columns = one head
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        uint32_t r[32];
                        tmem_ld_32x32(tbase + c * 32, r);
                        tmem_ld_wait();
                        const float* bp = bias_s + half * 256 + c * 32;
                        const int head = c & 3;
                        const bool is_gate = half == 1 && c >= 4;
                        const bool is_vt = half == 1 && c < 4 && p.vt_pitch > 0;
                        if (is_vt) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) stg[e * STG_PITCH + lane] = __float2bfloat16(__uint_as_float(r[e]) + bp[e]);
                            __syncwarp();
#pragma unroll
                            for (int pass = 0; pass < 4; ++pass) {
                                int dd = pass * 8 + (lane >> 2), piece = lane & 3;
                                int col = pos0 + quarter * 32 + piece * 8;
                                if (col + 8 <= p.vt_pitch)
                                    *reinterpret_cast<uint4*>(p.v + (((long long)line * 4 + head) * 32 + dd) * p.vt_pitch + col) =
                                        *reinterpret_cast<const uint4*>(stg + dd * STG_PITCH + piece * 8);
                            }
                            __syncwarp();
                        } else if (flat >= 0) {
                            uint4 o[4];
                            uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                float v0 = __uint_as_float(r[2 * e]) + bp[2 * e], v1 = __uint_as_float(r[2 * e + 1]) + bp[2 * e + 1];
                                if (is_gate) { v0 = sigmoid_tanh(v0); v1 = sigmoid_tanh(v1); }
                                ow[e] = pack_bf16x2(v0, v1);
                            }
                            __nv_bfloat16* dst;
                            if (is_gate) dst = p.g + flat * KC + head * 32;
                            else {
                                __nv_bfloat16* base = half == 0 ? (c < 4 ? p.q : p.k) : p.v;
                                dst = base + (((long long)line * 4 + head) * span + pos0 + row) * 32;
                            }
#pragma unroll
                            for (int e = 0; e < 4; ++e) reinterpret_cast<uint4*>(dst)[e] = o[e];
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B->acc_empty[half]);
            }
            ++acc_cnt;
        }
        if (!ok && lane == 0) atomicOr(status, DEV_STATUS_MBAR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int MODE>
static int launch(const Args& a, cudaStream_t st) {
    unsigned int* status = device_status_word();
    B200PF_REQUIRE(status, B200PF_ERR_CUDA, "row512: no device status word");
    B200PF_CUDA(cudaFuncSetAttribute(row512_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int span = a.transposed ? a.rows : a.n, lines = a.transposed ? a.n : a.rows;
    long long tiles = (long long)lines * ((span + TM - 1) / TM);
    row512_kernel<MODE><<<(unsigned)(tiles < sms ? tiles : sms), THREADS, SMEM_BYTES, st>>>(a, status);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

int launch_trimul(const Args& a, cudaStream_t st) { return launch<MODE_TRIMUL>(a, st); }
int launch_triatt(const Args& a, cudaStream_t st) { return launch<MODE_TRIATT>(a, st); }

}  // namespace r512
}  // namespace b200pf
