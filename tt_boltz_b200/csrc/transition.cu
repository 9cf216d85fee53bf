// Pair transition: z += W3( silu(W1 LN(z)) * (W2 LN(z)) ), the 512-wide hidden never leaves the SM.
//
// A CTA owns 256 pair positions (8 warps x 32).  The weights (384 KB in bf16) do not fit in
// shared memory, so they are streamed from L2 in 8 steps of 64 hidden channels with a
// two-stage cp.async ring shared by the CTA.  Per step and warp:
//   for each group of 16 hidden channels: f = tile(32x128) . W12grp^T (32 columns = 16 fc1 | 16 fc2)
//   h = silu(f1) * f2 stays in registers and is re-used directly as the A operand of the
//   second GEMM (accumulator layout == A-fragment layout), out(32x128) += h . W3grp^T.
//
// Host packing (tt_boltz_b200/weights.py):
//   w12 [1024][128]: 32 groups of 32 rows = 16 fc1 rows then the 16 fc2 rows of the same hidden
//                    channels, LN gain folded in;  bias12 [1024] fp32 in the same order;
//   w3  [8][128][64]: per step, the 64 matching columns of fc3 ([out][hidden]).
#include "rowtile.cuh"

namespace b200pf {

constexpr int T_STEPS = 8;
constexpr int W3_PITCH = 64 + 8;
constexpr int W12_STEP_BYTES = 128 * APITCH * 2;      // 34,816
constexpr int W3_STEP_BYTES = 128 * W3_PITCH * 2;     // 18,432
constexpr int T_STAGE_BYTES = W12_STEP_BYTES + W3_STEP_BYTES;
constexpr int TRANSITION_SMEM = 2 * T_STAGE_BYTES + 1024 * 4 + WARPS * A_TILE_BYTES;   // 180,224

struct TransitionArgs {
    float* z;
    const __nv_bfloat16* w12;
    const __nv_bfloat16* w3;
    const float* bias12;
    long long rows_flat;
};

__device__ __forceinline__ void transition_issue_step(uint8_t* stage, const TransitionArgs& p, int step) {
    __nv_bfloat16* w12_s = reinterpret_cast<__nv_bfloat16*>(stage);
    __nv_bfloat16* w3_s = reinterpret_cast<__nv_bfloat16*>(stage + W12_STEP_BYTES);
    const __nv_bfloat16* g12 = p.w12 + (long long)step * 128 * KC;
    const __nv_bfloat16* g3 = p.w3 + (long long)step * 128 * 64;
    for (int i = threadIdx.x; i < 128 * 16; i += blockDim.x) {
        int r = i >> 4, c = i & 15;
        cp_async16(w12_s + r * APITCH + c * 8, g12 + r * KC + c * 8);
    }
    for (int i = threadIdx.x; i < 128 * 8; i += blockDim.x) {
        int r = i >> 3, c = i & 7;
        cp_async16(w3_s + r * W3_PITCH + c * 8, g3 + r * 64 + c * 8);
    }
    cp_async_commit();
}

__global__ void __launch_bounds__(WARPS * 32, 1) transition_kernel(TransitionArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* stages = smem;
    float* bias_s = reinterpret_cast<float*>(smem + 2 * T_STAGE_BYTES);
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem + 2 * T_STAGE_BYTES + 1024 * 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __nv_bfloat16* tile = tiles + warp * (UNIT * APITCH);
    const uint32_t tile_addr = smem_u32(tile);
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) bias_s[i] = p.bias12[i];
    const int g = lane >> 2, t = lane & 3;
    const long long cta_tiles = (p.rows_flat + WARPS * UNIT - 1) / (WARPS * UNIT);

    for (long long ct = blockIdx.x; ct < cta_tiles; ct += gridDim.x) {
        const long long base = ct * (WARPS * UNIT) + warp * UNIT;
        __syncthreads();                               // previous tile done with both weight stages
        transition_issue_step(stages, p, 0);
        ln_rows_to_tile([&](int l) -> const float* { return base + l < p.rows_flat ? p.z + (base + l) * KC : nullptr; },
                        tile, lane);
        __syncwarp();
        float out[2][16][4];
        zero_acc(out);
#pragma unroll 1
        for (int step = 0; step < T_STEPS; ++step) {
            cp_async_wait<0>();
            __syncthreads();                           // step's weights visible; other stage free
            if (step + 1 < T_STEPS) transition_issue_step(stages + ((step + 1) & 1) * T_STAGE_BYTES, p, step + 1);
            const uint32_t w12_addr = smem_u32(stages + (step & 1) * T_STAGE_BYTES);
            const uint32_t w3_addr = w12_addr + W12_STEP_BYTES;
#pragma unroll 1
            for (int sub = 0; sub < 4; ++sub) {
                float f[2][4][4];
                zero_acc(f);
                warp_gemm_smemA<4>(tile_addr, w12_addr, APITCH, sub * 32, lane, f);
                // h = silu(f1) * f2 for 16 hidden channels -> A fragments of one k16 step
                uint32_t hfrag[2][4];
                const float* b1 = bias_s + step * 128 + sub * 32;
#pragma unroll
                for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        float h[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            int col = nt * 8 + 2 * t + (e & 1);
                            float f1 = f[mi][nt][e] + b1[col];
                            float f2 = f[mi][nt + 2][e] + b1[16 + col];
                            h[e] = f1 * sigmoidf_(f1) * f2;
                        }
                        hfrag[mi][nt * 2] = pack_bf16x2(h[0], h[1]);       // row g
                        hfrag[mi][nt * 2 + 1] = pack_bf16x2(h[2], h[3]);   // row g + 8
                    }
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    uint32_t b[4];
                    load_b_frag2(w3_addr, W3_PITCH, np * 16, sub * 16, lane, b);
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        mma_bf16(out[mi][np * 2], hfrag[mi], b[0], b[1]);
                        mma_bf16(out[mi][np * 2 + 1], hfrag[mi], b[2], b[3]);
                    }
                }
            }
        }
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                long long f = base + mi * 16 + g + hh * 8;
                if (f >= p.rows_flat) continue;
                float* zr = p.z + f * KC + 2 * t;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) {
                    float2 zv = *reinterpret_cast<float2*>(zr + nt * 8);
                    zv.x += out[mi][nt][hh * 2];
                    zv.y += out[mi][nt][hh * 2 + 1];
                    *reinterpret_cast<float2*>(zr + nt * 8) = zv;
                }
            }
    }
}

}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_transition_z(float* z, const b200pf_bf16* w12, const float* bias12,
                                   const b200pf_bf16* w3, long long n_rows_flat, void* stream) {
    B200PF_REQUIRE(z && w12 && bias12 && w3 && n_rows_flat > 0, B200PF_ERR_INVALID, "transition_z: bad argument");
    B200PF_REQUIRE(aligned16(z) && aligned16(w12) && aligned16(w3), B200PF_ERR_INVALID,
                   "transition_z: pointers must be 16-byte aligned");
    TransitionArgs p{z, (const __nv_bfloat16*)w12, (const __nv_bfloat16*)w3, bias12, n_rows_flat};
    B200PF_SMEM_ATTR_ONCE(transition_kernel, TRANSITION_SMEM);
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long tiles = (n_rows_flat + WARPS * UNIT - 1) / (WARPS * UNIT);
    transition_kernel<<<(unsigned)(tiles < sms ? tiles : sms), WARPS * 32, TRANSITION_SMEM, (cudaStream_t)stream>>>(p);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}
