// Warp-level bf16 tensor-core helpers (mma.sync m16n8k16 + ldmatrix) shared by the row-tile
// kernels and the attention kernel.
#pragma once

#include "common.cuh"

namespace b200pf {

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// d += a (16x16, row) * b (16x8, col), fp32 accumulate.
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Operand tiles in shared memory use a row pitch of K + 8 bf16 (16 bytes of padding), which
// makes every ldmatrix phase hit 8 distinct 16-byte bank groups.
constexpr int KC = 128;            // channel count of the pair representation
constexpr int APITCH = KC + 8;     // elements

// A fragment (16 rows x 16 k) of a row-major [rows][APITCH] tile.
__device__ __forceinline__ void load_a_frag(uint32_t tile_addr, int pitch_elems, int row0, int k0, int lane,
                                            uint32_t (&a)[4]) {
    uint32_t addr = tile_addr + (uint32_t)(((row0 + (lane & 15)) * pitch_elems + k0 + ((lane >> 4) << 3)) * 2);
    ldsm_x4(addr, a[0], a[1], a[2], a[3]);
}
// B fragments for two adjacent n-tiles (16 output columns x 16 k) of a weight tile stored
// [n][pitch] (k contiguous): b[0..1] -> n-tile at n0, b[2..3] -> n-tile at n0 + 8.
__device__ __forceinline__ void load_b_frag2(uint32_t w_addr, int pitch_elems, int n0, int k0, int lane,
                                             uint32_t (&b)[4]) {
    int row = n0 + (lane & 7) + ((lane >> 4) << 3);
    int col = k0 + (((lane >> 3) & 1) << 3);
    ldsm_x4(w_addr + (uint32_t)((row * pitch_elems + col) * 2), b[0], b[1], b[2], b[3]);
}

}  // namespace b200pf
