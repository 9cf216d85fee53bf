// Shared host/device helpers for the b200pf kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200pf.h"

namespace b200pf {

// ---- host side: error reporting and launch accounting ------------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
unsigned int* device_status_word();   // device address of the status word, cached per device

#define B200PF_REQUIRE(cond, code, ...)              \
    do {                                             \
        if (!(cond)) {                               \
            ::b200pf::set_error(__VA_ARGS__);        \
            return (code);                           \
        }                                            \
    } while (0)

#define B200PF_CUDA(call)                                                              \
    do {                                                                               \
        cudaError_t e__ = (call);                                                      \
        if (e__ != cudaSuccess) {                                                      \
            ::b200pf::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                                __FILE__, __LINE__);                                   \
            return B200PF_ERR_CUDA;                                                    \
        }                                                                              \
    } while (0)

#define B200PF_LAUNCH_CHECK()                                                          \
    do {                                                                               \
        ::b200pf::count_launch();                                                      \
        cudaError_t e__ = cudaGetLastError();                                          \
        if (e__ != cudaSuccess) {                                                      \
            ::b200pf::set_error("kernel launch failed: %s (%s:%d)",                    \
                                cudaGetErrorString(e__), __FILE__, __LINE__);          \
            return B200PF_ERR_CUDA;                                                    \
        }                                                                              \
    } while (0)

// Raises a kernel's dynamic shared-memory limit the first time the call site runs on a device (the attribute
// is per device and sticks), instead of on every launch.
#define B200PF_SMEM_ATTR_ONCE(kernel, bytes)                                                         \
    do {                                                                                             \
        static bool done__[64] = {false};                                                            \
        int d__ = 0;                                                                                 \
        B200PF_CUDA(cudaGetDevice(&d__));                                                            \
        if (d__ < 0 || d__ >= 64 || !done__[d__]) {                                                  \
            B200PF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes))); \
            if (d__ >= 0 && d__ < 64) done__[d__] = true;                                            \
        }                                                                                            \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- device side -------------------------------------------------------------------------
constexpr float LN_EPS = 1e-5f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_precise(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Status codes kernels may OR into the device status word (never trap, never spin forever).
constexpr unsigned int DEV_STATUS_MBAR_TIMEOUT = 1u;
constexpr unsigned int DEV_STATUS_BAD_INDEX    = 2u;
constexpr unsigned int DEV_STATUS_PEER_TIMEOUT = 4u;   // a cross-rank barrier gave up waiting for a peer

}  // namespace b200pf
