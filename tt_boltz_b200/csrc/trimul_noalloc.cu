// Triangle multiplication for callers that cannot allocate device memory.
//
// The three stages of the triangle multiplication (producer -> contraction -> epilogue) hand
// their intermediate a / b / x planes to each other through global memory.  Normally the host
// owns that scratch (a torch tensor).  Some hosts cannot provide it: a plugin that runs inside
// someone else's memory pool with a fixed budget, a callback invoked while the allocator is
// locked, an inference server that forbids allocation after start-up.  For them this file keeps
// the scratch in a file-scope device array that exists for as long as the library is loaded.
//
// The array name is only meaningful to device code; host code asks the runtime for its device
// address once per device and passes that address to the kernels.
#include <mutex>

#include "common.cuh"

namespace b200pf {

constexpr int NOALLOC_MAX_N = 128;                                  // largest token count served
constexpr int NOALLOC_CH = 128;
constexpr size_t NOALLOC_PLANE_ELEMS = (size_t)NOALLOC_CH * NOALLOC_MAX_N * NOALLOC_MAX_N;
constexpr size_t NOALLOC_BYTES = 3 * NOALLOC_PLANE_ELEMS * sizeof(__nv_bfloat16);   // a, b, x: 12 MiB

static __device__ __align__(256) unsigned char g_trimul_scratch[NOALLOC_BYTES];

// Device address of the scratch array on the current device (looked up once per device).
static int scratch_address(__nv_bfloat16** out) {
    static std::mutex mu;
    static void* ptrs[64] = {nullptr};
    int dev = 0;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_REQUIRE(dev >= 0 && dev < 64, B200PF_ERR_UNSUPPORTED, "tri_mul_noalloc: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_trimul_scratch);
        B200PF_REQUIRE(e == cudaSuccess && p != nullptr, B200PF_ERR_CUDA,
                       "tri_mul_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        ptrs[dev] = p;
    }
    *out = static_cast<__nv_bfloat16*>(ptrs[dev]);
    return B200PF_OK;
}

}  // namespace b200pf

using namespace b200pf;

extern "C" int b200pf_tri_mul_noalloc(float* z, const uint8_t* mask, const float* ln_gamma, const float* ln_beta,
                                      const b200pf_bf16* w_pg,
                                      const b200pf_bf16* w_pout, const b200pf_bf16* w_gout,
                                      const float* wsum, const float* wb,
                                      int n, int incoming, void* stream) {
    B200PF_REQUIRE(n > 0, B200PF_ERR_INVALID, "tri_mul_noalloc: n must be positive");
    B200PF_REQUIRE(n <= NOALLOC_MAX_N, B200PF_ERR_UNSUPPORTED,
                   "tri_mul_noalloc: n = %d exceeds the built-in scratch (at most %d tokens); use the "
                   "producer / contract / epilogue entry points with caller-owned planes instead", n, NOALLOC_MAX_N);
    __nv_bfloat16* base = nullptr;
    int rc = scratch_address(&base);
    if (rc != B200PF_OK) return rc;
    const int pitch = (n + 7) / 8 * 8;
    const long long plane_stride = (long long)n * pitch;
    __nv_bfloat16* a = base;
    __nv_bfloat16* b = base + NOALLOC_PLANE_ELEMS;
    __nv_bfloat16* x = base + 2 * NOALLOC_PLANE_ELEMS;
    // The producer writes every element the contraction reads and the contraction every element
    // the epilogue reads (padding columns included), so nothing has to be cleared between calls.
    b200pf_plane_out oa{a, plane_stride, 0, 0}, ob{b, plane_stride, 0, 0};
    rc = b200pf_trimul_producer(z, mask, ln_gamma, ln_beta, w_pg, &oa, &ob, pitch, n, n, incoming, stream);
    if (rc != B200PF_OK) return rc;
    b200pf_planes pa{a, plane_stride, 0, pitch, n, n, 1, 0}, pb{b, plane_stride, 0, pitch, n, n, 1, 0};
    rc = b200pf_trimul_contract(&pa, &pb, nullptr, nullptr, reinterpret_cast<b200pf_bf16*>(x), plane_stride, pitch,
                                0, 0, NOALLOC_CH, 0, stream);
    if (rc != B200PF_OK) return rc;
    return b200pf_trimul_epilogue_tc(z, reinterpret_cast<const b200pf_bf16*>(x), plane_stride, pitch, ln_gamma, ln_beta,
                                     w_pout, w_gout, wsum, wb, n, n, stream);
}
