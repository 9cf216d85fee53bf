// Library-wide host state of the C ABI: last-error text, launch counter, device status word.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace b200pf {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

__device__ unsigned int g_dev_status = 0;

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

unsigned int* device_status_word() {
    static std::mutex mu;
    static unsigned int* ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dev_status) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<unsigned int*>(p);
    }
    return ptrs[dev];
}

}  // namespace b200pf

extern "C" {

int b200pf_version(void) { return 100; }

const char* b200pf_last_error(void) { return b200pf::g_err; }

long long b200pf_launch_count(void) { return b200pf::g_launches.load(); }

int b200pf_device_status(void* stream) {
    unsigned int* p = b200pf::device_status_word();
    B200PF_REQUIRE(p != nullptr, B200PF_ERR_CUDA, "no device status word (no CUDA device?)");
    unsigned int v = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B200PF_CUDA(cudaMemcpyAsync(&v, p, sizeof(v), cudaMemcpyDeviceToHost, st));
    B200PF_CUDA(cudaStreamSynchronize(st));
    if (v != 0) {
        B200PF_CUDA(cudaMemsetAsync(p, 0, sizeof(v), st));
        B200PF_CUDA(cudaStreamSynchronize(st));
        b200pf::set_error("device status word = 0x%x (1 = a bounded mbarrier wait ran out, 2 = index check, 4 = a cross-rank barrier gave up on a peer)", v);
    }
    return static_cast<int>(v);
}

}  // extern "C"
