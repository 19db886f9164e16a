// Error text, version and the device status word of libllamatov_b200.so.
#include <stdarg.h>
#include <string.h>

#include "lt_common.cuh"

namespace lt {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static unsigned long long g_launches = 0;
void count_launches(int n) { __atomic_fetch_add(&g_launches, (unsigned long long)n, __ATOMIC_RELAXED); }

static int g_chained = 0;
bool chained_launch() { return __atomic_load_n(&g_chained, __ATOMIC_RELAXED) != 0; }

__device__ int g_status_word = 0;

int* device_status_ptr() {
    // One word per device.  The address is looked up once per device (first launch on that
    // device, which precedes any stream capture) and handed to kernels as an argument.
    static int* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cache[dev] == nullptr) {
        int* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_status_word) != cudaSuccess) return nullptr;
        cache[dev] = p;
    }
    return cache[dev];
}

}  // namespace lt

extern "C" const char* lt_last_error(void) { return lt::g_err; }

extern "C" const char* lt_version(void) { return "llamatov_b200 0.1 (sm_100a)"; }

extern "C" unsigned long long lt_launch_count(void) { return __atomic_load_n(&lt::g_launches, __ATOMIC_RELAXED); }

extern "C" int lt_set_chained_launch(int on) {
    return __atomic_exchange_n(&lt::g_chained, on ? 1 : 0, __ATOMIC_RELAXED);
}

extern "C" int lt_device_status(unsigned int* h_status, void* stream) {
    LT_REQUIRE(h_status != nullptr, "lt_device_status: null output");
    cudaStream_t s = (cudaStream_t)stream;
    int* p = lt::device_status_ptr();
    LT_REQUIRE(p != nullptr, "lt_device_status: status word unavailable");
    int v = 0;
    LT_CUDA(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, s));
    LT_CUDA(cudaMemsetAsync(p, 0, sizeof(int), s));
    LT_CUDA(cudaStreamSynchronize(s));
    *h_status = (unsigned int)v;
    return LT_OK;
}
