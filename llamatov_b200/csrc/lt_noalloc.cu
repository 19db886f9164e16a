// lt_q8_linear_static: the decode linear (quantise the fp32 activation, then the Q8_0 GEMV)
// for callers that must not allocate device memory.
//
// The ordinary route is lt_quant_q8 followed by lt_q8_gemv, with the quantised activation
// (K int8 + K/32 fp16) living in scratch the caller allocated.  Some callers cannot do that:
// a plugin that is handed the host application's buffers and is forbidden to call cudaMalloc
// (the host owns a fixed memory budget and a foreign allocation would break its accounting),
// or code that runs inside a region where an allocation would synchronise the device or
// invalidate what is being recorded.  For them the scratch lives in the library image itself:
// a file-scope __device__ array that every GPU loading the library holds until the process
// exits (LT_STATIC_MAX_K + LT_STATIC_MAX_K/16 bytes = 17 KiB).
#include "lt_common.cuh"

#define LT_STATIC_MAX_K 16384

namespace {

// [0, MAX_K): int8 quants; [MAX_K, MAX_K + MAX_K/16): fp16 scales.
static __device__ __align__(256) unsigned char g_static_scratch[LT_STATIC_MAX_K + LT_STATIC_MAX_K / 16];

// In host code the array's name only stands for the symbol; the address a kernel can use
// has to be asked for, once per device, with that device current.
unsigned char* static_scratch_for_current_device() {
    static unsigned char* cache[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        lt::set_error("lt_q8_linear_static: cannot identify the current device");
        return nullptr;
    }
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            lt::set_error("lt_q8_linear_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cache[dev] = static_cast<unsigned char*>(p);
    }
    return cache[dev];
}

}  // namespace

extern "C" int lt_q8_linear_static_max_k(void) { return LT_STATIC_MAX_K; }

extern "C" int lt_q8_linear_static(const int8_t* Wq, const uint16_t* Wd, const float* X, const float* Resid,
                                   float* Y, int M, int K, void* stream) {
    LT_REQUIRE(Wq && Wd && X && Y, "lt_q8_linear_static: null pointer");
    LT_REQUIRE(M > 0, "lt_q8_linear_static: M=%d must be positive", M);
    LT_REQUIRE(K > 0 && K % 32 == 0, "lt_q8_linear_static: K=%d must be a positive multiple of 32", K);
    LT_REQUIRE(K <= LT_STATIC_MAX_K,
               "lt_q8_linear_static: K=%d exceeds the built-in scratch (max K = %d); use lt_quant_q8 + lt_q8_gemv "
               "with caller scratch", K, LT_STATIC_MAX_K);
    unsigned char* scratch = static_scratch_for_current_device();
    if (scratch == nullptr) return LT_ERR_CUDA;
    int8_t* xq = reinterpret_cast<int8_t*>(scratch);
    uint16_t* xd = reinterpret_cast<uint16_t*>(scratch + LT_STATIC_MAX_K);
    // Every byte the GEMV reads (K quants, K/32 scales) is rewritten by the quantiser first, so
    // what an earlier call left behind never shows; nothing here needs to start at zero.
    int rc = lt_quant_q8(X, xq, xd, K, 1, stream);
    if (rc != LT_OK) return rc;
    return lt_q8_gemv(Wq, Wd, xq, xd, Resid, Y, M, K, 1, stream);
}
