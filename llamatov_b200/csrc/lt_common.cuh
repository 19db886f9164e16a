// Shared helpers for the sm_100a kernels and their C-ABI launchers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/llamatov_b200.h"

namespace lt {

// Thread-local text of the last failure, returned by lt_last_error().
void set_error(const char* fmt, ...);

// Device status word shared by all kernels of the library (0 = clean).  Kernels
// never trap: on a bad length / out-of-range index they skip the access and OR a
// bit into this word; lt_device_status() reads and clears it.
int* device_status_ptr();

// Number of kernel launches this library has enqueued in this process (lt_launch_count()).
void count_launches(int n);

inline int check_launch(const char* what, int n = 1, cudaError_t launched = cudaSuccess) {
    count_launches(n);
    cudaError_t e = launched != cudaSuccess ? launched : cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
        return LT_ERR_CUDA;
    }
    return LT_OK;
}

// Chained launches (lt_set_chained_launch): kernels of the one-sequence decode operators are enqueued with
// programmatic stream serialisation, so that a kernel's CTAs may become resident while its predecessor in
// the stream is still running.  Such a kernel calls chain_release() at its start (lets ITS successor be
// scheduled), may fetch what no predecessor writes (weights) and calls chain_wait() before it touches
// anything else; chain_wait() returns when the predecessor has completed and its writes are visible.  Both
// calls do nothing in a kernel that was launched the ordinary way.
bool chained_launch();

__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... P, typename... A>
inline cudaError_t launch_chained(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    if (chained_launch()) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

#define LT_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            lt::set_error(__VA_ARGS__);       \
            return LT_ERR_INVALID;            \
        }                                     \
    } while (0)

#define LT_CUDA(call)                                                        \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) {                                            \
            lt::set_error("%s: %s", #call, cudaGetErrorString(e__));         \
            return LT_ERR_CUDA;                                              \
        }                                                                    \
    } while (0)

// Per-device "done once" flags.  cudaFuncSetAttribute and occupancy are per-device properties, so a
// launcher that caches either must key the cache by the current device (a process may drive several
// GPUs).  first() returns true exactly once per device (racing threads may both see true: the guarded
// calls are idempotent).
struct PerDeviceOnce {
    bool done[64] = {};
    bool first() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
        if (done[dev]) return false;
        done[dev] = true;
        return true;
    }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- device helpers

// 128-bit streaming load of weights: read-only path, do not keep in L1.
__device__ __forceinline__ int4 ld_stream_v4(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned short ld_stream_u16(const void* p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// exact integer dot of one 32-byte Q8_0 block held as two int4
__device__ __forceinline__ int block_dot(const int4& w0, const int4& w1, const int4& x0, const int4& x1) {
    int s = 0;
    s = __dp4a(w0.x, x0.x, s); s = __dp4a(w0.y, x0.y, s);
    s = __dp4a(w0.z, x0.z, s); s = __dp4a(w0.w, x0.w, s);
    s = __dp4a(w1.x, x1.x, s); s = __dp4a(w1.y, x1.y, s);
    s = __dp4a(w1.z, x1.z, s); s = __dp4a(w1.w, x1.w, s);
    return s;
}

// The frozen fp32 step of the Q8_0 GEMV: acc = fma(wd*xd, (float)isum, acc), one rounding
// for the product of the scales and one for the fused multiply-add.
__device__ __forceinline__ float q8_accum(float wd, float xd, int isum, float acc) {
    return __fmaf_rn(__fmul_rn(wd, xd), (float)isum, acc);
}

// 5-level shuffle-down tree over the 32 lane partials (s = 16, 8, 4, 2, 1); lane 0 holds
// the row result.
__device__ __forceinline__ float warp_tree_sum(float acc) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, s));
    return acc;
}

// Activation quantiser for one value of a 32-block whose lanes hold the block:
// amax over the warp, d = amax/127 (1 if amax == 0), stored as fp16; q = clamp(rint(v / f32(d))).
__device__ __forceinline__ int quant_lane(float v, __half* d_out) {
    float a = fabsf(v);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        float o = __shfl_xor_sync(0xffffffffu, a, s);
        if (o > a) a = o;
    }
    float d = (a > 0.0f) ? __fdiv_rn(a, 127.0f) : 1.0f;
    __half dh = __float2half_rn(d);
    *d_out = dh;
    float dq = __half2float(dh);
    int q = (int)rintf(__fdiv_rn(v, dq));
    q = q < -127 ? -127 : (q > 127 ? 127 : q);
    return q;
}

__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

}  // namespace lt
