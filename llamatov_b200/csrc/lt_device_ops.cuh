// Device functions shared by the stand-alone kernels and the fused decode step, so that
// both execute literally the same arithmetic.
#pragma once
#include "lt_common.cuh"

namespace lt {

// NeoX half-split rotation of one (x1, x2) pair of a head at integer position `pos`:
// freq = powf(theta, -(2j)/hd), ang = pos * freq, o1 = x1*cos - x2*sin, o2 = x1*sin + x2*cos.
// The reference kernel's source leaves the two output expressions to nvcc's default
// contraction; compiled for sm_100a it comes out as
//     o1 = fma(x1, cos, -(x2*sin))      o2 = fma(x2, cos, x1*sin)
// (found by comparing the explicit candidates with the reference's own kernel bit for bit on
// the GPU, which the parity tests keep doing).  It is written out here so that no context can
// change it.  The angle part depends only on (j, pos), so a fused kernel may evaluate it before
// its input has arrived.
__device__ __forceinline__ void rope_trig(int j, int hd, float theta, int pos, float& c, float& s) {
    float p = (float)pos;
    float freq = powf(theta, -(2.0f * (float)j) / (float)hd);
    float ang = p * freq;
    c = cosf(ang);
    s = sinf(ang);
}
__device__ __forceinline__ void rope_rotate(float x1, float x2, float c, float s, float& o1, float& o2) {
    o1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
    o2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
}
__device__ __forceinline__ void rope_pair(float x1, float x2, int j, int hd, float theta, int pos, float& o1,
                                          float& o2) {
    float c, s;
    rope_trig(j, hd, theta, pos, c, s);
    rope_rotate(x1, x2, c, s, o1, o2);
}

// ---- RMSNorm and quantiser over a vector in shared memory, for kernels that fuse them as a prologue
// sum of squares in the declared 256-lane order; the block has exactly 256 threads
__device__ __forceinline__ float block_rms_sumsq(const float* sF, int N, float* sred) {
    const int t = threadIdx.x;
    float local = 0.0f;
    if (t < 256)
        for (int j = t; j < N; j += 256) local = __fmaf_rn(sF[j], sF[j], local);
    if (t < 256) sred[t] = local;
    __syncthreads();
    if (t < 32) {
        const float* p = sred;   // levels 128, 64, 32 in the declared pairing, then 16 .. 1
        const float a = __fadd_rn(__fadd_rn(p[t], p[t + 128]), __fadd_rn(p[t + 64], p[t + 192]));
        const float b = __fadd_rn(__fadd_rn(p[t + 32], p[t + 160]), __fadd_rn(p[t + 96], p[t + 224]));
        const float v = warp_tree_sum(__fadd_rn(a, b));
        if (t == 0) sred[256] = v;
    }
    __syncthreads();
    return sred[256];
}

// quantise N floats of shared memory (optionally (x*inv)*w first) into sXq / sXd; all warps
__device__ __forceinline__ void block_quant(const float* sF, const float* sW, float inv, int N, int8_t* sXq,
                                            __half* sXd) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int nblk = N >> 5;
    for (int b0 = warp; b0 < nblk; b0 += 2 * nw) {
        float v[2], a[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int b = b0 + k * nw;
            const int j = (b < nblk ? b : b0) * 32 + lane;
            float x = sF[j];
            if (sW != nullptr) x = __fmul_rn(__fmul_rn(x, inv), sW[j]);
            v[k] = x;
            a[k] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(x))));
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int b = b0 + k * nw;
            if (b < nblk) {
                const float d = (a[k] > 0.0f) ? __fdiv_rn(a[k], 127.0f) : 1.0f;
                const __half dh = __float2half_rn(d);
                int q = (int)rintf(__fdiv_rn(v[k], __half2float(dh)));
                q = q < -127 ? -127 : (q > 127 ? 127 : q);
                sXq[b * 32 + lane] = (int8_t)q;
                if (lane == 0) sXd[b] = dh;
            }
        }
    }
}

}  // namespace lt
