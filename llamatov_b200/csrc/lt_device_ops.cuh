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

}  // namespace lt
