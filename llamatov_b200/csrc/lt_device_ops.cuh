// Device functions shared by the stand-alone kernels and the fused decode step, so that
// both execute literally the same arithmetic.
#pragma once
#include "lt_common.cuh"

namespace lt {

// NeoX half-split rotation of one (x1, x2) pair of a head at integer position `pos`:
// freq = powf(theta, -(2j)/hd), ang = pos * freq, o1 = x1*cos - x2*sin, o2 = x1*sin + x2*cos.
// The two output expressions are left to the compiler's default contraction on purpose:
// that is what the reference kernel's source does, and the result is compared with it bit
// for bit on the GPU.  The angle part depends only on (j, pos), so a fused kernel may evaluate
// it before its input has arrived.
__device__ __forceinline__ void rope_trig(int j, int hd, float theta, int pos, float& c, float& s) {
    float p = (float)pos;
    float freq = powf(theta, -(2.0f * (float)j) / (float)hd);
    float ang = p * freq;
    c = cosf(ang);
    s = sinf(ang);
}
__device__ __forceinline__ void rope_rotate(float x1, float x2, float c, float s, float& o1, float& o2) {
    o1 = x1 * c - x2 * s;
    o2 = x1 * s + x2 * c;
}
__device__ __forceinline__ void rope_pair(float x1, float x2, int j, int hd, float theta, int pos, float& o1,
                                          float& o2) {
    float c, s;
    rope_trig(j, hd, theta, pos, c, s);
    rope_rotate(x1, x2, c, s, o1, o2);
}

}  // namespace lt
