// Q8_0 quantiser and GEMV / GEMM in the fold order of the reference's COMPILED CPU PATH
// (bpd-substrate/bench/bpd_cpu.c:4096-4126, bpd_gemm_q8_0_cpu.c:53-132,205-260, which mirror ggml's AVX
// kernels), so that the GPU result can be compared bit for bit with that library as well as with the
// resident engine's declared order.  Not used by the decode engine; a parity mode.
//
//   quantiser   d = fp16(amax/127), id = 127/amax (0 if amax == 0), q = rint(x * id)
//   one token   8 float lanes; lanes 0-3 take the even blocks, lanes 4-7 the odd ones; lane k sums the bytes
//               4k..4k+3 of both 16-byte halves of its block (exact int), then acc = d*float(isum) + acc with
//               TWO roundings (multiply, then add); blocks in pairs, an odd last block is not visited
//   2+ tokens   tiles of 4 or 2 tokens: every block feeds all 8 lanes (lane k = bytes 4k..4k+3), same two
//               roundings; an odd last token falls back to the one-token form
//   result      ((l4+l0) + (l6+l2)) + ((l5+l1) + (l7+l3))
// Mapping: a thread is one lane of one (token, row) result, eight threads per result, shuffles for the sum.
#include "lt_common.cuh"

namespace lt {

__global__ void __launch_bounds__(256) k_quant_q8_ggml(const float* __restrict__ X, int8_t* __restrict__ Xq,
                                                        __half* __restrict__ Xd, long nblocks) {
    const long b = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (b >= nblocks) return;
    const float v = X[b * 32 + lane];
    float a = fabsf(v);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, a, s);
        if (o > a) a = o;
    }
    if (lane == 0) Xd[b] = __float2half_rn(__fdiv_rn(a, 127.0f));
    const float id = a != 0.0f ? __fdiv_rn(127.0f, a) : 0.0f;
    Xq[b * 32 + lane] = (int8_t)(int)rintf(__fmul_rn(v, id));
}

__global__ void __launch_bounds__(256)
k_q8_gemm_ggml(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd, const int8_t* __restrict__ Xq,
               const __half* __restrict__ Xd, float* __restrict__ Y, int M, int K, int T) {
    const int nb = K >> 5;
    const long res = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;   // (token, row) index
    const int k = threadIdx.x & 7;
    const bool on = res < (long)T * M;
    const int t = on ? (int)(res / M) : 0, n = on ? (int)(res - (long)t * M) : 0;
    const int8_t* wq = Wq + (long)n * K;
    const __half* wd = Wd + (long)n * nb;
    const int8_t* xq = Xq + (long)t * K;
    const __half* xd = Xd + (long)t * nb;
    const bool vec = (T & 1) && t == T - 1;
    float acc = 0.0f;
    if (on) {
        if (vec) {
            const int h = k >> 2, kk = k & 3;
            for (int b = h; b < (nb & ~1); b += 2) {   // pairs (2p, 2p+1) with 2p + 1 < nb
                const int is = __dp4a(*(const int*)(wq + b * 32 + 4 * kk), *(const int*)(xq + b * 32 + 4 * kk), 0) +
                               __dp4a(*(const int*)(wq + b * 32 + 16 + 4 * kk), *(const int*)(xq + b * 32 + 16 + 4 * kk), 0);
                const float dl = __fmul_rn(__half2float(wd[b]), __half2float(xd[b]));
                acc = __fadd_rn(__fmul_rn(dl, (float)is), acc);
            }
        } else {
            for (int b = 0; b < nb; b++) {
                const int is = __dp4a(*(const int*)(wq + b * 32 + 4 * k), *(const int*)(xq + b * 32 + 4 * k), 0);
                const float sc = __fmul_rn(__half2float(wd[b]), __half2float(xd[b]));
                acc = __fadd_rn(__fmul_rn(sc, (float)is), acc);
            }
        }
    }
    // hsum_float_8 over the eight lanes of a result
    acc = __fadd_rn(__shfl_down_sync(0xffffffffu, acc, 4, 8), acc);
    acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 2, 8));
    acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 1, 8));
    if (on && k == 0) Y[(long)t * M + n] = acc;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_quant_q8_ggml(const float* X, int8_t* Xq, uint16_t* Xd, int K, int rows, void* stream) {
    LT_REQUIRE(X && Xq && Xd, "lt_quant_q8_ggml: null pointer");
    LT_REQUIRE(K > 0 && K % 32 == 0 && rows > 0, "lt_quant_q8_ggml: K=%d must be a positive multiple of 32, rows=%d > 0", K, rows);
    const long nblocks = (long)rows * (K / 32);
    k_quant_q8_ggml<<<(unsigned)((nblocks + 7) / 8), 256, 0, (cudaStream_t)stream>>>(X, Xq, (__half*)Xd, nblocks);
    return check_launch("lt_quant_q8_ggml");
}

extern "C" int lt_q8_gemm_ggml(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, float* Y,
                               int M, int K, int T, void* stream) {
    LT_REQUIRE(Wq && Wd && Xq && Xd && Y, "lt_q8_gemm_ggml: null pointer");
    LT_REQUIRE(M > 0 && T > 0 && K > 0 && K % 32 == 0, "lt_q8_gemm_ggml: M=%d T=%d K=%d (K a multiple of 32)", M, T, K);
    LT_REQUIRE((reinterpret_cast<uintptr_t>(Wq) & 3u) == 0 && (reinterpret_cast<uintptr_t>(Xq) & 3u) == 0,
               "lt_q8_gemm_ggml: Wq and Xq must be 4-byte aligned");
    const long threads = (long)T * M * 8;
    k_q8_gemm_ggml<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        Wq, (const __half*)Wd, Xq, (const __half*)Xd, Y, M, K, T);
    return check_launch("lt_q8_gemm_ggml");
}
