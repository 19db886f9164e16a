// Decode attention (one query token) over the resident fp32 KV cache, GQA.
//
// Frozen arithmetic, per query head h (kv head hk = h / (nh/nkv)), L = *len:
//   score_t = (fold_i fma(q[h,i], K[t,hk,i], .)) * scale      for t < L,  -1e30 for t >= L
//   mx      = max over t  (64 strided lanes, then a tree; exact in any order)
//   p_t     = __expf(score_t - mx)
//   Z       = 64 lanes, lane r sums t = r, r+64, ... ascending; tree s = 32 .. 1
//   out_d   = (left fold over t < L of fma(p_t, V[t,hk,d], .)) / Z
// Nothing stored at positions >= L may influence the result.
//
// Mapping: one CTA per query head; scores and exponentials are spread over all threads
// (each is independent), the two softmax reductions run on the frozen 64-lane layout, the
// V sum runs one thread per output element.
#include "lt_common.cuh"

namespace lt {

constexpr int ATTN_THREADS = 256;

// Z in the frozen order from the probabilities in shared memory (masked entries hold +0).
__device__ __forceinline__ float softmax_denominator(const float* sh, int maxt, float* red) {
    int d = threadIdx.x;
    if (d < 64) {
        float ls = 0.0f;
        for (int t = d; t < maxt; t += 64) ls = __fadd_rn(ls, sh[t]);
        red[d] = ls;
    }
    __syncthreads();
    if (d < 32) {
        float v = __fadd_rn(red[d], red[d + 32]);
        v = warp_tree_sum(v);
        if (d == 0) red[0] = v;
    }
    __syncthreads();
    float Z = red[0];
    __syncthreads();
    return Z;
}

__device__ __forceinline__ float block_max(const float* sh, int maxt, float* red) {
    int d = threadIdx.x;
    if (d < 64) {
        float m = -1e30f;
        for (int t = d; t < maxt; t += 64) m = fmaxf(m, sh[t]);
        red[d] = m;
    }
    __syncthreads();
    if (d < 32) {
        float v = fmaxf(red[d], red[d + 32]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
        if (d == 0) red[0] = v;
    }
    __syncthreads();
    float mx = red[0];
    __syncthreads();
    return mx;
}

// grid = nh (one CTA per query head); dynamic shared = maxt floats.
__global__ void __launch_bounds__(ATTN_THREADS)
k_attn_decode_masked(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                     const int* __restrict__ len_ptr, float* __restrict__ OUT, int hd, int nh, int nkv, float scale,
                     int maxt, int* status) {
    extern __shared__ float sh[];
    __shared__ float red[64];
    const int h = blockIdx.x;
    const int d = threadIdx.x;
    int L = *len_ptr;
    if (L < 0 || L > maxt) {
        if (d == 0) atomicOr(status, (int)LT_STATUS_BAD_LENGTH);
        L = L < 0 ? 0 : maxt;
    }
    const int rep = nh / nkv, hk = h / rep;
    const float* qh = Q + (long)h * hd;
    for (int t = d; t < maxt; t += ATTN_THREADS) {
        float v = -1e30f;
        if (t < L) {
            const float4* Kt = (const float4*)(K + ((long)t * nkv + hk) * hd);
            const float4* q4 = (const float4*)qh;
            float s = 0.0f;
            for (int i = 0; i < (hd >> 2); i++) {
                float4 kk = Kt[i];
                float4 qq = q4[i];
                s = __fmaf_rn(qq.x, kk.x, s);
                s = __fmaf_rn(qq.y, kk.y, s);
                s = __fmaf_rn(qq.z, kk.z, s);
                s = __fmaf_rn(qq.w, kk.w, s);
            }
            v = __fmul_rn(s, scale);
        }
        sh[t] = v;
    }
    __syncthreads();
    const float mx = block_max(sh, maxt, red);
    for (int t = d; t < maxt; t += ATTN_THREADS) sh[t] = __expf(__fsub_rn(sh[t], mx));
    __syncthreads();
    const float Z = softmax_denominator(sh, maxt, red);
    if (d < hd) {
        const float* Vd = V + (long)hk * hd + d;
        const long stride = (long)nkv * hd;
        float acc = 0.0f;
        int t = 0;
        for (; t + 4 <= L; t += 4) {  // loads batched, fold order unchanged
            float v0 = Vd[(long)t * stride], v1 = Vd[(long)(t + 1) * stride];
            float v2 = Vd[(long)(t + 2) * stride], v3 = Vd[(long)(t + 3) * stride];
            acc = __fmaf_rn(sh[t], v0, acc);
            acc = __fmaf_rn(sh[t + 1], v1, acc);
            acc = __fmaf_rn(sh[t + 2], v2, acc);
            acc = __fmaf_rn(sh[t + 3], v3, acc);
        }
        for (; t < L; t++) acc = __fmaf_rn(sh[t], Vd[(long)t * stride], acc);
        OUT[(long)h * hd + d] = __fdiv_rn(acc, Z);
    }
}

}  // namespace lt

using namespace lt;

extern "C" int lt_attn_decode_masked(const float* Q, const float* K, const float* V, const int* len, float* OUT,
                                     int hd, int nh, int nkv, float scale, int maxt, void* stream) {
    LT_REQUIRE(Q && K && V && len && OUT, "lt_attn_decode_masked: null pointer");
    LT_REQUIRE(hd > 0 && hd % 4 == 0 && hd <= ATTN_THREADS, "lt_attn_decode_masked: hd=%d must be a multiple of 4, at most %d", hd, ATTN_THREADS);
    LT_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "lt_attn_decode_masked: nh=%d must be a positive multiple of nkv=%d", nh, nkv);
    LT_REQUIRE(maxt > 0 && maxt <= 49152, "lt_attn_decode_masked: maxt=%d out of range (1..49152)", maxt);
    LT_REQUIRE(aligned16(Q) && aligned16(K), "lt_attn_decode_masked: Q and K must be 16-byte aligned");
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_attn_decode_masked: status word unavailable");
    size_t smem = (size_t)maxt * sizeof(float);
    if (smem > 48 * 1024)
        LT_CUDA(cudaFuncSetAttribute(k_attn_decode_masked, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    k_attn_decode_masked<<<nh, ATTN_THREADS, smem, (cudaStream_t)stream>>>(Q, K, V, len, OUT, hd, nh, nkv, scale, maxt,
                                                                         st);
    return check_launch("lt_attn_decode_masked");
}
