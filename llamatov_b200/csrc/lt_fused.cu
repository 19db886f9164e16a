// One decode step as a chain of FUSED kernels linked by programmatic dependent launch.
//
// Five kernels per layer (q|k|v, attention, o_proj, gate|up, down), an LM-head kernel and a
// final argmax kernel.  Each kernel (a) lets its successor start launching at once
// (griddepcontrol.launch_dependents), (b) fetches everything that does not depend on its
// predecessor -- its weight rows, norm weights, cached K/V rows -- into shared memory with
// asynchronous copies, and only then (c) waits for the predecessor's results
// (griddepcontrol.wait).  Launch latency and the weight stream therefore overlap the
// predecessor's execution; what stays serial is a short activation prologue and the fold.
//
// Activations are quantised where they are produced whenever a producer owns whole 32-blocks
// (attention heads, gate|up blocks), so that the consumer's prologue is a plain copy.
// The arithmetic of every op is the per-op kernels' (same device functions, same orders), so
// the step is bit-identical to the chain of per-op launches.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

__device__ __forceinline__ unsigned fsmem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fcp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(fsmem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void fcp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(fsmem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void fcp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// asynchronous copy of one weight row (K quants, K/32 scales; K % 64 == 0) into shared memory
__device__ __forceinline__ void prefetch_row(unsigned char* dst, const int8_t* Wq, const __half* Wd, long row, int K,
                                             int lane) {
    const int nb = K >> 5;
    const int8_t* q = Wq + row * K;
    for (int c = lane; c < (K >> 4); c += 32) fcp_async16(dst + c * 16, q + c * 16);
    const unsigned char* d = (const unsigned char*)(Wd + row * nb);
    for (int c = lane; c < (nb >> 1); c += 32) fcp_async4(dst + K + c * 4, d + c * 4);
}

// fold one row held in shared memory (layout of prefetch_row) with the activation in sXq / sXd
__device__ __forceinline__ float fold_row(const unsigned char* w, int K, const int8_t* sXq, const __half* sXd, int lane) {
    const int nb = K >> 5;
    const __half* wd = (const __half*)(w + K);
    float acc = 0.0f;
    for (int b = lane; b < nb; b += 32) {
        const int4* wp = (const int4*)(w + b * 32);
        const int4* xp = (const int4*)(sXq + b * 32);
        const int4 w0 = wp[0], w1 = wp[1], x0 = xp[0], x1 = xp[1];
        acc = q8_accum(__half2float(wd[b]), __half2float(sXd[b]), block_dot(w0, w1, x0, x1), acc);
    }
    return acc;
}

struct FusedArgs {
    const int8_t* Wq; const __half* Wd; int M, K;
    // activation: f32 vector (+ norm weight) to be quantised here, or an already quantised one
    const float* x; const float* normw; float eps;
    const int8_t* xq; const __half* xd;
    // embedding gather for the first kernel of a step
    const int* tok; const int8_t* emb_q; const __half* emb_d; int V; float* x_copy;
    // epilogue
    const float* add; float* out;
    int* len_incr; int max_seq;
    int* status;
};

// shared layout of k_fused_gemv: sXq[K] | sXd[K/32] (pad 16) | sred[272] | sF[K] | sW[K] | rows[8][K + K/16 (+pad)]
__device__ __forceinline__ int row_stride(int K) { return ((K + (K >> 4)) + 15) & ~15; }

// PRO: 0 = activation arrives quantised, 1 = f32 vector -> rmsnorm -> quant, 2 = embedding row -> rmsnorm -> quant
template <int PRO>
__global__ void __launch_bounds__(256) k_fused_gemv(const FusedArgs a) {
    extern __shared__ __align__(16) unsigned char fsm[];
    const int K = a.K, nb = K >> 5;
    int8_t* sXq = (int8_t*)fsm;
    __half* sXd = (__half*)(fsm + K);
    size_t off = ((size_t)K + nb * 2 + 15) & ~(size_t)15;
    float* sred = (float*)(fsm + off);
    off += 272 * 4;
    float* sF = (float*)(fsm + off);
    float* sW = sF + (PRO ? K : 0);
    off += (PRO ? (size_t)2 * K * 4 : 0);
    unsigned char* rows = fsm + off;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long row = (long)blockIdx.x * 8 + warp;

    pdl_launch_dependents();
    // ---- independent of the predecessor: this warp's weight row, the norm weight
    if (row < a.M) prefetch_row(rows + (size_t)warp * row_stride(K), a.Wq, a.Wd, row, K, lane);
    if (PRO)
        for (int c = threadIdx.x; c < (K >> 2); c += 256) fcp_async16(sW + c * 4, a.normw + c * 4);
    float addv = 0.0f;
    pdl_wait();
    // ---- activation
    if (PRO == 0) {
        for (int c = threadIdx.x; c < (K >> 4); c += 256) ((int4*)sXq)[c] = __ldcg((const int4*)a.xq + c);
        for (int c = threadIdx.x; c < (nb >> 1); c += 256) ((unsigned*)sXd)[c] = __ldcg((const unsigned*)a.xd + c);
    } else if (PRO == 1) {
        for (int j = threadIdx.x; j < K; j += 256) sF[j] = __ldcg(a.x + j);
    } else {
        int t = __ldcg(a.tok);
        if (t < 0 || t >= a.V) {
            if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(a.status, (int)LT_STATUS_BAD_TOKEN);
            t = t < 0 ? 0 : a.V - 1;
        }
        for (int j = threadIdx.x; j < K; j += 256) {
            const float v = __fmul_rn(__half2float(a.emb_d[(size_t)t * nb + (j >> 5)]), (float)a.emb_q[(size_t)t * K + j]);
            sF[j] = v;
            if (blockIdx.x == 0) a.x_copy[j] = v;
        }
    }
    if (a.add != nullptr && lane == 0 && row < a.M) addv = __ldcg(a.add + row);
    if (a.len_incr != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        const int p = __ldcg(a.len_incr);
        if (p >= 0 && p < a.max_seq) *a.len_incr = p + 1;
    }
    fcp_async_wait_all();
    __syncthreads();
    if (PRO) {
        const float ss = block_rms_sumsq(sF, K, sred);
        const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)K), a.eps));
        block_quant(sF, sW, inv, K, sXq, sXd);
        __syncthreads();
    }
    if (row < a.M) {
        float v = warp_tree_sum(fold_row(rows + (size_t)warp * row_stride(K), K, sXq, sXd, lane));
        if (lane == 0) {
            if (a.add != nullptr) v = __fadd_rn(v, addv);
            a.out[row] = v;
        }
    }
}

// gate|up: one CTA per 32-row block of the FFN (16 warps, two row pairs each).  The CTA forms
// v = silu(gate)*up for its block and quantises it, so the down projection receives Q8_0.
struct GateUpArgs {
    const int8_t* Wq; const __half* Wd; int F, K;      // [2F, K], rows gate | up
    const float* x; const float* normw; float eps;
    int8_t* vq; __half* vd;                            // [F], [F/32]
};

__global__ void __launch_bounds__(512) k_fused_gateup(const GateUpArgs a) {
    extern __shared__ __align__(16) unsigned char fsm[];
    const int K = a.K, nb = K >> 5;
    int8_t* sXq = (int8_t*)fsm;
    __half* sXd = (__half*)(fsm + K);
    size_t off = ((size_t)K + nb * 2 + 15) & ~(size_t)15;
    float* sred = (float*)(fsm + off);
    off += 272 * 4;
    float* sv = (float*)(fsm + off);      // 32 activations of the block
    off += 32 * 4;
    float* sF = (float*)(fsm + off);
    float* sW = sF + K;
    off += (size_t)2 * K * 4;
    unsigned char* rows = fsm + off;      // 64 rows: gate[32] then up[32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long blk = blockIdx.x;
    const int rs = row_stride(K);

    pdl_launch_dependents();
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int i = warp * 2 + k;
        prefetch_row(rows + (size_t)i * rs, a.Wq, a.Wd, blk * 32 + i, K, lane);
        prefetch_row(rows + (size_t)(32 + i) * rs, a.Wq, a.Wd, (long)a.F + blk * 32 + i, K, lane);
    }
    for (int c = threadIdx.x; c < (K >> 2); c += 512) fcp_async16(sW + c * 4, a.normw + c * 4);
    pdl_wait();
    for (int j = threadIdx.x; j < K; j += 512) sF[j] = __ldcg(a.x + j);
    fcp_async_wait_all();
    __syncthreads();
    const float ss = block_rms_sumsq(sF, K, sred);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)K), a.eps));
    block_quant(sF, sW, inv, K, sXq, sXd);
    __syncthreads();
    float acc[4];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int i = warp * 2 + k;
        acc[k] = fold_row(rows + (size_t)i * rs, K, sXq, sXd, lane);
        acc[2 + k] = fold_row(rows + (size_t)(32 + i) * rs, K, sXq, sXd, lane);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
#pragma unroll
        for (int k = 0; k < 4; k++) acc[k] = __fadd_rn(acc[k], __shfl_down_sync(0xffffffffu, acc[k], s));
    }
    if (lane == 0) {
        sv[warp * 2] = silu_mul(acc[0], acc[2]);
        sv[warp * 2 + 1] = silu_mul(acc[1], acc[3]);
    }
    __syncthreads();
    if (warp == 0) {
        __half dh;
        const int q = quant_lane(sv[lane], &dh);
        a.vq[blk * 32 + lane] = (int8_t)q;
        if (lane == 0) a.vd[blk] = dh;
    }
}

// attention: one CTA per query head, 256 threads; rope + KV append + masked attention, output
// quantised (a head is hd/32 whole blocks).
struct AttnArgs {
    const float* qkv; float* kcache; float* vcache; const int* len;
    int8_t* aq; __half* ad;
    int hd, nh, nkv, maxt, vcap; float theta, scale;
    int* status;
};

__global__ void __launch_bounds__(256) k_fused_attn(const AttnArgs a) {
    extern __shared__ __align__(16) unsigned char fsm[];
    float* sh = (float*)fsm;
    const int hd = a.hd, hd4 = hd >> 2, nh = a.nh, nkv = a.nkv, maxt = a.maxt, kst = hd + 4;
    float* sQ = sh + maxt;
    float* sKn = sQ + hd;
    float* sVn = sKn + hd;
    float* so = sVn + hd;
    float* red = so + hd;              // 64 + 2
    float* sV = red + 68;
    float* sK = sV + (size_t)a.vcap * hd;
    const int h = blockIdx.x, tid = threadIdx.x;
    const int nq = nh * hd, nk = nkv * hd, rep = nh / nkv, hk = h / rep;

    pdl_launch_dependents();
    // the cache length was last changed by the previous step: readable before the wait
    int pos = __ldcg(a.len);
    const bool room = (pos >= 0 && pos < maxt);
    if (!room) {
        if (tid == 0) atomicOr(a.status, (int)LT_STATUS_KV_OVERFLOW);
        pos = pos < 0 ? 0 : maxt;
    }
    const int L = room ? pos + 1 : pos, Lc = room ? pos : L;
    const bool staged = (L <= a.vcap);
    if (staged) {
        for (int e = tid; e < Lc * hd4; e += 256) {
            const int t = e / hd4, c = e - t * hd4;
            const size_t g = ((size_t)t * nkv + hk) * hd + c * 4;
            fcp_async16(sK + (size_t)t * kst + c * 4, a.kcache + g);
            fcp_async16(sV + (size_t)t * hd + c * 4, a.vcache + g);
        }
    }
    // rope angles depend on the position only: evaluated before the predecessor is awaited
    const int half = hd >> 1;
    float rc = 1.0f, rs = 0.0f;
    if (tid < half) rope_trig(tid, hd, a.theta, pos, rc, rs);
    else if (tid >= 64 && tid < 64 + half) rope_trig(tid - 64, hd, a.theta, pos, rc, rs);
    pdl_wait();
    if (tid < half) {
        float o1, o2;
        rope_rotate(__ldcg(a.qkv + h * hd + tid), __ldcg(a.qkv + h * hd + tid + half), rc, rs, o1, o2);
        sQ[tid] = o1; sQ[tid + half] = o2;
    } else if (tid >= 64 && tid < 64 + half) {
        const int j = tid - 64;
        float o1, o2;
        rope_rotate(__ldcg(a.qkv + nq + hk * hd + j), __ldcg(a.qkv + nq + hk * hd + j + half), rc, rs, o1, o2);
        sKn[j] = o1; sKn[j + half] = o2;
        if (room && staged) { sK[(size_t)pos * kst + j] = o1; sK[(size_t)pos * kst + j + half] = o2; }
    } else if (tid >= 128 && tid < 128 + hd) {
        const int j = tid - 128;
        const float v = __ldcg(a.qkv + nq + nk + hk * hd + j);
        sVn[j] = v;
        if (room && staged) sV[(size_t)pos * hd + j] = v;
    }
    fcp_async_wait_all();
    __syncthreads();
    if (room && (h % rep) == 0 && tid < hd) {
        a.kcache[((size_t)pos * nkv + hk) * hd + tid] = sKn[tid];
        a.vcache[((size_t)pos * nkv + hk) * hd + tid] = sVn[tid];
    }
    for (int t = tid; t < maxt; t += 256) {
        float v = -1e30f;
        if (t < L) {
            const float4* K4 = staged ? (const float4*)(sK + (size_t)t * kst)
                                      : ((room && t == pos) ? (const float4*)sKn
                                                            : (const float4*)(a.kcache + ((size_t)t * nkv + hk) * hd));
            const float4* q4 = (const float4*)sQ;
            float s = 0.0f;
#pragma unroll 4
            for (int i = 0; i < hd4; i++) {
                const float4 kk = K4[i];
                const float4 qq = q4[i];
                s = __fmaf_rn(qq.x, kk.x, s);
                s = __fmaf_rn(qq.y, kk.y, s);
                s = __fmaf_rn(qq.z, kk.z, s);
                s = __fmaf_rn(qq.w, kk.w, s);
            }
            v = __fmul_rn(s, a.scale);
        }
        sh[t] = v;
    }
    __syncthreads();
    if (tid < 64) {
        float m = -1e30f;
        for (int t = tid; t < maxt; t += 64) m = fmaxf(m, sh[t]);
        red[tid] = m;
    }
    __syncthreads();
    if (tid < 32) {
        float v = fmaxf(red[tid], red[tid + 32]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
        if (tid == 0) red[64] = v;
    }
    __syncthreads();
    const float mx = red[64];
    for (int t = tid; t < maxt; t += 256) sh[t] = __expf(__fsub_rn(sh[t], mx));
    __syncthreads();
    if (tid < 64) {
        float ls = 0.0f;
        for (int t = tid; t < maxt; t += 64) ls = __fadd_rn(ls, sh[t]);
        red[tid] = ls;
    }
    __syncthreads();
    if (tid < 32) {
        float v = __fadd_rn(red[tid], red[tid + 32]);
        v = warp_tree_sum(v);
        if (tid == 0) red[65] = v;
    }
    __syncthreads();
    const float Z = red[65];
    if (tid < hd) {
        float acc = 0.0f;
        if (staged) {
#pragma unroll 4
            for (int t = 0; t < L; t++) acc = __fmaf_rn(sh[t], sV[(size_t)t * hd + tid], acc);
        } else {
            const float* Vd = a.vcache + (size_t)hk * hd + tid;
            const size_t stride = (size_t)nkv * hd;
            int t = 0;
            for (; t + 8 <= Lc; t += 8) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = Vd[(size_t)(t + k) * stride];
#pragma unroll
                for (int k = 0; k < 8; k++) acc = __fmaf_rn(sh[t + k], v[k], acc);
            }
            for (; t < Lc; t++) acc = __fmaf_rn(sh[t], Vd[(size_t)t * stride], acc);
            if (room) acc = __fmaf_rn(sh[pos], sVn[tid], acc);
        }
        so[tid] = __fdiv_rn(acc, Z);
    }
    __syncthreads();
    // quantise the head's output: hd/32 blocks, one warp each
    const int warp = tid >> 5, lane = tid & 31;
    if (warp < (hd >> 5)) {
        __half dh;
        const int q = quant_lane(so[warp * 32 + lane], &dh);
        a.aq[h * hd + warp * 32 + lane] = (int8_t)q;
        if (lane == 0) a.ad[(h * hd >> 5) + warp] = dh;
    }
}

// LM head: prologue as k_fused_gemv<1>, then a grid-stride walk over the vocabulary rows with
// the weights streamed from global memory; each CTA leaves its best (value, index).
struct LmArgs {
    const int8_t* Wq; const __half* Wd; int V, K;
    const float* x; const float* normw; float eps;
    float* logits; float* part_val; int* part_idx;
};

__global__ void __launch_bounds__(256) k_fused_lmhead(const LmArgs a) {
    extern __shared__ __align__(16) unsigned char fsm[];
    const int K = a.K, nb = K >> 5;
    int8_t* sXq = (int8_t*)fsm;
    __half* sXd = (__half*)(fsm + K);
    size_t off = ((size_t)K + nb * 2 + 15) & ~(size_t)15;
    float* sred = (float*)(fsm + off);
    off += 272 * 4;
    float* sF = (float*)(fsm + off);
    float* sW = sF + K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int R = 4;
    const long warps_total = (long)gridDim.x * 8;
    long r0 = ((long)blockIdx.x * 8 + warp) * R;

    pdl_launch_dependents();
    for (int c = threadIdx.x; c < (K >> 2); c += 256) fcp_async16(sW + c * 4, a.normw + c * 4);
    // first group of rows: weights into registers before the predecessor is awaited
    int4 w0[R], w1[R];
    float wd[R];
    const bool one_block = (nb <= 32);
#pragma unroll
    for (int r = 0; r < R; r++) {
        w0[r] = make_int4(0, 0, 0, 0); w1[r] = w0[r]; wd[r] = 0.0f;
        if (one_block && lane < nb && r0 + r < a.V) {
            const int8_t* p = a.Wq + (r0 + r) * K + lane * 32;
            w0[r] = ld_stream_v4(p);
            w1[r] = ld_stream_v4(p + 16);
            wd[r] = __half2float(__ushort_as_half(ld_stream_u16(a.Wd + (r0 + r) * nb + lane)));
        }
    }
    pdl_wait();
    for (int j = threadIdx.x; j < K; j += 256) sF[j] = __ldcg(a.x + j);
    fcp_async_wait_all();
    __syncthreads();
    const float ss = block_rms_sumsq(sF, K, sred);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)K), a.eps));
    block_quant(sF, sW, inv, K, sXq, sXd);
    __syncthreads();
    float bestv = -3.4e38f;
    int besti = 2147483647;
    bool first = one_block;
    for (; r0 < a.V; r0 += warps_total * R) {
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] = 0.0f;
        for (int b = lane; b < nb; b += 32) {
            if (!first) {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    if (r0 + r < a.V) {
                        const int8_t* p = a.Wq + (r0 + r) * K + (long)b * 32;
                        w0[r] = ld_stream_v4(p);
                        w1[r] = ld_stream_v4(p + 16);
                        wd[r] = __half2float(__ushort_as_half(ld_stream_u16(a.Wd + (r0 + r) * nb + b)));
                    } else {
                        w0[r] = make_int4(0, 0, 0, 0); w1[r] = w0[r]; wd[r] = 0.0f;
                    }
                }
            }
            const int4* xp = (const int4*)(sXq + b * 32);
            const int4 x0 = xp[0], x1 = xp[1];
            const float xd = __half2float(sXd[b]);
#pragma unroll
            for (int r = 0; r < R; r++) acc[r] = q8_accum(wd[r], xd, block_dot(w0[r], w1[r], x0, x1), acc[r]);
        }
        first = false;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
#pragma unroll
            for (int r = 0; r < R; r++) acc[r] = __fadd_rn(acc[r], __shfl_down_sync(0xffffffffu, acc[r], s));
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; r++) {
                const long row = r0 + r;
                if (row < a.V) {
                    a.logits[row] = acc[r];
                    if (acc[r] > bestv || (acc[r] == bestv && (int)row < besti)) { bestv = acc[r]; besti = (int)row; }
                }
            }
        }
    }
    // block best (lane 0 of each warp holds a candidate)
    float* bv = sred;
    int* bi = (int*)(sred + 8);
    if (lane == 0) { bv[warp] = bestv; bi[warp] = besti; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = bv[0];
        int i = bi[0];
        for (int w = 1; w < 8; w++)
            if (bv[w] > v || (bv[w] == v && bi[w] < i)) { v = bv[w]; i = bi[w]; }
        a.part_val[blockIdx.x] = v;
        a.part_idx[blockIdx.x] = i;
    }
}

struct FinalArgs {
    const float* part_val; const int* part_idx; int nparts;
    int* out_tok; int* tok; int* history; int* step; int hist_cap;
};

__global__ void __launch_bounds__(256) k_fused_argmax(const FinalArgs a) {
    __shared__ float sv[8];
    __shared__ int si[8];
    pdl_launch_dependents();
    pdl_wait();
    float bv = -3.4e38f;
    int bi = 2147483647;
    for (int c = threadIdx.x; c < a.nparts; c += 256) {
        const float v = __ldcg(a.part_val + c);
        const int i = __ldcg(a.part_idx + c);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        *a.out_tok = bi;
        if (a.tok != nullptr) *a.tok = bi;
        if (a.history != nullptr) {
            const int s = *a.step;
            if (s >= 0 && s < a.hist_cap) a.history[s] = bi;
            *a.step = s + 1;
        }
    }
}

template <typename Kern, typename Args>
static int launch_pdl(Kern kern, const Args& args, int grid, int block, size_t smem, cudaStream_t s, const char* what) {
    if (smem > 48 * 1024) LT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args);
    if (e != cudaSuccess) {
        set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
        return LT_ERR_CUDA;
    }
    count_launches(1);
    return LT_OK;
}

static size_t gemv_smem(int K, bool pro) {
    size_t off = ((size_t)K + (K >> 5) * 2 + 15) & ~(size_t)15;
    off += 272 * 4;
    if (pro) off += (size_t)2 * K * 4;
    off += (size_t)8 * ((K + (K >> 4) + 15) & ~15);
    return off;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_decode_step_pdl(const lt_decode_desc* d, void* stream) {
    LT_REQUIRE(d != nullptr, "lt_decode_step_pdl: null descriptor");
    LT_REQUIRE(d->layers && d->h_layers && d->out_norm && d->lm_q && d->lm_d && d->logits && d->out_tok && d->part_val &&
                   d->part_idx && d->ws_x && d->ws_x1 && d->ws_qkv && d->ws_att && d->ws_v,
               "lt_decode_step_pdl: null pointer in descriptor (h_layers is the host copy of the layer array)");
    LT_REQUIRE(d->tok != nullptr ? (d->emb_q && d->emb_d) : (d->x != nullptr),
               "lt_decode_step_pdl: needs either a device token with the embedding table or a preloaded input row");
    const int E = d->E, F = d->F, hd = d->hd, nq = d->nh * hd, nk = d->nkv * hd, nqkv = nq + 2 * nk;
    LT_REQUIRE(E % 64 == 0 && F % 64 == 0 && nq % 64 == 0, "lt_decode_step_pdl: E, F and nh*hd must be multiples of 64");
    LT_REQUIRE(hd == 32 || hd == 64 || hd == 128, "lt_decode_step_pdl: hd=%d must be 32, 64 or 128", hd);
    LT_REQUIRE(d->nkv > 0 && d->nh % d->nkv == 0 && d->max_seq % 4 == 0, "lt_decode_step_pdl: bad head / cache geometry");
    cudaStream_t s = (cudaStream_t)stream;
    int* status = d->status ? d->status : device_status_ptr();
    LT_REQUIRE(status != nullptr, "lt_decode_step_pdl: status word unavailable");
    int dev = 0, sms = 148, smem_max = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    LT_REQUIRE(gemv_smem(F, false) <= (size_t)smem_max && gemv_smem(E, true) <= (size_t)smem_max,
               "lt_decode_step_pdl: model dimensions need more shared memory than one SM has");

    float* x = (float*)d->ws_x;             // residual stream
    float* x1 = (float*)d->ws_x1;
    float* qkv = (float*)d->ws_qkv;
    int8_t* aq = (int8_t*)d->ws_att;
    __half* ad = (__half*)((unsigned char*)d->ws_att + nq);
    int8_t* vq = (int8_t*)d->ws_v;
    __half* vd = (__half*)((unsigned char*)d->ws_v + F);

    // attention shared memory: probabilities, q / new k / new v / out, reductions, staged K and V rows
    const size_t att_fixed = ((size_t)d->max_seq + 4 * hd + 68) * 4;
    const size_t att_row = (size_t)hd * 4 + (size_t)(hd + 4) * 4;
    int vcap = (int)(((size_t)smem_max - 2048 - att_fixed) / att_row);
    if (vcap > d->max_seq) vcap = d->max_seq;
    const size_t att_smem = att_fixed + (size_t)vcap * att_row;
    const size_t gu_smem = (((size_t)E + (E >> 5) * 2 + 15) & ~(size_t)15) + 272 * 4 + 32 * 4 + (size_t)2 * E * 4 +
                           (size_t)64 * ((E + (E >> 4) + 15) & ~15);
    LT_REQUIRE(gu_smem <= (size_t)smem_max, "lt_decode_step_pdl: gate|up block does not fit shared memory (E=%d)", E);

    for (int il = 0; il < d->n_layers; il++) {
        const lt_decode_layer* ly = d->h_layers + il;
        int rc;
        {   // q|k|v
            FusedArgs a = {};
            a.Wq = ly->qkv_q; a.Wd = (const __half*)ly->qkv_d; a.M = nqkv; a.K = E;
            a.normw = ly->attn_norm; a.eps = d->eps; a.add = ly->qkv_bias; a.out = qkv; a.status = status;
            if (il == 0 && d->tok != nullptr) {
                a.tok = d->tok; a.emb_q = d->emb_q; a.emb_d = (const __half*)d->emb_d; a.V = d->V; a.x_copy = x;
                rc = launch_pdl(k_fused_gemv<2>, a, (nqkv + 7) / 8, 256, gemv_smem(E, true), s, "lt_decode_step_pdl(qkv)");
            } else {
                a.x = (il == 0) ? d->x : x;
                rc = launch_pdl(k_fused_gemv<1>, a, (nqkv + 7) / 8, 256, gemv_smem(E, true), s, "lt_decode_step_pdl(qkv)");
            }
            if (rc != LT_OK) return rc;
        }
        {   // attention
            AttnArgs a = {};
            a.qkv = qkv; a.kcache = ly->kcache; a.vcache = ly->vcache; a.len = ly->len; a.aq = aq; a.ad = ad;
            a.hd = hd; a.nh = d->nh; a.nkv = d->nkv; a.maxt = d->max_seq; a.vcap = vcap; a.theta = d->theta;
            a.scale = d->scale; a.status = status;
            rc = launch_pdl(k_fused_attn, a, d->nh, 256, att_smem, s, "lt_decode_step_pdl(attn)");
            if (rc != LT_OK) return rc;
        }
        {   // o_proj + residual (x, or the input row for layer 0 in host mode)
            FusedArgs a = {};
            a.Wq = ly->o_q; a.Wd = (const __half*)ly->o_d; a.M = E; a.K = nq; a.xq = aq; a.xd = ad;
            a.add = (il == 0 && d->tok == nullptr) ? d->x : x; a.out = x1; a.len_incr = ly->len; a.max_seq = d->max_seq;
            a.status = status;
            rc = launch_pdl(k_fused_gemv<0>, a, (E + 7) / 8, 256, gemv_smem(nq, false), s, "lt_decode_step_pdl(o)");
            if (rc != LT_OK) return rc;
        }
        {   // gate|up -> quantised silu(gate)*up
            GateUpArgs a = {};
            a.Wq = ly->gu_q; a.Wd = (const __half*)ly->gu_d; a.F = F; a.K = E; a.x = x1; a.normw = ly->ffn_norm;
            a.eps = d->eps; a.vq = vq; a.vd = vd;
            rc = launch_pdl(k_fused_gateup, a, F / 32, 512, gu_smem, s, "lt_decode_step_pdl(gateup)");
            if (rc != LT_OK) return rc;
        }
        {   // down + residual
            FusedArgs a = {};
            a.Wq = ly->down_q; a.Wd = (const __half*)ly->down_d; a.M = E; a.K = F; a.xq = vq; a.xd = vd; a.add = x1;
            a.out = x; a.status = status;
            rc = launch_pdl(k_fused_gemv<0>, a, (E + 7) / 8, 256, gemv_smem(F, false), s, "lt_decode_step_pdl(down)");
            if (rc != LT_OK) return rc;
        }
    }
    {
        LmArgs a = {};
        a.Wq = d->lm_q; a.Wd = (const __half*)d->lm_d; a.V = d->V; a.K = E; a.x = x; a.normw = d->out_norm; a.eps = d->eps;
        a.logits = d->logits; a.part_val = d->part_val; a.part_idx = d->part_idx;
        const int grid = sms * 4;
        const size_t smem = (((size_t)E + (E >> 5) * 2 + 15) & ~(size_t)15) + 272 * 4 + (size_t)2 * E * 4;
        int rc = launch_pdl(k_fused_lmhead, a, grid, 256, smem, s, "lt_decode_step_pdl(lm)");
        if (rc != LT_OK) return rc;
        FinalArgs f = {};
        f.part_val = d->part_val; f.part_idx = d->part_idx; f.nparts = grid; f.out_tok = d->out_tok; f.tok = d->tok;
        f.history = d->history; f.step = d->step; f.hist_cap = d->hist_cap;
        rc = launch_pdl(k_fused_argmax, f, 1, 256, 0, s, "lt_decode_step_pdl(argmax)");
        if (rc != LT_OK) return rc;
    }
    return LT_OK;
}

extern "C" int lt_decode_pdl_num_parts(void) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms * 4;
}
