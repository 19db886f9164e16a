// Decode step operators for a batch of sequences and for long contexts.
//
// Same per-(sequence, head) arithmetic as the one-sequence kernels (lt_elementwise.cu,
// lt_attn.cu) -- the reference has no batched engine, its contract is that every sequence gets
// the one-sequence result (bpd/lib/dev_residency.py:1344-1350).  What differs is the spread of
// the work: the attention of one (sequence, head) is three launches, so that a long context is
// scanned by many CTAs while every fp32 fold keeps its frozen order:
//   scores   one thread per cached position (sequential-i fma, * scale), all query heads of a
//            KV head from one read of the K row                -> S[b, h, t]
//   softmax  one CTA per (b, h): max, __expf, Z on the 64-lane strided layout + tree -> P, Z
//   V sum    one thread per output element, left fold over t, the query heads of a KV head
//            sharing the V rows                                -> OUT[b, h, d] = fold / Z
// The KV caches of the batch are one buffer per layer, [B][max_seq][nkv*hd], with a device
// length per sequence.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

constexpr int BT = 256;
constexpr int MAX_REP = 8;   // query heads per KV head handled together

// ------------------------------------------------------------------ rope, one position per row
__global__ void k_rope_batch(float* __restrict__ X, int ld, const int* __restrict__ pos, int nrows, int n_head, int hd,
                             float theta) {
    const int half = hd / 2;
    const long total = (long)nrows * n_head * half;
    const long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const int j = gid % half;
    const long hr = gid / half;
    const int head = hr % n_head;
    const int row = hr / n_head;
    const long base = (long)row * ld + (long)head * hd;
    float o1, o2;
    rope_pair(X[base + j], X[base + j + half], j, hd, theta, pos[row], o1, o2);
    X[base + j] = o1;
    X[base + j + half] = o2;
}

// ------------------------------------------------------------------ append one row per sequence
__global__ void k_append_kv_batch(float* __restrict__ kbase, const float* __restrict__ ksrc, float* __restrict__ vbase,
                                  const float* __restrict__ vsrc, int src_ld, int* __restrict__ lens, int width,
                                  int max_seq, int incr, int* status) {
    const int b = blockIdx.x;
    const int L = lens[b];
    const bool ok = L >= 0 && L < max_seq;
    if (ok) {
        const long off = ((long)b * max_seq + L) * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            kbase[off + i] = ksrc[(long)b * src_ld + i];
            vbase[off + i] = vsrc[(long)b * src_ld + i];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ok) atomicOr(status, (int)LT_STATUS_KV_OVERFLOW);
        else if (incr) lens[b] = L + 1;
    }
}

// ------------------------------------------------------------------ rope + append in one launch
// grid (chunks, B): a CTA rotates 256 (x1, x2) pairs of the row's q and k heads at position lens[b];
// rotated k pairs and the CTA's slice of the v row go straight to the cache at that position.  The
// last CTA of a sequence to finish (a ticket per sequence, self-resetting) advances the length, when
// every CTA of the sequence has long read it.  Same values as k_rope_batch + k_append_kv_batch.
__global__ void __launch_bounds__(256)
k_rope_append_batch(float* __restrict__ X, int ld, int n_qhead, int n_kvhead, int hd, float theta,
                    float* __restrict__ kbase, float* __restrict__ vbase, int* __restrict__ lens, int max_seq,
                    int* __restrict__ ticket, int* status) {
    chain_release();
    chain_wait();
    const int b = blockIdx.y;
    const int L = lens[b];
    const bool ok = L >= 0 && L < max_seq;
    const int half = hd / 2;
    float* row = X + (long)b * ld;
    const int pairs = (n_qhead + n_kvhead) * half;
    const int width = n_kvhead * hd;
    const long off = ((long)b * max_seq + (ok ? L : 0)) * width;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < pairs) {
        const int head = i / half, j = i - head * half;
        const long base = (long)head * hd;
        float o1, o2;
        rope_pair(row[base + j], row[base + j + half], j, hd, theta, L, o1, o2);
        row[base + j] = o1;
        row[base + j + half] = o2;
        if (ok && head >= n_qhead) {
            const long kb = off + (long)(head - n_qhead) * hd;
            kbase[kb + j] = o1;
            kbase[kb + j + half] = o2;
        }
    }
    if (ok) {   // this CTA's slice of the v row
        const float* vsrc = row + (long)(n_qhead + n_kvhead) * hd;
        for (int c = blockIdx.x * 256 + threadIdx.x; c < width; c += gridDim.x * 256) vbase[off + c] = vsrc[c];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int t = atomicAdd(&ticket[b], 1);
        if (t == (int)gridDim.x - 1) {
            ticket[b] = 0;
            if (!ok) atomicOr(status, (int)LT_STATUS_KV_OVERFLOW);
            else lens[b] = L + 1;
        }
    }
}

// ------------------------------------------------------------------ attention, phase 1: scores
// grid (tiles of SC_PT positions, nkv, B); S[(b*nh + h)*s_ld + t].  The CTA brings its SC_PT K rows into shared
// memory with asynchronous copies by all threads (coalesced; 16-byte chunk c of row p lands at chunk
// c ^ (p & 7)), then a thread folds one (position, query head) score, s = fold_i fma(q[i], k[i], s), from
// shared memory without bank conflicts.
constexpr int SC_PT = 64;

__device__ __forceinline__ void sc_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}

__global__ void __launch_bounds__(BT)
k_attn_scores(const float* __restrict__ Q, int q_ld, const float* __restrict__ K, const int* __restrict__ lens,
              float* __restrict__ S, int s_ld, int hd, int nh, int nkv, float scale, int max_seq, int* status) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float sc_smem[];
    const int b = blockIdx.z, hk = blockIdx.y;
    const int rep = nh / nkv;
    float* qs = sc_smem;                 // [rep][hd]
    float* ks = qs + rep * hd;           // [SC_PT][hd], swizzled
    int L = lens[b];
    if (L < 0 || L > max_seq) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, (int)LT_STATUS_BAD_LENGTH);
        L = L < 0 ? 0 : max_seq;
    }
    const int t0 = blockIdx.x * SC_PT;
    if (t0 >= L) return;
    const int n = L - t0 < SC_PT ? L - t0 : SC_PT;
    const int cpr = hd >> 2;
    const float* Kb = K + (((long)b * max_seq + t0) * nkv + hk) * hd;
    const long kstride = (long)nkv * hd;
    for (int i = threadIdx.x; i < n * cpr; i += BT) {
        const int row = i / cpr, c = i - row * cpr;
        sc_cp_async16(ks + (size_t)row * hd + ((c ^ (row & 7)) << 2), Kb + (long)row * kstride + c * 4);
    }
    for (int i = threadIdx.x; i < rep * hd; i += BT) qs[i] = Q[(long)b * q_ld + (long)hk * rep * hd + i];
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    const int p = threadIdx.x & (SC_PT - 1);
    if (p >= n) return;
    const float4* Kt = (const float4*)(ks + (size_t)p * hd);
    const int sw = p & 7;
    for (int r = threadIdx.x / SC_PT; r < rep; r += BT / SC_PT) {
        const float4* qr = (const float4*)(qs + r * hd);
        float s = 0.0f;
        for (int i0 = 0; i0 < cpr; i0 += 8) {   // hd is a multiple of 32
            float4 kk[8];
#pragma unroll
            for (int u = 0; u < 8; u++) kk[u] = Kt[(i0 + u) ^ sw];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float4 qq = qr[i0 + u];
                s = __fmaf_rn(qq.x, kk[u].x, s);
                s = __fmaf_rn(qq.y, kk[u].y, s);
                s = __fmaf_rn(qq.z, kk[u].z, s);
                s = __fmaf_rn(qq.w, kk[u].w, s);
            }
        }
        S[((long)b * nh + hk * rep + r) * s_ld + t0 + p] = __fmul_rn(s, scale);
    }
}

// ------------------------------------------------------------------ phase 2: softmax numerators and Z
// grid (nh, B); the row is staged in shared memory (max_seq floats)
__global__ void __launch_bounds__(BT)
k_attn_softmax(float* __restrict__ S, int s_ld, const int* __restrict__ lens, float* __restrict__ Z, int nh,
               int max_seq) {
    chain_release();
    chain_wait();
    extern __shared__ float sh[];
    __shared__ float red[64];
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    int L = lens[b];
    L = L < 0 ? 0 : (L > max_seq ? max_seq : L);
    float* row = S + ((long)b * nh + h) * s_ld;
    for (int t = d; t < L; t += BT) sh[t] = row[t];
    __syncthreads();
    // max (exact in any order; the one-sequence kernel also scans the masked -1e30 entries)
    if (d < 64) {
        float m = -1e30f;
        for (int t = d; t < L; t += 64) m = fmaxf(m, sh[t]);
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
    const float mx = red[0];
    __syncthreads();
    for (int t = d; t < L; t += BT) {
        const float p = __expf(__fsub_rn(sh[t], mx));
        sh[t] = p;
        row[t] = p;
    }
    __syncthreads();
    // Z: lane r sums t = r, r+64, ... ascending; masked entries of the one-sequence kernel add +0
    if (d < 64) {
        float ls = 0.0f;
        for (int t = d; t < L; t += 64) ls = __fadd_rn(ls, sh[t]);
        red[d] = ls;
    }
    __syncthreads();
    if (d < 32) {
        float v = __fadd_rn(red[d], red[d + 32]);
        v = warp_tree_sum(v);
        if (d == 0) Z[(long)b * nh + h] = v;
    }
}

// ------------------------------------------------------------------ phase 3: V sum
// grid (hd/32, nkv, B), block = 32 output elements x rep query heads.  The fold over t is one
// dependent chain per output element; what can be spread is the loading: the CTA stages tiles of
// PV_TT positions (its 32 columns of V, and the probabilities of its heads) in shared memory with
// asynchronous copies, one tile ahead of the fold.
// PV_TT positions per tile: 128 when few CTAs stream the cache, 64 for a batch (smaller CTAs: all of them resident at once)
// tiles in flight per CTA: 4 when few CTAs stream the cache (one sequence: each CTA's V stream is
// latency-bound otherwise), 2 when the batch supplies CTAs enough and residency matters more
constexpr size_t pv_smem(int stages, int tt) { return (size_t)stages * (tt * 32 + MAX_REP * tt) * sizeof(float); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}

template <int PV_STAGES, int PV_TT>
__global__ void __launch_bounds__(32 * MAX_REP)
k_attn_pv(const float* __restrict__ P, int s_ld, const float* __restrict__ V, const int* __restrict__ lens,
          const float* __restrict__ Z, float* __restrict__ OUT, int out_ld, int hd, int nh, int nkv, int max_seq,
          int8_t* __restrict__ Xq, __half* __restrict__ Xd) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float pv_buf[];
    float (*vt)[PV_TT][32] = (float (*)[PV_TT][32])pv_buf;                                  // [stage][t][d]
    float (*pt)[MAX_REP][PV_TT] = (float (*)[MAX_REP][PV_TT])(pv_buf + PV_STAGES * PV_TT * 32);   // [stage][head][t]
    const int b = blockIdx.z, hk = blockIdx.y;
    const int rep = nh / nkv;
    const int dl = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int d0 = blockIdx.x * 32;
    const int h = hk * rep + r;
    int L = lens[b];
    L = L < 0 ? 0 : (L > max_seq ? max_seq : L);
    const float* Vb = V + ((long)b * max_seq * nkv + hk) * hd + d0;
    const long vs = (long)nkv * hd;
    const float* Pb = P + ((long)b * nh + (long)hk * rep) * s_ld;
    const int nthreads = 32 * rep;
    const int tiles = (L + PV_TT - 1) / PV_TT;

    auto stage = [&](int k) {   // always commits a group, so that group k is tile k
        if (k < tiles) {
            const int buf = k % PV_STAGES, t0 = k * PV_TT;
            for (int i = threadIdx.x; i < PV_TT * 8; i += nthreads) {
                const int row = i >> 3, c = i & 7;
                if (t0 + row < L) cp_async16(&vt[buf][row][c * 4], Vb + (long)(t0 + row) * vs + c * 4);
            }
            for (int i = threadIdx.x; i < rep * (PV_TT / 4); i += nthreads) {
                const int hr = i / (PV_TT / 4), c = i - hr * (PV_TT / 4);
                if (t0 + c * 4 < L) cp_async16(&pt[buf][hr][c * 4], Pb + (long)hr * s_ld + t0 + c * 4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc = 0.0f;
    for (int k = 0; k < PV_STAGES - 1; k++) stage(k);
    for (int k = 0; k < tiles; k++) {
        stage(k + PV_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(PV_STAGES - 1) : "memory");
        __syncthreads();
        const int buf = k % PV_STAGES;
        const int n = L - k * PV_TT < PV_TT ? L - k * PV_TT : PV_TT;
        const float* pr = pt[buf][r];
        const float* vc = &vt[buf][0][dl];
        int t = 0;
        // the fold is one dependent chain; the shared-memory reads of 16 steps are issued together, ahead of it
        for (; t + 16 <= n; t += 16) {
            float pp[16], vv[16];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float4 p4 = *(const float4*)(pr + t + 4 * u);
                pp[4 * u] = p4.x; pp[4 * u + 1] = p4.y; pp[4 * u + 2] = p4.z; pp[4 * u + 3] = p4.w;
            }
#pragma unroll
            for (int u = 0; u < 16; u++) vv[u] = vc[(t + u) * 32];
#pragma unroll
            for (int u = 0; u < 16; u++) acc = __fmaf_rn(pp[u], vv[u], acc);
        }
        for (; t < n; t++) acc = __fmaf_rn(pr[t], vc[t * 32], acc);
        __syncthreads();
    }
    const float o = __fdiv_rn(acc, Z[(long)b * nh + h]);
    OUT[(long)b * out_ld + (long)h * hd + d0 + dl] = o;
    if (Xq != nullptr) {   // a warp holds one whole 32-block of the attention row: quantise it here
        __half dh;
        const int q = quant_lane(o, &dh);
        const long col = (long)h * hd + d0 + dl;
        Xq[(long)b * nh * hd + col] = (int8_t)q;
        if (dl == 0) Xd[((long)b * nh * hd + col) >> 5] = dh;
    }
}

// ------------------------------------------------------------------ attention, declared split order
// The reference's second declared order for decode attention, reduction_order(attn_decode_split, ...)
// (bpd/lib/ir_param_axes.pl:307-346; kernel text bpd/kernelgen/experimental/attn_decode_split.cu, launched
// with 64 threads by bpd/kernelgen/referee/gatebench_attn_split.py): the positions are cut into S contiguous
// ranges of ceil(L/S); each range takes its own max, exponentiates against it, sums Z on 64 strided lanes +
// tree and left-folds its V sum; a second launch rescales the ranges by exp(local max - global max) and
// adds them in ascending range order.  S is part of the order (fix it per captured graph).  It is a
// re-canonicalisation of the one-pass order, not a faster way to the same bits; what it buys is that the
// dependent V-sum chain is L/S long.
// grid (S, nkv, B); a CTA serves the rep query heads of its KV head.  scratch: partM, partZ [B][nh][S],
// partO [B][nh][S][hd].
constexpr int SPLIT_PT = 64;   // positions per staged V tile

__global__ void __launch_bounds__(1024)
k_attn_split(const float* Q, int q_ld, float* K, float* V,      // K, V, lens: written too when X != NULL, so no __restrict__
             int* lens, float* __restrict__ partM, float* __restrict__ partZ,
             float* __restrict__ partO, int hd, int nh, int nkv, float scale, int max_seq, int per_max, int kstage,
             int* status, const float* X, float theta, int* ticket) {
    // X != NULL: the row arrives as q | k | v straight from the projection (q_ld floats apart, Q = X).  The CTA
    // rotates its own query heads while its K rows are on the way (k_rope at position lens[b]); the CTA whose
    // range ends with the new position rotates the row's k head and appends k and v to the cache first; the last
    // CTA of the sequence to finish advances lens[b] (self-resetting ticket).  Same values as
    // k_rope_append_batch followed by this kernel.
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float sp_smem[];
    const int S = gridDim.x, sp = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int rep = nh / nkv;
    float* qs = sp_smem;                 // [rep][hd]
    float* red = qs + rep * hd;          // [rep][64]
    float* mz = red + rep * 64;          // [rep] local max
    float* sh = mz + ((rep + 3) & ~3);   // [rep][per_max] scores, then exponentials
    const int tid = threadIdx.x;
    const bool fused = X != nullptr;
    const int L0 = lens[b];
    const bool room = L0 >= 0 && L0 < max_seq;          // fused: the new row fits
    int L = fused && room ? L0 + 1 : L0;
    if (L < 0 || L > max_seq) {
        if (tid == 0 && sp == 0) atomicOr(status, (int)LT_STATUS_BAD_LENGTH);
        L = L < 0 ? 0 : max_seq;
    }
    const int per = (L + S - 1) / S;
    const int p0 = sp * per;
    int p1 = p0 + per;
    if (p1 > L) p1 = L;
    const int rangeN = p1 > p0 ? p1 - p0 : 0;
    if (fused && room && L0 >= p0 && L0 < p1) {     // this CTA's range ends with the new position: append it first
        const int half = hd >> 1;
        const float* xr = X + (long)b * q_ld;
        const float* ksrc = xr + (long)nh * hd + (long)hk * hd;
        const float* vsrc = xr + (long)(nh + nkv) * hd + (long)hk * hd;
        float* kdst = K + (((long)b * max_seq + L0) * nkv + hk) * hd;
        float* vdst = V + (((long)b * max_seq + L0) * nkv + hk) * hd;
        for (int j = tid; j < half; j += blockDim.x) {
            float o1, o2;
            rope_pair(ksrc[j], ksrc[j + half], j, hd, theta, L0, o1, o2);
            kdst[j] = o1;
            kdst[j + half] = o2;
        }
        for (int c = tid; c < hd; c += blockDim.x) vdst[c] = vsrc[c];
        __threadfence();
        __syncthreads();
    }
    // Everything the CTA will read is requested at once with asynchronous copies: the K rows of the range
    // (kstage: they fit beside the rest; 16-byte chunk c of row t lands at chunk c ^ (t & 7), so that the
    // one-thread-per-position reads below are free of bank conflicts) and the first two V tiles.
    float* vt = sh + (size_t)rep * per_max;   // [2][SPLIT_PT][hd]
    float* ks = vt + 2 * (size_t)SPLIT_PT * hd;   // [per_max][hd], swizzled (kstage only)
    const float* Vb = V + (((long)b * max_seq + p0) * nkv + hk) * hd;
    const long vs = (long)nkv * hd;
    const int cpr = hd >> 2;                  // 16-byte chunks per row
    const int ntile = (rangeN + SPLIT_PT - 1) / SPLIT_PT;
    auto stage = [&](int k) {
        if (k < ntile) {
            float* dst = vt + (size_t)(k & 1) * SPLIT_PT * hd;
            const int t0 = k * SPLIT_PT;
            for (int i = tid; i < SPLIT_PT * cpr; i += blockDim.x) {
                const int row = i / cpr, c = i - row * cpr;
                if (t0 + row < rangeN) cp_async16(dst + row * hd + c * 4, Vb + (long)(t0 + row) * vs + c * 4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (kstage) {
        const float* Kb = K + (((long)b * max_seq + p0) * nkv + hk) * hd;
        for (int i = tid; i < rangeN * cpr; i += blockDim.x) {
            const int row = i / cpr, c = i - row * cpr;
            cp_async16(ks + (size_t)row * hd + ((c ^ (row & 7)) << 2), Kb + (long)row * vs + c * 4);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    stage(0);
    stage(1);
    if (fused) {
        const int half = hd >> 1;
        const float* qsrc = X + (long)b * q_ld + (long)hk * rep * hd;
        for (int i = tid; i < rep * half; i += blockDim.x) {
            const int r = i / half, j = i - r * half;
            float o1, o2;
            rope_pair(qsrc[r * hd + j], qsrc[r * hd + j + half], j, hd, theta, L0, o1, o2);
            qs[r * hd + j] = o1;
            qs[r * hd + j + half] = o2;
        }
    } else {
        for (int i = tid; i < rep * hd; i += blockDim.x) qs[i] = Q[(long)b * q_ld + (long)hk * rep * hd + i];
    }
    asm volatile("cp.async.wait_group 2;" ::: "memory");     // the K rows have landed (the V tiles may be in flight)
    __syncthreads();
    // scores of the range, once: s = fold_i fma(q[i], K[t, i], s), then * scale
    for (int t = p0 + tid; t < p1; t += blockDim.x) {
        const int tl = t - p0;
        const float4* Kt = kstage ? (const float4*)(ks + (size_t)tl * hd)
                                  : (const float4*)(K + (((long)b * max_seq + t) * nkv + hk) * hd);
        const int sw = kstage ? (tl & 7) : 0;
        float s[MAX_REP];
#pragma unroll
        for (int r = 0; r < MAX_REP; r++) s[r] = 0.0f;
        for (int i0 = 0; i0 < (hd >> 2); i0 += 8) {
            float4 kk[8];
#pragma unroll
            for (int u = 0; u < 8; u++) kk[u] = Kt[(i0 + u) ^ sw];
#pragma unroll
            for (int u = 0; u < 8; u++) {
#pragma unroll
                for (int r = 0; r < MAX_REP; r++) {
                    if (r < rep) {
                        const float4 qq = ((const float4*)(qs + r * hd))[i0 + u];
                        s[r] = __fmaf_rn(qq.x, kk[u].x, s[r]);
                        s[r] = __fmaf_rn(qq.y, kk[u].y, s[r]);
                        s[r] = __fmaf_rn(qq.z, kk[u].z, s[r]);
                        s[r] = __fmaf_rn(qq.w, kk[u].w, s[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MAX_REP; r++)
            if (r < rep) sh[r * per_max + tl] = __fmul_rn(s[r], scale);
    }
    __syncthreads();
    // per head on 64 lanes: local max, exponentials against it, Z (lane l sums t = l, l+64, ... of the range;
    // tree 32, 16, ..., 1)
    const int groups = blockDim.x >> 6, grp = tid >> 6, l64 = tid & 63;
    for (int r0 = 0; r0 < rep; r0 += groups) {
        const int r = r0 + grp;
        const bool on = r < rep;
        float* row = sh + (on ? r : 0) * per_max;
        float m = -1e30f;
        if (on)
            for (int t = l64; t < rangeN; t += 64) m = fmaxf(m, row[t]);
        if (on) red[r * 64 + l64] = m;
        __syncthreads();
        if (on && l64 < 32) {
            float v = fmaxf(red[r * 64 + l64], red[r * 64 + l64 + 32]);
#pragma unroll
            for (int s2 = 16; s2 > 0; s2 >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s2));
            if (l64 == 0) mz[r] = rangeN > 0 ? v : -1e30f;
        }
        __syncthreads();
        float ls = 0.0f;
        if (on) {
            const float lmx = mz[r];
            for (int t = l64; t < rangeN; t += 64) {
                const float p = __expf(__fsub_rn(row[t], lmx));
                row[t] = p;
                ls = __fadd_rn(ls, p);
            }
            red[r * 64 + l64] = ls;
        }
        __syncthreads();
        if (on && l64 < 32) {
            float v = __fadd_rn(red[r * 64 + l64], red[r * 64 + l64 + 32]);
            v = warp_tree_sum(v);
            if (l64 == 0) {
                const long o = ((long)b * nh + hk * rep + r) * S + sp;
                partM[o] = mz[r];
                partZ[o] = v;
            }
        }
        __syncthreads();
    }
    // partial V sum: left fold over the range, one thread per (head, output element).  The V rows of the
    // range arrive in tiles of SPLIT_PT positions (asynchronous copies by all threads, coalesced), two tiles
    // ahead of the fold, so that the chain never waits on global memory.
    const bool fold = tid < rep * hd;
    const int fr = fold ? tid / hd : 0, fd = fold ? tid - fr * hd : 0;
    const float* prow = sh + fr * per_max;
    float acc = 0.0f;
    for (int k = 0; k < ntile; k++) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");     // tile k has landed, tile k+1 may be in flight
        __syncthreads();
        if (fold) {
            const float* vc = vt + (size_t)(k & 1) * SPLIT_PT * hd + fd;
            const float* pr = prow + k * SPLIT_PT;
            const int n = rangeN - k * SPLIT_PT < SPLIT_PT ? rangeN - k * SPLIT_PT : SPLIT_PT;
            int t = 0;
            for (; t + 8 <= n; t += 8) {   // reads batched, fold order unchanged
                float pp[8], vv[8];
#pragma unroll
                for (int u = 0; u < 8; u++) { pp[u] = pr[t + u]; vv[u] = vc[(t + u) * hd]; }
#pragma unroll
                for (int u = 0; u < 8; u++) acc = __fmaf_rn(pp[u], vv[u], acc);
            }
            for (; t < n; t++) acc = __fmaf_rn(pr[t], vc[t * hd], acc);
        }
        __syncthreads();
        stage(k + 2);      // into the buffer just folded
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (fold) partO[(((long)b * nh + hk * rep + fr) * S + sp) * hd + fd] = acc;
    if (fused) {
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const int t = atomicAdd(&ticket[b], 1);
            if (t == (int)(gridDim.x * gridDim.y) - 1) {
                ticket[b] = 0;
                if (room) lens[b] = L0 + 1;
                else atomicOr(status, (int)LT_STATUS_KV_OVERFLOW);
            }
        }
    }
}

// grid (nh, B), block hd: global max over the ranges, w = __expf(local max - global max),
// Z = fold fma(w, partZ, Z), O = fold fma(w, partO, O) in ascending range order, OUT = O / Z
__global__ void k_attn_split_combine(const float* __restrict__ partM, const float* __restrict__ partZ,
                                     const float* __restrict__ partO, float* __restrict__ OUT, int out_ld, int hd, int nh,
                                     int S, int8_t* __restrict__ Xq, __half* __restrict__ Xd) {
    chain_release();
    chain_wait();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const long o = ((long)b * nh + h) * S;
    float M = -1e30f;
    for (int sp = 0; sp < S; sp++) M = fmaxf(M, partM[o + sp]);
    float Z = 0.0f, acc = 0.0f;
    for (int s0 = 0; s0 < S; s0 += 16) {      // 16 ranges' loads in flight together; fold order unchanged
        float pm[16], pz[16], po[16];
#pragma unroll
        for (int u = 0; u < 16; u++) {
            const int sp = s0 + u < S ? s0 + u : S - 1;
            pm[u] = partM[o + sp]; pz[u] = partZ[o + sp]; po[u] = partO[(o + sp) * hd + d];
        }
#pragma unroll
        for (int u = 0; u < 16; u++) {
            if (s0 + u < S) {
                const float w = __expf(__fsub_rn(pm[u], M));
                Z = __fmaf_rn(w, pz[u], Z);
                acc = __fmaf_rn(w, po[u], acc);
            }
        }
    }
    const float y = __fdiv_rn(acc, Z);
    OUT[(long)b * out_ld + (long)h * hd + d] = y;
    if (Xq != nullptr) {   // hd is a multiple of 32: a warp holds one 32-block of the output row
        __half dh;
        const int q = quant_lane(y, &dh);
        const long col = ((long)b * nh + h) * hd + d;
        Xq[col] = (int8_t)q;
        if ((d & 31) == 0) Xd[col >> 5] = dh;
    }
}

}  // namespace lt

using namespace lt;

extern "C" int lt_rope_batch(float* X, int ld, const int* pos, int nrows, int n_head, int hd, float theta,
                             void* stream) {
    LT_REQUIRE(X && pos, "lt_rope_batch: null pointer");
    LT_REQUIRE(nrows > 0 && n_head > 0 && hd > 0 && hd % 2 == 0 && ld >= n_head * hd,
               "lt_rope_batch: nrows=%d n_head=%d hd=%d ld=%d", nrows, n_head, hd, ld);
    const long total = (long)nrows * n_head * (hd / 2);
    k_rope_batch<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(X, ld, pos, nrows, n_head, hd, theta);
    return check_launch("lt_rope_batch");
}

extern "C" int lt_append_kv_batch(float* kbase, const float* ksrc, float* vbase, const float* vsrc, int src_ld,
                                  int* lens, int width, int max_seq, int B, int incr, void* stream) {
    LT_REQUIRE(kbase && ksrc && vbase && vsrc && lens, "lt_append_kv_batch: null pointer");
    LT_REQUIRE(width > 0 && max_seq > 0 && B > 0 && src_ld >= width, "lt_append_kv_batch: width=%d max_seq=%d B=%d src_ld=%d",
               width, max_seq, B, src_ld);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_append_kv_batch: status word unavailable");
    const int threads = width >= 1024 ? 1024 : ((width + 31) / 32) * 32;
    k_append_kv_batch<<<B, threads, 0, (cudaStream_t)stream>>>(kbase, ksrc, vbase, vsrc, src_ld, lens, width, max_seq,
                                                              incr, st);
    return check_launch("lt_append_kv_batch");
}

extern "C" int lt_rope_append_batch(float* X, int ld, int n_qhead, int n_kvhead, int hd, float theta, float* kbase,
                                    float* vbase, int* lens, int max_seq, int B, int* ticket, void* stream) {
    LT_REQUIRE(X && kbase && vbase && lens && ticket, "lt_rope_append_batch: null pointer");
    LT_REQUIRE(n_qhead > 0 && n_kvhead > 0 && hd > 0 && hd % 2 == 0 && B > 0 && max_seq > 0 &&
                   ld >= (n_qhead + 2 * n_kvhead) * hd,
               "lt_rope_append_batch: n_qhead=%d n_kvhead=%d hd=%d ld=%d B=%d max_seq=%d", n_qhead, n_kvhead, hd, ld, B, max_seq);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_rope_append_batch: status word unavailable");
    const int pairs = (n_qhead + n_kvhead) * (hd / 2);
    const cudaError_t e = launch_chained(k_rope_append_batch, dim3((pairs + 255) / 256, B), dim3(256), 0,
                                         (cudaStream_t)stream, X, ld, n_qhead, n_kvhead, hd, theta, kbase, vbase, lens,
                                         max_seq, ticket, st);
    return check_launch("lt_rope_append_batch", 1, e);
}

extern "C" long lt_attn_decode_batch_scratch_floats(int nh, int max_seq, int B) {
    const long s_ld = ((long)max_seq + 3) & ~3L;
    return (long)B * nh * s_ld + (long)B * nh;
}

extern "C" int lt_attn_decode_batch(const float* Q, int q_ld, const float* K, const float* V, const int* lens,
                                    float* OUT, int out_ld, float* scratch, int hd, int nh, int nkv, float scale,
                                    int max_seq, int B, int8_t* Xq, uint16_t* Xd, void* stream) {
    LT_REQUIRE((Xq == nullptr) == (Xd == nullptr), "lt_attn_decode_batch: Xq and Xd are given together or not at all");
    LT_REQUIRE(Q && K && V && lens && OUT && scratch, "lt_attn_decode_batch: null pointer");
    LT_REQUIRE(hd > 0 && hd % 32 == 0, "lt_attn_decode_batch: hd=%d must be a positive multiple of 32", hd);
    LT_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= MAX_REP,
               "lt_attn_decode_batch: nh=%d must be a multiple of nkv=%d with at most %d query heads per KV head", nh, nkv, MAX_REP);
    LT_REQUIRE(max_seq > 0 && max_seq <= 49152 && B > 0 && B <= 65535, "lt_attn_decode_batch: max_seq=%d (1..49152) B=%d", max_seq, B);
    LT_REQUIRE(q_ld >= nh * hd && out_ld >= nh * hd && q_ld % 4 == 0, "lt_attn_decode_batch: q_ld=%d out_ld=%d", q_ld, out_ld);
    LT_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(scratch), "lt_attn_decode_batch: Q, K, V and scratch must be 16-byte aligned");
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_attn_decode_batch: status word unavailable");
    cudaStream_t s = (cudaStream_t)stream;
    const int s_ld = (max_seq + 3) & ~3;
    float* S = scratch;
    float* Z = scratch + (long)B * nh * s_ld;
    const int rep = nh / nkv;
    const size_t sc_bytes = ((size_t)rep * hd + (size_t)SC_PT * hd) * sizeof(float);
    LT_REQUIRE(sc_bytes <= 200 * 1024, "lt_attn_decode_batch: hd=%d needs %zu bytes of shared memory for a K tile", hd, sc_bytes);
    static PerDeviceOnce attr_once;
    if (attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_attn_scores, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LT_CUDA(cudaFuncSetAttribute(k_attn_softmax, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LT_CUDA(cudaFuncSetAttribute(k_attn_pv<4, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pv_smem(4, 128)));
        LT_CUDA(cudaFuncSetAttribute(k_attn_pv<2, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pv_smem(2, 64)));
    }
    cudaError_t e = launch_chained(k_attn_scores, dim3((max_seq + SC_PT - 1) / SC_PT, nkv, B), dim3(BT), sc_bytes, s, Q,
                                   q_ld, K, lens, S, s_ld, hd, nh, nkv, scale, max_seq, st);
    if (e == cudaSuccess)
        e = launch_chained(k_attn_softmax, dim3(nh, B), dim3(BT), (size_t)max_seq * sizeof(float), s, S, s_ld, lens, Z, nh,
                           max_seq);
    if (e == cudaSuccess) {
        if ((long)(hd / 32) * nkv * B >= 592)
            e = launch_chained(k_attn_pv<2, 64>, dim3(hd / 32, nkv, B), dim3(32 * rep), pv_smem(2, 64), s, S, s_ld, V, lens, Z, OUT,
                               out_ld, hd, nh, nkv, max_seq, Xq, (__half*)Xd);
        else
            e = launch_chained(k_attn_pv<4, 128>, dim3(hd / 32, nkv, B), dim3(32 * rep), pv_smem(4, 128), s, S, s_ld, V, lens, Z, OUT,
                               out_ld, hd, nh, nkv, max_seq, Xq, (__half*)Xd);
    }
    return check_launch("lt_attn_decode_batch", 3, e);
}

extern "C" long lt_attn_decode_split_scratch_floats(int nh, int hd, int nsplit, int B) {
    return (long)B * nh * nsplit * (2 + (long)hd);
}

static int attn_split_launch(const char* what, const float* Q, int q_ld, const float* K, const float* V, const int* lens,
                             float* OUT, int out_ld, float* scratch, int hd, int nh, int nkv, float scale, int max_seq,
                             int B, int nsplit, int8_t* Xq, uint16_t* Xd, const float* X, float theta, int* ticket,
                             void* stream) {
    LT_REQUIRE(Q && K && V && lens && OUT && scratch, "%s: null pointer", what);
    LT_REQUIRE(hd > 0 && hd % 32 == 0 && hd <= 1024, "%s: hd=%d must be a multiple of 32, at most 1024", what, hd);
    LT_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= MAX_REP,
               "%s: nh=%d must be a multiple of nkv=%d with at most %d query heads per KV head", what, nh, nkv, MAX_REP);
    LT_REQUIRE(nsplit >= 1 && nsplit <= 1024, "%s: nsplit=%d (1..1024)", what, nsplit);
    LT_REQUIRE(max_seq > 0 && B > 0 && B <= 65535, "%s: max_seq=%d B=%d", what, max_seq, B);
    LT_REQUIRE(q_ld >= nh * hd && out_ld >= nh * hd && q_ld % 4 == 0, "%s: q_ld=%d out_ld=%d", what, q_ld, out_ld);
    LT_REQUIRE((Xq == nullptr) == (Xd == nullptr), "%s: Xq and Xd are given together or not at all", what);
    LT_REQUIRE(Xq == nullptr || out_ld == nh * hd, "%s: the quantised output needs out_ld == nh*hd", what);
    LT_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V), "%s: Q, K and V must be 16-byte aligned", what);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "%s: status word unavailable", what);
    cudaStream_t s = (cudaStream_t)stream;
    const int rep = nh / nkv;
    const int per_max = (((max_seq + nsplit - 1) / nsplit) + 3) & ~3;
    size_t smem = ((size_t)rep * hd + rep * 64 + ((rep + 3) & ~3) + (size_t)rep * per_max + 2 * (size_t)SPLIT_PT * hd) *
                  sizeof(float);
    LT_REQUIRE(smem <= 200 * 1024, "%s: max_seq=%d / nsplit=%d needs %zu bytes of shared memory", what, max_seq, nsplit, smem);
    // the K rows of a range are staged in shared memory too when they fit beside the rest
    const size_t kbytes = (size_t)per_max * hd * sizeof(float);
    const int kstage = smem + kbytes <= 227 * 1024 ? 1 : 0;
    if (kstage) smem += kbytes;
    static PerDeviceOnce attr_once;
    if (attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_attn_split, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    }
    int threads = ((rep * hd + 31) / 32) * 32;
    if (threads < 256) threads = 256;
    if (threads > 1024) threads = 1024;
    float* partM = scratch;
    float* partZ = partM + (long)B * nh * nsplit;
    float* partO = partZ + (long)B * nh * nsplit;
    cudaError_t e = launch_chained(k_attn_split, dim3(nsplit, nkv, B), dim3(threads), smem, s, Q, q_ld, (float*)K, (float*)V,
                                   (int*)lens, partM, partZ, partO, hd, nh, nkv, scale, max_seq, per_max, kstage, st, X, theta,
                                   ticket);
    if (e == cudaSuccess)
        e = launch_chained(k_attn_split_combine, dim3(nh, B), dim3(hd), 0, s, partM, partZ, partO, OUT, out_ld, hd, nh,
                           nsplit, Xq, (__half*)Xd);
    return check_launch(what, 2, e);
}

extern "C" int lt_attn_decode_split(const float* Q, int q_ld, const float* K, const float* V, const int* lens,
                                    float* OUT, int out_ld, float* scratch, int hd, int nh, int nkv, float scale,
                                    int max_seq, int B, int nsplit, int8_t* Xq, uint16_t* Xd, void* stream) {
    return attn_split_launch("lt_attn_decode_split", Q, q_ld, K, V, lens, OUT, out_ld, scratch, hd, nh, nkv, scale, max_seq, B,
                             nsplit, Xq, Xd, nullptr, 0.0f, nullptr, stream);
}

extern "C" int lt_rope_attn_decode_split(const float* X, int ld, float* K, float* V, int* lens, float* OUT, int out_ld,
                                         float* scratch, int hd, int nh, int nkv, float theta, float scale, int max_seq,
                                         int B, int nsplit, int* ticket, int8_t* Xq, uint16_t* Xd, void* stream) {
    LT_REQUIRE(X && ticket, "lt_rope_attn_decode_split: null pointer");
    LT_REQUIRE(ld >= (nh + 2 * nkv) * hd, "lt_rope_attn_decode_split: ld=%d is shorter than a q|k|v row", ld);
    return attn_split_launch("lt_rope_attn_decode_split", X, ld, K, V, lens, OUT, out_ld, scratch, hd, nh, nkv, scale, max_seq,
                             B, nsplit, Xq, Xd, X, theta, ticket, stream);
}
