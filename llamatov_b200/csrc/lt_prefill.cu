// Row-batched forms of the decode operators, for prefilling a prompt in one pass.
//
// The reference prefills by running its one-token step once per prompt token
// (bpd/lib/dev_residency.py:1344-1350) and requires any batched form to give the same
// numbers.  Every kernel here therefore computes, for row r of the batch, exactly what the
// one-token kernel computes for that token: same fold orders, same device functions.  What
// changes is only how the work is spread: rows share one launch, and the causal attention
// reads each cached K/V row once per tile of query rows instead of once per query.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

// ------------------------------------------------------------------ embedding rows
__global__ void k_embed_q8_rows(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd,
                                const int* __restrict__ toks, float* __restrict__ out, int E, int V, int nrows,
                                int* status) {
    chain_release();
    chain_wait();
    const int r = blockIdx.x;
    if (r >= nrows) return;
    int t = toks[r];
    if (t < 0 || t >= V) {
        if (threadIdx.x == 0) atomicOr(status, (int)LT_STATUS_BAD_TOKEN);
        t = t < 0 ? 0 : V - 1;
    }
    const int nb = E >> 5;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float q = (float)Wq[(long)t * E + i];
        const float d = __half2float(Wd[(long)t * nb + (i >> 5)]);
        out[(long)r * E + i] = __fmul_rn(q, d);
    }
}

// ------------------------------------------------------------------ rope rows
// row r of X (row stride ld floats, n_head heads of hd at the row start) is rotated at position *pos0 + r
__global__ void k_rope_rows(float* __restrict__ X, int ld, const int* __restrict__ pos0, int nrows, int n_head, int hd,
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
    rope_pair(X[base + j], X[base + j + half], j, hd, theta, *pos0 + row, o1, o2);
    X[base + j] = o1;
    X[base + j + half] = o2;
}

// ------------------------------------------------------------------ KV append rows
// rows 0..nrows-1 of ksrc / vsrc (row stride src_ld) go to cache positions *len .. *len+nrows-1
__global__ void k_append_kv_rows(float* __restrict__ kbase, const float* __restrict__ ksrc, float* __restrict__ vbase,
                                 const float* __restrict__ vsrc, int src_ld, const int* __restrict__ len, int width,
                                 int max_seq, int nrows, int* status) {
    const int L = *len;
    if (L < 0 || L + nrows > max_seq) {
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, (int)LT_STATUS_KV_OVERFLOW);
        return;
    }
    const long total = (long)nrows * width;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int r = (int)(i / width), c = (int)(i - (long)r * width);
        kbase[(long)(L + r) * width + c] = ksrc[(long)r * src_ld + c];
        vbase[(long)(L + r) * width + c] = vsrc[(long)r * src_ld + c];
    }
}
__global__ void k_add_len(int* len, int n, int max_seq) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int L = *len;
        if (L >= 0 && L + n <= max_seq) *len = L + n;
    }
}

// ------------------------------------------------------------------ silu * up -> quant, strided rows
__global__ void k_silu_mul_quant_rows(const float* __restrict__ G, const float* __restrict__ U, int ld,
                                      int8_t* __restrict__ Xq, __half* __restrict__ Xd, int K, int rows) {
    chain_release();
    chain_wait();
    const int nb = K >> 5;
    const long blk = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= (long)rows * nb) return;
    const int r = (int)(blk / nb), b = (int)(blk - (long)r * nb);
    const long src = (long)r * ld + (long)b * 32 + lane;
    const float v = silu_mul(G[src], U[src]);
    __half d;
    const int q = quant_lane(v, &d);
    Xq[(long)r * K + (long)b * 32 + lane] = (int8_t)q;
    if (lane == 0) Xd[(long)r * nb + b] = d;
}

// ------------------------------------------------------------------ causal attention over a chunk of rows
// Row r of the chunk is the query at cache position L0 + r, L0 = *len - nrows (the chunk's K/V rows
// are already appended), and sees L_r = L0 + r + 1 positions.  Per (row, head) the arithmetic is the
// one-token kernel's (lt_attn.cu): sequential-i fma scores, * scale, max, __expf, Z on 64 strided
// lanes + tree, left-fold V sum, / Z.
constexpr int PF_THREADS = 256;
constexpr int PF_KTILE = 128;            // K rows staged per tile: two threads per position

template <int HD, int QT>
__global__ void __launch_bounds__(PF_THREADS, QT <= 8 ? 3 : 1)
k_attn_prefill(const float* __restrict__ Q, int q_ld, const float* __restrict__ K, const float* __restrict__ V,
               const int* __restrict__ len_ptr, float* __restrict__ OUT, int out_ld, int nh, int nkv, float scale,
               int nrows, int maxt, int* status) {
    extern __shared__ __align__(16) float pf_smem[];
    float* qs = pf_smem;                 // [QT][HD]
    float* red = qs + QT * HD;           // [QT][64]
    float* zs = red + QT * 64;           // [QT] max, then Z
    float* kt = zs + ((QT + 3) & ~3);    // [PF_KTILE][HD + 4] one tile of K rows (rows padded: conflict-free 16-byte reads)
    float* sc = kt + PF_KTILE * (HD + 4);   // [QT][ld], ld = maxt rounded up to 4 floats
    const int ld = (maxt + 3) & ~3;
    const int tid = threadIdx.x;
    const int h = blockIdx.y;
    const int r0 = blockIdx.x * QT;
    int Lafter = *len_ptr;
    if (Lafter < nrows || Lafter > maxt) {
        if (tid == 0) atomicOr(status, (int)LT_STATUS_BAD_LENGTH);
        return;
    }
    const int L0 = Lafter - nrows;
    const int nq = nrows - r0 < QT ? nrows - r0 : QT;   // query rows of this tile
    const int Lmax = L0 + r0 + nq;                      // positions the last row sees
    const int hk = h / (nh / nkv);

    for (int i = tid; i < QT * HD; i += PF_THREADS) {
        const int qi = i / HD, d = i - qi * HD;
        qs[i] = qi < nq ? Q[(long)(r0 + qi) * q_ld + (long)h * HD + d] : 0.0f;
    }
    __syncthreads();

    // scores: K rows go through shared memory in tiles of PF_KTILE positions (coalesced 16-byte asynchronous
    // copies; a thread reading its own row straight from global memory touches a new sector with every load).
    // A position of the tile is served by two threads, QT/2 queries each; each (row, query) score is the same
    // sequential-i fma chain as in the one-token kernel.
    constexpr int KST = HD + 4, QH = QT / 2;
    const int p = tid & (PF_KTILE - 1), qh = tid / PF_KTILE;
    for (int t0 = 0; t0 < Lmax; t0 += PF_KTILE) {
        const int nt = Lmax - t0 < PF_KTILE ? Lmax - t0 : PF_KTILE;
        for (int e = tid; e < nt * (HD / 4); e += PF_THREADS) {
            const int r = e / (HD / 4), c = e - r * (HD / 4);
            const float* src = K + ((long)(t0 + r) * nkv + hk) * HD + c * 4;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(kt + r * KST + c * 4)),
                         "l"(src) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        if (p < nt) {
            const int t = t0 + p;
            const float4* Kt = (const float4*)(kt + p * KST);
            float s[QH];
#pragma unroll
            for (int qi = 0; qi < QH; qi++) s[qi] = 0.0f;
#pragma unroll 4
            for (int i = 0; i < HD / 4; i++) {
                const float4 kk = Kt[i];
#pragma unroll
                for (int qi = 0; qi < QH; qi++) {
                    const float4 qq = ((const float4*)(qs + (qh * QH + qi) * HD))[i];
                    s[qi] = __fmaf_rn(qq.x, kk.x, s[qi]);
                    s[qi] = __fmaf_rn(qq.y, kk.y, s[qi]);
                    s[qi] = __fmaf_rn(qq.z, kk.z, s[qi]);
                    s[qi] = __fmaf_rn(qq.w, kk.w, s[qi]);
                }
            }
#pragma unroll
            for (int qi = 0; qi < QH; qi++) {
                const int q = qh * QH + qi;
                sc[q * ld + t] = t < L0 + r0 + q + 1 ? __fmul_rn(s[qi], scale) : -1e30f;
            }
        }
        __syncthreads();        // the tile is rewritten
    }

    // softmax per query row on the frozen 64-lane layout: 4 rows at a time, 64 threads each
    const int grp = tid >> 6, l64 = tid & 63;
    for (int qb = 0; qb < QT; qb += 4) {
        const int qi = qb + grp;
        float* row = sc + qi * ld;
        float m = -1e30f;
        for (int t = l64; t < Lmax; t += 64) m = fmaxf(m, row[t]);
        red[qi * 64 + l64] = m;
        __syncthreads();
        if (l64 < 32) {
            float v = fmaxf(red[qi * 64 + l64], red[qi * 64 + l64 + 32]);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
            if (l64 == 0) zs[qi] = v;
        }
        __syncthreads();
        const float mx = zs[qi];
        for (int t = l64; t < Lmax; t += 64) row[t] = __expf(__fsub_rn(row[t], mx));
        __syncthreads();
        float ls = 0.0f;
        for (int t = l64; t < Lmax; t += 64) ls = __fadd_rn(ls, row[t]);
        red[qi * 64 + l64] = ls;
        __syncthreads();
        if (l64 < 32) {
            float v = __fadd_rn(red[qi * 64 + l64], red[qi * 64 + l64 + 32]);
            v = warp_tree_sum(v);
            if (l64 == 0) zs[qi] = v;
        }
        __syncthreads();
    }

    // V sum: thread = (row group, two neighbouring output elements); a V row is read once per group as 8-byte
    // loads and serves the group's rows, so the loop is bound by its FMAs, not by loads
    constexpr int DV = 2;
    constexpr int TPG = HD / DV;             // threads per row group
    constexpr int NG = PF_THREADS / TPG;     // row groups
    constexpr int RPG = (QT + NG - 1) / NG;  // rows per group
    const int g = tid / TPG, d = (tid - g * TPG) * DV;
    float2 acc[RPG];
    int Lr[RPG];
#pragma unroll
    for (int k = 0; k < RPG; k++) {
        acc[k] = make_float2(0.0f, 0.0f);
        const int qi = g + k * NG;
        Lr[k] = qi < nq ? L0 + r0 + qi + 1 : 0;
    }
    const float* Vd = V + (long)hk * HD + d;
    const long vstride = (long)nkv * HD;
    // positions every row of the tile sees: four at a time, the probabilities as one 16-byte load
    const int Lcommon = (L0 + r0 + 1) & ~3;
    int t = 0;
    for (; t < Lcommon; t += 4) {
        const float2 v0 = *(const float2*)(Vd + (long)t * vstride), v1 = *(const float2*)(Vd + (long)(t + 1) * vstride);
        const float2 v2 = *(const float2*)(Vd + (long)(t + 2) * vstride), v3 = *(const float2*)(Vd + (long)(t + 3) * vstride);
#pragma unroll
        for (int k = 0; k < RPG; k++) {
            if (g + k * NG < QT) {
                const float4 pr = *(const float4*)(sc + (g + k * NG) * ld + t);
                acc[k].x = __fmaf_rn(pr.x, v0.x, acc[k].x); acc[k].y = __fmaf_rn(pr.x, v0.y, acc[k].y);
                acc[k].x = __fmaf_rn(pr.y, v1.x, acc[k].x); acc[k].y = __fmaf_rn(pr.y, v1.y, acc[k].y);
                acc[k].x = __fmaf_rn(pr.z, v2.x, acc[k].x); acc[k].y = __fmaf_rn(pr.z, v2.y, acc[k].y);
                acc[k].x = __fmaf_rn(pr.w, v3.x, acc[k].x); acc[k].y = __fmaf_rn(pr.w, v3.y, acc[k].y);
            }
        }
    }
    for (; t < Lmax; t++) {   // the causal edge: row by row
        const float2 v = *(const float2*)(Vd + (long)t * vstride);
#pragma unroll
        for (int k = 0; k < RPG; k++) {
            const int qi = g + k * NG;
            if (t < Lr[k]) {
                const float pr = sc[qi * ld + t];
                acc[k].x = __fmaf_rn(pr, v.x, acc[k].x);
                acc[k].y = __fmaf_rn(pr, v.y, acc[k].y);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < RPG; k++) {
        const int qi = g + k * NG;
        if (qi < nq) {
            const float z = zs[qi];
            *(float2*)(OUT + (long)(r0 + qi) * out_ld + (long)h * HD + d) = make_float2(__fdiv_rn(acc[k].x, z), __fdiv_rn(acc[k].y, z));
        }
    }
}

// ---- the same attention for 16 query rows per CTA (one CTA of 512 threads per SM).  A tile of K (then V) rows
// serves 16 query rows (half the L2 traffic of the 8-row kernel above), the next tile's asynchronous copy runs
// while this one is used (two buffers; the copies then cost ~1 k cycles per tile, barriers included, and nothing
// waits for them), and the first V tile is requested before the softmax.  What is left is shared-memory reads
// per fused multiply-add, so both folds are blocked in registers: a score thread owns two positions and four
// query rows (two K reads and four broadcast q reads per 32 FMAs), a V-sum thread two neighbouring output
// elements of two query rows.  Every (row, head) result is the one-token kernel's, bit for bit.
constexpr int PW_THREADS = 512;
constexpr int PW_QT = 16;
constexpr int PW_TILE = 128;             // positions per staged tile of K or V rows

template <int HD>
__global__ void __launch_bounds__(PW_THREADS, 1)
k_attn_prefill_wide(const float* __restrict__ Q, int q_ld, const float* __restrict__ K, const float* __restrict__ V,
                    const int* __restrict__ len_ptr, float* __restrict__ OUT, int out_ld, int nh, int nkv, float scale,
                    int nrows, int maxt, int* status) {
    constexpr int QT = PW_QT, KST = HD + 4;
    extern __shared__ __align__(16) float pf_smem[];
    float* qs = pf_smem;                     // [QT][HD]
    float* red = qs + QT * HD;               // [QT][64]
    float* zs = red + QT * 64;               // [QT] max, then Z
    float* tiles = zs + QT;                  // [2][PW_TILE][KST]
    float* sc = tiles + 2 * PW_TILE * KST;   // [QT][ld]
    const int ld = (maxt + 3) & ~3;
    const int tid = threadIdx.x;
    const int h = blockIdx.y;
    const int r0 = blockIdx.x * QT;
    const int Lafter = *len_ptr;
    if (Lafter < nrows || Lafter > maxt) {
        if (tid == 0) atomicOr(status, (int)LT_STATUS_BAD_LENGTH);
        return;
    }
    const int L0 = Lafter - nrows;
    const int nq = nrows - r0 < QT ? nrows - r0 : QT;   // query rows of this tile
    const int Lmax = L0 + r0 + nq;                      // positions the last row sees
    const int hk = h / (nh / nkv);
    const long rstride = (long)nkv * HD;                // floats between two positions of a cache

    auto copy_tile = [&](const float* base, int t0, float* dst) {     // positions [t0, t0 + PW_TILE) of head hk, one commit group
        const int nt = Lmax - t0 < PW_TILE ? Lmax - t0 : PW_TILE;
        const float* src = base + (long)hk * HD + (long)t0 * rstride;
        for (int e = tid; e < nt * (HD / 4); e += PW_THREADS) {
            const int r = e / (HD / 4), c = e - r * (HD / 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst + r * KST + c * 4)),
                         "l"(src + (long)r * rstride + c * 4) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    copy_tile(K, 0, tiles);
    for (int i = tid; i < QT * HD; i += PW_THREADS) {
        const int qi = i / HD, d = i - qi * HD;
        qs[i] = qi < nq ? Q[(long)(r0 + qi) * q_ld + (long)h * HD + d] : 0.0f;
    }

    // ---- scores: a thread owns two positions of the tile (p and p + 64) and four query rows: eight chains fed by two
    // 16-byte reads of K rows and four broadcast reads of q per four elements (half the shared-memory traffic per
    // fused multiply-add of one position per thread); 256 threads fold, all copy
    constexpr int QH = 4, PH = PW_TILE / 2;
    const int p = tid & (PH - 1), qh = tid / PH;
    for (int t0 = 0, buf = 0; t0 < Lmax; t0 += PW_TILE, buf ^= 1) {
        const bool more = t0 + PW_TILE < Lmax;
        if (more) copy_tile(K, t0 + PW_TILE, tiles + (buf ^ 1) * PW_TILE * KST);
        if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                    // tile t0 has landed (and, first pass, the q rows are stored)
        const int nt = Lmax - t0 < PW_TILE ? Lmax - t0 : PW_TILE;
        if (qh < QT / QH && p < nt) {
            const bool two = p + PH < nt;
            const float4* Ka = (const float4*)(tiles + buf * PW_TILE * KST + p * KST);
            const float4* Kb = (const float4*)(tiles + buf * PW_TILE * KST + (two ? p + PH : p) * KST);
            const float4* Qt = (const float4*)(qs + qh * QH * HD);
            float sa[QH], sb[QH];
#pragma unroll
            for (int qi = 0; qi < QH; qi++) { sa[qi] = 0.0f; sb[qi] = 0.0f; }
#pragma unroll 4
            for (int i = 0; i < HD / 4; i++) {
                const float4 ka = Ka[i], kb = Kb[i];
                float4 qq[QH];
#pragma unroll
                for (int qi = 0; qi < QH; qi++) qq[qi] = Qt[qi * (HD / 4) + i];
#pragma unroll
                for (int qi = 0; qi < QH; qi++) { sa[qi] = __fmaf_rn(qq[qi].x, ka.x, sa[qi]); sb[qi] = __fmaf_rn(qq[qi].x, kb.x, sb[qi]); }
#pragma unroll
                for (int qi = 0; qi < QH; qi++) { sa[qi] = __fmaf_rn(qq[qi].y, ka.y, sa[qi]); sb[qi] = __fmaf_rn(qq[qi].y, kb.y, sb[qi]); }
#pragma unroll
                for (int qi = 0; qi < QH; qi++) { sa[qi] = __fmaf_rn(qq[qi].z, ka.z, sa[qi]); sb[qi] = __fmaf_rn(qq[qi].z, kb.z, sb[qi]); }
#pragma unroll
                for (int qi = 0; qi < QH; qi++) { sa[qi] = __fmaf_rn(qq[qi].w, ka.w, sa[qi]); sb[qi] = __fmaf_rn(qq[qi].w, kb.w, sb[qi]); }
            }
#pragma unroll
            for (int qi = 0; qi < QH; qi++) {
                const int q = qh * QH + qi;
                const int ta = t0 + p, tb2 = ta + PH;
                sc[q * ld + ta] = ta < L0 + r0 + q + 1 ? __fmul_rn(sa[qi], scale) : -1e30f;
                if (two) sc[q * ld + tb2] = tb2 < L0 + r0 + q + 1 ? __fmul_rn(sb[qi], scale) : -1e30f;
            }
        }
        __syncthreads();                    // the tile may be overwritten, the scores are visible
    }
    // the first V tile travels while the softmax runs
    copy_tile(V, 0, tiles);

    // ---- softmax per query row on the frozen 64-lane layout: 8 rows at a time, 64 threads each
    const int grp = tid >> 6, l64 = tid & 63;
    for (int qb = 0; qb < QT; qb += PW_THREADS / 64) {
        const int qi = qb + grp;
        float* row = sc + qi * ld;
        float m = -1e30f;
        for (int t = l64; t < Lmax; t += 64) m = fmaxf(m, row[t]);
        red[qi * 64 + l64] = m;
        __syncthreads();
        if (l64 < 32) {
            float v = fmaxf(red[qi * 64 + l64], red[qi * 64 + l64 + 32]);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
            if (l64 == 0) zs[qi] = v;
        }
        __syncthreads();
        const float mx = zs[qi];
        float ls = 0.0f;
        for (int t = l64; t < Lmax; t += 64) {      // a lane sums what it has just written: no barrier in between
            const float e = __expf(__fsub_rn(row[t], mx));
            row[t] = e;
            ls = __fadd_rn(ls, e);
        }
        red[qi * 64 + l64] = ls;
        __syncthreads();
        if (l64 < 32) {
            float v = __fadd_rn(red[qi * 64 + l64], red[qi * 64 + l64 + 32]);
            v = warp_tree_sum(v);
            if (l64 == 0) zs[qi] = v;
        }
        __syncthreads();
    }

    // ---- V sum: thread = (group of two query rows, two neighbouring output elements); 256 threads fold, all copy
    constexpr int DV = 2, TPG = HD / DV, RPG = 2, NG = QT / RPG;
    static_assert(NG * TPG <= PW_THREADS, "row groups");
    const int g = tid / TPG, d = (tid - g * TPG) * DV;
    const bool folds = g < NG;
    float2 acc[RPG];
    int Lr[RPG];
#pragma unroll
    for (int k = 0; k < RPG; k++) {
        acc[k] = make_float2(0.0f, 0.0f);
        const int qi = g * RPG + k;
        Lr[k] = (folds && qi < nq) ? L0 + r0 + qi + 1 : 0;
    }
    // positions every row of the tile sees are folded four at a time, the probabilities as one 16-byte read
    const int Lcommon = (L0 + r0 + 1) & ~3;
    for (int t0 = 0, buf = 0; t0 < Lmax; t0 += PW_TILE, buf ^= 1) {
        const bool more = t0 + PW_TILE < Lmax;
        if (more) copy_tile(V, t0 + PW_TILE, tiles + (buf ^ 1) * PW_TILE * KST);
        if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (folds) {
            const float* vt = tiles + buf * PW_TILE * KST + d;
            const float* pr0 = sc + (g * RPG) * ld;
            const int te = more ? t0 + PW_TILE : Lmax;
            const int tv = (te < Lcommon ? te : Lcommon) & ~3;
            int t = t0;
            for (; t + 4 <= tv; t += 4) {
                float2 v[4];
                float4 pr[RPG];
#pragma unroll
                for (int j = 0; j < 4; j++) v[j] = *(const float2*)(vt + (t + j - t0) * KST);
#pragma unroll
                for (int k = 0; k < RPG; k++) pr[k] = *(const float4*)(pr0 + k * ld + t);
#pragma unroll
                for (int k = 0; k < RPG; k++) { acc[k].x = __fmaf_rn(pr[k].x, v[0].x, acc[k].x); acc[k].y = __fmaf_rn(pr[k].x, v[0].y, acc[k].y); }
#pragma unroll
                for (int k = 0; k < RPG; k++) { acc[k].x = __fmaf_rn(pr[k].y, v[1].x, acc[k].x); acc[k].y = __fmaf_rn(pr[k].y, v[1].y, acc[k].y); }
#pragma unroll
                for (int k = 0; k < RPG; k++) { acc[k].x = __fmaf_rn(pr[k].z, v[2].x, acc[k].x); acc[k].y = __fmaf_rn(pr[k].z, v[2].y, acc[k].y); }
#pragma unroll
                for (int k = 0; k < RPG; k++) { acc[k].x = __fmaf_rn(pr[k].w, v[3].x, acc[k].x); acc[k].y = __fmaf_rn(pr[k].w, v[3].y, acc[k].y); }
            }
            for (; t < te; t++) {   // the causal edge: row by row
                const float2 v = *(const float2*)(vt + (t - t0) * KST);
#pragma unroll
                for (int k = 0; k < RPG; k++) {
                    if (t < Lr[k]) {
                        const float pr = pr0[k * ld + t];
                        acc[k].x = __fmaf_rn(pr, v.x, acc[k].x);
                        acc[k].y = __fmaf_rn(pr, v.y, acc[k].y);
                    }
                }
            }
        }
        __syncthreads();                    // the tile may be overwritten
    }
#pragma unroll
    for (int k = 0; k < RPG; k++) {
        const int qi = g * RPG + k;
        if (folds && qi < nq) {
            const float z = zs[qi];
            *(float2*)(OUT + (long)(r0 + qi) * out_ld + (long)h * HD + d) = make_float2(__fdiv_rn(acc[k].x, z), __fdiv_rn(acc[k].y, z));
        }
    }
}

template <int HD>
static size_t attn_prefill_wide_smem(int maxt) {
    return ((size_t)PW_QT * HD + PW_QT * 64 + PW_QT + (size_t)2 * PW_TILE * (HD + 4) + (size_t)PW_QT * ((maxt + 3) & ~3)) * sizeof(float);
}

template <int HD>
static int launch_attn_prefill_wide(const float* Q, int q_ld, const float* K, const float* V, const int* len, float* OUT,
                                    int out_ld, int nh, int nkv, float scale, int nrows, int maxt, cudaStream_t s) {
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_attn_prefill: status word unavailable");
    const size_t smem = attn_prefill_wide_smem<HD>(maxt);
    static PerDeviceOnce attr_once;
    if (attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_attn_prefill_wide<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    }
    dim3 grid((nrows + PW_QT - 1) / PW_QT, nh);
    k_attn_prefill_wide<HD><<<grid, PW_THREADS, smem, s>>>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, st);
    return check_launch("lt_attn_prefill");
}

template <int HD, int QT>
static int launch_attn_prefill(const float* Q, int q_ld, const float* K, const float* V, const int* len, float* OUT,
                               int out_ld, int nh, int nkv, float scale, int nrows, int maxt, cudaStream_t s) {
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_attn_prefill: status word unavailable");
    const size_t smem = ((size_t)QT * HD + QT * 64 + ((QT + 3) & ~3) + (size_t)PF_KTILE * (HD + 4) +
                         (size_t)QT * ((maxt + 3) & ~3)) * sizeof(float);
    LT_REQUIRE(smem <= 200 * 1024, "lt_attn_prefill: maxt=%d needs %zu bytes of shared memory", maxt, smem);
    static PerDeviceOnce attr_once;
    if (attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_attn_prefill<HD, QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    dim3 grid((nrows + QT - 1) / QT, nh);
    k_attn_prefill<HD, QT><<<grid, PF_THREADS, smem, s>>>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt,
                                                         st);
    return check_launch("lt_attn_prefill");
}

template <int HD>
static int pick_attn_prefill(const float* Q, int q_ld, const float* K, const float* V, const int* len, float* OUT,
                             int out_ld, int nh, int nkv, float scale, int nrows, int maxt, cudaStream_t s) {
    // query rows per tile: 8 while three CTAs of score rows fit an SM (the V sum and the softmax are
    // chains of dependent operations, resident warps hide them), else 4; 16 only for short chunks (16 rows
    // with one CTA per SM was measured 6 % slower at 2048 positions)
    // 16 rows per CTA with double-buffered tiles where the score rows of 16 queries fit one SM beside them
    if (nrows >= 2 * PW_QT && attn_prefill_wide_smem<HD>(maxt) <= 227 * 1024 && aligned16(V))
        return launch_attn_prefill_wide<HD>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, s);
    const size_t per_row = (size_t)((maxt + 3) & ~3) + HD + 65;
    const size_t tile = (size_t)PF_KTILE * (HD + 4) * sizeof(float);
    if (16 * per_row * sizeof(float) + tile <= 72 * 1024)
        return launch_attn_prefill<HD, 16>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, s);
    if (8 * per_row * sizeof(float) + tile <= 110 * 1024 || 4 * per_row * sizeof(float) + tile > 200 * 1024 / 2)
        return launch_attn_prefill<HD, 8>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, s);
    return launch_attn_prefill<HD, 4>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, s);
}

}  // namespace lt

using namespace lt;

extern "C" int lt_embed_q8_rows(const int8_t* Wq, const uint16_t* Wd, const int* toks, float* out, int E, int V,
                                int nrows, void* stream) {
    LT_REQUIRE(Wq && Wd && toks && out, "lt_embed_q8_rows: null pointer");
    LT_REQUIRE(E > 0 && E % 32 == 0 && V > 0 && nrows > 0, "lt_embed_q8_rows: E=%d (multiple of 32) V=%d nrows=%d", E, V, nrows);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_embed_q8_rows: status word unavailable");
    const cudaError_t e = launch_chained(k_embed_q8_rows, dim3(nrows), dim3(256), 0, (cudaStream_t)stream, Wq,
                                         (const __half*)Wd, toks, out, E, V, nrows, st);
    return check_launch("lt_embed_q8_rows", 1, e);
}

extern "C" int lt_rope_rows(float* X, int ld, const int* pos0, int nrows, int n_head, int hd, float theta,
                            void* stream) {
    LT_REQUIRE(X && pos0, "lt_rope_rows: null pointer");
    LT_REQUIRE(nrows > 0 && n_head > 0 && hd > 0 && hd % 2 == 0 && ld >= n_head * hd,
               "lt_rope_rows: nrows=%d n_head=%d hd=%d ld=%d", nrows, n_head, hd, ld);
    const long total = (long)nrows * n_head * (hd / 2);
    k_rope_rows<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(X, ld, pos0, nrows, n_head, hd, theta);
    return check_launch("lt_rope_rows");
}

extern "C" int lt_append_kv_rows(float* kbase, const float* ksrc, float* vbase, const float* vsrc, int src_ld, int* len,
                                 int width, int max_seq, int nrows, int incr, void* stream) {
    LT_REQUIRE(kbase && ksrc && vbase && vsrc && len, "lt_append_kv_rows: null pointer");
    LT_REQUIRE(width > 0 && max_seq > 0 && nrows > 0 && src_ld >= width,
               "lt_append_kv_rows: width=%d max_seq=%d nrows=%d src_ld=%d", width, max_seq, nrows, src_ld);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_append_kv_rows: status word unavailable");
    const long total = (long)nrows * width;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    k_append_kv_rows<<<blocks, 256, 0, (cudaStream_t)stream>>>(kbase, ksrc, vbase, vsrc, src_ld, len, width, max_seq,
                                                              nrows, st);
    int n = 1;
    if (incr) {
        k_add_len<<<1, 32, 0, (cudaStream_t)stream>>>(len, nrows, max_seq);
        n = 2;
    }
    return check_launch("lt_append_kv_rows", n);
}

extern "C" int lt_silu_mul_quant_rows(const float* g, const float* u, int ld, int8_t* Xq, uint16_t* Xd, int K, int rows,
                                      void* stream) {
    LT_REQUIRE(g && u && Xq && Xd, "lt_silu_mul_quant_rows: null pointer");
    LT_REQUIRE(K > 0 && K % 32 == 0 && rows > 0 && ld >= K, "lt_silu_mul_quant_rows: K=%d rows=%d ld=%d", K, rows, ld);
    const long blocks32 = (long)rows * (K / 32);
    const cudaError_t e = launch_chained(k_silu_mul_quant_rows, dim3((unsigned)((blocks32 + 7) / 8)), dim3(256), 0,
                                         (cudaStream_t)stream, g, u, ld, Xq, (__half*)Xd, K, rows);
    return check_launch("lt_silu_mul_quant_rows", 1, e);
}

extern "C" int lt_attn_prefill(const float* Q, int q_ld, const float* K, const float* V, const int* len, float* OUT,
                               int out_ld, int hd, int nh, int nkv, float scale, int nrows, int maxt, void* stream) {
    LT_REQUIRE(Q && K && V && len && OUT, "lt_attn_prefill: null pointer");
    LT_REQUIRE(hd == 64 || hd == 128, "lt_attn_prefill: hd=%d (64 and 128 are built)", hd);
    LT_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "lt_attn_prefill: nh=%d must be a positive multiple of nkv=%d", nh, nkv);
    LT_REQUIRE(nrows > 0 && maxt >= nrows && maxt <= 12000, "lt_attn_prefill: nrows=%d maxt=%d (maxt in nrows..12000)", nrows, maxt);
    LT_REQUIRE(q_ld >= nh * hd && out_ld >= nh * hd && q_ld % 4 == 0, "lt_attn_prefill: q_ld=%d out_ld=%d", q_ld, out_ld);
    LT_REQUIRE(out_ld % 2 == 0 && (reinterpret_cast<uintptr_t>(OUT) & 7u) == 0 && (reinterpret_cast<uintptr_t>(V) & 7u) == 0,
               "lt_attn_prefill: OUT and V must be 8-byte aligned, out_ld even");
    LT_REQUIRE(aligned16(Q) && aligned16(K), "lt_attn_prefill: Q and K must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return pick_attn_prefill<64>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, s);
    return pick_attn_prefill<128>(Q, q_ld, K, V, len, OUT, out_ld, nh, nkv, scale, nrows, maxt, s);
}
