// Small streaming kernels of the decode step: activation quantiser, silu*mul (+quant),
// RMSNorm, RoPE, KV append, argmax, embedding gather.  All are latency-bound at decode
// sizes; they exist as stand-alone launches for the per-op interface and as building
// blocks whose arithmetic the fused kernels repeat verbatim.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

// ------------------------------------------------------------------ quantiser
// one warp per 32-block, lane = element
__global__ void __launch_bounds__(256) k_quant_q8(const float* __restrict__ X, int8_t* __restrict__ Xq,
                                                   __half* __restrict__ Xd, long nblocks) {
    long b = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (b >= nblocks) return;
    float v = X[b * 32 + lane];
    __half dh;
    int q = quant_lane(v, &dh);
    if (lane == 0) Xd[b] = dh;
    Xq[b * 32 + lane] = (int8_t)q;
}

__global__ void __launch_bounds__(256) k_silu_mul_quant(const float* __restrict__ g, const float* __restrict__ u,
                                                         int8_t* __restrict__ Xq, __half* __restrict__ Xd,
                                                         long nblocks) {
    long b = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (b >= nblocks) return;
    long i = b * 32 + lane;
    float v = silu_mul(g[i], u[i]);
    __half dh;
    int q = quant_lane(v, &dh);
    if (lane == 0) Xd[b] = dh;
    Xq[i] = (int8_t)q;
}

__global__ void k_silu_mul(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ y, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = silu_mul(g[i], u[i]);
}

__global__ void k_add(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, int n) {
    chain_release();
    chain_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fadd_rn(a[i], b[i]);
}

// ------------------------------------------------------------------ RMSNorm
// Sum of squares in the declared order: 256 lanes, lane t folds j = t, t+256, ... with a
// fused multiply-add, then the pairwise tree s = 128 .. 1 (p[t] += p[t+s]).  The three
// widest levels go through shared memory, the five narrowest are warp-0 shuffles, which
// add exactly the same pairs.
__device__ __forceinline__ float rms_sumsq_256(const float* __restrict__ xr, int N, float* sred) {
    int t = threadIdx.x;
    float local = 0.0f;
    for (int j = t; j < N; j += 256) {
        float v = xr[j];
        local = __fmaf_rn(v, v, local);
    }
    sred[t] = local;
    __syncthreads();
    if (t < 128) sred[t] = __fadd_rn(sred[t], sred[t + 128]);
    __syncthreads();
    if (t < 64) sred[t] = __fadd_rn(sred[t], sred[t + 64]);
    __syncthreads();
    if (t < 32) {
        float v = __fadd_rn(sred[t], sred[t + 32]);
        v = warp_tree_sum(v);
        if (t == 0) sred[0] = v;
    }
    __syncthreads();
    return sred[0];
}

__global__ void __launch_bounds__(256) k_rmsnorm(const float* __restrict__ x, const float* __restrict__ w,
                                                  float* __restrict__ y, int M, int N, float eps) {
    __shared__ float sred[256];
    int row = blockIdx.x;
    if (row >= M) return;
    const float* xr = x + (long)row * N;
    float* yr = y + (long)row * N;
    float ss = rms_sumsq_256(xr, N, sred);
    float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)N), eps));
    for (int j = threadIdx.x; j < N; j += 256) yr[j] = __fmul_rn(__fmul_rn(xr[j], inv), w[j]);
}

// RMSNorm and the activation quantiser in one launch (row per CTA): the normalised value goes
// straight into the warp-wide block quantiser (a warp holds one 32-block per round), the same two
// computations as k_rmsnorm followed by k_quant_q8.
__global__ void __launch_bounds__(256) k_rmsnorm_quant(const float* __restrict__ x, const float* __restrict__ w,
                                                        float* __restrict__ y, int8_t* __restrict__ Xq,
                                                        __half* __restrict__ Xd, int M, int N, float eps) {
    __shared__ float sred[256];
    int row = blockIdx.x;
    if (row >= M) return;
    const float* xr = x + (long)row * N;
    float ss = rms_sumsq_256(xr, N, sred);
    float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)N), eps));
    const int nb = N >> 5;
    for (int j0 = threadIdx.x; j0 < N; j0 += 256 * 8) {   // eight rounds of loads in flight, then their quantisers
        float xv[8], wv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int j = j0 + u * 256;
            xv[u] = j < N ? xr[j] : 0.0f;
            wv[u] = j < N ? w[j] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int j = j0 + u * 256;
            if (j < N) {      // N is a multiple of 32: a warp is in or out as a whole
                const float v = __fmul_rn(__fmul_rn(xv[u], inv), wv[u]);
                if (y != nullptr) y[(long)row * N + j] = v;
                __half dh;
                const int q = quant_lane(v, &dh);
                Xq[(long)row * N + j] = (int8_t)q;
                if ((threadIdx.x & 31) == 0) Xd[(long)row * nb + (j >> 5)] = dh;
            }
        }
    }
}

// ------------------------------------------------------------------ RoPE
__global__ void k_rope(float* __restrict__ X, const int* __restrict__ pos, int nrows, int n_head, int hd,
                       float theta) {
    int half = hd / 2;
    long total = (long)nrows * n_head * half;
    long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    int j = gid % half;
    long hr = gid / half;
    int head = hr % n_head;
    int row = hr / n_head;
    long base = (long)row * n_head * hd + (long)head * hd;
    float o1, o2;
    rope_pair(X[base + j], X[base + j + half], j, hd, theta, pos[row], o1, o2);
    X[base + j] = o1;
    X[base + j + half] = o2;
}

// ------------------------------------------------------------------ KV append
__global__ void k_append_kv(float* __restrict__ kbase, const float* __restrict__ ksrc, float* __restrict__ vbase,
                            const float* __restrict__ vsrc, int* len, int width, int max_seq, int incr,
                            int* status) {
    int L = *len;
    bool ok = (L >= 0 && L < max_seq);
    if (ok) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            long off = (long)L * width + i;
            kbase[off] = ksrc[i];
            vbase[off] = vsrc[i];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ok) atomicOr(status, (int)LT_STATUS_KV_OVERFLOW);
        else if (incr) *len = L + 1;
    }
}

__global__ void k_incr_len(int* len) {
    if (threadIdx.x == 0 && blockIdx.x == 0) *len += 1;
}

// ------------------------------------------------------------------ argmax
struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best block_best(Best m) {
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        Best o;
        o.v = __shfl_xor_sync(0xffffffffu, m.v, s);
        o.i = __shfl_xor_sync(0xffffffffu, m.i, s);
        m = better(m, o);
    }
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) { sv[warp] = m.v; si[warp] = m.i; }
    __syncthreads();
    if (warp == 0) {
        Best r;
        r.v = lane < nw ? sv[lane] : -3.4e38f;
        r.i = lane < nw ? si[lane] : 2147483647;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            Best o;
            o.v = __shfl_xor_sync(0xffffffffu, r.v, s);
            o.i = __shfl_xor_sync(0xffffffffu, r.i, s);
            r = better(r, o);
        }
        m = r;
    }
    return m;  // valid in warp 0
}

constexpr int ARGMAX_BLOCKS = 296;  // two per SM

__global__ void __launch_bounds__(256) k_argmax_s1(const float* __restrict__ x, int n, float* __restrict__ pval,
                                                    int* __restrict__ pidx) {
    chain_release();
    chain_wait();
    Best m;
    m.v = -3.4e38f;
    m.i = 2147483647;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        Best c;
        c.v = x[i];
        c.i = (int)i;
        m = better(m, c);
    }
    m = block_best(m);
    if (threadIdx.x == 0) { pval[blockIdx.x] = m.v; pidx[blockIdx.x] = m.i; }
}

__global__ void __launch_bounds__(256) k_argmax_s2(const float* __restrict__ pval, const int* __restrict__ pidx,
                                                    int nparts, int* __restrict__ out_idx) {
    chain_release();
    chain_wait();
    Best m;
    m.v = -3.4e38f;
    m.i = 2147483647;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) {
        Best c;
        c.v = pval[i];
        c.i = pidx[i];
        m = better(m, c);
    }
    m = block_best(m);
    if (threadIdx.x == 0) *out_idx = m.i;
}

// ------------------------------------------------------------------ embedding gather
__global__ void k_embed_q8(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd, const int* __restrict__ tok,
                           float* __restrict__ out, int E, int V, int* status) {
    int t = *tok;
    if (t < 0 || t >= V) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, (int)LT_STATUS_BAD_TOKEN);
        t = t < 0 ? 0 : V - 1;
    }
    int nb = E / 32;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < E; i += gridDim.x * blockDim.x)
        out[i] = __fmul_rn(__half2float(Wd[(long)t * nb + (i >> 5)]), (float)Wq[(long)t * E + i]);
}

// ------------------------------------------------------------------ token history
__global__ void k_token_record(const int* __restrict__ tok, int* __restrict__ history, int* __restrict__ step,
                               int capacity) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int s = *step;
        if (s >= 0 && s < capacity) history[s] = *tok;
        *step = s + 1;
    }
}

}  // namespace lt

using namespace lt;

// One token through a captured step, for a host loop that feeds every token back itself: the token id from
// page-locked memory -> the graph -> the chosen token back into page-locked memory -> one wait.  Four runtime
// calls behind one entry point: the caller's per-token cost is this call, not four trips through its binding.
extern "C" int lt_graph_replay_token(void* graph_exec, void* stream, const int* h_tok, int* d_tok, const int* d_out,
                                     int* h_out) {
    LT_REQUIRE(graph_exec && h_tok && d_tok && d_out && h_out, "lt_graph_replay_token: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    LT_CUDA(cudaMemcpyAsync(d_tok, h_tok, sizeof(int), cudaMemcpyHostToDevice, s));
    LT_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, s));
    LT_CUDA(cudaMemcpyAsync(h_out, d_out, sizeof(int), cudaMemcpyDeviceToHost, s));
    LT_CUDA(cudaStreamSynchronize(s));
    return LT_OK;
}

extern "C" int lt_token_record(const int* tok, int* history, int* step, int capacity, void* stream) {
    LT_REQUIRE(tok && history && step && capacity > 0, "lt_token_record: bad argument");
    k_token_record<<<1, 32, 0, (cudaStream_t)stream>>>(tok, history, step, capacity);
    return check_launch("lt_token_record");
}

extern "C" int lt_quant_q8(const float* X, int8_t* Xq, uint16_t* Xd, int K, int rows, void* stream) {
    LT_REQUIRE(X && Xq && Xd, "lt_quant_q8: null pointer");
    LT_REQUIRE(K > 0 && K % 32 == 0 && rows > 0, "lt_quant_q8: K=%d must be a positive multiple of 32, rows=%d > 0", K, rows);
    long nblocks = (long)rows * (K / 32);
    unsigned grid = (unsigned)((nblocks + 7) / 8);
    k_quant_q8<<<grid, 256, 0, (cudaStream_t)stream>>>(X, Xq, (__half*)Xd, nblocks);
    return check_launch("lt_quant_q8");
}

extern "C" int lt_silu_mul_quant(const float* g, const float* u, int8_t* Xq, uint16_t* Xd, int K, int rows,
                                 void* stream) {
    LT_REQUIRE(g && u && Xq && Xd, "lt_silu_mul_quant: null pointer");
    LT_REQUIRE(K > 0 && K % 32 == 0 && rows > 0, "lt_silu_mul_quant: K=%d must be a positive multiple of 32, rows=%d > 0", K, rows);
    long nblocks = (long)rows * (K / 32);
    unsigned grid = (unsigned)((nblocks + 7) / 8);
    k_silu_mul_quant<<<grid, 256, 0, (cudaStream_t)stream>>>(g, u, Xq, (__half*)Xd, nblocks);
    return check_launch("lt_silu_mul_quant");
}

extern "C" int lt_silu_mul(const float* g, const float* u, float* y, int n, void* stream) {
    LT_REQUIRE(g && u && y && n > 0, "lt_silu_mul: bad argument");
    k_silu_mul<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(g, u, y, n);
    return check_launch("lt_silu_mul");
}

extern "C" int lt_add(const float* a, const float* b, float* y, int n, void* stream) {
    LT_REQUIRE(a && b && y && n > 0, "lt_add: bad argument");
    const cudaError_t e = launch_chained(k_add, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, a, b, y, n);
    return check_launch("lt_add", 1, e);
}

extern "C" int lt_rmsnorm(const float* x, const float* w, float* y, int M, int N, float eps, void* stream) {
    LT_REQUIRE(x && w && y, "lt_rmsnorm: null pointer");
    LT_REQUIRE(M > 0 && N > 0, "lt_rmsnorm: M=%d N=%d must be positive", M, N);
    k_rmsnorm<<<M, 256, 0, (cudaStream_t)stream>>>(x, w, y, M, N, eps);
    return check_launch("lt_rmsnorm");
}

extern "C" int lt_rmsnorm_quant(const float* x, const float* w, float* y, int8_t* Xq, uint16_t* Xd, int M, int N,
                                float eps, void* stream) {
    LT_REQUIRE(x && w && Xq && Xd, "lt_rmsnorm_quant: null pointer");
    LT_REQUIRE(M > 0 && N > 0 && N % 32 == 0, "lt_rmsnorm_quant: M=%d, N=%d must be a positive multiple of 32", M, N);
    k_rmsnorm_quant<<<M, 256, 0, (cudaStream_t)stream>>>(x, w, y, Xq, (__half*)Xd, M, N, eps);
    return check_launch("lt_rmsnorm_quant");
}

extern "C" int lt_rope(float* X, const int* pos, int nrows, int n_head, int hd, float theta, void* stream) {
    LT_REQUIRE(X && pos, "lt_rope: null pointer");
    LT_REQUIRE(nrows > 0 && n_head > 0 && hd > 0 && hd % 2 == 0, "lt_rope: nrows=%d n_head=%d hd=%d (hd must be even)", nrows, n_head, hd);
    long total = (long)nrows * n_head * (hd / 2);
    k_rope<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(X, pos, nrows, n_head, hd, theta);
    return check_launch("lt_rope");
}

extern "C" int lt_append_kv(float* kbase, const float* ksrc, float* vbase, const float* vsrc, int* len, int width,
                            int max_seq, int incr, void* stream) {
    LT_REQUIRE(kbase && ksrc && vbase && vsrc && len, "lt_append_kv: null pointer");
    LT_REQUIRE(width > 0 && max_seq > 0, "lt_append_kv: width=%d max_seq=%d must be positive", width, max_seq);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_append_kv: status word unavailable");
    int threads = width >= 1024 ? 1024 : ((width + 31) / 32) * 32;
    k_append_kv<<<1, threads, 0, (cudaStream_t)stream>>>(kbase, ksrc, vbase, vsrc, len, width, max_seq, incr, st);
    return check_launch("lt_append_kv");
}

extern "C" int lt_incr_len(int* len, void* stream) {
    LT_REQUIRE(len, "lt_incr_len: null pointer");
    k_incr_len<<<1, 1, 0, (cudaStream_t)stream>>>(len);
    return check_launch("lt_incr_len");
}

extern "C" int lt_argmax_scratch_bytes(void) { return ARGMAX_BLOCKS * 8; }

extern "C" int lt_argmax(const float* x, int n, void* partials, int* out_idx, void* stream) {
    LT_REQUIRE(x && partials && out_idx, "lt_argmax: null pointer");
    LT_REQUIRE(n > 0, "lt_argmax: n=%d must be > 0 (an empty input has no index)", n);
    float* pval = (float*)partials;
    int* pidx = (int*)(pval + ARGMAX_BLOCKS);
    int blocks = (n + 255) / 256;
    if (blocks > ARGMAX_BLOCKS) blocks = ARGMAX_BLOCKS;
    cudaError_t e = launch_chained(k_argmax_s1, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, n, pval, pidx);
    if (e == cudaSuccess)
        e = launch_chained(k_argmax_s2, dim3(1), dim3(256), 0, (cudaStream_t)stream, pval, pidx, blocks, out_idx);
    return check_launch("lt_argmax", 2, e);
}

extern "C" int lt_embed_q8(const int8_t* Wq, const uint16_t* Wd, const int* tok, float* out, int E, int V,
                           void* stream) {
    LT_REQUIRE(Wq && Wd && tok && out, "lt_embed_q8: null pointer");
    LT_REQUIRE(E > 0 && E % 32 == 0 && V > 0, "lt_embed_q8: E=%d must be a positive multiple of 32, V=%d > 0", E, V);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_embed_q8: status word unavailable");
    k_embed_q8<<<(E + 255) / 256, 256, 0, (cudaStream_t)stream>>>(Wq, (const __half*)Wd, tok, out, E, V, st);
    return check_launch("lt_embed_q8");
}
