// One decode step (one token through all layers, final norm, LM head and argmax) as ONE
// persistent kernel: a CTA per SM, the weight stream decoupled from the dependency chain.
//
// Why: at batch 1 a 0.5B model streams ~525 MB per token (80 us at HBM speed) but the step
// is a chain of ~120 dependent phases; as separate launches each phase costs microseconds of
// launch latency during which HBM idles.  Weights do not depend on activations, so here a
// producer warp per CTA runs ahead of the chain and keeps a ring of shared-memory stages
// filled with the weight rows this CTA will need next (bulk async copies, global -> shared,
// completion on an mbarrier; no multicast), across phase and layer boundaries.  The consumer
// warps wait at a grid barrier only for the small activation vectors.
//
// Arithmetic is the per-op kernels' arithmetic, repeated verbatim (same device functions):
//   P1  x -> rmsnorm(attn_norm) -> quant -> [q|k|v] GEMV + bias
//   P2  rope(q,k at *len) -> append k,v at *len -> masked attention (one CTA per query head)
//   P3  quant(att) -> o_proj GEMV + x -> x1            (*len += 1)
//   P4  rmsnorm(ffn_norm)(x1) -> quant -> [gate|up] GEMV
//   P5  silu(gate)*up -> quant -> down GEMV + x1 -> x
//   LM  rmsnorm(out_norm)(x) -> quant -> LM-head GEMV -> logits, argmax
// so the step is bit-identical to the chain of per-op launches.
//
// Every wait (grid barrier, mbarrier) is bounded by a clock limit; on expiry the kernel sets
// LT_STATUS_WAIT_TIMEOUT, stops waiting anywhere, drains its copies and returns.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

constexpr int DEC_THREADS = 512;
constexpr int DEC_CWARPS = 15;                  // consumer warps; warp 15 is the producer
constexpr int DEC_CTHREADS = DEC_CWARPS * 32;
constexpr int DEC_STAGE_BYTES = 32768;          // weight rows per stage (quants + scales)
constexpr int DEC_STAGE_STRIDE = DEC_STAGE_BYTES + 128;
constexpr long long DEC_WAIT_CLOCKS = 2000000000LL;   // ~1 s at 2 GHz

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bulk async copy global -> this CTA's shared memory, completion counted on an mbarrier
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DEC_CTHREADS) : "memory"); }

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct Shared {
    unsigned long long full[8];
    unsigned long long empty[8];
    float sred[256];
    float red64[64];
    float best_v[DEC_CWARPS];
    int best_i[DEC_CWARPS];
    volatile int abort_flag;
    int pos;
};

// bounded wait on an mbarrier phase; returns false (and raises the abort flag) on expiry
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, Shared* S, int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (S->abort_flag) return false;
        if ((++spins & 1023u) == 0 && (*(volatile int*)status & (int)LT_STATUS_WAIT_TIMEOUT)) {
            S->abort_flag = 1;      // another CTA gave up: do not wait for it
            return false;
        }
        if (clock64() - t0 > DEC_WAIT_CLOCKS) {
            S->abort_flag = 1;
            atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
            return false;
        }
    }
    return true;
}

// Grid barrier for the consumer warps of all CTAs.  `epoch` counts barriers of this launch;
// the counter is monotonic within a launch and reset by the last CTA to leave the kernel.
__device__ __forceinline__ void grid_sync(unsigned* ctr, unsigned& epoch, unsigned nctas, Shared* S, int* status) {
    consumer_sync();
    epoch += 1;
    if (threadIdx.x == 0 && !S->abort_flag) {
        __threadfence();
        atomicAdd(ctr, 1u);
        const unsigned target = epoch * nctas;
        long long t0 = clock64();
        unsigned spins = 0;
        while (ld_acquire_u32(ctr) < target) {
            if ((++spins & 255u) == 0 && (*(volatile int*)status & (int)LT_STATUS_WAIT_TIMEOUT)) {
                S->abort_flag = 1;  // another CTA gave up: do not wait for it
                break;
            }
            if (clock64() - t0 > DEC_WAIT_CLOCKS) {
                S->abort_flag = 1;
                atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
                break;
            }
        }
        __threadfence();
    }
    consumer_sync();
}

// optional phase-boundary time stamps (thread 0 of CTA 0 and of the last CTA)
struct Tracer {
    long long* buf;
    int n;
    __device__ __forceinline__ void init(const lt_decode_desc& P) {
        buf = nullptr; n = 0;
        if (P.trace != nullptr && threadIdx.x == 0) {
            if (blockIdx.x == 0) buf = P.trace;
            else if (blockIdx.x == gridDim.x - 1) buf = P.trace + (16 * P.n_layers + 8);
        }
    }
    __device__ __forceinline__ void stamp() {
        if (buf != nullptr) buf[n++] = clock64();
    }
};

struct GemvDesc {
    const int8_t* Wq;
    const __half* Wd;
    int M, K;
};

__device__ __forceinline__ GemvDesc phase_desc(const lt_decode_desc& P, int idx) {
    GemvDesc d;
    const int L = P.n_layers;
    const int nq = P.nh * P.hd, nk = P.nkv * P.hd;
    if (idx >= 4 * L) {
        d.Wq = P.lm_q; d.Wd = (const __half*)P.lm_d; d.M = P.V; d.K = P.E;
        return d;
    }
    const lt_decode_layer* ly = P.layers + (idx >> 2);
    switch (idx & 3) {
        case 0: d.Wq = ly->qkv_q; d.Wd = (const __half*)ly->qkv_d; d.M = nq + 2 * nk; d.K = P.E; break;
        case 1: d.Wq = ly->o_q; d.Wd = (const __half*)ly->o_d; d.M = P.E; d.K = nq; break;
        case 2: d.Wq = ly->gu_q; d.Wd = (const __half*)ly->gu_d; d.M = 2 * P.F; d.K = P.E; break;
        default: d.Wq = ly->down_q; d.Wd = (const __half*)ly->down_d; d.M = P.E; d.K = P.F; break;
    }
    return d;
}

__device__ __forceinline__ void cta_rows(int M, int& r0, int& r1) {
    r0 = (int)(((long long)M * blockIdx.x) / gridDim.x);
    r1 = (int)(((long long)M * (blockIdx.x + 1)) / gridDim.x);
}
__device__ __forceinline__ int rows_per_chunk(int K) {
    int rc = DEC_STAGE_BYTES / (K + (K >> 4));
    return rc < 1 ? 1 : rc;
}

// ---------------------------------------------------------------- producer
__device__ void producer_loop(const lt_decode_desc& P, unsigned char* ring, int nstages, Shared* S) {
    unsigned cnt = 0;
    const int nphases = 4 * P.n_layers + 1;
    for (int idx = 0; idx < nphases; idx++) {
        GemvDesc d = phase_desc(P, idx);
        int r0, r1;
        cta_rows(d.M, r0, r1);
        const int nb = d.K >> 5;
        const int RC = rows_per_chunk(d.K);
        for (int r = r0; r < r1; r += RC, cnt++) {
            const int n = (r1 - r < RC) ? (r1 - r) : RC;
            const unsigned stage = cnt % nstages;
            if (cnt >= (unsigned)nstages) {
                if (!mbar_wait(&S->empty[stage], ((cnt / nstages) - 1) & 1, S, P.status)) return;
            }
            unsigned char* dst = ring + (size_t)stage * DEC_STAGE_STRIDE;
            const unsigned qbytes = (unsigned)n * d.K;
            const size_t d0 = ((size_t)r * nb * 2) & ~(size_t)15;
            const size_t d1 = (((size_t)(r + n) * nb * 2) + 15) & ~(size_t)15;
            const unsigned dbytes = (unsigned)(d1 - d0);
            mbar_expect_tx(&S->full[stage], qbytes + dbytes);
            bulk_g2s(dst, d.Wq + (size_t)r * d.K, qbytes, &S->full[stage]);
            bulk_g2s(dst + qbytes, (const unsigned char*)d.Wd + d0, dbytes, &S->full[stage]);
        }
    }
}

// ---------------------------------------------------------------- consumer: GEMV phase
enum { EPI_BIAS = 0, EPI_RESID = 1, EPI_NONE = 2, EPI_LOGITS = 3 };

template <int EPI>
__device__ __forceinline__ void consume_gemv(const lt_decode_desc& P, const GemvDesc& d, unsigned char* ring,
                                             int nstages, unsigned& cnt, Shared* S, const int8_t* sXq,
                                             const __half* sXd, const float* add, float* out, float& bestv,
                                             int& besti) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int r0, r1;
    cta_rows(d.M, r0, r1);
    const int K = d.K, nb = K >> 5;
    const int RC = rows_per_chunk(K);
    for (int r = r0; r < r1; r += RC, cnt++) {
        const int n = (r1 - r < RC) ? (r1 - r) : RC;
        const unsigned stage = cnt % nstages;
        const bool ok = mbar_wait(&S->full[stage], (cnt / nstages) & 1, S, P.status);
        const unsigned char* base = ring + (size_t)stage * DEC_STAGE_STRIDE;
        const size_t doff = ((size_t)r * nb * 2) & 15;
        const __half* wdbase = (const __half*)(base + (size_t)n * K + doff);
        if (ok) {
            for (int i = warp; i < n; i += DEC_CWARPS) {
                const unsigned char* wq = base + (size_t)i * K;
                const __half* wd = wdbase + (size_t)i * nb;
                float acc = 0.0f;
                for (int b = lane; b < nb; b += 32) {
                    const int4* wp = (const int4*)(wq + b * 32);
                    const int4* xp = (const int4*)(sXq + b * 32);
                    int4 w0 = wp[0], w1 = wp[1];
                    int4 x0 = xp[0], x1 = xp[1];
                    acc = q8_accum(__half2float(wd[b]), __half2float(sXd[b]), block_dot(w0, w1, x0, x1), acc);
                }
                float v = warp_tree_sum(acc);
                if (lane == 0) {
                    const int row = r + i;
                    if (EPI == EPI_BIAS) {
                        if (add != nullptr) v = __fadd_rn(v, __ldg(add + row));
                    } else if (EPI == EPI_RESID) {
                        v = __fadd_rn(v, __ldcg(add + row));
                    }
                    out[row] = v;
                    if (EPI == EPI_LOGITS) {
                        if (v > bestv || (v == bestv && row < besti)) { bestv = v; besti = row; }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&S->empty[stage]);
    }
}

// ---------------------------------------------------------------- consumer: prologues
// sum of squares in the declared 256-lane order over a vector staged in shared memory
__device__ __forceinline__ float cta_rms_sumsq(const float* sF, int N, Shared* S) {
    const int t = threadIdx.x;
    if (t < 256) {
        float local = 0.0f;
        for (int j = t; j < N; j += 256) local = __fmaf_rn(sF[j], sF[j], local);
        S->sred[t] = local;
    }
    consumer_sync();
    if (t < 128) S->sred[t] = __fadd_rn(S->sred[t], S->sred[t + 128]);
    consumer_sync();
    if (t < 64) S->sred[t] = __fadd_rn(S->sred[t], S->sred[t + 64]);
    consumer_sync();
    if (t < 32) {
        float v = __fadd_rn(S->sred[t], S->sred[t + 32]);
        v = warp_tree_sum(v);
        if (t == 0) S->sred[0] = v;
    }
    consumer_sync();
    return S->sred[0];
}

// sF holds x; writes quant(rmsnorm(x) * w) into sXq / sXd
__device__ __forceinline__ void prologue_rms_quant(const float* sF, const float* __restrict__ normw, int N, float eps,
                                                   int8_t* sXq, __half* sXd, Shared* S) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float ss = cta_rms_sumsq(sF, N, S);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)N), eps));
    for (int b = warp; b < (N >> 5); b += DEC_CWARPS) {
        const int j = b * 32 + lane;
        float v = __fmul_rn(__fmul_rn(sF[j], inv), __ldg(normw + j));
        __half dh;
        int q = quant_lane(v, &dh);
        sXq[j] = (int8_t)q;
        if (lane == 0) sXd[b] = dh;
    }
    consumer_sync();
}

__device__ __forceinline__ void stage_vector(const float* __restrict__ g, float* sF, int N) {
    for (int j = threadIdx.x; j < N; j += DEC_CTHREADS) sF[j] = __ldcg(g + j);
    consumer_sync();
}

__device__ __forceinline__ void prologue_quant(const float* __restrict__ g, int N, int8_t* sXq, __half* sXd) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int b = warp; b < (N >> 5); b += DEC_CWARPS) {
        const int j = b * 32 + lane;
        __half dh;
        int q = quant_lane(__ldcg(g + j), &dh);
        sXq[j] = (int8_t)q;
        if (lane == 0) sXd[b] = dh;
    }
    consumer_sync();
}

__device__ __forceinline__ void prologue_silu_quant(const float* __restrict__ g, const float* __restrict__ u, int N,
                                                    int8_t* sXq, __half* sXd) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int b = warp; b < (N >> 5); b += DEC_CWARPS) {
        const int j = b * 32 + lane;
        float v = silu_mul(__ldcg(g + j), __ldcg(u + j));
        __half dh;
        int q = quant_lane(v, &dh);
        sXq[j] = (int8_t)q;
        if (lane == 0) sXd[b] = dh;
    }
    consumer_sync();
}

// ---------------------------------------------------------------- consumer: attention phase
// One CTA per query head.  sAtt: [maxt] probabilities, then hd (q) + hd (new k) + hd (new v)
// floats, then the V staging area of vcap rows.
__device__ void attention_phase(const lt_decode_desc& P, const lt_decode_layer* ly, float* sAtt, int vcap,
                                Shared* S) {
    const int h = blockIdx.x;
    const int tid = threadIdx.x;
    const int hd = P.hd, nh = P.nh, nkv = P.nkv, maxt = P.max_seq;
    const int nq = nh * hd, nk = nkv * hd;
    const int rep = nh / nkv, hk = h / rep;
    float* sh = sAtt;
    float* sQ = sAtt + maxt;
    float* sKn = sQ + hd;
    float* sVn = sKn + hd;
    float* sV = sVn + hd;

    int pos = __ldcg(ly->len);
    const bool room = (pos >= 0 && pos < maxt);
    if (!room) {
        if (tid == 0) atomicOr(P.status, (int)LT_STATUS_KV_OVERFLOW);
        pos = pos < 0 ? 0 : maxt;
    }
    const int L = room ? pos + 1 : pos;      // attention length after the append
    // rope of this head's q and of the kv head's k at position pos; v is copied
    const int half = hd >> 1;
    if (tid < half) {
        float o1, o2;
        rope_pair(__ldcg(P.qkv + h * hd + tid), __ldcg(P.qkv + h * hd + tid + half), tid, hd, P.theta, pos, o1, o2);
        sQ[tid] = o1; sQ[tid + half] = o2;
    } else if (tid >= 64 && tid < 64 + half) {
        const int j = tid - 64;
        float o1, o2;
        rope_pair(__ldcg(P.qkv + nq + hk * hd + j), __ldcg(P.qkv + nq + hk * hd + j + half), j, hd, P.theta, pos, o1, o2);
        sKn[j] = o1; sKn[j + half] = o2;
    } else if (tid >= 256 && tid < 256 + hd) {
        sVn[tid - 256] = __ldcg(P.qkv + nq + nk + hk * hd + (tid - 256));
    }
    consumer_sync();
    if (room && (h % rep) == 0 && tid < hd) {
        ly->kcache[((size_t)pos * nkv + hk) * hd + tid] = sKn[tid];
        ly->vcache[((size_t)pos * nkv + hk) * hd + tid] = sVn[tid];
    }
    // scores
    for (int t = tid; t < maxt; t += DEC_CTHREADS) {
        float v = -1e30f;
        if (t < L) {
            const float* Kt = (room && t == pos) ? sKn : ly->kcache + ((size_t)t * nkv + hk) * hd;
            const float4* K4 = (const float4*)Kt;
            const float4* q4 = (const float4*)sQ;
            float s = 0.0f;
            for (int i = 0; i < (hd >> 2); i++) {
                float4 kk = K4[i];
                float4 qq = q4[i];
                s = __fmaf_rn(qq.x, kk.x, s);
                s = __fmaf_rn(qq.y, kk.y, s);
                s = __fmaf_rn(qq.z, kk.z, s);
                s = __fmaf_rn(qq.w, kk.w, s);
            }
            v = __fmul_rn(s, P.scale);
        }
        sh[t] = v;
    }
    // stage V rows (independent of the scores) while the scores settle
    const bool staged = (L <= vcap);
    if (staged) {
        const int hq = hd >> 2;
        for (int e = tid; e < L * hq; e += DEC_CTHREADS) {
            const int t = e / hq, c = e - t * hq;
            const float4* src = (room && t == pos) ? (const float4*)sVn : (const float4*)(ly->vcache + ((size_t)t * nkv + hk) * hd);
            ((float4*)sV)[(size_t)t * hq + c] = src[c];
        }
    }
    consumer_sync();
    // max over the frozen 64-lane layout (exact in any order)
    if (tid < 64) {
        float m = -1e30f;
        for (int t = tid; t < maxt; t += 64) m = fmaxf(m, sh[t]);
        S->red64[tid] = m;
    }
    consumer_sync();
    if (tid < 32) {
        float v = fmaxf(S->red64[tid], S->red64[tid + 32]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
        if (tid == 0) S->red64[0] = v;
    }
    consumer_sync();
    const float mx = S->red64[0];
    consumer_sync();
    for (int t = tid; t < maxt; t += DEC_CTHREADS) sh[t] = __expf(__fsub_rn(sh[t], mx));
    consumer_sync();
    if (tid < 64) {
        float ls = 0.0f;
        for (int t = tid; t < maxt; t += 64) ls = __fadd_rn(ls, sh[t]);
        S->red64[tid] = ls;
    }
    consumer_sync();
    if (tid < 32) {
        float v = __fadd_rn(S->red64[tid], S->red64[tid + 32]);
        v = warp_tree_sum(v);
        if (tid == 0) S->red64[0] = v;
    }
    consumer_sync();
    const float Z = S->red64[0];
    if (tid < hd) {
        float acc = 0.0f;
        if (staged) {
            for (int t = 0; t < L; t++) acc = __fmaf_rn(sh[t], sV[(size_t)t * hd + tid], acc);
        } else {
            const float* Vd = ly->vcache + (size_t)hk * hd + tid;
            const size_t stride = (size_t)nkv * hd;
            const int Lc = room ? pos : L;      // rows that live in the cache
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
        P.att[h * hd + tid] = __fdiv_rn(acc, Z);
    }
    consumer_sync();
}

// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(DEC_THREADS, 1) k_decode_step(const lt_decode_desc P, int nstages, int kmax,
                                                                int fmax, int vcap) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;
    size_t off = (size_t)nstages * DEC_STAGE_STRIDE;
    Shared* S = (Shared*)(smem + off);
    off += (sizeof(Shared) + 127) & ~(size_t)127;
    int8_t* sXq = (int8_t*)(smem + off);
    off += ((size_t)kmax + 127) & ~(size_t)127;
    __half* sXd = (__half*)(smem + off);
    off += ((size_t)(kmax >> 5) * 2 + 127) & ~(size_t)127;
    float* sF = (float*)(smem + off);
    off += ((size_t)fmax * 4 + 127) & ~(size_t)127;
    float* sAtt = (float*)(smem + off);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < nstages; s++) {
            mbar_init(&S->full[s], 1);
            mbar_init(&S->empty[s], DEC_CWARPS);
        }
        S->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == DEC_CWARPS) {       // producer warp: one lane streams weights for the whole step
        if ((tid & 31) == 0) producer_loop(P, ring, nstages, S);
        return;
    }

    // ------------------------------------------------------------ consumers
    const unsigned nctas = gridDim.x;
    unsigned epoch = 0, cnt = 0;
    const int E = P.E, F = P.F, nq = P.nh * P.hd;
    float bestv = -3.4e38f;
    int besti = 2147483647;
    float dummy_v = 0.0f;
    int dummy_i = 0;
    Tracer tr;
    tr.init(P);
    tr.stamp();

    // x for layer 0: gathered from the Q8_0 table by the device token, or preloaded by the host
    if (P.tok != nullptr) {
        int t = *P.tok;
        if (t < 0 || t >= P.V) {
            if (tid == 0 && blockIdx.x == 0) atomicOr(P.status, (int)LT_STATUS_BAD_TOKEN);
            t = t < 0 ? 0 : P.V - 1;
        }
        const int nbE = E >> 5;
        for (int j = tid; j < E; j += DEC_CTHREADS) {
            float v = __fmul_rn(__half2float(((const __half*)P.emb_d)[(size_t)t * nbE + (j >> 5)]),
                                (float)P.emb_q[(size_t)t * E + j]);
            sF[j] = v;
            if (blockIdx.x == 0) P.x[j] = v;
        }
        consumer_sync();
    } else {
        stage_vector(P.x, sF, E);
    }

    for (int il = 0; il < P.n_layers; il++) {
        const lt_decode_layer* ly = P.layers + il;
        // P1: rmsnorm + quant -> q|k|v
        if (il > 0) stage_vector(P.x, sF, E);
        prologue_rms_quant(sF, ly->attn_norm, E, P.eps, sXq, sXd, S);
        tr.stamp();
        consume_gemv<EPI_BIAS>(P, phase_desc(P, 4 * il + 0), ring, nstages, cnt, S, sXq, sXd, ly->qkv_bias, P.qkv,
                               dummy_v, dummy_i);
        tr.stamp();
        grid_sync(P.sync, epoch, nctas, S, P.status);
        tr.stamp();
        // P2: rope + append + attention
        if ((int)blockIdx.x < P.nh) attention_phase(P, ly, sAtt, vcap, S);
        tr.stamp();
        grid_sync(P.sync, epoch, nctas, S, P.status);
        tr.stamp();
        // P3: o_proj + residual; the cache length advances now that every head has read it
        if (blockIdx.x == 0 && tid == 0) {
            int p = __ldcg(ly->len);
            if (p >= 0 && p < P.max_seq) *ly->len = p + 1;
        }
        prologue_quant(P.att, nq, sXq, sXd);
        tr.stamp();
        consume_gemv<EPI_RESID>(P, phase_desc(P, 4 * il + 1), ring, nstages, cnt, S, sXq, sXd, P.x, P.x1, dummy_v,
                                dummy_i);
        tr.stamp();
        grid_sync(P.sync, epoch, nctas, S, P.status);
        tr.stamp();
        // P4: rmsnorm + quant -> gate|up
        stage_vector(P.x1, sF, E);
        prologue_rms_quant(sF, ly->ffn_norm, E, P.eps, sXq, sXd, S);
        tr.stamp();
        consume_gemv<EPI_NONE>(P, phase_desc(P, 4 * il + 2), ring, nstages, cnt, S, sXq, sXd, nullptr, P.gu, dummy_v,
                               dummy_i);
        tr.stamp();
        grid_sync(P.sync, epoch, nctas, S, P.status);
        tr.stamp();
        // P5: silu*up + quant -> down + residual
        prologue_silu_quant(P.gu, P.gu + F, F, sXq, sXd);
        tr.stamp();
        consume_gemv<EPI_RESID>(P, phase_desc(P, 4 * il + 3), ring, nstages, cnt, S, sXq, sXd, P.x1, P.x, dummy_v,
                                dummy_i);
        tr.stamp();
        grid_sync(P.sync, epoch, nctas, S, P.status);
        tr.stamp();
    }
    // LM head + argmax
    stage_vector(P.x, sF, E);
    prologue_rms_quant(sF, P.out_norm, E, P.eps, sXq, sXd, S);
    tr.stamp();
    consume_gemv<EPI_LOGITS>(P, phase_desc(P, 4 * P.n_layers), ring, nstages, cnt, S, sXq, sXd, nullptr, P.logits,
                             bestv, besti);
    tr.stamp();
    if ((tid & 31) == 0) { S->best_v[warp] = bestv; S->best_i[warp] = besti; }
    consumer_sync();
    if (tid == 0) {
        float bv = S->best_v[0];
        int bi = S->best_i[0];
        for (int w = 1; w < DEC_CWARPS; w++) {
            float v = S->best_v[w];
            int i = S->best_i[w];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        P.part_val[blockIdx.x] = bv;
        P.part_idx[blockIdx.x] = bi;
    }
    grid_sync(P.sync, epoch, nctas, S, P.status);
    if (blockIdx.x == 0 && warp == 0) {
        const int lane = tid & 31;
        float bv = -3.4e38f;
        int bi = 2147483647;
        for (int c = lane; c < (int)nctas; c += 32) {
            float v = __ldcg(P.part_val + c);
            int i = __ldcg(P.part_idx + c);
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            int oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            *P.out_tok = bi;
            if (P.tok != nullptr) *P.tok = bi;
            if (P.history != nullptr) {
                int s = *P.step;
                if (s >= 0 && s < P.hist_cap) P.history[s] = bi;
                *P.step = s + 1;
            }
        }
    }
    // the last CTA to get here resets the barrier counters for the next launch
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(P.sync + 1, 1u) == nctas - 1) {
            P.sync[0] = 0;
            P.sync[1] = 0;
            __threadfence();
        }
    }
}

struct DecodeGeometry {
    int nstages, kmax, fmax, vcap;
    size_t smem;
    int ctas;
};

static int decode_geometry(const lt_decode_desc* d, DecodeGeometry* g) {
    int dev = 0, sms = 0, smem_max = 0;
    LT_CUDA(cudaGetDevice(&dev));
    LT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    LT_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const int nq = d->nh * d->hd;
    g->kmax = d->E > d->F ? d->E : d->F;
    if (nq > g->kmax) g->kmax = nq;
    g->fmax = d->E > nq ? d->E : nq;
    size_t fixed = ((sizeof(Shared) + 127) & ~(size_t)127) + (((size_t)g->kmax + 127) & ~(size_t)127) +
                   (((size_t)(g->kmax >> 5) * 2 + 127) & ~(size_t)127) + (((size_t)g->fmax * 4 + 127) & ~(size_t)127);
    size_t att_fixed = ((size_t)d->max_seq + 3 * d->hd) * 4;
    // at least 3 stages for the ring; the rest goes to V staging (up to max_seq rows)
    size_t avail = (size_t)smem_max - 1024;
    if (fixed + att_fixed + 3 * (size_t)DEC_STAGE_STRIDE > avail) {
        set_error("lt_decode_step: model dimensions need more shared memory than one SM has");
        return LT_ERR_UNSUPPORTED;
    }
    size_t left = avail - fixed - att_fixed;
    size_t vrow = (size_t)d->hd * 4;
    size_t vwant = (size_t)d->max_seq * vrow;
    int nst = 4;
    if (left >= 4 * (size_t)DEC_STAGE_STRIDE + vwant) {
        g->vcap = d->max_seq;
        nst = (int)((left - vwant) / DEC_STAGE_STRIDE);
    } else {
        nst = (int)(left / DEC_STAGE_STRIDE);
        if (nst > 4) nst = 4;
        g->vcap = (int)((left - (size_t)nst * DEC_STAGE_STRIDE) / vrow);
    }
    if (nst > 8) nst = 8;
    g->nstages = nst;
    g->smem = (size_t)nst * DEC_STAGE_STRIDE + fixed + att_fixed + (size_t)g->vcap * vrow + 128;
    g->ctas = sms;
    return LT_OK;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_decode_step(const lt_decode_desc* d, void* stream) {
    LT_REQUIRE(d != nullptr, "lt_decode_step: null descriptor");
    LT_REQUIRE(d->layers && d->out_norm && d->lm_q && d->lm_d && d->x && d->x1 && d->qkv && d->att && d->gu &&
                   d->logits && d->out_tok && d->sync && d->part_val && d->part_idx,
               "lt_decode_step: null pointer in descriptor");
    LT_REQUIRE(d->tok == nullptr || (d->emb_q && d->emb_d), "lt_decode_step: device token loop needs the embedding table");
    LT_REQUIRE(d->n_layers > 0 && d->E > 0 && d->F > 0 && d->V > 0 && d->max_seq > 0, "lt_decode_step: bad dimensions");
    LT_REQUIRE(d->E % 32 == 0 && d->F % 32 == 0 && (d->nh * d->hd) % 32 == 0, "lt_decode_step: E, F and nh*hd must be multiples of 32");
    LT_REQUIRE(d->hd % 4 == 0 && d->hd <= 128, "lt_decode_step: hd=%d must be a multiple of 4, at most 128", d->hd);
    LT_REQUIRE(d->nkv > 0 && d->nh % d->nkv == 0, "lt_decode_step: nh must be a multiple of nkv");
    LT_REQUIRE(d->max_seq % 4 == 0, "lt_decode_step: max_seq=%d must be a multiple of 4", d->max_seq);
    const int nq = d->nh * d->hd, nk = d->nkv * d->hd;
    // the scale rows of each matrix are fetched in 16-byte windows: the array must end on one
    const long long ms[5] = {(long long)(nq + 2 * nk) * (d->E / 32), (long long)d->E * (nq / 32),
                             (long long)2 * d->F * (d->E / 32), (long long)d->E * (d->F / 32),
                             (long long)d->V * (d->E / 32)};
    for (int i = 0; i < 5; i++)
        LT_REQUIRE(ms[i] % 8 == 0, "lt_decode_step: a weight matrix has M*K/32 = %lld scales, not a multiple of 8", ms[i]);
    DecodeGeometry g;
    int rc = decode_geometry(d, &g);
    if (rc != LT_OK) return rc;
    LT_REQUIRE(d->nh <= g.ctas, "lt_decode_step: more query heads (%d) than SMs (%d)", d->nh, g.ctas);
    LT_CUDA(cudaFuncSetAttribute(k_decode_step, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
    lt_decode_desc P = *d;
    if (P.status == nullptr) P.status = device_status_ptr();
    LT_REQUIRE(P.status != nullptr, "lt_decode_step: status word unavailable");
    int nstages = g.nstages, kmax = g.kmax, fmax = g.fmax, vcap = g.vcap;
    void* args[] = {&P, &nstages, &kmax, &fmax, &vcap};
    // cooperative launch: all CTAs are resident together, which the grid barrier relies on
    LT_CUDA(cudaLaunchCooperativeKernel((const void*)k_decode_step, dim3(g.ctas), dim3(DEC_THREADS), args, g.smem,
                                        (cudaStream_t)stream));
    count_launches(1);
    return LT_OK;
}

extern "C" int lt_decode_num_ctas(void) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}
