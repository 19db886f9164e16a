// One decode step (one token through all layers, final norm, LM head and argmax) as ONE
// persistent kernel: a CTA per SM, the weight stream decoupled from the dependency chain.
//
// Why: at batch 1 a 0.5B model streams ~525 MB per token (80 us at HBM speed) but the step
// is a chain of ~120 dependent phases; as separate launches each phase costs microseconds of
// launch latency during which HBM idles.  Two things are done about that here.
//
// (1) Weights do not depend on activations, so a producer warp per CTA runs ahead of the
//     chain and keeps a ring of shared-memory stages filled with the weight rows this CTA
//     will need next (bulk async copies global -> shared, completion on an mbarrier, no
//     multicast), across phase and layer boundaries.
// (2) The phases are chained by DATA, not by grid barriers.  Every activation element that
//     crosses CTAs is stored as one 8-byte word {fp32 value, 32-bit tag}; the tag names the
//     token and layer that produced it.  A consumer simply loads the vector it needs and
//     retries the elements whose tag is not yet the expected one, so the cost of a phase
//     boundary is one L2 round trip after the last producer's store, with no fence, no
//     counter and no second round trip.  Value and tag travel in the same naturally aligned
//     store, so they can never be seen apart.  Buffer reuse is safe without barriers because
//     every rewrite of a buffer is separated from its last read by a full all-to-all phase
//     (nobody can produce layer l+1's q|k|v before every CTA has finished layer l).
//
// Arithmetic is the per-op kernels' arithmetic, repeated verbatim (same device functions):
//   P1  x -> rmsnorm(attn_norm) -> quant -> [q|k|v] GEMV + bias
//   P2  rope(q,k at *len) -> append k,v at *len -> masked attention (one CTA per query head)
//   P3  quant(att) -> o_proj GEMV + x -> x1            (*len += 1)
//   P4  rmsnorm(ffn_norm)(x1) -> quant -> gate rows, then up rows of the same indices;
//       v = silu(gate)*up is formed in the CTA that holds both
//   P5  quant(v) -> down GEMV + x1 -> x
//   LM  rmsnorm(out_norm)(x) -> quant -> LM-head GEMV -> logits, argmax
// so the step is bit-identical to the chain of per-op launches.
//
// Every wait (data tags, mbarriers, the one grid barrier before the argmax) is bounded by a
// clock limit; on expiry the kernel sets LT_STATUS_WAIT_TIMEOUT, stops waiting anywhere,
// drains its copies and returns.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

constexpr int DEC_THREADS = 512;
constexpr int DEC_CWARPS = 15;                  // consumer warps; warp 15 is the producer
constexpr int DEC_CTHREADS = DEC_CWARPS * 32;
constexpr int DEC_STAGE_BYTES = 32768;          // weight rows per stage (quants + scales)
constexpr int DEC_STAGE_STRIDE = DEC_STAGE_BYTES + 128;
constexpr int DEC_ILP = 4;                      // rows one warp folds together
constexpr int DEC_MAX_LAYERS = 128;
constexpr int DEC_ROWBUF = DEC_CTHREADS;        // per-CTA rows whose epilogue operand is staged
constexpr long long DEC_WAIT_CLOCKS = 2000000000LL;   // ~1 s at 2 GHz
#ifndef DEC_POLL_BACKOFF_NS
#define DEC_POLL_BACKOFF_NS 200
#endif

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
// 16-byte asynchronous copy global -> shared (no register staging)
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DEC_CTHREADS) : "memory"); }
// barrier of the consumer warps that also ANDs a predicate over them
__device__ __forceinline__ bool consumer_all(bool pred) {
    unsigned r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((unsigned)pred), "n"(DEC_CTHREADS)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// tagged activation element: {value, tag} in one 8-byte word
__device__ __forceinline__ void st_tagged(float2* p, float v, unsigned tag) { __stcg(p, make_float2(v, __uint_as_float(tag))); }

enum { KIND_QKV = 0, KIND_O = 1, KIND_GU = 2, KIND_DOWN = 3, KIND_LM = 4, KIND_COUNT = 5 };

struct Shared {
    unsigned long long full[8];
    unsigned long long empty[8];
    float sred[256];
    float red64[64];
    float add[DEC_ROWBUF];      // bias of this CTA's q|k|v rows
    float gate[DEC_ROWBUF];     // gate results of this CTA's rows, until the up rows arrive
    int lens[DEC_MAX_LAYERS];   // cache lengths at kernel entry (attention CTAs)
    lt_decode_layer ly[2];      // descriptor of the current and of the next layer
    int row0[KIND_COUNT], row1[KIND_COUNT];   // this CTA's row range per matrix kind
    int rc[KIND_COUNT];                        // rows per ring stage per matrix kind
    float best_v[DEC_CWARPS];
    int best_i[DEC_CWARPS];
    volatile int abort_flag;
};

__device__ __forceinline__ bool wait_expired(long long t0, unsigned& spins, Shared* S, int* status) {
    if (S->abort_flag) return true;
    if ((++spins & 63u) == 0) {
        if (*(volatile int*)status & (int)LT_STATUS_WAIT_TIMEOUT) { S->abort_flag = 1; return true; }   // another CTA gave up
        if (clock64() - t0 > DEC_WAIT_CLOCKS) {
            S->abort_flag = 1;
            atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
            return true;
        }
    }
    return false;
}

// bounded wait on an mbarrier phase; returns false on expiry
__device__ __noinline__ bool mbar_wait_slow(unsigned long long* bar, unsigned parity, Shared* S, int* status) {
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity))
        if (wait_expired(t0, spins, S, status)) return false;
    return true;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, Shared* S, int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, S, status);
}

// optional time stamps (thread 0 of CTA 0 and of the last CTA): pairs (id, SM clock)
constexpr int DEC_TRACE_CAP = 8192;      // entries per traced CTA
struct Tracer {
    long long* buf;
    int n;
    __device__ __forceinline__ void init(const lt_decode_desc& P) {
        buf = nullptr; n = 0;
        if (P.trace != nullptr && threadIdx.x == 0) {
            if (blockIdx.x == 0) buf = P.trace;
            else if (blockIdx.x == gridDim.x - 1) buf = P.trace + 2 * DEC_TRACE_CAP;
        }
    }
    __device__ __forceinline__ void stamp(int id) {
        if (buf != nullptr && n < DEC_TRACE_CAP) { buf[2 * n] = id; buf[2 * n + 1] = clock64(); n++; }
    }
};

// The one grid barrier of the step (before the final argmax); counter reset by the last CTA to
// leave the kernel.
__device__ __forceinline__ void grid_sync_once(unsigned* ctr, unsigned nctas, Shared* S, int* status) {
    consumer_sync();
    if (threadIdx.x == 0 && !S->abort_flag) {
        __threadfence();
        atomicAdd(ctr, 1u);
        const long long t0 = clock64();
        unsigned spins = 0;
        while (ld_acquire_u32(ctr) < nctas)
            if (wait_expired(t0, spins, S, status)) break;
    }
    consumer_sync();
}

// ---------------------------------------------------------------- phases
// Five weight phases per layer (q|k|v, o, gate, up, down) and the LM head.  The gate and up
// matrices are the two halves of the concatenated [2F, E] matrix; a CTA takes the same row
// range of both halves.
enum { PH_QKV = 0, PH_O = 1, PH_GATE = 2, PH_UP = 3, PH_DOWN = 4, PH_PER_LAYER = 5, PH_LM = 5 };

struct GemvDesc {
    const int8_t* Wq;
    const __half* Wd;
    int K, kind;
};

__device__ __forceinline__ GemvDesc phase_desc(const lt_decode_desc& P, const lt_decode_layer* ly, int ph) {
    GemvDesc d;
    switch (ph) {
        case PH_QKV: d.Wq = ly->qkv_q; d.Wd = (const __half*)ly->qkv_d; d.K = P.E; d.kind = KIND_QKV; break;
        case PH_O: d.Wq = ly->o_q; d.Wd = (const __half*)ly->o_d; d.K = P.nh * P.hd; d.kind = KIND_O; break;
        case PH_GATE: d.Wq = ly->gu_q; d.Wd = (const __half*)ly->gu_d; d.K = P.E; d.kind = KIND_GU; break;
        case PH_UP:
            d.Wq = ly->gu_q + (size_t)P.F * P.E;
            d.Wd = (const __half*)ly->gu_d + (size_t)P.F * (P.E >> 5);
            d.K = P.E; d.kind = KIND_GU;
            break;
        case PH_DOWN: d.Wq = ly->down_q; d.Wd = (const __half*)ly->down_d; d.K = P.F; d.kind = KIND_DOWN; break;
        default: d.Wq = P.lm_q; d.Wd = (const __half*)P.lm_d; d.K = P.E; d.kind = KIND_LM; break;
    }
    return d;
}

__device__ __forceinline__ void cta_rows(int M, int& r0, int& r1) {
    r0 = (int)(((long long)M * blockIdx.x) / gridDim.x);
    r1 = (int)(((long long)M * (blockIdx.x + 1)) / gridDim.x);
}
// rows per ring stage: as many as fit, at most DEC_ILP per consumer warp
__device__ __forceinline__ int rows_per_chunk(int K) {
    int rc = DEC_STAGE_BYTES / (K + (K >> 4));
    if (rc > DEC_CWARPS * DEC_ILP) rc = DEC_CWARPS * DEC_ILP;
    return rc < 1 ? 1 : rc;
}

// ---------------------------------------------------------------- producer
__device__ __forceinline__ void producer_loop(const lt_decode_desc& P, unsigned char* ring, int nstages, Shared* S) {
    int stage = 0;
    unsigned fill = 0;          // how many times the ring has wrapped
    for (int il = 0; il <= P.n_layers; il++) {
      const bool lm = (il == P.n_layers);
      for (int ph = lm ? PH_LM : 0; ph < (lm ? PH_LM + 1 : PH_PER_LAYER); ph++) {
        // descriptors are read from global memory: the producer runs ahead of the consumers
        const GemvDesc d = phase_desc(P, lm ? P.layers : P.layers + il, ph);
        const int r0 = S->row0[d.kind], r1 = S->row1[d.kind];
        const int nb = d.K >> 5;
        const int RC = S->rc[d.kind];
        for (int r = r0; r < r1; r += RC) {
            const int n = (r1 - r < RC) ? (r1 - r) : RC;
            if (fill > 0) {
                if (!mbar_wait(&S->empty[stage], (fill - 1) & 1, S, P.status)) return;
            }
            unsigned char* dst = ring + (size_t)stage * DEC_STAGE_STRIDE;
            const unsigned qbytes = (unsigned)n * d.K;
            // the scale rows are fetched as the enclosing 16-byte aligned window
            const size_t a0 = (size_t)(reinterpret_cast<uintptr_t>(d.Wd + (size_t)r * nb));
            const size_t d0 = a0 & ~(size_t)15;
            const size_t d1 = (a0 + (size_t)n * nb * 2 + 15) & ~(size_t)15;
            const unsigned dbytes = (unsigned)(d1 - d0);
            mbar_expect_tx(&S->full[stage], qbytes + dbytes);
            bulk_g2s(dst, d.Wq + (size_t)r * d.K, qbytes, &S->full[stage]);
            bulk_g2s(dst + qbytes, reinterpret_cast<const void*>(d0), dbytes, &S->full[stage]);
            if (++stage == nstages) { stage = 0; fill++; }
        }
      }
    }
}

// ---------------------------------------------------------------- consumer helpers
// Load n tagged elements into shared memory (values only), retrying the ones whose tag is not
// yet `want`.  All loads of a round are in flight together; a round ends in one consumer
// barrier that also tells whether every element has arrived, and a failed round backs off for
// a moment: polling that is too eager steals L2 bandwidth from the CTAs still producing
// (measured: per-warp free-running polls made the step slower).
template <int B>
__device__ __forceinline__ void wait_vector(const float2* __restrict__ g, float* s, int n, unsigned want, Shared* S,
                                            int* status) {
    float2 v[B];
    bool have[B];
#pragma unroll
    for (int k = 0; k < B; k++) have[k] = (k * DEC_CTHREADS + (int)threadIdx.x >= n);
    const long long t0 = clock64();
    unsigned spins = 0;
    for (;;) {
#pragma unroll
        for (int k = 0; k < B; k++)
            if (!have[k]) v[k] = __ldcg(g + k * DEC_CTHREADS + threadIdx.x);
        bool ok = true;
#pragma unroll
        for (int k = 0; k < B; k++) {
            if (!have[k]) have[k] = (__float_as_uint(v[k].y) == want);
            ok = ok && have[k];
        }
        if (consumer_all(ok)) break;
        if (threadIdx.x == 0) wait_expired(t0, spins, S, status);
        if (S->abort_flag) break;
        __nanosleep(DEC_POLL_BACKOFF_NS);
    }
#pragma unroll
    for (int k = 0; k < B; k++) {
        const int j = k * DEC_CTHREADS + threadIdx.x;
        if (j < n) s[j] = v[k].x;
    }
}

// quant(rmsnorm(x) * w) (sW != NULL) or quant(x) (sW == NULL) of a vector staged in shared memory
// into sXq / sXd.  The sum of squares follows the declared 256-lane order.  Each warp quantises
// up to four 32-blocks together so that their dependent chains overlap.
__device__ __forceinline__ void quant_from_smem(const float* sF, const float* sW, int N, float eps, int8_t* sXq,
                                                __half* sXd, Shared* S) {
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    float inv = 1.0f;
    if (sW != nullptr) {
        if (t < 256) {
            float local = 0.0f;
            for (int j = t; j < N; j += 256) local = __fmaf_rn(sF[j], sF[j], local);
            S->sred[t] = local;
        }
        consumer_sync();
        if (t < 32) {
            // levels 128, 64, 32 of the pairwise tree for lane t, in the declared pairing:
            // p[t] += p[t+128]; p[t] += p[t+64]; p[t] += p[t+32]
            const float* p = S->sred;
            const float a = __fadd_rn(__fadd_rn(p[t], p[t + 128]), __fadd_rn(p[t + 64], p[t + 192]));
            const float b = __fadd_rn(__fadd_rn(p[t + 32], p[t + 160]), __fadd_rn(p[t + 96], p[t + 224]));
            float v = warp_tree_sum(__fadd_rn(a, b));      // levels 16 .. 1
            if (t == 0) S->red64[0] = v;
        }
        consumer_sync();
        inv = rsqrtf(__fadd_rn(__fdiv_rn(S->red64[0], (float)N), eps));
    }
    const int nblk = N >> 5;
    for (int b0 = warp; b0 < nblk; b0 += 4 * DEC_CWARPS) {
        float v[4], a[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int b = b0 + k * DEC_CWARPS;
            const int j = (b < nblk ? b : b0) * 32 + lane;
            float x = sF[j];
            if (sW != nullptr) x = __fmul_rn(__fmul_rn(x, inv), sW[j]);
            v[k] = x;
            a[k] = fabsf(x);
        }
        // amax over the 32 lanes: the bit patterns of non-negative floats order like unsigned
        // integers, so one integer max-reduction gives the same maximum as a compare tree
#pragma unroll
        for (int k = 0; k < 4; k++) a[k] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(a[k])));
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int b = b0 + k * DEC_CWARPS;
            if (b < nblk) {
                const float d = (a[k] > 0.0f) ? __fdiv_rn(a[k], 127.0f) : 1.0f;
                const __half dh = __float2half_rn(d);
                const float dq = __half2float(dh);
                int q = (int)rintf(__fdiv_rn(v[k], dq));
                q = q < -127 ? -127 : (q > 127 ? 127 : q);
                sXq[b * 32 + lane] = (int8_t)q;
                if (lane == 0) sXd[b] = dh;
            }
        }
    }
    consumer_sync();
}

// ---------------------------------------------------------------- consumer: attention phase
// One CTA per query head.  Every global load of the phase is issued before the first use:
// all cached K and V rows of the head's KV group go to shared memory by 16-byte asynchronous
// copies (no registers), then the head's q / k / v slices (tagged, produced by P1 of this
// layer) are awaited.  K rows are padded by 4 floats so that one-row-per-thread reads do not
// collide on banks.
// sAtt: [maxt] probabilities, hd (q) + hd (new k) + hd (new v) floats, vcap V rows, vcap K rows.
__device__ __forceinline__ void attention_phase(const lt_decode_desc& P, const lt_decode_layer* ly, int pos,
                                                unsigned tag, float* sAtt, int vcap, Shared* S) {
    const int h = blockIdx.x;
    const int tid = threadIdx.x;
    const int hd = P.hd, hd4 = hd >> 2, nh = P.nh, nkv = P.nkv, maxt = P.max_seq;
    const int nq = nh * hd, nk = nkv * hd;
    const int rep = nh / nkv, hk = h / rep;
    const int kst = hd + 4;                  // padded K row stride in floats
    float* sh = sAtt;
    float* sQ = sAtt + maxt;
    float* sKn = sQ + hd;
    float* sVn = sKn + hd;
    float* sV = sVn + hd;
    float* sK = sV + (size_t)vcap * hd;
    const float2* qkv = (const float2*)P.ws_qkv;

    const bool room = (pos >= 0 && pos < maxt);
    if (!room) {
        if (tid == 0) atomicOr(P.status, (int)LT_STATUS_KV_OVERFLOW);
        pos = pos < 0 ? 0 : maxt;
    }
    const int L = room ? pos + 1 : pos;      // attention length after the append
    const int Lc = room ? pos : L;           // rows that already live in the cache
    const bool staged = (L <= vcap);
    // (1) cached K and V rows -> shared memory, asynchronously
    if (staged) {
        for (int e = tid; e < Lc * hd4; e += DEC_CTHREADS) {
            const int t = e / hd4, c = e - t * hd4;
            const size_t g = ((size_t)t * nkv + hk) * hd + c * 4;
            cp_async16(sK + (size_t)t * kst + c * 4, ly->kcache + g);
            cp_async16(sV + (size_t)t * hd + c * 4, ly->vcache + g);
        }
    }
    // (2) the q / k / v slices of the new token: three groups of hd/2 threads, two elements each
    const int half = hd >> 1;
    int role = -1, j = 0;
    const float2* src = qkv;
    if (tid >= 256 && tid < 256 + half) { role = 0; j = tid - 256; src = qkv + h * hd; }
    else if (tid >= 320 && tid < 320 + half) { role = 1; j = tid - 320; src = qkv + nq + hk * hd; }
    else if (tid >= 384 && tid < 384 + half) { role = 2; j = tid - 384; src = qkv + nq + nk + hk * hd; }
    float2 e1 = make_float2(0.0f, 0.0f), e2 = e1;
    {
        bool have = (role < 0);
        const long long t0 = clock64();
        unsigned spins = 0;
        for (;;) {
            if (!have) {
                e1 = __ldcg(src + j);
                e2 = __ldcg(src + j + half);
                have = (__float_as_uint(e1.y) == tag) && (__float_as_uint(e2.y) == tag);
            }
            if (consumer_all(have)) break;
            if (tid == 0) wait_expired(t0, spins, S, P.status);
            if (S->abort_flag) break;
            __nanosleep(DEC_POLL_BACKOFF_NS);
        }
    }
    if (role == 0) {
        float o1, o2;
        rope_pair(e1.x, e2.x, j, hd, P.theta, pos, o1, o2);
        sQ[j] = o1; sQ[j + half] = o2;
    } else if (role == 1) {
        float o1, o2;
        rope_pair(e1.x, e2.x, j, hd, P.theta, pos, o1, o2);
        sKn[j] = o1; sKn[j + half] = o2;
        if (room && staged) { sK[(size_t)pos * kst + j] = o1; sK[(size_t)pos * kst + j + half] = o2; }
    } else if (role == 2) {
        sVn[j] = e1.x; sVn[j + half] = e2.x;
        if (room && staged) { sV[(size_t)pos * hd + j] = e1.x; sV[(size_t)pos * hd + j + half] = e2.x; }
    }
    cp_async_wait_all();
    consumer_sync();
    if (room && (h % rep) == 0 && tid < hd) {
        ly->kcache[((size_t)pos * nkv + hk) * hd + tid] = sKn[tid];
        ly->vcache[((size_t)pos * nkv + hk) * hd + tid] = sVn[tid];
    }
    // scores: thread t owns positions t, t + 480, ...
    for (int t = tid; t < maxt; t += DEC_CTHREADS) {
        float v = -1e30f;
        if (t < L) {
            const float4* K4 = staged ? (const float4*)(sK + (size_t)t * kst)
                                      : ((room && t == pos) ? (const float4*)sKn
                                                            : (const float4*)(ly->kcache + ((size_t)t * nkv + hk) * hd));
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
            v = __fmul_rn(s, P.scale);
        }
        sh[t] = v;
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
        if (tid == 0) S->sred[0] = v;
    }
    consumer_sync();
    const float mx = S->sred[0];
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
        if (tid == 0) S->sred[1] = v;
    }
    consumer_sync();
    const float Z = S->sred[1];
    if (tid < hd) {
        float acc = 0.0f;
        if (staged) {
#pragma unroll 4
            for (int t = 0; t < L; t++) acc = __fmaf_rn(sh[t], sV[(size_t)t * hd + tid], acc);
        } else {
            const float* Vd = ly->vcache + (size_t)hk * hd + tid;
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
        st_tagged((float2*)P.ws_att + h * hd + tid, __fdiv_rn(acc, Z), tag);
    }
    consumer_sync();
}

// ---------------------------------------------------------------- the kernel
enum { EPI_QKV = 0, EPI_O = 1, EPI_GATE = 2, EPI_UP = 3, EPI_DOWN = 4, EPI_LOGITS = 5 };

__global__ void __launch_bounds__(DEC_THREADS, 1)
k_decode_step(const __grid_constant__ lt_decode_desc P, int nstages, int kmax, int fmax, int vcap) {
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
    float* sW = (float*)(smem + off);
    off += ((size_t)fmax * 4 + 127) & ~(size_t)127;
    float* sRes = (float*)(smem + off);       // residual rows of this CTA for the o_proj / down epilogues
    off += (size_t)2 * DEC_ROWBUF * 4;
    float* sAtt = (float*)(smem + off);       // attention area; doubles as the staging area of v in P5

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int E = P.E, F = P.F, nq = P.nh * P.hd, nqkv = nq + 2 * P.nkv * P.hd, L = P.n_layers;
    if (tid == 0) {
        for (int s = 0; s < nstages; s++) {
            mbar_init(&S->full[s], 1);
            mbar_init(&S->empty[s], DEC_CWARPS);
        }
        S->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid < KIND_COUNT) {
        const int M = tid == KIND_QKV ? nqkv : (tid == KIND_GU ? F : (tid == KIND_LM ? P.V : E));
        const int Kk = tid == KIND_O ? nq : (tid == KIND_DOWN ? F : E);
        int a, b;
        cta_rows(M, a, b);
        S->row0[tid] = a; S->row1[tid] = b;
        S->rc[tid] = rows_per_chunk(Kk);
    }
    __syncthreads();

    if (warp == DEC_CWARPS) {       // producer warp: one lane streams weights for the whole step
        if (lane == 0) producer_loop(P, ring, nstages, S);
        return;
    }

    // ------------------------------------------------------------ consumers
    const unsigned nctas = gridDim.x;
    int stage = 0;
    unsigned fill = 0;
    float bestv = -3.4e38f;
    int besti = 2147483647;
    Tracer tr;
    tr.init(P);
    tr.stamp(101);
    // tags of this step: token counter * (L+1) + layer + 1
    const unsigned tag0 = __ldcg(P.epoch) * (unsigned)(L + 1) + 1u;

    constexpr int LY_WORDS = (int)(sizeof(lt_decode_layer) / 8);
    if (tid < LY_WORDS) ((unsigned long long*)&S->ly[0])[tid] = ((const unsigned long long*)P.layers)[tid];
    if ((int)blockIdx.x < P.nh)
        for (int l = tid; l < L; l += DEC_CTHREADS) S->lens[l] = __ldcg(P.layers[l].len);

    // x for layer 0: gathered from the Q8_0 table by the device token, or preloaded by the host
    {
        const float* nw0 = P.layers[0].attn_norm;
        if (P.tok != nullptr) {
            int t = *P.tok;
            if (t < 0 || t >= P.V) {
                if (tid == 0 && blockIdx.x == 0) atomicOr(P.status, (int)LT_STATUS_BAD_TOKEN);
                t = t < 0 ? 0 : P.V - 1;
            }
            const int nbE = E >> 5;
            for (int j = tid; j < E; j += DEC_CTHREADS) {
                const __half dh = ((const __half*)P.emb_d)[(size_t)t * nbE + (j >> 5)];
                const int8_t q = P.emb_q[(size_t)t * E + j];
                const float nw = __ldg(nw0 + j);
                sF[j] = __fmul_rn(__half2float(dh), (float)q);
                sW[j] = nw;
            }
        } else {
            for (int j = tid; j < E; j += DEC_CTHREADS) {
                const float xv = __ldcg(P.x + j);
                const float nw = __ldg(nw0 + j);
                sF[j] = xv;
                sW[j] = nw;
            }
        }
    }
    consumer_sync();

    const int nph = PH_PER_LAYER * L + 1;
    int il = 0, ph = 0;
    for (int idx = 0; idx < nph; idx++, ph++) {
        if (ph == PH_PER_LAYER && il < L) { ph = 0; il++; }
        const bool lm = (il >= L);
        if (lm) ph = PH_LM;
        const lt_decode_layer* ly = &S->ly[il & 1];
        const unsigned tag = tag0 + (unsigned)il;           // data produced in this layer
        int epi = EPI_LOGITS;
        // ---------------- prologue: fetch the activation, quantise it into sXq / sXd
        if (ph == PH_QKV || ph == PH_LM) {
            // prefetch the next layer's descriptor (visible after this phase's barriers)
            if (!lm && il + 1 < L && tid < LY_WORDS)
                ((unsigned long long*)&S->ly[(il + 1) & 1])[tid] = ((const unsigned long long*)(P.layers + il + 1))[tid];
            const float* nw = lm ? P.out_norm : ly->attn_norm;
            const float* bias = lm ? nullptr : ly->qkv_bias;
            const int br0 = S->row0[KIND_QKV], bnr = S->row1[KIND_QKV] - br0;
            if (il > 0) {
                float nwv[4], bv = 0.0f;
                if (bias != nullptr && tid < bnr) bv = __ldg(bias + br0 + tid);
#pragma unroll
                for (int k = 0; k < 4; k++) { const int j = k * DEC_CTHREADS + tid; nwv[k] = (j < E) ? __ldg(nw + j) : 0.0f; }
                wait_vector<4>((const float2*)P.ws_x, sF, E, tag - 1u, S, P.status);
#pragma unroll
                for (int k = 0; k < 4; k++) { const int j = k * DEC_CTHREADS + tid; if (j < E) sW[j] = nwv[k]; }
                if (bias != nullptr && tid < bnr) S->add[tid] = bv;
            } else {
                if (bias != nullptr && tid < bnr) S->add[tid] = __ldg(bias + br0 + tid);
            }
            consumer_sync();
            if (!lm) {      // residual rows of x for the o_proj epilogue of this layer
                const int r0 = S->row0[KIND_O], nr = S->row1[KIND_O] - r0;
                if (tid < nr) sRes[tid] = sF[r0 + tid];
            }
            tr.stamp(11);
            quant_from_smem(sF, sW, E, P.eps, sXq, sXd, S);
            epi = lm ? EPI_LOGITS : EPI_QKV;
            tr.stamp(12);
        } else if (ph == PH_O) {
            // P2 first: rope + append + attention on the head CTAs
            if ((int)blockIdx.x < P.nh) {
                attention_phase(P, ly, S->lens[il], tag, sAtt, vcap, S);
            }
            tr.stamp(13);
            // the cache length advances (every head works from the lengths read at kernel entry)
            if (blockIdx.x == 0 && tid == 0) {
                int p = __ldcg(ly->len);
                if (p >= 0 && p < P.max_seq) *ly->len = p + 1;
            }
            wait_vector<4>((const float2*)P.ws_att, sF, nq, tag, S, P.status);
            consumer_sync();
            tr.stamp(14);
            quant_from_smem(sF, nullptr, nq, 0.0f, sXq, sXd, S);
            epi = EPI_O;
            tr.stamp(15);
        } else if (ph == PH_GATE) {
            float nwv[4];
#pragma unroll
            for (int k = 0; k < 4; k++) { const int j = k * DEC_CTHREADS + tid; nwv[k] = (j < E) ? __ldg(ly->ffn_norm + j) : 0.0f; }
            wait_vector<4>((const float2*)P.ws_x1, sF, E, tag, S, P.status);
#pragma unroll
            for (int k = 0; k < 4; k++) { const int j = k * DEC_CTHREADS + tid; if (j < E) sW[j] = nwv[k]; }
            consumer_sync();
            {               // residual rows of x1 for the down epilogue of this layer
                const int r0 = S->row0[KIND_DOWN], nr = S->row1[KIND_DOWN] - r0;
                if (tid < nr) sRes[DEC_ROWBUF + tid] = sF[r0 + tid];
            }
            tr.stamp(16);
            quant_from_smem(sF, sW, E, P.eps, sXq, sXd, S);
            epi = EPI_GATE;
            tr.stamp(17);
        } else if (ph == PH_UP) {
            consumer_sync();        // every gate value of this CTA is in shared memory
            epi = EPI_UP;
        } else {    // PH_DOWN
            wait_vector<12>((const float2*)P.ws_v, sAtt, F, tag, S, P.status);
            consumer_sync();
            tr.stamp(18);
            quant_from_smem(sAtt, nullptr, F, 0.0f, sXq, sXd, S);
            epi = EPI_DOWN;
            tr.stamp(19);
        }

        // ---------------- weight phase: fold this CTA's rows, one copy of the code for all phases
        const GemvDesc d = phase_desc(P, ly, ph);
        const int r0 = S->row0[d.kind], r1 = S->row1[d.kind];
        const int K = d.K, nb = K >> 5;
        const int RC = S->rc[d.kind];
        for (int r = r0; r < r1; r += RC) {
            const int n = (r1 - r < RC) ? (r1 - r) : RC;
            const bool ok = mbar_wait(&S->full[stage], fill & 1, S, P.status);
            tr.stamp(21);
            const unsigned char* base = ring + (size_t)stage * DEC_STAGE_STRIDE;
            const size_t doff = (size_t)(reinterpret_cast<uintptr_t>(d.Wd + (size_t)r * nb)) & 15;
            const __half* wdbase = (const __half*)(base + (size_t)n * K + doff);
            const int nv = (n - warp + DEC_CWARPS - 1) / DEC_CWARPS;     // this warp's rows of the chunk (<= DEC_ILP)
            if (ok && nv > 0) {
                // A warp folds up to DEC_ILP rows together (rows warp, warp+15, ... of the chunk):
                // the block loop is outermost, so each row keeps its own ascending-block fma chain
                // and its own 5-level shuffle tree while the chains of different rows overlap.
                float acc[DEC_ILP];
#pragma unroll
                for (int k = 0; k < DEC_ILP; k++) acc[k] = 0.0f;
                for (int b = lane; b < nb; b += 32) {
                    const int4* xp = (const int4*)(sXq + b * 32);
                    const int4 x0 = xp[0], x1 = xp[1];
                    const float xd = __half2float(sXd[b]);
#pragma unroll
                    for (int k = 0; k < DEC_ILP; k++) {
                        if (k < nv) {       // warp-uniform
                            const int i = warp + k * DEC_CWARPS;
                            const int4* wp = (const int4*)(base + (size_t)i * K + b * 32);
                            const int4 w0 = wp[0], w1 = wp[1];
                            const float wd = __half2float(wdbase[(size_t)i * nb + b]);
                            acc[k] = q8_accum(wd, xd, block_dot(w0, w1, x0, x1), acc[k]);
                        }
                    }
                }
#pragma unroll
                for (int s = 16; s > 0; s >>= 1) {
#pragma unroll
                    for (int k = 0; k < DEC_ILP; k++) acc[k] = __fadd_rn(acc[k], __shfl_down_sync(0xffffffffu, acc[k], s));
                }
                float v = acc[0];       // lane k finishes row k
#pragma unroll
                for (int k = 1; k < DEC_ILP; k++) {
                    const float t = __shfl_sync(0xffffffffu, acc[k], 0);
                    if (lane == k) v = t;
                }
                if (lane < nv) {
                    const int row = r + warp + lane * DEC_CWARPS;
                    const int li = row - r0;
                    switch (epi) {
                        case EPI_QKV:
                            if (ly->qkv_bias != nullptr) v = __fadd_rn(v, S->add[li]);
                            st_tagged((float2*)P.ws_qkv + row, v, tag);
                            break;
                        case EPI_O:
                            v = __fadd_rn(v, sRes[li]);
                            st_tagged((float2*)P.ws_x1 + row, v, tag);
                            break;
                        case EPI_GATE: S->gate[li] = v; break;
                        case EPI_UP: st_tagged((float2*)P.ws_v + row, silu_mul(S->gate[li], v), tag); break;
                        case EPI_DOWN:
                            v = __fadd_rn(v, sRes[DEC_ROWBUF + li]);
                            st_tagged((float2*)P.ws_x + row, v, tag);
                            break;
                        default:
                            P.logits[row] = v;
                            if (v > bestv || (v == bestv && row < besti)) { bestv = v; besti = row; }
                            break;
                    }
                }
            }
            __syncwarp();
            tr.stamp(22);
            if (lane == 0) mbar_arrive(&S->empty[stage]);
            if (++stage == nstages) { stage = 0; fill++; }
        }
        tr.stamp(30 + ph);
    }

    // ---------------- argmax: lanes 0..DEC_ILP-1 of every warp hold candidates
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bestv, s);
        int oi = __shfl_xor_sync(0xffffffffu, besti, s);
        if (ov > bestv || (ov == bestv && oi < besti)) { bestv = ov; besti = oi; }
    }
    if (lane == 0) { S->best_v[warp] = bestv; S->best_i[warp] = besti; }
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
    grid_sync_once(P.sync, nctas, S, P.status);
    if (blockIdx.x == 0 && warp == 0) {
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
    tr.stamp(118);
    // the last CTA to get here resets the barrier counters and advances the token counter
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(P.sync + 1, 1u) == nctas - 1) {
            P.sync[0] = 0;
            P.sync[1] = 0;
            *P.epoch = *P.epoch + 1u;
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
    const size_t r128 = 127;
    size_t fixed = ((sizeof(Shared) + r128) & ~r128) + (((size_t)g->kmax + r128) & ~r128) +
                   (((size_t)(g->kmax >> 5) * 2 + r128) & ~r128) + 2 * (((size_t)g->fmax * 4 + r128) & ~r128) +
                   (size_t)2 * DEC_ROWBUF * 4;
    const size_t att_fixed = ((size_t)d->max_seq + 3 * d->hd) * 4;
    const size_t vrow = (size_t)d->hd * 4 + (size_t)(d->hd + 4) * 4;     // one staged V row + one padded K row
    const size_t v_stage = (size_t)d->F * 4;      // P5 stages v in the attention area
    const size_t avail = (size_t)smem_max - 1024;
    const size_t min_area = att_fixed > v_stage ? att_fixed : v_stage;
    if (fixed + min_area + 2 * (size_t)DEC_STAGE_STRIDE > avail) {
        set_error("lt_decode_step: model dimensions need more shared memory than one SM has");
        return LT_ERR_UNSUPPORTED;
    }
    // ring first (3 stages, fewer only if the model leaves no room), then as many staged K/V
    // rows as fit (up to max_seq), then a deeper ring if room is left
    size_t left = avail - fixed;
    int nst = 3;
    while (nst > 2 && (size_t)nst * DEC_STAGE_STRIDE + min_area > left) nst--;
    size_t area = left - (size_t)nst * DEC_STAGE_STRIDE;
    size_t want = att_fixed + (size_t)d->max_seq * vrow;
    if (want < v_stage) want = v_stage;
    if (area > want) {
        while (nst < 8 && area >= want + (size_t)DEC_STAGE_STRIDE) { nst++; area -= DEC_STAGE_STRIDE; }   // spare room: deepen the ring
        area = want;
    }
    g->nstages = nst;
    g->vcap = area > att_fixed ? (int)((area - att_fixed) / vrow) : 0;
    if (g->vcap > d->max_seq) g->vcap = d->max_seq;
    g->smem = (size_t)nst * DEC_STAGE_STRIDE + fixed + area + 128;
    g->ctas = sms;
    return LT_OK;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_decode_step(const lt_decode_desc* d, void* stream) {
    LT_REQUIRE(d != nullptr, "lt_decode_step: null descriptor");
    LT_REQUIRE(d->layers && d->out_norm && d->lm_q && d->lm_d && d->logits && d->out_tok && d->sync && d->epoch &&
                   d->part_val && d->part_idx && d->ws_x && d->ws_x1 && d->ws_qkv && d->ws_att && d->ws_v,
               "lt_decode_step: null pointer in descriptor");
    LT_REQUIRE(d->tok != nullptr ? (d->emb_q && d->emb_d) : (d->x != nullptr),
               "lt_decode_step: needs either a device token with the embedding table or a preloaded input row");
    LT_REQUIRE(d->n_layers > 0 && d->n_layers <= DEC_MAX_LAYERS && d->E > 0 && d->F > 0 && d->V > 0 && d->max_seq > 0,
               "lt_decode_step: bad dimensions");
    LT_REQUIRE(d->E % 32 == 0 && d->F % 32 == 0 && (d->nh * d->hd) % 32 == 0, "lt_decode_step: E, F and nh*hd must be multiples of 32");
    LT_REQUIRE(d->E <= 4 * DEC_CTHREADS && d->nh * d->hd <= 4 * DEC_CTHREADS && d->F <= 12 * DEC_CTHREADS,
               "lt_decode_step: this build handles E and nh*hd up to %d and F up to %d", 4 * DEC_CTHREADS, 12 * DEC_CTHREADS);
    LT_REQUIRE(d->hd == 32 || d->hd == 64 || d->hd == 128, "lt_decode_step: hd=%d must be 32, 64 or 128", d->hd);
    LT_REQUIRE(d->nkv > 0 && d->nh % d->nkv == 0, "lt_decode_step: nh must be a multiple of nkv");
    LT_REQUIRE(d->max_seq % 4 == 0, "lt_decode_step: max_seq=%d must be a multiple of 4", d->max_seq);
    const int nq = d->nh * d->hd, nk = d->nkv * d->hd;
    // scale rows are fetched in 16-byte windows: every matrix (and the up half of gate|up) must
    // hold a multiple of 8 scales so that no window crosses the end of its array
    const long long ms[6] = {(long long)(nq + 2 * nk) * (d->E / 32), (long long)d->E * (nq / 32),
                             (long long)d->F * (d->E / 32), (long long)2 * d->F * (d->E / 32),
                             (long long)d->E * (d->F / 32), (long long)d->V * (d->E / 32)};
    for (int i = 0; i < 6; i++)
        LT_REQUIRE(ms[i] % 8 == 0, "lt_decode_step: a weight matrix has %lld scales, not a multiple of 8", ms[i]);
    DecodeGeometry g;
    int rc = decode_geometry(d, &g);
    if (rc != LT_OK) return rc;
    LT_REQUIRE(d->nh <= g.ctas, "lt_decode_step: more query heads (%d) than SMs (%d)", d->nh, g.ctas);
    const int widest = d->F > nq + 2 * nk ? d->F : nq + 2 * nk;
    LT_REQUIRE(widest / g.ctas + 1 <= DEC_ROWBUF, "lt_decode_step: more rows per CTA than the epilogue buffers hold");
    LT_CUDA(cudaFuncSetAttribute(k_decode_step, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
    lt_decode_desc P = *d;
    if (P.status == nullptr) P.status = device_status_ptr();
    LT_REQUIRE(P.status != nullptr, "lt_decode_step: status word unavailable");
    int nstages = g.nstages, kmax = g.kmax, fmax = g.fmax, vcap = g.vcap;
    void* args[] = {&P, &nstages, &kmax, &fmax, &vcap};
    // cooperative launch: all CTAs are resident together, which the data-flow waits rely on
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
