// One decode step (one token through all layers, final norm, LM head and argmax) as ONE
// persistent kernel: a CTA per SM, the weight stream decoupled from the dependency chain, and
// FOUR cross-SM exchanges per layer.
//
// Why: at batch 1 a 0.5B model streams ~525 MB per token (80 us at HBM speed), but the step is a
// chain of dependent phases; what a phase costs is not its bytes but the hand-over of a small
// activation vector from every SM to every SM through L2.  So the step is organised to need as
// few hand-overs as the arithmetic allows, and to make each one a single L2 round trip.
//
// Roles (one cooperative launch, grid = number of SMs, 512 threads; warp 15 of every CTA only
// issues bulk copies):
//   * CTAs [0, nh) are ATTENTION CTAs, one per query head.  The head's q rows and its KV group's
//     k rows of the q|k|v matrix (2*hd rows) are resident in shared memory for the next layer
//     before the layer's input arrives, the cached V rows of the group are staged in shared
//     memory and the cached K rows sit in registers (one position per thread).  From the layer
//     input x the CTA computes RMSNorm -> quantiser -> its q and k rows -> rope -> KV append ->
//     masked attention -> quantised head output, with block barriers only.
//   * the other CTAs are GEMV CTAs.  Each owns a fixed slice of the rows of every other matrix:
//     the v rows of q|k|v, o_proj, whole 32-row blocks of gate|up (so that silu(gate)*up is
//     quantised where it is produced), down, and (together with the attention CTAs) the LM head.
//     A producer warp fetches the CTA's rows with bulk async copies (no multicast), ahead of the
//     dependency chain: within the layers every slice has a FIXED place in shared memory (a slot
//     per phase, refilled with the next layer's slice once this layer's has been folded -- the
//     large ones while the attention CTAs work, so that the refills do not travel through L2
//     during a hand-over -- so a phase finds its rows early and at addresses that never change);
//     the LM head, many times the size of shared memory, streams through a ring of stages over
//     the same area.  All weight copies are marked "evict first" in L2.
//
// Per layer:   x --(1)--> attention CTAs: q,k,attention -> a(q8)          GEMV CTAs: v rows
//              a --(2)--> o_proj + x -> x1 --(3)--> rmsnorm, gate|up, silu*up -> v(q8)
//              v --(4)--> down + x1 -> x'
// Every element that crosses CTAs is one 8-byte word {payload, tag}; the tag names the token and
// the layer.  A consumer loads the words it needs and retries those whose tag is not yet the
// expected one: payload and tag travel in one naturally aligned store, so no fence, flag or
// counter is involved.  A buffer is rewritten only after a full all-to-all hand-over separates
// the rewrite from its last read, so single buffers suffice.  Quantised vectors travel packed
// (4 int8 per word, one fp16 scale per word).
//
// Arithmetic is the per-op kernels' arithmetic (same device functions, same frozen orders), so
// the step is bit-identical to the chain of per-op launches.
//
// Every wait (tags, mbarriers) is bounded by a clock limit; on expiry the kernel sets
// LT_STATUS_WAIT_TIMEOUT, stops waiting anywhere, lets its copies land and returns.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"

namespace lt {

constexpr int DEC_THREADS = 512;
constexpr int DEC_CWARPS = 15;                  // consumer warps; warp 15 is the producer
constexpr int DEC_CTHREADS = DEC_CWARPS * 32;
constexpr int DEC_STAGE_BYTES = 32768;          // weight rows per ring stage (quants + scales)
constexpr int DEC_STAGE_STRIDE = DEC_STAGE_BYTES + 128;
constexpr int DEC_MAX_STAGES = 8;
constexpr int DEC_ILP = 4;                      // rows one warp folds together
constexpr int DEC_MAX_LAYERS = 128;
constexpr int DEC_XB = 4;                       // E <= 256 * DEC_XB (words of x polled per thread)
constexpr int DEC_VB = 4;                       // F/4 + F/32 <= DEC_CTHREADS * DEC_VB
constexpr int DEC_AB = 4;                       // nq/4 + nq/32 <= DEC_CTHREADS * DEC_AB
constexpr int DEC_NREP = 32;                    // copies of every hand-over buffer (one per lane of the storing warp)
constexpr unsigned DEC_FIRST_LOOK_DELAY_NS = 200;      // pause of a GEMV CTA between its preparation and its first look
constexpr long long DEC_WAIT_CLOCKS = 2000000000LL;   // ~1 s at 2 GHz
constexpr long long DEC_DRAIN_CLOCKS = 4000000LL;     // ~2 ms: copies in flight after a give-up

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
// bulk async copy global -> this CTA's shared memory, completion counted on an mbarrier, with an L2 eviction
// policy for the lines it touches.  Every weight byte passes through L2 once per
// token: marked "evict first", the stream leaves the small hot set (hand-over words, KV rows, norm weights)
// in L2 instead of sweeping it out (measured: 1.2-1.8 % of the step; asking L2 to KEEP a part of the LM head
// from token to token instead was slower at every fraction tried)
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, unsigned bytes, unsigned long long* bar,
                                              unsigned long long policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// 16-byte asynchronous copy global -> shared (no register staging)
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DEC_CTHREADS) : "memory"); }
__device__ __forceinline__ void pair_sync() { asm volatile("bar.sync 2, 64;" ::: "memory"); }   // warps 0 and 1

// tagged element: {payload, tag} in one 8-byte word
__device__ __forceinline__ void st_tagged(float2* p, float v, unsigned tag) { __stcg(p, make_float2(v, __uint_as_float(tag))); }
__device__ __forceinline__ void st_tagged_u32(float2* p, unsigned v, unsigned tag) {
    __stcg(p, make_float2(__uint_as_float(v), __uint_as_float(tag)));
}

// A hand-over buffer of n words exists DEC_NREP times (replica r at g + r*n); CTA c reads replica
// c % DEC_NREP, so that no L2 line is polled by more than a few SMs.  A warp stores one word to all
// replicas with one instruction (lane = replica).
__device__ __forceinline__ void st_tagged_all(float2* g, int n, int idx, unsigned payload, unsigned tag, int nrep) {
    const int lane = threadIdx.x & 31;
    if (lane < nrep) __stcg(g + (size_t)lane * n + idx, make_float2(__uint_as_float(payload), __uint_as_float(tag)));
}

struct GemvConst {
    unsigned big;       // shared address of the big area (slot p at big + SL.off[p])
    unsigned db[4];     // scale rows of slot p relative to the slot (p = 2: offset of a chunk's scale rows within their 16-byte window)
    int v0, nv, e0, ne, b0, nbk;    // the CTA's slices: first v row / count, first o_proj and down row / count, first FFN block / count
};

struct Shared {
    unsigned long long full[DEC_MAX_STAGES];
    unsigned long long empty[DEC_MAX_STAGES];
    unsigned long long sfull[4], sempty[4]; // GEMV CTA: the slots of the four layer phases
    unsigned long long wfull, wempty;       // attention CTA: the head's resident q|k rows
    unsigned long long att_done;            // attention CTA: layers finished, the big area is free for the LM ring
    float sred[256];                        // RMSNorm lane partials (the declared 256 lanes)
    float red[64], red2[64];                // softmax lane partials
    float sv[2][32];                        // silu(gate)*up of the FFN blocks being folded
    float bias[256];                        // attention CTA: bias of its q rows, then of its k rows
    float qk[256];                          // attention CTA: q rows then k rows before rope
    // plan of a full LM-head set, remembered per warp relative to the stage bases: [warp][qrel 4 | drel 4 |
    // chunk of row k (4 x 8 bits) | nset | nch | nv]
    unsigned memo[DEC_CWARPS][12];
    float vn[128];                          // attention CTA: the new v row of its group
    int lens[DEC_MAX_LAYERS];               // cache lengths at kernel entry
    float best_v[DEC_CWARPS];
    int best_i[DEC_CWARPS];
    volatile int abort_flag;
    int nrep;                               // copies of the hand-over buffers in use (1..DEC_NREP)
    GemvConst gc;                           // GEMV CTA: what does not change from layer to layer
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
__device__ __forceinline__ bool mbar_wait_slow(unsigned long long* bar, unsigned parity, Shared* S, int* status) {
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

// Spin until every word this thread is responsible for carries the tag `want`.  The thread's
// words are g[first + k*stride], k < nwords <= 4, as far as they lie below n (first < 0: none).
// All outstanding loads of a look are in flight together; threads spin independently (no barrier
// inside the loop); `pause_ns` is slept between two looks.  Returns false if the wait was given up.
//
// Everything in this kernel is inlined and must stay in registers: with the shared-memory carve-out
// this kernel needs, L1 has next to nothing left, so a thread's stack (spills, arrays passed by
// pointer to a real function) lives in L2 -- which the weight stream sweeps all the time -- and every
// access to it is a memory round trip on the critical path.  (Measured: a few hundred bytes of stack
// per thread made the step 1.6x slower.)
template <typename Sink>
__device__ __forceinline__ bool poll_words(const float2* __restrict__ g, int n, int first, int stride, int nwords,
                                           unsigned want, Sink sink, Shared* S, int* status, unsigned pause_ns) {
    // sink(k, payload) takes word k when it has arrived (no copy of the words is kept in registers)
    unsigned pending = 0;
#pragma unroll
    for (int k = 0; k < 4; k++)
        if (k < nwords && first >= 0 && first + k * stride < n) pending |= 1u << k;
    if (!pending) return true;
    const long long t0 = clock64();
    unsigned spins = 0;
    for (;;) {
        float2 w[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (pending & (1u << k)) w[k] = __ldcg(g + first + k * stride);
#pragma unroll
        for (int k = 0; k < 4; k++)
            if ((pending & (1u << k)) && __float_as_uint(w[k].y) == want) { sink(k, w[k].x); pending &= ~(1u << k); }
        if (!pending) return true;
        if (wait_expired(t0, spins, S, status)) return false;
        if (pause_ns) __nanosleep(pause_ns);
    }
}

// optional time stamps (thread 0 of CTA 0 and of the last CTA): pairs (id, SM clock)
constexpr int DEC_TRACE_CAP = 8192;      // entries per traced CTA
struct Tracer {
    long long* buf;
    int n;
    __device__ __forceinline__ void init(const lt_decode_desc& P) {
        buf = nullptr; n = 0;
        if (P.trace != nullptr && threadIdx.x == 0) {
            const unsigned second = P.trace_cta > 0 ? (unsigned)P.trace_cta : gridDim.x - 1;
            if (blockIdx.x == 0) buf = P.trace;
            else if (blockIdx.x == second) buf = P.trace + 2 * DEC_TRACE_CAP;
        }
    }
    __device__ __forceinline__ void stamp(int id) {
        if (buf != nullptr && n < DEC_TRACE_CAP) { buf[2 * n] = id; buf[2 * n + 1] = clock64(); n++; }
    }
};

// Diagnostics, second form: with a trace buffer and trace_layer = l >= 0, thread 0 of EVERY CTA stores the
// global timer at the arrival of each phase's input (slots 0..3) and at the end of each phase (slots 4..7) of
// layer l, in the last 8 * gridDim.x entries of the trace buffer: one layer's hand-overs on one clock.
__device__ __forceinline__ void layer_timeline(const lt_decode_desc& P, int il, int slot) {
    if (P.trace != nullptr && threadIdx.x == 0 && il == P.trace_layer) {
        unsigned long long gt;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
        P.trace[4 * DEC_TRACE_CAP - 8 * (int)gridDim.x + 8 * (int)blockIdx.x + slot] = (long long)gt;
    }
}

// ---------------------------------------------------------------- weight ring
struct Ring {
    unsigned char* base;
    unsigned long long* full;
    unsigned long long* empty;
    int nstages;
    int stage;
    unsigned fill;      // how many times the ring has wrapped
    __device__ __forceinline__ void advance() { if (++stage == nstages) { stage = 0; fill++; } }
};

// rows per ring stage: as many as fit, at most DEC_ILP per consumer warp
__device__ __forceinline__ int rows_per_chunk(int K) {
    int rc = DEC_STAGE_BYTES / (K + (K >> 4));
    if (rc > DEC_CWARPS * DEC_ILP) rc = DEC_CWARPS * DEC_ILP;
    return rc < 1 ? 1 : rc;
}
// ... of the LM head, which is streamed for many sets: if a stage holds more than half a set of
// DEC_CWARPS * DEC_ILP rows, half a set per stage, so that two stages give every warp DEC_ILP rows
__device__ __forceinline__ int rows_per_chunk_lm(int K) {
    const int rc = rows_per_chunk(K), half = DEC_CWARPS * DEC_ILP / 2;
    return (rc > half && rc < 2 * half) ? half : rc;
}

// producer side: rows [r0, r1) of a matrix with row length K, chunk by chunk
// gate: the first use of stage gate_stage (and so of every later stage) waits for that barrier phase first
// (the ring lies over memory that is still being read until then); nullptr = no gate.
__device__ __forceinline__ bool produce_segment(Ring& R, const int8_t* Wq, const __half* Wd, int r0, int r1, int K, int RC,
                                                Shared* S, int* status, unsigned long long* gate = nullptr,
                                                unsigned gate_parity = 0, int gate_stage = 0) {
    const unsigned long long pol = l2_policy_evict_first();
    const int nb = K >> 5;
    for (int r = r0; r < r1; r += RC) {
        const int n = (r1 - r < RC) ? (r1 - r) : RC;
        if (R.fill > 0) {
            if (!mbar_wait(&R.empty[R.stage], (R.fill - 1) & 1, S, status)) return false;
        } else if (gate != nullptr && R.stage == gate_stage) {
            if (!mbar_wait(gate, gate_parity, S, status)) return false;
        }
        unsigned char* dst = R.base + (size_t)R.stage * DEC_STAGE_STRIDE;
        const unsigned qbytes = (unsigned)n * K;
        // the scale rows are fetched as the enclosing 16-byte aligned window
        const size_t a0 = (size_t)(reinterpret_cast<uintptr_t>(Wd + (size_t)r * nb));
        const size_t d0 = a0 & ~(size_t)15;
        const size_t d1 = (a0 + (size_t)n * nb * 2 + 15) & ~(size_t)15;
        const unsigned dbytes = (unsigned)(d1 - d0);
        mbar_expect_tx(&R.full[R.stage], qbytes + dbytes);
        bulk_g2s_hint(dst, Wq + (size_t)r * K, qbytes, &R.full[R.stage], pol);
        bulk_g2s_hint(dst + qbytes, reinterpret_cast<const void*>(d0), dbytes, &R.full[R.stage], pol);
        R.advance();
    }
    return true;
}

// After a give-up the consumers no longer wait for the stages: before the CTA may exit, the
// producer lets the copies it has armed land (bounded), so that none arrives in shared memory
// that already belongs to another kernel's CTA.
__device__ __forceinline__ void producer_drain(const Ring& R) {
    const long long t0 = clock64();
    for (int s = 0; s < R.nstages; s++) {
        // the last phase armed on stage s: fill (if s < R.stage this wrap already armed it) or fill - 1
        const bool armed_this_wrap = s < R.stage;
        if (!armed_this_wrap && R.fill == 0) continue;
        const unsigned parity = (armed_this_wrap ? R.fill : R.fill - 1) & 1;
        while (!mbar_try_wait(&R.full[s], parity))
            if (clock64() - t0 > DEC_DRAIN_CLOCKS) return;
    }
}

// ---- slots: where a GEMV CTA keeps its slice of the four layer matrices.  Slot p (phase p) holds rows
// [r0, r0 + n) of a matrix as n*K quant bytes followed by the 16-byte aligned window of their scales; the
// gate|up slot holds, block after block, the gate chunk and the up chunk (32 rows each, same format) at
// a fixed pitch.  Offsets are the same in every CTA (sized for the largest share).
struct DecSlots {
    int off[4];         // byte offset of slot p in the big area
    int chunk;          // pitch of a 32-row chunk in the gate|up slot
};

// producer: request rows [r, r + n) of a matrix into shared memory at dst; returns the bytes requested
__device__ __forceinline__ unsigned slot_request(unsigned char* dst, const int8_t* Wq, const __half* Wd, int r, int n, int K,
                                                 unsigned long long* bar) {
    const int nb = K >> 5;
    const unsigned qbytes = (unsigned)n * K;
    const size_t a0 = (size_t)(reinterpret_cast<uintptr_t>(Wd + (size_t)r * nb));
    const size_t d0 = a0 & ~(size_t)15;
    const size_t d1 = (a0 + (size_t)n * nb * 2 + 15) & ~(size_t)15;
    const unsigned dbytes = (unsigned)(d1 - d0);
    const unsigned long long pol = l2_policy_evict_first();
    bulk_g2s_hint(dst, Wq + (size_t)r * K, qbytes, bar, pol);
    bulk_g2s_hint(dst + qbytes, reinterpret_cast<const void*>(d0), dbytes, bar, pol);
    return qbytes + dbytes;
}
__device__ __forceinline__ unsigned slot_bytes(const __half* Wd, int r, int n, int K) {
    const int nb = K >> 5;
    const size_t a0 = (size_t)(reinterpret_cast<uintptr_t>(Wd + (size_t)r * nb));
    return (unsigned)n * K + (unsigned)(((a0 + (size_t)n * nb * 2 + 15) & ~(size_t)15) - (a0 & ~(size_t)15));
}

enum { EPI_V = 0, EPI_O = 1, EPI_DOWN = 2, EPI_LOGITS = 3 };

struct EpiCtx {
    Tracer tr;
    const lt_decode_desc* P;
    const lt_decode_layer* ly;
    Shared* S;
    const float* resid;     // residual vector in shared memory (EPI_O, EPI_DOWN)
    unsigned tag;
    int pos, room;          // EPI_V: where the new cache row goes
    int nq, nk;
    float bestv;
    int besti;
};

// The two 16-byte halves of lane L's 32-byte block are read in swapped order by the lanes whose
// bit 2 is set: a quarter-warp's eight 16-byte reads then fall on all 32 banks (plain lane*32
// addressing makes lanes L and L+4 collide).  The block dot is an integer sum: any order is exact.
__device__ __forceinline__ int lane_swizzle() { return ((threadIdx.x >> 2) & 1) << 4; }

__device__ __forceinline__ int4 lds128(unsigned addr) {
    int4 v;
    asm("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_half(unsigned addr) {
    unsigned short h;
    asm("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
    return __half2float(__ushort_as_half(h));
}

// rows a warp folds together: shared addresses of the quants and of the scales of each row
template <int NR>
struct RowSetN {
    unsigned q[NR];
    unsigned d[NR];
};
typedef RowSetN<DEC_ILP> RowSet;

// Fold up to NR rows of shared memory against the quantised activation at shared addresses
// xq / xd: lane L folds blocks L, L+32, ... in ascending order (the frozen chain), then the 5-level
// shuffle tree; the chains of the rows overlap.  Returns in lane k (k < nv) the result of row k.
// The first nv (warp-uniform) rows are valid.
template <int NR>
__device__ __forceinline__ float fold_rows(const RowSetN<NR>& rs, int nb, int nv, unsigned xq, unsigned xd) {
    const int lane = threadIdx.x & 31;
    const unsigned sw = (unsigned)lane_swizzle();
    float acc[NR];
#pragma unroll
    for (int k = 0; k < NR; k++) acc[k] = 0.0f;
#pragma unroll (NR == 1 ? 4 : (NR <= 4 ? 2 : 1))
    for (int b = lane; b < nb; b += 32) {
        const int4 x0 = lds128(xq + b * 32 + sw);
        const int4 x1 = lds128(xq + b * 32 + (sw ^ 16u));
        const float xs = lds_half(xd + b * 2);
#pragma unroll
        for (int k = 0; k < NR; k++) {
            if (k < nv) {       // warp-uniform
                const int4 w0 = lds128(rs.q[k] + b * 32 + sw);
                const int4 w1 = lds128(rs.q[k] + b * 32 + (sw ^ 16u));
                const float wd = lds_half(rs.d[k] + b * 2);
                acc[k] = q8_accum(wd, xs, block_dot(w0, w1, x0, x1), acc[k]);
            }
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
#pragma unroll
        for (int k = 0; k < NR; k++) acc[k] = __fadd_rn(acc[k], __shfl_down_sync(0xffffffffu, acc[k], s));
    }
    float v = acc[0];       // lane k takes row k
#pragma unroll
    for (int k = 1; k < NR; k++) {
        const float t = __shfl_sync(0xffffffffu, acc[k], 0);
        if (lane == k) v = t;
    }
    return v;
}

constexpr int DEC_MAXCH = 4;    // chunks of one segment that are folded together

// consumer side of a segment = rows [r0, r1) of a matrix with row length K, streamed through the ring (the LM
// head).  Up to DEC_MAXCH chunks are taken together as one SET and their rows dealt to the warps (row j of
// the set to warp j % 15); a warp folds up to DEC_ILP rows together.  Work is split in two so that everything
// that does not depend on the activation (waiting for the weight stages, every address, the epilogue's
// operand) is done BEFORE the hand-over is awaited, and only the fold and the store come after it.
struct SegPlan {
    RowSet rs;
    int r;          // first row of the set
    int nset, nch, nv;
    float add;      // epilogue operand of this lane's row (bias / residual)
    bool ok;
};

// memo: the plan of a full set relative to its stages' base addresses is the same for every full set of the
// segment (same chunking, and a set's scale rows start a whole number of 16-byte units after the previous set's):
// memo_mode 1 = compute it and remember it, 2 = take it from the memo (a fraction of the arithmetic), 0 = neither.
__device__ __forceinline__ SegPlan seg_prepare(int epi, const Ring& R, const __half* Wd, int r0, int r, int r1, int K,
                                               int RC, EpiCtx& C, unsigned* memo, int memo_mode) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = K >> 5;
    SegPlan sp;
    sp.r = r;
    sp.ok = true;
    unsigned cb[DEC_MAXCH];
    if (memo_mode == 2) {
        sp.nset = (int)memo[9]; sp.nch = (int)memo[10]; sp.nv = (int)memo[11];
        Ring R2 = R;
#pragma unroll
        for (int c = 0; c < DEC_MAXCH; c++) {
            cb[c] = 0;
            if (c < sp.nch) {
                sp.ok = mbar_wait(&R2.full[R2.stage], R2.fill & 1, C.S, C.P->status) && sp.ok;
                cb[c] = smem_u32(R2.base + (size_t)R2.stage * DEC_STAGE_STRIDE);
                R2.advance();
            }
        }
        const unsigned ck = memo[8];
#pragma unroll
        for (int k = 0; k < DEC_ILP; k++) {
            const unsigned c = (ck >> (8 * k)) & 0xffu;
            unsigned base = cb[0];
#pragma unroll
            for (int cc = 1; cc < DEC_MAXCH; cc++)
                if (c == (unsigned)cc) base = cb[cc];
            sp.rs.q[k] = base + memo[k];
            sp.rs.d[k] = base + memo[4 + k];
        }
    } else {
        // the set: chunks with nset rows from row r on, at most DEC_MAXCH chunks and DEC_CWARPS * DEC_ILP rows
        int nset = r1 - r;
        if (nset > DEC_MAXCH * RC) nset = DEC_MAXCH * RC;
        if (nset > DEC_CWARPS * DEC_ILP) nset = (DEC_CWARPS * DEC_ILP / RC > 0 ? DEC_CWARPS * DEC_ILP / RC : 1) * RC;
        if (nset > r1 - r) nset = r1 - r;
        sp.nset = nset;
        sp.nch = (nset + RC - 1) / RC;
        sp.nv = (nset - warp + DEC_CWARPS - 1) / DEC_CWARPS;     // this warp's rows of the set (<= DEC_ILP)
        unsigned qrel[DEC_ILP], drel[DEC_ILP], ck = 0;
#pragma unroll
        for (int k = 0; k < DEC_ILP; k++) { qrel[k] = 0; drel[k] = 0; }
        Ring R2 = R;
#pragma unroll
        for (int c = 0; c < DEC_MAXCH; c++) {
            cb[c] = 0;
            if (c < sp.nch) {
                sp.ok = mbar_wait(&R2.full[R2.stage], R2.fill & 1, C.S, C.P->status) && sp.ok;
                const int rc0 = r + c * RC;
                const int n = (r + nset - rc0 < RC) ? (r + nset - rc0) : RC;
                cb[c] = smem_u32(R2.base + (size_t)R2.stage * DEC_STAGE_STRIDE);
                const unsigned cdrel = (unsigned)(n * K) + (unsigned)(reinterpret_cast<uintptr_t>(Wd + (size_t)rc0 * nb) & 15);
#pragma unroll
                for (int k = 0; k < DEC_ILP; k++) {
                    const int i = warp + k * DEC_CWARPS - c * RC;       // row k of this warp, relative to chunk c
                    if (c == 0) drel[k] = cdrel;                        // (unused slots point at valid memory)
                    if (i >= 0 && i < n) {
                        qrel[k] = (unsigned)(i * K);
                        drel[k] = cdrel + (unsigned)(i * nb * 2);
                        ck |= (unsigned)c << (8 * k);
                    }
                }
                R2.advance();
            }
        }
#pragma unroll
        for (int k = 0; k < DEC_ILP; k++) {
            const unsigned c = (ck >> (8 * k)) & 0xffu;
            unsigned base = cb[0];
#pragma unroll
            for (int cc = 1; cc < DEC_MAXCH; cc++)
                if (c == (unsigned)cc) base = cb[cc];
            sp.rs.q[k] = base + qrel[k];
            sp.rs.d[k] = base + drel[k];
        }
        if (memo_mode == 1 && lane == 0) {
#pragma unroll
            for (int k = 0; k < DEC_ILP; k++) { memo[k] = qrel[k]; memo[4 + k] = drel[k]; }
            memo[8] = ck; memo[9] = (unsigned)sp.nset; memo[10] = (unsigned)sp.nch; memo[11] = (unsigned)sp.nv;
        }
    }
    sp.add = 0.0f;
    if (lane < sp.nv) {
        const int row = r + warp + lane * DEC_CWARPS;
        if (epi == EPI_V) { if (C.ly->qkv_bias != nullptr) sp.add = __ldg(C.ly->qkv_bias + row); }
        else if (epi == EPI_O || epi == EPI_DOWN) sp.add = C.resid[row];
    }
    return sp;
}

// The same for a slot: rows [r0, r0 + n) of the matrix lie at shared address sbase, their scale rows at dbase;
// the set is rows i0 .. of them, dealt to the warps as above.  Nothing but a wait for the slot
// (first set only) and a few multiplications: the addresses do not depend on the layer.
__device__ __forceinline__ SegPlan slot_prepare(int epi, unsigned sbase, unsigned dbase, int r0, int i0, int n, int K,
                                                unsigned long long* bar, unsigned parity, EpiCtx& C) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = K >> 5;
    SegPlan sp;
    sp.r = r0 + i0;
    sp.nch = 0;
    int m = n - i0;
    if (m > DEC_CWARPS * DEC_ILP) m = DEC_CWARPS * DEC_ILP;
    sp.nset = m;
    sp.nv = m > warp ? (m - warp + DEC_CWARPS - 1) / DEC_CWARPS : 0;
    sp.ok = (i0 > 0 || n <= 0) ? true : mbar_wait(bar, parity, C.S, C.P->status);
#pragma unroll
    for (int k = 0; k < DEC_ILP; k++) {
        int i = i0 + warp + k * DEC_CWARPS;
        if (i >= n) i = n > 0 ? n - 1 : 0;      // (unused rows point at valid memory)
        sp.rs.q[k] = sbase + (unsigned)(i * K);
        sp.rs.d[k] = dbase + (unsigned)(i * nb * 2);
    }
    sp.add = 0.0f;
    if (lane < sp.nv) {
        const int row = sp.r + warp + lane * DEC_CWARPS;
        if (epi == EPI_V) { if (C.ly->qkv_bias != nullptr) sp.add = __ldg(C.ly->qkv_bias + row); }
        else if (epi == EPI_O || epi == EPI_DOWN) sp.add = C.resid[row];
    }
    return sp;
}

__device__ __forceinline__ void seg_finish(int epi, const SegPlan& sp, Ring& R, int K, const int8_t* sXq, const __half* sXd,
                                           EpiCtx& C) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const lt_decode_desc& P = *C.P;
    float v = 0.0f;
    if (sp.ok && sp.nv == 1) {
        // one long row per warp (down): its rounds' loads and block dots all in flight, only the fma chain is serial
        RowSetN<1> r1;
        r1.q[0] = sp.rs.q[0]; r1.d[0] = sp.rs.d[0];
        v = fold_rows<1>(r1, K >> 5, 1, smem_u32(sXq), smem_u32(sXd));
    } else if (sp.ok && sp.nv > 0) {
        v = fold_rows<DEC_ILP>(sp.rs, K >> 5, sp.nv, smem_u32(sXq), smem_u32(sXd));
    }
    // the stages are no longer read: hand them back before the epilogue
    __syncwarp();
    for (int c = 0; c < sp.nch; c++) {
        if (lane == 0) mbar_arrive(&R.empty[R.stage]);
        R.advance();
    }
    if (sp.ok && sp.nv > 0) {
        const int row = sp.r + warp + lane * DEC_CWARPS;       // lanes < nv
        if (epi == EPI_V) {
            // row of the v section: bias, hand-over to the attention CTAs of its KV group, cache row
            if (lane < sp.nv) {
                const int vr = row - (C.nq + C.nk);     // index within the v section
                if (C.ly->qkv_bias != nullptr) v = __fadd_rn(v, sp.add);
                st_tagged((float2*)P.ws_qkv + vr, v, C.tag);
                if (C.room) C.ly->vcache[(size_t)C.pos * C.nk + vr] = v;
            }
        } else if (epi == EPI_O || epi == EPI_DOWN) {
            // residual add, then the lanes store the row's word to the copies of the buffer
            v = __fadd_rn(v, sp.add);
            float2* g = (float2*)(epi == EPI_O ? P.ws_x1 : P.ws_x);
            if (C.S->nrep == 1) {       // one copy: lane k stores row k itself
                if (lane < sp.nv) st_tagged(g + row, v, C.tag);
            } else
            for (int k = 0; k < sp.nv; k++) {
                const float vk = __shfl_sync(0xffffffffu, v, k);
                st_tagged_all(g, P.E, sp.r + warp + k * DEC_CWARPS, __float_as_uint(vk), C.tag, C.S->nrep);
            }
        } else {
            if (lane < sp.nv) {
                P.logits[row] = v;
                if (v > C.bestv || (v == C.bestv && row < C.besti)) { C.bestv = v; C.besti = row; }
            }
        }
    }
}

// one warp: quantise the 32-block whose lane values are `val` and publish it packed at block index b
// of a vector of n elements, in every copy of the buffer (nw = n/4 + n/32 words per copy)
__device__ __forceinline__ void publish_block_q8(float2* g, int n, int b, float val, unsigned tag, int nrep) {
    const int nw = (n >> 2) + (n >> 5);
    __half dh;
    const unsigned q = (unsigned)quant_lane(val, &dh) & 0xffu;
    unsigned w = q;
    w |= __shfl_down_sync(0xffffffffu, q, 1) << 8;
    w |= __shfl_down_sync(0xffffffffu, q, 2) << 16;
    w |= __shfl_down_sync(0xffffffffu, q, 3) << 24;
    if (nrep == 1) {        // one copy: the lanes that hold a word store it themselves, one instruction
        const int lane = threadIdx.x & 31;
        if ((lane & 3) == 0) st_tagged_u32(g + b * 8 + (lane >> 2), w, tag);
        if (lane == 0) st_tagged_u32(g + (n >> 2) + b, (unsigned)__half_as_ushort(dh), tag);
        return;
    }
    for (int i = 0; i < 8; i++) {
        const unsigned wi = __shfl_sync(0xffffffffu, w, 4 * i);
        st_tagged_all(g, nw, b * 8 + i, wi, tag, nrep);
    }
    st_tagged_all(g, nw, (n >> 2) + b, (unsigned)__half_as_ushort(dh), tag, nrep);
}

// gate|up of up to two whole 32-row FFN blocks [b, b + nbk) of the CTA's gate|up slot (chunk j of the slot
// at sbase + j*pitch: gate and up of the CTA's first block, gate and up of its second, ...); a warp folds gate row i and up row i of two
// rows of a block side by side (rows i = warp, warp+15; warps 0 and 1 then rows 30 and 31), forms
// silu(gate)*up where both results land, and the blocks are then quantised and published by one warp each.
struct FfnPlan {
    unsigned cbase[4], cwd[4];      // shared addresses of the chunks: gate, up of block b, gate, up of block b+1
    bool ok;
};

__device__ __forceinline__ FfnPlan ffn_prepare(unsigned sbase, unsigned pitch, unsigned dalign, int b0, int b, int nbk, int E) {
    FfnPlan fp;
    fp.ok = true;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        fp.cbase[c] = 0; fp.cwd[c] = 0;
        if (c < 2 * nbk) {
            // gate chunk, then up chunk of a block; a chunk's scale rows start a whole number of 16-byte units
            // after the matrix's first scale (32 rows of E/32 scales, F rows more for the up chunk)
            fp.cbase[c] = sbase + (unsigned)((b - b0) * 2 + c) * pitch;
            fp.cwd[c] = fp.cbase[c] + (unsigned)(32 * E) + dalign;
        }
    }
    return fp;
}

__device__ __forceinline__ void ffn_finish(const FfnPlan& fp, int F, int b, int nbk, bool more, int E,
                                           const int8_t* sXq, const __half* sXd, EpiCtx& C) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = E >> 5;
    const unsigned xq = smem_u32(sXq), xd = smem_u32(sXd);
    const int items = (32 - warp + DEC_CWARPS - 1) / DEC_CWARPS;     // rows of a block this warp folds: 3 for warps 0 and 1, else 2
    if (nbk == 2 && fp.ok) {
        // two blocks in ONE pass: their 64 FFN rows j = warp, warp + 15, ... (up to five per warp), gate and up row
        // of each side by side.  A pass costs a fixed ~0.5 us plus ~0.1 us per row of a warp, so one pass of ten
        // rows is shorter than two passes of six
        const int items2 = (64 - warp + DEC_CWARPS - 1) / DEC_CWARPS;
        RowSetN<10> rs;
#pragma unroll
        for (int k = 0; k < 10; k++) {
            int j = warp + (k >> 1) * DEC_CWARPS;       // FFN row within the two blocks
            if (j > 63) j = 63;
            const int bi = j >> 5, i = j & 31;
            const unsigned q0 = (k & 1) ? (bi ? fp.cbase[3] : fp.cbase[1]) : (bi ? fp.cbase[2] : fp.cbase[0]);
            const unsigned d0 = (k & 1) ? (bi ? fp.cwd[3] : fp.cwd[1]) : (bi ? fp.cwd[2] : fp.cwd[0]);
            rs.q[k] = q0 + (unsigned)(i * E);
            rs.d[k] = d0 + (unsigned)(i * nb * 2);
        }
        const float v = fold_rows<10>(rs, nb, 2 * items2, xq, xd);   // lanes 2k, 2k+1: gate, up of FFN row warp + 15 k
        const float u = __shfl_down_sync(0xffffffffu, v, 1);
        if (lane < 2 * items2 && (lane & 1) == 0) {
            const int j = warp + (lane >> 1) * DEC_CWARPS;
            C.S->sv[j >> 5][j & 31] = silu_mul(v, u);
        }
    } else
    for (int bi = 0; bi < nbk && fp.ok; bi++) {
        const unsigned gq = bi ? fp.cbase[2] : fp.cbase[0], uq = bi ? fp.cbase[3] : fp.cbase[1];
        const unsigned gd = bi ? fp.cwd[2] : fp.cwd[0], ud = bi ? fp.cwd[3] : fp.cwd[1];
        RowSetN<6> rs;
#pragma unroll
        for (int k = 0; k < 6; k++) {
            int i = warp + (k >> 1) * DEC_CWARPS;
            if (i > 31) i = 31;
            rs.q[k] = ((k & 1) ? uq : gq) + (unsigned)(i * E);
            rs.d[k] = ((k & 1) ? ud : gd) + (unsigned)(i * nb * 2);
        }
        const float v = fold_rows<6>(rs, nb, 2 * items, xq, xd);     // lanes 2j, 2j+1: gate, up of row warp + 15 j
        const float u = __shfl_down_sync(0xffffffffu, v, 1);
        if (lane < 2 * items && (lane & 1) == 0) C.S->sv[bi][warp + (lane >> 1) * DEC_CWARPS] = silu_mul(v, u);
    }
    consumer_sync();
    if (warp < nbk) publish_block_q8((float2*)C.P->ws_v, F, b + warp, C.S->sv[warp][lane], C.tag, C.S->nrep);
    if (more) consumer_sync();      // sv is rewritten by the next group
}

// ---------------------------------------------------------------- activation prologue
// quant(rmsnorm(x) * w) of the vector in sF whose 256 declared RMSNorm lane partials are in S->sred,
// into sXq / sXd.  1/rms: tree levels 128, 64, 32 in registers (p[t] += p[t+128]; += p[t+64];
// += p[t+32] for lane t), levels 16 .. 1 by shuffles; every warp evaluates it for itself (same
// operations in the same order: same bits).  Then the 15 consumer warps quantise two blocks each at a
// time so that their dependent chains overlap.
__device__ __forceinline__ void norm_quant(const float* sF, const float* sW, int N, float eps, int8_t* sXq, __half* sXd,
                                        const Shared* S) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* sred = S->sred;
    const float a = __fadd_rn(__fadd_rn(sred[lane], sred[lane + 128]), __fadd_rn(sred[lane + 64], sred[lane + 192]));
    const float b = __fadd_rn(__fadd_rn(sred[lane + 32], sred[lane + 160]), __fadd_rn(sred[lane + 96], sred[lane + 224]));
    float ss = warp_tree_sum(__fadd_rn(a, b));
    ss = __shfl_sync(0xffffffffu, ss, 0);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)N), eps));
    const int nblk = N >> 5;
    for (int b0 = warp; b0 < nblk; b0 += 2 * DEC_CWARPS) {
        float v[2], m[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int bb = b0 + k * DEC_CWARPS;
            const int j = (bb < nblk ? bb : b0) * 32 + lane;
            const float x = __fmul_rn(__fmul_rn(sF[j], inv), sW[j]);
            v[k] = x;
            // amax over the 32 lanes: bit patterns of non-negative floats order like unsigned integers
            m[k] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(x))));
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int bb = b0 + k * DEC_CWARPS;
            if (bb < nblk) {
                const float d = (m[k] > 0.0f) ? __fdiv_rn(m[k], 127.0f) : 1.0f;
                const __half dh = __float2half_rn(d);
                int q = (int)rintf(__fdiv_rn(v[k], __half2float(dh)));
                q = q < -127 ? -127 : (q > 127 ? 127 : q);
                sXq[bb * 32 + lane] = (int8_t)q;
                if (lane == 0) sXd[bb] = dh;
            }
        }
    }
}

// The layer input x (E tagged words) -> sF, with the declared RMSNorm lane partials
// p_t = fold_{j = t, t+256, ...} fma(x_j, x_j, .) formed by the thread that fetched them.
// from_smem: x is already in sF (first layer: embedding row), only the partials are formed.
__device__ __forceinline__ void fetch_x(const float2* g, unsigned want, bool from_smem, float* sF, int E, Shared* S,
                                     int* status, unsigned pause_ns) {
    const int t = threadIdx.x;
    if (t < 256) {
        float p = 0.0f;
        if (from_smem) {
            for (int j = t; j < E; j += 256) p = __fmaf_rn(sF[j], sF[j], p);
        } else {
            poll_words(g + (size_t)(blockIdx.x % S->nrep) * E, E, t, 256, DEC_XB, want,
                             [&](int k, float x) { sF[t + k * 256] = x; }, S, status, pause_ns);
#pragma unroll
            for (int k = 0; k < DEC_XB; k++) {       // the declared lane partial: this thread's words in ascending order
                const int j = t + k * 256;
                if (j < E) { const float x = sF[j]; p = __fmaf_rn(x, x, p); }
            }
        }
        S->sred[t] = p;
    }
}

// a packed quantised vector (n/4 words of 4 int8, then n/32 words of one fp16 scale) -> sXq / sXd
__device__ __forceinline__ void fetch_q8(const float2* g, unsigned want, int n, int8_t* sXq, __half* sXd, Shared* S, int* status,
                                      unsigned pause_ns) {
    const int nw = (n >> 2) + (n >> 5);
    poll_words(g + (size_t)(blockIdx.x % S->nrep) * nw, nw, threadIdx.x, DEC_CTHREADS, 4, want,
                     [&](int k, float x) {
                         const int i = threadIdx.x + k * DEC_CTHREADS;
                         if (i < (n >> 2)) ((unsigned*)sXq)[i] = __float_as_uint(x);
                         else sXd[i - (n >> 2)] = __ushort_as_half((unsigned short)(__float_as_uint(x) & 0xffffu));
                     }, S, status, pause_ns);
}

struct Areas {
    int8_t* xq0; __half* xd0;       // quantised activation of the phases whose row length is E
    int8_t* xq1; __half* xd1;       // ... whose row length is nh*hd or F
    float* fa; float* fb;           // x and x1 of the layer (fp32)
    float* w;                       // norm weight
    float* sh;                      // attention probabilities [max_seq]
    float* q; float* kn;            // rotated q and new k of the head
    unsigned char* big;             // ring stages (GEMV CTA) / resident q|k rows + staged V rows (attention CTA)
};

// ---------------------------------------------------------------- attention CTA, one layer
template <int HD>
__device__ __forceinline__ void attention_layer(const lt_decode_desc& P, const lt_decode_layer* ly, int il, unsigned tag0,
                                                const Areas& A, int vcap, Shared* S, Tracer& tr) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x;
    const int E = P.E, nb = E >> 5, nh = P.nh, nkv = P.nkv, maxt = P.max_seq;
    const int nq = nh * HD, nk = nkv * HD, rep = nh / nkv, hk = h / rep;
    constexpr int HD4 = HD / 4, HALF = HD / 2;
    const unsigned tag = tag0 + (unsigned)il;
    const unsigned backoff = (unsigned)P.poll_ns;
    float* sV = (float*)(A.big + (size_t)2 * HD * (E + 2 * nb));

    int pos = S->lens[il];
    const bool room = (pos >= 0 && pos < maxt);
    if (!room) {
        if (tid == 0) atomicOr(P.status, (int)LT_STATUS_KV_OVERFLOW);
        pos = pos < 0 ? 0 : maxt;
    }
    const int L = room ? pos + 1 : pos;      // attention length after the append
    const int Lc = room ? pos : L;           // rows that already live in the cache
    const int vst = Lc < vcap ? Lc : vcap;   // cached V rows staged in shared memory

    // ---- before the layer input is awaited: everything that does not depend on it
    // cached K rows in registers: position tid/2, the even thread holds the first half of the row,
    // the odd thread the second half (the score's fma chain runs through the even thread, then the odd)
    constexpr int HD8 = HD / 8;
    constexpr int KPOS = DEC_CTHREADS / 2;   // positions held in registers
    float4 kr[HD8];
#pragma unroll
    for (int i = 0; i < HD8; i++) kr[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if ((tid >> 1) < Lc) {
        const float4* kp = (const float4*)(ly->kcache + ((size_t)(tid >> 1) * nkv + hk) * HD) + (tid & 1) * HD8;
#pragma unroll
        for (int i = 0; i < HD8; i++) kr[i] = __ldcg(kp + i);
    }
    for (int e = tid; e < vst * HD4; e += DEC_CTHREADS) {
        const int t = e / HD4, c = e - t * HD4;
        cp_async16(sV + (size_t)t * HD + c * 4, ly->vcache + ((size_t)t * nkv + hk) * HD + c * 4);
    }
    for (int j = tid; j < E; j += DEC_CTHREADS) A.w[j] = __ldg(ly->attn_norm + j);
    if (tid < 2 * HD && ly->qkv_bias != nullptr)
        S->bias[tid] = __ldg(ly->qkv_bias + (tid < HD ? h * HD + tid : nq + hk * HD + (tid - HD)));
    float rc = 1.0f, rs = 0.0f;              // rope angle of pair tid: the same for q and k
    if (tid < HALF) rope_trig(tid, HD, P.theta, pos, rc, rs);

    // the head's resident q|k rows were requested a layer ago
    const bool wok = mbar_wait(&S->wfull, (unsigned)il & 1u, S, P.status);
    // ---- layer input -> RMSNorm -> quantiser
    fetch_x((const float2*)P.ws_x, tag - 1u, il == 0, A.fa, E, S, P.status, backoff);
    consumer_sync();
    tr.stamp(11);
    norm_quant(A.fa, A.w, E, P.eps, A.xq0, A.xd0, S);
    consumer_sync();
    tr.stamp(111);
    // ---- the head's q rows and its group's k rows (resident): rows warp, warp+15, ... four at a time
    {
        const unsigned wq = smem_u32(A.big);
        const unsigned wd = wq + (unsigned)(2 * HD * E);
        constexpr int AILP = 5;     // 2*hd = 128 rows over 15 warps: two passes of up to 5 rows
        for (int i0 = warp; i0 < 2 * HD && wok; i0 += DEC_CWARPS * AILP) {
            const int left = (2 * HD - i0 + DEC_CWARPS - 1) / DEC_CWARPS;
            const int nv = left < AILP ? left : AILP;
            RowSetN<AILP> rs;
#pragma unroll
            for (int k = 0; k < AILP; k++) {
                int i = i0 + k * DEC_CWARPS;
                if (i >= 2 * HD) i = 2 * HD - 1;
                rs.q[k] = wq + (unsigned)(i * E);
                rs.d[k] = wd + (unsigned)(i * nb * 2);
            }
            float v = fold_rows<AILP>(rs, nb, nv, smem_u32(A.xq0), smem_u32(A.xd0));
            const int i = i0 + lane * DEC_CWARPS;
            if (lane < nv) {
                if (ly->qkv_bias != nullptr) v = __fadd_rn(v, S->bias[i]);
                S->qk[i] = v;
            }
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&S->wempty);      // this warp no longer reads the resident rows
    consumer_sync();
    tr.stamp(12);
    // ---- rope of q and k (pair tid), KV append of the k row
    if (tid < HALF) {
        float o1, o2;
        rope_rotate(S->qk[tid], S->qk[tid + HALF], rc, rs, o1, o2);
        A.q[tid] = o1; A.q[tid + HALF] = o2;
        rope_rotate(S->qk[HD + tid], S->qk[HD + tid + HALF], rc, rs, o1, o2);
        A.kn[tid] = o1; A.kn[tid + HALF] = o2;
        if (room && (h % rep) == 0) {
            float* kc = ly->kcache + ((size_t)pos * nkv + hk) * HD;
            kc[tid] = o1; kc[tid + HALF] = o2;
        }
    }
    cp_async_wait_all();
    consumer_sync();
    // ---- scores: threads 2t, 2t+1 own position t (cached row in registers, the new row from shared memory)
    {
        const int t = tid >> 1, hf = tid & 1;
        if (room && t == pos) {
            const float4* k4 = (const float4*)A.kn + hf * HD8;
#pragma unroll
            for (int i = 0; i < HD8; i++) kr[i] = k4[i];
        }
        const float4* q4 = (const float4*)A.q + hf * HD8;
        float s = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            if (hf == half) {
#pragma unroll
                for (int i = 0; i < HD8; i++) {
                    const float4 qq = q4[i];
                    s = __fmaf_rn(qq.x, kr[i].x, s); s = __fmaf_rn(qq.y, kr[i].y, s);
                    s = __fmaf_rn(qq.z, kr[i].z, s); s = __fmaf_rn(qq.w, kr[i].w, s);
                }
            }
            if (half == 0) {        // the odd thread continues the chain of its even neighbour
                const float se = __shfl_sync(0xffffffffu, s, lane & ~1);
                if (hf == 1) s = se;
            }
        }
        if (hf == 1 && t < L) A.sh[t] = __fmul_rn(s, P.scale);
    }
    for (int t = tid + KPOS; t < L; t += DEC_CTHREADS) {     // contexts longer than the registers hold
        const float4* k4 = (room && t == pos) ? (const float4*)A.kn
                                              : (const float4*)(ly->kcache + ((size_t)t * nkv + hk) * HD);
        const float4* q4 = (const float4*)A.q;
        float s = 0.0f;
#pragma unroll 4
        for (int i = 0; i < HD4; i++) {
            const float4 qq = q4[i], kk = k4[i];
            s = __fmaf_rn(qq.x, kk.x, s); s = __fmaf_rn(qq.y, kk.y, s);
            s = __fmaf_rn(qq.z, kk.z, s); s = __fmaf_rn(qq.w, kk.w, s);
        }
        A.sh[t] = __fmul_rn(s, P.scale);
    }
    consumer_sync();
    tr.stamp(13);
    // ---- softmax in the declared 64-lane layout, V fold, quantiser: warps 0 and 1.  Positions
    // beyond L hold -1e30 / contribute exp() = +0 in the declared order: leaving them out gives
    // the same maximum and the same sums.
    if (warp == 2) {
        // the new v row of the group comes from the GEMV CTAs: fetched by an otherwise idle warp
        // while warps 0 and 1 do the softmax
        if (room) {
            for (int j = lane; j < HD; j += 32) {
                poll_words((const float2*)P.ws_qkv, nk, hk * HD + j, 0, 1, tag, [&](int, float x) { S->vn[j] = x; }, S,
                           P.status, backoff);
            }
        }
        asm volatile("bar.sync 3, 96;" ::: "memory");
    }
    if (tid < 64) {
        float m = -1e30f;
        for (int t = tid; t < L; t += 64) m = fmaxf(m, A.sh[t]);
        S->red[tid] = m;
        pair_sync();
        float mx = fmaxf(S->red[lane], S->red[lane + 32]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        float ls = 0.0f;
        for (int t = tid; t < L; t += 64) {
            const float e = __expf(__fsub_rn(A.sh[t], mx));
            A.sh[t] = e;
            ls = __fadd_rn(ls, e);
        }
        S->red2[tid] = ls;
        pair_sync();
        float Z = warp_tree_sum(__fadd_rn(S->red2[lane], S->red2[lane + 32]));
        Z = __shfl_sync(0xffffffffu, Z, 0);
        float out = 0.0f;
        if (tid < HD) {
            float acc = 0.0f;
#pragma unroll 4
            for (int t = 0; t < vst; t++) acc = __fmaf_rn(A.sh[t], sV[(size_t)t * HD + tid], acc);
            if (vst < Lc) {
                const float* Vd = ly->vcache + (size_t)hk * HD + tid;
                const size_t stride = (size_t)nkv * HD;
                int t = vst;
                for (; t + 8 <= Lc; t += 8) {
                    float v[8];
#pragma unroll
                    for (int k = 0; k < 8; k++) v[k] = __ldcg(Vd + (size_t)(t + k) * stride);
#pragma unroll
                    for (int k = 0; k < 8; k++) acc = __fmaf_rn(A.sh[t + k], v[k], acc);
                }
                for (; t < Lc; t++) acc = __fmaf_rn(A.sh[t], __ldcg(Vd + (size_t)t * stride), acc);
            }
            asm volatile("bar.sync 3, 96;" ::: "memory");       // warp 2 has the new v row
            if (room) acc = __fmaf_rn(A.sh[pos], S->vn[tid], acc);
            out = __fdiv_rn(acc, Z);
        } else {
            asm volatile("bar.sync 3, 96;" ::: "memory");
        }
        if (warp < (HD >> 5)) publish_block_q8((float2*)P.ws_att, nq, (h * HD >> 5) + warp, out, tag, S->nrep);
    }
    tr.stamp(14);
    consumer_sync();        // the shared-memory areas of this layer may be rewritten
}

// ---------------------------------------------------------------- GEMV CTA, one phase of one layer

__device__ __forceinline__ void gemv_phase(const int PH, const lt_decode_desc& P, const lt_decode_layer* lys, int il, int L, unsigned tag0,
                                           const DecSlots& SL, const Areas& A, Shared* S, EpiCtx& C) {
    const GemvConst& GC = S->gc;
    const int tid = threadIdx.x, lane = tid & 31;
    const int E = P.E, F = P.F;
    const lt_decode_layer* ly = lys + il;
    const unsigned tag = tag0 + (unsigned)il;
    const unsigned backoff = (unsigned)P.poll_ns;
    const int epi = PH == 0 ? EPI_V : (PH == 1 ? EPI_O : EPI_DOWN);
    const int K = PH == 1 ? C.nq : (PH == 3 ? F : E);
    const int r0 = PH == 0 ? C.nq + C.nk + GC.v0 : (PH == 2 ? GC.b0 : GC.e0);
    const int n = PH == 0 ? GC.nv : (PH == 2 ? GC.nbk : GC.ne);
    const unsigned sb = GC.big + (unsigned)(PH == 0 ? SL.off[0] : (PH == 1 ? SL.off[1] : (PH == 2 ? SL.off[2] : SL.off[3])));
    const unsigned db = PH == 2 ? GC.db[2] : sb + GC.db[PH];
    const int pitch = SL.chunk;
    C.ly = ly; C.tag = tag;
    if (PH == 0) {
        const int pos = S->lens[il];
        C.room = (pos >= 0 && pos < P.max_seq);
        C.pos = pos;
    }
    if (PH == 1) C.resid = A.fa;
    if (PH == 3) C.resid = A.fb;
    // ---- before the hand-over is awaited: the slot of the phase, every address, the epilogue's operands,
    // the norm weight of the next phase (into registers)
    SegPlan sp;
    FfnPlan fp;
    if (PH == 2) {
        fp = ffn_prepare(sb, (unsigned)pitch, db, r0, r0, n < 2 ? n : 2, E);
        if (n > 0) fp.ok = mbar_wait(&S->sfull[2], (unsigned)il & 1u, S, P.status);
    } else {
        sp = slot_prepare(epi, sb, db, r0, 0, n, K, &S->sfull[PH], (unsigned)il & 1u, C);
    }
    float nwr[DEC_XB / 2];
    if (PH & 1) {
        const float* nw = PH == 1 ? ly->ffn_norm : (il + 1 < L ? lys[il + 1].attn_norm : P.out_norm);
#pragma unroll
        for (int k = 0; k < DEC_XB / 2; k++) {
            const int j = tid + k * DEC_CTHREADS;
            nwr[k] = j < E ? __ldg(nw + j) : 0.0f;
        }
    }
    C.tr.stamp(20);
    // a short pause before the first look at a vector that is being stored right now: the reads of 134 SMs on a
    // line delay the stores to it (a first look issued before the preparation cost 15 %; 200 ns of quiet gain
    // 1-1.4 %, 300 ns and more lose again).  Not before the attention output, which is microseconds away.
    if (PH != 1 && !(PH == 0 && il == 0)) __nanosleep(DEC_FIRST_LOOK_DELAY_NS);
    // ---- the hand-over, then what depends on it
    if ((PH & 1) == 0) {
        float* sF = PH == 0 ? A.fa : A.fb;
        fetch_x((const float2*)(PH == 0 ? P.ws_x : P.ws_x1), PH == 0 ? tag - 1u : tag, PH == 0 && il == 0, sF, E, S, P.status, backoff);
        consumer_sync();
        C.tr.stamp(21 + PH);
        norm_quant(sF, A.w, E, P.eps, A.xq0, A.xd0, S);
        consumer_sync();
    } else {
        fetch_q8((const float2*)(PH == 1 ? P.ws_att : P.ws_v), tag, PH == 1 ? C.nq : F, A.xq1, A.xd1, S, P.status, backoff);
        // the norm weight of the next phase; every read of A.w in the previous phase is past a barrier
#pragma unroll
        for (int k = 0; k < DEC_XB / 2; k++) {
            const int j = tid + k * DEC_CTHREADS;
            if (j < E) A.w[j] = nwr[k];
        }
        consumer_sync();
        C.tr.stamp(21 + PH);
    }
    layer_timeline(P, il, PH);
    const int8_t* sXq = (PH & 1) ? A.xq1 : A.xq0;
    const __half* sXd = (PH & 1) ? A.xd1 : A.xd0;
    if (PH == 2) {
        const bool ok2 = fp.ok;
        for (int b = r0; b < r0 + n; b += 2) {
            if (b > r0) {
                fp = ffn_prepare(sb, (unsigned)pitch, db, r0, b, r0 + n - b < 2 ? r0 + n - b : 2, E);
                fp.ok = ok2;
            }
            ffn_finish(fp, F, b, r0 + n - b < 2 ? r0 + n - b : 2, b + 2 < r0 + n, E, sXq, sXd, C);
        }
    } else {
        Ring none;      // (a slot's rows are not ring stages: nothing is handed back per set)
        none.base = nullptr; none.full = nullptr; none.empty = nullptr; none.nstages = 1; none.stage = 0; none.fill = 0;
        for (;;) {
            seg_finish(epi, sp, none, K, sXq, sXd, C);
            const int i = sp.r - r0 + sp.nset;
            if (i >= n) break;
            const bool ok1 = sp.ok;
            sp = slot_prepare(epi, sb, db, r0, i, n, K, &S->sfull[PH], (unsigned)il & 1u, C);
            sp.ok = ok1;
        }
    }
    // this warp no longer reads the slot: the next layer's slice may be requested
    __syncwarp();
    if (lane == 0 && (n > 0 || PH == 0)) mbar_arrive(&S->sempty[PH]);     // (phase 0 is also the producer's cue: always)
    C.tr.stamp(25 + PH);
    layer_timeline(P, il, 4 + PH);
}

// ---------------------------------------------------------------- the kernel
template <int HD>
__global__ void __launch_bounds__(DEC_THREADS, 1)
k_decode_step(const __grid_constant__ lt_decode_desc P, int nstages, int nstages_att, int vcap, int fixed_bytes,
              const DecSlots SL) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int E = P.E, F = P.F, nq = P.nh * HD, nk = P.nkv * HD, L = P.n_layers, nbE = E >> 5;
    const int kmax1 = nq > F ? nq : F;
    // fixed areas (the same in both roles), then the big area
    Areas A;
    Shared* S = (Shared*)smem;
    size_t off = (sizeof(Shared) + 127) & ~(size_t)127;
    A.xq0 = (int8_t*)(smem + off); off += ((size_t)E + 127) & ~(size_t)127;
    A.xd0 = (__half*)(smem + off); off += ((size_t)nbE * 2 + 127) & ~(size_t)127;
    A.xq1 = (int8_t*)(smem + off); off += ((size_t)kmax1 + 127) & ~(size_t)127;
    A.xd1 = (__half*)(smem + off); off += ((size_t)(kmax1 >> 5) * 2 + 127) & ~(size_t)127;
    A.fa = (float*)(smem + off); off += ((size_t)E * 4 + 127) & ~(size_t)127;
    A.fb = (float*)(smem + off); off += ((size_t)E * 4 + 127) & ~(size_t)127;
    A.w = (float*)(smem + off); off += ((size_t)E * 4 + 127) & ~(size_t)127;
    A.sh = (float*)(smem + off); off += ((size_t)P.max_seq * 4 + 127) & ~(size_t)127;
    A.q = (float*)(smem + off); off += (size_t)HD * 4;
    A.kn = (float*)(smem + off); off += (size_t)HD * 4;
    off = (off + 127) & ~(size_t)127;
    // the layer descriptors, copied once: the producer thread walks them far ahead of the consumers and
    // must not pay a memory round trip per pointer
    lt_decode_layer* lys = (lt_decode_layer*)(smem + off);
    A.big = smem + fixed_bytes;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int G = (int)gridDim.x, NG = G - P.nh;
    const bool att = (int)blockIdx.x < P.nh;
    const int g = (int)blockIdx.x - P.nh;               // index among the GEMV CTAs
    if (tid == 0) {
        for (int s = 0; s < DEC_MAX_STAGES; s++) {
            mbar_init(&S->full[s], 1);
            mbar_init(&S->empty[s], DEC_CWARPS);
        }
        for (int p = 0; p < 4; p++) {
            mbar_init(&S->sfull[p], 1);
            mbar_init(&S->sempty[p], DEC_CWARPS);
        }
        mbar_init(&S->wfull, 1);
        mbar_init(&S->wempty, DEC_CWARPS);
        mbar_init(&S->att_done, 1);
        S->abort_flag = 0;
        S->nrep = (P.poll_looks >= 1 && P.poll_looks <= DEC_NREP) ? P.poll_looks : DEC_NREP;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    {
        constexpr int LY_WORDS = (int)(sizeof(lt_decode_layer) / 8);
        for (int i = tid; i < L * LY_WORDS; i += DEC_THREADS)
            ((unsigned long long*)lys)[i] = __ldg((const unsigned long long*)P.layers + i);
    }
    __syncthreads();

    // this CTA's share of every matrix
    int v0 = 0, v1 = 0, e0 = 0, e1 = 0, b0 = 0, b1 = 0;
    if (!att) {
        v0 = (int)(((long long)nk * g) / NG); v1 = (int)(((long long)nk * (g + 1)) / NG);
        e0 = (int)(((long long)E * g) / NG); e1 = (int)(((long long)E * (g + 1)) / NG);
        b0 = (int)(((long long)(F >> 5) * g) / NG); b1 = (int)(((long long)(F >> 5) * (g + 1)) / NG);
    }

    // ------------------------------------------------------------ producer warp
    if (warp == DEC_CWARPS) {
        if (lane != 0) return;
        // this CTA's rows of the LM head and the ring they stream through
        const int l0 = (int)(((long long)P.V * blockIdx.x) / G), l1 = (int)(((long long)P.V * (blockIdx.x + 1)) / G);
        Ring R;
        R.base = A.big; R.full = S->full; R.empty = S->empty; R.stage = 0; R.fill = 0;
        R.nstages = att ? nstages_att : nstages;

        bool ok = true;
        if (att) {
            const int h = blockIdx.x, hk = h / (P.nh / P.nkv);
            const unsigned qb = (unsigned)HD * E, db = (unsigned)HD * nbE * 2;
            int armed = -1;         // last layer whose resident rows were requested
            for (int il = 0; il < L && ok; il++) {
                const lt_decode_layer* ly = lys + il;
                if (il > 0) ok = mbar_wait(&S->wempty, (unsigned)(il - 1) & 1u, S, P.status);
                if (!ok) break;
                armed = il;
                mbar_expect_tx(&S->wfull, 2 * (qb + db));
                const unsigned long long pol = l2_policy_evict_first();
                bulk_g2s_hint(A.big, ly->qkv_q + (size_t)h * HD * E, qb, &S->wfull, pol);
                bulk_g2s_hint(A.big + qb, ly->qkv_q + ((size_t)nq + (size_t)hk * HD) * E, qb, &S->wfull, pol);
                bulk_g2s_hint(A.big + 2 * (size_t)qb, (const __half*)ly->qkv_d + (size_t)h * HD * nbE, db, &S->wfull, pol);
                bulk_g2s_hint(A.big + 2 * (size_t)qb + db, (const __half*)ly->qkv_d + ((size_t)nq + (size_t)hk * HD) * nbE, db,
                              &S->wfull, pol);
            }
            if (ok) ok = mbar_wait(&S->att_done, 0u, S, P.status);
            if ((!ok || S->abort_flag) && armed >= 0) {     // gave up: let the requested rows land before the CTA exits
                const long long t0 = clock64();
                while (!mbar_try_wait(&S->wfull, (unsigned)armed & 1u))
                    if (clock64() - t0 > DEC_DRAIN_CLOCKS) break;
            }
            if (ok) ok = produce_segment(R, P.lm_q, (const __half*)P.lm_d, l0, l1, E, rows_per_chunk_lm(E), S, P.status);
        } else {
            // the slots: the v slice of layer il is requested as soon as that of layer il - 1 has been folded; the
            // others (o_proj, gate|up, down) wait until phase 0 of layer il has been folded as well, i.e. until the
            // GEMV CTAs start waiting for the attention CTAs: requested right after their own fold, all CTAs'
            // refills (18 MB) would travel through L2 exactly while x1, silu(gate)*up and x are handed over
            int armed[4] = {-1, -1, -1, -1};
            const int nrows[4] = {v1 - v0, e1 - e0, b1 - b0, e1 - e0};
            for (int il = 0; il < L && ok; il++) {
                const lt_decode_layer* ly = lys + il;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if (nrows[p] <= 0 || !ok) continue;
                    if (il > 0) ok = mbar_wait(&S->sempty[p], (unsigned)(il - 1) & 1u, S, P.status);
                    if (ok && il > 0 && p >= 1) ok = mbar_wait(&S->sempty[0], (unsigned)il & 1u, S, P.status);
                    if (!ok) continue;
                    unsigned char* dst = A.big + SL.off[p];
                    armed[p] = il;
                    if (p == 0) {
                        const __half* Wd = (const __half*)ly->qkv_d;
                        mbar_expect_tx(&S->sfull[0], slot_bytes(Wd, nq + nk + v0, v1 - v0, E));
                        slot_request(dst, ly->qkv_q, Wd, nq + nk + v0, v1 - v0, E, &S->sfull[0]);
                    } else if (p == 1) {
                        const __half* Wd = (const __half*)ly->o_d;
                        mbar_expect_tx(&S->sfull[1], slot_bytes(Wd, e0, e1 - e0, nq));
                        slot_request(dst, ly->o_q, Wd, e0, e1 - e0, nq, &S->sfull[1]);
                    } else if (p == 2) {
                        const __half* Wd = (const __half*)ly->gu_d;
                        unsigned total = 0;
                        for (int b = b0; b < b1; b++) total += slot_bytes(Wd, b * 32, 32, E) + slot_bytes(Wd, F + b * 32, 32, E);
                        mbar_expect_tx(&S->sfull[2], total);
                        for (int b = b0; b < b1; b++) {
                            slot_request(dst + (size_t)(2 * (b - b0)) * SL.chunk, ly->gu_q, Wd, b * 32, 32, E, &S->sfull[2]);
                            slot_request(dst + (size_t)(2 * (b - b0) + 1) * SL.chunk, ly->gu_q, Wd, F + b * 32, 32, E, &S->sfull[2]);
                        }
                    } else {
                        const __half* Wd = (const __half*)ly->down_d;
                        mbar_expect_tx(&S->sfull[3], slot_bytes(Wd, e0, e1 - e0, F));
                        slot_request(dst, ly->down_q, Wd, e0, e1 - e0, F, &S->sfull[3]);
                    }
                }
            }
            // the LM-head ring lies over the slots: its stages below the down slot may be requested once the
            // last layer's v, o_proj and gate|up slices have been folded, the others after its down slice
#pragma unroll
            for (int p = 0; p < 3; p++)
                if (ok && nrows[p] > 0) ok = mbar_wait(&S->sempty[p], (unsigned)(L - 1) & 1u, S, P.status);
            if (ok)
                ok = produce_segment(R, P.lm_q, (const __half*)P.lm_d, l0, l1, E, rows_per_chunk_lm(E), S, P.status,
                                     nrows[3] > 0 ? &S->sempty[3] : nullptr, (unsigned)(L - 1) & 1u, SL.off[3] / DEC_STAGE_STRIDE);
            if (!ok || S->abort_flag) {       // gave up: let the requested slices land before the CTA exits
                const long long t0 = clock64();
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if (armed[p] < 0) continue;
                    while (!mbar_try_wait(&S->sfull[p], (unsigned)armed[p] & 1u))
                        if (clock64() - t0 > DEC_DRAIN_CLOCKS) break;
                }
            }
        }
        if (!ok || S->abort_flag) producer_drain(R);
        return;
    }

    // ------------------------------------------------------------ consumers
    Tracer tr;
    tr.init(P);
    tr.stamp(1);
    const unsigned backoff = (unsigned)P.poll_ns;
    // tags of this step: token counter * (L+2) + layer + 1 (never 0 = "never written"); the argmax partials use tag0 + L
    const unsigned tag0 = __ldcg(P.epoch) * (unsigned)(L + 2) + 1u;
    for (int l = tid; l < L; l += DEC_CTHREADS) S->lens[l] = __ldcg(lys[l].len);
    // x of layer 0: gathered from the Q8_0 table by the device token, or preloaded by the host
    if (P.tok != nullptr) {
        int t = __ldcg(P.tok);
        if (t < 0 || t >= P.V) {
            if (tid == 0 && blockIdx.x == 0) atomicOr(P.status, (int)LT_STATUS_BAD_TOKEN);
            t = t < 0 ? 0 : P.V - 1;
        }
        for (int j = tid; j < E; j += DEC_CTHREADS)
            A.fa[j] = __fmul_rn(__half2float(((const __half*)P.emb_d)[(size_t)t * nbE + (j >> 5)]), (float)P.emb_q[(size_t)t * E + j]);
    } else {
        for (int j = tid; j < E; j += DEC_CTHREADS) A.fa[j] = __ldcg(P.x + j);
    }
    consumer_sync();

    // ---- attention CTAs: their own loop over the layers
    if (att) {
        for (int il = 0; il < L; il++) attention_layer<HD>(P, lys + il, il, tag0, A, vcap, S, tr);
        if (tid == 0) mbar_arrive(&S->att_done);        // every warp is past the last layer's final barrier
        for (int j = tid; j < E; j += DEC_CTHREADS) A.w[j] = __ldg(P.out_norm + j);
    } else {
        for (int j = tid; j < E; j += DEC_CTHREADS) A.w[j] = __ldg(lys[0].attn_norm + j);
    }

    // ---- GEMV CTAs: four weight phases per layer.  Phase p of layer il:
    //   0  x  -> RMSNorm -> quantiser -> this CTA's v rows             (x of layer il: tag of layer il - 1)
    //   1  quantised attention output -> o_proj + x -> x1
    //   2  x1 -> RMSNorm -> quantiser -> gate|up blocks -> quantised silu(gate)*up
    //   3  quantised FFN activation -> down + x1 -> x of the next layer
    EpiCtx C;
    C.tr = tr; C.P = &P; C.S = S; C.nq = nq; C.nk = nk; C.bestv = -3.4e38f; C.besti = 2147483647;
    C.resid = A.fa; C.tag = 0; C.pos = 0; C.room = 0; C.ly = lys;
    if (!att) {
        // what a phase needs of its slot does not depend on the layer (the launcher checks that a matrix kind's
        // scale arrays are aligned alike in every layer): computed once
        if (tid == 0) {
            GemvConst GC;
            GC.big = smem_u32(A.big);
            GC.v0 = v0; GC.nv = v1 - v0; GC.e0 = e0; GC.ne = e1 - e0; GC.b0 = b0; GC.nbk = b1 - b0;
            GC.db[0] = (unsigned)((v1 - v0) * E) + (unsigned)(reinterpret_cast<uintptr_t>((const __half*)lys[0].qkv_d + (size_t)(nq + nk + v0) * nbE) & 15);
            GC.db[1] = (unsigned)((e1 - e0) * nq) + (unsigned)(reinterpret_cast<uintptr_t>((const __half*)lys[0].o_d + (size_t)e0 * (nq >> 5)) & 15);
            GC.db[2] = (unsigned)(reinterpret_cast<uintptr_t>(lys[0].gu_d) & 15);
            GC.db[3] = (unsigned)((e1 - e0) * F) + (unsigned)(reinterpret_cast<uintptr_t>((const __half*)lys[0].down_d + (size_t)e0 * (F >> 5)) & 15);
            S->gc = GC;
        }
        consumer_sync();
        for (int idx = 0; idx < 4 * L; idx++) gemv_phase(idx & 3, P, lys, idx >> 2, L, tag0, SL, A, S, C);
    }

    // ---- the LM head, every CTA: final x -> RMSNorm (output norm) -> quantiser -> this CTA's rows of the
    // LM-head matrix, streamed through the ring, with the running argmax
    {
        const int l0 = (int)(((long long)P.V * blockIdx.x) / G), l1 = (int)(((long long)P.V * (blockIdx.x + 1)) / G);
        Ring R;
        R.base = A.big; R.full = S->full; R.empty = S->empty; R.stage = 0; R.fill = 0;
        R.nstages = att ? nstages_att : nstages;
        const unsigned tag = tag0 + (unsigned)L;
        C.ly = lys + (L - 1); C.tag = tag;
        const __half* Wd = (const __half*)P.lm_d;
        const int RC = rows_per_chunk_lm(E);
        // the full sets take their plan from the memo from the second set on
        const int full_lm = DEC_CWARPS * DEC_ILP;
        const bool lm_memo = l1 - l0 >= full_lm && 2 * RC == full_lm && (RC * nbE * 2) % 16 == 0;
        SegPlan sp = seg_prepare(EPI_LOGITS, R, Wd, l0, l0, l1, E, RC, C, S->memo[warp], lm_memo ? 1 : 0);
        C.tr.stamp(20);
        fetch_x((const float2*)P.ws_x, tag - 1u, false, A.fa, E, S, P.status, backoff);
        consumer_sync();
        C.tr.stamp(21);
        norm_quant(A.fa, A.w, E, P.eps, A.xq0, A.xd0, S);
        consumer_sync();
        for (;;) {
            seg_finish(EPI_LOGITS, sp, R, E, A.xq0, A.xd0, C);
            const int r = sp.r + sp.nset;
            if (r >= l1) break;
            sp = seg_prepare(EPI_LOGITS, R, Wd, l0, r, l1, E, RC, C, S->memo[warp], (lm_memo && l1 - r >= full_lm) ? 2 : 0);
        }
        C.tr.stamp(25);
    }
    C.tr.stamp(32);
    float bestv = C.bestv;
    int besti = C.besti;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bestv, s);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, s);
        if (ov > bestv || (ov == bestv && oi < besti)) { bestv = ov; besti = oi; }
    }
    if (lane == 0) { S->best_v[warp] = bestv; S->best_i[warp] = besti; }
    consumer_sync();
    const unsigned ptag = tag0 + (unsigned)L;
    if (tid == 0) {
        float bv = S->best_v[0];
        int bi = S->best_i[0];
        for (int w = 1; w < DEC_CWARPS; w++) {
            const float v = S->best_v[w];
            const int i = S->best_i[w];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        st_tagged((float2*)P.ws_part + 2 * blockIdx.x, bv, ptag);
        st_tagged_u32((float2*)P.ws_part + 2 * blockIdx.x + 1, (unsigned)bi, ptag);
    }
    // the last CTA collects the partial results of all CTAs and ends the step
    if ((int)blockIdx.x == G - 1 && warp == 0) {
        float bv = -3.4e38f;
        int bi = 2147483647;
        for (int c = lane; c < G; c += 32) {
            float pv = -3.4e38f, pi = __uint_as_float(2147483647u);
            poll_words((const float2*)P.ws_part, 2 * G, 2 * c, 1, 2, ptag, [&](int k, float x) { if (k == 0) pv = x; else pi = x; }, S,
                       P.status, backoff);
            const float v = pv;
            const int i = (int)__float_as_uint(pi);
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        // every CTA has delivered its result, so every CTA has read the token, the lengths and the
        // token counter of this step: they may advance now
        for (int l = lane; l < L; l += 32) {
            int* lp = lys[l].len;
            const int p = __ldcg(lp);
            if (p >= 0 && p < P.max_seq) *lp = p + 1;
        }
        if (lane == 0) {
            *P.out_tok = bi;
            if (P.tok != nullptr) *P.tok = bi;
            if (P.history != nullptr) {
                const int s = *P.step;
                if (s >= 0 && s < P.hist_cap) P.history[s] = bi;
                *P.step = s + 1;
            }
            *P.epoch = *P.epoch + 1u;
        }
    }
    C.tr.stamp(99);
}

struct DecodeGeometry {
    DecSlots slots;
    int nstages, nstages_att, vcap, fixed_bytes;
    size_t smem;
    int ctas;
};

static size_t up128(size_t v) { return (v + 127) & ~(size_t)127; }

static int decode_geometry(const lt_decode_desc* d, DecodeGeometry* g) {
    int dev = 0, sms = 0, smem_max = 0;
    LT_CUDA(cudaGetDevice(&dev));
    LT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    LT_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const int E = d->E, F = d->F, hd = d->hd, nq = d->nh * hd;
    const int kmax1 = nq > F ? nq : F;
    size_t fixed = up128(sizeof(Shared)) + up128(E) + up128((size_t)(E >> 5) * 2) + up128(kmax1) +
                   up128((size_t)(kmax1 >> 5) * 2) + 3 * up128((size_t)E * 4) + up128((size_t)d->max_seq * 4) +
                   (size_t)2 * hd * 4;
    fixed = up128(fixed) + up128((size_t)d->n_layers * sizeof(lt_decode_layer));
    const size_t avail = (size_t)smem_max - 256;
    // attention CTA: the head's q rows and its group's k rows (quants, then scales), then staged V rows
    const size_t wreg = (size_t)2 * hd * (E + (E >> 5) * 2);
    if (fixed + wreg + (size_t)hd * 4 > avail || fixed + 2 * (size_t)DEC_STAGE_STRIDE > avail) {
        set_error("lt_decode_step: model dimensions need more shared memory than one SM has "
                  "(2*hd rows of q|k|v must stay resident: hd=%d, E=%d)", hd, E);
        return LT_ERR_UNSUPPORTED;
    }
    size_t vrows = (avail - fixed - wreg) / ((size_t)hd * 4);
    if (vrows > (size_t)d->max_seq) vrows = (size_t)d->max_seq;
    g->vcap = (int)vrows;
    int nst = (int)((avail - fixed) / DEC_STAGE_STRIDE);
    if (nst > DEC_MAX_STAGES) nst = DEC_MAX_STAGES;
    g->nstages = nst;
    if (nst < DEC_MAXCH) {
        set_error("lt_decode_step: shared memory leaves only %d ring stages (needs %d)", nst, DEC_MAXCH);
        return LT_ERR_UNSUPPORTED;
    }
    // the LM-head ring of an attention CTA lives in its big area once the layers are done
    const size_t big_att = wreg + vrows * (size_t)hd * 4;
    int nsa = (int)(big_att / DEC_STAGE_STRIDE);
    if (nsa > DEC_MAX_STAGES) nsa = DEC_MAX_STAGES;
    size_t big = (size_t)nst * DEC_STAGE_STRIDE;
    if (nsa < 2) {          // tiny models: make room for two stages
        nsa = 2;
        if (big < 2 * (size_t)DEC_STAGE_STRIDE) big = 2 * (size_t)DEC_STAGE_STRIDE;
    }
    if (big_att > big) big = big_att;
    // GEMV CTA: the slots of the four layer phases, sized for the largest share of a CTA
    {
        const int NG = sms - d->nh > 0 ? sms - d->nh : 1;
        const int nk = d->nkv * hd, nbE = E >> 5;
        const size_t mV = (size_t)(nk + NG - 1) / NG, mE = (size_t)(E + NG - 1) / NG, mB = (size_t)((F >> 5) + NG - 1) / NG;
        const size_t chunk = up128((size_t)32 * E + (size_t)32 * nbE * 2 + 32);
        const size_t sz[4] = {up128(mV * E + mV * nbE * 2 + 32), up128(mE * nq + mE * (nq >> 5) * 2 + 32), mB * 2 * chunk,
                              up128(mE * F + mE * (F >> 5) * 2 + 32)};
        size_t o = 0;
        for (int p = 0; p < 4; p++) { g->slots.off[p] = (int)o; o += sz[p]; }
        g->slots.chunk = (int)chunk;
        if (fixed + o > avail) {
            set_error("lt_decode_step: a CTA's share of one layer (%zu bytes) does not fit shared memory beside %zu fixed bytes",
                      o, fixed);
            return LT_ERR_UNSUPPORTED;
        }
        if (o > big) big = o;
    }
    g->nstages_att = nsa;
    g->fixed_bytes = (int)fixed;
    g->smem = fixed + big;
    g->ctas = sms;
    if (g->smem > (size_t)smem_max) {
        set_error("lt_decode_step: shared-memory plan exceeds the SM (%zu > %d)", g->smem, smem_max);
        return LT_ERR_UNSUPPORTED;
    }
    return LT_OK;
}

static int decode_check(const lt_decode_desc* d, DecodeGeometry* g) {
    LT_REQUIRE(d != nullptr, "lt_decode_step: null descriptor");
    LT_REQUIRE(d->layers && d->h_layers && d->out_norm && d->lm_q && d->lm_d && d->logits && d->out_tok && d->epoch &&
                   d->ws_part && d->ws_x && d->ws_x1 && d->ws_qkv && d->ws_att && d->ws_v,
               "lt_decode_step: null pointer in descriptor");
    LT_REQUIRE(d->tok != nullptr ? (d->emb_q && d->emb_d) : (d->x != nullptr),
               "lt_decode_step: needs either a device token with the embedding table or a preloaded input row");
    LT_REQUIRE(d->n_layers > 0 && d->n_layers <= DEC_MAX_LAYERS && d->E > 0 && d->F > 0 && d->V > 0 && d->max_seq > 0,
               "lt_decode_step: bad dimensions");
    LT_REQUIRE(d->poll_ns >= 0 && d->poll_ns <= 100000, "lt_decode_step: poll_ns=%d out of range", d->poll_ns);
    LT_REQUIRE(d->poll_looks >= 0 && d->poll_looks <= DEC_NREP, "lt_decode_step: %d workspace copies out of range (0..%d)", d->poll_looks, DEC_NREP);
    const int nq = d->nh * d->hd, nk = d->nkv * d->hd;
    if (!(d->hd == 32 || d->hd == 64)) {
        set_error("lt_decode_step: hd=%d (this kernel keeps a cached K row in registers: hd 32 or 64)", d->hd);
        return LT_ERR_UNSUPPORTED;
    }
    const int fmax = DEC_CTHREADS * DEC_VB * 32 / 9 / 32 * 32, qmax = DEC_CTHREADS * DEC_AB * 32 / 9 / 32 * 32;
    // a 32-row block of gate|up must fit one ring stage
    const int emax = DEC_STAGE_BYTES / 34 / 32 * 32 < 256 * DEC_XB ? DEC_STAGE_BYTES / 34 / 32 * 32 : 256 * DEC_XB;
    if (!(d->E % 32 == 0 && d->F % 32 == 0 && d->E <= emax && d->F <= fmax && nq <= qmax &&
          d->F + d->F / 16 <= DEC_STAGE_BYTES)) {
        set_error("lt_decode_step: this kernel handles E <= %d, F <= %d, nh*hd <= %d (multiples of 32); got E=%d F=%d nh*hd=%d",
                  emax, fmax, qmax, d->E, d->F, nq);
        return LT_ERR_UNSUPPORTED;
    }
    LT_REQUIRE(d->nkv > 0 && d->nh % d->nkv == 0, "lt_decode_step: nh must be a multiple of nkv");
    // scale rows are fetched in 16-byte windows: every matrix must hold a multiple of 8 scales so that no
    // window crosses the end of its array; the resident q|k rows need 16-byte aligned scale rows
    const long long ms[5] = {(long long)(nq + 2 * nk) * (d->E / 32), (long long)d->E * (nq / 32),
                             (long long)2 * d->F * (d->E / 32), (long long)d->E * (d->F / 32),
                             (long long)d->V * (d->E / 32)};
    for (int i = 0; i < 5; i++)
        LT_REQUIRE(ms[i] % 8 == 0, "lt_decode_step: a weight matrix has %lld scales, not a multiple of 8", ms[i]);
    LT_REQUIRE(((long long)d->hd * (d->E / 32) * 2) % 16 == 0, "lt_decode_step: hd*E/32 scales of a head must fill whole 16-byte units");
    for (int il = 0; il < d->n_layers; il++) {
        const lt_decode_layer* ly = d->h_layers + il;
        LT_REQUIRE(ly->attn_norm && ly->qkv_q && ly->qkv_d && ly->o_q && ly->o_d && ly->ffn_norm && ly->gu_q && ly->gu_d &&
                       ly->down_q && ly->down_d && ly->kcache && ly->vcache && ly->len,
                   "lt_decode_step: null pointer in layer %d", il);
        LT_REQUIRE(aligned16(ly->qkv_q) && aligned16(ly->qkv_d) && aligned16(ly->o_q) && aligned16(ly->gu_q) &&
                       aligned16(ly->down_q) && aligned16(ly->kcache) && aligned16(ly->vcache),
                   "lt_decode_step: weights and caches of layer %d must be 16-byte aligned", il);
    }
    LT_REQUIRE(aligned16(d->lm_q), "lt_decode_step: the LM-head matrix must be 16-byte aligned");
    for (int il = 1; il < d->n_layers; il++) {
        const lt_decode_layer *a = d->h_layers, *b = d->h_layers + il;
        // (the kernel works out once, from the first layer, where the scale rows of a slice lie in its slot)
        LT_REQUIRE(((uintptr_t)a->qkv_d & 15) == ((uintptr_t)b->qkv_d & 15) && ((uintptr_t)a->o_d & 15) == ((uintptr_t)b->o_d & 15) &&
                       ((uintptr_t)a->down_d & 15) == ((uintptr_t)b->down_d & 15) && ((uintptr_t)a->gu_d & 15) == ((uintptr_t)b->gu_d & 15) &&
                       (a->qkv_bias == nullptr) == (b->qkv_bias == nullptr),
                   "lt_decode_step: the scale arrays of layer %d are aligned differently from layer 0's", il);
    }
    int rc = decode_geometry(d, g);
    if (rc != LT_OK) return rc;
    if (d->nh + 1 > g->ctas || nk > 64 * (g->ctas - d->nh)) {
        set_error("lt_decode_step: %d query heads / %d v rows are too many for %d SMs", d->nh, nk, g->ctas);
        return LT_ERR_UNSUPPORTED;
    }
    return LT_OK;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_decode_step_supported(const lt_decode_desc* d) {
    DecodeGeometry g;
    return decode_check(d, &g) == LT_OK ? 1 : 0;
}

extern "C" int lt_decode_step(const lt_decode_desc* d, void* stream) {
    DecodeGeometry g;
    int rc = decode_check(d, &g);
    if (rc != LT_OK) return rc;
    lt_decode_desc P = *d;
    if (P.status == nullptr) P.status = device_status_ptr();
    LT_REQUIRE(P.status != nullptr, "lt_decode_step: status word unavailable");
    int nstages = g.nstages, nsa = g.nstages_att, vcap = g.vcap, fixed = g.fixed_bytes;
    DecSlots slots = g.slots;
    void* args[] = {&P, &nstages, &nsa, &vcap, &fixed, &slots};
    const void* kern = d->hd == 32 ? (const void*)k_decode_step<32> : (const void*)k_decode_step<64>;
    LT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
    // cooperative launch: all CTAs are resident together, which the data-flow waits rely on
    LT_CUDA(cudaLaunchCooperativeKernel(kern, dim3(g.ctas), dim3(DEC_THREADS), args, g.smem, (cudaStream_t)stream));
    count_launches(1);
    return LT_OK;
}

extern "C" int lt_decode_ws_replicas(void) { return DEC_NREP; }

extern "C" int lt_decode_num_ctas(void) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}
