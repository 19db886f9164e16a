// Device-side view of an lt_comm (one-shot exchange over peer stores) shared by the all-reduce kernel and by
// the GEMV that pushes its partial rows itself.
//
// Protocol.  Every rank owns a staging buffer [2 users][2][world][max_n] of 8-byte words {fp32 value, u32 tag}
// that its peers map through CUDA IPC.  An exchange of element i has a number, counted in device memory on
// every rank alike (the same sequence of calls runs on every rank; a captured graph's launch arguments never
// change): the writer stores {value, number} into slot [number & 1][its rank][i] of EVERY rank's buffer, the
// reader polls slot [number & 1][r][i] of its OWN buffer until the tag equals the number.  Data and "arrived"
// travel in one aligned 8-byte store: no fence, no flag.  A rank can be at most one exchange ahead of its
// slowest peer (finishing exchange k needs every peer's words of exchange k, which a peer sends only after it
// has left exchange k-1), so two slots by parity suffice.  The counters belong to whoever owns the element for
// good: the all-reduce kernel counts per CTA (CTA c always owns elements 1024c ..), the GEMV with the
// all-reduce epilogue counts per row (its grid depends on the matrix); the two users have separate halves of
// the buffer.  Waits are bounded (LT_STATUS_WAIT_TIMEOUT).  One process per GPU: the kernels of different
// ranks wait on each other and must never share a GPU.
#pragma once
#include "lt_common.cuh"

namespace lt {

constexpr long long COMM_WAIT_LIMIT = 2000000000LL;   // SM clocks (about a second) before a wait gives up

constexpr int COMM_USER_ALLREDUCE = 0, COMM_USER_GEMV = 1;

struct CommDev {
    float2* stage[LT_COMM_MAX_RANKS];    // stage[r]: rank r's staging buffer as mapped here
    unsigned* ctr;                       // exchanges completed: [max_ctas] per all-reduce CTA, then [max_n] per GEMV row
    int rank, world, max_n, max_ctas;
};

inline CommDev comm_dev(const lt_comm* c) {
    CommDev C;
    for (int r = 0; r < LT_COMM_MAX_RANKS; r++) C.stage[r] = (float2*)c->stage[r];
    C.ctr = c->ctr; C.rank = c->rank; C.world = c->world; C.max_n = c->max_n; C.max_ctas = c->max_ctas;
    return C;
}

__device__ __forceinline__ float2 ld_volatile_f2(const float2* p) {
    float2 v;
    asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_volatile_f4(const float2* p) {      // two neighbouring words, 16-byte aligned
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ long comm_slot(const CommDev& C, int user, unsigned number, int src, long i) {
    return (((long)user * 2 + (long)(number & 1u)) * C.world + src) * C.max_n + i;
}

// value i of rank `src` in exchange `number`, from this rank's own staging memory; false after a timeout
__device__ __forceinline__ bool comm_take(const CommDev& C, int user, unsigned number, int src, long i, long long t0,
                                          int* status, float& v) {
    const float2* p = C.stage[C.rank] + comm_slot(C, user, number, src, i);
    float2 w = ld_volatile_f2(p);
    while (__float_as_uint(w.y) != number) {
        if (clock64() - t0 > COMM_WAIT_LIMIT) {
            atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
            return false;
        }
        w = ld_volatile_f2(p);
    }
    v = w.x;
    return true;
}

// store value i of this rank for exchange `number` into every rank's staging memory
__device__ __forceinline__ void comm_push(const CommDev& C, int user, unsigned number, long i, float v) {
    const long slot = comm_slot(C, user, number, C.rank, i);
    const float2 w = make_float2(v, __uint_as_float(number));
    for (int r = 0; r < C.world; r++) C.stage[r][slot] = w;
}

}  // namespace lt
