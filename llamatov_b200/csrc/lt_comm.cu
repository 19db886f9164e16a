// One-shot all-reduce (sum) of a small fp32 vector over the GPUs of one node, fused with the
// residual add that follows it in the tensor-parallel decode step:
//     out = resid + ((part_0 + part_1) + part_2 + ... )          (rank order, the same bits on every rank)
// One kernel per rank: a thread pushes its four elements of the local partial into every rank's staging
// memory (plain peer stores over NVLink), then takes the elements of all ranks from its own memory and folds
// them in rank order.  No data crosses NVLink twice, nothing is read from a peer, no multicast object is
// involved.  The exchange protocol is in lt_comm.cuh.
#include <string.h>

#include "lt_comm.cuh"

namespace lt {

constexpr int LT_ALLREDUCE_TWO_STAGE_MIN = 32768;   // elements
constexpr int COMM_THREADS = 256;
constexpr int COMM_CHUNK = COMM_THREADS * 4;        // floats per CTA

// TREE: the partials are summed pairwise, p[t] + p[t + s] for s = world/2 .. 1 (world a power of two): the last
// levels of the GEMV contract's lane tree when the ranks hold lane subsets (lt_q8_gemv_lanes); otherwise in
// rank order.
template <bool TREE>
__global__ void __launch_bounds__(COMM_THREADS)
k_allreduce_add(const CommDev C, const float* __restrict__ part, const float* __restrict__ resid,
                float* __restrict__ out, int n, int* status) {
    chain_release();
    chain_wait();
    __shared__ unsigned s_number;
    const int tid = threadIdx.x;
    if (tid == 0) s_number = C.ctr[blockIdx.x] + 1u;
    __syncthreads();
    const unsigned number = s_number;
    constexpr int U = COMM_USER_ALLREDUCE;
    const int i = blockIdx.x * COMM_CHUNK + tid * 4;
    if (i < n) {
        const float4 v = *(const float4*)(part + i);
        {   // four tagged words as two 16-byte stores per rank (each 8-byte word still carries its own tag)
            const long slot = comm_slot(C, U, number, C.rank, i);
            const float tg = __uint_as_float(number);
            const float4 w0 = make_float4(v.x, tg, v.y, tg), w1 = make_float4(v.z, tg, v.w, tg);
            for (int r = 0; r < C.world; r++) {
                float4* d = (float4*)(C.stage[r] + slot);
                d[0] = w0;
                d[1] = w1;
            }
        }
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float p[TREE ? LT_COMM_MAX_RANKS : 1][4];
        bool ok = true;
        const long long t0 = clock64();
#pragma unroll
        for (int r = 0; r < LT_COMM_MAX_RANKS; r++) {
            if (r < C.world && ok) {
                const float2* src = C.stage[C.rank] + comm_slot(C, U, number, r, i);
#pragma unroll
                for (int e = 0; e < 4; e += 2) {      // two words per 16-byte load, both tags checked
                    float4 w = ld_volatile_f4(src + e);
                    while (__float_as_uint(w.y) != number || __float_as_uint(w.w) != number) {
                        if (clock64() - t0 > COMM_WAIT_LIMIT) {
                            atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
                            ok = false;
                            break;
                        }
                        w = ld_volatile_f4(src + e);
                    }
                    if (TREE) {
                        p[TREE ? r : 0][e] = w.x; p[TREE ? r : 0][e + 1] = w.z;
                    } else {
                        a[e] = r == 0 ? w.x : __fadd_rn(a[e], w.x);
                        a[e + 1] = r == 0 ? w.z : __fadd_rn(a[e + 1], w.z);
                    }
                }
            } else if (TREE) {
#pragma unroll
                for (int e = 0; e < 4; e++) p[TREE ? r : 0][e] = 0.0f;
            }
        }
        if (TREE) {
#pragma unroll
            for (int s = LT_COMM_MAX_RANKS / 2; s > 0; s >>= 1) {
                if (s < C.world) {
#pragma unroll
                    for (int t = 0; t < s; t++)
#pragma unroll
                        for (int e = 0; e < 4; e++) p[TREE ? t : 0][e] = __fadd_rn(p[TREE ? t : 0][e], p[TREE ? t + s : 0][e]);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; e++) a[e] = p[0][e];
        }
        if (ok) {
            float4 y = make_float4(a[0], a[1], a[2], a[3]);
            if (resid != nullptr) {
                const float4 x = *(const float4*)(resid + i);
                y.x = __fadd_rn(x.x, y.x); y.y = __fadd_rn(x.y, y.y); y.z = __fadd_rn(x.z, y.z); y.w = __fadd_rn(x.w, y.w);
            }
            *(float4*)(out + i) = y;
        }
    }
    __syncthreads();
    if (tid == 0) C.ctr[blockIdx.x] = number;
}

// Two-stage form for long vectors on four or more ranks: the one-shot form stores world * n words per rank,
// this one 2 * n.  CTA c's 1024 elements are OWNED by rank c % world: every rank stores its partial of the
// chunk into the owner's staging memory only (slot [its rank]); the owner folds all ranks' partials in rank
// order, adds the residual, writes its own output and stores the finished words into the other ranks'
// staging memory (slot [owner], which stage one leaves unused there); the others take them from their own
// memory.  Same additions in the same order as the one-shot form: the same bits on every rank.
__global__ void __launch_bounds__(COMM_THREADS)
k_allreduce_add_2stage(const CommDev C, const float* __restrict__ part, const float* __restrict__ resid,
                       float* __restrict__ out, int n, int* status) {
    chain_release();
    chain_wait();
    __shared__ unsigned s_number;
    const int tid = threadIdx.x;
    if (tid == 0) s_number = C.ctr[blockIdx.x] + 1u;
    __syncthreads();
    const unsigned number = s_number;
    constexpr int U = COMM_USER_ALLREDUCE;
    const int i = blockIdx.x * COMM_CHUNK + tid * 4;
    const int owner = (int)(blockIdx.x % (unsigned)C.world);
    if (i < n) {
        const float tg = __uint_as_float(number);
        const long long t0 = clock64();
        bool ok = true;
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float4 v = *(const float4*)(part + i);
        if (C.rank != owner) {
            float4* d = (float4*)(C.stage[owner] + comm_slot(C, U, number, C.rank, i));
            d[0] = make_float4(v.x, tg, v.y, tg);
            d[1] = make_float4(v.z, tg, v.w, tg);
            // the finished words arrive in this rank's memory, slot [owner]
            const float2* src = C.stage[C.rank] + comm_slot(C, U, number, owner, i);
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                float4 w = ld_volatile_f4(src + e);
                while (__float_as_uint(w.y) != number || __float_as_uint(w.w) != number) {
                    if (clock64() - t0 > COMM_WAIT_LIMIT) {
                        atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
                        ok = false;
                        break;
                    }
                    w = ld_volatile_f4(src + e);
                }
                a[e] = w.x; a[e + 1] = w.z;
            }
        } else {
            const float mine[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int r = 0; r < LT_COMM_MAX_RANKS; r++) {
                if (r < C.world && ok) {
                    float p[4];
                    if (r == C.rank) {
#pragma unroll
                        for (int e = 0; e < 4; e++) p[e] = mine[e];
                    } else {
                        const float2* src = C.stage[C.rank] + comm_slot(C, U, number, r, i);
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            float4 w = ld_volatile_f4(src + e);
                            while (__float_as_uint(w.y) != number || __float_as_uint(w.w) != number) {
                                if (clock64() - t0 > COMM_WAIT_LIMIT) {
                                    atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
                                    ok = false;
                                    break;
                                }
                                w = ld_volatile_f4(src + e);
                            }
                            p[e] = w.x; p[e + 1] = w.z;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; e++) a[e] = r == 0 ? p[e] : __fadd_rn(a[e], p[e]);
                }
            }
            if (resid != nullptr) {
                const float4 x = *(const float4*)(resid + i);
                a[0] = __fadd_rn(x.x, a[0]); a[1] = __fadd_rn(x.y, a[1]); a[2] = __fadd_rn(x.z, a[2]); a[3] = __fadd_rn(x.w, a[3]);
            }
            if (ok) {
                const long slot = comm_slot(C, U, number, owner, i);
                const float4 w0 = make_float4(a[0], tg, a[1], tg), w1 = make_float4(a[2], tg, a[3], tg);
                for (int r = 0; r < C.world; r++) {
                    if (r == C.rank) continue;
                    float4* d = (float4*)(C.stage[r] + slot);
                    d[0] = w0;
                    d[1] = w1;
                }
            }
        }
        if (ok) *(float4*)(out + i) = make_float4(a[0], a[1], a[2], a[3]);
    }
    __syncthreads();
    if (tid == 0) C.ctr[blockIdx.x] = number;
}

// ---------------------------------------------------------------- greedy token of B rows over the ranks
// Each rank holds a vocabulary slice [v0, v0 + nv) of the logits of B sequences.  Stage 1: ARGROW_BLOCKS
// CTAs per row reduce a strided share to (max, lowest index).  Stage 2 (one CTA, a warp per row): the row's
// partials -> this rank's (max, global index); with more than one rank the pair is pushed to every rank as
// two tagged words (elements 2b, 2b+1 of the all-reduce user's CTA 0: the same counter an lt_allreduce_add
// call advances, so the exchange numbers stay in step on all ranks), every rank takes all pairs from its own
// memory and keeps the maximum, lowest index on ties: the same token on every rank, no host step.
constexpr int ARGROW_BLOCKS = 32;

struct BestR {
    float v;
    int i;
};
__device__ __forceinline__ BestR better_r(BestR a, BestR b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ BestR warp_best_r(BestR m) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        BestR o;
        o.v = __shfl_xor_sync(0xffffffffu, m.v, s);
        o.i = __shfl_xor_sync(0xffffffffu, m.i, s);
        m = better_r(m, o);
    }
    return m;
}

__global__ void __launch_bounds__(256)
k_argmax_rows_part(const float* __restrict__ x, long ld, int nv, float* __restrict__ pval, int* __restrict__ pidx) {
    chain_release();
    chain_wait();
    __shared__ float sv[8];
    __shared__ int si[8];
    const int b = blockIdx.y;
    const float* row = x + (size_t)b * ld;
    BestR m;
    m.v = -3.4e38f; m.i = 2147483647;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < nv; i += ARGROW_BLOCKS * 256) {
        BestR c;
        c.v = row[i]; c.i = i;
        m = better_r(m, c);
    }
    m = warp_best_r(m);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = m.v; si[warp] = m.i; }
    __syncthreads();
    if (warp == 0) {
        BestR r;
        r.v = lane < 8 ? sv[lane] : -3.4e38f;
        r.i = lane < 8 ? si[lane] : 2147483647;
        r = warp_best_r(r);
        if (lane == 0) { pval[b * ARGROW_BLOCKS + blockIdx.x] = r.v; pidx[b * ARGROW_BLOCKS + blockIdx.x] = r.i; }
    }
}

template <bool EXCHANGE>
__global__ void __launch_bounds__(1024)
k_argmax_rows_final(const CommDev C, const float* __restrict__ pval, const int* __restrict__ pidx, int v0, int B,
                    int* __restrict__ tok, int* status) {
    chain_release();
    chain_wait();
    __shared__ unsigned s_number;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
    if (EXCHANGE) {
        if (tid == 0) s_number = C.ctr[0] + 1u;
        __syncthreads();
    }
    const unsigned number = EXCHANGE ? s_number : 0u;
    constexpr int U = COMM_USER_ALLREDUCE;
    for (int b = warp; b < B; b += nw) {
        BestR m;
        m.v = lane < ARGROW_BLOCKS ? pval[b * ARGROW_BLOCKS + lane] : -3.4e38f;
        m.i = lane < ARGROW_BLOCKS ? pidx[b * ARGROW_BLOCKS + lane] : 2147483647;
        m = warp_best_r(m);
        if (m.i != 2147483647) m.i += v0;       // (a row without any value above the sentinel keeps the sentinel index)
        if (EXCHANGE) {
            if (lane == 0) {
                comm_push(C, U, number, 2 * b, m.v);
                comm_push(C, U, number, 2 * b + 1, __int_as_float(m.i));
            }
            BestR r;
            r.v = -3.4e38f; r.i = 2147483647;
            bool ok = true;
            if (lane < C.world) {
                const long long t0 = clock64();
                float fv = 0.0f, fi = 0.0f;
                ok = comm_take(C, U, number, lane, 2 * b, t0, status, fv) && comm_take(C, U, number, lane, 2 * b + 1, t0, status, fi);
                if (ok) { r.v = fv; r.i = __float_as_int(fi); }
            }
            r = warp_best_r(r);
            ok = __all_sync(0xffffffffu, ok);
            if (lane == 0 && ok) tok[b] = r.i;
        } else {
            if (lane == 0) tok[b] = m.i;
        }
    }
    if (EXCHANGE) {
        __syncthreads();
        if (tid == 0) C.ctr[0] = number;
    }
}

}  // namespace lt

using namespace lt;

extern "C" int lt_argmax_rows_scratch_bytes(int B) { return B > 0 ? B * ARGROW_BLOCKS * 8 : 0; }

extern "C" int lt_argmax_rows(const lt_comm* comm, const float* logits, long ld, int nv, int v0, int B, void* partials,
                              int* tok, void* stream) {
    LT_REQUIRE(logits && partials && tok, "lt_argmax_rows: null pointer");
    LT_REQUIRE(nv > 0 && B > 0 && ld >= nv && v0 >= 0, "lt_argmax_rows: nv=%d B=%d ld=%ld v0=%d", nv, B, ld, v0);
    const bool exchange = comm != nullptr && comm->world > 1;
    if (exchange)
        LT_REQUIRE(2 * B <= comm->max_n && 2 * B <= COMM_CHUNK, "lt_argmax_rows: B=%d rows need %d exchange words (max %d)",
                   B, 2 * B, comm->max_n < COMM_CHUNK ? comm->max_n : COMM_CHUNK);
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_argmax_rows: status word unavailable");
    float* pval = (float*)partials;
    int* pidx = (int*)(pval + (size_t)B * ARGROW_BLOCKS);
    cudaError_t e = launch_chained(k_argmax_rows_part, dim3(ARGROW_BLOCKS, B), dim3(256), 0, (cudaStream_t)stream, logits, ld, nv,
                                   pval, pidx);
    if (e == cudaSuccess) {
        const int threads = B >= 32 ? 1024 : 32 * B;
        CommDev C = {};
        if (exchange) {
            C = comm_dev(comm);
            e = launch_chained(k_argmax_rows_final<true>, dim3(1), dim3(threads), 0, (cudaStream_t)stream, C,
                               (const float*)pval, (const int*)pidx, v0, B, tok, st);
        } else {
            e = launch_chained(k_argmax_rows_final<false>, dim3(1), dim3(threads), 0, (cudaStream_t)stream, C,
                               (const float*)pval, (const int*)pidx, v0, B, tok, st);
        }
    }
    return check_launch("lt_argmax_rows", 2, e);
}

extern "C" int lt_comm_alloc(int world, int max_n, lt_comm* comm, unsigned char* handle) {
    LT_REQUIRE(comm && handle, "lt_comm_alloc: null pointer");
    LT_REQUIRE(world >= 1 && world <= LT_COMM_MAX_RANKS, "lt_comm_alloc: world=%d (1..%d)", world, LT_COMM_MAX_RANKS);
    LT_REQUIRE(max_n > 0 && max_n % 4 == 0, "lt_comm_alloc: max_n=%d must be a positive multiple of 4", max_n);
    memset(comm, 0, sizeof(*comm));
    comm->world = world; comm->max_n = max_n;
    comm->max_ctas = (max_n + COMM_CHUNK - 1) / COMM_CHUNK;
    const size_t sb = (size_t)2 * 2 * world * max_n * sizeof(float2);     // two users x two parities
    const size_t cb = ((size_t)comm->max_ctas + max_n) * sizeof(unsigned);
    void *s = nullptr, *c = nullptr;
    LT_CUDA(cudaMalloc(&s, sb));
    LT_CUDA(cudaMalloc(&c, cb));
    LT_CUDA(cudaMemset(s, 0, sb));          // tag 0 = never written (call counts start at 1)
    LT_CUDA(cudaMemset(c, 0, cb));
    LT_CUDA(cudaDeviceSynchronize());
    comm->local_stage = (float*)s; comm->ctr = (unsigned*)c;
    cudaIpcMemHandle_t hs;
    LT_CUDA(cudaIpcGetMemHandle(&hs, s));
    static_assert(sizeof(cudaIpcMemHandle_t) == LT_COMM_HANDLE_BYTES, "IPC handle size");
    memcpy(handle, &hs, LT_COMM_HANDLE_BYTES);
    return LT_OK;
}

extern "C" int lt_comm_connect(lt_comm* comm, int rank, const unsigned char* all_handles) {
    LT_REQUIRE(comm && all_handles && comm->local_stage, "lt_comm_connect: call lt_comm_alloc first");
    LT_REQUIRE(rank >= 0 && rank < comm->world, "lt_comm_connect: rank=%d of %d", rank, comm->world);
    comm->rank = rank;
    for (int r = 0; r < comm->world; r++) {
        if (r == rank) {
            comm->stage[r] = comm->local_stage;
            continue;
        }
        cudaIpcMemHandle_t hs;
        memcpy(&hs, all_handles + (size_t)r * LT_COMM_HANDLE_BYTES, LT_COMM_HANDLE_BYTES);
        void* s = nullptr;
        LT_CUDA(cudaIpcOpenMemHandle(&s, hs, cudaIpcMemLazyEnablePeerAccess));
        comm->stage[r] = (float*)s;
    }
    return LT_OK;
}

extern "C" int lt_comm_free(lt_comm* comm) {
    LT_REQUIRE(comm, "lt_comm_free: null pointer");
    for (int r = 0; r < comm->world; r++) {
        if (r == comm->rank) continue;
        if (comm->stage[r]) cudaIpcCloseMemHandle(comm->stage[r]);
    }
    if (comm->local_stage) cudaFree(comm->local_stage);
    if (comm->ctr) cudaFree(comm->ctr);
    memset(comm, 0, sizeof(*comm));
    return LT_OK;
}

extern "C" int lt_allreduce_add(const lt_comm* comm, const float* part, const float* resid, float* out, int n,
                                void* stream) {
    LT_REQUIRE(comm && part && out, "lt_allreduce_add: null pointer");
    LT_REQUIRE(n > 0 && n % 4 == 0 && n <= comm->max_n, "lt_allreduce_add: n=%d must be a multiple of 4, at most %d", n, comm->max_n);
    LT_REQUIRE(aligned16(part) && aligned16(out) && (resid == nullptr || aligned16(resid)),
               "lt_allreduce_add: vectors must be 16-byte aligned");
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_allreduce_add: status word unavailable");
    const CommDev C = comm_dev(comm);
    const int ctas = (n + COMM_CHUNK - 1) / COMM_CHUNK;
    // long vectors on four or more ranks: the two-stage form (2n instead of world*n words stored per rank)
    const bool two_stage = comm->world >= 4 && n >= LT_ALLREDUCE_TWO_STAGE_MIN;
    const cudaError_t e = two_stage ? launch_chained(k_allreduce_add_2stage, dim3(ctas), dim3(COMM_THREADS), 0, (cudaStream_t)stream,
                                                     C, part, resid, out, n, st)
                                    : launch_chained(k_allreduce_add<false>, dim3(ctas), dim3(COMM_THREADS), 0, (cudaStream_t)stream,
                                                     C, part, resid, out, n, st);
    return check_launch("lt_allreduce_add", 1, e);
}

extern "C" int lt_allreduce_add_tree(const lt_comm* comm, const float* part, const float* resid, float* out, int n,
                                     void* stream) {
    LT_REQUIRE(comm && part && out, "lt_allreduce_add_tree: null pointer");
    LT_REQUIRE((comm->world & (comm->world - 1)) == 0, "lt_allreduce_add_tree: world=%d must be a power of two", comm->world);
    LT_REQUIRE(n > 0 && n % 4 == 0 && n <= comm->max_n, "lt_allreduce_add_tree: n=%d must be a multiple of 4, at most %d", n, comm->max_n);
    LT_REQUIRE(aligned16(part) && aligned16(out) && (resid == nullptr || aligned16(resid)),
               "lt_allreduce_add_tree: vectors must be 16-byte aligned");
    int* st = device_status_ptr();
    LT_REQUIRE(st != nullptr, "lt_allreduce_add_tree: status word unavailable");
    const CommDev C = comm_dev(comm);
    const int ctas = (n + COMM_CHUNK - 1) / COMM_CHUNK;
    const cudaError_t e = launch_chained(k_allreduce_add<true>, dim3(ctas), dim3(COMM_THREADS), 0, (cudaStream_t)stream, C,
                                         part, resid, out, n, st);
    return check_launch("lt_allreduce_add_tree", 1, e);
}
