// One-shot all-reduce (sum) of a small fp32 vector over the GPUs of one node, fused with the
// residual add that follows it in the tensor-parallel decode step:
//     out = resid + ((part_0 + part_1) + part_2 + ... )          (rank order, the same bits on every rank)
//
// Every rank owns a staging buffer that its peers map through CUDA IPC.  One kernel per rank: a thread
// stores its four elements of the local partial into slot [my rank] of EVERY rank's staging buffer as
// 8-byte words {value, tag} (plain peer stores over NVLink; the tag is the call count), then polls the
// words of all ranks in its own memory until their tags match and folds the values in rank order.  Data
// and "it has arrived" travel in the same aligned 8-byte store, so there is no fence and no separate
// flag on the path.  No data crosses NVLink twice, nothing is read from a peer, no multicast object is
// involved.  Waits are bounded (LT_STATUS_WAIT_TIMEOUT).
//
// Tags: a CTA counts its own calls in device memory (the launch arguments of a captured graph never
// change); staging is double-buffered by the count's parity: a rank can run at most one all-reduce ahead
// of its slowest peer, because finishing call k needs every peer's words of call k, which a peer only
// sends after it has left call k-1.  One process per GPU; the kernels of different ranks wait on each
// other and therefore must never share a GPU.
#include <string.h>

#include "lt_common.cuh"

namespace lt {

constexpr int COMM_THREADS = 256;
constexpr int COMM_CHUNK = COMM_THREADS * 4;        // floats per CTA
constexpr long long COMM_WAIT_LIMIT = 2000000000LL; // SM clocks (about a second) before a wait gives up

struct CommDev {
    float2* stage[LT_COMM_MAX_RANKS];    // stage[r]: rank r's staging buffer [2][world][max_n] of {value, tag}
    unsigned* ctr;                       // this rank's call counters [max_ctas]
    int rank, world, max_n, max_ctas;
};

__device__ __forceinline__ float2 ld_volatile_f2(const float2* p) {
    float2 v;
    asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(COMM_THREADS)
k_allreduce_add(const CommDev C, const float* __restrict__ part, const float* __restrict__ resid,
                float* __restrict__ out, int n, int* status) {
    chain_release();
    chain_wait();
    __shared__ unsigned s_epoch;
    const int c = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) s_epoch = C.ctr[c] + 1;
    __syncthreads();
    const unsigned epoch = s_epoch;
    const float tag = __uint_as_float(epoch);
    const int par = (int)(epoch & 1u);
    const int i = c * COMM_CHUNK + tid * 4;
    if (i < n) {
        // 1. my four elements, tagged, into slot [my rank] of every rank's staging buffer
        const float4 v = *(const float4*)(part + i);
        const long slot = ((long)par * C.world + C.rank) * C.max_n + i;
        for (int r = 0; r < C.world; r++) {
            float2* d = C.stage[r] + slot;
            d[0] = make_float2(v.x, tag); d[1] = make_float2(v.y, tag);
            d[2] = make_float2(v.z, tag); d[3] = make_float2(v.w, tag);
        }
        // 2. every rank's four elements from my own memory, folded in rank order
        const float2* mine = C.stage[C.rank] + (long)par * C.world * C.max_n + i;
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        bool ok = true;
        const long long t0 = clock64();
        for (int r = 0; r < C.world && ok; r++) {
            const float2* src = mine + (long)r * C.max_n;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float2 w = ld_volatile_f2(src + e);
                while (__float_as_uint(w.y) != epoch) {
                    if (clock64() - t0 > COMM_WAIT_LIMIT) {
                        atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
                        ok = false;
                        break;
                    }
                    w = ld_volatile_f2(src + e);
                }
                a[e] = r == 0 ? w.x : __fadd_rn(a[e], w.x);
            }
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
    if (tid == 0) C.ctr[c] = epoch;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_comm_alloc(int world, int max_n, lt_comm* comm, unsigned char* handle) {
    LT_REQUIRE(comm && handle, "lt_comm_alloc: null pointer");
    LT_REQUIRE(world >= 1 && world <= LT_COMM_MAX_RANKS, "lt_comm_alloc: world=%d (1..%d)", world, LT_COMM_MAX_RANKS);
    LT_REQUIRE(max_n > 0 && max_n % 4 == 0, "lt_comm_alloc: max_n=%d must be a positive multiple of 4", max_n);
    memset(comm, 0, sizeof(*comm));
    comm->world = world; comm->max_n = max_n;
    comm->max_ctas = (max_n + COMM_CHUNK - 1) / COMM_CHUNK;
    const size_t sb = (size_t)2 * world * max_n * sizeof(float2);
    void *s = nullptr, *c = nullptr;
    LT_CUDA(cudaMalloc(&s, sb));
    LT_CUDA(cudaMalloc(&c, (size_t)comm->max_ctas * sizeof(unsigned)));
    LT_CUDA(cudaMemset(s, 0, sb));          // tag 0 = never written (call counts start at 1)
    LT_CUDA(cudaMemset(c, 0, (size_t)comm->max_ctas * sizeof(unsigned)));
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
    CommDev C;
    for (int r = 0; r < LT_COMM_MAX_RANKS; r++) C.stage[r] = (float2*)comm->stage[r];
    C.ctr = comm->ctr; C.rank = comm->rank; C.world = comm->world; C.max_n = comm->max_n; C.max_ctas = comm->max_ctas;
    const int ctas = (n + COMM_CHUNK - 1) / COMM_CHUNK;
    const cudaError_t e = launch_chained(k_allreduce_add, dim3(ctas), dim3(COMM_THREADS), 0, (cudaStream_t)stream, C, part,
                                         resid, out, n, st);
    return check_launch("lt_allreduce_add", 1, e);
}
