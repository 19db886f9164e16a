// One-shot all-reduce (sum) of a small fp32 vector over the GPUs of one node, fused with the
// residual add that follows it in the tensor-parallel decode step:
//     out = resid + ((part_0 + part_1) + part_2 + ... )          (rank order, the same bits on every rank)
//
// Every rank owns a staging buffer and a flag array that its peers map through CUDA IPC.  One
// kernel per rank: a CTA copies its chunk of the local partial into slot [my rank] of EVERY rank's
// staging buffer with plain peer stores over NVLink, publishes a flag per destination
// (release, system scope), waits until the flags of all ranks have arrived in its own memory
// (acquire, bounded) and then folds the `world` local copies in rank order.  No data crosses
// NVLink twice, nothing is read from a peer, no multicast object is involved.
//
// Epochs: a CTA counts its own calls in device memory (the launch arguments of a captured graph
// never change), flag values are those counts, and staging is double-buffered by the count's
// parity: a rank can run at most one all-reduce ahead of its slowest peer, because finishing
// call k needs every peer's flag for k, which a peer only sends after it has left call k-1.
// One process per GPU; the kernels of different ranks wait on each other and therefore must
// never share a GPU.
#include <string.h>

#include "lt_common.cuh"

namespace lt {

constexpr int COMM_THREADS = 256;
constexpr int COMM_CHUNK = COMM_THREADS * 4;        // floats per CTA
constexpr long long COMM_WAIT_LIMIT = 2000000000LL; // SM clocks (about a second) before a wait gives up

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct CommDev {
    float* stage[LT_COMM_MAX_RANKS];     // stage[r]: rank r's staging buffer [2][world][max_n]
    unsigned* flags[LT_COMM_MAX_RANKS];  // flags[r]: rank r's flags [2][world][max_ctas]
    unsigned* ctr;                       // this rank's call counters [max_ctas]
    int rank, world, max_n, max_ctas;
};

__global__ void __launch_bounds__(COMM_THREADS)
k_allreduce_add(const CommDev C, const float* __restrict__ part, const float* __restrict__ resid,
                float* __restrict__ out, int n, int* status) {
    __shared__ unsigned s_epoch;
    __shared__ int s_fail;
    const int c = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) {
        s_epoch = C.ctr[c] + 1;
        s_fail = 0;
    }
    __syncthreads();
    const unsigned epoch = s_epoch;
    const int par = (int)(epoch & 1u);
    const int i = c * COMM_CHUNK + tid * 4;
    const long slot = ((long)par * C.world + C.rank) * C.max_n;
    // 1. my chunk of the partial into slot [my rank] of every rank's staging buffer
    if (i < n) {
        const float4 v = *(const float4*)(part + i);
        for (int r = 0; r < C.world; r++) *(float4*)(C.stage[r] + slot + i) = v;
    }
    __threadfence_system();
    __syncthreads();
    // 2. tell every rank that this chunk of mine has landed
    if (tid < C.world) st_release_sys(C.flags[tid] + ((long)par * C.world + C.rank) * C.max_ctas + c, epoch);
    // 3. wait for every rank's chunk in my own memory
    if (tid < C.world) {
        const unsigned* f = C.flags[C.rank] + ((long)par * C.world + tid) * C.max_ctas + c;
        const long long t0 = clock64();
        while (ld_acquire_sys(f) != epoch) {
            if (clock64() - t0 > COMM_WAIT_LIMIT) {
                s_fail = 1;
                atomicOr(status, (int)LT_STATUS_WAIT_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();
    // 4. fold the copies in rank order, add the residual
    if (i < n && !s_fail) {
        const float* mine = C.stage[C.rank] + (long)par * C.world * C.max_n + i;
        float4 a = __ldcg((const float4*)mine);
        for (int r = 1; r < C.world; r++) {
            const float4 b = __ldcg((const float4*)(mine + (long)r * C.max_n));
            a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
        }
        if (resid != nullptr) {
            const float4 x = *(const float4*)(resid + i);
            a.x = __fadd_rn(x.x, a.x); a.y = __fadd_rn(x.y, a.y); a.z = __fadd_rn(x.z, a.z); a.w = __fadd_rn(x.w, a.w);
        }
        *(float4*)(out + i) = a;
    }
    if (tid == 0) C.ctr[c] = epoch;
}

}  // namespace lt

using namespace lt;

extern "C" int lt_comm_alloc(int world, int max_n, lt_comm* comm, unsigned char* handles) {
    LT_REQUIRE(comm && handles, "lt_comm_alloc: null pointer");
    LT_REQUIRE(world >= 1 && world <= LT_COMM_MAX_RANKS, "lt_comm_alloc: world=%d (1..%d)", world, LT_COMM_MAX_RANKS);
    LT_REQUIRE(max_n > 0 && max_n % 4 == 0, "lt_comm_alloc: max_n=%d must be a positive multiple of 4", max_n);
    memset(comm, 0, sizeof(*comm));
    comm->world = world; comm->max_n = max_n;
    comm->max_ctas = (max_n + COMM_CHUNK - 1) / COMM_CHUNK;
    const size_t sb = (size_t)2 * world * max_n * sizeof(float);
    const size_t fb = (size_t)2 * world * comm->max_ctas * sizeof(unsigned);
    void *s = nullptr, *f = nullptr, *c = nullptr;
    LT_CUDA(cudaMalloc(&s, sb));
    LT_CUDA(cudaMalloc(&f, fb));
    LT_CUDA(cudaMalloc(&c, (size_t)comm->max_ctas * sizeof(unsigned)));
    LT_CUDA(cudaMemset(s, 0, sb));
    LT_CUDA(cudaMemset(f, 0, fb));
    LT_CUDA(cudaMemset(c, 0, (size_t)comm->max_ctas * sizeof(unsigned)));
    LT_CUDA(cudaDeviceSynchronize());
    comm->local_stage = (float*)s; comm->local_flags = (unsigned*)f; comm->ctr = (unsigned*)c;
    cudaIpcMemHandle_t hs, hf;
    LT_CUDA(cudaIpcGetMemHandle(&hs, s));
    LT_CUDA(cudaIpcGetMemHandle(&hf, f));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handles, &hs, 64);
    memcpy(handles + 64, &hf, 64);
    return LT_OK;
}

extern "C" int lt_comm_connect(lt_comm* comm, int rank, const unsigned char* all_handles) {
    LT_REQUIRE(comm && all_handles && comm->local_stage, "lt_comm_connect: call lt_comm_alloc first");
    LT_REQUIRE(rank >= 0 && rank < comm->world, "lt_comm_connect: rank=%d of %d", rank, comm->world);
    comm->rank = rank;
    for (int r = 0; r < comm->world; r++) {
        if (r == rank) {
            comm->stage[r] = comm->local_stage;
            comm->flags[r] = comm->local_flags;
            continue;
        }
        cudaIpcMemHandle_t hs, hf;
        memcpy(&hs, all_handles + (size_t)r * 128, 64);
        memcpy(&hf, all_handles + (size_t)r * 128 + 64, 64);
        void *s = nullptr, *f = nullptr;
        LT_CUDA(cudaIpcOpenMemHandle(&s, hs, cudaIpcMemLazyEnablePeerAccess));
        LT_CUDA(cudaIpcOpenMemHandle(&f, hf, cudaIpcMemLazyEnablePeerAccess));
        comm->stage[r] = (float*)s; comm->flags[r] = (unsigned*)f;
    }
    return LT_OK;
}

extern "C" int lt_comm_free(lt_comm* comm) {
    LT_REQUIRE(comm, "lt_comm_free: null pointer");
    for (int r = 0; r < comm->world; r++) {
        if (r == comm->rank) continue;
        if (comm->stage[r]) cudaIpcCloseMemHandle(comm->stage[r]);
        if (comm->flags[r]) cudaIpcCloseMemHandle(comm->flags[r]);
    }
    if (comm->local_stage) cudaFree(comm->local_stage);
    if (comm->local_flags) cudaFree(comm->local_flags);
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
    for (int r = 0; r < LT_COMM_MAX_RANKS; r++) {
        C.stage[r] = comm->stage[r];
        C.flags[r] = comm->flags[r];
    }
    C.ctr = comm->ctr; C.rank = comm->rank; C.world = comm->world; C.max_n = comm->max_n; C.max_ctas = comm->max_ctas;
    const int ctas = (n + COMM_CHUNK - 1) / COMM_CHUNK;
    k_allreduce_add<<<ctas, COMM_THREADS, 0, (cudaStream_t)stream>>>(C, part, resid, out, n, st);
    return check_launch("lt_allreduce_add");
}
