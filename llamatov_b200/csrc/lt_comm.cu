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

}  // namespace lt

using namespace lt;

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
    const cudaError_t e = launch_chained(k_allreduce_add<false>, dim3(ctas), dim3(COMM_THREADS), 0, (cudaStream_t)stream, C,
                                         part, resid, out, n, st);
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
