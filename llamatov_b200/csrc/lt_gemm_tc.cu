// Q8_0 skinny GEMM / prefill GEMM on the 5th-generation tensor cores (tcgen05, kind::i8).
//
// Same arithmetic contract as the GEMV (lt_gemv.cu), per output row n and activation column t:
//   lane L in 0..31:  acc_L = 0;  for b = L, L+32, ... < K/32 (ascending):
//       isum  = sum_i Wq[n, 32b+i] * Xq[t, 32b+i]                    (exact int32)
//       acc_L = fma( f32(Wd[n,b]) * f32(Xd[t,b]), (float)isum, acc_L )
//   Y[t, n] = tree over the 32 lane values, s = 16, 8, 4, 2, 1: acc_l += acc_{l+s}   (+ Resid[n])
//
// The integer part is the dense contraction: one tcgen05.mma (M = 128 weight rows, N = NT
// activation columns, K = 32 bytes) produces the isum of one Q8_0 block for 128 x NT outputs as
// int32 in tensor memory.  Each block needs its own accumulator (the fp32 scale differs per
// block), so the fp32 part runs on the CUDA cores: epilogue warps read a block's 128 x NT int32
// from TMEM, scale and fold them in exactly the order above.  The "lanes" of the contract are
// plain registers here: thread = one weight row (TMEM lane) x CW columns, and the blocks are
// visited so that a row needs few live partials:
//   groups of CB adjacent lanes (CB blocks = one shared-memory chunk of CB*32 bytes per row) are
//   visited in bit-reversed group order; inside a group the rounds r = 0, 1, ... (block
//   CB*g + i + 32 r) extend the CB lane accumulators in ascending order; a finished group is
//   pushed on a log2(32/CB)-deep stack that performs the s = 16, 8, ... levels of the tree as
//   soon as both operands exist; the last log2(CB) levels combine the CB stacks at the end.
//
// Pipeline per CTA (persistent over tiles of 128 rows x NT columns):
//   warp EW   : producer, TMA tiled loads (hardware swizzle) of weight and activation chunks
//               into a ring of shared-memory stages; a stage = one chunk of CB blocks
//   warp EW+1 : one thread issues the CB MMAs of a stage into a ring of TMEM slots and commits
//   warps 0..EW-1 : epilogue, TMEM -> registers -> fp32 fold -> Y
// Every wait is bounded: after the limit a CTA sets LT_STATUS_WAIT_TIMEOUT, all its later waits
// return at once, it drains and frees its tensor memory.
#include <cuda.h>

#include "lt_common.cuh"

namespace lt {
namespace tc {

constexpr int TM = 128;          // weight rows per tile (MMA M, TMEM lanes)
constexpr int TMEM_COLS = 256;   // allocated tensor-memory columns (two CTAs may share an SM)
constexpr long long WAIT_LIMIT = 3000000000LL;  // SM clocks (> 1 s) before a wait gives up

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

// Bounded wait.  *abort_flag (shared) is set by the first wait of the CTA that runs out of time;
// from then on every wait returns immediately so that all roles run to the end of their loops.
template <int SLEEP_NS = 0>
__device__ __forceinline__ void mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                          int* status) {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if (*abort_flag) return;
        if (clock64() - t0 > WAIT_LIMIT) {
            *abort_flag = 1;
            atomicOr(status, LT_STATUS_WAIT_TIMEOUT);
            return;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] = A[smem] * B[smem], int8 x int8 -> int32, overwriting D
__device__ __forceinline__ void mma_i8(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                       unsigned idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// K-major shared-memory operand descriptor.  Rows are `row_bytes` apart inside an 8-row swizzle
// atom, atoms follow each other every 8*row_bytes (the stride byte offset); the leading byte
// offset is unused for swizzled K-major operands whose K extent fits the swizzle width.
template <int CB>
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
    constexpr unsigned long long layout = CB == 4 ? 2ull : (CB == 2 ? 4ull : 6ull);  // 128B / 64B / 32B swizzle
    constexpr unsigned long long sbo = (8ull * CB * 32ull) >> 4;
    return (unsigned long long)((addr >> 4) & 0x3FFFu) | (1ull << 16) | (sbo << 32) | (1ull << 46) | (layout << 61);
}

template <int CW>
__device__ __forceinline__ void tmem_ld(unsigned taddr, int (&v)[CW]);
template <>
__device__ __forceinline__ void tmem_ld<4>(unsigned taddr, int (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<8>(unsigned taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<16>(unsigned taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
// Completes the TMEM loads of this thread.  The loaded registers are passed through the
// statement (eight at a time) so that no use of them can be scheduled above the wait.
__device__ __forceinline__ void reg_fence4(int* v) {
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3])::"memory");
}
template <int N, int CB, int CW>
__device__ __forceinline__ void tmem_ld_wait(int (&v)[CB][CW]) {
    static_assert(N == CB * CW && CW % 4 == 0, "register count");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < CB; i++)
#pragma unroll
        for (int c = 0; c < CW; c += 4) reg_fence4(&v[i][c]);
}

constexpr int ilog2(int v) { return v <= 1 ? 0 : 1 + ilog2(v >> 1); }

struct Params {
    const __half* Wd;
    const __half* Xd;
    const float* Resid;
    float* Y;
    int* status;
    int M, K, T;
    int row_tiles, t_tiles;
    int resid_ld;   // 0: Resid[n] for every column (bias); else Resid[t * resid_ld + n]
};

template <int NT, int CB, int EW>
struct Cfg {
    static constexpr int CW = NT * 4 / EW;             // columns per epilogue thread
    static constexpr int G = 32 / CB;                  // lane groups
    static constexpr int LV = ilog2(G);                // stack depth
    static constexpr int MW = 2;                       // MMA-issuing warps
    static constexpr int THREADS = (EW + 1 + MW) * 32;
    static constexpr int W_STAGE = CB * TM * 32;       // bytes: one stage = one chunk of CB blocks
    static constexpr int X_STAGE = CB * NT * 32;
    static constexpr int STAGE = W_STAGE + ((X_STAGE + 1023) / 1024) * 1024;
    static constexpr int NSTAGE = CB == 4 ? 4 : (CB == 2 ? 6 : 8);
    static constexpr int SLOT_COLS = CB * NT;
    static constexpr int NSLOT = TMEM_COLS / SLOT_COLS;
    static constexpr int LB = CB * CW <= 16 ? CB : (CB >= 2 && CW <= 8 ? 2 : 1);   // blocks per TMEM round trip
    static_assert(EW % 4 == 0 && (CW == 4 || CW == 8 || CW == 16), "epilogue shape");
    static_assert(NSLOT >= 2 && NSLOT <= 16 && (NSLOT & (NSLOT - 1)) == 0, "TMEM slots");
    static_assert(W_STAGE % 1024 == 0, "stages keep 1024-byte alignment");
};

struct Barriers {
    unsigned long long full[8], empty[8];
    unsigned long long tfull[16], tempty[16];
    unsigned tmem_base;
    int abort_flag;
    int next_start[32];   // per visiting position: first block of the next group that has blocks, -1 = none
};

template <int NT, int CB, int EW>
__global__ void __launch_bounds__(Cfg<NT, CB, EW>::THREADS, 1)
k_q8_gemm_tc(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params P) {
    using C = Cfg<NT, CB, EW>;
    constexpr int CW = C::CW, G = C::G, LV = C::LV, NSLOT = C::NSLOT, NSTAGE = C::NSTAGE, LB = C::LB, MW = C::MW;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte aligned carve-up: stages (weights, then activations), barriers, activation scales
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Barriers* B = (Barriers*)(base + NSTAGE * C::STAGE);
    float* xs = (float*)((unsigned char*)B + 1024);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = P.K >> 5;
    const int tiles = P.row_tiles * P.t_tiles;
    volatile int* abort_flag = &B->abort_flag;

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&B->full[s], 1);
            mbar_init(&B->empty[s], 1);
        }
        for (int s = 0; s < NSLOT; s++) {
            mbar_init(&B->tfull[s], 1);
            mbar_init(&B->tempty[s], EW);
        }
        B->abort_flag = 0;
        for (int gi = 0; gi < G; gi++) {
            int nxt = -1;
            for (int gj = gi + 1; gj < G && nxt < 0; gj++) {
                const int b0 = CB * (int)(__brev((unsigned)gj) >> (32 - LV));
                if (b0 < nb) nxt = b0;
            }
            B->next_start[gi] = nxt;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == EW + 1) {   // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&B->tmem_base)),
                     "r"((unsigned)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = B->tmem_base;

    // chunks per tile: groups in bit-reversed order, rounds ascending; identical in all three roles
    if (warp == EW) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            unsigned it = 0;   // chunks issued
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const int rt = tile / P.t_tiles, tt = tile - rt * P.t_tiles;
                const int row0 = rt * TM, t0 = tt * NT;
                for (int gi = 0; gi < G; gi++) {
                    const int g = (int)(__brev((unsigned)gi) >> (32 - LV));
                    for (int b0 = CB * g; b0 < nb; b0 += 32, it++) {
                        const int s = it % NSTAGE;
                        unsigned char* st = base + s * C::STAGE;
                        mbar_wait<64>(&B->empty[s], ((it / NSTAGE) & 1) ^ 1, abort_flag, P.status);
                        mbar_expect_tx(&B->full[s], C::W_STAGE + C::X_STAGE);
                        tma_load_2d(st, &tmW, b0 * 32, row0, &B->full[s]);
                        tma_load_2d(st + C::W_STAGE, &tmX, b0 * 32, t0, &B->full[s]);
                    }
                }
            }
        }
    } else if (warp >= EW + 1) {
        // ------------------------------------------------------------------ MMA issue
        // MW warps share the chunks round-robin (a chunk has its own stage and slot, so the warps
        // are independent); issuing, not the tensor pipe, limits these small MMAs.
        if (lane == 0) {
            // instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = NT, M = 128
            constexpr unsigned idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NT >> 3) << 17) |
                                       ((unsigned)(TM >> 4) << 24);
            const unsigned long long wdesc0 = smem_desc<CB>(smem_u32(base));
            const unsigned long long xdesc0 = smem_desc<CB>(smem_u32(base) + C::W_STAGE);
            const unsigned chunks = (unsigned)(nb / CB);
            int my_tiles = 0;
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) my_tiles++;
            const unsigned total = (unsigned)my_tiles * chunks;
            for (unsigned it = (unsigned)(warp - (EW + 1)); it < total; it += MW) {
                const unsigned s = it % NSTAGE, slot = it % NSLOT;
                mbar_wait<32>(&B->full[s], (it / NSTAGE) & 1, abort_flag, P.status);
                mbar_wait<32>(&B->tempty[slot], ((it / NSLOT) & 1) ^ 1, abort_flag, P.status);
                tc_fence_after();
                // descriptors differ from the first stage's only in the start address (16-byte units)
                const unsigned long long wd0 = wdesc0 + (unsigned long long)(s * (C::STAGE >> 4));
                const unsigned long long xd0 = xdesc0 + (unsigned long long)(s * (C::STAGE >> 4));
                const unsigned d0 = tmem + slot * C::SLOT_COLS;
#pragma unroll
                for (int i = 0; i < CB; i++)   // block i = the i-th 32-byte slice of the swizzled rows
                    mma_i8(d0 + i * NT, wd0 + 2 * i, xd0 + 2 * i, idesc);
                mma_commit(&B->empty[s]);     // the stage may be refilled once these MMAs have read it
                mma_commit(&B->tfull[slot]);  // and the slot holds the block sums
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        // A thread walks its row's blocks in the visiting order.  While it folds a block, the
        // TMEM load of the next block and the global load of the next weight scales are in flight.
        const int q = warp & 3, cg = warp >> 2;
        const int col0 = cg * CW;
        const unsigned lane_addr = ((unsigned)(q * 32) << 16) + (unsigned)col0;
        int my_tiles = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) my_tiles++;
        const unsigned total = (unsigned)my_tiles * (unsigned)(nb / CB);   // chunks this thread consumes
        unsigned it = 0;                                                   // chunks consumed so far
        auto scale_row = [&](int tile) {   // this thread's row of weight scales in a tile (row 0 if out of range)
            int r = (tile / P.t_tiles) * TM + q * 32 + lane;
            if (r >= P.M) r = 0;
            return P.Wd + (long)r * nb;
        };
        auto scales_at = [&](const __half* p) {   // the CB scales of blocks b .. b+CB-1
            uint2 w = make_uint2(0u, 0u);
            if (CB == 4) w = __ldg((const uint2*)p);
            else if (CB == 2) w.x = __ldg((const unsigned*)p);
            else w.x = __ldg((const unsigned short*)p);
            return w;
        };
        uint2 wnext = make_uint2(0u, 0u);
        if (total > 0) wnext = scales_at(scale_row(blockIdx.x));

        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int rt = tile / P.t_tiles, tt = tile - rt * P.t_tiles;
            const int row = rt * TM + q * 32 + lane, t0 = tt * NT;
            const bool row_ok = row < P.M;
            const __half* wdrow = scale_row(tile);
            const __half* wdrow_next = scale_row(tile + gridDim.x < tiles ? tile + (int)gridDim.x : tile);

            // activation scales of this column tile: xs[b][c] = f32(Xd[t0 + c, b])
            asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory");
            for (int c = warp; c < NT; c += EW) {
                const bool ok = t0 + c < P.T;
                const __half* xr = P.Xd + (long)(ok ? t0 + c : 0) * nb;
                for (int b = lane; b < nb; b += 32) xs[b * NT + c] = ok ? __half2float(xr[b]) : 0.0f;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory");

            float stack[CB][LV > 0 ? LV : 1][CW];
            float fin[CB][CW];
#pragma unroll
            for (int gi = 0; gi < G; gi++) {
                const int g = (int)(__brev((unsigned)gi) >> (32 - LV));
                float leaf[CB][CW];
#pragma unroll
                for (int i = 0; i < CB; i++)
#pragma unroll
                    for (int c = 0; c < CW; c++) leaf[i][c] = 0.0f;

                for (int b0 = CB * g; b0 < nb; b0 += 32) {
                    const uint2 wcur = wnext;
                    {   // scales of the next chunk: next round of this group, else the next group that
                        // has blocks, else the first chunk of the next tile
                        const __half* np = wdrow + b0 + 32;
                        if (b0 + 32 >= nb) {
                            const int ns = B->next_start[gi];
                            np = ns < 0 ? wdrow_next : wdrow + ns;
                        }
                        wnext = scales_at(np);
                    }
                    // all CB blocks of the chunk in one round trip to tensor memory
                    const unsigned slot = it % NSLOT;
                    const unsigned taddr = tmem + lane_addr + slot * C::SLOT_COLS;
                    mbar_wait(&B->tfull[slot], (it / NSLOT) & 1, abort_flag, P.status);
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < CB; h += LB) {   // LB blocks per round trip to tensor memory
                        int v[LB][CW];
#pragma unroll
                        for (int i = 0; i < LB; i++) tmem_ld<CW>(taddr + (h + i) * NT, v[i]);
                        tmem_ld_wait<LB * CW>(v);
                        if (h + LB == CB) {
                            // the chunk's sums are in registers: hand the slot back to the MMA warp
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&B->tempty[slot]);
                            it++;
                        }
#pragma unroll
                        for (int j = 0; j < LB; j++) {
                            const int i = h + j;
                            const unsigned short wbits =
                                CB == 4 ? (unsigned short)((i < 2 ? wcur.x : wcur.y) >> ((i & 1) * 16))
                                        : (unsigned short)(wcur.x >> ((i & 1) * 16));
                            const float wd = __half2float(__ushort_as_half(wbits));
                            const float4* xp = (const float4*)(xs + (b0 + i) * NT + col0);
#pragma unroll
                            for (int c4 = 0; c4 < CW / 4; c4++) {
                                const float4 x = xp[c4];
                                leaf[i][4 * c4] = __fmaf_rn(__fmul_rn(wd, x.x), (float)v[j][4 * c4], leaf[i][4 * c4]);
                                leaf[i][4 * c4 + 1] =
                                    __fmaf_rn(__fmul_rn(wd, x.y), (float)v[j][4 * c4 + 1], leaf[i][4 * c4 + 1]);
                                leaf[i][4 * c4 + 2] =
                                    __fmaf_rn(__fmul_rn(wd, x.z), (float)v[j][4 * c4 + 2], leaf[i][4 * c4 + 2]);
                                leaf[i][4 * c4 + 3] =
                                    __fmaf_rn(__fmul_rn(wd, x.w), (float)v[j][4 * c4 + 3], leaf[i][4 * c4 + 3]);
                            }
                        }
                    }
                }
                // push the finished group: levels whose left operand is already there are added now
#pragma unroll
                for (int i = 0; i < CB; i++) {
                    bool placed = false;
#pragma unroll
                    for (int lv = 0; lv < LV; lv++) {
                        if (!placed) {
                            if ((gi >> lv) & 1) {
#pragma unroll
                                for (int c = 0; c < CW; c++) leaf[i][c] = __fadd_rn(stack[i][lv][c], leaf[i][c]);
                            } else {
#pragma unroll
                                for (int c = 0; c < CW; c++) stack[i][lv][c] = leaf[i][c];
                                placed = true;
                            }
                        }
                    }
                    if (!placed) {
#pragma unroll
                        for (int c = 0; c < CW; c++) fin[i][c] = leaf[i][c];
                    }
                }
            }
            // last levels of the tree across the CB lanes of a group: strides CB/2, ..., 1
#pragma unroll
            for (int s = CB / 2; s >= 1; s >>= 1)
#pragma unroll
                for (int i = 0; i < s; i++)
#pragma unroll
                    for (int c = 0; c < CW; c++) fin[i][c] = __fadd_rn(fin[i][c], fin[i + s][c]);

            if (row_ok) {
#pragma unroll
                for (int c = 0; c < CW; c++) {
                    const int t = t0 + col0 + c;
                    if (t < P.T) {
                        float y = fin[0][c];
                        if (P.Resid != nullptr) y = __fadd_rn(y, P.Resid[(long)t * P.resid_ld + row]);
                        P.Y[(long)t * P.M + row] = y;
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && warp == EW && lane == 0) {
        // a wait ran out: give bulk copies still in flight time to land before the CTA leaves
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
    }
    __syncthreads();
    if (warp == EW + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------- host side

typedef CUresult (*encode_fn_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_fn_t encode_fn() {
    static encode_fn_t fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (encode_fn_t)p;
    }
    return fn;
}

// 2-D byte tensor [rows][K] (row-major), box = box_k bytes x box_rows rows, hardware swizzle of box_k bytes
static int make_map(CUtensorMap* m, const void* ptr, int rows, int K, int box_k, int box_rows) {
    encode_fn_t fn = encode_fn();
    if (fn == nullptr) {
        set_error("lt_q8_gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
        return LT_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)box_k, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw = box_k == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                         : (box_k == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("lt_q8_gemm_tc: cuTensorMapEncodeTiled failed (%d) for rows=%d K=%d box=%dx%d", (int)r, rows, K,
                  box_k, box_rows);
        return LT_ERR_CUDA;
    }
    return LT_OK;
}

template <int NT, int CB, int EW>
static int launch(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, const float* Resid,
                  int resid_ld, float* Y, int M, int K, int T, cudaStream_t s) {
    using C = Cfg<NT, CB, EW>;
    const int nb = K / 32;
    CUtensorMap tmW, tmX;
    int rc = make_map(&tmW, Wq, M, K, CB * 32, TM);
    if (rc != LT_OK) return rc;
    rc = make_map(&tmX, Xq, T, K, CB * 32, NT);
    if (rc != LT_OK) return rc;
    const size_t smem = 1024 + (size_t)C::NSTAGE * C::STAGE + 1024 + (size_t)nb * NT * 4;
    LT_REQUIRE(smem <= 220 * 1024, "lt_q8_gemm_tc: K=%d needs %zu bytes of shared memory per CTA", K, smem);
    static PerDeviceOnce attr_once;
    if (attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_q8_gemm_tc<NT, CB, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    }
    Params P;
    P.Wd = (const __half*)Wd; P.Xd = (const __half*)Xd; P.Resid = Resid; P.Y = Y;
    P.status = device_status_ptr();
    LT_REQUIRE(P.status != nullptr, "lt_q8_gemm_tc: status word unavailable");
    P.M = M; P.K = K; P.T = T; P.resid_ld = resid_ld;
    P.row_tiles = (M + TM - 1) / TM;
    P.t_tiles = (T + NT - 1) / NT;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long tiles = (long)P.row_tiles * P.t_tiles;
    const int grid = (int)(tiles < sms ? tiles : sms);
    k_q8_gemm_tc<NT, CB, EW><<<grid, C::THREADS, smem, s>>>(tmW, tmX, P);
    return check_launch("lt_q8_gemm_tc");
}

}  // namespace tc
}  // namespace lt

using namespace lt;

extern "C" int lt_q8_gemm_tc(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                             const float* Resid, int resid_ld, float* Y, int M, int K, int T, int variant,
                             void* stream) {
    LT_REQUIRE(Wq && Wd && Xq && Xd && Y, "lt_q8_gemm_tc: null pointer");
    LT_REQUIRE(M > 0 && T > 0, "lt_q8_gemm_tc: M=%d T=%d must be positive", M, T);
    LT_REQUIRE(K > 0 && K % 128 == 0, "lt_q8_gemm_tc: K=%d must be a positive multiple of 128", K);
    LT_REQUIRE(aligned16(Wq) && aligned16(Xq), "lt_q8_gemm_tc: Wq and Xq must be 16-byte aligned");
    LT_REQUIRE(resid_ld == 0 || resid_ld >= M, "lt_q8_gemm_tc: resid_ld=%d must be 0 or at least M=%d", resid_ld, M);
    LT_REQUIRE(Resid == nullptr || resid_ld != 0 || T == 1 || (const void*)Y != (const void*)Resid,
               "lt_q8_gemm_tc: Y may alias Resid only when Resid has one row per column");
    cudaStream_t s = (cudaStream_t)stream;
    if (variant == 0) variant = 1;
    if (variant == 1) return tc::launch<16, 4, 8>(Wq, Wd, Xq, Xd, Resid, resid_ld, Y, M, K, T, s);
    if (variant == 2) return tc::launch<32, 1, 8>(Wq, Wd, Xq, Xd, Resid, resid_ld, Y, M, K, T, s);
    if (variant == 3) return tc::launch<16, 4, 16>(Wq, Wd, Xq, Xd, Resid, resid_ld, Y, M, K, T, s);
    set_error("lt_q8_gemm_tc: unknown variant %d", variant);
    return LT_ERR_INVALID;
}

