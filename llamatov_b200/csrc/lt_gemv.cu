// Q8_0 GEMV / skinny GEMM, HBM-bound: the weight matrix is streamed once, the (small)
// quantised activation sits in shared memory.
//
// Arithmetic contract, per output row n and activation column t:
//   lane L in 0..31:  acc_L = 0;  for b = L, L+32, ... < K/32 (ascending):
//       isum = sum_i Wq[n, 32b+i] * Xq[t, 32b+i]            (exact int32, dp4a)
//       acc_L = fma( f32(Wd[n,b]) * f32(Xd[t,b]), (float)isum, acc_L )
//   Y[t, n] = tree over lanes, s = 16, 8, 4, 2, 1: acc_l += acc_{l+s}   (+ Resid[n])
// Only the fp32 order is frozen; loads and integer work are scheduled freely.
//
// Mapping: one warp owns R consecutive rows at a time and keeps the loads of all R rows
// in flight together (R * (2 x 128-bit + 1 x 16-bit) per lane), lane = block index mod 32,
// exactly the lane of the contract, so the per-lane fold and the shuffle tree need no
// re-association.  Warps walk the matrix with a grid stride sized to the SM count.
#include "lt_common.cuh"
#include "lt_device_ops.cuh"
#include "lt_comm.cuh"

namespace lt {

constexpr int GEMV_WARPS = 8;      // warps per CTA
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

template <int R, int TB>
__global__ void __launch_bounds__(GEMV_THREADS)
k_q8_gemv(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd, const int8_t* __restrict__ Xq,
          const __half* __restrict__ Xd, const float* __restrict__ Resid, float* __restrict__ Y, int M, int K,
          int T) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nb = K >> 5;
    // shared: TB columns of (K int8 + nb fp16), each column padded to 16 bytes
    const int col_stride = ((K + nb * 2 + 15) >> 4) << 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long warps_total = (long)gridDim.x * GEMV_WARPS;
    const long gwarp = (long)blockIdx.x * GEMV_WARPS + warp;

    {   // T <= TB: one pass over the matrix serves every column
        const int t0 = 0;
        const int tcount = T;
        for (int c = 0; c < tcount; c++) {
            const int4* src = (const int4*)(Xq + (long)(t0 + c) * K);
            int4* dst = (int4*)(smem + c * col_stride);
            for (int i = threadIdx.x; i < (K >> 4); i += GEMV_THREADS) dst[i] = src[i];
            __half* dsth = (__half*)(smem + c * col_stride + K);
            const __half* srch = Xd + (long)(t0 + c) * nb;
            for (int i = threadIdx.x; i < nb; i += GEMV_THREADS) dsth[i] = srch[i];
        }
        __syncthreads();

        for (long r0 = gwarp * R; r0 < M; r0 += warps_total * R) {
            float acc[R][TB];
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int c = 0; c < TB; c++) acc[r][c] = 0.0f;

            for (int b = lane; b < nb; b += 32) {
                int4 w0[R], w1[R];
                float wd[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    long row = r0 + r;
                    if (row < M) {
                        const int8_t* p = Wq + row * K + (long)b * 32;
                        w0[r] = ld_stream_v4(p);
                        w1[r] = ld_stream_v4(p + 16);
                        wd[r] = __half2float(__ushort_as_half(ld_stream_u16(Wd + row * nb + b)));
                    } else {
                        w0[r] = make_int4(0, 0, 0, 0);
                        w1[r] = make_int4(0, 0, 0, 0);
                        wd[r] = 0.0f;
                    }
                }
#pragma unroll
                for (int c = 0; c < TB; c++) {
                    if (c < tcount) {
                        const int4* xp = (const int4*)(smem + c * col_stride + b * 32);
                        int4 x0 = xp[0], x1 = xp[1];
                        float xd = __half2float(((const __half*)(smem + c * col_stride + K))[b]);
#pragma unroll
                        for (int r = 0; r < R; r++)
                            acc[r][c] = q8_accum(wd[r], xd, block_dot(w0[r], w1[r], x0, x1), acc[r][c]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
#pragma unroll
                for (int c = 0; c < TB; c++) {
                    float v = warp_tree_sum(acc[r][c]);
                    long row = r0 + r;
                    if (lane == 0 && row < M && c < tcount) {
                        if (Resid != nullptr) v = __fadd_rn(v, Resid[row]);
                        Y[(long)(t0 + c) * M + row] = v;
                    }
                }
            }
        }
    }
}

// One activation column (the decode GEMV), tuned for latency as well as bandwidth: a warp owns R
// rows and keeps U rounds of every row's blocks in flight (R * U * 34 bytes per lane) before it
// folds them, so short matrices are one or two round trips to memory instead of K/1024.  The
// fold itself walks the rounds in ascending block order, the lane chain of the contract.
//
// PRO: the activation arrives as an fp32 vector and is RMS-normalised and quantised here, by every CTA
// for itself (the arithmetic of lt_rmsnorm + lt_quant_q8), while the first rows of every warp are on their
// way from DRAM to L2; Xq then names the fp32 vector, Xd the norm weight.
//
// Groups of R rows go to the warps with a grid stride (group cta*8 + warp, then + 8*grid): the warps of a CTA
// read neighbouring rows and the matrix is swept front to back.  Dealing the rows so that every SM gets an
// equal share (contiguous shares per CTA, or round-robin over CTAs first) was measured 10-20 % slower on the
// large shapes: an SM then touches many distant pages at once.
//
// MODE 2 (tensor parallel, this rank holds a K-slice of the rows): the result of a row is a partial sum; the
// warp pushes it into every rank's staging memory as soon as it is folded, and when all its rows are out it
// takes the partials of all ranks from its own staging memory and writes
// Y[n] = Resid[n] + ((part_0 + part_1) + ...) in rank order (lt_comm.cuh) -- the all-reduce rides in the GEMV,
// the exchange overlaps the rest of the weight stream.
constexpr int GEMV_PLAIN = 0, GEMV_NORM = 1, GEMV_ALLREDUCE = 2;
template <int R, int U, int MODE>
__global__ void __launch_bounds__(GEMV_THREADS, (R == 1 && U <= 4) ? 4 : (R * U <= 4 ? 3 : 2))
k_q8_gemv1(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd, const void* __restrict__ Xq_,
           const void* __restrict__ Xd_, float eps, const float* __restrict__ Resid, float* __restrict__ Y, int M,
           int K, const CommDev C, int* status) {
    constexpr bool PRO = MODE == GEMV_NORM;
    extern __shared__ __align__(16) unsigned char smem[];
    const int nb = K >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long groups = ((long)M + R - 1) / R;
    const long g_step = (long)GEMV_WARPS * gridDim.x;
    int4 w0[U][R], w1[U][R];
    unsigned short wd[U][R];
    // the tile (rows r0 .. r0+R-1, blocks b0, b0+32, ..) of this lane
    auto load_tile = [&](long r0, int b0) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int b = b0 + 32 * u;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const long row = r0 + r;
                if (b < nb && row < M) {
                    const int8_t* p = Wq + row * K + (long)b * 32;
                    w0[u][r] = ld_stream_v4(p);
                    w1[u][r] = ld_stream_v4(p + 16);
                    wd[u][r] = ld_stream_u16(Wd + row * nb + b);
                } else {
                    w0[u][r] = make_int4(0, 0, 0, 0);
                    w1[u][r] = make_int4(0, 0, 0, 0);
                    wd[u][r] = 0;
                }
            }
        }
    };
    // Weights do not depend on the predecessor in the stream: the first tile is requested before the wait,
    // and the second one is pulled into L2, so the head of the weight stream overlaps the predecessor's tail
    // (chained launch) and the activation prologue.
    chain_release();
    const long g_first = (long)blockIdx.x * GEMV_WARPS + warp;
    const long r_first = g_first * R;
    if (g_first < groups) {
        load_tile(r_first, lane);
        long r2 = r_first;
        int b2 = lane + 32 * U;
        if (b2 >= nb) { r2 = (g_first + g_step) * R; b2 = lane; }
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int r = 0; r < R; r++)
                if (b2 + 32 * u < nb && r2 + r < M)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(Wq + (r2 + r) * K + (long)(b2 + 32 * u) * 32));
    }
    // shared (PRO): sXq[K] | sXd[nb] (pad 16) | sred[272] | sF[K] | sW[K]
    float* sred = (float*)(smem + (((size_t)K + nb * 2 + 15) & ~(size_t)15));
    float* sF = sred + 272;
    float* sW = sF + K;
    if (PRO) {      // the norm weight is a constant of the model: on its way before the wait
        const float* normw = (const float*)Xd_;
        for (int c = threadIdx.x; c < (K >> 2); c += GEMV_THREADS)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(sW + c * 4)),
                         "l"(normw + c * 4) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    chain_wait();
    if (PRO) {
        const float4* X4 = (const float4*)Xq_;
        for (int c = threadIdx.x; c < (K >> 2); c += GEMV_THREADS) ((float4*)sF)[c] = X4[c];
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float ss = block_rms_sumsq(sF, K, sred);
        const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)K), eps));
        block_quant(sF, sW, inv, K, (int8_t*)smem, (__half*)(smem + K));
    } else {
        const int4* src = (const int4*)Xq_;
        int4* dst = (int4*)smem;
        for (int i = threadIdx.x; i < (K >> 4); i += GEMV_THREADS) dst[i] = src[i];
        __half* dsth = (__half*)(smem + K);
        const __half* Xd = (const __half*)Xd_;
        for (int i = threadIdx.x; i < nb; i += GEMV_THREADS) dsth[i] = Xd[i];
    }
    __syncthreads();
    const __half* xds = (const __half*)(smem + K);
    const unsigned* rowctr = MODE == GEMV_ALLREDUCE ? C.ctr + C.max_ctas : nullptr;     // exchanges completed, per row

    bool loaded = true;
    for (long g = g_first; g < groups; g += g_step) {
        const long r0 = g * R;
        unsigned number[R];
        if (MODE == GEMV_ALLREDUCE) {     // asked for early: the answer is there when the row is folded
#pragma unroll
            for (int r = 0; r < R; r++) number[r] = r0 + r < M ? rowctr[r0 + r] + 1u : 0u;
        }
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] = 0.0f;
        for (int b0 = lane; b0 < nb; b0 += 32 * U) {
            if (!loaded) load_tile(r0, b0);
            loaded = false;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int b = b0 + 32 * u;
                if (b < nb) {
                    const int4* xp = (const int4*)(smem + b * 32);
                    const int4 x0 = xp[0], x1 = xp[1];
                    const float xd = __half2float(xds[b]);
#pragma unroll
                    for (int r = 0; r < R; r++)
                        acc[r] = q8_accum(__half2float(__ushort_as_half(wd[u][r])), xd,
                                          block_dot(w0[u][r], w1[u][r], x0, x1), acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            float v = warp_tree_sum(acc[r]);
            const long row = r0 + r;
            if (lane == 0 && row < M) {
                if (MODE == GEMV_ALLREDUCE) {
                    comm_push(C, COMM_USER_GEMV, number[r], row, v);
                } else {
                    if (Resid != nullptr) v = __fadd_rn(v, Resid[row]);
                    Y[row] = v;
                }
            }
        }
    }
    if (MODE == GEMV_ALLREDUCE) {
        // the rows of this warp, one per lane: partials of all ranks in rank order, then the residual
        const long n_rows = g_first < groups ? ((groups - g_first + g_step - 1) / g_step) * R : 0;
        const long long t0 = clock64();
        for (long idx = lane; idx < n_rows; idx += 32) {
            const long row = (g_first + (idx / R) * g_step) * R + idx % R;
            if (row < M) {
                const unsigned num = rowctr[row] + 1u;
                float a = 0.0f;
                bool ok = true;
                for (int r = 0; r < C.world && ok; r++) {
                    float x = 0.0f;
                    ok = comm_take(C, COMM_USER_GEMV, num, r, row, t0, status, x);
                    a = r == 0 ? x : __fadd_rn(a, x);
                }
                if (ok) {
                    if (Resid != nullptr) a = __fadd_rn(Resid[row], a);
                    Y[row] = a;
                }
                // the exchange is counted whether or not it completed: every rank pushed this row with this
                // number, so the ranks' numbers must stay in step after a wait that gave up
                const_cast<unsigned*>(rowctr)[row] = num;
            }
        }
    }
}

// Wide skinny GEMM (8 < T <= TW): one warp per row, the row's blocks stay in registers while
// all T columns are folded, so the matrix is still read exactly once.  The activation
// columns come from global memory through L1/L2 (T*K bytes, cache resident).  Same lane /
// fold / tree order per (row, column) as the GEMV.  At these widths the integer dot
// products, not HBM, set the pace.
template <int TW>
__global__ void __launch_bounds__(GEMV_THREADS)
k_q8_gemm_wide(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd, const int8_t* __restrict__ Xq,
               const __half* __restrict__ Xd, const float* __restrict__ Resid, float* __restrict__ Y, int M, int K,
               int T) {
    const int nb = K >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long warps_total = (long)gridDim.x * GEMV_WARPS;
    for (long row = (long)blockIdx.x * GEMV_WARPS + warp; row < M; row += warps_total) {
        float acc[TW];
#pragma unroll
        for (int c = 0; c < TW; c++) acc[c] = 0.0f;
        for (int b = lane; b < nb; b += 32) {
            const int8_t* p = Wq + row * K + (long)b * 32;
            int4 w0 = ld_stream_v4(p), w1 = ld_stream_v4(p + 16);
            float wd = __half2float(__ushort_as_half(ld_stream_u16(Wd + row * nb + b)));
#pragma unroll
            for (int c = 0; c < TW; c++) {
                if (c < T) {
                    const int4* xp = (const int4*)(Xq + (long)c * K + (long)b * 32);
                    int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                    float xd = __half2float(__ldg(Xd + (long)c * nb + b));
                    acc[c] = q8_accum(wd, xd, block_dot(w0, w1, x0, x1), acc[c]);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < TW; c++) {
            float v = warp_tree_sum(acc[c]);
            if (lane == 0 && c < T) {
                if (Resid != nullptr) v = __fadd_rn(v, Resid[row]);
                Y[(long)c * M + row] = v;
            }
        }
    }
}

static int gemv_grid(long row_groups) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long ctas = (row_groups + GEMV_WARPS - 1) / GEMV_WARPS;
    long cap = (long)sms * 8;  // up to 8 resident CTAs of 256 threads per SM
    return (int)(ctas > cap ? cap : ctas);
}

// Lane-subset GEMV for a tensor-parallel row split that keeps the bits of one GPU.  A group of g ranks
// deals the Q8_0 blocks of a row round-robin: rank r holds blocks b = r (mod g), i.e. exactly the blocks of
// the contract's lanes L = r (mod g).  In the rank's local matrix (blocks j = (b - r) / g) the chain of
// lane L = r + g*m is blocks j = m, m + 32/g, m + 2*32/g, ...: the contract with LN = 32/g lanes.  The tree
// levels s >= g pair lanes of one rank (local levels s/g = LN/2 .. 1); the levels s < g pair ranks and are
// done by whoever sums the partials, in the order p[t] + p[t + s] for s = g/2 .. 1.  A warp folds G rows at
// once (LN lanes per row).  Y[t*M + n] = the rank's partial of (row n, column t).
template <int G>
__global__ void __launch_bounds__(GEMV_THREADS)
k_q8_gemv_lanes(const int8_t* __restrict__ Wq, const __half* __restrict__ Wd, const int8_t* __restrict__ Xq,
                const __half* __restrict__ Xd, float* __restrict__ Y, int M, int K, int T) {
    constexpr int LN = 32 / G;
    const int nb = K >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LN, m = lane % LN;
    const long warps_total = (long)gridDim.x * GEMV_WARPS;
    chain_release();
    chain_wait();
    for (long rg = (long)blockIdx.x * GEMV_WARPS + warp; rg * G < M; rg += warps_total) {
        const long row = rg * G + sub;
        const bool live = row < M;
        for (int t = 0; t < T; t++) {
            float acc = 0.0f;
            if (live) {
                const int8_t* wrow = Wq + row * K;
                const __half* drow = Wd + row * nb;
                const int8_t* xrow = Xq + (long)t * K;
                const __half* xdrow = Xd + (long)t * nb;
                int j = m;
                for (; j + 3 * LN < nb; j += 4 * LN) {       // four blocks of the chain in flight
                    int4 w0[4], w1[4];
                    unsigned short wd[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int8_t* p = wrow + (long)(j + u * LN) * 32;
                        w0[u] = ld_stream_v4(p); w1[u] = ld_stream_v4(p + 16);
                        wd[u] = ld_stream_u16(drow + j + u * LN);
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int4* xp = (const int4*)(xrow + (long)(j + u * LN) * 32);
                        const int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                        acc = q8_accum(__half2float(__ushort_as_half(wd[u])), __half2float(__ldg(xdrow + j + u * LN)),
                                       block_dot(w0[u], w1[u], x0, x1), acc);
                    }
                }
                for (; j < nb; j += LN) {
                    const int8_t* p = wrow + (long)j * 32;
                    const int4 w0 = ld_stream_v4(p), w1 = ld_stream_v4(p + 16);
                    const int4* xp = (const int4*)(xrow + (long)j * 32);
                    const int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                    acc = q8_accum(__half2float(__ushort_as_half(ld_stream_u16(drow + j))), __half2float(__ldg(xdrow + j)),
                                   block_dot(w0, w1, x0, x1), acc);
                }
            }
#pragma unroll
            for (int s = LN / 2; s > 0; s >>= 1) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, s, LN));
            if (live && m == 0) Y[(long)t * M + row] = acc;
        }
    }
}

template <int G>
static int launch_gemv_lanes(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, float* Y, int M,
                             int K, int T, cudaStream_t s) {
    const int ctas = gemv_grid(((long)M + G - 1) / G);
    const cudaError_t e = launch_chained(k_q8_gemv_lanes<G>, dim3((unsigned)ctas), dim3(GEMV_THREADS), 0, s, Wq,
                                         (const __half*)Wd, Xq, (const __half*)Xd, Y, M, K, T);
    return check_launch("lt_q8_gemv_lanes", 1, e);
}


template <int TW>
static int launch_gemm_wide(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                            const float* Resid, float* Y, int M, int K, int T, cudaStream_t s) {
    k_q8_gemm_wide<TW><<<gemv_grid(M), GEMV_THREADS, 0, s>>>(Wq, (const __half*)Wd, Xq, (const __half*)Xd, Resid, Y,
                                                            M, K, T);
    return check_launch("lt_q8_gemv(wide)");
}

template <int R, int TB>
static int launch_gemv(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                       const float* Resid, float* Y, int M, int K, int T, cudaStream_t s) {
    const int nb = K / 32;
    const int col_stride = ((K + nb * 2 + 15) / 16) * 16;
    const size_t smem = (size_t)col_stride * TB;
    static PerDeviceOnce attr_once;
    if (smem > 48 * 1024 && attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_q8_gemv<R, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    LT_REQUIRE(smem <= 200 * 1024, "lt_q8_gemv: K=%d needs %zu bytes of shared memory per CTA (limit 204800)", K, smem);
    int ctas = gemv_grid(((long)M + R - 1) / R);
    k_q8_gemv<R, TB><<<(unsigned)ctas, GEMV_THREADS, smem, s>>>(Wq, (const __half*)Wd, Xq, (const __half*)Xd, Resid,
                                                             Y, M, K, T);
    return check_launch("lt_q8_gemv");
}

template <int R, int U, int MODE>
static int launch_gemv1(const int8_t* Wq, const uint16_t* Wd, const void* Xq, const void* Xd, float eps,
                        const float* Resid, float* Y, int M, int K, const CommDev& C, cudaStream_t s) {
    constexpr bool PRO = MODE == GEMV_NORM;
    const int nb = K / 32;
    const size_t smem = (size_t)((K + nb * 2 + 15) / 16) * 16 + (PRO ? (size_t)(272 + 2 * K) * 4 : 0);
    static PerDeviceOnce attr_once;
    if (smem > 48 * 1024 && attr_once.first()) {
        LT_CUDA(cudaFuncSetAttribute(k_q8_gemv1<R, U, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    LT_REQUIRE(smem <= 200 * 1024, "lt_q8_gemv: K=%d needs %zu bytes of shared memory per CTA (limit 204800)", K, smem);
    // one wave: as many CTAs as are resident at once (by this instantiation's registers and shared memory)
    // occupancy of this instantiation, cached per device and shared-memory size
    struct Occ { int per_sm, sms; size_t smem; };
    static Occ occ[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    Occ local = {};
    Occ& oc = (dev >= 0 && dev < 64) ? occ[dev] : local;
    if (oc.per_sm == 0 || oc.smem != smem) {
        cudaDeviceGetAttribute(&oc.sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&oc.per_sm, k_q8_gemv1<R, U, MODE>, GEMV_THREADS, smem) !=
                cudaSuccess || oc.per_sm < 1)
            oc.per_sm = 1;
        oc.smem = smem;
    }
    const int per_sm = oc.per_sm, sms = oc.sms;
    // CTAs for one round of all warps, at most the resident wave (the warps loop).  With the all-reduce
    // epilogue every CTA must be resident (CTAs of different ranks wait on each other): never more than a wave.
    const long need = (((long)M + R - 1) / R + GEMV_WARPS - 1) / GEMV_WARPS;
    const long cap = (long)sms * per_sm;
    const int ctas = (int)(need < cap ? need : cap);
    int* st = nullptr;
    if (MODE == GEMV_ALLREDUCE) {
        st = device_status_ptr();
        LT_REQUIRE(st != nullptr, "lt_q8_gemv_allreduce: status word unavailable");
    }
    cudaError_t e;
    if (MODE == GEMV_ALLREDUCE) {
        // warps of different ranks wait for each other's rows: every CTA must be resident, which only a
        // cooperative launch guarantees (the grid is at most one wave by construction)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ctas);
        cfg.blockDim = dim3(GEMV_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeCooperative;
        at[0].val.cooperative = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, k_q8_gemv1<R, U, MODE>, Wq, (const __half*)Wd, Xq, Xd, eps, Resid, Y, M, K, C, st);
    } else {
        e = launch_chained(k_q8_gemv1<R, U, MODE>, dim3((unsigned)ctas), dim3(GEMV_THREADS), smem, s, Wq,
                           (const __half*)Wd, Xq, Xd, eps, Resid, Y, M, K, C, st);
    }
    return check_launch("lt_q8_gemv", 1, e);
}

// rows per warp by matrix height (enough warps to fill the GPU), rounds in flight by row length
template <int MODE>
static int dispatch_gemv1(const int8_t* Wq, const uint16_t* Wd, const void* Xq, const void* Xd, float eps,
                          const float* Resid, float* Y, int M, int K, const CommDev& C, cudaStream_t s) {
    const int rounds = (K / 32 + 31) / 32;
    if (MODE != GEMV_ALLREDUCE) {
        if (M >= 32768) {
            if (rounds >= 2) return launch_gemv1<4, 2, MODE == GEMV_ALLREDUCE ? GEMV_PLAIN : MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
            return launch_gemv1<4, 1, MODE == GEMV_ALLREDUCE ? GEMV_PLAIN : MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
        }
        if (M >= 8192) {
            if (rounds >= 3) return launch_gemv1<2, 4, MODE == GEMV_ALLREDUCE ? GEMV_PLAIN : MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
            if (rounds == 2) return launch_gemv1<2, 2, MODE == GEMV_ALLREDUCE ? GEMV_PLAIN : MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
            return launch_gemv1<2, 1, MODE == GEMV_ALLREDUCE ? GEMV_PLAIN : MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
        }
    }
    if (rounds >= 5) return launch_gemv1<1, 8, MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
    if (rounds >= 3) return launch_gemv1<1, 4, MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
    if (rounds == 2) return launch_gemv1<1, 2, MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
    return launch_gemv1<1, 1, MODE>(Wq, Wd, Xq, Xd, eps, Resid, Y, M, K, C, s);
}

}  // namespace lt

using namespace lt;

extern "C" int lt_q8_gemv(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                          const float* Resid, float* Y, int M, int K, int T, void* stream) {
    LT_REQUIRE(Wq && Wd && Xq && Xd && Y, "lt_q8_gemv: null pointer");
    LT_REQUIRE(M > 0 && T > 0, "lt_q8_gemv: M=%d T=%d must be positive", M, T);
    LT_REQUIRE(K > 0 && K % 32 == 0, "lt_q8_gemv: K=%d must be a positive multiple of 32", K);
    LT_REQUIRE(aligned16(Wq) && aligned16(Xq), "lt_q8_gemv: Wq and Xq must be 16-byte aligned");
    LT_REQUIRE((reinterpret_cast<uintptr_t>(Wd) & 1u) == 0 && (reinterpret_cast<uintptr_t>(Xd) & 1u) == 0,
               "lt_q8_gemv: scale pointers must be 2-byte aligned");
    LT_REQUIRE(T == 1 || Resid == nullptr || Y != Resid, "lt_q8_gemv: Y may alias Resid only when T == 1");
    cudaStream_t s = (cudaStream_t)stream;
    if (T == 1) return dispatch_gemv1<GEMV_PLAIN>(Wq, Wd, Xq, Xd, 0.0f, Resid, Y, M, K, CommDev{}, s);
    if (T <= 2) return launch_gemv<4, 2>(Wq, Wd, Xq, Xd, Resid, Y, M, K, T, s);
    if (T <= 4) return launch_gemv<2, 4>(Wq, Wd, Xq, Xd, Resid, Y, M, K, T, s);
    if (T <= 8) return launch_gemv<2, 8>(Wq, Wd, Xq, Xd, Resid, Y, M, K, T, s);
    // wider batches: block dots on the tensor cores when the row length allows the tiled loads
    if (K % 128 == 0 && (T == 1 || Resid == nullptr || Y != Resid))
        return lt_q8_gemm_tc(Wq, Wd, Xq, Xd, Resid, 0, Y, M, K, T, 0, stream);
    // otherwise chunks of up to 64 columns, each chunk one pass over the matrix with dp4a
    const int nb = K / 32;
    for (int t0 = 0; t0 < T; t0 += 64) {
        int tc = T - t0 < 64 ? T - t0 : 64;
        const int8_t* xq = Xq + (long)t0 * K;
        const uint16_t* xd = Xd + (long)t0 * nb;
        float* y = Y + (long)t0 * M;
        int rc;
        if (tc <= 16) rc = launch_gemm_wide<16>(Wq, Wd, xq, xd, Resid, y, M, K, tc, s);
        else if (tc <= 32) rc = launch_gemm_wide<32>(Wq, Wd, xq, xd, Resid, y, M, K, tc, s);
        else rc = launch_gemm_wide<64>(Wq, Wd, xq, xd, Resid, y, M, K, tc, s);
        if (rc != LT_OK) return rc;
    }
    return LT_OK;
}

extern "C" int lt_q8_gemv_lanes(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, float* Y, int M,
                                int K, int T, int group, void* stream) {
    LT_REQUIRE(Wq && Wd && Xq && Xd && Y, "lt_q8_gemv_lanes: null pointer");
    LT_REQUIRE(M > 0 && T > 0, "lt_q8_gemv_lanes: M=%d T=%d must be positive", M, T);
    LT_REQUIRE(K > 0 && K % 32 == 0, "lt_q8_gemv_lanes: K=%d must be a positive multiple of 32", K);
    LT_REQUIRE(aligned16(Wq) && aligned16(Xq), "lt_q8_gemv_lanes: Wq and Xq must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    switch (group) {
        case 1: return launch_gemv_lanes<1>(Wq, Wd, Xq, Xd, Y, M, K, T, s);
        case 2: return launch_gemv_lanes<2>(Wq, Wd, Xq, Xd, Y, M, K, T, s);
        case 4: return launch_gemv_lanes<4>(Wq, Wd, Xq, Xd, Y, M, K, T, s);
        case 8: return launch_gemv_lanes<8>(Wq, Wd, Xq, Xd, Y, M, K, T, s);
        default: break;
    }
    set_error("lt_q8_gemv_lanes: group=%d must be 1, 2, 4 or 8", group);
    return LT_ERR_INVALID;
}

extern "C" int lt_rmsnorm_q8_gemv(const int8_t* Wq, const uint16_t* Wd, const float* X, const float* normw, float eps,
                                  const float* Resid, float* Y, int M, int K, void* stream) {
    LT_REQUIRE(Wq && Wd && X && normw && Y, "lt_rmsnorm_q8_gemv: null pointer");
    LT_REQUIRE(M > 0, "lt_rmsnorm_q8_gemv: M=%d must be positive", M);
    LT_REQUIRE(K > 0 && K % 32 == 0, "lt_rmsnorm_q8_gemv: K=%d must be a positive multiple of 32", K);
    LT_REQUIRE(aligned16(Wq), "lt_rmsnorm_q8_gemv: Wq must be 16-byte aligned");
    LT_REQUIRE((reinterpret_cast<uintptr_t>(Wd) & 1u) == 0, "lt_rmsnorm_q8_gemv: Wd must be 2-byte aligned");
    LT_REQUIRE(Y != X, "lt_rmsnorm_q8_gemv: Y must not alias X (every CTA reads all of X)");
    LT_REQUIRE(aligned16(X) && aligned16(normw), "lt_rmsnorm_q8_gemv: X and normw must be 16-byte aligned");
    return dispatch_gemv1<GEMV_NORM>(Wq, Wd, X, normw, eps, Resid, Y, M, K, CommDev{}, (cudaStream_t)stream);
}

extern "C" int lt_q8_gemv_allreduce(const lt_comm* comm, const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq,
                                    const uint16_t* Xd, const float* Resid, float* Y, int M, int K, void* stream) {
    LT_REQUIRE(comm && Wq && Wd && Xq && Xd && Y, "lt_q8_gemv_allreduce: null pointer");
    LT_REQUIRE(comm->local_stage != nullptr && comm->world >= 1, "lt_q8_gemv_allreduce: comm is not connected");
    LT_REQUIRE(M > 0 && M <= comm->max_n, "lt_q8_gemv_allreduce: M=%d must be positive, at most the comm's max_n=%d", M, comm->max_n);
    LT_REQUIRE(K > 0 && K % 32 == 0, "lt_q8_gemv_allreduce: K=%d must be a positive multiple of 32", K);
    LT_REQUIRE(aligned16(Wq) && aligned16(Xq), "lt_q8_gemv_allreduce: Wq and Xq must be 16-byte aligned");
    LT_REQUIRE((reinterpret_cast<uintptr_t>(Wd) & 1u) == 0 && (reinterpret_cast<uintptr_t>(Xd) & 1u) == 0,
               "lt_q8_gemv_allreduce: scale pointers must be 2-byte aligned");
    return dispatch_gemv1<GEMV_ALLREDUCE>(Wq, Wd, Xq, Xd, 0.0f, Resid, Y, M, K, comm_dev(comm), (cudaStream_t)stream);
}
