/*
 * lt_oracle.c -- CPU restatement of the reference's on-device Q8_0 decode arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA path: it is
 * compiled by oracle/build.py and loaded by tests/, by the smoke check and by the
 * cpu_baseline / reference legs of bench.py.  Nothing in the product package may
 * link, import or call it.
 *
 * Every function follows one reference kernel (paths are relative to the
 * reference project root):
 *   lto_quant_q8           bpd/lib/dev_residency.py:867-886   (k_quant_q8; host twin
 *                          bpd/lib/fact_dispatch.py:383-391)
 *   lto_silu_mul_quant     bpd/lib/dev_residency.py:573-593   (k_silu_mul_quant)
 *   lto_q8_gemv[_addres]   bpd/kernelgen/emitters/q8_0_from_facts.pl:476,483-516
 *                          (declared order + canonical-serial rendering), epilogue :412
 *   lto_q8_gemv_leftfold   bpd/kernelgen/emitters/q8_0_from_facts.pl:525-540 (thread-per-row
 *                          dp4a/scalar modes used by the host-roundtrip path)
 *   lto_quant_q8_ggml      bpd-substrate/bench/bpd_cpu.c:4096-4126 (the compiled CPU path's quantiser:
 *                          q = rint(x * (127/amax)))
 *   lto_q8_gemm_ggml       bpd-substrate/bench/bpd_gemm_q8_0_cpu.c:53-78 (one token: 8 lanes, block pairs,
 *                          mul then add, hsum_float_8), :80-132 (tiles of 2 or 4 tokens: 8 lanes per block
 *                          halves) and the token grouping of the dispatcher :205-260
 *   lto_rmsnorm            bpd/kernelgen/emitters/norm_softmax_from_facts.pl:49,117-144
 *   lto_rope               bpd/kernelgen/emitters/rope_from_facts.pl:48-65
 *   lto_append_kv_incr     bpd/lib/dev_residency.py:303-315
 *   lto_attn_decode_masked bpd/lib/dev_residency.py:1956-2009
 *   lto_attn_decode_split  bpd/kernelgen/experimental/attn_decode_split.cu (declared order
 *                          bpd/lib/ir_param_axes.pl:307-346; 64-thread launch of
 *                          bpd/kernelgen/referee/gatebench_attn_split.py)
 *   lto_argmax             bpd/lib/dev_residency.py:226-271
 *   lto_embed_q8           bpd/lib/dev_residency.py:1357-1358 (row of the dequantised table)
 *   lto_decode_token       bpd/lib/dev_residency.py:1381-1477,1596-1623 (op sequence)
 *
 * Arithmetic rules restated here: fp32 everywhere, a fused multiply-add wherever
 * the reference kernel's `acc += a*b` is contracted by nvcc (fmaf below), IEEE
 * division, rint = round-half-even.  Built with -ffp-contract=off so the C
 * compiler adds no contraction of its own.
 *
 * Device-numerics class: rsqrtf, expf, __expf, powf, cosf, sinf are CUDA device
 * functions whose last bits are not reproducible on a CPU.  This file uses libm
 * for them; tests compare those ops with a tolerance and everything else
 * (integer dots, quantised bytes, the GEMV fp32 order, argmax) bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- fp16 <-> fp32 */

float lto_h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal half: value = man * 2^-24; normalise */
            int e = -1;
            do { e++; man <<= 1; } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, like __float2half / numpy astype(float16) */
uint16_t lto_f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0u));
    }
    if (ax >= 0x477ff000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) { /* < 2^-25 (or == 2^-25, tie to even 0) */
        return sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    int shift;
    uint32_t hexp;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    uint32_t out;
    if (hexp == 0) {
        out = q; /* q may reach 0x400 -> smallest normal, encoding is continuous */
    } else {
        out = ((hexp - 1) << 10) + q; /* q carries the implicit bit (0x400..0x800) */
    }
    return (uint16_t)(sign | out);
}

/* ---------------------------------------------------------------- quantisers */

static inline int8_t quant_one(float v, float dq) {
    float r = v / dq;
    /* CUDA float->int conversion saturates and maps NaN to 0; then the kernel clamps. */
    if (r != r) return 0;
    if (r >= 127.0f) return 127;
    if (r <= -127.0f) return -127;
    int q = (int)rintf(r);
    if (q < -127) q = -127;
    if (q > 127) q = 127;
    return (int8_t)q;
}

static void quant_block(const float* v, int8_t* q, uint16_t* d_out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
        float a = fabsf(v[i]);
        if (a > amax) amax = a;
    }
    float d = (amax > 0.0f) ? amax / 127.0f : 1.0f;
    uint16_t dh = lto_f2h(d);
    *d_out = dh;
    float dq = lto_h2f(dh);
    for (int i = 0; i < 32; i++) q[i] = quant_one(v[i], dq);
}

void lto_quant_q8(const float* X, int8_t* Xq, uint16_t* Xd, int K) {
    int nb = K / 32;
    for (int b = 0; b < nb; b++) quant_block(X + 32 * b, Xq + 32 * b, Xd + b);
}

/* silu(g)*u exactly as written in the kernel: (g / (1 + expf(-g))) * u */
static inline float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

void lto_silu_mul(const float* g, const float* u, float* y, int K) {
    for (int i = 0; i < K; i++) y[i] = silu_mul(g[i], u[i]);
}

void lto_silu_mul_quant(const float* g, const float* u, int8_t* Xq, uint16_t* Xd, int K) {
    int nb = K / 32;
    float v[32];
    for (int b = 0; b < nb; b++) {
        for (int i = 0; i < 32; i++) v[i] = silu_mul(g[32 * b + i], u[32 * b + i]);
        quant_block(v, Xq + 32 * b, Xd + b);
    }
}

/* ---------------------------------------------------------------- Q8_0 GEMV */

static inline int block_isum(const int8_t* w, const int8_t* x) {
    int s = 0;
    for (int i = 0; i < 32; i++) s += (int)w[i] * (int)x[i];
    return s;
}

/* integer block dots only (exact): out[row*nb + b] */
void lto_q8_block_isums(const int8_t* Wq, const int8_t* Xq, int32_t* out, int M, int K) {
    int nb = K / 32;
    for (long r = 0; r < M; r++)
        for (int b = 0; b < nb; b++)
            out[r * nb + b] = block_isum(Wq + r * K + 32 * b, Xq + 32 * b);
}

static inline float gemv_row(const int8_t* wq, const uint16_t* wd, const int8_t* Xq,
                             const float* xdf, int nb) {
    float lane[32];
    for (int L = 0; L < 32; L++) {
        float acc = 0.0f;
        for (int b = L; b < nb; b += 32) {
            int isum = block_isum(wq + 32 * b, Xq + 32 * b);
            float s = lto_h2f(wd[b]) * xdf[b];
            acc = fmaf(s, (float)isum, acc);
        }
        lane[L] = acc;
    }
    for (int s = 16; s > 0; s >>= 1)
        for (int t = 0; t < s; t++) lane[t] = lane[t] + lane[t + s];
    return lane[0];
}

/* Y[M] (+Resid). Resid may be NULL. Rows are independent, so the row loop may run
 * on several host threads without changing a single bit. */
void lto_q8_gemv_addres(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq,
                        const uint16_t* Xd, const float* Resid, float* Y, int M, int K) {
    int nb = K / 32;
    float* xdf = (float*)malloc(sizeof(float) * (size_t)nb);
    for (int b = 0; b < nb; b++) xdf[b] = lto_h2f(Xd[b]);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < M; r++) {
        float acc = gemv_row(Wq + r * K, Wd + r * nb, Xq, xdf, nb);
        Y[r] = Resid ? acc + Resid[r] : acc;
    }
    free(xdf);
}

void lto_q8_gemv(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                 float* Y, int M, int K) {
    lto_q8_gemv_addres(Wq, Wd, Xq, Xd, NULL, Y, M, K);
}

/* batch of T activation columns, each reduced independently: Y[t*M + r] */
void lto_q8_gemm(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                 float* Y, int M, int K, int T) {
    int nb = K / 32;
    for (int t = 0; t < T; t++)
        lto_q8_gemv_addres(Wq, Wd, Xq + (long)t * K, Xd + (long)t * nb, NULL, Y + (long)t * M, M, K);
}

/* the older thread-per-row order: plain left fold over blocks */
void lto_q8_gemv_leftfold(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq,
                          const uint16_t* Xd, float* Y, int M, int K) {
    int nb = K / 32;
    for (long r = 0; r < M; r++) {
        float acc = 0.0f;
        for (int b = 0; b < nb; b++) {
            int isum = block_isum(Wq + r * K + 32 * b, Xq + 32 * b);
            float s = lto_h2f(Wd[r * nb + b]) * lto_h2f(Xd[b]);
            acc = fmaf(s, (float)isum, acc);
        }
        Y[r] = acc;
    }
}

/* ---------------------------------------------------------------- RMSNorm */

float lto_rms_sumsq(const float* x, int N) {
    float p[256];
    for (int t = 0; t < 256; t++) {
        float acc = 0.0f;
        for (int j = t; j < N; j += 256) acc = fmaf(x[j], x[j], acc);
        p[t] = acc;
    }
    for (int s = 128; s > 0; s >>= 1)
        for (int t = 0; t < s; t++) p[t] = p[t] + p[t + s];
    return p[0];
}

/* inv_override: when non-NULL its value replaces rsqrtf(...) so a test can feed the
 * device's own rsqrtf result and compare the rest of the kernel bit for bit. */
void lto_rmsnorm(const float* x, const float* w, float* y, int M, int N, float eps,
                 const float* inv_override) {
    for (long i = 0; i < M; i++) {
        const float* row = x + i * N;
        float ss = lto_rms_sumsq(row, N);
        float inv = inv_override ? inv_override[i] : 1.0f / sqrtf(ss / (float)N + eps);
        for (int j = 0; j < N; j++) y[i * N + j] = (row[j] * inv) * w[j];
    }
}

/* ---------------------------------------------------------------- RoPE */

void lto_rope(float* X, const int* pos, int nrows, int n_head, int hd, float theta) {
    int half = hd / 2;
    for (long row = 0; row < nrows; row++)
        for (int head = 0; head < n_head; head++)
            for (int j = 0; j < half; j++) {
                float p = (float)pos[row];
                float freq = powf(theta, -(2.0f * (float)j) / (float)hd);
                float ang = p * freq;
                float c = cosf(ang), s = sinf(ang);
                long base = row * n_head * hd + (long)head * hd;
                float x1 = X[base + j], x2 = X[base + j + half];
                /* contraction of the reference kernel as nvcc compiles it for sm_100a
                 * (checked against the reference's own kernel on the GPU) */
                X[base + j] = fmaf(x1, c, -(x2 * s));
                X[base + j + half] = fmaf(x2, c, x1 * s);
            }
}

/* ---------------------------------------------------------------- KV append */

void lto_append_kv_incr(float* kbase, const float* ksrc, float* vbase, const float* vsrc,
                        int* len, int width) {
    int L = *len;
    memcpy(kbase + (long)L * width, ksrc, sizeof(float) * (size_t)width);
    memcpy(vbase + (long)L * width, vsrc, sizeof(float) * (size_t)width);
    *len = L + 1;
}

/* ---------------------------------------------------------------- the compiled CPU path's order ("ggml order") */

/* Activation quantiser of the reference's C library: d = fp16(amax/127), id = 127/amax (0 when amax == 0),
 * q = rint(x * id).  Differs from lto_quant_q8 (q = rint(x / f32(d))) in the last bit of some quants. */
void lto_quant_q8_ggml(const float* x, int8_t* q, uint16_t* d, int K) {
    int nb = K / 32;
    for (int b = 0; b < nb; b++) {
        const float* xb = x + (long)b * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; j++) {
            float av = xb[j] < 0 ? -xb[j] : xb[j];
            if (av > amax) amax = av;
        }
        d[b] = lto_f2h(amax / 127.f);
        float id = (amax != 0.0f) ? 127.f / amax : 0.0f;
        for (int j = 0; j < 32; j++) q[(long)b * 32 + j] = (int8_t)rintf(xb[j] * id);
    }
}

static int isum4(const int8_t* w, const int8_t* a) {
    return (int)w[0] * a[0] + (int)w[1] * a[1] + (int)w[2] * a[2] + (int)w[3] * a[3];
}
static float hsum8(const float* l) {   /* ((l4+l0)+(l6+l2)) + ((l5+l1)+(l7+l3)) */
    float r0 = l[4] + l[0], r1 = l[5] + l[1], r2 = l[6] + l[2], r3 = l[7] + l[3];
    float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

/* Y[t*M + n].  One token (or the odd last one): lanes 0-3 take the even blocks, lanes 4-7 the odd ones, lane k
 * the bytes 4k..4k+3 of both 16-byte halves; acc = d*float(isum) + acc (two roundings).  Tokens in tiles of
 * 4 or 2: every block feeds all 8 lanes (lanes 0-3 the first half, 4-7 the second half). */
void lto_q8_gemm_ggml(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, float* Y,
                      int M, int K, int T) {
    int nb = K / 32;
    for (int t = 0; t < T; t++) {
        int vec = (T & 1) && t == T - 1;      /* the dispatcher's last group of one token */
        const int8_t* xq = Xq + (long)t * K;
        const uint16_t* xd = Xd + (long)t * nb;
#pragma omp parallel for schedule(static)
        for (int n = 0; n < M; n++) {
            const int8_t* wq = Wq + (long)n * K;
            const uint16_t* wd = Wd + (long)n * nb;
            float l[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (vec) {
                for (int b = 0; b + 1 < nb; b += 2) {
                    for (int h = 0; h < 2; h++) {
                        int bb = b + h;
                        float dl = lto_h2f(wd[bb]) * lto_h2f(xd[bb]);
                        for (int k = 0; k < 4; k++) {
                            int is = isum4(wq + bb * 32 + 4 * k, xq + bb * 32 + 4 * k) +
                                     isum4(wq + bb * 32 + 16 + 4 * k, xq + bb * 32 + 16 + 4 * k);
                            float pr = dl * (float)is;
                            l[4 * h + k] = pr + l[4 * h + k];
                        }
                    }
                }
            } else {
                for (int b = 0; b < nb; b++) {
                    float sc = lto_h2f(wd[b]) * lto_h2f(xd[b]);
                    for (int k = 0; k < 8; k++) {
                        int is = isum4(wq + b * 32 + 4 * k, xq + b * 32 + 4 * k);
                        float pr = sc * (float)is;
                        l[k] = pr + l[k];
                    }
                }
            }
            Y[(long)t * M + n] = hsum8(l);
        }
    }
}

/* ---------------------------------------------------------------- attention */

/* exp_fn selects the exponential: 0 = expf (libm), used as stand-in for __expf */
void lto_attn_decode_masked(const float* Q, const float* K, const float* V, int L, float* OUT,
                            int hd, int nh, int nkv, float scale, int maxt) {
    float* sh = (float*)malloc(sizeof(float) * (size_t)maxt);
    int rep = nh / nkv;
    for (int h = 0; h < nh; h++) {
        int hk = h / rep;
        const float* qh = Q + (long)h * hd;
        for (int t = 0; t < maxt; t++) {
            if (t < L) {
                const float* Kt = K + ((long)t * nkv + hk) * hd;
                float s = 0.0f;
                for (int i = 0; i < hd; i++) s = fmaf(qh[i], Kt[i], s);
                sh[t] = s * scale;
            } else {
                sh[t] = -1e30f;
            }
        }
        float red[64];
        for (int r = 0; r < 64; r++) {
            float m = -1e30f;
            for (int t = r; t < maxt; t += 64) m = fmaxf(m, sh[t]);
            red[r] = m;
        }
        for (int s2 = 32; s2 > 0; s2 >>= 1)
            for (int r = 0; r < s2; r++) red[r] = fmaxf(red[r], red[r + s2]);
        float mx = red[0];
        for (int t = 0; t < maxt; t++) sh[t] = expf(sh[t] - mx);
        for (int r = 0; r < 64; r++) {
            float ls = 0.0f;
            for (int t = r; t < maxt; t += 64) ls += sh[t];
            red[r] = ls;
        }
        for (int s2 = 32; s2 > 0; s2 >>= 1)
            for (int r = 0; r < s2; r++) red[r] = red[r] + red[r + s2];
        float Z = red[0];
        for (int d = 0; d < hd; d++) {
            float acc = 0.0f;
            for (int t = 0; t < L; t++) acc = fmaf(sh[t], V[((long)t * nkv + hk) * hd + d], acc);
            OUT[(long)h * hd + d] = acc / Z;
        }
    }
    free(sh);
}

/* The second declared order: S contiguous ranges of ceil(L/S) positions; per range local max,
 * expf against it, Z on 64 strided lanes + tree (32..1), left-fold V sum; combine in ascending
 * range order with w = expf(local max - global max), Z = fma(w, partZ, Z), O = fma(w, partO, O). */
void lto_attn_decode_split(const float* Q, const float* K, const float* V, int L, float* OUT,
                           int hd, int nh, int nkv, float scale, int S) {
    int rep = nh / nkv;
    int per = (L + S - 1) / S;
    float* sh = (float*)malloc(sizeof(float) * (size_t)(per > 0 ? per : 1));
    float* pM = (float*)malloc(sizeof(float) * (size_t)S);
    float* pZ = (float*)malloc(sizeof(float) * (size_t)S);
    float* pO = (float*)malloc(sizeof(float) * (size_t)S * hd);
    for (int h = 0; h < nh; h++) {
        int hk = h / rep;
        const float* qh = Q + (long)h * hd;
        for (int sp = 0; sp < S; sp++) {
            int p0 = sp * per, p1 = p0 + per;
            if (p1 > L) p1 = L;
            int n = p1 > p0 ? p1 - p0 : 0;
            float m = -1e30f;
            for (int t = p0; t < p1; t++) {
                const float* Kt = K + ((long)t * nkv + hk) * hd;
                float s = 0.0f;
                for (int i = 0; i < hd; i++) s = fmaf(qh[i], Kt[i], s);
                s = s * scale;
                sh[t - p0] = s;
                m = fmaxf(m, s);
            }
            float lmx = n > 0 ? m : -1e30f;
            pM[sp] = lmx;
            for (int t = 0; t < n; t++) sh[t] = expf(sh[t] - lmx);
            float red[64];
            for (int r = 0; r < 64; r++) {
                float ls = 0.0f;
                for (int t = r; t < n; t += 64) ls += sh[t];
                red[r] = ls;
            }
            for (int s2 = 32; s2 > 0; s2 >>= 1)
                for (int r = 0; r < s2; r++) red[r] += red[r + s2];
            pZ[sp] = red[0];
            for (int d = 0; d < hd; d++) {
                float acc = 0.0f;
                for (int t = p0; t < p1; t++) acc = fmaf(sh[t - p0], V[((long)t * nkv + hk) * hd + d], acc);
                pO[(long)sp * hd + d] = acc;
            }
        }
        float M = -1e30f;
        for (int sp = 0; sp < S; sp++) M = fmaxf(M, pM[sp]);
        for (int d = 0; d < hd; d++) {
            float Z = 0.0f, acc = 0.0f;
            for (int sp = 0; sp < S; sp++) {
                float w = expf(pM[sp] - M);
                Z = fmaf(w, pZ[sp], Z);
                acc = fmaf(w, pO[(long)sp * hd + d], acc);
            }
            OUT[(long)h * hd + d] = acc / Z;
        }
    }
    free(sh); free(pM); free(pZ); free(pO);
}


/* ---------------------------------------------------------------- argmax */

int lto_argmax(const float* x, int n) {
    float bestv = -3.4e38f;
    int besti = 2147483647;
    for (int i = 0; i < n; i++) {
        float v = x[i];
        if (v > bestv || (v == bestv && i < besti)) { bestv = v; besti = i; }
    }
    return besti;
}

/* ---------------------------------------------------------------- embedding */

/* row `tok` of the dequantised table: f32(d) * q (exact product) */
void lto_embed_q8(const int8_t* Wq, const uint16_t* Wd, int tok, float* out, int E) {
    int nb = E / 32;
    for (int i = 0; i < E; i++)
        out[i] = lto_h2f(Wd[(long)tok * nb + i / 32]) * (float)Wq[(long)tok * E + i];
}

/* ---------------------------------------------------------------- whole token */

typedef struct {
    const int8_t* wq;
    const uint16_t* wd;
} lto_q8w;

typedef struct {
    const float* attn_norm;   /* [E] */
    lto_q8w qkv;              /* [(nh+2nkv)*hd, E] rows q|k|v */
    const float* qkv_bias;    /* [(nh+2nkv)*hd] or NULL */
    lto_q8w o;                /* [E, nh*hd] */
    const float* ffn_norm;    /* [E] */
    lto_q8w gateup;           /* [2F, E] rows gate|up */
    lto_q8w down;             /* [E, F] */
    float* kcache;            /* [max_seq, nkv*hd] */
    float* vcache;
    int* len;                 /* host int: valid positions */
} lto_layer;

typedef struct {
    int n_layers, E, nh, nkv, hd, F, V, max_seq;
    float eps, theta;
    const lto_layer* layers;
    const float* out_norm;    /* [E] */
    lto_q8w lm_head;          /* [V, E] */
    lto_q8w embd;             /* [V, E] embedding table (Q8_0 rows) */
} lto_model;

/* One decode step: token id in, logits[V] out; caches and lengths advance.
 * Returns the greedy token.  scratch: caller-provided float workspace of at least
 * 4*E + 3*qkv + 2*F floats plus E+F bytes is avoided -- we malloc once per call. */
int lto_decode_token(const lto_model* m, int tok, float* logits) {
    int E = m->E, nh = m->nh, nkv = m->nkv, hd = m->hd, F = m->F;
    int nq = nh * hd, nk = nkv * hd, nqkv = nq + 2 * nk;
    int maxK = E > F ? E : F;
    float* x = (float*)malloc(sizeof(float) * (size_t)E);
    float* h = (float*)malloc(sizeof(float) * (size_t)E);
    float* x1 = (float*)malloc(sizeof(float) * (size_t)E);
    float* qkv = (float*)malloc(sizeof(float) * (size_t)nqkv);
    float* att = (float*)malloc(sizeof(float) * (size_t)nq);
    float* gu = (float*)malloc(sizeof(float) * (size_t)(2 * F));
    int8_t* xq = (int8_t*)malloc((size_t)maxK);
    uint16_t* xd = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(maxK / 32));
    float scale = (float)pow((double)hd, -0.5);

    lto_embed_q8(m->embd.wq, m->embd.wd, tok, x, E);
    for (int il = 0; il < m->n_layers; il++) {
        const lto_layer* ly = &m->layers[il];
        lto_rmsnorm(x, ly->attn_norm, h, 1, E, m->eps, NULL);
        lto_quant_q8(h, xq, xd, E);
        lto_q8_gemv_addres(ly->qkv.wq, ly->qkv.wd, xq, xd, ly->qkv_bias, qkv, nqkv, E);
        int pos = *ly->len;
        lto_rope(qkv, &pos, 1, nh + nkv, hd, m->theta);
        lto_append_kv_incr(ly->kcache, qkv + nq, ly->vcache, qkv + nq + nk, ly->len, nk);
        lto_attn_decode_masked(qkv, ly->kcache, ly->vcache, *ly->len, att, hd, nh, nkv, scale,
                               m->max_seq);
        lto_quant_q8(att, xq, xd, nq);
        lto_q8_gemv_addres(ly->o.wq, ly->o.wd, xq, xd, x, x1, E, nq);
        lto_rmsnorm(x1, ly->ffn_norm, h, 1, E, m->eps, NULL);
        lto_quant_q8(h, xq, xd, E);
        lto_q8_gemv_addres(ly->gateup.wq, ly->gateup.wd, xq, xd, NULL, gu, 2 * F, E);
        lto_silu_mul_quant(gu, gu + F, xq, xd, F);
        lto_q8_gemv_addres(ly->down.wq, ly->down.wd, xq, xd, x1, x, E, F);
    }
    lto_rmsnorm(x, m->out_norm, h, 1, E, m->eps, NULL);
    lto_quant_q8(h, xq, xd, E);
    lto_q8_gemv_addres(m->lm_head.wq, m->lm_head.wd, xq, xd, NULL, logits, m->V, E);
    int best = lto_argmax(logits, m->V);
    free(x); free(h); free(x1); free(qkv); free(att); free(gu); free(xq); free(xd);
    return best;
}

/* n > 0: use n OpenMP threads from now on (a launcher may have exported OMP_NUM_THREADS=1) */
void lto_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int lto_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
