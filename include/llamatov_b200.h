/*
 * llamatov_b200.h -- C ABI of libllamatov_b200.so: the sm_100a kernels of the Q8_0
 * transformer decode path, as host launchers.
 *
 * Conventions
 *   - every pointer argument is a DEVICE pointer unless its name starts with `h_`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - launchers only enqueue work: no allocation, no synchronisation, no host<->device
 *     copy, so every one of them may be recorded into a CUDA graph;
 *   - return value 0 = LT_OK; otherwise an LT_ERR_* code, with text in lt_last_error();
 *   - Q8_0 data is the split layout of the reference's resident engine: quants
 *     int8[rows*K] row-major and scales fp16[rows*K/32] (bit patterns, uint16_t);
 *   - K is always a multiple of 32; Wq and Xq must be 16-byte aligned.
 *
 * Each entry point names the reference interface it replaces (path inside the
 * reference project : line).  The reference launches these as C-linkage kernels
 * through cuLaunchKernel; here the grid/block/shared-memory choice is inside the launcher.
 */
#ifndef LLAMATOV_B200_H
#define LLAMATOV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LT_OK 0
#define LT_ERR_INVALID 1     /* bad argument (shape, alignment, null pointer) */
#define LT_ERR_CUDA 2        /* a CUDA runtime call or launch failed */
#define LT_ERR_UNSUPPORTED 3 /* valid request this build does not implement */

/* bits of the device status word (lt_device_status) */
#define LT_STATUS_KV_OVERFLOW 1u  /* append beyond max_seq was skipped */
#define LT_STATUS_BAD_LENGTH 2u   /* attention saw len < 0 or len > maxt; clamped */
#define LT_STATUS_BAD_TOKEN 4u    /* embedding gather saw a token id outside [0, V) */
#define LT_STATUS_WAIT_TIMEOUT 8u /* a bounded on-device wait gave up */

/* Text of the last error raised on the calling thread ("" if none). */
const char* lt_last_error(void);

/* Library version string. */
const char* lt_version(void);

/* Kernel launches this library has enqueued so far in this process (captured launches count
 * once, at capture). */
unsigned long long lt_launch_count(void);

/* Chained launches for the one-sequence decode operators (lt_q8_gemv with T = 1, lt_rmsnorm_q8_gemv,
 * lt_rope_append_batch, lt_attn_decode_batch, lt_attn_decode_split, lt_silu_mul_quant_rows, lt_embed_q8_rows,
 * lt_argmax, lt_add, lt_allreduce_add): when on, these kernels are enqueued with programmatic stream
 * serialisation; each lets its successor be scheduled at once, fetches its first weight rows, and only then
 * waits for its predecessor to complete, so launch latency and the head of the weight stream overlap the
 * predecessor's tail.  Results are unchanged.  Process-wide, off by default; returns the previous setting.
 * A captured graph keeps the setting it was recorded with. */
int lt_set_chained_launch(int on);

/* Reads the device status word of the current device into *h_status and clears it.
 * Synchronises `stream`.  Not capturable. */
int lt_device_status(unsigned int* h_status, void* stream);

/* ---- activation quantiser --------------------------------------------------------
 * replaces k_quant_q8 (bpd/lib/dev_residency.py:867-904, _launch_quant).
 * X f32[rows*K] -> Xq int8[rows*K], Xd fp16[rows*K/32]; one warp per 32-block:
 * d = fp16(amax/127) (1.0 when amax == 0), q = clamp(rint(v / f32(d)), +-127). */
int lt_quant_q8(const float* X, int8_t* Xq, uint16_t* Xd, int K, int rows, void* stream);

/* replaces k_silu_mul_quant (bpd/lib/dev_residency.py:573-605, _launch_silu_quant):
 * v = (g / (1 + expf(-g))) * u, then the quantiser above. */
int lt_silu_mul_quant(const float* g, const float* u, int8_t* Xq, uint16_t* Xd, int K, int rows,
                      void* stream);

/* replaces k_silu_mul and k_add (bpd/lib/dev_residency.py:545-566), the unfused forms. */
int lt_silu_mul(const float* g, const float* u, float* y, int n, void* stream);
int lt_add(const float* a, const float* b, float* y, int n, void* stream);

/* ---- Q8_0 GEMV / skinny GEMM --------------------------------------------------------
 * replaces k_q8_0_gemv, mode tiled_v4 (bpd/kernelgen/emitters/q8_0_from_facts.pl:212-253;
 * launched from bpd/lib/dev_residency.py:953-975,1152-1162) and k_q8_0_gemv_addres
 * (q8_0_from_facts.pl:374-416; dev_residency.py:1021-1032).
 * Y[t*M + n] = tree32( lane L: fold over blocks b = L, L+32, ... of
 *                      fma(f32(Wd[n,b]) * f32(Xd[t,b]), (float)isum(n,b,t), acc) ) (+ Resid[n])
 * which is the declared reduction_order(q8_gemv_dp4a, lanes(32), strided, accum(fma),
 * tree(shfl_down,5)) (q8_0_from_facts.pl:476).  T activation columns are reduced
 * independently (T = 1 is the decode GEMV).  Resid may be NULL; when given it has M
 * entries and is added to every column (bias or residual stream).  Y must not alias Resid
 * unless T == 1. */
int lt_q8_gemv(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
               const float* Resid, float* Y, int M, int K, int T, void* stream);

/* The same contract (same lane fold, same tree, bit-identical results) for wider activation
 * batches, with the integer block dots on the tensor cores: one tcgen05.mma kind::i8 per Q8_0
 * block gives the int32 sums of 128 weight rows x one tile of columns in tensor memory, the
 * fp32 scale-and-fold runs in the frozen order on the CUDA cores.  This is the batched form the
 * reference does not have (its prefill loops the per-token GEMV and requires batched results to
 * equal the per-token ones, bpd/lib/dev_residency.py:1344-1350).  K must be a multiple of 128.
 * variant: 0 = default (1); 1 = 16-column tiles, 128-byte weight chunks, 8 epilogue warps (the matrix
 * streams once from HBM in 128-byte rows; fastest measured at every width); 2 = 32-column tiles,
 * 32-byte chunks (fewest live partials per thread); 3 = as 1 with 16 epilogue warps.
 * Resid: NULL, or a bias of M entries added to every column (resid_ld = 0), or one row per
 * column, Resid[t * resid_ld + n] (the residual stream of a prefill; Y may then alias Resid).
 * lt_q8_gemv forwards to this entry for T > 8 when K allows it. */
int lt_q8_gemm_tc(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd,
                  const float* Resid, int resid_ld, float* Y, int M, int K, int T, int variant,
                  void* stream);

/* ---- RMSNorm --------------------------------------------------------------------------
 * replaces k_rmsnorm, mode block_row (bpd/kernelgen/emitters/norm_softmax_from_facts.pl:83-108;
 * launched from bpd/lib/dev_residency.py:757-781): 256 strided lanes fold fma(x,x,.), 8-level
 * pairwise tree, inv = rsqrtf(ss/N + eps), y = (x*inv)*w.  M rows of N. */
int lt_rmsnorm(const float* x, const float* w, float* y, int M, int N, float eps, void* stream);

/* lt_rmsnorm followed by lt_quant_q8 in one launch (the reference's RMS-quant production pairing,
 * bpd/kernelgen/referee/rms_quant_prod_ab.py); y may be NULL when only the quantised row is wanted. */
int lt_rmsnorm_quant(const float* x, const float* w, float* y, int8_t* Xq, uint16_t* Xd, int M, int N, float eps,
                     void* stream);

/* lt_rmsnorm + lt_quant_q8 + lt_q8_gemv (one column) in one launch, for the decode step's q|k|v and
 * gate|up projections: the reference's RMS->quant seam and its QFUSED GEMV, which quantises x into shared
 * memory itself (bpd/lib/dev_residency.py:937-948), taken one step further: every CTA normalises and quantises the K-vector X for itself in
 * shared memory, with the same arithmetic as the separate launches, then folds its rows.
 * Y[n] = sum over the Q8_0 row n and quant((X*inv)*normw) (+ Resid[n]); Y must not alias X. */
int lt_rmsnorm_q8_gemv(const int8_t* Wq, const uint16_t* Wd, const float* X, const float* normw, float eps,
                       const float* Resid, float* Y, int M, int K, void* stream);

/* ---- RoPE ------------------------------------------------------------------------------
 * replaces k_rope (bpd/kernelgen/emitters/rope_from_facts.pl:40-69; launched from
 * bpd/lib/dev_residency.py:701-742).  NeoX half-split rotation in place of X[nrows, n_head*hd]
 * at the positions pos[nrows] (device ints). */
int lt_rope(float* X, const int* pos, int nrows, int n_head, int hd, float theta, void* stream);

/* ---- KV cache append ----------------------------------------------------------------
 * replaces k_append_kv_incr / k_append_kv / k_incr_len (bpd/lib/dev_residency.py:281-316,
 * 464-521).  Writes ksrc/vsrc[width] at row *len of the position-major caches, then (when
 * incr != 0) *len += 1.  A row index >= max_seq is skipped and flagged. */
int lt_append_kv(float* kbase, const float* ksrc, float* vbase, const float* vsrc, int* len,
                 int width, int max_seq, int incr, void* stream);
int lt_incr_len(int* len, void* stream);

/* ---- decode attention ------------------------------------------------------------------
 * replaces k_attn_decode_masked (bpd/lib/dev_residency.py:1955-2031): one query token, GQA,
 * fp32 position-major cache [t][kvhead][d], valid length read from *len, positions >= len
 * masked; frozen reduction orders (64-lane max and sum, left-fold V sum).  maxt is the
 * capacity the reference compiles in as MAXT. */
int lt_attn_decode_masked(const float* Q, const float* K, const float* V, const int* len,
                          float* OUT, int hd, int nh, int nkv, float scale, int maxt,
                          void* stream);

/* ---- argmax ----------------------------------------------------------------------------
 * replaces k_argmax_s1 + k_argmax_s2 (bpd/lib/dev_residency.py:225-272,1074-1110): index of
 * the maximum, lowest index on ties.  `partials` is caller scratch of lt_argmax_scratch_bytes()
 * bytes. */
int lt_argmax(const float* x, int n, void* partials, int* out_idx, void* stream);
int lt_argmax_scratch_bytes(void);

/* ---- embedding gather ------------------------------------------------------------------
 * replaces the host lookup of the dequantised table row (bpd/lib/dev_residency.py:1357-1358,
 * 1761-1764): out[i] = f32(Wd[tok, i/32]) * Wq[tok, i], token id read from device memory. */
int lt_embed_q8(const int8_t* Wq, const uint16_t* Wd, const int* tok, float* out, int E, int V,
                void* stream);

/* ---- one decode step as one persistent kernel ---------------------------------------------
 * replaces the captured graph of one token forward, i.e. the whole body of
 * forward_pass_resident for one token plus _compute_folded_logits and argmax_dev
 * (bpd/lib/dev_residency.py:1381-1477,1596-1623,1812-1815; ~315 kernel nodes per token in the
 * reference): per layer rmsnorm+quant -> q|k|v GEMV+bias -> rope -> KV append -> masked
 * attention -> quant -> o_proj GEMV + residual -> rmsnorm+quant -> gate|up GEMV -> silu*up
 * quant -> down GEMV + residual; then final rmsnorm+quant -> LM-head GEMV -> argmax.  The
 * arithmetic of every op is the per-op entry point's, so results are bit-identical to the
 * chain of per-op launches.  One CTA per SM, cooperative launch.  CTAs [0, nh) each serve one
 * query head (its q rows and its KV group's k rows stay resident in shared memory, cached K rows
 * in registers, cached V rows staged in shared memory: rmsnorm -> q,k -> rope -> append ->
 * attention -> quantised head output without leaving the SM); the other CTAs own fixed row slices
 * of the v rows, o_proj, gate|up (whole 32-row blocks), down and the LM head, streamed through a
 * shared-memory ring by bulk async copies that run ahead of the dependency chain.  Four hand-overs
 * per layer go through tagged 8-byte words in the workspaces (no grid barrier).  Capturable.
 * Launches that share workspaces must not overlap on the GPU.
 *
 * All pointers are device pointers.  Each Q8_0 matrix must have a scale count (rows*K/32)
 * that is a multiple of 8 and 16-byte aligned bases.  Limits of this kernel: hd 32 or 64,
 * E <= 1024, F <= 6816, nh*hd <= 3392, nh < number of SMs; lt_decode_step_supported() tells
 * (1/0) whether a descriptor fits, lt_decode_step returns LT_ERR_UNSUPPORTED otherwise (use
 * lt_decode_step_pdl then). */
typedef struct lt_decode_layer {
    const float* attn_norm;    /* [E] */
    const int8_t* qkv_q;       /* [(nh+2*nkv)*hd, E] rows q|k|v */
    const uint16_t* qkv_d;
    const float* qkv_bias;     /* [(nh+2*nkv)*hd] or NULL */
    const int8_t* o_q;         /* [E, nh*hd] */
    const uint16_t* o_d;
    const float* ffn_norm;     /* [E] */
    const int8_t* gu_q;        /* [2F, E] rows gate|up */
    const uint16_t* gu_d;
    const int8_t* down_q;      /* [E, F] */
    const uint16_t* down_d;
    float* kcache;             /* [max_seq, nkv*hd] fp32, position-major */
    float* vcache;
    int* len;                  /* valid positions; rope position of the new token */
} lt_decode_layer;

typedef struct lt_decode_desc {
    int n_layers, E, nh, nkv, hd, F, V, max_seq;
    float eps, theta, scale;   /* scale = hd^-0.5 as fp32 */
    int hist_cap;
    const lt_decode_layer* layers;  /* device array [n_layers] */
    const float* out_norm;     /* [E] */
    const int8_t* lm_q;        /* [V, E] */
    const uint16_t* lm_d;
    const int8_t* emb_q;       /* [V, E] embedding table (needed when tok != NULL) */
    const uint16_t* emb_d;
    const float* x;            /* [E] input embedding row, read when tok == NULL (plain fp32, written by the host) */
    /* workspaces, 8 bytes per element, zero before first use.  lt_decode_step stores {payload, u32 tag}
     * words and keeps R = lt_decode_ws_replicas() copies of ws_x, ws_x1, ws_att and ws_v (each SM polls
     * one copy), so those four need R times the element counts given here. */
    void* ws_x;                /* [E] */
    void* ws_x1;               /* [E] */
    void* ws_qkv;              /* [(nh+2*nkv)*hd] (lt_decode_step keeps the new v row in the first nkv*hd elements) */
    void* ws_att;              /* [nh*hd] (lt_decode_step: packed Q8_0, nh*hd/4 + nh*hd/32 elements used) */
    void* ws_v;                /* [F] silu(gate)*up (lt_decode_step: packed Q8_0) */
    float* logits;             /* [V] */
    int* tok;                  /* device token: read at the start, overwritten with the argmax; NULL = x preloaded */
    int* out_tok;              /* argmax of the logits */
    int* history;              /* optional: history[*step] = token; *step += 1 */
    int* step;
    unsigned int* sync;        /* unused (kept for layout) */
    unsigned int* epoch;       /* [1] token counter that stamps the workspaces, zero before the first launch;
                                  advanced by every launch (wraps after 2^32/(n_layers+2) tokens) */
    float* part_val;           /* [lt_decode_num_ctas()] */
    int* part_idx;             /* [lt_decode_num_ctas()] */
    int* status;               /* device status word; NULL = the library's own */
    long long* trace;          /* optional [2][8192][2] (id, SM clock) stamps of CTA 0 and of the last CTA
                                  (diagnostics); NULL in production */
    const lt_decode_layer* h_layers; /* HOST copy of the layer array (launch-time checks; walked by lt_decode_step_pdl) */
    void* ws_part;             /* lt_decode_step: tagged workspace [2 * lt_decode_num_ctas()] for the per-CTA argmax results */
    int poll_ns;               /* lt_decode_step: pause between two looks at hand-over words that have not arrived
                                  (0 = none); with several looks in flight, their spacing */
    int poll_looks;            /* lt_decode_step: copies of the hand-over workspaces in use, 1..lt_decode_ws_replicas() (0 = all) */
    int trace_cta;             /* lt_decode_step, diagnostics: the second traced CTA (0 = the last one) */
    int trace_layer;           /* lt_decode_step, diagnostics: with `trace` set and trace_layer = l >= 0, thread 0 of every
                                * CTA stores the global timer (ns) at the arrival of the input of each of layer l's four
                                * phases and at the end of each phase, in the last 8 * lt_decode_num_ctas() entries of the
                                * trace buffer ([cta][arrival 0..3, end 0..3]); negative = off */
} lt_decode_desc;

int lt_decode_step(const lt_decode_desc* h_desc, void* stream);
int lt_decode_step_supported(const lt_decode_desc* h_desc);
int lt_decode_ws_replicas(void);
int lt_decode_num_ctas(void);

/* The same step, same descriptor and bit-identical results, as a chain of fused kernels (five
 * per layer + LM head + argmax) linked by programmatic dependent launch: every kernel prefetches
 * its weights (and cached K/V rows, rope angles) while its predecessor is still running, then
 * waits for the predecessor (griddepcontrol.wait).  The workspaces are used as plain buffers
 * here (no tags); epoch and sync are not used.  part_val / part_idx need
 * lt_decode_pdl_num_parts() entries. */
int lt_decode_step_pdl(const lt_decode_desc* h_desc, void* stream);
int lt_decode_pdl_num_parts(void);

/* ---- row-batched operators for prefilling a prompt in one pass ---------------------------
 * The reference prefills by running its one-token step once per prompt token
 * (bpd/lib/dev_residency.py:1344-1350, forward_pass_resident recursing over the tokens) and
 * requires a batched form to give the same numbers.  Each entry below computes for row r exactly
 * what the one-token operator computes for that token; together with lt_rmsnorm / lt_quant_q8
 * (rows) and lt_q8_gemm_tc they make a prompt chunk one pass over the weights.
 *
 * lt_embed_q8_rows      rows of lt_embed_q8: out[r, :] = dequantised table row of toks[r].
 * lt_rope_rows          k_rope (rope_from_facts.pl:40-69) on row r at position *pos0 + r; a row holds
 *                       n_head heads of hd floats at its start, rows are ld floats apart.
 * lt_append_kv_rows     k_append_kv_incr (dev_residency.py:303-315) for nrows rows: row r goes to cache
 *                       position *len + r; then *len += nrows when incr != 0.  Overflow sets
 *                       LT_STATUS_KV_OVERFLOW and appends nothing.
 * lt_silu_mul_quant_rows  lt_silu_mul_quant with gate and up rows ld floats apart.
 * lt_attn_prefill       k_attn_decode_masked (dev_residency.py:1955-2010) for the nrows rows just
 *                       appended: *len is the length after the append, row r is the query at position
 *                       *len - nrows + r and sees the positions up to and including its own.
 *                       maxt >= *len bounds the shared-memory score rows (<= 12000). */
int lt_embed_q8_rows(const int8_t* Wq, const uint16_t* Wd, const int* toks, float* out, int E, int V,
                     int nrows, void* stream);
int lt_rope_rows(float* X, int ld, const int* pos0, int nrows, int n_head, int hd, float theta, void* stream);
int lt_append_kv_rows(float* kbase, const float* ksrc, float* vbase, const float* vsrc, int src_ld, int* len,
                      int width, int max_seq, int nrows, int incr, void* stream);
int lt_silu_mul_quant_rows(const float* g, const float* u, int ld, int8_t* Xq, uint16_t* Xd, int K, int rows,
                           void* stream);
int lt_attn_prefill(const float* Q, int q_ld, const float* K, const float* V, const int* len, float* OUT,
                    int out_ld, int hd, int nh, int nkv, float scale, int nrows, int maxt, void* stream);

/* ---- decode operators for a batch of sequences / long contexts ------------------------------
 * No batched engine exists in the reference; its contract is that every sequence gets the
 * one-sequence result.  The KV caches of a batch are one buffer per layer,
 * [B][max_seq][nkv*hd] fp32, with one device length per sequence (lens[B]).
 *
 * lt_rope_batch         k_rope with one position per row: row r (ld floats apart) at pos[r].
 * lt_append_kv_batch    k_append_kv_incr per sequence: row b goes to position lens[b] of cache b,
 *                       then lens[b] += 1 when incr != 0; a full cache sets LT_STATUS_KV_OVERFLOW.
 * lt_attn_decode_batch  k_attn_decode_masked (bpd/lib/dev_residency.py:1955-2010) for B query rows,
 *                       lens[b] = length after the append.  Three launches (scores over position
 *                       chunks, softmax per head, V sum per output element) so that a long context
 *                       is scanned by many CTAs; every fold keeps the frozen order, results are
 *                       bit-identical to lt_attn_decode_masked.  Xq / Xd (both or neither): the Q8_0
 *                       quantisation of the output rows (lt_quant_q8) written by the same launch.  scratch holds
 *                       lt_attn_decode_batch_scratch_floats(nh, max_seq, B) floats, 16-byte aligned. */
int lt_rope_batch(float* X, int ld, const int* pos, int nrows, int n_head, int hd, float theta, void* stream);
int lt_append_kv_batch(float* kbase, const float* ksrc, float* vbase, const float* vsrc, int src_ld, int* lens,
                       int width, int max_seq, int B, int incr, void* stream);
long lt_attn_decode_batch_scratch_floats(int nh, int max_seq, int B);
int lt_attn_decode_batch(const float* Q, int q_ld, const float* K, const float* V, const int* lens, float* OUT,
                         int out_ld, float* scratch, int hd, int nh, int nkv, float scale, int max_seq, int B,
                         int8_t* Xq, uint16_t* Xd, void* stream);
/* lt_rope_batch on the q and k heads of row b at position lens[b], then lt_append_kv_batch of the row's k|v
 * part, in one launch; a row is q heads | k heads | v heads, ld floats apart.  ticket: B ints of device
 * scratch, zero before the first call (the kernel leaves them zero). */
int lt_rope_append_batch(float* X, int ld, int n_qhead, int n_kvhead, int hd, float theta, float* kbase,
                         float* vbase, int* lens, int max_seq, int B, int* ticket, void* stream);

/* lt_attn_decode_split: decode attention in the reference's second declared order,
 * reduction_order(attn_decode_split, ...) (bpd/lib/ir_param_axes.pl:307-346; kernel text
 * bpd/kernelgen/experimental/attn_decode_split.cu, launched with 64 threads by
 * bpd/kernelgen/referee/gatebench_attn_split.py): nsplit contiguous ranges of ceil(L/nsplit) positions, each
 * with its own max / exponentials / 64-lane Z / left-fold V sum, combined by exp(local max - global max) in
 * ascending range order.  nsplit is part of the order (fix it per captured graph); nsplit = 1 gives the bits
 * of lt_attn_decode_masked.  The reference keeps this order banked, not wired into production; here it is
 * opt-in for long contexts, where it shortens the dependent V-sum chain to L/nsplit.  Same cache layout and
 * arguments as lt_attn_decode_batch; scratch holds lt_attn_decode_split_scratch_floats(nh, hd, nsplit, B). */
long lt_attn_decode_split_scratch_floats(int nh, int hd, int nsplit, int B);
int lt_attn_decode_split(const float* Q, int q_ld, const float* K, const float* V, const int* lens, float* OUT,
                         int out_ld, float* scratch, int hd, int nh, int nkv, float scale, int max_seq, int B,
                         int nsplit, int8_t* Xq, uint16_t* Xd, void* stream);
/* lt_rope_append_batch followed by lt_attn_decode_split in the same two launches the attention needs anyway:
 * X holds the rows q | k | v as the projection wrote them (ld floats apart); every CTA of the range kernel
 * rotates its own query heads (k_rope at position lens[b]), the CTA whose range ends with the new position
 * rotates the row's k head and appends k and v to the cache before it reads its range, and the last CTA of a
 * sequence to finish advances lens[b].  X itself is not modified.  ticket: B ints of device scratch, zero
 * before the first call (left zero).  Same values, cache rows and lengths as the two separate calls; a full
 * cache sets LT_STATUS_KV_OVERFLOW and appends nothing. */
int lt_rope_attn_decode_split(const float* X, int ld, float* K, float* V, int* lens, float* OUT, int out_ld,
                              float* scratch, int hd, int nh, int nkv, float theta, float scale, int max_seq, int B,
                              int nsplit, int* ticket, int8_t* Xq, uint16_t* Xd, void* stream);

/* ---- parity mode: the fold order of the reference's compiled CPU path ---------------------------
 * lt_quant_q8_ggml / lt_q8_gemm_ggml reproduce bpd_quant_q8_0_cpu and bpd_qmatmul_q8_0_llamafile_cpu
 * (bpd-substrate/bench/bpd_cpu.c:4096-4126,4419-4447; bpd_gemm_q8_0_cpu.c:53-132,205-260) bit for bit:
 * q = rint(x * 127/amax); 8 float lanes per result, multiply then add (two roundings), hsum_float_8; one
 * token (or an odd last token) folds block pairs into lane halves, tokens in tiles fold every block into
 * all 8 lanes.  Y[t*M + n].  Not used by the decode engine (which keeps the resident engine's declared
 * order, lt_q8_gemv); for comparing a GPU result with that CPU library. */
int lt_quant_q8_ggml(const float* X, int8_t* Xq, uint16_t* Xd, int K, int rows, void* stream);
int lt_q8_gemm_ggml(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, float* Y,
                    int M, int K, int T, void* stream);

/* ---- all-reduce over the GPUs of one node, fused with the residual add ---------------------
 * No counterpart in the reference (it is single-GPU).  For the tensor-parallel decode step:
 * out = resid + (part_0 + part_1 + ... in rank order), the same bits on every rank.  Each rank owns
 * a staging buffer that its peers map through CUDA IPC; one kernel per rank stores its partial into
 * every rank's staging memory as {value, call-count tag} words (plain peer stores), polls the words of
 * all ranks in its own memory (bounded: LT_STATUS_WAIT_TIMEOUT) and folds them.  One process per GPU.
 * Setup: every rank calls lt_comm_alloc (fills LT_COMM_HANDLE_BYTES handle bytes), the ranks exchange
 * the handle bytes by any host means, every rank calls lt_comm_connect with all of them (world *
 * LT_COMM_HANDLE_BYTES bytes, rank order), then a host barrier before the first lt_allreduce_add. */
#define LT_COMM_MAX_RANKS 8
#define LT_COMM_HANDLE_BYTES 64
typedef struct lt_comm {
    int rank, world, max_n, max_ctas;
    float* stage[LT_COMM_MAX_RANKS];      /* stage[r]: rank r's staging buffer as mapped in this process */
    float* local_stage;
    unsigned int* ctr;                    /* exchange counters (device): per all-reduce CTA, then per GEMV row */
} lt_comm;
int lt_comm_alloc(int world, int max_n, lt_comm* comm, unsigned char* handle);
int lt_comm_connect(lt_comm* comm, int rank, const unsigned char* all_handles);
/* lt_comm_free unmaps the peers' buffers and frees this rank's: no kernel of ANY rank that uses the comm may
 * still be running -- synchronise the device, then pass a host barrier over all ranks, then call it. */
int lt_comm_free(lt_comm* comm);
int lt_allreduce_add(const lt_comm* comm, const float* part, const float* resid, float* out, int n,
                     void* stream);
/* The same exchange with the partials summed pairwise, p[t] + p[t + s] for s = world/2 .. 1 (world a power of
 * two): the order in which the GEMV contract's lane tree (bpd/kernelgen/emitters/q8_0_from_facts.pl:476) joins
 * lanes t and t + s.  With lt_q8_gemv_lanes partials this gives the bits of the one-GPU GEMV. */
int lt_allreduce_add_tree(const lt_comm* comm, const float* part, const float* resid, float* out, int n,
                          void* stream);

/* Greedy tokens of B sequences whose logits are split by vocabulary over the ranks of a comm: this rank
 * holds columns [v0, v0 + nv) as logits[b*ld + i].  Two launches: per-row partial maxima, then one CTA that
 * finishes each row, pushes this rank's (maximum, global index) to every rank as two tagged words (the
 * lt_allreduce_add exchange, elements 2b and 2b+1 of its first CTA, so the call must come at the same place
 * of the call sequence on every rank) and keeps the maximum over the ranks, lowest index on ties (the
 * reference's k_argmax_s1 / k_argmax_s2 rule, bpd/lib/dev_residency.py:226-271): tok[b] is the same on every
 * rank, with no host step in between.  comm NULL or world 1: no exchange, tok[b] = v0 + local index.
 * `partials` is caller scratch of lt_argmax_rows_scratch_bytes(B) bytes; 2*B <= 1024 and <= max_n of the comm.
 * Bounded waits (LT_STATUS_WAIT_TIMEOUT; tok[b] is left unwritten for a row whose wait gave up). */
int lt_argmax_rows(const lt_comm* comm, const float* logits, long ld, int nv, int v0, int B, void* partials,
                   int* tok, void* stream);
int lt_argmax_rows_scratch_bytes(int B);

/* Partial GEMV of a tensor-parallel row split that keeps the one-GPU bits.  The `group` ranks deal the Q8_0
 * blocks of every row round-robin (rank r holds blocks b = r mod group, i.e. the blocks of the contract's
 * lanes L = r mod group, q8_0_from_facts.pl:476); Wq / Wd are this rank's blocks, K its share of the row
 * length.  Lane chains in ascending block order and the tree levels that stay inside a rank; Y[t*M + n] is
 * the rank's partial.  Summing the ranks' partials in lt_allreduce_add_tree's order gives lt_q8_gemv's result
 * on the whole matrix bit for bit.  group 1, 2, 4 or 8 (group 1 = lt_q8_gemv). */
int lt_q8_gemv_lanes(const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq, const uint16_t* Xd, float* Y, int M,
                     int K, int T, int group, void* stream);

/* The tensor-parallel row-split projection (o_proj, down) of one sequence with the all-reduce inside the
 * GEMV: this rank folds its K-slice of every row (lt_q8_gemv arithmetic), a warp stores each finished partial
 * into every rank's staging memory at once and, when its rows are out, takes the partials of all ranks from
 * its own staging memory: Y[n] = Resid[n] + ((part_0[n] + part_1[n]) + ...) in rank order, the same bits as
 * lt_q8_gemv followed by lt_allreduce_add.  Same call sequence and the same M, K on every rank; M <= max_n of
 * the comm; Y may alias Resid.  Bounded waits (LT_STATUS_WAIT_TIMEOUT); a row's exchange is counted even
 * when its wait gave up, so the ranks stay in step.  Warps of different ranks wait for each other, so the
 * kernel is launched cooperatively (at most one resident wave): one process per GPU, nothing else may hold
 * the GPU's SMs for good while it runs. */
int lt_q8_gemv_allreduce(const lt_comm* comm, const int8_t* Wq, const uint16_t* Wd, const int8_t* Xq,
                         const uint16_t* Xd, const float* Resid, float* Y, int M, int K, void* stream);

/* ---- decode linear without caller scratch ----------------------------------------------
 * No counterpart in the reference (its engine allocates scratch with cuMemAlloc or from a
 * slab it owns).  Y[M] = W . quant(X[K]) (+ Resid), the same arithmetic as lt_quant_q8
 * followed by lt_q8_gemv with T = 1, for callers that may not allocate device memory: the
 * quantised activation lives in a 17 KiB __device__ array inside the library, which every
 * GPU that loads the library keeps until the process exits.
 *   - K must not exceed lt_q8_linear_static_max_k() (16384); larger K is rejected with
 *     LT_ERR_INVALID and a message, nothing is launched.
 *   - The first call on each device looks the array's address up; make that call before any
 *     stream capture begins on that device.
 *   - The entry point calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - All calls share the one array and it keeps the last call's contents (each call
 *     overwrites every byte it later reads).  Two calls whose kernels overlap on the GPU
 *     (different streams, or concurrent graphs) race on it: serialise them. */
int lt_q8_linear_static(const int8_t* Wq, const uint16_t* Wd, const float* X, const float* Resid,
                        float* Y, int M, int K, void* stream);
int lt_q8_linear_static_max_k(void);

/* ---- on-device token loop ---------------------------------------------------------------
 * no reference counterpart as a kernel: the reference copies the chosen token to the host
 * after every step (bpd/lib/dev_residency.py:1812-1818).  history[*step] = *tok; *step += 1;
 * lets a captured step feed its own argmax to the next replay and keeps the token trace. */
int lt_token_record(const int* tok, int* history, int* step, int capacity, void* stream);

/* Host-side helper for a loop that feeds every token back from the host (the reference's
 * GraphRunner.replay_token, bpd/lib/dev_residency.py:1626 ff.): copies the 4-byte token id from page-locked
 * h_tok to d_tok, launches graph_exec (a cudaGraphExec_t whose step reads d_tok and leaves the chosen token in
 * d_out), copies d_out to page-locked h_out and waits for the stream.  One call per token. */
int lt_graph_replay_token(void* graph_exec, void* stream, const int* h_tok, int* d_tok, const int* d_out, int* h_out);

#ifdef __cplusplus
}
#endif
#endif /* LLAMATOV_B200_H */
