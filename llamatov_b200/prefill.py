"""Prompt prefill in one pass over the weights.

The reference prefills by running its one-token step once per prompt token
(`forward_pass_resident` recursing, bpd/lib/dev_residency.py:1344-1350) and demands that a
batched form give the same numbers.  `prefill_resident` here runs the same layer sequence
(bpd/lib/dev_residency.py:1381-1477) on all rows of a prompt chunk at once: row-batched
RMSNorm / quantiser / rope / append, the Q8_0 GEMMs on the tensor cores (`lt_q8_gemm_tc`),
causal attention over the rows just appended (`lt_attn_prefill`).  Every row gets exactly the
arithmetic the one-token step would give it, so the KV cache, the final hidden state and the
logits are bit-identical to the token-by-token prefill (tests/test_gpu_prefill.py).

Several sequences can be prefilled together (`toks` of shape [B, T], one KV-cache list per
sequence): the GEMMs then run over B*T rows, rope / append / attention per sequence.
"""
import numpy as np
import torch

from . import _lib
from . import dev_residency as dr
from .fact_dispatch import Q8Weight

# Rows per pass.  The activations of a pass stay resident (a [rows, 2F] fp32 gate|up buffer is
# the largest); 16384 rows of the 0.5B architecture are 0.6 GB.
MAX_ROWS = 16384


def _embedding_rows(w, toks_flat, E):
    """[n, E] fp32 rows of the embedding table on the device."""
    n = int(toks_flat.numel())
    out = torch.empty((n, E), dtype=torch.float32, device="cuda")
    emb = w["token_embd.weight"]
    if isinstance(dr._np(emb), Q8Weight):
        dWq, dWd, V, _ = dr._weights(dr._np(emb))
        dt = toks_flat.to(device="cuda", dtype=torch.int32)
        _lib.call("lt_embed_q8_rows", dWq, dWd, dt.data_ptr(), out.data_ptr(), E, V, n, dr._stream())
        torch.cuda.current_stream().synchronize()
    else:
        rows = np.stack([dr._embedding_row(w, int(t), E) for t in toks_flat.tolist()])
        out.copy_(torch.from_numpy(rows))
    return out


def supported(cfg, w):
    """The batched path needs row lengths that the tiled weight loads accept and a head size
    the chunk attention is built for; anything else prefills token by token."""
    E = cfg["n_embd"]
    hd = E // cfg["n_head"]
    F = dr._fused_gateup_weight(w, "blk.0")[2][0]
    return E % 128 == 0 and F % 128 == 0 and (cfg["n_head"] * hd) % 128 == 0 and hd in (64, 128)


def prefill_resident(w, cfg, toks, kv_caches, want_logits=True):
    """Run a prompt (chunk) through all layers with batched rows.

    toks: int tensor [T] or [B, T].  kv_caches: the per-layer cache list of the sequence (or a
    list of B such lists); caches are created on first use exactly as the one-token path does.
    Positions continue from each cache's current length.  Returns the logits of the last row
    of the last sequence as a [1, 1, V] tensor, like `forward_pass_resident`.
    """
    if toks.dim() == 1:
        toks = toks.reshape(1, -1)
        kv_caches = [kv_caches]
    B, T = int(toks.shape[0]), int(toks.shape[1])
    if B * T > MAX_ROWS:
        raise RuntimeError(f"prefill_resident: {B}x{T} rows exceed MAX_ROWS={MAX_ROWS}; split the prompt in chunks")
    nh, nkv, E = cfg["n_head"], cfg["n_head_kv"], cfg["n_embd"]
    hd = E // nh
    nq, nk = nh * hd, nkv * hd
    nl = cfg["n_layers"]
    eps, theta = float(cfg["norm_eps"]), float(cfg["rope_theta"])
    scale = float(np.float32(hd ** -0.5))
    R = B * T
    st = dr._stream
    f32 = dict(dtype=torch.float32, device="cuda")
    i8 = dict(dtype=torch.int8, device="cuda")
    i16 = dict(dtype=torch.int16, device="cuda")

    x = _embedding_rows(w, toks.reshape(-1), E)                  # residual stream [R, E]
    x1 = torch.empty((R, E), **f32)
    h = torch.empty((R, E), **f32)
    F = dr._fused_gateup_weight(w, "blk.0")[2][0]
    qkv = torch.empty((R, nq + 2 * nk), **f32)
    att = torch.empty((R, nq), **f32)
    gu = torch.empty((R, 2 * F), **f32)
    kmax = max(E, nq, F)
    xq = torch.empty(R * kmax, **i8)
    xd = torch.empty(R * (kmax // 32), **i16)

    def gemm(Wt, K, N, y, resid=None, resid_ld=0):
        dWq, dWd, n_, k_ = dr._weights(Wt)
        assert n_ == N and k_ == K, (n_, N, k_, K)
        _lib.call("lt_q8_gemm_tc", dWq, dWd, xq.data_ptr(), xd.data_ptr(),
                  None if resid is None else dr._vp(resid), resid_ld, y.data_ptr(), N, K, R, 0, st())

    for il in range(nl):
        p = f"blk.{il}"
        _lib.call("lt_rmsnorm", x.data_ptr(), dr._dev_const(dr._np(w[f"{p}.attn_norm.weight"])), h.data_ptr(),
                  R, E, eps, st())
        _lib.call("lt_quant_q8", h.data_ptr(), xq.data_ptr(), xd.data_ptr(), E, R, st())
        Wqkv, bcat, _ = dr._fused_qkv_weight(w, p)
        gemm(Wqkv, E, nq + 2 * nk, qkv, None if bcat is None else dr._dev_const(bcat), 0)
        for b in range(B):
            caches = kv_caches[b]
            if caches[il] is None:
                caches[il] = dr.DeviceKVCache(dr._KV_MAX_SEQ, nkv, hd)
            c = caches[il]
            lp = c._ensure_len_ptr(seed=True)
            if c.length + T > c.max_seq:
                raise RuntimeError(f"KV cache overflow: {c.length}+{T} > {c.max_seq}")
            rows = qkv[b * T:(b + 1) * T]
            _lib.call("lt_rope_rows", rows.data_ptr(), nq + 2 * nk, lp, T, nh + nkv, hd, theta, st())
            _lib.call("lt_append_kv_rows", c.k_ptr, rows.data_ptr() + nq * 4, c.v_ptr,
                      rows.data_ptr() + (nq + nk) * 4, nq + 2 * nk, lp, c.width, c.max_seq, T, 1, st())
            c.length += T
            _lib.call("lt_attn_prefill", rows.data_ptr(), nq + 2 * nk, c.k_ptr, c.v_ptr, lp,
                      att[b * T:(b + 1) * T].data_ptr(), nq, hd, nh, nkv, scale, T, c.length, st())
        _lib.call("lt_quant_q8", att.data_ptr(), xq.data_ptr(), xd.data_ptr(), nq, R, st())
        gemm(dr._np(w[f"{p}.attn_output.weight"]), nq, E, x1, x.data_ptr(), E)
        _lib.call("lt_rmsnorm", x1.data_ptr(), dr._dev_const(dr._np(w[f"{p}.ffn_norm.weight"])), h.data_ptr(),
                  R, E, eps, st())
        _lib.call("lt_quant_q8", h.data_ptr(), xq.data_ptr(), xd.data_ptr(), E, R, st())
        Wgu, _b, (ng, _nu) = dr._fused_gateup_weight(w, p)
        gemm(Wgu, E, 2 * F, gu)
        _lib.call("lt_silu_mul_quant_rows", gu.data_ptr(), gu.data_ptr() + F * 4, 2 * F, xq.data_ptr(),
                  xd.data_ptr(), F, R, st())
        gemm(dr._np(w[f"{p}.ffn_down.weight"]), F, E, x, x1.data_ptr(), E)

    # the last row's hidden state goes where the one-token path leaves it
    _rin, rout = dr._ensure_resid(E)
    dr._memcpy_dtod(dr._addr(rout.ptr), x[R - 1].data_ptr(), E * 4)
    if not want_logits:
        torch.cuda.synchronize()
        return None
    dr._ensure_logits_buf(E, w)
    dr._ensure_logits_scratch(E)
    lbuf = dr._compute_folded_logits(w, cfg, E)
    torch.cuda.synchronize()
    return torch.from_numpy(lbuf.to_host()).reshape(1, 1, lbuf.n)
