"""GPU parity: every kernel of the decode path, called through the C ABI, against the CPU
oracle on the same seeded inputs.  Bit-exact wherever the arithmetic is reproducible on a
CPU (quantised bytes, integer dots, the GEMV fp32 order, argmax, KV rows); a stated
tolerance where a CUDA device function (rsqrtf, expf, __expf, powf, sinf, cosf) is involved."""
import ctypes

import numpy as np
import pytest
import torch

from llamatov_b200 import _lib, synth
from tests.gpu_util import bits, dev, gpu_gemv, gpu_quant, host, stream, ulp_diff

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ quantiser
@pytest.mark.parametrize("K", [32, 896, 4864, 4096, 14336])
def test_quant_bit_exact(oracle, K):
    rng = np.random.default_rng(K)
    x = rng.standard_normal(K).astype(np.float32)
    xq, xd = gpu_quant(x)
    oq, od = oracle.quant_q8(x)
    assert np.array_equal(host(xq), oq)
    assert np.array_equal(host(xd, np.uint16), od.view(np.uint16))


def test_quant_golden_and_edges(oracle, golden_dir):
    import os
    g = np.load(os.path.join(golden_dir, "quantize_q8_0.npz"))
    for n in sorted({k.split("__")[0] for k in g.files}):
        xq, xd = gpu_quant(g[n + "__x"])
        assert np.array_equal(host(xq), g[n + "__q"]), n
        assert np.array_equal(host(xd, np.uint16), g[n + "__d"]), n


def test_quant_batched_rows(oracle):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 896)).astype(np.float32)
    xq, xd = gpu_quant(x, rows=5)
    for r in range(5):
        oq, od = oracle.quant_q8(x[r])
        assert np.array_equal(host(xq).reshape(5, -1)[r], oq)
        assert np.array_equal(host(xd, np.uint16).reshape(5, -1)[r], od.view(np.uint16))


def test_silu_mul_quant(oracle):
    rng = np.random.default_rng(6)
    K = 4864
    g = (rng.standard_normal(K) * 2).astype(np.float32)
    u = rng.standard_normal(K).astype(np.float32)
    dg, du = dev(g), dev(u)
    xq = torch.empty(K, dtype=torch.int8, device="cuda")
    xd = torch.empty(K // 32, dtype=torch.int16, device="cuda")
    _lib.call("lt_silu_mul_quant", dg.data_ptr(), du.data_ptr(), xq.data_ptr(), xd.data_ptr(), K, 1, stream())
    y = torch.empty(K, dtype=torch.float32, device="cuda")
    _lib.call("lt_silu_mul", dg.data_ptr(), du.data_ptr(), y.data_ptr(), K, stream())
    v = host(y)
    # device expf differs from libm by a few ULP: the activation itself within 4 ULP ...
    assert ulp_diff(v, oracle.silu_mul(g, u)).max() <= 4
    # ... and the fused kernel is bit-identical to quantising the device's own activation
    oq, od = oracle.quant_q8(v)
    assert np.array_equal(host(xq), oq)
    assert np.array_equal(host(xd, np.uint16), od.view(np.uint16))


# ------------------------------------------------------------------ GEMV
GEMV_SHAPES = [(4864, 896), (896, 896), (128, 896), (896, 4864), (1152, 896), (9728, 896),
               (4096, 4096), (1024, 14336), (37, 64), (1, 32), (515, 1056)]


@pytest.mark.parametrize("M,K", GEMV_SHAPES)
def test_gemv_bit_exact(oracle, M, K):
    Wq, Wd, x = synth.gemv_case(M, K, seed=0)
    dWq, dWd = dev(Wq), dev(Wd)
    xq, xd = gpu_quant(x[0])
    oq, od = oracle.quant_q8(x[0])
    assert np.array_equal(host(xq), oq) and np.array_equal(host(xd, np.uint16), od.view(np.uint16))
    y = host(gpu_gemv(dWq, dWd, xq, xd, M, K))
    want = oracle.q8_gemv(Wq, Wd, oq, od, M, K)
    assert ulp_diff(y, want).max() == 0
    assert np.array_equal(bits(y), bits(want))
    # residual / bias epilogue
    r = np.random.default_rng(1).standard_normal(M).astype(np.float32)
    y2 = host(gpu_gemv(dWq, dWd, xq, xd, M, K, resid=dev(r)))
    assert np.array_equal(bits(y2), bits(oracle.q8_gemv(Wq, Wd, oq, od, M, K, resid=r)))


def test_gemv_lm_head_shape(oracle):
    M, K = 151936, 896
    Wq, Wd, x = synth.gemv_case(M, K, seed=0)
    xq, xd = gpu_quant(x[0])
    y = host(gpu_gemv(dev(Wq), dev(Wd), xq, xd, M, K))
    want = oracle.q8_gemv(Wq, Wd, *oracle.quant_q8(x[0]), M, K)
    assert np.array_equal(bits(y), bits(want))


@pytest.mark.parametrize("M,K", [(14336, 4096), (128256, 4096), (4096, 14336)])
def test_gemv_llama_shapes_bit_exact(oracle, M, K):
    """The Llama-3-8B-architecture shapes of the sweep at one column, against the CPU oracle (rows sampled for
    the vocabulary-sized matrix so that the oracle stays within seconds; the GPU computes all rows)."""
    Wq, Wd, x = synth.gemv_case(M, K, seed=3)
    xq, xd = gpu_quant(x[0])
    y = host(gpu_gemv(dev(Wq), dev(Wd), xq, xd, M, K))
    oq, od = oracle.quant_q8(x[0])
    nb = K // 32
    if M > 20000:
        rows = np.unique(np.concatenate([np.arange(0, 64), np.arange(M - 64, M),
                                         np.random.default_rng(0).integers(0, M, size=4096)]))
        Wq_s = np.ascontiguousarray(Wq.reshape(M, K)[rows]).reshape(-1)
        Wd_s = np.ascontiguousarray(Wd.reshape(M, nb)[rows]).reshape(-1)
        want = oracle.q8_gemv(Wq_s, Wd_s, oq, od, len(rows), K)
        assert np.array_equal(bits(y[rows]), bits(want))
    else:
        assert np.array_equal(bits(y), bits(oracle.q8_gemv(Wq, Wd, oq, od, M, K)))


@pytest.mark.parametrize("T", [4, 16, 64])
def test_skinny_gemm_wide_matrix_bit_exact(oracle, T):
    """Batches of 4, 16 and 64 columns on a 4096-row matrix (dp4a path and tensor-core path)."""
    M, K = 4096, 4096
    Wq, Wd, x = synth.gemv_case(M, K, T=T, seed=40 + T)
    xq, xd = gpu_quant(x, rows=T)
    y = host(gpu_gemv(dev(Wq), dev(Wd), xq, xd, M, K, T=T)).reshape(T, M)
    want = oracle.q8_gemm(Wq, Wd, host(xq), host(xd, np.uint16), M, K, T)
    assert np.array_equal(bits(y), bits(want))


@pytest.mark.parametrize("T", [2, 3, 4, 8, 16, 33, 64, 70])
@pytest.mark.parametrize("M,K", [(896, 896), (300, 4864), (200, 1056)])
def test_skinny_gemm_bit_exact(oracle, M, K, T):
    Wq, Wd, x = synth.gemv_case(M, K, T=T, seed=T)
    xq, xd = gpu_quant(x, rows=T)
    r = np.random.default_rng(2).standard_normal(M).astype(np.float32)
    y = host(gpu_gemv(dev(Wq), dev(Wd), xq, xd, M, K, T=T, resid=dev(r))).reshape(T, M)
    want = oracle.q8_gemm(Wq, Wd, host(xq), host(xd, np.uint16), M, K, T) + r[None, :]
    assert np.array_equal(bits(y), bits(want))


def gpu_gemm_tc(dWq, dWd, dXq, dXd, M, K, T, variant, resid=None, resid_ld=0):
    y = torch.full((T * M,), float("nan"), dtype=torch.float32, device="cuda")
    _lib.call("lt_q8_gemm_tc", dWq.data_ptr(), dWd.data_ptr(), dXq.data_ptr(), dXd.data_ptr(),
              None if resid is None else resid.data_ptr(), resid_ld, y.data_ptr(), M, K, T, variant, stream())
    return y


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("M,K,T", [(128, 128, 16), (128, 896, 16), (896, 896, 64), (300, 4864, 33), (1152, 896, 70),
                                   (256, 4096, 5), (200, 14336, 17), (4864, 896, 257)])
def test_tensor_core_gemm_bit_exact(oracle, M, K, T, variant):
    Wq, Wd, x = synth.gemv_case(M, K, T=T, seed=T + variant)
    xq, xd = gpu_quant(x, rows=T)
    r = np.random.default_rng(2).standard_normal(M).astype(np.float32)
    dWq, dWd = dev(Wq), dev(Wd)
    want = oracle.q8_gemm(Wq, Wd, host(xq), host(xd, np.uint16), M, K, T)
    y = host(gpu_gemm_tc(dWq, dWd, xq, xd, M, K, T, variant)).reshape(T, M)
    assert np.array_equal(bits(y), bits(want))
    y = host(gpu_gemm_tc(dWq, dWd, xq, xd, M, K, T, variant, resid=dev(r))).reshape(T, M)
    assert np.array_equal(bits(y), bits(want + r[None, :]))
    # one residual row per column (the residual stream of a prefill)
    R = np.random.default_rng(3).standard_normal((T, M)).astype(np.float32)
    y = host(gpu_gemm_tc(dWq, dWd, xq, xd, M, K, T, variant, resid=dev(R), resid_ld=M)).reshape(T, M)
    assert np.array_equal(bits(y), bits(want + R))
    assert _lib.device_status() == set()


@pytest.mark.parametrize("M,K,T", [(4864, 896, 1), (96, 896, 5), (64, 4864, 4), (33, 1024, 2), (50, 896, 7)])
def test_ggml_order_mode_bit_exact(oracle, M, K, T):
    # the fold order of the reference's compiled CPU path (the oracle restatement is pinned to that
    # library bit for bit on the CPU, tests/test_oracle_golden.py)
    Wq, Wd, x = synth.gemv_case(M, K, T=T, seed=T)
    dx = dev(x.reshape(-1))
    xq = torch.empty(T * K, dtype=torch.int8, device="cuda"); xd = torch.empty(T * K // 32, dtype=torch.int16, device="cuda")
    _lib.call("lt_quant_q8_ggml", dx.data_ptr(), xq.data_ptr(), xd.data_ptr(), K, T, stream())
    oq = np.stack([oracle.quant_q8_ggml(x[t])[0] for t in range(T)])
    od = np.stack([oracle.quant_q8_ggml(x[t])[1] for t in range(T)])
    assert np.array_equal(host(xq).reshape(T, K), oq)
    assert np.array_equal(host(xd, np.uint16).reshape(T, -1), od.view(np.uint16))
    y = torch.empty(T * M, dtype=torch.float32, device="cuda")
    dWq, dWd = dev(Wq), dev(Wd)
    _lib.call("lt_q8_gemm_ggml", dWq.data_ptr(), dWd.data_ptr(), xq.data_ptr(), xd.data_ptr(), y.data_ptr(),
              M, K, T, stream())
    want = oracle.q8_gemm_ggml(Wq, Wd, oq, od, M, K, T)
    assert np.array_equal(bits(host(y).reshape(T, M)), bits(want))


def test_gemv_linearity_full_size():
    # size-independent property at the LM-head size: W(x1 quantised) + W(x2 quantised) rows are
    # independent of which other rows are computed (row-slice consistency), and the result does
    # not depend on the launch (two calls, bitwise equal).
    M, K = 151936, 896
    Wq, Wd, x = synth.gemv_case(M, K, seed=3)
    dWq, dWd = dev(Wq), dev(Wd)
    xq, xd = gpu_quant(x[0])
    y1 = host(gpu_gemv(dWq, dWd, xq, xd, M, K))
    y2 = host(gpu_gemv(dWq, dWd, xq, xd, M, K))
    assert np.array_equal(bits(y1), bits(y2))
    lo = 70000
    ys = host(gpu_gemv(dWq[lo * K:], dWd[lo * (K // 32):], xq, xd, M - lo, K))
    assert np.array_equal(bits(ys), bits(y1[lo:]))


def test_gemv_rejects_bad_arguments():
    t = torch.zeros(64, dtype=torch.int8, device="cuda")
    rc = _lib.lib().lt_q8_gemv(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 1, 40, 1, None)
    assert rc == 1 and "multiple of 32" in _lib.last_error()


# ------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("M,N,eps", [(1, 896, 1e-6), (3, 4096, 1e-5), (2, 100, 1e-6)])
def test_rmsnorm(oracle, M, N, eps):
    rng = np.random.default_rng(N)
    x = rng.standard_normal((M, N)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(N)).astype(np.float32)
    dx, dw = dev(x), dev(w)
    y = torch.empty_like(dx)
    _lib.call("lt_rmsnorm", dx.data_ptr(), dw.data_ptr(), y.data_ptr(), M, N, eps, stream())
    got = host(y)
    want = oracle.rmsnorm(x, w, eps)
    # rsqrtf (device) vs 1/sqrtf (host): at most 2 ULP on inv, so <= 3 ULP on y
    assert ulp_diff(got, want).max() <= 4
    # the sum of squares and everything after rsqrtf are bit-exact: recover inv from a unit
    # weight / unit element and replay the oracle with the device's own inv
    ones = dev(np.ones(N, np.float32))
    probe = dx.clone(); probe[:, 0] = 1.0
    y1 = torch.empty_like(dx)
    _lib.call("lt_rmsnorm", probe.data_ptr(), ones.data_ptr(), y1.data_ptr(), M, N, eps, stream())
    inv = host(y1)[:, 0].copy()                    # (1*inv)*1 == inv exactly
    xp = x.copy(); xp[:, 0] = 1.0
    want2 = oracle.rmsnorm(xp, np.ones(N, np.float32), eps, inv_override=inv)
    assert np.array_equal(bits(host(y1)), bits(want2))


# ------------------------------------------------------------------ RoPE
def test_rmsnorm_quant_equals_the_two_launches():
    rng = np.random.default_rng(5)
    M, N = 3, 4096
    x = rng.standard_normal((M, N)).astype(np.float32) * 3
    w = (1 + 0.1 * rng.standard_normal(N)).astype(np.float32)
    dx, dw = dev(x.reshape(-1)), dev(w)
    y = torch.empty(M * N, device="cuda"); y2 = torch.empty(M * N, device="cuda")
    xq = torch.empty(M * N, dtype=torch.int8, device="cuda"); xd = torch.empty(M * N // 32, dtype=torch.int16, device="cuda")
    xq2 = torch.empty_like(xq); xd2 = torch.empty_like(xd)
    _lib.call("lt_rmsnorm", dx.data_ptr(), dw.data_ptr(), y.data_ptr(), M, N, 1e-5, stream())
    _lib.call("lt_quant_q8", y.data_ptr(), xq.data_ptr(), xd.data_ptr(), N, M, stream())
    _lib.call("lt_rmsnorm_quant", dx.data_ptr(), dw.data_ptr(), y2.data_ptr(), xq2.data_ptr(), xd2.data_ptr(), M, N, 1e-5,
              stream())
    assert np.array_equal(bits(host(y)), bits(host(y2)))
    assert np.array_equal(host(xq), host(xq2)) and np.array_equal(host(xd), host(xd2))
    _lib.call("lt_rmsnorm_quant", dx.data_ptr(), dw.data_ptr(), None, xq2.data_ptr(), xd2.data_ptr(), M, N, 1e-5, stream())
    assert np.array_equal(host(xq), host(xq2)) and np.array_equal(host(xd), host(xd2))


@pytest.mark.parametrize("M,K", [(1152, 896), (9728, 896), (6144, 4096), (28672, 4096), (151936, 896), (40, 14336)])
def test_rmsnorm_q8_gemv_equals_the_three_launches(M, K):
    """The projection with the RMSNorm + quantiser prologue gives the bits of lt_rmsnorm, lt_quant_q8, lt_q8_gemv."""
    rng = np.random.default_rng(M + K)
    Wq = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    Wd = (np.abs(rng.standard_normal((M, K // 32))) * 0.02).astype(np.float16)
    x = rng.standard_normal(K).astype(np.float32) * 2
    w = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    res = rng.standard_normal(M).astype(np.float32)
    dWq, dWd, dx, dw, dres = dev(Wq.reshape(-1)), dev(Wd.view(np.int16).reshape(-1)), dev(x), dev(w), dev(res)
    h = torch.empty(K, device="cuda")
    xq = torch.empty(K, dtype=torch.int8, device="cuda"); xd = torch.empty(K // 32, dtype=torch.int16, device="cuda")
    y = torch.empty(M, device="cuda"); y2 = torch.empty(M, device="cuda")
    for resid in (None, dres):
        rp = None if resid is None else resid.data_ptr()
        _lib.call("lt_rmsnorm", dx.data_ptr(), dw.data_ptr(), h.data_ptr(), 1, K, 1e-5, stream())
        _lib.call("lt_quant_q8", h.data_ptr(), xq.data_ptr(), xd.data_ptr(), K, 1, stream())
        _lib.call("lt_q8_gemv", dWq.data_ptr(), dWd.data_ptr(), xq.data_ptr(), xd.data_ptr(), rp, y.data_ptr(), M, K, 1,
                  stream())
        _lib.call("lt_rmsnorm_q8_gemv", dWq.data_ptr(), dWd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 1e-5, rp,
                  y2.data_ptr(), M, K, stream())
        assert np.array_equal(bits(host(y)), bits(host(y2)))


@pytest.mark.parametrize("theta,hd,nh", [(1e6, 64, 16), (5e5, 128, 40)])
def test_rope(oracle, theta, hd, nh):
    rng = np.random.default_rng(int(hd))
    for pos in (0, 1, 31, 159, 4095):
        x = rng.standard_normal((1, nh * hd)).astype(np.float32)
        dx = dev(x)
        dp = torch.tensor([pos], dtype=torch.int32, device="cuda")
        _lib.call("lt_rope", dx.data_ptr(), dp.data_ptr(), 1, nh, hd, theta, stream())
        got = host(dx)
        want = oracle.rope(x, [pos], nh, hd, theta)
        # powf/sinf/cosf are device functions: angle error ~ pos * 1e-7, values O(1)
        tol = 2e-6 + pos * 4e-7
        assert np.max(np.abs(got - want)) <= tol, (pos, np.max(np.abs(got - want)))
        if pos == 0:
            assert np.array_equal(bits(got), bits(x))
        # rotation preserves the norm of every pair
        h = hd // 2
        g = got.reshape(nh, hd); xx = x.reshape(nh, hd)
        assert np.allclose(g[:, :h] ** 2 + g[:, h:] ** 2, xx[:, :h] ** 2 + xx[:, h:] ** 2, rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------ KV append
def test_append_kv_and_overflow_flag():
    width, max_seq = 128, 4
    kb = torch.zeros(max_seq * width, device="cuda"); vb = torch.zeros(max_seq * width, device="cuda")
    ln = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = []
    for i in range(max_seq):
        k = torch.full((width,), float(i + 1), device="cuda"); v = -k
        rows.append((k, v))
        _lib.call("lt_append_kv", kb.data_ptr(), k.data_ptr(), vb.data_ptr(), v.data_ptr(), ln.data_ptr(), width,
                  max_seq, 1, stream())
    assert int(ln.item()) == max_seq
    assert torch.equal(kb.view(max_seq, width)[:, 0].cpu(), torch.arange(1, max_seq + 1, dtype=torch.float32))
    assert torch.equal(vb, -kb)
    assert _lib.device_status() == set()
    # one more append is refused, flagged, and changes nothing
    before = kb.clone()
    _lib.call("lt_append_kv", kb.data_ptr(), rows[0][0].data_ptr(), vb.data_ptr(), rows[0][1].data_ptr(),
              ln.data_ptr(), width, max_seq, 1, stream())
    assert _lib.device_status() == {"kv_overflow"}
    assert torch.equal(kb, before) and int(ln.item()) == max_seq
    assert _lib.device_status() == set()
    # wide rows (Llama-3-8B: 1024) and no-increment form
    width = 1024
    kb = torch.zeros(3 * width, device="cuda"); vb = torch.zeros(3 * width, device="cuda")
    ln = torch.tensor([1], dtype=torch.int32, device="cuda")
    k = torch.randn(width, device="cuda"); v = torch.randn(width, device="cuda")
    _lib.call("lt_append_kv", kb.data_ptr(), k.data_ptr(), vb.data_ptr(), v.data_ptr(), ln.data_ptr(), width, 3, 0, stream())
    assert int(ln.item()) == 1 and torch.equal(kb[width:2 * width], k) and torch.equal(vb[width:2 * width], v)
    _lib.call("lt_incr_len", ln.data_ptr(), stream())
    assert int(ln.item()) == 2


# ------------------------------------------------------------------ attention
def _attn(q, kc, vc, L, hd, nh, nkv, maxt):
    out = torch.empty(nh * hd, device="cuda")
    ln = torch.tensor([L], dtype=torch.int32, device="cuda")
    _lib.call("lt_attn_decode_masked", q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ln.data_ptr(), out.data_ptr(),
              hd, nh, nkv, float(np.float32(hd ** -0.5)), maxt, stream())
    return host(out)


@pytest.mark.parametrize("nh,nkv,hd,maxt", [(14, 2, 64, 256), (32, 8, 128, 512)])
def test_attention_vs_oracle_and_poison(oracle, nh, nkv, hd, maxt):
    rng = np.random.default_rng(hd)
    q = rng.standard_normal(nh * hd).astype(np.float32)
    kc = rng.standard_normal((maxt, nkv, hd)).astype(np.float32)
    vc = rng.standard_normal((maxt, nkv, hd)).astype(np.float32)
    dq = dev(q)
    for L in (1, 2, maxt // 2, maxt - 1, maxt):
        got = _attn(dq, dev(kc), dev(vc), L, hd, nh, nkv, maxt)
        want = oracle.attn_decode_masked(q, kc, vc, L, hd, nh, nkv, np.float32(hd ** -0.5), maxt)
        # __expf (device) vs expf (host): bound from the reference's own soft gate, 5e-6
        assert np.max(np.abs(got - want)) < 5e-6, L
        # poison: NaN / Inf / garbage beyond L must not change a single bit
        kp, vp = kc.copy(), vc.copy()
        kp[L:] = np.nan; vp[L:] = np.inf
        got_p = _attn(dq, dev(kp), dev(vp), L, hd, nh, nkv, maxt)
        assert np.array_equal(bits(got), bits(got_p)), L
        kp[L:] = 1e30; vp[L:] = -1e30
        assert np.array_equal(bits(got), bits(_attn(dq, dev(kp), dev(vp), L, hd, nh, nkv, maxt)))
    assert _lib.device_status() == set()


def test_attention_bad_length_is_flagged_not_faulted():
    nh, nkv, hd, maxt = 4, 2, 32, 64
    q = torch.randn(nh * hd, device="cuda"); kc = torch.randn(maxt * nkv * hd, device="cuda"); vc = torch.randn_like(kc)
    _attn(q, kc, vc, maxt + 5, hd, nh, nkv, maxt)
    assert _lib.device_status() == {"bad_length"}


# ------------------------------------------------------------------ argmax / embedding
def test_argmax_exact(oracle):
    rng = np.random.default_rng(0)
    part = torch.empty(_lib.lib().lt_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    for n in (1, 5, 255, 256, 257, 151936, 128256):
        v = rng.standard_normal(n).astype(np.float32)
        dv = dev(v)
        _lib.call("lt_argmax", dv.data_ptr(), n, part.data_ptr(), out.data_ptr(), stream())
        assert int(out.item()) == oracle.argmax(v) == int(np.argmax(v))
    v = np.zeros(151936, np.float32); v[[777, 90000, 151935]] = 3.5      # ties -> lowest index
    dv = dev(v)
    _lib.call("lt_argmax", dv.data_ptr(), v.size, part.data_ptr(), out.data_ptr(), stream())
    assert int(out.item()) == 777
    v[:] = -np.inf                                                       # reference sentinel
    dv = dev(v)
    _lib.call("lt_argmax", dv.data_ptr(), v.size, part.data_ptr(), out.data_ptr(), stream())
    assert int(out.item()) == oracle.argmax(v) == 2147483647


def test_argmax_rows_exact(oracle):
    """lt_argmax_rows without a comm: every row's argmax (lowest index on ties) plus the slice offset v0, rows
    taken from a wider matrix (ld > nv)."""
    rng = np.random.default_rng(1)
    for B, nv, ld, v0 in ((1, 5, 5, 0), (3, 257, 300, 1000), (32, 16032, 16032, 16032 * 3), (40, 4097, 4100, 7),
                          (2, 151936, 151936, 0)):
        m = rng.standard_normal((B, ld)).astype(np.float32)
        if nv > 300:
            m[0, [nv - 1, 17, 200]] = 9.0                               # ties -> lowest index
            m[B - 1, :nv] = -np.inf                                      # reference sentinel
        if ld > nv:
            m[:, nv:] = 100.0                                            # outside the slice: must be ignored
        dm = dev(m)
        part = torch.empty(_lib.lib().lt_argmax_rows_scratch_bytes(B), dtype=torch.uint8, device="cuda")
        out = torch.full((B,), -5, dtype=torch.int32, device="cuda")
        _lib.call("lt_argmax_rows", None, dm.data_ptr(), ld, nv, v0, B, part.data_ptr(), out.data_ptr(), stream())
        got = host(out)
        for b in range(B):
            want = oracle.argmax(m[b, :nv])
            assert int(got[b]) == (want + v0 if want != 2147483647 else want), (B, nv, b)
    assert not _lib.device_status()


def test_embed_gather(oracle):
    V, E = 1000, 896
    Wq, Wd, _ = synth.gemv_case(V, E, seed=5)
    dWq, dWd = dev(Wq), dev(Wd)
    out = torch.empty(E, device="cuda")
    for tok in (0, 1, 999):
        dt = torch.tensor([tok], dtype=torch.int32, device="cuda")
        _lib.call("lt_embed_q8", dWq.data_ptr(), dWd.data_ptr(), dt.data_ptr(), out.data_ptr(), E, V, stream())
        assert np.array_equal(bits(host(out)), bits(oracle.embed_q8(Wq, Wd, tok, E)))
    dt = torch.tensor([V], dtype=torch.int32, device="cuda")
    _lib.call("lt_embed_q8", dWq.data_ptr(), dWd.data_ptr(), dt.data_ptr(), out.data_ptr(), E, V, stream())
    assert _lib.device_status() == {"bad_token"}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_in_one_process(oracle):
    """Function attributes and occupancy are per device: a GEMV that needs more than 48 KB of dynamic shared
    memory on cuda:1 after the same call on cuda:0, both against the oracle."""
    M, K = 256, 8192
    Wq, Wd, x = synth.gemv_case(M, K, T=1, seed=31)
    xq, xd = oracle.quant_q8(x[0])
    want = oracle.q8_gemv(Wq, Wd, xq, xd, M, K)
    for d in (0, 1, 0):
        with torch.cuda.device(d):
            dWq, dWd = dev(Wq), dev(Wd)
            dxq, dxd = dev(xq), dev(xd)
            y = torch.empty(M, dtype=torch.float32, device="cuda")
            _lib.call("lt_q8_gemv", dWq.data_ptr(), dWd.data_ptr(), dxq.data_ptr(), dxd.data_ptr(), None, y.data_ptr(), M, K, 1, stream())
            torch.cuda.synchronize()
            assert np.array_equal(bits(host(y)), bits(want)), d
            assert _lib.device_status() == set()
