"""CPU: the oracle (oracle/lt_oracle.c) against the golden vectors produced by the
reference's own Python host functions (tests/golden/make_golden.py), plus self-checks of
the restated arithmetic that need no reference (fp16 conversion, integer dots, the
declared reduction orders against straightforward numpy renderings)."""
import os

import numpy as np
import pytest


def _ulp_diff(a, b):
    a = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7fffffff), a)
    b = np.where(b < 0, -(b & 0x7fffffff), b)
    return np.abs(a - b)


def test_f16_conversion_all_halfs(oracle):
    # every fp16 bit pattern round-trips, and f2h agrees with numpy on random floats
    hs = np.arange(65536, dtype=np.uint16)
    for h in hs[::7]:
        f = hs[h:h + 1].view(np.float16).astype(np.float32)[0]
        got = oracle.h2f(h)
        if np.isnan(f):
            assert np.isnan(got)
        else:
            assert got == f
            assert oracle.f2h(f) == h or (f == 0 and (oracle.f2h(f) & 0x7fff) == 0)
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 1e3, 7e4)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f2h(x) for x in xs], np.uint16)
    assert np.array_equal(got, want)
    # exact ties: halfway between two adjacent halfs rounds to even
    for h in (0x3c00, 0x3c01, 0x0001, 0x03ff, 0x7bfe):
        a = np.array([h, h + 1], np.uint16).view(np.float16).astype(np.float64)
        mid = np.float32((a[0] + a[1]) / 2)
        assert oracle.f2h(mid) == (h if h % 2 == 0 else h + 1)


def test_quantize_q8_0_matches_reference(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "quantize_q8_0.npz"))
    names = sorted({k.split("__")[0] for k in g.files})
    assert names
    for n in names:
        x, q, d = g[n + "__x"], g[n + "__q"], g[n + "__d"]
        xq, xd = oracle.quant_q8(x)
        assert np.array_equal(xd.view(np.uint16), d), n
        assert np.array_equal(xq, q), n


def test_weight_quantizer_matches_reference(golden_dir):
    # the product's host weight quantiser (a mirror of the reference's) on the same matrix
    from llamatov_b200 import fact_dispatch as fd
    g = np.load(os.path.join(golden_dir, "quantize_weight_q8_0.npz"))
    Wq, Wd, N, K = fd._quantize_weight_q8_0(g["W"])
    assert (N, K) == (int(g["N"]), int(g["K"]))
    assert np.array_equal(Wq, g["Wq"]) and np.array_equal(Wd.view(np.uint16), g["Wd"])
    # and the activation quantiser of the product's host side against the oracle
    x = g["W"][:, 0].copy()
    q, d = fd.quantize_q8_0(x)
    from oracle import oracle as o
    oq, od = o.quant_q8(x)
    assert np.array_equal(q, oq) and np.array_equal(d.view(np.uint16), od.view(np.uint16))


def test_synth_quant_rows_idempotent():
    # quantise -> dequantise -> quantise reproduces the blocks (the fp32 boundary and the
    # direct Q8_0 boundary carry the same weights)
    from llamatov_b200 import synth, fact_dispatch as fd
    rng = np.random.default_rng(3)
    w = synth._rand_q8(rng, 40, 96, 0.02)
    Wq, Wd, N, K = fd._quantize_weight_q8_0(w.dequant())
    assert np.array_equal(Wq, w.Wq) and np.array_equal(Wd.view(np.uint16), w.Wd.view(np.uint16))


def test_dequant_matches_reference(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "dequant_q8_0.npz"))
    K, N = int(g["K"]), int(g["N"])
    raw = g["raw"]
    d = raw[:, :2].copy().view(np.uint16).reshape(-1)
    q = raw[:, 2:].copy().view(np.int8).reshape(-1)
    for n in range(N):
        row = oracle.embed_q8(q, d, n, K)
        assert np.array_equal(row, g["deq"][:, n])


def test_rope_soft_vs_reference(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "rope_soft.npz"))
    nh, nkv, hd = int(g["nh"]), int(g["nkv"]), int(g["hd"])
    for theta in (1e6, 5e5):
        got_q = oracle.rope(g["q"][0], g["pos"], nh, hd, theta)
        got_k = oracle.rope(g["k"][0], g["pos"], nkv, hd, theta)
        assert np.max(np.abs(got_q - g[f"q_{theta:g}"][0])) < 2e-4   # position 159: angle error ~1e-5
        assert np.max(np.abs(got_k - g[f"k_{theta:g}"][0])) < 2e-4
    # position 0 is the identity, exactly
    q0 = oracle.rope(g["q"][0][:1], [0], nh, hd, 1e6)
    assert np.array_equal(q0, g["q"][0][:1])


def test_rmsnorm_soft_vs_reference(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "rmsnorm_soft.npz"))
    y = oracle.rmsnorm(g["x"], g["w"], float(g["eps"]))
    assert np.max(np.abs(y - g["y"]) / (np.abs(g["y"]) + 1e-6)) < 5e-6


def test_rms_sumsq_order(oracle):
    # numpy rendering of the declared order: 256 strided lanes (fma emulated exactly in
    # float64: x*x is exact in double, one rounding of the sum to fp32), pairwise tree
    rng = np.random.default_rng(5)
    for N in (896, 4096, 100, 256, 1):
        x = rng.standard_normal(N).astype(np.float32)
        p = np.zeros(256, np.float32)
        for t in range(256):
            acc = np.float32(0)
            for j in range(t, N, 256):
                acc = np.float32(np.float64(x[j]) * np.float64(x[j]) + np.float64(acc))
            p[t] = acc
        s = 128
        while s > 0:
            p[:s] = p[:s] + p[s:2 * s]
            s //= 2
        assert oracle.rms_sumsq(x) == p[0]


def _gemv_numpy(Wq, Wd, Xq, Xd, M, K):
    """Declared order in numpy.  fma(s, i, acc) with s*i exact in float64 (24+20 bits) and a
    single rounding of the double sum: acc is fp32, product < 2^53 significant bits, but the
    double addition may round before the fp32 rounding; use Python fractions for exactness."""
    from fractions import Fraction
    nb = K // 32
    W = Wq.reshape(M, nb, 32).astype(np.int64)
    X = Xq.reshape(nb, 32).astype(np.int64)
    isum = (W * X[None]).sum(axis=2)
    wd = Wd.reshape(M, nb).astype(np.float32)
    xd = Xd.astype(np.float32)
    y = np.zeros(M, np.float32)
    for r in range(M):
        lanes = np.zeros(32, np.float32)
        for L in range(32):
            acc = np.float32(0)
            for b in range(L, nb, 32):
                s = np.float32(wd[r, b] * xd[b])
                exact = Fraction(float(s)) * int(isum[r, b]) + Fraction(float(acc))
                acc = _round_fraction_f32(exact)
            lanes[L] = acc
        s = 16
        while s > 0:
            lanes[:s] = lanes[:s] + lanes[s:2 * s]
            s //= 2
        y[r] = lanes[0]
    return y, isum


def _round_fraction_f32(fr):
    """Round an exact rational to the nearest fp32 (ties to even)."""
    from fractions import Fraction
    if fr == 0:
        return np.float32(0)
    d = float(fr)                       # correctly rounded to double
    f = np.float32(d)
    # double rounding guard: if the double sits exactly halfway between two floats, decide exactly
    lo = np.nextafter(f, np.float32(-np.inf)); hi = np.nextafter(f, np.float32(np.inf))
    best = f
    for c in (lo, hi):
        if abs(Fraction(float(c)) - fr) < abs(Fraction(float(best)) - fr):
            best = c
        elif abs(Fraction(float(c)) - fr) == abs(Fraction(float(best)) - fr):
            if (np.float32(c).view(np.uint32) & 1) == 0:
                best = c
    return np.float32(best)


@pytest.mark.parametrize("M,K", [(7, 32), (5, 896), (3, 4864), (4, 1056)])
def test_gemv_order_and_integer_dots(oracle, M, K):
    from llamatov_b200 import synth
    Wq, Wd, x = synth.gemv_case(M, K, seed=M * 1000 + K)
    Xq, Xd = oracle.quant_q8(x[0])
    y = oracle.q8_gemv(Wq, Wd, Xq, Xd, M, K)
    want, isum = _gemv_numpy(Wq, Wd, Xq, Xd, M, K)
    assert np.array_equal(oracle.q8_block_isums(Wq, Xq, M, K), isum.astype(np.int32))
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    # residual epilogue = one fp32 add
    r = np.linspace(-1, 1, M).astype(np.float32)
    assert np.array_equal(oracle.q8_gemv(Wq, Wd, Xq, Xd, M, K, resid=r), y + r)
    # float64 dequantise-then-dot agrees to fp32 rounding noise
    deq = Wq.reshape(M, K).astype(np.float64) * np.repeat(Wd.reshape(M, -1).astype(np.float64), 32, axis=1)
    xdq = Xq.astype(np.float64) * np.repeat(Xd.astype(np.float64), 32)
    ref = deq @ xdq
    assert np.max(np.abs(y - ref)) <= 1e-5 * np.max(np.abs(ref)) + 1e-6
    # batch: each column independent
    Wq2, Wd2, xs = synth.gemv_case(M, K, T=3, seed=9)
    cols = [oracle.quant_q8(xs[t]) for t in range(3)]
    XQ = np.concatenate([c[0] for c in cols]); XD = np.concatenate([c[1] for c in cols])
    Y = oracle.q8_gemm(Wq2, Wd2, XQ, XD, M, K, 3)
    for t in range(3):
        assert np.array_equal(Y[t], oracle.q8_gemv(Wq2, Wd2, cols[t][0], cols[t][1], M, K))


def test_attention_against_float64(oracle):
    rng = np.random.default_rng(11)
    nh, nkv, hd, maxt = 4, 2, 32, 64
    for L in (1, 2, 33, 64):
        q = rng.standard_normal(nh * hd).astype(np.float32)
        kc = rng.standard_normal((maxt, nkv, hd)).astype(np.float32)
        vc = rng.standard_normal((maxt, nkv, hd)).astype(np.float32)
        scale = hd ** -0.5
        out = oracle.attn_decode_masked(q, kc, vc, L, hd, nh, nkv, scale, maxt)
        # poison beyond L must not change a bit
        kc2, vc2 = kc.copy(), vc.copy()
        kc2[L:] = np.nan; vc2[L:] = np.inf
        out2 = oracle.attn_decode_masked(q, kc2, vc2, L, hd, nh, nkv, scale, maxt)
        assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))
        for h in range(nh):
            hk = h // (nh // nkv)
            s = (kc[:L, hk].astype(np.float64) @ q[h * hd:(h + 1) * hd].astype(np.float64)) * scale
            p = np.exp(s - s.max()); p /= p.sum()
            ref = p @ vc[:L, hk].astype(np.float64)
            assert np.max(np.abs(out[h * hd:(h + 1) * hd] - ref)) < 5e-6


def test_argmax_ties_and_sentinel(oracle):
    x = np.array([1, 5, 5, 3, 5], np.float32)
    assert oracle.argmax(x) == 1
    assert oracle.argmax(np.array([-np.inf, -np.inf], np.float32)) == 2147483647   # reference sentinel
    rng = np.random.default_rng(2)
    v = rng.standard_normal(151936).astype(np.float32)
    assert oracle.argmax(v) == int(np.argmax(v))


def test_oracle_engine_runs_and_is_deterministic(oracle):
    from llamatov_b200 import synth
    m = synth.make_model("tiny", seed=1)
    om = synth.oracle_model(m)
    e1 = oracle.OracleEngine(om, max_seq=32)
    e2 = oracle.OracleEngine(om, max_seq=32)
    toks = [3, 77, 500, 12]
    l1 = [e1.step(t)[0] for t in toks]
    l2 = [e2.step(t)[0] for t in toks]
    for a, b in zip(l1, l2):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        assert np.all(np.isfinite(a))
    assert int(e1.lens[0]) == len(toks)
    # the step composition equals the per-op functions chained by hand (first layer, first token)
    cfg = m["cfg"]; E = cfg["n_embd"]; ly = om["layers"][0]
    x = oracle.embed_q8(*om["token_embd"], 3, E)
    h = oracle.rmsnorm(x, ly["attn_norm"], cfg["norm_eps"])
    xq, xd = oracle.quant_q8(h)
    nqkv = (cfg["n_head"] + 2 * cfg["n_head_kv"]) * cfg["hd"]
    qkv = oracle.q8_gemv(*ly["qkv"], xq, xd, nqkv, E, resid=ly["qkv_bias"])
    nq = cfg["n_head"] * cfg["hd"]; nk = cfg["n_head_kv"] * cfg["hd"]
    e3 = oracle.OracleEngine(om, max_seq=32)
    e3.step(3)
    # position 0: rope is the identity, so the cached K/V rows are the raw projections
    assert np.array_equal(e3.kc[0][0], qkv[nq:nq + nk])
    assert np.array_equal(e3.vc[0][0], qkv[nq + nk:])


def test_ggml_order_restatement_equals_the_reference_cpu_library(oracle):
    """oracle/_ref/libbpd_cpu.so is the reference's own C code compiled here: its quantiser and its Q8_0
    matmul (one token, tiles, odd last token) against the restatement, bit for bit."""
    import ctypes
    from llamatov_b200 import synth
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libbpd_cpu.so")
    if not os.path.exists(so):
        pytest.skip("reference CPU library not built (no reference checkout)")
    L = ctypes.CDLL(so)
    mm = L.bpd_qmatmul_q8_0_llamafile_cpu; mm.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3; mm.restype = None
    qf = L.bpd_quant_q8_0_cpu; qf.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]; qf.restype = None
    for (M, K, T) in [(4864, 896, 1), (96, 896, 5), (64, 4864, 4), (33, 1024, 2), (50, 896, 7)]:
        Wq, Wd, x = synth.gemv_case(M, K, T=T, seed=T)
        nb = K // 32
        blocks = np.empty((M * nb, 34), np.uint8)
        blocks[:, :2] = Wd.view(np.uint8).reshape(M * nb, 2); blocks[:, 2:] = Wq.view(np.uint8).reshape(M * nb, 32)
        xa = np.ascontiguousarray(x, np.float32); ya = np.zeros(T * M, np.float32)
        mm(blocks.ctypes.data, xa.ctypes.data, ya.ctypes.data, M, T, K)
        qs, ds = [], []
        for t in range(T):
            q, d = oracle.quant_q8_ggml(x[t]); qs.append(q); ds.append(d)
            raw = np.zeros(nb * 34, np.uint8)
            qf(np.ascontiguousarray(x[t]).ctypes.data, raw.ctypes.data, K)
            raw = raw.reshape(nb, 34)
            assert np.array_equal(raw[:, 2:].copy().view(np.int8).reshape(-1), q)
            assert np.array_equal(raw[:, :2].copy().view(np.uint16).reshape(-1), d.view(np.uint16))
        y = oracle.q8_gemm_ggml(Wq, Wd, np.stack(qs), np.stack(ds), M, K, T)
        assert np.array_equal(y.reshape(-1).view(np.uint32), ya.view(np.uint32)), (M, K, T)
