"""ctypes front end of the CPU oracle (oracle/lt_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and bench.py's
cpu_baseline / reference legs.  The product package never imports it.

Parity status: pinned by (a) the reference's own host quantisers run in the build
container (tests/golden/make_golden.py -> tests/golden/*.npz) and (b) the reference's
own CUDA kernel texts compiled for sm_100a (oracle/_ref/*.cubin, compared on the GPU by
tests/test_ref_device_parity.py).  The reference stores no numeric golden vectors for
this path.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblt_oracle.so")
_lib = None

c_i8p = ctypes.POINTER(ctypes.c_int8)
c_u16p = ctypes.POINTER(ctypes.c_uint16)
c_f32p = ctypes.POINTER(ctypes.c_float)
c_i32p = ctypes.POINTER(ctypes.c_int32)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_lt_oracle_build", os.path.join(_HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        _lib = ctypes.CDLL(_SO)
        _lib.lto_h2f.restype = ctypes.c_float
        _lib.lto_h2f.argtypes = [ctypes.c_uint16]
        _lib.lto_f2h.restype = ctypes.c_uint16
        _lib.lto_f2h.argtypes = [ctypes.c_float]
        _lib.lto_rms_sumsq.restype = ctypes.c_float
        _lib.lto_argmax.restype = ctypes.c_int
        _lib.lto_decode_token.restype = ctypes.c_int
        _lib.lto_num_threads.restype = ctypes.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(t)


def _f32(a):
    return np.ascontiguousarray(a, np.float32)


def quant_q8(x):
    """x f32[K] -> (Xq int8[K], Xd float16[K/32])"""
    x = _f32(x).reshape(-1)
    K = x.size
    xq = np.empty(K, np.int8)
    xd = np.empty(K // 32, np.uint16)
    lib().lto_quant_q8(_p(x, c_f32p), _p(xq, c_i8p), _p(xd, c_u16p), ctypes.c_int(K))
    return xq, xd.view(np.float16)


def silu_mul(g, u):
    g = _f32(g).reshape(-1); u = _f32(u).reshape(-1)
    y = np.empty_like(g)
    lib().lto_silu_mul(_p(g, c_f32p), _p(u, c_f32p), _p(y, c_f32p), ctypes.c_int(g.size))
    return y


def silu_mul_quant(g, u):
    g = _f32(g).reshape(-1); u = _f32(u).reshape(-1)
    K = g.size
    xq = np.empty(K, np.int8)
    xd = np.empty(K // 32, np.uint16)
    lib().lto_silu_mul_quant(_p(g, c_f32p), _p(u, c_f32p), _p(xq, c_i8p), _p(xd, c_u16p), ctypes.c_int(K))
    return xq, xd.view(np.float16)


def _w(Wq, Wd):
    Wq = np.ascontiguousarray(Wq, np.int8).reshape(-1)
    Wd = np.ascontiguousarray(Wd).reshape(-1)
    if Wd.dtype == np.float16:
        Wd = Wd.view(np.uint16)
    assert Wd.dtype == np.uint16
    return Wq, Wd


def q8_gemv(Wq, Wd, Xq, Xd, M, K, resid=None):
    Wq, Wd = _w(Wq, Wd)
    Xq, Xd = _w(Xq, Xd)
    y = np.empty(M, np.float32)
    r = None if resid is None else _f32(resid).reshape(-1)
    lib().lto_q8_gemv_addres(_p(Wq, c_i8p), _p(Wd, c_u16p), _p(Xq, c_i8p), _p(Xd, c_u16p),
                             None if r is None else _p(r, c_f32p), _p(y, c_f32p),
                             ctypes.c_int(M), ctypes.c_int(K))
    return y


def q8_gemm(Wq, Wd, Xq, Xd, M, K, T):
    """T activation columns, each reduced independently -> Y[T, M]."""
    Wq, Wd = _w(Wq, Wd)
    Xq, Xd = _w(Xq, Xd)
    y = np.empty((T, M), np.float32)
    lib().lto_q8_gemm(_p(Wq, c_i8p), _p(Wd, c_u16p), _p(Xq, c_i8p), _p(Xd, c_u16p), _p(y, c_f32p),
                      ctypes.c_int(M), ctypes.c_int(K), ctypes.c_int(T))
    return y


def q8_gemv_leftfold(Wq, Wd, Xq, Xd, M, K):
    Wq, Wd = _w(Wq, Wd)
    Xq, Xd = _w(Xq, Xd)
    y = np.empty(M, np.float32)
    lib().lto_q8_gemv_leftfold(_p(Wq, c_i8p), _p(Wd, c_u16p), _p(Xq, c_i8p), _p(Xd, c_u16p),
                               _p(y, c_f32p), ctypes.c_int(M), ctypes.c_int(K))
    return y


def q8_block_isums(Wq, Xq, M, K):
    Wq = np.ascontiguousarray(Wq, np.int8).reshape(-1)
    Xq = np.ascontiguousarray(Xq, np.int8).reshape(-1)
    out = np.empty((M, K // 32), np.int32)
    lib().lto_q8_block_isums(_p(Wq, c_i8p), _p(Xq, c_i8p), _p(out, c_i32p), ctypes.c_int(M), ctypes.c_int(K))
    return out


def rms_sumsq(x):
    x = _f32(x).reshape(-1)
    return np.float32(lib().lto_rms_sumsq(_p(x, c_f32p), ctypes.c_int(x.size)))


def rmsnorm(x, w, eps, inv_override=None):
    x = _f32(x)
    N = x.shape[-1]
    M = x.size // N
    w = _f32(w).reshape(-1)
    y = np.empty_like(x)
    inv = None if inv_override is None else _f32(inv_override).reshape(-1)
    lib().lto_rmsnorm(_p(x, c_f32p), _p(w, c_f32p), _p(y, c_f32p), ctypes.c_int(M), ctypes.c_int(N),
                      ctypes.c_float(eps), None if inv is None else _p(inv, c_f32p))
    return y


def rope(x, pos, n_head, hd, theta):
    """x f32[nrows, n_head*hd] (copied), pos int[nrows] -> roped copy."""
    x = _f32(x).copy().reshape(-1, n_head * hd)
    pos = np.ascontiguousarray(np.asarray(pos).reshape(-1), np.int32)
    lib().lto_rope(_p(x, c_f32p), _p(pos, c_i32p), ctypes.c_int(x.shape[0]), ctypes.c_int(n_head),
                   ctypes.c_int(hd), ctypes.c_float(theta))
    return x


def attn_decode_masked(q, kc, vc, L, hd, nh, nkv, scale, maxt):
    q = _f32(q).reshape(-1); kc = _f32(kc).reshape(-1); vc = _f32(vc).reshape(-1)
    out = np.empty(nh * hd, np.float32)
    lib().lto_attn_decode_masked(_p(q, c_f32p), _p(kc, c_f32p), _p(vc, c_f32p), ctypes.c_int(L),
                                 _p(out, c_f32p), ctypes.c_int(hd), ctypes.c_int(nh), ctypes.c_int(nkv),
                                 ctypes.c_float(scale), ctypes.c_int(maxt))
    return out


def quant_q8_ggml(x):
    """The reference C library's activation quantiser (q = rint(x * 127/amax))."""
    x = _f32(x).reshape(-1)
    K = x.size
    q = np.empty(K, np.int8); d = np.empty(K // 32, np.uint16)
    lib().lto_quant_q8_ggml(_p(x, c_f32p), _p(q, c_i8p), _p(d, c_u16p), ctypes.c_int(K))
    return q, d.view(np.float16)


def q8_gemm_ggml(Wq, Wd, Xq, Xd, M, K, T=1):
    """Y [T, M] in the fold order of the reference's compiled CPU path."""
    Wq, Wd = _w(Wq, Wd)
    Xq = np.ascontiguousarray(Xq, np.int8).reshape(-1)
    Xd = np.ascontiguousarray(Xd).reshape(-1)
    Xd = Xd.view(np.uint16) if Xd.dtype != np.uint16 else Xd
    y = np.empty(T * M, np.float32)
    lib().lto_q8_gemm_ggml(_p(Wq, c_i8p), _p(Wd, c_u16p), _p(Xq, c_i8p), _p(Xd, c_u16p), _p(y, c_f32p),
                           ctypes.c_int(M), ctypes.c_int(K), ctypes.c_int(T))
    return y.reshape(T, M)


def attn_decode_split(q, kc, vc, L, hd, nh, nkv, scale, nsplit):
    """Decode attention in the declared split order (one sequence)."""
    q = _f32(q).reshape(-1); kc = _f32(kc).reshape(-1); vc = _f32(vc).reshape(-1)
    out = np.empty(nh * hd, np.float32)
    lib().lto_attn_decode_split(_p(q, c_f32p), _p(kc, c_f32p), _p(vc, c_f32p), ctypes.c_int(L),
                                _p(out, c_f32p), ctypes.c_int(hd), ctypes.c_int(nh), ctypes.c_int(nkv),
                                ctypes.c_float(scale), ctypes.c_int(nsplit))
    return out


def argmax(x):
    x = _f32(x).reshape(-1)
    return int(lib().lto_argmax(_p(x, c_f32p), ctypes.c_int(x.size)))


def embed_q8(Wq, Wd, tok, E):
    Wq, Wd = _w(Wq, Wd)
    out = np.empty(E, np.float32)
    lib().lto_embed_q8(_p(Wq, c_i8p), _p(Wd, c_u16p), ctypes.c_int(tok), _p(out, c_f32p), ctypes.c_int(E))
    return out


def f2h(x):
    return np.uint16(lib().lto_f2h(ctypes.c_float(float(np.float32(x)))))


def h2f(h):
    return np.float32(lib().lto_h2f(ctypes.c_uint16(int(h))))


def num_threads():
    return int(lib().lto_num_threads())


def set_threads(n):
    """Use n OpenMP threads (torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks)."""
    lib().lto_set_threads(ctypes.c_int(int(n)))


# ------------------------------------------------------------------ whole-model engine

class _Q8W(ctypes.Structure):
    _fields_ = [("wq", ctypes.c_void_p), ("wd", ctypes.c_void_p)]


class _Layer(ctypes.Structure):
    _fields_ = [("attn_norm", ctypes.c_void_p), ("qkv", _Q8W), ("qkv_bias", ctypes.c_void_p),
                ("o", _Q8W), ("ffn_norm", ctypes.c_void_p), ("gateup", _Q8W), ("down", _Q8W),
                ("kcache", ctypes.c_void_p), ("vcache", ctypes.c_void_p), ("len", ctypes.c_void_p)]


class _Model(ctypes.Structure):
    _fields_ = [("n_layers", ctypes.c_int), ("E", ctypes.c_int), ("nh", ctypes.c_int), ("nkv", ctypes.c_int),
                ("hd", ctypes.c_int), ("F", ctypes.c_int), ("V", ctypes.c_int), ("max_seq", ctypes.c_int),
                ("eps", ctypes.c_float), ("theta", ctypes.c_float),
                ("layers", ctypes.c_void_p), ("out_norm", ctypes.c_void_p), ("lm_head", _Q8W), ("embd", _Q8W)]


class OracleEngine:
    """CPU decode engine with the reference's production op sequence.

    `model` is the dict made by the synthetic-model generator: per layer the concatenated
    Q8_0 weights as (Wq int8[N*K], Wd float16[N*K/32]) plus the fp32 norm weights and bias.
    """

    def __init__(self, model, max_seq=256):
        cfg = model["cfg"]
        self.cfg = cfg
        self.max_seq = max_seq
        self._keep = []
        L = cfg["n_layers"]
        nk = cfg["n_head_kv"] * cfg["hd"]
        layers = (_Layer * L)()

        def ptr(a):
            self._keep.append(a)
            return a.ctypes.data

        def q8(pair):
            wq, wd = _w(*pair)
            return _Q8W(ptr(wq), ptr(wd))
        self.kc, self.vc, self.lens = [], [], np.zeros(L, np.int32)
        for i, ly in enumerate(model["layers"]):
            kc = np.zeros((max_seq, nk), np.float32); vc = np.zeros((max_seq, nk), np.float32)
            self.kc.append(kc); self.vc.append(vc)
            layers[i] = _Layer(ptr(_f32(ly["attn_norm"])), q8(ly["qkv"]),
                               ptr(_f32(ly["qkv_bias"])) if ly.get("qkv_bias") is not None else None,
                               q8(ly["o"]), ptr(_f32(ly["ffn_norm"])), q8(ly["gateup"]), q8(ly["down"]),
                               kc.ctypes.data, vc.ctypes.data, self.lens.ctypes.data + 4 * i)
        self._layers = layers
        self.m = _Model(L, cfg["n_embd"], cfg["n_head"], cfg["n_head_kv"], cfg["hd"], cfg["n_ffn"],
                        cfg["vocab"], max_seq, cfg["norm_eps"], cfg["rope_theta"],
                        ctypes.addressof(layers), ptr(_f32(model["output_norm"])),
                        q8(model["lm_head"]), q8(model["token_embd"]))
        self.V = cfg["vocab"]

    def step(self, tok):
        """One token in, (logits f32[V], greedy token) out; the caches advance."""
        logits = np.empty(self.V, np.float32)
        nxt = lib().lto_decode_token(ctypes.byref(self.m), ctypes.c_int(int(tok)), _p(logits, c_f32p))
        return logits, int(nxt)

    def reset(self):
        self.lens[:] = 0
