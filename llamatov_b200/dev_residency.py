"""Device-resident decode engine with the names and call contract of the reference's
bpd/lib/dev_residency.py: activations flow op -> op as device pointers (`DevTensor`), the KV
cache lives on the GPU (`DeviceKVCache`), `forward_pass_resident` runs one token through
the layer loop and `GraphRunner` captures that step into a CUDA graph and replays it.

What differs from the reference is underneath the names: kernels are precompiled sm_100a
code in libllamatov_b200.so reached through its C ABI (no runtime code generation), device
memory is held by torch tensors, launches go to torch's current stream, and graph capture
uses torch.cuda.CUDAGraph.  Only the reference's production ensemble
(`PRODUCTION_PROFILE`, bpd/lib/dev_residency.py:1221-1230) is implemented; the flags it
turns off name code paths that do not exist here and are refused.

Reference lines for each function are given in its docstring.
"""
import ctypes
import os

import numpy as np
import torch

from . import _lib
from . import fact_dispatch as fd
from .fact_dispatch import Q8Weight

# --------------------------------------------------------------------------- profile
# bpd/lib/dev_residency.py:1221-1247.  The flags are kept as module attributes because the
# reference's referees read and assert them; this engine always runs the production ensemble.
PRODUCTION_PROFILE = {
    "_DEVICE_KV_CACHE": True, "_DEVICE_ATTN": True, "_MASKED_ATTN": True,
    "_GRAPH_PREP": True, "_KV_MAX_SEQ": 256, "_ATTN_SPLIT_K": False,
    "_DEVICE_LOGITS": True, "_QFUSED": False, "_GEMV_TILED_V4_QFUSED": False, "_KV_QUANT_Q8": False,
    "_ADDRES_FUSED": True, "_BIAS_FOLD": True, "_RMS_BLOCKROW": True,
    "_GEMV_TILED": True, "_GEMV_TILED_V4": True, "_GEMV_TILED_BM": 16,
    "_QUANT_PAR": True, "_ARGMAX2": True, "_FUSE_QKV": True, "_FUSE_GATEUP": True,
    "_APPEND_KV_FUSED": True, "_APPEND_INCR_FUSED": True, "_RESID_CARRY_FUSED": True,
    "_ROPE_QK_FUSED": True, "_SILU_QUANT_FUSED": True,
}
for _k, _v in PRODUCTION_PROFILE.items():
    globals()[_k] = _v
_HOST_OPS = set()
_GATE_COMPOSITIONS = True
# flags whose non-production value selects a reference code path this engine does not have
_FIXED_FLAGS = ("_DEVICE_KV_CACHE", "_DEVICE_ATTN", "_MASKED_ATTN", "_GRAPH_PREP", "_ATTN_SPLIT_K",
                "_DEVICE_LOGITS", "_QFUSED", "_GEMV_TILED_V4_QFUSED", "_KV_QUANT_Q8")


def apply_production_profile():
    """Set every flag of the production ensemble; returns a copy of the profile
    (bpd/lib/dev_residency.py:1231-1240)."""
    g = globals()
    for k, v in PRODUCTION_PROFILE.items():
        g[k] = v
    _SLAB.enabled = True
    return dict(PRODUCTION_PROFILE)


def attest_profile():
    """Live values of the profile flags (bpd/lib/dev_residency.py:1241-1247)."""
    g = globals()
    live = {k: g.get(k) for k in PRODUCTION_PROFILE}
    live["_SLAB.enabled"] = _SLAB.enabled
    return live


def assert_certified_composition():
    """Refuse flag combinations that have no certified kernel ensemble
    (bpd/lib/dev_residency.py:1259-1281).  Here that is any departure from the production
    value of a flag in _FIXED_FLAGS."""
    if not _GATE_COMPOSITIONS:
        return
    live = attest_profile()
    bad = [k for k in _FIXED_FLAGS if k != "_KV_MAX_SEQ" and live[k] != PRODUCTION_PROFILE[k]]
    if bad:
        raise RuntimeError(
            "UNCERTIFIED COMPOSITION REFUSED by the config-profile gate: %s differ from the production "
            "profile; this engine implements the production ensemble only. Run apply_production_profile()."
            % ", ".join(bad))


# --------------------------------------------------------------------------- plumbing

def _stream():
    """cudaStream_t of torch's current stream (the capture stream while a graph is recorded)."""
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _capturing():
    return torch.cuda.is_current_stream_capturing()


def _vp(p):
    return p if isinstance(p, ctypes.c_void_p) else ctypes.c_void_p(int(p))


def _addr(p):
    return p.value if isinstance(p, ctypes.c_void_p) else int(p)


class _SlabArena:
    """Bump arena for per-layer scratch: one device buffer, fixed offsets, reset per layer
    (bpd/lib/dev_residency.py:149-176).  Fixed pointers are what makes the step capturable."""
    __slots__ = ("enabled", "base", "cap", "off", "_align", "_buf")

    def __init__(self):
        self.enabled = True
        self.base = None; self.cap = 0; self.off = 0; self._align = 256; self._buf = None

    def ensure(self, nbytes):
        if self.base is None:
            self.cap = max(int(nbytes), 8 << 20)
            self._buf = torch.empty(self.cap, dtype=torch.uint8, device="cuda")
            self.base = ctypes.c_void_p(self._buf.data_ptr())

    def alloc(self, nbytes):
        self.ensure(nbytes)
        a = (int(nbytes) + self._align - 1) & ~(self._align - 1)
        if self.off + a > self.cap:
            raise RuntimeError(f"slab overflow: need {self.off + a}, cap {self.cap}")
        p = ctypes.c_void_p(self.base.value + self.off)
        self.off += a
        return p

    def reset(self):
        self.off = 0


_SLAB = _SlabArena()
_SCRATCH = []


def free_scratch():
    """Rewind the arena (bpd/lib/dev_residency.py:139-146)."""
    if _SLAB.enabled:
        _SLAB.reset()
    else:
        _SCRATCH.clear()


def _scratch_alloc(nbytes):
    if _SLAB.enabled:
        return _SLAB.alloc(nbytes)
    t = torch.empty(int(nbytes), dtype=torch.uint8, device="cuda")
    _SCRATCH.append(t)
    return ctypes.c_void_p(t.data_ptr())


class DevTensor:
    """Device-resident fp32 activation: pointer + shape (bpd/lib/dev_residency.py:387-415)."""
    __slots__ = ("ptr", "shape", "n", "nbytes", "_owns", "_t")

    def __init__(self, ptr, shape, owns=True, _t=None):
        self.ptr = _vp(ptr); self.shape = tuple(shape)
        self.n = int(np.prod(shape)) if len(self.shape) else 1
        self.nbytes = self.n * 4; self._owns = owns; self._t = _t

    @staticmethod
    def from_host(arr):
        a = np.ascontiguousarray(np.asarray(arr, np.float32))
        t = torch.from_numpy(a).cuda()
        return DevTensor(t.data_ptr(), a.shape, True, t)

    @staticmethod
    def empty(shape):
        n = int(np.prod(shape))
        t = torch.empty(n, dtype=torch.float32, device="cuda")
        return DevTensor(t.data_ptr(), shape, True, t)

    def to_host(self):
        torch.cuda.synchronize()
        out = np.empty(self.shape, np.float32)
        _memcpy_dtoh(out, self.ptr, self.nbytes)
        return out

    def free(self):
        if self._owns and self.ptr:
            self._t = None; self.ptr = None


_cudart = None


def _rt():
    global _cudart
    if _cudart is None:
        _cudart = ctypes.CDLL("libcudart.so.12")
        _cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        _cudart.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    return _cudart


def _memcpy_dtoh(host_arr, dptr, nbytes):
    r = _rt().cudaMemcpy(host_arr.ctypes.data, _vp(dptr), nbytes, 2)
    if r != 0:
        raise RuntimeError(f"cudaMemcpy DtoH failed: {r}")


def _memcpy_htod(dptr, host_arr, nbytes):
    r = _rt().cudaMemcpyAsync(_vp(dptr), host_arr.ctypes.data, nbytes, 1, _stream())
    if r != 0:
        raise RuntimeError(f"cudaMemcpyAsync HtoD failed: {r}")


def _memcpy_dtod(dst, src, nbytes):
    """Device-to-device copy on the current stream (bpd/lib/dev_residency.py:331-338)."""
    r = _rt().cudaMemcpyAsync(_vp(dst), _vp(src), nbytes, 3, _stream())
    if r != 0:
        raise RuntimeError(f"cudaMemcpyAsync DtoD failed: {r}")


def _empty_dev(shape):
    if _SLAB.enabled:
        n = int(np.prod(shape))
        return DevTensor(_SLAB.alloc(n * 4), shape, owns=False)
    return DevTensor.empty(shape)


def _slice_dev(t, start, length):
    """View of t[start:start+length], no copy (bpd/lib/dev_residency.py:1308-1311)."""
    return DevTensor(ctypes.c_void_p(_addr(t.ptr) + start * 4), (length,), owns=False)


_DEV_CONST = {}


def _dev_const(arr):
    """Upload-once cache for norm weights and biases, keyed by length and three samples
    (bpd/lib/dev_residency.py:784-792)."""
    a = np.ascontiguousarray(np.asarray(arr, np.float32)).reshape(-1)
    key = (a.shape[0], float(a[0]), float(a[a.shape[0] // 2]), float(a[-1]))
    hit = _DEV_CONST.get(key)
    if hit is not None:
        return hit[0]
    if _capturing():
        raise RuntimeError("constant upload during graph capture: warm every weight in seed()")
    t = torch.from_numpy(a).cuda()
    _DEV_CONST[key] = (ctypes.c_void_p(t.data_ptr()), t)
    return _DEV_CONST[key][0]


def _np(w):
    if isinstance(w, Q8Weight):
        return w
    return w.detach().cpu().numpy() if hasattr(w, "detach") else w


# --------------------------------------------------------------------------- KV cache

class DeviceKVCache:
    """Per-layer fp32 K and V buffers [max_seq, nkv*hd], position-major, with a device-side
    length counter (bpd/lib/dev_residency.py:418-541)."""
    __slots__ = ("max_seq", "nkv", "hd", "width", "k_ptr", "v_ptr", "length", "elem_bytes", "len_ptr",
                 "_k", "_v", "_len")

    def __init__(self, max_seq, nkv, hd, elem_bytes=4):
        if elem_bytes != 4:
            raise RuntimeError("DeviceKVCache: only fp32 (elem_bytes=4) is implemented")
        self.max_seq = int(max_seq); self.nkv = int(nkv); self.hd = int(hd)
        self.width = self.nkv * self.hd
        self.elem_bytes = 4
        self._k = torch.zeros(self.max_seq * self.width, dtype=torch.float32, device="cuda")
        self._v = torch.zeros(self.max_seq * self.width, dtype=torch.float32, device="cuda")
        self.k_ptr = ctypes.c_void_p(self._k.data_ptr())
        self.v_ptr = ctypes.c_void_p(self._v.data_ptr())
        self.length = 0
        self.len_ptr = None
        self._len = None

    def _row_off(self, pos):
        return pos * self.width * self.elem_bytes

    def _ensure_len_ptr(self, seed=True):
        """Device int holding the length.  seed=True writes the host mirror into it (never
        during capture: the captured step advances it on the device)."""
        if self.len_ptr is None:
            self._len = torch.zeros(1, dtype=torch.int32, device="cuda")
            self.len_ptr = ctypes.c_void_p(self._len.data_ptr())
            seed = True
        if seed:
            if _capturing():
                raise RuntimeError("length seeding during graph capture")
            self._len.fill_(self.length)
        return self.len_ptr

    def incr_len_dev(self):
        _lib.call("lt_incr_len", self.len_ptr, _stream())

    def append(self, k_dev_ptr, v_dev_ptr, count=1):
        """Copy `count` rows at the host-known offset, advance the host length."""
        n = count * self.width * self.elem_bytes
        if self.length + count > self.max_seq:
            raise RuntimeError(f"KV cache overflow: {self.length}+{count} > {self.max_seq}")
        _memcpy_dtod(_addr(self.k_ptr) + self._row_off(self.length), k_dev_ptr, n)
        _memcpy_dtod(_addr(self.v_ptr) + self._row_off(self.length), v_dev_ptr, n)
        self.length += count

    def append_at_len(self, k_dev_ptr, v_dev_ptr):
        """Append one row at the device-side length, no increment."""
        _lib.call("lt_append_kv", self.k_ptr, _vp(k_dev_ptr), self.v_ptr, _vp(v_dev_ptr), self.len_ptr,
                  self.width, self.max_seq, 0, _stream())

    def append_at_len_incr(self, k_dev_ptr, v_dev_ptr):
        """Append at *len and *len += 1 in one launch; always folds the increment (any width)."""
        _lib.call("lt_append_kv", self.k_ptr, _vp(k_dev_ptr), self.v_ptr, _vp(v_dev_ptr), self.len_ptr,
                  self.width, self.max_seq, 1, _stream())
        return True

    def _slice_host(self, ptr):
        torch.cuda.synchronize()
        n = self.length * self.width
        out = np.empty(n, np.float32)
        if n:
            _memcpy_dtoh(out, ptr, n * 4)
        return out.reshape(self.length, self.nkv, self.hd)

    def k_slice_host(self):
        return self._slice_host(self.k_ptr)

    def v_slice_host(self):
        return self._slice_host(self.v_ptr)

    def free(self):
        self._k = None; self._v = None; self.k_ptr = None; self.v_ptr = None


# --------------------------------------------------------------------------- per-op launchers

def _launch_quant(dX_ptr, dXq, dXd, K):
    """k_quant_q8 (bpd/lib/dev_residency.py:891-904)."""
    _lib.call("lt_quant_q8", _vp(dX_ptr), dXq, dXd, K, 1, _stream())


def _launch_silu_quant(g_ptr, u_ptr, dXq, dXd, K):
    """k_silu_mul_quant (bpd/lib/dev_residency.py:597-604)."""
    _lib.call("lt_silu_mul_quant", _vp(g_ptr), _vp(u_ptr), dXq, dXd, K, 1, _stream())


def silu_mul_dev(g, u):
    y = _empty_dev(g.shape)
    _lib.call("lt_silu_mul", g.ptr, u.ptr, y.ptr, g.n, _stream())
    return y


def add_dev(a, b):
    y = _empty_dev(a.shape)
    _lib.call("lt_add", a.ptr, b.ptr, y.ptr, a.n, _stream())
    return y


_RMS_OUT_OVERRIDE = None


def rms_norm_dev(x, weight_np, eps=1e-6):
    """RMSNorm, device in -> device out (bpd/lib/dev_residency.py:746-781)."""
    M = 1 if x.shape[0:-1] == () else int(np.prod(x.shape[:-1]))
    N = x.shape[-1]
    dW = _dev_const(weight_np)
    y = _RMS_OUT_OVERRIDE if _RMS_OUT_OVERRIDE is not None else _empty_dev(x.shape)
    _lib.call("lt_rmsnorm", x.ptr, dW, y.ptr, M, N, float(eps), _stream())
    return y


def rms_norm_dev_into(x, weight_np, eps, out):
    """RMSNorm into a given fixed buffer (bpd/lib/dev_residency.py:1130-1137)."""
    global _RMS_OUT_OVERRIDE
    _RMS_OUT_OVERRIDE = out
    try:
        return rms_norm_dev(x, weight_np, eps)
    finally:
        _RMS_OUT_OVERRIDE = None


def _weights(weight_np):
    Wq, Wd, N, K = fd._quantize_weight_q8_0(_np(weight_np))
    key = (Wq.ctypes.data, Wd.ctypes.data, Wq.nbytes)
    if _capturing() and key not in fd._DEV_WEIGHT_CACHE:
        raise RuntimeError("weight upload during graph capture: warm every weight in seed()")
    dWq, dWd = fd._dev_weight(Wq, Wd)
    return dWq, dWd, N, K


def q8_linear_dev(x, weight_np, mode="dp4a", rms_src=None):
    """y = x @ W with W in Q8_0: quantise x on the device, GEMV, result stays on the device
    (bpd/lib/dev_residency.py:905-985)."""
    dWq, dWd, N, K = _weights(weight_np)
    nb = K // 32
    dXq = _scratch_alloc(K); dXd = _scratch_alloc(nb * 2)
    _launch_quant(x.ptr, dXq, dXd, K)
    y = _empty_dev((N,))
    _lib.call("lt_q8_gemv", dWq, dWd, dXq, dXd, None, y.ptr, N, K, 1, _stream())
    return y


def q8_linear_add_residual_dev(x, weight_np, resid, mode="dp4a", out=None, silu_src=None):
    """y = (x @ W) + resid with the add folded into the GEMV store; `out` names a fixed
    destination; `silu_src=(g, u)` makes the activation silu(g)*u, quantised in one launch
    (bpd/lib/dev_residency.py:988-1045)."""
    dWq, dWd, N, K = _weights(weight_np)
    nb = K // 32
    dXq = _scratch_alloc(K); dXd = _scratch_alloc(nb * 2)
    if silu_src is not None:
        _g, _u = silu_src
        _launch_silu_quant(_g.ptr, _u.ptr, dXq, dXd, K)
    else:
        _launch_quant(x.ptr, dXq, dXd, K)
    y = out if out is not None else _empty_dev((N,))
    _lib.call("lt_q8_gemv", dWq, dWd, dXq, dXd, resid.ptr, y.ptr, N, K, 1, _stream())
    return y


def q8_linear_dev_into(x, weight_np, out, mode="dp4a", xq=None, xd=None):
    """GEMV into a given fixed buffer, optionally with fixed quantiser scratch
    (bpd/lib/dev_residency.py:1139-1172)."""
    dWq, dWd, N, K = _weights(weight_np)
    nb = K // 32
    dXq = xq if xq is not None else _scratch_alloc(K)
    dXd = xd if xd is not None else _scratch_alloc(nb * 2)
    _launch_quant(x.ptr, dXq, dXd, K)
    _lib.call("lt_q8_gemv", dWq, dWd, dXq, dXd, None, out.ptr, N, K, 1, _stream())
    return out


def q8_linear_dev_bias(x, weight_np, bias_t=None):
    """Q8 linear with the bias folded into the GEMV store as its "residual"
    (bpd/lib/dev_residency.py:1177-1193)."""
    if bias_t is not None and not isinstance(bias_t, int):
        bias_np = _np(bias_t)
        bd = DevTensor(_dev_const(bias_np), (int(np.asarray(bias_np).shape[0]),), owns=False)
        return q8_linear_add_residual_dev(x, weight_np, bd)
    return q8_linear_dev(x, weight_np)


_FUSED_W_CACHE = {}


def _as_q8(t):
    t = _np(t)
    if isinstance(t, Q8Weight):
        return t
    Wq, Wd, N, K = fd._quantize_weight_q8_0(t)
    return Q8Weight(Wq, Wd, N, K)


def _fused_qkv_weight(w, p):
    """Concatenate q, k, v along the output dimension, once (bpd/lib/dev_residency.py:1283-1297).
    Rows are quantised independently, so concatenating the quantised rows equals quantising
    the concatenated matrix."""
    key = (id(w), p, "qkv")
    cached = _FUSED_W_CACHE.get(key)
    if cached is None:
        ws = [_as_q8(w[f"{p}.attn_{n}.weight"]) for n in "qkv"]
        bq = w.get(f"{p}.attn_q.bias")
        bcat = None
        if bq is not None:
            bcat = np.concatenate([np.asarray(_np(w[f"{p}.attn_{n}.bias"]), np.float32) for n in "qkv"])
        cached = (Q8Weight.concat(ws), bcat, tuple(x.N for x in ws))
        _FUSED_W_CACHE[key] = cached
    return cached


def _fused_gateup_weight(w, p):
    """(bpd/lib/dev_residency.py:1299-1306)"""
    key = (id(w), p, "gateup")
    cached = _FUSED_W_CACHE.get(key)
    if cached is None:
        ws = [_as_q8(w[f"{p}.ffn_gate.weight"]), _as_q8(w[f"{p}.ffn_up.weight"])]
        cached = (Q8Weight.concat(ws), None, tuple(x.N for x in ws))
        _FUSED_W_CACHE[key] = cached
    return cached


def qkv_fused_dev(x, w, p):
    """One GEMV over q|k|v (+bias); returns three views (bpd/lib/dev_residency.py:1313-1319)."""
    Wcat, bcat, (nq, nk, nv) = _fused_qkv_weight(w, p)
    y = q8_linear_dev_bias(x, Wcat, bcat)
    return _slice_dev(y, 0, nq), _slice_dev(y, nq, nk), _slice_dev(y, nq + nk, nv)


def gateup_fused_dev(x, w, p, rms_src=None):
    """One GEMV over gate|up; returns two views (bpd/lib/dev_residency.py:1321-1326)."""
    Wcat, _b, (ng, nu) = _fused_gateup_weight(w, p)
    y = q8_linear_dev(x, Wcat)
    return _slice_dev(y, 0, ng), _slice_dev(y, ng, nu)


def rope_dev_inplace_devpos(x_dev, pos_dev_ptr, n_head, hd, theta):
    """RoPE in place, position read from a device int (bpd/lib/dev_residency.py:701-720)."""
    _lib.call("lt_rope", x_dev.ptr, _vp(pos_dev_ptr), 1, n_head, hd, float(theta), _stream())
    return x_dev


def rope_dev_qk_fused(qk_dev_ptr, pos_dev_ptr, nh, nkv, hd, theta):
    """One launch over the contiguous q|k heads (bpd/lib/dev_residency.py:722-741)."""
    _lib.call("lt_rope", _vp(qk_dev_ptr), _vp(pos_dev_ptr), 1, nh + nkv, hd, float(theta), _stream())


def rope_dev_inplace(x_dev, pos_int, n_head, hd, theta):
    """RoPE at a host-known position (bpd/lib/dev_residency.py:676-698); not capturable."""
    p = torch.tensor([int(pos_int)], dtype=torch.int32, device="cuda")
    _lib.call("lt_rope", x_dev.ptr, p.data_ptr(), 1, n_head, hd, float(theta), _stream())
    _SCRATCH.append(p)
    return x_dev


def rope_dev(x_np, positions_np, n_head, hd, theta):
    """Host round-trip RoPE of [nrows, n_head*hd] (bpd/lib/dev_residency.py:649-673)."""
    xa = np.ascontiguousarray(x_np, np.float32)
    dx = torch.from_numpy(xa.copy()).cuda()
    dp = torch.from_numpy(np.ascontiguousarray(np.asarray(positions_np).reshape(-1), np.int32)).cuda()
    _lib.call("lt_rope", dx.data_ptr(), dp.data_ptr(), xa.shape[0], n_head, hd, float(theta), _stream())
    return dx.cpu().numpy()


def attn_decode_from_cache_masked(q_dev_ptr, cache, nh, scale, len_dev_ptr, maxt):
    """Masked decode attention over the device cache (bpd/lib/dev_residency.py:2016-2031)."""
    out = _empty_dev((nh * cache.hd,))
    _lib.call("lt_attn_decode_masked", _vp(q_dev_ptr), cache.k_ptr, cache.v_ptr, _vp(len_dev_ptr), out.ptr,
              cache.hd, nh, cache.nkv, float(np.float32(scale)), int(maxt), _stream())
    return out


def attn_decode_from_cache(q_dev_ptr, cache, nh, scale):
    """Variable-length form (bpd/lib/dev_residency.py:2033-2047): same arithmetic with the
    capacity set to the current length."""
    lp = cache._ensure_len_ptr()
    return attn_decode_from_cache_masked(q_dev_ptr, cache, nh, scale, lp, max(cache.length, 1))


_ARGMAX_BUF = None
_ARGMAX_PARTIALS = None


def _ensure_argmax_buf():
    global _ARGMAX_BUF, _ARGMAX_PARTIALS
    if _ARGMAX_BUF is None:
        t = torch.zeros(1, dtype=torch.int32, device="cuda")
        s = torch.empty(_lib.lib().lt_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
        _ARGMAX_BUF = (ctypes.c_void_p(t.data_ptr()), t)
        _ARGMAX_PARTIALS = (ctypes.c_void_p(s.data_ptr()), s)
    return _ARGMAX_BUF[0]


def argmax_dev(logits_ptr, n, out_ptr=None):
    """Device argmax, lowest index on ties (bpd/lib/dev_residency.py:1074-1110)."""
    if out_ptr is None:
        out_ptr = _ensure_argmax_buf()
    _ensure_argmax_buf()
    assert n > 0, f"argmax_dev: n={n} (must be >0)"
    _lib.call("lt_argmax", _vp(logits_ptr), int(n), _ARGMAX_PARTIALS[0], _vp(out_ptr), _stream())
    return out_ptr


# --------------------------------------------------------------------------- fixed buffers
_RESID_IN = None
_RESID_OUT = None
_LOGITS_BUF = None
_LOGITS_RMS = None
_LOGITS_XQ = None
_LOGITS_XD = None
_FIXED_KEEP = []
_DEVICE_EMBED = None     # (dWq, dWd, token pointer, V) while the on-device token loop is recorded


def _ensure_resid(E):
    """Fixed residual input / carry buffers (bpd/lib/dev_residency.py:126-134)."""
    global _RESID_IN, _RESID_OUT
    if _RESID_IN is None or _RESID_IN.n != E:
        _RESID_IN = DevTensor.empty((E,)); _RESID_IN._owns = False
        _RESID_OUT = DevTensor.empty((E,)); _RESID_OUT._owns = False
    return _RESID_IN, _RESID_OUT


def _lm_head(w):
    return w.get("output.weight", w.get("token_embd.weight"))


def _ensure_logits_buf(E, w):
    """Fixed logits buffer; warms the output-weight and final-norm caches
    (bpd/lib/dev_residency.py:1051-1063)."""
    global _LOGITS_BUF
    lm = _np(_lm_head(w))
    N = lm.shape[1] if lm.shape[0] == E else lm.shape[0]
    if _LOGITS_BUF is None or _LOGITS_BUF.n != N:
        _LOGITS_BUF = DevTensor.empty((N,)); _LOGITS_BUF._owns = False
        _weights(lm)
        _dev_const(_np(w["output_norm.weight"]))
    return _LOGITS_BUF


def _ensure_logits_scratch(E):
    """(bpd/lib/dev_residency.py:1119-1127)"""
    global _LOGITS_RMS, _LOGITS_XQ, _LOGITS_XD
    if _LOGITS_RMS is None or _LOGITS_RMS.n != E:
        _LOGITS_RMS = DevTensor.empty((E,)); _LOGITS_RMS._owns = False
        xq = torch.empty(E, dtype=torch.int8, device="cuda")
        xd = torch.empty(E // 32, dtype=torch.int16, device="cuda")
        _FIXED_KEEP.extend([xq, xd])
        _LOGITS_XQ = ctypes.c_void_p(xq.data_ptr()); _LOGITS_XD = ctypes.c_void_p(xd.data_ptr())
    return _LOGITS_RMS, _LOGITS_XQ, _LOGITS_XD


def reset_engine_state():
    """Drop every module-level buffer and cache (a fresh engine for another model)."""
    global _RESID_IN, _RESID_OUT, _LOGITS_BUF, _LOGITS_RMS, _LOGITS_XQ, _LOGITS_XD, _ARGMAX_BUF, _ARGMAX_PARTIALS
    _RESID_IN = _RESID_OUT = _LOGITS_BUF = _LOGITS_RMS = _LOGITS_XQ = _LOGITS_XD = None
    _ARGMAX_BUF = _ARGMAX_PARTIALS = None
    _FIXED_KEEP.clear(); _DEV_CONST.clear(); _FUSED_W_CACHE.clear()
    fd._DEV_WEIGHT_CACHE.clear(); fd._Q8_WEIGHT_CACHE.clear()
    _SLAB.reset()


def _embedding_row(w, tok, E):
    """fp32 row of the (dequantised) embedding table for one token id, on the host
    (bpd/lib/dev_residency.py:1357-1358)."""
    emb = w["token_embd.weight"]
    if isinstance(emb, Q8Weight):
        t = int(tok)
        nb = E // 32
        q = emb.Wq[t * E:(t + 1) * E].astype(np.float32).reshape(nb, 32)
        d = emb.Wd[t * nb:(t + 1) * nb].astype(np.float32).reshape(nb, 1)
        return np.ascontiguousarray((q * d).reshape(E))
    row = emb.T[tok] if emb.shape[0] < emb.shape[1] else emb[tok]
    return np.ascontiguousarray(row.reshape(E).numpy(), np.float32)


# --------------------------------------------------------------------------- forward

def forward_pass_resident(w, cfg, tok, positions, kv_cache):
    """One token through the device-resident layer loop; several tokens by recursion, one at
    a time, so prefill and decode share one arithmetic (bpd/lib/dev_residency.py:1328-1593).
    Returns logits [1, 1, V] (None while a graph is being captured)."""
    nh, nkv = cfg["n_head"], cfg["n_head_kv"]
    hd = cfg["n_embd"] // nh
    nl = cfg["n_layers"]
    if tok.numel() > 1 and _BATCHED_PREFILL and not _capturing() and _DEVICE_EMBED is None:
        from . import prefill as _pf
        if _pf.supported(cfg, w):
            flat = tok.reshape(-1)
            last = None
            for c0 in range(0, flat.numel(), _pf.MAX_ROWS):
                last = _pf.prefill_resident(w, cfg, flat[c0:c0 + _pf.MAX_ROWS], kv_cache,
                                            want_logits=c0 + _pf.MAX_ROWS >= flat.numel())
            return last
    if tok.numel() > 1:
        toks = tok.reshape(-1).tolist(); poss = positions.reshape(-1).tolist()
        last = None
        for ti, pi in zip(toks, poss):
            last = forward_pass_resident(w, cfg, torch.tensor([ti]), torch.tensor([pi]), kv_cache)
        return last
    E = cfg["n_embd"]
    capturing = _capturing()
    _resid_in, _resid_carry = _ensure_resid(E)
    if _DEVICE_EMBED is not None:
        # on-device token loop: the row is gathered from the Q8_0 table by the token id that
        # the previous step's argmax left in device memory
        dWq, dWd, tok_ptr, V = _DEVICE_EMBED
        _lib.call("lt_embed_q8", dWq, dWd, tok_ptr, _resid_in.ptr, E, V, _stream())
    elif not capturing:
        row = _embedding_row(w, int(tok.reshape(-1)[0]), E)
        _memcpy_htod(_resid_in.ptr, row, E * 4)
        torch.cuda.current_stream().synchronize()      # `row` is pageable host memory
    x_resident = _resid_in
    eps = cfg["norm_eps"]
    theta = cfg["rope_theta"]
    for il in range(nl):
        p = f"blk.{il}"
        xd = x_resident
        hdv = rms_norm_dev(xd, _np(w[f"{p}.attn_norm.weight"]), eps)
        qd, kd, vd = qkv_fused_dev(hdv, w, p)
        cache = kv_cache[il]
        if cache is None:
            if capturing:
                raise RuntimeError("KV cache allocation during graph capture: seed() first")
            cache = DeviceKVCache(_KV_MAX_SEQ, nkv, hd); kv_cache[il] = cache
        lp = cache._ensure_len_ptr(seed=not capturing)
        # position = length before the append; attention sees the length after it
        rope_dev_qk_fused(qd.ptr, lp, nh, nkv, hd, theta)
        cache.append_at_len_incr(kd.ptr, vd.ptr)
        cache.length += 1
        yd = attn_decode_from_cache_masked(qd.ptr, cache, nh, hd ** -0.5, lp, cache.max_seq)
        xres = q8_linear_add_residual_dev(yd, w[f"{p}.attn_output.weight"], xd)
        h2 = rms_norm_dev(xres, _np(w[f"{p}.ffn_norm.weight"]), eps)
        g, u = gateup_fused_dev(h2, w, p)
        q8_linear_add_residual_dev(g, w[f"{p}.ffn_down.weight"], xres, out=_resid_carry, silu_src=(g, u))
        x_resident = _resid_carry
        free_scratch()
    _compute_folded_logits(w, cfg, E)
    if capturing:
        return None
    torch.cuda.synchronize()
    lbuf = _ensure_logits_buf(E, w)
    return torch.from_numpy(lbuf.to_host()).reshape(1, 1, lbuf.n)


def _compute_folded_logits(w, cfg, E):
    """Final RMSNorm + LM-head GEMV into fixed buffers (bpd/lib/dev_residency.py:1596-1623)."""
    if _RESID_OUT is None:
        raise RuntimeError("_compute_folded_logits requires the device residual chain (_RESID_OUT)")
    lbuf = _ensure_logits_buf(E, w)
    rms_out, xq, xd = _ensure_logits_scratch(E)
    rms_norm_dev_into(DevTensor(_RESID_OUT.ptr, (E,), owns=False), _np(w["output_norm.weight"]),
                      cfg["norm_eps"], rms_out)
    q8_linear_dev_into(rms_out, _lm_head(w), lbuf, xq=xq, xd=xd)
    return lbuf


# --------------------------------------------------------------------------- fused decode step
# GraphRunner records the token step either as ~320 per-op kernel nodes (False, the reference's
# structure), as a chain of fused kernels linked by programmatic dependent launch ("pdl",
# lt_decode_step_pdl: 122 nodes) or as ONE persistent kernel ("persistent", lt_decode_step).
# Same arithmetic, bit-identical results in every mode; the eager forward_pass_resident keeps
# the per-op launches and is the parity baseline.
_FUSED_STEP = "persistent"
# pause (ns) between two looks at hand-over words that have not arrived yet, in the one-kernel step
_POLL_NS = int(os.environ.get("LLAMATOV_POLL_NS", "0"))
# copies of the hand-over buffers in use (each SM polls copy SM % n): 1 .. lt_decode_ws_replicas()
_POLL_LOOKS = int(os.environ.get("LLAMATOV_WS_COPIES", "1"))
_WS_TUNE = os.environ.get("LLAMATOV_WS_TUNE", "1") != "0"          # time the step at several workspace positions, keep the fastest
_WS_CANDIDATES = int(os.environ.get("LLAMATOV_WS_CANDIDATES", "12"))
_WS_ROUNDS = int(os.environ.get("LLAMATOV_WS_ROUNDS", "1"))          # sweeps over the vectors

# A prompt of several tokens runs as one batched pass (prefill.prefill_resident) when the
# architecture allows it; False keeps the reference's token-by-token recursion.  Both give the
# same bits.
_BATCHED_PREFILL = True


class _DecLayer(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "attn_norm", "qkv_q", "qkv_d", "qkv_bias", "o_q", "o_d", "ffn_norm", "gu_q", "gu_d",
        "down_q", "down_d", "kcache", "vcache", "len")]


class _DecDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("n_layers", "E", "nh", "nkv", "hd", "F", "V", "max_seq")] + \
               [(n, ctypes.c_float) for n in ("eps", "theta", "scale")] + [("hist_cap", ctypes.c_int)] + \
               [(n, ctypes.c_void_p) for n in (
                   "layers", "out_norm", "lm_q", "lm_d", "emb_q", "emb_d", "x", "ws_x", "ws_x1", "ws_qkv", "ws_att",
                   "ws_v", "logits", "tok", "out_tok", "history", "step", "sync", "epoch", "part_val", "part_idx",
                   "status", "trace", "h_layers", "ws_part")] + [("poll_ns", ctypes.c_int), ("poll_looks", ctypes.c_int), ("trace_cta", ctypes.c_int), ("trace_layer", ctypes.c_int)]


def _ws_layout(sizes, candidates):
    """Arena layout of the hand-over workspaces, in floats: vector i (sizes[i] floats) may sit at
    region[i] + c * pitch[i], c < candidates.  The pitch is an odd number of 256-byte units at least as long as
    the vector (candidate windows of a vector never overlap, and they shift line by line against the L2 slice
    interleave); regions follow each other with 4 KB between them.  Returns (pitch, region, total)."""
    pitch = [(((n * 4 + 255) // 256) | 1) * 64 for n in sizes]
    region = [0]
    for pch in pitch[:-1]:
        region.append(region[-1] + pch * candidates + 1024)
    return pitch, region, region[-1] + pitch[-1] * candidates + 1024


class FusedDecodeStep:
    """Descriptor + workspace of lt_decode_step for one model and its KV caches.  Every weight
    pointer comes from the same upload caches the per-op path uses (no second copy)."""

    def __init__(self, w, cfg, kv, tok_ptr=None, history=None, step=None, hist_cap=0):
        nh, nkv, E = cfg["n_head"], cfg["n_head_kv"], cfg["n_embd"]
        hd = E // nh
        L = cfg["n_layers"]
        self._keep = []
        layers = (_DecLayer * L)()
        F = None
        for il in range(L):
            p = f"blk.{il}"
            Wqkv, bcat, _ = _fused_qkv_weight(w, p)
            Wgu, _, (ng, _nu) = _fused_gateup_weight(w, p)
            F = ng
            qq, qd, _, _ = _weights(Wqkv)
            oq, od, _, _ = _weights(w[f"{p}.attn_output.weight"])
            gq, gd, _, _ = _weights(Wgu)
            dq, dd, _, _ = _weights(w[f"{p}.ffn_down.weight"])
            c = kv[il]
            if c is None:
                raise RuntimeError("FusedDecodeStep: KV caches must exist (run seed() first)")
            c._ensure_len_ptr(seed=False)
            layers[il] = _DecLayer(_addr(_dev_const(_np(w[f"{p}.attn_norm.weight"]))), _addr(qq), _addr(qd),
                                   _addr(_dev_const(bcat)) if bcat is not None else None, _addr(oq), _addr(od),
                                   _addr(_dev_const(_np(w[f"{p}.ffn_norm.weight"]))), _addr(gq), _addr(gd),
                                   _addr(dq), _addr(dd), _addr(c.k_ptr), _addr(c.v_ptr), _addr(c.len_ptr))
        raw = np.frombuffer(bytes(layers), dtype=np.uint8).copy()
        self._layers_dev = torch.from_numpy(raw).cuda()
        self._layers_host = layers
        lq, ld, V, _ = _weights(_lm_head(w))
        eq, ed = None, None
        if tok_ptr is not None:
            eq, ed, _, _ = _weights(_np(w["token_embd.weight"]))
        nq, nk = nh * hd, nkv * hd
        # partial-argmax slots: one per CTA of the persistent kernel / per CTA of the fused LM-head kernel
        nct = max(_lib.lib().lt_decode_num_ctas(), _lib.lib().lt_decode_pdl_num_parts())
        f32 = dict(dtype=torch.float32, device="cuda")
        # tagged workspaces: {value, tag} pairs, zero tags = "never written"
        rep = _lib.lib().lt_decode_ws_replicas() if _POLL_LOOKS != 1 else 1      # copies of four of the vectors in use
        # the hand-over workspaces (five tagged vectors and the argmax slots) live side by side in one arena; where
        # in it is chosen by tune_placement()
        self._ws_sizes = [2 * n for n in (rep * E, rep * E, nq + 2 * nk, rep * nq, rep * F)] + [4 * nct]
        self._ws_pitch, self._ws_region, total = _ws_layout(self._ws_sizes, _WS_CANDIDATES)
        self._ws_arena = torch.zeros(total, **f32)
        self._kv = kv
        self._place(0)
        self.sync = torch.zeros(2, dtype=torch.int32, device="cuda")
        self.epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.part_val = torch.zeros(nct, **f32); self.part_idx = torch.zeros(nct, dtype=torch.int32, device="cuda")
        resid_in, _ = _ensure_resid(E)
        lbuf = _ensure_logits_buf(E, w)
        out_tok = _ensure_argmax_buf()
        max_seq = kv[0].max_seq
        self.desc = _DecDesc(L, E, nh, nkv, hd, F, V, max_seq, float(cfg["norm_eps"]), float(cfg["rope_theta"]),
                             float(np.float32(hd ** -0.5)), int(hist_cap),
                             self._layers_dev.data_ptr(), _addr(_dev_const(_np(w["output_norm.weight"]))),
                             _addr(lq), _addr(ld), None if eq is None else _addr(eq), None if ed is None else _addr(ed),
                             _addr(resid_in.ptr), self.ws[0].data_ptr(), self.ws[1].data_ptr(),
                             self.ws[2].data_ptr(), self.ws[3].data_ptr(), self.ws[4].data_ptr(), _addr(lbuf.ptr),
                             None if tok_ptr is None else int(tok_ptr), _addr(out_tok),
                             None if history is None else int(history), None if step is None else int(step),
                             self.sync.data_ptr(), self.epoch.data_ptr(), self.part_val.data_ptr(),
                             self.part_idx.data_ptr(), None, None, ctypes.addressof(self._layers_host),
                             self.ws_part.data_ptr(), int(_POLL_NS), int(_POLL_LOOKS), int(os.environ.get("LLAMATOV_TRACE_CTA", "0")), int(os.environ.get("LLAMATOV_TRACE_LAYER", "-1")))
        self.mode = "persistent" if _FUSED_STEP is True else _FUSED_STEP
        if self.mode == "persistent" and not _lib.lib().lt_decode_step_supported(ctypes.byref(self.desc)):
            self.mode = "pdl"       # the one-kernel step keeps 2*hd rows of q|k|v resident per SM: small models only

    def _place(self, cands):
        """Point workspace i at candidate position cands[i] of its own region of the arena (an int = the same for
        all): region start + candidate * pitch, the pitch an odd number of 256-byte units, so that the candidates
        of a vector fall on different L2 slices line by line."""
        if isinstance(cands, int):
            cands = [cands] * len(self._ws_sizes)
        views = []
        for i, n in enumerate(self._ws_sizes):
            o = self._ws_region[i] + cands[i] * self._ws_pitch[i]
            views.append(self._ws_arena[o:o + n])
        self.ws = views[:5]
        self.ws_part = views[5]
        if getattr(self, "desc", None) is not None:
            d = self.desc
            d.ws_x, d.ws_x1, d.ws_qkv, d.ws_att, d.ws_v = (v.data_ptr() for v in self.ws)
            d.ws_part = self.ws_part.data_ptr()
        self.placement = list(cands)

    def tune_placement(self, steps=6):
        """Choose where the hand-over workspaces live.  The one-kernel step is bound by the latency of small vectors
        handed from every SM to every SM through L2; a hand-over is complete when its LAST line has arrived, and how
        long a line takes depends on the L2 slice its address falls on: the same kernel ran between 365 and 423 us
        per token on one GPU with nothing changed but the workspaces' addresses.  So a few steps are timed with each
        vector at each candidate position of its region (one vector after the other, the best position kept), and
        the fastest combination stays.  Device state that a step advances -- cache lengths, token, history -- is put
        back afterwards; the cache rows written past the length are overwritten by the real steps.
        Returns the list of (placement, us per step) tried."""
        if self.mode != "persistent" or not _WS_TUNE or _WS_CANDIDATES < 2:
            return []
        if any(c.length + steps > c.max_seq for c in self._kv):
            return []
        pending = _lib.device_status()      # (read and cleared: say so rather than swallow it)
        if pending:
            import warnings
            warnings.warn(f"device status {sorted(pending)} was pending when the decode step's workspaces were placed")
        d = self.desc
        lens = [c._len.clone() for c in self._kv]
        saved = (d.tok, d.out_tok, d.history, d.step)
        tok = torch.zeros(1, dtype=torch.int32, device="cuda"); out = torch.zeros(1, dtype=torch.int32, device="cuda")
        d.tok = tok.data_ptr() if saved[0] else None
        d.out_tok = out.data_ptr(); d.history = None; d.step = None
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        tried = []

        def time_at(cands):
            self._place(cands)
            for c, l in zip(self._kv, lens):
                c._len.copy_(l)
            tok.zero_()
            for i in range(steps):
                if i == 2:
                    e0.record(torch.cuda.current_stream())
                self.launch()
            e1.record(torch.cuda.current_stream())
            e1.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (steps - 2)
            tried.append((list(cands), us))
            return us

        try:
            best = [0] * len(self._ws_sizes)
            best_us = time_at(best)
            for rnd in range(_WS_ROUNDS):
                for i in range(len(self._ws_sizes)):        # one vector after the other
                    for cand in range(_WS_CANDIDATES):
                        if cand == best[i]:
                            continue
                        trial = list(best); trial[i] = cand
                        us = time_at(trial)
                        if us < best_us:
                            best, best_us = trial, us
        finally:
            for c, l in zip(self._kv, lens):
                c._len.copy_(l)
            d.tok, d.out_tok, d.history, d.step = saved
            torch.cuda.synchronize()
        if "wait_timeout" in _lib.device_status():
            raise RuntimeError("lt_decode_step: a wait ran out while the workspace placement was being chosen")
        self._place(best)
        self.placement_us = tried
        return tried

    def enable_trace(self):
        """Diagnostics: SM-clock stamps of CTA 0 and of the last CTA at every phase boundary."""
        n = 8192                     # (id, clock) pairs per traced CTA
        self.trace = torch.zeros(2 * 2 * n, dtype=torch.int64, device="cuda")
        self.desc.trace = self.trace.data_ptr()
        return n

    def launch(self):
        if self.mode == "pdl":
            _lib.check(_lib.lib().lt_decode_step_pdl(ctypes.byref(self.desc), _stream()), "lt_decode_step_pdl")
        else:
            _lib.check(_lib.lib().lt_decode_step(ctypes.byref(self.desc), _stream()), "lt_decode_step")


class GraphRunner:
    """Captures one decode step into a CUDA graph and replays it per token
    (bpd/lib/dev_residency.py:1626-1818): seed() runs the prompt eagerly and settles every
    fixed pointer, capture() records one step, replay_logits()/replay_token() write the
    token's embedding row into the fixed input buffer, launch the graph and read the result."""

    def __init__(self, w, cfg, kv_cache):
        self.w = w; self.cfg = cfg; self.kv = kv_cache
        self.E = cfg["n_embd"]
        self.graph = None
        self.captured = False
        self.stream = torch.cuda.Stream()
        self._tok_host = None

    def seed(self, first_tok, first_pos):
        assert _GRAPH_PREP, "GraphRunner requires the device position/length path"
        assert_certified_composition()
        _ensure_resid(self.E)
        if not _SLAB.enabled:
            raise RuntimeError("GraphRunner requires the slab arena (fixed pointers)")
        if _HOST_OPS:
            raise RuntimeError(f"GraphRunner cannot capture with host-op toggles active: {_HOST_OPS}")
        _ensure_logits_buf(self.E, self.w)
        _ensure_logits_scratch(self.E)
        _ensure_argmax_buf()
        if first_tok.numel() > 1:
            # the prompt but its last token in one batched pass; the last token takes the one-token
            # path, which settles every fixed scratch pointer the captured step will use
            ft, fp = first_tok.reshape(-1), first_pos.reshape(-1)
            forward_pass_resident(self.w, self.cfg, ft[:-1], fp[:-1], self.kv)
            first_tok, first_pos = ft[-1:], fp[-1:]
        logits = forward_pass_resident(self.w, self.cfg, first_tok, first_pos, self.kv)
        torch.cuda.synchronize()
        self._weight_cache_frozen = (frozenset(_DEV_CONST.keys()), frozenset(fd._DEV_WEIGHT_CACHE.keys()),
                                     frozenset(fd._Q8_WEIGHT_CACHE.keys()))
        return logits

    def _assert_weight_cache_frozen(self):
        if not hasattr(self, "_weight_cache_frozen"):
            return
        now = (frozenset(_DEV_CONST.keys()), frozenset(fd._DEV_WEIGHT_CACHE.keys()),
               frozenset(fd._Q8_WEIGHT_CACHE.keys()))
        for label, snap, cur in zip(("_DEV_CONST", "_DEV_WEIGHT_CACHE", "_Q8_WEIGHT_CACHE"),
                                    self._weight_cache_frozen, now):
            added = cur - snap
            if added:
                raise RuntimeError(f"weight cache {label} grew after seed() (added {len(added)} entries): "
                                   "the graph holds the seed-time pointers")

    def capture(self, tok, pos):
        """Record one decode step.  The step's device side effects (cache append, length
        increment) do not run during capture, so the host length mirrors are restored."""
        self._assert_weight_cache_frozen()
        lens = [c.length for c in self.kv]
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        n0 = _lib.launch_count()
        self.fused = bool(_FUSED_STEP)
        self._tok_in = None
        if self.fused:
            # When the embedding table is a Q8_0 table (dequantising its blocks reproduces the rows the host
            # lookup returns), the captured step gathers the row itself from a token id in device memory: a
            # replay then uploads 4 bytes instead of looking the row up and dequantising it on the host.
            if self._q8_exact_table(int(tok.reshape(-1)[0])):
                self._tok_in = torch.zeros(1, dtype=torch.int32, device="cuda")
                self._step_host = FusedDecodeStep(self.w, self.cfg, self.kv, tok_ptr=self._tok_in.data_ptr())
            else:
                self._step_host = FusedDecodeStep(self.w, self.cfg, self.kv)
            with torch.cuda.stream(self.stream):
                self._step_host.tune_placement()
            torch.cuda.synchronize()
            n0 = _lib.launch_count()
            with torch.cuda.graph(g, stream=self.stream):
                self._step_host.launch()
        else:
            with torch.cuda.graph(g, stream=self.stream):
                forward_pass_resident(self.w, self.cfg, tok, pos, self.kv)
        self.launches_per_token = _lib.launch_count() - n0
        for c, n in zip(self.kv, lens):
            c.length = n
        self._assert_weight_cache_frozen()
        self.graph = g
        self.captured = True

    def _q8_exact_table(self, probe_tok):
        """True if token_embd.weight is exactly representable as Q8_0 (checked on sample rows); uploads it."""
        emb = _np(self.w["token_embd.weight"])
        before = (frozenset(_DEV_CONST.keys()), frozenset(fd._DEV_WEIGHT_CACHE.keys()), frozenset(fd._Q8_WEIGHT_CACHE.keys()))
        Wq, Wd, V, K = fd._quantize_weight_q8_0(emb)
        if K != self.E:
            return False
        nb = K // 32
        for t in (0, V // 2, V - 1, int(probe_tok) % V):
            deq = (Wq[t * K:(t + 1) * K].astype(np.float32).reshape(nb, 32) *
                   Wd[t * nb:(t + 1) * nb].astype(np.float32).reshape(nb, 1)).reshape(K)
            if not np.array_equal(deq, _embedding_row(self.w, t, K)):
                return False
        _weights(emb)       # an untied table is not used by the host-row step: upload it now
        if hasattr(self, "_weight_cache_frozen") and before == self._weight_cache_frozen:
            self._weight_cache_frozen = (frozenset(_DEV_CONST.keys()), frozenset(fd._DEV_WEIGHT_CACHE.keys()),
                                         frozenset(fd._Q8_WEIGHT_CACHE.keys()))
        return True

    def input_bytes_per_replay(self):
        """Host-to-device bytes a replay uploads: the token id, or the embedding row."""
        return 4 if getattr(self, "_tok_in", None) is not None else self.E * 4

    def _ensure_pinned(self):
        if getattr(self, "_pin_row", None) is None:     # page-locked staging: the copies below are truly asynchronous
            self._pin_row = torch.empty(self.E, dtype=torch.float32).pin_memory()
            self._pin_row_np = self._pin_row.numpy()
            self._pin_idx = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._pin_idx_np = self._pin_idx.numpy()
            self._pin_tok = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._pin_tok_np = self._pin_tok.numpy()

    def _launch(self, tok):
        assert self.captured, "call capture() before replay"
        self._ensure_pinned()
        if self._tok_in is not None:
            self._pin_tok_np[0] = int(tok)
            with torch.cuda.stream(self.stream):
                _memcpy_htod(ctypes.c_void_p(self._tok_in.data_ptr()), self._pin_tok_np, 4)
                self.graph.replay()
        else:
            np.copyto(self._pin_row_np, _embedding_row(self.w, int(tok), self.E))
            with torch.cuda.stream(self.stream):
                _memcpy_htod(_RESID_IN.ptr, self._pin_row_np, self.E * 4)
                self.graph.replay()
        for c in self.kv:
            c.length += 1

    # ---- on-device token loop: embedding gather and argmax inside the captured step, so that
    # consecutive replays need no host work at all (the reference reads the token back and
    # uploads the next embedding row every step, bpd/lib/dev_residency.py:1806-1818).
    def capture_device_loop(self, first_tok, capacity=4096):
        """Record embed(tok_dev) -> layers -> logits -> argmax -> tok_dev, history[step++] = tok.
        Call after seed().  `first_tok` is the token the first replay consumes."""
        global _DEVICE_EMBED
        self._assert_weight_cache_frozen()
        emb = _np(self.w["token_embd.weight"])
        _weights(emb)       # an untied table is not used by the host-driven step: upload it now
        self._weight_cache_frozen = (frozenset(_DEV_CONST.keys()), frozenset(fd._DEV_WEIGHT_CACHE.keys()),
                                     frozenset(fd._Q8_WEIGHT_CACHE.keys()))
        Wq, Wd, V, K = fd._quantize_weight_q8_0(emb)
        if K != self.E:
            raise RuntimeError("token_embd.weight must be [n_embd, vocab]")
        # the gather is exact only if the table is a Q8_0 table: check rows against the host lookup
        nb = K // 32
        for t in (0, V // 2, V - 1, int(first_tok)):
            deq = (Wq[t * K:(t + 1) * K].astype(np.float32).reshape(nb, 32) *
                   Wd[t * nb:(t + 1) * nb].astype(np.float32).reshape(nb, 1)).reshape(K)
            if not np.array_equal(deq, _embedding_row(self.w, t, K)):
                raise RuntimeError("token_embd.weight is not exactly representable as Q8_0; "
                                   "the on-device token loop would change the embedding")
        dWq, dWd, _, _ = _weights(emb)
        self._tok_dev = torch.tensor([int(first_tok)], dtype=torch.int32, device="cuda")
        self._hist = torch.zeros(capacity, dtype=torch.int32, device="cuda")
        self._step = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._hist_cap = capacity
        lens = [c.length for c in self.kv]
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        n0 = _lib.launch_count()
        if _FUSED_STEP:
            self._step_dev = FusedDecodeStep(self.w, self.cfg, self.kv, tok_ptr=self._tok_dev.data_ptr(),
                                             history=self._hist.data_ptr(), step=self._step.data_ptr(),
                                             hist_cap=capacity)
            with torch.cuda.stream(self.stream):
                self._step_dev.tune_placement()
            torch.cuda.synchronize()
            n0 = _lib.launch_count()
            with torch.cuda.graph(g, stream=self.stream):
                self._step_dev.launch()
        else:
            _DEVICE_EMBED = (dWq, dWd, ctypes.c_void_p(self._tok_dev.data_ptr()), V)
            try:
                with torch.cuda.graph(g, stream=self.stream):
                    forward_pass_resident(self.w, self.cfg, torch.tensor([0]), torch.tensor([0]), self.kv)
                    argmax_dev(_LOGITS_BUF.ptr, _LOGITS_BUF.n, self._tok_dev.data_ptr())
                    _lib.call("lt_token_record", self._tok_dev.data_ptr(), self._hist.data_ptr(),
                              self._step.data_ptr(), capacity, _stream())
            finally:
                _DEVICE_EMBED = None
        self.launches_per_step = _lib.launch_count() - n0
        for c, n in zip(self.kv, lens):
            c.length = n
        self._assert_weight_cache_frozen()
        self.loop_graph = g

    def reset_device_loop(self, first_tok):
        """Start the device loop over: next replay consumes `first_tok`, the token history is empty."""
        self.stream.synchronize()
        self._tok_dev.fill_(int(first_tok))
        self._step.zero_()
        torch.cuda.synchronize()

    def replay_device(self, n):
        """n decode steps back to back on the device; no host work between them."""
        with torch.cuda.stream(self.stream):
            for _ in range(n):
                self.loop_graph.replay()
        for c in self.kv:
            c.length += n

    def device_tokens(self):
        """Tokens chosen by the device loop so far."""
        self.stream.synchronize()
        n = min(int(self._step.item()), self._hist_cap)
        return self._hist[:n].cpu().tolist()

    def replay_logits(self, tok):
        self._launch(tok)
        self.stream.synchronize()
        return torch.from_numpy(_LOGITS_BUF.to_host()).reshape(1, 1, _LOGITS_BUF.n)

    def _raw_exec(self):
        """The cudaGraphExec_t of the captured step, if this torch exposes it (else None: the calls go one by one)."""
        if getattr(self, "_exec_ptr", None) is None:
            try:
                self._exec_ptr = int(self.graph.raw_cuda_graph_exec())
            except Exception:
                self._exec_ptr = 0
        return self._exec_ptr or None

    def replay_token(self, tok):
        """Replay, device argmax, 4 bytes back to the host."""
        assert _LOGITS_BUF is not None, "replay_token requires device logits"
        if self.fused and self._tok_in is not None and self.captured and self._raw_exec() is not None:
            # token id up, graph, chosen token down, one wait: one call into the library
            self._ensure_pinned()
            self._pin_tok_np[0] = int(tok)
            _lib.call("lt_graph_replay_token", ctypes.c_void_p(self._exec_ptr), ctypes.c_void_p(self.stream.cuda_stream),
                      self._pin_tok_np.ctypes.data, ctypes.c_void_p(self._tok_in.data_ptr()), _vp(_ensure_argmax_buf()),
                      self._pin_idx_np.ctypes.data)
            for c in self.kv:
                c.length += 1
            return int(self._pin_idx_np[0])
        self._launch(tok)
        ab = _ensure_argmax_buf()
        if not self.fused:          # the fused step already left the argmax in the buffer
            with torch.cuda.stream(self.stream):
                argmax_dev(_LOGITS_BUF.ptr, _LOGITS_BUF.n, ab)
        with torch.cuda.stream(self.stream):
            r = _rt().cudaMemcpyAsync(self._pin_idx_np.ctypes.data, _vp(ab), 4, 2, _stream())
        if r != 0:
            raise RuntimeError(f"cudaMemcpyAsync DtoH failed: {r}")
        self.stream.synchronize()          # the one host wait of the step
        return int(self._pin_idx_np[0])
