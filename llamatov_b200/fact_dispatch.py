"""Host side of the Q8_0 path: weight / activation quantisers and the upload-once weight
cache, with the names and behaviour of the reference's bpd/lib/fact_dispatch.py
(`quantize_q8_0` :383-391, `_quantize_weight_q8_0` :255-282, `_dev_weight` :286-299,
`q8_0_linear_from_fp32` :356-381, `rms_norm_fact` :437-463).

The reference builds kernels at first use (Prolog emitter -> nvcc -> cubin) and launches
them through the driver API; here the kernels are precompiled into libllamatov_b200.so
and reached through its C ABI, and device memory is held by torch tensors.
"""
import ctypes

import numpy as np

from . import _lib

_Q8_WEIGHT_CACHE = {}
_DEV_WEIGHT_CACHE = {}


class Q8Weight:
    """A weight that is already Q8_0: quants int8[N*K] by output row and fp16 scales
    [N*K/32].  Accepted wherever the reference interface takes the fp32 [K, N] matrix, so
    that a model stored as Q8_0 blocks skips the dequantise / requantise detour."""
    __slots__ = ("Wq", "Wd", "N", "K", "bias")

    def __init__(self, Wq, Wd, N, K):
        self.Wq = np.ascontiguousarray(Wq, np.int8).reshape(-1)
        Wd = np.ascontiguousarray(Wd).reshape(-1)
        self.Wd = Wd.view(np.float16) if Wd.dtype == np.uint16 else Wd.astype(np.float16, copy=False)
        self.N = int(N); self.K = int(K)
        assert self.Wq.size == self.N * self.K and self.Wd.size == self.N * (self.K // 32)

    @property
    def shape(self):
        return (self.K, self.N)

    def numpy(self):
        return self

    def dequant(self):
        """fp32 [K, N] matrix (exact: f32(d) * q)."""
        w = self.Wq.reshape(self.N, self.K // 32, 32).astype(np.float32) * \
            self.Wd.reshape(self.N, self.K // 32, 1).astype(np.float32)
        return np.ascontiguousarray(w.reshape(self.N, self.K).T)

    @staticmethod
    def concat(ws):
        """Concatenate along the output dimension (rows)."""
        K = ws[0].K
        assert all(w.K == K for w in ws)
        return Q8Weight(np.concatenate([w.Wq for w in ws]), np.concatenate([w.Wd for w in ws]),
                        sum(w.N for w in ws), K)


def quantize_q8_0(vec):
    """1-D fp32 vector -> (q int8[K], d fp16[K/32]); per 32-block d = fp16(amax/127)
    (1.0 for an all-zero block), q = clip(round(v / f32(d)), -127, 127)."""
    K = vec.shape[0]
    nb = K // 32
    v = np.ascontiguousarray(vec, np.float32).reshape(nb, 32)
    amax = np.max(np.abs(v), axis=1)
    d = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float16)
    q = np.clip(np.round(v / d[:, None].astype(np.float32)), -127, 127).astype(np.int8)
    return q.reshape(K), d


def _quantize_weight_q8_0(weight2d):
    """fp32 weight [K, N] -> (Wq int8[N*K], Wd fp16[N*K/32], N, K), row n = weight[:, n].
    Cached by shape plus four sampled elements, like the reference.  A Q8Weight passes
    through untouched."""
    if isinstance(weight2d, Q8Weight):
        return weight2d.Wq, weight2d.Wd, weight2d.N, weight2d.K
    W = np.ascontiguousarray(np.asarray(weight2d, np.float32))
    flat = W.reshape(-1)
    n = flat.size
    samp = (float(flat[0]), float(flat[n // 3]), float(flat[n // 2]), float(flat[-1])) if n >= 4 else (float(flat.sum()),)
    key = (W.shape, n) + samp
    hit = _Q8_WEIGHT_CACHE.get(key)
    if hit is not None:
        return hit
    K, N = W.shape
    if K % 32 != 0:
        raise RuntimeError("Q8_0 needs K %% 32 == 0, got K=%d" % K)
    nb = K // 32
    Wq = np.empty((N, K), np.int8)
    Wd = np.empty((N, nb), np.float16)
    step = max(1, (1 << 24) // max(K, 1))      # rows per chunk: bounds temporaries to ~64 MB
    for r0 in range(0, N, step):
        blocks = np.ascontiguousarray(W[:, r0:r0 + step].T).reshape(-1, nb, 32)
        amax = np.max(np.abs(blocks), axis=2)
        d = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float16)
        q = np.clip(np.round(blocks / d[:, :, None].astype(np.float32)), -127, 127).astype(np.int8)
        Wq[r0:r0 + step] = q.reshape(-1, K)
        Wd[r0:r0 + step] = d
    res = (Wq.reshape(N * K), Wd.reshape(N * nb), N, K)
    _Q8_WEIGHT_CACHE[key] = res
    return res


def _dev_weight(Wq, Wd):
    """Upload (Wq, Wd) once; returns (dWq, dWd) as ctypes.c_void_p device pointers.  Keyed by
    the identity of the host arrays (stable: they live in the weight cache)."""
    import torch
    key = (Wq.ctypes.data, Wd.ctypes.data, Wq.nbytes)
    hit = _DEV_WEIGHT_CACHE.get(key)
    if hit is not None:
        return hit[0], hit[1]
    tq = torch.from_numpy(np.ascontiguousarray(Wq, np.int8)).cuda()
    td = torch.from_numpy(np.ascontiguousarray(Wd, np.float16).view(np.int16)).cuda()
    ent = (ctypes.c_void_p(tq.data_ptr()), ctypes.c_void_p(td.data_ptr()), tq, td, Wq, Wd)
    _DEV_WEIGHT_CACHE[key] = ent
    return ent[0], ent[1]


def _stream_handle():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def q8_0_linear_from_fp32(x, weight, mode="dp4a"):
    """y = x @ weight with the weight quantised to Q8_0 and the activation quantised per
    row, computed by the GEMV kernel.  x[K] or [T, K]; weight [K, N] -> y[N] or [T, N].
    Host round trip (upload x, download y), like the reference's function of this name.
    `mode` is accepted for signature compatibility; every mode maps to the one kernel."""
    import torch
    is_torch = hasattr(x, "numpy")
    xn = x.detach().cpu().numpy() if is_torch else np.asarray(x, np.float32)
    wn = weight.detach().cpu().numpy() if hasattr(weight, "detach") else weight
    Wq, Wd, N, K = _quantize_weight_q8_0(wn)
    dWq, dWd = _dev_weight(Wq, Wd)
    rows = np.ascontiguousarray(xn.reshape(-1, K), np.float32)
    T = rows.shape[0]
    dx = torch.from_numpy(rows).cuda()
    xq = torch.empty(T * K, dtype=torch.int8, device="cuda")
    xd = torch.empty(T * (K // 32), dtype=torch.int16, device="cuda")
    y = torch.empty(T * N, dtype=torch.float32, device="cuda")
    s = _stream_handle()
    _lib.call("lt_quant_q8", dx.data_ptr(), xq.data_ptr(), xd.data_ptr(), K, T, s)
    _lib.call("lt_q8_gemv", dWq, dWd, xq.data_ptr(), xd.data_ptr(), None, y.data_ptr(), N, K, T, s)
    out = y.cpu().numpy().reshape(T, N)
    yy = out[0] if xn.ndim == 1 else out.reshape(xn.shape[:-1] + (N,))
    return torch.from_numpy(np.ascontiguousarray(yy)) if is_torch else yy


def rms_norm_fact(x, weight, eps=1e-5):
    """RMSNorm in the declared 256-lane order, host round trip.  Accepts/returns torch or numpy."""
    import torch
    is_torch = hasattr(x, "numpy")
    xn = x.detach().cpu().numpy() if is_torch else np.asarray(x, np.float32)
    wn = weight.detach().cpu().numpy() if hasattr(weight, "detach") else np.asarray(weight, np.float32)
    shape = xn.shape
    N = shape[-1]
    M = int(np.prod(shape[:-1])) if xn.ndim > 1 else 1
    dx = torch.from_numpy(np.ascontiguousarray(xn.reshape(M, N), np.float32)).cuda()
    dw = torch.from_numpy(np.ascontiguousarray(wn, np.float32)).cuda()
    y = torch.empty_like(dx)
    _lib.call("lt_rmsnorm", dx.data_ptr(), dw.data_ptr(), y.data_ptr(), M, N, float(eps), _stream_handle())
    out = y.cpu().numpy().reshape(shape)
    return torch.from_numpy(out) if is_torch else out
