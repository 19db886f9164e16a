"""Helpers for the GPU parity tests: call the C ABI with torch device buffers."""
import ctypes

import numpy as np
import torch

from llamatov_b200 import _lib


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.int16)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


def host(t, dtype=None):
    a = t.cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def gpu_quant(x, rows=1):
    x = np.ascontiguousarray(x, np.float32).reshape(rows, -1)
    K = x.shape[1]
    dx = dev(x)
    xq = torch.empty(rows * K, dtype=torch.int8, device="cuda")
    xd = torch.empty(rows * (K // 32), dtype=torch.int16, device="cuda")
    _lib.call("lt_quant_q8", dx.data_ptr(), xq.data_ptr(), xd.data_ptr(), K, rows, stream())
    return xq, xd


def gpu_gemv(dWq, dWd, dXq, dXd, M, K, T=1, resid=None):
    y = torch.empty(T * M, dtype=torch.float32, device="cuda")
    _lib.call("lt_q8_gemv", dWq.data_ptr(), dWd.data_ptr(), dXq.data_ptr(), dXd.data_ptr(),
              None if resid is None else resid.data_ptr(), y.data_ptr(), M, K, T, stream())
    return y


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def ulp_diff(a, b):
    a = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7fffffff), a)
    b = np.where(b < 0, -(b & 0x7fffffff), b)
    return np.abs(a - b)
