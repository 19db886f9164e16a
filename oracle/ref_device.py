"""Run the reference's own CUDA kernels (oracle/_ref/*.cubin, compiled for sm_100a from the
reference checkout by oracle/build.py) on the GPU, for bit comparison with the product
kernels and as a same-box timing bar.

TEST INFRASTRUCTURE ONLY.  Launch geometry follows the reference's launch sites in
bpd/lib/dev_residency.py (cited per function).  Device memory is passed as torch tensors.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
_cu = None
_mods = {}


def available():
    return os.path.exists(os.path.join(REF_DIR, "q8_gemv_tiled_v4.cubin"))


def _driver():
    global _cu
    if _cu is None:
        torch.cuda.init()
        torch.zeros(1, device="cuda")          # makes the primary context current
        _cu = ctypes.CDLL("libcuda.so.1")
        _cu.cuInit(0)
    return _cu


def _func(cubin, kname):
    cu = _driver()
    key = (cubin, kname)
    if key not in _mods:
        if cubin not in _mods:
            mod = ctypes.c_void_p()
            r = cu.cuModuleLoad(ctypes.byref(mod), os.path.join(REF_DIR, cubin + ".cubin").encode())
            if r != 0:
                raise RuntimeError(f"cuModuleLoad({cubin}) = {r}")
            _mods[cubin] = mod
        fn = ctypes.c_void_p()
        r = cu.cuModuleGetFunction(ctypes.byref(fn), _mods[cubin], kname.encode())
        if r != 0:
            raise RuntimeError(f"cuModuleGetFunction({kname}) = {r}")
        _mods[key] = fn
    return _mods[key]


def _launch(fn, grid, block, shmem, args):
    cu = _driver()
    conv = []
    for a in args:
        if isinstance(a, torch.Tensor):
            conv.append(ctypes.c_void_p(a.data_ptr()))
        elif isinstance(a, float):
            conv.append(ctypes.c_float(a))
        elif isinstance(a, int):
            conv.append(ctypes.c_int(a))
        else:
            conv.append(a)
    argv = (ctypes.c_void_p * len(conv))(*[ctypes.cast(ctypes.byref(a), ctypes.c_void_p) for a in conv])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if shmem > 48 * 1024:
        cu.cuFuncSetAttribute(fn, 8, ctypes.c_int(shmem))   # MAX_DYNAMIC_SHARED_SIZE_BYTES
    r = cu.cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, shmem, stream, argv, None)
    if r != 0:
        raise RuntimeError(f"cuLaunchKernel = {r}")


def quant_q8(X, Xq, Xd, K):
    """k_quant_q8, warp per block (launch: bpd/lib/dev_residency.py:898-904)."""
    nb = K // 32
    _launch(_func("quant_q8_par", "k_quant_q8"), (nb + 7) // 8, 256, 0, [X, Xq, Xd, K])


def silu_mul_quant(g, u, Xq, Xd, K):
    """(launch: bpd/lib/dev_residency.py:597-604)"""
    nb = K // 32
    _launch(_func("silu_mul_quant", "k_silu_mul_quant"), (nb + 7) // 8, 256, 0, [g, u, Xq, Xd, K])


def q8_gemv(Wq, Wd, Xq, Xd, Y, M, K, resid=None):
    """k_q8_0_gemv / k_q8_0_gemv_addres, BM=16 (launch: bpd/lib/dev_residency.py:971-972,1031-1032)."""
    nb = K // 32
    grid, block, shmem = (M + 15) // 16, 512, K + nb * 2
    if resid is None:
        _launch(_func("q8_gemv_tiled_v4", "k_q8_0_gemv"), grid, block, shmem, [Wq, Wd, Xq, Xd, Y, M, K])
    else:
        _launch(_func("q8_gemv_tiled_v4_addres", "k_q8_0_gemv_addres"), grid, block, shmem,
                [Wq, Wd, Xq, Xd, resid, Y, M, K])


def q8_gemv_canonical_serial(Wq, Wd, Xq, Xd, Y, M, K):
    _launch(_func("q8_gemv_canonical_serial", "k_q8_0_gemv"), (M + 63) // 64, 64, 0, [Wq, Wd, Xq, Xd, Y, M, K])


def rmsnorm(x, w, y, M, N, eps_tag="1e-06"):
    """k_rmsnorm block_row (launch: bpd/lib/dev_residency.py:773-777)."""
    _launch(_func("rmsnorm_blockrow_" + eps_tag, "k_rmsnorm"), M, 256, 1024, [x, w, y, M, N])


def rope(X, pos, nrows, n_head, hd, theta_tag="1e6"):
    """k_rope (launch: bpd/lib/dev_residency.py:737-741)."""
    total = nrows * n_head * (hd // 2)
    _launch(_func("rope_" + theta_tag, "k_rope"), (total + 255) // 256, 256, 0, [X, pos, nrows, n_head, hd])


def append_kv_incr(kb, ks, vb, vs, length, width):
    """k_append_kv_incr (launch: bpd/lib/dev_residency.py:515-520); width <= 128."""
    assert width <= 128
    _launch(_func("append_at_len", "k_append_kv_incr"), 1, 128, 0, [kb, ks, vb, vs, length, width])


def attn_decode_masked(Q, K, V, length, OUT, hd, nh, nkv, scale, maxt):
    """k_attn_decode_masked (launch: bpd/lib/dev_residency.py:2023-2030)."""
    _launch(_func(f"attn_decode_masked_{maxt}", "k_attn_decode_masked"), nh, 256, maxt * 4 + 256,
            [Q, K, V, length, OUT, hd, nh, nkv, float(scale)])


def attn_decode_split(Q, K, V, length, partM, partZ, partO, OUT, hd, nh, nkv, scale, nsplit, maxt=256):
    """k_attn_decode_split + k_attn_decode_combine with the referee's launch geometry: 64 threads per
    (head, range) block (bpd/kernelgen/referee/gatebench_attn_split.py)."""
    assert hd <= 64, "the reference launches this kernel with 64 threads: hd <= 64"
    name = f"attn_decode_split_{nsplit}"
    _launch(_func(name, "k_attn_decode_split"), nh * nsplit, 64, maxt * 4 + 1024 * 4,
            [Q, K, V, length, partM, partZ, partO, hd, nh, nkv, float(scale)])
    _launch(_func(name, "k_attn_decode_combine"), nh, hd, 0, [partM, partZ, partO, OUT, hd, nh])


def argmax2(x, n, pval, pidx, out):
    """k_argmax_s1 + k_argmax_s2, 256 stage-1 blocks (launch: bpd/lib/dev_residency.py:1096-1103)."""
    _launch(_func("argmax2", "k_argmax_s1"), 256, 256, 0, [x, n, 256, pval, pidx])
    _launch(_func("argmax2", "k_argmax_s2"), 1, 256, 0, [pval, pidx, 256, out])
