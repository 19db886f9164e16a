"""ctypes binding of libllamatov_b200.so (the C ABI declared in include/llamatov_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails, a RuntimeError
is raised with the library's own error text.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libllamatov_b200.so")
_lib = None

LT_OK = 0
STATUS_BITS = {1: "kv_overflow", 2: "bad_length", 4: "bad_token", 8: "wait_timeout"}

_vp = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float
_l = ctypes.c_long

# name -> argtypes (all return int unless listed in _RESTYPES)
SIGNATURES = {
    "lt_device_status": [ctypes.POINTER(ctypes.c_uint), _vp],
    "lt_quant_q8": [_vp, _vp, _vp, _i, _i, _vp],
    "lt_silu_mul_quant": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "lt_silu_mul": [_vp, _vp, _vp, _i, _vp],
    "lt_add": [_vp, _vp, _vp, _i, _vp],
    "lt_q8_gemv": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "lt_q8_gemm_tc": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "lt_quant_q8_ggml": [_vp, _vp, _vp, _i, _i, _vp],
    "lt_q8_gemm_ggml": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "lt_rmsnorm": [_vp, _vp, _vp, _i, _i, _f, _vp],
    "lt_rmsnorm_quant": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp],
    "lt_q8_gemv_allreduce": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lt_rmsnorm_q8_gemv": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _vp],
    "lt_rope": [_vp, _vp, _i, _i, _i, _f, _vp],
    "lt_append_kv": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "lt_incr_len": [_vp, _vp],
    "lt_attn_decode_masked": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "lt_argmax": [_vp, _i, _vp, _vp, _vp],
    "lt_argmax_scratch_bytes": [],
    "lt_argmax_rows_scratch_bytes": [_i],
    "lt_embed_q8": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "lt_token_record": [_vp, _vp, _vp, _i, _vp],
    "lt_graph_replay_token": [_vp, _vp, _vp, _vp, _vp, _vp],
    "lt_embed_q8_rows": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "lt_rope_rows": [_vp, _i, _vp, _i, _i, _i, _f, _vp],
    "lt_append_kv_rows": [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "lt_silu_mul_quant_rows": [_vp, _vp, _i, _vp, _vp, _i, _i, _vp],
    "lt_attn_prefill": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp],
    "lt_rope_batch": [_vp, _i, _vp, _i, _i, _i, _f, _vp],
    "lt_append_kv_batch": [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "lt_attn_decode_batch": [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp],
    "lt_attn_decode_split": [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _f, _i, _i, _i, _vp, _vp, _vp],
    "lt_rope_attn_decode_split": [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _f, _f, _i, _i, _i, _vp, _vp, _vp, _vp],
    "lt_rope_append_batch": [_vp, _i, _i, _i, _i, _f, _vp, _vp, _vp, _i, _i, _vp, _vp],
    "lt_comm_alloc": [_i, _i, _vp, _vp],
    "lt_comm_connect": [_vp, _i, _vp],
    "lt_comm_free": [_vp],
    "lt_allreduce_add": [_vp, _vp, _vp, _vp, _i, _vp],
    "lt_allreduce_add_tree": [_vp, _vp, _vp, _vp, _i, _vp],
    "lt_argmax_rows": [_vp, _vp, _l, _i, _i, _i, _vp, _vp, _vp],
    "lt_q8_gemv_lanes": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lt_q8_linear_static": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lt_q8_linear_static_max_k": [],
    "lt_decode_step": [_vp, _vp],
    "lt_decode_step_supported": [_vp],
    "lt_decode_num_ctas": [],
    "lt_decode_ws_replicas": [],
    "lt_decode_step_pdl": [_vp, _vp],
    "lt_decode_pdl_num_parts": [],
}
_RESTYPES = {"lt_last_error": ctypes.c_char_p, "lt_version": ctypes.c_char_p,
             "lt_launch_count": ctypes.c_ulonglong}
# name -> (argtypes, restype) for the entries that return something other than a status code
_QUERIES = {"lt_attn_decode_batch_scratch_floats": ([_i, _i, _i], ctypes.c_long),
            "lt_attn_decode_split_scratch_floats": ([_i, _i, _i, _i], ctypes.c_long),
            "lt_set_chained_launch": ([_i], ctypes.c_int)}


def lib():
    """The loaded library (loads on first use)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libllamatov_b200.so is not built (%s). Run `python -m llamatov_b200.build`; "
                "this package has no CPU or PyTorch fallback." % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        for name, rt in _RESTYPES.items():
            fn = getattr(L, name)
            fn.argtypes = []
            fn.restype = rt
        for name, (args, rt) in _QUERIES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = rt
        _lib = L
    return _lib


def last_error():
    return lib().lt_last_error().decode("utf-8", "replace")


def check(rc, what=""):
    """Raise RuntimeError if a launcher returned a non-zero code."""
    if rc != LT_OK:
        raise RuntimeError("llamatov_b200 %s failed (code %d): %s" % (what, rc, last_error()))


def call(name, *args):
    check(getattr(lib(), name)(*args), name)


def launch_count():
    return int(lib().lt_launch_count())


def device_status(stream=None):
    """Read and clear the device status word; returns the set of flag names."""
    v = ctypes.c_uint(0)
    check(lib().lt_device_status(ctypes.byref(v), stream), "lt_device_status")
    return {n for bit, n in STATUS_BITS.items() if v.value & bit}
