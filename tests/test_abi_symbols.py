"""CPU: the C-ABI library loads and exports every entry point include/llamatov_b200.h
declares; the Python binding table names exactly those; argument validation (which runs on
the host before any launch) returns error codes and text instead of raising across the ABI."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "llamatov_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lt_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    from llamatov_b200 import _lib
    names = _declared()
    assert "lt_q8_gemv" in names and "lt_last_error" in names and len(names) >= 15
    L = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} declared in the header but not exported"
    bound = set(_lib.SIGNATURES) | set(_lib._RESTYPES) | set(_lib._QUERIES)
    assert bound == set(names), (sorted(bound - set(names)), sorted(set(names) - bound))


def test_argument_validation_without_gpu():
    from llamatov_b200 import _lib
    L = _lib.lib()
    assert b"sm_100a" in L.lt_version()
    one = ctypes.c_void_p(256)     # never dereferenced: validation fails first
    assert L.lt_q8_gemv(one, one, one, one, None, one, 4, 48, 1, None) == 1
    assert "multiple of 32" in _lib.last_error()
    assert L.lt_q8_gemv(None, one, one, one, None, one, 4, 64, 1, None) == 1
    assert "null" in _lib.last_error()
    assert L.lt_q8_gemv(ctypes.c_void_p(260), one, one, one, None, one, 4, 64, 1, None) == 1
    assert "aligned" in _lib.last_error()
    assert L.lt_argmax(one, 0, one, one, None) == 1
    assert L.lt_rope(one, one, 1, 2, 63, 1e6, None) == 1
    assert L.lt_attn_decode_masked(one, one, one, one, one, 64, 14, 4, 0.125, 256, None) == 1
    assert "multiple of nkv" in _lib.last_error()
    with pytest.raises(RuntimeError):
        _lib.check(1, "probe")


def test_missing_library_fails_loudly(monkeypatch):
    from llamatov_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libllamatov_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
