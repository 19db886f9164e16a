"""GPU: lt_q8_linear_static, the decode linear for callers that cannot allocate.

A host application that lends this library its buffers may forbid any cudaMalloc from plugin
code (its memory budget is fixed), and code running while a stream is being recorded must not
allocate either.  For those callers the quantised activation lives in a __device__ array
inside the library instead of caller scratch.  This test calls the entry point through the
C ABI twice in a row -- a long activation first, a short one second, so that stale bytes of
the first call sit right behind the second call's data -- and requires the results to equal,
bit for bit, what lt_quant_q8 + lt_q8_gemv produce with caller-allocated scratch.  It also
checks that an activation longer than the built-in scratch is refused with a clear message.

The file name sorts last on purpose: pytest collects it after every other test, and it must
pass both alone in a fresh process and after the rest of the suite."""
import numpy as np
import pytest
import torch

from llamatov_b200 import _lib, synth
from tests.gpu_util import bits, dev, gpu_gemv, gpu_quant, host, stream

pytestmark = pytest.mark.gpu


def _static_linear(dWq, dWd, dx, M, K, resid=None):
    y = torch.empty(M, dtype=torch.float32, device="cuda")
    _lib.call("lt_q8_linear_static", dWq.data_ptr(), dWd.data_ptr(), dx.data_ptr(),
              None if resid is None else resid.data_ptr(), y.data_ptr(), M, K, stream())
    return y


def test_static_scratch_linear_matches_caller_scratch_on_two_calls_in_a_row():
    cases = [(896, 4864, 11), (1152, 896, 12)]          # long K first, then short K
    prepared = []
    for M, K, seed in cases:
        Wq, Wd, x = synth.gemv_case(M, K, seed=seed)
        r = np.random.default_rng(seed).standard_normal(M).astype(np.float32)
        prepared.append((M, K, dev(Wq), dev(Wd), dev(x[0]), dev(r), x[0]))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    got = [_static_linear(dWq, dWd, dx, M, K, resid=dr) for (M, K, dWq, dWd, dx, dr, _) in prepared]
    torch.cuda.synchronize()
    # the outputs were allocated by the test (torch); the entry point itself took nothing more
    assert free_before - torch.cuda.mem_get_info()[0] <= 4 << 20
    for (M, K, dWq, dWd, dx, dr, x), y in zip(prepared, got):
        xq, xd = gpu_quant(x)
        want = gpu_gemv(dWq, dWd, xq, xd, M, K, resid=dr)
        assert np.array_equal(bits(host(y)), bits(host(want))), (M, K)
    # same inputs again: the array kept the last call's bytes, the answer does not change
    M, K, dWq, dWd, dx, dr, _ = prepared[0]
    again = _static_linear(dWq, dWd, dx, M, K, resid=dr)
    assert np.array_equal(bits(host(again)), bits(host(got[0])))
    assert _lib.device_status() == set()


def test_static_scratch_rejects_oversized_k():
    max_k = _lib.lib().lt_q8_linear_static_max_k()
    assert max_k == 16384
    t = torch.zeros(64, dtype=torch.float32, device="cuda")
    rc = _lib.lib().lt_q8_linear_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 1,
                                        max_k + 32, stream())
    assert rc == 1 and "exceeds the built-in scratch" in _lib.last_error()
    rc = _lib.lib().lt_q8_linear_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 1, 48, stream())
    assert rc == 1 and "multiple of 32" in _lib.last_error()


def test_static_scratch_at_the_maximum_k():
    M, K = 64, 16384
    Wq, Wd, x = synth.gemv_case(M, K, seed=5)
    dWq, dWd, dx = dev(Wq), dev(Wd), dev(x[0])
    y = _static_linear(dWq, dWd, dx, M, K)
    xq, xd = gpu_quant(x[0])
    assert np.array_equal(bits(host(y)), bits(host(gpu_gemv(dWq, dWd, xq, xd, M, K))))


def test_static_scratch_linear_inside_a_captured_graph():
    """A caller that is recording a stream: one eager call first (function attributes, occupancy and the
    symbol address are settled outside the capture), then the same call recorded into a CUDA graph and
    replayed twice -- the bits of the eager result, no allocation by the entry point during capture or replay."""
    M, K = 896, 4864
    Wq, Wd, x = synth.gemv_case(M, K, seed=21)
    r = np.random.default_rng(21).standard_normal(M).astype(np.float32)
    dWq, dWd, dx, dr = dev(Wq), dev(Wd), dev(x[0]), dev(r)
    eager = host(_static_linear(dWq, dWd, dx, M, K, resid=dr)).copy()
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        rc = _lib.lib().lt_q8_linear_static(dWq.data_ptr(), dWd.data_ptr(), dx.data_ptr(), dr.data_ptr(), y.data_ptr(),
                                            M, K, stream())
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert np.array_equal(bits(host(y)), bits(eager))
    assert free_before - torch.cuda.mem_get_info()[0] <= 1 << 20
    assert _lib.device_status() == set()
