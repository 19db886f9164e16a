"""GPU: the batched / long-context decode operators against the one-sequence operators they
must reproduce bit for bit."""
import os

import numpy as np
import pytest
import torch

from llamatov_b200 import _lib
from tests.gpu_util import bits, dev, host, stream

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hd,nh,nkv,max_seq,lens", [(64, 14, 2, 256, [1, 37, 256]), (128, 32, 8, 4100, [4097, 1000]),
                                                  (128, 4, 1, 4224, [4097])])
def test_batched_attention_equals_one_sequence_attention(hd, nh, nkv, max_seq, lens):
    rng = np.random.default_rng(nh)
    B = len(lens)
    width = nkv * hd
    K = (rng.standard_normal((B, max_seq, width)) * 0.3).astype(np.float32)
    V = (rng.standard_normal((B, max_seq, width)) * 0.3).astype(np.float32)
    for b, L in enumerate(lens):                       # nothing beyond a length may be read
        K[b, L:] = np.nan; V[b, L:] = np.nan
    Q = rng.standard_normal((B, nh * hd)).astype(np.float32)
    dK, dV, dQ = dev(K.reshape(-1)), dev(V.reshape(-1)), dev(Q.reshape(-1))
    dl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = float(np.float32(hd ** -0.5))
    nscr = _lib.lib().lt_attn_decode_batch_scratch_floats(nh, max_seq, B)
    scratch = torch.empty(nscr, dtype=torch.float32, device="cuda")
    out = torch.full((B * nh * hd,), float("nan"), device="cuda")
    xq = torch.empty(B * nh * hd, dtype=torch.int8, device="cuda")
    xd = torch.empty(B * nh * hd // 32, dtype=torch.int16, device="cuda")
    _lib.call("lt_attn_decode_batch", dQ.data_ptr(), nh * hd, dK.data_ptr(), dV.data_ptr(), dl.data_ptr(),
              out.data_ptr(), nh * hd, scratch.data_ptr(), hd, nh, nkv, scale, max_seq, B, xq.data_ptr(), xd.data_ptr(),
              stream())
    got = host(out).reshape(B, nh * hd)
    # the quantised rows equal lt_quant_q8 of the output
    xq2 = torch.empty_like(xq); xd2 = torch.empty_like(xd)
    _lib.call("lt_quant_q8", out.data_ptr(), xq2.data_ptr(), xd2.data_ptr(), nh * hd, B, stream())
    assert np.array_equal(host(xq), host(xq2)) and np.array_equal(host(xd), host(xd2))
    one = torch.empty(nh * hd, device="cuda")
    for b in range(B):
        _lib.call("lt_attn_decode_masked", dQ[b * nh * hd:].data_ptr(), dK[b * max_seq * width:].data_ptr(),
                  dV[b * max_seq * width:].data_ptr(), dl[b:].data_ptr(), one.data_ptr(), hd, nh, nkv, scale, max_seq,
                  stream())
        assert np.array_equal(bits(got[b]), bits(host(one))), b
    assert _lib.device_status() == set()


def test_batched_rope_and_append():
    rng = np.random.default_rng(0)
    B, nh, nkv, hd, max_seq = 5, 4, 2, 64, 16
    ld = (nh + 2 * nkv) * hd
    X = rng.standard_normal((B, ld)).astype(np.float32)
    pos = np.array([0, 3, 15, 7, 7], np.int32)
    dX = dev(X.reshape(-1)); dp = torch.from_numpy(pos).cuda()
    _lib.call("lt_rope_batch", dX.data_ptr(), ld, dp.data_ptr(), B, nh + nkv, hd, 5e5, stream())
    got = host(dX).reshape(B, ld)
    for b in range(B):                                  # one row at a time through lt_rope
        row = dev(X[b, :(nh + nkv) * hd].copy())
        _lib.call("lt_rope", row.data_ptr(), dp[b:].data_ptr(), 1, nh + nkv, hd, 5e5, stream())
        assert np.array_equal(bits(got[b, :(nh + nkv) * hd]), bits(host(row)))
        assert np.array_equal(bits(got[b, (nh + nkv) * hd:]), bits(X[b, (nh + nkv) * hd:]))   # v untouched
    width = nkv * hd
    kc = torch.zeros(B * max_seq * width, device="cuda"); vc = torch.zeros(B * max_seq * width, device="cuda")
    lens = torch.tensor([0, 3, 15, 16, 7], dtype=torch.int32, device="cuda")     # sequence 3 is full
    _lib.call("lt_append_kv_batch", kc.data_ptr(), dX.data_ptr() + nh * hd * 4, vc.data_ptr(),
              dX.data_ptr() + (nh + nkv) * hd * 4, ld, lens.data_ptr(), width, max_seq, B, 1, stream())
    assert _lib.device_status() == {"kv_overflow"}
    assert lens.tolist() == [1, 4, 16, 16, 8]
    k = host(kc).reshape(B, max_seq, width); v = host(vc).reshape(B, max_seq, width)
    for b, L in enumerate([0, 3, 15, None, 7]):
        if L is None:
            assert not k[b].any()
            continue
        assert np.array_equal(bits(k[b, L]), bits(got[b, nh * hd:(nh + nkv) * hd]))
        assert np.array_equal(bits(v[b, L]), bits(got[b, (nh + nkv) * hd:]))
        assert np.count_nonzero(k[b].any(axis=1)) == 1
    # the fused launch: same rows, caches and lengths as the two launches
    dX2 = dev(X.reshape(-1))
    kc2 = torch.zeros_like(kc); vc2 = torch.zeros_like(vc)
    lens2 = torch.tensor([0, 3, 15, 16, 7], dtype=torch.int32, device="cuda")
    ticket = torch.zeros(B, dtype=torch.int32, device="cuda")
    _lib.call("lt_rope_append_batch", dX2.data_ptr(), ld, nh, nkv, hd, 5e5, kc2.data_ptr(), vc2.data_ptr(),
              lens2.data_ptr(), max_seq, B, ticket.data_ptr(), stream())
    assert ticket.tolist() == [0] * B
    assert _lib.device_status() == {"kv_overflow"}
    assert lens2.tolist() == [1, 4, 16, 16, 8]
    g2 = host(dX2).reshape(B, ld)
    for b in (0, 1, 2, 4):
        assert np.array_equal(bits(g2[b]), bits(got[b]))
    assert np.array_equal(bits(host(kc2)), bits(host(kc))) and np.array_equal(bits(host(vc2)), bits(host(vc)))


def _split_case(hd, nh, nkv, max_seq, lens, seed):
    rng = np.random.default_rng(seed)
    B = len(lens)
    width = nkv * hd
    K = (rng.standard_normal((B, max_seq, width)) * 0.3).astype(np.float32)
    V = (rng.standard_normal((B, max_seq, width)) * 0.3).astype(np.float32)
    for b, L in enumerate(lens):
        K[b, L:] = np.nan; V[b, L:] = np.nan
    Q = (rng.standard_normal((B, nh * hd)) * 0.3).astype(np.float32)
    return Q, K, V


def _gpu_split(Q, K, V, lens, hd, nh, nkv, max_seq, ns, quant=False):
    B = len(lens)
    dK, dV, dQ = dev(K.reshape(-1)), dev(V.reshape(-1)), dev(Q.reshape(-1))
    dl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scratch = torch.empty(_lib.lib().lt_attn_decode_split_scratch_floats(nh, hd, ns, B), device="cuda")
    out = torch.full((B * nh * hd,), float("nan"), device="cuda")
    xq = torch.empty(B * nh * hd, dtype=torch.int8, device="cuda") if quant else None
    xd = torch.empty(B * nh * hd // 32, dtype=torch.int16, device="cuda") if quant else None
    _lib.call("lt_attn_decode_split", dQ.data_ptr(), nh * hd, dK.data_ptr(), dV.data_ptr(), dl.data_ptr(), out.data_ptr(),
              nh * hd, scratch.data_ptr(), hd, nh, nkv, float(np.float32(hd ** -0.5)), max_seq, B, ns,
              None if xq is None else xq.data_ptr(), None if xd is None else xd.data_ptr(), stream())
    return out, xq, xd, (dQ, dK, dV, dl)


@pytest.mark.parametrize("ns", [2, 4])
@pytest.mark.parametrize("L", [1, 3, 40, 64, 120, 255, 256])
def test_split_order_attention_equals_the_reference_kernel(ns, L):
    # the reference's own split kernel (compiled for this GPU) with the referee's 64-thread launch
    from oracle import ref_device as ref
    if not ref.available() or not os.path.exists(os.path.join(ref.REF_DIR, f"attn_decode_split_{ns}.cubin")):
        pytest.skip("reference kernels not built")
    hd, nh, nkv, max_seq = 64, 14, 2, 256
    Q, K, V = _split_case(hd, nh, nkv, max_seq, [L], seed=L)
    out, _, _, (dQ, dK, dV, dl) = _gpu_split(Q, K, V, [L], hd, nh, nkv, max_seq, ns)
    pm = torch.empty(nh * ns, device="cuda"); pz = torch.empty(nh * ns, device="cuda")
    po = torch.empty(nh * ns * hd, device="cuda"); want = torch.empty(nh * hd, device="cuda")
    ref.attn_decode_split(dQ, dK, dV, dl, pm, pz, po, want, hd, nh, nkv, float(np.float32(hd ** -0.5)), ns, max_seq)
    assert np.array_equal(bits(host(out)), bits(host(want)))
    assert _lib.device_status() == set()


@pytest.mark.parametrize("hd,nh,nkv,max_seq,lens,ns", [(128, 32, 8, 4352, [4100, 1000, 7], 16), (64, 14, 2, 300, [300, 33], 3),
                                                      (128, 4, 1, 4352, [4097], 32)])
def test_split_order_attention_vs_oracle_and_one_range_equals_frozen_order(oracle, hd, nh, nkv, max_seq, lens, ns):
    Q, K, V = _split_case(hd, nh, nkv, max_seq, lens, seed=ns)
    B = len(lens)
    out, xq, xd, (dQ, dK, dV, dl) = _gpu_split(Q, K, V, lens, hd, nh, nkv, max_seq, ns, quant=True)
    got = host(out).reshape(B, nh * hd)
    scale = float(np.float32(hd ** -0.5))
    for b, L in enumerate(lens):
        want = oracle.attn_decode_split(Q[b], np.nan_to_num(K[b]), np.nan_to_num(V[b]), L, hd, nh, nkv, scale, ns)
        assert np.max(np.abs(got[b] - want)) < 5e-6          # __expf vs libm
    xq2 = torch.empty_like(xq); xd2 = torch.empty_like(xd)
    _lib.call("lt_quant_q8", out.data_ptr(), xq2.data_ptr(), xd2.data_ptr(), nh * hd, B, stream())
    assert np.array_equal(host(xq), host(xq2)) and np.array_equal(host(xd), host(xd2))
    # one range: the bits of the frozen one-pass order
    one, _, _, _ = _gpu_split(Q, K, V, lens, hd, nh, nkv, max_seq, 1)
    frozen = torch.empty(B * nh * hd, device="cuda")
    scr = torch.empty(_lib.lib().lt_attn_decode_batch_scratch_floats(nh, max_seq, B), device="cuda")
    _lib.call("lt_attn_decode_batch", dQ.data_ptr(), nh * hd, dK.data_ptr(), dV.data_ptr(), dl.data_ptr(),
              frozen.data_ptr(), nh * hd, scr.data_ptr(), hd, nh, nkv, scale, max_seq, B, None, None, stream())
    assert np.array_equal(bits(host(one)), bits(host(frozen)))
    assert _lib.device_status() == set()


@pytest.mark.parametrize("hd,nh,nkv,max_seq,lens,ns", [(128, 8, 2, 300, [257, 0, 31], 4), (64, 14, 2, 96, [95, 96, 5], 3),
                                                        (128, 32, 8, 4200, [4096], 16)])
def test_rope_append_inside_the_split_kernel_equals_the_separate_launches(hd, nh, nkv, max_seq, lens, ns):
    """lt_rope_attn_decode_split == lt_rope_append_batch + lt_attn_decode_split: output bits, quantised output,
    cache rows, lengths; a full cache (length == max_seq) appends nothing and is reported."""
    rng = np.random.default_rng(hd + nh + ns)
    B = len(lens)
    ld = (nh + 2 * nkv) * hd
    theta = 5e5
    scale = float(np.float32(hd ** -0.5))
    X = rng.standard_normal((B, ld)).astype(np.float32)
    K = (rng.standard_normal((B, max_seq, nkv * hd)) * 0.3).astype(np.float32)
    V = (rng.standard_normal((B, max_seq, nkv * hd)) * 0.3).astype(np.float32)
    res = []
    for fused in (False, True):
        dX, dK, dV = dev(X.reshape(-1)), dev(K.reshape(-1)), dev(V.reshape(-1))
        dl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        ticket = torch.zeros(B, dtype=torch.int32, device="cuda")
        out = torch.zeros(B * nh * hd, device="cuda")
        xq = torch.zeros(B * nh * hd, dtype=torch.int8, device="cuda")
        xd = torch.zeros(B * nh * hd // 32, dtype=torch.int16, device="cuda")
        scr = torch.empty(_lib.lib().lt_attn_decode_split_scratch_floats(nh, hd, ns, B), device="cuda")
        for _ in range(2):       # two steps: the second one reads the row the first one appended
            if fused:
                _lib.call("lt_rope_attn_decode_split", dX.data_ptr(), ld, dK.data_ptr(), dV.data_ptr(), dl.data_ptr(),
                          out.data_ptr(), nh * hd, scr.data_ptr(), hd, nh, nkv, theta, scale, max_seq, B, ns,
                          ticket.data_ptr(), xq.data_ptr(), xd.data_ptr(), stream())
            else:
                dXw = dX.clone()
                _lib.call("lt_rope_append_batch", dXw.data_ptr(), ld, nh, nkv, hd, theta, dK.data_ptr(), dV.data_ptr(),
                          dl.data_ptr(), max_seq, B, ticket.data_ptr(), stream())
                _lib.call("lt_attn_decode_split", dXw.data_ptr(), ld, dK.data_ptr(), dV.data_ptr(), dl.data_ptr(),
                          out.data_ptr(), nh * hd, scr.data_ptr(), hd, nh, nkv, scale, max_seq, B, ns, xq.data_ptr(),
                          xd.data_ptr(), stream())
        torch.cuda.synchronize()
        status = _lib.device_status()
        res.append((bits(host(out)), host(xq), host(xd), bits(host(dK)), bits(host(dV)), host(dl), host(ticket), status))
    for a, b in zip(res[0][:7], res[1][:7]):
        assert np.array_equal(a, b)
    assert res[0][7] == res[1][7]
    assert ("kv_overflow" in res[1][7]) == any(l >= max_seq - 1 for l in lens)
