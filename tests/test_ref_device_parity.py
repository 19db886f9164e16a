"""GPU parity against the REFERENCE'S OWN kernels: the CUDA texts of the reference's resident
engine and Prolog emitters, compiled for sm_100a into oracle/_ref/*.cubin where a reference
checkout was present (oracle/build.py), launched here with the reference's launch geometry.
Every comparison is bit for bit, including the ops whose device functions (rsqrtf, expf,
__expf, powf, sinf, cosf) a CPU cannot reproduce.  Inputs follow the reference's pair-gate
procedures (seeded numpy, shapes 896x4864 / 151936x896 / 896x896, K in {896, 4864})."""
import numpy as np
import pytest
import torch

from llamatov_b200 import _lib, synth
from oracle import ref_device as ref
from tests.gpu_util import bits, dev, gpu_gemv, host, stream

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref.available(), reason="oracle/_ref cubins not built (no reference checkout at build time)")]


def _pairgate_inputs(M, K, seed=8):
    # bpd/kernelgen/referee/gemv_canonical_pairgate.py:23-42
    rs = np.random.RandomState(seed)
    nb = K // 32
    Wq = rs.randint(-127, 128, size=M * K).astype(np.int8)
    Wd = (rs.randn(M * nb) * 0.1).astype(np.float16)
    Xq = rs.randint(-127, 128, size=K).astype(np.int8)
    Xd = (rs.randn(nb) * 0.1).astype(np.float16)
    return Wq, Wd, Xq, Xd


@pytest.mark.parametrize("M,K", [(896, 4864), (151936, 896), (896, 896), (4864, 896), (1152, 896), (4096, 14336)])
def test_gemv_vs_reference_kernels(oracle, M, K):
    Wq, Wd, Xq, Xd = _pairgate_inputs(M, K)
    dWq, dWd, dXq, dXd = dev(Wq), dev(Wd), dev(Xq), dev(Xd)
    mine = host(gpu_gemv(dWq, dWd, dXq, dXd, M, K))
    y = torch.empty(M, device="cuda")
    ref.q8_gemv(dWq, dWd, dXq, dXd, y, M, K)
    theirs = host(y)
    assert np.array_equal(bits(mine), bits(theirs))
    # the CPU oracle agrees with the reference kernel too (pins the oracle)
    assert np.array_equal(bits(oracle.q8_gemv(Wq, Wd, Xq, Xd, M, K)), bits(theirs))
    if M <= 4864:
        ys = torch.empty(M, device="cuda")
        ref.q8_gemv_canonical_serial(dWq, dWd, dXq, dXd, ys, M, K)
        assert np.array_equal(bits(host(ys)), bits(theirs))
    r = dev(np.random.RandomState(1).randn(M).astype(np.float32))
    y2 = torch.empty(M, device="cuda")
    ref.q8_gemv(dWq, dWd, dXq, dXd, y2, M, K, resid=r)
    assert np.array_equal(bits(host(gpu_gemv(dWq, dWd, dXq, dXd, M, K, resid=r))), bits(host(y2)))


@pytest.mark.parametrize("K", [896, 4864, 4096])
def test_quant_vs_reference_kernel(K):
    x = dev(np.random.RandomState(7).randn(K).astype(np.float32))
    a_q = torch.empty(K, dtype=torch.int8, device="cuda"); a_d = torch.empty(K // 32, dtype=torch.int16, device="cuda")
    b_q = torch.empty_like(a_q); b_d = torch.empty_like(a_d)
    _lib.call("lt_quant_q8", x.data_ptr(), a_q.data_ptr(), a_d.data_ptr(), K, 1, stream())
    ref.quant_q8(x, b_q, b_d, K)
    assert torch.equal(a_q, b_q) and torch.equal(a_d, b_d)


def test_silu_quant_vs_reference_kernel():
    K = 4864
    rs = np.random.RandomState(4)
    g = dev((rs.randn(K) * 3).astype(np.float32)); u = dev(rs.randn(K).astype(np.float32))
    a_q = torch.empty(K, dtype=torch.int8, device="cuda"); a_d = torch.empty(K // 32, dtype=torch.int16, device="cuda")
    b_q = torch.empty_like(a_q); b_d = torch.empty_like(a_d)
    _lib.call("lt_silu_mul_quant", g.data_ptr(), u.data_ptr(), a_q.data_ptr(), a_d.data_ptr(), K, 1, stream())
    ref.silu_mul_quant(g, u, b_q, b_d, K)
    assert torch.equal(a_q, b_q) and torch.equal(a_d, b_d)


@pytest.mark.parametrize("N,tag,eps", [(896, "1e-06", 1e-6), (4096, "1e-05", 1e-5)])
def test_rmsnorm_vs_reference_kernel(N, tag, eps):
    rs = np.random.RandomState(9)
    x = dev(rs.randn(2, N).astype(np.float32)); w = dev((1 + 0.1 * rs.randn(N)).astype(np.float32))
    a = torch.empty_like(x); b = torch.empty_like(x)
    _lib.call("lt_rmsnorm", x.data_ptr(), w.data_ptr(), a.data_ptr(), 2, N, eps, stream())
    ref.rmsnorm(x, w, b, 2, N, tag)
    assert np.array_equal(bits(host(a)), bits(host(b)))


@pytest.mark.parametrize("theta,tag,hd,nh", [(1e6, "1e6", 64, 16), (5e5, "5e5", 128, 40)])
def test_rope_vs_reference_kernel(theta, tag, hd, nh):
    rs = np.random.RandomState(3)
    for pos in (0, 1, 33, 159, 255, 4095):
        x = rs.randn(nh * hd).astype(np.float32)
        a = dev(x); b = dev(x)
        p = torch.tensor([pos], dtype=torch.int32, device="cuda")
        _lib.call("lt_rope", a.data_ptr(), p.data_ptr(), 1, nh, hd, theta, stream())
        ref.rope(b, p, 1, nh, hd, tag)
        assert np.array_equal(bits(host(a)), bits(host(b))), pos


@pytest.mark.parametrize("nh,nkv,hd,maxt", [(14, 2, 64, 256), (32, 8, 128, 512)])
def test_attention_vs_reference_kernel(nh, nkv, hd, maxt):
    rs = np.random.RandomState(5)
    q = dev(rs.randn(nh * hd).astype(np.float32))
    kc = dev(rs.randn(maxt * nkv * hd).astype(np.float32)); vc = dev(rs.randn(maxt * nkv * hd).astype(np.float32))
    scale = float(np.float32(hd ** -0.5))
    for L in (1, 2, maxt // 2, maxt - 1, maxt):
        ln = torch.tensor([L], dtype=torch.int32, device="cuda")
        a = torch.empty(nh * hd, device="cuda"); b = torch.empty(nh * hd, device="cuda")
        _lib.call("lt_attn_decode_masked", q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ln.data_ptr(), a.data_ptr(),
                  hd, nh, nkv, scale, maxt, stream())
        ref.attn_decode_masked(q, kc, vc, ln, b, hd, nh, nkv, scale, maxt)
        assert np.array_equal(bits(host(a)), bits(host(b))), L


def test_argmax_and_append_vs_reference_kernels():
    rs = np.random.RandomState(6)
    v = rs.randn(151936).astype(np.float32); v[[5000, 120000]] = v.max() + 1
    dv = dev(v)
    part = torch.empty(_lib.lib().lt_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    a = torch.zeros(1, dtype=torch.int32, device="cuda"); b = torch.zeros(1, dtype=torch.int32, device="cuda")
    pv = torch.empty(256, device="cuda"); pi = torch.empty(256, dtype=torch.int32, device="cuda")
    _lib.call("lt_argmax", dv.data_ptr(), v.size, part.data_ptr(), a.data_ptr(), stream())
    ref.argmax2(dv, v.size, pv, pi, b)
    assert int(a.item()) == int(b.item()) == 5000
    width = 128
    ka = torch.zeros(8 * width, device="cuda"); va = torch.zeros_like(ka); kb = torch.zeros_like(ka); vb = torch.zeros_like(ka)
    la = torch.tensor([3], dtype=torch.int32, device="cuda"); lb = la.clone()
    k = dev(rs.randn(width).astype(np.float32)); vv = dev(rs.randn(width).astype(np.float32))
    _lib.call("lt_append_kv", ka.data_ptr(), k.data_ptr(), va.data_ptr(), vv.data_ptr(), la.data_ptr(), width, 8, 1, stream())
    ref.append_kv_incr(kb, k, vb, vv, lb, width)
    assert torch.equal(ka, kb) and torch.equal(va, vb) and int(la.item()) == int(lb.item()) == 4
