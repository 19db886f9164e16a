"""GPU: the tensor-parallel batched decoder.  On one GPU (world 1) against the CPU oracle engine and
against itself (batch of sequences == the sequences one by one; graph replay == eager); on two or
more GPUs (NCCL, one process per GPU) against world 1: identical greedy tokens, logits within the
re-association tolerance."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from llamatov_b200 import _lib, synth, tp

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-3


def _cfg(m):
    return m["cfg"]


def test_world1_matches_oracle_engine(oracle):
    m = synth.make_model("tiny-llama", seed=4)
    dec = tp.TPDecoder(_cfg(m), batch=1, max_seq=64, model=m)
    eng = oracle.OracleEngine(synth.oracle_model(m), max_seq=64)
    tok = 11
    dec.set_tokens([tok])
    for i in range(10):
        dec.step()
        torch.cuda.synchronize()
        lg, nxt = eng.step(tok)
        got = dec.logits[0].cpu().numpy()
        assert np.max(np.abs(got - lg)) < LOGIT_TOL, i
        top2 = np.partition(lg, -2)[-2:]
        tok = int(dec.tok[0].item())
        if top2[1] - top2[0] > 2 * LOGIT_TOL:
            assert tok == nxt
    assert all(int(l[0].item()) == 10 for l in dec.lens)
    assert _lib.device_status() == set()


def test_batch_equals_sequences_one_by_one_and_graph_equals_eager():
    m = synth.make_model("tiny-llama", seed=6)
    starts = [3, 77, 500]
    d3 = tp.TPDecoder(_cfg(m), batch=3, max_seq=64, model=m)
    d3.fill_cache(5, seed=9)
    d3.set_tokens(starts)
    eager = d3.run(8)
    for b, s in enumerate(starts):
        d = tp.TPDecoder(_cfg(m), batch=1, max_seq=64, model=m)
        d.fill_cache(5, seed=9)
        for il in range(len(d.kc)):       # sequence b's cache rows
            w = d.plan.nk_l
            d.kc[il].view(1, 64, w)[0].copy_(d3.kc[il].view(3, 64, w)[b]); d.vc[il].view(1, 64, w)[0].copy_(d3.vc[il].view(3, 64, w)[b])
            d.kc[il].view(1, 64, w)[0, 5:].zero_(); d.vc[il].view(1, 64, w)[0, 5:].zero_()
        d.set_tokens([s])
        assert np.array_equal(d.run(8)[:, 0], eager[:, b]), b
    g3 = tp.TPDecoder(_cfg(m), batch=3, max_seq=64, model=m)
    g3.fill_cache(5, seed=9)
    g3.set_tokens(starts)
    g3.step(); first = g3.tok.clone()
    g3.capture()                      # its warm-up step runs (2 steps so far); the recorded pass does not
    torch.cuda.synchronize()
    rest = g3.run(6)
    assert np.array_equal(first.cpu().numpy(), eager[0])
    assert np.array_equal(rest, eager[2:8])
    assert _lib.device_status() == set()


@pytest.mark.parametrize("attn_split", [0, 4])
def test_chained_launches_give_the_same_bits(attn_split):
    """One sequence, eager and from a graph: programmatic launch chaining changes when kernels start, not what
    they compute."""
    m = synth.make_model("tiny-llama", seed=11)
    out = {}
    for chained in (False, True):
        d = tp.TPDecoder(_cfg(m), batch=1, max_seq=64, model=m, attn_split=attn_split, chained=chained)
        d.fill_cache(7, seed=4)
        d.set_tokens([19])
        toks, logits = [], []
        for _ in range(5):
            d.step()
            torch.cuda.synchronize()
            toks.append(int(d.tok[0].item())); logits.append(d.logits.cpu().numpy().copy())
        d.capture()
        torch.cuda.synchronize()
        more = d.run(6)
        out[chained] = (np.array(toks), np.concatenate(logits, axis=0), more, d.logits.cpu().numpy().copy())
    for a, b in zip(out[False], out[True]):
        assert np.array_equal(a.view(np.int32) if a.dtype == np.float32 else a, b.view(np.int32) if b.dtype == np.float32 else b)
    assert _lib.device_status() == set()


@pytest.mark.parametrize("g", [2, 4, 8])
@pytest.mark.parametrize("shape", [(96, 896 * 2, 1), (64, 14336, 1), (40, 4864, 3)])
def test_exact_row_split_partials_sum_to_the_one_gpu_bits(g, shape):
    """The exact tensor-parallel row split, all ranks' shares computed on this one GPU: rank r holds the Q8_0
    blocks b = r mod g of every row, lt_q8_gemv_lanes folds its lanes, and the partials added in the lane
    tree's order (p[t] + p[t + s], s = g/2 .. 1, plain fp32 adds on the host) must equal lt_q8_gemv on the
    whole matrix bit for bit (which the kernel tests pin to the oracle)."""
    from tests.gpu_util import dev, gpu_gemv, gpu_quant, host, stream
    M, K, T = shape
    nb = K // 32
    if nb % g:
        pytest.skip("blocks do not deal evenly")
    Wq, Wd, x = synth.gemv_case(M, K, T=T, seed=11 + g)
    xq, xd = gpu_quant(x, rows=T)
    want = host(gpu_gemv(dev(Wq), dev(Wd), xq, xd, M, K, T))
    Wq3 = Wq.reshape(M, nb, 32); Wd2 = Wd.reshape(M, nb)
    xq3 = host(xq).reshape(T, nb, 32); xd2 = host(xd).reshape(T, nb)
    parts = []
    for r in range(g):
        wq = np.ascontiguousarray(Wq3[:, r::g, :]).reshape(-1); wd = np.ascontiguousarray(Wd2[:, r::g]).reshape(-1)
        lxq = dev(np.ascontiguousarray(xq3[:, r::g, :]).reshape(-1)); lxd = dev(np.ascontiguousarray(xd2[:, r::g]).reshape(-1))
        dwq, dwd = dev(wq), dev(wd)             # (named: a temporary's memory may be handed out again before the launch runs)
        y = torch.empty(T * M, dtype=torch.float32, device="cuda")
        _lib.call("lt_q8_gemv_lanes", dwq.data_ptr(), dwd.data_ptr(), lxq.data_ptr(), lxd.data_ptr(), y.data_ptr(),
                  M, K // g, T, g, stream())
        torch.cuda.synchronize()
        parts.append(host(y).copy())
    s = g // 2
    while s >= 1:
        for t_ in range(s):
            parts[t_] = (parts[t_] + parts[t_ + s]).astype(np.float32)
        s //= 2
    assert np.array_equal(parts[0].view(np.uint32), want.view(np.uint32))
    assert _lib.device_status() == set()


def test_exchange_wait_gives_up_and_the_context_stays_usable():
    """A rank whose peer never delivers: the bounded waits of the all-reduce kernel and of the GEMV with the
    all-reduce epilogue run out (about a second), the kernels return, the status word says wait_timeout, the
    exchange counters still advance (the ranks stay in step), and the GPU keeps working.  The "peer" is a second
    rank slot that points at this rank's own staging memory, which nobody fills: no fault, no hang."""
    import ctypes
    from tests.gpu_util import dev, gpu_gemv, gpu_quant, host, stream
    c = tp._CommStruct()
    handles = (ctypes.c_ubyte * 64)()
    n = 1024
    _lib.call("lt_comm_alloc", 2, n, ctypes.byref(c), handles)
    try:
        c.rank = 0
        c.stage[0] = c.local_stage
        c.stage[1] = c.local_stage            # rank 1's words are expected here and never come
        part = torch.ones(n, device="cuda"); out = torch.zeros(n, device="cuda")
        _lib.call("lt_allreduce_add", ctypes.byref(c), part.data_ptr(), None, out.data_ptr(), n, stream())
        torch.cuda.synchronize()
        assert "wait_timeout" in _lib.device_status()
        M, K = 64, 256
        Wq, Wd, x = synth.gemv_case(M, K, seed=1)
        xq, xd = gpu_quant(x[0])
        y = torch.zeros(M, device="cuda")
        dWq, dWd = dev(Wq), dev(Wd)
        for _ in range(2):      # twice: the second call must not find the row counters out of step with its own pushes
            _lib.call("lt_q8_gemv_allreduce", ctypes.byref(c), dWq.data_ptr(), dWd.data_ptr(), xq.data_ptr(),
                      xd.data_ptr(), None, y.data_ptr(), M, K, stream())
            torch.cuda.synchronize()
            assert "wait_timeout" in _lib.device_status()
        # the context is intact: an ordinary GEMV still gives the oracle-pinned bits
        y2 = host(gpu_gemv(dWq, dWd, xq, xd, M, K))
        assert np.isfinite(y2).all() and _lib.device_status() == set()
    finally:
        c.stage[1] = None
        torch.cuda.synchronize()
        _lib.call("lt_comm_free", ctypes.byref(c))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_world2_matches_world1(tmp_path):
    """Two ranks under torch.distributed.run (tests/tp_worker.py) against this process at world 1."""
    import subprocess
    m = synth.make_model("tiny-llama", seed=8)
    ref = tp.TPDecoder(m["cfg"], batch=2, max_seq=64, model=m)
    ref.fill_cache(6, seed=2)
    ref.set_tokens([5, 600])
    rt, rl = [], []
    for _ in range(6):
        ref.step(); torch.cuda.synchronize()
        rt.append(ref.tok.cpu().numpy().copy()); rl.append(ref.logits.cpu().numpy().copy())
    ref.step()                        # the warm-up step of the workers' capture()
    rmore = ref.run(3)
    # the exact row split of `down` alone: the worker ranks run TPDecoder._row_split(exact=True) on a seeded
    # [E, F] matrix and activation; here the same product on one GPU with lt_q8_gemv (+ residual)
    from tests.gpu_util import dev, gpu_gemv, gpu_quant, host
    E_, F_ = m["cfg"]["n_embd"], m["cfg"]["n_ffn"]
    Wq, Wd, xx = synth.gemv_case(E_, F_, T=1, seed=77)
    xq, xd = gpu_quant(xx, rows=1)
    resid = np.random.default_rng(78).standard_normal(E_).astype(np.float32)
    want_down = host(gpu_gemv(dev(Wq), dev(Wd), xq, xd, E_, F_, 1, resid=dev(resid)))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(root, "tests", "tp_worker.py"), str(tmp_path)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    r = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = [np.load(os.path.join(str(tmp_path), f"rank{k}.npz")) for k in range(2)]
    V = m["cfg"]["vocab"]
    full = np.concatenate([res[0]["logits"], res[1]["logits"]], axis=1)[:, :V]      # vocabulary halves side by side
    want = np.concatenate(rl, axis=0)
    assert np.max(np.abs(full - want)) < LOGIT_TOL
    for k in range(2):
        assert np.array_equal(res[k]["toks"], np.stack(rt)), k
        assert np.array_equal(res[k]["more"], rmore), k
        assert int(res[k]["status"]) == 0
        assert int(res[k]["p2p_equals_nccl"]) == 1
        # exact row split of down: both exchange paths give the one-GPU bits
        for name in ("down_exact_p2p", "down_exact_nccl"):
            assert np.array_equal(res[k][name].view(np.uint32), want_down.view(np.uint32)), (k, name)


def _run_comm_worker(tmp_path, world):
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(root, "tests", "comm_worker.py"), str(tmp_path)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    r = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for k in range(world):
        res = np.load(os.path.join(str(tmp_path), f"comm{k}.npz"))
        assert int(res["ok_sum"]) == 1, k          # all-reduce = the rank-order fp32 sum, bit for bit
        assert int(res["ok_tok"]) == 1, k          # tokens over vocabulary slices = argmax of the whole rows
        assert int(res["status"]) == 0, k


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_exchange_kernels_world2(tmp_path):
    """lt_allreduce_add and lt_argmax_rows called directly on two ranks (tests/comm_worker.py)."""
    _run_comm_worker(tmp_path, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_exchange_kernels_world4(tmp_path):
    """The same on four ranks, where long vectors take the two-stage all-reduce."""
    _run_comm_worker(tmp_path, 4)
