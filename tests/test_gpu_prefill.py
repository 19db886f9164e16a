"""GPU: the batched prompt prefill (row-batched operators + tensor-core GEMM + chunk attention)
against the reference's own way of prefilling, one token at a time through the decode step.
The two must agree bit for bit: logits, every KV-cache row, device lengths."""
import ctypes

import numpy as np
import pytest
import torch

from llamatov_b200 import _lib, dev_residency as dr, prefill, synth
from tests.gpu_util import bits, dev, host, stream

pytestmark = pytest.mark.gpu


def _fresh(arch, seed=0, **kw):
    dr.reset_engine_state()
    dr.apply_production_profile()
    m = synth.make_model(arch, seed=seed, **kw)
    w, cfg = synth.reference_weights(m)
    return m, w, cfg


def _prefill(w, cfg, prompt, batched, max_seq=256):
    dr._BATCHED_PREFILL = batched
    dr._KV_MAX_SEQ = max_seq
    try:
        kv = [None] * cfg["n_layers"]
        logits = dr.forward_pass_resident(w, cfg, torch.tensor(prompt), torch.arange(len(prompt)), kv)
    finally:
        dr._BATCHED_PREFILL = True
    return logits.reshape(-1).numpy().copy(), kv


@pytest.mark.parametrize("arch,T", [("tiny-llama", 1 + 16), ("tiny-llama", 37), ("tiny-qwen64", 70), ("tiny-qwen64", 150)])
def test_batched_prefill_equals_token_by_token(arch, T):
    m, w, cfg = _fresh(arch, seed=3)
    assert prefill.supported(cfg, w)
    prompt = np.random.default_rng(T).integers(0, m["cfg"]["vocab"], size=T).tolist()
    la, kva = _prefill(w, cfg, prompt, batched=False)
    lb, kvb = _prefill(w, cfg, prompt, batched=True)
    assert np.array_equal(bits(la), bits(lb))
    for ca, cb in zip(kva, kvb):
        assert ca.length == cb.length == T
        assert int(ca._len.item()) == int(cb._len.item()) == T
        assert np.array_equal(bits(ca.k_slice_host()), bits(cb.k_slice_host()))
        assert np.array_equal(bits(ca.v_slice_host()), bits(cb.v_slice_host()))
    assert _lib.device_status() == set()


@pytest.mark.parametrize("batch", [1, 8])
def test_qwen05b_prefill_2048_tokens_equals_token_by_token_on_a_sample(batch):
    """BASELINE config 3 at its stated size: Qwen2.5-0.5B architecture (depth cut to 4 layers so that the
    token-by-token arm, 2048 decode steps, stays within the test budget; every operator runs at the full
    widths and the full 2048 rows), batch 1 and batch 8.  Batched prefill against the reference's way
    (one token at a time through the decode step): last-position logits bit-equal, and 64 sampled KV rows
    of every layer bit-equal, for the first and the last sequence of the batch."""
    T = 2048
    m, w, cfg = _fresh("qwen2.5-0.5b", seed=0, n_layers=4)
    V = m["cfg"]["vocab"]
    rng = np.random.default_rng(batch)
    prompts = rng.integers(0, V, size=(batch, T))
    dr._KV_MAX_SEQ = T
    try:
        kvs = [[None] * cfg["n_layers"] for _ in range(batch)]
        # (prefill_resident returns the logits of the last sequence's last position)
        lb = prefill.prefill_resident(w, cfg, torch.from_numpy(prompts.astype(np.int64)), kvs).reshape(-1).numpy().copy() \
            if batch > 1 else prefill_chunks(w, cfg, prompts[0], kvs[0])
        rows = np.sort(rng.choice(T, size=64, replace=False))
        for s in sorted({0, batch - 1}):
            la, kva = _prefill(w, cfg, prompts[s].tolist(), batched=False, max_seq=T)
            if s == batch - 1:
                assert np.array_equal(bits(la), bits(lb)), s
            for ca, cb in zip(kva, kvs[s]):
                assert ca.length == cb.length == T
                assert np.array_equal(bits(ca.k_slice_host()[rows]), bits(cb.k_slice_host()[rows]))
                assert np.array_equal(bits(ca.v_slice_host()[rows]), bits(cb.v_slice_host()[rows]))
            for c in kva:
                c.free()
        assert _lib.device_status() == set()
    finally:
        dr._KV_MAX_SEQ = 256


def prefill_chunks(w, cfg, prompt, kv):
    """One sequence through prefill_resident in chunks of its row capacity; returns the last logits."""
    last = None
    for c0 in range(0, len(prompt), prefill.MAX_ROWS):
        last = prefill.prefill_resident(w, cfg, torch.from_numpy(np.asarray(prompt[c0:c0 + prefill.MAX_ROWS], np.int64)), kv,
                                        want_logits=c0 + prefill.MAX_ROWS >= len(prompt))
    return last.reshape(-1).numpy().copy()


def test_prefill_in_two_chunks_then_decode():
    # a second chunk continues from the cache of the first; decoding afterwards continues from both
    m, w, cfg = _fresh("tiny-qwen64", seed=5)
    V = m["cfg"]["vocab"]
    prompt = np.random.default_rng(1).integers(0, V, size=90).tolist()
    la, kva = _prefill(w, cfg, prompt, batched=False)
    dr._KV_MAX_SEQ = 256
    kv = [None] * cfg["n_layers"]
    prefill.prefill_resident(w, cfg, torch.tensor(prompt[:50]), kv, want_logits=False)
    lb = prefill.prefill_resident(w, cfg, torch.tensor(prompt[50:]), kv).reshape(-1).numpy()
    assert np.array_equal(bits(la), bits(lb))
    nxt = int(np.argmax(la))
    a = dr.forward_pass_resident(w, cfg, torch.tensor([nxt]), torch.tensor([90]), kva).reshape(-1).numpy()
    b = dr.forward_pass_resident(w, cfg, torch.tensor([nxt]), torch.tensor([90]), kv).reshape(-1).numpy()
    assert np.array_equal(bits(a), bits(b))


def test_prefill_of_two_sequences_together():
    m, w, cfg = _fresh("tiny-llama", seed=7)
    V = m["cfg"]["vocab"]
    rng = np.random.default_rng(2)
    p0, p1 = rng.integers(0, V, size=40).tolist(), rng.integers(0, V, size=40).tolist()
    _, kv0 = _prefill(w, cfg, p0, batched=False)
    l1, kv1 = _prefill(w, cfg, p1, batched=False)
    dr._KV_MAX_SEQ = 256
    kvs = [[None] * cfg["n_layers"], [None] * cfg["n_layers"]]
    lb = prefill.prefill_resident(w, cfg, torch.tensor([p0, p1]), kvs).reshape(-1).numpy()
    assert np.array_equal(bits(l1), bits(lb))
    for ref, got in ((kv0, kvs[0]), (kv1, kvs[1])):
        for ca, cb in zip(ref, got):
            assert np.array_equal(bits(ca.k_slice_host()), bits(cb.k_slice_host()))
            assert np.array_equal(bits(ca.v_slice_host()), bits(cb.v_slice_host()))


def test_prefill_overflow_is_refused_on_the_host_and_flagged_on_the_device():
    m, w, cfg = _fresh("tiny-llama", seed=1)
    dr._KV_MAX_SEQ = 32
    kv = [None] * cfg["n_layers"]
    with pytest.raises(RuntimeError, match="overflow"):
        prefill.prefill_resident(w, cfg, torch.arange(40) % 600, kv)
    dr._KV_MAX_SEQ = 256
    # device side: rows that do not fit are not written and the length stays
    width, max_seq = 8, 4
    kb = torch.zeros(max_seq * width, device="cuda"); vb = torch.zeros(max_seq * width, device="cuda")
    src = torch.ones(3 * width, device="cuda")
    ln = torch.tensor([2], dtype=torch.int32, device="cuda")
    _lib.call("lt_append_kv_rows", kb.data_ptr(), src.data_ptr(), vb.data_ptr(), src.data_ptr(), width,
              ln.data_ptr(), width, max_seq, 3, 1, stream())
    assert _lib.device_status() == {"kv_overflow"}
    assert int(ln.item()) == 2 and float(kb.sum().item()) == 0.0


@pytest.mark.parametrize("hd,nh,nkv", [(64, 14, 2), (128, 8, 2)])
def test_chunk_attention_equals_one_token_attention(hd, nh, nkv):
    # rows appended after 37 cached positions; every row against lt_attn_decode_masked at its own length
    rng = np.random.default_rng(hd)
    L0, T, maxseq = 37, 45, 128
    width = nkv * hd
    K = (rng.standard_normal((maxseq, width)) * 0.5).astype(np.float32)
    Vv = rng.standard_normal((maxseq, width)).astype(np.float32)
    K[L0 + T:] = np.nan; Vv[L0 + T:] = np.nan          # nothing beyond the length may be read
    Q = rng.standard_normal((T, nh * hd)).astype(np.float32)
    dK, dV, dQ = dev(K.reshape(-1)), dev(Vv.reshape(-1)), dev(Q.reshape(-1))
    scale = float(np.float32(hd ** -0.5))
    out = torch.full((T * nh * hd,), float("nan"), device="cuda")
    ln = torch.tensor([L0 + T], dtype=torch.int32, device="cuda")
    _lib.call("lt_attn_prefill", dQ.data_ptr(), nh * hd, dK.data_ptr(), dV.data_ptr(), ln.data_ptr(), out.data_ptr(),
              nh * hd, hd, nh, nkv, scale, T, L0 + T, stream())
    got = host(out).reshape(T, nh * hd)
    one = torch.empty(nh * hd, device="cuda")
    for r in range(T):
        ln1 = torch.tensor([L0 + r + 1], dtype=torch.int32, device="cuda")
        _lib.call("lt_attn_decode_masked", dQ[r * nh * hd:].data_ptr(), dK.data_ptr(), dV.data_ptr(), ln1.data_ptr(),
                  one.data_ptr(), hd, nh, nkv, scale, maxseq, stream())
        assert np.array_equal(bits(got[r]), bits(host(one))), r
    assert _lib.device_status() == set()
