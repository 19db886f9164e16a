"""GPU: the device-resident decode engine (forward_pass_resident / GraphRunner, the
reference's entry points) against the CPU oracle engine, plus the reference's own
graph-replay == eager contract (bit-exact logits, tokens, device length, cache rows)."""
import numpy as np
import pytest
import torch

from llamatov_b200 import dev_residency as dr, synth
from tests.gpu_util import bits

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-3          # max-abs on logits (north-star tolerance for the non-reproducible ops)


def _fresh(arch, seed=0, **kw):
    dr.reset_engine_state()
    dr.apply_production_profile()
    m = synth.make_model(arch, seed=seed, **kw)
    w, cfg = synth.reference_weights(m)
    return m, w, cfg


def _prompt(V, n, seed=0):
    return np.random.default_rng(seed).integers(0, V, size=n).tolist()


def _run_gpu_eager(w, cfg, prompt, n_new):
    kv = [None] * cfg["n_layers"]
    toks = list(prompt)
    logits = dr.forward_pass_resident(w, cfg, torch.tensor(prompt), torch.arange(len(prompt)), kv)
    out = [logits.reshape(-1).numpy().copy()]
    for _ in range(n_new):
        nxt = int(np.argmax(out[-1]))
        toks.append(nxt)
        logits = dr.forward_pass_resident(w, cfg, torch.tensor([nxt]), torch.tensor([len(toks) - 1]), kv)
        out.append(logits.reshape(-1).numpy().copy())
    return toks, out, kv


@pytest.mark.parametrize("arch", ["tiny", "tiny-llama"])
def test_eager_decode_matches_oracle(oracle, arch):
    m, w, cfg = _fresh(arch, seed=1)
    V = m["cfg"]["vocab"]
    prompt = _prompt(V, 5)
    n_new = 12
    toks, logits, kv = _run_gpu_eager(w, cfg, prompt, n_new)
    eng = oracle.OracleEngine(synth.oracle_model(m), max_seq=dr._KV_MAX_SEQ)
    for t in prompt[:-1]:
        eng.step(t)
    o_logits = []
    # teacher-forced on the GPU's tokens so that one near-tie cannot cascade; token identity is
    # asserted wherever the oracle's top-1 margin exceeds the drift bound
    for t in toks[len(prompt) - 1:]:
        lg, _ = eng.step(t)
        o_logits.append(lg)
    assert len(o_logits) == len(logits) == n_new + 1
    for i, (a, b) in enumerate(zip(logits, o_logits)):
        assert np.max(np.abs(a - b)) < LOGIT_TOL, (i, np.max(np.abs(a - b)))
        top2 = np.partition(b, -2)[-2:]
        if top2[1] - top2[0] > 2 * LOGIT_TOL:
            assert int(np.argmax(a)) == int(np.argmax(b))
    # device caches equal the oracle's rows up to the rope tolerance; lengths exact
    L = len(toks)
    for il, c in enumerate(kv):
        assert c.length == L == int(eng.lens[il])
        assert int(c._len.item()) == L
        k = c.k_slice_host().reshape(L, -1)
        assert np.max(np.abs(k - eng.kc[il][:L])) < 1e-3
    assert dr._lib.device_status() == set()


def test_fp32_weight_boundary_equals_q8_boundary():
    # the reference interface hands fp32 [K, N] matrices; re-quantising them must give the
    # same device results as handing the Q8_0 blocks directly
    m, w_q8, cfg = _fresh("tiny", seed=2)
    prompt = _prompt(m["cfg"]["vocab"], 4)
    _, a, _ = _run_gpu_eager(w_q8, cfg, prompt, 3)
    dr.reset_engine_state(); dr.apply_production_profile()
    w_f32, _ = synth.reference_weights(m, dequantize=True)
    _, b, _ = _run_gpu_eager(w_f32, cfg, prompt, 3)
    for x, y in zip(a, b):
        assert np.array_equal(bits(x), bits(y))


@pytest.fixture(params=["pdl", "persistent", False], ids=["fused-pdl", "fused-persistent", "per-op-graph"])
def fused(request):
    old = dr._FUSED_STEP
    dr._FUSED_STEP = request.param
    yield request.param
    dr._FUSED_STEP = old


@pytest.mark.parametrize("arch", ["tiny", "tiny-llama"])
def test_graph_replay_equals_eager_bit_exact(fused, arch):
    # the reference's graph referee contract (bpd/kernelgen/referee/gr_referee.py:11-18,184-215);
    # with the fused step this is also the bit-exactness test of the persistent decode kernel
    # against the chain of per-op kernels
    m, w, cfg = _fresh(arch, seed=3)
    V = m["cfg"]["vocab"]
    prompt = _prompt(V, 6, seed=1)
    n_new = 10
    e_toks, e_logits, e_kv = _run_gpu_eager(w, cfg, prompt, n_new)
    e_rows = [c.k_slice_host().copy() for c in e_kv]

    dr.reset_engine_state(); dr.apply_production_profile()
    kv = [None] * cfg["n_layers"]
    gr = dr.GraphRunner(w, cfg, kv)
    lg = gr.seed(torch.tensor(prompt), torch.arange(len(prompt)))
    assert np.array_equal(bits(lg.reshape(-1).numpy()), bits(e_logits[0]))
    nxt = int(np.argmax(lg.reshape(-1).numpy()))
    gr.capture(torch.tensor([nxt]), torch.tensor([len(prompt)]))
    assert all(int(c._len.item()) == len(prompt) for c in kv)      # capture executed nothing
    toks = list(prompt)
    for i in range(n_new):
        toks.append(nxt)
        lg = gr.replay_logits(nxt).reshape(-1).numpy()
        assert np.array_equal(bits(lg), bits(e_logits[i + 1])), i
        nxt = int(np.argmax(lg))
    assert toks == e_toks
    for c, rows in zip(kv, e_rows):
        assert int(c._len.item()) == c.length == len(toks)
        assert np.array_equal(bits(c.k_slice_host()), bits(rows))
    # replay_token: device argmax == host argmax of the same logits
    t_dev = gr.replay_token(nxt)
    assert t_dev == int(np.argmax(dr._LOGITS_BUF.to_host()))
    if fused == "persistent":
        assert gr.launches_per_token == 1
    elif fused == "pdl":
        assert gr.launches_per_token == 5 * cfg["n_layers"] + 2
    assert dr._lib.device_status() == set()


def test_workspace_placement_is_chosen_by_timing_and_changes_no_bits():
    """The one-kernel step places its hand-over workspaces by timing a few steps per candidate position before
    the graph is captured: the trials leave no trace (lengths back, tokens and logits equal to an engine whose
    workspaces stay at the first position)."""
    old = (dr._FUSED_STEP, dr._WS_TUNE)
    runs = {}
    try:
        for tune in (True, False):
            dr._FUSED_STEP, dr._WS_TUNE = "persistent", tune
            m, w, cfg = _fresh("tiny-qwen64", seed=5)
            prompt = _prompt(m["cfg"]["vocab"], 5, seed=2)
            dr.reset_engine_state(); dr.apply_production_profile()
            kv = [None] * cfg["n_layers"]
            gr = dr.GraphRunner(w, cfg, kv)
            lg = gr.seed(torch.tensor(prompt), torch.arange(len(prompt)))
            nxt = int(np.argmax(lg.reshape(-1).numpy()))
            gr.capture(torch.tensor([nxt]), torch.tensor([len(prompt)]))
            assert gr._step_host.mode == "persistent"
            assert all(int(c._len.item()) == len(prompt) for c in kv)
            tried = getattr(gr._step_host, "placement_us", [])
            assert (len(tried) > 1) == tune
            out = []
            for _ in range(8):
                lgt = gr.replay_logits(nxt).reshape(-1).numpy().copy()
                nxt = int(np.argmax(lgt))
                out.append((nxt, bits(lgt)))
            runs[tune] = out
            assert dr._lib.device_status() == set()
    finally:
        dr._FUSED_STEP, dr._WS_TUNE = old
    for (ta, la), (tb, lb) in zip(runs[True], runs[False]):
        assert ta == tb and np.array_equal(la, lb)


@pytest.mark.parametrize("arch", ["tiny", "tiny-llama"])
def test_device_token_loop_equals_host_driven_loop(fused, arch):
    m, w, cfg = _fresh(arch, seed=6)
    prompt = _prompt(m["cfg"]["vocab"], 5, seed=2)
    n_new = 14
    kv = [None] * cfg["n_layers"]
    gr = dr.GraphRunner(w, cfg, kv)
    lg = gr.seed(torch.tensor(prompt), torch.arange(len(prompt)))
    first = int(np.argmax(lg.reshape(-1).numpy()))
    gr.capture(torch.tensor([first]), torch.tensor([len(prompt)]))
    tok, host_toks = first, []
    for _ in range(n_new):
        tok = gr.replay_token(tok)
        host_toks.append(tok)
    rows = [c.k_slice_host().copy() for c in kv]
    # rewind the caches to the end of the prompt and run the same steps with no host in the loop
    for c in kv:
        c.length = len(prompt); c._len.fill_(len(prompt))
    gr.capture_device_loop(first, capacity=8)      # history shorter than the run: must not overflow
    gr.replay_device(n_new)
    got = gr.device_tokens()
    assert got == host_toks[:8]
    assert int(gr._tok_dev.item()) == host_toks[-1]
    for c, r in zip(kv, rows):
        assert int(c._len.item()) == c.length == len(prompt) + n_new
        assert np.array_equal(bits(c.k_slice_host()), bits(r))
    assert dr._lib.device_status() == set()


@pytest.mark.parametrize("mode", ["pdl", "persistent"])
def test_fused_step_kv_overflow_is_flagged_not_faulted(mode):
    m, w, cfg = _fresh("tiny", seed=7)
    dr._KV_MAX_SEQ = 8
    old = dr._FUSED_STEP
    dr._FUSED_STEP = mode
    try:
        kv = [None] * cfg["n_layers"]
        gr = dr.GraphRunner(w, cfg, kv)
        gr.seed(torch.tensor([1, 2, 3]), torch.arange(3))
        gr.capture(torch.tensor([4]), torch.tensor([3]))
        t = 4
        for _ in range(5):
            t = gr.replay_token(t)
        assert dr._lib.device_status() == set()
        assert int(kv[0]._len.item()) == 8
        gr.replay_token(t)                           # ninth position: refused, flagged
        assert "kv_overflow" in dr._lib.device_status()
        assert int(kv[0]._len.item()) == 8
    finally:
        dr._FUSED_STEP = old
        dr.apply_production_profile()


def test_capture_preconditions_are_loud():
    m, w, cfg = _fresh("tiny", seed=4)
    kv = [None] * cfg["n_layers"]
    gr = dr.GraphRunner(w, cfg, kv)
    with pytest.raises(AssertionError):
        gr.replay_logits(1)
    dr._QFUSED = True
    with pytest.raises(RuntimeError, match="UNCERTIFIED"):
        gr.seed(torch.tensor([1]), torch.tensor([0]))
    dr.apply_production_profile()
    assert dr.attest_profile()["_QFUSED"] is False


def test_kv_overflow_is_flagged():
    m, w, cfg = _fresh("tiny", seed=5)
    dr._KV_MAX_SEQ = 4
    try:
        kv = [None] * cfg["n_layers"]
        for i in range(5):
            dr.forward_pass_resident(w, cfg, torch.tensor([i + 1]), torch.tensor([i]), kv)
        assert "kv_overflow" in dr._lib.device_status()
    finally:
        dr.apply_production_profile()


def test_qwen05b_greedy_128_tokens_identical_to_reference_kernels(oracle):
    """Full-size configuration: Qwen2.5-0.5B architecture, 32-token prompt, 128 greedy tokens with
    the token loop on the device (fused step), against
      (a) the REFERENCE'S OWN KERNELS chained in the reference's op sequence on this GPU
          (oracle/ref_engine.py): logits bit-identical, tokens identical -- the north-star rule;
      (b) the CPU oracle engine, whose libm transcendentals differ from the CUDA device functions
          in the last bits; over 24 layers that drift reaches a few 1e-2 on logits of O(1), so the
          bound here is loose (0.25) and tokens must agree wherever the oracle's top-1 margin
          exceeds twice the observed drift."""
    from oracle import ref_device, ref_engine
    m, w, cfg = _fresh("qwen2.5-0.5b", seed=0)
    V = m["cfg"]["vocab"]
    prompt = _prompt(V, 32)
    n_new = 128
    kv = [None] * cfg["n_layers"]
    gr = dr.GraphRunner(w, cfg, kv)
    lg = gr.seed(torch.tensor(prompt), torch.arange(32)).reshape(-1).numpy()
    first = int(np.argmax(lg))
    gr.capture_device_loop(first, capacity=256)
    gr.replay_device(n_new)
    toks = gr.device_tokens()
    assert len(toks) == n_new and dr._lib.device_status() == set()
    last_logits = dr._LOGITS_BUF.to_host().reshape(-1)
    seq = [first] + toks
    # (a) the reference's kernels on this GPU
    if ref_device.available():
        re = ref_engine.RefEngine(m, max_seq=dr._KV_MAX_SEQ)
        for t in prompt:
            rl, rnext = re.step(t)
        assert np.array_equal(bits(rl), bits(lg)), "prompt logits differ from the reference kernels"
        assert rnext == first
        for i in range(n_new):
            rl, rnext = re.step(seq[i])
            assert rnext == seq[i + 1], (i, rnext, seq[i + 1])
        assert np.array_equal(bits(rl), bits(last_logits)), "logits after 128 tokens differ from the reference kernels"
    # (b) the CPU oracle
    eng = oracle.OracleEngine(synth.oracle_model(m), max_seq=dr._KV_MAX_SEQ)
    for t in prompt:
        ol, _ = eng.step(t)
    drift = float(np.max(np.abs(ol - lg)))
    decisive = agree = 0
    for i in range(n_new):
        ol, onext = eng.step(seq[i])
        top2 = np.partition(ol, -2)[-2:]
        if i == n_new - 1:
            drift = max(drift, float(np.max(np.abs(ol - last_logits))))
        if top2[1] - top2[0] > 0.2:
            decisive += 1
            assert onext == seq[i + 1], (i, onext, seq[i + 1])
        agree += int(onext == seq[i + 1])
    print(f"qwen2.5-0.5b: {agree}/{n_new} tokens identical to the CPU oracle, {decisive} decisive steps, "
          f"max logit drift vs CPU oracle {drift:.4f}")
    assert drift < 0.25
    assert agree >= n_new - 8


def test_generate_from_gguf_equals_engine_on_the_same_weights(tmp_path):
    # the reference's runner entry points: write a synthetic model as GGUF, load it back as Q8_0 blocks,
    # generate through the graph runner, compare with eager decoding on the original arrays
    from llamatov_b200 import decode_fact, llamatov_run as R
    m, w, cfg = _fresh("tiny-qwen64", seed=11)
    a = cfg["arch"]
    md = {"general.architecture": a, f"{a}.block_count": cfg["n_layers"], f"{a}.attention.head_count": cfg["n_head"],
          f"{a}.attention.head_count_kv": cfg["n_head_kv"], f"{a}.embedding_length": cfg["n_embd"],
          f"{a}.rope.freq_base": float(cfg["rope_theta"]), f"{a}.attention.layer_norm_rms_epsilon": float(cfg["norm_eps"])}
    path = str(tmp_path / "m.gguf")
    R.write_gguf(path, md, w)
    prompt = _prompt(m["cfg"]["vocab"], 6, seed=4)
    want, _, _ = _run_gpu_eager(w, cfg, prompt, 10)
    dr.reset_engine_state()
    got = R.generate(path, prompt, 10, verbose=False)
    assert got == want
    dr.reset_engine_state()
    got2 = decode_fact.decode(path, prompt, 10)
    assert got2 == want
