"""CPU: the GGUF reader / writer and the reference-shaped loaders (llamatov_b200.llamatov_run):
dq8_0 against the reference's own output (tests/golden/dequant_q8_0.npz), a write -> parse -> load
round trip of a synthetic model, Q8_0 blocks arriving unchanged."""
import os

import numpy as np
import pytest
import torch

from llamatov_b200 import decode_fact, llamatov_run as R, synth
from llamatov_b200.fact_dispatch import Q8Weight


def test_dq8_0_matches_reference_golden(golden_dir, tmp_path):
    g = np.load(os.path.join(golden_dir, "dequant_q8_0.npz"))
    K, N = int(g["K"]), int(g["N"])
    p = tmp_path / "blocks.bin"
    g["raw"].tofile(p)
    got = R.dq8_0(str(p), 0, K * N, [K, N]).numpy()
    assert got.shape == (K, N) and np.array_equal(got, g["deq"])
    w = R.q8_0_blocks(str(p), 0, K * N, [K, N])
    assert np.array_equal(w.dequant(), g["deq"])


def _export(tmp_path, arch="tiny-qwen64"):
    m = synth.make_model(arch, seed=3)
    w, cfg = synth.reference_weights(m)
    a = cfg["arch"]
    md = {"general.architecture": a, f"{a}.block_count": cfg["n_layers"], f"{a}.attention.head_count": cfg["n_head"],
          f"{a}.attention.head_count_kv": cfg["n_head_kv"], f"{a}.embedding_length": cfg["n_embd"],
          f"{a}.rope.freq_base": float(cfg["rope_theta"]), f"{a}.attention.layer_norm_rms_epsilon": float(cfg["norm_eps"])}
    path = str(tmp_path / "model.gguf")
    R.write_gguf(path, md, w)
    return m, w, cfg, path


def test_gguf_round_trip(tmp_path):
    m, w, cfg, path = _export(tmp_path)
    md, ts, do = R.parse_gguf(path)
    assert md["general.architecture"] == "qwen2" and set(ts) == set(w) and do % 32 == 0
    cfg2, w2 = decode_fact.load_model(path)
    for k in cfg2:       # float metadata are fp32 in the file: the value the kernels use anyway
        assert cfg2[k] == cfg[k] or np.float32(cfg2[k]) == np.float32(cfg[k]), k
    for n, t in w.items():
        u = w2[n]
        if isinstance(t, Q8Weight):
            assert isinstance(u, Q8Weight) and (u.N, u.K) == (t.N, t.K)
            assert np.array_equal(u.Wq, t.Wq) and np.array_equal(u.Wd.view(np.uint16), t.Wd.view(np.uint16))
        else:
            assert torch.equal(u, t)
    # the fp32 route of the reference loader: same logical [K, N] matrix
    _c, w3 = R.load_model(path, q8_blocks=False)
    n = "blk.0.ffn_down.weight"
    assert tuple(w3[n].shape) == w[n].shape and np.array_equal(w3[n].numpy(), w[n].dequant())


def test_step_tensors_and_refusals(tmp_path):
    tok, pos = decode_fact.step_tensors([5, 6, 7], 0)
    assert tok.tolist() == [5, 6, 7] and pos.tolist() == [0, 1, 2]
    tok, pos = decode_fact.step_tensors([5, 6, 7, 9], 2)
    assert tok.tolist() == [9] and pos.tolist() == [3]
    with pytest.raises(RuntimeError, match="no CPU execution path"):
        R.generate("x.gguf", [1], 2, device="cpu")
    with pytest.raises(NotImplementedError):
        decode_fact.forward_pass({}, {}, None, None, [], lin=decode_fact.fp32lin)
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"NOPE" + b"\0" * 32)
    with pytest.raises(ValueError, match="Not GGUF"):
        R.parse_gguf(str(bad))
