"""The reference's KV-cache decode driver (bpd/decode_fact.py) on the device-resident engine.

Kept entry points: `load_model(path) -> (cfg, w)` (:39-51), `step_tensors(generated, step)` (:105-111,
prefill at step 0, one token afterwards), `forward_pass(w, cfg, tok, positions, kv_cache, lin, rms)`
(:54-102) and `decode(path, input_ids, n_tokens, mode)` (:114-141).  In the reference `forward_pass`
is a host loop that sends every linear through the GPU and back (`q8lin`, the "int8" arm) or runs
torch fp32 (`fp32lin`, its reference arm).  Here the int8 arm is the whole layer loop on the device
(`dev_residency.forward_pass_resident`): `kv_cache` is the list of `DeviceKVCache`, `lin` must be
`q8lin` and `rms` is accepted for signature compatibility (the device path applies the same
`norm_eps`).  The fp32 arm is the reference's own torch code and is not reproduced.
"""
import time

import torch

from . import dev_residency as dr
from . import fact_dispatch as fd
from . import llamatov_run as R


def q8lin(h, w, b=None):
    """The Q8_0 linear through the host boundary (bpd/decode_fact.py:23-28): one GEMV per call."""
    y = fd.q8_0_linear_from_fp32(h, w)
    if b is not None and not isinstance(b, int):
        y = y + b
    return y


def fp32lin(h, w, b=None):
    raise NotImplementedError("the fp32 arm is the reference's torch code (bpd/decode_fact.py:31-36); "
                              "this package runs the Q8_0 arm only")


def load_model(path):
    """Parse GGUF, build cfg, load tensors; Q8_0 matrices stay Q8_0 blocks."""
    cfg, w = R.load_model(path)
    cfg = {k: cfg[k] for k in ("n_layers", "n_head", "n_head_kv", "n_embd", "rope_theta", "norm_eps", "arch")}
    return cfg, w


def forward_pass(w, cfg, tok, positions, kv_cache, lin=q8lin, rms=None):
    """One forward over `tok` (all prompt ids at step 0, the last id afterwards); returns logits
    [1, 1, vocab] of the last position and advances the device KV caches."""
    if lin is not q8lin:
        raise NotImplementedError("forward_pass: only lin=q8lin (the Q8_0 device path) is implemented")
    return dr.forward_pass_resident(w, cfg, tok, positions, kv_cache)


def step_tensors(generated, step):
    """The per-step (tok, positions) pair: prefill at step 0, one-token decode after."""
    if step == 0:
        return torch.tensor(generated, dtype=torch.long), torch.arange(len(generated))
    return torch.tensor([generated[-1]], dtype=torch.long), torch.tensor([len(generated) - 1])


def decode(path, input_ids, n_tokens=10, mode="int8", preloaded=None):
    """Eager KV-cache decode, one `forward_pass` per step (the reference's loop; `llamatov_run.generate`
    is the graph-replay form)."""
    if mode != "int8":
        raise NotImplementedError("decode: mode='int8' only")
    cfg, w = preloaded if preloaded is not None else load_model(path)
    nl = cfg["n_layers"]
    print(f"Arch {cfg['arch']} layers {nl} heads {cfg['n_head']}/{cfg['n_head_kv']} embd {cfg['n_embd']}", flush=True)
    dr.apply_production_profile()
    dr._KV_MAX_SEQ = max(dr._KV_MAX_SEQ, len(input_ids) + n_tokens + 1)
    kv_cache = [None] * nl
    generated = list(input_ids)
    step_times = []
    for step in range(n_tokens):
        t_step = time.time()
        tok, positions = step_tensors(generated, step)
        logits = forward_pass(w, cfg, tok, positions, kv_cache, q8lin, None)
        nxt = int(logits[0, -1].argmax().item())
        generated.append(nxt)
        step_times.append(time.time() - t_step)
    dec = step_times[1:]
    if dec:
        print(f"DECODE tok/s: {len(dec) / sum(dec):.2f} ({sum(dec) / len(dec) * 1000:.1f}ms/token), "
              f"prefill={step_times[0]:.2f}s", flush=True)
    print(f"GENERATED: {generated[len(input_ids):]}", flush=True)
    return generated
