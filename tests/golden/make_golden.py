#!/usr/bin/env python3
"""Generate tests/golden/*.npz by running the REFERENCE's own Python host functions in a
container that has the reference checkout (it does not travel to the GPU box; the vectors
do).  Usage:  python tests/golden/make_golden.py [--reference /path/to/LlamaTov]

What is pinned, and by which reference function:
  quantize_q8_0.npz        bpd/lib/fact_dispatch.py:383-391   quantize_q8_0(vec)
                           (the device k_quant_q8 is written to match it bit for bit,
                            bpd/lib/dev_residency.py:806,867-886)
  quantize_weight_q8_0.npz bpd/lib/fact_dispatch.py:255-282   _quantize_weight_q8_0(W[K,N])
  rope_soft.npz            bpd/llamatov_run.py:516-550        apply_rope (torch; a soft,
                           non-bit-exact reference for k_rope, as the reference itself says)
  rmsnorm_soft.npz         bpd/llamatov_run.py:513-514        rms_norm (torch; soft)
  dequant_q8_0.npz         bpd/llamatov_run.py:184-207        dq8_0 on a synthetic 34-byte-block file

The reference stores no numeric fixture for the GEMV, attention or decode results; those
are pinned on the GPU against the reference's own kernels compiled for sm_100a
(oracle/_ref/*.cubin, built by oracle/build.py).
"""
import argparse
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def inputs_for_quant(rng):
    cases = {}
    for K in (32, 896, 4864):
        cases[f"randn_{K}"] = rng.standard_normal(K).astype(np.float32)
    x = rng.standard_normal(256).astype(np.float32)
    x[0:32] = 0.0                                   # all-zero block -> d = 1.0
    x[32:64] *= 1e-6                                # tiny magnitudes (fp16 subnormal scale)
    x[64:96] *= 1e4                                 # large magnitudes
    x[96:128] = np.linspace(-1, 1, 32, dtype=np.float32)
    x[128:160] = np.float32(0.5) * np.arange(-16, 16, dtype=np.float32)   # exact .5 ties after scaling
    x[160] = np.float32(3.0e38)                     # near fp32 max in a block of small values
    cases["edge_256"] = x
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LLAMATOV_REFERENCE"),
                    help="path of the reference checkout (or set LLAMATOV_REFERENCE)")
    a = ap.parse_args()
    if not a.reference:
        ap.error("give --reference or set LLAMATOV_REFERENCE")
    os.environ.setdefault("FACT_CUBIN_CACHE", tempfile.mkdtemp(prefix="fact_cubins_"))
    sys.path.insert(0, os.path.join(a.reference, "bpd", "lib"))
    sys.path.insert(0, os.path.join(a.reference, "bpd"))
    import fact_dispatch as rfd          # the reference's module
    import llamatov_run as R             # the reference's module
    import torch

    rng = np.random.default_rng(20260612)

    out = {}
    for name, x in inputs_for_quant(rng).items():
        q, d = rfd.quantize_q8_0(x)
        out[name + "__x"] = x
        out[name + "__q"] = q
        out[name + "__d"] = d.view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "quantize_q8_0.npz"), **out)

    W = (rng.standard_normal((96, 24)) * 0.05).astype(np.float32)      # [K=96, N=24]
    W[0:32, 3] = 0.0                                                   # an all-zero block
    Wq, Wd, N, K = rfd._quantize_weight_q8_0(W)
    np.savez_compressed(os.path.join(HERE, "quantize_weight_q8_0.npz"), W=W, Wq=Wq, Wd=Wd.view(np.uint16),
                        N=np.int32(N), K=np.int32(K))

    nh, nkv, hd = 4, 2, 64
    q = rng.standard_normal((1, 3, nh * hd)).astype(np.float32)
    k = rng.standard_normal((1, 3, nkv * hd)).astype(np.float32)
    pos = np.array([0, 7, 159], np.int64)
    rope = {}
    for theta in (1e6, 5e5):
        qr, kr = R.apply_rope(torch.from_numpy(q), torch.from_numpy(k), nh, hd, theta, positions=torch.from_numpy(pos))
        rope[f"q_{theta:g}"] = qr.numpy(); rope[f"k_{theta:g}"] = kr.numpy()
    np.savez_compressed(os.path.join(HERE, "rope_soft.npz"), q=q, k=k, pos=pos, nh=np.int32(nh), nkv=np.int32(nkv),
                        hd=np.int32(hd), **rope)

    x = rng.standard_normal((3, 896)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(896)).astype(np.float32)
    y = R.rms_norm(torch.from_numpy(x), torch.from_numpy(w), 1e-6).numpy()
    np.savez_compressed(os.path.join(HERE, "rmsnorm_soft.npz"), x=x, w=w, y=y, eps=np.float32(1e-6))

    # dq8_0: write 34-byte blocks (fp16 scale + 32 int8) for a [ne0=K=64, ne1=N=5] tensor
    K2, N2 = 64, 5
    nb = N2 * K2 // 32
    d = (np.abs(rng.standard_normal(nb)) * 0.02).astype(np.float16)
    qs = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8)
    raw = np.empty((nb, 34), np.uint8)
    raw[:, :2] = d.view(np.uint8).reshape(nb, 2)
    raw[:, 2:] = qs.view(np.uint8)
    with tempfile.NamedTemporaryFile(suffix=".bin", delete=False) as f:
        f.write(raw.tobytes()); path = f.name
    deq = R.dq8_0(path, 0, N2 * K2, (K2, N2)).numpy()              # [K, N]
    os.unlink(path)
    np.savez_compressed(os.path.join(HERE, "dequant_q8_0.npz"), raw=raw, deq=deq, K=np.int32(K2), N=np.int32(N2))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
