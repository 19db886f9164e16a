"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (there are no model files): a Q8_0 matrix + activation for the GEMV cases
and random-initialised Q8_0 transformer weights of a named architecture.

Weights of a model are drawn as fp32 N(0, sigma) and quantised with the engine's own weight
rule (fact_dispatch._quantize_weight_q8_0), which maps each block's largest magnitude to
+-127; re-quantising the dequantised matrix then reproduces the same blocks, so the fp32
boundary and the direct Q8_0 boundary carry identical weights.
"""
import numpy as np

from .fact_dispatch import Q8Weight

ARCHS = {
    # Qwen2.5-0.5B architecture
    "qwen2.5-0.5b": dict(n_layers=24, n_embd=896, n_head=14, n_head_kv=2, hd=64, n_ffn=4864,
                         norm_eps=1e-6, rope_theta=1e6, vocab=151936, qkv_bias=True, tied=True, arch="qwen2"),
    # Llama-3-8B architecture
    "llama-3-8b": dict(n_layers=32, n_embd=4096, n_head=32, n_head_kv=8, hd=128, n_ffn=14336,
                       norm_eps=1e-5, rope_theta=5e5, vocab=128256, qkv_bias=False, tied=False, arch="llama"),
    # small shapes for tests (same structure: GQA, bias, tied head)
    "tiny": dict(n_layers=2, n_embd=128, n_head=4, n_head_kv=2, hd=32, n_ffn=256,
                 norm_eps=1e-6, rope_theta=1e6, vocab=512, qkv_bias=True, tied=True, arch="qwen2"),
    "tiny-qwen64": dict(n_layers=2, n_embd=256, n_head=4, n_head_kv=2, hd=64, n_ffn=384,
                        norm_eps=1e-6, rope_theta=1e6, vocab=512, qkv_bias=True, tied=True, arch="qwen2"),
    "tiny-llama": dict(n_layers=2, n_embd=256, n_head=4, n_head_kv=2, hd=64, n_ffn=512,
                       norm_eps=1e-5, rope_theta=5e5, vocab=640, qkv_bias=False, tied=False, arch="llama"),
}


def gemv_case(N, K, T=1, seed=0):
    """Benchmark GEMV input: per block d = fp16(|N(0,1)| * 0.02), q ~ U{-127..127};
    x ~ N(0,1) fp32 [T, K].  numpy.random.default_rng(seed)."""
    rng = np.random.default_rng(seed)
    nb = K // 32
    Wd = (np.abs(rng.standard_normal((N, nb), dtype=np.float32)) * np.float32(0.02)).astype(np.float16)
    Wq = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    x = rng.standard_normal((T, K), dtype=np.float32)
    return Wq.reshape(-1), Wd.reshape(-1), x


def _quant_rows(W):
    """W fp32 [N, K] (rows = outputs) -> Q8Weight, the engine's weight rule, chunked."""
    N, K = W.shape
    nb = K // 32
    Wq = np.empty((N, K), np.int8)
    Wd = np.empty((N, nb), np.float16)
    step = max(1, (1 << 24) // K)
    for r0 in range(0, N, step):
        blocks = W[r0:r0 + step].reshape(-1, nb, 32)
        amax = np.max(np.abs(blocks), axis=2)
        d = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float16)
        q = np.clip(np.round(blocks / d[:, :, None].astype(np.float32)), -127, 127).astype(np.int8)
        Wq[r0:r0 + step] = q.reshape(-1, K)
        Wd[r0:r0 + step] = d
    return Q8Weight(Wq.reshape(-1), Wd.reshape(-1), N, K)


def _rand_q8(rng, N, K, sigma):
    W = rng.standard_normal((N, K), dtype=np.float32)
    W *= np.float32(sigma)
    return _quant_rows(W)


def make_model(arch="qwen2.5-0.5b", seed=0, n_layers=None, sigma=0.02):
    """Random-init Q8_0 model.  Returns {"cfg", "token_embd", "lm_head", "output_norm", "layers"}
    where each matrix is a Q8Weight and each layer holds the concatenated q|k|v and gate|up
    matrices the engine runs."""
    a = dict(ARCHS[arch])
    if n_layers is not None:
        a["n_layers"] = n_layers
    rng = np.random.default_rng(seed)
    E, nh, nkv, hd, F, V = a["n_embd"], a["n_head"], a["n_head_kv"], a["hd"], a["n_ffn"], a["vocab"]
    nq, nk = nh * hd, nkv * hd
    layers = []
    for _ in range(a["n_layers"]):
        ly = {
            "attn_norm": (1.0 + 0.1 * rng.standard_normal(E, dtype=np.float32)).astype(np.float32),
            "qkv": _rand_q8(rng, nq + 2 * nk, E, sigma),
            "qkv_bias": (0.02 * rng.standard_normal(nq + 2 * nk, dtype=np.float32)).astype(np.float32)
            if a["qkv_bias"] else None,
            "o": _rand_q8(rng, E, nq, sigma),
            "ffn_norm": (1.0 + 0.1 * rng.standard_normal(E, dtype=np.float32)).astype(np.float32),
            "gateup": _rand_q8(rng, 2 * F, E, sigma),
            "down": _rand_q8(rng, E, F, sigma),
        }
        layers.append(ly)
    embd = _rand_q8(rng, V, E, sigma)
    lm = embd if a["tied"] else _rand_q8(rng, V, E, sigma)
    cfg = dict(n_layers=a["n_layers"], n_head=nh, n_head_kv=nkv, n_embd=E, rope_theta=a["rope_theta"],
               norm_eps=a["norm_eps"], arch=a["arch"], hd=hd, n_ffn=F, vocab=V, tied=a["tied"], name=arch)
    return {"cfg": cfg, "token_embd": embd, "lm_head": lm,
            "output_norm": (1.0 + 0.1 * rng.standard_normal(E, dtype=np.float32)).astype(np.float32),
            "layers": layers}


def _rows(w, r0, r1):
    nb = w.K // 32
    return Q8Weight(w.Wq[r0 * w.K:r1 * w.K], w.Wd[r0 * nb:r1 * nb], r1 - r0, w.K)


def reference_weights(model, dequantize=False):
    """(w, cfg) in the reference's data model: GGUF tensor names -> matrices [K_in, N_out].
    With dequantize=True the matrices are fp32 torch tensors (what the reference's loader
    returns); otherwise they are Q8Weight objects, which the engine accepts in their place."""
    import torch
    cfg = {k: model["cfg"][k] for k in ("n_layers", "n_head", "n_head_kv", "n_embd", "rope_theta", "norm_eps", "arch")}
    c = model["cfg"]
    nq, nk = c["n_head"] * c["hd"], c["n_head_kv"] * c["hd"]
    F = c["n_ffn"]

    def mat(q8):
        return torch.from_numpy(q8.dequant()) if dequantize else q8

    def vec(v):
        return torch.from_numpy(np.ascontiguousarray(v, np.float32))
    w = {"token_embd.weight": mat(model["token_embd"]), "output_norm.weight": vec(model["output_norm"])}
    if not c["tied"]:
        w["output.weight"] = mat(model["lm_head"])
    for i, ly in enumerate(model["layers"]):
        p = f"blk.{i}"
        w[f"{p}.attn_norm.weight"] = vec(ly["attn_norm"])
        w[f"{p}.attn_q.weight"] = mat(_rows(ly["qkv"], 0, nq))
        w[f"{p}.attn_k.weight"] = mat(_rows(ly["qkv"], nq, nq + nk))
        w[f"{p}.attn_v.weight"] = mat(_rows(ly["qkv"], nq + nk, nq + 2 * nk))
        if ly["qkv_bias"] is not None:
            w[f"{p}.attn_q.bias"] = vec(ly["qkv_bias"][:nq])
            w[f"{p}.attn_k.bias"] = vec(ly["qkv_bias"][nq:nq + nk])
            w[f"{p}.attn_v.bias"] = vec(ly["qkv_bias"][nq + nk:])
        w[f"{p}.attn_output.weight"] = mat(ly["o"])
        w[f"{p}.ffn_norm.weight"] = vec(ly["ffn_norm"])
        w[f"{p}.ffn_gate.weight"] = mat(_rows(ly["gateup"], 0, F))
        w[f"{p}.ffn_up.weight"] = mat(_rows(ly["gateup"], F, 2 * F))
        w[f"{p}.ffn_down.weight"] = mat(ly["down"])
    return w, cfg


def oracle_model(model):
    """The same model as plain arrays for the CPU checker: (Wq, Wd) pairs."""
    def pair(q8):
        return (q8.Wq, q8.Wd)
    out = {"cfg": model["cfg"], "token_embd": pair(model["token_embd"]), "lm_head": pair(model["lm_head"]),
           "output_norm": model["output_norm"], "layers": []}
    for ly in model["layers"]:
        out["layers"].append({"attn_norm": ly["attn_norm"], "qkv": pair(ly["qkv"]), "qkv_bias": ly["qkv_bias"],
                              "o": pair(ly["o"]), "ffn_norm": ly["ffn_norm"], "gateup": pair(ly["gateup"]),
                              "down": pair(ly["down"])})
    return out
