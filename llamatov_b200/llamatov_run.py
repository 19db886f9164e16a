#!/usr/bin/env python3
"""The reference's benchmark-runner entry points for the Q8_0 decode path (bpd/llamatov_run.py):
GGUF parsing, tensor loading, `load_model`, `generate` and the command line -- with the model
running on the device-resident engine of this package.

  python -m llamatov_b200.llamatov_run model.gguf 1,415,6557 20 --generate

What is kept: `parse_gguf(path) -> (metadata, tensors, data_offset)` (bpd/llamatov_run.py:9-29),
`lt(path, do, info)` (:497-511) for F32 / F16 / Q8_0 tensors, `dq8_0` (:184-207), the torch
`rms_norm` / `apply_rope` helpers (:513-550, the reference's "soft" checks), `load_model` (:933-952)
and `generate` (:955-1177) with their argument meaning.  What differs: `load_model(..., q8_blocks=True)`
(the default) hands Q8_0 tensors to the engine as their 34-byte blocks (`fact_dispatch.Q8Weight`)
instead of dequantising to fp32 and re-quantising -- the same bits arrive on the device either way,
since a block's largest element re-quantises to +-127 -- and `generate` decodes on the GPU through
`dev_residency.GraphRunner`; there is no CPU execution path here (device="cpu" is refused).
Only the llama / qwen2 block structure with Q8_0 / F32 / F16 tensors is in scope; other tensor types
and architectures of the reference's runner are refused with an error that says so.
`write_gguf` is the inverse of the parser, for exporting synthetic models and for the tests.
"""
import struct
import sys
import time

import numpy as np
import torch

from .fact_dispatch import Q8Weight

GGUF_MAGIC = 0x46554747
_T_F32, _T_F16, _T_Q8_0 = 0, 1, 8


# --------------------------------------------------------------------------- parser

def rv(f, vt):
    """One metadata value of GGUF value type `vt` (bpd/llamatov_run.py:31-40)."""
    if vt == 4: return struct.unpack("<I", f.read(4))[0]
    if vt == 5: return struct.unpack("<i", f.read(4))[0]
    if vt == 6: return struct.unpack("<f", f.read(4))[0]
    if vt == 7: return bool(struct.unpack("<?", f.read(1))[0])
    if vt == 8:
        n = struct.unpack("<Q", f.read(8))[0]
        return f.read(n).decode()
    if vt == 9:
        at = struct.unpack("<I", f.read(4))[0]
        c = struct.unpack("<Q", f.read(8))[0]
        return [rv(f, at) for _ in range(c)]
    if vt == 10: return struct.unpack("<Q", f.read(8))[0]
    f.read({0: 1, 1: 1, 2: 2, 3: 2, 11: 8, 12: 8}.get(vt, 4))
    return None


def parse_gguf(path):
    """(metadata dict, {name: (dims, type, offset)}, data offset); dims are GGUF order, ne0 fastest."""
    with open(path, "rb") as f:
        magic = struct.unpack("<I", f.read(4))[0]
        if magic != GGUF_MAGIC:
            raise ValueError(f"Not GGUF: {magic:#x}")
        struct.unpack("<I", f.read(4))            # version
        nt = struct.unpack("<Q", f.read(8))[0]
        nkv = struct.unpack("<Q", f.read(8))[0]
        md = {}
        for _ in range(nkv):
            kl = struct.unpack("<Q", f.read(8))[0]
            k = f.read(kl).decode()
            vt = struct.unpack("<I", f.read(4))[0]
            md[k] = rv(f, vt)
        ts = {}
        for _ in range(nt):
            nl = struct.unpack("<Q", f.read(8))[0]
            n = f.read(nl).decode()
            nd = struct.unpack("<I", f.read(4))[0]
            dims = [struct.unpack("<Q", f.read(8))[0] for _ in range(nd)]
            tt = struct.unpack("<I", f.read(4))[0]
            off = struct.unpack("<Q", f.read(8))[0]
            ts[n] = (dims, tt, off)
        al = md.get("general.alignment", 32)
        do = (f.tell() + al - 1) // al * al
    return md, ts, do


def _q8_blocks(path, off, nel):
    nb = nel // 32
    raw = np.fromfile(path, dtype=np.uint8, count=nb * 34, offset=off).reshape(nb, 34)
    d = raw[:, :2].copy().view(np.float16).reshape(nb)
    q = raw[:, 2:].copy().view(np.int8)
    return q, d


def dq8_0(path, off, nel, shape):
    """Q8_0 tensor -> fp32 torch tensor in the reference's logical shape ([ne0, ne1] for matrices):
    y = f32(d) * q per 34-byte block."""
    q, d = _q8_blocks(path, off, nel)
    y = d.astype(np.float32)[:, None] * q.astype(np.float32)
    if len(shape) == 2:
        ne0, ne1 = shape
        return torch.from_numpy(y.reshape(ne1, ne0).T.copy())
    return torch.from_numpy(y.reshape(shape).copy())


def q8_0_blocks(path, off, nel, shape):
    """Q8_0 matrix [ne0 = K, ne1 = N] -> Q8Weight, the blocks as stored (no fp32 detour)."""
    if len(shape) != 2:
        raise ValueError("q8_0_blocks: matrices only")
    K, N = int(shape[0]), int(shape[1])
    q, d = _q8_blocks(path, off, nel)
    return Q8Weight(q.reshape(-1), d, N, K)


def lt(path, do, info, q8_blocks=False):
    """Load one tensor (bpd/llamatov_run.py:497-511).  Matrices come back as [ne0, ne1] = [K_in, N_out]."""
    dims, tt, ro = info
    off = do + ro
    cnt = 1
    for d in dims:
        cnt *= d
    if tt == _T_F32 or tt == _T_F16:
        a = np.fromfile(path, dtype="float32" if tt == _T_F32 else "float16", count=cnt, offset=off).astype("float32")
        t = torch.from_numpy(a.copy())
        return t.reshape(dims[::-1]).T.contiguous() if len(dims) == 2 else t.reshape(dims)
    if tt == _T_Q8_0:
        return q8_0_blocks(path, off, cnt, dims) if (q8_blocks and len(dims) == 2) else dq8_0(path, off, cnt, dims)
    raise NotImplementedError(f"GGUF tensor type {tt}: only F32, F16 and Q8_0 are in scope of this package")


# --------------------------------------------------------------------------- writer

def write_gguf(path, metadata, tensors, alignment=32):
    """Write a GGUF v3 file.  metadata: {key: int | float | str | bool}; tensors: {name: 1-D float32
    array | fp32 [K, N] matrix (stored F32) | Q8Weight (stored Q8_0)}."""
    def kv(k, v):
        b = struct.pack("<Q", len(k.encode())) + k.encode()
        if isinstance(v, bool):
            return b + struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return b + struct.pack("<II", 4, v)
        if isinstance(v, float):
            return b + struct.pack("<If", 6, v)
        s = str(v).encode()
        return b + struct.pack("<IQ", 8, len(s)) + s
    md = dict(metadata); md.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(md)) + b"".join(kv(k, v) for k, v in md.items())
    infos, blobs, off = b"", [], 0
    for name, t in tensors.items():
        if isinstance(t, Q8Weight):
            nb = t.N * (t.K // 32)
            raw = np.empty((nb, 34), np.uint8)
            raw[:, :2] = t.Wd.view(np.uint8).reshape(nb, 2)
            raw[:, 2:] = t.Wq.view(np.uint8).reshape(nb, 32)
            dims, tt, blob = [t.K, t.N], _T_Q8_0, raw.tobytes()
        else:
            a = np.asarray(t.numpy() if hasattr(t, "numpy") else t, np.float32)
            if a.ndim == 2:                       # [K, N] logical -> stored by output row
                dims, blob = [a.shape[0], a.shape[1]], np.ascontiguousarray(a.T).tobytes()
            else:
                dims, blob = [a.shape[0]], np.ascontiguousarray(a).tobytes()
            tt = _T_F32
        nm = name.encode()
        infos += struct.pack("<Q", len(nm)) + nm + struct.pack("<I", len(dims)) + b"".join(
            struct.pack("<Q", int(d)) for d in dims) + struct.pack("<IQ", tt, off)
        blobs.append((off, blob))
        off = (off + len(blob) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + infos)
        do = (f.tell() + alignment - 1) // alignment * alignment
        for o, blob in blobs:
            f.seek(do + o)
            f.write(blob)
        f.truncate(do + off)


# --------------------------------------------------------------------------- soft torch helpers

def rms_norm(x, w, eps=1e-6):
    return w * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))


def apply_rope(q, k, n_head, head_dim, theta=500000.0, positions=None):
    """NeoX half-split rotation of q and k ([B, T, heads*head_dim]) at `positions` (default 0..T-1)."""
    B, T, _ = q.shape
    q = q.view(B, T, n_head, head_dim)
    k = k.view(B, T, k.shape[-1] // head_dim, head_dim)
    half = head_dim // 2
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(T, dtype=torch.float32) if positions is None else positions.to(torch.float32)
    ang = torch.outer(t, freqs)
    c = torch.cos(ang)[None, :, None, :]; s = torch.sin(ang)[None, :, None, :]

    def rot(x):
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)
    return rot(q).reshape(B, T, -1), rot(k).reshape(B, T, -1)


# --------------------------------------------------------------------------- model, generation

def _cfg_from(md):
    arch = md.get("general.architecture", "llama")
    if arch not in ("llama", "qwen2"):
        raise NotImplementedError(f"architecture {arch!r}: only the llama / qwen2 block structure is in scope")
    return {"arch": arch,
            "n_layers": md.get(f"{arch}.block_count", 12),
            "n_head": md.get(f"{arch}.attention.head_count", 12),
            "n_head_kv": md.get(f"{arch}.attention.head_count_kv", md.get(f"{arch}.attention.head_count", 12)),
            "head_dim": md.get(f"{arch}.attention.key_length", None),
            "n_embd": md.get(f"{arch}.embedding_length", 768),
            "rope_theta": md.get(f"{arch}.rope.freq_base", 500000.0),
            "norm_eps": md.get(f"{arch}.attention.layer_norm_rms_epsilon",
                               md.get(f"{arch}.attention.layer_norm_epsilon", 1e-5))}


def load_model(path, device="cuda", q8_blocks=True):
    """(cfg, w) for `generate(..., preloaded=(cfg, w))` and the device-resident engine."""
    md, ts, do = parse_gguf(path)
    cfg = _cfg_from(md)
    w = {n: lt(path, do, info, q8_blocks=q8_blocks) for n, info in ts.items()}
    return cfg, w


def generate(path, input_ids, n_tokens=20, device="cuda", preloaded=None, verbose=True):
    """Greedy generation with the KV cache on the device: prompt prefill, one captured decode step,
    graph replays.  Returns the full id list (prompt + generated), like the reference."""
    from . import dev_residency as dr
    if device == "cpu":
        raise RuntimeError("llamatov_b200 has no CPU execution path; run the reference for device='cpu'")
    if not torch.cuda.is_available():
        raise RuntimeError("llamatov_b200.generate needs a CUDA device")
    t0 = time.time()
    cfg, w = preloaded if preloaded is not None else load_model(path)
    nl = cfg["n_layers"]
    if verbose:
        print(f"=== LlamaTov Generate ===\nModel: {path}")
        print(f"Arch: {cfg['arch']}, layers: {nl}, heads: {cfg['n_head']}/{cfg['n_head_kv']}, embd: {cfg['n_embd']}")
        print(f"Loaded {len(w)} tensors in {time.time() - t0:.1f}s")
    dr.apply_production_profile()
    dr._KV_MAX_SEQ = max(dr._KV_MAX_SEQ, len(input_ids) + n_tokens + 1)
    kv = [None] * nl
    runner = dr.GraphRunner(w, cfg, kv)
    generated = list(input_ids)
    t1 = time.time()
    logits = runner.seed(torch.tensor(generated, dtype=torch.long), torch.arange(len(generated)))
    nxt = int(logits.reshape(-1).argmax().item())
    generated.append(nxt)
    t_prefill = time.time() - t1
    if n_tokens > 1:
        runner.capture(torch.tensor([nxt]), torch.tensor([len(generated) - 1]))
        t2 = time.time()
        for _ in range(n_tokens - 1):
            nxt = runner.replay_token(nxt)
            generated.append(nxt)
        dt = time.time() - t2
        if verbose:
            print(f"DECODE tok/s: {(n_tokens - 1) / dt:.2f} ({dt / (n_tokens - 1) * 1000:.2f}ms/token), prefill={t_prefill:.2f}s")
    if verbose:
        print(f"GENERATED: {generated[len(input_ids):]}")
    return generated


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    args = [a for a in argv if not a.startswith("--")]
    p = args[0] if args else "models/model.gguf"
    ids = [int(x) for x in args[1].split(",")] if len(args) > 1 else [1, 15043]
    n = int(args[2]) if len(args) > 2 else 20
    if "--cpu" in argv:
        raise SystemExit("llamatov_b200 has no CPU execution path")
    generate(p, ids, n)


if __name__ == "__main__":
    main()
