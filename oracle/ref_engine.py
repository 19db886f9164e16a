"""The reference's decode step run with the REFERENCE'S OWN KERNELS on this GPU.

TEST INFRASTRUCTURE ONLY.  Chains the kernels of oracle/_ref/*.cubin (the reference's CUDA
texts compiled for sm_100a) in the reference's production op sequence
(bpd/lib/dev_residency.py:1381-1477 per layer, :1596-1623 for the logits, :1074-1110 argmax)
with the reference's launch geometry (oracle/ref_device.py).  What comes out is what the
reference engine itself computes on a B200, so the product engine can be compared with it
bit for bit at full model size, including the ops whose device functions a CPU cannot
reproduce.  Host side is plain Python + torch allocations; speed is irrelevant here."""
import numpy as np
import torch

from . import ref_device as ref


def _dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


class RefEngine:
    def __init__(self, model, max_seq=256):
        """`model`: dict from llamatov_b200.synth.make_model (Q8Weight matrices, fp32 vectors)."""
        c = model["cfg"]
        self.c = c
        self.max_seq = max_seq
        assert max_seq in (256, 512), "reference attention cubins are built for MAXT 256 and 512"
        self.eps_tag = {1e-6: "1e-06", 1e-5: "1e-05"}[float(c["norm_eps"])]
        self.theta_tag = {1e6: "1e6", 5e5: "5e5", 1e4: "1e4"}[float(c["rope_theta"])]
        E, nh, nkv, hd, F, V = c["n_embd"], c["n_head"], c["n_head_kv"], c["hd"], c["n_ffn"], c["vocab"]
        self.layers = []
        for ly in model["layers"]:
            d = {k: (_dev(ly[k].Wq), _dev(ly[k].Wd)) for k in ("qkv", "o", "gateup", "down")}
            d["attn_norm"] = _dev(ly["attn_norm"]); d["ffn_norm"] = _dev(ly["ffn_norm"])
            d["bias"] = _dev(ly["qkv_bias"]) if ly["qkv_bias"] is not None else None
            d["k"] = torch.zeros(max_seq * nkv * hd, device="cuda"); d["v"] = torch.zeros(max_seq * nkv * hd, device="cuda")
            d["len"] = torch.zeros(1, dtype=torch.int32, device="cuda")
            self.layers.append(d)
        self.emb = model["token_embd"]
        self.lm = (_dev(model["lm_head"].Wq), _dev(model["lm_head"].Wd))
        self.out_norm = _dev(model["output_norm"])
        f = dict(dtype=torch.float32, device="cuda")
        K = max(E, F)
        self.xq = torch.empty(K, dtype=torch.int8, device="cuda"); self.xd = torch.empty(K // 32, dtype=torch.int16, device="cuda")
        self.h = torch.empty(E, **f); self.qkv = torch.empty((nh + 2 * nkv) * hd, **f); self.att = torch.empty(nh * hd, **f)
        self.x = torch.empty(E, **f); self.x1 = torch.empty(E, **f); self.gu = torch.empty(2 * F, **f)
        self.logits = torch.empty(V, **f)
        self.pv = torch.empty(256, **f); self.pi = torch.empty(256, dtype=torch.int32, device="cuda")
        self.tok = torch.zeros(1, dtype=torch.int32, device="cuda")

    def _embed(self, t):
        E = self.c["n_embd"]; nb = E // 32
        q = self.emb.Wq[t * E:(t + 1) * E].astype(np.float32).reshape(nb, 32)
        d = self.emb.Wd[t * nb:(t + 1) * nb].astype(np.float32).reshape(nb, 1)
        return torch.from_numpy((q * d).reshape(E)).cuda()

    def _linear(self, W, x, K, M, out, resid=None):
        ref.quant_q8(x, self.xq, self.xd, K)
        ref.q8_gemv(W[0], W[1], self.xq, self.xd, out, M, K, resid=resid)

    def step(self, tok):
        """One token; returns (logits numpy [V], greedy token)."""
        c = self.c
        E, nh, nkv, hd, F, V = c["n_embd"], c["n_head"], c["n_head_kv"], c["hd"], c["n_ffn"], c["vocab"]
        nq, nk = nh * hd, nkv * hd
        scale = float(np.float32(hd ** -0.5))
        self.x.copy_(self._embed(int(tok)))
        for ly in self.layers:
            ref.rmsnorm(self.x, ly["attn_norm"], self.h, 1, E, self.eps_tag)
            if ly["bias"] is not None:
                self._linear(ly["qkv"], self.h, E, nq + 2 * nk, self.qkv, resid=ly["bias"])
            else:
                self._linear(ly["qkv"], self.h, E, nq + 2 * nk, self.qkv)
            ref.rope(self.qkv, ly["len"], 1, nh + nkv, hd, self.theta_tag)
            assert nk <= 128, "k_append_kv_incr handles width <= 128"
            ref.append_kv_incr(ly["k"], self.qkv[nq:], ly["v"], self.qkv[nq + nk:], ly["len"], nk)
            ref.attn_decode_masked(self.qkv, ly["k"], ly["v"], ly["len"], self.att, hd, nh, nkv, scale, self.max_seq)
            self._linear(ly["o"], self.att, nq, E, self.x1, resid=self.x)
            ref.rmsnorm(self.x1, ly["ffn_norm"], self.h, 1, E, self.eps_tag)
            self._linear(ly["gateup"], self.h, E, 2 * F, self.gu)
            ref.silu_mul_quant(self.gu, self.gu[F:], self.xq, self.xd, F)
            ref.q8_gemv(ly["down"][0], ly["down"][1], self.xq, self.xd, self.x, E, F, resid=self.x1)
        ref.rmsnorm(self.x, self.out_norm, self.h, 1, E, self.eps_tag)
        self._linear(self.lm, self.h, E, V, self.logits)
        ref.argmax2(self.logits, V, self.pv, self.pi, self.tok)
        torch.cuda.synchronize()
        return self.logits.cpu().numpy(), int(self.tok.item())
