"""Tensor-parallel decode of a Q8_0 transformer over the GPUs of one node, one process per GPU.

The reference engine is single-GPU (bpd/lib/dev_residency.py); this module shards the same layer
sequence (dev_residency.py:1381-1477) for models too large to be worth running on one GPU:

  column split (rows of W):  q|k|v by KV-head group, gate|up, LM head (vocabulary).  A rank's rows
                             are whole reductions, so its outputs are bit-identical to one GPU's.
  row split (K of W):        o_proj and down.  Each rank folds its K slice in the frozen order and
                             the partial sums meet in an all-reduce (sum) of [batch, hidden] fp32;
                             rank order of the sum is fixed, every rank gets the same bits.  The
                             association differs from one GPU's single fold: tolerance class.
  exact row split of down:   the Q8_0 blocks of the FFN dimension are dealt round-robin over the ranks
                             (rank r: blocks b = r mod g, gate|up rows dealt to match), so a rank holds
                             whole lanes of the GEMV contract (lane = block mod 32): its partial is the
                             contract's lane chains plus the tree levels that stay inside the rank
                             (lt_q8_gemv_lanes), and the all-reduce adds the partials in the order of the
                             tree's last levels (lt_allreduce_add_tree): the bits of one GPU at the same
                             bytes on the wire.  For up to 8 sequences per step (the GEMV path).
  attention / KV cache:      head-parallel, every rank caches only its KV heads; no exchange.
  next token:                local (max, index) per sequence, all-gather, lowest index wins ties.

`ShardPlan` and the argmax combination are plain host code (tested on CPU with gloo);
`TPDecoder` drives the C-ABI kernels and `torch.distributed` (NCCL) on the GPUs.
"""
import ctypes

import numpy as np
import torch

from . import _lib


class ShardPlan:
    """Which rows / K ranges of every matrix a rank owns."""

    def __init__(self, cfg, world):
        self.world = int(world)
        self.E = cfg["n_embd"]; self.nh = cfg["n_head"]; self.nkv = cfg["n_head_kv"]
        self.hd = cfg["hd"]; self.F = cfg["n_ffn"]; self.V = cfg["vocab"]
        g = self.world
        if self.nkv % g != 0:
            raise ValueError(f"{self.nkv} KV heads do not split over {g} ranks")
        if (self.F // g) % 128 != 0 or self.F % g != 0:
            raise ValueError(f"FFN width {self.F} does not split over {g} ranks in multiples of 128")
        self.nkv_l = self.nkv // g
        self.nh_l = self.nh // g
        self.nq_l = self.nh_l * self.hd
        self.nk_l = self.nkv_l * self.hd
        self.F_l = self.F // g
        self.V_l = -(-self.V // g)            # rows per rank, the last rank may hold fewer

    def qkv_rows(self, rank):
        """Row ranges (q, k, v) of the fused [nq + 2 nk, E] matrix owned by `rank`."""
        nq, nk = self.nh * self.hd, self.nkv * self.hd
        q = (rank * self.nq_l, (rank + 1) * self.nq_l)
        k = (nq + rank * self.nk_l, nq + (rank + 1) * self.nk_l)
        v = (nq + nk + rank * self.nk_l, nq + nk + (rank + 1) * self.nk_l)
        return q, k, v

    def o_cols(self, rank):
        return rank * self.nq_l, (rank + 1) * self.nq_l

    def gateup_rows(self, rank):
        """Row ranges (gate, up) of the fused [2F, E] matrix."""
        return (rank * self.F_l, (rank + 1) * self.F_l), (self.F + rank * self.F_l, self.F + (rank + 1) * self.F_l)

    def down_cols(self, rank):
        return rank * self.F_l, (rank + 1) * self.F_l

    # ---- exact row split of down: Q8_0 blocks dealt round-robin
    def ffn_blocks(self, rank):
        """Blocks (32 FFN columns each) of rank `rank`: b = rank mod world."""
        return list(range(rank, self.F // 32, self.world))

    def gateup_rows_dealt(self, rank):
        """Row ranges of the fused [2F, E] matrix: the gate rows, then the up rows, of the rank's blocks."""
        bl = self.ffn_blocks(rank)
        return [(32 * b, 32 * b + 32) for b in bl] + [(self.F + 32 * b, self.F + 32 * b + 32) for b in bl]

    def vocab_rows(self, rank):
        return min(self.V, rank * self.V_l), min(self.V, (rank + 1) * self.V_l)


def combine_argmax(vals, idxs):
    """vals, idxs: [world, B] local maxima and their GLOBAL indices -> [B] winning indices;
    ties go to the lowest index (dev_residency.py:226-271 keeps the lowest index on ties)."""
    best = vals.max(dim=0, keepdim=True).values
    cand = torch.where(vals == best, idxs, torch.full_like(idxs, torch.iinfo(idxs.dtype).max))
    return cand.min(dim=0).values


def take_rows(Wq, Wd, K, ranges):
    """Rows of a Q8_0 matrix given as tensors Wq [N, K] int8, Wd [N, K/32]."""
    return (torch.cat([Wq[a:b] for a, b in ranges]).contiguous(), torch.cat([Wd[a:b] for a, b in ranges]).contiguous())


def take_blocks(Wq, Wd, first, step):
    """Blocks first, first + step, ... of every row."""
    N, K = Wq.shape
    return (Wq.view(N, K // 32, 32)[:, first::step, :].reshape(N, -1).contiguous(), Wd[:, first::step].contiguous())


def take_cols(Wq, Wd, k0, k1):
    """K range [k0, k1) (whole 32-blocks) of every row."""
    assert k0 % 32 == 0 and k1 % 32 == 0
    return Wq[:, k0:k1].contiguous(), Wd[:, k0 // 32:k1 // 32].contiguous()


def random_q8(N, K, gen, device, sigma=0.02):
    """Seeded random-init weights N(0, sigma) quantised to Q8_0 on the device with the engine's weight rule
    (bpd/lib/fact_dispatch.py:255-282: per 32-block d = fp16(amax/127), 1.0 if 0; q = clip(round(w / f32(d))))."""
    Wq = torch.empty((N, K), dtype=torch.int8, device=device)
    Wd = torch.empty((N, K // 32), dtype=torch.float16, device=device)
    step = max(1, (1 << 26) // K)
    for r0 in range(0, N, step):
        r1 = min(N, r0 + step)
        w = torch.randn((r1 - r0, K // 32, 32), generator=gen, dtype=torch.float32, device=device) * sigma
        d = (w.abs().amax(dim=-1) / 127.0).to(torch.float16)
        d = torch.where(d == 0, torch.ones_like(d), d)
        Wd[r0:r1] = d
        Wq[r0:r1] = torch.clamp(torch.round(w / d.float().unsqueeze(-1)), -127, 127).to(torch.int8).view(r1 - r0, K)
    return Wq, Wd


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _CommStruct(ctypes.Structure):
    """struct lt_comm of include/llamatov_b200.h."""
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("max_n", ctypes.c_int), ("max_ctas", ctypes.c_int),
                ("stage", ctypes.c_void_p * 8), ("local_stage", ctypes.c_void_p), ("ctr", ctypes.c_void_p)]


class P2PComm:
    """The one-shot all-reduce over peer memory (lt_allreduce_add): staging buffers mapped through CUDA
    IPC, handles exchanged over the process group that already exists."""

    def __init__(self, rank, world, max_n, group=None):
        import torch.distributed as dist
        self.c = _CommStruct()
        handles = (ctypes.c_ubyte * 64)()
        _lib.call("lt_comm_alloc", world, max_n, ctypes.byref(self.c), handles)
        mine = bytes(handles)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=group)
        allh = (ctypes.c_ubyte * (64 * world)).from_buffer_copy(b"".join(gathered))
        _lib.call("lt_comm_connect", ctypes.byref(self.c), rank, allh)
        torch.cuda.synchronize()
        dist.barrier(group=group)          # every rank's buffers exist and are zero before the first store

    def allreduce_add(self, part, resid, out, n):
        _lib.call("lt_allreduce_add", ctypes.byref(self.c), part.data_ptr(), None if resid is None else resid.data_ptr(),
                  out.data_ptr(), n, _stream())

    def allreduce_add_tree(self, part, resid, out, n):
        """The same with the partials summed in the lane tree's order (exact row split, lt_q8_gemv_lanes)."""
        _lib.call("lt_allreduce_add_tree", ctypes.byref(self.c), part.data_ptr(), None if resid is None else resid.data_ptr(),
                  out.data_ptr(), n, _stream())

    def free(self, group=None):
        """No kernel of any rank may still be storing into the buffers: device sync, host barrier, then free."""
        import torch.distributed as dist
        if self.c.local_stage:
            torch.cuda.synchronize()
            if dist.is_initialized() and self.c.world > 1:
                dist.barrier(group=group)
            _lib.call("lt_comm_free", ctypes.byref(self.c))


class _W:
    """One resident Q8_0 matrix shard."""
    __slots__ = ("q", "d", "N", "K")

    def __init__(self, Wq, Wd):
        self.q = Wq.contiguous(); self.d = Wd.contiguous().view(torch.int16)
        self.N, self.K = int(Wq.shape[0]), int(Wq.shape[1])


class TPDecoder:
    """Batched greedy decode of a random-init Q8_0 model, sharded over `world` ranks.

    Every rank builds the full matrices from the same seed and keeps its shard, so the
    model is the same at every world size (token streams can be compared against world 1).
    """

    def __init__(self, cfg, rank=0, world=1, batch=1, max_seq=4352, seed=0, group=None, device=None, model=None,
                 comm="nccl", attn_split=0, chained=False, fused_allreduce=True, exact_split=False):
        self.chained = bool(chained)
        self.fused_rope = True            # split order: rope + append inside the range kernel
        self.fused_allreduce = bool(fused_allreduce)     # comm="p2p", one sequence: all-reduce inside the GEMV
        self.cfg = dict(cfg); self.rank = rank; self.world = world; self.B = int(batch)
        self.max_seq = int(max_seq); self.group = group
        self.dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.plan = p = ShardPlan(cfg, world)
        E, L = p.E, cfg["n_layers"]
        # exact row split of down (blocks dealt round-robin): world a power of two up to 8, GEMV path
        self.exact = bool(exact_split) and world in (2, 4, 8) and self.B <= 8 and (p.F // 32) % world == 0
        f32 = dict(dtype=torch.float32, device=self.dev)
        if model is not None:
            src = self._from_model(model)
        else:
            src = self._random(seed)
        self.layers = []
        for _ in range(L):
            an = next(src)
            Wq, Wd = next(src)
            qkv = _W(*take_rows(Wq, Wd, E, self.plan.qkv_rows(rank)))
            Wq, Wd = next(src)
            o = _W(*take_cols(Wq, Wd, *p.o_cols(rank)))
            fn = next(src)
            Wq, Wd = next(src)
            gu = _W(*take_rows(Wq, Wd, E, p.gateup_rows_dealt(rank) if self.exact else p.gateup_rows(rank)))
            Wq, Wd = next(src)
            down = _W(*(take_blocks(Wq, Wd, rank, world) if self.exact else take_cols(Wq, Wd, *p.down_cols(rank))))
            del Wq, Wd
            self.layers.append(dict(attn_norm=an, qkv=qkv, o=o, ffn_norm=fn, gateup=gu, down=down))
        self.out_norm = next(src)
        Wq, Wd = next(src)
        self.embd = _W(Wq, Wd)                                   # replicated (gather of B rows per step)
        lq, ld = next(src)
        v0, v1 = p.vocab_rows(rank)
        self.lm = _W(lq[v0:v1], ld[v0:v1]); self.v0 = v0
        del lq, ld, src
        # caches: [B, max_seq, nkv_l * hd] per layer, lengths per sequence
        wl = p.nk_l
        self.kc = [torch.zeros(self.B * self.max_seq * wl, **f32) for _ in range(L)]
        self.vc = [torch.zeros(self.B * self.max_seq * wl, **f32) for _ in range(L)]
        self.lens = [torch.zeros(self.B, dtype=torch.int32, device=self.dev) for _ in range(L)]
        # fixed workspaces (the step is graph-capturable)
        B = self.B
        kmax = max(E, p.nq_l, p.F_l)
        self.tok = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self.x = torch.empty((B, E), **f32); self.x1 = torch.empty((B, E), **f32)
        self.h = torch.empty((B, E), **f32); self.part = torch.empty((B, E), **f32)
        self.gpart = torch.empty((world, B, E), **f32) if (self.exact and comm == "nccl") else None
        self.qkv = torch.empty((B, p.nq_l + 2 * p.nk_l), **f32)
        self.att = torch.empty((B, p.nq_l), **f32)
        self.gu = torch.empty((B, 2 * p.F_l), **f32)
        self.xq = torch.empty(B * kmax, dtype=torch.int8, device=self.dev)
        self.xd = torch.empty(B * (kmax // 32), dtype=torch.int16, device=self.dev)
        self.logits = torch.empty((B, max(1, v1 - v0)), **f32)
        # attn_split = S > 0: the reference's declared split order with S ranges (fixed for the captured graph);
        # 0: the one-pass frozen order
        self.attn_split = int(attn_split)
        n = _lib.lib().lt_attn_decode_batch_scratch_floats(p.nh_l, self.max_seq, B)
        if self.attn_split > 0:
            n = max(n, _lib.lib().lt_attn_decode_split_scratch_floats(p.nh_l, p.hd, self.attn_split, B))
        self.scratch = torch.empty(n, **f32)
        self.amax_part = torch.empty(_lib.lib().lt_argmax_rows_scratch_bytes(B) // 4, **f32)
        self.loc_idx = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self.ticket = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self.pair = torch.zeros((B, 2), **f32)                   # (value, global index as float bits) per sequence
        self.gath = torch.zeros((world, B, 2), **f32)
        self.graph = None
        self.history = []
        self.allreduce_calls = 0
        # comm: "nccl" = torch.distributed all-reduce + a separate residual add; "p2p" = the one-shot
        # peer-store all-reduce with the residual add folded in
        self.comm = None
        if world > 1 and comm == "p2p":
            self.comm = P2PComm(rank, world, B * E, group)
        elif comm not in ("nccl", "p2p"):
            raise ValueError(f"comm={comm!r}")

    # ------------------------------------------------------------------ weights
    def _random(self, seed):
        """The full matrices in layer order, drawn on the device from one seeded generator."""
        p, cfg = self.plan, self.cfg
        E = p.E
        gen = torch.Generator(device=self.dev); gen.manual_seed(seed)
        f32 = dict(dtype=torch.float32, device=self.dev)
        for _ in range(cfg["n_layers"]):
            yield 1.0 + 0.1 * torch.randn(E, generator=gen, **f32)
            yield random_q8(p.nh * p.hd + 2 * p.nkv * p.hd, E, gen, self.dev)
            yield random_q8(E, p.nh * p.hd, gen, self.dev)
            yield 1.0 + 0.1 * torch.randn(E, generator=gen, **f32)
            yield random_q8(2 * p.F, E, gen, self.dev)
            yield random_q8(E, p.F, gen, self.dev)
        yield 1.0 + 0.1 * torch.randn(E, generator=gen, **f32)
        emb = random_q8(p.V, E, gen, self.dev)
        yield emb
        yield emb if cfg.get("tied", False) else random_q8(p.V, E, gen, self.dev)

    def _from_model(self, model):
        """The same sequence from a host model (llamatov_b200.synth.make_model); no q/k/v bias."""
        def q8(w):
            Wq = torch.from_numpy(np.ascontiguousarray(w.Wq).reshape(w.N, w.K)).to(self.dev)
            Wd = torch.from_numpy(np.ascontiguousarray(w.Wd).view(np.int16).reshape(w.N, w.K // 32)).to(self.dev)
            return Wq, Wd.view(torch.float16)

        def vec(a):
            return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(self.dev)
        for ly in model["layers"]:
            if ly["qkv_bias"] is not None:
                raise ValueError("TPDecoder: q/k/v bias is not supported (Llama-type models)")
            yield vec(ly["attn_norm"]); yield q8(ly["qkv"]); yield q8(ly["o"])
            yield vec(ly["ffn_norm"]); yield q8(ly["gateup"]); yield q8(ly["down"])
        yield vec(model["output_norm"])
        yield q8(model["token_embd"])
        yield q8(model["lm_head"])

    # ------------------------------------------------------------------ state
    def fill_cache(self, ctx, seed=1):
        """KV caches pre-filled to `ctx` positions with N(0,1) * 0.3; the values of a (layer, sequence) do
        not depend on the world size or the batch size."""
        p = self.plan
        gen = torch.Generator(device=self.dev)
        wl, wfull = p.nk_l, p.nkv * p.hd
        c0 = self.rank * wl
        for il in range(len(self.layers)):
            kc = self.kc[il].view(self.B, self.max_seq, wl); vc = self.vc[il].view(self.B, self.max_seq, wl)
            for b in range(self.B):
                gen.manual_seed(seed * 1000003 + il * 4099 + b)        # one draw per (layer, sequence)
                full = torch.randn((2, ctx, wfull), generator=gen, dtype=torch.float32, device=self.dev) * 0.3
                kc[b, :ctx] = full[0, :, c0:c0 + wl]
                vc[b, :ctx] = full[1, :, c0:c0 + wl]
            self.lens[il].fill_(ctx)

    def set_tokens(self, toks):
        self.tok.copy_(torch.as_tensor(toks, dtype=torch.int32).to(self.dev))

    # ------------------------------------------------------------------ one step
    def _gemm(self, W, y, T, resid=None, resid_ld=0):
        if T == 1 and resid_ld in (0, W.N):
            _lib.call("lt_q8_gemv", W.q.data_ptr(), W.d.data_ptr(), self.xq.data_ptr(), self.xd.data_ptr(),
                      None if resid is None else resid.data_ptr(), y.data_ptr(), W.N, W.K, 1, _stream())
        else:
            _lib.call("lt_q8_gemm_tc", W.q.data_ptr(), W.d.data_ptr(), self.xq.data_ptr(), self.xd.data_ptr(),
                      None if resid is None else resid.data_ptr(), resid_ld, y.data_ptr(), W.N, W.K, T, 0, _stream())

    def _norm_quant(self, x, w):
        """RMSNorm + activation quantiser of the B rows.  One launch when there are rows enough to fill the
        GPU (a row is one CTA); for a few rows the quantiser spreads better as its own launch."""
        B, E = self.B, self.plan.E
        eps = float(self.cfg["norm_eps"])
        if B >= 16:
            _lib.call("lt_rmsnorm_quant", x.data_ptr(), w.data_ptr(), None, self.xq.data_ptr(), self.xd.data_ptr(),
                      B, E, eps, _stream())
        else:
            _lib.call("lt_rmsnorm", x.data_ptr(), w.data_ptr(), self.h.data_ptr(), B, E, eps, _stream())
            _lib.call("lt_quant_q8", self.h.data_ptr(), self.xq.data_ptr(), self.xd.data_ptr(), E, B, _stream())

    def _norm_gemm(self, x, w, W, y):
        """y = W . quant(rmsnorm(x) * w) for the B rows; one launch for a single sequence (the projection's
        CTAs normalise and quantise the row themselves), else the quantiser launch(es) and the GEMM."""
        if self.B == 1:
            _lib.call("lt_rmsnorm_q8_gemv", W.q.data_ptr(), W.d.data_ptr(), x.data_ptr(), w.data_ptr(),
                      float(self.cfg["norm_eps"]), None, y.data_ptr(), W.N, W.K, _stream())
        else:
            self._norm_quant(x, w)
            self._gemm(W, y, self.B)

    def _allreduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)
            self.allreduce_calls += 1

    def _row_split(self, W, resid, out, exact=False):
        """out = resid + sum over ranks of (W_rank . x_rank): one fold on one rank (the residual rides
        in the GEMV store, the reference's add-residual form); an all-reduce of partials otherwise.
        exact: W holds this rank's round-robin blocks; lane partials, summed in the lane tree's order."""
        B, E = self.B, self.plan.E
        if self.world == 1:
            self._gemm(W, out, B, resid, E)
        elif exact:
            _lib.call("lt_q8_gemv_lanes", W.q.data_ptr(), W.d.data_ptr(), self.xq.data_ptr(), self.xd.data_ptr(),
                      self.part.data_ptr(), W.N, W.K, B, self.world, _stream())
            if self.comm is not None:
                self.comm.allreduce_add_tree(self.part, resid, out, B * E)
            else:
                torch.distributed.all_gather_into_tensor(self.gpart.view(-1), self.part.view(-1), group=self.group)
                s = self.world // 2
                while s >= 1:       # p[t] + p[t + s], s = world/2 .. 1 (IEEE fp32 adds)
                    self.gpart[:s] = self.gpart[:s] + self.gpart[s:2 * s]
                    s //= 2
                _lib.call("lt_add", resid.data_ptr(), self.gpart[0].data_ptr(), out.data_ptr(), B * E, _stream())
            self.allreduce_calls += 1
        elif self.comm is not None and B == 1 and self.fused_allreduce:
            # one sequence: the partial rows are exchanged by the GEMV itself
            _lib.call("lt_q8_gemv_allreduce", ctypes.byref(self.comm.c), W.q.data_ptr(), W.d.data_ptr(),
                      self.xq.data_ptr(), self.xd.data_ptr(), resid.data_ptr(), out.data_ptr(), W.N, W.K, _stream())
            self.allreduce_calls += 1
        elif self.comm is not None:
            self._gemm(W, self.part, B)
            self.comm.allreduce_add(self.part, resid, out, B * E)
            self.allreduce_calls += 1
        else:
            self._gemm(W, self.part, B)
            self._allreduce(self.part)
            _lib.call("lt_add", resid.data_ptr(), self.part.data_ptr(), out.data_ptr(), B * E, _stream())

    def step(self):
        """One greedy decode step for the B sequences: tokens in self.tok -> next tokens in self.tok.
        With chained=True the one-sequence operators are enqueued as chained launches (lt_set_chained_launch)."""
        prev = _lib.lib().lt_set_chained_launch(1 if self.chained else 0)
        try:
            self._step()
        finally:
            _lib.lib().lt_set_chained_launch(prev)

    def _step(self):
        p, cfg, B = self.plan, self.cfg, self.B
        E, hd = p.E, p.hd
        eps, theta = float(cfg["norm_eps"]), float(cfg["rope_theta"])
        scale = float(np.float32(hd ** -0.5))
        st = _stream
        qld = p.nq_l + 2 * p.nk_l
        _lib.call("lt_embed_q8_rows", self.embd.q.data_ptr(), self.embd.d.data_ptr(), self.tok.data_ptr(),
                  self.x.data_ptr(), E, p.V, B, st())
        for il, ly in enumerate(self.layers):
            self._norm_gemm(self.x, ly["attn_norm"], ly["qkv"], self.qkv)
            lens = self.lens[il]
            if self.attn_split > 0 and self.fused_rope:
                # rope, append and the attention ranges in one launch; the quantised output from the combine
                _lib.call("lt_rope_attn_decode_split", self.qkv.data_ptr(), qld, self.kc[il].data_ptr(),
                          self.vc[il].data_ptr(), lens.data_ptr(), self.att.data_ptr(), p.nq_l, self.scratch.data_ptr(),
                          hd, p.nh_l, p.nkv_l, theta, scale, self.max_seq, B, self.attn_split, self.ticket.data_ptr(),
                          self.xq.data_ptr(), self.xd.data_ptr(), st())
                self._row_split(ly["o"], self.x, self.x1)
                self._norm_gemm(self.x1, ly["ffn_norm"], ly["gateup"], self.gu)
                _lib.call("lt_silu_mul_quant_rows", self.gu.data_ptr(), self.gu.data_ptr() + p.F_l * 4, 2 * p.F_l,
                          self.xq.data_ptr(), self.xd.data_ptr(), p.F_l, B, st())
                self._row_split(ly["down"], self.x1, self.x, exact=self.exact)
                continue
            _lib.call("lt_rope_append_batch", self.qkv.data_ptr(), qld, p.nh_l, p.nkv_l, hd, theta,
                      self.kc[il].data_ptr(), self.vc[il].data_ptr(), lens.data_ptr(), self.max_seq, B,
                      self.ticket.data_ptr(), st())
            # attention output and its Q8_0 quantisation (the o_proj input) from one launch chain
            if self.attn_split > 0:
                _lib.call("lt_attn_decode_split", self.qkv.data_ptr(), qld, self.kc[il].data_ptr(),
                          self.vc[il].data_ptr(), lens.data_ptr(), self.att.data_ptr(), p.nq_l, self.scratch.data_ptr(),
                          hd, p.nh_l, p.nkv_l, scale, self.max_seq, B, self.attn_split, self.xq.data_ptr(),
                          self.xd.data_ptr(), st())
            else:
                _lib.call("lt_attn_decode_batch", self.qkv.data_ptr(), qld, self.kc[il].data_ptr(),
                          self.vc[il].data_ptr(), lens.data_ptr(), self.att.data_ptr(), p.nq_l, self.scratch.data_ptr(),
                          hd, p.nh_l, p.nkv_l, scale, self.max_seq, B, self.xq.data_ptr(), self.xd.data_ptr(), st())
            self._row_split(ly["o"], self.x, self.x1)
            self._norm_gemm(self.x1, ly["ffn_norm"], ly["gateup"], self.gu)
            _lib.call("lt_silu_mul_quant_rows", self.gu.data_ptr(), self.gu.data_ptr() + p.F_l * 4, 2 * p.F_l,
                      self.xq.data_ptr(), self.xd.data_ptr(), p.F_l, B, st())
            self._row_split(ly["down"], self.x1, self.x, exact=self.exact)
        self._norm_gemm(self.x, self.out_norm, self.lm, self.logits)
        nv = self.lm.N
        ld = int(self.logits.stride(0))
        if self.world == 1 or self.comm is not None:
            # the rows' maxima, the exchange of (maximum, global index) over the ranks and the lowest-index
            # combine in two launches; the token lands in self.tok on every rank
            _lib.call("lt_argmax_rows", None if self.comm is None else ctypes.byref(self.comm.c), self.logits.data_ptr(), ld, nv,
                      self.v0, B, self.amax_part.data_ptr(), self.tok.data_ptr(), st())
        else:
            _lib.call("lt_argmax_rows", None, self.logits.data_ptr(), ld, nv, 0, B, self.amax_part.data_ptr(),
                      self.loc_idx.data_ptr(), st())
            idx = self.loc_idx.long()
            self.pair[:, 0] = self.logits.gather(1, idx.view(B, 1)).view(B)
            self.pair[:, 1] = (idx + self.v0).to(torch.int32).view(torch.float32)      # index carried as bits
            torch.distributed.all_gather_into_tensor(self.gath.view(-1), self.pair.view(-1), group=self.group)
            vals = self.gath[:, :, 0]
            idxs = self.gath[:, :, 1].contiguous().view(torch.int32)
            self.tok.copy_(combine_argmax(vals, idxs))

    # ------------------------------------------------------------------ graph
    def capture(self):
        """Record step() (kernels and collectives) into a CUDA graph.  One warm-up step runs first (it is a
        real decode step: lengths advance, tokens move on); the recorded pass itself executes nothing."""
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()                       # warm-up: NCCL channels, function attributes
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = _lib.launch_count()
        with torch.cuda.graph(g, stream=side):
            self.step()
        self.launches_per_step = _lib.launch_count() - n0
        self.graph = g
        return g

    def run(self, steps):
        """`steps` decode steps (graph replays when captured); returns the tokens [steps, B] on the host.
        Raises if a device wait gave up or a bound was hit during the run (the tokens would be garbage)."""
        out = []
        for _ in range(steps):
            if self.graph is not None:
                self.graph.replay()
            else:
                self.step()
            out.append(self.tok.clone())
        torch.cuda.synchronize()
        st = _lib.device_status()
        if st:
            raise RuntimeError(f"TPDecoder.run: device status {sorted(st)} (rank {self.rank})")
        return torch.stack(out).cpu().numpy()

    def close(self):
        """Release what lives outside torch's allocator (the peer-mapped staging buffers); every rank calls it."""
        self.graph = None
        if self.comm is not None:
            self.comm.free(self.group)
            self.comm = None
