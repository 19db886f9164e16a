"""CPU: the host side of the tensor-parallel decode -- the shard plan, the argmax combination
and, over gloo with world_size 2, the arithmetic of the two splits with the CPU checker standing
in for the device kernels (row split = partial folds + all-reduce, column split = exact rows)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llamatov_b200 import synth
from llamatov_b200.tp import ShardPlan, combine_argmax, take_cols, take_rows


@pytest.mark.parametrize("arch,world", [("llama-3-8b", 1), ("llama-3-8b", 2), ("llama-3-8b", 4), ("llama-3-8b", 8),
                                        ("tiny-llama", 2)])
def test_shard_plan_partitions_every_matrix(arch, world):
    a = synth.ARCHS[arch]
    cfg = dict(n_embd=a["n_embd"], n_head=a["n_head"], n_head_kv=a["n_head_kv"], hd=a["hd"], n_ffn=a["n_ffn"],
               vocab=a["vocab"])
    p = ShardPlan(cfg, world)
    nq, nk = a["n_head"] * a["hd"], a["n_head_kv"] * a["hd"]
    seen = np.zeros(nq + 2 * nk, int); gu = np.zeros(2 * a["n_ffn"], int)
    oc = np.zeros(nq, int); dc = np.zeros(a["n_ffn"], int); vr = np.zeros(a["vocab"], int)
    for r in range(world):
        for lo, hi in p.qkv_rows(r):
            seen[lo:hi] += 1
        for lo, hi in p.gateup_rows(r):
            gu[lo:hi] += 1
        lo, hi = p.o_cols(r); oc[lo:hi] += 1
        lo, hi = p.down_cols(r); dc[lo:hi] += 1
        lo, hi = p.vocab_rows(r); vr[lo:hi] += 1
        # a rank's query heads attend to the KV heads it caches
        q, k, _ = p.qkv_rows(r)
        rep = a["n_head"] // a["n_head_kv"]
        assert q[0] // a["hd"] // rep == (k[0] - nq) // a["hd"]
    for cover in (seen, gu, oc, dc, vr):
        assert (cover == 1).all()
    assert p.nq_l % 32 == 0 and p.F_l % 128 == 0


def test_shard_plan_refuses_what_does_not_split():
    cfg = dict(n_embd=896, n_head=14, n_head_kv=2, hd=64, n_ffn=4864, vocab=151936)
    with pytest.raises(ValueError):
        ShardPlan(cfg, 4)           # 2 KV heads over 4 ranks
    with pytest.raises(ValueError):
        ShardPlan(dict(cfg, n_head_kv=14, n_ffn=4864), 7)


def test_combine_argmax_lowest_index_wins_ties():
    vals = torch.tensor([[1.0, 5.0, 2.0], [3.0, 5.0, 2.0]])
    idxs = torch.tensor([[7, 40, 9], [107, 12, 3]], dtype=torch.int32)
    assert combine_argmax(vals, idxs).tolist() == [107, 12, 3]


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as o
    N, K = 96, 1024
    Wq, Wd, x = synth.gemv_case(N, K, seed=5)
    xq, xd = o.quant_q8(x[0])
    full = o.q8_gemv(Wq, Wd, xq, xd, N, K)
    tWq = torch.from_numpy(Wq.reshape(N, K)); tWd = torch.from_numpy(Wd.view(np.int16).reshape(N, K // 32))
    # row split: this rank's K half, partial fold, all-reduce
    k0, k1 = rank * K // world, (rank + 1) * K // world
    cq, cd = take_cols(tWq, tWd, k0, k1)
    part = o.q8_gemv(cq.numpy().reshape(-1), cd.numpy().view(np.float16).reshape(-1), xq[k0:k1], xd[k0 // 32:k1 // 32],
                     N, k1 - k0)
    t = torch.from_numpy(np.ascontiguousarray(part, np.float32).copy())
    dist.all_reduce(t)
    rel = float(np.max(np.abs(t.numpy() - full) / np.maximum(np.abs(full), 1e-6)))
    # column split: this rank's rows are exact
    r0, r1 = rank * N // world, (rank + 1) * N // world
    rq, rd = take_rows(tWq, tWd, K, [(r0, r1)])
    rows = o.q8_gemv(rq.numpy().reshape(-1), rd.numpy().view(np.float16).reshape(-1), xq, xd, r1 - r0, K)
    exact = bool(np.array_equal(np.asarray(rows, np.float32).view(np.uint32), np.asarray(full[r0:r1], np.float32).view(np.uint32)))
    # next token: local maxima with global indices, all-gather, lowest index wins
    loc = int(np.argmax(full[r0:r1]))
    pair = torch.tensor([[float(full[r0 + loc]), float(r0 + loc)]])
    gath = [torch.zeros_like(pair) for _ in range(world)]
    dist.all_gather(gath, pair)
    g = torch.stack(gath)                                # [world, 1, 2]
    tok = int(combine_argmax(g[:, :, 0], g[:, :, 1].to(torch.int32))[0])
    # every rank holds the same reduced bits
    chk = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(chk, t)
    same = all(torch.equal(chk[0], c) for c in chk)
    out.put((rank, rel, exact, tok, int(np.argmax(full)), same))
    dist.destroy_process_group()


def test_splits_over_gloo_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps: p.start()
    res = sorted(q.get(timeout=180) for _ in ps)
    for p in ps: p.join(timeout=60)
    for rank, rel, exact, tok, want, same in res:
        assert rel < 1e-5           # re-associated fold: the tolerance stated for a GEMV output
        assert exact                # rows of a column split are bit-identical
        assert tok == want and same
