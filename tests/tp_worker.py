"""Rank program of tests/test_gpu_tp.py::test_world2_matches_world1 (run under torch.distributed.run):
decodes the tiny model tensor-parallel over NCCL, eagerly and from a captured graph, and leaves
tokens and logits in <outdir>/rank<k>.npz."""
import datetime
import os
import sys
import traceback

import numpy as np
import torch
import torch.distributed as dist


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    out = sys.argv[1]
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    from llamatov_b200 import _lib, synth, tp
    m = synth.make_model("tiny-llama", seed=8)
    res = {}
    for comm in ("nccl", "p2p"):
        # batch 2 runs the batched operators; the chained-launch form is exercised with the peer-store all-reduce
        d = tp.TPDecoder(m["cfg"], rank=rank, world=world, batch=2, max_seq=64, model=m, comm=comm,
                         chained=(comm == "p2p"))
        d.fill_cache(6, seed=2)
        d.set_tokens([5, 600])
        toks, logits = [], []
        for _ in range(6):
            d.step()
            torch.cuda.synchronize()
            toks.append(d.tok.cpu().numpy().copy()); logits.append(d.logits.cpu().numpy().copy())
        d.capture()
        more = d.run(3)
        res[comm] = (np.stack(toks), np.concatenate(logits, axis=0), more)
    # one sequence: the chained one-sequence operators (fused norm + GEMV, peer-store all-reduce) against the
    # plain launches with NCCL
    one = {}
    for comm in ("nccl", "p2p"):
        d = tp.TPDecoder(m["cfg"], rank=rank, world=world, batch=1, max_seq=64, model=m, comm=comm, attn_split=2,
                         chained=(comm == "p2p"))
        d.fill_cache(6, seed=3)
        d.set_tokens([41])
        d.step(); d.step()
        torch.cuda.synchronize()
        lg = d.logits.cpu().numpy().copy()
        d.capture()
        one[comm] = (lg, d.run(4))
    # the exact row split of `down`: this rank's round-robin blocks of a seeded matrix and activation
    from tests.gpu_util import dev, gpu_quant, host
    E_, F_ = m["cfg"]["n_embd"], m["cfg"]["n_ffn"]
    Wq, Wd, xx = synth.gemv_case(E_, F_, T=1, seed=77)
    xq, xd = gpu_quant(xx, rows=1)
    resid = torch.from_numpy(np.random.default_rng(78).standard_normal(E_).astype(np.float32)).cuda()
    nb = F_ // 32
    tWq = torch.from_numpy(Wq.reshape(E_, F_)).cuda(); tWd = torch.from_numpy(Wd.reshape(E_, nb).view(np.int16)).cuda()
    down = {}
    for comm in ("p2p", "nccl"):
        d = tp.TPDecoder(m["cfg"], rank=rank, world=world, batch=1, max_seq=64, model=m, comm=comm, exact_split=True)
        assert d.exact
        W = tp._W(*tp.take_blocks(tWq, tWd.view(torch.float16), rank, world))
        d.xq[:F_ // world] = xq.view(nb, 32)[rank::world].reshape(-1)
        d.xd[:nb // world] = xd[rank::world]
        yout = torch.empty((1, E_), dtype=torch.float32, device="cuda")
        d._row_split(W, resid, yout, exact=True)
        torch.cuda.synchronize()
        down[comm] = yout.cpu().numpy().reshape(-1).copy()
        # ... and a few whole steps with the dealt gate|up / down shards stay finite and flag nothing
        d.fill_cache(6, seed=5); d.set_tokens([9]); d.step(); d.step()
        torch.cuda.synchronize()
        assert np.isfinite(d.logits.cpu().numpy()).all()
        d.close()
    one_same = all(np.array_equal(a, b) for a, b in zip(one["nccl"], one["p2p"]))
    status = _lib.device_status()
    same = one_same and all(np.array_equal(a, b) for a, b in zip(res["nccl"], res["p2p"]))      # two ranks: one addition, same bits
    toks, logits, more = res["p2p"]
    np.savez(os.path.join(out, f"rank{rank}.npz"), toks=toks, logits=logits, more=more, status=np.int32(len(status)),
             p2p_equals_nccl=np.int32(same), down_exact_p2p=down["p2p"], down_exact_nccl=down["nccl"])
    dist.barrier()
    torch.cuda.synchronize()


if __name__ == "__main__":
    code = 0
    try:
        main()
    except Exception:
        traceback.print_exc()
        code = 1
    sys.stdout.flush(); sys.stderr.flush()
    os._exit(code)        # no interpreter teardown: a process group being destroyed can wait on its peer
