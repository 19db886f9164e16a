"""Rank program of tests/test_gpu_tp.py::test_exchange_kernels_world{2,4} (run under torch.distributed.run): the
peer-store exchanges called directly.  lt_allreduce_add on a short vector (one-shot form) and on a long one (the
two-stage form from four ranks on) against the same sum formed from gathered partials in rank order, and
lt_argmax_rows over vocabulary slices against numpy on the whole matrix.  Results in <outdir>/comm<k>.npz."""
import datetime
import os
import sys
import traceback

import numpy as np
import torch
import torch.distributed as dist


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    outdir = sys.argv[1]
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    import ctypes
    from llamatov_b200 import _lib, tp
    nmax = 1 << 17
    comm = tp.P2PComm(rank, world, nmax)
    ok_sum = True
    for rep, n in enumerate((4096, 1 << 16, 1 << 17, 40960, 4096)):
        g = torch.Generator(device="cuda"); g.manual_seed(100 * rep + rank)
        part = torch.randn(n, generator=g, device="cuda") * (10.0 ** (rank - 1))
        g2 = torch.Generator(device="cuda"); g2.manual_seed(7 + rep)
        resid = torch.randn(n, generator=g2, device="cuda")
        out = torch.empty(n, device="cuda")
        comm.allreduce_add(part, resid, out, n)
        parts = [torch.empty(n, device="cuda") for _ in range(world)]
        dist.all_gather(parts, part)
        acc = parts[0].clone()
        for r in range(1, world):
            acc = acc + parts[r]                # fp32 additions in rank order, one rounding each
        want = resid + acc
        torch.cuda.synchronize()
        ok_sum = ok_sum and bool(torch.equal(out.view(torch.int32), want.view(torch.int32)))
    # greedy tokens over vocabulary slices
    ok_tok = True
    for B, V in ((1, 1000 * world), (32, 16032 * world), (5, 257 * world)):
        rng = np.random.default_rng(B)
        full = rng.standard_normal((B, V)).astype(np.float32)
        nv = V // world
        full[0, [nv - 1, nv, V - 1]] = 11.0                 # a tie across ranks: lowest index wins
        if B > 2:
            full[2, 3 * nv // 2 % V] = 12.0
        mine = torch.from_numpy(np.ascontiguousarray(full[:, rank * nv:(rank + 1) * nv])).cuda()
        partb = torch.empty(_lib.lib().lt_argmax_rows_scratch_bytes(B), dtype=torch.uint8, device="cuda")
        tok = torch.full((B,), -1, dtype=torch.int32, device="cuda")
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.call("lt_argmax_rows", ctypes.byref(comm.c), mine.data_ptr(), nv, nv, rank * nv, B, partb.data_ptr(), tok.data_ptr(), st)
        torch.cuda.synchronize()
        ok_tok = ok_tok and np.array_equal(tok.cpu().numpy(), np.argmax(full, axis=1).astype(np.int32))
        # ... and an all-reduce after it keeps the exchange numbers in step
        n = 4096
        part = torch.full((n,), float(rank + 1), device="cuda"); out = torch.empty(n, device="cuda")
        comm.allreduce_add(part, None, out, n)
        torch.cuda.synchronize()
        ok_sum = ok_sum and bool((out == float(world * (world + 1) // 2)).all())
    status = _lib.device_status()
    np.savez(os.path.join(outdir, f"comm{rank}.npz"), ok_sum=np.int32(ok_sum), ok_tok=np.int32(ok_tok), status=np.int32(len(status)))
    comm.free()
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
