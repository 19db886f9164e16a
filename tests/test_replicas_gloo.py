"""CPU, world_size 2 over gloo: the multi-GPU path of the 0.5B configuration is N independent
replicas; what the ranks share is the measurement (barrier, max over ranks, token agreement)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from llamatov_b200 import replicas
    from oracle import oracle as o
    from llamatov_b200 import synth
    # every rank decodes the same tiny model with the CPU checker standing in for the device path
    m = synth.make_model("tiny", seed=0)
    eng = o.OracleEngine(synth.oracle_model(m), max_seq=32)
    tok, toks = 3, []
    for _ in range(6):
        _, tok = eng.step(tok); toks.append(tok)
    replicas.barrier()
    elapsed = 10.0 * (rank + 1)                    # rank 1 is the slow one
    tput, ms = replicas.replica_throughput(6, elapsed)
    same = replicas.all_equal(toks)
    differ = replicas.all_equal(toks if rank == 0 else toks[:-1] + [toks[-1] + 1])
    out.put((rank, tput, ms, same, differ))
    dist.destroy_process_group()


def test_replica_measurement_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps: p.start()
    res = sorted(q.get(timeout=120) for _ in ps)
    for p in ps: p.join(timeout=60)
    for rank, tput, ms, same, differ in res:
        assert ms == 20.0                          # max over ranks
        assert abs(tput - 2 * 6 / 0.020) < 1e-6    # both replicas' tokens over the slowest time
        assert same is True and differ is False


def test_single_process_passthrough():
    from llamatov_b200 import replicas
    assert replicas.max_over_ranks(3.5) == 3.5
    assert replicas.replica_throughput(10, 5.0) == (2000.0, 5.0)
    assert replicas.all_equal([1, 2, 3])
