"""Multi-GPU helper for models that do not shard (the Qwen2.5-0.5B architecture has 2 KV heads
and 0.5 GB of weights): every rank runs an independent replica of the decode path; there is no
data-path collective.  Only the measurement is collective: a barrier around the timed region
and the maximum of the per-rank device times."""
import torch
import torch.distributed as dist


def barrier():
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def max_over_ranks(value, device="cpu"):
    """Maximum of a per-rank scalar (elapsed time) over all ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def replica_throughput(units_per_rank, elapsed_ms_this_rank, device="cpu"):
    """Whole-job throughput of N independent replicas: all ranks' units over the slowest
    rank's time.  Returns (units per second, max elapsed ms)."""
    world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
    ms = max_over_ranks(elapsed_ms_this_rank, device)
    return world * units_per_rank / (ms * 1e-3), ms


def all_equal(tokens, device="cpu"):
    """True when every rank holds the same token list (replicas of a deterministic decode)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return True
    t = torch.tensor(list(tokens), dtype=torch.int64, device=device)
    lo = t.clone(); hi = t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return bool(torch.equal(lo, hi))
