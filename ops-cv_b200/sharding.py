"""Batch sharding of the resampling operators across the GPUs of one box.

Every operator of this library is independent per image n (grid sampler: grid[n] with input[n]; the backward
passes write grad_input[n] and grad_grid[n] only), so the box-level split is a contiguous split along N with
rank-local tensors and no data-path collective. What ranks exchange is only bookkeeping: a barrier around the
timed region, the maximum of the device times and the sum of the units processed. These helpers are that
bookkeeping; they work on any torch.distributed backend (nccl on the GPUs, gloo in the CPU tests).
"""
import datetime

import torch


def shard_range(n, world, rank):
    """[begin, end) of the images rank `rank` of `world` owns: contiguous, sizes differ by at most one, the first
    n % world ranks take the extra image."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(int(n), world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch(t, world, rank):
    """The rank's slice of a batch-major tensor (a view: dimension 0 is N for NCHW, NHWC and grids alike)."""
    b, e = shard_range(t.shape[0], world, rank)
    return t[b:e]


def max_over_ranks(values, dist=None, device=None):
    """Element-wise maximum over ranks of a list of floats (device times): the box time of a step is that of its
    slowest rank."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(v) for v in values]
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def sum_over_ranks(values, dist=None, device=None):
    """Element-wise sum over ranks (bytes or pixels processed)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(v) for v in values]
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.tolist()


def box_throughput(units_per_rank, ms_per_rank, dist=None, device=None):
    """Whole-box throughput in units per second: all ranks' units divided by the slowest rank's time."""
    total = sum_over_ranks([units_per_rank], dist, device)[0]
    worst = max_over_ranks([ms_per_rank], dist, device)[0]
    return total / (worst * 1e-3)


class RankLost(RuntimeError):
    """A rank did not check in for a step within the time limit (it exited, hung or never joined)."""


class StepGuard:
    """Host-side liveness check between steps of a batch-sharded job. There is no data-path collective whose failure
    would reveal a lost rank, so every rank checks in on the process group's store before a step
    (`guard.check_in(step)`) and waits, with a time limit, for the check-ins of all others; a rank that exited or
    hung between steps makes the others raise RankLost instead of entering the step (and instead of waiting in the
    next barrier for ever). Ranks must leave only between steps, with none of their kernels in flight; this class is
    pure host logic and touches no GPU."""

    def __init__(self, store, world, rank, timeout_s=5.0, tag="opscv"):
        self.store, self.world, self.rank = store, world, rank
        self.timeout = datetime.timedelta(seconds=timeout_s)
        self.tag = tag

    def check_in(self, step):
        self.store.set(f"{self.tag}/step{step}/rank{self.rank}", "1")
        keys = [f"{self.tag}/step{step}/rank{r}" for r in range(self.world) if r != self.rank]
        missing = []
        for key in keys:  # one key at a time, so that the message can name the rank
            try:
                self.store.wait([key], self.timeout)
            except Exception:  # noqa: BLE001 - the store raises a backend-specific timeout error
                missing.append(int(key.rsplit("rank", 1)[1]))
        if missing:
            raise RankLost(f"step {step}: no check-in from rank(s) {missing} within {self.timeout.total_seconds():.1f} s")
