"""Host-side logic of the multi-GPU path, run as world_size-2 gloo ranks on the CPU.

The box-level split is a contiguous split along N with no data-path collective. These tests check the split
itself, that per-image independence really holds for every operator family (the oracle applied to the shards
equals the oracle applied to the whole batch, bit for bit, including the backward outputs), and the
bookkeeping reductions the benchmark uses (slowest rank's time, summed units).
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _batch(seed, n):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, 3, 9, 11)).astype(np.float32)
    grid = rng.uniform(-1.1, 1.1, (n, 6, 7, 2)).astype(np.float32)
    go = rng.standard_normal((n, 3, 6, 7)).astype(np.float32)
    return x, grid, go


def _run_ops(o, x, grid, go):
    """A forward and a backward of each family on one (sub-)batch."""
    out = {}
    out["nearest"] = o.nearest2d_fwd(x, (18, 22))
    out["bilinear"] = o.bilinear2d_fwd(x, (13, 17), False)
    out["aa"] = o.bicubic_aa_fwd(x, (4, 5), False)
    out["aa_bwd"] = o.bicubic_aa_bwd(out["aa"], x.shape[2:], False)
    out["gs"] = o.grid_sampler2d_fwd(x, grid, 0, 0, False)
    gi, gg = o.grid_sampler2d_bwd(go, x, grid, 0, 0, False)
    out["gs_gi"], out["gs_gg"] = gi, gg
    return out


def _worker(rank, world, port, n, q):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    import oracle as o
    entry.load_package()
    from opscv_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, grid, go = _batch(7, n)
        b, e = sharding.shard_range(n, world, rank)
        mine = _run_ops(o, x[b:e], grid[b:e], go[b:e])
        # gather the shards on every rank (test bookkeeping only: the product path has no collective)
        gathered = [None] * world
        dist.all_gather_object(gathered, {k: np.asarray(v) for k, v in mine.items()})
        ms = sharding.max_over_ranks([10.0 + rank, 5.0 - rank], dist)
        units = sharding.sum_over_ranks([e - b], dist)
        thr = sharding.box_throughput(float(e - b), 10.0 + rank, dist)
        if rank == 0:
            q.put((gathered, ms, units, thr))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [4, 5])
def test_two_rank_split_matches_whole_batch(oracle, n):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    gathered, ms, units, thr = q.get()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    whole = _run_ops(oracle, *_batch(7, n))
    for key, ref in whole.items():
        got = np.concatenate([g[key] for g in gathered], axis=0)
        assert got.shape == np.asarray(ref).shape, key
        assert np.array_equal(got, np.asarray(ref)), key  # per-image independence: bit-identical
    assert ms == [11.0, 5.0]
    assert units == [float(n)]
    assert thr == pytest.approx(n / 11.0e-3)


def test_shard_range_covers_batch():
    entry = __import__("__graft_entry__")
    entry.load_package()
    from opscv_b200 import sharding
    for n in (0, 1, 7, 8, 512, 513):
        for world in (1, 2, 4, 8):
            edges = [sharding.shard_range(n, world, r) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            for (b0, e0), (b1, _) in zip(edges, edges[1:]):
                assert e0 == b1 and e0 >= b0
            sizes = [e - b for b, e in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)
    t = torch.arange(10).reshape(5, 2)
    assert torch.equal(torch.cat([sharding.shard_batch(t, 2, r) for r in range(2)]), t)


def _liveness_worker(rank, world, port, q):
    """Rank 1 leaves after step 1 (between steps, nothing in flight); rank 0 must notice at step 2."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from opscv_b200 import sharding
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=20))
    guard = sharding.StepGuard(store, world, rank, timeout_s=1.5)
    done = []
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                q.put((rank, "left", done))
                return
            guard.check_in(step)
            done.append(step)
        q.put((rank, "finished", done))
    except sharding.RankLost as exc:
        q.put((rank, "lost: " + str(exc), done))
        if rank == 0:
            import time
            time.sleep(0.5)  # keep the store alive until the message is out


def test_a_rank_that_leaves_between_steps_is_reported():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_liveness_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, what, done = q.get(timeout=60)
        results[rank] = (what, done)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert results[1] == ("left", [0, 1])
    what, done = results[0]
    assert done == [0, 1] and what.startswith("lost: step 2") and "[1]" in what  # reported, not waited for
