"""World-size-2 CPU test (gloo) of the replica sharding logic: disjoint balanced seed shards,
super-batch cutting, count all-gather and the max-time / summed-units reduction."""
import importlib.util
import os
import socket
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_shard():
    # the package __init__ needs the native libraries; shard.py itself is pure host logic
    spec = importlib.util.spec_from_file_location("gsb_shard", os.path.join(ROOT, "gsampler_b200", "shard.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist

    shard = _load_shard()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    seeds = torch.arange(1001, dtype=torch.int64)
    mine = shard.shard_seeds(seeds, rank, world)
    batches = shard.super_batches(mine, batch=64, per_step=4)
    n = sum(int(s.numel()) for s, _ in batches)
    counts = shard.gather_counts(n)
    t, total = shard.reduce_timing(10.0 * (rank + 1), n)
    q.put((rank, mine.tolist(), [p.tolist() for _, p in batches], counts, t, total))
    dist.destroy_process_group()


def test_two_rank_sharding():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, s0, p0, c0, t0, n0), (r1, s1, p1, c1, t1, n1) = res
    assert sorted(s0 + s1) == list(range(1001)) and not set(s0) & set(s1)
    assert abs(len(s0) - len(s1)) <= 1
    assert c0 == c1 == [len(s0), len(s1)]
    assert t0 == t1 == 20.0 and n0 == n1 == 1001
    for ptrs, n in ((p0, len(s0)), (p1, len(s1))):
        assert all(len(p) == 5 for p in ptrs)
        assert sum(p[-1] for p in ptrs) == n
        assert ptrs[0] == [0, 64, 128, 192, 256]
        assert ptrs[-1][-1] == n - 256 * (len(ptrs) - 1)


def test_bounds_edge_cases():
    shard = _load_shard()
    assert [shard.shard_bounds(5, r, 8) for r in range(8)] == [(0, 1), (1, 2), (2, 3), (3, 4), (4, 5),
                                                               (5, 5), (5, 5), (5, 5)]
    assert shard.shard_bounds(0, 0, 1) == (0, 0)
    assert shard.gather_counts(7) == [7]
    assert shard.reduce_timing(3.5, 9) == (3.5, 9)
    sb = shard.super_batches(torch.arange(10), batch=4, per_step=2)
    assert [p.tolist() for _, p in sb] == [[0, 4, 8], [0, 2, 2]]
