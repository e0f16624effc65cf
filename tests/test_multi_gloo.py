"""The N > 1 host logic on CPU with the gloo backend, world size 2: row-shard
bounds, column gather layout, and that a sharded oracle product reassembled by
the all-gather equals the unsharded product bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from mojolearn_b200 import parallel


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)
        x = rng.standard_normal((5, 300)).astype(np.float32)
        w = rng.standard_normal((64, 300)).astype(np.float32)
        lo, hi = parallel.shard_bounds(64, rank, world)
        part = oracle.gemm(x, w[lo:hi].copy(), oracle.OP_NT)  # this rank's output columns, full k
        full = parallel.gather_columns(torch.from_numpy(part)).numpy()
        want = oracle.gemm(x, w, oracle.OP_NT)
        ok = full.tobytes() == want.tobytes()
        # KV caches re-cut from sequence shards to head shards: [b/g, heads, L, hd] on every rank -> [b, heads/g, L, hd]
        cache = torch.arange(4 * 6 * 3 * 2, dtype=torch.float32).reshape(4, 6, 3, 2)  # the whole [b, heads, L, hd]
        mine = cache[rank * 2:(rank + 1) * 2].contiguous()
        got = parallel.exchange_heads(mine, world)
        ok = ok and torch.equal(got, cache[:, rank * 3:(rank + 1) * 3].contiguous())
        out.put((rank, ok, (lo, hi)))
    except Exception as exc:  # report instead of leaving the parent to time out
        out.put((rank, False, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_sharded_columns_reassemble_bit_for_bit():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[2] for r in results) == [(0, 32), (32, 64)]
    assert all(r[1] for r in results)


def test_exchange_plan_keeps_the_first_gather_apart():
    plan = parallel.ExchangePlan(8, first_zone=2 << 20, total_bytes=(2 << 20) + (80 << 20))
    shapes = [(32, 256), (32, 256), (32, 1024), (32, 256)] * 2 + [(32, 6288)]
    for step in range(2):  # every step places its gathers at the same offsets
        plan.begin_step()
        placed = [plan.place(m, w) for m, w in shapes]
        assert [p[0] for p in placed] == list(range(len(shapes)))
        offsets = [p[1] for p in placed]
        assert offsets[0] == 0 and offsets[1] == 2 << 20
        sizes = [m * w * 8 * 8 for m, w in shapes]  # world x (word, tag) pairs
        for i in range(1, len(shapes) - 1):
            assert offsets[i + 1] >= offsets[i] + sizes[i] and offsets[i] % 256 == 0
    plan.begin_step()
    assert not plan.fits(64, 50304)  # wider than the first gather's zone: the caller falls back to the process group
    plan.place(32, 256)
    assert plan.needs_closing_gather()
    with pytest.raises(RuntimeError):
        plan.begin_step()  # a step of one gather cannot order the reuse of its area
    plan.place(1, 2)       # the closing gather the exchange adds by itself
    plan.begin_step()


def test_shard_bounds_refusals():
    assert parallel.shard_bounds(50304, 3, 8) == (3 * 6288, 4 * 6288)
    with pytest.raises(ValueError):
        parallel.shard_bounds(10, 0, 3)
    with pytest.raises(ValueError):
        parallel.shard_bounds(8, 2, 2)
