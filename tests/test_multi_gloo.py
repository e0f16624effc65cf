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
        out.put((rank, full.tobytes() == want.tobytes(), (lo, hi)))
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


def test_shard_bounds_refusals():
    assert parallel.shard_bounds(50304, 3, 8) == (3 * 6288, 4 * 6288)
    with pytest.raises(ValueError):
        parallel.shard_bounds(10, 0, 3)
    with pytest.raises(ValueError):
        parallel.shard_bounds(8, 2, 2)
