"""Batch sharding across ranks (the only multi-GPU scheme of this path): world_size-2 gloo ranks on
CPU, each computing its shard with the oracle, must reproduce the unsharded result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sharding = cases.pkg.sharding
    oracle = cases.ge.load_oracle()
    total = 6
    lo, hi = sharding.shard_range(total, world, rank)
    # weights come from their own RandomState stream, so every shard size sees the same model
    js_full, pb_full, x_full = cases.wl.mobilenet_v1(batch=total, size=32)
    js, pb, _ = cases.wl.mobilenet_v1(batch=hi - lo, size=32)
    part = oracle.run_model(js, pb, x_full[lo:hi])
    parts = [None] * world
    dist.all_gather_object(parts, part)
    # timing reduction used by the benchmark: the slowest rank defines the step time
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        whole = oracle.run_model(js_full, pb_full, x_full)
        q.put((np.array_equal(np.concatenate(parts), whole), float(t.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_full_batch():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok, tmax = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok
    assert tmax == 2.0


def test_shard_ranges_cover_the_batch():
    sharding = cases.pkg.sharding
    for total in (1, 7, 64, 256):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and b >= a
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
