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


def _graph(build, batch=4, **finish):
    b = cases.wl.GraphBuilder(seed=1)
    x = b.var("data", (batch, 4, 6, 6), 8)
    return b.finish(build(b, x, batch), **finish)[0]


_NOT_SEPARABLE = {
    "sum_over_batch": lambda b, x, n: b.op("sum", [x], (4, 6, 6), {"axis": (0,), "keepdims": False, "exclude": False}),
    "sum_exclude_keeps_channel_only": lambda b, x, n: b.op("sum", [x], (4,), {"axis": (1,), "keepdims": False, "exclude": True}),
    "reshape_folds_batch": lambda b, x, n: b.op("reshape", [x], (n * 4, 36), {"shape": (n * 4, 36)}),
    "transpose_moves_batch": lambda b, x, n: b.op("transpose", [x], (4, n, 6, 6), {"axes": (1, 0, 2, 3)}),
    "concat_along_batch": lambda b, x, n: b.op("concatenate", [x, x], (2 * n, 4, 6, 6), {"axis": 0}),
    "take_flat": lambda b, x, n: b.op("take", [x, b.var("idx", (n, 3), 16, np.zeros((n, 3), np.int32))], (n, 3), {}),
    "batch_shaped_parameter": lambda b, x, n: b.op(
        "broadcast_add", [x, b.var("p", (n, 4, 6, 6), 8, np.ones((n, 4, 6, 6), np.int32))], (n, 4, 6, 6)),
    "slice_of_batch": lambda b, x, n: b.op("strided_slice", [x], (n - 1, 4, 6, 6), {"begin": (1, 0, 0, 0), "end": (n, 4, 6, 6), "stride": (1, 1, 1, 1)}),
}


@pytest.mark.parametrize("name", sorted(_NOT_SEPARABLE))
def test_unseparable_graph_is_refused(name):
    sharding = cases.pkg.sharding
    js = _graph(_NOT_SEPARABLE[name])
    why = sharding.batch_separable(js)
    assert why is not None, name
    # the refusal comes before any model is loaded: no GPU is needed to see it
    with pytest.raises(ValueError, match="cannot be sharded"):
        sharding.ShardedModel(lambda batch: (js, b"", None), 4, [0, 0])


def test_heads_and_postprocess_are_refused():
    sharding = cases.pkg.sharding
    relu = lambda b, x, n: b.op("relu", [x], (n, 4, 6, 6))
    assert sharding.batch_separable(_graph(relu)) is None
    assert "argmax" in sharding.batch_separable(_graph(relu, postprocess="argmax"))
    assert "detection" in sharding.batch_separable(_graph(relu, postprocess="detection"))
    b = cases.wl.GraphBuilder(seed=1)
    x = b.var("data", (4, 4, 6, 6), 8)
    js = b.finish([b.op("relu", [x], (4, 4, 6, 6)), b.op("abs", [x], (4, 4, 6, 6))])[0]
    assert "heads" in sharding.batch_separable(js)


def test_separable_verdict_holds_on_the_oracle():
    """Every benchmark network passes the check, and for those the shards of a batch reproduce the
    whole (small sizes, CPU oracle)."""
    sharding = cases.pkg.sharding
    oracle = cases.ge.load_oracle()
    builds = {
        "ssd_tail": lambda n: cases.wl.ssd_tail(batch=n, anchors=96, top_k=20),
        "ssd_full": lambda n: cases.wl.ssd_full(batch=n, size=64),
    }
    for name, build in builds.items():
        js, pb, x = build(4)
        assert sharding.batch_separable(js) is None, name
        whole = oracle.run_model(js, pb, x)
        parts = []
        for r in range(2):
            lo, hi = sharding.shard_range(4, 2, r)
            js_r, pb_r, _ = build(hi - lo)
            parts.append(oracle.run_model(js_r, pb_r, x[lo:hi]))
        assert np.array_equal(np.concatenate(parts), whole), name
