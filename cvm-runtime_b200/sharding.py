"""Batch sharding across the GPUs of one box.

Every operator on this path is independent across the batch dimension (convolutions, pooling,
element-wise, dense rows; get_valid_counts / non_max_suppression loop over batches,
src/runtime/cpu/ops/nms.cc:44,68), so a batch is split into contiguous shards, one model handle
per GPU with its own weight replica, no collective on the data path.  The reference C-ABI has no
multi-device notion (src/core/c_api.cc:29-36): the sharding lives above it, one handle and one
host thread per GPU.
"""
import threading

import numpy as np

from . import runtime as rt


def shard_range(total, world, rank):
    """Contiguous [lo, hi) of `total` items owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class ShardedModel:
    """`build(batch)` -> (graph_json, params_blob, example_input) is called once per distinct shard
    size; shard r runs on GPU `devices[r]`.  Works for single-head models whose output is
    concatenated along the batch (SaveTensor modes 3 and 4, src/core/model.cc:248-262)."""

    def __init__(self, build, total_batch, devices):
        self.devices = list(devices)
        self.spans = [shard_range(total_batch, len(self.devices), r) for r in range(len(self.devices))]
        self.nets = []
        for dev, (lo, hi) in zip(self.devices, self.spans):
            if hi == lo:
                self.nets.append(None)
                continue
            js, pb, _ = build(hi - lo)
            self.nets.append(rt.CVMAPILoadModel(js, pb, dev))

    def infer(self, x):
        outs = [None] * len(self.nets)
        errs = []

        def work(r):
            try:
                lo, hi = self.spans[r]
                if self.nets[r] is not None:
                    outs[r] = rt.inference_bytes(self.nets[r], np.ascontiguousarray(x[lo:hi]))
            except Exception as e:  # a failing shard fails the whole call
                errs.append(e)

        threads = [threading.Thread(target=work, args=(r,)) for r in range(len(self.nets))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errs:
            raise errs[0]
        return np.concatenate([o for o in outs if o is not None])

    def free(self):
        for n in self.nets:
            if n is not None:
                rt.CVMAPIFreeModel(n)
        self.nets = []
