"""Batch sharding across the GPUs of one box.

The operators of the image and detection networks are independent across the batch dimension
(convolutions, pooling, element-wise, dense rows; get_valid_counts / non_max_suppression loop
over batches, src/runtime/cpu/ops/nms.cc:44,68), so a batch is split into contiguous shards, one
model handle per GPU with its own weight replica, no collective on the data path.  The reference
C-ABI has no multi-device notion (src/core/c_api.cc:29-36): the sharding lives above it, one
handle and one host thread per GPU.

Two limits.  (1) Not every graph is separable along the batch: a reshape that folds the batch
axis, a reduction over axis 0, a take without an axis, a parameter of the batch's shape, the
argmax and detection post-processing (which pick over the whole output) are not.
`batch_separable()` checks a graph node by node and `ShardedModel` refuses what fails it.
(2) non_max_suppression RETURNS FROM THE WHOLE CALL at the first image whose valid count is not
positive (nms.cc:76-79): the images after it keep whatever the output buffer held.  In a shard
that holds only later images they are processed normally, so on such an input the sharded and
the unsharded bytes differ for those later images.  The sharded result is the well-defined one
(the unsharded one depends on stale memory); callers that need the reference's exact bytes on
such inputs run unsharded.
"""
import json
import threading

import numpy as np

from . import runtime as rt


def shard_range(total, world, rank):
    """Contiguous [lo, hi) of `total` items owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _ints(text):
    """'(2, 3)' / '[2, 3]' / '2' / 'None' -> list of ints (None for an absent value)."""
    t = str(text).strip()
    if t in ("None", ""):
        return None
    t = t.strip("()[]")
    return [int(v) for v in t.replace(" ", "").split(",") if v not in ("", "None")]


_ROWWISE = {
    "conv2d", "dense", "max_pool2d", "upsampling", "relu", "clip", "cvm_clip", "cvm_right_shift",
    "cvm_left_shift", "cvm_precision", "abs", "negative", "flatten", "get_valid_counts",
    "non_max_suppression",
}
_BINARY = {
    "elemwise_add", "elemwise_sub", "broadcast_add", "broadcast_sub", "broadcast_mul", "broadcast_div",
    "broadcast_max", "broadcast_greater", "where", "cvm_lut",
}


def batch_separable(graph_json):
    """None when running the graph on a slice of the batch gives that slice of the full result,
    else a sentence saying which node stands in the way.  Conservative: a shape that is not
    recognised is refused."""
    g = json.loads(graph_json) if isinstance(graph_json, (str, bytes)) else graph_json
    nodes, shapes = g["nodes"], g["attrs"]["shape"][1]
    row_ptr = g["node_row_ptr"]
    op_attrs = g["attrs"].get("op_attrs", [None, [None] * len(nodes)])[1]
    if len(g["heads"]) != 1:
        return "%d heads: their bytes interleave per head, not per image" % len(g["heads"])
    if g.get("postprocess") in ("argmax", "detection"):
        return "the %s post-processing selects over the whole output" % g["postprocess"]
    data = [i for i in g["arg_nodes"] if nodes[i]["name"] == "data"]
    if len(data) != 1:
        return "no input named data"
    batch = shapes[row_ptr[data[0]]][0]
    is_param = [n["op"] == "null" and n["name"] != "data" for n in nodes]
    for nid, n in enumerate(nodes):
        if n["op"] == "null":
            continue
        op = n["attrs"]["func_name"]
        at = json.loads(op_attrs[nid]) if op_attrs[nid] else {}
        where = "%s %s" % (op, n["name"])
        ins = [(e[0], shapes[row_ptr[e[0]] + e[1]]) for e in n["inputs"]]
        outs = [shapes[k] for k in range(row_ptr[nid], row_ptr[nid + 1])]
        for sh in outs:
            if not sh or sh[0] != batch:
                return "%s: output shape %s does not lead with the batch" % (where, sh)
        acts = [(src, sh) for src, sh in ins if not is_param[src]]
        for src, sh in acts:
            if not sh or sh[0] != batch:
                return "%s: operand of shape %s does not lead with the batch" % (where, sh)
        if op not in ("conv2d", "dense"):
            for src, sh in ins:
                if is_param[src] and batch > 1 and len(sh) == len(outs[0]) and sh[0] == batch and op != "cvm_lut":
                    return "%s: parameter of the batch's shape %s" % (where, sh)
        if op in _ROWWISE or op in _BINARY:
            if op == "cvm_lut" and not is_param[ins[1][0]]:
                return "%s: table computed from the batch" % where
            continue
        if op in ("reshape", "squeeze", "expand_dims"):
            if op == "squeeze" and (_ints(at.get("axis")) is None or 0 in [a % len(ins[0][1]) for a in _ints(at.get("axis"))]):
                if batch == 1:
                    return "%s: may remove the batch axis" % where
            if op == "expand_dims" and int(at.get("axis", 0)) % (len(ins[0][1]) + 1) == 0:
                return "%s: inserts an axis before the batch" % where
            continue   # leading extent preserved (checked above): rows stay rows
        if op in ("sum", "max"):
            nd = len(ins[0][1])
            axis = [a % nd for a in (_ints(at.get("axis")) or [])]
            exclude = str(at.get("exclude", "False")) == "True"
            reduced = [a for a in range(nd) if (a in axis) != exclude] if axis else list(range(nd))
            if 0 in reduced:
                return "%s: reduces over the batch axis" % where
            continue
        if op == "concatenate":
            if int(at.get("axis", 1)) % len(outs[0]) == 0:
                return "%s: joins along the batch axis" % where
            continue
        if op == "transpose":
            axes = _ints(at.get("axes"))
            if not axes or axes[0] % len(outs[0]) != 0:
                return "%s: moves the batch axis" % where
            continue
        if op == "strided_slice":
            begin, end, stride = _ints(at.get("begin")) or [0], _ints(at.get("end")) or [], _ints(at.get("stride")) or [1]
            if begin[0] != 0 or (stride[0] if stride else 1) != 1 or outs[0][0] != ins[0][1][0]:
                return "%s: cuts the batch axis" % where
            continue
        if op == "slice_like":
            axis = _ints(at.get("axis"))
            if not axis or 0 in [a % len(outs[0]) for a in axis]:
                return "%s: slices the batch axis" % where
            continue
        if op == "repeat":
            if int(at.get("axis", 0)) % len(outs[0]) == 0:
                return "%s: repeats along the batch axis" % where
            continue
        if op == "tile":
            reps = _ints(at.get("reps")) or []
            if len(reps) >= len(outs[0]) and reps[len(reps) - len(outs[0])] != 1 or len(reps) > len(ins[0][1]):
                return "%s: tiles the batch axis" % where
            continue
        if op == "take":
            axis = at.get("axis")
            if axis in (None, "None") or int(axis) % len(ins[0][1]) == 0 or not is_param[ins[1][0]]:
                return "%s: gathers across the batch" % where
            continue
        return "%s: not known to be independent across the batch" % where
    return None


class ShardedModel:
    """`build(batch)` -> (graph_json, params_blob, example_input) is called once per distinct shard
    size; shard r runs on GPU `devices[r]`.  Works for single-head models whose output is
    concatenated along the batch (SaveTensor modes 3 and 4, src/core/model.cc:248-262); a graph
    that `batch_separable()` does not pass is refused with ValueError before anything is loaded."""

    def __init__(self, build, total_batch, devices):
        self.devices = list(devices)
        self.spans = [shard_range(total_batch, len(self.devices), r) for r in range(len(self.devices))]
        self.nets = []
        built = []
        for lo, hi in self.spans:
            built.append(build(hi - lo) if hi > lo else None)
            if built[-1] is not None:
                why = batch_separable(built[-1][0])
                if why is not None:
                    raise ValueError("graph cannot be sharded along the batch: " + why)
        for dev, b in zip(self.devices, built):
            self.nets.append(None if b is None else rt.CVMAPILoadModel(b[0], b[1], dev))

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
