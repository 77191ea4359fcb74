"""Seeded differential fuzzing of the model loader (and, for mutants the reference accepts, of the
operators): small valid models with one or two random edits to their graph JSON.  The reference's
verdict on every mutant (load status, and output + gas when it loads) is a committed fixture
written by tests/golden/make_golden.py; the tests replay the same mutants against the library.

The loader contract being probed: src/runtime/graph_runtime.h:216-436 (JSON reader),
src/runtime/graph_runtime.cc:53-250 (Init / CheckAttr / SetupStorage / SetupOpExecs),
src/cvm/top/**/*.cc (attribute parsers, shape and precision inference).
"""
import json

import numpy as np

import cases

wl = cases.wl

ATTR_VALUES = ["0", "1", "2", "3", "-1", "7", "8", "16", "31", "32", "33", "100", "(0, 0)", "(1, 1)", "(2, 2)",
               "(1, 2)", "(3, 3)", "[1]", "(0,)", "(1,)", "(-1,)", "(0, 1)", "(1, 0)", "True", "False", "abc", "",
               "NHWC", "1.5", "(1, 1, 1)", "None"]
PRECISIONS = [-1, 0, 1, 2, 7, 8, 9, 15, 16, 17, 30, 31, 32, 33]
SWAPS = ["relu", "abs", "negative", "clip", "cvm_clip", "cvm_right_shift", "cvm_left_shift", "cvm_precision",
         "flatten", "elemwise_add", "elemwise_sub", "broadcast_add", "broadcast_sub", "broadcast_mul",
         "broadcast_max", "broadcast_div", "broadcast_greater", "max", "sum", "transpose", "squeeze",
         "expand_dims", "max_pool2d", "upsampling", "repeat", "tile", "conv2d", "dense", "concatenate"]


# Refusals this library adds to the reference's checks.  The reference accepts these models and
# then (1) indexes the weight tensor by the attributes (out of bounds, or with another tensor's
# strides), or (2) runs a storage plan in which live entries share a buffer, so operators read
# values a later operator already overwrote.
STRICTER = ("does not match attributes", "storage plan:")


def is_documented_refusal(text):
    return any(k in text for k in STRICTER)


def bases():
    """name -> (graph dict, params blob, data precision)."""
    out = {}
    for name, thunk in (
            ("chain", lambda: wl.conv_chain(1, channels=32, size=8)),
            ("tail", lambda: wl.ssd_tail(batch=1, anchors=60, top_k=10)),
            ("mobilenet", lambda: wl.mobilenet_v1(batch=1, size=32)),
            ("ssd", lambda: wl.ssd_full(batch=1, size=64))):
        js, pb, x = thunk()
        out[name] = (json.loads(js), pb, x)
    return out


def _op_nodes(g):
    return [i for i, n in enumerate(g["nodes"]) if n["op"] != "null"]


def _mutate(g, rng):
    """One random edit; returns a short description."""
    nodes = g["nodes"]
    rp = g["node_row_ptr"]
    attrs = g["attrs"]
    ops = _op_nodes(g)
    kind = rng.randint(0, 12)
    if kind == 0:      # attribute value
        nid = ops[rng.randint(len(ops))]
        d = json.loads(attrs["op_attrs"][1][nid])
        if d:
            k = sorted(d)[rng.randint(len(d))]
            d[k] = ATTR_VALUES[rng.randint(len(ATTR_VALUES))]
            attrs["op_attrs"][1][nid] = json.dumps(d)
            return "attr %s.%s=%s" % (nodes[nid]["name"], k, d[k])
        d["axis"] = "1"
        attrs["op_attrs"][1][nid] = json.dumps(d)
        return "attr %s +axis" % nodes[nid]["name"]
    if kind == 1:      # attribute removed
        nid = ops[rng.randint(len(ops))]
        d = json.loads(attrs["op_attrs"][1][nid])
        if d:
            k = sorted(d)[rng.randint(len(d))]
            del d[k]
            attrs["op_attrs"][1][nid] = json.dumps(d)
            return "attr %s -%s" % (nodes[nid]["name"], k)
        return "noop"
    if kind == 2:      # one shape extent
        e = rng.randint(len(attrs["shape"][1]))
        s = list(attrs["shape"][1][e])
        if s:
            a = rng.randint(len(s))
            s[a] = max(0, s[a] + [-1, 1, 1, 2, -s[a], s[a]][rng.randint(6)])
            if int(np.prod(s, dtype=np.int64)) > (1 << 22):
                return "noop"
            attrs["shape"][1][e] = s
            return "shape[%d][%d]=%d" % (e, a, s[a])
        return "noop"
    if kind == 3:      # shape rank
        e = rng.randint(len(attrs["shape"][1]))
        s = list(attrs["shape"][1][e])
        if rng.randint(2) and s:
            s.pop(rng.randint(len(s)))
        else:
            s.insert(rng.randint(len(s) + 1), 1)
        attrs["shape"][1][e] = s
        return "rank[%d]=%d" % (e, len(s))
    if kind == 4:      # declared precision
        e = rng.randint(len(attrs["precision"][1]))
        attrs["precision"][1][e] = PRECISIONS[rng.randint(len(PRECISIONS))]
        return "precision[%d]=%d" % (e, attrs["precision"][1][e])
    if kind == 5:      # storage plan
        e = rng.randint(len(attrs["storage_id"][1]))
        attrs["storage_id"][1][e] = int(rng.randint(-1, len(attrs["storage_id"][1]) + 1))
        return "storage[%d]=%d" % (e, attrs["storage_id"][1][e])
    if kind == 6:      # rewire one input
        nid = ops[rng.randint(len(ops))]
        ins = nodes[nid]["inputs"]
        if ins:
            k = rng.randint(len(ins))
            ins[k] = [int(rng.randint(0, len(nodes))), int(rng.randint(0, 2) if rng.randint(4) == 0 else 0), 0]
            return "input %s[%d]=%s" % (nodes[nid]["name"], k, ins[k])
        return "noop"
    if kind == 7:      # operator swapped
        nid = ops[rng.randint(len(ops))]
        nodes[nid]["attrs"]["func_name"] = SWAPS[rng.randint(len(SWAPS))]
        return "func %s=%s" % (nodes[nid]["name"], nodes[nid]["attrs"]["func_name"])
    if kind == 8:      # arity fields
        nid = ops[rng.randint(len(ops))]
        k = ["num_inputs", "num_outputs", "flatten_data"][rng.randint(3)]
        nodes[nid]["attrs"][k] = str(rng.randint(0, 4))
        return "%s %s=%s" % (nodes[nid]["name"], k, nodes[nid]["attrs"][k])
    if kind == 9:      # heads (inside the entry table: past it the reference reads out of bounds)
        if rng.randint(2):
            g["heads"].append([int(rng.randint(0, len(nodes))), 0, 0])
        else:
            nid = int(rng.randint(0, len(nodes)))
            idx = int(rng.randint(0, 2))
            if rp[nid] + idx >= rp[-1]:
                idx = 0
            g["heads"][rng.randint(len(g["heads"]))] = [nid, idx, 0]
        return "heads=%s" % g["heads"]
    if kind == 10:     # tables
        k = rng.randint(4)
        if k == 0:
            rp[rng.randint(len(rp))] += int(rng.randint(-1, 2))
        elif k == 1:
            g["arg_nodes"][rng.randint(len(g["arg_nodes"]))] = int(rng.randint(0, len(nodes)))
        elif k == 2:
            attrs["dltype"][1][rng.randint(len(attrs["dltype"][1]))] = ["int8", "int32", "float32", "uint8", "int64"][rng.randint(5)]
        else:
            g["version"] = ["cvm_1.0.0", "cvm_1.1.0", "cvm_1.2.0", ""][rng.randint(4)]
        return "table %d" % k
    # node record
    nid = rng.randint(len(nodes))
    k = rng.randint(3)
    if k == 0:
        nodes[nid]["name"] = nodes[rng.randint(len(nodes))]["name"]
    elif k == 1:
        nodes[nid]["precision"] = int(PRECISIONS[rng.randint(len(PRECISIONS))])
    else:
        nodes[nid]["op"] = ["null", "cvm_op", "tvm_op"][rng.randint(3)]
    return "node %d field %d" % (nid, k)


def data_for(g, x, seed):
    """Seeded input for a mutant: the base input when the data entry kept its shape, else fresh
    values of the declared precision (None when the declared entry is unusable)."""
    shape = g["attrs"]["shape"][1][0]
    prec = g["attrs"]["precision"][1][0]
    if list(x.shape) == list(shape):
        return x
    n = int(np.prod(shape, dtype=np.int64)) if shape else 1
    if n <= 0 or n > (1 << 22) or not (1 <= prec <= 32):
        return None
    a = (1 << (min(prec, 31) - 1)) - 1
    rng = np.random.RandomState(seed)
    return rng.randint(-a, a + 1, size=shape).astype(x.dtype)


def fuzz_cases(count=1000, seed=20240607):
    """name -> (graph_json bytes, params blob, input ndarray or None, description)."""
    rng = np.random.RandomState(seed)
    base = bases()
    names = sorted(base)
    out = {}
    for i in range(count):
        bname = names[i % len(names)]
        g0, pb, x = base[bname]
        g = json.loads(json.dumps(g0))
        desc = [_mutate(g, rng)]
        if rng.randint(4) == 0:
            desc.append(_mutate(g, rng))
        out["fuzz_%03d_%s" % (i, bname)] = (json.dumps(g).encode(), pb, data_for(g, x, i), "; ".join(desc))
    return out
