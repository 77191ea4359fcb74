"""Seeded random operator graphs: a differential test of the lowering (chain fusion, residual joins,
int8 / int32 storage decisions, layout changes) against the reference's CPU runtime.

Each graph starts from an int8 image, applies 4..14 random operators drawn from the whole operator
set (src/cvm/top/**: convolutions of every kind the kernels distinguish, dense, pooling,
element-wise and broadcast arithmetic, shifts and clips, reductions, concatenation and the
transform operators) to random earlier results, and ends in one or two heads.  Precisions are
tracked only roughly; a graph whose precision inference fails in the reference is kept as a
refusal case.  The reference's verdict (load status, inference status, SHA-256 of the output) is
the committed fixture tests/golden/random_graphs.npz, written by tests/golden/make_golden.py.
"""
import numpy as np

import cases

wl = cases.wl


class _T:
    """A live tensor: graph entry, shape, rough precision."""

    def __init__(self, e, shape, prec):
        self.e, self.shape, self.prec = e, list(shape), prec


def _narrow(g, rng, t):
    """Back to 8 bits the way quantised models do it."""
    if rng.randint(3) == 0:
        y = g.op("cvm_clip", [t.e], t.shape, {"precision": 8})
    else:
        y = g.op("cvm_right_shift", [t.e], t.shape, {"precision": 8, "shift_bit": int(rng.randint(1, 12))})
    return _T(y, t.shape, 8)


def _conv(g, rng, t):
    n, c, h, w = t.shape
    kind = rng.randint(5)
    k = int([1, 3, 3, 5, 2][rng.randint(5)])
    stride = int([1, 1, 2, 3][rng.randint(4)])
    dil = 2 if (k == 3 and rng.randint(5) == 0) else 1
    pad = int(rng.randint(0, k // 2 + 2))
    groups = 1
    oc = int([8, 16, 24, 32, 40, 64, 96, 128][rng.randint(8)])
    if kind == 0 and c > 1:                      # depthwise
        groups, oc = c, c
    elif kind == 1 and c % 4 == 0:               # grouped
        groups = 4
        oc = (oc // 4) * 4
    dk = dil * (k - 1) + 1
    if h + 2 * pad < dk or w + 2 * pad < dk:
        return None
    y = g.conv(t.e, oc, k, stride, pad, groups=groups, relu=bool(rng.randint(2)),
               shift=[None, None, 0, int(rng.randint(1, 14))][rng.randint(4)], dilation=dil, bias=bool(rng.randint(4)))
    s = g.shape_of(y)
    last = g.nodes[y[0]]["attrs"]["func_name"]
    return _T(y, s, 8 if last == "cvm_right_shift" else 26)


def _step(g, rng, live):
    """Appends one random operator; returns the new tensor or None when nothing applied."""
    t = live[rng.randint(len(live))]
    r = len(t.shape)
    kind = rng.randint(28)
    if kind <= 4 and r == 4:
        if t.prec > 8:
            t = _narrow(g, rng, t)
            live.append(t)
        return _conv(g, rng, t)
    if kind == 5 and r == 2:
        if t.prec > 8:
            t = _narrow(g, rng, t)
            live.append(t)
        units = int([10, 32, 64, 100][rng.randint(4)])
        y = g.dense(t.e, units, shift=[None, 0, 9][rng.randint(3)], relu=bool(rng.randint(2)), bias=bool(rng.randint(3)))
        last = g.nodes[y[0]]["attrs"]["func_name"]
        return _T(y, g.shape_of(y), 8 if last == "cvm_right_shift" else 26)
    if kind == 6:
        f = ["relu", "abs", "negative", "cvm_precision"][rng.randint(4)]
        return _T(g.op(f, [t.e], t.shape), t.shape, t.prec if f != "cvm_precision" else 6)
    if kind == 7:
        lo, hi = sorted(int(v) for v in rng.randint(-300, 300, size=2))
        if lo == hi:
            hi += 1
        return _T(g.op("clip", [t.e], t.shape, {"a_min": lo, "a_max": hi}), t.shape, 10)
    if kind == 8:
        p = int(rng.randint(1, 17))
        return _T(g.op("cvm_clip", [t.e], t.shape, {"precision": p}), t.shape, p)
    if kind == 9:
        p = int(rng.randint(2, 17))
        return _T(g.op("cvm_right_shift", [t.e], t.shape, {"precision": p, "shift_bit": int(rng.randint(1, 10))}), t.shape, p)
    # cvm_left_shift is left out: the reference's CPU operator throws on every call (it converts its
    # attribute handle to a string, src/runtime/cpu/ops/elemwise.cc:183), so it has no CPU verdict.
    if kind == 10 and r >= 2 and 1 in t.shape[1:]:
        ax = 1 + t.shape[1:].index(1)
        s = t.shape[:ax] + t.shape[ax + 1:]
        return _T(g.op("squeeze", [t.e], s, {"axis": (ax,)}), s, t.prec)
    if kind in (11, 12):
        same = [u for u in live if u.shape == t.shape and u is not t]
        if same and max(t.prec, same[0].prec) < 31:
            u = same[rng.randint(len(same))]
            f = ["elemwise_add", "elemwise_sub"][rng.randint(2)]
            return _T(g.op(f, [t.e, u.e], t.shape), t.shape, max(t.prec, u.prec) + 1)
        return None
    if kind == 13 and t.prec <= 16:
        f = "broadcast_" + ["add", "sub", "mul", "max", "div", "greater"][rng.randint(6)]
        bshape = [(1,), (t.shape[-1],), tuple([t.shape[1]] + [1] * (r - 2)) if r >= 3 else (1,)][rng.randint(3)]
        val = rng.randint(-100, 101, size=bshape).astype(np.int32)
        if f == "broadcast_div" and rng.randint(2):
            val[val == 0] = 3
        b = g.var("c%d" % len(g.nodes), bshape, 8, val)
        prec = {"broadcast_mul": t.prec + 8, "broadcast_add": t.prec + 1, "broadcast_sub": t.prec + 1}.get(f, t.prec)
        return _T(g.op(f, [t.e, b], t.shape), t.shape, prec)
    if kind == 14 and r == 4:
        n, c, h, w = t.shape
        k = int(rng.randint(2, 4))
        s = int(rng.randint(1, 3))
        pad = int(rng.randint(0, k // 2 + 1))
        if h + 2 * pad < k or w + 2 * pad < k:
            return None
        y = g.max_pool(t.e, k, s, pad)
        return _T(y, g.shape_of(y), t.prec)
    if kind == 15 and r == 4 and t.shape[2] * t.shape[3] <= 64:
        sc = int(rng.randint(2, 4))
        s = [t.shape[0], t.shape[1], t.shape[2] * sc, t.shape[3] * sc]
        return _T(g.op("upsampling", [t.e], s, {"scale": sc}), s, t.prec)
    if kind == 16:
        ax = int(rng.randint(0, r))
        mates = [u for u in live if len(u.shape) == r and u is not t
                 and all(a == b for i, (a, b) in enumerate(zip(u.shape, t.shape)) if i != ax)]
        if not mates:
            return None
        u = mates[rng.randint(len(mates))]
        s = list(t.shape)
        s[ax] += u.shape[ax]
        return _T(g.op("concatenate", [t.e, u.e], s, {"axis": ax}), s, max(t.prec, u.prec))
    if kind == 17 and r >= 2:
        f = ["sum", "max"][rng.randint(2)]
        axes = sorted(set(int(a) for a in rng.randint(1, r, size=rng.randint(1, 3))))
        keep = bool(rng.randint(2))
        s = [d if i not in axes else 1 for i, d in enumerate(t.shape)] if keep else [d for i, d in enumerate(t.shape) if i not in axes]
        red = int(np.prod([t.shape[a] for a in axes]))
        prec = t.prec + (int(np.ceil(np.log2(red))) if f == "sum" and red > 1 else 0)
        if prec > 32:
            return None
        return _T(g.op(f, [t.e], s, {"axis": tuple(axes), "keepdims": keep, "exclude": False}), s, prec)
    if kind == 18:
        perm = [int(p) for p in rng.permutation(r)]
        s = [t.shape[p] for p in perm]
        return _T(g.op("transpose", [t.e], s, {"axes": tuple(perm)}), s, t.prec)
    if kind == 19 and r >= 2:
        n = int(np.prod(t.shape[1:]))
        if rng.randint(2):
            return _T(g.op("flatten", [t.e], [t.shape[0], n]), [t.shape[0], n], t.prec)
        if n % 4 == 0:
            s = [t.shape[0], 4, n // 4]
            return _T(g.op("reshape", [t.e], s, {"shape": tuple(s)}), s, t.prec)
        return None
    if kind == 20:
        begin, end = [], []
        for d in t.shape:
            b = int(rng.randint(0, d))
            e = int(rng.randint(b + 1, d + 1))
            begin.append(b)
            end.append(e)
        s = [e - b for b, e in zip(begin, end)]
        return _T(g.op("strided_slice", [t.e], s, {"begin": tuple(begin), "end": tuple(end)}), s, t.prec)
    if kind == 21 and int(np.prod(t.shape)) <= 4096:
        ax = int(rng.randint(0, r))
        rep = int(rng.randint(2, 4))
        s = list(t.shape)
        s[ax] *= rep
        return _T(g.op("repeat", [t.e], s, {"repeats": rep, "axis": ax}), s, t.prec)
    if kind == 22 and int(np.prod(t.shape)) <= 4096:
        reps = [int(v) for v in rng.randint(1, 3, size=r)]
        s = [d * k for d, k in zip(t.shape, reps)]
        return _T(g.op("tile", [t.e], s, {"reps": tuple(reps)}), s, t.prec)
    if kind == 23:
        s = [t.shape[0], 1] + t.shape[1:]
        if len(s) > 6:
            return None
        return _T(g.op("expand_dims", [t.e], s, {"axis": 1, "num_newaxis": 1}), s, t.prec)
    if kind == 24:
        mates = [u for u in live if len(u.shape) == r and u is not t and any(a < b for a, b in zip(u.shape, t.shape))]
        if not mates:
            return None
        u = mates[rng.randint(len(mates))]
        axes = [i for i in range(r) if u.shape[i] <= t.shape[i]]
        if not axes:
            return None
        if len(axes) > 1 and rng.randint(2):
            axes = axes[:rng.randint(1, len(axes))]
        s = [u.shape[i] if i in axes else t.shape[i] for i in range(r)]
        attrs = None if len(axes) == r and rng.randint(2) else {"axis": tuple(axes)}
        return _T(g.op("slice_like", [t.e, u.e], s, attrs), s, t.prec)
    if kind == 25:
        axis = None if rng.randint(3) == 0 else int(rng.randint(0, r))
        ishape = tuple(int(v) for v in rng.randint(1, 5, size=rng.randint(1, 3)))
        n = int(np.prod(t.shape)) if axis is None else t.shape[axis]
        idx = rng.randint(-3, n + 3, size=ishape).astype(np.int32)
        iv = g.var("i%d" % len(g.nodes), ishape, 16, idx)
        s = list(ishape) if axis is None else t.shape[:axis] + list(ishape) + t.shape[axis + 1:]
        if len(s) > 6:
            return None
        return _T(g.op("take", [t.e, iv], s, None if axis is None else {"axis": axis}), s, t.prec)
    if kind == 26 and t.prec <= 10:
        in_dim = int(rng.randint(4, 300))
        tp = int([8, 12, 16][rng.randint(3)])
        a = (1 << (tp - 1)) - 1
        table = rng.randint(-a, a + 1, size=(in_dim,)).astype(np.int32)
        tv = g.var("t%d" % len(g.nodes), (in_dim,), tp, table)
        return _T(g.op("cvm_lut", [t.e, tv], t.shape, {"in_dim": in_dim}), t.shape, tp)
    if kind == 27 and t.prec <= 16:
        same = [u for u in live if u.shape == t.shape and u is not t]
        if len(same) < 1:
            return None
        u = same[rng.randint(len(same))]
        v = same[rng.randint(len(same))]
        return _T(g.op("where", [t.e, u.e, v.e], t.shape), t.shape, max(t.prec, u.prec, v.prec))
    return None


def random_graph(seed):
    """(graph_json, params_blob, input) for one seed."""
    rng = np.random.RandomState(seed)
    g = wl.GraphBuilder(seed)
    n = int(rng.randint(1, 4))
    c = int([3, 8, 16, 32, 32, 64][rng.randint(6)])
    h = int(rng.randint(4, 15))
    w = int(rng.randint(4, 15))
    x = rng.randint(-127, 128, size=(n, c, h, w)).astype(np.int8)
    live = [_T(g.var("data", x.shape, 8), x.shape, 8)]
    steps = int(rng.randint(4, 15))
    tries = 0
    while steps > 0 and tries < 200:
        tries += 1
        t = _step(g, rng, live)
        if t is None:
            continue
        if int(np.prod(t.shape)) > (1 << 18):
            break
        live.append(t)
        steps -= 1
    heads = [live[-1].e]
    if len(live) > 2 and rng.randint(10) == 0:
        other = live[rng.randint(1, len(live) - 1)]
        if other.e != heads[0]:
            heads.append(other.e)
    js, pb = g.finish(heads)
    return js, pb, x


def random_tail(seed):
    """A detection tail (get_valid_counts -> non_max_suppression, nms.cc:42-140) on boxes built to
    hit the corners of the CPU loop: tied scores, negative class ids, identical, empty and inverted
    boxes, every relation between top_k / max_output_size / valid count, several 512-box sweep
    blocks, and (sometimes) the operator's input as a second head."""
    rng = np.random.RandomState(seed)
    b = int(rng.randint(1, 5))
    n = int([rng.randint(1, 40), rng.randint(40, 300), rng.randint(500, 1300)][rng.randint(3)])
    style = rng.randint(3)
    rows = np.zeros((b, n, 6), np.int32)
    if style == 0:      # coarse grid: many exact ties and identical boxes
        rows[..., 0] = rng.randint(-1, 3, size=(b, n))
        rows[..., 1] = rng.randint(0, 8, size=(b, n)) * 1000
        rows[..., 2:4] = rng.randint(0, 6, size=(b, n, 2)) * 10
        rows[..., 4:6] = rows[..., 2:4] + rng.randint(-1, 4, size=(b, n, 2)) * 10
    elif style == 1:    # ordinary detections
        rows[..., 0] = rng.randint(0, 5, size=(b, n))
        rows[..., 1] = rng.randint(0, 1 << 15, size=(b, n))
        rows[..., 2:4] = rng.randint(0, 200, size=(b, n, 2))
        rows[..., 4:6] = rows[..., 2:4] + rng.randint(1, 120, size=(b, n, 2))
    else:               # clustered boxes, a few negative ids, full-range coordinates
        centers = rng.randint(-3000, 3000, size=(b, 4, 2))
        pick = rng.randint(0, 4, size=(b, n))
        rows[..., 0] = np.where(rng.rand(b, n) < 0.1, -1, rng.randint(0, 3, size=(b, n)))
        rows[..., 1] = rng.randint(0, 300, size=(b, n)) * 100
        c = centers[np.arange(b)[:, None], pick]
        rows[..., 2:4] = c + rng.randint(-40, 40, size=(b, n, 2))
        rows[..., 4:6] = rows[..., 2:4] + rng.randint(0, 90, size=(b, n, 2))
    rows = np.clip(rows, -32767, 32767).astype(np.int32)
    g = wl.GraphBuilder(seed)
    d = g.var("data", (b, n, 6), 16)
    thr = int([-1, 0, 999, 2000, 5000, 20000, 40000][rng.randint(7)])
    # An image without a valid box ends the CPU operator (nms.cc:76-79, `return 0`) and leaves the
    # output rows of every later image uninitialised; only the last image may be empty here.
    if ((rows[:-1, :, 1] > thr).sum(axis=1) <= 0).any():
        thr = -1
    vc, boxes = g.op("get_valid_counts", [d], [(b,), (b, n, 6)], {"score_threshold": thr})
    y = g.op("non_max_suppression", [boxes, vc], (b, n, 6), {
        "iou_threshold": int([1, 25, 50, 75, 100, 101, 1000][rng.randint(7)]),
        "top_k": int([-1, -1, 0, 1, 5, max(1, n // 2), n, n + 5][rng.randint(8)]),
        "max_output_size": int([-1, -1, 0, 1, 3, n][rng.randint(6)]),
        "force_suppress": bool(rng.randint(2)), "id_index": 0, "score_index": 1, "coord_start": 2,
        "return_indices": False, "invalid_to_bottom": True})
    heads = [y]
    if rng.randint(4) == 0:
        heads.append(boxes)
    js, pb = g.finish(heads)
    return js, pb, rows


COUNT = 600
TAILS = 300


def random_cases(count=COUNT, first_seed=5000, tails=TAILS):
    table = {"rand_%03d" % i: (lambda s=first_seed + i: random_graph(s)) for i in range(count)}
    table.update({"tail_%03d" % i: (lambda s=first_seed + i: random_tail(s)) for i in range(tails)})
    return table
