"""Seeded synthetic CVM models: graph JSON + params blob + input bytes for the benchmark and
parity configurations.

Wire formats follow the reference loader: graph JSON as read by CvmRuntime::Load
(src/runtime/graph_runtime.h:208-436; every node attribute value is a JSON string, graph
attributes are [type_tag, list] pairs) and the params blob of load_param_dict
(src/runtime/param_dict.cc:14-38) with NDArray records (include/cvm/runtime/ndarray.h:430-556).
storage ids obey the aliasing rule of PrepareGraphWithVersion (graph_runtime.cc:143-177): only
the listed element-wise / reshape-like operators may write into one of their own inputs.

No dataset is involved: weights, biases and inputs are drawn from numpy RandomState streams, one
RandomState(seed) consumed in node-creation order (weight, then bias, per layer) and a separate
RandomState(input_seed) for the network input.
"""
import json
import math
import struct

import numpy as np

ND_MAGIC = 0xDD5E40F096B4A13F
LIST_MAGIC = 0xF7E58D4F05049CB7

# Operators whose output may share storage with an input (graph_runtime.cc:151-158).
INPLACE_OPS = {"flatten", "relu", "expand_dims", "reshape", "squeeze", "abs", "cvm_precision",
               "elemwise_add", "elemwise_sub", "clip", "cvm_clip", "cvm_right_shift",
               "cvm_left_shift"}


def ndarray_bytes(a):
    a = np.ascontiguousarray(a)
    bits = a.dtype.itemsize * 8
    return (struct.pack("<QQ", ND_MAGIC, 0) + struct.pack("<ii", 1, 0) + struct.pack("<i", a.ndim)
            + struct.pack("<BBH", 0, bits, 1) + struct.pack("<%dq" % a.ndim, *a.shape)
            + struct.pack("<q", a.nbytes) + a.tobytes())


def params_blob(params):
    """Serialise {name: int8/int32 ndarray} in the reference's NDArray-list format."""
    out = [struct.pack("<QQ", LIST_MAGIC, 0), struct.pack("<Q", len(params))]
    for k in params:
        kb = k.encode()
        out.append(struct.pack("<Q", len(kb)) + kb)
    out.append(struct.pack("<Q", len(params)))
    for k in params:
        out.append(ndarray_bytes(params[k]))
    return b"".join(out)


def attr_str(v):
    if isinstance(v, bool):
        return "True" if v else "False"
    if isinstance(v, (tuple, list)):
        return "(" + ", ".join(str(int(x)) for x in v) + ("," if len(v) == 1 else "") + ")"
    return str(v)


class GraphBuilder:
    """Builds a `cvm_1.0.0` graph node by node and plans storage ids by liveness."""

    def __init__(self, seed=0):
        self.nodes, self.op_attrs, self.shapes, self.prec = [], [], [], []
        self.node_outputs = []          # number of outputs per node
        self.params = {}
        self.rng = np.random.RandomState(seed)
        self.counts = {}

    # -- entries are (node_id, output_index)
    def shape_of(self, e):
        return self.shapes[self._eid(e)]

    def _eid(self, e):
        return sum(self.node_outputs[:e[0]]) + e[1]

    def var(self, name, shape, precision, value=None):
        self.nodes.append({"op": "null", "name": name, "inputs": []})
        self.op_attrs.append("{}")
        self.node_outputs.append(1)
        self.shapes.append([int(s) for s in shape])
        self.prec.append(int(precision))
        if value is not None:
            self.params[name] = value
        return (len(self.nodes) - 1, 0)

    def op(self, func, inputs, out_shapes, attrs=None):
        if out_shapes and not isinstance(out_shapes[0], (list, tuple)):
            out_shapes = [out_shapes]
        i = self.counts.get(func, 0)
        self.counts[func] = i + 1
        self.nodes.append({
            "op": "cvm_op", "name": "%s_%d" % (func, i),
            "attrs": {"func_name": func, "num_inputs": str(len(inputs)),
                      "num_outputs": str(len(out_shapes)), "flatten_data": "0"},
            "inputs": [[e[0], e[1], 0] for e in inputs]})
        self.op_attrs.append(json.dumps({k: attr_str(v) for k, v in (attrs or {}).items()}))
        self.node_outputs.append(len(out_shapes))
        for s in out_shapes:
            self.shapes.append([int(x) for x in s])
            self.prec.append(-1)
        nid = len(self.nodes) - 1
        return (nid, 0) if len(out_shapes) == 1 else [(nid, k) for k in range(len(out_shapes))]

    # -- random parameters
    def weight8(self, shape):
        return self.rng.randint(-127, 128, size=shape).astype(np.int8)

    def bias32(self, n):
        return self.rng.randint(-(1 << 16), (1 << 16) + 1, size=(n,)).astype(np.int32)

    # -- layers
    @staticmethod
    def default_shift(k):
        # keeps roughly half of the activations non-zero through the depth of the network
        return max(1, int(round(5.8 + 0.5 * math.log2(k))))

    def conv(self, x, oc, k, stride=1, pad=0, groups=1, relu=True, shift=None, dilation=1, bias=True):
        n, c, h, w = self.shape_of(x)
        i = len(self.params)
        icg = c // groups
        ins = [x, self.var("w%d" % i, (oc, icg, k, k), 8, self.weight8((oc, icg, k, k)))]
        if bias:
            ins.append(self.var("b%d" % i, (oc,), 18, self.bias32(oc)))
        dk = dilation * (k - 1) + 1
        oh, ow = (h + 2 * pad - dk) // stride + 1, (w + 2 * pad - dk) // stride + 1
        y = self.op("conv2d", ins, (n, oc, oh, ow), {
            "channels": oc, "kernel_size": (k, k), "strides": (stride, stride), "padding": (pad, pad),
            "dilation": (dilation, dilation), "groups": groups, "layout": "NCHW",
            "kernel_layout": "OIHW", "use_bias": bias})
        if relu:
            y = self.op("relu", [y], self.shape_of(y))
        if shift is None:
            shift = self.default_shift(icg * k * k)
        if shift:
            y = self.op("cvm_right_shift", [y], self.shape_of(y), {"precision": 8, "shift_bit": shift})
        return y

    def dense(self, x, units, shift=None, relu=False, bias=True):
        n, k = self.shape_of(x)
        i = len(self.params)
        ins = [x, self.var("w%d" % i, (units, k), 8, self.weight8((units, k)))]
        if bias:
            ins.append(self.var("b%d" % i, (units,), 18, self.bias32(units)))
        y = self.op("dense", ins, (n, units), {"units": units, "use_bias": bias})
        if relu:
            y = self.op("relu", [y], self.shape_of(y))
        if shift is not None:
            if shift == 0:
                shift = self.default_shift(k)
            y = self.op("cvm_right_shift", [y], self.shape_of(y), {"precision": 8, "shift_bit": shift})
        return y

    def max_pool(self, x, k, stride, pad):
        n, c, h, w = self.shape_of(x)
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        return self.op("max_pool2d", [x], (n, c, oh, ow), {
            "pool_size": (k, k), "strides": (stride, stride), "padding": (pad, pad),
            "layout": "NCHW", "ceil_mode": False})

    def global_sum(self, x, shift=5):
        n, c, h, w = self.shape_of(x)
        s = self.op("sum", [x], (n, c), {"axis": (2, 3), "keepdims": False, "exclude": False})
        return self.op("cvm_right_shift", [s], (n, c), {"precision": 8, "shift_bit": shift})

    # -- finish
    def finish(self, heads, postprocess=None, version=None):
        """Returns (graph_json_bytes, params_blob_bytes)."""
        if isinstance(heads, tuple):
            heads = [heads]
        n_nodes = len(self.nodes)
        row_ptr = [0]
        for k in self.node_outputs:
            row_ptr.append(row_ptr[-1] + k)
        n_entries = row_ptr[-1]
        eid = lambda nid, idx: row_ptr[nid] + idx
        last_use = [-1] * n_entries
        for nid, nd in enumerate(self.nodes):
            for e in nd["inputs"]:
                last_use[eid(e[0], e[1])] = nid
        for h in heads:
            last_use[eid(h[0], h[1])] = 10 ** 9
        size = lambda e: int(np.prod(self.shapes[e])) * 4
        sid = [-1] * n_entries
        pool_size, free, owner_live = [], [], {}
        for nid, nd in enumerate(self.nodes):
            outs = [eid(nid, k) for k in range(self.node_outputs[nid])]
            if nd["op"] == "null":
                sid[outs[0]] = len(pool_size)
                pool_size.append(size(outs[0]))
                continue
            func = nd["attrs"]["func_name"]
            in_eids = [eid(e[0], e[1]) for e in nd["inputs"]]
            for oe in outs:
                got = None
                if func in INPLACE_OPS and len(outs) == 1:
                    for je in in_eids:
                        src_is_var = self.nodes[self._node_of(je, row_ptr)]["op"] == "null"
                        shared = [k for k in range(n_entries) if sid[k] == sid[je] and k != je and last_use[k] > nid]
                        if (not src_is_var and last_use[je] == nid and not shared
                                and pool_size[sid[je]] >= size(oe) and in_eids.count(je) == 1):
                            got = sid[je]
                            break
                if got is None:
                    if free:
                        free.sort(key=lambda t: abs(pool_size[t] - size(oe)))
                        got = free.pop(0)
                        pool_size[got] = max(pool_size[got], size(oe))
                    else:
                        got = len(pool_size)
                        pool_size.append(size(oe))
                sid[oe] = got
            out_sids = {sid[o] for o in outs}
            for je in set(in_eids):
                src_is_var = self.nodes[self._node_of(je, row_ptr)]["op"] == "null"
                if src_is_var or last_use[je] != nid or sid[je] in out_sids:
                    continue
                if any(sid[k] == sid[je] and last_use[k] > nid for k in range(n_entries) if k != je and sid[k] >= 0):
                    continue
                if sid[je] not in free:
                    free.append(sid[je])
        graph = {
            "nodes": self.nodes,
            "arg_nodes": [i for i, nd in enumerate(self.nodes) if nd["op"] == "null"],
            "node_row_ptr": row_ptr,
            "heads": [[h[0], h[1], 0] for h in heads],
            "attrs": {
                "op_attrs": ["list_str", self.op_attrs],
                "dltype": ["list_str", ["int32"] * n_entries],
                "precision": ["list_int", self.prec],
                "storage_id": ["list_int", sid],
                "shape": ["list_shape", self.shapes],
            },
        }
        if postprocess is not None:
            graph["postprocess"] = postprocess
        if version is not None:
            graph["version"] = version
        self.storage_bytes = sum(pool_size)
        return json.dumps(graph).encode(), params_blob(self.params)

    @staticmethod
    def _node_of(e, row_ptr):
        lo = 0
        while row_ptr[lo + 1] <= e:
            lo += 1
        return lo


# ---------------------------------------------------------------------------------------------
# The five configurations
# ---------------------------------------------------------------------------------------------
def conv_chain(batch=1, seed=0, channels=64, size=56):
    """C1: conv2d 3x3 s1 p1 (+bias) -> cvm_right_shift 8 -> cvm_clip 8.  One RandomState(seed)
    stream: input, weight, bias.  Returns (json, params, input int8 NCHW)."""
    rng = np.random.RandomState(seed)
    x = rng.randint(-127, 128, size=(batch, channels, size, size)).astype(np.int8)
    w = rng.randint(-127, 128, size=(channels, channels, 3, 3)).astype(np.int8)
    b = rng.randint(-(1 << 16), (1 << 16) + 1, size=(channels,)).astype(np.int32)
    g = GraphBuilder(seed)
    d = g.var("data", x.shape, 8)
    wv = g.var("w", w.shape, 8, w)
    bv = g.var("b", b.shape, 18, b)
    y = g.op("conv2d", [d, wv, bv], x.shape, {
        "channels": channels, "kernel_size": [3, 3], "strides": (1, 1), "padding": (1, 1),
        "dilation": (1, 1), "groups": 1, "layout": "NCHW", "kernel_layout": "OIHW", "use_bias": True})
    y = g.op("cvm_right_shift", [y], x.shape, {"precision": 8, "shift_bit": 8})
    y = g.op("cvm_clip", [y], x.shape, {"precision": 8})
    js, pb = g.finish(y)
    return js, pb, x


def image_input(batch, size=224, input_seed=7):
    return np.random.RandomState(input_seed).randint(-127, 128, size=(batch, 3, size, size)).astype(np.int8)


def resnet50(batch=1, seed=0, size=224, input_seed=7, classes=1000):
    """C2: ResNet-50 v1 (bottleneck 3-4-6-3), every conv followed by [relu] + cvm_right_shift(8 bit),
    joins as elemwise_add -> relu -> cvm_clip, global average as sum + shift, dense to `classes`."""
    g = GraphBuilder(seed)
    x = g.var("data", (batch, 3, size, size), 8)
    y = g.conv(x, 64, 7, 2, 3)
    y = g.max_pool(y, 3, 2, 1)
    for stage, (blocks, mid) in enumerate([(3, 64), (4, 128), (6, 256), (3, 512)]):
        for b in range(blocks):
            stride = 2 if (b == 0 and stage > 0) else 1
            out = mid * 4
            sc = y
            if b == 0:
                sc = g.conv(y, out, 1, stride, 0, relu=False)
            z = g.conv(y, mid, 1, 1, 0)
            z = g.conv(z, mid, 3, stride, 1)
            z = g.conv(z, out, 1, 1, 0, relu=False)
            a = g.op("elemwise_add", [z, sc], g.shape_of(z))
            a = g.op("relu", [a], g.shape_of(a))
            y = g.op("cvm_clip", [a], g.shape_of(a), {"precision": 8})
    s = g.global_sum(y)
    o = g.dense(s, classes)
    js, pb = g.finish(o)
    return js, pb, image_input(batch, size, input_seed)


def mobilenet_v1(batch=1, seed=0, size=224, input_seed=7, classes=1000):
    """C3: MobileNet v1 1.0: 3x3/2 stem, 13 x [depthwise 3x3 + pointwise 1x1], sum + shift, dense."""
    g = GraphBuilder(seed)
    x = g.var("data", (batch, 3, size, size), 8)
    y = g.conv(x, 32, 3, 2, 1)
    cfg = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2)] + [(512, 1)] * 5 + [(1024, 2), (1024, 1)]
    for oc, s in cfg:
        c = g.shape_of(y)[1]
        y = g.conv(y, c, 3, s, 1, groups=c)
        y = g.conv(y, oc, 1, 1, 0)
    s_ = g.global_sum(y)
    o = g.dense(s_, classes)
    js, pb = g.finish(o)
    return js, pb, image_input(batch, size, input_seed)


def vgg19(batch=1, seed=0, size=224, input_seed=7, classes=1000, fc=4096):
    """C4: VGG-19: 16 conv 3x3 s1 p1 in five groups with 2x2/2 max pooling, flatten, three dense."""
    g = GraphBuilder(seed)
    y = g.var("data", (batch, 3, size, size), 8)
    for n, c in [(2, 64), (2, 128), (4, 256), (4, 512), (4, 512)]:
        for _ in range(n):
            y = g.conv(y, c, 3, 1, 1)
        y = g.max_pool(y, 2, 2, 0)
    n_, c_, h_, w_ = g.shape_of(y)
    y = g.op("flatten", [y], (n_, c_ * h_ * w_))
    y = g.dense(y, fc, 0, True)
    y = g.dense(y, fc, 0, True)
    o = g.dense(y, classes)
    js, pb = g.finish(o)
    return js, pb, image_input(batch, size, input_seed)


SSD_ANCHORS = 64 * 64 * 4 + 32 * 32 * 6 + 16 * 16 * 6 + 8 * 8 * 6 + 4 * 4 * 6 + 2 * 2 * 4 + 4  # 24564


def ssd_boxes(batch, anchors=SSD_ANCHORS, seed=0, classes=21, image=512):
    """Synthetic detection rows [class id, score, x1, y1, x2, y2], int32."""
    rng = np.random.RandomState(seed)
    ids = rng.randint(0, classes, size=(batch, anchors))
    score = rng.randint(0, 1 << 15, size=(batch, anchors))
    x1 = rng.randint(0, image - 32, size=(batch, anchors))
    y1 = rng.randint(0, image - 32, size=(batch, anchors))
    w = rng.randint(1, 200, size=(batch, anchors))
    h = rng.randint(1, 200, size=(batch, anchors))
    x2 = np.minimum(x1 + w, image)
    y2 = np.minimum(y1 + h, image)
    return np.stack([ids, score, x1, y1, x2, y2], axis=-1).astype(np.int32)


def ssd_tail(batch=1, anchors=SSD_ANCHORS, score_threshold=1 << 14, iou_threshold=45, top_k=400,
             max_output_size=-1, force_suppress=False, seed=0):
    """C5 tail: get_valid_counts -> non_max_suppression over (batch, anchors, 6) int32 rows."""
    g = GraphBuilder(seed)
    d = g.var("data", (batch, anchors, 6), 16)
    vc, boxes = g.op("get_valid_counts", [d], [(batch,), (batch, anchors, 6)],
                     {"score_threshold": score_threshold})
    y = g.op("non_max_suppression", [boxes, vc], (batch, anchors, 6), {
        "iou_threshold": iou_threshold, "top_k": top_k, "max_output_size": max_output_size,
        "force_suppress": force_suppress, "id_index": 0, "score_index": 1, "coord_start": 2,
        "return_indices": False, "invalid_to_bottom": True})
    js, pb = g.finish(y)
    return js, pb, ssd_boxes(batch, anchors, seed)


def ssd_backbone(batch=1, seed=0, size=512, input_seed=7, classes=21):
    """C5 convolutional part: MobileNet-1.0 backbone at 512x512, four extra stride-2 stages, and a
    3x3 class head (A*classes channels) and box head (A*4) on each of the seven feature maps; the
    head outputs are flattened and concatenated into one (batch, total) tensor."""
    g = GraphBuilder(seed)
    x = g.var("data", (batch, 3, size, size), 8)
    y = g.conv(x, 32, 3, 2, 1)
    feats = []
    cfg = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2)] + [(512, 1)] * 5 + [(1024, 2), (1024, 1)]
    for idx, (oc, s) in enumerate(cfg):
        c = g.shape_of(y)[1]
        y = g.conv(y, c, 3, s, 1, groups=c)
        y = g.conv(y, oc, 1, 1, 0)
        if idx in (4, 10, 12):       # 64x64x256, 32x32x512, 16x16x1024
            feats.append(y)
    for oc in (512, 512, 256, 256):  # 8, 4, 2, 1
        y = g.conv(y, oc // 2, 1, 1, 0)
        y = g.conv(y, oc, 3, 2, 1)
        feats.append(y)
    outs = []
    for f, a in zip(feats, (4, 6, 6, 6, 6, 4, 4)):
        for ch in (a * classes, a * 4):
            hd = g.conv(f, ch, 3, 1, 1, relu=False)
            n_, c_, h_, w_ = g.shape_of(hd)
            outs.append(g.op("flatten", [hd], (n_, c_ * h_ * w_)))
    total = sum(g.shape_of(o)[1] for o in outs)
    y = g.op("concatenate", outs, (batch, total), {"axis": 1})
    js, pb = g.finish(y)
    return js, pb, image_input(batch, size, input_seed)


def ssd_full(batch=1, seed=0, size=128, input_seed=7, classes=8, score_threshold=20, iou_threshold=45,
             top_k=100):
    """Image to boxes in one graph (the C5 backbone and heads joined to the C5 tail): per feature map
    the class and box heads are transposed to channels-last, reshaped to (batch, anchors, .) and
    concatenated over the maps; score = max over the classes, a small class id from comparisons of
    class logits (there is no argmax operator), boxes = clip(anchor + (delta >> 2)); the rows
    [id, score, x1, y1, x2, y2] go through get_valid_counts and non_max_suppression."""
    g = GraphBuilder(seed)
    x = g.var("data", (batch, 3, size, size), 8)
    y = g.conv(x, 32, 3, 2, 1)
    feats = []
    cfg = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2)] + [(512, 1)] * 5 + [(1024, 2), (1024, 1)]
    for idx, (oc, s) in enumerate(cfg):
        c = g.shape_of(y)[1]
        y = g.conv(y, c, 3, s, 1, groups=c)
        y = g.conv(y, oc, 1, 1, 0)
        if idx in (4, 10, 12):
            feats.append(y)
    for oc in (512, 512, 256, 256):
        y = g.conv(y, oc // 2, 1, 1, 0)
        y = g.conv(y, oc, 3, 2, 1)
        feats.append(y)
    cls_parts, box_parts = [], []
    for f, a in zip(feats, (4, 6, 6, 6, 6, 4, 4)):
        for ch, last, parts in ((a * classes, classes, cls_parts), (a * 4, 4, box_parts)):
            hd = g.conv(f, ch, 3, 1, 1, relu=False)
            n_, c_, h_, w_ = g.shape_of(hd)
            t = g.op("transpose", [hd], (n_, h_, w_, c_), {"axes": (0, 2, 3, 1)})
            parts.append(g.op("reshape", [t], (n_, h_ * w_ * a, last), {"shape": (0, -1, last)}))
    total = sum(g.shape_of(o)[1] for o in cls_parts)
    cls = g.op("concatenate", cls_parts, (batch, total, classes), {"axis": 1})
    box = g.op("concatenate", box_parts, (batch, total, 4), {"axis": 1})
    score = g.op("max", [cls], (batch, total, 1), {"axis": (2,), "keepdims": True, "exclude": False})

    def column(k):
        return g.op("strided_slice", [cls], (batch, total, 1), {"begin": (0, 0, k), "end": (batch, total, k + 1)})
    c0, c1, c2 = column(0), column(1), column(2)
    gt1 = g.op("broadcast_greater", [c1, c0], (batch, total, 1))
    gt2 = g.op("broadcast_greater", [c2, c0], (batch, total, 1))
    cid = g.op("elemwise_add", [gt1, gt2], (batch, total, 1))
    rng = np.random.RandomState(seed + 1)
    ax = rng.randint(0, size - 40, size=(1, total, 1))
    ay = rng.randint(0, size - 40, size=(1, total, 1))
    aw = rng.randint(8, 40, size=(1, total, 1))
    ah = rng.randint(8, 40, size=(1, total, 1))
    anchors = np.concatenate([ax, ay, ax + aw, ay + ah], axis=2).astype(np.int32)
    anc = g.var("anchors", anchors.shape, 10, anchors)
    delta = g.op("cvm_right_shift", [box], (batch, total, 4), {"precision": 6, "shift_bit": 2})
    moved = g.op("broadcast_add", [delta, anc], (batch, total, 4))
    boxes = g.op("clip", [moved], (batch, total, 4), {"a_min": 0, "a_max": size})
    rows = g.op("concatenate", [cid, score, boxes], (batch, total, 6), {"axis": 2})
    vc, kept = g.op("get_valid_counts", [rows], [(batch,), (batch, total, 6)], {"score_threshold": score_threshold})
    out = g.op("non_max_suppression", [kept, vc], (batch, total, 6), {
        "iou_threshold": iou_threshold, "top_k": top_k, "max_output_size": -1, "force_suppress": False,
        "id_index": 0, "score_index": 1, "coord_start": 2, "return_indices": False, "invalid_to_bottom": True})
    js, pb = g.finish(out)
    return js, pb, image_input(batch, size, input_seed)


def conv_ops_per_image(graph_json):
    """2 * MACs of every conv2d (groups = 1 and grouped) and dense node, for one image."""
    gj = json.loads(graph_json)
    shapes = gj["attrs"]["shape"][1]
    row_ptr = gj["node_row_ptr"]
    total = 0
    for nid, nd in enumerate(gj["nodes"]):
        if nd["op"] == "null":
            continue
        fn = nd["attrs"]["func_name"]
        if fn in ("conv2d", "dense"):
            w = shapes[row_ptr[nd["inputs"][1][0]]]
            o = shapes[row_ptr[nid]]
            total += 2 * int(np.prod(o[1:])) * int(np.prod(w[1:]))
    return total
