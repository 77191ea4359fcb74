"""Seeded parity cases shared by the golden-fixture generator and the tests.

Every case is (graph_json, params_blob, input ndarray).  Single-operator graphs follow the
reference's op-level harness (tests/test_op.cc:478-661: attributes + inputs -> outputs, including
expected failures); model cases follow its model-level harness (tests/test_model.cc:94-235).
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

pkg = ge.load_package()
wl = pkg.workloads


def single_op(func, data, data_prec, attrs, out_shapes, params=(), seed=0, head=None, data_pos=0):
    """Graph `data (+ params) -> func -> heads`.  `params` is a list of (ndarray, precision);
    `head` selects one output of a multi-output operator; `data_pos` is the position of the
    runtime input among the operator's inputs."""
    g = wl.GraphBuilder(seed)
    ins = []
    for i, (arr, prec) in enumerate(params):
        ins.append(g.var("p%d" % i, arr.shape, prec, arr))
    ins.insert(data_pos, g.var("data", data.shape, data_prec))
    out = g.op(func, ins, out_shapes, attrs)
    heads = out if isinstance(out, list) else [out]
    if head is not None:
        heads = [heads[head]]
    js, pb = g.finish(heads)
    return js, pb, data


def rnd(rng, shape, prec):
    a = (1 << (prec - 1)) - 1
    arr = rng.randint(-a, a + 1, size=shape)
    return arr.astype(np.int8 if prec <= 8 else np.int32)


def conv_case(seed, n, c, h, w, oc, k, stride=1, pad=0, dil=1, groups=1, bias=True, shift=None, relu=False):
    rng = np.random.RandomState(seed)
    g = wl.GraphBuilder(seed)
    x = rnd(rng, (n, c, h, w), 8)
    d = g.var("data", x.shape, 8)
    y = g.conv(d, oc, k, stride, pad, groups=groups, relu=relu, shift=shift if shift else 0, dilation=dil, bias=bias)
    js, pb = g.finish(y)
    return js, pb, x


def nms_writeback_case():
    """non_max_suppression overwrites the rows of its INPUT outside the top_k (cpu/ops/nms.cc:93-97).
    Here that input is read three times: by a cvm_clip before the operator (which must see the rows
    as they were, although its only consumer -- an elemwise_add with the operator's output -- comes
    after it, so a fused clip+add would run too late), by the operator, and by an elemwise_add after
    it (which must see the overwritten rows)."""
    b, n = 2, 120
    g = wl.GraphBuilder(0)
    d = g.var("data", (b, n, 6), 16)
    vc, boxes = g.op("get_valid_counts", [d], [(b,), (b, n, 6)], {"score_threshold": 1 << 13})
    c = g.op("cvm_clip", [boxes], (b, n, 6), {"precision": 10})
    y = g.op("non_max_suppression", [boxes, vc], (b, n, 6), {
        "iou_threshold": 45, "top_k": 12, "max_output_size": -1, "force_suppress": False, "id_index": 0,
        "score_index": 1, "coord_start": 2, "return_indices": False, "invalid_to_bottom": True})
    s1 = g.op("elemwise_add", [c, y], (b, n, 6), {})
    s2 = g.op("elemwise_add", [s1, boxes], (b, n, 6), {})
    js, pb = g.finish(s2)
    return js, pb, wl.ssd_boxes(b, n, 3, classes=4, image=128)


def model_cases():
    """name -> thunk; small enough for the CPU oracle to finish in seconds."""
    return {
        "nms_input_writeback_order": nms_writeback_case,
        "conv_chain_s14": lambda: wl.conv_chain(batch=1, channels=32, size=14),
        "conv_chain_b3": lambda: wl.conv_chain(batch=3, channels=64, size=20),
        "resnet50_s64": lambda: wl.resnet50(batch=1, size=64),
        "mobilenet_s64": lambda: wl.mobilenet_v1(batch=2, size=64),
        "vgg19_s32": lambda: wl.vgg19(batch=2, size=32, fc=64),
        "ssd_backbone_s128": lambda: wl.ssd_backbone(batch=1, size=128),
        "ssd_full_s128": lambda: wl.ssd_full(batch=2, size=128),
        "ssd_tail_b2": lambda: wl.ssd_tail(batch=2, anchors=600, top_k=50),
        "ssd_tail_mos": lambda: wl.ssd_tail(batch=2, anchors=500, top_k=-1, max_output_size=20),
        "ssd_tail_force": lambda: wl.ssd_tail(batch=1, anchors=700, top_k=200, force_suppress=True, score_threshold=100),
        "ssd_tail_none_valid": lambda: wl.ssd_tail(batch=1, anchors=300, top_k=10, score_threshold=1 << 15),
    }


def fullsize_cases():
    """The benchmark configurations at (or near) their real sizes.  Too large for byte fixtures: the
    golden file keeps the SHA-256 and the length of the reference CPU runtime's output."""
    return {
        "conv_chain_b16": lambda: wl.conv_chain(batch=16),
        "resnet50_b32": lambda: wl.resnet50(batch=32),
        "mobilenet_b32": lambda: wl.mobilenet_v1(batch=32),
        "vgg19_b4": lambda: wl.vgg19(batch=4),
        "ssd_tail_b64_t16384": lambda: wl.ssd_tail(batch=64),
        "ssd_tail_b64_t100": lambda: wl.ssd_tail(batch=64, score_threshold=100),
        # fewer valid rows than top_k (about 125 of 24564 score above 32600)
        "ssd_tail_b64_t32600": lambda: wl.ssd_tail(batch=64, score_threshold=32600),
        # no top_k limit: every valid row (about half of them) goes through the suppression sweep
        "ssd_tail_b4_all_rows": lambda: wl.ssd_tail(batch=4, top_k=-1),
        "ssd_tail_b4_force_out100": lambda: wl.ssd_tail(batch=4, top_k=2000, max_output_size=100, force_suppress=True),
        "ssd_backbone_512_b1": lambda: wl.ssd_backbone(batch=1),
        "ssd_full_512_b1": lambda: wl.ssd_full(batch=1, size=512, classes=21),
        "ssd_full_512_b2": lambda: wl.ssd_full(batch=2, size=512, classes=21),
    }


def op_cases():
    """name -> thunk for single-operator graphs, edge cases included."""
    c = {}
    r = np.random.RandomState(1234)

    def add(name, thunk):
        c[name] = thunk

    # conv2d: tensor-core shapes, strides, dilation, padding, odd channel counts, groups
    add("conv_tc_3x3", lambda: conv_case(1, 2, 32, 9, 11, 64, 3, 1, 1, shift=9))
    add("conv_tc_1x1_s2", lambda: conv_case(2, 3, 64, 10, 10, 32, 1, 2, 0, shift=8))
    add("conv_tc_dil2", lambda: conv_case(3, 1, 32, 12, 12, 48, 3, 1, 2, dil=2, shift=9))
    add("conv_tc_5x5_s2_nobias", lambda: conv_case(4, 2, 32, 13, 13, 40, 5, 2, 2, bias=False, shift=10))
    add("conv_tc_int32_out", lambda: conv_case(5, 1, 64, 6, 6, 24, 3, 1, 1, shift=0))
    add("conv_stem_7x7", lambda: conv_case(6, 2, 3, 30, 30, 16, 7, 2, 3, shift=8, relu=True))
    # image stems on the tensor cores (1..4 input channels, 32/64/128 output channels)
    add("conv_stem_fused_7x7_s2", lambda: conv_case(30, 2, 3, 32, 32, 64, 7, 2, 3, shift=8, relu=True))
    add("conv_stem_fused_3x3_s2_oc32", lambda: conv_case(31, 3, 3, 33, 30, 32, 3, 2, 1, shift=7, relu=True))
    add("conv_stem_fused_3x3_s1_oc128", lambda: conv_case(32, 1, 3, 17, 48, 128, 3, 1, 1, shift=7))
    add("conv_stem_fused_wide_row", lambda: conv_case(33, 1, 1, 6, 300, 32, 5, 1, 2, shift=6, relu=True))
    add("conv_stem_fused_4ch_nobias", lambda: conv_case(34, 2, 4, 20, 16, 64, 5, 2, 0, bias=False, shift=8))
    add("conv_stem_fused_1x1", lambda: conv_case(35, 2, 2, 9, 16, 32, 1, 1, 0, shift=3))
    add("conv_stem_fused_s3_rows", lambda: conv_case(36, 1, 3, 37, 32, 64, 7, 3, 2, shift=8, relu=True))
    # more stems for the folded-stride kernel: odd heights, one and two channels, the widest filter,
    # an input row wider than one TMA box (two boxes of 144 columns)
    add("conv_stem_fused_3x3_s2_odd_h", lambda: conv_case(37, 3, 3, 37, 64, 32, 3, 2, 1, shift=7, relu=True))
    add("conv_stem_fused_5x5_s1_2ch", lambda: conv_case(38, 2, 2, 19, 32, 64, 5, 1, 2, shift=8))
    add("conv_stem_fused_8x8_s2_1ch", lambda: conv_case(39, 2, 1, 40, 48, 32, 8, 2, 3, shift=8, relu=True))
    add("conv_stem_fused_7x7_s2_two_boxes", lambda: conv_case(40, 1, 3, 21, 288, 64, 7, 2, 3, shift=9, relu=True))
    add("conv_stem_fused_4x4_s1_pad0", lambda: conv_case(41, 2, 4, 12, 16, 128, 4, 1, 0, shift=8))
    # 3x3 over 128 -> 128 channels: both channel blocks of the weights resident in shared memory
    add("conv_halo_resident_128", lambda: conv_case(42, 2, 128, 20, 24, 128, 3, 1, 1, shift=10, relu=True))
    # depthwise 3x3 over an image wide enough that a band of rows needs more than 48 KB of shared memory
    add("depthwise_3x3_wide_band", lambda: conv_case(43, 1, 32, 9, 256, 32, 3, 1, 1, groups=32, shift=6, relu=True))
    add("depthwise_3x3_s2_wide_band", lambda: conv_case(44, 1, 64, 11, 192, 64, 3, 2, 1, groups=64, shift=6))
    # depthwise 3x3 stride 1 over more shapes: ragged 28 x 28 images, a wide 32-channel image, four
    # channel blocks without bias, no padding, 96 = 3 x 32 channels, 1024 channels; and an ordinary
    # 32 -> 64 channel layer whose image is whole 8 x 16 pixel patches
    add("depthwise_3x3_64ch_28x28", lambda: conv_case(45, 2, 64, 28, 28, 64, 3, 1, 1, groups=64, shift=6, relu=True))
    add("depthwise_3x3_32ch_32x40", lambda: conv_case(46, 1, 32, 32, 40, 32, 3, 1, 1, groups=32, shift=6))
    add("depthwise_3x3_256ch_nobias", lambda: conv_case(47, 3, 256, 14, 14, 256, 3, 1, 1, groups=256, bias=False, shift=5))
    add("depthwise_3x3_pad0", lambda: conv_case(48, 1, 128, 18, 18, 128, 3, 1, 0, groups=128, shift=6))
    add("depthwise_3x3_96ch", lambda: conv_case(49, 2, 96, 16, 16, 96, 3, 1, 1, groups=96, shift=6, relu=True))
    add("depthwise_3x3_1024ch", lambda: conv_case(50, 1, 1024, 16, 16, 1024, 3, 1, 1, groups=1024, shift=6, relu=True))
    # (128 channels and more run on the tensor cores as groups of 32 channels: ragged patches, three N tiles)
    add("depthwise_3x3_128ch_28x28", lambda: conv_case(52, 2, 128, 28, 28, 128, 3, 1, 1, groups=128, shift=6, relu=True))
    add("depthwise_3x3_384ch", lambda: conv_case(53, 1, 384, 16, 24, 384, 3, 1, 1, groups=384, shift=6))
    add("conv_tc_3x3_32ch_patches", lambda: conv_case(51, 2, 32, 16, 24, 64, 3, 1, 1, shift=9, relu=True))
    # narrow 1x1 layers, which the executor runs with 4 or 2 neighbouring pixels folded into the
    # channels (block-diagonal weights): 32 -> 64 (fold 4), 64 -> 64 with int32 output and a pixel
    # count that only 2 divides, 25 pixels (no fold), 64 -> 128 without bias (fold 2)
    add("conv_1x1_fold4", lambda: conv_case(54, 2, 32, 12, 10, 64, 1, 1, 0, shift=7, relu=True))
    add("conv_1x1_fold2_int32", lambda: conv_case(55, 1, 64, 9, 6, 64, 1, 1, 0, shift=0))
    add("conv_1x1_odd_pixels", lambda: conv_case(56, 1, 32, 5, 5, 32, 1, 1, 0, shift=6))
    add("conv_1x1_fold2_nobias", lambda: conv_case(57, 2, 64, 8, 8, 128, 1, 1, 0, bias=False, shift=7))
    # batch 8: the inference uploads the batch in four chunks and runs the stem per chunk
    add("conv_stem_fused_b8_chunked", lambda: conv_case(38, 8, 3, 20, 16, 32, 3, 2, 1, shift=7, relu=True))
    def stem_generic():
        rng = np.random.RandomState(37)
        g = wl.GraphBuilder(37)
        x = rnd(rng, (2, 3, 18, 32), 8)
        d = g.var("data", x.shape, 8)
        y = g.conv(d, 64, 3, 1, 1, relu=True, shift=7)
        y = g.op("cvm_clip", [y], g.shape_of(y), {"precision": 6})
        y = g.op("negative", [y], g.shape_of(y))
        js, pb = g.finish(y)
        return js, pb, x
    add("conv_stem_fused_generic_chain", stem_generic)
    def head_transpose(pool_after):
        # conv -> transpose(0, 2, 3, 1) -> reshape, as detection heads do (the transpose of a
        # channels-last buffer is an alias), and the same transpose read by max_pool2d (a real copy)
        def f():
            rng = np.random.RandomState(58)
            g = wl.GraphBuilder(58)
            x = rnd(rng, (2, 32, 6, 10), 8)
            d = g.var("data", x.shape, 8)
            y = g.conv(d, 48, 3, 1, 1, relu=False, shift=8)
            t = g.op("transpose", [y], (2, 6, 10, 48), {"axes": (0, 2, 3, 1)})
            if pool_after:
                t = g.op("max_pool2d", [t], (2, 6, 5, 24), {"pool_size": (2, 2), "strides": (2, 2), "padding": (0, 0), "ceil_mode": False})
                r = g.op("reshape", [t], (2, 720), {"shape": (2, 720)})
            else:
                r = g.op("reshape", [t], (2, 60, 48), {"shape": (2, 60, 48)})
            js, pb = g.finish(r)
            return js, pb, x
        return f
    add("head_transpose_reshape", head_transpose(False))
    add("head_transpose_pool", head_transpose(True))
    add("conv_odd_channels", lambda: conv_case(7, 1, 5, 8, 8, 7, 3, 1, 1, shift=7))
    add("conv_depthwise", lambda: conv_case(8, 2, 32, 10, 10, 32, 3, 1, 1, groups=32, shift=6, relu=True))
    add("conv_depthwise_s2", lambda: conv_case(9, 1, 48, 9, 9, 48, 3, 2, 1, groups=48, shift=6))
    add("conv_grouped", lambda: conv_case(10, 1, 12, 7, 7, 8, 3, 1, 0, groups=4, shift=7))

    def join_case(seed, sub, relu, clip_attrs, other_first=False, oc=64):
        """conv -> cvm_right_shift -> elemwise add/sub with a second int8 tensor -> [relu] -> clip:
        the residual join that the executor folds into the convolution."""
        def f():
            rng = np.random.RandomState(seed)
            g = wl.GraphBuilder(seed)
            x = rnd(rng, (2, 32, 9, 7), 8)
            d = g.var("data", x.shape, 8)
            y = g.conv(d, oc, 3, 1, 1, relu=False, shift=9)
            other = g.var("res", g.shape_of(y), 8, rnd(rng, g.shape_of(y), 8))
            ins = [other, y] if other_first else [y, other]
            z = g.op("elemwise_sub" if sub else "elemwise_add", ins, g.shape_of(y))
            if relu:
                z = g.op("relu", [z], g.shape_of(z))
            z = g.op(clip_attrs[0], [z], g.shape_of(z), clip_attrs[1])
            js, pb = g.finish(z)
            return js, pb, x
        return f
    add("conv_join_add_relu_clip", join_case(13, False, True, ("cvm_clip", {"precision": 8})))
    add("conv_join_sub_clip", join_case(14, True, False, ("clip", {"a_min": -100, "a_max": 90})))
    add("conv_join_rsub_clip", join_case(15, True, False, ("cvm_clip", {"precision": 7}), other_first=True))
    add("conv_join_add_oc48", join_case(16, False, True, ("cvm_clip", {"precision": 8}), oc=48))

    # 3x3 stride-1 filters over 64 / 128 channels: the M tile is an 8 x 16 pixel patch whose input
    # halo is staged once per 64-channel block (partial patches at the right / bottom edges, one
    # and two channel blocks, both output widths, padding 0 and 2, relu, residual join)
    add("conv_halo_c64_56", lambda: conv_case(40, 2, 64, 56, 56, 64, 3, 1, 1, shift=9, relu=True))
    add("conv_halo_c128_28", lambda: conv_case(41, 3, 128, 28, 28, 128, 3, 1, 1, shift=10))
    add("conv_halo_c64_oc128_edges", lambda: conv_case(42, 2, 64, 37, 27, 128, 3, 1, 1, shift=9, relu=True))
    add("conv_halo_c128_oc32_pad0", lambda: conv_case(43, 1, 128, 34, 42, 32, 3, 1, 0, shift=10, bias=False))
    add("conv_halo_c64_pad2", lambda: conv_case(44, 2, 64, 30, 30, 64, 3, 1, 2, shift=9))

    # output channel counts that are not a multiple of 8 (detection heads): tensor-core kernel on
    # channels padded to 32, real channels copied out; int32 and int8 outputs
    add("conv_tc_oc126_int32", lambda: conv_case(46, 2, 64, 9, 11, 126, 3, 1, 1, shift=0))
    add("conv_tc_oc84_shift", lambda: conv_case(47, 3, 96, 7, 5, 84, 3, 1, 1, shift=9, relu=True))
    add("conv_tc_oc21_1x1", lambda: conv_case(48, 2, 32, 6, 6, 21, 1, 1, 0, shift=7, bias=False))

    def halo_join():
        rng = np.random.RandomState(45)
        g = wl.GraphBuilder(45)
        x = rnd(rng, (2, 64, 40, 48), 8)
        d = g.var("data", x.shape, 8)
        y = g.conv(d, 64, 3, 1, 1, relu=False, shift=9)
        z = g.op("elemwise_add", [y, d], g.shape_of(y))
        z = g.op("relu", [z], g.shape_of(z))
        z = g.op("cvm_clip", [z], g.shape_of(z), {"precision": 8})
        js, pb = g.finish(z)
        return js, pb, x
    add("conv_halo_join", halo_join)

    def dense_case(seed, m, k, units, bias=True):
        def f():
            g = wl.GraphBuilder(seed)
            x = rnd(np.random.RandomState(seed), (m, k), 8)
            d = g.var("data", x.shape, 8)
            y = g.dense(d, units, bias=bias)
            js, pb = g.finish(y)
            return js, pb, x
        return f
    add("dense_tc", dense_case(11, 5, 64, 24))
    add("dense_odd", dense_case(12, 3, 50, 10, bias=False))

    # dense layers of a few rows over a long reduction: cut along K into tiles of their own,
    # partial sums added by a second kernel that also applies the chain
    def dense_long_k(seed, m, k, units, second=None, relu=True):
        def f():
            g = wl.GraphBuilder(seed)
            x = rnd(np.random.RandomState(seed), (m, k), 8)
            d = g.var("data", x.shape, 8)
            y = g.dense(d, units, shift=0, relu=relu)
            if second:
                y = g.dense(y, second)          # int32 head straight from the sums
            js, pb = g.finish(y)
            return js, pb, x
        return f
    add("dense_k_slices_int8", dense_long_k(13, 7, 4096, 512))
    add("dense_k_slices_chain", dense_long_k(14, 33, 2048, 1024, second=256, relu=False))
    add("dense_k_slices_head", lambda: (lambda g, x: (lambda d: g.finish(g.dense(d, 256)) + (x,))(g.var("data", x.shape, 8)))(
        wl.GraphBuilder(15), rnd(np.random.RandomState(15), (4, 3072), 8)))

    def unary(func, attrs, prec=16, shape=(2, 3, 5, 7), seed=20, special=None):
        def f():
            rng = np.random.RandomState(seed)
            x = rnd(rng, shape, prec)
            if special is not None:
                flat = x.reshape(-1)
                flat[:len(special)] = special
            return single_op(func, x, prec, attrs, [list(shape)])
        return f
    big = [(1 << 31) - 1, -(1 << 31) + 1, 0, 1, -1, 255, -256, 1 << 30]
    add("relu", unary("relu", None))
    add("abs", unary("abs", None, prec=32, special=big))
    add("negative", unary("negative", None, prec=32, special=big))
    add("cvm_precision", unary("cvm_precision", None, prec=32, special=big))
    add("clip", unary("clip", {"a_min": -100, "a_max": 77}))
    add("clip_wide", unary("clip", {"a_min": -100000, "a_max": 5}, prec=32, special=big))
    add("cvm_clip_8", unary("cvm_clip", {"precision": 8}))
    add("cvm_clip_1", unary("cvm_clip", {"precision": 1}))
    add("cvm_clip_20", unary("cvm_clip", {"precision": 20}, prec=32, special=big))
    add("rshift_8_8", unary("cvm_right_shift", {"precision": 8, "shift_bit": 8}, prec=24))
    add("rshift_1_8", unary("cvm_right_shift", {"precision": 8, "shift_bit": 1}, prec=32, special=big))
    add("rshift_p1", unary("cvm_right_shift", {"precision": 1, "shift_bit": 3}, prec=32, special=big))
    add("rshift_b31", unary("cvm_right_shift", {"precision": 8, "shift_bit": 31}, prec=32, special=big))
    add("rshift_b32", unary("cvm_right_shift", {"precision": 8, "shift_bit": 32}, prec=32, special=big))
    add("rshift_noclip", unary("cvm_right_shift", {"precision": 8, "shift_bit": 24}, prec=32, special=big))
    add("rshift_noclip_b1", unary("cvm_right_shift", {"precision": 31, "shift_bit": 1}, prec=32, special=big))
    add("rshift_16_5", unary("cvm_right_shift", {"precision": 16, "shift_bit": 5}, prec=32, special=big))

    def binary(func, shape_a, shape_b, out_shape, pa=8, pb_=8, seed=30, zero_b=False):
        def f():
            rng = np.random.RandomState(seed)
            a = rnd(rng, shape_a, pa)
            b = rnd(rng, shape_b, pb_)
            if zero_b:
                b.reshape(-1)[::3] = 0
            return single_op(func, a, pa, None, [list(out_shape)], params=[(b, pb_)])
        return f
    add("elemwise_add", binary("elemwise_add", (2, 4, 3, 5), (2, 4, 3, 5), (2, 4, 3, 5), 16, 16))
    add("elemwise_sub", binary("elemwise_sub", (3, 7), (3, 7), (3, 7), 30, 30))
    for op in ("add", "sub", "mul", "max", "div", "greater"):
        add("broadcast_%s_scalar" % op, binary("broadcast_" + op, (2, 3, 4, 5), (1,), (2, 3, 4, 5), 12, 12, zero_b=False))
        add("broadcast_%s_chan" % op, binary("broadcast_" + op, (2, 6, 4, 5), (6, 1, 1), (2, 6, 4, 5), 12, 12, zero_b=(op == "div")))
        add("broadcast_%s_nd" % op, binary("broadcast_" + op, (3, 1, 5), (2, 1, 4, 1), (2, 3, 4, 5), 10, 10, zero_b=(op == "div")))
    add("broadcast_div_zero_scalar", lambda: single_op(
        "broadcast_div", rnd(np.random.RandomState(3), (4, 5), 16), 16, None, [[4, 5]],
        params=[(np.zeros((1,), np.int32), 16)]))

    def pool(seed, shape, k, s, p, ceil=False, prec=8, pad1=False):
        def f():
            rng = np.random.RandomState(seed)
            x = rnd(rng, shape, prec)
            n, ch, h, w = shape
            if ceil:
                oh, ow = -(-(h + 2 * p - k) // s) + 1, -(-(w + 2 * p - k) // s) + 1
            else:
                oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
            attrs = {"pool_size": (k, k), "strides": (s, s), "padding": (p,) if pad1 else (p, p), "ceil_mode": ceil}
            return single_op("max_pool2d", x, prec, attrs, [[n, ch, oh, ow]])
        return f
    add("max_pool_3x3_s2", pool(40, (2, 16, 11, 11), 3, 2, 1))
    add("max_pool_2x2", pool(41, (1, 5, 8, 6), 2, 2, 0))
    add("max_pool_ceil", pool(42, (1, 16, 10, 10), 3, 2, 0, ceil=True))
    add("max_pool_int32", pool(43, (1, 4, 9, 9), 3, 1, 1, prec=20, pad1=True))
    # channel-vector forms: 2x2 stride 2, 3x3 stride 1 with padding, 3x3 stride 2 over odd sizes,
    # 2x2 in ceil mode (the last window reaches past the image)
    add("max_pool_2x2_vec", pool(44, (2, 32, 12, 10), 2, 2, 0))
    add("max_pool_3x3_s1_vec", pool(45, (1, 32, 7, 9), 3, 1, 1))
    add("max_pool_3x3_s2_odd_vec", pool(46, (2, 64, 13, 15), 3, 2, 1))
    add("max_pool_2x2_ceil_vec", pool(47, (1, 16, 9, 7), 2, 2, 0, ceil=True))

    add("upsampling", lambda: single_op("upsampling", rnd(np.random.RandomState(50), (2, 16, 4, 5), 8), 8,
                                        {"scale": 2}, [[2, 16, 8, 10]]))
    add("upsampling_x3_int32", lambda: single_op("upsampling", rnd(np.random.RandomState(51), (1, 3, 3, 2), 20), 20,
                                                 {"scale": 3}, [[1, 3, 9, 6]]))

    def concat(seed, shapes, axis, prec=8):
        def f():
            rng = np.random.RandomState(seed)
            arrs = [rnd(rng, s, prec) for s in shapes]
            out = list(shapes[0])
            ax = axis if axis >= 0 else axis + len(out)
            out[ax] = sum(s[ax] for s in shapes)
            return single_op("concatenate", arrs[0], prec, {"axis": axis}, [out],
                             params=[(a, prec) for a in arrs[1:]])
        return f
    add("concat_channels", concat(60, [(2, 16, 4, 4), (2, 32, 4, 4), (2, 16, 4, 4)], 1))
    add("concat_anchor_axis", concat(61, [(2, 10, 6), (2, 7, 6)], 1, prec=16))
    add("concat_last_neg", concat(62, [(3, 4, 2), (3, 4, 5)], -1, prec=12))
    add("concat_h", concat(63, [(1, 3, 4, 5), (1, 3, 2, 5)], 2))

    def red(func, seed, shape, axis, keepdims=False, exclude=False, prec=8, out=None):
        def f():
            rng = np.random.RandomState(seed)
            x = rnd(rng, shape, prec)
            nd = len(shape)
            ax = sorted(a + nd if a < 0 else a for a in axis)
            real = ax if not exclude else [i for i in range(nd) if i not in ax]
            if not ax and not exclude:
                real = list(range(nd))
            if len(real) == nd:
                oshape = [1] * nd if keepdims else [1]
            elif not real:
                oshape = list(shape)
            elif keepdims:
                oshape = [1 if i in real else shape[i] for i in range(nd)]
            else:
                oshape = [shape[i] for i in range(nd) if i not in real]
            return single_op(func, x, prec, {"axis": tuple(axis), "keepdims": keepdims, "exclude": exclude}, [oshape])
        return f
    add("sum_hw", red("sum", 70, (2, 32, 7, 7), (2, 3)))
    add("sum_hw_keep", red("sum", 71, (2, 16, 3, 3), (2, 3), keepdims=True))
    add("sum_all", red("sum", 72, (3, 4, 5), ()))
    add("max_all_negative", lambda: single_op("max", -np.abs(rnd(np.random.RandomState(73), (4, 6), 8)) - 1, 8,
                                              {"axis": (), "keepdims": False, "exclude": False}, [[1]]))
    add("max_axis1", red("max", 74, (3, 5, 4), (1,)))
    add("sum_exclude", red("sum", 75, (2, 3, 4, 5), (1,), exclude=True))
    add("sum_channel_keep", red("sum", 76, (2, 6, 4, 4), (1,), keepdims=True))
    add("sum_size1_quirk", red("sum", 77, (3, 2, 1), (1,)))       # cpu index-map quirk, reduce.cc:66-89
    add("max_axes_neg", red("max", 78, (2, 3, 4), (-1, 0)))

    def reshape_like(func, seed, shape, attrs, out, prec=8):
        def f():
            return single_op(func, rnd(np.random.RandomState(seed), shape, prec), prec, attrs, [out])
        return f
    add("flatten_4d", reshape_like("flatten", 80, (2, 16, 3, 5), None, [2, 240]))
    add("reshape_4d_to_3d", reshape_like("reshape", 81, (2, 8, 3, 5), {"shape": (0, -1, 5)}, [2, 24, 5]))
    add("reshape_2d_to_4d", reshape_like("reshape", 82, (2, 60), {"shape": (2, 4, 3, 5)}, [2, 4, 3, 5]))
    add("expand_dims", reshape_like("expand_dims", 83, (3, 4), {"axis": 1, "num_newaxis": 2}, [3, 1, 1, 4], prec=12))
    add("squeeze", reshape_like("squeeze", 84, (3, 1, 4, 1), {"axis": (1, 3)}, [3, 4], prec=12))

    # index-map transforms, take / cvm_lut, where
    def xform(func, seed, shape, attrs, out, prec=8):
        def f():
            return single_op(func, rnd(np.random.RandomState(seed), shape, prec), prec, attrs, [out])
        return f
    add("transpose_default", xform("transpose", 110, (3, 4, 5), None, [5, 4, 3], prec=12))
    add("transpose_nchw_to_nhwc", xform("transpose", 111, (2, 16, 3, 5), {"axes": (0, 2, 3, 1)}, [2, 3, 5, 16]))
    add("transpose_120", xform("transpose", 112, (4, 3, 6), {"axes": (1, 2, 0)}, [3, 6, 4], prec=16))
    add("transpose_neg_axes", xform("transpose", 113, (2, 3, 4, 5), {"axes": (-1, 0, -2, 1)}, [5, 2, 4, 3]))
    add("transpose_2d", xform("transpose", 114, (7, 33), {"axes": (1, 0)}, [33, 7], prec=20))
    add("transpose_6d", xform("transpose", 115, (2, 3, 2, 3, 2, 3), {"axes": (5, 3, 1, 4, 2, 0)}, [3, 3, 3, 2, 2, 2]))
    add("strided_slice_basic", xform("strided_slice", 120, (3, 8, 6), {"begin": (0, 1), "end": (2, 7), "stride": (1, 2)}, [2, 3, 6], prec=12))
    add("strided_slice_neg_stride", xform("strided_slice", 121, (5, 9), {"begin": (4, -1), "end": (0, 2), "stride": (-2, -3)}, [2, 2], prec=16))
    add("strided_slice_neg_begin_4d", xform("strided_slice", 122, (2, 8, 6, 6), {"begin": (0, -6, 1, 0), "end": (2, 8, 5, 6)}, [2, 6, 4, 6]))
    add("strided_slice_clamped", xform("strided_slice", 123, (6, 5), {"begin": (-100, 2), "end": (100, 100)}, [6, 3], prec=10))
    add("strided_slice_anchor_cols", xform("strided_slice", 124, (2, 50, 6), {"begin": (0, 0, 2), "end": (2, 50, 6)}, [2, 50, 4], prec=16))

    def slice_like(seed, shape, like, axis, out, prec=8):
        def f():
            rng = np.random.RandomState(seed)
            attrs = {"axis": axis} if axis is not None else None
            return single_op("slice_like", rnd(rng, shape, prec), prec, attrs, [out],
                             params=[(rnd(rng, like, 8), 8)])
        return f
    add("slice_like_all", slice_like(130, (4, 6, 5), (2, 6, 3), None, [2, 6, 3], prec=12))
    add("slice_like_axes", slice_like(131, (2, 16, 7, 9), (2, 3, 5, 6), (2, 3), [2, 16, 5, 6]))
    add("slice_like_neg_axis", slice_like(132, (3, 10), (7, 4), (-1,), [3, 4], prec=16))
    add("repeat_axis0", xform("repeat", 140, (3, 4), {"repeats": 2, "axis": 0}, [6, 4], prec=12))
    add("repeat_channels", xform("repeat", 141, (2, 8, 3, 3), {"repeats": 3, "axis": 1}, [2, 24, 3, 3]))
    add("repeat_last_neg", xform("repeat", 142, (2, 3, 5), {"repeats": 4, "axis": -1}, [2, 3, 20], prec=16))
    add("tile_same_rank", xform("tile", 150, (2, 3), {"reps": (2, 3)}, [4, 9], prec=12))
    add("tile_more_reps", xform("tile", 151, (3, 2), {"reps": (2, 1, 2)}, [2, 3, 4], prec=16))
    add("tile_fewer_reps", xform("tile", 152, (2, 4, 3, 5), {"reps": (2, 2)}, [2, 4, 6, 10]))
    add("tile_6d", xform("tile", 153, (2, 1, 3, 2, 1, 2), {"reps": (2, 2, 1, 2, 3, 2)}, [4, 2, 3, 4, 3, 4]))

    def take(seed, shape, idx_shape, axis, out, prec=8, idx_range=None, data_is_index=False):
        def f():
            rng = np.random.RandomState(seed)
            x = rnd(rng, shape, prec)
            n = int(np.prod(shape)) if axis is None else shape[axis]
            lo, hi = idx_range if idx_range else (-3, n + 3)   # out-of-range indices are clamped
            idx = rng.randint(lo, hi, size=idx_shape).astype(np.int32)
            attrs = {"axis": axis} if axis is not None else None
            if data_is_index:
                return single_op("take", idx, 16, attrs, [out], params=[(x, prec)], data_pos=1)
            return single_op("take", x, prec, attrs, [out], params=[(idx, 16)])
        return f
    add("take_flat", take(160, (4, 5, 3), (7, 2), None, [7, 2], prec=12))
    add("take_axis0_embedding", take(161, (50, 16), (3, 9), 0, [3, 9, 16], data_is_index=True))
    add("take_axis1", take(162, (3, 6, 4), (5,), 1, [3, 5, 4], prec=16))
    add("take_axis_neg_4d", take(163, (2, 8, 3, 5), (2, 2), -1, [2, 8, 3, 2, 2]))
    add("take_axis2_4d_out", take(164, (2, 8, 7), (3, 5), 2, [2, 8, 3, 5]))

    def lut(seed, shape, in_dim, table_prec, idx_prec):
        def f():
            rng = np.random.RandomState(seed)
            table = rnd(rng, (in_dim,), table_prec)
            a = (1 << (idx_prec - 1)) - 1
            idx = rng.randint(-2 if idx_prec > 8 else -a, a + 1, size=shape).astype(np.int8 if idx_prec <= 8 else np.int32)
            return single_op("cvm_lut", idx, idx_prec, {"in_dim": in_dim}, [list(shape)], params=[(table, table_prec)])
        return f
    add("cvm_lut_int8_index", lut(170, (2, 16, 5, 5), 100, 16, 8))
    add("cvm_lut_wide_index", lut(171, (3, 40), 300, 8, 10))

    def where(seed, shape, rows, cond_is_data=True, prec=8):
        def f():
            rng = np.random.RandomState(seed)
            cshape = (shape[0],) if rows else shape
            cond = (rng.randint(0, 3, size=cshape) - 1).astype(np.int8)   # -1, 0, 1
            x, y = rnd(rng, shape, prec), rnd(rng, shape, prec)
            if cond_is_data:
                return single_op("where", cond, 8, None, [list(shape)], params=[(x, prec), (y, prec)])
            return single_op("where", x, prec, None, [list(shape)], params=[(cond, 8), (y, prec)], data_pos=1)
        return f
    add("where_elementwise", where(180, (2, 16, 3, 5), False))
    add("where_elementwise_int32", where(181, (6, 7), False, cond_is_data=False, prec=20))
    add("where_1d", where(182, (9,), False, prec=16))

    def gvc(seed, b, n, k, thr, head=1):
        def f():
            rng = np.random.RandomState(seed)
            x = rng.randint(-50, 1000, size=(b, n, k)).astype(np.int32)
            return single_op("get_valid_counts", x, 16, {"score_threshold": thr}, [[b], [b, n, k]], head=head)
        return f
    add("gvc_k6", gvc(90, 3, 257, 6, 400))
    add("gvc_k6_count", gvc(90, 3, 257, 6, 400, head=0))
    add("gvc_k5_all", gvc(91, 2, 40, 5, -100))
    add("gvc_none", gvc(92, 2, 33, 6, 5000))
    add("gvc_big", gvc(93, 2, 3000, 6, 300))

    def nms_direct(seed, b, n, vcs, **kw):
        """non_max_suppression fed by parameters, so valid_count and ids can be arbitrary."""
        def f():
            rng = np.random.RandomState(seed)
            rows = wl.ssd_boxes(b, n, seed, classes=4, image=64)
            if kw.pop("neg_ids", False):
                rows[:, ::5, 0] = -1
            if kw.pop("ties", False):
                rows[:, :, 1] = rng.randint(0, 6, size=(b, n))
            g = wl.GraphBuilder(seed)
            d = g.var("data", rows.shape, 16)
            vc = g.var("vc", (b,), 16, np.array(vcs, np.int32))
            attrs = {"iou_threshold": 30, "top_k": -1, "max_output_size": -1, "force_suppress": False,
                     "id_index": 0, "score_index": 1, "coord_start": 2, "return_indices": False,
                     "invalid_to_bottom": True}
            attrs.update(kw)
            y = g.op("non_max_suppression", [d, vc], rows.shape, attrs)
            js, pb = g.finish(y)
            return js, pb, rows
        return f
    add("nms_basic", nms_direct(100, 2, 300, [300, 150]))
    add("nms_neg_ids", nms_direct(101, 2, 200, [200, 120], neg_ids=True))
    add("nms_neg_ids_force", nms_direct(102, 1, 200, [180], neg_ids=True, force_suppress=True))
    add("nms_ties_topk", nms_direct(103, 2, 700, [700, 650], ties=True, top_k=600))
    add("nms_topk0", nms_direct(104, 1, 50, [40], top_k=0))
    add("nms_mos", nms_direct(105, 2, 120, [100, 120], max_output_size=7, iou_threshold=60))
    add("nms_vc_over_n", nms_direct(106, 1, 64, [1000], iou_threshold=101))
    add("nms_large_block", nms_direct(107, 1, 1300, [1300], iou_threshold=70))
    return c


def malformed_cases():
    """name -> (graph_json, params_blob): models the loader must refuse, with the reference's
    status class.  Derived from the conv chain by editing its JSON."""
    js, pb, _ = wl.conv_chain(batch=1, channels=32, size=8)
    base = json.loads(js)
    out = {}

    def mut(name, fn, params=pb):
        g = json.loads(json.dumps(base))
        fn(g)
        out[name] = (json.dumps(g).encode(), params)

    out["not_json"] = (b"{nodes: [", pb)
    mut("unknown_top_key", lambda g: g.update({"bogus": 1}))
    mut("missing_heads", lambda g: g.pop("heads"))
    mut("unknown_op", lambda g: g["nodes"][3]["attrs"].update({"func_name": "conv3d"}))
    mut("bad_op_type", lambda g: g["nodes"][3].update({"op": "tvm_op"}))
    mut("unknown_attr", lambda g: g["attrs"]["op_attrs"][1].__setitem__(4, json.dumps({"precision": "8", "shift_bit": "8", "foo": "1"})))
    mut("missing_required_attr", lambda g: g["attrs"]["op_attrs"][1].__setitem__(4, json.dumps({"precision": "8"})))
    mut("bad_int_attr", lambda g: g["attrs"]["op_attrs"][1].__setitem__(5, json.dumps({"precision": "eight"})))
    mut("attrs_on_plain_op", lambda g: g["attrs"]["op_attrs"][1].__setitem__(0, "{}") or g["nodes"][5]["attrs"].update({"func_name": "relu"}))
    mut("wrong_num_inputs", lambda g: g["nodes"][3]["inputs"].pop())
    mut("storage_alias_conv", lambda g: g["attrs"]["storage_id"][1].__setitem__(3, 0))
    mut("negative_storage_id", lambda g: g["attrs"]["storage_id"][1].__setitem__(4, -1))
    mut("shape_too_many_dims", lambda g: g["attrs"]["shape"][1].__setitem__(2, [1] * 7))
    mut("wrong_output_shape", lambda g: g["attrs"]["shape"][1].__setitem__(3, [1, 32, 9, 8]))
    mut("wrong_bias_shape", lambda g: g["attrs"]["shape"][1].__setitem__(2, [31]))
    mut("precision_too_big", lambda g: g["attrs"]["precision"][1].__setitem__(0, 33))
    mut("input_precision_9", lambda g: g["attrs"]["precision"][1].__setitem__(0, 9))
    mut("variable_without_precision", lambda g: g["attrs"]["precision"][1].__setitem__(1, -1))
    mut("device_index_set", lambda g: g["attrs"].update({"device_index": ["list_int", [0] * 6]}))
    mut("dltype_int8", lambda g: g["attrs"]["dltype"][1].__setitem__(0, "int8"))
    mut("bad_row_ptr", lambda g: g["node_row_ptr"].__setitem__(2, 5))
    mut("bad_arg_nodes", lambda g: g.update({"arg_nodes": [0, 1]}))
    mut("version_unknown", lambda g: g.update({"version": "cvm_2.0.0"}))
    mut("not_topological", lambda g: g["nodes"][3]["inputs"].__setitem__(0, [4, 0, 0]))
    mut("duplicate_names", lambda g: g["nodes"][1].update({"name": "data"}))
    mut("shift_bit_0", lambda g: g["attrs"]["op_attrs"][1].__setitem__(4, json.dumps({"precision": "8", "shift_bit": "0"})))
    mut("kernel_exceeds_input", lambda g: (g["attrs"]["op_attrs"][1].__setitem__(3, g["attrs"]["op_attrs"][1][3].replace('"[3, 3]"', '"[30, 30]"'))))
    mut("params_missing", lambda g: None, params=wl.params_blob({}))
    mut("params_bad_magic", lambda g: None, params=b"\x00" * 64)
    big = np.full((32,), 1 << 20, np.int32)
    w = np.zeros((32, 32, 3, 3), np.int8)
    mut("param_out_of_range", lambda g: None, params=wl.params_blob({"w": w, "b": big}))
    mut("param_wrong_shape", lambda g: None, params=wl.params_blob({"w": w[:, :, :2], "b": big // 8192}))
    mut("param_unknown_name", lambda g: None, params=wl.params_blob({"w": w, "b": big // 8192, "zz": w}))
    mut("version_1_1_0_ok", lambda g: g.update({"version": "cvm_1.1.0"}))
    # cvm_1.1.0 recomputes both tables; the reference indexes the missing one before that and
    # crashes, so this case has no golden status (recorded as -11).
    mut("version_1_1_0_no_tables", lambda g: (g.update({"version": "cvm_1.1.0"}), g.pop("node_row_ptr"), g.pop("arg_nodes")))
    mut("postprocess_argmax_ok", lambda g: g.update({"postprocess": "argmax"}))

    # transform operators with attributes or shapes their shape inference refuses
    def bad_op(name, func, shape, attrs, out_shape, params=(), prec=8):
        j, p, _ = single_op(func, np.zeros(shape, np.int8), prec, attrs, [out_shape], params=params)
        out[name] = (j, p)
    bad_op("transpose_repeated_axis", "transpose", (2, 3, 4), {"axes": (0, 1, 1)}, [2, 3, 3])
    bad_op("transpose_axis_count", "transpose", (2, 3, 4), {"axes": (1, 0)}, [3, 2, 4])
    bad_op("transpose_wrong_out_shape", "transpose", (2, 3, 4), {"axes": (2, 0, 1)}, [4, 3, 2])
    bad_op("tile_zero_rep", "tile", (2, 3), {"reps": (2, 0)}, [4, 3])
    bad_op("tile_default_reps", "tile", (2, 3), None, [2, 3])
    bad_op("repeat_zero", "repeat", (2, 3), {"repeats": 0, "axis": 0}, [2, 3])
    bad_op("repeat_bad_axis", "repeat", (2, 3), {"repeats": 2, "axis": 2}, [2, 3])
    bad_op("repeat_missing_repeats", "repeat", (2, 3), {"axis": 0}, [2, 3])
    bad_op("strided_slice_empty", "strided_slice", (4, 5), {"begin": (2, 0), "end": (2, 5)}, [1, 5])
    bad_op("strided_slice_zero_stride", "strided_slice", (4, 5), {"begin": (0, 0), "end": (2, 5), "stride": (1, 0)}, [2, 5])
    bad_op("strided_slice_wrong_direction", "strided_slice", (4, 5), {"begin": (0,), "end": (3,), "stride": (-1,)}, [3, 5])
    bad_op("slice_like_exceeds", "slice_like", (2, 3), None, [4, 3], params=[(np.zeros((4, 3), np.int8), 8)])
    bad_op("slice_like_rank_mismatch", "slice_like", (2, 3, 4), None, [2, 3, 4], params=[(np.zeros((2, 3), np.int8), 8)])
    bad_op("slice_like_bad_axis", "slice_like", (2, 3, 4), {"axis": (2,)}, [2, 3, 4], params=[(np.zeros((2, 3), np.int8), 8)])
    bad_op("take_bad_axis", "take", (3, 4), {"axis": 2}, [3, 2], params=[(np.zeros((2,), np.int32), 16)])
    bad_op("take_axis_not_int", "take", (3, 4), {"axis": "x"}, [3, 2], params=[(np.zeros((2,), np.int32), 16)])
    bad_op("cvm_lut_in_dim_mismatch", "cvm_lut", (3, 4), {"in_dim": 9}, [3, 4], params=[(np.zeros((10,), np.int8), 8)])
    bad_op("where_xy_mismatch", "where", (3, 4), None, [3, 4],
           params=[(np.zeros((3, 4), np.int8), 8), (np.zeros((3, 5), np.int8), 8)])
    bad_op("where_cond_rows_mismatch", "where", (2,), None, [3, 4],
           params=[(np.zeros((3, 4), np.int8), 8), (np.zeros((3, 4), np.int8), 8)])
    return out
