"""Parity of the CUDA path, through the C-ABI, against the oracle: bit-exact on every case.

Small cases are checked three ways (committed fixtures from the reference CPU runtime, the numpy
restatement, and the reference library itself when it travelled with the repository); full-size
configurations are checked through batch independence and other size-independent properties."""
import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu

MODELS = list(cases.model_cases())
OPS = list(cases.op_cases())


@pytest.mark.parametrize("name", MODELS)
def test_models_match_golden_and_oracle(name, gpu_run, oracle, golden):
    js, pb, x = cases.model_cases()[name]()
    got = gpu_run(js, pb, x)
    assert np.array_equal(got, golden["model/%s/out" % name]), "differs from the reference fixture"
    assert np.array_equal(got, oracle.run_model(js, pb, x)), "differs from the oracle"


@pytest.mark.parametrize("name", OPS)
def test_ops_match_golden_and_oracle(name, gpu_run, oracle, golden):
    js, pb, x = cases.op_cases()[name]()
    got = gpu_run(js, pb, x)
    assert np.array_equal(got, golden["op/%s/out" % name]), "differs from the reference fixture"
    assert np.array_equal(got, oracle.run_model(js, pb, x)), "differs from the oracle"


def test_queries_match_reference(rt, golden):
    for name in ("conv_chain_s14", "resnet50_s64", "ssd_tail_b2"):
        js, pb, x = cases.model_cases()[name]()
        meta = golden["model/%s/meta" % name]
        net = rt.CVMAPILoadModel(js, pb, 0)
        try:
            assert rt.CVMAPIGetInputLength(net) == meta[0]
            assert rt.CVMAPIGetOutputLength(net) == meta[1]
            assert rt.CVMAPIGetStorageSize(net) == meta[2]
            if meta[3] == 0:
                assert rt.CVMAPIGetGasFromModel(net) == meta[4]
            assert rt.CVMAPIGetVersion(net) == "cvm_1.0.0"
            assert rt.CVMAPIGetPreprocessMethod(net) == ""
            assert rt.CVMAPIGetInputTypeSize(net) in (1, 4)
        finally:
            rt.CVMAPIFreeModel(net)


@pytest.mark.parametrize("seed", [1, 2, 3])
@pytest.mark.parametrize("batch", [1, 5])
def test_conv_chain_seeds(seed, batch, gpu_run, oracle, wl):
    """Config 1 (64 -> 64 channels, 3x3, 56x56) over seeds and batch sizes."""
    js, pb, x = wl.conv_chain(batch=batch, seed=seed)
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))


def test_random_conv_shapes(gpu_run, oracle):
    """Random strides / dilations / paddings / channel counts, tensor-core and CUDA-core paths."""
    rng = np.random.RandomState(2024)
    for i in range(24):
        c = int(rng.choice([3, 8, 32, 64, 96, 128]))
        groups = 1 if rng.rand() < 0.7 else int(rng.choice([g for g in (2, 4, c) if c % g == 0]))
        oc = int(rng.choice([8, 16, 24, 32, 64, 136])) // groups * groups or groups
        k = int(rng.choice([1, 2, 3, 5]))
        dil = int(rng.choice([1, 1, 2]))
        stride = int(rng.choice([1, 1, 2, 3]))
        pad = int(rng.randint(0, k * dil // 2 + 1))
        h, w = int(rng.randint(6, 19)), int(rng.randint(6, 19))
        if dil * (k - 1) + 1 > min(h, w) + 2 * pad:
            continue
        js, pb, x = cases.conv_case(100 + i, int(rng.randint(1, 4)), c, h, w, oc, k, stride, pad, dil,
                                    groups=groups, bias=bool(rng.rand() < 0.7), shift=int(rng.randint(0, 12)),
                                    relu=bool(rng.rand() < 0.5))
        assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x)), (i, c, oc, k, stride, pad, dil, groups)


def test_random_bottlenecks(gpu_run, oracle, wl):
    """Residual bottleneck blocks on random shapes: 1x1 reduce, 3x3 (stride 1: spatial-patch TMA,
    stride 2: im2col-mode TMA), 1x1 expand fused with the join, identity or projection shortcut;
    odd spatial sizes and batches give partial tiles, small channel counts give several
    (tap, channel block) units per ring stage."""
    rng = np.random.RandomState(77)
    for i in range(14):
        mid = int(rng.choice([32, 64, 128]))
        out = mid * int(rng.choice([2, 4]))
        cin = out if rng.rand() < 0.4 else int(rng.choice([32, 64, 96, 256]))
        stride = 1 if cin == out and rng.rand() < 0.7 else int(rng.choice([1, 2]))
        batch = int(rng.randint(1, 10))
        h, w = int(rng.randint(5, 23)), int(rng.randint(5, 23))
        g = wl.GraphBuilder(300 + i)
        x = cases.rnd(rng, (batch, cin, h, w), 8)
        d = g.var("data", x.shape, 8)
        sc = d
        if cin != out or stride != 1:
            sc = g.conv(d, out, 1, stride, 0, relu=False)
        z = g.conv(d, mid, 1, 1, 0)
        z = g.conv(z, mid, 3, stride, 1)
        z = g.conv(z, out, 1, 1, 0, relu=False)
        a = g.op("elemwise_add", [z, sc] if rng.rand() < 0.5 else [sc, z], g.shape_of(z))
        if rng.rand() < 0.8:
            a = g.op("relu", [a], g.shape_of(a))
        y = g.op("cvm_clip", [a], g.shape_of(a), {"precision": int(rng.choice([8, 8, 7]))})
        js, pb = g.finish(y)
        assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x)), (i, cin, mid, out, stride, batch, h, w)


def test_random_halo_convolutions(gpu_run, oracle, wl):
    """3x3 stride-1 filters over 64 / 128 channels on random shapes: the halo form of the patch
    tile (8 x 16 pixel patches, partial at the right / bottom edges, one or two 64-channel blocks,
    32..128 output channels, padding 0..2), bare, with relu, and fused with a residual join."""
    rng = np.random.RandomState(91)
    for i in range(12):
        c = int(rng.choice([64, 128]))
        oc = int(rng.choice([32, 64, 96, 128]))
        pad = int(rng.choice([0, 1, 1, 2]))
        batch = int(rng.randint(1, 4))
        h, w = int(rng.randint(9, 61)), int(rng.randint(9, 61))
        g = wl.GraphBuilder(500 + i)
        x = cases.rnd(rng, (batch, c, h, w), 8)
        d = g.var("data", x.shape, 8)
        y = g.conv(d, oc, 3, 1, pad, relu=bool(rng.randint(2)), shift=int(rng.randint(7, 12)), bias=bool(rng.randint(3)))
        if pad == 1 and oc == c and rng.rand() < 0.7:
            y = g.op("elemwise_add", [y, d], g.shape_of(y))
            y = g.op("cvm_clip", [y], g.shape_of(y), {"precision": 8})
        js, pb = g.finish(y)
        assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x)), (i, c, oc, pad, batch, h, w)


def test_input_is_clamped_to_its_precision(gpu_run, oracle, wl):
    """graph_runtime.cc:379-386: -128 enters the network as -127."""
    js, pb, x = wl.conv_chain(batch=1, channels=32, size=8)
    x = x.copy()
    x.reshape(-1)[::7] = -128
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))


def test_postprocess_argmax(gpu_run, oracle, wl):
    g = wl.GraphBuilder(5)
    d = g.var("data", (6, 64), 8)
    y = g.dense(d, 40, shift=9)
    js, pb = g.finish(y, postprocess="argmax")
    x = np.random.RandomState(5).randint(-127, 128, size=(6, 64)).astype(np.int8)
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))


def test_multi_head_detection_interleave(gpu_run, oracle, wl):
    """model.cc:200-246: heads with equal row counts are interleaved row-wise."""
    g = wl.GraphBuilder(6)
    d = g.var("data", (4, 32), 8)
    a = g.dense(d, 8, shift=8)
    b = g.dense(d, 16)
    js, pb = g.finish([a, b], postprocess="detection")
    x = np.random.RandomState(6).randint(-127, 128, size=(4, 32)).astype(np.int8)
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))


def test_api_errors_on_a_loaded_model(rt, wl):
    import ctypes
    js, pb, x = wl.conv_chain(batch=1, channels=32, size=8)
    net = rt.CVMAPILoadModel(js, pb, 0)
    try:
        out = np.zeros(rt.CVMAPIGetOutputLength(net), np.uint8)
        lib = rt.lib()
        st = lib.CVMAPIInference(net, x.ctypes.data_as(ctypes.c_char_p), x.nbytes - 1, out.ctypes.data_as(ctypes.c_char_p))
        assert st == rt.ERROR_LOGIC          # wrong input length, model.cc:155
        assert lib.CVMAPIInference(net, None, x.nbytes, out.ctypes.data_as(ctypes.c_char_p)) == rt.ERROR_RUNTIME
        assert lib.CVMAPIInference(net, x.ctypes.data_as(ctypes.c_char_p), x.nbytes, out.ctypes.data_as(ctypes.c_char_p)) == 0
    finally:
        rt.CVMAPIFreeModel(net)
    with pytest.raises(rt.CVMError) as e:
        rt.CVMAPILoadModel(js, pb, 99)       # no such GPU
    assert e.value.status == rt.ERROR_RUNTIME


def test_accepted_variants_load(rt, golden_status):
    for name in ("version_1_1_0_ok", "version_1_1_0_no_tables", "postprocess_argmax_ok"):
        js, pb = cases.malformed_cases()[name]
        net = rt.CVMAPILoadModel(js, pb, 0)
        rt.CVMAPIFreeModel(net)


def test_fuzzed_models_accepted_like_the_reference(rt, golden_fuzz):
    """Mutants the reference loads: same load status, same inference status, same output bytes."""
    import ctypes
    import hashlib
    import fuzz_cases
    table = fuzz_cases.fuzz_cases()
    names = list(table)
    assert names == golden_fuzz["names"].tolist()
    wrong = []
    ran = 0
    for i, name in enumerate(names):
        if int(golden_fuzz["load"][i]) != 0:
            continue
        js, pb, x, desc = table[name]
        net = ctypes.c_void_p()
        st = rt.lib().CVMAPILoadModel(js, len(js), pb, len(pb), ctypes.byref(net), 1, 0)
        if st != 0:
            if not (st == rt.ERROR_LOGIC and fuzz_cases.is_documented_refusal(rt.last_error())):
                wrong.append((name, desc, "load", st, rt.last_error()))
            continue
        try:
            if x is None:
                continue
            n_out = ctypes.c_ulonglong()
            rt.lib().CVMAPIGetOutputLength(net, ctypes.byref(n_out))
            out = np.zeros(n_out.value, np.uint8)
            xc = np.ascontiguousarray(x)
            ist = rt.lib().CVMAPIInference(net, xc.ctypes.data_as(ctypes.c_char_p), ctypes.c_int(xc.nbytes),
                                           out.ctypes.data_as(ctypes.c_char_p))
            want = int(golden_fuzz["infer"][i])
            if ist != want:
                wrong.append((name, desc, "infer status", want, ist))
            elif want == 0:
                ran += 1
                digest = "%s:%d" % (hashlib.sha256(out.tobytes()).hexdigest(), out.nbytes)
                if digest != str(golden_fuzz["out_sha"][i]):
                    wrong.append((name, desc, "output differs"))
        finally:
            rt.lib().CVMAPIFreeModel(net)
    assert ran >= 250
    assert not wrong, wrong


def test_random_graphs_match_the_reference(rt, golden_random):
    """Random operator graphs (tests/random_graphs.py): load status, inference status and output
    bytes as the reference's CPU runtime gave them."""
    import ctypes
    import hashlib
    import random_graphs
    table = random_graphs.random_cases()
    names = list(table)
    assert names == golden_random["names"].tolist()
    wrong = []
    ran = 0
    for i, name in enumerate(names):
        want_load = int(golden_random["load"][i])
        if want_load not in (0, 1, 2):
            continue
        js, pb, x = table[name]()
        net = ctypes.c_void_p()
        st = rt.lib().CVMAPILoadModel(js, len(js), pb, len(pb), ctypes.byref(net), 1, 0)
        if st != want_load:
            wrong.append((name, "load", want_load, st, rt.last_error()))
        if st != 0:
            continue
        try:
            n_out = ctypes.c_ulonglong()
            rt.lib().CVMAPIGetOutputLength(net, ctypes.byref(n_out))
            out = np.zeros(n_out.value, np.uint8)
            ist = rt.lib().CVMAPIInference(net, x.ctypes.data_as(ctypes.c_char_p), ctypes.c_int(x.nbytes),
                                           out.ctypes.data_as(ctypes.c_char_p))
            want = int(golden_random["infer"][i])
            if ist != want:
                wrong.append((name, "infer status", want, ist, rt.last_error()))
            elif want == 0:
                ran += 1
                digest = "%s:%d" % (hashlib.sha256(out.tobytes()).hexdigest(), out.nbytes)
                if digest != str(golden_random["out_sha"][i]):
                    wrong.append((name, "output differs"))
        finally:
            rt.lib().CVMAPIFreeModel(net)
    assert ran >= 700
    assert not wrong, wrong


# ---------------------------------------------------------------------------------------------
# full-size configurations: SHA-256 of the reference CPU runtime's own output
# ---------------------------------------------------------------------------------------------
FULLSIZE = list(cases.fullsize_cases())


@pytest.mark.parametrize("name", FULLSIZE)
def test_fullsize_matches_reference_digest(name, gpu_run, golden_fullsize):
    """The benchmark configurations at their real sizes (512 x 512 SSD graphs, 24564-anchor tails at
    batch 64, ResNet-50 / MobileNet batch 32, VGG-19 batch 4): the bytes CVMAPIInference returns
    hash to what the reference CPU runtime returned for the same model and input."""
    import hashlib
    js, pb, x = cases.fullsize_cases()[name]()
    want_sha, want_len, input_sha = golden_fullsize[name]
    assert hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest() == input_sha, "the seeded input changed"
    got = gpu_run(js, pb, x)
    assert got.nbytes == want_len
    assert hashlib.sha256(got.tobytes()).hexdigest() == want_sha, "differs from the reference's output"


# ---------------------------------------------------------------------------------------------
# full-size configurations: size-independent properties
# ---------------------------------------------------------------------------------------------
def test_resnet50_batch256_batch_independence(rt, gpu_run, oracle, wl):
    """ResNet-50 at the benchmark batch: image i of the batch-256 run equals the same image run in
    a batch of 4, and that small batch equals the oracle."""
    js, pb, x = wl.resnet50(batch=256)
    big = gpu_run(js, pb, x).view(np.int32).reshape(256, 1000)
    js4, pb4, _ = wl.resnet50(batch=4)
    for lo in (0, 124, 252):
        small = gpu_run(js4, pb4, x[lo:lo + 4]).view(np.int32).reshape(4, 1000)
        assert np.array_equal(big[lo:lo + 4], small)
    assert np.array_equal(gpu_run(js4, pb4, x[:4]), oracle.run_model(js4, pb4, x[:4]))
    # replays are deterministic, also dozens of them back to back from a pageable and from a
    # page-locked buffer (the per-chunk kernels of the leading operators then follow one another as
    # closely as they ever do: this is where a missing ordering between the roles of a kernel shows)
    import torch
    net = rt.CVMAPILoadModel(js, pb, 0)
    try:
        a = rt.inference_bytes(net, x).copy()
        b = rt.inference_bytes(net, x).copy()
        assert np.array_equal(a, b) and np.array_equal(a.view(np.int32).reshape(256, 1000), big)
        out = np.empty_like(a)
        flat = np.ascontiguousarray(x).reshape(-1).view(np.uint8)
        pinned = torch.empty(flat.size, dtype=torch.uint8, pin_memory=True)
        pinned.numpy()[:] = flat
        for src in (flat.copy(), pinned.numpy()):
            for _ in range(30):
                rt.inference_bytes(net, src, out)
            assert np.array_equal(out, a)
    finally:
        rt.CVMAPIFreeModel(net)


def test_chunked_prefix_matches_oracle(gpu_run, oracle, wl):
    """Batch 8 divides into four chunks: the stem, the pooling and the first bottleneck blocks run
    chunk by chunk (upload / compute overlap) before the rest of the network runs on the batch."""
    js, pb, x = wl.resnet50(batch=8, size=64)
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))
    js, pb, x = wl.vgg19(batch=8, size=32, fc=64)
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))


@pytest.mark.parametrize("builder,batch,small", [("mobilenet_v1", 64, 2), ("vgg19", 16, 1)])
def test_large_batch_matches_small_batches(builder, batch, small, gpu_run, oracle, wl):
    js, pb, x = getattr(wl, builder)(batch=batch)
    big = gpu_run(js, pb, x).view(np.int32).reshape(batch, 1000)
    jss, pbs, _ = getattr(wl, builder)(batch=small)
    for lo in (0, batch - small):
        got = gpu_run(jss, pbs, x[lo:lo + small])
        assert np.array_equal(big[lo:lo + small], got.view(np.int32).reshape(small, 1000))
    assert np.array_equal(gpu_run(jss, pbs, x[:small]), oracle.run_model(jss, pbs, x[:small]))


def test_ssd_tail_full_size_properties(gpu_run, wl):
    """24564 anchors, batch 64: per image the kept rows are sorted by score, come from the input,
    respect top_k, are padded with -1, and running NMS on its own output changes nothing."""
    b, n = 64, wl.SSD_ANCHORS
    js, pb, x = wl.ssd_tail(batch=b)
    y = gpu_run(js, pb, x).view(np.int32).reshape(b, n, 6)
    for i in (0, 31, 63):
        kept = y[i][y[i, :, 0] >= 0]
        assert 0 < len(kept) <= 400
        assert np.all(y[i, len(kept):] == -1)
        assert np.all(np.diff(kept[:, 1]) <= 0)
        rows = {tuple(r) for r in x[i].tolist()}
        assert all(tuple(r) in rows for r in kept.tolist())
        assert kept[:, 1].min() > (1 << 14)
    again = gpu_run(js, pb, np.where(y < 0, 0, y).astype(np.int32)).view(np.int32).reshape(b, n, 6)
    for i in (0, 63):
        k0 = y[i][y[i, :, 0] >= 0]
        k1 = again[i][again[i, :, 0] >= 0]
        assert np.array_equal(k0, k1)


def test_ssd_tail_full_size_against_oracle_batch1(gpu_run, oracle, wl):
    js, pb, x = wl.ssd_tail(batch=1)
    assert np.array_equal(gpu_run(js, pb, x), oracle.run_model(js, pb, x))


def test_sharded_model_equals_single_handle(pkg, gpu_run, wl):
    """ShardedModel over one GPU used twice: same bytes as one handle holding the whole batch."""
    build = lambda b: wl.mobilenet_v1(batch=b, size=64)
    js, pb, x = build(6)
    whole = gpu_run(js, pb, x)
    sm = pkg.sharding.ShardedModel(build, 6, [0, 0])
    try:
        assert np.array_equal(sm.infer(x), whole)
    finally:
        sm.free()


def test_activation_memory_is_planned_by_lifetime(rt, wl, oracle):
    """Buffers that are never live together share physical memory (the result is checked against
    the oracle like every other case, here once more on the handle whose memory is inspected), and
    what the handle reports is what it holds."""
    js, pb, x = wl.mobilenet_v1(batch=16, size=160)
    net = rt.CVMAPILoadModel(js, pb, 0)
    try:
        buffers, physical = rt.activation_bytes(net)
        assert buffers > 0, "the planner did not run"
        assert 0 < physical < buffers
        assert physical % (2 << 20) == 0            # whole 2 MiB chunks
        assert rt.device_bytes(net) >= physical
        got = rt.inference_bytes(net, x)
        assert np.array_equal(got, oracle.run_model(js, pb, x))
        assert np.array_equal(got, rt.inference_bytes(net, x)), "second run on the shared memory differs"
    finally:
        rt.CVMAPIFreeModel(net)
