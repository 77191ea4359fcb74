"""The numpy restatement (oracle/) against the reference's own CPU runtime: through the committed
fixtures everywhere, and directly when oracle/_ref has been built here."""
import hashlib

import numpy as np
import pytest

import cases

ALL = [("model", n) for n in cases.model_cases()] + [("op", n) for n in cases.op_cases()]


def _thunk(group, name):
    return (cases.model_cases() if group == "model" else cases.op_cases())[name]


@pytest.mark.parametrize("group,name", ALL)
def test_oracle_matches_golden(group, name, oracle, golden):
    js, pb, x = _thunk(group, name)()
    key = "%s/%s" % (group, name)
    shas = golden[key + "/sha"].tolist()
    got_sha = [hashlib.sha256(b).hexdigest() for b in (js, pb, np.ascontiguousarray(x).tobytes())]
    assert got_sha == shas, "case generator is not deterministic"
    out = oracle.run_model(js, pb, x)
    want = golden[key + "/out"]
    assert out.shape == want.shape
    assert np.array_equal(out, want)


def test_oracle_byte_widths(oracle, golden):
    for group, name in ALL:
        js, pb, x = _thunk(group, name)()
        it = oracle.Interpreter(js, pb)
        meta = golden["%s/%s/meta" % (group, name)]
        assert it.input_bytes() * x.size == meta[0], name
        assert len(golden["%s/%s/out" % (group, name)]) == meta[1], name


@pytest.mark.parametrize("name", ["conv_chain_s14", "ssd_tail_b2", "mobilenet_s64"])
def test_oracle_matches_reference_library(name, oracle):
    if not oracle.ref_lib.available():
        pytest.skip("oracle/_ref not built in this environment")
    js, pb, x = cases.model_cases()[name]()
    assert np.array_equal(oracle.run_model(js, pb, x), oracle.ref_lib.run_model(js, pb, x))


@pytest.mark.parametrize("name", ["conv_chain_b16", "ssd_tail_b64_t32600", "ssd_full_512_b1"])
def test_oracle_matches_fullsize_digest(name, oracle, golden_fullsize):
    """The numpy restatement against the reference's digests of the full-size configurations (the
    ones it finishes in seconds; the GPU suite checks all of them)."""
    js, pb, x = cases.fullsize_cases()[name]()
    want_sha, want_len, input_sha = golden_fullsize[name]
    assert hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest() == input_sha
    out = oracle.run_model(js, pb, x)
    assert out.nbytes == want_len and hashlib.sha256(out.tobytes()).hexdigest() == want_sha


def test_right_shift_corners(oracle):
    """Branch structure of cpu/ops/elemwise.cc:129-147 on hand-checked values."""
    f = oracle.cvm_oracle.cvm_right_shift
    x = np.array([255, -255, 128, -128, 127, 383, -384, (1 << 31) - 1, -(1 << 31) + 1])
    assert f(x, 1, 8).tolist() == [127, -127, 64, -64, 64, 127, -127, 127, -127]
    assert f(x, 8, 8).tolist() == [1, -1, 1, 0, 0, 1, -1, 127, -127]
    assert f(x, 31, 8).tolist() == [0, -1, 0, -1, 0, 0, -1, 0, -1]
    assert f(np.array([(1 << 31) - 1]), 24, 8).tolist() == [128]          # p + b = 32: no clip
    assert f(np.array([(1 << 31) - 1]), 1, 31).tolist() == [-(1 << 30)]   # int32 "+1" wraps
    assert f(x, 3, 1).tolist() == [0] * len(x)


def test_iou_values(oracle):
    iou = oracle.cvm_oracle.iou
    assert iou((0, 0, 10, 10), (0, 0, 10, 10)) == 100
    assert iou((0, 0, 10, 10), (5, 0, 15, 10)) == 33
    assert iou((0, 0, 10, 10), (10, 10, 20, 20)) == 0
    assert iou((0, 0, 0, 0), (0, 0, 0, 0)) == 0
