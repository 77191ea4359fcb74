"""The allocation-free NMS entry point (cvmk_non_max_suppression_static) against the regular one.

Callers that may not allocate device memory (inside a stream capture, in a loop that must never
synchronise, or under a fixed memory budget) use the variant whose scratch is a fixed array inside
the library.  It must give exactly the bytes of cvmk_non_max_suppression, call after call, even
though every call reuses the same scratch and finds the previous call's data in it, and both must
give the bytes of the CPU oracle.  This file is
collected last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


class NmsDesc(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("valid_count", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("B", ctypes.c_int32), ("N", ctypes.c_int32), ("max_output_size", ctypes.c_int32),
                ("iou_threshold", ctypes.c_int32), ("top_k", ctypes.c_int32), ("force_suppress", ctypes.c_int32),
                ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_int64),
                ("x_writeback", ctypes.c_void_p)]


def _rows(batch, n, seed):
    rows = cases.wl.ssd_boxes(batch, n, seed, classes=5, image=128)
    vc = np.random.RandomState(seed).randint(n // 2, n + 1, size=(batch,)).astype(np.int32)
    return rows, vc


def test_static_scratch_matches_regular_entry_point(rt, oracle):
    """Several calls in a row through the C-ABI, each finding the previous call's scratch: the
    static-scratch entry point returns the bytes of the regular entry point and of the CPU oracle
    (cpu/ops/nms.cc:65-140 restated in numpy).  The calls also cover the corner rules through the
    shared array: forced suppression across classes, rows with a negative class id (they end the
    scan), an image without valid rows (it ends the whole call: later images keep what the output
    buffer held), top_k = 0."""
    import torch
    lib = rt.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    #        batch  n    seed top_k  max_out force  special
    calls = [(3,    900,  11, 300,   -1,     0,     None),
             (2,    1400, 12, -1,    25,     0,     None),
             (3,    900,  13, 300,   -1,     1,     "negative_ids"),
             (3,    700,  14, 200,   -1,     0,     "empty_image"),
             (2,    500,  15, 0,     -1,     0,     None),
             (3,    900,  11, 300,   -1,     0,     None)]
    for call, (batch, n, seed, top_k, mos, force, special) in enumerate(calls):
        rows, vc = _rows(batch, n, seed)
        if special == "negative_ids":
            rng = np.random.RandomState(seed)
            rows[:, rng.randint(0, n, size=12), 0] = -1
        if special == "empty_image":
            vc[1] = 0           # image 1 has no valid rows: the call ends there, image 2 is not touched
        x = torch.from_numpy(rows).to(dev)
        v = torch.from_numpy(vc).to(dev)
        y_ref = torch.full_like(x, 7)
        y_new = torch.full_like(x, 7)
        need = lib.cvmk_nms_scratch_bytes(batch, n)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        d = NmsDesc(x.data_ptr(), v.data_ptr(), y_ref.data_ptr(), batch, n, mos, 40, top_k, force,
                    scratch.data_ptr(), need)
        assert lib.cvmk_non_max_suppression(ctypes.byref(d), stream) == 0, lib.cvmk_last_error()
        rc = lib.cvmk_non_max_suppression_static(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(v.data_ptr()),
                                                 ctypes.c_void_p(y_new.data_ptr()), batch, n, mos, 40, top_k, force, stream)
        assert rc == 0, lib.cvmk_last_error()
        torch.cuda.synchronize()
        a, b = y_ref.cpu().numpy(), y_new.cpu().numpy()
        assert np.array_equal(a, b), "call %d differs from the regular entry point" % call   # integer output: exact
        want = oracle.cvm_oracle.non_max_suppression(rows, vc, 40, top_k, mos, bool(force),
                                                     y_init=np.full_like(rows, 7))
        assert np.array_equal(b, want), "call %d differs from the CPU oracle" % call
        assert np.array_equal(x.cpu().numpy(), rows), "the static variant never writes into its input"
        if special is None and top_k != 0:
            assert (b[:, :, 0] >= 0).any()


def test_static_scratch_refuses_oversized_problems(rt):
    import torch
    lib = rt.lib()
    torch.cuda.set_device(0)
    batch, n = 64, cases.wl.SSD_ANCHORS          # needs 37.7 MB of scratch, the array holds 8 MiB
    assert lib.cvmk_nms_scratch_bytes(batch, n) > (8 << 20)
    x = torch.zeros((1, 8, 6), dtype=torch.int32, device="cuda")
    rc = lib.cvmk_non_max_suppression_static(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                             ctypes.c_void_p(x.data_ptr()), batch, n, -1, 45, 400, 0, None)
    assert rc == 1
    assert b"needs" in lib.cvmk_last_error()
    torch.cuda.synchronize()
