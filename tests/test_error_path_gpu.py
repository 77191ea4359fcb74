"""The bounded-wait error path, end to end, without making any kernel fail.

Every spin in the tensor-core kernels is a bounded mbarrier wait: when it runs out the CTA raises a
flag, its roles leave their loops, the kernel ORs a code into the model's status word and returns;
CVMAPIInference then answers ERROR_RUNTIME.  Two halves are exercised here: the device half with a
kernel whose only job is to wait on a barrier that nothing arrives at (a short limit, so the wait
gives up after a fraction of a millisecond and the kernel returns normally), and the host half by
writing a status word the way such a kernel would.
"""
import ctypes

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports(rt):
    word, clocks = rt.wait_timeout(64)
    assert word == (0x100 | 5)          # what a convolution kernel would have ORed into its status word
    assert 0 < clocks < 2_000_000_000   # it did wait, and for a bounded time (64 polls of about 2 us)
    longer, clocks2 = rt.wait_timeout(512)
    assert longer == word and clocks2 > clocks
    # the context is intact: ordinary work still runs
    js, pb, x = cases.model_cases()["conv_chain_s14"]()
    net = rt.CVMAPILoadModel(js, pb, 0)
    try:
        rt.inference_bytes(net, x)
    finally:
        rt.CVMAPIFreeModel(net)


def test_status_word_becomes_error_runtime_and_handle_stays_usable(rt, golden):
    js, pb, x = cases.model_cases()["conv_chain_s14"]()
    net = rt.CVMAPILoadModel(js, pb, 0)
    try:
        want = golden["model/conv_chain_s14/out"]
        assert np.array_equal(rt.inference_bytes(net, x), want)
        rt.set_status_word(net, 0x103)
        out = np.zeros(rt.CVMAPIGetOutputLength(net), np.uint8)
        arr = np.ascontiguousarray(x)
        st = rt.lib().CVMAPIInference(net, arr.ctypes.data_as(ctypes.c_char_p), ctypes.c_int(arr.nbytes),
                                      out.ctypes.data_as(ctypes.c_char_p))
        assert st == rt.ERROR_RUNTIME
        assert "wait ran out" in rt.last_error()
        # the word was cleared: the same handle answers correctly again
        assert np.array_equal(rt.inference_bytes(net, x), want)
    finally:
        rt.CVMAPIFreeModel(net)
