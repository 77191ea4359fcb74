"""ctypes driver of the UNMODIFIED reference CPU runtime built by oracle/Makefile into
oracle/_ref/libcvm_runtime_ref.so.  TEST INFRASTRUCTURE ONLY: used to pin the numpy restatement,
to generate the fixtures under tests/golden/, and as the timed CPU baseline of bench.py.
It drives the reference through its own C-ABI (src/core/c_api.cc), device_type 0 = CPU backend,
2 = formal backend.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(HERE, "_ref", "libcvm_runtime_ref.so")
_LIB = None


def available():
    return os.path.exists(REF_LIB)


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(REF_LIB)
    return _LIB


class RefModel:
    """One model loaded into the reference runtime."""

    def __init__(self, graph_json, params_blob, device_type=0):
        self.net = ctypes.c_void_p()
        self.status = lib().CVMAPILoadModel(graph_json, len(graph_json), params_blob, len(params_blob),
                                            ctypes.byref(self.net), device_type, 0)
        self.loaded = self.status == 0

    def _ull(self, name):
        v = ctypes.c_ulonglong()
        st = getattr(lib(), name)(self.net, ctypes.byref(v))
        return st, v.value

    def input_length(self):
        return self._ull("CVMAPIGetInputLength")[1]

    def output_length(self):
        return self._ull("CVMAPIGetOutputLength")[1]

    def storage_size(self):
        return self._ull("CVMAPIGetStorageSize")[1]

    def gas(self):
        return self._ull("CVMAPIGetGasFromModel")

    def infer(self, data):
        """Returns (status, output bytes as uint8)."""
        data = np.ascontiguousarray(data)
        out = np.zeros(self.output_length(), np.uint8)
        st = lib().CVMAPIInference(self.net, data.ctypes.data_as(ctypes.c_char_p), ctypes.c_int(data.nbytes),
                                   out.ctypes.data_as(ctypes.c_char_p))
        return st, out

    def free(self):
        if self.loaded:
            lib().CVMAPIFreeModel(self.net)
            self.loaded = False


def run_model(graph_json, params_blob, data, device_type=0):
    m = RefModel(graph_json, params_blob, device_type)
    if not m.loaded:
        raise RuntimeError("reference refused the model (status %d)" % m.status)
    st, out = m.infer(data)
    m.free()
    if st != 0:
        raise RuntimeError("reference inference failed (status %d)" % st)
    return out
