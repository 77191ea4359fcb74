"""ctypes binding of libcvm_runtime.so, mirroring the reference's Python binding
(python/cvm/_ctypes/runtime.py:12-159): same function names, same argument meaning, a raised
error for every non-zero status.  The library is loaded from this directory; there is no
fallback when it (or a GPU) is missing.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcvm_runtime.so")
MEASURE_LIB_PATH = os.path.join(HERE, "libcvm_measure.so")
MEASURE_SYMBOLS = ["cvmk_measure_i8_mma_rate", "cvmk_measure_i8_mma_rate_window", "cvmk_measure_wait_timeout",
                   "cvmk_measure_last_error"]

SUCCEED, ERROR_LOGIC, ERROR_RUNTIME = 0, 1, 2

API_SYMBOLS = [
    "CVMAPILoadModel", "CVMAPIFreeModel", "CVMAPIInference", "CVMAPIGetVersion",
    "CVMAPIGetPreprocessMethod", "CVMAPIGetInputLength", "CVMAPIGetOutputLength",
    "CVMAPIGetInputTypeSize", "CVMAPIGetOutputTypeSize", "CVMAPIGetStorageSize",
    "CVMAPIGetGasFromModel", "CVMAPIGetGasFromGraphFile",
]
KERNEL_SYMBOLS = [
    "cvmk_im2col_pack", "cvmk_stem_pack", "cvmk_stem_pack_supported",
    "cvmk_conv2d_stem_supported", "cvmk_conv2d_stem_weight_bytes", "cvmk_conv2d_stem_pack_weights",
    "cvmk_conv2d_stem_prepare", "cvmk_conv2d_stem_launch",
    "cvmk_conv2d_tc_supported", "cvmk_conv2d_tc_workspace_bytes", "cvmk_conv2d_tc_prepare", "cvmk_conv2d_tc_launch", "cvmk_elemwise",
    "cvmk_transpose_batched", "cvmk_strided", "cvmk_strided_batch", "cvmk_take", "cvmk_where", "cvmk_reduce", "cvmk_max_pool2d", "cvmk_conv2d_direct", "cvmk_get_valid_counts", "cvmk_get_valid_counts_clamped",
    "cvmk_nms_scratch_bytes", "cvmk_non_max_suppression", "cvmk_non_max_suppression_static",
    "cvmk_last_error",
]


class CVMError(RuntimeError):
    """A C-ABI call returned ERROR_LOGIC (1) or ERROR_RUNTIME (2)."""

    def __init__(self, status, what, text=""):
        super().__init__("%s returned status %d%s" % (what, status, ": " + text if text else ""))
        self.status = status
        self.text = text


_LIB = None


def lib():
    """The loaded shared library (raises if it has not been built)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise OSError("%s not found: build it with `python cvm-runtime_b200/build.py`" % LIB_PATH)
        _LIB = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        _LIB.cvmk_last_error.restype = ctypes.c_char_p
        _LIB.CVMXLastError.restype = ctypes.c_char_p
        _LIB.cvmk_nms_scratch_bytes.restype = ctypes.c_int64
    return _LIB


_MEASURE = None


def measure_lib():
    """libcvm_measure.so: measurement and self-test helpers, kept out of the runtime library."""
    global _MEASURE
    if _MEASURE is None:
        if not os.path.exists(MEASURE_LIB_PATH):
            raise OSError("%s not found: build it with `python cvm-runtime_b200/build.py`" % MEASURE_LIB_PATH)
        _MEASURE = ctypes.CDLL(MEASURE_LIB_PATH)
        _MEASURE.cvmk_measure_last_error.restype = ctypes.c_char_p
    return _MEASURE


def last_error():
    """Text of the last failing C-ABI call of this thread."""
    return (lib().CVMXLastError() or b"").decode("utf-8", "replace")


def check_call(status, what="CVMAPI call"):
    if status != SUCCEED:
        raise CVMError(status, what, last_error())


NetworkHandle = ctypes.c_void_p


def CVMAPILoadModel(json_str, param_bytes, device_id=0, device_type=1):
    """Load a model from its graph JSON and params blob onto GPU `device_id`."""
    net = NetworkHandle()
    if isinstance(json_str, str):
        json_str = json_str.encode("utf-8")
    check_call(lib().CVMAPILoadModel(
        ctypes.c_char_p(json_str), ctypes.c_int(len(json_str)),
        ctypes.c_char_p(param_bytes), ctypes.c_int(len(param_bytes)),
        ctypes.byref(net), ctypes.c_int(device_type), ctypes.c_int(device_id)), "CVMAPILoadModel")
    return net


def CVMAPIFreeModel(net):
    check_call(lib().CVMAPIFreeModel(net), "CVMAPIFreeModel")


def _get_ull(name, net):
    size = ctypes.c_ulonglong()
    check_call(getattr(lib(), name)(net, ctypes.byref(size)), name)
    return size.value


def CVMAPIGetInputLength(net):
    return _get_ull("CVMAPIGetInputLength", net)


def CVMAPIGetInputTypeSize(net):
    return _get_ull("CVMAPIGetInputTypeSize", net)


def CVMAPIGetOutputLength(net):
    return _get_ull("CVMAPIGetOutputLength", net)


def CVMAPIGetOutputTypeSize(net):
    return _get_ull("CVMAPIGetOutputTypeSize", net)


def CVMAPIGetStorageSize(net):
    return _get_ull("CVMAPIGetStorageSize", net)


def CVMAPIGetGasFromModel(net):
    return _get_ull("CVMAPIGetGasFromModel", net)


def CVMAPIGetGasFromGraphFile(json_str):
    if isinstance(json_str, str):
        json_str = json_str.encode("utf-8")
    gas = ctypes.c_ulonglong()
    check_call(lib().CVMAPIGetGasFromGraphFile(ctypes.c_char_p(json_str), ctypes.byref(gas)),
               "CVMAPIGetGasFromGraphFile")
    return gas.value


def CVMAPIGetVersion(net):
    buf = ctypes.create_string_buffer(64)
    check_call(lib().CVMAPIGetVersion(net, buf), "CVMAPIGetVersion")
    return buf.value.decode()


def CVMAPIGetPreprocessMethod(net):
    buf = ctypes.create_string_buffer(64)
    check_call(lib().CVMAPIGetPreprocessMethod(net, buf), "CVMAPIGetPreprocessMethod")
    return buf.value.decode()


def inference_bytes(net, input_data, out=None):
    """CVMAPIInference on raw bytes (or a contiguous numpy array); returns the output bytes as a
    numpy uint8 array (written into `out` when given)."""
    if isinstance(input_data, np.ndarray):
        arr = np.ascontiguousarray(input_data)
        in_ptr = arr.ctypes.data_as(ctypes.c_char_p)
        in_len = arr.nbytes
    else:
        arr = input_data
        in_ptr = ctypes.c_char_p(input_data)
        in_len = len(input_data)
    if out is None:
        out = np.zeros(CVMAPIGetOutputLength(net), dtype=np.uint8)  # argmax mode leaves a tail unwritten
    check_call(lib().CVMAPIInference(net, in_ptr, ctypes.c_int(in_len),
                                     out.ctypes.data_as(ctypes.c_char_p)), "CVMAPIInference")
    return out


def CVMAPIInference(net, input_data):
    """Reference-compatible form: returns the outputs as a list of Python ints."""
    raw = inference_bytes(net, input_data)
    otype = CVMAPIGetOutputTypeSize(net)
    return raw.view(np.int8 if otype == 1 else np.int32).astype(np.int64).tolist()


# ---- measurement helpers (include/cvm/c_api_ext.h) --------------------------------------------
def step_count(net):
    """Kernel launches per inference."""
    return _get_ull("CVMXStepCount", net)


def device_bytes(net):
    return _get_ull("CVMXDeviceBytes", net)


def activation_bytes(net):
    """(sum of the planned activation buffers' sizes, device memory that backs them)."""
    a, b = ctypes.c_ulonglong(), ctypes.c_ulonglong()
    check_call(lib().CVMXActivationBytes(net, ctypes.byref(a), ctypes.byref(b)), "CVMXActivationBytes")
    return int(a.value), int(b.value)


def replay_device(net, iters):
    """Device milliseconds for `iters` kernel-only replays (input of the last inference)."""
    ms = ctypes.c_float()
    check_call(lib().CVMXReplayDevice(net, ctypes.c_int(iters), ctypes.byref(ms)), "CVMXReplayDevice")
    return ms.value


def measure_i8_mma_rate(n=256, reps=20000):
    """Measured int8 tensor-core rate of the current GPU in TOP/s (tcgen05.mma kind::i8, M = 128,
    N = n, K = 32 issued back to back on every SM)."""
    tops = ctypes.c_double()
    rc = measure_lib().cvmk_measure_i8_mma_rate(ctypes.c_int(n), ctypes.c_int(reps), ctypes.byref(tops))
    if rc != 0:
        raise RuntimeError("cvmk_measure_i8_mma_rate failed (%d): %s" % (rc, measure_lib().cvmk_measure_last_error().decode()))
    return tops.value


def measure_i8_mma_rate_window(n, reps, row_bytes, a_offset_rows, group_stride_rows):
    """The rate with the A operand read as a window of a staged halo: rows of `row_bytes`, starting
    `a_offset_rows` rows into the tile, 8-row groups `group_stride_rows` rows apart (TOP/s)."""
    tops = ctypes.c_double()
    rc = measure_lib().cvmk_measure_i8_mma_rate_window(ctypes.c_int(n), ctypes.c_int(reps), ctypes.c_int(row_bytes),
                                                       ctypes.c_int(a_offset_rows), ctypes.c_int(group_stride_rows),
                                                       ctypes.byref(tops))
    if rc != 0:
        raise RuntimeError("cvmk_measure_i8_mma_rate_window failed (%d): %s" % (rc, measure_lib().cvmk_measure_last_error().decode()))
    return tops.value


def wait_timeout(limit=64):
    """Lets a bounded device-side wait run out (a barrier nothing arrives at, `limit` polls of about
    2 us); returns (status word, SM clocks waited)."""
    word, clocks = ctypes.c_int(0), ctypes.c_longlong(0)
    rc = measure_lib().cvmk_measure_wait_timeout(ctypes.c_uint(limit), ctypes.byref(word), ctypes.byref(clocks))
    if rc != 0:
        raise RuntimeError("cvmk_measure_wait_timeout failed (%d): %s" % (rc, measure_lib().cvmk_measure_last_error().decode()))
    return word.value, clocks.value


def set_status_word(net, code):
    """Writes `code` into the model's device status word, as a kernel whose bounded wait ran out
    would (include/cvm/c_api_ext.h)."""
    check_call(lib().CVMXSetStatusWord(net, ctypes.c_int(code)), "CVMXSetStatusWord")


def profile_steps(net, input_data):
    """[(operator label, milliseconds)] of one launch-by-launch pass."""
    arr = np.ascontiguousarray(input_data)
    buf = ctypes.create_string_buffer(1 << 20)
    check_call(lib().CVMXProfileSteps(net, arr.ctypes.data_as(ctypes.c_char_p), ctypes.c_int(arr.nbytes),
                                      buf, ctypes.c_int(len(buf))), "CVMXProfileSteps")
    rows = []
    for line in buf.value.decode().splitlines():
        label, ms = line.rsplit("\t", 1)
        rows.append((label, float(ms)))
    return rows
