"""Host-side contract without a GPU: the library loads, exports every declared symbol, answers the
graph-only queries like the reference, and refuses malformed models with the reference's status."""
import ctypes
import os
import re

import numpy as np
import pytest

import cases

ROOT = cases.ROOT


def declared_symbols():
    names = []
    for rel in ("include/cvm/c_api.h", "include/cvm/c_api_ext.h", "include/cvmk_kernels.h"):
        text = open(os.path.join(ROOT, rel)).read()
        names += re.findall(r"^(?:CVM_DLL|CVMK_API)\s+[\w\s\*]*?\b(\w+)\s*\(", text, flags=re.M)
    return names


def test_library_exports_every_declared_symbol(rt):
    lib = rt.lib()
    names = declared_symbols()
    assert len(names) >= 12 + 4 + 12
    for n in rt.API_SYMBOLS + rt.KERNEL_SYMBOLS:
        assert n in names, n
    for n in names:
        assert hasattr(lib, n), "libcvm_runtime.so does not export " + n


def test_measure_library_exports_its_symbols(rt):
    """libcvm_measure.so (measurement / self-test helpers) is a library of its own: the runtime
    library exports none of its symbols."""
    text = open(os.path.join(ROOT, "include/cvmk_measure.h")).read()
    names = re.findall(r"^CVMK_API\s+[\w\s\*]*?\b(\w+)\s*\(", text, flags=re.M)
    assert sorted(names) == sorted(rt.MEASURE_SYMBOLS)
    for n in names:
        assert hasattr(rt.measure_lib(), n), "libcvm_measure.so does not export " + n
        assert not hasattr(rt.lib(), n), "libcvm_runtime.so should not export " + n


def test_gas_matches_reference(rt, golden):
    for group, table in (("model", cases.model_cases()), ("op", cases.op_cases())):
        for name, thunk in table.items():
            js, _, _ = thunk()
            meta = golden["%s/%s/meta" % (group, name)]
            if meta[3] == 0:
                assert rt.CVMAPIGetGasFromGraphFile(js) == meta[4], name


def test_gas_limit_is_a_logic_error(rt, wl):
    js, _, _ = wl.resnet50(batch=256)
    with pytest.raises(rt.CVMError) as e:
        rt.CVMAPIGetGasFromGraphFile(js)       # 3.2e12 > 2^40, infer_attr.cc:97-99
    assert e.value.status == rt.ERROR_LOGIC
    js, _, _ = wl.resnet50(batch=32)
    assert rt.CVMAPIGetGasFromGraphFile(js) > 0


@pytest.mark.parametrize("name", list(cases.malformed_cases()))
def test_malformed_models_fail_like_the_reference(name, rt, golden_status):
    want = golden_status[name]
    if want not in (1, 2):
        pytest.skip("accepted (or crashed) by the reference: covered by the GPU tests")
    js, pb = cases.malformed_cases()[name]
    net = ctypes.c_void_p()
    st = rt.lib().CVMAPILoadModel(js, len(js), pb, len(pb), ctypes.byref(net), 1, 0)
    assert st == want


def test_fuzzed_models_are_refused_like_the_reference(rt, golden_fuzz):
    """Every mutant the reference refuses is refused with the same status class; gas of the
    accepted ones matches (graph-only query, no GPU)."""
    import fuzz_cases
    table = fuzz_cases.fuzz_cases()
    names = list(table)
    assert names == golden_fuzz["names"].tolist()
    wrong = []
    refused = stricter = 0
    for i, name in enumerate(names):
        js, pb, _, desc = table[name]
        want = int(golden_fuzz["load"][i])
        if want in (1, 2):
            refused += 1
            net = ctypes.c_void_p()
            st = rt.lib().CVMAPILoadModel(js, len(js), pb, len(pb), ctypes.byref(net), 1, 0)
            if st == 0:
                rt.lib().CVMAPIFreeModel(net)
            if st != want:
                wrong.append((name, desc, want, st))
        elif want == 0 and int(golden_fuzz["gas_status"][i]) == 0:
            try:
                gas = rt.CVMAPIGetGasFromGraphFile(js)
            except rt.CVMError as e:
                if e.status == rt.ERROR_LOGIC and fuzz_cases.is_documented_refusal(e.text):
                    stricter += 1
                    continue
                gas = "status %d" % e.status
            if gas != int(golden_fuzz["gas"][i]):
                wrong.append((name, desc, "gas %d" % int(golden_fuzz["gas"][i]), gas))
    assert refused >= 500 and stricter <= 80
    assert not wrong, wrong


def test_null_arguments_are_runtime_errors(rt):
    lib = rt.lib()
    v = ctypes.c_ulonglong()
    assert lib.CVMAPIGetInputLength(None, ctypes.byref(v)) == 2
    assert lib.CVMAPIInference(None, None, 0, None) == 2
    assert lib.CVMAPIFreeModel(None) == 0
    js, pb, _ = cases.wl.conv_chain(1, channels=32, size=8)
    net = ctypes.c_void_p()
    assert lib.CVMAPILoadModel(js, len(js), pb, len(pb), ctypes.byref(net), 7, 0) == 2   # bad device type
    assert lib.CVMAPILoadModel(js, len(js), pb, len(pb), ctypes.byref(net), 0, 0) == 2   # no CPU path
    assert lib.CVMAPILoadModel(js, len(js), b"", 0, ctypes.byref(net), 1, 0) == 1        # empty params


def test_workload_shapes(wl):
    js, pb, x = wl.resnet50(1)
    assert x.shape == (1, 3, 224, 224) and x.dtype == np.int8
    assert abs(wl.conv_ops_per_image(js) - 8.18e9) < 0.05e9
    assert wl.SSD_ANCHORS == 24564
