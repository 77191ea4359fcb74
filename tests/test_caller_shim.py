"""The library driven through the reference's own caller-side shim.

The reference's Go package binds the runtime with kernel/dlopen.h: dlopen(RTLD_NOW|RTLD_GLOBAL) and
one dlsym per call behind dl_CVMAPI* wrappers (kernel/dlopen.h:11-78), in the call order of
kernel/libcvm.go:57-133.  There is no Go toolchain here, but that shim is plain C:
tests/caller_shim/go_shim_caller.c includes the header from the reference checkout (it is not
copied into this repository) and replays the sequence.  The program is compiled where the
reference tree is available ($CVM_REFERENCE_ROOT, or a `reference` directory beside the
repository) into tests/caller_shim/build/, which travels with the repository but stays out of its
history; where neither the tree nor the binary exists the tests skip.
"""
import os
import subprocess

import numpy as np
import pytest

import cases

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "caller_shim", "go_shim_caller.c")
BIN = os.path.join(HERE, "caller_shim", "build", "go_shim_caller")


def reference_root():
    return os.environ.get("CVM_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


def build_caller():
    """Compiles the caller against <reference>/kernel/dlopen.h; returns the binary or None."""
    header = os.path.join(reference_root(), "kernel", "dlopen.h")
    if os.path.exists(header):
        stale = not os.path.exists(BIN) or os.path.getmtime(BIN) < max(os.path.getmtime(SRC), os.path.getmtime(header))
        if stale:
            os.makedirs(os.path.dirname(BIN), exist_ok=True)
            subprocess.check_call(["gcc", "-O1", "-Wall", "-Wno-unused-function", "-I" + os.path.dirname(header),
                                   SRC, "-o", BIN, "-ldl"])
    return BIN if os.path.exists(BIN) else None


def run_caller(binary, lib_path, case, tmp_path, device_type):
    js, pb, x = cases.model_cases()[case]()
    paths = {k: str(tmp_path / (case + "." + k)) for k in ("json", "params", "input", "output")}
    open(paths["json"], "wb").write(js if isinstance(js, bytes) else js.encode())
    open(paths["params"], "wb").write(pb)
    open(paths["input"], "wb").write(np.ascontiguousarray(x).tobytes())
    p = subprocess.run([binary, lib_path, paths["json"], paths["params"], paths["input"], paths["output"],
                        str(device_type), "0"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    fields = dict(tok[1:].split("=", 1) for tok in p.stdout.split() if tok.startswith("@") and "=" in tok)
    out = np.fromfile(paths["output"], dtype=np.uint8) if os.path.exists(paths["output"]) else None
    return p.returncode, fields, out, p.stderr


def check(fields, out, golden, case, version):
    meta = golden["model/%s/meta" % case]
    assert fields["load"] == "0" and fields["infer"] == "0" and fields["infer2"] == "0" and fields["free"] == "0"
    assert int(fields["input_length"]) == meta[0]
    assert int(fields["output_length"]) == meta[1]
    assert int(fields["storage"]) == meta[2]
    if meta[3] == 0:
        assert fields["gas_status"] == "0" and int(fields["gas"]) == meta[4]
        assert fields["gas_file_status"] == "0" and int(fields["gas_file"]) == meta[4]
    if version is not None:
        assert fields["version"] == "[%s]" % version
    assert fields["method"] == "[]"
    assert np.array_equal(out, golden["model/%s/out" % case])


CASES = ["conv_chain_s14", "resnet50_s64", "ssd_tail_b2"]   # int8 head, int32 logits, int32 detection rows


@pytest.mark.parametrize("case", CASES)
def test_shim_harness_against_reference_library(case, tmp_path, golden, oracle):
    """The harness itself, on the CPU: the reference's own library through the reference's own shim
    must reproduce the committed fixtures (which came from that library through ctypes)."""
    binary = build_caller()
    if binary is None or not oracle.ref_lib.available():
        pytest.skip("needs the reference checkout (kernel/dlopen.h) and oracle/_ref")
    rc, fields, out, err = run_caller(binary, oracle.ref_lib.REF_LIB, case, tmp_path, 0)
    assert rc == 0, (rc, fields, err)
    # The reference never fills the version buffer: its `get_version` function wants an array handle
    # and CVMModel passes a char* (src/runtime/graph_runtime.cc:733-742, src/core/model.cc:75-80), so
    # the caller reads whatever the stack held.  Not compared.
    check(fields, out, golden, case, None)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES)
def test_library_through_reference_shim(case, tmp_path, golden, pkg):
    """libcvm_runtime.so of this repository behind the reference's dlopen shim, device_type 1 (GPU)."""
    binary = build_caller()
    if binary is None:
        pytest.skip("tests/caller_shim/build/go_shim_caller was not built (no reference checkout)")
    rc, fields, out, err = run_caller(binary, pkg.LIB, case, tmp_path, 1)
    assert rc == 0, (rc, fields, err)
    check(fields, out, golden, case, "cvm_1.0.0")
