"""Host-side functions of the kernel C-ABI that run without a device.

tests/kernel_abi/host_fns.c is plain C: it includes include/cvmk_kernels.h (so the header is
checked to be a C header), links with the runtime library and prints what
cvmk_conv2d_tc_workspace_bytes(), cvmk_conv2d_stem_weight_bytes() and
cvmk_conv2d_stem_pack_weights() return.  The packed filter is compared with the operand order the
header documents, restated here with numpy.
"""
import os
import shutil
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "kernel_abi", "host_fns.c")
BIN = os.path.join(HERE, "kernel_abi", "build", "host_fns")
LIBDIR = os.path.join(ROOT, "cvm-runtime_b200")
LIB = os.path.join(LIBDIR, "libcvm_runtime.so")


@pytest.fixture(scope="module")
def host_fns():
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    if not os.path.exists(LIB):
        import __graft_entry__
        __graft_entry__.build()
    stale = not os.path.exists(BIN) or os.path.getmtime(BIN) < max(os.path.getmtime(SRC), os.path.getmtime(LIB))
    if stale:
        os.makedirs(os.path.dirname(BIN), exist_ok=True)
        subprocess.check_call(["gcc", "-O1", "-Wall", "-Werror", "-std=c11", "-I" + os.path.join(ROOT, "include"), SRC,
                               "-o", BIN, "-L" + LIBDIR, "-lcvm_runtime", "-Wl,-rpath," + LIBDIR])

    def run(*args):
        env = dict(os.environ)
        for k in [k for k in env if k.startswith("CVM_B200_")]:
            del env[k]
        p = subprocess.run([BIN] + [str(a) for a in args], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                           env=env, timeout=60)
        assert p.returncode == 0, p.stderr
        return dict(tok[1:].split("=", 1) for tok in p.stdout.split() if tok.startswith("@"))
    return run


def test_long_reductions_of_few_rows_ask_for_scratch(host_fns):
    # a dense layer of 8 rows over K = 25088 (VGG fc6) has 16 output tiles: it is cut along K, and the
    # scratch is rows x slices x OC int32 partial sums with a slice count that divides the K blocks
    f = host_fns("workspace", 8, 1, 1, 25088, 4096, 1, 1)
    assert f["supported"] == "1"
    ws = int(f["workspace"])
    assert ws > 0 and ws % (8 * 4096 * 4) == 0
    slices = ws // (8 * 4096 * 4)
    assert slices >= 2 and (25088 // 128) % slices == 0


@pytest.mark.parametrize("shape", [(256, 56, 56, 64, 256, 1, 1),      # many tiles already
                                   (32, 14, 14, 512, 512, 3, 3),      # not a 1x1 layer
                                   (8, 1, 1, 512, 1000, 1, 1),        # short K
                                   (200, 1, 1, 25088, 4096, 1, 1)])   # more rows than one tile
def test_other_shapes_ask_for_no_scratch(host_fns, shape):
    f = host_fns("workspace", *shape)
    assert f["workspace"] == "0"


def packed_reference(C, OC, KH, KW, S):
    """The documented operand order: for filter row ky' and tap pair j two blocks (taps 2j, 2j + 1)
    of OC rows x 16 bytes; byte (a * S + b) * C + c of a row is w[oc][c][S ky' + a][S kx' + b]."""
    oc, c, ky, kx = np.meshgrid(np.arange(OC), np.arange(C), np.arange(KH), np.arange(KW), indexing="ij")
    w = ((oc * 131 + c * 31 + ky * 7 + kx) % 255 - 127).astype(np.int8)
    khp, kwp = -(-KH // S), -(-KW // S)
    nj = (kwp + 1) // 2
    out = np.zeros((khp, nj, 2, OC, 16), dtype=np.int8)
    for kyp in range(khp):
        for kxp in range(kwp):
            for a in range(S):
                for b in range(S):
                    y, x = S * kyp + a, S * kxp + b
                    if y < KH and x < KW:
                        out[kyp, kxp // 2, kxp & 1, :, (a * S + b) * C:(a * S + b) * C + C] = w[:, :, y, x]
    return out


@pytest.mark.parametrize("shape", [(2, 224, 224, 3, 64, 7, 7, 2, 3),     # ResNet / SSD stems
                                   (2, 224, 224, 3, 32, 3, 3, 2, 1),     # MobileNet stem
                                   (1, 64, 64, 1, 128, 8, 8, 2, 0),
                                   (1, 32, 48, 2, 32, 5, 5, 1, 2),
                                   (1, 32, 32, 4, 64, 4, 4, 1, 0)])
def test_stem_filter_operand_order(host_fns, tmp_path, shape):
    N, H, W, C, OC, KH, KW, S, pad = shape
    path = tmp_path / "packed.bin"
    f = host_fns("stem", *shape, path)
    assert f["supported"] == "1" and f["pack"] == "0"
    want = packed_reference(C, OC, KH, KW, S)
    assert int(f["weight_bytes"]) == want.size
    got = np.fromfile(path, dtype=np.int8)
    np.testing.assert_array_equal(got, want.reshape(-1))


@pytest.mark.parametrize("shape", [(1, 224, 224, 5, 64, 7, 7, 2, 3),     # five channels
                                   (1, 224, 224, 3, 48, 7, 7, 2, 3),     # output channels not 32 / 64 / 128
                                   (1, 224, 200, 3, 64, 7, 7, 2, 3),     # width not a multiple of 16
                                   (1, 224, 224, 3, 64, 9, 9, 2, 3),     # filter wider than 8
                                   (1, 224, 224, 3, 64, 7, 7, 3, 3)])    # stride 3
def test_stem_refuses_what_it_cannot_run(host_fns, tmp_path, shape):
    f = host_fns("stem", *shape, tmp_path / "none.bin")
    assert f["supported"] == "0" and int(f["weight_bytes"]) < 0 and f["pack"] == "-1"
    assert not (tmp_path / "none.bin").exists()


@pytest.mark.parametrize("shape,ok", [((256, 56, 56, 128, 4, 3, 1), "1"),    # MobileNet: 128 channels as 4 groups of 32
                                      ((256, 14, 14, 512, 16, 3, 1), "1"),
                                      ((1, 16, 16, 1024, 32, 3, 1), "1"),
                                      ((256, 56, 56, 128, 2, 3, 1), "0"),    # groups of 64 channels
                                      ((256, 56, 56, 128, 4, 3, 2), "0"),    # stride 2
                                      ((256, 56, 56, 128, 4, 5, 1), "0"),    # 5 x 5
                                      ((256, 7, 7, 1024, 32, 3, 1), "0")])   # a 7 x 7 image wastes most of an 8 x 16 tile
def test_grouped_convolutions_the_tensor_core_kernel_takes(host_fns, shape, ok):
    assert host_fns("grouped", *shape)["supported"] == ok
