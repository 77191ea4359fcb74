import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import __graft_entry__ as ge  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the sm_100a kernels through the C-ABI)")


@pytest.fixture(scope="session")
def pkg():
    p = ge.load_package()
    if not os.path.exists(p.LIB):
        p.build()
    return p


@pytest.fixture(scope="session")
def rt(pkg):
    return pkg.runtime


@pytest.fixture(scope="session")
def wl(pkg):
    return pkg.workloads


@pytest.fixture(scope="session")
def oracle():
    return ge.load_oracle()


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "outputs.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def golden_status():
    d = np.load(os.path.join(ROOT, "tests", "golden", "load_status.npz"))
    return dict(zip(d["names"].tolist(), d["status"].tolist()))


@pytest.fixture(scope="session")
def golden_fuzz():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "fuzz.npz")))


@pytest.fixture(scope="session")
def golden_random():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "random_graphs.npz")))


@pytest.fixture(scope="session")
def golden_fullsize():
    d = np.load(os.path.join(ROOT, "tests", "golden", "fullsize.npz"))
    return {n: (str(s), int(b), str(i)) for n, s, b, i in zip(d["names"].tolist(), d["sha"].tolist(),
                                                              d["nbytes"].tolist(), d["input_sha"].tolist())}


@pytest.fixture(scope="session")
def gpu_run(rt):
    """Runs (json, params, input) through the C-ABI on cuda:0 and returns the output bytes."""
    def run(js, pb, x, device=0):
        net = rt.CVMAPILoadModel(js, pb, device)
        try:
            return rt.inference_bytes(net, x).copy()
        finally:
            rt.CVMAPIFreeModel(net)
    return run
