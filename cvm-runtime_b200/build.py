"""Builds libcvm_runtime.so (host runtime + sm_100a kernels) and libcvm_measure.so (measurement and
self-test helpers, include/cvmk_measure.h) in-tree with nvcc.

libcvm_runtime.so is the product: the C-ABI of include/cvm/c_api.h on top of the kernel launchers
of include/cvmk_kernels.h.  Nothing here links or loads anything under oracle/.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libcvm_runtime.so")
MEASURE_LIB = os.path.join(HERE, "libcvm_measure.so")

KERNEL_SRCS = ["common.cu", "conv_tc.cu", "conv_stem.cu", "conv_direct.cu", "elemwise.cu", "transform.cu", "nms.cu"]
HOST_SRCS = ["ops.cc", "graph.cc", "executor.cc", "c_api.cc"]
MEASURE_SRCS = ["measure.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
]


def _newer(src, dst):
    return not os.path.exists(dst) or os.path.getmtime(src) > os.path.getmtime(dst)


def build(force=False, verbose=False):
    """Compile every translation unit that changed and link the shared library."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    inc = ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(HERE, "csrc", "kernels"),
           "-I" + os.path.join(HERE, "csrc", "host")]
    headers = []
    for d in (os.path.join(ROOT, "include"), os.path.join(ROOT, "include", "cvm"),
              os.path.join(HERE, "csrc", "kernels"), os.path.join(HERE, "csrc", "host")):
        headers += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".h", ".cuh"))]
    newest_header = max(os.path.getmtime(h) for h in headers)
    objs, measure_objs, procs = [], [], []
    for sub, names in (("kernels", KERNEL_SRCS), ("host", HOST_SRCS), ("measure", MEASURE_SRCS)):
        for name in names:
            src = os.path.join(HERE, "csrc", sub, name)
            obj = os.path.join(objdir, name + ".o")
            (measure_objs if sub == "measure" else objs).append(obj)
            stale = force or _newer(src, obj) or newest_header > os.path.getmtime(obj)
            if stale:
                cmd = [nvcc] + NVCC_FLAGS + inc + ["-x", "cu", "-c", src, "-o", obj]
                if verbose:
                    print(" ".join(cmd))
                procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for name, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            failed = True
            sys.stderr.write("nvcc failed on %s:\n%s\n" % (name, out))
        elif verbose and out.strip():
            print(out)
    if failed:
        raise RuntimeError("build of libcvm_runtime.so failed")
    if procs or not os.path.exists(LIB):
        subprocess.check_call([nvcc, "-shared", "-o", LIB] + objs + ["-lcudart"])
    if procs or not os.path.exists(MEASURE_LIB):
        subprocess.check_call([nvcc, "-shared", "-o", MEASURE_LIB] + measure_objs + ["-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
