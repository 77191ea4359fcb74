"""Generates tests/golden/*.npz from the reference's own CPU runtime (oracle/_ref, built by
`make -C oracle ref` from the unmodified reference sources).  Run in a container that has the
reference tree; the fixtures it writes are committed and travel where the reference does not.

    python tests/golden/make_golden.py
"""
import hashlib
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import cases  # noqa: E402

oracle = cases.ge.load_oracle()


def sha(b):
    return hashlib.sha256(bytes(b)).hexdigest()


def main():
    ref = oracle.ref_lib
    if not ref.available():
        raise SystemExit("oracle/_ref/libcvm_runtime_ref.so is missing: run `make -C oracle ref` first")
    out = {}
    for group, table in (("model", cases.model_cases()), ("op", cases.op_cases())):
        for name, thunk in table.items():
            js, pb, x = thunk()
            m = ref.RefModel(js, pb, 0)
            assert m.loaded, (name, m.status)
            st, y = m.infer(x)
            assert st == 0, (name, st)
            gst, gas = m.gas()
            key = "%s/%s" % (group, name)
            out[key + "/out"] = y
            out[key + "/meta"] = np.array([m.input_length(), m.output_length(), m.storage_size(), gst, gas], np.int64)
            out[key + "/sha"] = np.array([sha(js), sha(pb), sha(np.ascontiguousarray(x).tobytes())])
            m.free()
    np.savez_compressed(os.path.join(HERE, "outputs.npz"), **out)
    # one process per malformed model: the reference may crash on some of them
    status = {}
    for name in cases.malformed_cases():
        code = ("import sys; sys.path.insert(0, %r); import cases; o = cases.ge.load_oracle(); "
                "js, pb = cases.malformed_cases()[%r]; m = o.ref_lib.RefModel(js, pb, 0); "
                "sys.stdout.flush(); import os; os._exit(100 + m.status)" % (os.path.dirname(HERE), name))
        rc = subprocess.run([sys.executable, "-c", code], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL).returncode
        status[name] = rc - 100 if rc >= 100 else rc
    np.savez(os.path.join(HERE, "load_status.npz"), names=np.array(list(status)), status=np.array(list(status.values())))
    print("wrote %d outputs, %d load statuses" % (len(out) // 3, len(status)))
    for k, v in status.items():
        print("  %-28s -> %d" % (k, v))


if __name__ == "__main__":
    main()
