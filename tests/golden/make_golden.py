"""Generates tests/golden/*.npz from the reference's own CPU runtime (oracle/_ref, built by
`make -C oracle ref` from the unmodified reference sources).  Run in a container that has the
reference tree; the fixtures it writes are committed and travel where the reference does not.

    python tests/golden/make_golden.py              # everything
    python tests/golden/make_golden.py --fullsize   # only the digests of the full-size configurations
    python tests/golden/make_golden.py --outputs    # only outputs.npz and load_status.npz
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


def fullsize_golden():
    """tests/golden/fullsize.npz: SHA-256 and length of the reference's output on the full-size
    configurations of tests/cases.py (one process each: some of them hold gigabytes)."""
    names = list(cases.fullsize_cases())
    digests, sizes, inputs = [], [], []
    for name in names:
        code = ("import sys, hashlib; sys.path.insert(0, %r); import cases, numpy as np; o = cases.ge.load_oracle(); "
                "js, pb, x = cases.fullsize_cases()[%r](); y = o.ref_lib.run_model(js, pb, x); "
                "sys.stdout.write('\\nDIGEST %%s %%d %%s\\n' %% (hashlib.sha256(y.tobytes()).hexdigest(), y.nbytes, "
                "hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest()))" % (os.path.dirname(HERE), name))
        out = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, check=True).stdout
        line = [l for l in out.splitlines() if l.startswith("DIGEST ")][-1].split()
        digests.append(line[1])
        sizes.append(int(line[2]))
        inputs.append(line[3])
        print("  %-24s %s %d" % (name, line[1][:16], int(line[2])))
    np.savez(os.path.join(HERE, "fullsize.npz"), names=np.array(names), sha=np.array(digests),
             nbytes=np.array(sizes, np.int64), input_sha=np.array(inputs))


def fuzz_worker(start, path):
    """Runs mutants start.. against the reference, one JSON line each; a `begin` line first so the
    parent can tell which mutant took the process down."""
    import json
    import fuzz_cases
    ref = oracle.ref_lib
    table = fuzz_cases.fuzz_cases()
    names = list(table)
    with open(path, "a") as f:
        for i in range(start, len(names)):
            js, pb, x, _ = table[names[i]]
            f.write(json.dumps({"begin": i}) + "\n")
            f.flush()
            os.fsync(f.fileno())
            m = ref.RefModel(js, pb, 0)
            rec = {"i": i, "load": int(m.status), "infer": -1, "out": "", "gas_status": -1, "gas": 0}
            if m.loaded:
                gst, gas = m.gas()
                rec["gas_status"], rec["gas"] = int(gst), int(gas)
                if x is not None:
                    st, y = m.infer(x)
                    rec["infer"] = int(st)
                    if st == 0:
                        rec["out"] = sha(y.tobytes()) + ":%d" % y.nbytes
                m.free()
            f.write(json.dumps(rec) + "\n")
            f.flush()


def fuzz_golden():
    """tests/golden/fuzz.npz: the reference's verdict on every mutant of tests/fuzz_cases.py.
    load = -100 marks a mutant that crashed or hung the reference process."""
    import json
    import fuzz_cases
    names = list(fuzz_cases.fuzz_cases())
    path = os.path.join(HERE, "_fuzz_progress.jsonl")
    if os.path.exists(path):
        os.remove(path)
    recs = {}
    start = 0
    while start < len(names):
        try:
            subprocess.run([sys.executable, os.path.abspath(__file__), "--fuzz-worker", str(start), path],
                           stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, timeout=600)
        except subprocess.TimeoutExpired:
            pass
        last_begin = None
        for line in open(path):
            r = json.loads(line)
            if "begin" in r:
                last_begin = r["begin"]
            else:
                recs[r["i"]] = r
        if last_begin is None:
            raise SystemExit("fuzz worker produced nothing")
        if last_begin not in recs:
            recs[last_begin] = {"i": last_begin, "load": -100, "infer": -1, "out": "", "gas_status": -1, "gas": 0}
        start = max(recs) + 1
    os.remove(path)
    out = {"names": np.array(names)}
    out["load"] = np.array([recs[i]["load"] for i in range(len(names))], np.int32)
    out["infer"] = np.array([recs[i]["infer"] for i in range(len(names))], np.int32)
    out["gas_status"] = np.array([recs[i]["gas_status"] for i in range(len(names))], np.int32)
    out["gas"] = np.array([recs[i]["gas"] for i in range(len(names))], np.int64)
    out["out_sha"] = np.array([recs[i]["out"] for i in range(len(names))])   # "sha256:length" or ""
    np.savez_compressed(os.path.join(HERE, "fuzz.npz"), **out)
    load = out["load"]
    print("fuzz: %d mutants: %d accepted (%d inferred), %d logic errors, %d runtime errors, %d crashed the reference"
          % (len(names), int((load == 0).sum()), int((out["infer"] == 0).sum()), int((load == 1).sum()),
             int((load == 2).sum()), int((load == -100).sum())))


def random_worker(start, path):
    import json
    import random_graphs
    ref = oracle.ref_lib
    table = random_graphs.random_cases()
    names = list(table)
    with open(path, "a") as f:
        for i in range(start, len(names)):
            js, pb, x = table[names[i]]()
            f.write(json.dumps({"begin": i}) + "\n")
            f.flush()
            os.fsync(f.fileno())
            m = ref.RefModel(js, pb, 0)
            rec = {"i": i, "load": int(m.status), "infer": -1, "out": ""}
            if m.loaded:
                st, y = m.infer(x)
                rec["infer"] = int(st)
                if st == 0:
                    rec["out"] = sha(y.tobytes()) + ":%d" % y.nbytes
                m.free()
            f.write(json.dumps(rec) + "\n")
            f.flush()


def random_golden():
    """tests/golden/random_graphs.npz: the reference's verdict on every graph of tests/random_graphs.py."""
    import json
    import random_graphs
    names = list(random_graphs.random_cases())
    path = os.path.join(HERE, "_random_progress.jsonl")
    if os.path.exists(path):
        os.remove(path)
    recs = {}
    start = 0
    while start < len(names):
        try:
            subprocess.run([sys.executable, os.path.abspath(__file__), "--random-worker", str(start), path],
                           stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, timeout=900)
        except subprocess.TimeoutExpired:
            pass
        last_begin = None
        for line in open(path):
            r = json.loads(line)
            if "begin" in r:
                last_begin = r["begin"]
            else:
                recs[r["i"]] = r
        if last_begin is None:
            raise SystemExit("random-graph worker produced nothing")
        if last_begin not in recs:
            recs[last_begin] = {"i": last_begin, "load": -100, "infer": -1, "out": ""}
        start = max(recs) + 1
    os.remove(path)
    out = {"names": np.array(names),
           "load": np.array([recs[i]["load"] for i in range(len(names))], np.int32),
           "infer": np.array([recs[i]["infer"] for i in range(len(names))], np.int32),
           "out_sha": np.array([recs[i]["out"] for i in range(len(names))])}
    np.savez_compressed(os.path.join(HERE, "random_graphs.npz"), **out)
    print("random graphs: %d: %d ran, %d refused at load, %d failed at inference, %d crashed the reference"
          % (len(names), int((out["infer"] == 0).sum()), int(((out["load"] == 1) | (out["load"] == 2)).sum()),
             int(((out["load"] == 0) & (out["infer"] > 0)).sum()), int((out["load"] == -100).sum())))


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--random-worker":
        random_worker(int(sys.argv[2]), sys.argv[3])
    elif len(sys.argv) > 1 and sys.argv[1] == "--random":
        random_golden()
    elif len(sys.argv) > 1 and sys.argv[1] == "--fuzz-worker":
        fuzz_worker(int(sys.argv[2]), sys.argv[3])
    elif len(sys.argv) > 1 and sys.argv[1] == "--fuzz":
        fuzz_golden()
    elif len(sys.argv) > 1 and sys.argv[1] == "--fullsize":
        fullsize_golden()
    elif len(sys.argv) > 1 and sys.argv[1] == "--outputs":
        main()
    else:
        main()
        fuzz_golden()
        random_golden()
        fullsize_golden()
