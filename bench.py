"""Benchmark of the operator hot path: int8 ResNet-50 images/s through the C-ABI on N B200s, with
the other two figures of the headline metric (conv2d int8 TOP/s, NMS boxes/s) measured beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload resnet50|mobilenet|vgg19|conv_chain|ssd_tail|ssd_backbone|ssd_full] [--batch B]

One step = one inference of the per-GPU batch (default: synthetic MRT-style quantized ResNet-50
v1, batch 256).  With N > 1 (launched through torch.distributed.run) every rank holds its own
weight replica and its own batch: no collective is on the data path, throughput scales weakly.

Printed JSON (rank 0):
  value        units/s with the input resident in device memory: CUDA events around K kernel-only
               replays, max over ranks, median over R back-to-back repetitions of the K-step region
               (R chosen so that the repetitions last about 1.5 s; `ms_per_step_best` is the best one)
  e2e          units/s through CVMAPIInference with host buffers (upload, kernels, download and the
               output conversion inside the timed region), page-locked and pageable caller buffers
  roofline     the dominant kernel (tcgen05 convolution, or NMS) against the rate measured in this run
  extra        (1 GPU) conv2d TOP/s on the conv chain and the VGG-19 layers, NMS boxes/s at batch 1 and
               64, MobileNet images/s, GB/s of the bandwidth-bound kernels
  strong       (N > 1) the same network with a global batch of 256 split over the N GPUs
  cpu_baseline the reference CPU runtime on this machine's cores: one thread, all threads, and one
               single-thread process per core on batch shards (clean child processes)
`--impl reference` times the reference's own CPU runtime (oracle/_ref) on the same configuration.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

METRIC = "int8 ResNet-50 images/s"
UNITS = {"resnet50": "images/s", "mobilenet": "images/s", "vgg19": "images/s", "conv_chain": "images/s",
         "ssd_tail": "boxes/s", "ssd_backbone": "images/s", "ssd_full": "images/s"}
# VGG-19: the reference refuses graphs whose int32 pool exceeds 4 GiB, i.e. batch 256 in one graph;
# its configuration is batch 256 over 8 GPUs = 32 per handle.
DEFAULT_BATCH = {"ssd_tail": 64, "vgg19": 32, "ssd_backbone": 32, "ssd_full": 8}
L2_BYTES = 126e6
REGION_SECONDS = 1.5     # length of the device-timed region (all repetitions together)


def make_workload(wl, name, batch):
    if name == "resnet50":
        return wl.resnet50(batch)
    if name == "mobilenet":
        return wl.mobilenet_v1(batch)
    if name == "vgg19":
        return wl.vgg19(batch)
    if name == "conv_chain":
        return wl.conv_chain(batch)
    if name == "ssd_tail":
        return wl.ssd_tail(batch)
    if name == "ssd_backbone":
        return wl.ssd_backbone(batch)
    if name == "ssd_full":   # image -> boxes in one graph: backbone, heads, transposes / concats, valid counts, NMS
        return wl.ssd_full(batch, size=512, classes=21)
    raise SystemExit("unknown workload " + name)


def units_per_step(name, batch, wl):
    return batch * wl.SSD_ANCHORS if name == "ssd_tail" else batch


def activation_bytes(graph_json):
    """Elements every operator of the graph writes per step (one byte each where the tensor is held
    as int8, which is all of them in the image networks)."""
    gj = json.loads(graph_json)
    shapes = gj["attrs"]["shape"][1]
    rp = gj["node_row_ptr"]
    return sum(int(np.prod(shapes[rp[nid]])) for nid, nd in enumerate(gj["nodes"]) if nd["op"] != "null")


def fits_l2(graph_json):
    return activation_bytes(graph_json) < 2 * L2_BYTES


def config_of(workload, batch, world, graph_json):
    """The configuration record; identical for both arms (`--impl ours` and `--impl reference`)."""
    act = activation_bytes(graph_json)
    l2 = ("operators write %.0f M elements per step against a %.0f MB L2: " % (act / 1e6, L2_BYTES / 1e6)) + (
        "the working set fits L2, so every step is timed on its own with a 256 MB buffer overwritten in front of it"
        if fits_l2(graph_json) else "inputs larger than L2, no flush between steps")
    return {"workload": "%s batch %d per GPU (global batch %d), seeded synthetic int8 weights/inputs"
                        % (workload, batch, batch * world),
            "parallelism": "batch-sharded replicas x%d, no collective" % world, "l2": l2}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML in-process every
    2 ms (read-only queries), nvidia-smi polling as the fallback."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
                   ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index, uuid=None):
        self.gpu = gpu_index
        self.uuid = uuid
        self.rows = []
        self.proc = None
        self.nvml = None
        self.handle = None
        self.stop_flag = threading.Event()
        self.sm, self.smax, self.reasons = [], [], set()

    def _nvml_open(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if self.uuid:
                for cand in (self.uuid, "GPU-" + self.uuid):
                    try:
                        h = pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:
                        h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.nvml, self.handle = pynvml, h
            self.smax.append(float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)))
            return True
        except Exception:
            self.nvml = None
            return False

    def _nvml_loop(self):
        nv, h = self.nvml, self.handle
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                if reasons_fn:
                    mask = int(reasons_fn(h))
                    for name, bit in self.REASON_BITS:
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._nvml_open():
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([t.strip() for t in line.split(",")])

    def stop(self):
        if self.nvml:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                    "sm_max_mhz": max(self.smax) if self.smax else None, "samples": len(self.sm),
                    "reasons": sorted(self.reasons), "source": "nvml, 2 ms period"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi, 200 ms period"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------
# CPU legs: the reference CPU runtime (oracle/_ref, else the numpy port) in clean child processes
# ---------------------------------------------------------------------------------------------
def cpu_child(workload, batch, repeats, handshake, warm=1):
    """Child process body: loads the sample model into the reference runtime, runs `warm` untimed
    inferences, then times `repeats` inferences.  With `handshake` it prints READY and waits for a
    line on stdin first, so that several children can be started together.  Prints one JSON line."""
    pkg = ge.load_package()
    oracle = ge.load_oracle()
    wl = pkg.workloads
    js, pb, x = make_workload(wl, workload, batch)
    if oracle.ref_lib.available():
        m = oracle.ref_lib.RefModel(js, pb, 0)
        if not m.loaded:
            raise SystemExit("reference refused the sample model")
        run = lambda: m.infer(x)
        kind = "reference"
    else:
        run = lambda: oracle.run_model(js, pb, x)
        kind = "port"
    for _ in range(max(1, warm)):   # warm: first touch of the pool
        run()
    if handshake:
        sys.stdout.write("READY\n")
        sys.stdout.flush()
        sys.stdin.readline()
    t0 = time.perf_counter()
    for _ in range(repeats):
        run()
    dt = time.perf_counter() - t0
    sys.stdout.write("\n" + json.dumps({"seconds": dt, "repeats": repeats, "batch": batch, "kind": kind}) + "\n")
    sys.stdout.flush()


def _child_cmd(workload, batch, repeats, handshake, warm=1):
    return [sys.executable, os.path.abspath(__file__), "--cpu-child", workload, str(batch), str(repeats),
            "1" if handshake else "0", str(warm)]


def _child_env(threads):
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = str(threads)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "OMP_PROC_BIND", "GOMP_CPU_AFFINITY"):
        env.pop(k, None)
    return env


def _last_json(text):
    for line in reversed(text.splitlines()):
        line = line.strip()
        if line.startswith("{") and line.endswith("}"):
            return json.loads(line)
    raise RuntimeError("CPU child printed no result: " + text[-400:])


def cpu_run(workload, batch, repeats, threads, warm=1):
    """One child process with `threads` OpenMP threads; returns its timing record."""
    out = subprocess.run(_child_cmd(workload, batch, repeats, False, warm), env=_child_env(threads), check=True,
                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True).stdout
    r = _last_json(out)
    return r


def cpu_process_parallel(workload, batch_each, repeats, procs):
    """`procs` single-thread processes, each on its own shard of `batch_each` images, started together."""
    children = [subprocess.Popen(_child_cmd(workload, batch_each, repeats, True), env=_child_env(1),
                                 stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                for _ in range(procs)]
    for c in children:
        while True:
            line = c.stdout.readline()
            if not line:
                raise RuntimeError("CPU child ended before it was ready")
            if line.strip() == "READY":
                break
    t0 = time.perf_counter()
    for c in children:
        c.stdin.write("go\n")
        c.stdin.flush()
    results = [_last_json(c.communicate()[0]) for c in children]
    wall = time.perf_counter() - t0
    return results, wall


CPU_SAMPLES = {   # workload: (batch for one thread, batch for all threads, batch per process)
    "resnet50": (4, 16, 2), "mobilenet": (8, 32, 4), "vgg19": (1, 4, 1), "conv_chain": (16, 64, 8),
    "ssd_tail": (8, 16, 4), "ssd_backbone": (1, 2, 1), "ssd_full": (1, 2, 1),
}


def cpu_baseline(workload, wl):
    """The three CPU figures: one thread, all threads, one single-thread process per core."""
    cores = os.cpu_count() or 1
    b1, ball, bproc = CPU_SAMPLES[workload]
    per_image = units_per_step(workload, 1, wl)
    one = cpu_run(workload, b1, 1, 1)
    allt = cpu_run(workload, ball, 2, cores)
    results, wall = cpu_process_parallel(workload, bproc, 2, cores)
    v_one = per_image * one["batch"] * one["repeats"] / one["seconds"]
    v_all = per_image * allt["batch"] * allt["repeats"] / allt["seconds"]
    v_proc = per_image * sum(r["batch"] * r["repeats"] for r in results) / max(r["seconds"] for r in results)
    unit = UNITS[workload]
    return {
        "value": v_all, "unit": unit, "cores": cores, "kind": allt["kind"],
        "sample": "%s batch %d, 2 timed inferences after 1 warm-up, OpenMP threads = %d (clean child process)"
                  % (workload, ball, cores),
        "one_thread": {"value": v_one, "unit": unit, "cores": 1,
                       "sample": "%s batch %d, 1 timed inference after 1 warm-up, OMP_NUM_THREADS=1" % (workload, b1)},
        "process_parallel": {"value": v_proc, "unit": unit, "cores": cores,
                             "sample": "%d single-thread processes, each %s batch %d x 2 inferences, started "
                                       "together; total units / slowest process (wall %.2f s)"
                                       % (cores, workload, bproc, wall)},
    }


def run_reference(args, wl, rank, world):
    """The reference arm: the reference's own CPU runtime with every host thread; one step = one
    inference of a bounded sample (the configuration's batch does not fit the time allowed)."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    _, ball, _ = CPU_SAMPLES[args.workload]
    r = cpu_run(args.workload, ball, args.steps, cores, warm=max(1, args.warmup))
    dt = r["seconds"] / r["repeats"]
    units = units_per_step(args.workload, ball, wl)
    value = units / dt
    sample = ("each step = one %s batch-%d inference on the host cores (OpenMP threads = %d); the rate does not "
              "depend on the batch: the reference walks the batch serially" % (args.workload, ball, cores))
    line = {
        "impl": "reference", "metric": METRIC if args.workload == "resnet50" else args.workload + " " + UNITS[args.workload],
        "value": value, "unit": UNITS[args.workload], "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32 storage, int8 products (reference CPU)", "data": "synthetic",
        "config": config_of(args.workload, args.batch, world, make_workload(wl, args.workload, args.batch)[0]),
        "cpu_baseline": {"value": value, "unit": UNITS[args.workload], "cores": cores, "kind": r["kind"], "sample": sample},
        "e2e": {"value": value, "unit": UNITS[args.workload], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# graph arithmetic: operations and compulsory bytes per node
# ---------------------------------------------------------------------------------------------
def node_table(graph_json):
    """{node name: dict(op, x shape, w shape, out shape, ops, bytes)} for conv2d / dense / max_pool2d
    / sum nodes.  ops = 2 * MACs; bytes = inputs + outputs at one byte per activation (every such
    tensor of the benchmark networks is held as int8), weights one byte, bias four."""
    gj = json.loads(graph_json)
    shapes = gj["attrs"]["shape"][1]
    rp = gj["node_row_ptr"]
    attrs = gj["attrs"]["op_attrs"][1]
    out = {}
    for nid, nd in enumerate(gj["nodes"]):
        if nd["op"] == "null":
            continue
        fn = nd["attrs"]["func_name"]
        if fn not in ("conv2d", "dense", "max_pool2d", "sum"):
            continue
        xs = shapes[rp[nd["inputs"][0][0]] + nd["inputs"][0][1]]
        o = shapes[rp[nid]]
        rec = {"op": fn, "x": xs, "out": o, "ops": 0, "groups": 1, "w": None,
               "bytes": int(np.prod(xs)) + int(np.prod(o))}
        if fn in ("conv2d", "dense"):
            w = shapes[rp[nd["inputs"][1][0]]]
            rec["w"] = w
            rec["groups"] = int(json.loads(attrs[nid]).get("groups", "1"))
            rec["ops"] = 2 * int(np.prod(o)) * int(np.prod(w[1:]))
            rec["bytes"] += int(np.prod(w)) + 4 * int(w[0])
        out[nd["name"]] = rec
    return out


def tc_conv_ops(graph_json):
    """2 * MACs of the conv2d / dense nodes that run on the tensor-core kernel (groups = 1,
    input channels a multiple of 32, output channels a multiple of 8)."""
    total = 0
    for rec in node_table(graph_json).values():
        if rec["op"] in ("conv2d", "dense") and rec["groups"] == 1 and rec["x"][1] % 32 == 0 and rec["w"][0] % 8 == 0:
            total += rec["ops"]
    return total


def label_name(label):
    """'conv2d:conv2d_3[tc]' -> ('conv2d_3', 'tc'); 'max_pool2d:max_pool2d_0' -> ('max_pool2d_0', '')."""
    kind = ""
    if label.endswith("]") and "[" in label:
        kind = label[label.rfind("[") + 1:-1]
        label = label[:label.rfind("[")]
    parts = label.split(":")
    return (parts[1] if len(parts) > 1 else parts[0]), kind


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Harness:
    """Process-wide pieces of the GPU arm: device, rank plumbing, timing helpers."""

    def __init__(self, args):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the operator path has no CPU fallback")
        torch.cuda.set_device(self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist_mod
            self.dist = dist_mod
            self.dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        pkg = ge.load_package()
        self.wl, self.rt = pkg.workloads, pkg.runtime
        self.args = args
        try:
            self.gpu_uuid = str(torch.cuda.get_device_properties(self.local_rank).uuid)
        except Exception:
            self.gpu_uuid = None

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if not self.dist:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def h2d_rate(self, nbytes, reps=12):
        """GB/s of plain page-locked -> device copies of `nbytes`, every rank copying at the same
        time (barrier before the timed copies, slowest rank counts): the rate the box gives the
        uploads of an end-to-end step when all GPUs ask at once."""
        torch = self.torch
        src = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
        dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        for _ in range(2):
            dst.copy_(src, non_blocking=True)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        e1.record()
        e1.synchronize()
        ms = self.max_over_ranks(e0.elapsed_time(e1))
        self.barrier()
        return nbytes * reps / (ms * 1e-3) / 1e9

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()
            self.dist = None

    def measure(self, workload, batch, steps, warmup, region_s=REGION_SECONDS, e2e=True, sample_clocks=False,
                profile=True, flush=False):
        """Loads one model and times it: device-resident replays (R repetitions of exactly `steps`
        steps, each bracketed by a barrier), the C-ABI loop with host buffers, and one
        launch-by-launch pass for the per-kernel table.  With `flush` (models whose tensors fit the
        L2) every step is replayed and timed on its own, and a 256 MB buffer is overwritten in front
        of it, outside the timed events."""
        rt, wl, torch = self.rt, self.wl, self.torch
        js, pb, x = make_workload(wl, workload, batch)
        if flush is None:
            flush = fits_l2(js)
        net = rt.CVMAPILoadModel(js, pb, self.local_rank)
        out = np.empty(rt.CVMAPIGetOutputLength(net), dtype=np.uint8)
        res = {"workload": workload, "batch": batch, "launches": int(rt.step_count(net)),
               "units": units_per_step(workload, batch, wl), "graph_json": js,
               "device_bytes": int(rt.device_bytes(net)), "in_bytes": int(x.nbytes), "out_bytes": int(out.nbytes)}
        res["activation_bytes"] = dict(zip(("buffers", "physical"), rt.activation_bytes(net)))
        rt.inference_bytes(net, x, out)

        # ---- end to end through the C-ABI: a page-locked caller buffer (uploaded in place) and an
        # ordinary pageable numpy buffer (staged by the library), upload + download inside the region
        if e2e:
            pinned = torch.empty(x.nbytes, dtype=torch.uint8, pin_memory=True)
            x_pinned = pinned.numpy()
            x_pinned[:] = np.ascontiguousarray(x).view(np.uint8).reshape(-1)

            def e2e_loop(buf):
                for _ in range(warmup):
                    rt.inference_bytes(net, buf, out)
                times = []
                spent = 0.0
                while spent < region_s / 3 or len(times) < 3:
                    self.barrier()
                    t0 = time.perf_counter()
                    for _ in range(steps):
                        rt.inference_bytes(net, buf, out)
                    torch.cuda.synchronize()
                    dt = self.max_over_ranks(time.perf_counter() - t0)
                    times.append(dt)
                    spent += dt
                    if len(times) >= 64:
                        break
                return statistics.median(times) / steps, min(times) / steps, len(times)
            res["e2e_pageable"] = e2e_loop(x)
            res["e2e_pinned"] = e2e_loop(x_pinned)

        # ---- device-resident
        rt.replay_device(net, max(warmup, 3))
        sampler = None
        if sample_clocks and self.rank == 0:
            sampler = ClockSampler(self.local_rank, self.gpu_uuid)
            sampler.start()
        times = []
        spent = 0.0
        scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
        while spent < region_s or len(times) < 3:
            self.barrier()
            if flush:
                ms = 0.0
                for _ in range(steps):
                    scratch.fill_(1)
                    torch.cuda.synchronize()
                    ms += rt.replay_device(net, 1)
                ms = self.max_over_ranks(ms)
            else:
                ms = self.max_over_ranks(rt.replay_device(net, steps))
            times.append(ms)
            spent += ms * 1e-3
            if len(times) >= 256:
                break
        self.barrier()
        res["clocks"] = sampler.stop() if sampler else None
        res["dev_ms_median"] = statistics.median(times) / steps
        res["dev_ms_best"] = min(times) / steps
        res["repeats"] = len(times)
        res["flushed"] = bool(flush)

        # ---- per-kernel attribution (launch by launch, CUDA events in between; rank 0)
        res["rows"] = []
        if profile and self.rank == 0:
            reps = 3
            acc = {}
            order = []
            for _ in range(reps):
                for i, (label, ms) in enumerate(rt.profile_steps(net, x)):
                    key = (i, label)
                    if key not in acc:
                        acc[key] = 0.0
                        order.append(key)
                    acc[key] += ms
            res["rows"] = [(label, acc[(i, label)] / reps) for i, label in order]
        rt.CVMAPIFreeModel(net)
        return res


def kernels_table(rows):
    agg = {}
    for label, ms in rows:
        _, kind = label_name(label)
        kind = kind or label.split(":")[0]
        a = agg.setdefault(kind, [0, 0.0])
        a[0] += 1
        a[1] += ms
    total = sum(v[1] for v in agg.values())
    return {k: {"launches_per_step": v[0], "ms_per_step": v[1], "share": v[1] / total if total else 0.0}
            for k, v in agg.items()}


def layer_rates(res, want_kind=None):
    """Per launch: TOP/s (tensor-core layers) and GB/s against the compulsory bytes."""
    table = node_table(res["graph_json"])
    out = []
    for label, ms in res["rows"]:
        name, kind = label_name(label)
        rec = table.get(name)
        if rec is None or (want_kind and kind not in want_kind):
            continue
        out.append({"name": name, "kind": kind or rec["op"], "x": rec["x"], "w": rec["w"], "ms": ms,
                    "tops": rec["ops"] / (ms * 1e-3) / 1e12 if ms > 0 else None,
                    "gbs": rec["bytes"] / (ms * 1e-3) / 1e9 if ms > 0 else None})
    return out


def run_ours(args):
    h = Harness(args)
    rt, wl = h.rt, h.wl
    rank, world = h.rank, h.world
    head = h.measure(args.workload, args.batch, args.steps, args.warmup, sample_clocks=True, flush=None)
    h2d_gbs = h.h2d_rate(head["in_bytes"])
    peaks = measured_peaks()
    line = None
    if rank == 0:
        kernels = kernels_table(head["rows"])
        roofline = None
        peak_i8 = rt.measure_i8_mma_rate(256, 20000)
        if "tc" in kernels:
            tc_ops = tc_conv_ops(head["graph_json"])
            tc_ms = kernels["tc"]["ms_per_step"]
            achieved = tc_ops / (tc_ms * 1e-3) / 1e12
            roofline = {
                "kernel": "conv_tc_kernel (tcgen05 kind::i8 implicit GEMM, all groups=1 conv2d + dense)",
                "bound": "tensor", "achieved": achieved, "peak": peak_i8, "unit": "TFLOP/s",
                "frac": achieved / peak_i8, "traffic": None,
                "note": "int8 multiply-accumulates counted as 2 ops (TOP/s); achieved = ops of the tensor-core "
                        "launches / the sum of their CUDA-event times in a launch-by-launch pass (the graph "
                        "replay overlaps launches and is faster); peak = the int8 tcgen05.mma rate measured in "
                        "this run (M128 N256 K32 instructions back to back on all SMs); against 2 x the %s "
                        "bf16 cuBLAS figures the fraction is %.3f (sustained %.1f) / %.3f (burst %.1f), against "
                        "the nominal 4500 dense TOP/s %.3f; launches_per_step=%d, avg launch %.1f us; traffic: "
                        "not captured in this run (ncu summaries under profiles/)" % (
                            peaks["source"], achieved / (2.0 * peaks["bf16_sustained"]), peaks["bf16_sustained"],
                            achieved / (2.0 * peaks["bf16"]), peaks["bf16"], achieved / 4500.0,
                            kernels["tc"]["launches_per_step"],
                            1e3 * tc_ms / max(1, kernels["tc"]["launches_per_step"])),
                "kernels": kernels,
            }
            # The kernel runs layers of very different shape: some cannot be faster than their
            # compulsory bytes over the HBM copy rate, others than their ops over the MMA rate.  The
            # sum over layers of the larger of the two is the floor of this kernel on this network
            # (bytes: input + output + weights + bias of a layer at one byte per activation; the
            # int8 operand of a fused residual add is not counted, so the floor is on the low side).
            floor_ms = 0.0
            for x in layer_rates(head, want_kind=("tc",)):
                rec = node_table(head["graph_json"])[x["name"]]
                floor_ms += 1e3 * max(rec["ops"] / (peak_i8 * 1e12), rec["bytes"] / (peaks["hbm_gbs"] * 1e9))
            roofline["layer_floor"] = {"ms_per_step": floor_ms, "frac": floor_ms / tc_ms if tc_ms else None,
                                       "note": "sum over the kernel's launches of max(ops / measured int8 MMA rate, compulsory "
                                               "bytes / measured HBM copy rate); frac = that floor / the launches' summed time"}
        elif "non_max_suppression" in kernels:
            nbytes = 2.0 * args.batch * wl.SSD_ANCHORS * 6 * 4
            ms = kernels["non_max_suppression"]["ms_per_step"]
            achieved = nbytes / (ms * 1e-3) / 1e9
            roofline = {"kernel": "nms_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                        "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None, "kernels": kernels}
        total_units = head["units"] * world
        e2e_med, e2e_best, e2e_reps = head["e2e_pinned"]
        line = {
            "metric": METRIC if args.workload == "resnet50" else args.workload + " " + UNITS[args.workload],
            "value": total_units / (head["dev_ms_median"] * 1e-3), "unit": UNITS[args.workload], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["dev_ms_median"],
            "ms_per_step_best": head["dev_ms_best"], "repeats": head["repeats"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 operands, int32 accumulate", "data": "synthetic",
            "config": config_of(args.workload, args.batch, world, head["graph_json"]),
            "timing": "median over %d repetitions of %d device-timed steps (CUDA events on the model's stream, "
                      "max over ranks per repetition)" % (head["repeats"], args.steps),
            "e2e": {"value": total_units / e2e_med, "unit": UNITS[args.workload],
                    "h2d_bytes_per_step": head["in_bytes"], "d2h_bytes_per_step": head["out_bytes"] + 4,
                    "ms_per_step": 1e3 * e2e_med, "ms_per_step_best": 1e3 * e2e_best, "repeats": e2e_reps,
                    "input": "page-locked host buffer",
                    "pageable_input_value": total_units / head["e2e_pageable"][0],
                    # what the uploads alone would allow: every rank copying its input at once
                    "h2d_copy_gbs_per_gpu": h2d_gbs,
                    "upload_bound_value": total_units / (head["in_bytes"] / (h2d_gbs * 1e9))},
            "gpu_launches": head["launches"] * args.steps * head["repeats"],
            "device_bytes": head["device_bytes"], "activation_bytes": head["activation_bytes"],
            "clocks": head["clocks"], "roofline": roofline,
        }

    # ---- strong scaling: the same network with the global batch 256 split over the ranks
    if world > 1 and not args.no_extra and args.workload == "resnet50" and 256 % world == 0:
        per = 256 // world
        s = h.measure(args.workload, per, args.steps, args.warmup, region_s=0.75, profile=False)
        if rank == 0:
            line["strong"] = {
                "global_batch": 256, "per_gpu": per, "n_gpus": world,
                "value": 256 / (s["dev_ms_median"] * 1e-3), "unit": UNITS[args.workload],
                "ms_per_step": s["dev_ms_median"], "ms_per_step_best": s["dev_ms_best"],
                "e2e_value": 256 / s["e2e_pinned"][0], "e2e_ms_per_step": 1e3 * s["e2e_pinned"][0],
                "e2e_pageable_value": 256 / s["e2e_pageable"][0]}

    # ---- the other figures of the metric (one GPU)
    if world == 1 and rank == 0 and not args.no_extra and args.workload == "resnet50":
        line["extra"] = extras(h, args, peak_i8, peaks)

    h.barrier()
    h.close()
    if rank == 0:
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload, wl)
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)


def extras(h, args, peak_i8, peaks):
    """conv2d TOP/s (conv chain, VGG-19 layers), NMS boxes/s, MobileNet, bandwidth kernels."""
    K, W = args.steps, args.warmup
    ex = {"note": "same run, same GPU; device-resident CUDA-event medians; fractions are of the rates measured "
                  "in this run (int8 tensor: %.0f TOP/s) and of the %s HBM copy rate (%.0f GB/s)"
                  % (peak_i8, peaks["source"], peaks["hbm_gbs"])}
    tops = {}
    for b in (64, 256):
        r = h.measure("conv_chain", b, K, W, region_s=0.4, flush=None)
        conv = [x for x in layer_rates(r) if x["kind"] == "tc"]
        ops = tc_conv_ops(r["graph_json"])
        rec = {"graph_ms_per_step": r["dev_ms_median"], "images_per_s": b / (r["dev_ms_median"] * 1e-3),
               "e2e_images_per_s": b / r["e2e_pinned"][0]}
        if conv:
            rec.update({"conv_kernel_ms": conv[0]["ms"], "tops": conv[0]["tops"], "frac": conv[0]["tops"] / peak_i8})
        else:
            rec.update({"tops": ops / (r["dev_ms_median"] * 1e-3) / 1e12})
        tops["conv_chain_b%d" % b] = rec
    for b in (32, 64):
        r = h.measure("vgg19", b, K, W, region_s=0.4, e2e=(b == 32))
        layers = layer_rates(r, want_kind=("tc",))
        big = [x for x in layers if x["w"] and len(x["w"]) == 4 and x["w"][2] == 3 and x["x"][1] >= 256]
        ops_big = sum(node_table(r["graph_json"])[x["name"]]["ops"] for x in big)
        ms_big = sum(x["ms"] for x in big)
        rec = {"graph_ms_per_step": r["dev_ms_median"], "images_per_s": b / (r["dev_ms_median"] * 1e-3),
               "conv3x3_256_512ch": {"layers": len(big), "tops": ops_big / (ms_big * 1e-3) / 1e12 if ms_big else None,
                                     "frac": ops_big / (ms_big * 1e-3) / 1e12 / peak_i8 if ms_big else None,
                                     "best_layer_tops": max(x["tops"] for x in big) if big else None,
                                     "worst_layer_tops": min(x["tops"] for x in big) if big else None},
               "all_tc_layers_tops": tc_conv_ops(r["graph_json"]) / (sum(x["ms"] for x in layers) * 1e-3) / 1e12,
               "fc6_25088x4096": next(({"ms": x["ms"], "tops": x["tops"], "weight_gbs": x["gbs"]} for x in layers
                                       if x["w"] and len(x["w"]) == 2 and x["w"][1] == 25088), None)}
        if b == 32:
            rec["e2e_images_per_s"] = b / r["e2e_pinned"][0]
        tops["vgg19_b%d" % b] = rec
    ex["conv2d_tops"] = tops

    nms = {}
    for b in (1, 64):
        r = h.measure("ssd_tail", b, K, W, region_s=0.3, flush=None)
        kt = kernels_table(r["rows"])
        nbytes = 2.0 * b * h.wl.SSD_ANCHORS * 6 * 4
        rec = {"boxes_per_s": r["units"] / (r["dev_ms_median"] * 1e-3), "ms_per_step": r["dev_ms_median"],
               "e2e_boxes_per_s": r["units"] / r["e2e_pinned"][0], "e2e_ms_per_step": 1e3 * r["e2e_pinned"][0]}
        for k, v in kt.items():
            rec[k + "_ms"] = v["ms_per_step"]
            if k in ("non_max_suppression", "get_valid_counts"):
                rec[k + "_gbs"] = nbytes / (v["ms_per_step"] * 1e-3) / 1e9
                rec[k + "_frac_hbm"] = rec[k + "_gbs"] / peaks["hbm_gbs"]
        nms["ssd_tail_b%d" % b] = rec
    ex["nms_boxes_per_s"] = nms

    r = h.measure("mobilenet", 256, K, W, region_s=0.4)
    dw = [x for x in layer_rates(r) if x["kind"] == "dw"]
    ex["mobilenet_b256"] = {
        "images_per_s": 256 / (r["dev_ms_median"] * 1e-3), "ms_per_step": r["dev_ms_median"],
        "e2e_images_per_s": 256 / r["e2e_pinned"][0],
        "depthwise3x3": {"layers": len(dw), "gbs_min": min(x["gbs"] for x in dw) if dw else None,
                         "gbs_max": max(x["gbs"] for x in dw) if dw else None,
                         "gbs_all": (sum(node_table(r["graph_json"])[x["name"]]["bytes"] for x in dw) /
                                     (sum(x["ms"] for x in dw) * 1e-3) / 1e9) if dw else None,
                         "ms": sum(x["ms"] for x in dw)}}
    if ex["mobilenet_b256"]["depthwise3x3"]["gbs_all"]:
        ex["mobilenet_b256"]["depthwise3x3"]["frac_hbm"] = ex["mobilenet_b256"]["depthwise3x3"]["gbs_all"] / peaks["hbm_gbs"]
    return ex


def main():
    if len(sys.argv) > 1 and sys.argv[1] == "--cpu-child":
        cpu_child(sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), sys.argv[5] == "1", int(sys.argv[6]))
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50", choices=sorted(UNITS))
    ap.add_argument("--batch", type=int, default=None, help="images per GPU (default 256; ssd_tail 64)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra metrics / strong-scaling block")
    ap.add_argument("--inferences", type=int, default=0,
                    help="profiling aid: load the workload, run this many plain inferences through the C-ABI and exit "
                         "(no timing, no JSON line); what a profiler capture of a few launches needs")
    args = ap.parse_args()
    if args.batch is None:
        args.batch = DEFAULT_BATCH.get(args.workload, 256)
    if args.impl == "reference":
        pkg = ge.load_package()
        run_reference(args, pkg.workloads, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")))
        return
    if args.inferences > 0:
        pkg = ge.load_package()
        js, pb, x = make_workload(pkg.workloads, args.workload, args.batch)
        net = pkg.runtime.CVMAPILoadModel(js, pb, 0)
        for _ in range(args.inferences):
            pkg.runtime.inference_bytes(net, x)
        pkg.runtime.CVMAPIFreeModel(net)
        print("ran %d inference(s) of %s batch %d" % (args.inferences, args.workload, args.batch))
        return
    args.warmup = max(args.warmup, 3)
    run_ours(args)


if __name__ == "__main__":
    main()
