#!/usr/bin/env python3
"""Benchmark of the quantized-inference hot path: ResNet-50 v1.5 int8 images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the network over one batch (64 images per GPU) of seeded
synthetic uint8 input, built through the tim::vx API (tim-vx_b200/samples).
Work shards by batch: every rank owns a full replica on its own GPU and there
is no collective on the data path ("scaling": "weak").

Printed on rank 0, one JSON line:
  value     images/s over all GPUs, inputs already resident in HBM, timed with
            CUDA events on the launching stream, max over ranks
  e2e       images/s through Tensor::CopyDataToTensor -> Graph::Run ->
            Tensor::CopyDataFromTensor with pinned host buffers inside the timed region; the
            steps are shared by --e2e-threads host threads (default 3), each with its own
            replica of the graph, so that one replica's copies overlap the other's kernels
  roofline  the dominant kernel (the tcgen05 int8 GEMM over all its launches of one
            step), per-kernel CUDA-event times measured live by b2vx_graph_profile;
            int8_peak_measured is the tensor pipe's dense int8 rate from an issue-rate
            microbenchmark run on the spot (b2vx_measure_int8_peak)
  sustained the same graph replayed back to back for at least two seconds, with the
            median SM clock and power sampled meanwhile
  configs   (N=1, default workload) one number each for the other benchmark
            configurations: LeNet, the convolution sweep, MobileNetV2, the GEMM sweep,
            the decode-like FullyConnected shapes and the 64 Mi-element Add
  cpu_baseline  the CPU oracle (a restatement, "port") on a bounded sample, rank 0, N=1

--impl reference times that CPU oracle as the reference arm (the reference's own
arithmetic sits in a closed driver that is not in its tree, so there is no
reference binary to run).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tim-vx_b200"))

SAMPLES_LIB = os.path.join(ROOT, "tim-vx_b200", "samples", "libb2vx_samples.so")
SAMPLES_ORACLE_LIB = os.path.join(ROOT, "oracle", "_build", "libb2vx_samples_oracle.so")


def load_samples(path):
    lib = C.CDLL(path)
    vp = C.c_void_p
    lib.b2vx_net_create.restype = vp
    lib.b2vx_net_create.argtypes = [C.c_char_p, C.c_int32, C.c_uint64, C.c_int32]
    lib.b2vx_net_destroy.argtypes = [vp]
    lib.b2vx_net_input_bytes.restype = C.c_size_t
    lib.b2vx_net_input_bytes.argtypes = [vp]
    lib.b2vx_net_output_bytes.restype = C.c_size_t
    lib.b2vx_net_output_bytes.argtypes = [vp]
    lib.b2vx_net_synthetic_input.argtypes = [vp, C.c_uint64, vp]
    lib.b2vx_net_set_input.restype = C.c_int32
    lib.b2vx_net_set_input.argtypes = [vp, vp]
    lib.b2vx_net_run.restype = C.c_int32
    lib.b2vx_net_run.argtypes = [vp]
    lib.b2vx_net_get_output.restype = C.c_int32
    lib.b2vx_net_get_output.argtypes = [vp, vp]
    lib.b2vx_net_graph_handle.restype = vp
    lib.b2vx_net_graph_handle.argtypes = [vp]
    lib.b2vx_net_macs_per_image.restype = C.c_uint64
    lib.b2vx_net_macs_per_image.argtypes = [vp]
    return lib


TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic.json")


def dram_traffic(workload, batch):
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel's launches in one step, as
    recorded from an ncu capture by --traffic-from; None when no capture of this workload is on file."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f).get("%s:%d" % (workload, batch))
        return rec
    except (OSError, ValueError):
        return None


def record_traffic(args):
    """--traffic-from <csv>: sums dram__bytes_read.sum and dram__bytes_write.sum per kernel over the launches listed
    in an `ncu --csv --metrics dram__bytes_read.sum,dram__bytes_write.sum` log of one step of this workload and
    stores the dominant kernel's total, with the commit the tree is at, in profiles/dram_traffic.json."""
    import csv
    unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    per = {}
    with open(args.traffic_from) as f:
        rows = [r for r in csv.reader(l for l in f if l.startswith('"'))]
    hdr = rows[0]
    ki, mi, ui, vi = hdr.index("Kernel Name"), hdr.index("Metric Name"), hdr.index("Metric Unit"), hdr.index("Metric Value")
    launches = {}
    for r in rows[1:]:
        if r[mi] not in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            continue
        name = r[ki].split("(")[0].split("::")[-1]
        per[name] = per.get(name, 0.0) + float(r[vi].replace(",", "")) * unit.get(r[ui], 1.0)
        if r[mi] == "dram__bytes_read.sum":
            launches[name] = launches.get(name, 0) + 1
    top = max(per, key=lambda n: per[n])
    # both instantiations of the GEMM kernel count as one kernel
    total = sum(v for n, v in per.items() if n.split("<")[0] == top.split("<")[0])
    count = sum(v for n, v in launches.items() if n.split("<")[0] == top.split("<")[0])
    try:
        commit = subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], capture_output=True, text=True).stdout.strip()
    except OSError:
        commit = ""
    try:
        with open(TRAFFIC_FILE) as f:
            table = json.load(f)
    except (OSError, ValueError):
        table = {}
    table["%s:%d" % (args.workload, args.batch)] = {"bytes": total, "kernel": top.split("<")[0], "launches": count, "commit": commit,
                                                    "source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one step"}
    with open(TRAFFIC_FILE, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
        f.write("\n")
    print(json.dumps(table["%s:%d" % (args.workload, args.batch)]))
    return 0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons, watts = [], None, set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 8:
                continue
            try:
                mhz.append(float(f[1]))
                mx = float(f[2])
                watts.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        watts.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz), "power_w": watts[len(watts) // 2] if watts else None}



class NetWorkload:
    """A sample network (tim-vx_b200/samples) built through the tim::vx C++ API."""

    def __init__(self, lib_path, name, batch, seed, device):
        self.lib = load_samples(lib_path)
        self.net = self.lib.b2vx_net_create(name.encode(), batch, seed, device)
        assert self.net, "network creation failed"
        self.in_bytes = self.lib.b2vx_net_input_bytes(self.net)
        self.out_bytes = self.lib.b2vx_net_output_bytes(self.net)
        self.units = batch
        macs = self.lib.b2vx_net_macs_per_image(self.net)
        self.ops = 2 * macs * batch
        self.metric, self.unit = "%s_int8_images_per_sec" % name, "images/s"
        self.scale = 1.0        # metric units per processed unit
        self.describe = {"resnet50": "resnet50 v1.5 int8, 224x224x3 uint8 input, batch %d per GPU, per-channel int8 weights",
                         "mobilenetv2": "mobilenetv2-1.0 uint8 asymmetric, 224x224x3 input, batch %d per GPU",
                         "lenet": "lenet-5 uint8 asymmetric, 28x28x1 input, batch %d per GPU"}.get(name, name + " batch %d") % batch

    def graph_handle(self):
        return C.c_void_p(self.lib.b2vx_net_graph_handle(self.net))

    def synthetic_input(self, seed, ptr):
        self.lib.b2vx_net_synthetic_input(self.net, seed, C.c_void_p(ptr))

    def set_input(self, ptr):
        assert self.lib.b2vx_net_set_input(self.net, C.c_void_p(ptr)) == 0

    def run(self):
        assert self.lib.b2vx_net_run(self.net) == 0

    def get_output(self, ptr):
        assert self.lib.b2vx_net_get_output(self.net, C.c_void_p(ptr)) == 0

    def close(self):
        self.lib.b2vx_net_destroy(self.net)


class OpWorkload:
    """One operator (tim-vx_b200/opworkloads.py) built through the b2vx C ABI."""

    def __init__(self, lib_path, spec, batch, seed, device):
        import numpy as np
        import pyb2vx as B
        import opworkloads
        self.B = B
        self.g = B.Graph(B.load(lib_path), device)
        rng = np.random.default_rng(seed)
        self.w = opworkloads.build(spec, batch, self.g, rng)
        self.g.compile()
        self.in_sizes = [a.nbytes for _, a in self.w["inputs"]]
        self.in_bytes = sum(self.in_sizes)
        self.out_sizes = [int(np.prod(self.g.shape(t))) for t in self.w["outputs"]]
        self.out_bytes = sum(self.out_sizes)
        self.units = self.w["units"]
        self.ops = self.w["ops"]
        kind = spec.split(":")[0]
        if kind == "add":
            self.metric, self.unit, self.scale = "quantized_add_gbytes_per_sec", "GB/s", 3.0 / 1e9
        elif kind in ("concat", "transpose"):
            self.metric, self.unit, self.scale = kind + "_gbytes_per_sec", "GB/s", 2.0 / 1e9   # each element read and written once
        elif kind == "fcchain":
            self.metric, self.unit, self.scale = "fullyconnected_chain_gbytes_per_sec", "GB/s", self.w["bytes"] / self.units / 1e9
        else:
            self.metric = "conv2d_int8_tops" if kind in ("conv", "convadd") else "fullyconnected_int8_tops"
            self.unit, self.scale = "TOP/s", self.ops / self.units / 1e12
        self.describe = self.w["name"]

    def graph_handle(self):
        return self.g.g

    def synthetic_input(self, seed, ptr):
        off = 0
        for (_, a), n in zip(self.w["inputs"], self.in_sizes):
            C.memmove(ptr + off, a.ctypes.data, n)
            off += n

    def set_input(self, ptr):
        off = 0
        for (t, _), n in zip(self.w["inputs"], self.in_sizes):
            self.g.write_ptr(t, ptr + off, n)
            off += n

    def run(self):
        self.g.run()

    def get_output(self, ptr):
        off = 0
        for t, n in zip(self.w["outputs"], self.out_sizes):
            self.g.read_ptr(t, ptr + off, n)
            off += n

    def close(self):
        self.g.close()


def make_workload(args, oracle, batch, device):
    if ":" in args.workload:
        import pyb2vx as B
        lib_path = B.PRODUCT_LIB
        if oracle:   # the CPU baseline / reference arm: the one place outside tests/ that runs the oracle
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import oracle_paths
            lib_path = oracle_paths.ORACLE_LIB
        return OpWorkload(lib_path, args.workload, batch, args.seed, device)
    return NetWorkload(SAMPLES_ORACLE_LIB if oracle else SAMPLES_LIB, args.workload, batch, args.seed, device)


def run_reference(args):
    """Reference arm: the CPU oracle (a port of the path; see module docstring) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # all host threads this process may use (torchrun exports OMP_NUM_THREADS=1 to its workers)
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    if not os.path.exists(SAMPLES_ORACLE_LIB):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")], stdout=subprocess.DEVNULL)
    import numpy as np
    sample = args.cpu_batch
    if ":" in args.workload:
        import opworkloads
        args.workload, sample_note = opworkloads.cpu_sample(args.workload)
    else:
        sample_note = "%d images per step (bounded sample of the %d-image batch)" % (sample, args.batch)
    wl = make_workload(args, True, sample, 0)
    x = np.empty(wl.in_bytes, np.uint8)
    y = np.empty(wl.out_bytes, np.uint8)
    wl.synthetic_input(args.seed, x.ctypes.data)
    for _ in range(args.warmup):
        wl.set_input(x.ctypes.data)
        wl.run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.set_input(x.ctypes.data)
        wl.run()
        wl.get_output(y.ctypes.data)
    dt = time.perf_counter() - t0
    value = wl.units * args.steps / dt * wl.scale
    cores = C.CDLL(os.path.join(ROOT, "oracle", "_build", "liboracle_ops.so")).orc_num_threads()
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "%s; on host cores: %s" % (wl.describe, sample_note)},
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": cores, "kind": "port",
                         "sample": "%s x %d steps" % (sample_note, args.steps)},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    wl.close()
    return 0


def cpu_baseline_subprocess(args):
    """Runs the oracle in a child process (both sample libraries define the same symbols)."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", args.workload, "--batch", str(args.batch), "--steps", "2",
           "--warmup", "1", "--cpu-batch", str(args.cpu_batch), "--seed", str(args.seed)]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        for line in out.stdout.splitlines():
            if line.startswith("{"):
                return json.loads(line)["cpu_baseline"]
    except Exception as e:   # noqa: BLE001 - reported in the JSON line instead of failing the bench
        return {"value": None, "unit": None, "cores": 0, "kind": "port", "sample": "failed: %s" % e}
    return {"value": None, "unit": None, "cores": 0, "kind": "port", "sample": "no output: %s" % out.stderr[-200:]}


class ArgsView:
    """The few fields make_workload reads, for the extra configurations."""

    def __init__(self, workload, seed):
        self.workload, self.seed = workload, seed


def time_replays(blib, graph, stream, steps, flush):
    """Milliseconds of `steps` replays of a compiled graph on `stream`, inputs resident; with `flush`, a buffer larger
    than the L2 is rewritten before every replay and every replay has its own pair of events."""
    import torch
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            assert blib.b2vx_graph_run_async(graph) == 0
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        flush.fill_(1)
        a.record(stream)
        assert blib.b2vx_graph_run_async(graph) == 0
        b.record(stream)
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs)


def time_replays_streams(blib, lanes, steps):
    """Milliseconds of `steps` replays shared round-robin by the graph replicas in `lanes` ((graph handle, torch stream)
    pairs), each replica on its own stream with its own resident input: kernels of different replicas overlap wherever
    one leaves SMs idle (a layer with fewer tiles than SMs, the tail of a launch, its prologue).  Timed from an event all
    streams wait for to an event that waits for all streams."""
    import torch
    main = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for _, st in lanes:
        st.wait_event(e0)
    for i in range(steps):
        assert blib.b2vx_graph_run_async(lanes[i % len(lanes)][0]) == 0
    for _, st in lanes:
        done = torch.cuda.Event()
        done.record(st)
        main.wait_event(done)
    e1.record(main)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def kernel_table(blib, graph, B, iters, step_ms):
    """Per-kernel times of one step: b2vx_graph_profile puts an event pair around every launch, which costs about
    2 us apiece and breaks the overlap of consecutive kernels, so the event times add up to more than a step of the
    timed region; a kernel's time inside the timed region is taken as its share of the event total times the step."""
    assert blib.b2vx_graph_profile(graph, iters) == 0
    n = C.c_uint32()
    blib.b2vx_graph_kernel_count(graph, C.byref(n))
    per = {}
    for i in range(n.value):
        k = B.KernelInfo()
        blib.b2vx_graph_kernel_info(graph, i, C.byref(k))
        name = k.name.decode().split("(")[0]
        d = per.setdefault(name, {"launches": 0, "ms": 0.0, "ops": 0, "bytes": 0})
        d["launches"] += 1
        d["ms"] += k.last_ms
        d["ops"] += k.ops
        d["bytes"] += k.bytes
    total = sum(d["ms"] for d in per.values()) or 1.0
    for d in per.values():
        d["ms_events"] = d["ms"]
        d["ms"] = d["ms"] / total * step_ms
    return per, n.value


def layer_table(blib, B, graph, stream, args, wl, int8_measured):
    """One line per kernel launch of a step.  A launch's ceiling time is max(ops / int8 peak, algorithmic bytes / HBM copy
    rate); its time inside a step is its event time scaled by step / sum of event times (the events serialise launches
    that overlap in the replayed graph and add about 2 us apiece)."""
    peaks = measured_peaks()
    int8_peak = int8_measured if int8_measured else 2.0 * peaks["bf16_sustained"]
    for _ in range(max(3, args.warmup)):
        assert blib.b2vx_graph_run_async(graph) == 0
    assert blib.b2vx_graph_sync(graph) == 0
    step_ms = min(time_replays(blib, graph, stream, args.steps, None) for _ in range(5)) / args.steps   # best of five rounds
    assert blib.b2vx_graph_profile(graph, max(3, args.profile_iters)) == 0
    n = C.c_uint32()
    blib.b2vx_graph_kernel_count(graph, C.byref(n))
    rows = []
    for i in range(n.value):
        k = B.KernelInfo()
        blib.b2vx_graph_kernel_info(graph, i, C.byref(k))
        rows.append((k.name.decode(), -1 if k.node_index == 0xFFFFFFFF else k.node_index, k.last_ms, k.ops, k.bytes))
    total = sum(r[2] for r in rows) or 1.0
    print("# %s, batch %d: step %.4f ms, %d launches, sum of event times %.4f ms; int8 peak %.0f TOP/s (%s), HBM %.0f GB/s (%s)"
          % (args.workload, args.batch, step_ms, len(rows), total, int8_peak, "measured" if int8_measured else "assumed",
             peaks["hbm_gbs"], peaks["source"]))
    print("# %3s %-44s %5s %9s %9s %9s %8s %8s %6s" % ("i", "kernel", "node", "event_us", "step_us", "ceil_us", "TOP/s", "GB/s", "frac"))
    ceil_total = 0.0
    for i, (name, node, ms, ops, nbytes) in enumerate(rows):
        us = ms / total * step_ms * 1e3
        ceil_us = max(ops / (int8_peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e6
        ceil_total += ceil_us
        print("%5d %-44s %5d %9.2f %9.2f %9.2f %8.1f %8.1f %6.3f" % (i, name[:44], node, ms * 1e3, us, ceil_us, ops / (us * 1e-6) / 1e12 if us else 0.0,
                                                                       nbytes / (us * 1e-6) / 1e9 if us else 0.0, ceil_us / us if us else 0.0))
    print("# sum of ceilings %.1f us = %.3f of the step" % (ceil_total, ceil_total / (step_ms * 1e3)))
    wl.close()
    return 0


def roofline_of(t, hbm_gbs, int8_peak):
    """Achieved rate of one kernel record (ops, bytes, ms) against the roofline min(int8 peak, intensity x HBM)."""
    ai = t["ops"] / max(t["bytes"], 1)
    ridge = int8_peak * 1e12 / (hbm_gbs * 1e9)
    sec = max(t["ms"], 1e-9) / 1e3
    if t["ops"] and ai >= ridge:
        achieved = t["ops"] / sec / 1e12
        return {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak}
    achieved = t["bytes"] / sec / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs}


# The benchmark configurations beside the headline one (workload, batch), timed at N=1 into "configs".
EXTRA_CONFIGS = [("lenet", 1), ("lenet", 256),
                 ("conv:3:64:64:56:1", 1), ("conv:3:64:64:56:1", 32), ("conv:3:64:64:56:1", 256),
                 ("conv:1:64:64:56:1", 256), ("conv:3:64:64:56:2", 256),
                 ("mobilenetv2", 64),
                 ("gemm:1024:1024:1024", 1), ("gemm:2048:2048:2048", 1), ("gemm:4096:4096:4096", 1), ("gemm:8192:8192:8192", 1),
                 ("gemm:1:4096:4096", 1), ("gemm:16:4096:4096", 1), ("gemm:1:8192:8192", 1), ("gemm:16:8192:8192", 1),
                 ("fcchain:1:4096:12", 1), ("fcchain:16:4096:12", 1), ("fcchain:1:8192:4", 1), ("fcchain:16:8192:4", 1),
                 ("add:67108864", 1)]


def run_configs(blib, B, stream, seed, device, hbm_gbs, int8_peak, flush):
    """One record per extra configuration: whole-graph value in the configuration's unit (layout conversion of the
    graph's inputs and outputs included), and the dominant kernel's rate against its roofline."""
    import torch
    out = []
    for spec, batch in EXTRA_CONFIGS:
        rec = {"workload": spec, "batch": batch}
        try:
            wl = make_workload(ArgsView(spec, seed), False, batch, device)
            g = wl.graph_handle()
            assert blib.b2vx_graph_set_stream(g, C.c_void_p(stream.cuda_stream)) == 0
            host_in = torch.empty(wl.in_bytes, dtype=torch.uint8).pin_memory()
            wl.synthetic_input(seed, host_in.data_ptr())
            wl.set_input(host_in.data_ptr())
            for _ in range(3):
                assert blib.b2vx_graph_run_async(g) == 0
            assert blib.b2vx_graph_sync(g) == 0
            steps = 10
            ms = time_replays(blib, g, stream, steps, flush if wl.in_bytes + wl.out_bytes < 256 * 1024 * 1024 else None)
            assert blib.b2vx_graph_sync(g) == 0
            step_ms = ms / steps
            per, launches = kernel_table(blib, g, B, 2, step_ms)
            top = max(per, key=lambda n: per[n]["ms"])
            roof = roofline_of(per[top], hbm_gbs, int8_peak)
            rec.update({"metric": wl.metric, "value": wl.units / (step_ms / 1e3) * wl.scale, "unit": wl.unit, "ms_per_step": step_ms,
                        "launches": launches, "kernel": top, "kernel_ms": per[top]["ms"], "bound": roof["bound"],
                        "achieved": roof["achieved"], "achieved_unit": roof["unit"], "frac": roof["frac"]})
            wl.close()
        except Exception as e:   # noqa: BLE001 - one failing configuration must not lose the headline line
            rec["error"] = str(e)[:200]
        out.append(rec)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None,
                    help="resnet50 (default), mobilenetv2, lenet, or one operator: conv:k:cin:cout:hw:stride, "
                         "convadd:k:cin:cout:hw:stride, gemm:m:n:k, fcchain:m:n:layers, add:elements, concat:c1:c2:hw, transpose:c:hw "
                         "(tim-vx_b200/opworkloads.py)")
    ap.add_argument("--net", default="resnet50", help="older spelling of --workload for the networks")
    ap.add_argument("--batch", type=int, default=64, help="images per GPU per step")
    ap.add_argument("--cpu-batch", type=int, default=4, help="images per step of the CPU baseline sample")
    ap.add_argument("--seed", type=int, default=2024)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer loop (profiler captures)")
    ap.add_argument("--no-configs", action="store_true", help="skip the extra configurations (N=1, default workload)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second sustained replay")
    ap.add_argument("--streams", type=int, default=3,
                    help="graph replicas replayed concurrently, each on its own CUDA stream with its own resident batch (the device-resident "
                         "value; 1 = one graph back to back, which the line also reports as single_stream)")
    ap.add_argument("--e2e-threads", type=int, default=4,
                    help="host threads (each with its own graph replica and pinned buffers) sharing the steps of the end-to-end loop")
    ap.add_argument("--e2e-repeats", type=int, default=5, help="the end-to-end loop times this many rounds of --steps steps")
    ap.add_argument("--profile-iters", type=int, default=3)
    ap.add_argument("--layer-table", action="store_true",
                    help="print one line per kernel launch of a step (event time, share-scaled time, achieved rate, roofline "
                         "ceiling time and the ratio of the two) instead of the JSON line")
    ap.add_argument("--traffic-from", default=None,
                    help="an ncu --csv log with dram__bytes_read.sum / dram__bytes_write.sum of one step of --workload at --batch: "
                         "record the dominant kernel's DRAM traffic in profiles/dram_traffic.json and exit")
    args = ap.parse_args()
    default_workload = args.workload is None and args.net == "resnet50" and args.batch == 64
    if args.workload is None:
        args.workload = args.net
    if args.traffic_from:
        return record_traffic(args)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import pyb2vx as B

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert os.path.exists(SAMPLES_LIB), "libb2vx_samples.so is not built: python -c 'import __graft_entry__ as g; g.build()'"
    blib = B.load(B.PRODUCT_LIB)
    wl = make_workload(args, False, args.batch, local_rank)
    graph = wl.graph_handle()
    stream = torch.cuda.Stream()   # a non-default stream: the library takes NULL to mean "its own"
    torch.cuda.set_stream(stream)
    assert blib.b2vx_graph_set_stream(graph, C.c_void_p(stream.cuda_stream)) == 0
    in_bytes, out_bytes = wl.in_bytes, wl.out_bytes
    host_in = torch.empty(in_bytes, dtype=torch.uint8).pin_memory()
    host_out = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
    wl.synthetic_input(args.seed + rank, host_in.data_ptr())
    wl.set_input(host_in.data_ptr())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The tensor pipe's dense int8 rate, measured here and now on rank 0's GPU (well under a second)
    int8_measured = None
    if rank == 0:
        tops, sms = C.c_double(0.0), C.c_int32(0)
        if blib.b2vx_measure_int8_peak(local_rank, 5, C.byref(tops), C.byref(sms)) == 0 and tops.value > 0:
            int8_measured = tops.value

    # A pass that touches less than the L2 (126 MB) would be served from cache on repeat: write a
    # buffer larger than L2 between timed passes and time each pass with its own pair of events.
    flush = None
    if in_bytes + out_bytes < 256 * 1024 * 1024 and ":" in args.workload:
        flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    if args.layer_table:
        return layer_table(blib, B, graph, stream, args, wl, int8_measured)

    # ---- device-resident timing
    for _ in range(args.warmup):
        assert blib.b2vx_graph_run_async(graph) == 0
    assert blib.b2vx_graph_sync(graph) == 0
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    single_elapsed = time_replays(blib, graph, stream, args.steps, flush)
    barrier()
    assert blib.b2vx_graph_sync(graph) == 0, "a kernel reported a device-side timeout"
    # ---- the same with --streams replicas in flight (not for the L2-flushed single-operator passes)
    n_lanes = max(1, args.streams) if flush is None else 1
    lanes, lane_workloads = [(graph, stream)], []
    for _ in range(1, n_lanes):
        r = make_workload(args, False, args.batch, local_rank)
        rs = torch.cuda.Stream()
        assert blib.b2vx_graph_set_stream(r.graph_handle(), C.c_void_p(rs.cuda_stream)) == 0
        r.set_input(host_in.data_ptr())
        for _ in range(max(2, args.warmup)):
            assert blib.b2vx_graph_run_async(r.graph_handle()) == 0
        assert blib.b2vx_graph_sync(r.graph_handle()) == 0
        lanes.append((r.graph_handle(), rs))
        lane_workloads.append(r)
    elapsed = single_elapsed
    if n_lanes > 1:
        time_replays_streams(blib, lanes, len(lanes))   # one untimed round
        barrier()
        elapsed = time_replays_streams(blib, lanes, args.steps)
        barrier()
        for g, _ in lanes:
            assert blib.b2vx_graph_sync(g) == 0, "a kernel reported a device-side timeout"
    ms = torch.tensor([elapsed], device="cuda")
    single_ms = torch.tensor([single_elapsed], device="cuda")
    # ---- end to end through the public calls, host buffers pinned
    # Every step copies its input from pinned host memory, runs, and copies its result back, all through the
    # synchronous public calls.  As in the reference's multi-thread sample, --e2e-threads host threads each own
    # a replica of the graph and their own pinned buffers and take the steps in turn, so one replica's copies
    # overlap the other's kernels; 1 gives the strictly serial copy-run-copy loop.  The threads are started and
    # parked behind a barrier before the clock starts, and the timed region is --e2e-repeats rounds of --steps steps.
    e2e_steps = 0 if args.no_e2e else args.steps * max(1, args.e2e_repeats)
    n_host = max(1, min(args.e2e_threads, e2e_steps)) if e2e_steps else 1
    replicas = [(wl, host_in, host_out)]
    for _ in range(1, n_host):
        r = make_workload(args, False, args.batch, local_rank)
        rin = torch.empty(in_bytes, dtype=torch.uint8).pin_memory()
        rout = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
        rin.copy_(host_in)
        replicas.append((r, rin, rout))

    def feed(replica, count, gate=None):
        r, rin, rout = replica
        torch.cuda.set_device(local_rank)   # a new host thread starts on device 0
        if gate is not None:
            gate.wait()
        for _ in range(count):
            r.set_input(rin.data_ptr())
            r.run()
            r.get_output(rout.data_ptr())

    for rep in replicas if e2e_steps else []:
        feed(rep, 2)
    counts = [e2e_steps // n_host + (1 if k < e2e_steps % n_host else 0) for k in range(n_host)]
    gate = threading.Barrier(n_host)
    threads = [threading.Thread(target=feed, args=(rep, cnt, gate)) for rep, cnt in zip(replicas[1:], counts[1:])]
    for t in threads:
        t.start()
    barrier()
    t0 = time.perf_counter()
    if e2e_steps:
        feed(replicas[0], counts[0], gate)
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    e2e_ms = torch.tensor([1e3 * (time.perf_counter() - t0)], device="cuda")
    if n_host > 1:
        assert torch.equal(replicas[0][2], replicas[1][2]), "graph replicas disagree on the same input"
    for r, _, _ in replicas[1:]:
        r.close()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(single_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    ms, single_ms, e2e_ms = float(ms.item()), float(single_ms.item()), float(e2e_ms.item())

    # ---- sustained: the same graph back to back for at least two seconds, clocks and power sampled meanwhile
    sustained = None
    if not args.no_sustained and flush is None:
        step_ms = ms / args.steps
        n_sus = max(args.steps, int(2200.0 / max(step_ms, 1e-3)))
        sus_sampler = ClockSampler(local_rank)
        if rank == 0:
            sus_sampler.start()
        barrier()
        sus_ms = torch.tensor([time_replays_streams(blib, lanes, n_sus) if n_lanes > 1 else time_replays(blib, graph, stream, n_sus, None)],
                              device="cuda")
        barrier()
        sus_clocks = sus_sampler.stop() if rank == 0 else None
        if world > 1:
            dist.all_reduce(sus_ms, op=dist.ReduceOp.MAX)
        if rank == 0:
            sus_ms = float(sus_ms.item())
            sustained = {"value": wl.units * world * n_sus / (sus_ms / 1e3) * wl.scale, "unit": wl.unit, "steps": n_sus, "streams": n_lanes,
                         "seconds": sus_ms / 1e3, "ms_per_step": sus_ms / n_sus, "sm_mhz_median": sus_clocks["sm_mhz"],
                         "power_w_median": sus_clocks.get("power_w"), "reasons": sus_clocks["reasons"],
                         "ms_per_step_x_mhz": (sus_ms / n_sus) * sus_clocks["sm_mhz"] if sus_clocks["sm_mhz"] else None}

    if rank == 0:
        units = wl.units * world * args.steps
        value = units / (ms / 1e3) * wl.scale
        e2e_value = wl.units * world * e2e_steps / (e2e_ms / 1e3) * wl.scale if e2e_steps else None
        # ---- roofline of the dominant kernel, per-kernel CUDA events measured live; a kernel's time is its share of the
        # single-stream step (with several replicas in flight kernels overlap and a per-kernel time is not defined)
        step_ms = single_ms / args.steps
        per, n_kernels = kernel_table(blib, graph, B, args.profile_iters, step_ms)
        top = max(per, key=lambda n: per[n]["ms"])
        peaks = measured_peaks()
        int8_assumed = 2.0 * peaks["bf16_sustained"]
        int8_peak = int8_measured if int8_measured else int8_assumed
        t = per[top]
        roof = roofline_of(t, peaks["hbm_gbs"], int8_peak)
        traffic = dram_traffic(args.workload, args.batch)
        roof.update({"traffic": traffic["bytes"] if traffic else None, "traffic_record": traffic,
                     "kernel": top, "launches_per_step": t["launches"], "kernel_ms_per_step": t["ms"],
                     "kernel_ms_per_step_events": t["ms_events"],
                     "timing": "per-kernel CUDA events (b2vx_graph_profile) give the shares; kernel time = share x measured step",
                     "share_of_step": t["ms"] / step_ms, "tops": t["ops"] / (t["ms"] / 1e3) / 1e12 if t["ms"] else None,
                     "algorithmic_bytes": t["bytes"], "algorithmic_ops": t["ops"],
                     "int8_peak_measured": int8_measured,
                     "int8_peak_measured_how": "tcgen05.mma.kind::i8 issue-rate microbenchmark on every SM, operands in shared memory, best of 5 x 10 ms",
                     "int8_peak_assumed": int8_assumed,
                     "frac_of_int8_peak": (t["ops"] / (t["ms"] / 1e3) / 1e12) / int8_peak if t["ms"] and t["ops"] else None,
                     "frac_of_hbm": (t["bytes"] / (t["ms"] / 1e3) / 1e9) / peaks["hbm_gbs"] if t["ms"] else None,
                     "peak_source": peaks["source"],
                     "per_kernel_ms": {n: round(d["ms"], 4) for n, d in sorted(per.items(), key=lambda kv: -kv[1]["ms"])},
                     "per_kernel_ms_events": {n: round(d["ms_events"], 4) for n, d in sorted(per.items(), key=lambda kv: -kv[1]["ms"])}})
        configs = None
        if world == 1 and default_workload and not args.no_configs:
            cfg_flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
            configs = run_configs(blib, B, stream, args.seed, local_rank, peaks["hbm_gbs"], int8_peak, cfg_flush)
            del cfg_flush
        cpu = None if (args.no_cpu_baseline or world > 1) else cpu_baseline_subprocess(args)
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic",
            "config": {"workload": wl.describe,
                       "parallelism": "batch-sharded replicas, no collective", "units_per_step": wl.units * world,
                       "streams": n_lanes,
                       "step": "one replay of one graph replica over its resident batch; the %d replicas of a GPU, each on its own CUDA "
                               "stream, take the steps in turn and overlap" % n_lanes if n_lanes > 1 else "one replay of the graph",
                       "l2": ("a 192 MB buffer is rewritten between timed passes (L2 flush); each pass has its own events"
                              if flush is not None else "the per-step working set exceeds the 126 MB L2")},
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                    "ms_per_step": e2e_ms / e2e_steps if e2e_steps else None, "host_threads": n_host,
                    "steps": e2e_steps, "repeats": max(1, args.e2e_repeats) if e2e_steps else 0},
            "gpu_launches": n_kernels * args.steps,
            "single_stream": {"value": wl.units * world * args.steps / (single_ms / 1e3) * wl.scale, "unit": wl.unit,
                              "ms_per_step": single_ms / args.steps},
            "roofline": roof, "sustained": sustained, "cpu_baseline": cpu, "clocks": clocks, "configs": configs,
        }
        print(json.dumps(line))
    for r in lane_workloads:
        r.close()
    wl.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
