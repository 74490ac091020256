#!/usr/bin/env python
"""Benchmark of the B200-native glades feed-forward path.

    python bench.py --gpus N --steps K --warmup W            our arm (one JSON line on rank 0)
    python bench.py --impl reference --gpus N ...            the CPU arm (rank 0 only)

Workload (default `wide_mlp`): the wide-MLP teacher-student training config -- student
1024-4096(ReLU)-4096(ReLU)-1024(softmax), cross-entropy, SGD lr 1e-2, minibatch 8192 split evenly
over the N GPUs with one gradient all-reduce per step; inputs ~ N(0,1) generated on the device by
the counter-based generator, labels = argmax of a fixed seeded 1024-4096(ReLU)-1024 teacher.  One
step = one minibatch window (forward, backward, update).  Batched arithmetic mode: aligned windows,
frozen weights inside a window, plain error sum, softmax + cross-entropy head (none of which the
reference has; its own arithmetic is non-finite on this shape after the first sample).

`value`   train samples/s with the windows already resident in HBM (CUDA events on the library's
          stream, max over ranks).
`e2e`     the same step through gl_train_window_host_submit / _result (inference: gl_forward_host_submit
          / _result): every window's rows start in pinned HOST memory and are copied in by the call, and
          every window's loss (inference: plus every row's predicted class) is read back; two windows
          are in flight so the copy of one overlaps the compute of the other.
`roofline` the tensor-core layer-product kernel: algorithmic flop of its launches / their summed
          CUDA-event durations, against the measured dense bf16 peak of MEASURED_PEAKS.json.
`cpu_baseline` the CPU restatement of the same batched arithmetic (oracle port, all host cores)
          on a small sample of the same window.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

SEED = 0x474C4144  # "GLAD"

WORKLOADS = {
    # name: sizes, activations, global batch, lr, momentum, kind
    "wide_mlp": dict(sizes=[1024, 4096, 4096, 1024], acts=["relu", "relu", "softmax"], batch=8192, lr=1e-2, momentum=0.0,
                     out="classification", kind="train"),
    "window_regressor": dict(sizes=[32, 256, 256, 1], acts=["relu", "relu", "linear"], batch=1024, lr=1e-3, momentum=0.9,
                             out="regression", kind="train", params=[0.0, 0.0, 1.0], resident_rows=1 << 21),
    "batched_inference": dict(sizes=[784, 2048, 2048, 10], acts=["relu", "relu", "softmax"], batch=65536, lr=0.0,
                              momentum=0.0, out="classification", kind="infer"),
}


def flop_per_sample(sizes, train):
    P = sum(sizes[i] * sizes[i + 1] for i in range(len(sizes) - 1))
    return (6 * P - 2 * sizes[0] * sizes[1]) if train else 2 * P


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], tensor=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1400.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and the clock-event reasons while the timed region runs: NVML queries
    from a thread every few milliseconds (read-only), or `nvidia-smi -lms` where NVML's Python
    module is missing."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        try:
            self.gpu = int(vis.split(",")[gpu_index]) if vis else gpu_index
        except (ValueError, IndexError):
            self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.stop_flag = False
        self.sm, self.mx, self.reasons = [], [], set()

    def _nvml_loop(self, nv, h):
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                for bit, name in self.REASON_BITS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread:
            self.stop_flag = True
            self.thread.join(timeout=2)
            if self.sm:
                out.update(sm_mhz=float(np.median(self.sm)), sm_max_mhz=float(max(self.mx)), reasons=sorted(self.reasons),
                           samples=len(self.sm), source="nvml")
            return out
        if not self.proc:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    c = [v.strip() for v in line.split(",")]
                    if len(c) < 9:
                        continue
                    try:
                        sm.append(float(c[1]))
                        mx.append(float(c[2]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                       c[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm),
                       source="nvidia-smi")
        return out


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


class Plumbing:
    """torch.distributed (one process per GPU) for barriers, the max over ranks and the hand-over
    of the library's NCCL id; the data path's collective is the library's own all-reduce."""

    def __init__(self, world):
        self.world = world
        self.td = None
        if world > 1:
            import torch
            import torch.distributed as td
            self.torch = torch
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            td.init_process_group(backend="gloo")
            self.td = td

    def barrier(self):
        if self.td:
            self.td.barrier()

    def max(self, v):
        if not self.td:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64)
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t[0])

    def sum(self, v):
        if not self.td:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64)
        self.td.all_reduce(t, op=self.td.ReduceOp.SUM)
        return float(t[0])

    def bcast_bytes(self, b, src=0):
        if not self.td:
            return b
        lst = [b]
        self.td.broadcast_object_list(lst, src=src)
        return lst[0]

    def close(self):
        if self.td:
            self.td.destroy_process_group()


def dev_alloc(L, nbytes, dev):
    p = C.c_void_p()
    if L.gl_device_alloc(C.byref(p), nbytes, dev) != 0:
        raise RuntimeError(L.gl_last_error().decode())
    return p


def fill_shard(L, d_ptr, nwin, lb, gb, rank, width, seed, stream, dist, scale, offset, dev):
    """Fills this rank's rows of `nwin` global windows from ONE global table [nwin * gb][width] of the
    counter-based stream (seed, stream): window i of the rank holds global rows [i*gb + rank*lb, ... + lb).
    The table -- and with it every global window -- is the same for any number of ranks."""
    for i in range(nwin):
        first = (i * gb + rank * lb) * width
        dst = C.c_void_p(d_ptr.value + i * lb * width * 4)
        if L.gl_synth_fill_at(dst, lb * width, first, seed, stream, dist, scale, offset, dev) != 0:
            raise RuntimeError(L.gl_last_error().decode())


def build_wide_mlp_data(g, w, nwin, lb, gb, dev, rank):
    """Resident synthetic shard: X ~ N(0,1) on the device, Y = one-hot argmax of the seeded teacher."""
    L = g.lib()
    rows = nwin * lb
    n_in, n_out = w["sizes"][0], w["sizes"][-1]
    dX = dev_alloc(L, rows * n_in * 4, dev)
    dY = dev_alloc(L, rows * n_out * 4, dev)
    # stream 0 = data: every rank fills its own rows of the one global table
    fill_shard(L, dX, nwin, lb, gb, rank, n_in, SEED + 4, 0, 1, 1.0, 0.0, dev)
    rng = np.random.default_rng(SEED + 41)
    tsz = [n_in, 4096, n_out]
    tw = np.concatenate([(rng.standard_normal(tsz[i] * tsz[i + 1]) / np.sqrt(tsz[i])).astype(np.float32)
                         for i in range(2)])
    td = g.make_desc(tsz, ["relu", "linear"], "regression", batch=8192, lr=0.0, params=[0.0, 1.0],
                     mode=g.MODE_BATCHED, device=dev)
    teacher = g.Net(td)
    teacher.set_weights(tw, None)
    teacher.set_data_device(dX.value, None, rows)  # forward only: no expected rows, no metrics
    labels = np.empty(rows, np.int32)
    step = 65536
    for r0 in range(0, rows, step):
        cnt = min(step, rows - r0)
        _, am, _ = teacher.forward(r0, cnt, want_outputs=False)
        labels[r0:r0 + cnt] = am
    teacher.close()
    labels = np.maximum(labels, 0)
    assert L.gl_onehot_fill(dY, labels.ctypes.data_as(C.c_void_p), rows, n_out, 1.0, 0.0, dev) == 0, L.gl_last_error()
    return dX, dY, labels


def student_weights(sizes):
    rng = np.random.default_rng(SEED + 42)
    parts = []
    for i in range(len(sizes) - 1):
        a = 1.0 / np.sqrt(sizes[i])
        parts.append(rng.uniform(-a, a, sizes[i] * sizes[i + 1]).astype(np.float32))
    return np.concatenate(parts)


def cpu_port_baseline(g, w, sample_rows, threads=None):
    """Times the CPU port of the same batched arithmetic on a sample of one window: training steps on the
    blocked fp32 variant (oracle/fastport.c: register-tiled products, OpenMP over the host cores, checked
    against the double-accumulating restatement by the CPU tests), inference on the restatement's forward.
    Test infrastructure used as the reported CPU baseline only."""
    o = ge.import_oracle()
    sizes = w["sizes"]
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    # set explicitly: a launcher may have exported OMP_NUM_THREADS=1 (torchrun does); `cores` is what really runs
    cores = o.set_threads(threads or avail)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((sample_rows, sizes[0])).astype(np.float32)
    y = np.zeros((sample_rows, sizes[-1]), np.float32)
    y[np.arange(sample_rows), rng.integers(0, sizes[-1], sample_rows)] = 1.0
    d = g.make_desc(sizes, w["acts"], w["out"], batch=sample_rows, lr=w["lr"], momentum=w["momentum"],
                    params=w.get("params"), mode=g.MODE_BATCHED)
    S = o.Restate(d, x, y, g.Metrics)
    S.set_weights(student_weights(sizes), None)
    t0 = time.time()
    if w["kind"] == "train":
        S.train_window_fast(0, sample_rows)
    else:
        S.forward_block(0, sample_rows)
    dt = time.time() - t0
    S.close()
    return sample_rows / dt, cores, dt


def _ref_worker(job):
    """One single-threaded run of the reference's own compiled code (oracle/_ref) on `rows` rows."""
    name, rows, seed = job
    g = ge.import_package()
    o = ge.import_oracle()
    w = WORKLOADS[name]
    sizes = w["sizes"]
    rng = np.random.default_rng(seed)
    x = rng.random((rows, sizes[0]), dtype=np.float32) if w["kind"] == "infer" else \
        rng.standard_normal((rows, sizes[0])).astype(np.float32)
    y = np.full((rows, sizes[-1]), 0.01, np.float32)
    # the reference has no softmax: its native head (per-node sigmoid) stands in, same flop count
    acts = ["sigmoid" if a == "softmax" else a for a in w["acts"]]
    d = g.make_desc(sizes, acts, w["out"], batch=min(rows, w["batch"]), lr=w["lr"], momentum=w["momentum"],
                    params=w.get("params"), mode=g.MODE_REFERENCE)
    R = o.Reference(d, x, y, g.Metrics)
    R.set_weights(student_weights(sizes), None)
    t0 = time.perf_counter()
    if w["kind"] == "train":
        R.train_public(1)
    else:
        R.test_public()
    dt = time.perf_counter() - t0
    R.close()
    return rows, dt


def cpu_reference_baseline(name, rows_per_proc, procs):
    """The compiled reference on the host cores.  Training is sequential by construction (one process);
    inference rows are independent, so `procs` single-threaded processes run disjoint rows side by side
    and their rows/s add up."""
    import multiprocessing as mp
    jobs = [(name, rows_per_proc, 11 + i) for i in range(procs)]
    if procs == 1:
        res = [_ref_worker(jobs[0])]
    else:
        with mp.get_context("spawn").Pool(procs) as pool:
            res = pool.map(_ref_worker, jobs)
    return sum(r / dt for r, dt in res), max(dt for _, dt in res)


# bounded samples of the compiled reference per workload: rows per process, processes
REF_SAMPLES = {"batched_inference": (16, "all"), "window_regressor": (768, 1)}


def cpu_baseline_for(g, name, w):
    """(value, cores, kind, sample text) of the CPU figure reported beside a workload: the reference's own
    compiled code where a bounded sample of it can be timed, else the CPU port."""
    o = ge.import_oracle()
    if name in REF_SAMPLES and o.have_reference():
        rows, procs = REF_SAMPLES[name]
        procs = min(os.cpu_count() or 1, 8) if procs == "all" else procs
        v, dt = cpu_reference_baseline(name, rows, procs)
        head = " (per-node sigmoid head: the reference has no softmax)" if "softmax" in w["acts"] else ""
        return v, procs, "reference", ("%d rows in each of %d single-threaded process(es) of the compiled reference%s, "
                                       "%.1f s" % (rows, procs, head, dt)), dt
    train = w["kind"] == "train"
    rows = min(w["batch"], 8192) if train else 2048
    v, cores, dt = cpu_port_baseline(g, w, rows)
    note = "; the compiled reference needs ~669 s per training row at this shape (forward 2.6 s, backward 666 s)" \
        if name == "wide_mlp" else ""
    how = "blocked fp32 products, OpenMP on %d threads" % cores if train else "double accumulation, OpenMP on %d threads" % cores
    return v, cores, "port", ("%d rows of one window, CPU port of the same batched arithmetic (%s), %.1f s%s"
                              % (rows, how, dt, note)), dt


def workload_config(name, w, world):
    """The part of `config` that names the workload; the same for our arm and the reference arm."""
    train = w["kind"] == "train"
    gb = w["batch"]
    return {"workload": name, "sizes": w["sizes"], "global_batch": gb, "per_gpu_rows": gb // world if train else gb,
            "mode": "batched", "head": w["acts"][-1], "lr": w["lr"], "parallelism": "dp%d" % world}


def run_reference_arm(args, g, w, rank, world):
    """The CPU arm: the reference's own compiled code (oracle/_ref) on a bounded sample where that is
    feasible (inference rows, the window regressor's training rows).  For the wide MLP it needs ~669 s
    for ONE training row (forward 2.6 s, backward 666 s: the output layer copies the whole expected row
    per edge, network.cpp:605-606), so the arm times the CPU port of the same arithmetic there and says
    so in `cpu_baseline.kind` / `.sample`."""
    if rank != 0:
        return
    vals, secs = [], []
    cores = kind = sample = None
    for i in range(args.warmup + args.steps):
        v, cores, kind, sample, dt = cpu_baseline_for(g, args.workload, w)
        if i >= args.warmup:
            vals.append(v)
            secs.append(dt)
    value = float(np.mean(vals))
    unit = "samples/s" if w["kind"] == "train" else "rows/s"
    line = {
        "impl": "reference", "metric": "train_samples_per_s" if w["kind"] == "train" else "infer_rows_per_s",
        "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean(secs)), "higher_is_better": True,
        "scaling": "strong" if w["kind"] == "train" else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w, world),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if args.workload == "wide_mlp":
        # the compiled reference itself on this shape, timed once on one core of the development box (not
        # re-run here: one row takes eleven minutes and its arithmetic leaves the finite range)
        line["reference_measured_once"] = {"seconds_per_training_row": 668.7, "forward_s": 2.6, "backward_s": 666.0,
                                           "samples_per_s": 1.0 / 668.7, "cores": 1, "finite": False}
    print(json.dumps(line), flush=True)


SMALL = {
    # config 1 at the only learning rate where the reference stays finite (0.01, interleaved class rows)
    "tiny_classifier": dict(sizes=[4, 16, 3], acts=["sigmoid", "sigmoid"], out="classification", batch=1, lr=0.01,
                            momentum=0.9, rows=150, epochs=200, modes=["reference"]),
    # config 2: all 2^10 binary vectors, parity target
    "parity_net": dict(sizes=[10, 32, 32, 1], acts=["tanh", "tanh", "sigmoid"], out="regression", batch=32, lr=0.05,
                       momentum=0.0, rows=1024, epochs=500, modes=["reference", "batched"]),
}


def small_data(name, w):
    rng = np.random.default_rng(SEED + 1)
    if name == "parity_net":
        idx = np.arange(1024)
        x = ((idx[:, None] >> np.arange(9, -1, -1)) & 1).astype(np.float32)
        y = (x.sum(1) % 2).astype(np.float32)[:, None]
        a = 1.0
    else:
        means = rng.uniform(-2, 2, (3, 4))
        cls = np.arange(w["rows"]) % 3
        x = (means[cls] + 0.5 * rng.standard_normal((w["rows"], 4))).astype(np.float32)
        y = np.full((w["rows"], 3), 0.01, np.float32)
        y[np.arange(w["rows"]), cls] = 0.99
        a = 0.5
    nw = sum(w["sizes"][i] * w["sizes"][i + 1] for i in range(len(w["sizes"]) - 1))
    return x, y, rng.uniform(-a, a, nw).astype(np.float32)


def run_small(args, g, name):
    """The two small configs (sequential by construction, one GPU): whole training runs in one launch.
    One step = `epochs` epochs over the data set; value = samples/s; the CPU figure beside it is the
    reference's own compiled code (oracle/_ref) when it is present, else the CPU port."""
    w = dict(SMALL[name])
    if args.epochs > 0:
        w["epochs"] = args.epochs
    x, y, w0 = small_data(name, w)
    peaks = measured_peaks()
    o = ge.import_oracle()
    for mode_name in w["modes"]:
        mode = g.MODE_REFERENCE if mode_name == "reference" else g.MODE_BATCHED
        d = g.make_desc(w["sizes"], w["acts"], w["out"], batch=w["batch"], lr=w["lr"], momentum=w["momentum"], mode=mode)
        net = g.Net(d)
        times, e2e = [], []
        sampler = ClockSampler(0)
        for i in range(args.warmup + args.steps):
            if i == args.warmup:
                sampler.start()
            t0 = time.perf_counter()
            net.set_weights(w0, None)
            net.set_data(x, y)                       # host rows in, every step
            m = net.train_epochs(w["epochs"])        # metrics (loss) read back
            dt = time.perf_counter() - t0
            if i >= args.warmup:
                times.append(m.device_ms / 1000.0)
                e2e.append(dt)
        clocks = sampler.stop()
        samples = w["rows"] * w["epochs"]
        value = samples / float(np.mean(times))
        bytes_per_sample = 4 * (w["sizes"][0] + w["sizes"][-1])
        t0 = time.perf_counter()
        if mode_name == "reference" and o.have_reference():
            R = o.Reference(d, x, y, g.Metrics)
            R.set_weights(w0, None)
            cpu_epochs = max(1, w["epochs"] // 10)
            t0 = time.perf_counter()
            R.train_public(cpu_epochs)
            kind = "reference"
        else:
            S = o.Restate(d, x, y, g.Metrics)
            S.set_weights(w0, None)
            cpu_epochs = max(1, w["epochs"] // 10)
            t0 = time.perf_counter()
            for _ in range(cpu_epochs):
                if mode_name == "reference":
                    S.epoch(0)
                else:
                    for r0 in range(0, w["rows"], w["batch"]):
                        S.train_window(r0, min(w["batch"], w["rows"] - r0))
            kind = "port"
        cpu_dt = time.perf_counter() - t0
        line = {
            "metric": "train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean(times)), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "sizes": w["sizes"], "mode": mode_name, "batch": w["batch"], "lr": w["lr"],
                       "epochs_per_step": w["epochs"], "rows": w["rows"],
                       "l2": "data set far smaller than L2: the run is a sequential dependent chain, not a bandwidth test"},
            "e2e": {"value": samples / float(np.mean(e2e)), "unit": "samples/s",
                    "h2d_bytes_per_step": int(x.nbytes + y.nbytes + w0.nbytes), "d2h_bytes_per_step": 32},
            "gpu_launches": args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": value * bytes_per_sample / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": value * bytes_per_sample / 1e9 / peaks["hbm"], "traffic": None,
                         "note": "latency-bound: %s" % ("strictly sequential per-sample SGD" if mode_name == "reference"
                                                        else "one window of %d rows at a time on one SM" % w["batch"])},
            "cpu_baseline": {"value": w["rows"] * cpu_epochs / cpu_dt, "unit": "samples/s", "cores": 1, "kind": kind,
                             "sample": "%d epochs (%.1f s)" % (cpu_epochs, cpu_dt)},
            "final_accuracy": m.total_accuracy, "nonfinite": m.nonfinite,
        }
        print(json.dumps(line), flush=True)
        net.close()


def run_standardize(args, g):
    """The step in front of the loop: standardisation of a raw table that lies in HBM (gl_standardize_table).
    One step = one 1 M x 33 table (the window regressor's data set: 32 inputs and the target, 138 MB, larger than
    L2), min-max scaling.  value = rows/s resident; e2e = the same from a pinned host table, copy in and
    standardised matrices back out included.  HBM roofline: algorithmic bytes = the table read once and the
    standardised matrices written once (the kernels read the table twice: extrema, then transform)."""
    o = ge.import_oracle()
    L = g.lib()
    rows, cols = 1 << 20, 33
    kind = np.zeros(cols, np.int32)
    classes = np.zeros(cols, np.int32)
    outs = np.zeros(cols, np.int32)
    outs[-1] = 1
    d_raw = dev_alloc(L, rows * cols * 4, 0)
    assert L.gl_synth_fill(d_raw, rows * cols, SEED + 9, 0, 1, 4.0, 0.0, 0) == 0
    nx, ny = C.c_int32(), C.c_int32()
    ptrs = (kind.ctypes.data_as(C.c_void_p), classes.ctypes.data_as(C.c_void_p), outs.ctypes.data_as(C.c_void_p))
    assert L.gl_standardize_table(d_raw, rows, cols, *ptrs, 0, None, C.byref(nx), None, C.byref(ny), None, 0) == 0
    d_x = dev_alloc(L, rows * nx.value * 4, 0)
    d_y = dev_alloc(L, rows * ny.value * 4, 0)
    import torch
    sampler = ClockSampler(0)
    times = []
    for i in range(args.warmup + args.steps):
        if i == args.warmup:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()   # the entry point works on the legacy default stream, which torch's current stream is
        st = L.gl_standardize_table(d_raw, rows, cols, *ptrs, 0, d_x, C.byref(nx), d_y, C.byref(ny), None, 0)
        ev1.record()
        torch.cuda.synchronize()
        assert st == 0, L.gl_last_error()
        if i >= args.warmup:
            times.append(ev0.elapsed_time(ev1) / 1000.0)
    clocks = sampler.stop()
    # end to end: pinned host table in, standardised matrices out
    h_raw, h_x, h_y = C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert L.gl_host_alloc_pinned(C.byref(h_raw), rows * cols * 4) == 0
    assert L.gl_host_alloc_pinned(C.byref(h_x), rows * nx.value * 4) == 0
    assert L.gl_host_alloc_pinned(C.byref(h_y), rows * ny.value * 4) == 0
    L.gl_memcpy_d2h(h_raw, d_raw, rows * cols * 4, 0)
    e2e = []
    for i in range(3 + min(args.steps, 10)):
        t0 = time.perf_counter()
        L.gl_memcpy_h2d(d_raw, h_raw, rows * cols * 4, 0)
        assert L.gl_standardize_table(d_raw, rows, cols, *ptrs, 0, d_x, C.byref(nx), d_y, C.byref(ny), None, 0) == 0
        L.gl_memcpy_d2h(h_x, d_x, rows * nx.value * 4, 0)
        L.gl_memcpy_d2h(h_y, d_y, rows * ny.value * 4, 0)
        if i >= 3:
            e2e.append(time.perf_counter() - t0)
    peaks = measured_peaks()
    t = float(np.mean(times))
    alg_bytes = rows * cols * 4 + rows * (nx.value + ny.value) * 4
    cpu = None
    if not args.no_cpu_baseline:
        sample = 1 << 17
        raw = o.synth_fill(sample * cols, SEED + 9, 0, 1, 4.0, 0.0).reshape(sample, cols)
        t0 = time.perf_counter()
        o.standardize_table(raw, [0] * cols, list(outs), 0, nx.value, ny.value)
        dt = time.perf_counter() - t0
        cpu = {"value": sample / dt, "unit": "rows/s", "cores": 1, "kind": "port",
               "sample": "%d rows x %d columns, C restatement of NumberInput::standardizeInputTable (pinned bit for bit to the "
                         "reference's code), %.2f s" % (sample, cols, dt)}
    line = {
        "metric": "standardize_rows_per_s", "value": rows / t, "unit": "rows/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * t, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "standardize", "rows": rows, "cols": cols, "flag": "minmax",
                   "l2": "inputs larger than L2: a 138 MB table is read and 138 MB of matrices are written per step"},
        "e2e": {"value": rows / float(np.mean(e2e)), "unit": "rows/s", "h2d_bytes_per_step": rows * cols * 4,
                "d2h_bytes_per_step": rows * (nx.value + ny.value) * 4},
        "gpu_launches": 2 * args.steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "minmax_kernel + transform_kernel (one call)", "achieved": alg_bytes / t / 1e9,
                     "peak": peaks["hbm"], "unit": "GB/s", "frac": alg_bytes / t / 1e9 / peaks["hbm"], "traffic": None,
                     "peak_source": peaks["source"] + " copy bandwidth",
                     "note": "the call reads the extrema back to the host between its two kernels (the layout of the "
                             "outputs depends on them); the kernels read the table twice, 414 MB of traffic per call"},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wide_mlp", choices=sorted(WORKLOADS) + sorted(SMALL) + ["standardize"])
    ap.add_argument("--windows", type=int, default=0, help="resident windows per GPU (default: steps+warmup, max 64)")
    ap.add_argument("--gemm", default="auto", choices=["auto", "ffma", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the workload's global batch (diagnostic runs, e.g. 1024 = one GPU's share of the 8-GPU step)")
    ap.add_argument("--epochs", type=int, default=0, help="small workloads: epochs per step (default: the config's)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    rank, world, local = dist_env()
    g = ge.import_package()
    if args.workload == "standardize":
        if rank == 0 and args.impl == "ours":
            run_standardize(args, g)
        return
    if args.workload in SMALL:
        if rank == 0 and args.impl == "ours":
            run_small(args, g, args.workload)
        return
    w = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        w["batch"] = args.batch
    if args.impl == "reference":
        run_reference_arm(args, g, w, rank, world)
        return
    if g.device_count() < 1:
        raise SystemExit("bench.py needs a B200: the library has no CPU path")
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    plumb = Plumbing(world)
    dev = local
    L = g.lib()
    sizes = w["sizes"]
    train = w["kind"] == "train"
    gb = w["batch"]
    if gb % world:
        raise SystemExit("global batch %d does not split over %d GPUs" % (gb, world))
    lb = gb // world if train else gb  # training splits the window; inference shards whole batches
    nwin = args.windows or min(64, args.steps + args.warmup)
    if not args.windows and train and nwin * lb * (sizes[0] + sizes[-1]) * 4 < 2 * 126e6 and "resident_rows" in w:
        # small rows: keep the config's whole data set resident so that the windows the steps touch are
        # larger than L2 together and each step reads rows no earlier step has touched
        nwin = max(nwin, w["resident_rows"] // gb)
    rows = nwin * lb
    gemm = {"auto": g.GEMM_AUTO, "ffma": g.GEMM_FFMA, "tcgen05": g.GEMM_TCGEN05}[args.gemm]

    d = g.make_desc(sizes, w["acts"], w["out"], batch=gb, lr=w["lr"], momentum=w["momentum"], params=w.get("params"),
                    mode=g.MODE_BATCHED, gemm=gemm, device=dev)
    net = g.Net(d)
    net.set_weights(student_weights(sizes), None)
    if args.workload == "wide_mlp":
        dX, dY, labels = build_wide_mlp_data(g, w, nwin, lb, gb, dev, rank)
    else:
        dX = dev_alloc(L, rows * sizes[0] * 4, dev)
        dY = dev_alloc(L, rows * sizes[-1] * 4, dev)
        dist, sc, off = (0, 1.0, 0.0) if args.workload == "batched_inference" else (1, 1.0, 0.0)
        # training: the rank's rows of each global window; inference: the rank's own whole batches
        # (batch i of rank k is global batch i * world + k), both cut from one global table
        tgb, trank = (gb, rank) if train else (gb * world, rank)
        fill_shard(L, dX, nwin, lb, tgb, trank, sizes[0], SEED, 0, dist, sc, off, dev)
        fill_shard(L, dY, nwin, lb, tgb, trank, sizes[-1], SEED + 7, 3, 0, 0.98, 0.01, dev)
        labels = None
    net.set_data_device(dX.value, dY.value, rows)
    if world > 1 and train:
        uid = (C.c_char * 128)()
        if rank == 0:
            assert L.gl_dp_unique_id(uid) == 0, L.gl_last_error()
        uid_bytes = plumb.bcast_bytes(bytes(uid.raw))
        net.dp_init(rank, world, uid_bytes)
        net.dp_set_window(gb, rank * lb)
    dp_mode = net.dp_mode()

    def step(i, want_metrics=False):
        r0 = (i % nwin) * lb
        if train:
            return net.train_window(r0, lb, want_metrics)
        return net.forward(r0, lb, want_outputs=False, want_argmax=False)[2]

    # ---- resident timing (`value`): K steps per region, no per-launch events inside it; the region is run
    # three times back to back and the fastest is reported (all three are in the line, `region_ms`): a
    # region of a few tens of milliseconds is exposed to one-off stalls, which can only add time, and the
    # later regions run under the 1 kW power cap at a lower clock (the `clocks` record covers all three)
    m_first = step(0, True)
    for i in range(1, args.warmup):
        step(i)
    net.sync()
    launches0 = net.kernel_launches()
    sampler = ClockSampler(dev)
    sampler.start()
    regions = []
    for rep in range(3):
        plumb.barrier()
        net.timer_start()
        for i in range(args.steps):
            step(args.warmup + rep * args.steps + i)
        r_ms = net.timer_stop()
        net.sync()
        plumb.barrier()
        regions.append(plumb.max(r_ms))
    clocks = sampler.stop()
    launches = (net.kernel_launches() - launches0) // 3
    ms = float(np.min(regions))
    samples_per_step = gb if train else gb * world
    value = samples_per_step * args.steps / (ms / 1000.0)
    # ---- a separate, untimed-for-`value` pass with per-launch events around the layer products (roofline)
    net.profile_enable(True)
    net.timer_start()
    for i in range(args.steps):
        step(args.warmup + i)
    prof_ms = plumb.max(net.timer_stop())
    net.sync()
    plumb.barrier()
    prof = net.profile_read()
    net.profile_enable(False)
    m_last = step(0, True) if train else None

    # ---- end to end through the host-buffer entry point (`e2e`)
    n_pin = 2
    xb = lb * sizes[0] * 4
    yb = lb * sizes[-1] * 4
    pins = []
    for _ in range(n_pin):
        px, py = C.c_void_p(), C.c_void_p()
        assert L.gl_host_alloc_pinned(C.byref(px), xb) == 0 and L.gl_host_alloc_pinned(C.byref(py), yb) == 0
        pins.append((px, py))
    for k, (px, py) in enumerate(pins):
        L.gl_memcpy_d2h(px, C.c_void_p(dX.value + k * xb), xb, dev)
        L.gl_memcpy_d2h(py, C.c_void_p(dY.value + k * yb), yb, dev)
    mm = g.Metrics()
    h_out = np.empty(8, np.float32)
    h_arg = np.empty(lb, np.int32)  # inference: every batch's predicted classes are read back

    def e2e_submit(i):
        px, py = pins[i % n_pin]
        if L.gl_train_window_host_submit(net.h, px, py, lb) != 0:
            raise RuntimeError(L.gl_last_error().decode())

    def e2e_result():
        if L.gl_train_window_host_result(net.h, C.byref(mm)) != 0:
            raise RuntimeError(L.gl_last_error().decode())
        return mm.total_error

    def e2e_run(count):
        """count steps, each with its own host->device copy and its own loss read-back; training keeps two
        windows in flight so that the copy of one overlaps the compute of the other."""
        if not train:
            def fsubmit(i):
                px, py = pins[i % n_pin]
                if L.gl_forward_host_submit(net.h, px, py, lb) != 0:
                    raise RuntimeError(L.gl_last_error().decode())

            def fresult():
                if L.gl_forward_host_result(net.h, h_arg.ctypes.data_as(C.c_void_p), C.byref(mm)) != 0:
                    raise RuntimeError(L.gl_last_error().decode())

            fsubmit(0)
            for i in range(1, count):
                fsubmit(i)
                fresult()
            fresult()
            return
        e2e_submit(0)
        for i in range(1, count):
            e2e_submit(i)
            e2e_result()
        e2e_result()

    e2e_run(3)
    plumb.barrier()
    e2e_steps = max(3, min(args.steps, 20))
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    dt = time.perf_counter() - t0
    plumb.barrier()
    dt = plumb.max(dt)
    e2e_value = samples_per_step * e2e_steps / dt
    # the loss / accuracy sums (2 doubles) and the status words (4 ints) read back every step; inference also
    # reads back the predicted class of every row
    d2h_bytes = 16 + 16 + (0 if train else 4 * lb)

    # ---- roofline of the dominant kernel
    peaks = measured_peaks()
    tc = prof["tc"]
    ff = prof["ffma"]
    if tc["ms"] == 0 and ff["ms"] == 0:
        # no per-layer product ran: the whole step is one fused kernel (whole-window cooperative kernel)
        bytes_per_sample = 4 * (sizes[0] + sizes[-1])
        gbs = value * bytes_per_sample / 1e9
        roofline = {
            "bound": "hbm", "kernel": "grid_fused_kernel (whole window in one cooperative launch, fp32 FFMA)",
            "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"], "traffic": None,
            "peak_source": peaks["source"] + " copy bandwidth",
            "launches": int(launches), "avg_launch_ms": ms / max(1, int(launches)),
            "algorithmic_bytes_per_launch": bytes_per_sample * samples_per_step,
            "fp32_tflops": flop_per_sample(sizes, train) * value / 1e12,
            "note": "algorithmic bytes = input row + target row per sample; the step is far from the HBM bound (arithmetic "
                    "intensity %d flop/B): it is bound by fp32 FFMA issue and shared-memory latency on %d-row windows, see "
                    "fp32_tflops" % (flop_per_sample(sizes, train) // bytes_per_sample, lb),
        }
        dom = None
    else:
        dom = tc if tc["ms"] >= ff["ms"] else ff
        dom_name = "gemm_tc_kernel (TMA + tcgen05 kind::tf32, 3xTF32)" if dom is tc else "gemm_ffma_kernel (fp32 FFMA)"
        achieved = dom["flop"] / (dom["ms"] / 1000.0) / 1e12 if dom["ms"] > 0 else 0.0
        roofline = {
            "bound": "tensor", "kernel": dom_name, "achieved": achieved, "peak": peaks["tensor"], "unit": "TFLOP/s",
            "frac": achieved / peaks["tensor"],
            # DRAM bytes per launch of this kernel from one ncu capture of this very workload (5.81 GB over
            # the 8 products of a step); null elsewhere
            "traffic": 0.726e9 if (dom is tc and args.workload == "wide_mlp" and world == 1) else None,
            "peak_source": peaks["source"] + " dense bf16 (sustained)",
            "launches": dom["launches"], "avg_launch_ms": dom["ms"] / max(1, dom["launches"]),
            "algorithmic_flop_per_launch": dom["flop"] / max(1, dom["launches"]),
            "note": "achieved counts algorithmic fp32 flop (2*M*N*K per product); the 3xTF32 mode issues 3 TF32 MMAs per "
                    "product term, so the tensor pipe runs at 3x this figure and the mode's own ceiling is peak/6",
            "frac_of_3xtf32_ceiling": achieved / (peaks["tensor"] / 6.0),
            # cuBLAS TF32 GEMM measured on this pool's B200s the way the bf16 peak was (8192^3, best of 10,
            # CUDA events): 745.6 TFLOP/s burst, 591.7 over 300 in a row; a 3xTF32 product can reach a third
            "frac_of_cublas_tf32_third": achieved / (745.6 / 3.0),
            "share_of_step_ms": dom["ms"] / prof_ms if prof_ms > 0 else None,
        }

    # sum and sum of magnitudes of the final weights (after warm-up, the timed regions, the profiled pass
    # and the end-to-end steps: the same sequence of global windows for every N)
    checksum = None
    if train and rank == 0:
        wfin, bfin = net.get_weights()
        checksum = {"sum": float(np.sum(wfin, dtype=np.float64)), "sum_abs": float(np.sum(np.abs(wfin), dtype=np.float64)),
                    "bias": [float(v) for v in bfin]}
    line = None
    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            v, cores, kind, sample, _ = cpu_baseline_for(g, args.workload, w)
            cpu = {"value": v, "unit": "samples/s" if train else "rows/s", "cores": cores, "kind": kind, "sample": sample}
        line = {
            "metric": "train_samples_per_s" if train else "infer_rows_per_s",
            "value": value, "unit": "samples/s" if train else "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if train else "weak",
            "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, fp32 accumulate)" if (dom is not None and dom is tc) else "f32",
            "data": "synthetic",
            "config": dict(workload_config(args.workload, w, world), **{
                       "resident_windows_per_gpu": nwin,
                       "timed_region": "fastest of 3 back-to-back regions of %d steps each (CUDA events, max over ranks; all "
                                       "three in region_ms); per-launch events only in a separate pass" % args.steps,
                       "l2": ("inputs larger than L2: every step streams a distinct %.0f MB window plus %.0f MB of weights and "
                              "%.0f MB of activations and deltas" % (lb * (sizes[0] + sizes[-1]) * 4 / 1e6, net.nw * 4 / 1e6,
                                                                       2 * lb * sum(sizes) * 4 / 1e6))
                             if lb * sum(sizes) * 8 + net.nw * 4 > 126e6 else
                             "inputs larger than L2: %d resident windows (%.0f MB) and every step reads a window no earlier step "
                             "has touched; the weights and the window's scratch (%.1f MB) stay in L2 by design"
                             % (nwin, nwin * lb * (sizes[0] + sizes[-1]) * 4 / 1e6, (2 * lb * sum(sizes) + net.nw) * 4 / 1e6),
                       "gradient_exchange": {0: None, 1: "NCCL all-reduce per layer, overlapped with the backward pass",
                                             2: "row bands stored into their owner's memory by the gradient product's "
                                                "epilogue over NVLink; owner sums, updates, writes every replica's staging "
                                                "vector; each rank commits a layer after its last reader of the old weights"}[dp_mode]}),
            "e2e": {"value": e2e_value, "unit": "samples/s" if train else "rows/s", "h2d_bytes_per_step": xb + yb,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "region_ms": regions,
            # the same global windows are trained for every number of GPUs (one global table, see fill_shard), so
            # these three agree across N up to the fp32 summation order
            "loss_first_window": m_first.total_error if m_first else None,
            "loss_after": m_last.total_error if m_last else None,
            "weights_checksum": checksum,
            "flop_per_sample": flop_per_sample(sizes, train),
            "step_tflops": flop_per_sample(sizes, train) * samples_per_step / (ms / args.steps / 1000.0) / 1e12,
        }
        print(json.dumps(line), flush=True)
    net.close()
    plumb.close()


if __name__ == "__main__":
    main()
