#!/usr/bin/env python3
"""Benchmark of the batched MLP forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--dtype int8] [--batch 65536] [--math exact|fast] [--all-dtypes]

The default line also carries a `train` object: the data-parallel Adam training configuration at the same rank count,
and, on one GPU, an `other_configs` object: the wide BF16 net at 16384 rows and the large INT4 net at 1 and 64 rows,
each measured by this script in a child process (`--workload wide|large`), so that every configuration is in one run.

One "step" is one forward pass of the 784-512-1000-10 MLP (weights stored in
the chosen .nn precision, INT8 by default) over one batch of 65536 synthetic
U[0,1) rows per GPU.  Ranks are independent (weights replicated, rows sharded,
no collective), so scaling is weak: `value` is all ranks' rows per second.

  value     device-resident throughput: inputs and outputs in HBM, K steps timed
            with CUDA events on the launching stream, max over ranks
  e2e       the same call with HOST (pinned) buffers: H2D of the batch and D2H
            of the result inside the timed region
  roofline  the dominant kernel of the path that ran (config.path): the one-launch
            three-layer kernel or the per-layer tcgen05 GEMM -- algorithmic FLOPs of
            its launches / their summed device time (event pairs recorded by the
            library around each launch), against the measured bf16 peak; the GEMV or
            weight-streaming kernel for small batches -- packed weight bytes / time,
            against the measured HBM bandwidth
  cpu_baseline  the reference's own CPU forward (built from its sources into
            oracle/_ref) or, if that is absent, the C restatement in oracle/,
            timed on this host's cores on a bounded sample of the same batch

`--impl reference` runs only that CPU arm and prints the same JSON shape.
"""
import argparse
import atexit
import ctypes
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOPO = [784, 512, 1000, 10]
FLOP_PER_SAMPLE = 2 * (784 * 512 + 512 * 1000 + 1000 * 10)       # 1 846 816

# name -> (topology, activation names, default dtype, default batch, weight gain, input distribution)
WORKLOADS = {
    "mlp":   ([784, 512, 1000, 10], "A", "int8", 65536, 2.0, "uniform"),
    "wide":  ([4096, 8192, 8192, 8192, 8192, 4096, 1000], "W", "bf16", 16384, 1.0, "normal"),
    "large": ([8192, 16384, 16384, 8192, 1000], "L", "int4", 1, 2.0, "normal"),
}
BITS = {"fp32": 32, "fp16": 16, "bf16": 16, "int8": 8, "int4": 4, "int2": 2}


def flops_per_sample(topo):
    return 2 * sum(a * b for a, b in zip(topo[:-1], topo[1:]))


def algorithmic_bytes(topo, dtype, batch):
    """Weights and biases once in their stored precision (+4-byte abs-max per integer array), input and output rows."""
    bits, extra = BITS[dtype], (4 if dtype.startswith("int") else 0)
    total = 0
    for a, b in zip(topo[:-1], topo[1:]):
        total += (a * b * bits + 7) // 8 + extra + (b * bits + 7) // 8 + extra
    return total + batch * topo[0] * 4 + batch * topo[-1] * 4
METRIC = "mlp_forward_samples_per_sec"
PRECS = ["fp32", "fp16", "bf16", "int8", "int4", "int2"]


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="mlp", choices=list(WORKLOADS), help="mlp = the benchmark line; wide/large = the other configurations")
    ap.add_argument("--dtype", default=None, choices=PRECS)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--math", default="auto", choices=["auto", "exact", "fast"])
    ap.add_argument("--all-dtypes", action="store_true", help="also report every stored precision (fewer steps each); on by default for the mlp workload")
    ap.add_argument("--one-dtype", action="store_true", help="skip the per-dtype table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-train", action="store_true", help="skip the training leg of the mlp workload")
    ap.add_argument("--no-others", action="store_true", help="skip the other configurations (wide, large) of the default line")
    ap.add_argument("--train", action="store_true", help="secondary line: data-parallel Adam training steps (256 rows per GPU per step) instead of inference")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    args.topo, args.dtype, args.batch = w[0], args.dtype or w[2], args.batch or w[3]
    return args


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons sampled (read-only, through NVML) while the timed region runs;
    falls back to polling nvidia-smi when the NVML binding is missing."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.sm = []
        self.reasons = set()
        self.sm_max = None
        self._stop = threading.Event()
        self._t = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[gpu_index]) if visible and visible.split(",")[gpu_index].isdigit() else gpu_index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.sm.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
        mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
            else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        for name, bit in (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40), ("sw_power_cap", 0x4)):
            if mask & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        if not out:
            return
        r = [c.strip() for c in out.splitlines()[0].split(",")]
        self.sm.append(float(r[1]))
        self.sm_max = float(r[2])
        for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
            if r[col].lower().startswith("active"):
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.002 if self._nvml else 0.05)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["unsampled"]}
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(sm), "source": "nvml" if self._nvml else "nvidia-smi"}


def make_net_file(spg, dtype, tmpdir, workload="mlp"):
    from spingalett_b200 import configs as nets
    if workload == "mlp":
        return nets.make_net_file(spg, os.path.join(tmpdir, f"mlp_{dtype}.nn"), nets.A_TOPO, nets.A_ACTS,
                                  spg.abi.PRECISION_NAMES[dtype], seed=1234, reference_rng=True)
    topo, acts = (nets.W_TOPO, nets.W_ACTS) if workload == "wide" else (nets.L_TOPO, nets.L_ACTS)
    return nets.make_net_file(spg, os.path.join(tmpdir, f"{workload}_{dtype}.nn"), topo, acts,
                              spg.abi.PRECISION_NAMES[dtype], gain=WORKLOADS[workload][4], seed=77)


def make_inputs(workload, batch, width, seed):
    from spingalett_b200 import configs as nets
    return nets.uniform_inputs(batch, width, seed) if WORKLOADS[workload][5] == "uniform" else nets.normal_inputs(batch, width, seed)


def cpu_arm(path, x, steps, warmup, sample_rows):
    """Times the reference's CPU forward (or the oracle port) on `sample_rows` rows per step."""
    from oracle import Oracle, OracleNet, Reference
    xs = np.ascontiguousarray(x[:sample_rows])
    cores = os.cpu_count() or 1
    if Reference.available():
        R = Reference
        lib = R.lib()
        lib.spingalett_set_num_threads(cores)
        net = R.load(path)
        blas = bool(lib.refh_has_blas())
        if blas:
            lib.refh_blas_threads(cores)
            lib.spingalett_set_compute_mode(2)      # COMPUTE_OPENBLAS
            ws = lib.refh_ws_create(net, sample_rows)
            run = lambda: lib.refh_ws_forward(net, ws, xs.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), sample_rows)
            how = "reference batch_forward (OpenBLAS sgemm + its own bias/activation/softmax passes)"
        else:
            lib.spingalett_set_compute_mode(1)      # COMPUTE_OPENMP
            run = lambda: R.forward_batch(net, xs)
            how = "reference forward() per sample (OpenMP)"
        kind = "reference"
    else:
        net = OracleNet.from_file(path)
        run = lambda: net.forward_batch(xs)
        kind, how = "port", "oracle C restatement, OpenMP over rows"
        cores = Oracle.threads()
    for _ in range(max(1, warmup)):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    return {"value": sample_rows * steps / dt, "unit": "samples/s", "cores": cores, "kind": kind,
            "sample": f"{sample_rows} rows x {steps} steps of the same batch; {how}", "ms_per_step": dt / steps * 1e3}


def workload_name(args):
    """One description of the configuration, shared by both arms."""
    dist_name = "U[0,1)" if WORKLOADS[args.workload][5] == "uniform" else "N(0,1)"
    return (f"MLP {'-'.join(map(str, args.topo))} forward, weights stored {args.dtype} (.nn), batch {args.batch} per GPU, "
            f"{dist_name} fp32 inputs")


def reference_net_file(dtype, tmpdir, workload):
    """The same .nn file as make_net_file(), written by the reference library itself (its own generator stream after
    rng_seed for the benchmark MLP, the same numpy draws for the two large nets, its own save_spingalett), so the
    reference arm never loads this repository's library."""
    from oracle import Reference as R
    from spingalett_b200 import abi, configs
    path = os.path.join(tmpdir, f"{workload}_{dtype}_ref.nn")
    if workload == "mlp":
        net = R.build_net(configs.A_TOPO, configs.A_ACTS, abi.WEIGHT_INITIALIZATION_HE, seed=1234)
    else:
        topo, acts = (configs.W_TOPO, configs.W_ACTS) if workload == "wide" else (configs.L_TOPO, configs.L_ACTS)
        net = R.build_net(topo, acts, abi.WEIGHT_INITIALIZATION_NONE)

        class _View:                      # what configs.fill_normal writes into
            weights, biases = R.weights(net), R.biases(net)
        configs.fill_normal(_View, topo, WORKLOADS[workload][4], 77)
    R.save(net, path, abi.PRECISION_NAMES[dtype])
    R.free(net)
    return path


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import Reference
    tmpdir = tempfile.mkdtemp(prefix="spg_bench_")
    atexit.register(shutil.rmtree, tmpdir, ignore_errors=True)      # the .nn files of the large nets are hundreds of MB
    if Reference.available():
        path = reference_net_file(args.dtype, tmpdir, args.workload)
    else:
        import spingalett_b200 as spg      # no reference build here: the oracle port reads a file this library writes
        spg.lib().spingalett_set_verbose(False)
        path = make_net_file(spg, args.dtype, tmpdir, args.workload)
    x = make_inputs(args.workload, args.batch, args.topo[0], 4321)
    r = cpu_arm(path, x, args.steps, args.warmup, args.batch)
    line = {"metric": METRIC, "value": r["value"], "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": workload_name(args), "batch_per_gpu": args.batch,
                       "note": "the reference dequantises the file to fp32 at load and computes in fp32 (OpenBLAS sgemm)"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def measure(spg, net, torch, x_dev, y_dev, x_pin, y_pin, batch, steps, warmup, dist, local_rank):
    """Returns (device ms/step, e2e ms/step, kernel ms, kernel launches, launches, clocks)."""
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(3, warmup)):
        net.forward_batch_ptr(x_dev.data_ptr(), batch, y_dev.data_ptr())
    net.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clk:
        l0 = spg.kernel_launches()
        start.record()
        for _ in range(steps):
            net.forward_batch_ptr(x_dev.data_ptr(), batch, y_dev.data_ptr())
        stop.record()
        barrier()
        launches = spg.kernel_launches() - l0
        # the same steps again with an event pair around every launch of the dominant kernel (roofline timing);
        # kept out of the loop above because an event between two kernels stops the next layer from starting
        # its weight fetch under the tail of the one before it
        net.profile(True)
        for _ in range(steps):
            net.forward_batch_ptr(x_dev.data_ptr(), batch, y_dev.data_ptr())
        net.synchronize()
        k_ms, k_cnt = net.profile_read()
        net.profile(False)
    dev_ms = reduce_max(start.elapsed_time(stop)) / steps

    # end to end: pinned host buffers through the public call, copies inside the timed region
    for _ in range(2):
        net.forward_batch_ptr(x_pin.data_ptr(), batch, y_pin.data_ptr())
    barrier()
    e2e_steps = max(3, steps // 4)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        net.forward_batch_ptr(x_pin.data_ptr(), batch, y_pin.data_ptr())      # returns with the result on the host
    torch.cuda.synchronize()
    e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3) / e2e_steps
    # the same call on ordinary (pageable) host arrays, which is what a C caller of the reference API passes
    x_page, y_page = x_pin.numpy().copy(), np.empty_like(y_pin.numpy())
    net.forward_batch_ptr(x_page.ctypes.data, batch, y_page.ctypes.data)
    barrier()
    t0 = time.perf_counter()
    for _ in range(2):
        net.forward_batch_ptr(x_page.ctypes.data, batch, y_page.ctypes.data)
    torch.cuda.synchronize()
    measure.pageable_ms = reduce_max((time.perf_counter() - t0) * 1e3) / 2
    return dev_ms, e2e_ms, k_ms, k_cnt, launches, clk.summary()


def run_train(args):
    """Training configuration: MLP 784-512-1000-10, fp32, 256 rows per GPU per step, cross-entropy, Adam lr 1e-3; with more
    than one rank the flat gradient is all-reduced over NCCL every step.  One train() call runs `steps` optimiser steps
    (100 epochs over 20*256 rows in shuffled mini-batches of 256, so that the per-call costs - allocation, upload, read-back - weigh a few percent); CUDA events on the library's stream bracket the call,
    the upload of the host arrays and the read-back of weights and optimiser state included."""
    import torch
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")
    import spingalett_b200 as spg
    lib = spg.lib()
    lib.spingalett_set_verbose(False)
    lib.spingalett_set_device(local)
    if world > 1:
        uid = np.zeros(128, np.uint8)
        if rank == 0:
            assert lib.spingalett_dist_unique_id(uid.ctypes.data) == 0
        t = torch.from_numpy(uid)
        dist.broadcast(t, 0)
        assert lib.spingalett_dist_init(rank, world, t.numpy().ctypes.data) == 0
    topo = [784, 512, 1000, 10]
    net = spg.Network.build(topo, [spg.abi.ACT_RELU, spg.abi.ACT_RELU, spg.abi.ACT_SOFTMAX], spg.abi.WEIGHT_INITIALIZATION_HE, seed=1234)
    net.set_stream(torch.cuda.current_stream().cuda_stream)
    epochs = max(args.steps, 20) * 5
    steps = epochs * 20
    rng = np.random.default_rng(100 + rank)
    rows = 256 * 20
    x = rng.random((rows, 784), dtype=np.float32)
    tg = np.zeros((rows, 10), np.float32)
    tg[np.arange(rows), rng.integers(0, 10, rows)] = 1.0
    kw = dict(epochs=epochs, batch_size=256, strategy=spg.abi.STRATEGY_SMALL_BATCH, learning_rate=1e-3)
    net.train(x[:256 * 8], tg[:256 * 8], **dict(kw, epochs=1))                      # warm-up: allocations, NCCL channels
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = spg.kernel_launches()
    e0.record()
    net.train(x, tg, **kw)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = spg.kernel_launches() - l0
    if dist is not None:
        tt = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    if rank == 0:
        print(json.dumps({"metric": "mlp_train_samples_per_sec", "value": 256 * steps * world / (ms * 1e-3), "unit": "samples/s", "n_gpus": world,
                          "steps": steps, "warmup": 8, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic",
                          "config": {"workload": "MLP 784-512-1000-10 training, 256 rows per GPU per step, cross-entropy, Adam lr 1e-3, one train() call of %d epochs over 5120 rows " % epochs +
                                                 "(host arrays in, weights and optimiser state back to the host at the end)",
                                     "collective": "NCCL all-reduce of 924930 fp32 gradients per step" if world > 1 else "none"},
                          "e2e": {"value": 256 * steps * world / (ms * 1e-3), "unit": "samples/s",
                                  "h2d_bytes_per_step": int((x.nbytes + tg.nbytes + 3 * 924930 * 4) // steps),
                                  "d2h_bytes_per_step": int((4 * 924930 * 4) // steps),
                                  "note": "train() takes host arrays and returns host arrays: the timed region is the call"},
                          "gpu_launches": int(launches)}))
    if world > 1:
        lib.spingalett_dist_shutdown()
        dist.barrier()
        dist.destroy_process_group()
    net.free()


def train_leg(spg, torch, dist, rank, world, epochs):
    """The training configuration at this rank count: MLP 784-512-1000-10 from the reference's generator stream, fp32, 256 rows
    per GPU per step, cross-entropy, Adam lr 1e-3; with more than one rank the gradient is exchanged over NVLink every step.
    One train() call of `epochs` epochs over 20*256 rows per rank (host arrays in, weights and optimiser state back to the
    host at the end); device time of the call, max over ranks."""
    lib = spg.lib()
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            host = np.zeros(128, np.uint8)
            assert lib.spingalett_dist_unique_id(host.ctypes.data) == 0
            uid.copy_(torch.from_numpy(host))
        dist.broadcast(uid, 0)
        host = uid.cpu().numpy()
        assert lib.spingalett_dist_init(rank, world, host.ctypes.data) == 0
    net = spg.Network.build(TOPO, [spg.abi.ACT_RELU, spg.abi.ACT_RELU, spg.abi.ACT_SOFTMAX], spg.abi.WEIGHT_INITIALIZATION_HE, seed=1234)
    net.set_stream(torch.cuda.current_stream().cuda_stream)
    steps = epochs * 20
    rng = np.random.default_rng(100 + rank)
    rows = 256 * 20
    x = rng.random((rows, 784), dtype=np.float32)
    tg = np.zeros((rows, 10), np.float32)
    tg[np.arange(rows), rng.integers(0, 10, rows)] = 1.0
    kw = dict(batch_size=256, strategy=spg.abi.STRATEGY_SMALL_BATCH, learning_rate=1e-3)
    net.train(x[:256 * 8], tg[:256 * 8], epochs=1, **kw)                  # warm-up: allocations, communicator channels
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    # The call is ten launches per 0.12 ms step issued by one host thread, so a descheduled host shows at once: two
    # identical calls, both reported (calls_ms), the faster one taken (max over ranks of each call first).
    calls = []
    for _ in range(2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = spg.kernel_launches()
        e0.record()
        net.train(x, tg, epochs=epochs, **kw)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = spg.kernel_launches() - l0
        if dist is not None:
            tt = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        calls.append(ms)
    ms = min(calls)
    if dist is not None:
        lib.spingalett_dist_shutdown()
    net.free()
    return {"metric": "mlp_train_samples_per_sec", "value": 256 * steps * world / (ms * 1e-3), "unit": "samples/s",
            "ms_per_step": ms / steps, "steps": steps, "world": world, "rows_per_gpu_per_step": 256, "dtype": "f32",
            "gpu_launches": int(launches), "calls_ms": [round(c, 3) for c in calls],
            "collective": "gradient exchange of 924930 fp32 values per step over NVLink" if world > 1 else "none",
            "note": "one train() call: host arrays in, weights and optimiser state back on the host at the end, inside the timed region; the faster of two identical calls (calls_ms)"}


def other_configs():
    """The wide BF16 net (16384 rows, AUTO) and the large INT4 net (1 row: GEMV; 64 rows: weight streaming), each run by
    this script in a child process once the parent's measurement is over; a short form of each child's line is kept.
    A child that fails leaves its error text in its place: the parent's line does not depend on it."""
    out = {}
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")}
    for key, extra in (("wide_bf16_b16384_auto", ["--workload", "wide", "--steps", "5"]),
                       ("large_int4_b1", ["--workload", "large", "--batch", "1"]),
                       ("large_int4_b64", ["--workload", "large", "--batch", "64"])):
        cmd = [sys.executable, os.path.abspath(__file__), *extra, "--one-dtype", "--no-cpu"]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env)
            d = json.loads(r.stdout.strip().splitlines()[-1])
            rf = d.get("roofline") or {}
            out[key] = {"value": d["value"], "unit": d["unit"], "ms_per_step": d["ms_per_step"], "steps": d["steps"],
                        "workload": d["config"]["workload"], "path": d["config"]["path"], "dtype": d["dtype"],
                        "e2e": d["e2e"]["value"], "gpu_launches": d["gpu_launches"], "clocks": d.get("clocks"),
                        "roofline": {k: rf.get(k) for k in ("bound", "achieved", "peak", "unit", "frac", "whole_step_frac", "kernel")}}
        except Exception as e:                      # noqa: BLE001 - reported, not fatal
            out[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    if args.train:
        return run_train(args)

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    import spingalett_b200 as spg
    lib = spg.lib()
    lib.spingalett_set_verbose(False)
    assert lib.spingalett_set_device(local_rank) == 0
    spg.set_math_mode({"exact": spg.abi.MATH_EXACT, "fast": spg.abi.MATH_FAST, "auto": spg.abi.MATH_AUTO}[args.math])
    pk = peaks()
    tmpdir = tempfile.mkdtemp(prefix=f"spg_bench_r{rank}_")
    atexit.register(shutil.rmtree, tmpdir, ignore_errors=True)      # the .nn files of the large nets are hundreds of MB
    batch = args.batch

    topo = args.topo
    x = make_inputs(args.workload, batch, topo[0], 4321 + rank)
    x_dev = torch.from_numpy(x).cuda()
    y_dev = torch.empty((batch, topo[-1]), dtype=torch.float32, device="cuda")
    x_pin = torch.from_numpy(x).pin_memory()
    y_pin = torch.empty((batch, topo[-1]), dtype=torch.float32).pin_memory()

    def run_dtype(dtype, steps, warmup):
        path = make_net_file(spg, dtype, tmpdir, args.workload)
        net = spg.Network.load(path)
        net.set_stream(torch.cuda.current_stream().cuda_stream)
        res = measure(spg, net, torch, x_dev, y_dev, x_pin, y_pin, batch, steps, warmup, dist, local_rank)
        path_taken = spg.last_path()
        net.free()
        return path, res, path_taken

    path, (dev_ms, e2e_ms, k_ms, k_cnt, launches, clocks), path_taken = run_dtype(args.dtype, args.steps, args.warmup)
    value = batch * world / (dev_ms * 1e-3)
    e2e_value = batch * world / (e2e_ms * 1e-3)
    passes = 2 if args.math == "exact" else 1
    compute = {"exact": "bf16(hi+lo)xbf16->f32", "fast": "f16xf16->f32", "auto": "f16xf16->f32 + exact recompute of low-margin rows"}[args.math]
    if path_taken == "gemv" and args.dtype in ("int8", "int4", "int2"):
        compute = "s8 digits x s8 -> s32 (exact sums of 28-bit fixed-point activations)"
    elif path_taken in ("gemv", "wstream"):
        compute = "bf16 terms x bf16 -> f32 (exact products)"
    line = {
        "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": compute, "data": "synthetic",
        "config": {"workload": workload_name(args), "batch_per_gpu": batch, "math_mode": args.math, "path": path_taken,
                   "l2": ("inputs (205 MB per batch) and activations exceed the 126 MB L2; no explicit flush" if args.workload == "mlp"
                          else "the stored weights streamed every step (>= 136 MB) exceed the 126 MB L2; no explicit flush"),
                   "sharding": "rows across ranks, weights replicated, no collective"},
        "e2e": {"value": e2e_value, "unit": "samples/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": batch * topo[0] * 4, "d2h_bytes_per_step": batch * topo[-1] * 4,
                "host_buffers": "pinned", "pageable_value": batch * world / (measure.pageable_ms * 1e-3),
                "pageable_ms_per_step": measure.pageable_ms},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if k_cnt and path_taken.startswith("tcgen05"):
        fused = path_taken == "tcgen05-fused"
        flops = flops_per_sample(topo) * batch * args.steps      # algorithmic: 2*N*sum(in*out), one term per product
        k_ms_eff = min(k_ms, dev_ms * args.steps)                # event pairs around single launches cannot undercut the timed loop
        achieved = flops / (k_ms_eff * 1e-3) / 1e12
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "mlp3_fused_traffic.json" if fused else "gemm_tc_traffic.json")
        if os.path.exists(tpath):
            traffic = json.load(open(tpath)).get(f"{args.workload}_{args.dtype}_{args.math}_{batch}")
        line["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                            "frac": achieved / pk["bf16_tflops"], "traffic": traffic,
                            "kernel": "spg_mlp3_fused_kernel" if fused else "spg_gemm_tc_kernel",
                            "launches": int(k_cnt), "kernel_ms_per_step": k_ms_eff / args.steps,
                            "peak_source": pk["source"] + " burst bf16", "tensor_passes_per_product": passes,
                            "executed_frac": achieved * passes / pk["bf16_tflops"],
                            "whole_step_frac": flops / (dev_ms * args.steps * 1e-3) / 1e12 / pk["bf16_tflops"],
                            "note": ("frac: the one launch per step that computes all three layers of all rows (event pair around it); "
                                     "whole_step_frac: the same FLOPs over ms_per_step, which in AUTO also holds the exact "
                                     "recomputation of the low-margin rows (per-layer kernels on a percent or two of the rows)")
                                    if fused else "frac: summed device time of the layer kernels (event pairs); whole_step_frac: over ms_per_step"}
    elif k_cnt:
        nbytes = algorithmic_bytes(topo, args.dtype, batch)      # per step, all layers (one kernel launch per layer)
        achieved = nbytes * args.steps / (k_ms * 1e-3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "gemv_traffic.json")
        if os.path.exists(tpath):
            traffic = json.load(open(tpath)).get(f"{args.workload}_{args.dtype}_{batch}")
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                            "frac": achieved / pk["hbm_gbs"], "traffic": traffic,
                            "kernel": "spg_wstream_kernel" if path_taken == "wstream" else "spg_gemv_kernel",
                            "launches": int(k_cnt), "kernel_ms_per_step": k_ms / args.steps,
                            "algorithmic_bytes_per_step": nbytes, "peak_source": pk["source"] + " copy bandwidth",
                            "whole_step_frac": nbytes / (dev_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                            "note": "frac: event pairs around each layer kernel in a separate pass (events keep a layer from "
                                    "prefetching weights under the previous one); whole_step_frac: algorithmic bytes / ms_per_step "
                                    "of the timed loop, staging and softmax included"}
    if (args.all_dtypes or args.workload == "mlp") and not args.one_dtype:
        per = {}
        for dt in PRECS:
            _, (d_ms, e_ms, km, kc, _, _), _ = run_dtype(dt, max(5, args.steps // 2), 3)
            ktf = (flops_per_sample(topo) * batch * max(5, args.steps // 2) / (km * 1e-3) / 1e12) if kc else None
            per[dt] = {"value": batch * world / (d_ms * 1e-3), "e2e": batch * world / (e_ms * 1e-3),
                       "kernel_tflops": ktf, "roofline_frac": (ktf / pk["bf16_tflops"]) if ktf else None}
        line["per_dtype"] = per
    if args.workload == "mlp" and not args.no_train:
        line["train"] = train_leg(spg, torch, dist, rank, world, max(40, args.steps * 2))
    if rank == 0 and world == 1 and not args.no_cpu:
        sample = min(batch, 16384 if args.workload == "mlp" else 64)
        cb = cpu_arm(path, x, 3, 1, sample)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if args.workload == "mlp" and world == 1 and not args.no_others and not args.one_dtype:
        torch.cuda.synchronize()
        del x_dev, y_dev, x_pin, y_pin
        torch.cuda.empty_cache()
        line["other_configs"] = other_configs()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
