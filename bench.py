"""Throughput of the ViT training step (forward + backward + clip + AdamW).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2]
    python bench.py --impl reference ...      # the reference's CPU path

One step = one call of the reference's vit_model_train_batch_smoothed on one
synthetic batch.  The host side is the reference's unmodified C code
(transformer-in-c_b200/host/libvithost.so, built from the reference sources);
with the B200 backend enabled every op it dispatches runs as one of this
repository's CUDA kernels.  Prints ONE JSON line (rank 0).  Workloads quoted on
a fixed global batch (cfg5: 4096 images per optimiser step whatever the GPU
count) run each rank's share as micro-batches with gradient accumulation, one
optimiser call and one gradient exchange per step ("scaling": "strong").

The headline numbers of the line are the workload named by --workload (cfg2,
the configuration the metric is quoted on).  Unless --no-cfg5 is given the
line also carries a "cfg5" object: the data-parallel configuration (d 512, 12
layers, global batch 4096) measured the same way at the same GPU count, so a
run at 1, 2, 4 and 8 GPUs yields its strong-scaling curve.

Timed quantities (three passes of K steps each, after W warm-up steps)
  e2e    wall clock over K steps called with HOST buffers: per step the host
         copies images + labels in, the backend uploads them, and the loss is
         read back.  The `synchronize` slot is deferred in this pass
         (vitb200_set_deferred_synchronize; --strict-synchronize turns that
         off), so the host's share of a step overlaps the device's backward
         pass of the step before; the pass ends with a device synchronise.
  value  K more steps, counting only the time the device stream was busy
         between the first op after the uploads and the synchronise that ends
         the step (two CUDA events on the backend's stream, nothing else in
         it): throughput with the batch already resident in HBM.
  roofline  K more steps with a CUDA event pair around every op; the op with
         the largest share is reported: achieved = its algorithmic bytes (or
         flops) / that time.  ms_per_step_with_op_events is this pass's step.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

import importlib.util

REPO = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.join(REPO, "transformer-in-c_b200")
# The reference's unmodified host code, compiled twice by oracle/build_ref.py:
# the copy that drives the backend in the timed steps, and the copy that only
# runs the CPU loops (the cpu_baseline legs and --impl reference).
HOST_LIBRARY = os.path.join(PACKAGE, "host", "libvithost.so")
CPU_LIBRARY = os.path.join(REPO, "oracle", "_ref", "libvithost.so")


def load_module(name, path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


# (channels, height, width, patch, d_model, heads, layers, classes), batch
WORKLOADS = {
    "cfg1": ((1, 28, 28, 4, 128, 8, 4, 11), 32),
    "cfg2": ((1, 28, 28, 4, 128, 8, 4, 11), 2048),
    "cfg3": ((1, 28, 28, 2, 256, 8, 6, 11), 512),
    "cfg4": ((1, 64, 64, 2, 384, 6, 12, 11), 64),
    "cfg5": ((1, 28, 28, 2, 512, 8, 12, 11), 512),
}
# Workloads quoted on a fixed GLOBAL batch: every rank takes global / world
# images per optimiser step, in micro-batches of the size above (gradient
# accumulation), so the total work is the same at every GPU count.
GLOBAL_BATCH = {"cfg5": 4096}
LR, WD, SMOOTHING = 1e-3, 0.05, 0.1
TENSOR_OPS = {"gemm", "gemm_backward", "multi_head_attention",
              "multi_head_attention_backward"}


def measured_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
        return (float(peaks["hbm_gbs"]),
                float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])),
                "measured")
    return 6650.0, 1400.0, "fallback"


def measure_tf32_peak(seconds=2.0):
    """Dense TF32 rate of this GPU, measured here because no recorded peak
    exists for it: a cuBLAS FP32 matmul with TF32 allowed, 8192^3, as a burst
    (20 products) and sustained over `seconds`.  The library call only
    supplies the denominator of the contractions' roofline fractions."""
    import torch
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    n = 8192
    a = torch.randn(n, n, device="cuda")
    b = torch.randn(n, n, device="cuda")
    c = torch.empty(n, n, device="cuda")

    def timed(count):
        begin = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(count):
            torch.matmul(a, b, out=c)
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / 1e3

    timed(3)
    burst_seconds = timed(20)
    burst = 2.0 * n ** 3 * 20 / burst_seconds / 1e12
    count = max(20, int(seconds / (burst_seconds / 20)))
    sustained = 2.0 * n ** 3 * count / timed(count) / 1e12
    torch.backends.cuda.matmul.allow_tf32 = previous
    del a, b, c
    torch.cuda.empty_cache()
    return {"burst_tflops": burst, "sustained_tflops": sustained,
            "how": f"torch.matmul fp32 8192^3 with TF32 allowed: 20 products, "
                   f"then {count} products"}


def recorded_traffic(kernel, workload, batch):
    """dram__bytes_read + dram__bytes_write per launch of `kernel` from the ncu
    capture summarised under profiles/ (the JSON beside the summary names the
    capture's workload, batch and source commit), scaled to this batch by the
    rows processed; None when no capture of this kernel and workload exists."""
    path = os.path.join(REPO, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    for entry in json.load(open(path)).get("captures", []):
        if entry["kernel"] == kernel and entry["workload"] == workload:
            return entry["bytes_per_launch"] * batch / entry["batch"]
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region
    runs (read-only query; nothing is changed on the GPU)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device),
                 "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *unused):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.process:
            return
        time.sleep(0.15)
        self.process.terminate()
        out, _ = self.process.communicate()
        clocks, reasons, maximum = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                 "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maximum = float(parts[1])
            except ValueError:
                continue
            for name, state in zip(names, parts[2:6]):
                if state.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.summary = {"sm_mhz": float(np.median(clocks)),
                            "sm_max_mhz": maximum, "reasons": sorted(reasons)}


def pinned_like(array):
    """Copy of `array` in page-locked host memory (torch owns the pages)."""
    import torch
    tensor = torch.from_numpy(array).pin_memory()
    return tensor, tensor.numpy()


def cpu_reference_rate(vh, host_lib, config, seconds_budget, max_batch=32):
    """images/s of the reference's CPU code on one core, on a bounded sample:
    a batch sized from a one-image probe so the timed steps fit the budget."""
    probe = vh.VitHost(host_lib, config, 1)
    images, labels = vh.synthetic_batch(1, config[1], config[2], config[7], 77)
    start = time.perf_counter()
    probe.train_step(images, labels, LR, WD, None, SMOOTHING)
    per_image = time.perf_counter() - start
    probe.close()
    batch = int(max(1, min(max_batch, seconds_budget / (2.0 * per_image))))
    host = vh.VitHost(host_lib, config, batch)
    images, labels = vh.synthetic_batch(batch, config[1], config[2], config[7], 78)
    steps = 2
    start = time.perf_counter()
    for _ in range(steps):
        host.train_step(images, labels, LR, WD, None, SMOOTHING)
    elapsed = time.perf_counter() - start
    host.close()
    return batch * steps / elapsed, batch, steps


# The trainer's augmentation settings (reference examples/organ_smnist.c:142-151)
# for pixels in [0, 1].
AUGMENTATION = {
    "max_shift_pixels": 2.0, "max_rotation_degrees": 10.0,
    "max_scale_delta": 0.1, "max_brightness_delta": 0.05,
    "max_contrast_delta": 0.1, "noise_standard_deviation": 0.01,
    "erasing_probability": 0.25, "erasing_max_side_fraction": 0.4,
    "erasing_value": 0.5, "minimum_value": 0.0, "maximum_value": 1.0,
}


def augmentation_measurement(backend, host_lib, batch, channels, height, width,
                             steps, with_cpu):
    """The batch augmentation that precedes every training step in the
    reference's trainer (examples/organ_smnist.c:594-612), on the device:
    `e2e` with page-locked host buffers in and out (both copies inside the
    timed calls), `value` from the kernels' own CUDA events; beside them the
    reference's C code on one host core over a bounded sample."""
    rng = np.random.RandomState(11)
    pixels = (rng.randint(0, 256, size=(batch, channels, height, width))
              .astype(np.float32) / np.float32(255.0))
    keep_in, source = pinned_like(pixels)
    keep_out, destination = pinned_like(np.zeros_like(pixels))
    state = 1
    for _ in range(3):
        status, _, state = backend.augment(AUGMENTATION, state, source, destination)
        assert status == 0
    backend.profile(True)
    start = time.perf_counter()
    for _ in range(steps):
        status, _, state = backend.augment(AUGMENTATION, state, source, destination)
    elapsed = time.perf_counter() - start
    kernel_ms = sum(e["ms"] for e in backend.profile_entries()
                    if e["name"] == "data_augmentation")
    backend.profile(False)
    images = batch * steps
    hbm_peak, _, peak_source = measured_peaks()
    result = {
        "metric": "augmented images/s", "unit": "images/s",
        "settings": "reference trainer defaults",
        "batch": batch, "image": [channels, height, width],
        "value": images / (kernel_ms / 1e3),
        "e2e": {"value": images / elapsed,
                "h2d_bytes_per_step": int(pixels.nbytes) + batch * 48,
                "d2h_bytes_per_step": int(pixels.nbytes)},
        # One read and one write of every pixel.
        "roofline": {"bound": "hbm", "achieved": 2 * pixels.nbytes * steps /
                     (kernel_ms / 1e3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                     "peak_source": peak_source},
    }
    result["roofline"]["frac"] = result["roofline"]["achieved"] / hbm_peak
    if with_cpu:
        golden = load_module("make_augmentation_golden", os.path.join(
            REPO, "tests", "golden", "make_augmentation_golden.py"))
        lib = golden.reference_library()
        sample = pixels[:min(batch, 512)]
        start = time.perf_counter()
        golden.reference_apply(lib, AUGMENTATION, 1, sample)
        cpu_seconds = time.perf_counter() - start
        result["cpu_baseline"] = {
            "value": len(sample) / cpu_seconds, "unit": "images/s", "cores": 1,
            "kind": "reference",
            "sample": f"reference data_augmentation_apply, {len(sample)} images, one call"}
    del keep_in, keep_out
    return result


def dataset_measurement(vh, backend, batch, height, width, steps, with_cpu):
    """Batches out of a device-resident dataset (include/vitb200_dataset.h):
    gather by the shuffled order, integer -> [0, 1] -> normalised float, the
    work the reference's trainer does on the host once per dataset and per
    epoch (examples/organ_smnist.c:75-139).  `value` from the kernel's own CUDA
    events, `e2e` with a page-locked host destination (copy inside the call);
    algorithmic bytes: one stored byte read and one float written per pixel."""
    rng = np.random.RandomState(5)
    samples = 8 * batch
    pixels = rng.randint(0, 256, size=(samples, height, width)).astype(np.uint16)
    labels = rng.randint(0, 11, size=samples).astype(np.uintp)
    dataset = vh.Dataset(backend, pixels=pixels, labels=labels)
    mean, inverse = dataset.statistics()
    dataset.shuffle(1)
    keep, destination = pinned_like(np.zeros((batch, height * width), np.float32))
    for index in range(3):
        dataset.batch(index * batch, batch, mean, inverse, destination)
    backend.profile(True)
    start = time.perf_counter()
    for index in range(steps):
        status, _, _ = dataset.batch((index % 8) * batch, batch, mean, inverse,
                                     destination)
        assert status == 0
    elapsed = time.perf_counter() - start
    kernel_ms = sum(e["ms"] for e in backend.profile_entries()
                    if e["name"] == "dataset_batch")
    backend.profile(False)
    dataset.close()
    del keep
    hbm_peak, _, peak_source = measured_peaks()
    moved = 5.0 * batch * height * width * steps
    result = {
        "metric": "dataset batch images/s", "unit": "images/s", "batch": batch,
        "samples": samples, "storage": "uint8",
        "value": batch * steps / (kernel_ms / 1e3),
        "e2e": {"value": batch * steps / elapsed, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 4 * batch * height * width},
        "roofline": {"bound": "hbm", "achieved": moved / (kernel_ms / 1e3) / 1e9,
                     "peak": hbm_peak, "unit": "GB/s", "peak_source": peak_source},
    }
    result["roofline"]["frac"] = result["roofline"]["achieved"] / hbm_peak
    if with_cpu:
        dataset_reference = load_module("dataset_reference", os.path.join(
            REPO, "tests", "dataset_reference.py"))
        timed = dataset_reference.time_reference(samples, height, width)
        if timed:
            result["cpu_baseline"] = {
                "value": samples / timed["shuffle_seconds"], "unit": "images/s",
                "cores": 1, "kind": "reference",
                "sample": f"reference trainer shuffle_dataset over {samples} "
                          f"images in memory (its batches are slices of the "
                          f"shuffled array), mean of 3; its one-off "
                          f"normalize_dataset took "
                          f"{1e3 * timed['normalise_seconds']:.1f} ms"}
    return result


def reference_cuda_rate(config, batch, warmup=2, steps=5):
    """Secondary baseline: the reference's own CUDA backend (src/cuda_backend.cu,
    cuBLAS FP32 SGEMM + managed memory + its SIMT kernels) compiled unmodified
    for sm_100a by oracle/build_ref.py, on the same GPU and workload, in a
    process of its own.  None when that binary is not present or fails."""
    binary = os.path.join(REPO, "oracle", "_ref", "reference_cuda_step")
    if not os.path.exists(binary):
        return None
    command = [binary, *[str(v) for v in config], str(batch), str(warmup), str(steps)]
    try:
        done = subprocess.run(command, capture_output=True, text=True, timeout=240)
        if done.returncode != 0:
            return None
        result = json.loads(done.stdout.strip().splitlines()[-1])
    except (subprocess.TimeoutExpired, ValueError, IndexError):
        return None
    return {"value": result["images_per_second"], "unit": "images/s",
            "ms_per_step": result["ms_per_step"], "batch": batch, "steps": steps,
            "kind": "reference src/cuda_backend.cu built for sm_100a (cuBLAS FP32, "
                    "managed memory), wall clock around the same train calls"}


def reference_replica(args):
    """One replica of the reference arm: a model of its own on its own sample,
    `--warmup` untimed and `--steps` timed CPU train steps; prints the time."""
    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    config, _ = WORKLOADS[args.workload]
    lib = vh.load_host_library(CPU_LIBRARY, visible_to_backend=False)
    host = vh.VitHost(lib, config, args.batch)
    images, labels = vh.synthetic_batch(args.batch, config[1], config[2], config[7],
                                        100 + args.replica)
    for _ in range(args.warmup):
        host.train_step(images, labels, LR, WD, None, SMOOTHING)
    start = time.perf_counter()
    for _ in range(args.steps):
        host.train_step(images, labels, LR, WD, None, SMOOTHING)
    print(json.dumps(time.perf_counter() - start), flush=True)
    host.close()


def run_reference(args, vh, config, batch, rank, world):
    """The reference's own CPU implementation of the step, timed on this
    machine's host cores.  The code is single-threaded on Linux
    (reference src/ops.c:52-55), so all cores are used as independent
    replicas, each stepping its own model on its own sample."""
    if rank != 0:
        return None
    cpu_lib = vh.load_host_library(CPU_LIBRARY, visible_to_backend=False)
    probe = vh.VitHost(cpu_lib, config, 1)
    images, labels = vh.synthetic_batch(1, config[1], config[2], config[7], 77)
    start = time.perf_counter()
    probe.train_step(images, labels, LR, WD, None, SMOOTHING)
    per_image = time.perf_counter() - start
    probe.close()
    total_steps = args.steps + args.warmup
    budget = 150.0
    sample = int(max(1, min(batch, 32, budget / (total_steps * per_image))))
    replicas = max(1, min(os.cpu_count() or 1, 64))
    children = [subprocess.Popen(
        [sys.executable, os.path.abspath(__file__), "--impl", "reference-replica",
         "--workload", args.workload, "--batch", str(sample), "--replica", str(i),
         "--steps", str(args.steps), "--warmup", str(args.warmup)],
        stdout=subprocess.PIPE, text=True) for i in range(replicas)]
    times = [float(json.loads(child.communicate()[0].strip().splitlines()[-1]))
             for child in children]
    elapsed = max(times)
    value = replicas * sample * args.steps / elapsed
    line = {
        "impl": "reference", "metric": "train images/s", "value": value,
        "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "vit": list(config),
                   "batch_per_gpu": batch, "global_batch": batch,
                   "timed_batch_per_replica": sample, "replicas": replicas,
                   "parallelism": "dp1"},
        "cpu_baseline": {
            "value": value, "unit": "images/s", "cores": replicas,
            "kind": "reference",
            "sample": f"{replicas} independent replicas of the reference's "
                      f"single-threaded CPU train step, batch {sample} each, "
                      f"{args.steps} steps (per-image cost is batch-independent)"},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    return line


def measure(vh, backend, host_lib, workload, config, batch, micro_batches, steps,
            warmup, rank, local_rank, world, tf32_peak, strict_synchronize=False):
    """`warmup` untimed and 3 x `steps` timed optimiser steps of one workload
    (one pass for the end-to-end rate, one for device time, one with an event
    pair around every op for the per-op table); returns the fields of a bench
    line."""
    import torch
    import torch.distributed as dist
    backend.set_gradient_accumulation(micro_batches)
    host = vh.VitHost(host_lib, config, batch)
    images, labels = vh.synthetic_batch(batch * micro_batches, config[1],
                                        config[2], config[7], 1234 + rank)
    keep_images, images = pinned_like(images)
    keep_labels, labels = pinned_like(labels.astype(np.int64))
    labels = labels.view(np.uintp)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if micro_batches > 1:
            return host.train_step_accumulated(images, labels, micro_batches,
                                               LR, WD, None, SMOOTHING)
        return host.train_step_raw(images, labels, LR, WD, None, SMOOTHING)

    declined = backend.declined_ops()
    # The warm-up already runs the way the end-to-end pass does (see below), so
    # that its one-time set-up (a second device buffer for the batch, staging
    # memory for the loss) is not part of the timed steps.
    backend.set_deferred_synchronize(0 if strict_synchronize else 1)
    for _ in range(warmup):
        step()

    # ---- e2e: host buffers in, loss out, wall clock ----------------------
    # The way a training program would run it: the `synchronize` slot deferred
    # (vitb200_set_deferred_synchronize), so that the host's part of the next
    # step (zeroing, the memcpy of the next batch into the input tensor, its
    # upload) overlaps the device's backward pass of this one.  Each step still
    # returns its own loss; the barrier below waits for the device.
    backend.set_deferred_synchronize(0 if strict_synchronize else 1)
    barrier()
    counters = backend.memory_counters()
    start = time.perf_counter()
    step_ends = []
    for _ in range(steps):
        loss = step()
        step_ends.append(time.perf_counter())
    barrier()
    e2e_seconds = time.perf_counter() - start
    backend.set_deferred_synchronize(0)
    step_ms = [round(1e3 * (b - a), 3) for a, b in zip([start] + step_ends, step_ends)]
    moved = backend.memory_counters()
    h2d_per_step = (moved["h2d_bytes"] - counters["h2d_bytes"]) / steps
    d2h_per_step = (moved["d2h_bytes"] - counters["d2h_bytes"]) / steps

    # ---- value: device time over K steps --------------------------------
    # Two CUDA events on the backend's stream around each stretch of device
    # work (from the first kernel enqueued after a host synchronisation to the
    # next synchronisation), summed over the K steps; nothing else is recorded
    # in the stream, so chained launches stay chained.
    barrier()
    backend.device_busy_ms(reset=True)
    launches = backend.kernel_launches()
    paths = backend.kernel_paths()
    with ClockSampler(local_rank) as clocks:
        for _ in range(steps):
            loss = step()
        busy_ms = backend.device_busy_ms(reset=True)
    barrier()
    launches = backend.kernel_launches() - launches
    paths = {k: v - paths[k] for k, v in backend.kernel_paths().items()}

    # ---- per-op roofline: an event pair around every op -----------------
    backend.profile(True)
    for _ in range(steps):
        step()
    profiled_ms = backend.device_busy_ms(reset=True)
    barrier()
    entries = backend.profile_entries()
    backend.profile(False)
    declined = backend.declined_ops() - declined

    busy = torch.tensor([busy_ms, e2e_seconds], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(busy, op=dist.ReduceOp.MAX)
    busy_ms, e2e_seconds = float(busy[0]), float(busy[1])
    images_per_step = batch * micro_batches * world
    value = images_per_step * steps / (busy_ms / 1e3)
    e2e_value = images_per_step * steps / e2e_seconds

    hbm_peak, bf16_peak, peak_source = measured_peaks()
    # The contractions take TF32 operands: their roof is the TF32 rate
    # measured on this GPU by this run (sustained figure: the kernels are
    # timed inside a long step).
    tensor_peak = tf32_peak["sustained_tflops"] if tf32_peak else 0.44 * bf16_peak
    tensor_source = ("TF32 matmul measured by this run" if tf32_peak
                     else "0.44 x recorded BF16 rate (TF32 rate not measured by this run: "
                          "several ranks, or --no-tf32-peak)")
    top = max(entries, key=lambda e: e["ms"])
    kernel_name = top["name"]
    traffic_kernel = None
    if top["name"] in ("gemm", "gemm_backward"):
        # Both ops are launches of one kernel (one per forward product, two per
        # gradient pair, each timed as one entry): judge it as a whole.
        parts = [e for e in entries if e["name"] in ("gemm", "gemm_backward")]
        kernel_launches = sum(e["calls"] for e in parts)
        top = {"name": "gemm_tc_kernel", "ms": sum(e["ms"] for e in parts),
               "bytes": sum(e["bytes"] for e in parts),
               "flops": sum(e["flops"] for e in parts), "calls": kernel_launches}
        kernel_name = "gemm_tc_kernel (ops gemm + gemm_backward)"
        traffic_kernel = "gemm_tc_kernel"
    seconds = top["ms"] / 1e3
    tensor_bound = (top["name"] in TENSOR_OPS | {"gemm_tc_kernel"} and
                    top["flops"] / (tensor_peak * 1e12) >
                    top["bytes"] / (hbm_peak * 1e9))
    if tensor_bound:
        achieved, peak, unit = top["flops"] / seconds / 1e12, tensor_peak, "TFLOP/s"
    else:
        achieved, peak, unit = top["bytes"] / seconds / 1e9, hbm_peak, "GB/s"
    traffic = (recorded_traffic(traffic_kernel, workload, batch)
               if traffic_kernel and not tensor_bound else None)
    roofline = {
        "bound": "tensor" if tensor_bound else "hbm", "kernel": kernel_name,
        "achieved": achieved, "peak": peak, "unit": unit,
        "frac": achieved / peak,
        "peak_source": tensor_source if tensor_bound else peak_source,
        "traffic": traffic,
        "algorithmic_per_launch": (top["flops"] if tensor_bound else top["bytes"]) /
                                  max(top["calls"], 1),
        "launch_ms": top["ms"] / top["calls"],
        "share_of_device_time": top["ms"] / sum(e["ms"] for e in entries),
    }
    if tensor_bound:
        roofline["frac_of_recorded_bf16_rate"] = achieved / bf16_peak
    breakdown = {e["name"]: round(e["ms"] / steps, 4)
                 for e in sorted(entries, key=lambda e: -e["ms"])[:24]}
    # Every op against the roofline that bounds it: algorithmic bytes (and
    # flops for the contractions) over the CUDA-event time of its launches.
    by_op = {}
    for e in sorted(entries, key=lambda e: -e["ms"])[:16]:
        if e["ms"] <= 0.0:
            continue
        op = {"ms_per_step": round(e["ms"] / steps, 4),
              "launches_per_step": round(e["calls"] / steps, 1),
              "GB/s": round(e["bytes"] / e["ms"] / 1e6, 1),
              "frac_hbm": round(e["bytes"] / e["ms"] / 1e6 / hbm_peak, 3)}
        if e["flops"] > 0.0:
            op["TFLOP/s"] = round(e["flops"] / e["ms"] / 1e9, 1)
            op["frac_tf32"] = round(e["flops"] / e["ms"] / 1e9 / tensor_peak, 3)
        by_op[e["name"]] = op

    result = {
        "metric": "train images/s", "value": value, "unit": "images/s",
        "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": busy_ms / steps, "higher_is_better": True,
        "scaling": "strong" if micro_batches > 1 or workload in GLOBAL_BATCH
                   else "weak",
        "vs_baseline": None,
        "dtype": "tf32", "data": "synthetic",
        "config": {"workload": workload, "vit": list(config),
                   "batch_per_gpu": batch * micro_batches,
                   "micro_batch": batch, "micro_batches_per_step": micro_batches,
                   "global_batch": images_per_step,
                   "precision": "TF32 operands on the tensor cores, FP32 storage, "
                                "accumulation, softmax, normalisation and optimiser",
                   "parallelism": f"dp{world}" + (
                       " (batch sharded by sample, NCCL all-reduce of gradients "
                       "overlapped with backward)" if world > 1 else ""),
                   "l2": "per-step working set (activations + gradients) far "
                         "exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks.summary,
        "e2e": {"value": e2e_value, "unit": "images/s",
                "h2d_bytes_per_step": h2d_per_step,
                "d2h_bytes_per_step": d2h_per_step,
                "ms_per_step": 1e3 * e2e_seconds / steps,
                "synchronize_slot": "waits" if strict_synchronize else "deferred",
                "ms_of_each_step_on_rank0": step_ms},
        "gpu_launches": launches,
        "ms_per_step_with_op_events": profiled_ms / steps,
        "declined_ops": declined,
        "kernel_paths": paths,
        "roofline": roofline,
        "ms_per_step_by_op": breakdown,
        "roofline_by_op": by_op,
        "loss": loss,
    }
    if world > 1:
        result["dp"] = backend.dp_counters()
    host.close()
    del keep_images, keep_labels
    return result


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours",
                        choices=["ours", "reference", "reference-replica"])
    parser.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    parser.add_argument("--batch", type=int, default=0,
                        help="override the workload's batch (per GPU)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-cfg5", action="store_true",
                        help="leave out the data-parallel configuration's object")
    parser.add_argument("--cfg5-steps", type=int, default=3)
    parser.add_argument("--no-tf32-peak", action="store_true",
                        help="do not measure the TF32 matmul rate first (keeps "
                             "library kernels out of a profiler's launch list)")
    parser.add_argument("--strict-synchronize", action="store_true",
                        help="end-to-end pass with a `synchronize` slot that "
                             "waits for the device, as the reference's does")
    parser.add_argument("--replica", type=int, default=0, help=argparse.SUPPRESS)
    parser.add_argument("--global-batch", type=int, default=-1,
                        help="images per optimiser step over all GPUs; 0 = one "
                             "micro-batch per GPU, -1 = the workload's own")
    args = parser.parse_args()
    if args.impl == "reference-replica":
        reference_replica(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and rank == 0:
        print(f"bench.py: --gpus {args.gpus} but the launcher started {world} "
              f"rank(s); measuring {world}", file=sys.stderr)
    config, batch = WORKLOADS[args.workload]
    if args.batch:
        batch = args.batch

    def micro_batch_count(workload, micro_batch):
        total = (GLOBAL_BATCH.get(workload, 0) if args.global_batch < 0
                 else args.global_batch)
        if not total:
            return 1
        if total % (world * micro_batch):
            parser.error(f"global batch {total} is not a multiple of "
                         f"{world} GPUs x micro-batch {micro_batch}")
        return total // (world * micro_batch)

    micro_batches = micro_batch_count(args.workload, batch)

    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    if args.impl == "reference":
        line = run_reference(args, vh, config, batch, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    import torch
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    os.environ["VITB200_DEVICE"] = str(local_rank)

    # The TF32 roof, before the backend holds any memory.  With several ranks
    # only a single-GPU run measures it (the ranks would share the power and
    # the result would not be a per-GPU peak).
    tf32_peak = (measure_tf32_peak()
                 if world == 1 and not args.no_tf32_peak else None)

    host_lib = vh.load_host_library(HOST_LIBRARY)
    backend = vh.Backend()          # raises without the library or a B200
    if world > 1:
        # One NCCL communicator of our own for the gradient exchange; its id
        # travels through torch.distributed.
        holder = [backend.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(holder, src=0)
        backend.dp_init(rank, world, holder[0])
    backend.enable()
    line = measure(vh, backend, host_lib, args.workload, config, batch,
                   micro_batches, args.steps, args.warmup, rank, local_rank,
                   world, tf32_peak, args.strict_synchronize)
    if tf32_peak:
        line["tf32_peak"] = tf32_peak
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        cpu_lib = vh.load_host_library(CPU_LIBRARY, visible_to_backend=False)
        rate, sample_batch, sample_steps = cpu_reference_rate(
            vh, cpu_lib, config, seconds_budget=12.0)
        line["cpu_baseline"] = {
            "value": rate, "unit": "images/s", "cores": 1, "kind": "reference",
            "sample": f"reference CPU train step (single-threaded on Linux), "
                      f"batch {sample_batch}, {sample_steps} steps"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        secondary = reference_cuda_rate(config, batch)
        if secondary:
            line["reference_cuda"] = secondary
    if rank == 0 and world == 1:
        line["augmentation"] = augmentation_measurement(
            backend, host_lib, batch, config[0], config[1], config[2],
            args.steps, with_cpu=not args.no_cpu_baseline)
    if rank == 0 and world == 1:
        line["dataset"] = dataset_measurement(
            vh, backend, batch, config[1], config[2], args.steps,
            with_cpu=not args.no_cpu_baseline)
    if not args.no_cfg5 and args.workload != "cfg5":
        # The data-parallel configuration at this GPU count: the same global
        # batch of 4096 whatever the count, micro-batches of 512.
        cfg5_config, cfg5_batch = WORKLOADS["cfg5"]
        torch.cuda.empty_cache()
        line["cfg5"] = measure(
            vh, backend, host_lib, "cfg5", cfg5_config, cfg5_batch,
            micro_batch_count("cfg5", cfg5_batch), args.cfg5_steps, 3, rank,
            local_rank, world, tf32_peak, args.strict_synchronize)
    backend.disable()
    backend.dp_shutdown()
    backend.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
