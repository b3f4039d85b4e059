#!/usr/bin/env python
"""Benchmark of the hot path: ResNet-50 v1.5 fp32-accurate inference (images/s) as a NeoML CDnn on the B200 math engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The timed call is NeoML's own `CDnn::RunOnce()` on the engine that NeoML's factory returns (`CreateGpuMathEngine` /
`IGpuMathEngineManager` of the hosted libNeoMathEngine.so: the B200 engine); NeoML itself is built unmodified.
N > 1 is launched by torch.distributed.run (one rank per GPU); inference is batch-sharded with no data-path
collective (weak scaling: every rank runs the full per-GPU batch).  Rank 0 prints ONE JSON line.

A step is one forward pass over one synthetic batch (256 x 224 x 224 x 3, uniform[0,1], seeded; He-normal weights with
the BatchNorm folded into the free terms).  `value` is timed with the batch already resident in HBM (the source
layer's blob), CUDA events on the engine's stream; `e2e` is the same through the calls a NeoML user makes with HOST
buffers: per step `CDnnBlob::CopyFrom(host)` of the batch from pinned memory, `RunOnce()`, `CopyTo(host)` of the
probabilities and arg-max indices.  `roofline` describes the dominant kernel (the tcgen05 contraction) from CUDA-event
timings of every contraction launch in three extra, instrumented steps.  `cpu_baseline` / `--impl reference` time the
same CDnn on the reference's own CPU math engine (oracle/_ref: NeoML and NeoMathEngine built unmodified), one engine
per host thread on slices of the same 256-image batch.

Other modes: --sweep (per-GPU batch 1/32/256/1024 on 1/2/4/8 engines of ONE process made by NeoML's
CreateDistributedCudaMathEngines, one host thread per engine; plain and double-buffered input loop), --transformer (configuration 4 as a CDnn), --ops and
--products (kernel-level figures at the configurations' sizes).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "resnet50_fp32_infer_images_per_s"
UNIT = "images/s"
IMAGE = (224, 224, 3)
WORKLOAD = "resnet50_v1.5_infer_b256_224x224x3"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    ap.add_argument("--precision", type=int, default=0, help="0 = 3xTF32 (default), 1 = TF32 opt-in")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-peak", action="store_true", help="skip the TF32 peak measurement (profiler captures)")
    ap.add_argument("--layers", action="store_true", help="print the per-contraction timing table to stderr")
    ap.add_argument("--settle-seconds", type=float, default=3.0,
                    help="upper bound of the untimed settling phase (20-step blocks until two agree within 2 %%); "
                         "0 for profiler captures")
    ap.add_argument("--ops", action="store_true",
                    help="instead of the network: time the bandwidth-bound kernels at the configs' sizes (one JSON line each)")
    ap.add_argument("--products", action="store_true",
                    help="time the dense contractions of the other configs (config 1 convolution, config 2 MobileNetV2 "
                         "block, config 4 FC and attention products, config 5 matrix products) against the tensor roofline")
    ap.add_argument("--sweep", action="store_true",
                    help="per-GPU batch 1/32/256/1024 on 1/2/4/8 engines of one process (CreateDistributedCudaMathEngines)")
    ap.add_argument("--only", default="", help="with --products: run only the cases whose name contains this text")
    ap.add_argument("--transformer", action="store_true", help="configuration 4 (12 encoder layers, 64 x 512 x 768) as a CDnn")
    ap.add_argument("--kernel-options", type=int, default=0,
                    help="diagnostic switches of the contraction launcher (16 gather kernel, 32 no split K, 64 no "
                         "programmatic dependent launch); for A/B timing only")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------- CPU legs
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference_arm(args):
    """The reference's own CPU path for the same step: the ResNet-50 CDnn on NeoML's CPU math engine (oracle/_ref:
    NeoML and NeoMathEngine compiled unmodified), one engine and one host thread per slice of the 256-image batch --
    NeoML's multi-core model (CDistributedInference).  Every step copies its slice from host memory into the source
    blob, runs, and copies probabilities and arg-max indices back."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from neoml_b200 import cdnn, resnet50
    ref_dir = ROOT / "oracle" / "_ref"
    if not (ref_dir / "libcdnn_host.so").exists():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref is not built (make -C oracle ref needs a NeoML checkout)"}))
        return
    cdnn.use_directory(ref_dir)
    cdnn.load()
    batch = args.batch
    threads = 1
    while threads * 2 <= host_cores() and batch % (threads * 2) == 0:
        threads *= 2
    per = batch // threads
    model = cdnn.Model.resnet50(resnet50.make_weights())
    x = np.random.default_rng(1234).uniform(0, 1, (batch, *IMAGE)).astype(np.float32)
    out_floats = per * (resnet50.CLASSES + 1)
    out = np.empty(threads * out_floats, np.float32)
    reps = cdnn.Replicas("cpu", model, count=threads)
    for i in range(threads):
        reps.net(i).set_input("in", x[i * per:(i + 1) * per])
    seconds = reps.time_steps(args.warmup, args.steps, "in", x.ctypes.data, x.size // threads, "probs,argmax",
                              out.ctypes.data, out_floats * 4)
    reps.close()
    ips = batch * args.steps / seconds
    sample = (f"ResNet-50 CDnn, {threads} CPU engines x {per} images = one {batch}-image step, {args.steps} timed steps "
              f"after {args.warmup} warm-up; sgemm = MLAS (no MKL on this host)")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(ips, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * seconds / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": WORKLOAD if batch == 256 else f"resnet50_v1.5_infer_b{batch}", "per_gpu_batch": batch,
                   "step": f"one {batch}-image batch: {threads} host threads x {per} images, host buffers in and out",
                   "engine": "reference CPU math engine (MLAS sgemm) under the reference's CDnn"},
        "cpu_baseline": {"value": round(ips, 3), "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": round(ips, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------- GPU arm
class ClockSampler:
    """nvidia-smi clocks and throttle reasons of this rank's GPU, sampled every 50 ms; started before the warm-up
    steps (the tool needs a few hundred ms to come up) and stopped after the timed regions."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # "under load" = the samples whose board power is within 40 % of the highest one seen
        load = [c for c, w in zip(sm, pw) if w >= 0.6 * max(pw)] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(load),
                "power_w_max": max(pw) if pw else None}


class HostedEngine:
    """A GPU engine from NeoML's factory plus the two things a benchmark needs beyond the NeoML interface: the CUDA
    stream the engine enqueues on (for events) and the kernel library's launch counter."""

    def __init__(self, device: int, precision: int):
        import torch
        from neoml_b200 import _capi, cdnn
        self.torch, self.cdnn = torch, cdnn
        self.kernels = _capi.load()
        cdnn.load()
        self.hosted = ctypes.CDLL(str(cdnn.directory() / "libNeoMathEngine.so"))
        self.hosted.nb200_engine_stream.restype = ctypes.c_void_p
        self.hosted.nb200_engine_stream.argtypes = [ctypes.c_void_p]
        # entry `device` of IGpuMathEngineManager; flags: the reference's TF32 opt-in bit
        self.engine = cdnn.Engine("manager", device=device, flags=2 if precision == 1 else 0)
        ptr = self.hosted.nb200_engine_stream(self.engine.ptr)
        if not ptr:
            raise SystemExit("the GPU engine NeoML's factory returned is not the B200 engine")
        self.stream = torch.cuda.ExternalStream(ptr, device=device)

    def record(self, event):
        # the call also makes the engine launch anything it still holds back for fusion
        self.hosted.nb200_engine_stream(self.engine.ptr)
        event.record(self.stream)

    def timed(self, fn) -> float:
        """Milliseconds of fn() on the engine's stream."""
        start, stop = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        self.record(start)
        fn()
        self.record(stop)
        stop.synchronize()
        return start.elapsed_time(stop)


def settle(engine: HostedEngine, step, budget_s: float):
    """Untimed 20-step blocks until two consecutive blocks agree within 2 % (clocks and power settle on a box that has
    been idle), bounded by budget_s.  Returns the block times in ms per step."""
    blocks = []
    t0 = time.perf_counter()
    while budget_s > 0 and time.perf_counter() - t0 < budget_s:
        blocks.append(engine.timed(lambda: [step() for _ in range(20)]) / 20)
        if len(blocks) >= 2 and abs(blocks[-1] - blocks[-2]) <= 0.02 * blocks[-1]:
            break
    return blocks


def measure_tf32_peak(torch, seconds: float = 2.0):
    """Dense TF32 tensor throughput of this GPU, measured the way MEASURED_PEAKS.json's bf16 figure was: a library
    8192^3 product (torch.matmul with TF32 allowed), best of 10 single calls (burst) and back to back for `seconds`
    (sustained).  Yardstick only: nothing of the product path runs here."""
    n = 8192
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        best = float("inf")
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(10):
            s.record()
            torch.matmul(a, b, out=c)
            e.record()
            e.synchronize()
            best = min(best, s.elapsed_time(e))
        reps = max(10, int(seconds * 1e3 / best))
        s.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e.record()
        e.synchronize()
        sustained_ms = s.elapsed_time(e) / reps
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return {"burst_tflops": round(flops / best / 1e9, 1), "sustained_tflops": round(flops / sustained_ms / 1e9, 1),
            "how": f"torch.matmul fp32 with TF32 allowed, {n}^3: best of 10 (burst), {reps} calls back to back (sustained)"}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from neoml_b200 import cdnn, resnet50, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    eng = HostedEngine(local, args.precision)
    lib = eng.kernels
    if lib.nb200_device_count() < 1:
        raise SystemExit("libneoml_b200.so sees no sm_100 device")
    if args.kernel_options:
        lib.nb200_debug_set_contraction_trace(None, 0, args.kernel_options)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    batch = args.batch
    model = cdnn.Model.resnet50(resnet50.make_weights())
    net = cdnn.Net(eng.engine, model)
    rng = np.random.default_rng(1234 + rank)
    host_x = torch.from_numpy(rng.uniform(0, 1, (batch, *IMAGE)).astype(np.float32)).pin_memory()
    dims = (1, batch, 1, IMAGE[0], IMAGE[1], 1, IMAGE[2])
    net.set_input_ptr("in", host_x.data_ptr(), dims)       # the source blob now holds the batch in HBM
    host_out = torch.empty(batch * (resnet50.CLASSES + 1), dtype=torch.float32).pin_memory()
    step = net.run

    # ---- device-resident timing -------------------------------------------------------------------------
    sampler = ClockSampler(local)
    sampler.start()
    step()
    settle_blocks = settle(eng, step, args.settle_seconds)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    launches0 = lib.nb200_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    eng.record(start)
    for _ in range(args.steps):
        step()
    eng.record(stop)
    barrier()
    launches = lib.nb200_launch_count() - launches0
    ms_total = start.elapsed_time(stop)

    # ---- end to end: what a NeoML user calls, host buffers in and out --------------------------------------------------
    def e2e(n):
        return net.time_steps(n, "probs,argmax", source="in", input_ptr=host_x.data_ptr(),
                              output_ptr=host_out.data_ptr(), output_bytes=host_out.numel() * 4, double_buffered=True)
    e2e(2)
    barrier()
    t0 = time.perf_counter()
    e2e(args.steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()

    # a step is as slow as its slowest rank
    ms_total, e2e_ms = sharding.max_over_ranks([ms_total, e2e_s * 1e3], device="cuda")

    status = lib.nb200_device_status(None, 0)
    if status != 0:
        raise SystemExit(f"a kernel reported a bounded-wait timeout (status {status:#x}); no number is reported")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (rank 0, three instrumented steps) --------------------------------------------
    # The library brackets every contraction launch with CUDA events on its stream (operand preparation, allocations and
    # host gaps stay outside) and notes the algorithmic flops of the call each launch belongs to.
    timed_steps = 3
    lib.nb200_debug_time_contractions(1)
    step()                                                  # creates the library's events; not counted
    torch.cuda.synchronize()
    lib.nb200_debug_time_contractions(1)                    # clears the list
    for _ in range(timed_steps):
        step()
    eng.record(stop)
    stop.synchronize()
    lib.nb200_debug_time_contractions(0)
    cap = 4096
    times, flop = (ctypes.c_float * cap)(), (ctypes.c_double * cap)()
    got = lib.nb200_debug_contraction_records(ctypes.cast(times, ctypes.c_void_p), ctypes.cast(flop, ctypes.c_void_p), cap)
    if got <= 0 or got % timed_steps:
        raise SystemExit(f"the library timed {got} contraction launches over {timed_steps} steps")
    tc_launches = got // timed_steps
    kernel_ms = [sum(times[i + s * tc_launches] for s in range(timed_steps)) / timed_steps for i in range(tc_launches)]
    layer_flops = [flop[i] for i in range(tc_launches)]
    flops = sum(layer_flops)
    expected = resnet50.flops_per_image() * batch
    if abs(flops - expected) > 1e-6 * expected:
        raise SystemExit(f"the timed launches account for {flops:.4e} flops, the network has {expected:.4e}")
    tc_ms = sum(kernel_ms)
    if args.layers:
        for i, (f, t) in enumerate(zip(layer_flops, kernel_ms)):
            print(f"launch {i:3d} {f / 1e9:9.2f} GFLOP {t:8.3f} ms {f / t / 1e9:8.1f} TFLOP/s", file=sys.stderr)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        pk = json.loads(peaks_path.read_text())
        peak_tf, peak_src = float(pk["bf16_tflops_sustained"]), "MEASURED_PEAKS.json bf16_tflops_sustained (of measured)"
    else:
        peak_tf, peak_src = 1390.7, "fallback: sustained cuBLAS bf16, an earlier measurement (of fallback)"
    achieved_tf = flops / (tc_ms * 1e-3) / 1e12
    mma_per_product = 3 if args.precision == 0 else 1
    tf32 = None if args.no_peak else measure_tf32_peak(torch)
    if tf32 is not None:
        eff_peak, eff_src = tf32["sustained_tflops"] / mma_per_product, "TF32 sustained, measured in this run"
    else:
        eff_peak, eff_src = peak_tf / 2 / mma_per_product, "bf16 sustained / 2 (not measured in this run)"
    act_bytes = resnet50.contraction_bytes_per_image() * batch + resnet50.weight_bytes()
    roofline = {
        "bound": "tensor", "kernel": "contraction_tc_kernel (tcgen05 kind::tf32, implicit-GEMM conv + FC)",
        "achieved": round(achieved_tf, 2), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(achieved_tf / peak_tf, 4),
        "peak_source": peak_src,
        "traffic": round(TRAFFIC_MB_PER_IMAGE * 1e6 * batch / max(tc_launches, 1) / 1e9, 4),
        "traffic_unit": "GB per launch (average)",
        "traffic_source": TRAFFIC_SOURCE,
        "algorithmic_bytes_per_launch_gb": round(act_bytes / max(tc_launches, 1) / 1e9, 4),
        "launches_per_step": tc_launches, "ms_per_step_in_kernel": round(tc_ms, 3),
        "algorithmic_gflop_per_step": round(flops / 1e9, 2),
        "tf32_peak_measured": tf32,
        "effective_peak_for_this_arithmetic": round(eff_peak, 1),
        "effective_peak_source": f"{eff_src}, / {mma_per_product} MMAs per product",
        "frac_of_effective_peak": round(achieved_tf / eff_peak, 4),
        "whole_step_frac_of_effective_peak": round(flops / (ms_total / args.steps * 1e-3) / 1e12 / eff_peak, 4),
        "note": "peak is dense bf16; this arithmetic is TF32 (3 MMAs per product in the default 3xTF32 mode), "
                "algorithmic flops counted once",
    }

    images = batch * world * args.steps
    ms_step = ms_total / args.steps
    line = {
        "metric": METRIC, "value": round(images / (ms_total * 1e-3), 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (3xTF32 split on tcgen05, fp32 accumulate)" if args.precision == 0 else "tf32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD if batch == 256 else f"resnet50_v1.5_infer_b{batch}",
                   "per_gpu_batch": batch, "global_batch": batch * world, "parallelism": f"batch-sharded x{world}",
                   "call": "NeoML CDnn::RunOnce on the engine from IGpuMathEngineManager::CreateMathEngine",
                   "fused_epilogues": "by the engine (conv -> add -> ReLU calls folded at run time)",
                   "settle_blocks_ms_per_step": [round(b, 3) for b in settle_blocks],
                   "l2": "inputs and activations larger than L2 (154 MB batch, 822 MB stem output)"},
        "clocks": dict(clocks, ms_times_mhz=round(ms_step * clocks["sm_mhz"], 1) if clocks.get("sm_mhz") else None),
        "e2e": {"value": round(images / (e2e_ms * 1e-3), 2), "unit": UNIT,
                "h2d_bytes_per_step": host_x.numel() * 4, "d2h_bytes_per_step": host_out.numel() * 4,
                "ms_per_step": round(e2e_ms / args.steps, 3),
                "loop": "per step: CDnnBlob::CopyFrom(pinned host batch) into the idle one of two source blobs, "
                        "CDnn::RunOnce, CopyTo(host) of probabilities and arg-max; the copy of step i+1 is issued "
                        "right after RunOnce of step i and overlaps its kernels"},
        "gpu_launches": int(launches),
        "roofline": roofline,
    }
    if world == 1 and not args.no_cpu_baseline:
        # in a process of its own: the reference's NeoMathEngine library and the hosted one carry the same soname
        try:
            r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "3", "--warmup", "1",
                                "--batch", str(batch)], capture_output=True, text=True, timeout=600)
            ref = json.loads(r.stdout.strip().splitlines()[-1])
            line["cpu_baseline"] = ref.get("cpu_baseline") or {"value": None, "unit": UNIT, "cores": 0, "kind": "reference",
                                                               "sample": ref.get("unavailable", "no line")}
        except Exception as exc:  # the baseline is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": f"failed: {exc}"}
    print(json.dumps(line), flush=True)
    net.close()
    if world > 1:
        dist.destroy_process_group()


# DRAM traffic of the contraction launches: dram__bytes_read.sum + dram__bytes_write.sum of the 54 launches of one
# batch-64 step in an ncu capture, per image; activations dominate, so it scales with the batch.  A constant from
# that capture, not a figure of this run.
TRAFFIC_MB_PER_IMAGE = 85.0
TRAFFIC_SOURCE = "constant: ncu capture of a batch-64 step (54 launches, 5.44 GB), scaled by the batch; not measured in this run"


def run_sweep(args):
    """Configuration 5's scaling sweep the way NeoML distributes a network: ONE process, the engines made by
    CreateDistributedCudaMathEngines, one host thread per engine, every engine a replica of the ResNet-50 CDnn on its
    own per-GPU batch (host buffers in and out every step).  One JSON line per (engines, batch)."""
    import torch
    from neoml_b200 import cdnn, resnet50
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --sweep needs CUDA devices: the product path has no CPU fallback")
    cdnn.load()
    visible = torch.cuda.device_count()
    model = cdnn.Model.resnet50(resnet50.make_weights())
    batches = [1, 32, 256, 1024]
    x = torch.rand(max(batches), *IMAGE).pin_memory()
    rows = []
    for n in [g for g in (1, 2, 4, 8) if g <= min(visible, args.gpus)]:
        reps = cdnn.Replicas("gpu", model, devices=list(range(n)))
        out = torch.empty(n * max(batches) * (resnet50.CLASSES + 1)).pin_memory()
        for b in batches:
            for i in range(n):
                reps.net(i).set_input_ptr("in", x.data_ptr(), (1, b, 1, IMAGE[0], IMAGE[1], 1, IMAGE[2]))
            steps = {1: 200, 32: 60, 256: args.steps, 1024: max(4, args.steps // 2)}[b]
            per_out = b * (resnet50.CLASSES + 1) * 4
            secs = reps.time_steps(max(args.warmup, 3), steps, "in", x.data_ptr(), 0, "probs,argmax", out.data_ptr(), per_out)
            secs2 = reps.time_steps(max(args.warmup, 3), steps, "in", x.data_ptr(), 0, "probs,argmax", out.data_ptr(), per_out,
                                    double_buffered=True)
            row = {"mode": "sweep", "engines": n, "per_gpu_batch": b, "steps": steps,
                   "images_per_s": round(n * b * steps / secs, 1), "ms_per_step": round(1e3 * secs / steps, 3),
                   "double_buffered_images_per_s": round(n * b * steps / secs2, 1),
                   "double_buffered_ms_per_step": round(1e3 * secs2 / steps, 3),
                   "call": "CreateDistributedCudaMathEngines, one host thread per engine, host buffers in and out; "
                           "double_buffered: the input copy of step i+1 is issued before the results of step i are read"}
            rows.append(row)
            print(json.dumps(row), flush=True)
        reps.close()
    base = {r["per_gpu_batch"]: r["images_per_s"] for r in rows if r["engines"] == 1}
    base2 = {r["per_gpu_batch"]: r["double_buffered_images_per_s"] for r in rows if r["engines"] == 1}
    print(json.dumps({"mode": "sweep_summary", "scaling_vs_one_engine": {
        f"b{r['per_gpu_batch']}_x{r['engines']}": round(r["images_per_s"] / base[r["per_gpu_batch"]], 3) for r in rows},
        "double_buffered_scaling_vs_one_engine": {
        f"b{r['per_gpu_batch']}_x{r['engines']}": round(r["double_buffered_images_per_s"] / base2[r["per_gpu_batch"]], 3)
        for r in rows}}))


def run_transformer(args):
    """Configuration 4 as a NeoML CDnn on the GPU engine: 12 x CTransformerEncoderLayer, 64 x 512 x 768, 12 heads,
    FFN 3072, GELU, mask input.  Algorithmic flops per layer: 4 FC products of 32768 x 768 x 768 (Q, K, V, output),
    the FFN pair 32768 x 768 x 3072 twice, and the two attention products 768 x (512 x 512 x 64)."""
    import numpy as np
    import torch
    from neoml_b200 import cdnn
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --transformer needs a CUDA device: the product path has no CPU fallback")
    eng = HostedEngine(0, args.precision)
    layers, b, s, hid, heads, ffn = 12, 64, 512, 768, 12, 3072
    model = cdnn.Model.transformer(layers, hid, heads, ffn, seed=7, sigma=0.02, mask=True)
    net = cdnn.Net(eng.engine, model)
    rng = np.random.default_rng(404)
    net.set_input("in", rng.standard_normal((b, s, hid)).astype(np.float32))
    net.set_input("mask", np.zeros((s, s), np.float32), (1, 1, 1, 1, s, 1, s))
    tokens = b * s
    flops = layers * (2.0 * tokens * hid * hid * 4 + 2.0 * tokens * hid * ffn * 2 + 2.0 * (b * heads) * s * s * (hid // heads) * 2)
    net.run()
    settle(eng, net.run, args.settle_seconds)
    lib = eng.kernels
    launches0 = lib.nb200_launch_count()
    ms = eng.timed(lambda: [net.run() for _ in range(args.steps)]) / args.steps
    launches = (lib.nb200_launch_count() - launches0) // args.steps
    tf32 = None if args.no_peak else measure_tf32_peak(torch)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak_tf = float(json.loads(peaks_path.read_text())["bf16_tflops_sustained"]) if peaks_path.exists() else 1390.7
    mma = 3 if args.precision == 0 else 1
    eff = (tf32["sustained_tflops"] if tf32 else peak_tf / 2) / mma
    tf = flops / ms / 1e9
    print(json.dumps({"mode": "transformer", "workload": "transformer_encoder_12x_b64_s512_h768 (CDnn::RunOnce)",
                      "ms_per_step": round(ms, 3), "sequences_per_s": round(b / ms * 1e3, 1), "launches_per_step": int(launches),
                      "algorithmic_gflop_per_step": round(flops / 1e9, 1),
                      "roofline": {"bound": "tensor (whole step, bandwidth-bound passes included)", "achieved": round(tf, 1),
                                   "peak": peak_tf, "unit": "TFLOP/s", "frac": round(tf / peak_tf, 4),
                                   "tf32_peak_measured": tf32, "effective_peak_for_this_arithmetic": round(eff, 1),
                                   "frac_of_effective_peak": round(tf / eff, 3)}}))
    net.close()


def run_ops(args):
    """The bandwidth-bound kernels of the path at the sizes the configs give them, against the measured HBM peak.
    Algorithmic bytes = unique input elements * 4 + output elements * 4 (in place counts read + write).  Every tensor
    is larger than L2 (126 MB) or the op is repeated over several buffers so that L2 does not serve the reads."""
    import torch
    from neoml_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --ops needs a CUDA device: the product path has no CPU fallback")
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else 6650.0
    peak_src = "MEASURED_PEAKS.json hbm_gbs (of measured)" if peaks_path.exists() else "fallback: 6.65 TB/s, an earlier measurement (of fallback)"
    dev = "cuda"
    n = args.batch            # images of config 3; --batch 128 halves every tensor (for profiler captures)
    tb = max(1, 64 * n // 256)  # sequences of config 4
    rnd = lambda *shape: torch.rand(*shape, device=dev)
    zero = torch.zeros(1, device=dev)
    cases = []
    # config 3 (ResNet-50, batch 256): activations of the stem and of stage 1
    a, b2 = rnd(n, 112, 112, 64), rnd(n, 112, 112, 64)              # 822 MB each at batch 256
    cases.append((f"VectorAdd {n}x112x112x64 (stem output size)", lambda: ops.VectorAdd(a, b2, result=a), 3 * a.numel() * 4))
    cases.append((f"VectorReLU {n}x112x112x64 in place", lambda: ops.VectorReLU(a, result=a, threshold=zero), 2 * a.numel() * 4))
    padded = torch.empty(n, 114, 114, 64, device=dev)
    cases.append((f"BlobResizeImage {n}x112x112x64 +1 each side", lambda: ops.BlobResizeImage(a, 1, 1, 1, 1, 0, 0.0, result=padded),
                  (a.numel() + padded.numel()) * 4))
    pooled = torch.empty(n, 56, 56, 64, device=dev)
    cases.append((f"BlobMaxPooling 3x3/2 on {n}x114x114x64", lambda: ops.BlobMaxPooling(padded, (3, 3), (2, 2), result=pooled),
                  (padded.numel() + pooled.numel()) * 4))
    feat = rnd(4 * n, 7, 7, 2048)                                    # 411 MB: global mean pool of a batch-1024 shard
    cases.append((f"SumMatrixRows {4 * n}x49x2048 (global pool)", lambda: ops.SumMatrixRows(4 * n, feat, 49, 2048), feat.numel() * 4))
    # config 2: depthwise 3x3 of the MobileNetV2 block
    dwx, dww, dwb = rnd(max(1, n // 4), 56, 56, 192), rnd(3, 3, 192), rnd(192)
    dwy = torch.empty_like(dwx)
    cases.append((f"BlobChannelwiseConvolution 3x3 {max(1, n // 4)}x56x56x192", lambda: ops.BlobChannelwiseConvolution(
        dwx, dww, dwb, result=dwy, padding=(1, 1), act=ops.ACT_RELU, act_param=6.0), 2 * dwx.numel() * 4))
    # config 4 (transformer, batch 64 x seq 512): scores, projections
    heads = 12 * tb
    scores = rnd(heads * 512, 512)                                  # 805 MB at batch 64 x 12 heads
    cases.append((f"MatrixSoftmaxByRows {heads * 512}x512 in place", lambda: ops.MatrixSoftmaxByRows(scores, heads * 512, 512, result=scores),
                  2 * scores.numel() * 4))
    mask = rnd(512 * 512)
    cases.append((f"AddVectorToMatrixRows {heads} x 262144 (mask)", lambda: ops.AddVectorToMatrixRows(1, scores, mask, heads, 512 * 512, result=scores),
                  2 * scores.numel() * 4))
    scale = torch.full((1,), 0.125, device=dev)
    cases.append((f"VectorMultiply {heads}x512x512 (score scale)", lambda: ops.vector_op("MULTIPLY", scores.view(-1), scalar=scale, result=scores.view(-1)),
                  2 * scores.numel() * 4))
    cases.append((f"scale + mask + MatrixSoftmaxByRows {heads * 512}x512 as one pass (engine fusion)",
                  lambda: ops.MatrixSoftmaxByRowsFused(scores, heads * 512, 512, scale=scale, row_bias=mask, bias_rows=512, result=scores),
                  2 * scores.numel() * 4 + mask.numel() * 4))
    q = rnd(tb * 512 * 12 * 64)                                      # 100 MB: four of them rotate to defeat L2
    qs = [rnd(tb * 512 * 12 * 64) for _ in range(4)]
    qt = torch.empty_like(q)
    rot = {"i": 0}

    def transpose():
        rot["i"] = (rot["i"] + 1) % 4
        return ops.TransposeMatrix(tb, qs[rot["i"]], 512, 1, 12, 64, result=qt)
    cases.append((f"TransposeMatrix [{tb},512,12,64] -> [{tb},12,512,64]", transpose, 2 * q.numel() * 4))
    side = 8192 * n // 256 if n >= 64 else 2048                       # 268 MB at the full size
    big, big_t = rnd(side, side), torch.empty(side, side, device=dev)
    cases.append((f"TransposeMatrix {side}x{side} (the transposing pass of MultiplyMatrixByMatrix)",
                  lambda: ops.TransposeMatrix(1, big, side, 1, side, 1, result=big_t), 2 * big.numel() * 4))
    vals = [rnd(12 * tb, 512, 64) for _ in range(4)]                  # 100 MB each: four rotate to defeat L2
    val_t = torch.empty(12 * tb, 64, 512, device=dev)

    def transpose_values():
        rot["i"] = (rot["i"] + 1) % 4
        return ops.TransposeMatrix(12 * tb, vals[rot["i"]], 512, 1, 64, 1, result=val_t)
    cases.append((f"TransposeMatrix {12 * tb} x [512,64] -> [64,512] (attention values)", transpose_values, 2 * val_t.numel() * 4))
    rows = tb * 512
    hid = rnd(rows, 3072)                                            # 403 MB
    cases.append((f"VectorSigmoid {rows}x3072 (GELU gate)", lambda: ops.vector_op("SIGMOID", hid.view(-1), result=hid.view(-1)), 2 * hid.numel() * 4))
    colsum = torch.empty(rows, device=dev)
    cases.append((f"SumMatrixColumns {rows}x3072 (layer norm)", lambda: ops.SumMatrixColumns(hid, rows, 3072, result=colsum), hid.numel() * 4))

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, fn, nbytes in cases:
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
        gbs = nbytes / ms / 1e6
        print(json.dumps({"op": name, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 1),
                          "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                       "frac": round(gbs / peak, 3), "peak_source": peak_src}}))


def run_products(args):
    """The dense contractions of configs 1, 2, 4 and 5 at full size: algorithmic flops (2*M*N*K, counted once) over the
    CUDA-event time of the public call (operand preparation and scratch allocation included), against the tensor peak
    of this arithmetic (measured sustained bf16 / 2 for TF32 / 3 MMAs per product for 3xTF32)."""
    import torch
    from neoml_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --products needs a CUDA device: the product path has no CPU fallback")
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["bf16_tflops_sustained"]) if peaks_path.exists() else 1390.7
    eff = peak / 2 / (3 if args.precision == 0 else 1)
    dev, prec = "cuda", args.precision
    rnd = lambda *shape: torch.rand(*shape, device=dev) - 0.5
    cases = []   # (name, algorithmic flops, setup): setup() allocates the operands and returns the call to time

    def cfg1():
        x1, f1, b1 = rnd(32, 56, 56, 64), rnd(64, 3, 3, 64), rnd(64)
        return lambda: ops.BlobConvolution(x1, f1, b1, padding=(1, 1), precision=prec)
    cases.append(("cfg1 BlobConvolution 32x56x56x64, 3x3 -> 64", 2.0 * 32 * 56 * 56 * 64 * 576, cfg1))

    def cfg2():
        x2, we, wd, wo = torch.rand(64, 56, 56, 32, device=dev), rnd(192, 32), rnd(3, 3, 192), rnd(32, 192) * 0.2
        be, bd, bo = rnd(192) * 0.2, rnd(192) * 0.2, rnd(32) * 0.2
        return lambda: ops.MobileNetV2Block(x2, we, be, wd, bd, wo, bo, stride=1, residual=True)
    cases.append(("cfg2 MobileNetV2Block 64x56x56x32 (expand 192)", 5.63e9, cfg2))

    # config 4: the FC products of an encoder layer (32768 tokens) and the per-head attention products
    for m, k, n in [(32768, 768, 768), (32768, 768, 3072), (32768, 3072, 768)]:
        def fc(m=m, k=k, n=n):
            a, b = rnd(m, k), rnd(n, k)
            return lambda: ops.MultiplyMatrixByTransposedMatrix(a, b, precision=prec)
        cases.append((f"cfg4 MultiplyMatrixByTransposedMatrix {m}x{k} * ({n}x{k})^T", 2.0 * m * k * n, fc))

    def qk():
        q, kk, sc = rnd(768, 512, 64), rnd(768, 512, 64), torch.empty(768, 512, 512, device=dev)
        return lambda: ops.BatchMultiplyMatrixByTransposedMatrix(q, kk, result=sc, precision=prec)
    cases.append(("cfg4 QK^T: batch 768, 512x64 * (512x64)^T", 2.0 * 768 * 512 * 512 * 64, qk))

    def pv():
        pr, v, ctx = torch.rand(768, 512, 512, device=dev), rnd(768, 512, 64), torch.empty(768, 512, 64, device=dev)
        return lambda: ops.MultiplyMatrixByMatrix(pr, v, result=ctx, precision=prec)
    cases.append(("cfg4 PV: batch 768, MultiplyMatrixByMatrix 512x512 * 512x64", 2.0 * 768 * 512 * 512 * 64, pv))

    if prec == 0:
        for masked in (False, True):
            def chain(masked=masked):
                q, kt4, v = rnd(768, 512, 64), rnd(768, 64, 512), rnd(768, 512, 64)
                scale4 = torch.full((1,), 0.125, device=dev)
                mask4 = torch.triu(torch.full((512, 512), -1e9, device=dev), diagonal=1) if masked else None
                return lambda: ops.AttentionScoresValues(q, kt4, v, scale=scale4, mask=mask4)
            cases.append(("cfg4 attention chain as one kernel: softmax(scale QK^T" + (" + mask" if masked else "")
                          + ") V, batch 768, 512 x 512 x 64", 4.0 * 768 * 512 * 512 * 64, chain))

    # config 5: square MultiplyMatrixByMatrix
    for size in (1024, 4096, 8192):
        def square(size=size):
            a, b, c = rnd(1, size, size), rnd(1, size, size), torch.empty(1, size, size, device=dev)
            return lambda: ops.MultiplyMatrixByMatrix(a, b, result=c, precision=prec)
        cases.append((f"cfg5 MultiplyMatrixByMatrix {size}^3", 2.0 * size ** 3, square))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, flops, setup in cases:
        if args.only and args.only not in name:
            continue
        fn = setup()
        for _ in range(max(args.warmup, 3) if not args.only else max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
        tf = flops / ms / 1e9
        print(json.dumps({"op": name, "ms": round(ms, 4), "algorithmic_gflop": round(flops / 1e9, 2),
                          "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s",
                                       "frac": round(tf / peak, 4), "effective_peak_for_this_arithmetic": round(eff, 1),
                                       "frac_of_effective_peak": round(tf / eff, 3)}}))
        del fn
        torch.cuda.empty_cache()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.sweep:
        run_sweep(args)
    elif args.transformer:
        run_transformer(args)
    elif args.products:
        run_products(args)
    elif args.ops:
        run_ops(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
