#!/usr/bin/env python
"""Benchmark of the hot path: ResNet-50 v1.5 fp32-accurate inference (images/s) through the B200 math-engine kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched by torch.distributed.run (one rank per GPU); inference is batch-sharded with no data-path
collective (weak scaling: every rank runs the full per-GPU batch).  Rank 0 prints ONE JSON line.

A step is one forward pass over one synthetic batch (256 x 224 x 224 x 3, uniform[0,1], seeded; He-normal weights with
the BatchNorm folded into the free terms).  `value` is timed with the batch already resident in HBM; `e2e` runs the
same call with the batch in pinned host memory, host->device copy and device->host read of the result inside the
timed region.  `roofline` describes the dominant kernel (the tcgen05 contraction) from CUDA-event timings of every
contraction launch in one extra, instrumented step.  `cpu_baseline` times the reference's own CPU math engine
(oracle/_ref) on a bounded sample of the same workload on this host's cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "resnet50_fp32_infer_images_per_s"
UNIT = "images/s"
IMAGE = (224, 224, 3)


SETTLE_STEPS = 12   # untimed steps ahead of the warm-up steps (see run_ours)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    ap.add_argument("--precision", type=int, default=0, help="0 = 3xTF32 (default), 1 = TF32 opt-in")
    ap.add_argument("--unfused", action="store_true", help="issue conv / add / ReLU as separate engine calls")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", action="store_true", help="print the per-contraction timing table to stderr")
    ap.add_argument("--graph", action="store_true",
                    help="capture the forward pass in a CUDA graph and replay it (small batches are launch-bound: "
                         "115 launches per pass)")
    ap.add_argument("--ops", action="store_true",
                    help="instead of the network: time the bandwidth-bound kernels at the configs' sizes (one JSON line each)")
    ap.add_argument("--settle", type=int, default=SETTLE_STEPS,
                    help="untimed steps ahead of the warm-up steps (clocks and power settle on a fresh box); 0 for profiler captures")
    ap.add_argument("--products", action="store_true",
                    help="time the dense contractions of the other configs (config 1 convolution, config 2 MobileNetV2 "
                         "block, config 4 FC and attention products, config 5 matrix products) against the tensor roofline")
    ap.add_argument("--kernel-options", type=int, default=0,
                    help="diagnostic switches of the contraction launcher (16 gather kernel, 32 no split K, 64 no "
                         "programmatic dependent launch); for A/B timing only")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU-baseline sample")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------- CPU legs
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_reference_run(per_thread_batch: int, rounds_budget_s: float, min_rounds: int, max_rounds: int, warm: int):
    """Times the reference CPU math engine (or, where it was not built, the plain-C oracle port) on ResNet-50:
    one engine per host thread, each thread a replica on its own slice of the batch -- the reference's own
    multi-core model (CDistributedInference).  Returns (images/s, ms per round, cores, kind, sample text)."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import numpy as np
    from neoml_b200 import resnet50
    import ref_backend
    from oracle_lib import Reference

    kind = "reference" if Reference.available() else "port"
    cores = host_cores() if kind == "reference" else 1
    weights = resnet50.make_weights()
    rng = np.random.default_rng(7)
    inputs = [rng.uniform(0, 1, (per_thread_batch, *IMAGE)).astype(np.float32) for _ in range(cores)]
    backends = [None] * cores
    barrier = threading.Barrier(cores + 1)
    stop = {"flag": False}

    def worker(i):
        backends[i] = ref_backend.RefBackend() if kind == "reference" else ref_backend.OracleBackend()
        while True:
            barrier.wait()
            if stop["flag"]:
                break
            resnet50.forward(backends[i], weights, inputs[i], fuse=False)
            barrier.wait()

    threads = [threading.Thread(target=worker, args=(i,), daemon=True) for i in range(cores)]
    for t in threads:
        t.start()
    times = []
    t_start = time.perf_counter()
    rounds = 0
    while True:
        barrier.wait()
        t0 = time.perf_counter()
        barrier.wait()
        dt = time.perf_counter() - t0
        rounds += 1
        if rounds > warm:
            times.append(dt)
        timed = len(times)
        if timed >= max_rounds or (timed >= min_rounds and time.perf_counter() - t_start > rounds_budget_s):
            break
    stop["flag"] = True
    barrier.wait()
    for t in threads:
        t.join()
    images = per_thread_batch * cores
    total = sum(times)
    ips = images * len(times) / total
    sample = (f"ResNet-50 forward, {cores} engine(s) x batch {per_thread_batch} per round, {len(times)} timed rounds "
              f"after {warm} warm-up; sgemm = MLAS (no MKL on this host)" if kind == "reference" else
              f"plain-C oracle port, 1 thread x batch {per_thread_batch}, {len(times)} rounds")
    return ips, 1e3 * total / len(times), cores, kind, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ips, ms, cores, kind, sample = cpu_reference_run(per_thread_batch=1, rounds_budget_s=0.0, min_rounds=args.steps,
                                                     max_rounds=args.steps, warm=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(ips, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "resnet50_v1.5_infer_b256_224x224x3", "per_gpu_batch": 256,
                   "step": f"bounded sample of the workload: {cores} host threads x 1 image per step",
                   "engine": "reference CPU math engine (MLAS sgemm)"},
        "cpu_baseline": {"value": round(ips, 3), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
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


class ContractionTimer:
    """CUDA events around every contraction launch of one instrumented step."""

    def __init__(self, torch):
        self.torch, self.records, self._start = torch, [], None

    def begin(self):
        self._start = self.torch.cuda.Event(enable_timing=True)
        self._start.record()

    def end(self, kind, flops):
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        self.records.append((kind, flops, self._start, e))

    def totals(self):
        self.torch.cuda.synchronize()
        ms = [(k, f, s.elapsed_time(e)) for k, f, s, e in self.records]
        return sum(f for _, f, _ in ms), sum(t for _, _, t in ms), len(ms), ms


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from neoml_b200 import _capi, resnet50, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _capi.load()
    if lib.nb200_device_count() < 1:
        raise SystemExit("libneoml_b200.so sees no sm_100 device")
    if args.kernel_options:
        lib.nb200_debug_set_contraction_trace(None, 0, args.kernel_options)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    batch = args.batch
    be = resnet50.EngineBackend(precision=args.precision)
    weights = be.upload(resnet50.make_weights())
    rng = np.random.default_rng(1234 + rank)
    host_x = torch.from_numpy(rng.uniform(0, 1, (batch, *IMAGE)).astype(np.float32)).pin_memory()
    dev_x = host_x.cuda()
    fuse = not args.unfused

    def eager_step(x):
        return resnet50.forward(be, weights, x, fuse=fuse)

    step = eager_step
    if args.graph:
        # The library allocates nothing and keeps no per-call host state, so a forward pass captures as it is: the
        # scratch and result tensors come from torch's capture-aware allocator, tensor maps travel as kernel arguments.
        for _ in range(3):
            eager_step(dev_x)       # one-time set-up (function attributes, driver entry points) happens outside capture
        torch.cuda.synchronize()
        graph_in = [dev_x, torch.empty_like(dev_x), torch.empty_like(dev_x)]   # the device loop and the two e2e buffers
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for buf in graph_in:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    out = eager_step(buf)
                graphs.append((g, out))
        torch.cuda.current_stream().wait_stream(side)

        def step(x):
            for buf, (g, out) in zip(graph_in, graphs):
                if buf.data_ptr() == x.data_ptr():
                    g.replay()
                    return out
            raise RuntimeError("graph replay needs one of the captured input buffers")

    # ---- device-resident timing -------------------------------------------------------------------------
    sampler = ClockSampler(local)
    sampler.start()
    # A fresh box needs a moment under load before clocks and power settle (a first timed loop right after three
    # warm-up steps has measured 15 % slow): a fixed number of extra untimed steps precedes the W warm-up steps.
    for _ in range(max(args.settle, 0)):
        step(dev_x)
    for _ in range(max(args.warmup, 3)):
        step(dev_x)
    barrier()
    launches0 = lib.nb200_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        probs, idx = step(dev_x)
    stop.record()
    barrier()
    launches = lib.nb200_launch_count() - launches0
    if args.graph:
        # a replayed graph launches the captured kernels without passing through the library's counter
        before = lib.nb200_launch_count()
        eager_step(dev_x)
        torch.cuda.synchronize()
        launches = (lib.nb200_launch_count() - before) * args.steps
    ms_total = start.elapsed_time(stop)

    # ---- end to end: pinned host batch -> device -> forward -> result back, double-buffered ---------------------------
    copy_stream = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    bufs = graph_in[1:] if args.graph else [torch.empty_like(dev_x) for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    host_idx = torch.empty(batch, dtype=torch.int32).pin_memory()
    host_probs = torch.empty((batch, resnet50.CLASSES), dtype=torch.float32).pin_memory()

    def e2e_loop(n):
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[b])  # the forward two steps ago has finished reading this buffer
                bufs[b].copy_(host_x, non_blocking=True)
                copied[b].record(copy_stream)
            main.wait_event(copied[b])
            p, ix = step(bufs[b])
            consumed[b].record(main)
            host_idx.copy_(ix, non_blocking=True)
            host_probs.copy_(p, non_blocking=True)
        torch.cuda.synchronize()

    for b in range(2):
        consumed[b].record(main)
    e2e_loop(2)
    barrier()
    t0 = time.perf_counter()
    e2e_loop(args.steps)
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

    # ---- roofline of the dominant kernel (rank 0, one instrumented step) -----------------------------------------------
    # The library brackets every contraction launch with CUDA events on its stream (operand preparation, allocations and
    # host gaps stay outside); the Python timer supplies the flops of each launch, in the same order.
    timer = ContractionTimer(torch)
    be_t = resnet50.EngineBackend(precision=args.precision, timer=timer)
    timed_steps = 3
    lib.nb200_debug_time_contractions(1)
    resnet50.forward(be_t, weights, dev_x, fuse=fuse)     # creates the library's events; not counted
    torch.cuda.synchronize()
    timer.records.clear()
    lib.nb200_debug_time_contractions(1)                   # clears the list
    for _ in range(timed_steps):
        resnet50.forward(be_t, weights, dev_x, fuse=fuse)
    torch.cuda.synchronize()
    lib.nb200_debug_time_contractions(0)
    flops, _, tc_launches, per_layer = timer.totals()
    times = (ctypes.c_float * tc_launches)()
    got = lib.nb200_debug_contraction_times(ctypes.cast(times, ctypes.c_void_p), tc_launches)
    if got != tc_launches:
        raise SystemExit(f"the library timed {got} contraction launches, the graph issued {tc_launches}")
    flops /= timed_steps
    tc_launches //= timed_steps
    kernel_ms = [sum(times[i + s * tc_launches] for s in range(timed_steps)) / timed_steps for i in range(tc_launches)]
    per_layer = [(k, f, kernel_ms[i]) for i, (k, f, _) in enumerate(per_layer[:tc_launches])]
    tc_ms = sum(kernel_ms)
    if args.layers:
        names = [sp.name for sp in resnet50.conv_specs()]
        order = ["stem"]
        for si, (_, _, blocks, _) in enumerate(resnet50.STAGES):
            for bi in range(blocks):
                p = f"s{si + 1}b{bi + 1}"
                order += ([p + "_down"] if bi == 0 else []) + [p + "_c1", p + "_c2", p + "_c3"]
        order.append("fc")
        assert len(order) == len(per_layer) and set(order) == set(names) | {"fc"}
        for name, (_, f, t) in zip(order, per_layer):
            print(f"{name:10s} {f / 1e9:9.2f} GFLOP {t:8.3f} ms {f / t / 1e9:8.1f} TFLOP/s", file=sys.stderr)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        pk = json.loads(peaks_path.read_text())
        peak_tf, peak_src = float(pk["bf16_tflops_sustained"]), "MEASURED_PEAKS.json bf16_tflops_sustained"
    else:
        peak_tf, peak_src = 1390.7, "fallback (MEASURED_PEAKS.json absent): sustained cuBLAS bf16 measured on this pool"
    achieved_tf = flops / (tc_ms * 1e-3) / 1e12
    mma_per_product = 3 if args.precision == 0 else 1
    eff_peak = peak_tf / 2 / mma_per_product  # TF32 runs at half the bf16 rate; 3xTF32 issues three MMAs per product
    roofline = {
        "bound": "tensor", "kernel": "contraction_tc_kernel (tcgen05 kind::tf32, implicit-GEMM conv + FC)",
        "achieved": round(achieved_tf, 2), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(achieved_tf / peak_tf, 4),
        "peak_source": peak_src,
        # ncu dram__bytes_read.sum + dram__bytes_write.sum of the 54 contraction launches of one batch-64 step is 5.44 GB
        # = 85.0 MB per image (profiles/resnet50_b256_launch_list.md); activations dominate, so it scales with the batch
        "traffic": round(85.0e6 * batch / max(tc_launches, 1) / 1e9, 4), "traffic_unit": "GB per launch (average)",
        "algorithmic_bytes_per_launch_gb": round(28.05 * batch / 256 / max(tc_launches, 1), 4),
        "launches_per_step": tc_launches, "ms_per_step_in_kernel": round(tc_ms, 3),
        "algorithmic_gflop_per_step": round(flops / 1e9, 2),
        "effective_peak_for_this_arithmetic": round(eff_peak, 1),
        "frac_of_effective_peak": round(achieved_tf / eff_peak, 4),
        "frac_ceiling_for_this_arithmetic": round(eff_peak / peak_tf, 4),
        "note": "peak is dense bf16; TF32 = 1/2 of it, 3xTF32 = 1/6 (algorithmic flops counted once)",
    }

    images = batch * world * args.steps
    line = {
        "metric": METRIC, "value": round(images / (ms_total * 1e-3), 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_total / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (3xTF32 split on tcgen05, fp32 accumulate)" if args.precision == 0 else "tf32",
        "data": "synthetic",
        "config": {"workload": "resnet50_v1.5_infer_b256_224x224x3" if batch == 256 else f"resnet50_v1.5_infer_b{batch}",
                   "per_gpu_batch": batch, "global_batch": batch * world, "parallelism": f"batch-sharded x{world}",
                   "fused_epilogues": fuse, "cuda_graph": bool(args.graph), "settle_steps_before_warmup": max(args.settle, 0), "l2": "inputs and activations larger than L2 (154 MB batch, 822 MB stem output)"},
        "clocks": clocks,
        "e2e": {"value": round(images / (e2e_ms * 1e-3), 2), "unit": UNIT,
                "h2d_bytes_per_step": host_x.numel() * 4, "d2h_bytes_per_step": host_idx.numel() * 4 + host_probs.numel() * 4,
                "ms_per_step": round(e2e_ms / args.steps, 3)},
        "gpu_launches": int(launches),
        "roofline": roofline,
    }
    if world == 1 and not args.no_cpu_baseline:
        try:
            ips, ms, cores, kind, sample = cpu_reference_run(per_thread_batch=1, rounds_budget_s=args.cpu_seconds,
                                                             min_rounds=2, max_rounds=50, warm=1)
            line["cpu_baseline"] = {"value": round(ips, 3), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}
        except Exception as exc:  # the baseline is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    peak_src = "MEASURED_PEAKS.json hbm_gbs" if peaks_path.exists() else "fallback: 6.65 TB/s measured on this pool earlier"
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
    cases = []
    # config 1: one 3x3 convolution, 32x56x56x64 -> 64
    x1, f1, b1 = rnd(32, 56, 56, 64), rnd(64, 3, 3, 64), rnd(64)
    cases.append(("cfg1 BlobConvolution 32x56x56x64, 3x3 -> 64", 2.0 * 32 * 56 * 56 * 64 * 576,
                  lambda: ops.BlobConvolution(x1, f1, b1, padding=(1, 1), precision=prec)))
    # config 2: MobileNetV2 block 64x56x56x32, expand 192, ReLU6 twice, residual
    x2, we, wd, wo = torch.rand(64, 56, 56, 32, device=dev), rnd(192, 32), rnd(3, 3, 192), rnd(32, 192) * 0.2
    be, bd, bo = rnd(192) * 0.2, rnd(192) * 0.2, rnd(32) * 0.2
    cases.append(("cfg2 MobileNetV2Block 64x56x56x32 (expand 192)", 5.63e9,
                  lambda: ops.MobileNetV2Block(x2, we, be, wd, bd, wo, bo, stride=1, residual=True)))
    # config 4: the FC products of an encoder layer (32768 tokens) and the per-head attention products
    for m, k, n in [(32768, 768, 768), (32768, 768, 3072), (32768, 3072, 768)]:
        a, b = rnd(m, k), rnd(n, k)
        cases.append((f"cfg4 MultiplyMatrixByTransposedMatrix {m}x{k} * ({n}x{k})^T", 2.0 * m * k * n,
                      lambda a=a, b=b: ops.MultiplyMatrixByTransposedMatrix(a, b, precision=prec)))
    q, kk, sc = rnd(768, 512, 64), rnd(768, 512, 64), torch.empty(768, 512, 512, device=dev)
    cases.append(("cfg4 QK^T: batch 768, 512x64 * (512x64)^T", 2.0 * 768 * 512 * 512 * 64,
                  lambda: ops.BatchMultiplyMatrixByTransposedMatrix(q, kk, result=sc, precision=prec)))
    pr, v, ctx = torch.rand(768, 512, 512, device=dev), rnd(768, 512, 64), torch.empty(768, 512, 64, device=dev)
    cases.append(("cfg4 PV: batch 768, MultiplyMatrixByMatrix 512x512 * 512x64", 2.0 * 768 * 512 * 512 * 64,
                  lambda: ops.MultiplyMatrixByMatrix(pr, v, result=ctx, precision=prec)))
    # config 5: square MultiplyMatrixByMatrix
    for size in (1024, 4096, 8192):
        a, b, c = rnd(1, size, size), rnd(1, size, size), torch.empty(1, size, size, device=dev)
        cases.append((f"cfg5 MultiplyMatrixByMatrix {size}^3", 2.0 * size ** 3,
                      lambda a=a, b=b, c=c: ops.MultiplyMatrixByMatrix(a, b, result=c, precision=prec)))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, flops, fn in cases:
        for _ in range(max(args.warmup, 3)):
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


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.products:
        run_products(args)
    elif args.ops:
        run_ops(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
