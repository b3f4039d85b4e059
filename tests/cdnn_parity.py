"""TEST INFRASTRUCTURE.  Runs one benchmark configuration as a NeoML CDnn twice -- on NeoML's own CPU math engine and
on the GPU engine the NeoMathEngine factory returns (CreateGpuMathEngine: the B200 engine in the hosted libraries) --
with the same model archive and the same seeded inputs, and prints one JSON line with the differences.

    python tests/cdnn_parity.py --config 3 [--scale full|small] [--cpu-threads 16] [--flags 0]

It runs in a process of its own (the hosted libNeoMathEngine.so and the oracle's carry the same soname).  The CPU side
uses one CPU engine per host thread on slices of the batch (what NeoML's CDistributedInference does,
NeoML/src/Dnn/DnnDistributed.cpp:551-607); the GPU side runs the whole batch on one engine.

Error figures: gate = max|g - w| / max(|w|, RMS(w)) (norm-wise); strict = the same with the floor 1e-3 * RMS(w).
Index outputs are compared bit for bit.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from neoml_b200 import cdnn, resnet50  # noqa: E402


def rel_err(got, want, floor):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    tau = floor * float(np.sqrt(np.mean(want * want))) + 1e-30
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), tau)))


def rng_for(seed):
    return np.random.Generator(np.random.Philox(seed))


def run_cpu_sliced(model, inputs: dict, sinks: list[str], threads: int, batch_axis_dims: dict):
    """inputs: name -> (array, dims7 or None, sliced?)   Slices along the array's first axis."""
    batch = next(a.shape[0] for a, _, sliced in inputs.values() if sliced)
    threads = max(1, min(threads, batch))
    while batch % threads:
        threads -= 1
    per = batch // threads
    reps = cdnn.Replicas("cpu", model, count=threads)
    try:
        sliced_name = None
        for i in range(threads):
            net = reps.net(i)
            for name, (a, dims, sliced) in inputs.items():
                if sliced:
                    sliced_name = name
                    part = a[i * per:(i + 1) * per]
                    d = None if dims is None else batch_axis_dims[name](per)
                    net.set_input(name, part, d)
                else:
                    net.set_input(name, a, dims)
        t0 = time.time()
        # one RunOnce per replica, all threads in parallel; outputs fetched afterwards
        src = inputs[sliced_name][0]
        flat = np.ascontiguousarray(src, np.float32)
        secs = reps.time_steps(0, 1, sliced_name, flat.ctypes.data, flat.size // threads, sinks[0], 0, 0)
        outs = {s: np.concatenate([reps.net(i).output(s).reshape(per, -1) for i in range(threads)]) for s in sinks}
        return outs, secs, threads, time.time() - t0
    finally:
        reps.close()


def run_gpu(model, inputs: dict, sinks: list[str], flags: int):
    eng = cdnn.Engine("gpu", flags=flags)
    try:
        net = cdnn.Net(eng, model)
        for name, (a, dims, _) in inputs.items():
            net.set_input(name, a, dims)
        net.run()
        first = {s: net.output(s) for s in sinks}
        t0 = time.time()
        net.run()
        outs = {s: net.output(s) for s in sinks}
        secs = time.time() - t0
        for s in sinks:  # the engine is deterministic: a second pass gives the same bits
            assert np.array_equal(first[s], outs[s]), f"{s}: two passes differ"
        batch = next(a.shape[0] for a, _, sliced in inputs.values() if sliced)
        outs = {s: o.reshape(batch, -1) for s, o in outs.items()}
        info = eng.info()
        net.close()
        return outs, secs, info
    finally:
        eng.close()


def config(n: str, scale: str):
    full = scale == "full"
    if n == "1":
        b, h, w, c, k = (32, 56, 56, 64, 64) if full else (3, 14, 14, 64, 64)
        r = rng_for(101)
        x = r.uniform(-1, 1, (b, h, w, c)).astype(np.float32)
        f = r.uniform(-1, 1, (k, 3, 3, c)).astype(np.float32)
        bias = r.uniform(-1, 1, k).astype(np.float32)
        return dict(name=f"config1 BlobConvolution {b}x{h}x{w}x{c} -> {k}, 3x3/1 pad 1",
                    model=cdnn.Model.conv(f, bias, padding=(1, 1)), inputs={"in": (x, None, True)}, sinks=["out"])
    if n == "2":
        b, h, w, c, e = (64, 56, 56, 32, 192) if full else (2, 14, 14, 32, 192)
        r = rng_for(202)
        x = r.uniform(0, 1, (b, h, w, c)).astype(np.float32)
        he = lambda shape, fan: (r.standard_normal(shape) * np.sqrt(2.0 / fan)).astype(np.float32)
        small = lambda m: r.uniform(-0.1, 0.1, m).astype(np.float32)
        return dict(name=f"config2 MobileNetV2Block {b}x{h}x{w}x{c}, expand {e}, ReLU6, residual",
                    model=cdnn.Model.mbv2(he((e, c), c), small(e), he((3, 3, e), 9), small(e), he((c, e), e), small(c)),
                    inputs={"in": (x, None, True)}, sinks=["out"])
    if n == "3":
        b, hw = (256, 224) if full else (4, 96)
        x = rng_for(303).uniform(0, 1, (b, hw, hw, 3)).astype(np.float32)
        return dict(name=f"config3 ResNet-50 v1.5 CDnn, batch {b} x {hw}x{hw}x3",
                    model=cdnn.Model.resnet50(resnet50.make_weights()), inputs={"in": (x, None, True)},
                    sinks=["probs", "argmax"])
    if n.startswith("4"):
        layers, b, s, hid, heads, ffn = (12, 64, 512, 768, 12, 3072) if full else (2, 4, 64, 128, 4, 256)
        x = rng_for(404).standard_normal((b, s, hid)).astype(np.float32)
        kind = {"4": "zeros", "4ones": "ones", "4causal": "causal"}[n]
        mask = {"zeros": np.zeros((s, s), np.float32), "ones": np.ones((s, s), np.float32),
                "causal": np.triu(np.ones((s, s), np.float32), 1)}[kind]
        return dict(name=f"config4 {layers} x CTransformerEncoderLayer, {b} x {s} x {hid}, {heads} heads, FFN {ffn}, "
                         f"mask {kind} (1 = ignored)",
                    model=cdnn.Model.transformer(layers, hid, heads, ffn, seed=7, sigma=0.02, mask=True),
                    inputs={"in": (x, None, True), "mask": (mask, (1, 1, 1, 1, s, 1, s), False)}, sinks=["out"])
    if n.startswith("5"):
        m = {"5a": 1024, "5b": 4096, "5c": 8192}[n] if full else {"5a": 96, "5b": 160, "5c": 256}[n]
        r = rng_for(505)
        a = r.uniform(-1, 1, (1, m, m)).astype(np.float32)
        bm = r.uniform(-1, 1, (1, m, m)).astype(np.float32)
        d = (1, 1, 1, m, 1, 1, m)
        return dict(name=f"config5 MultiplyMatrixByMatrix {m}^3 (CMatrixMultiplicationLayer)", model=cdnn.Model.matmul(),
                    inputs={"a": (a, d, True), "b": (bm, d, False)}, sinks=["out"], slice_dims={"a": lambda per: d},
                    unsliced=True)
    raise SystemExit(f"unknown config {n}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--scale", default="full", choices=["full", "small"])
    ap.add_argument("--cpu-threads", type=int, default=16)
    ap.add_argument("--flags", type=int, default=0, help="GPU engine flags (2 = the reference's TF32 opt-in)")
    ap.add_argument("--cpu-only", action="store_true", help="run the CPU side only (no GPU in this machine)")
    args = ap.parse_args()
    cdnn.load()
    cfg = config(args.config, args.scale)
    threads = 1 if cfg.get("unsliced") else args.cpu_threads
    want, cpu_secs, used, _ = run_cpu_sliced(cfg["model"], cfg["inputs"], cfg["sinks"], threads,
                                             cfg.get("slice_dims", {}))
    row = {"config": args.config, "scale": args.scale, "what": cfg["name"], "cpu_threads": used,
           "cpu_seconds": round(cpu_secs, 3)}
    if not args.cpu_only:
        got, gpu_secs, info = run_gpu(cfg["model"], cfg["inputs"], cfg["sinks"], args.flags)
        row["gpu_engine"] = info["name"]
        row["gpu_seconds_second_pass"] = round(gpu_secs, 4)
        for s in cfg["sinks"]:
            if want[s].dtype == np.int32:
                row[s + "_mismatches"] = int((want[s] != got[s]).sum())
                row[s + "_count"] = int(want[s].size)
            else:
                row[s + "_gate"] = rel_err(got[s], want[s], 1.0)
                row[s + "_strict"] = rel_err(got[s], want[s], 1e-3)
                row[s + "_finite"] = bool(np.isfinite(got[s]).all())
        if "probs" in want:
            top2 = np.sort(want["probs"], axis=1)[:, -2:]
            row["cpu_top2_margin_min_rel"] = float(((top2[:, 1] - top2[:, 0]) / top2[:, 1]).min())
    cfg["model"].close()
    print(json.dumps(row))


if __name__ == "__main__":
    main()
