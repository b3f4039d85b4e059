"""TEST INFRASTRUCTURE.  Runs one benchmark configuration as a NeoML CDnn twice -- on NeoML's own CPU math engine and
on the GPU engine the NeoMathEngine factory returns (CreateGpuMathEngine: the B200 engine in the hosted libraries) --
with the same model archive and the same seeded inputs, and prints one JSON line with the differences.

    python tests/cdnn_parity.py --config 3 [--scale full|small] [--cpu-threads 16] [--flags 0]

It runs in a process of its own (the hosted libNeoMathEngine.so and the oracle's carry the same soname).  The CPU side
uses one CPU engine per host thread on slices of the batch (what NeoML's CDistributedInference does,
NeoML/src/Dnn/DnnDistributed.cpp:551-607); the GPU side runs the whole batch on one engine.

Error figures: gate = max|g - w| / max(|w|, RMS(w)) (norm-wise); strict = the same with the floor 1e-3 * RMS(w).
Index outputs are compared bit for bit.  With --exact the same two figures are also given for each engine against an
evaluation in double precision (torch on the CPU, float64; configurations 1, 2, 3 -- its first 16 images -- and 5):
the distance of the reference's own CPU engine from the exact result is the yardstick for the other one.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import numpy as np

# torch (used by --exact) has to come first: importing it after NeoML's math-engine library has been loaded crashes
# inside torch's own start-up
try:
    import torch  # noqa: F401
except ImportError:
    pass

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


def exact_conv(x, f, bias, pad):
    import torch
    import torch.nn.functional as F
    y = F.conv2d(torch.from_numpy(x).double().permute(0, 3, 1, 2), torch.from_numpy(f).double().permute(0, 3, 1, 2),
                 torch.from_numpy(bias).double(), padding=pad)
    return y.permute(0, 2, 3, 1).numpy()


def exact_mbv2(x, we, be, wd, bd, wp, bp):
    import torch
    import torch.nn.functional as F
    t = torch.from_numpy(x).double()
    e = torch.clamp(t @ torch.from_numpy(we).double().T + torch.from_numpy(be).double(), 0, 6)
    c = we.shape[0]
    d = F.conv2d(e.permute(0, 3, 1, 2), torch.from_numpy(wd).double().permute(2, 0, 1).unsqueeze(1),
                 torch.from_numpy(bd).double(), padding=1, groups=c).permute(0, 2, 3, 1)
    d = torch.clamp(d, 0, 6)
    return (d @ torch.from_numpy(wp).double().T + torch.from_numpy(bp).double() + t).numpy()


def exact_resnet50(weights, x):
    """Probabilities in double precision, the same graph as neoml_b200.resnet50.forward."""
    import torch
    import torch.nn.functional as F
    w = {k: torch.from_numpy(v).double() for k, v in weights.items()}

    def conv(name, t, stride, pad, relu, residual=None):
        y = F.conv2d(t, w[name + ".w"].permute(0, 3, 1, 2), w[name + ".b"], stride=stride, padding=pad)
        if residual is not None:
            y = y + residual
        return torch.relu(y) if relu else y
    t = conv("stem", torch.from_numpy(x).double().permute(0, 3, 1, 2), 2, 3, True)
    t = F.max_pool2d(t, 3, 2, 1)
    for si, (mid, out, blocks, stride) in enumerate(resnet50.STAGES):
        for bi in range(blocks):
            s = stride if bi == 0 else 1
            p = f"s{si + 1}b{bi + 1}"
            shortcut = conv(p + "_down", t, s, 0, False) if bi == 0 else t
            u = conv(p + "_c1", t, 1, 0, True)
            u = conv(p + "_c2", u, s, 1, True)
            t = conv(p + "_c3", u, 1, 0, True, residual=shortcut)
    logits = t.mean(dim=(2, 3)) @ w["fc.w"].T + w["fc.b"]
    return torch.softmax(logits, dim=1).numpy()


def config(n: str, scale: str):
    full = scale == "full"
    if n == "1":
        b, h, w, c, k = (32, 56, 56, 64, 64) if full else (3, 14, 14, 64, 64)
        r = rng_for(101)
        x = r.uniform(-1, 1, (b, h, w, c)).astype(np.float32)
        f = r.uniform(-1, 1, (k, 3, 3, c)).astype(np.float32)
        bias = r.uniform(-1, 1, k).astype(np.float32)
        return dict(name=f"config1 BlobConvolution {b}x{h}x{w}x{c} -> {k}, 3x3/1 pad 1",
                    model=cdnn.Model.conv(f, bias, padding=(1, 1)), inputs={"in": (x, None, True)}, sinks=["out"],
                    exact=lambda: {"out": exact_conv(x, f, bias, 1).reshape(b, -1)})
    if n == "2":
        b, h, w, c, e = (64, 56, 56, 32, 192) if full else (2, 14, 14, 32, 192)
        r = rng_for(202)
        x = r.uniform(0, 1, (b, h, w, c)).astype(np.float32)
        he = lambda shape, fan: (r.standard_normal(shape) * np.sqrt(2.0 / fan)).astype(np.float32)
        small = lambda m: r.uniform(-0.1, 0.1, m).astype(np.float32)
        we, be, wd, bd, wp, bp = he((e, c), c), small(e), he((3, 3, e), 9), small(e), he((c, e), e), small(c)
        return dict(name=f"config2 MobileNetV2Block {b}x{h}x{w}x{c}, expand {e}, ReLU6, residual",
                    model=cdnn.Model.mbv2(we, be, wd, bd, wp, bp),
                    inputs={"in": (x, None, True)}, sinks=["out"],
                    exact=lambda: {"out": exact_mbv2(x, we, be, wd, bd, wp, bp).reshape(b, -1)})
    if n == "3":
        b, hw = (256, 224) if full else (4, 96)
        x = rng_for(303).uniform(0, 1, (b, hw, hw, 3)).astype(np.float32)
        weights = resnet50.make_weights()
        rows = min(b, 16)
        return dict(name=f"config3 ResNet-50 v1.5 CDnn, batch {b} x {hw}x{hw}x3",
                    model=cdnn.Model.resnet50(weights), inputs={"in": (x, None, True)},
                    sinks=["probs", "argmax"], exact=lambda: {"probs": exact_resnet50(weights, x[:rows])}, exact_rows=rows)
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
                    unsliced=True, exact=lambda: {"out": (a[0].astype(np.float64) @ bm[0].astype(np.float64)).reshape(1, -1)})
    raise SystemExit(f"unknown config {n}")


def run_all(args) -> None:
    import subprocess
    rows = []
    for c in ["1", "2", "3", "4", "4ones", "4causal", "5a", "5b", "5c"]:
        cmd = [sys.executable, __file__, "--config", c, "--scale", args.scale, "--cpu-threads", str(args.cpu_threads),
               "--flags", str(args.flags)] + (["--exact"] if args.exact else []) + (["--cpu-only"] if args.cpu_only else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise SystemExit(f"config {c} failed:\n{r.stdout[-1000:]}\n{r.stderr[-3000:]}")
        rows.append(json.loads(r.stdout.strip().splitlines()[-1]))
        print(json.dumps(rows[-1]), file=sys.stderr)
    fmt = lambda v: "-" if v is None else (f"{v:.2e}" if isinstance(v, float) else str(v))
    print("| config | what | gate (GPU vs CPU engine) | strict | CPU engine vs double: gate / strict | GPU engine vs double: gate / strict | index outputs |")
    print("|---|---|---|---|---|---|---|")
    for r in rows:
        sink = "probs" if any("probs" in k for k in r) else "out"
        idx = f"{r['argmax_count'] - r['argmax_mismatches']} / {r['argmax_count']} equal" if "argmax_count" in r else "-"
        print(f"| {r['config']} | {r['what']} | {fmt(r.get(sink + '_gate'))} | {fmt(r.get(sink + '_strict'))} | "
              f"{fmt(r.get('cpu_vs_exact_' + sink + '_gate'))} / {fmt(r.get('cpu_vs_exact_' + sink + '_strict'))} | "
              f"{fmt(r.get('gpu_vs_exact_' + sink + '_gate'))} / {fmt(r.get('gpu_vs_exact_' + sink + '_strict'))} | {idx} |")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, help="1, 2, 3, 4, 4ones, 4causal, 5a, 5b, 5c -- or 'all': every "
                    "configuration in a process of its own, the rows as a markdown table on stdout")
    ap.add_argument("--scale", default="full", choices=["full", "small"])
    ap.add_argument("--cpu-threads", type=int, default=16)
    ap.add_argument("--flags", type=int, default=0, help="GPU engine flags (2 = the reference's TF32 opt-in)")
    ap.add_argument("--cpu-only", action="store_true", help="run the CPU side only (no GPU in this machine)")
    ap.add_argument("--exact", action="store_true", help="also compare both engines with a double-precision evaluation")
    args = ap.parse_args()
    if args.config == "all":
        return run_all(args)
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
    if args.exact and "exact" in cfg:
        t0 = time.time()
        truth = cfg["exact"]()
        row["exact_seconds"] = round(time.time() - t0, 1)
        for s, t in truth.items():
            n = cfg.get("exact_rows", t.shape[0])
            row[f"cpu_vs_exact_{s}_gate"] = rel_err(want[s][:n], t, 1.0)
            row[f"cpu_vs_exact_{s}_strict"] = rel_err(want[s][:n], t, 1e-3)
            if not args.cpu_only:
                row[f"gpu_vs_exact_{s}_gate"] = rel_err(got[s][:n], t, 1.0)
                row[f"gpu_vs_exact_{s}_strict"] = rel_err(got[s][:n], t, 1e-3)
    cfg["model"].close()
    print(json.dumps(row))


if __name__ == "__main__":
    main()
