"""TEST INFRASTRUCTURE.  Writes tests/golden/engine_call_closure.json: for each benchmark graph, the IMathEngine
methods NeoML calls on the engine while it loads the model, reshapes and runs it (counts from one load + two runs at
a small size; the set does not depend on the size).  Needs the hosted libraries (make -C neoml_b200/host) and the
recording engine of gen_trace_engine.py built against them; run it where a NeoML checkout is available:

    python tests/closure/make_closure.py <libtrace_engine.so>
"""
from __future__ import annotations

import ctypes as C
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from neoml_b200 import cdnn, resnet50  # noqa: E402


class TraceEngine:
    kind = "trace"

    def __init__(self, lib):
        self.lib = lib
        lib.trace_engine_create.restype = C.c_void_p
        lib.trace_engine_calls.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        self.ptr = lib.trace_engine_create()

    def calls(self) -> dict[str, int]:
        buf = C.create_string_buffer(1 << 16)
        n = self.lib.trace_engine_calls(self.ptr, buf, len(buf))
        assert n >= 0
        return {k: int(v) for k, v in (line.split() for line in buf.value.decode().splitlines())}


def main() -> None:
    cdnn.load()
    trace = TraceEngine(C.CDLL(sys.argv[1], mode=C.RTLD_GLOBAL))
    rng = np.random.default_rng(0)
    f32 = lambda *s: rng.standard_normal(s).astype(np.float32)
    out = {}

    def record(name, model, inputs, sinks):
        trace.calls()
        net = cdnn.Net(trace, model)
        for _ in range(2):
            for k, v in inputs.items():
                net.set_input(k, *v) if isinstance(v, tuple) else net.set_input(k, v)
            net.run()
            for s in sinks:
                net.output(s)
        net.close()
        out[name] = trace.calls()
        print(name, len(out[name]), "methods")

    record("config1_blob_convolution", cdnn.Model.conv(f32(8, 3, 3, 8), f32(8), padding=(1, 1)),
           {"in": f32(2, 9, 9, 8)}, ["out"])
    record("config2_mobilenetv2_block",
           cdnn.Model.mbv2(f32(24, 8), f32(24), f32(3, 3, 24), f32(24), f32(8, 24), f32(8)),
           {"in": f32(2, 8, 8, 8)}, ["out"])
    record("config3_resnet50", cdnn.Model.resnet50(resnet50.make_weights()),
           {"in": np.abs(f32(1, 64, 64, 3))}, ["probs", "argmax"])
    record("config4_transformer_encoder", cdnn.Model.transformer(2, 64, 4, 128, mask=True),
           {"in": f32(2, 16, 64), "mask": (np.triu(np.ones((16, 16), np.float32), 1), (1, 1, 1, 1, 16, 1, 16))},
           ["out"])
    record("config5_matrix_product", cdnn.Model.matmul(),
           {"a": (f32(1, 32, 48), (1, 1, 1, 32, 1, 1, 48)), "b": (f32(1, 48, 40), (1, 1, 1, 48, 1, 1, 40))}, ["out"])
    target = ROOT / "tests" / "golden" / "engine_call_closure.json"
    target.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print("wrote", target)


if __name__ == "__main__":
    main()
