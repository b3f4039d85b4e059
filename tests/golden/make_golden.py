"""Generates tests/golden/reference_cpu_engine.npz: outputs of the reference's OWN CPU math engine
(oracle/_ref, built by `make -C oracle ref` from the NeoML sources) on the seeded cases of cases.py.

Run where a NeoML checkout exists:   make -C oracle ref && python tests/golden/make_golden.py
The .npz is committed; the parity tests and the oracle pin test read it and never need the checkout.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent / "oracle"))
sys.path.insert(0, str(HERE))

import cases  # noqa: E402
from oracle_lib import Reference  # noqa: E402


def main() -> None:
    ref = Reference()
    out = {}
    for name in cases.CONV_CASES:
        x, f, b, kw = cases.conv_inputs(name)
        out[f"conv/{name}"] = ref.blob_convolution(x, f, b, **kw)
    for name in cases.MMT_CASES:
        a, b, kw = cases.mmt_inputs(name)
        out[f"mmt/{name}"] = ref.multiply_matrix_by_transposed_matrix(a, b, **kw)
    for name in cases.MM_CASES:
        a, b = cases.mm_inputs(name)
        out[f"mm/{name}"] = ref.multiply_matrix_by_matrix(a, b)
    for name in cases.CHCONV_CASES:
        x, f, b, kw = cases.chconv_inputs(name)
        out[f"chconv/{name}"] = ref.blob_channelwise_convolution(x, f, b, **kw)
    for name in cases.MBV2_CASES:
        args, kw = cases.mbv2_inputs(name)
        out[f"mbv2/{name}"] = ref.mobilenetv2_block(*args, **kw)
    for name in cases.SOFTMAX_CASES:
        x, h, w = cases.softmax_inputs(name)
        out[f"softmax/{name}"] = ref.matrix_softmax_by_rows(x, h, w)
    ref.close()
    path = HERE / "reference_cpu_engine.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {path.stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
