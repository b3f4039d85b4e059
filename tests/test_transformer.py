"""Config 4 (transformer encoder layer as its engine-call sequence): the plain-C oracle against the reference CPU
engine on CPU; the B200 IMathEngine (real virtual calls through the shim) against the reference engine on the GPU."""
import numpy as np
import pytest

import transformer_graph as tg
from oracle_lib import TOL_FP32, gate_err

SMALL = dict(batch=2, seq=48, hidden=96, heads=4)       # head dim 24: nothing is a multiple of 32
MEDIUM = dict(batch=2, seq=128, hidden=256, heads=4)    # head dim 64, the production head size


def test_oracle_matches_reference_engine(oracle, reference):
    cfg = SMALL
    w = tg.make_weights(7000, cfg["hidden"], 4 * cfg["hidden"])
    x, mask = tg.make_inputs(7100, cfg["batch"], cfg["seq"], cfg["hidden"])
    want = tg.encoder_layer(reference, x, w, mask, **cfg)
    got = tg.encoder_layer(oracle, x, w, mask, **cfg)
    assert np.isfinite(want).all() and abs(float(want.std()) - 1.0) < 0.5     # layer-normed output
    assert gate_err(got, want) < TOL_FP32


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [SMALL, MEDIUM], ids=["small", "medium"])
def test_b200_engine_matches_reference_engine(reference, cfg):
    import torch
    from oracle_lib import ShimmedB200Engine
    if not ShimmedB200Engine.available():
        pytest.skip("libNeoMathEngineB200.so not built")
    w = tg.make_weights(7000, cfg["hidden"], 4 * cfg["hidden"])
    x, mask = tg.make_inputs(7100, cfg["batch"], cfg["seq"], cfg["hidden"])
    want = tg.encoder_layer(reference, x, w, mask, **cfg)
    e = ShimmedB200Engine()
    try:
        dw = {k: torch.from_numpy(v).cuda() for k, v in w.items()}
        got = tg.encoder_layer(e, torch.from_numpy(x).cuda(), dw, torch.from_numpy(mask).cuda(), **cfg)
        e.sync()
        got = got.cpu().numpy()
    finally:
        e.close()
    assert gate_err(got, want) < TOL_FP32
