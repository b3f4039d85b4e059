"""BASELINE config 3 in small form: ResNet-50 v1.5 through the B200 kernels against the same graph on the
reference's own CPU math engine (oracle/_ref; the plain-C oracle where that build is absent).
Probabilities within 1e-4 (norm-wise), argmax indices bit-exact.  Needs a B200."""
import numpy as np
import pytest
import torch

from neoml_b200 import resnet50
from oracle_lib import TOL_FP32, TOL_TF32, Reference, gate_err, rel_err

gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def net():
    assert torch.cuda.is_available()
    import ref_backend
    weights = resnet50.make_weights()
    batch = 4 if Reference.available() else 1
    x = np.random.default_rng(99).uniform(0, 1, (batch, 224, 224, 3)).astype(np.float32)
    cpu = ref_backend.RefBackend() if Reference.available() else ref_backend.OracleBackend()
    probs, idx = resnet50.forward(cpu, weights, x, fuse=False)
    return weights, x, probs, idx


@gpu
@pytest.mark.parametrize("precision,tol", [(0, TOL_FP32), (1, TOL_TF32)])
@pytest.mark.parametrize("fuse", [True, False])
def test_resnet50_matches_cpu_engine(net, precision, tol, fuse):
    weights, x, want_probs, want_idx = net
    be = resnet50.EngineBackend(precision=precision)
    probs, idx = resnet50.forward(be, be.upload(weights), torch.from_numpy(x).cuda(), fuse=fuse)
    probs, idx = probs.cpu().numpy(), idx.cpu().numpy()
    g, s = gate_err(probs, want_probs), rel_err(probs, want_probs)
    print(f"resnet50 precision={precision} fuse={fuse}: probabilities gate {g:.3e} strict {s:.3e}")
    assert g < tol
    # the top-2 margin of the CPU result is far above the numeric noise, so the index must agree exactly
    top2 = np.sort(want_probs, axis=1)[:, -2:]
    assert ((top2[:, 1] - top2[:, 0]) > 1e-3).all()
    assert np.array_equal(idx, want_idx)


@gpu
def test_resnet50_through_the_cpp_engine(net):
    """The same graph issued as IMathEngine virtual calls on CB200MathEngine (stack-allocated scratch, engine stream,
    handles): what a CDnn built on this engine executes."""
    import ref_backend
    from oracle_lib import ShimmedB200Engine
    if not ShimmedB200Engine.available():
        pytest.skip("libNeoMathEngineB200.so or the shim not built")
    weights, x, want_probs, want_idx = net
    be = ref_backend.ShimmedEngineBackend()
    try:
        probs, idx = resnet50.forward(be, be.upload(weights), torch.from_numpy(x).cuda(), fuse=False)
        be.impl.sync()
        probs, idx = probs.cpu().numpy(), idx.cpu().numpy()
    finally:
        be.close()
    g = gate_err(probs, want_probs)
    print(f"resnet50 through CB200MathEngine: probabilities gate {g:.3e}")
    assert g < TOL_FP32
    assert np.array_equal(idx, want_idx)


def test_flop_count_matches_published_figure():
    assert abs(resnet50.flops_per_image() / 1e9 - 8.178) < 0.01
    assert len(resnet50.conv_specs()) == 53


@gpu
def test_forward_pass_replays_from_a_cuda_graph(net):
    """The library allocates nothing and keeps no per-call host state: a captured forward pass replays bit for bit."""
    weights, x, _, _ = net
    be = resnet50.EngineBackend()
    dw = be.upload(weights)
    dx = torch.from_numpy(x).cuda()
    probs, idx = resnet50.forward(be, dw, dx, fuse=True)          # also the one-time set-up, outside capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            g_probs, g_idx = resnet50.forward(be, dw, dx, fuse=True)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        g_probs.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(g_probs, probs) and torch.equal(g_idx, idx)
