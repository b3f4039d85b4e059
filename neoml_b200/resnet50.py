"""ResNet-50 v1.5 as the sequence of math-engine calls a NeoML CDnn graph issues for it.

The graph is what NeoML builds from CConvLayer (+bias; BatchNorm folded into the free terms), CReLULayer,
CImageResizeLayer + CMaxPoolingLayer (the padded stem pool), CEltwiseSumLayer, CGlobalMeanPoolingLayer,
CFullyConnectedLayer, CSoftmaxLayer and CArgmaxLayer.  `forward()` walks it against any backend object that offers
the engine calls below, so the same description drives the B200 engine (EngineBackend here) and, in the tests and
the benchmark's CPU-baseline leg, the reference CPU engine.

v1.5: in each stage's first block the stride-2 sits on the 3x3 convolution.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

STAGES = [(64, 256, 3, 1), (128, 512, 4, 2), (256, 1024, 6, 2), (512, 2048, 3, 2)]  # mid, out, blocks, stride
CLASSES = 1000


@dataclass(frozen=True)
class ConvSpec:
    name: str
    c_in: int
    c_out: int
    k: int
    stride: int
    pad: int


def conv_specs() -> list[ConvSpec]:
    specs = [ConvSpec("stem", 3, 64, 7, 2, 3)]
    c_in = 64
    for si, (mid, out, blocks, stride) in enumerate(STAGES):
        for bi in range(blocks):
            s = stride if bi == 0 else 1
            p = f"s{si + 1}b{bi + 1}"
            specs.append(ConvSpec(p + "_c1", c_in, mid, 1, 1, 0))
            specs.append(ConvSpec(p + "_c2", mid, mid, 3, s, 1))
            specs.append(ConvSpec(p + "_c3", mid, out, 1, 1, 0))
            if bi == 0:
                specs.append(ConvSpec(p + "_down", c_in, out, 1, s, 0))
            c_in = out
    return specs


def flops_per_image(height: int = 224, width: int = 224) -> float:
    """2 * multiply-accumulates of all convolutions and the FC layer (no credit for padding taps)."""
    total = 0.0
    h, w = height, width
    sizes = {}
    # walk the graph once for spatial sizes
    def out(sz, k, s, p):
        return 1 + (sz + 2 * p - k) // s
    h, w = out(h, 7, 2, 3), out(w, 7, 2, 3)
    total += 2.0 * h * w * 64 * 147
    h, w = out(h, 3, 2, 1), out(w, 3, 2, 1)
    c_in = 64
    for mid, o, blocks, stride in STAGES:
        for bi in range(blocks):
            s = stride if bi == 0 else 1
            total += 2.0 * h * w * mid * c_in                 # 1x1 at the input resolution
            h2, w2 = out(h, 3, s, 1), out(w, 3, s, 1)
            total += 2.0 * h2 * w2 * mid * mid * 9            # 3x3 (carries the stride)
            total += 2.0 * h2 * w2 * o * mid                  # 1x1 expand
            if bi == 0:
                total += 2.0 * h2 * w2 * o * c_in             # projection shortcut
            h, w, c_in = h2, w2, o
    total += 2.0 * CLASSES * 2048
    del sizes
    return total


def contraction_bytes_per_image(height: int = 224, width: int = 224) -> float:
    """Algorithmic bytes the convolutions and the FC layer move per image: every input read once, every output
    written once, the shortcut read once by the block's last convolution (it rides in that epilogue); fp32."""
    def out(sz, k, s, p):
        return 1 + (sz + 2 * p - k) // s
    h, w = out(height, 7, 2, 3), out(width, 7, 2, 3)
    floats = height * width * 3 + h * w * 64
    h, w = out(h, 3, 2, 1), out(w, 3, 2, 1)
    c_in = 64
    for mid, o, blocks, stride in STAGES:
        for bi in range(blocks):
            s = stride if bi == 0 else 1
            h2, w2 = out(h, 3, s, 1), out(w, 3, s, 1)
            floats += h * w * c_in + h * w * mid              # 1x1 reduce
            floats += h * w * mid + h2 * w2 * mid             # 3x3
            floats += h2 * w2 * mid + 2 * h2 * w2 * o         # 1x1 expand: input, shortcut, output
            if bi == 0:
                floats += h * w * c_in + h2 * w2 * o          # projection shortcut
            h, w, c_in = h2, w2, o
    floats += 2048 + CLASSES
    return 4.0 * floats


def weight_bytes() -> float:
    return 4.0 * (sum(sp.c_out * sp.k * sp.k * sp.c_in + sp.c_out for sp in conv_specs()) + CLASSES * 2048 + CLASSES)


RESIDUAL_BRANCH_SCALE = 0.25  # folded BatchNorm scale of each block's last convolution


def make_weights(seed: int = 2024) -> dict[str, np.ndarray]:
    """He-normal filters [k, r, s, c] and small free terms (the folded BatchNorm), seeded.  The last convolution of
    every block carries a folded BatchNorm scale of 0.25, as a trained network's would be well below one there;
    without it nothing in a BN-folded random network bounds the residual stream and the 1000 logits saturate."""
    from numpy.random import Generator, Philox
    rng = Generator(Philox(seed))
    w = {}
    for sp in conv_specs():
        fan_in = sp.k * sp.k * sp.c_in
        w[sp.name + ".w"] = (rng.standard_normal((sp.c_out, sp.k, sp.k, sp.c_in), dtype=np.float32)
                             * np.float32(math.sqrt(2.0 / fan_in)))
        if sp.name.endswith("_c3"):
            w[sp.name + ".w"] *= np.float32(RESIDUAL_BRANCH_SCALE)
        w[sp.name + ".b"] = (rng.uniform(-0.1, 0.1, sp.c_out)).astype(np.float32)
    w["fc.w"] = rng.standard_normal((CLASSES, 2048), dtype=np.float32) * np.float32(math.sqrt(2.0 / 2048))
    w["fc.b"] = (rng.uniform(-0.1, 0.1, CLASSES)).astype(np.float32)
    return w


def forward(be, weights, x, fuse: bool = True):
    """Runs the graph on backend `be`.  With fuse=False the calls are exactly the per-layer sequence of the
    reference graph (conv, then ReLU; conv, eltwise sum, ReLU); with fuse=True bias/residual/ReLU ride in the
    convolution epilogue, which is what the engine's fusion of adjacent calls produces.
    Returns (probabilities [batch, 1000], argmax indices [batch])."""
    def conv(name, t, stride, pad, relu, residual=None):
        wt, b = weights[name + ".w"], weights[name + ".b"]
        if fuse:
            return be.conv(t, wt, b, stride, pad, relu=relu, residual=residual)
        y = be.conv(t, wt, b, stride, pad, relu=False, residual=None)
        if residual is not None:
            y = be.add(y, residual)
        return be.relu(y) if relu else y

    t = conv("stem", x, 2, 3, True)
    t = be.max_pool_3x3_s2_p1(t)
    for si, (mid, out, blocks, stride) in enumerate(STAGES):
        for bi in range(blocks):
            s = stride if bi == 0 else 1
            p = f"s{si + 1}b{bi + 1}"
            shortcut = conv(p + "_down", t, s, 0, False) if bi == 0 else t
            u = conv(p + "_c1", t, 1, 0, True)
            u = conv(p + "_c2", u, s, 1, True)
            t = conv(p + "_c3", u, 1, 0, True, residual=shortcut)
    pooled = be.global_mean(t)
    logits = be.fully_connected(pooled, weights["fc.w"], weights["fc.b"])
    probs = be.softmax(logits)
    return probs, be.argmax(probs)


class EngineBackend:
    """The B200 engine behind forward(): torch CUDA tensors in, C-ABI calls on the current stream.
    `timer` (optional) is called as timer(kind, flops) around each contraction for the roofline accounting."""

    def __init__(self, precision: int = 0, timer=None):
        import torch
        from . import ops
        self.torch, self.ops, self.precision, self.timer = torch, ops, precision, timer
        self._scalars = {}

    def _scalar(self, value: float, device):
        key = (value, str(device))
        if key not in self._scalars:
            self._scalars[key] = self.torch.tensor([value], dtype=self.torch.float32, device=device)
        return self._scalars[key]

    def upload(self, weights):
        return {k: self.torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in weights.items()}

    def conv(self, t, w, b, stride, pad, relu, residual):
        ops = self.ops
        flops = None
        if self.timer is not None:
            n, h, wd, _ = t.shape
            k, r, s, c = w.shape
            ho, wo = ops.conv_output_size(h, r, pad, stride), ops.conv_output_size(wd, s, pad, stride)
            flops = 2.0 * n * ho * wo * k * r * s * c
            self.timer.begin()
        y = ops.BlobConvolution(t, w, b, padding=(pad, pad), stride=(stride, stride), residual=residual,
                                act=ops.ACT_RELU if relu else ops.ACT_NONE, precision=self.precision)
        if self.timer is not None:
            self.timer.end("conv", flops)
        return y

    def add(self, a, b):
        return self.ops.VectorAdd(a, b, result=a)

    def relu(self, a):
        return self.ops.VectorReLU(a, result=a, threshold=self._scalar(0.0, a.device))

    def max_pool_3x3_s2_p1(self, t):
        # inputs are post-ReLU, so zero padding equals -inf padding
        padded = self.ops.BlobResizeImage(t, 1, 1, 1, 1, 0, 0.0)
        return self.ops.BlobMaxPooling(padded, (3, 3), (2, 2))

    def global_mean(self, t):
        n, h, w, c = t.shape
        s = self.ops.SumMatrixRows(n, t, h * w, c)
        return self.ops.vector_op("MULTIPLY", s, scalar=self._scalar(1.0 / (h * w), t.device), result=s)

    def fully_connected(self, x, w, b):
        if self.timer is not None:
            self.timer.begin()
        y = self.ops.MultiplyMatrixByTransposedMatrix(x, w, free_term=b, precision=self.precision)
        if self.timer is not None:
            self.timer.end("fc", 2.0 * x.shape[0] * w.shape[0] * w.shape[1])
        return y

    def softmax(self, x):
        return self.ops.MatrixSoftmaxByRows(x, x.shape[0], x.shape[1])

    def argmax(self, x):
        return self.ops.FindMaxValueInRows(x, x.shape[0], x.shape[1])[1]
