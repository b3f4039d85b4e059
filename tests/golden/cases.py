"""Seeded inputs and the case list shared by the golden-vector generator (make_golden.py) and the parity tests.

Inputs come from a counter-based splitmix64 generator written out here, so the same seed gives the same bytes on
any numpy version and on any machine; the golden files only need to store the reference engine's OUTPUTS.
"""
from __future__ import annotations

import numpy as np

_MASK = (1 << 64) - 1


def splitmix64(seed: int, n: int) -> np.ndarray:
    """n 64-bit outputs of splitmix64 started at `seed` (vectorised: state_i = seed + (i+1)*gamma)."""
    gamma = np.uint64(0x9E3779B97F4A7C15)
    idx = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed & _MASK) + idx * gamma
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def uniform(seed: int, shape, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    u = (splitmix64(seed, n) >> np.uint64(40)).astype(np.float64) / float(1 << 24)  # 24 random bits in [0,1)
    return (lo + (hi - lo) * u).astype(np.float32).reshape(shape)


def normal(seed: int, shape, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    u1 = ((splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) + 1.0) / float(1 << 53)
    u2 = (splitmix64(seed ^ 0x5DEECE66D, n) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (std * z).astype(np.float32).reshape(shape)


# ---- convolution: the edge cases of NeoMathEngine/test/src/inference/BlobConvolutionTest.cpp:113-400 in small form
# (1x1; stride larger than the filter; padding >= filter; dilation 3; one-pixel-high images; channels not a multiple
# of 4 or 32; filter count not a multiple of the tile) plus a tap-aligned C%32==0 case.
CONV_CASES = {
    # name: (batch,h,w,c, k,r,s, pad, stride, dil, free_term)
    "pointwise": (2, 7, 9, 16, 24, 1, 1, (0, 0), (1, 1), (1, 1), True),
    "pointwise_nobias": (1, 5, 6, 3, 5, 1, 1, (0, 0), (1, 1), (1, 1), False),
    "k3_pad1": (2, 9, 11, 5, 7, 3, 3, (1, 1), (1, 1), (1, 1), True),
    "k3_c32_tap": (2, 10, 12, 32, 40, 3, 3, (1, 1), (1, 1), (1, 1), True),
    "k3_c64_s2": (1, 13, 14, 64, 33, 3, 3, (1, 1), (2, 2), (1, 1), True),
    "stride_gt_filter": (2, 11, 13, 4, 6, 2, 2, (0, 0), (3, 4), (1, 1), True),
    "pad_w_ge_filter": (1, 6, 7, 3, 4, 2, 3, (1, 4), (1, 2), (1, 1), True),
    "dilation3": (1, 12, 13, 6, 5, 3, 3, (3, 3), (1, 1), (3, 3), True),
    "dil_mixed": (2, 11, 9, 32, 8, 3, 2, (2, 1), (2, 1), (2, 3), False),
    "tall_1px_wide": (1, 40, 1, 8, 9, 3, 1, (1, 0), (1, 1), (1, 1), True),
    "stem_7x7_s2_c3": (1, 30, 32, 3, 16, 7, 7, (3, 3), (2, 2), (1, 1), True),
    "k1_s2": (2, 8, 10, 32, 48, 1, 1, (0, 0), (2, 2), (1, 1), True),
    "wide_k": (1, 4, 5, 8, 300, 3, 3, (1, 1), (1, 1), (1, 1), True),
}


# Cases checked against the plain-C oracle only: with vertical padding >= filter height the reference CPU engine
# (this build: MLAS + AVX module, gcc 13) returns NaN / 1e38 garbage in the padded rows, so it cannot pin them.
CONV_CASES_ORACLE_ONLY = {
    "pad_h_ge_filter": (1, 6, 7, 3, 4, 2, 3, (3, 4), (1, 2), (1, 1), True),
    "pad_h_gt_filter_c32": (1, 5, 6, 32, 8, 2, 2, (3, 2), (1, 1), (1, 1), False),
}


def conv_inputs(name: str):
    table = CONV_CASES if name in CONV_CASES else CONV_CASES_ORACLE_ONLY
    b, h, w, c, k, r, s, pad, stride, dil, ft = table[name]
    if name not in CONV_CASES:
        seed = 1500 + 17 * sorted(CONV_CASES_ORACLE_ONLY).index(name)
        x = uniform(seed, (b, h, w, c))
        return x, uniform(seed + 1, (k, r, s, c)), uniform(seed + 2, (k,)) if ft else None, dict(
            padding=pad, stride=stride, dilation=dil)
    seed = 1000 + 17 * sorted(CONV_CASES).index(name)
    x = uniform(seed, (b, h, w, c))
    flt = uniform(seed + 1, (k, r, s, c))
    bias = uniform(seed + 2, (k,)) if ft else None
    return x, flt, bias, dict(padding=pad, stride=stride, dilation=dil)


# ---- matrix products: MultiplyMatrixByTransposedMatrixTest.cpp:38-64 draws sizes 1..500 and row strides >= width
MMT_CASES = {
    # name: (m, k, n, lda, ldb)
    "tiny": (1, 1, 1, 1, 1),
    "odd": (37, 53, 29, 53, 53),
    "strided": (33, 40, 21, 47, 44),
    "k_tail": (130, 70, 65, 70, 70),
    "aligned": (256, 128, 192, 128, 128),
    "long_k": (9, 500, 7, 500, 500),
}


def mmt_inputs(name: str):
    m, k, n, lda, ldb = MMT_CASES[name]
    seed = 2000 + 13 * sorted(MMT_CASES).index(name)
    return uniform(seed, (m, lda)), uniform(seed + 1, (n, ldb)), dict(m=m, k=k, n=n, lda=lda, ldb=ldb)


MM_CASES = {
    # name: (batch, m, k, n)
    "single": (1, 17, 23, 31),
    "batched_odd": (3, 17, 23, 31),
    "attention_qk": (4, 48, 64, 48),
    "attention_pv": (4, 48, 48, 64),
    "n1": (2, 5, 7, 1),
}


def mm_inputs(name: str):
    b, m, k, n = MM_CASES[name]
    seed = 3000 + 11 * sorted(MM_CASES).index(name)
    return uniform(seed, (b, m, k)), uniform(seed + 1, (b, k, n))


CHCONV_CASES = {
    # name: (batch,h,w,c, r,s, pad, stride, free_term)
    "k3_s1": (2, 10, 12, 24, 3, 3, (1, 1), (1, 1), True),
    "k3_s2": (2, 11, 13, 24, 3, 3, (1, 1), (2, 2), True),
    "c_odd": (1, 7, 8, 5, 3, 3, (1, 1), (1, 1), False),
    "k5": (1, 9, 9, 8, 5, 5, (2, 2), (1, 1), True),
}


def chconv_inputs(name: str):
    b, h, w, c, r, s, pad, stride, ft = CHCONV_CASES[name]
    seed = 4000 + 7 * sorted(CHCONV_CASES).index(name)
    return (uniform(seed, (b, h, w, c)), uniform(seed + 1, (r, s, c)), uniform(seed + 2, (c,)) if ft else None,
            dict(padding=pad, stride=stride))


# ---- MobileNetV2 block: the axes of NeoML/test/src/DnnMobileNetV2BlockTest.cpp:113-178
# (free-term presence, ReLU thresholds incl. none, stride, residual) in small form
MBV2_CASES = {
    # name: (batch,h,w,c_in,c_exp,c_out, stride, residual, act_exp, p_exp, act_dw, p_dw, biases(exp,dw,down))
    "relu6_res": (2, 12, 12, 8, 48, 8, 1, True, 1, 6.0, 1, 6.0, (True, True, True)),
    "relu6_s2": (2, 13, 11, 8, 48, 16, 2, False, 1, 6.0, 1, 6.0, (True, True, True)),
    "relu_nothr": (1, 9, 9, 8, 40, 8, 1, True, 1, 0.0, 1, 0.0, (True, False, True)),
    "hswish": (1, 8, 10, 16, 32, 24, 1, False, 2, 0.0, 2, 0.0, (False, True, False)),
    "nobias": (1, 6, 6, 4, 12, 4, 1, True, 1, 1.0, 1, 0.5, (False, False, False)),
}


def mbv2_inputs(name: str):
    b, h, w, ci, ce, co, stride, res, a1, p1, a2, p2, biases = MBV2_CASES[name]
    seed = 5000 + 19 * sorted(MBV2_CASES).index(name)
    x = uniform(seed, (b, h, w, ci), 0.0, 1.0)
    w_exp = normal(seed + 1, (ce, ci), float(np.sqrt(2.0 / ci)))
    w_dw = normal(seed + 2, (3, 3, ce), float(np.sqrt(2.0 / 9)))
    w_down = normal(seed + 3, (co, ce), float(np.sqrt(2.0 / ce)))
    b_exp = uniform(seed + 4, (ce,), -0.1, 0.1) if biases[0] else None
    b_dw = uniform(seed + 5, (ce,), -0.1, 0.1) if biases[1] else None
    b_down = uniform(seed + 6, (co,), -0.1, 0.1) if biases[2] else None
    kw = dict(stride=stride, residual=res, act_exp=a1, act_exp_param=p1, act_dw=a2, act_dw_param=p2)
    return (x, w_exp, b_exp, w_dw, b_dw, w_down, b_down), kw


SOFTMAX_CASES = {"narrow": (13, 37), "w512": (6, 512), "w1000": (3, 1000), "wide": (2, 1500), "one": (5, 1)}


def softmax_inputs(name: str):
    h, w = SOFTMAX_CASES[name]
    seed = 6000 + 5 * sorted(SOFTMAX_CASES).index(name)
    return uniform(seed, (h * w,), -8.0, 8.0), h, w
