"""Parity of the CUDA path against the reference CPU engine's committed outputs (tests/golden) and the plain-C
oracle, through the C ABI (neoml_b200.ops -> include/neoml_b200.h).  Needs a B200: run with -m gpu.

Tolerances (north-star contract): 1e-4 max relative error for the default 3xTF32 arithmetic, 1e-2 for opt-in TF32;
index outputs bit-exact.  The error metric is oracle_lib.gate_err (norm-wise: |g-w| / max(|w|, RMS(w))); the
strict-floor figure (floor 1e-3 x RMS) is printed alongside.
"""
import os

import numpy as np
import pytest
import torch

import cases
from oracle_lib import TOL_FP32, TOL_TF32, gate_err, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from neoml_b200 import _capi, ops as ops_mod
    assert _capi.load().nb200_device_count() >= 1, "no sm_100 device: the CUDA path cannot run (no fallback exists)"
    yield ops_mod
    torch.cuda.synchronize()
    assert _capi.load().nb200_device_status(None, 0) == 0, "a kernel reported a bounded-wait timeout"


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


PRECISIONS = [(0, TOL_FP32), (1, TOL_TF32), (2, TOL_FP32)]


def check(got, want, tol, what):
    g, s = gate_err(got, want), rel_err(got, want)
    print(f"{what}: gate {g:.3e} strict {s:.3e}")
    assert got.shape == want.shape
    assert np.isfinite(got).all(), what
    assert g < tol, f"{what}: {g:.3e} >= {tol}"


@pytest.mark.parametrize("prec,tol", PRECISIONS)
@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_blob_convolution_golden(ops, golden, oracle, name, prec, tol):
    x, f, b, kw = cases.conv_inputs(name)
    y = host(ops.BlobConvolution(dev(x), dev(f), dev(b), precision=prec, **kw))
    check(y, golden[f"conv/{name}"], tol, f"conv/{name}/ref")
    check(y, oracle.blob_convolution(x, f, b, **kw), tol, f"conv/{name}/oracle")


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES_ORACLE_ONLY))
def test_blob_convolution_oracle_only(ops, oracle, name):
    x, f, b, kw = cases.conv_inputs(name)
    y = host(ops.BlobConvolution(dev(x), dev(f), dev(b), **kw))
    check(y, oracle.blob_convolution(x, f, b, **kw), TOL_FP32, f"conv/{name}/oracle")


@pytest.mark.parametrize("name", ["stem_7x7_s2_c3", "k3_pad1", "dilation3", "pad_w_ge_filter"])
def test_blob_convolution_without_scratch(ops, golden, name):
    """Channel counts that are not a multiple of four: the element-wise gather (no scratch) and the widened-pixel
    path (scratch, the default of ops.BlobConvolution) must both match."""
    x, f, b, kw = cases.conv_inputs(name)
    y = host(ops.BlobConvolution(dev(x), dev(f), dev(b), use_scratch=False, **kw))
    check(y, golden[f"conv/{name}"], TOL_FP32, f"conv/{name}/no-scratch")


def test_blob_convolution_fused_tail(ops, oracle):
    """bias + residual + ReLU in the epilogue equals the unfused sequence."""
    x, f, b, kw = cases.conv_inputs("k3_c32_tap")
    want = oracle.blob_convolution(x, f, b, **kw)
    res = cases.uniform(77, want.shape)
    want = np.maximum(want + res, 0.0)
    y = host(ops.BlobConvolution(dev(x), dev(f), dev(b), residual=dev(res), act=ops.ACT_RELU, **kw))
    check(y, want, TOL_FP32, "conv fused tail")


def test_blob_convolution_unaligned_handles(ops, oracle):
    """NeoML handles may sit at any 4-byte offset: shift every operand by one float."""
    x, f, b, kw = cases.conv_inputs("k3_c32_tap")
    want = oracle.blob_convolution(x, f, b, **kw)

    def shifted(a):
        buf = torch.zeros(a.size + 1, dtype=torch.float32, device="cuda")
        buf[1:] = torch.from_numpy(a.ravel()).cuda()
        return buf[1:].view(a.shape)

    out = torch.zeros(want.size + 1, dtype=torch.float32, device="cuda")
    y = ops.BlobConvolution(shifted(x), shifted(f), shifted(b), result=out[1:].view(want.shape), **kw)
    check(host(y), want, TOL_FP32, "conv unaligned")


@pytest.mark.parametrize("prec,tol", PRECISIONS)
@pytest.mark.parametrize("name", sorted(cases.MMT_CASES))
def test_multiply_matrix_by_transposed_matrix(ops, golden, name, prec, tol):
    a, b, kw = cases.mmt_inputs(name)
    y = ops.MultiplyMatrixByTransposedMatrix(dev(a), dev(b), first_height=kw["m"], first_width=kw["k"],
                                             second_height=kw["n"], first_row_size=kw["lda"],
                                             second_row_size=kw["ldb"], precision=prec)
    check(host(y), golden[f"mmt/{name}"], tol, f"mmt/{name}")


def test_mmt_strided_result_and_bias(ops, oracle):
    a, b, kw = cases.mmt_inputs("strided")
    bias = cases.uniform(5, (kw["n"],))
    want = oracle.multiply_matrix_by_transposed_matrix(a, b, **kw) + bias
    out = torch.full((kw["m"], kw["n"] + 3), 7.0, dtype=torch.float32, device="cuda")
    ops.MultiplyMatrixByTransposedMatrix(dev(a), dev(b), out, first_height=kw["m"], first_width=kw["k"],
                                         second_height=kw["n"], first_row_size=kw["lda"], second_row_size=kw["ldb"],
                                         result_row_size=kw["n"] + 3, free_term=dev(bias))
    got = host(out)
    check(np.ascontiguousarray(got[:, :kw["n"]]), want, TOL_FP32, "mmt strided result")
    assert (got[:, kw["n"]:] == 7.0).all(), "columns beyond the result width were overwritten"


@pytest.mark.parametrize("prec,tol", PRECISIONS)
@pytest.mark.parametrize("name", sorted(cases.MM_CASES))
def test_multiply_matrix_by_matrix(ops, golden, name, prec, tol):
    a, b = cases.mm_inputs(name)
    check(host(ops.MultiplyMatrixByMatrix(dev(a), dev(b), precision=prec)), golden[f"mm/{name}"], tol, f"mm/{name}")
    # the kernel's own gather of the column-major operand (what a caller without scratch memory gets)
    check(host(ops.MultiplyMatrixByMatrix(dev(a), dev(b), precision=prec, use_scratch=False)), golden[f"mm/{name}"], tol,
          f"mm/{name} (no scratch)")


def test_batch_mmt(ops, oracle):
    a, b = cases.uniform(41, (3, 50, 70)), cases.uniform(42, (3, 33, 70))
    want = np.stack([oracle.multiply_matrix_by_transposed_matrix(a[i], b[i]) for i in range(3)])
    check(host(ops.BatchMultiplyMatrixByTransposedMatrix(dev(a), dev(b))), want, TOL_FP32, "batch mmt")


@pytest.mark.parametrize("name", sorted(cases.CHCONV_CASES))
def test_channelwise_convolution(ops, golden, name):
    x, f, b, kw = cases.chconv_inputs(name)
    check(host(ops.BlobChannelwiseConvolution(dev(x), dev(f), dev(b), **kw)), golden[f"chconv/{name}"], TOL_FP32,
          f"chconv/{name}")


@pytest.mark.parametrize("prec,tol", [(0, TOL_FP32), (1, TOL_TF32)])
@pytest.mark.parametrize("name", sorted(cases.MBV2_CASES))
def test_mobilenetv2_block(ops, golden, name, prec, tol):
    (x, we, be, wd, bd, wp, bp), kw = cases.mbv2_inputs(name)
    y = ops.MobileNetV2Block(dev(x), dev(we), dev(be), dev(wd), dev(bd), dev(wp), dev(bp), stride=kw["stride"],
                             residual=kw["residual"], expand_act=kw["act_exp"], expand_act_param=kw["act_exp_param"],
                             channelwise_act=kw["act_dw"], channelwise_act_param=kw["act_dw_param"], precision=prec)
    check(host(y), golden[f"mbv2/{name}"], tol, f"mbv2/{name}")


def test_mobilenetv2_block_in_place(ops, golden):
    (x, we, be, wd, bd, wp, bp), kw = cases.mbv2_inputs("relu6_res")
    xd = dev(x)
    ops.MobileNetV2Block(xd, dev(we), dev(be), dev(wd), dev(bd), dev(wp), dev(bp), result=xd, stride=1, residual=True)
    check(host(xd), golden["mbv2/relu6_res"], TOL_FP32, "mbv2 in place")


@pytest.mark.parametrize("name", sorted(cases.SOFTMAX_CASES))
def test_softmax(ops, golden, name):
    x, h, w = cases.softmax_inputs(name)
    xd = dev(x)
    check(host(ops.MatrixSoftmaxByRows(xd, h, w)), golden[f"softmax/{name}"], 1e-5, f"softmax/{name}")
    ops.MatrixSoftmaxByRows(xd, h, w, result=xd)  # in place
    check(host(xd), golden[f"softmax/{name}"], 1e-5, f"softmax/{name} in place")


def test_vector_ops(ops, oracle):
    from neoml_b200._capi import VEC_OPS
    for n in (1, 7, 1001, 4096):
        a = cases.uniform(11, (n,), -4, 4)
        b = cases.uniform(12, (n,), -4, 4)
        sc = torch.tensor([0.7], dtype=torch.float32, device="cuda")
        for op, name in enumerate(VEC_OPS):
            a_ = np.abs(a) + 0.1 if name in ("SQRT", "INV") else a
            b_ = np.abs(b) + 0.5 if name == "ELTWISE_DIV" else b
            got = host(ops.vector_op(name, dev(a_), dev(b_), scalar=sc, value=0.7))
            want = oracle.vector_op(op, a_, b_, 0.7)
            assert gate_err(got, want) < 1e-5, (name, n)  # fused multiply-add vs two roundings, expf vs exp


def test_sigmoid_gate_in_one_pass_equals_the_three_calls(ops, oracle):
    """y = sigmoid(a * s) * a (CGELULayer's fast form) as one pass: the bits of VectorMultiply, VectorSigmoid,
    VectorEltwiseMultiply run one after the other, and the oracle's chain to tolerance."""
    for n in (5, 1001, 1 << 16):
        a = cases.uniform(14, (n,), -6, 6)
        sc = torch.tensor([1.702], dtype=torch.float32, device="cuda")
        ad = dev(a)
        t = ops.vector_op("MULTIPLY", ad, scalar=sc)
        t = ops.vector_op("SIGMOID", t)
        three = host(ops.vector_op("ELTWISE_MUL", ad, t))
        one = host(ops.vector_op("SIGMOID_MUL", ad, scalar=sc))
        assert np.array_equal(one, three)
        want = oracle.vector_op(5, a, oracle.vector_op(10, oracle.vector_op(6, a, None, 1.702)))
        assert gate_err(one, want) < 1e-5


def test_vector_ops_unaligned_and_in_place(ops, oracle):
    a = cases.uniform(13, (1003,))
    buf = torch.zeros(1004, dtype=torch.float32, device="cuda")
    buf[1:] = dev(a)
    thr = torch.tensor([0.25], dtype=torch.float32, device="cuda")
    ops.vector_op("RELU", buf[1:], scalar=thr, result=buf[1:])
    assert np.array_equal(host(buf[1:]), oracle.vector_op(9, a, None, 0.25))
    assert float(buf[0]) == 0.0


def test_matrix_helpers(ops, oracle):
    for (bsz, h, w) in [(3, 5, 7), (2, 64, 768), (1, 300, 2048), (4, 49, 64)]:
        m = cases.uniform(21, (bsz * h * w,))
        v_bw, v_rows, v_w = cases.uniform(22, (bsz * w,)), cases.uniform(23, (bsz * h,)), cases.uniform(24, (w,))
        md = dev(m)
        assert np.array_equal(host(ops.AddVectorToMatrixRows(bsz, md, dev(v_bw), h, w)),
                              oracle.add_vector_to_matrix_rows(bsz, m, h, w, v_bw))
        assert np.array_equal(host(ops.AddVectorToMatrixColumns(md, dev(v_rows), bsz * h, w)),
                              oracle.add_vector_to_matrix_columns(m, bsz * h, w, v_rows))
        assert gate_err(host(ops.SumMatrixRows(bsz, md, h, w)), oracle.sum_matrix_rows(bsz, m, h, w)) < 1e-5
        init = cases.uniform(25, (bsz, w))
        assert gate_err(host(ops.SumMatrixRows(bsz, md, h, w, result=dev(init), add=True)),
                        oracle.sum_matrix_rows(bsz, m, h, w, init)) < 1e-5
        assert gate_err(host(ops.SumMatrixColumns(md, bsz * h, w)), oracle.sum_matrix_columns(m, bsz * h, w)) < 1e-5
        assert np.array_equal(host(ops.MultiplyDiagMatrixByMatrix(dev(v_rows), md, bsz * h, w)),
                              oracle.multiply_diag_matrix_by_matrix(v_rows, bsz * h, m, w))
        assert np.array_equal(host(ops.BatchMultiplyMatrixByDiagMatrix(1, md, bsz * h, w, dev(v_w), 0)),
                              oracle.multiply_matrix_by_diag_matrix(1, m, bsz * h, w, v_w, 0))
        assert np.array_equal(host(ops.BatchMultiplyMatrixByDiagMatrix(bsz, md, h, w, dev(v_bw), w)),
                              oracle.multiply_matrix_by_diag_matrix(bsz, m, h, w, v_bw, w))


def test_transpose(ops, oracle):
    # the last four are plain matrices with both extents a multiple of four: the 64 x 64-tile kernel, ragged tiles included
    for (b, h, m, w, c) in [(2, 3, 4, 5, 6), (2, 48, 1, 12, 64), (3, 50, 1, 70, 1), (1, 1, 1, 9, 4), (2, 33, 1, 1, 5),
                            (3, 100, 1, 36, 1), (2, 68, 1, 132, 1), (1, 256, 1, 512, 1), (5, 64, 1, 4, 1)]:
        t = cases.uniform(26, (b * h * m * w * c,))
        assert np.array_equal(host(ops.TransposeMatrix(b, dev(t), h, m, w, c)), oracle.transpose_matrix(b, t, h, m, w, c))


def test_argmax_bit_exact(ops, oracle):
    for (h, w) in [(13, 37), (256, 1000), (5, 1)]:
        am = cases.uniform(27, (h * w,))
        am[3 % am.size] = am.max()  # a tie: first maximum must win
        v, i = ops.FindMaxValueInRows(dev(am), h, w)
        ov, oi = oracle.find_max_value_in_rows(am, h, w)
        assert np.array_equal(host(v), ov) and np.array_equal(host(i), oi)
    am = cases.uniform(28, (2 * 6 * 37,))
    v, i = ops.FindMaxValueInColumns(2, dev(am), 6, 37)
    ov, oi = oracle.find_max_value_in_columns(2, am, 6, 37)
    assert np.array_equal(host(v), ov) and np.array_equal(host(i), oi)


def test_pooling_and_resize(ops, oracle):
    for shape in [(2, 9, 11, 6), (2, 10, 12, 8)]:
        x = cases.uniform(31, shape)
        y, idx = ops.BlobMaxPooling(dev(x), (3, 3), (2, 2), with_indices=True)
        want, _ = oracle.blob_max_pooling(x, (3, 3), (2, 2))
        assert np.array_equal(host(y), want)
        # every index points at a maximum of its window (the reference's index layout: offset inside the image)
        flat = x.reshape(shape[0], -1)
        picked = np.take_along_axis(flat, host(idx).reshape(shape[0], -1).astype(np.int64), axis=1)
        assert np.array_equal(picked.reshape(want.shape), want)
        assert rel_err(host(ops.BlobMeanPooling(dev(x), (3, 2), (2, 1))), oracle.blob_mean_pooling(x, (3, 2), (2, 1))) < 1e-6
        for pad in (0, 1, 2):
            assert np.array_equal(host(ops.BlobResizeImage(dev(x), 1, 2, 2, 1, pad, 0.5)),
                                  oracle.blob_resize_image(x, 1, 2, 2, 1, pad, 0.5))
        assert np.array_equal(host(ops.BlobResizeImage(dev(x), -1, -2, -2, 1, 0, 0.5)),
                              oracle.blob_resize_image(x, -1, -2, -2, 1, 0, 0.5))


def test_empty_inputs(ops):
    e = torch.empty(0, dtype=torch.float32, device="cuda")
    assert ops.vector_op("COPY", e, result=e).numel() == 0
    y = ops.MultiplyMatrixByTransposedMatrix(torch.empty((0, 8), device="cuda"), torch.ones((4, 8), device="cuda"))
    assert y.shape == (0, 4)


# ---- full-size checks through size-independent properties ------------------------------------------------------------

def test_config1_convolution_full_size(ops, oracle):
    """BASELINE config 1 (32x56x56x64, 64 filters 3x3, pad 1, bias): sampled outputs against the oracle, and
    linearity conv(x1 + x2) == conv(x1) + conv(x2) - bias over the whole tensor."""
    x1, x2 = cases.uniform(101, (32, 56, 56, 64)), cases.uniform(102, (32, 56, 56, 64))
    f, b = cases.uniform(103, (64, 3, 3, 64)), cases.uniform(104, (64,))
    fd, bd = dev(f), dev(b)
    y1 = ops.BlobConvolution(dev(x1), fd, bd, padding=(1, 1))
    y2 = ops.BlobConvolution(dev(x2), fd, bd, padding=(1, 1))
    y12 = ops.BlobConvolution(dev(x1 + x2), fd, bd, padding=(1, 1))
    lin = host(y1 + y2 - bd)
    check(host(y12), lin, 2e-4, "config1 linearity")  # two roundings of the inputs' sum on the right-hand side
    # oracle on 3 images
    want = oracle.blob_convolution(x1[:3], f, b, padding=(1, 1))
    check(host(y1)[:3], want, TOL_FP32, "config1 vs oracle (3 images)")
    # the exact-fp32 CUDA-core path on the full tensor
    y_simt = ops.BlobConvolution(dev(x1), fd, bd, padding=(1, 1), precision=ops.PREC_FP32_SIMT)
    check(host(y1), host(y_simt), TOL_FP32, "config1 tensor-core vs CUDA-core")


def test_config5_gemm_1024(ops, oracle):
    a, b = cases.uniform(111, (1024, 1024)), cases.uniform(112, (1024, 1024))
    y = ops.MultiplyMatrixByMatrix(dev(a), dev(b))
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    check(host(y), want, TOL_FP32, "gemm 1024 NN")
    yt = ops.MultiplyMatrixByTransposedMatrix(dev(a), dev(b))
    want_t = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32)
    check(host(yt), want_t, TOL_FP32, "gemm 1024 NT")
    y_tf32 = ops.MultiplyMatrixByMatrix(dev(a), dev(b), precision=ops.PREC_TF32)
    check(host(y_tf32), want, TOL_TF32, "gemm 1024 NN tf32")


@pytest.mark.parametrize("n", [4096, 8192])
def test_config5_gemm_large_by_random_projection(ops, n):
    """BASELINE config 5 (M = N = K = 4096 / 8192): the O(n^3) product is checked in O(n^2) on the host:
    (A B) v must equal A (B v) for random v (Freivalds), evaluated in float64; and rows sampled exactly."""
    rng = np.random.default_rng(500 + n)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    y = host(ops.MultiplyMatrixByMatrix(dev(a), dev(b)))
    a64 = a.astype(np.float64)
    for seed in range(3):
        v = np.random.default_rng(seed).uniform(-1, 1, (n,))
        want = a64 @ (b.astype(np.float64) @ v)
        got = y.astype(np.float64) @ v
        assert np.max(np.abs(got - want)) / np.sqrt(np.mean(want ** 2)) < TOL_FP32, f"projection {seed}"
    rows = rng.integers(0, n, 8)
    want_rows = (a64[rows] @ b.astype(np.float64)).astype(np.float32)
    check(y[rows], want_rows, TOL_FP32, f"gemm {n} sampled rows")


def test_config2_mobilenetv2_block_full_size(ops, reference):
    """BASELINE config 2 at its own size (64x56x56x32, expand 192, ReLU6, residual) against the reference CPU engine."""
    rng = np.random.default_rng(222)
    n, hw, c_in, c_exp = 64, 56, 32, 192
    x = rng.uniform(0, 1, (n, hw, hw, c_in)).astype(np.float32)
    w_exp = (rng.standard_normal((c_exp, c_in)) * np.sqrt(2.0 / c_in)).astype(np.float32)
    w_dw = (rng.standard_normal((3, 3, c_exp)) * np.sqrt(2.0 / 9)).astype(np.float32)
    w_down = (rng.standard_normal((c_in, c_exp)) * np.sqrt(2.0 / c_exp)).astype(np.float32)
    b_exp, b_dw = rng.uniform(-0.1, 0.1, c_exp).astype(np.float32), rng.uniform(-0.1, 0.1, c_exp).astype(np.float32)
    b_down = rng.uniform(-0.1, 0.1, c_in).astype(np.float32)
    want = reference.mobilenetv2_block(x, w_exp, b_exp, w_dw, b_dw, w_down, b_down, stride=1, residual=True)
    got = ops.MobileNetV2Block(dev(x), dev(w_exp), dev(b_exp), dev(w_dw), dev(b_dw), dev(w_down), dev(b_down),
                               stride=1, residual=True)
    check(host(got), want, TOL_FP32, "config2 block vs reference CPU engine")


def test_gather_kernel_agrees_with_the_tma_kernel(ops):
    """Shapes that normally ride on TMA, pushed through the cp.async gather instantiation (diagnostic option 16): the
    K order of the accumulation is the same, so the two kernels must agree bit for bit."""
    from neoml_b200 import _capi
    lib = _capi.load()
    x, f, b = dev(cases.uniform(61, (3, 20, 20, 64))), dev(cases.uniform(62, (80, 3, 3, 64))), dev(cases.uniform(63, (80,)))
    a, w = dev(cases.uniform(64, (300, 160))), dev(cases.uniform(65, (72, 160)))
    lib.nb200_debug_set_contraction_trace(None, 0, 32)   # one work item per tile in both kernels (the gather one never splits K)
    try:
        want_conv = ops.BlobConvolution(x, f, b, padding=(1, 1), act=ops.ACT_RELU)
        want_mmt = ops.MultiplyMatrixByTransposedMatrix(a, w)
        torch.cuda.synchronize()
        lib.nb200_debug_set_contraction_trace(None, 0, 16)
        got_conv = ops.BlobConvolution(x, f, b, padding=(1, 1), act=ops.ACT_RELU)
        got_mmt = ops.MultiplyMatrixByTransposedMatrix(a, w)
        torch.cuda.synchronize()
    finally:
        lib.nb200_debug_set_contraction_trace(None, 0, 0)
    assert torch.equal(got_conv, want_conv)
    assert torch.equal(got_mmt, want_mmt)


def test_split_k_convolutions(ops, oracle):
    """Few-tile convolutions cut their K loop into parts that run on otherwise idle SMs and are summed in a fixed
    order by a finishing pass: same answer as the oracle, the same bits on every run, and within rounding of the
    unsplit launch (diagnostic option 32) with bias, residual and every activation."""
    from neoml_b200 import _capi
    lib = _capi.load()
    shapes = [((1, 14, 14, 256), (64, 3, 3, 256), 1, 1),     # 2 tiles, 72 K blocks
              ((1, 7, 7, 512), (512, 1, 1, 512), 0, 1),      # pointwise, 1 x 4 tiles, 16 K blocks
              ((2, 9, 11, 96), (40, 5, 5, 96), 2, 2),        # ragged M and N, stride 2
              ((4, 28, 28, 128), (128, 3, 3, 128), 1, 1)]    # 25 tiles: a small split
    for i, (xs, fs, pad, stride) in enumerate(shapes):
        x, f, b = cases.uniform(400 + i, xs), cases.uniform(410 + i, fs) * 0.2, cases.uniform(420 + i, (fs[0],))
        want = oracle.blob_convolution(x, f, b, padding=(pad, pad), stride=(stride, stride))
        res = cases.uniform(430 + i, want.shape)
        dx, df, db, dres = dev(x), dev(f), dev(b), dev(res)
        for act, param, post in [(ops.ACT_NONE, 0.0, lambda v: v), (ops.ACT_RELU, 0.0, lambda v: np.maximum(v, 0)),
                                 (ops.ACT_RELU, 1.5, lambda v: np.clip(v, 0, 1.5)),
                                 (ops.ACT_HSWISH, 0.0, lambda v: v * np.clip(v + 3, 0, 6) / 6)]:
            launches = lib.nb200_launch_count()
            got = ops.BlobConvolution(dx, df, db, padding=(pad, pad), stride=(stride, stride), act=act, act_param=param,
                                      residual=dres)
            again = ops.BlobConvolution(dx, df, db, padding=(pad, pad), stride=(stride, stride), act=act, act_param=param,
                                        residual=dres)
            torch.cuda.synchronize()
            # contraction + the finishing pass that only a split launch has, behind the filter preparation that
            # convolutions with at least 1024 output positions get
            prepared = want.shape[0] * want.shape[1] * want.shape[2] >= 1024
            assert lib.nb200_launch_count() - launches == 2 * (2 + prepared), f"shape {i} did not split"
            assert torch.equal(got, again), f"shape {i}: split results differ between runs"
            check(host(got), post((want + res).astype(np.float64)).astype(np.float32), TOL_FP32, f"split conv {i} act {act}/{param}")
            lib.nb200_debug_set_contraction_trace(None, 0, 32)
            try:
                unsplit = ops.BlobConvolution(dx, df, db, padding=(pad, pad), stride=(stride, stride), act=act,
                                              act_param=param, residual=dres)
                torch.cuda.synchronize()
            finally:
                lib.nb200_debug_set_contraction_trace(None, 0, 0)
            # not tighter: the shorter accumulation chains of the parts are the more accurate of the two
            check(host(got), host(unsplit), TOL_FP32, f"split vs unsplit {i}")


def test_matrix_products_with_work_space(ops, oracle):
    """MultiplyMatrixByTransposedMatrix with scratch: the second operand is split once per call (tall products; the
    same bits as the in-kernel split), few-tile products split their K loop (classifier at small batch); batched
    and strided forms included."""
    from neoml_b200 import _capi
    lib = _capi.load()
    # tall, unsplit: prepared operand, bit-identical to the in-kernel conversion
    for (m, k, n) in [(1500, 160, 72), (1040, 96, 200)]:
        a, b = cases.uniform(500 + m, (m, k)), cases.uniform(501 + m, (n, k))
        da, db = dev(a), dev(b)
        launches = lib.nb200_launch_count()
        with_ws = ops.MultiplyMatrixByTransposedMatrix(da, db)
        assert lib.nb200_launch_count() - launches == 2          # preparation + product
        plain = ops.MultiplyMatrixByTransposedMatrix(da, db, use_scratch=False)
        assert torch.equal(with_ws, plain)
        check(host(with_ws), oracle.multiply_matrix_by_transposed_matrix(a, b), TOL_FP32, f"mmt with scratch {m}x{k}x{n}")
    # strided operands inside larger buffers
    m, k, n, lda, ldb, ldc = 1100, 64, 40, 80, 72, 48
    a, b = cases.uniform(520, (m, lda)), cases.uniform(521, (n, ldb))
    got = ops.MultiplyMatrixByTransposedMatrix(dev(a), dev(b), first_width=k, second_height=n, first_row_size=lda,
                                               second_row_size=ldb, result_row_size=ldc)
    check(host(got)[:, :n], oracle.multiply_matrix_by_transposed_matrix(a[:, :k].copy(), b[:, :k].copy()), TOL_FP32,
          "strided mmt with scratch")
    # few tiles, long K: split K (a classifier layer at batch 1 and 8), with bias
    for (m, k, n) in [(1, 2048, 1000), (8, 2048, 1000), (200, 1024, 256)]:
        a, b, bias = cases.uniform(530 + m, (m, k)), cases.uniform(531 + m, (n, k)) * 0.1, cases.uniform(532 + m, (n,))
        da, db, dbias = dev(a), dev(b), dev(bias)
        launches = lib.nb200_launch_count()
        got = ops.MultiplyMatrixByTransposedMatrix(da, db, free_term=dbias)
        assert lib.nb200_launch_count() - launches == 2          # product in K parts + finishing pass
        again = ops.MultiplyMatrixByTransposedMatrix(da, db, free_term=dbias)
        assert torch.equal(got, again)
        check(host(got), oracle.multiply_matrix_by_transposed_matrix(a, b) + bias, TOL_FP32, f"split mmt {m}x{k}x{n}")
    # batched, tall: prepared operand per batch entry
    bsz, m, k, n = 3, 1024, 64, 96
    a, b = cases.uniform(540, (bsz, m, k)), cases.uniform(541, (bsz, n, k))
    with_ws = ops.BatchMultiplyMatrixByTransposedMatrix(dev(a), dev(b))
    plain = ops.BatchMultiplyMatrixByTransposedMatrix(dev(a), dev(b), use_scratch=False)
    assert torch.equal(with_ws, plain)
    for i in range(bsz):
        check(host(with_ws)[i], oracle.multiply_matrix_by_transposed_matrix(a[i], b[i]), TOL_FP32, f"batched mmt {i}")


@pytest.mark.parametrize("stride", [1, 2])
def test_channelwise_convolution_large_images(ops, oracle, stride):
    """Depthwise 3x3 on images large enough for the TMA-staged kernel (tiles of 32 channels; here 144 channels leave a
    half-filled last tile, 57 x 45 pixels leave ragged tiles on both axes) and for the row-block kernel."""
    for i, (n, h, w, c) in enumerate([(16, 57, 45, 144), (40, 30, 29, 64), (3, 120, 130, 32)]):
        x, f, b = cases.uniform(600 + i, (n, h, w, c)), cases.uniform(610 + i, (3, 3, c)), cases.uniform(620 + i, (c,))
        want = oracle.blob_channelwise_convolution(x, f, b, padding=(1, 1), stride=(stride, stride))
        for act, param, post in [(ops.ACT_NONE, 0.0, lambda v: v), (ops.ACT_RELU, 6.0, lambda v: np.clip(v, 0, 6)),
                                 (ops.ACT_HSWISH, 0.0, lambda v: v * np.clip(v + 3, 0, 6) / 6)]:
            got = ops.BlobChannelwiseConvolution(dev(x * 4), dev(f), dev(b), padding=(1, 1), stride=(stride, stride),
                                                 act=act, act_param=param)
            want4 = oracle.blob_channelwise_convolution(x * 4, f, b, padding=(1, 1), stride=(stride, stride))
            check(host(got), post(want4.astype(np.float64)).astype(np.float32), TOL_FP32, f"depthwise {i} stride {stride} act {act}")
        assert want.shape == host(got).shape


def test_short_k_kernels_and_launch_timing(ops, oracle):
    """Contractions of at most four K blocks run on the short-K kernels (cross products added into the main
    accumulator, residual through a shared-memory ring, B resident for one or two K blocks); diagnostic option 128
    sends the same call to the general kernels.  Both must hold the fp32 bar, and differ only in the last bits.  The
    library's launch timing reports one duration per contraction launch."""
    from neoml_b200 import _capi
    import ctypes
    lib = _capi.load()
    shapes = [((6, 40, 40, 64), 256, True),      # K = 64: resident B, 2 column tiles, residual
              ((5, 28, 28, 128), 512, True),     # K = 128: ring without residency
              ((6, 40, 40, 32), 192, False),     # one K block, N = 192 (96-wide tiles)
              ((3, 17, 19, 96), 40, True)]       # ragged rows and columns
    lib.nb200_debug_time_contractions(1)
    launches = 0
    for i, (xs, k, with_res) in enumerate(shapes):
        x, f, b = cases.uniform(700 + i, xs), cases.uniform(710 + i, (k, 1, 1, xs[3])) * 0.3, cases.uniform(720 + i, (k,))
        want = oracle.blob_convolution(x, f, b)
        res = cases.uniform(730 + i, want.shape) if with_res else None
        ref = np.maximum(want + (res if with_res else 0), 0)
        dx, df, db, dres = dev(x), dev(f), dev(b), dev(res) if with_res else None
        short = ops.BlobConvolution(dx, df, db, residual=dres, act=ops.ACT_RELU)
        lib.nb200_debug_set_contraction_trace(None, 0, 128)
        try:
            general = ops.BlobConvolution(dx, df, db, residual=dres, act=ops.ACT_RELU)
            torch.cuda.synchronize()
        finally:
            lib.nb200_debug_set_contraction_trace(None, 0, 0)
        launches += 2
        check(host(short), ref, TOL_FP32, f"short-K {i}")
        check(host(general), ref, TOL_FP32, f"general {i}")
        check(host(short), host(general), 2e-5, f"short-K vs general {i}")
    lib.nb200_debug_time_contractions(0)
    times = (ctypes.c_float * 64)()
    n = lib.nb200_debug_contraction_times(ctypes.cast(times, ctypes.c_void_p), 64)
    assert n == launches
    assert all(0.0 < times[i] < 50.0 for i in range(n))      # milliseconds


def test_vectorised_helper_variants(ops, oracle):
    """The 16-byte forms of row sums, the channel-vector transpose and the strip max-pool against the oracle."""
    for (bsz, h, w) in [(3, 49, 2048), (1, 700, 260), (2, 5, 4)]:     # the second splits its rows over slices
        m = cases.uniform(71, (bsz * h * w,))
        assert gate_err(host(ops.SumMatrixRows(bsz, dev(m), h, w)), oracle.sum_matrix_rows(bsz, m, h, w)) < 1e-5
        init = cases.uniform(72, (bsz, w))
        assert gate_err(host(ops.SumMatrixRows(bsz, dev(m), h, w, result=dev(init), add=True)),
                        oracle.sum_matrix_rows(bsz, m, h, w, init)) < 1e-5
    for (b, h, mm, w, c) in [(2, 48, 1, 12, 64), (2, 5, 3, 7, 8), (1, 9, 1, 1, 4)]:
        t = cases.uniform(73, (b * h * mm * w * c,))
        assert np.array_equal(host(ops.TransposeMatrix(b, dev(t), h, mm, w, c)), oracle.transpose_matrix(b, t, h, mm, w, c))
    for shape in [(2, 23, 31, 8), (1, 7, 9, 64), (3, 3, 3, 4)]:          # odd sizes: partial strips at the right edge
        x = cases.uniform(74, shape)
        assert np.array_equal(host(ops.BlobMaxPooling(dev(x), (3, 3), (2, 2))), oracle.blob_max_pooling(x, (3, 3), (2, 2))[0])


def _attention_reference(q, kt, v, scale, mask):
    import torch
    s = torch.matmul(q.double(), kt.double())
    if scale is not None:
        s = s * float(scale)
    if mask is not None:
        s = s + mask.double()
    return torch.matmul(torch.softmax(s, dim=-1), v.double())


@pytest.mark.parametrize("case", [
    (3, 128, 128, False, 1.0), (2, 256, 384, True, 1.0), (2, 200, 260, True, 1.0), (5, 512, 512, True, 1.0),
    (2, 128, 512, False, 40.0),      # later key blocks dominate: the running reference of the softmax has to move
])
def test_attention_chain_as_one_kernel(ops, case):
    """softmax(scale * Q Kt + mask) V against a float64 evaluation: the same gate as the separate calls (1e-4 of the
    result's RMS).  The mask is NeoML's: -1e9 where a key is hidden (here: the causal triangle)."""
    import torch
    b, sq, st, masked, growth = case
    d = 64
    q = dev(cases.uniform(81, (b, sq, d)))
    kt = dev(cases.uniform(82, (b, d, st)))
    v = dev(cases.uniform(83, (b, st, d)))
    if growth != 1.0:
        kt[:, :, st // 2:] *= growth                       # scores of the second half are up to 40 x larger
    scale = torch.tensor([0.125], dtype=torch.float32, device="cuda")
    mask = None
    if masked:
        mask = torch.triu(torch.full((sq, st), -1e9, dtype=torch.float32, device="cuda"), diagonal=1 + max(st - sq, 0))
    got = ops.AttentionScoresValues(q, kt, v, scale=scale, mask=mask)
    want = _attention_reference(q, kt, v, 0.125, mask)
    torch.cuda.synchronize()
    assert ops.capi.load().nb200_device_status(None, 0) == 0
    err = (got.double() - want).abs().max() / want.pow(2).mean().sqrt()
    assert float(err) < 1e-4, float(err)
    # the engine's separate calls give the same to the same gate
    s = ops.MultiplyMatrixByMatrix(q, kt)
    s = s * 0.125 + (mask if mask is not None else 0.0)
    chain = ops.MultiplyMatrixByMatrix(torch.softmax(s, dim=-1).contiguous(), v)
    err_chain = (chain.double() - want).abs().max() / want.pow(2).mean().sqrt()
    assert float(err) < max(4.0 * float(err_chain), 2e-5), (float(err), float(err_chain))


def test_attention_chain_many_items_per_cta_is_exact_and_repeatable(ops):
    """Configuration 4's size (768 heads x 512 x 512): every CTA walks some twenty items, buffers are handed from one
    item to the next.  Three runs give the same bits, and every item meets the gate against float64."""
    import torch
    b, sq, st, d = 768, 512, 512, 64
    gen = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(b, sq, d, device="cuda", generator=gen)
    kt = torch.randn(b, d, st, device="cuda", generator=gen) * 0.3
    v = torch.randn(b, st, d, device="cuda", generator=gen)
    scale = torch.full((1,), 0.125, device="cuda")
    for mask in (None, torch.triu(torch.full((sq, st), -1e9, device="cuda"), diagonal=1)):
        runs = [ops.AttentionScoresValues(q, kt, v, scale=scale, mask=mask) for _ in range(3)]
        torch.cuda.synchronize()
        assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])
        worst = 0.0
        for i0 in range(0, b, 64):
            want = _attention_reference(q[i0:i0 + 64], kt[i0:i0 + 64], v[i0:i0 + 64], 0.125, mask)
            err = (runs[0][i0:i0 + 64].double() - want).abs().reshape(64 * 4, -1).amax(-1) / want.pow(2).mean().sqrt()
            worst = max(worst, float(err.max()))
        assert worst < 1e-4, worst


def test_attention_chain_refuses_what_it_does_not_cover(ops):
    import torch
    q = torch.zeros((1, 128, 32), device="cuda")
    kt = torch.zeros((1, 32, 128), device="cuda")
    with pytest.raises(Exception):
        ops.AttentionScoresValues(q, kt, q)                # depth 32: the separate calls are the way


def test_product_with_a_prepared_second_operand_equals_the_plain_call(ops):
    """nb200_multiply_matrix_by_transposed_matrix_prepared against the call that prepares per call: the same bits, with
    bias in the epilogue, for both precisions; short products report that they use no prepared operand."""
    import ctypes as C
    lib = ops.capi.load()
    ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    assert lib.nb200_matrix_product_prepared_floats(512, 96, 64, 64) == 0
    for m, k, n, prec in [(2048, 192, 160, ops.PREC_3XTF32), (1024, 64, 256, ops.PREC_TF32), (1500, 96, 100, ops.PREC_3XTF32)]:
        a, b, bias = dev(cases.uniform(96, (m, k))), dev(cases.uniform(97, (n, k))), dev(cases.uniform(98, (n,)))
        want = ops.MultiplyMatrixByTransposedMatrix(a, b, free_term=bias, precision=prec)
        floats = lib.nb200_matrix_product_prepared_floats(m, n, k, k)
        assert floats >= n * k
        prepared = torch.empty(floats, device="cuda")
        ops.capi.check("prepare", lib.nb200_matrix_product_prepare_second(None, ptr(b), n, k, k, ptr(prepared), prec))
        scratch = torch.empty(lib.nb200_matrix_product_scratch_floats(1, m, n, k, k) + 16, device="cuda")
        got = torch.full((m, n), float("nan"), device="cuda")
        epi = ops.capi.Epilogue(bias.data_ptr(), None, 0, ops.ACT_NONE, 0.0, 0, None)
        for _ in range(2):      # the prepared operand serves any number of calls
            ops.capi.check("product", lib.nb200_multiply_matrix_by_transposed_matrix_prepared(
                None, ptr(a), m, k, k, ptr(b), n, k, ptr(got), n, ptr(prepared), ptr(scratch), C.byref(epi), prec))
            torch.cuda.synchronize()
            assert torch.equal(got, want), (m, k, n, prec)


def test_normalisation_passes_equal_the_separate_calls(ops):
    """nb200_sum_matrix_columns_shifted and nb200_matrix_rows_cols_affine against the calls they stand for, bit for bit."""
    import ctypes as C
    lib = ops.capi.load()
    ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    for rows, width in [(5, 7), (64, 768), (33, 100)]:
        x = dev(cases.uniform(91, (rows, width)))
        a, b = dev(cases.uniform(92, (rows,))), dev(cases.uniform(93, (rows,), 0.5, 1.5))
        c, d = dev(cases.uniform(94, (width,), 0.5, 1.5)), dev(cases.uniform(95, (width,)))
        shifted = ops.AddVectorToMatrixColumns(x.reshape(-1), a, rows, width)
        squared = ops.vector_op("ELTWISE_MUL", shifted.reshape(-1), shifted.reshape(-1))
        for square, src in ((0, shifted), (1, squared)):
            got = torch.empty(rows, device="cuda")
            ops.capi.check("sum", lib.nb200_sum_matrix_columns_shifted(None, ptr(got), ptr(x), rows, width, ptr(a), square))
            assert torch.equal(got, ops.SumMatrixColumns(src.reshape(-1), rows, width))
        want = ops.MultiplyDiagMatrixByMatrix(b, shifted.reshape(-1), rows, width)
        want = ops.BatchMultiplyMatrixByDiagMatrix(1, want, rows, width, c, 0)
        want = ops.AddVectorToMatrixRows(1, want, d, rows, width)
        got = torch.empty(rows * width, device="cuda")
        ops.capi.check("affine", lib.nb200_matrix_rows_cols_affine(None, ptr(x), rows, width, ptr(a), 0, ptr(b), ptr(c), ptr(d), ptr(got)))
        torch.cuda.synchronize()
        assert torch.equal(got.reshape(-1), want.reshape(-1))


def test_padded_max_pool_equals_resize_then_pool(ops, oracle):
    """One pass over the unpadded image against BlobResizeImage followed by BlobMaxPooling on the oracle: bit-exact,
    including a border value above the data (it then wins at the edges) and uneven borders."""
    for shape, deltas, value in [((2, 23, 31, 8), (1, 1, 1, 1), 0.0), ((1, 8, 8, 64), (1, 1, 1, 1), 5.0),
                                 ((3, 7, 9, 4), (2, 0, 1, 3), -1.0), ((1, 112, 112, 64), (1, 1, 1, 1), 0.0)]:
        x = cases.uniform(75, shape)
        padded = oracle.blob_resize_image(x, *deltas, 0, value)
        want = oracle.blob_max_pooling(padded, (3, 3), (2, 2))[0]
        assert np.array_equal(host(ops.BlobMaxPoolingPadded(dev(x), deltas, value, (3, 3), (2, 2))), want)


def test_blob_convolution_random_shapes(ops, oracle):
    """Seeded random geometries against the plain-C oracle (120 by default, NB200_RANDOM_CASES sets another count:
    9 000 of them with another seed have been run, worst gate error 2.6e-5): channel counts on both sides of every
    path switch (row windows below 32 channels, im2col boxes at multiples of 32, gathers elsewhere), filters up to
    7x7, strides, dilations and paddings up to the filter size, one to eight images of up to 46 x 46 pixels, with
    and without free term, ReLU and residual, with and without caller scratch."""
    rng = np.random.default_rng(int(os.environ.get("NB200_RANDOM_SEED", "20240607")))
    channel_pool = [1, 2, 3, 4, 5, 7, 8, 12, 16, 24, 31, 32, 33, 48, 64, 96, 128, 160, 256]
    worst = 0.0
    for case in range(int(os.environ.get("NB200_RANDOM_CASES", "120"))):
        c = int(rng.choice(channel_pool))
        k = int(rng.choice([1, 3, 8, 16, 31, 32, 33, 64, 72, 96, 128, 130, 192, 256, 300]))
        r, s = int(rng.integers(1, 8)), int(rng.integers(1, 8))
        if c > 64:
            r, s = min(r, 3), min(s, 3)
        dil = (int(rng.integers(1, 3)), int(rng.integers(1, 3)))
        stride = (int(rng.integers(1, 4)), int(rng.integers(1, 4)))
        pad = (int(rng.integers(0, r)), int(rng.integers(0, s)))          # below the filter size: see cases.py on the reference
        h = int(rng.integers((r - 1) * dil[0] + 1, (r - 1) * dil[0] + 40))
        w = int(rng.integers((s - 1) * dil[1] + 1, (s - 1) * dil[1] + 40))
        n = int(rng.integers(1, 9))
        if n * h * w * c * k * r * s > 6e8:   # keeps the oracle's share of a case below a second
            continue
        x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
        f = rng.uniform(-1, 1, (k, r, s, c)).astype(np.float32)
        b = rng.uniform(-1, 1, (k,)).astype(np.float32) if rng.random() < 0.7 else None
        want = oracle.blob_convolution(x, f, b, padding=pad, stride=stride, dilation=dil)
        relu, with_res = bool(rng.random() < 0.5), bool(rng.random() < 0.4)
        res = rng.uniform(-1, 1, want.shape).astype(np.float32) if with_res else None
        if with_res:
            want = want + res
        if relu:
            want = np.maximum(want, 0.0)
        for scratch in (True, False):
            got = host(ops.BlobConvolution(dev(x), dev(f), dev(b), padding=pad, stride=stride, dilation=dil, residual=dev(res),
                                           act=ops.ACT_RELU if relu else ops.ACT_NONE, use_scratch=scratch))
            err = gate_err(got, want) if got.shape == want.shape else float("inf")
            worst = max(worst, err)
            assert err < TOL_FP32, \
                f"case {case}: n={n} h={h} w={w} c={c} k={k} r={r} s={s} pad={pad} stride={stride} dil={dil} relu={relu} " \
                f"res={with_res} scratch={scratch}: {err:.3e}"
    print(f"random convolutions: worst gate error {worst:.3e}")


def test_matrix_products_random_shapes(ops, oracle):
    """Forty seeded random products with row strides wider than the matrices, both orientations, batched."""
    rng = np.random.default_rng(777)
    for case in range(40):
        m, k, n = int(rng.integers(1, 300)), int(rng.integers(1, 300)), int(rng.integers(1, 300))
        lda, ldb = k + int(rng.integers(0, 9)), k + int(rng.integers(0, 9))
        a = rng.uniform(-1, 1, (m, lda)).astype(np.float32)
        b = rng.uniform(-1, 1, (n, ldb)).astype(np.float32)
        want = oracle.multiply_matrix_by_transposed_matrix(a, b, m=m, k=k, n=n, lda=lda, ldb=ldb)
        got = host(ops.MultiplyMatrixByTransposedMatrix(dev(a), dev(b), first_height=m, first_width=k, second_height=n,
                                                        first_row_size=lda, second_row_size=ldb))
        assert gate_err(got, want) < TOL_FP32, f"mmt case {case}: m={m} k={k} n={n} lda={lda} ldb={ldb}"
        batch = int(rng.integers(1, 4))
        a3 = rng.uniform(-1, 1, (batch, m, k)).astype(np.float32)
        b3 = rng.uniform(-1, 1, (batch, k, n)).astype(np.float32)
        want3 = oracle.multiply_matrix_by_matrix(a3, b3)
        for scratch in (True, False):
            got3 = host(ops.MultiplyMatrixByMatrix(dev(a3), dev(b3), use_scratch=scratch))
            assert gate_err(got3, want3) < TOL_FP32, f"mm case {case}: batch={batch} m={m} k={k} n={n} scratch={scratch}"


def test_forced_gather_on_a_few_channel_convolution_stays_inside_its_scratch():
    """The 3-channel stem shape with the gather kernel forced (diagnostic option 16): the row-window path must step
    aside BEFORE it writes anything, the channel-padding path then runs inside the caller's scratch; a guard region
    behind the scratch stays untouched and the result equals the one computed without scratch."""
    import ctypes as C
    from neoml_b200 import _capi, ops as O
    lib = _capi.load()
    n, h, w, c, k = 2, 37, 41, 3, 64
    ho, wo = O.conv_output_size(h, 7, 3, 2, 1), O.conv_output_size(w, 7, 3, 2, 1)
    desc = _capi.ConvDesc(n, h, w, c, k, 7, 7, 3, 3, 2, 2, 1, 1, ho, wo)
    need = lib.nb200_blob_convolution_scratch_floats(C.byref(desc))
    guard = 1 << 16
    sentinel = 12345.0
    buf = torch.full((need + guard,), sentinel, dtype=torch.float32, device="cuda")
    x, f, b = dev(cases.uniform(71, (n, h, w, c))), dev(cases.uniform(72, (k, 7, 7, c))), dev(cases.uniform(73, (k,)))
    epi = _capi.Epilogue(b.data_ptr(), None, 0, O.ACT_RELU, 0.0, 0)
    got = torch.empty((n, ho, wo, k), dtype=torch.float32, device="cuda")
    want = torch.empty_like(got)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    lib.nb200_debug_set_contraction_trace(None, 0, 16)
    try:
        _capi.check("BlobConvolution", lib.nb200_blob_convolution(stream, C.byref(desc), C.c_void_p(x.data_ptr()),
                    C.c_void_p(f.data_ptr()), C.c_void_p(got.data_ptr()), C.c_void_p(buf.data_ptr()), C.byref(epi), O.PREC_3XTF32))
        _capi.check("BlobConvolution", lib.nb200_blob_convolution(stream, C.byref(desc), C.c_void_p(x.data_ptr()),
                    C.c_void_p(f.data_ptr()), C.c_void_p(want.data_ptr()), None, C.byref(epi), O.PREC_3XTF32))
        torch.cuda.synchronize()
    finally:
        lib.nb200_debug_set_contraction_trace(None, 0, 0)
    assert bool((buf[need:] == sentinel).all()), "the call wrote past the scratch it was given"
    assert lib.nb200_device_status(stream, 0) == 0
    # two gather instantiations (16-byte pieces over widened pixels / single floats): same products, another order
    assert gate_err(got.cpu().numpy(), want.cpu().numpy()) < 1e-5


def test_sliced_row_sums_are_the_same_bits_on_every_run(ops, oracle):
    """Tall, narrow matrices split their rows over a thread-block cluster; the slices are added in a fixed order
    (distributed shared memory, no atomics), so repeated runs agree bit for bit."""
    for bsz, h, w in ((1, 20000, 64), (2, 4096, 37), (3, 1000, 128)):
        m = cases.uniform(81, (bsz * h * w,))
        md = dev(m)
        first = ops.SumMatrixRows(bsz, md, h, w)
        assert gate_err(host(first), oracle.sum_matrix_rows(bsz, m, h, w)) < 1e-5
        for _ in range(5):
            assert torch.equal(ops.SumMatrixRows(bsz, md, h, w), first)
        init = cases.uniform(82, (bsz * w,))
        acc = ops.SumMatrixRows(bsz, md, h, w, result=dev(init), add=True)
        assert gate_err(host(acc), oracle.sum_matrix_rows(bsz, m, h, w) + init.reshape(bsz, w)) < 1e-5


FUSED_MBV2 = [
    # batch, h, w, c_exp, c_out, residual, act1 (kind, param), act2, biases -- all with 32 input channels and stride 1:
    # the shapes the one-kernel form of the block covers (ragged tiles, every chunk count, both activations)
    (2, 8, 16, 32, 32, True, (1, 6.0), (1, 6.0), (True, True, True)),       # exactly one tile per image
    (1, 19, 23, 96, 32, True, (1, 6.0), (1, 6.0), (True, True, True)),      # ragged in both directions
    (3, 9, 33, 192, 32, True, (1, 0.0), (2, 0.0), (True, False, True)),     # ReLU without threshold, HSwish
    (2, 17, 5, 64, 16, False, (2, 0.0), (1, 6.0), (False, True, False)),    # narrower than a tile, 16 outputs
    (1, 24, 40, 96, 64, False, (1, 6.0), (1, 6.0), (True, True, True)),     # 64 outputs, three chunks
    (5, 14, 14, 96, 48, False, (1, 6.0), (1, 6.0), (True, True, True)),     # 48 outputs
]


@pytest.mark.parametrize("shape", FUSED_MBV2, ids=lambda s: "x".join(map(str, s[:5])))
@pytest.mark.parametrize("prec,tol", [(0, TOL_FP32), (1, TOL_TF32)], ids=["3xtf32", "tf32"])
def test_fused_mobilenetv2_block(ops, oracle, shape, prec, tol):
    b, h, w, ce, co, res, (a1, p1), (a2, p2), biases = shape
    seed = 8800 + 7 * FUSED_MBV2.index(shape)
    x = cases.uniform(seed, (b, h, w, 32), 0.0, 1.0)
    we = cases.normal(seed + 1, (ce, 32), float(np.sqrt(2.0 / 32)))
    wd = cases.normal(seed + 2, (3, 3, ce), float(np.sqrt(2.0 / 9)))
    wp = cases.normal(seed + 3, (co, ce), float(np.sqrt(2.0 / ce)))
    be = cases.uniform(seed + 4, (ce,), -0.1, 0.1) if biases[0] else None
    bd = cases.uniform(seed + 5, (ce,), -0.1, 0.1) if biases[1] else None
    bp = cases.uniform(seed + 6, (co,), -0.1, 0.1) if biases[2] else None
    kw = dict(stride=1, residual=res, act_exp=a1, act_exp_param=p1, act_dw=a2, act_dw_param=p2)
    want = oracle.mobilenetv2_block(x, we, be, wd, bd, wp, bp, **kw)
    from neoml_b200 import _capi
    lib = _capi.load()
    launches = lib.nb200_launch_count()
    y = ops.MobileNetV2Block(dev(x), dev(we), dev(be), dev(wd), dev(bd), dev(wp), dev(bp), stride=1, residual=res,
                             expand_act=a1, expand_act_param=p1, channelwise_act=a2, channelwise_act_param=p2,
                             precision=prec, one_kernel=True)
    got = host(y)
    assert lib.nb200_launch_count() - launches == 1, "the block did not run as one kernel"
    assert lib.nb200_device_status(None, 0) == 0
    check(got, want, tol, f"fused mbv2 {shape[:5]}")
    if res and prec == 0:
        # in place over the input, as NeoML calls it when it may: the result goes through the scratch
        xd = dev(x)
        ops.MobileNetV2Block(xd, dev(we), dev(be), dev(wd), dev(bd), dev(wp), dev(bp), result=xd, stride=1, residual=True,
                             expand_act=a1, expand_act_param=p1, channelwise_act=a2, channelwise_act_param=p2, one_kernel=True)
        assert np.array_equal(host(xd), got)


def test_mobilenetv2_block_random_shapes(ops, oracle):
    """Seeded random blocks against the plain-C oracle (80 by default, NB200_RANDOM_CASES sets another count; 7 700 with
    another seed have been run, worst gate error 8.8e-6): half of them in the shape class of the one-kernel form (32
    input channels, stride 1, up to 192 expanded and 64 output channels; where its shared memory does not hold the
    shape the three-launch form runs), half anywhere: images of 1 x 1 to 44 x 44 pixels, both strides, both
    activations with and without threshold, each free term present or not, the residual where the block allows one."""
    from neoml_b200 import _capi
    rng = np.random.default_rng(int(os.environ.get("NB200_RANDOM_SEED", "5150")))
    worst, one_kernel_runs = 0.0, 0
    for case in range(int(os.environ.get("NB200_RANDOM_CASES", "80"))):
        fused_class = case % 2 == 0
        b, h, w = int(rng.integers(1, 7)), int(rng.integers(1, 45)), int(rng.integers(1, 45))
        if fused_class:
            ci, stride = 32, 1
            ce, co = int(rng.choice([32, 64, 96, 128, 160, 192])), int(rng.choice([16, 32, 48, 64]))
        else:
            ci, stride = int(rng.choice([8, 16, 24, 32, 40, 64])), int(rng.choice([1, 2]))
            ce, co = int(rng.choice([16, 48, 96, 144, 192, 240])), int(rng.choice([8, 16, 24, 32, 64, 96]))
        res = bool(co == ci and stride == 1 and rng.random() < 0.6)
        a1 = (int(rng.choice([1, 2])), float(rng.choice([0.0, 6.0])))
        a2 = (int(rng.choice([1, 2])), float(rng.choice([0.0, 6.0])))
        x = rng.uniform(0, 1, (b, h, w, ci)).astype(np.float32)
        we = (rng.standard_normal((ce, ci)) * np.sqrt(2.0 / ci)).astype(np.float32)
        wd = (rng.standard_normal((3, 3, ce)) * np.sqrt(2.0 / 9)).astype(np.float32)
        wp = (rng.standard_normal((co, ce)) * np.sqrt(2.0 / ce)).astype(np.float32)
        be = rng.uniform(-0.1, 0.1, (ce,)).astype(np.float32) if rng.random() < 0.7 else None
        bd = rng.uniform(-0.1, 0.1, (ce,)).astype(np.float32) if rng.random() < 0.7 else None
        bp = rng.uniform(-0.1, 0.1, (co,)).astype(np.float32) if rng.random() < 0.7 else None
        want = oracle.mobilenetv2_block(x, we, be, wd, bd, wp, bp, stride=stride, residual=res, act_exp=a1[0],
                                        act_exp_param=a1[1], act_dw=a2[0], act_dw_param=a2[1])
        kw = dict(stride=stride, residual=res, expand_act=a1[0], expand_act_param=a1[1], channelwise_act=a2[0],
                  channelwise_act_param=a2[1])
        args = (dev(x), dev(we), dev(be), dev(wd), dev(bd), dev(wp), dev(bp))
        got = None
        if fused_class:
            try:
                got = host(ops.MobileNetV2Block(*args, one_kernel=True, **kw))
                one_kernel_runs += 1
            except _capi.Nb200Error:
                got = None                                   # the one-kernel form does not hold this shape
        if got is None:
            got = host(ops.MobileNetV2Block(*args, **kw))
        err = gate_err(got, want) if got.shape == want.shape else float("inf")
        worst = max(worst, err)
        assert err < TOL_FP32, f"case {case}: b={b} h={h} w={w} ci={ci} ce={ce} co={co} stride={stride} res={res} {a1} {a2}: {err:.3e}"
    assert _capi.load().nb200_device_status(None, 0) == 0
    print(f"random MobileNetV2 blocks: worst gate error {worst:.3e}, {one_kernel_runs} as one kernel")


def test_attention_chain_random_shapes(ops):
    """Seeded random attention shapes against a float64 evaluation (30 by default, NB200_RANDOM_CASES sets another
    count; 2 500 with NB200_RANDOM_SEED=77 have been run: worst 8.0e-5 of the result's RMS): 1 to 29 heads, 128 to 699 queries, 128 to 696 keys, no mask / the causal mask / a dense random mask, a scale
    of 0.05 to 0.25, and in three of ten cases keys whose second half is up to 40 x larger (the running reference of the
    softmax has to move)."""
    import torch
    rng = np.random.default_rng(int(os.environ.get("NB200_RANDOM_SEED", "31")))
    worst = 0.0
    for case in range(int(os.environ.get("NB200_RANDOM_CASES", "30"))):
        b, sq, st, d = int(rng.integers(1, 30)), int(rng.integers(128, 700)), 4 * int(rng.integers(32, 175)), 64
        q = dev(rng.uniform(-1, 1, (b, sq, d)).astype(np.float32))
        kt = dev(rng.uniform(-1, 1, (b, d, st)).astype(np.float32))
        v = dev(rng.uniform(-1, 1, (b, st, d)).astype(np.float32))
        grown = rng.random() < 0.3
        if grown:
            kt[:, :, st // 2:] *= float(rng.uniform(1, 40))
        # scores of a few hundred turn the 1e-6 of the 3xTF32 product into 1e-4 of a probability, in the separate calls
        # as in the kernel: with the large keys the scale stays at what a depth of 64 calls for
        factor = float(rng.uniform(0.05, 0.125 if grown else 0.25))
        scale = torch.tensor([factor], dtype=torch.float32, device="cuda")
        kind = rng.random()
        mask = None
        if kind < 0.35:
            mask = torch.triu(torch.full((sq, st), -1e9, dtype=torch.float32, device="cuda"), diagonal=1 + max(st - sq, 0))
        elif kind < 0.7:
            mask = dev(rng.uniform(-2, 2, (sq, st)).astype(np.float32))
        got = ops.AttentionScoresValues(q, kt, v, scale=scale, mask=mask)
        want = _attention_reference(q, kt, v, factor, mask)
        err = float((got.double() - want).abs().max() / want.pow(2).mean().sqrt())
        worst = max(worst, err)
        assert err < 1e-4, f"case {case}: heads={b} queries={sq} keys={st} mask kind {kind:.2f} scale {factor:.3f}: {err:.3e}"
    torch.cuda.synchronize()
    assert ops.capi.load().nb200_device_status(None, 0) == 0
    print(f"random attention shapes: worst {worst:.3e}")
