"""Pins the plain-C oracle: against the committed outputs of the reference's own CPU math engine
(tests/golden/reference_cpu_engine.npz) and, where oracle/_ref is built, against that engine live on the
operations that have no golden file.  CPU only."""
import numpy as np
import pytest

import cases
from oracle_lib import rel_err

# The oracle sums in double; the reference engine sums in fp32 in its own blocked order.  On outputs that cancel to
# ~0 the fp32 engine differs from the exact value by a few 1e-4 of (1e-3 x RMS), hence this bound for the pin.
PIN_TOL = 5e-4


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_conv_matches_reference(oracle, golden, name):
    x, f, b, kw = cases.conv_inputs(name)
    got = oracle.blob_convolution(x, f, b, **kw)
    want = golden[f"conv/{name}"]
    assert got.shape == want.shape
    assert rel_err(got, want) < PIN_TOL


@pytest.mark.parametrize("name", sorted(cases.MMT_CASES))
def test_mmt_matches_reference(oracle, golden, name):
    a, b, kw = cases.mmt_inputs(name)
    assert rel_err(oracle.multiply_matrix_by_transposed_matrix(a, b, **kw), golden[f"mmt/{name}"]) < PIN_TOL


@pytest.mark.parametrize("name", sorted(cases.MM_CASES))
def test_mm_matches_reference(oracle, golden, name):
    a, b = cases.mm_inputs(name)
    assert rel_err(oracle.multiply_matrix_by_matrix(a, b), golden[f"mm/{name}"]) < PIN_TOL


@pytest.mark.parametrize("name", sorted(cases.CHCONV_CASES))
def test_chconv_matches_reference(oracle, golden, name):
    x, f, b, kw = cases.chconv_inputs(name)
    assert rel_err(oracle.blob_channelwise_convolution(x, f, b, **kw), golden[f"chconv/{name}"]) < PIN_TOL


@pytest.mark.parametrize("name", sorted(cases.MBV2_CASES))
def test_mbv2_matches_reference(oracle, golden, name):
    args, kw = cases.mbv2_inputs(name)
    assert rel_err(oracle.mobilenetv2_block(*args, **kw), golden[f"mbv2/{name}"]) < PIN_TOL


@pytest.mark.parametrize("name", sorted(cases.SOFTMAX_CASES))
def test_softmax_matches_reference(oracle, golden, name):
    x, h, w = cases.softmax_inputs(name)
    assert rel_err(oracle.matrix_softmax_by_rows(x, h, w), golden[f"softmax/{name}"]) < 1e-5


def test_splitmix_known_answer():
    # first outputs of splitmix64 seeded with 0 (published test vector of the algorithm)
    z = cases.splitmix64(0, 3)
    assert [int(v) for v in z] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_vector_ops_live(oracle, reference):
    a = cases.uniform(11, (1001,), -4, 4)
    b = cases.uniform(12, (1001,), -4, 4)
    for op in range(19):
        a_ = np.abs(a) + 0.1 if op in (11, 12) else a
        b_ = np.abs(b) + 0.5 if op == 17 else b
        assert rel_err(oracle.vector_op(op, a_, b_, 0.7), reference.vector_op(op, a_, b_, 0.7)) < 1e-5, op


def test_matrix_helpers_live(oracle, reference):
    m = cases.uniform(21, (3 * 5 * 7,))
    v21, v15, v7 = cases.uniform(22, (21,)), cases.uniform(23, (15,)), cases.uniform(24, (7,))
    assert np.array_equal(oracle.add_vector_to_matrix_rows(3, m, 5, 7, v21), reference.add_vector_to_matrix_rows(3, m, 5, 7, v21))
    assert np.array_equal(oracle.add_vector_to_matrix_columns(m, 15, 7, v15), reference.add_vector_to_matrix_columns(m, 15, 7, v15))
    assert rel_err(oracle.sum_matrix_rows(3, m, 5, 7), reference.sum_matrix_rows(3, m, 5, 7)) < 1e-5
    init = cases.uniform(25, (3, 7))
    assert rel_err(oracle.sum_matrix_rows(3, m, 5, 7, init), reference.sum_matrix_rows(3, m, 5, 7, init)) < 1e-5
    assert rel_err(oracle.sum_matrix_columns(m, 15, 7), reference.sum_matrix_columns(m, 15, 7)) < 1e-5
    assert np.array_equal(oracle.multiply_diag_matrix_by_matrix(v15, 15, m, 7), reference.multiply_diag_matrix_by_matrix(v15, 15, m, 7))
    assert np.array_equal(oracle.multiply_matrix_by_diag_matrix(1, m, 15, 7, v7, 0), reference.multiply_matrix_by_diag_matrix(1, m, 15, 7, v7, 0))
    assert np.array_equal(oracle.multiply_matrix_by_diag_matrix(3, m, 5, 7, v21, 7), reference.multiply_matrix_by_diag_matrix(3, m, 5, 7, v21, 7))
    t = cases.uniform(26, (2 * 3 * 4 * 5 * 6,))
    assert np.array_equal(oracle.transpose_matrix(2, t, 3, 4, 5, 6), reference.transpose_matrix(2, t, 3, 4, 5, 6))
    am = cases.uniform(27, (13 * 37,))
    for fn in ("find_max_value_in_rows",):
        ov, oi = getattr(oracle, fn)(am, 13, 37)
        rv, ri = getattr(reference, fn)(am, 13, 37)
        assert np.array_equal(ov, rv) and np.array_equal(oi, ri)
    ov, oi = oracle.find_max_value_in_columns(2, am[:2 * 6 * 37], 6, 37)
    rv, ri = reference.find_max_value_in_columns(2, am[:2 * 6 * 37], 6, 37)
    assert np.array_equal(ov, rv) and np.array_equal(oi, ri)


def test_image_helpers_live(oracle, reference):
    x = cases.uniform(31, (2, 9, 11, 6))
    assert np.array_equal(oracle.blob_max_pooling(x, (3, 3), (2, 2))[0], reference.blob_max_pooling(x, (3, 3), (2, 2))[0])
    assert rel_err(oracle.blob_mean_pooling(x, (3, 2), (2, 1)), reference.blob_mean_pooling(x, (3, 2), (2, 1))) < 1e-5
    for pad in (0, 1, 2):
        assert np.array_equal(oracle.blob_resize_image(x, 1, 2, 2, 1, pad, 0.5), reference.blob_resize_image(x, 1, 2, 2, 1, pad, 0.5))
    assert np.array_equal(oracle.blob_resize_image(x, -1, -2, -2, 1, 0, 0.5), reference.blob_resize_image(x, -1, -2, -2, 1, 0, 0.5))


def test_reference_engine_roundtrip_through_the_shim(reference):
    """The engine-level shim calls (used on the GPU against the B200 engine) behave on the reference CPU engine."""
    x = cases.uniform(41, (1003,))
    y, (current, peak, pooled, pooled_after_cleanup) = reference.roundtrip(x)
    assert np.array_equal(y, 2 * x + 1)
    assert current >= 4 * x.size and peak >= current and pooled_after_cleanup == 0
    assert reference.info()[0] == 1      # MET_Cpu


def test_reference_engine_runs_the_rowwise_chain(reference):
    """The rowwise-chain driver of the shim on the reference CPU engine: shape and sanity of what the GPU test compares with."""
    import test_engine_gpu
    y = reference.rowwise_chain(*test_engine_gpu._rowwise_chain_inputs())
    assert y.shape == (2, 6, 5, 24) and np.isfinite(y).all() and float(np.abs(y).max()) > 0
