"""The C++ IMathEngine implementation (CB200MathEngine) exercised through real IMathEngine virtual calls.

The same C shim that drives the reference CPU engine (oracle/ref_shim.cpp) wraps device pointers into NeoML handles
and calls Init*/Blob*/Multiply*/... on the engine object created by the B200 factory; results are compared with the
reference CPU engine's committed outputs and the plain-C oracle.  Needs a B200 and oracle/_ref (for the shim and for
the libNeoMathEngine.so that provides IMathEngine's base-class symbols)."""
import numpy as np
import pytest
import torch

import cases
from oracle_lib import TOL_FP32, TOL_TF32, ShimmedB200Engine, gate_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine():
    assert torch.cuda.is_available()
    if not ShimmedB200Engine.available():
        pytest.skip("oracle/_ref or libNeoMathEngineB200.so not built")
    e = ShimmedB200Engine()
    yield e
    e.close()


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(e, t):
    e.sync()
    return t.cpu().numpy()


@pytest.mark.parametrize("name", sorted(cases.CONV_CASES))
def test_blob_convolution(engine, golden, name):
    x, f, b, kw = cases.conv_inputs(name)
    # the engine may hold the convolution back until the next call that touches data: like the blobs of a network, the
    # operands stay alive until the result has been read
    dx, df, db = dev(x), dev(f), dev(b)
    y = engine.blob_convolution(dx, df, db, **kw)
    assert gate_err(host(engine, y), golden[f"conv/{name}"]) < TOL_FP32


@pytest.mark.parametrize("name", sorted(cases.MMT_CASES))
def test_multiply_matrix_by_transposed_matrix(engine, golden, name):
    a, b, kw = cases.mmt_inputs(name)
    y = engine.multiply_matrix_by_transposed_matrix(dev(a), dev(b), **kw)
    assert gate_err(host(engine, y), golden[f"mmt/{name}"]) < TOL_FP32


@pytest.mark.parametrize("name", sorted(cases.MM_CASES))
def test_multiply_matrix_by_matrix(engine, golden, name):
    a, b = cases.mm_inputs(name)
    y = engine.multiply_matrix_by_matrix(dev(a), dev(b))
    assert gate_err(host(engine, y), golden[f"mm/{name}"]) < TOL_FP32


@pytest.mark.parametrize("name", sorted(cases.CHCONV_CASES))
def test_channelwise_convolution(engine, golden, name):
    x, f, b, kw = cases.chconv_inputs(name)
    y = engine.blob_channelwise_convolution(dev(x), dev(f), dev(b), **kw)
    assert gate_err(host(engine, y), golden[f"chconv/{name}"]) < TOL_FP32


@pytest.mark.parametrize("name", sorted(cases.MBV2_CASES))
def test_mobilenetv2_block(engine, golden, name):
    args, kw = cases.mbv2_inputs(name)
    y = engine.mobilenetv2_block(*[dev(a) for a in args], **kw)
    assert gate_err(host(engine, y), golden[f"mbv2/{name}"]) < TOL_FP32


@pytest.mark.parametrize("name", sorted(cases.SOFTMAX_CASES))
def test_softmax(engine, golden, name):
    x, h, w = cases.softmax_inputs(name)
    y = engine.matrix_softmax_by_rows(dev(x), h, w)
    assert gate_err(host(engine, y), golden[f"softmax/{name}"]) < 1e-5


def test_vector_and_matrix_helpers(engine, oracle):
    a, b = cases.uniform(11, (1001,), -4, 4), cases.uniform(12, (1001,), -4, 4)
    for op in (0, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18):
        a_ = np.abs(a) + 0.1 if op in (11, 12) else a
        b_ = np.abs(b) + 0.5 if op == 17 else b
        got = host(engine, engine.vector_op(op, dev(a_), dev(b_), 0.7))
        assert gate_err(got, oracle.vector_op(op, a_, b_, 0.7)) < 1e-5, op
    m = cases.uniform(21, (3 * 5 * 7,))
    v21, v15 = cases.uniform(22, (21,)), cases.uniform(23, (15,))
    assert np.array_equal(host(engine, engine.add_vector_to_matrix_rows(3, dev(m), 5, 7, dev(v21))),
                          oracle.add_vector_to_matrix_rows(3, m, 5, 7, v21))
    assert np.array_equal(host(engine, engine.add_vector_to_matrix_columns(dev(m), 15, 7, dev(v15))),
                          oracle.add_vector_to_matrix_columns(m, 15, 7, v15))
    assert gate_err(host(engine, engine.sum_matrix_rows(3, dev(m), 5, 7)), oracle.sum_matrix_rows(3, m, 5, 7)) < 1e-5
    assert gate_err(host(engine, engine.sum_matrix_columns(dev(m), 15, 7)), oracle.sum_matrix_columns(m, 15, 7)) < 1e-5
    t = cases.uniform(26, (2 * 3 * 4 * 5 * 6,))
    assert np.array_equal(host(engine, engine.transpose_matrix(2, dev(t), 3, 4, 5, 6)), oracle.transpose_matrix(2, t, 3, 4, 5, 6))
    am = cases.uniform(27, (13 * 37,))
    v, i = engine.find_max_value_in_rows(dev(am), 13, 37)
    ov, oi = oracle.find_max_value_in_rows(am, 13, 37)
    assert np.array_equal(host(engine, v), ov) and np.array_equal(host(engine, i), oi)


def test_pooling_and_resize(engine, oracle):
    x = cases.uniform(31, (2, 10, 12, 8))
    assert np.array_equal(host(engine, engine.blob_max_pooling(dev(x), (3, 3), (2, 2))[0]), oracle.blob_max_pooling(x, (3, 3), (2, 2))[0])
    assert gate_err(host(engine, engine.blob_mean_pooling(dev(x), (3, 2), (2, 1))), oracle.blob_mean_pooling(x, (3, 2), (2, 1))) < 1e-6
    for pad in (0, 1, 2):
        assert np.array_equal(host(engine, engine.blob_resize_image(dev(x), 1, 2, 2, 1, pad, 0.5)),
                              oracle.blob_resize_image(x, 1, 2, 2, 1, pad, 0.5))


def test_tf32_flag_selects_the_opt_in_arithmetic(golden):
    if not ShimmedB200Engine.available():
        pytest.skip("oracle/_ref or libNeoMathEngineB200.so not built")
    e = ShimmedB200Engine(flags=2)  # GpuMathEngineCublasUseTensorCoresTF32Flag
    try:
        a, b, kw = cases.mmt_inputs("aligned")
        y = host(e, e.multiply_matrix_by_transposed_matrix(dev(a), dev(b), **kw))
        err = gate_err(y, golden["mmt/aligned"])
        assert 1e-6 < err < TOL_TF32  # visibly TF32, and inside its own tolerance
    finally:
        e.close()


def test_engine_memory_exchange_and_gauges(engine):
    x = cases.uniform(41, (100_003,))
    y, (current, peak, pooled, pooled_after_cleanup) = engine.roundtrip(x)
    assert np.array_equal(y, 2 * x + 1)
    # one heap block of n floats is live when the gauges are read; the two stack variables pushed the peak higher
    assert current >= 4 * x.size and peak >= current + 4 * x.size
    assert pooled >= 4 * x.size          # the freed heap block is cached for reuse ...
    assert pooled_after_cleanup == 0     # ... until CleanUp() gives it back to the driver


def test_engine_identity(engine):
    kind, available, name, device = engine.info()
    assert kind == 2                     # MET_Cuda: NeoML code that branches on the engine type takes its GPU paths
    assert device == 0 and available > (1 << 30) and name


def test_training_methods_raise_instead_of_falling_back(engine):
    x = dev(cases.uniform(42, (64,)))
    assert engine.training_method_raises(x)


def test_in_place_add_and_relu_ride_in_the_convolution_epilogue(engine, oracle):
    """conv -> VectorAdd(y, r, y) -> VectorReLU(y, y) as a CDnn issues them: the engine holds the convolution back,
    folds the two in-place calls into its epilogue and launches once; the result is that of the three separate calls."""
    from neoml_b200 import _capi
    lib = _capi.load()
    x, f, b = cases.uniform(51, (2, 14, 14, 64)), cases.uniform(52, (96, 3, 3, 64)), cases.uniform(53, (96,))
    r = cases.uniform(54, (2, 14, 14, 96))
    want = np.maximum(oracle.blob_convolution(x, f, b, padding=(1, 1)) + r, 0.0)

    def run(fused: bool):
        dx, df, db, dr = dev(x), dev(f), dev(b), dev(r)
        engine.sync()
        before = lib.nb200_launch_count()
        y = engine.blob_convolution(dx, df, db, padding=(1, 1))
        if not fused:
            engine.sync()                                   # forces the convolution out before the next call
        engine.vector_op(3, y.reshape(-1), dr.reshape(-1), out=y.reshape(-1))       # VectorAdd in place
        engine.vector_op(9, y.reshape(-1), None, 0.0, out=y.reshape(-1))            # VectorReLU in place
        got = host(engine, y)
        return got, lib.nb200_launch_count() - before

    fused, fused_launches = run(True)
    plain, plain_launches = run(False)
    assert gate_err(fused, want) < TOL_FP32 and gate_err(plain, want) < TOL_FP32
    assert np.array_equal(fused, plain)                     # same arithmetic, same order of additions per element
    assert plain_launches == fused_launches + 2             # the add and the ReLU launched nothing of their own


def test_gpu_manager_lists_the_device_and_creates_engines(engine):
    """IGpuMathEngineManager as NeoML's device pickers use it: count, info, CreateMathEngine(index)."""
    import ctypes as C
    lib = engine.engine_lib
    lib.nb200_create_math_engine_manager.restype = C.c_void_p
    lib.nb200_manager_probe.restype = C.c_int
    lib.nb200_manager_probe.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_ulonglong), C.c_char_p, C.c_int]
    lib.nb200_destroy_math_engine_manager.argtypes = [C.c_void_p]
    lib.nb200_destroy_math_engine.argtypes = [C.c_void_p]
    manager = C.c_void_p(lib.nb200_create_math_engine_manager())
    try:
        created, memory, name = C.c_void_p(), C.c_ulonglong(0), C.create_string_buffer(256)
        count = lib.nb200_manager_probe(manager, 0, C.byref(created), C.byref(memory), name, 256)
        assert count == torch.cuda.device_count() >= 1
        assert b"B200" in name.value and memory.value > (100 << 30)
        assert created.value
        lib.nb200_destroy_math_engine(created)
        assert lib.nb200_manager_probe(manager, count, None, None, None, 0) == count     # out of range: nothing happens
    finally:
        lib.nb200_destroy_math_engine_manager(manager)


def test_in_place_scale_and_mask_ride_in_the_softmax(engine, oracle):
    """The score path of attention as CMultiheadAttentionLayer issues it, in place: VectorMultiply by a device scalar,
    AddVectorToMatrixRows of the mask, MatrixSoftmaxByRows.  The engine runs the three as one pass; the result is
    bit for bit that of the separate calls, which the oracle confirms to tolerance."""
    from neoml_b200 import _capi
    lib = _capi.load()
    heads, seq = 6, 48
    scores = cases.uniform(81, (heads * seq * seq,), -4, 4)
    mask = (np.triu(np.ones((seq, seq), np.float32), k=1) * -1e9).reshape(-1)
    want = oracle.matrix_softmax_by_rows(
        oracle.add_vector_to_matrix_rows(1, oracle.vector_op(6, scores, None, 0.125), heads, seq * seq, mask), heads * seq, seq)

    def run(fused: bool):
        x, m = dev(scores), dev(mask)
        engine.sync()
        before = lib.nb200_launch_count()
        engine.vector_op(6, x, None, 0.125, out=x)
        if not fused:
            engine.sync()
        engine.add_vector_to_matrix_rows(1, x, heads, seq * seq, m, out=x)
        if not fused:
            engine.sync()
        engine.matrix_softmax_by_rows(x, heads * seq, seq, out=x)
        return host(engine, x), lib.nb200_launch_count() - before

    fused, fused_launches = run(True)
    plain, plain_launches = run(False)
    assert np.array_equal(fused, plain)
    assert gate_err(fused, want) < 1e-5
    assert (fused_launches, plain_launches) == (1, 3)
    # a held-back multiply that nothing absorbs is simply launched by the next call
    y = dev(scores)
    engine.vector_op(6, y, None, 0.5, out=y)
    assert np.array_equal(host(engine, y), scores * np.float32(0.5))


def _rowwise_chain_inputs():
    n, h, w, c, k, cexp, kout = 2, 21, 18, 8, 16, 48, 24
    he = lambda seed, shape, fan: cases.normal(seed, shape, float(np.sqrt(2.0 / fan)))
    bias = lambda seed, m: cases.uniform(seed, (m,), -0.1, 0.1)
    return (cases.uniform(91, (n, h, w, c), 0, 1), he(92, (k, 3, 3, c), 9 * c), bias(93, k), he(94, (cexp, k), k), bias(95, cexp),
            he(96, (3, 3, cexp), 9), bias(97, cexp), he(98, (k, cexp), cexp), bias(99, k), he(100, (3, 3, k), 9), bias(101, k),
            he(102, (3, 3, k), 9), bias(103, k), he(104, (kout, k), k), bias(105, kout))


def test_rowwise_chain_matches_the_reference_cpu_engine(engine, reference):
    """A chain of eight rowwise operations (resize, pooling, conv + ReLU, MobileNetV2 block, channelwise conv + HSwish,
    channelwise-with-1x1) as the optimizer of NeoML emits them, on both engines through the same IMathEngine calls."""
    from neoml_b200 import _capi
    args = _rowwise_chain_inputs()
    want = reference.rowwise_chain(*args)
    held = [dev(a) for a in args]
    engine.sync()
    before = _capi.load().nb200_launch_count()
    got = engine.rowwise_chain(*held)
    result = host(engine, got)
    launches = _capi.load().nb200_launch_count() - before
    assert result.shape == want.shape == (2, 6, 5, 24)
    assert gate_err(result, want) < TOL_FP32
    # resize 1, pool 1, few-channel conv 4 (image padding, filter widening, filter preparation, contraction; ReLU folded
    # in), block 3, channelwise 1 (HSwish folded in), channelwise + 1x1 2: the two activations launch nothing
    assert launches == 12


@pytest.mark.parametrize("r,stride,residual,acts", [
    (3, 1, True, ((1, 6.0), (1, 6.0), (0, 0.0))),        # ReLU6 block with residual
    (5, 2, False, ((2, 0.0), (2, 0.0), (2, 0.0))),       # 5x5 / stride 2, HSwish everywhere
    (5, 1, True, ((2, 0.0), (1, 0.0), (1, 4.0))),
])
def test_mobilenetv3_block_matches_the_reference_cpu_engine(engine, reference, r, stride, residual, acts):
    """MobileNetV3PreSEBlock + MobileNetV3PostSEBlock (expand 1x1, channelwise r x r, squeeze-and-excite gate, down
    1x1, residual) on both engines through the same IMathEngine calls."""
    n, h, w, c, cexp = 3, 13, 11, 24, 72
    kout = c if residual else 40
    rng = np.random.default_rng(900 + r + stride)
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
    w_exp = (rng.standard_normal((cexp, c)) * np.sqrt(2.0 / c)).astype(np.float32)
    w_dw = (rng.standard_normal((r, r, cexp)) * np.sqrt(2.0 / (r * r))).astype(np.float32)
    w_down = (rng.standard_normal((kout, cexp)) * np.sqrt(2.0 / cexp)).astype(np.float32)
    b_exp, b_dw = rng.uniform(-0.1, 0.1, cexp).astype(np.float32), rng.uniform(-0.1, 0.1, cexp).astype(np.float32)
    b_down = rng.uniform(-0.1, 0.1, kout).astype(np.float32)
    se = rng.uniform(0, 1, (n, cexp)).astype(np.float32)       # what the block's pooled + FC + hard-sigmoid branch yields
    args = (x, w_exp, b_exp, w_dw, b_dw, se, w_down, b_down)
    want_mid, want = reference.mobilenetv3_block(*args, stride=stride, residual=residual, acts=acts)
    held = [dev(a) for a in args]
    engine.sync()
    got_mid, got = engine.mobilenetv3_block(*held, stride=stride, residual=residual, acts=acts)
    got_mid, got = host(engine, got_mid), host(engine, got)
    assert got.shape == want.shape and got_mid.shape == want_mid.shape
    assert gate_err(got_mid, want_mid) < TOL_FP32
    assert gate_err(got, want) < TOL_FP32


def test_two_engines_on_two_host_threads(golden):
    """One engine per host thread, as NeoML's replica drivers run them: both issue convolutions and products at the
    same time on their own streams; every result is still the golden one (no shared per-call state in the library)."""
    import threading
    if not ShimmedB200Engine.available():
        pytest.skip("libNeoMathEngineB200.so or the shim not built")
    engines = [ShimmedB200Engine(), ShimmedB200Engine()]
    names = sorted(cases.CONV_CASES)
    inputs = {n: cases.conv_inputs(n) for n in names}
    held = {n: tuple(dev(a) for a in inputs[n][:3]) for n in names}
    a, b, kw = cases.mmt_inputs("aligned")
    da, db = dev(a), dev(b)
    want = {n: np.array(golden[f"conv/{n}"]) for n in names}    # the archive reader is not for concurrent use
    want_mmt = np.array(golden["mmt/aligned"])
    failures = []

    def worker(e, order):
        try:
            for _ in range(3):
                for n in order:
                    dx, df, dbias = held[n]
                    y = e.blob_convolution(dx, df, dbias, **inputs[n][3])
                    m = e.multiply_matrix_by_transposed_matrix(da, db, **kw)
                    e.sync()
                    if gate_err(y.cpu().numpy(), want[n]) >= TOL_FP32 or gate_err(m.cpu().numpy(), want_mmt) >= TOL_FP32:
                        failures.append(n)
        except Exception as exc:  # noqa: BLE001 - reported below
            failures.append(repr(exc))

    threads = [threading.Thread(target=worker, args=(engines[0], names)),
               threading.Thread(target=worker, args=(engines[1], names[::-1]))]
    [t.start() for t in threads]
    [t.join() for t in threads]
    for e in engines:
        e.close()
    assert not failures, failures
