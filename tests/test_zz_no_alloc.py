"""nb200_blob_convolution_static_scratch: the channel-padded convolution whose work space is a fixed array inside the
library, for callers that cannot allocate.  Called through the C ABI and compared, bit for bit, with the existing
entry point (caller-provided scratch) on two calls in a row; the file sorts last so that it also runs after every
other GPU test has used the library."""
import ctypes as C

import pytest
import torch

import cases
from neoml_b200 import _capi as capi
from neoml_b200 import ops

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_FLOATS = 4 * 1024 * 1024  # NB200_STATIC_SCRATCH_FLOATS in include/neoml_b200.h


def _desc(n, h, w, c, k, r, s, pad, stride):
    ho = ops.conv_output_size(h, r, pad[0], stride[0], 1)
    wo = ops.conv_output_size(w, s, pad[1], stride[1], 1)
    return capi.ConvDesc(n, h, w, c, k, r, s, pad[0], pad[1], stride[0], stride[1], 1, 1, ho, wo), ho, wo


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    lib = capi.load()
    # the network stem in small: 3 channels, 7x7 stride 2 pad 3, free term + ReLU in the epilogue
    n, h, w, c, k = 2, 37, 41, 3, 64
    desc, ho, wo = _desc(n, h, w, c, k, 7, 7, (3, 3), (2, 2))
    need = lib.nb200_blob_convolution_scratch_floats(C.byref(desc))
    assert 0 < need <= STATIC_SCRATCH_FLOATS
    for call in range(2):
        # fresh inputs each time: a second call that still saw the first call's padded image would be caught
        x = torch.from_numpy(cases.uniform(9100 + call, (n, h, w, c))).cuda()
        f = torch.from_numpy(cases.uniform(9200 + call, (k, 7, 7, c))).cuda()
        b = torch.from_numpy(cases.uniform(9300 + call, (k,))).cuda()
        epi = capi.Epilogue(b.data_ptr(), None, 0, ops.ACT_RELU, 0.0, 0)
        want = torch.empty((n, ho, wo, k), dtype=torch.float32, device="cuda")
        got = torch.full_like(want, float("nan"))
        scratch = torch.empty(need, dtype=torch.float32, device="cuda")
        capi.check("BlobConvolution", lib.nb200_blob_convolution(
            _stream(), C.byref(desc), _ptr(x), _ptr(f), _ptr(want), _ptr(scratch), C.byref(epi), ops.PREC_3XTF32))
        torch.cuda.synchronize()
        # torch's own gauge only sees torch's allocator; the driver's free-memory figure sees any cudaMalloc
        reserved, free_before = torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0]
        capi.check("BlobConvolution(static scratch)", lib.nb200_blob_convolution_static_scratch(
            _stream(), C.byref(desc), _ptr(x), _ptr(f), _ptr(got), C.byref(epi), ops.PREC_3XTF32))
        torch.cuda.synchronize()
        assert torch.cuda.memory_reserved() == reserved
        if call == 1:   # the first call may load the kernels' code (module loading is lazy); the second one must not move
            assert torch.cuda.mem_get_info()[0] == free_before
        assert lib.nb200_device_status(_stream(), 0) == 0
        assert torch.equal(got, want), f"call {call}"


def test_shapes_beyond_the_fixed_work_space_are_refused():
    lib = capi.load()
    # 24 RGB 224x224 images need 24*224*224*4 floats of padded image: more than the fixed 4 Mi floats
    desc, ho, wo = _desc(24, 224, 224, 3, 64, 7, 7, (3, 3), (2, 2))
    assert lib.nb200_blob_convolution_scratch_floats(C.byref(desc)) > STATIC_SCRATCH_FLOATS
    launches = lib.nb200_launch_count()
    one = torch.zeros(16, device="cuda")  # never touched: the call is refused before anything is launched
    rc = lib.nb200_blob_convolution_static_scratch(_stream(), C.byref(desc), _ptr(one), _ptr(one), _ptr(one), None,
                                                   ops.PREC_3XTF32)
    assert rc == capi.ETOOBIG
    assert lib.nb200_launch_count() == launches
    assert b"capacity" in lib.nb200_error_string(rc)


def test_other_shapes_give_the_same_result_as_the_plain_entry_point():
    lib = capi.load()
    n, h, w, c, k = 1, 9, 10, 8, 16
    desc, ho, wo = _desc(n, h, w, c, k, 3, 3, (1, 1), (1, 1))
    x = torch.from_numpy(cases.uniform(9400, (n, h, w, c))).cuda()
    f = torch.from_numpy(cases.uniform(9401, (k, 3, 3, c))).cuda()
    got = torch.empty((n, ho, wo, k), dtype=torch.float32, device="cuda")
    capi.check("BlobConvolution(static scratch)", lib.nb200_blob_convolution_static_scratch(
        _stream(), C.byref(desc), _ptr(x), _ptr(f), _ptr(got), None, ops.PREC_3XTF32))
    torch.cuda.synchronize()
    assert torch.equal(got, ops.BlobConvolution(x, f, padding=(1, 1)))


@pytest.mark.parametrize("shape", [(4, 16, 16, 64, 64, "prepared filter"), (2, 14, 14, 256, 256, "split K")])
def test_the_work_space_paths_match_caller_scratch_bit_for_bit(shape):
    """The two ways the fixed array is written besides the padded image: the prepared filter (32-channel K blocks and
    at least 1024 output positions) and the split-K partial results taken from the array's tail."""
    lib = capi.load()
    n, h, w, c, k, _ = shape
    desc, ho, wo = _desc(n, h, w, c, k, 3, 3, (1, 1), (1, 1))
    need = lib.nb200_blob_convolution_scratch_floats(C.byref(desc))
    assert 0 < need <= STATIC_SCRATCH_FLOATS
    x = torch.from_numpy(cases.uniform(9500, (n, h, w, c))).cuda()
    f = torch.from_numpy(cases.uniform(9501, (k, 3, 3, c))).cuda()
    b = torch.from_numpy(cases.uniform(9502, (k,))).cuda()
    epi = capi.Epilogue(b.data_ptr(), None, 0, ops.ACT_NONE, 0.0, 0)
    want = torch.empty((n, ho, wo, k), dtype=torch.float32, device="cuda")
    scratch = torch.empty(need, dtype=torch.float32, device="cuda")
    capi.check("BlobConvolution", lib.nb200_blob_convolution(
        _stream(), C.byref(desc), _ptr(x), _ptr(f), _ptr(want), _ptr(scratch), C.byref(epi), ops.PREC_3XTF32))
    for call in range(2):
        got = torch.full_like(want, float("nan"))
        capi.check("BlobConvolution(static scratch)", lib.nb200_blob_convolution_static_scratch(
            _stream(), C.byref(desc), _ptr(x), _ptr(f), _ptr(got), C.byref(epi), ops.PREC_3XTF32))
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"
    assert lib.nb200_device_status(_stream(), 0) == 0
