"""ctypes binding of the C ABI declared in include/neoml_b200.h.

The shared library is built in-tree by ``python -m neoml_b200.build`` (neoml_b200/lib/libneoml_b200.so).
Nothing here falls back to another implementation: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libneoml_b200.so"

OK, EINVAL, ENODEVICE, ELAUNCH, EDEVICE, ETOOBIG = 0, -1, -2, -3, -4, -5
PREC_3XTF32, PREC_TF32, PREC_FP32_SIMT = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_HSWISH = 0, 1, 2

VEC_OPS = ["COPY", "FILL", "FILL_HANDLE", "ADD", "SUB", "ELTWISE_MUL", "MULTIPLY", "NEG_MULTIPLY", "ADD_VALUE",
           "RELU", "SIGMOID", "SQRT", "INV", "TANH", "EXP", "HSWISH", "ELTWISE_MAX", "ELTWISE_DIV", "MUL_ADD"]
VEC = {name: i for i, name in enumerate(VEC_OPS)}
VEC["SIGMOID_MUL"] = len(VEC_OPS)   # the library's own: three of the calls above in one pass (NB200_VEC_SIGMOID_MUL)


class Epilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("residual", C.c_void_p), ("ld_residual", C.c_int), ("act", C.c_int),
                ("act_param", C.c_float), ("accumulate", C.c_int), ("act_param_device", C.c_void_p)]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "h", "w", "c", "k", "r", "s", "pad_h", "pad_w", "stride_h",
                                       "stride_w", "dil_h", "dil_w", "ho", "wo")]


class ChConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "h", "w", "c", "r", "s", "pad_h", "pad_w", "stride_h", "stride_w",
                                       "ho", "wo")]


class Mbv2Desc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "h", "w", "c_in", "c_exp", "c_out", "stride", "residual",
                                       "act_exp", "act_dw")] + [("act_exp_param", C.c_float),
                                                                ("act_dw_param", C.c_float)]


_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_EP = C.POINTER(Epilogue)

# name -> (restype, argtypes); the single source of truth for tests that check exported symbols
SIGNATURES = {
    "nb200_version": (_i, []),
    "nb200_device_count": (_i, []),
    "nb200_error_string": (C.c_char_p, [_i]),
    "nb200_device_status": (_i, [_vp, _i]),
    "nb200_last_cuda_error": (C.c_char_p, []),
    "nb200_launch_count": (C.c_uint64, []),
    "nb200_multiply_matrix_by_transposed_matrix": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _EP, _i]),
    "nb200_batch_multiply_matrix_by_transposed_matrix": (_i, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _EP, _i]),
    "nb200_matrix_product_scratch_floats": (C.c_size_t, [_i, _i, _i, _i, _i]),
    "nb200_scale_channels_activation": (_i, [_vp, _i, _i, _i, _vp, _vp, _i, C.c_float, _vp]),
    "nb200_multiply_matrix_by_transposed_matrix_with_scratch": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _vp,
                                                                     _EP, _i]),
    "nb200_multiply_matrix_by_matrix": (_i, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _EP, _i]),
    "nb200_blob_convolution_scratch_floats": (C.c_size_t, [C.POINTER(ConvDesc)]),
    "nb200_blob_convolution": (_i, [_vp, C.POINTER(ConvDesc), _vp, _vp, _vp, _vp, _EP, _i]),
    "nb200_blob_convolution_prepared_filter_floats": (C.c_size_t, [C.POINTER(ConvDesc)]),
    "nb200_blob_convolution_prepare_filter": (_i, [_vp, C.POINTER(ConvDesc), _vp, _vp, _i]),
    "nb200_blob_convolution_with_prepared_filter": (_i, [_vp, C.POINTER(ConvDesc), _vp, _vp, _vp, _vp, _vp, _EP, _i]),
    "nb200_blob_convolution_static_scratch": (_i, [_vp, C.POINTER(ConvDesc), _vp, _vp, _vp, _EP, _i]),
    "nb200_blob_channelwise_convolution": (_i, [_vp, C.POINTER(ChConvDesc), _vp, _vp, _vp, _vp, _i, _f]),
    "nb200_mobilenetv2_scratch_floats": (C.c_size_t, [C.POINTER(Mbv2Desc)]),
    "nb200_mobilenetv2_block": (_i, [_vp, C.POINTER(Mbv2Desc), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "nb200_mobilenetv2_block_fused": (_i, [_vp, C.POINTER(Mbv2Desc), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "nb200_matrix_softmax_by_rows_fused": (_i, [_vp, _vp, _i, _i, _vp, _vp, _i, _vp]),
    "nb200_vector_op": (_i, [_vp, _i, _vp, _vp, _vp, _f, _vp, _i]),
    "nb200_vector_copy_int": (_i, [_vp, _vp, _vp, _i]),
    "nb200_vector_fill_int": (_i, [_vp, _i, _vp, _i]),
    "nb200_add_vector_to_matrix_rows": (_i, [_vp, _i, _vp, _vp, _i, _i, _vp]),
    "nb200_add_vector_to_matrix_columns": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "nb200_sum_matrix_rows": (_i, [_vp, _i, _vp, _vp, _i, _i, _i]),
    "nb200_sum_matrix_columns": (_i, [_vp, _vp, _vp, _i, _i]),
    "nb200_multiply_diag_matrix_by_matrix": (_i, [_vp, _vp, _i, _vp, _i, _vp]),
    "nb200_multiply_matrix_by_diag_matrix": (_i, [_vp, _i, _vp, _i, _i, _vp, _i, _vp]),
    "nb200_matrix_softmax_by_rows": (_i, [_vp, _vp, _i, _i, _vp]),
    "nb200_transpose_matrix": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp]),
    "nb200_find_max_value_in_rows": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "nb200_find_max_value_in_columns": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp]),
    "nb200_blob_max_pooling": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "nb200_matrix_product_prepared_floats": (C.c_size_t, [_i, _i, _i, _i]),
    "nb200_matrix_product_prepare_second": (_i, [_vp, _vp, _i, _i, _i, _vp, _i]),
    "nb200_multiply_matrix_by_transposed_matrix_prepared": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _EP, _i]),
    "nb200_sum_matrix_columns_shifted": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i]),
    "nb200_matrix_rows_cols_affine": (_i, [_vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp]),
    "nb200_attention_scores_values": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i]),
    "nb200_blob_max_pooling_padded": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp]),
    "nb200_blob_mean_pooling": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "nb200_blob_resize_image": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp]),
}

# Diagnostic entry points (neoml_b200/csrc/diagnostics.h): exported for the benchmark and the tests, not part of the
# product interface the public header declares
DIAGNOSTICS = {
    "nb200_debug_set_contraction_trace": (None, [_vp, _i, _i]),
    "nb200_debug_time_contractions": (None, [_i]),
    "nb200_debug_contraction_times": (_i, [_vp, _i]),
    "nb200_debug_contraction_records": (_i, [_vp, _vp, _i]),
    "nb200_debug_wait_probe": (_i, [_vp, C.c_ulonglong]),
}

_lib = None


class Nb200Error(RuntimeError):
    def __init__(self, fn: str, code: int):
        self.code = code
        msg = load().nb200_error_string(code).decode() if _lib is not None else str(code)
        if code in (ELAUNCH, ENODEVICE) and _lib is not None:
            msg += ": " + _lib.nb200_last_cuda_error().decode()
        super().__init__(f"{fn} failed: {msg} ({code})")


def load() -> C.CDLL:
    """Loads libneoml_b200.so and attaches the prototypes.  Raises if the library has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m neoml_b200.build` (no fallback exists)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in {**SIGNATURES, **DIAGNOSTICS}.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn: str, code: int) -> None:
    if code != OK:
        raise Nb200Error(fn, code)
