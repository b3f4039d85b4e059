"""Host-side mirror of the IMathEngine methods on the inference hot path, over torch CUDA tensors.

torch is used for device memory and streams only; every computation is a call into the C ABI
(include/neoml_b200.h) on the tensors' device pointers, enqueued on torch's current stream.
Method names and argument meaning follow NeoMathEngine/include/NeoMathEngine/NeoMathEngine.h; blobs are
channels-last ``[batch, height, width, channels]`` fp32 tensors, filters ``[count, height, width, channels]``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _capi as capi
from ._capi import (ACT_HSWISH, ACT_NONE, ACT_RELU, PREC_3XTF32, PREC_FP32_SIMT, PREC_TF32, VEC)  # noqa: F401


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensors only"
    return t.data_ptr()


def _f32(t: torch.Tensor) -> torch.Tensor:
    assert t.dtype == torch.float32
    return t


def _epilogue(bias=None, residual=None, ld_residual=0, act=ACT_NONE, act_param=0.0, accumulate=False,
              act_param_device=None):
    return capi.Epilogue(_ptr(bias), _ptr(residual), ld_residual, act, float(act_param), int(accumulate),
                         _ptr(act_param_device))


def conv_output_size(size: int, filt: int, pad: int, stride: int, dil: int = 1) -> int:
    """Output size rule of the reference (CpuMathEngineDnnConv.cpp:59-62)."""
    return 1 + (size - (filt - 1) * dil - 1 + 2 * pad) // stride


def MultiplyMatrixByTransposedMatrix(first, second, result=None, *, first_row_size=None, second_row_size=None,
                                     result_row_size=None, first_height=None, first_width=None, second_height=None,
                                     free_term=None, residual=None, act=ACT_NONE, act_param=0.0, accumulate=False,
                                     precision=PREC_3XTF32, use_scratch=True):
    """result[M x N] = first[M x K] * second[N x K]^T (+ fused tail).  2-D tensors give the shapes; pass explicit
    heights/widths/row sizes to address a sub-matrix of a larger buffer, as the reference allows.  With use_scratch
    (what the engine does with its stack allocator) the library gets work space for a prepared second operand and
    for split-K partial results."""
    m = first_height if first_height is not None else first.shape[0]
    k = first_width if first_width is not None else first.shape[1]
    n = second_height if second_height is not None else second.shape[0]
    lda = first_row_size if first_row_size is not None else k
    ldb = second_row_size if second_row_size is not None else k
    ldc = result_row_size if result_row_size is not None else n
    if result is None:
        result = torch.empty((m, ldc), dtype=torch.float32, device=first.device)
    epi = _epilogue(free_term, residual, ldc, act, act_param, accumulate)
    lib = capi.load()
    need = lib.nb200_matrix_product_scratch_floats(1, m, n, k, ldb) if use_scratch else 0
    if need:
        scratch = torch.empty(need, dtype=torch.float32, device=first.device)
        capi.check("MultiplyMatrixByTransposedMatrix", lib.nb200_multiply_matrix_by_transposed_matrix_with_scratch(
            _stream(), 1, _ptr(_f32(first)), m, k, lda, _ptr(_f32(second)), n, ldb, _ptr(result), ldc, _ptr(scratch),
            C.byref(epi), precision))
    else:
        capi.check("MultiplyMatrixByTransposedMatrix", lib.nb200_multiply_matrix_by_transposed_matrix(
            _stream(), _ptr(_f32(first)), m, k, lda, _ptr(_f32(second)), n, ldb, _ptr(result), ldc, C.byref(epi), precision))
    return result


def BatchMultiplyMatrixByTransposedMatrix(first, second, result=None, *, precision=PREC_3XTF32, use_scratch=True):
    """first [B, M, K], second [B, N, K] -> result [B, M, N]."""
    b, m, k = first.shape
    n = second.shape[1]
    if result is None:
        result = torch.empty((b, m, n), dtype=torch.float32, device=first.device)
    _batch_mmt(b, _f32(first), m, k, _f32(second), n, result, precision, use_scratch)
    return result


def _batch_mmt(b, first, m, k, second, n, result, precision, use_scratch):
    lib = capi.load()
    need = lib.nb200_matrix_product_scratch_floats(b, m, n, k, k) if use_scratch else 0
    if need:
        scratch = torch.empty(need, dtype=torch.float32, device=first.device)
        capi.check("BatchMultiplyMatrixByTransposedMatrix", lib.nb200_multiply_matrix_by_transposed_matrix_with_scratch(
            _stream(), b, _ptr(first), m, k, k, _ptr(second), n, k, _ptr(result), n, _ptr(scratch), None, precision))
    else:
        capi.check("BatchMultiplyMatrixByTransposedMatrix", lib.nb200_batch_multiply_matrix_by_transposed_matrix(
            _stream(), b, _ptr(first), m, k, _ptr(second), n, _ptr(result), None, precision))


def MultiplyMatrixByMatrix(first, second, result=None, *, precision=PREC_3XTF32, use_scratch=True):
    """first [B, M, K] (or [M, K]), second [B, K, N] (or [K, N]) -> result [B, M, N].
    With use_scratch (what the engine does with its stack allocator) the second operand is transposed once into
    scratch and the product runs as A * (B^T)^T on the TMA-fed path; without, the kernel gathers the column-major
    operand itself."""
    squeeze = first.dim() == 2
    if squeeze:
        first, second = first.unsqueeze(0), second.unsqueeze(0)
    b, m, k = first.shape
    n = second.shape[2]
    if result is None:
        result = torch.empty((b, m, n), dtype=torch.float32, device=first.device)
    lib = capi.load()
    if use_scratch and k >= 4 and n >= 4:
        transposed = torch.empty((b, n, k), dtype=torch.float32, device=first.device)
        capi.check("TransposeMatrix", lib.nb200_transpose_matrix(_stream(), b, _ptr(_f32(second)), k, 1, n, 1,
                                                                 _ptr(transposed)))
        _batch_mmt(b, _f32(first), m, k, transposed, n, result, precision, True)
    else:
        capi.check("MultiplyMatrixByMatrix", lib.nb200_multiply_matrix_by_matrix(
            _stream(), b, _ptr(_f32(first)), m, k, _ptr(_f32(second)), n, _ptr(result), None, precision))
    return result[0] if squeeze else result


def BlobConvolution(source, filter, free_term=None, result=None, *, padding=(0, 0), stride=(1, 1), dilation=(1, 1),
                    residual=None, act=ACT_NONE, act_param=0.0, precision=PREC_3XTF32, use_scratch=True):
    n, h, w, c = source.shape
    k, r, s, c2 = filter.shape
    assert c == c2
    ho = conv_output_size(h, r, padding[0], stride[0], dilation[0])
    wo = conv_output_size(w, s, padding[1], stride[1], dilation[1])
    if result is None:
        result = torch.empty((n, ho, wo, k), dtype=torch.float32, device=source.device)
    desc = capi.ConvDesc(n, h, w, c, k, r, s, padding[0], padding[1], stride[0], stride[1], dilation[0], dilation[1],
                         ho, wo)
    epi = _epilogue(free_term, residual, k, act, act_param)
    lib = capi.load()
    need = lib.nb200_blob_convolution_scratch_floats(C.byref(desc)) if use_scratch else 0
    scratch = torch.empty(need, dtype=torch.float32, device=source.device) if need else None
    capi.check("BlobConvolution", lib.nb200_blob_convolution(
        _stream(), C.byref(desc), _ptr(_f32(source)), _ptr(_f32(filter)), _ptr(result), _ptr(scratch), C.byref(epi),
        precision))
    return result


def BlobChannelwiseConvolution(source, filter, free_term=None, result=None, *, padding=(0, 0), stride=(1, 1),
                               act=ACT_NONE, act_param=0.0):
    n, h, w, c = source.shape
    r, s, c2 = filter.shape
    assert c == c2
    ho = conv_output_size(h, r, padding[0], stride[0])
    wo = conv_output_size(w, s, padding[1], stride[1])
    if result is None:
        result = torch.empty((n, ho, wo, c), dtype=torch.float32, device=source.device)
    desc = capi.ChConvDesc(n, h, w, c, r, s, padding[0], padding[1], stride[0], stride[1], ho, wo)
    capi.check("BlobChannelwiseConvolution", capi.load().nb200_blob_channelwise_convolution(
        _stream(), C.byref(desc), _ptr(_f32(source)), _ptr(_f32(filter)), _ptr(free_term), _ptr(result), act,
        float(act_param)))
    return result


def MobileNetV2Block(source, expand_filter, expand_free_term, channelwise_filter, channelwise_free_term, down_filter,
                     down_free_term, result=None, *, stride=1, residual=False, expand_act=ACT_RELU,
                     expand_act_param=6.0, channelwise_act=ACT_RELU, channelwise_act_param=6.0, scratch=None,
                     precision=PREC_3XTF32, one_kernel=False):
    """one_kernel: the block as a single kernel (nb200_mobilenetv2_block_fused; raises for shapes it does not cover)."""
    n, h, w, c_in = source.shape
    c_exp = expand_filter.shape[0]
    c_out = down_filter.shape[0]
    desc = capi.Mbv2Desc(n, h, w, c_in, c_exp, c_out, stride, int(residual), expand_act, channelwise_act,
                         float(expand_act_param), float(channelwise_act_param))
    lib = capi.load()
    need = lib.nb200_mobilenetv2_scratch_floats(C.byref(desc))
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.float32, device=source.device)
    ho, wo = conv_output_size(h, 3, 1, stride), conv_output_size(w, 3, 1, stride)
    if result is None:
        result = torch.empty((n, ho, wo, c_out), dtype=torch.float32, device=source.device)
    entry = lib.nb200_mobilenetv2_block_fused if one_kernel else lib.nb200_mobilenetv2_block
    capi.check("MobileNetV2Block", entry(
        _stream(), C.byref(desc), _ptr(source), _ptr(expand_filter), _ptr(expand_free_term), _ptr(channelwise_filter),
        _ptr(channelwise_free_term), _ptr(down_filter), _ptr(down_free_term), _ptr(result), _ptr(scratch), precision))
    return result


def vector_op(op: str, first=None, second=None, scalar=None, value=0.0, result=None, count=None):
    """Elementwise family; `op` is one of capi.VEC_OPS.  `scalar` is a 1-element device tensor where the reference
    takes a handle (VectorMultiply, VectorReLU threshold, ...)."""
    ref = first if first is not None else result
    if result is None:
        result = torch.empty_like(ref)
    n = count if count is not None else result.numel()
    capi.check("Vector" + op, capi.load().nb200_vector_op(
        _stream(), VEC[op], _ptr(first), _ptr(second), _ptr(scalar), float(value), _ptr(result), n))
    return result


def VectorReLU(first, result=None, threshold=None):
    if threshold is None:
        threshold = torch.zeros(1, dtype=torch.float32, device=first.device)
    return vector_op("RELU", first, scalar=threshold, result=result)


def VectorAdd(first, second, result=None):
    return vector_op("ADD", first, second, result=result)


def AddVectorToMatrixRows(batch, matrix, vector, height, width, result=None):
    if result is None:
        result = torch.empty_like(matrix)
    capi.check("AddVectorToMatrixRows", capi.load().nb200_add_vector_to_matrix_rows(
        _stream(), batch, _ptr(matrix), _ptr(result), height, width, _ptr(vector)))
    return result


def AddVectorToMatrixColumns(matrix, vector, height, width, result=None):
    if result is None:
        result = torch.empty_like(matrix)
    capi.check("AddVectorToMatrixColumns", capi.load().nb200_add_vector_to_matrix_columns(
        _stream(), _ptr(matrix), _ptr(result), height, width, _ptr(vector)))
    return result


def SumMatrixRows(batch, matrix, height, width, result=None, add=False):
    if result is None:
        result = torch.empty((batch, width), dtype=torch.float32, device=matrix.device)
    capi.check("SumMatrixRows", capi.load().nb200_sum_matrix_rows(
        _stream(), batch, _ptr(result), _ptr(matrix), height, width, int(add)))
    return result


def SumMatrixColumns(matrix, height, width, result=None):
    if result is None:
        result = torch.empty(height, dtype=torch.float32, device=matrix.device)
    capi.check("SumMatrixColumns", capi.load().nb200_sum_matrix_columns(
        _stream(), _ptr(result), _ptr(matrix), height, width))
    return result


def MultiplyDiagMatrixByMatrix(diag, matrix, height, width, result=None):
    if result is None:
        result = torch.empty_like(matrix)
    capi.check("MultiplyDiagMatrixByMatrix", capi.load().nb200_multiply_diag_matrix_by_matrix(
        _stream(), _ptr(diag), height, _ptr(matrix), width, _ptr(result)))
    return result


def BatchMultiplyMatrixByDiagMatrix(batch, matrix, height, width, diag, diag_stride, result=None):
    if result is None:
        result = torch.empty_like(matrix)
    capi.check("BatchMultiplyMatrixByDiagMatrix", capi.load().nb200_multiply_matrix_by_diag_matrix(
        _stream(), batch, _ptr(matrix), height, width, _ptr(diag), diag_stride, _ptr(result)))
    return result


def MatrixSoftmaxByRows(matrix, height, width, result=None):
    if result is None:
        result = torch.empty_like(matrix)
    capi.check("MatrixSoftmaxByRows", capi.load().nb200_matrix_softmax_by_rows(
        _stream(), _ptr(matrix), height, width, _ptr(result)))
    return result


def MatrixSoftmaxByRowsFused(matrix, height, width, scale=None, row_bias=None, bias_rows=0, result=None):
    """softmax over the rows of (matrix * *scale + row_bias[h % bias_rows]): what the engine launches when an in-place
    VectorMultiply by a device scalar and an in-place AddVectorToMatrixRows precede an in-place MatrixSoftmaxByRows."""
    if result is None:
        result = torch.empty_like(matrix)
    capi.check("MatrixSoftmaxByRows (fused)", capi.load().nb200_matrix_softmax_by_rows_fused(
        _stream(), _ptr(matrix), height, width, _ptr(scale), _ptr(row_bias), bias_rows, _ptr(result)))
    return result


def TransposeMatrix(batch, first, height, medium, width, channels, result=None):
    if result is None:
        result = torch.empty_like(first)
    capi.check("TransposeMatrix", capi.load().nb200_transpose_matrix(
        _stream(), batch, _ptr(first), height, medium, width, channels, _ptr(result)))
    return result


def FindMaxValueInRows(matrix, height, width, with_indices=True):
    vals = torch.empty(height, dtype=torch.float32, device=matrix.device)
    idx = torch.empty(height, dtype=torch.int32, device=matrix.device) if with_indices else None
    capi.check("FindMaxValueInRows", capi.load().nb200_find_max_value_in_rows(
        _stream(), _ptr(matrix), height, width, _ptr(vals), _ptr(idx)))
    return vals, idx


def FindMaxValueInColumns(batch, matrix, height, width):
    vals = torch.empty((batch, width), dtype=torch.float32, device=matrix.device)
    idx = torch.empty((batch, width), dtype=torch.int32, device=matrix.device)
    capi.check("FindMaxValueInColumns", capi.load().nb200_find_max_value_in_columns(
        _stream(), batch, _ptr(matrix), height, width, _ptr(vals), _ptr(idx)))
    return vals, idx


def BlobMaxPooling(source, filter_size, stride, result=None, with_indices=False):
    n, h, w, c = source.shape
    ho, wo = (h - filter_size[0]) // stride[0] + 1, (w - filter_size[1]) // stride[1] + 1
    if result is None:
        result = torch.empty((n, ho, wo, c), dtype=torch.float32, device=source.device)
    idx = torch.empty((n, ho, wo, c), dtype=torch.int32, device=source.device) if with_indices else None
    capi.check("BlobMaxPooling", capi.load().nb200_blob_max_pooling(
        _stream(), n, h, w, c, filter_size[0], filter_size[1], stride[0], stride[1], _ptr(source), _ptr(result),
        _ptr(idx)))
    return (result, idx) if with_indices else result


def AttentionScoresValues(q, kt, v, scale=None, mask=None, precision=PREC_3XTF32):
    """softmax(scale * q @ kt + mask) @ v per batch entry; q [b, sq, d], kt [b, d, st], v [b, st, d]; scale: a 1-element
    device tensor or None; mask [sq, st] or None."""
    b, sq, d = q.shape
    st = kt.shape[2]
    out = torch.empty((b, sq, d), dtype=torch.float32, device=q.device)
    capi.check("AttentionScoresValues", capi.load().nb200_attention_scores_values(
        _stream(), b, _ptr(q), _ptr(kt), _ptr(v), sq, d, st, _ptr(scale), _ptr(mask), _ptr(out), precision))
    return out


def BlobMaxPoolingPadded(source, deltas, default_value, filter_size, stride, result=None):
    """BlobResizeImage (constant padding; deltas = left, right, top, bottom) + BlobMaxPooling as one pass."""
    n, h, w, c = source.shape
    left, right, top, bottom = deltas
    ho = (h + top + bottom - filter_size[0]) // stride[0] + 1
    wo = (w + left + right - filter_size[1]) // stride[1] + 1
    if result is None:
        result = torch.empty((n, ho, wo, c), dtype=torch.float32, device=source.device)
    capi.check("BlobMaxPoolingPadded", capi.load().nb200_blob_max_pooling_padded(
        _stream(), n, h, w, c, left, right, top, bottom, float(default_value), filter_size[0], filter_size[1], stride[0],
        stride[1], _ptr(source), _ptr(result)))
    return result


def BlobMeanPooling(source, filter_size, stride, result=None):
    n, h, w, c = source.shape
    ho, wo = (h - filter_size[0]) // stride[0] + 1, (w - filter_size[1]) // stride[1] + 1
    if result is None:
        result = torch.empty((n, ho, wo, c), dtype=torch.float32, device=source.device)
    capi.check("BlobMeanPooling", capi.load().nb200_blob_mean_pooling(
        _stream(), n, h, w, c, filter_size[0], filter_size[1], stride[0], stride[1], _ptr(source), _ptr(result)))
    return result


def BlobResizeImage(source, delta_left, delta_right, delta_top, delta_bottom, padding=0, default_value=0.0,
                    result=None):
    n, h, w, c = source.shape
    if result is None:
        result = torch.empty((n, h + delta_top + delta_bottom, w + delta_left + delta_right, c), dtype=torch.float32,
                             device=source.device)
    capi.check("BlobResizeImage", capi.load().nb200_blob_resize_image(
        _stream(), n, h, w, c, delta_left, delta_right, delta_top, delta_bottom, padding, float(default_value),
        _ptr(source), _ptr(result)))
    return result
