/* neoml_b200.h -- C ABI of the B200 (sm_100a) kernel library behind a NeoML IMathEngine.
 *
 * Every entry point is the device-side body of one IMathEngine virtual (NeoMathEngine/include/NeoMathEngine/
 * NeoMathEngine.h, cited per function as NME.h:line).  Conventions:
 *   - all pointers are DEVICE pointers to fp32 / int32 data of the calling process, 4-byte aligned or better
 *     (NeoML handles may sit at any 4-byte offset; aligned fast paths are selected at run time);
 *   - sizes are element counts, exactly the ints the IMathEngine method receives;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, nothing synchronises;
 *   - the return value is 0 (NB200_OK) or a negative NB200_E* code; nothing throws, nothing allocates;
 *     the engine turns a non-zero code into IMathEngineExceptionHandler::OnAssert;
 *   - optional operands (free terms, residual) are NULL when absent, like the `const CConstFloatHandle*`
 *     arguments of the reference.
 * There is no CPU fallback: on a machine without a usable sm_100 device every compute call returns
 * NB200_ENODEVICE.
 */
#ifndef NEOML_B200_H
#define NEOML_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB200_API __attribute__((visibility("default")))

enum {
	NB200_OK = 0,
	NB200_EINVAL = -1,     /* bad argument (negative size, null required pointer, unsupported combination) */
	NB200_ENODEVICE = -2,  /* no sm_100 device / CUDA runtime error at launch */
	NB200_ELAUNCH = -3,    /* cudaGetLastError() after the launch was not cudaSuccess */
	NB200_EDEVICE = -4,    /* a kernel reported a bounded-wait timeout in the status word */
	NB200_ETOOBIG = -5     /* request exceeds a documented fixed capacity */
};

/* Arithmetic of the dense contractions.  The reference selects cuBLAS math modes with the engine flags
 * GpuMathEngineCublasUseTensorCores{Half,TF32}Flag (NME.h:1271-1274, CudaMathEngine.cu:56-65). */
enum {
	NB200_PREC_3XTF32 = 0, /* default: hi/lo TF32 split, 3 tcgen05 MMAs, fp32 accumulate; fp32-level accuracy */
	NB200_PREC_TF32 = 1,   /* opt-in single TF32 MMA (1e-2 tolerance class) */
	NB200_PREC_FP32_SIMT = 2 /* exact fp32 FMA on CUDA cores; diagnostic cross-check, slow */
};

/* Epilogue activations (TActivationFunction subset used by the rowwise descs, ActivationDesc.h:27-47). */
enum {
	NB200_ACT_NONE = 0,
	NB200_ACT_RELU = 1,   /* param > 0: min(max(x,0),param); else max(x,0)  (VectorReLU, NME.h:143-145) */
	NB200_ACT_HSWISH = 2, /* x * relu6(x+3) / 6 */
	NB200_ACT_SIGMOID_GATE = 3 /* x * sigmoid(x * param): CGELULayer's fast form (NeoML/src/Dnn/Layers/GELULayer.cpp:145-163,
	                            * param = 1.702) with the roundings of its three calls (NB200_VEC_SIGMOID_MUL) */
};

/* Optional fused tail of a contraction: y = act(acc + bias[n] (+ residual[m,n])).
 * The plain IMathEngine calls use bias only; the engine's fusion queue fills the rest. */
typedef struct nb200_epilogue {
	const float* bias;       /* [N] or NULL */
	const float* residual;   /* [M x N] with row stride ld_residual, or NULL; may alias the output */
	int ld_residual;
	int act;                 /* NB200_ACT_* */
	float act_param;         /* ReLU upper threshold (<=0: none) */
	int accumulate;          /* 1: y += result (the ...AndAdd variants); 0: overwrite */
	const float* act_param_device; /* optional: the ReLU threshold as one float in device memory, read by the kernel
	                                * (NeoML keeps it there: VectorReLU takes it as a handle, NME.h:143-145); NULL = use
	                                * act_param.  Lets the engine fuse a following VectorReLU without a host read. */
} nb200_epilogue;

/* ---- library ------------------------------------------------------------------------------------------- */
NB200_API int nb200_version(void);
/* Number of sm_100 devices visible; 0 when none (then every compute call fails with NB200_ENODEVICE). */
NB200_API int nb200_device_count(void);
NB200_API const char* nb200_error_string(int code);
/* Device-side status word of the calling thread's current device: 0 = clean, else the code of the first bounded
 * wait that gave up (kernel id << 8 | site).  Reading synchronises `stream`.  `reset` != 0 clears it. */
NB200_API int nb200_device_status(void* stream, int reset);
/* Text of the CUDA runtime error behind the calling thread's last NB200_ELAUNCH / NB200_ENODEVICE. */
NB200_API const char* nb200_last_cuda_error(void);
/* Kernels launched by this library in this process since load (for launch accounting in benchmarks). */
NB200_API uint64_t nb200_launch_count(void);

/* ---- dense contractions (tcgen05 / TMEM) ----------------------------------------------------------------- */
/* IBlasEngine::MultiplyMatrixByTransposedMatrix (NME.h:529-532):
 * C[M x N] (row stride ldc) = A[M x K] (row stride lda) * B[N x K]^T (row stride ldb). */
NB200_API int nb200_multiply_matrix_by_transposed_matrix(void* stream, const float* a, int m, int k, int lda,
	const float* b, int n, int ldb, float* c, int ldc, const nb200_epilogue* epi, int precision);
/* Batched overload (NME.h:533-535): `batch` contiguous problems of identical shape, dense strides. */
NB200_API int nb200_batch_multiply_matrix_by_transposed_matrix(void* stream, int batch, const float* a, int m,
	int k, const float* b, int n, float* c, const nb200_epilogue* epi, int precision);
/* Both overloads of IBlasEngine::MultiplyMatrixByTransposedMatrix (NME.h:529-535) with work space, the form the engine
 * calls: `batch` problems whose operands follow one another (A_b = a + b*m*lda, B_b = b + b*n*ldb, C_b = c + b*m*ldc).
 * `scratch` (NULL = none) holds nb200_matrix_product_scratch_floats(batch, m, n, k, ldb) floats of device memory:
 * for tall products the second operand is split for the tensor core once per call instead of tile by tile in every
 * CTA, and products with few output tiles (a classifier at batch 1) cut their K loop into parts summed in fixed order. */
NB200_API size_t nb200_matrix_product_scratch_floats(int batch, int m, int n, int k, int ldb);
NB200_API int nb200_multiply_matrix_by_transposed_matrix_with_scratch(void* stream, int batch, const float* a, int m,
	int k, int lda, const float* b, int n, int ldb, float* c, int ldc, float* scratch, const nb200_epilogue* epi,
	int precision);
/* The same product (NME.h:529-532, one problem) with the second operand prepared ahead of the call: a fully connected
 * layer's weights do not change between passes, so their tensor-core form (the lo part of the 3xTF32 split, or the
 * rounded copy for TF32) is made once -- nb200_matrix_product_prepared_floats(m, n, k, ldb) floats of device memory,
 * 16-byte aligned, 0 when a product of m rows does not use a prepared operand -- and handed to every call until the
 * weights change.  `scratch` then only serves split K (NULL allowed); prepared_b == NULL is the call above. */
NB200_API size_t nb200_matrix_product_prepared_floats(int m, int n, int k, int ldb);
NB200_API int nb200_matrix_product_prepare_second(void* stream, const float* b, int n, int k, int ldb, float* prepared,
	int precision);
NB200_API int nb200_multiply_matrix_by_transposed_matrix_prepared(void* stream, const float* a, int m, int k, int lda,
	const float* b, int n, int ldb, float* c, int ldc, const float* prepared_b, float* scratch, const nb200_epilogue* epi,
	int precision);
/* IBlasEngine::MultiplyMatrixByMatrix (NME.h:580-582): C_b[M x N] = A_b[M x K] * B_b[K x N], dense row-major. */
NB200_API int nb200_multiply_matrix_by_matrix(void* stream, int batch, const float* a, int m, int k,
	const float* b, int n, float* c, const nb200_epilogue* epi, int precision);
/* The score chain of CMultiheadAttentionLayer (NeoML/src/Dnn/Layers/MultiheadAttentionLayer.cpp:145-223) as one kernel:
 * batched MultiplyMatrixByMatrix (NME.h:580-582) of q [batch][seq_q x depth] by kt [batch][depth x seq_to],
 * VectorMultiply by *scale (NME.h:268; NULL = 1), AddVectorToMatrixRows of mask [seq_q x seq_to] (NME.h:419-420; the same
 * for every batch entry, NULL = none), MatrixSoftmaxByRows (NME.h:450), and the batched MultiplyMatrixByMatrix of the
 * probabilities by v [batch][seq_to x depth] -> out [batch][seq_q x depth].  The scores stay in tensor memory.
 * depth == 64, seq_q >= 128, seq_to >= 128 and a multiple of 4, 16-byte aligned operands, NB200_PREC_3XTF32;
 * NB200_EINVAL for anything else: issue the calls one by one then. */
NB200_API int nb200_attention_scores_values(void* stream, int batch, const float* q, const float* kt, const float* v,
	int seq_q, int depth, int seq_to, const float* scale, const float* mask, float* out, int precision);
/* IDnnEngine::InitBlobConvolution + BlobConvolution (NME.h:751-756; CPU CpuMathEngineDnnConv.cpp:43-73,391-431).
 * Channels-last blobs: x [batch,h,w,c], filter [k,r,s,c], y [batch,ho,wo,k];
 * ho = 1 + (h - (r-1)*dil_h - 1 + 2*pad_h) / stride_h (same for wo) must equal the values passed. */
typedef struct nb200_conv_desc {
	int batch, h, w, c;          /* source */
	int k, r, s;                 /* filter count, height, width */
	int pad_h, pad_w, stride_h, stride_w, dil_h, dil_w;
	int ho, wo;                  /* result */
} nb200_conv_desc;
/* `scratch` is optional (NULL = none): nb200_blob_convolution_scratch_floats(desc) floats of device memory for what
 * the fast paths prepare once per call: the filter split for the tensor core (lo part / rounded copy, so that no CTA
 * converts its filter tiles), and for few-channel images (the 3-channel network stem) a copy of the image with its
 * spatial padding and 4-channel pixels plus the filter widened to match; for convolutions with few output tiles
 * (small batches) also room for the partial results of a split K loop, which a finishing pass sums in a fixed order
 * (results do not vary from run to run).  The engine takes it from its block pool; without it the same result is
 * computed by slower in-kernel conversion and element-wise gathers, unsplit. */
NB200_API size_t nb200_blob_convolution_scratch_floats(const nb200_conv_desc* desc);
NB200_API int nb200_blob_convolution(void* stream, const nb200_conv_desc* desc, const float* x,
	const float* filter, float* y, float* scratch, const nb200_epilogue* epi, int precision);
/* The filter-only part of that preparation, made once and kept by the caller for as long as the filter's values do
 * not change (inference: for ever): nb200_blob_convolution_prepared_filter_floats(desc) floats (0: this shape prepares
 * nothing from the filter alone), filled by nb200_blob_convolution_prepare_filter for one `precision`; then
 * nb200_blob_convolution_with_prepared_filter is IDnnEngine::BlobConvolution (NME.h:751-756) without the per-call
 * filter pass.  `prepared` NULL behaves exactly like nb200_blob_convolution; results are the same bits either way. */
NB200_API size_t nb200_blob_convolution_prepared_filter_floats(const nb200_conv_desc* desc);
NB200_API int nb200_blob_convolution_prepare_filter(void* stream, const nb200_conv_desc* desc, const float* filter,
	float* prepared, int precision);
NB200_API int nb200_blob_convolution_with_prepared_filter(void* stream, const nb200_conv_desc* desc, const float* x,
	const float* filter, const float* prepared, float* y, float* scratch, const nb200_epilogue* epi, int precision);
/* No counterpart in the reference.  The same convolution for callers that cannot provide scratch memory at the moment
 * of the call (all device memory already in their own pool; a loop that must not stall on cudaMalloc; a fixed memory
 * budget): the work space (prepared filter, padded image) is a fixed array of NB200_STATIC_SCRATCH_FLOATS floats inside
 * the library's device module, and neither this call nor anything under it allocates or frees memory.
 *  - A shape whose prepared operands need more than NB200_STATIC_SCRATCH_FLOATS floats is refused with NB200_ETOOBIG
 *    before anything is launched (nb200_blob_convolution_scratch_floats(desc) is an upper bound of that need: it
 *    includes the optional room for a split K loop, which this entry point uses only as far as the array reaches).
 *  - The first call on each device looks the array up (and may load the module): make it during set-up, with that
 *    device current, before a stream capture begins.
 *  - One work space per device: calls that overlap in time on one device (other streams, other threads) race on it;
 *    calls on one stream are ordered.  Nothing in it needs to be zero beforehand. */
#define NB200_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024) /* 16 MiB: e.g. 19 padded RGB 224x224 images + a 7x7x64 filter */
NB200_API int nb200_blob_convolution_static_scratch(void* stream, const nb200_conv_desc* desc, const float* x,
	const float* filter, float* y, const nb200_epilogue* epi, int precision);

/* ---- depthwise / fused blocks ----------------------------------------------------------------------------- */
/* IDnnEngine::BlobChannelwiseConvolution (NME.h:766-771): x [batch,h,w,c], filter [r,s,c], y [batch,ho,wo,c]. */
typedef struct nb200_chconv_desc {
	int batch, h, w, c, r, s, pad_h, pad_w, stride_h, stride_w, ho, wo;
} nb200_chconv_desc;
NB200_API int nb200_blob_channelwise_convolution(void* stream, const nb200_chconv_desc* desc, const float* x,
	const float* filter, const float* free_term, float* y, int act, float act_param);
/* The squeeze-and-excite gate inside IDnnEngine::MobileNetV3PostSEBlock (NME.h:1078-1082; CPU
 * CpuMathEngineDnnChannelwiseConv.cpp:216-221): y[b][pixel][c] = act(x[b][pixel][c] * scale[b][c]); the engine runs
 * the block's 1x1 convolution on y with bias and residual in the epilogue. */
NB200_API int nb200_scale_channels_activation(void* stream, int batch, int pixels, int channels, const float* x,
	const float* scale, int act, float act_param, float* y);

/* IDnnEngine::InitRowwiseMobileNetV2 + MobileNetV2Block (NME.h:1095-1101,1069-1071;
 * CPU CpuRowwiseMobileNetV2.h:151-295):
 * y = [x +] W_down * act2( dw3x3( act1( W_exp * x + b_exp ) ) + b_dw ) + b_down.
 * x [batch,h,w,c_in]; w_exp [c_exp,c_in]; w_dw [3,3,c_exp]; w_down [c_out,c_exp]; y [batch,ho,wo,c_out].
 * `scratch` must hold nb200_mobilenetv2_scratch_floats(desc) floats (the engine takes it from StackAlloc). */
typedef struct nb200_mbv2_desc {
	int batch, h, w, c_in, c_exp, c_out, stride;
	int residual;               /* 1: add x (needs c_in == c_out, stride == 1); y may alias x */
	int act_exp, act_dw;        /* NB200_ACT_* */
	float act_exp_param, act_dw_param;
} nb200_mbv2_desc;
NB200_API size_t nb200_mobilenetv2_scratch_floats(const nb200_mbv2_desc* desc);
NB200_API int nb200_mobilenetv2_block(void* stream, const nb200_mbv2_desc* desc, const float* x,
	const float* w_exp, const float* b_exp, const float* w_dw, const float* b_dw,
	const float* w_down, const float* b_down, float* y, float* scratch, int precision);
/* The same block (NME.h:1095-1101,1069-1071) as ONE kernel that keeps the expanded activations on chip (DRAM traffic =
 * input + output + weights).  Shapes: stride 1, c_in = 32, c_exp a multiple of 32 up to 192, c_out a multiple of 16 up
 * to 64; anything else returns NB200_EINVAL.  `scratch` (batch*h*w*c_out floats + 4) is needed only when y overlaps x.
 * nb200_mobilenetv2_block takes this path by itself wherever the shape allows; the entry point exists so that a caller
 * (and the tests) can ask for it explicitly. */
NB200_API int nb200_mobilenetv2_block_fused(void* stream, const nb200_mbv2_desc* desc, const float* x,
	const float* w_exp, const float* b_exp, const float* w_dw, const float* b_dw,
	const float* w_down, const float* b_down, float* y, float* scratch, int precision);

/* ---- memory-bound vector / matrix ops ---------------------------------------------------------------------- */
/* Elementwise family (IVectorMathEngine, NME.h:69-384).  `op` selects the method; operands unused by an op
 * are NULL.  Scalars that NeoML keeps on the device arrive as device pointers (`scalar`); with scalar == NULL the ops
 * marked *scalar use `value` instead (true scalars: `value`). */
enum {
	NB200_VEC_COPY = 0,          /* VectorCopy           y = a                         NME.h:73  */
	NB200_VEC_FILL = 1,          /* VectorFill(value)    y = value                     NME.h:86  */
	NB200_VEC_FILL_HANDLE = 2,   /* VectorFill(handle)   y = *scalar                   NME.h:90  */
	NB200_VEC_ADD = 3,           /* VectorAdd            y = a + b                     NME.h:236 */
	NB200_VEC_SUB = 4,           /* VectorSub            y = a - b                     NME.h:249 */
	NB200_VEC_ELTWISE_MUL = 5,   /* VectorEltwiseMultiply y = a * b                    NME.h:279 */
	NB200_VEC_MULTIPLY = 6,      /* VectorMultiply       y = a * *scalar               NME.h:268 */
	NB200_VEC_NEG_MULTIPLY = 7,  /* VectorNegMultiply    y = -a * *scalar              NME.h:273 */
	NB200_VEC_ADD_VALUE = 8,     /* VectorAddValue       y = a + *scalar               NME.h:240 */
	NB200_VEC_RELU = 9,          /* VectorReLU           thr=*scalar; thr>0 ? min(max(a,0),thr) : max(a,0)  NME.h:144 */
	NB200_VEC_SIGMOID = 10,      /* VectorSigmoid        y = 1/(1+exp(-a))             NME.h:311 */
	NB200_VEC_SQRT = 11,         /* VectorSqrt                                         NME.h:299 */
	NB200_VEC_INV = 12,          /* VectorInv            y = 1/a                       NME.h:302 */
	NB200_VEC_TANH = 13,         /* VectorTanh                                         NME.h:319 */
	NB200_VEC_EXP = 14,          /* VectorExp                                          NME.h:215 */
	NB200_VEC_HSWISH = 15,       /* VectorHSwish                                       NME.h:162 */
	NB200_VEC_ELTWISE_MAX = 16,  /* VectorEltwiseMax                                   NME.h:169 */
	NB200_VEC_ELTWISE_DIV = 17,  /* VectorEltwiseDivide  y = a / b                     NME.h:291 */
	NB200_VEC_MUL_ADD = 18,      /* VectorMultiplyAndAdd y = a + b * *scalar           NME.h:259 */
	NB200_VEC_SIGMOID_MUL = 19,  /* VectorMultiply, VectorSigmoid, VectorEltwiseMultiply as CGELULayer chains them
	                                (NeoML/src/Dnn/Layers/GELULayer.cpp, the fast form): y = sigmoid(a * *scalar) * a,
	                                the same roundings as the three calls, one pass */
	NB200_VEC_OP_COUNT
};
NB200_API int nb200_vector_op(void* stream, int op, const float* a, const float* b, const float* scalar,
	float value, float* y, int count);
/* Int32 VectorCopy / VectorFill (NME.h:74,87). */
NB200_API int nb200_vector_copy_int(void* stream, const int* a, int* y, int count);
NB200_API int nb200_vector_fill_int(void* stream, int value, int* y, int count);

/* AddVectorToMatrixRows (NME.h:419-420): y[b][h][w] = x[b][h][w] + v[b][w]. */
NB200_API int nb200_add_vector_to_matrix_rows(void* stream, int batch, const float* x, float* y, int height,
	int width, const float* v);
/* AddVectorToMatrixColumns (NME.h:423-424): y[h][w] = x[h][w] + v[h]. */
NB200_API int nb200_add_vector_to_matrix_columns(void* stream, const float* x, float* y, int height, int width,
	const float* v);
/* SumMatrixRows / SumMatrixRowsAdd (NME.h:433-436): y[b][w] (+)= sum_h x[b][h][w]. */
NB200_API int nb200_sum_matrix_rows(void* stream, int batch, float* y, const float* x, int height, int width,
	int add);
/* SumMatrixColumns (NME.h:439-440): y[h] = sum_w x[h][w]. */
NB200_API int nb200_sum_matrix_columns(void* stream, float* y, const float* x, int height, int width);
/* AddVectorToMatrixColumns (NME.h:423-424) into a scratch matrix, optionally VectorEltwiseMultiply of it by itself
 * (NME.h:279), then SumMatrixColumns (NME.h:439-440) -- the variance step of CObjectNormalizationLayer
 * (NeoML/src/Dnn/Layers/ObjectNormalizationLayer.cpp:198-216) -- as one pass over x, the scratch matrix never written:
 * y[h] = sum_w f(x[h][w] + row_add[h]), f = identity or the square; same roundings and order of additions. */
NB200_API int nb200_sum_matrix_columns_shifted(void* stream, float* y, const float* x, int height, int width,
	const float* row_add, int square);
/* AddVectorToMatrixColumns (NME.h:423-424), MultiplyDiagMatrixByMatrix (NME.h:570-572), MultiplyMatrixByDiagMatrix
 * (NME.h:588-596), AddVectorToMatrixRows (NME.h:419-420) -- the normalise / scale / bias steps of
 * CObjectNormalizationLayer (ObjectNormalizationLayer.cpp:218-242) -- as one pass:
 * y[h][w] = (((x[h][w] + row_add[h]) [squared]) * row_mul[h]) * col_mul[w] + col_add[w]; a NULL vector skips its step;
 * each step is rounded by itself, so the result is the bits of the separate calls.  y may be x. */
NB200_API int nb200_matrix_rows_cols_affine(void* stream, const float* x, int height, int width, const float* row_add,
	int square, const float* row_mul, const float* col_mul, const float* col_add, float* y);
/* MultiplyDiagMatrixByMatrix (NME.h:570-572): y[i][j] = d[i] * x[i][j]. */
NB200_API int nb200_multiply_diag_matrix_by_matrix(void* stream, const float* d, int height, const float* x,
	int width, float* y);
/* BatchMultiplyMatrixByDiagMatrix / MultiplyMatrixByDiagMatrix (NME.h:588-596): y[b][i][j] = x[b][i][j] * d[b?][j];
 * diag_stride is `width` when each batch has its own diagonal, 0 when one diagonal serves all. */
NB200_API int nb200_multiply_matrix_by_diag_matrix(void* stream, int batch, const float* x, int height, int width,
	const float* d, int diag_stride, float* y);
/* MatrixSoftmaxByRows (NME.h:450): row-wise softmax, may run in place. */
NB200_API int nb200_matrix_softmax_by_rows(void* stream, const float* x, int height, int width, float* y);
/* The same with the attention chain's two preceding calls folded in (CMultiheadAttentionLayer: VectorMultiply by a
 * device scalar, NME.h:268-269, then AddVectorToMatrixRows of the mask, NME.h:419-420):
 * y = softmax_rows(x * *scale_device + row_bias[h % bias_rows][.]), each step rounded to fp32 like the separate calls.
 * Either of scale_device / row_bias may be NULL; width <= 1024 when one is given (NB200_ETOOBIG otherwise). */
NB200_API int nb200_matrix_softmax_by_rows_fused(void* stream, const float* x, int height, int width,
	const float* scale_device, const float* row_bias, int bias_rows, float* y);
/* TransposeMatrix (NME.h:599-603): x [batch][height][medium][width][channels] -> y [batch][width][medium][height][channels]. */
NB200_API int nb200_transpose_matrix(void* stream, int batch, const void* x, int height, int medium, int width,
	int channels, void* y);
/* FindMaxValueInRows (NME.h:466-469): per row max and (optional) first arg-max column index. */
NB200_API int nb200_find_max_value_in_rows(void* stream, const float* x, int height, int width, float* max_values,
	int* max_indices);
/* FindMaxValueInColumns (NME.h:472-474): per batch and column, max over rows and its first row index. */
NB200_API int nb200_find_max_value_in_columns(void* stream, int batch, const float* x, int height, int width,
	float* max_values, int* row_indices);
/* InitMaxPooling + BlobMaxPooling (NME.h:817-822): x [batch,h,w,c] -> y [batch,ho,wo,c], no padding;
 * max_indices (optional) receives the flat in-image index of each maximum. */
NB200_API int nb200_blob_max_pooling(void* stream, int batch, int h, int w, int c, int filter_h, int filter_w,
	int stride_h, int stride_w, const float* x, float* y, int* max_indices);
/* BlobResizeImage with constant padding (NME.h:708-716) followed by BlobMaxPooling (NME.h:817-822) as one pass: the
 * windows slide over x [batch,h,w,c] surrounded by pad_* rows / columns of pad_value; y is what pooling the padded
 * image would give, the padded image is never written.  3x3 windows with stride 2 and c % 4 == 0 only (the padded stem
 * pool of the ResNets); NB200_EINVAL for any other form: pad and pool with the two calls then. */
NB200_API int nb200_blob_max_pooling_padded(void* stream, int batch, int h, int w, int c, int pad_left, int pad_right,
	int pad_top, int pad_bottom, float pad_value, int filter_h, int filter_w, int stride_h, int stride_w, const float* x,
	float* y);
/* InitMeanPooling + BlobMeanPooling (NME.h:837-841). */
NB200_API int nb200_blob_mean_pooling(void* stream, int batch, int h, int w, int c, int filter_h, int filter_w,
	int stride_h, int stride_w, const float* x, float* y);
/* BlobResizeImage (NME.h:705-710): positive deltas pad, negative crop; padding 0 = constant(default_value),
 * 1 = edge, 2 = reflect (TBlobResizePadding, NME.h:61-66).  x [batch,h,w,c] -> y [batch,h+dt+db,w+dl+dr,c]. */
NB200_API int nb200_blob_resize_image(void* stream, int batch, int h, int w, int c, int delta_left, int delta_right,
	int delta_top, int delta_bottom, int padding, float default_value, const float* x, float* y);

#ifdef __cplusplus
}
#endif
#endif /* NEOML_B200_H */
