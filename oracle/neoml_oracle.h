/* TEST INFRASTRUCTURE ONLY -- not part of the product path.
 *
 * Plain-C restatement of what the NeoML CPU math engine computes for the operations on the inference hot path.
 * Every function follows the definition the reference implements (file:line cited at each definition in
 * neoml_oracle.c) with sums carried in double precision and rounded once, so it is the "exact" answer the
 * fp32 implementations (the reference CPU engine and the B200 kernels) are both measured against.
 * Pinned against the reference CPU engine itself: tests/golden/ holds outputs of the reference engine built from
 * its own sources (oracle/Makefile target `ref`), and tests/test_oracle.py checks this file against them.
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may load this library.
 */
#ifndef NEOML_ORACLE_H
#define NEOML_ORACLE_H

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_ACT_NONE = 0, ORACLE_ACT_RELU = 1, ORACLE_ACT_HSWISH = 2 };

void oracle_multiply_matrix_by_transposed_matrix(const float* a, int m, int k, int lda, const float* b, int n,
	int ldb, float* c, int ldc);
void oracle_multiply_matrix_by_matrix(int batch, const float* a, int m, int k, const float* b, int n, float* c);
void oracle_blob_convolution(int batch, int h, int w, int c, int k, int r, int s, int pad_h, int pad_w,
	int stride_h, int stride_w, int dil_h, int dil_w, const float* x, const float* filter, const float* free_term,
	float* y);
void oracle_blob_channelwise_convolution(int batch, int h, int w, int c, int r, int s, int pad_h, int pad_w,
	int stride_h, int stride_w, const float* x, const float* filter, const float* free_term, float* y);
void oracle_mobilenetv2_block(int batch, int h, int w, int c_in, int c_exp, int c_out, int stride, int residual,
	int act_exp, float act_exp_param, int act_dw, float act_dw_param, const float* x, const float* w_exp,
	const float* b_exp, const float* w_dw, const float* b_dw, const float* w_down, const float* b_down, float* y);
void oracle_vector_op(int op, const float* a, const float* b, float scalar, float* y, int count);
void oracle_add_vector_to_matrix_rows(int batch, const float* x, float* y, int height, int width, const float* v);
void oracle_add_vector_to_matrix_columns(const float* x, float* y, int height, int width, const float* v);
void oracle_sum_matrix_rows(int batch, float* y, const float* x, int height, int width, int add);
void oracle_sum_matrix_columns(float* y, const float* x, int height, int width);
void oracle_multiply_diag_matrix_by_matrix(const float* d, int height, const float* x, int width, float* y);
void oracle_multiply_matrix_by_diag_matrix(int batch, const float* x, int height, int width, const float* d,
	int diag_stride, float* y);
void oracle_matrix_softmax_by_rows(const float* x, int height, int width, float* y);
void oracle_transpose_matrix(int batch, const float* x, int height, int medium, int width, int channels, float* y);
void oracle_find_max_value_in_rows(const float* x, int height, int width, float* max_values, int* max_indices);
void oracle_find_max_value_in_columns(int batch, const float* x, int height, int width, float* max_values,
	int* row_indices);
void oracle_blob_max_pooling(int batch, int h, int w, int c, int fh, int fw, int sh, int sw, const float* x,
	float* y, int* max_indices);
void oracle_blob_mean_pooling(int batch, int h, int w, int c, int fh, int fw, int sh, int sw, const float* x,
	float* y);
void oracle_blob_resize_image(int batch, int h, int w, int c, int dl, int dr, int dt, int db, int padding,
	float default_value, const float* x, float* y);

#ifdef __cplusplus
}
#endif
#endif
