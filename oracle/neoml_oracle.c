/* TEST INFRASTRUCTURE ONLY -- see neoml_oracle.h.  Citations are paths inside the NeoML repository. */
#include "neoml_oracle.h"

#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

static float act_apply(float v, int act, float param)
{
	/* NeoMathEngine/src/CPU/Rowwise/CpuRowwiseMobileNetV2.h:151-295 applies ReLU(threshold) or HSwish between stages;
	   ReLU semantics: NeoMathEngine/include/NeoMathEngine/NeoMathEngine.h:143-145 */
	if(act == ORACLE_ACT_RELU) {
		v = v > 0.f ? v : 0.f;
		if(param > 0.f && v > param) v = param;
	} else if(act == ORACLE_ACT_HSWISH) {
		if(v <= -3.f) v = 0.f;
		else if(v < 3.f) v = v * (v + 3.f) / 6.f;
	}
	return v;
}

/* C = A * B^T with independent leading dimensions.
   NeoMathEngine/src/CPU/CpuMathEngineBlas.cpp:906-938 -> x86/CpuX86MathEngineBlasMkl.cpp:125-159 (sgemm NoTrans/Trans) */
void oracle_multiply_matrix_by_transposed_matrix(const float* a, int m, int k, int lda, const float* b, int n,
	int ldb, float* c, int ldc)
{
	for(int i = 0; i < m; ++i) {
		for(int j = 0; j < n; ++j) {
			double acc = 0.0;
			const float* ar = a + (size_t)i * lda;
			const float* br = b + (size_t)j * ldb;
			for(int t = 0; t < k; ++t) acc += (double)ar[t] * (double)br[t];
			c[(size_t)i * ldc + j] = (float)acc;
		}
	}
}

/* Batched C_b = A_b * B_b, dense row-major.  NeoMathEngine/src/CPU/CpuMathEngineBlas.cpp:846-864 */
void oracle_multiply_matrix_by_matrix(int batch, const float* a, int m, int k, const float* b, int n, float* c)
{
	double* row = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
	for(int bi = 0; bi < batch; ++bi) {
		const float* A = a + (size_t)bi * m * k;
		const float* B = b + (size_t)bi * k * n;
		float* C = c + (size_t)bi * m * n;
		for(int i = 0; i < m; ++i) {
			for(int j = 0; j < n; ++j) row[j] = 0.0;
			for(int t = 0; t < k; ++t) {
				const double av = A[(size_t)i * k + t];
				const float* br = B + (size_t)t * n;
				for(int j = 0; j < n; ++j) row[j] += av * (double)br[j];
			}
			for(int j = 0; j < n; ++j) C[(size_t)i * n + j] = (float)row[j];
		}
	}
	free(row);
}

/* Channels-last convolution with zero padding and dilation; filter layout [k][r][s][c].
   Definition: NeoMathEngine/src/CPU/CpuMathEngineDnnConv.cpp:43-73 (output size), :305-431 (im2col + sgemm + free term);
   the same sum is spelled out naively in NeoMathEngine/test/src/common/MeTestCommon.h:67-105. */
void oracle_blob_convolution(int batch, int h, int w, int c, int k, int r, int s, int pad_h, int pad_w,
	int stride_h, int stride_w, int dil_h, int dil_w, const float* x, const float* filter, const float* free_term,
	float* y)
{
	const int ho = 1 + (h - (r - 1) * dil_h - 1 + 2 * pad_h) / stride_h;
	const int wo = 1 + (w - (s - 1) * dil_w - 1 + 2 * pad_w) / stride_w;
	for(int n = 0; n < batch; ++n) {
		for(int oy = 0; oy < ho; ++oy) {
			for(int ox = 0; ox < wo; ++ox) {
				float* out = y + (((size_t)n * ho + oy) * wo + ox) * k;
				for(int f = 0; f < k; ++f) {
					double acc = free_term != NULL ? (double)free_term[f] : 0.0;
					for(int fy = 0; fy < r; ++fy) {
						const int iy = oy * stride_h - pad_h + fy * dil_h;
						if(iy < 0 || iy >= h) continue;
						for(int fx = 0; fx < s; ++fx) {
							const int ix = ox * stride_w - pad_w + fx * dil_w;
							if(ix < 0 || ix >= w) continue;
							const float* in = x + (((size_t)n * h + iy) * w + ix) * c;
							const float* fl = filter + (((size_t)f * r + fy) * s + fx) * c;
							for(int ch = 0; ch < c; ++ch) acc += (double)in[ch] * (double)fl[ch];
						}
					}
					out[f] = (float)acc;
				}
			}
		}
	}
}

/* Depthwise convolution, filter layout [r][s][c].
   NeoMathEngine/src/CPU/CpuMathEngineDnnChannelwiseConv.cpp:31-61 and CpuMathEngineDnnChannelwiseConv.h:294-... */
void oracle_blob_channelwise_convolution(int batch, int h, int w, int c, int r, int s, int pad_h, int pad_w,
	int stride_h, int stride_w, const float* x, const float* filter, const float* free_term, float* y)
{
	const int ho = 1 + (h - r + 2 * pad_h) / stride_h;
	const int wo = 1 + (w - s + 2 * pad_w) / stride_w;
	for(int n = 0; n < batch; ++n) {
		for(int oy = 0; oy < ho; ++oy) {
			for(int ox = 0; ox < wo; ++ox) {
				float* out = y + (((size_t)n * ho + oy) * wo + ox) * c;
				for(int ch = 0; ch < c; ++ch) {
					double acc = free_term != NULL ? (double)free_term[ch] : 0.0;
					for(int fy = 0; fy < r; ++fy) {
						const int iy = oy * stride_h - pad_h + fy;
						if(iy < 0 || iy >= h) continue;
						for(int fx = 0; fx < s; ++fx) {
							const int ix = ox * stride_w - pad_w + fx;
							if(ix < 0 || ix >= w) continue;
							acc += (double)x[(((size_t)n * h + iy) * w + ix) * c + ch]
								* (double)filter[((size_t)fy * s + fx) * c + ch];
						}
					}
					out[ch] = (float)acc;
				}
			}
		}
	}
}

/* y = [x +] W_down * act2(dw3x3(act1(W_exp * x + b_exp)) + b_dw) + b_down.
   NeoMathEngine/src/CPU/CpuMathEngineDnnRowwise.cpp:287-325 and Rowwise/CpuRowwiseMobileNetV2.h:151-295;
   the unfused composite the reference tests compare against: NeoML/test/src/DnnMobileNetV2BlockTest.cpp:23-106.
   Intermediates are kept in fp32 like both reference paths do. */
void oracle_mobilenetv2_block(int batch, int h, int w, int c_in, int c_exp, int c_out, int stride, int residual,
	int act_exp, float act_exp_param, int act_dw, float act_dw_param, const float* x, const float* w_exp,
	const float* b_exp, const float* w_dw, const float* b_dw, const float* w_down, const float* b_down, float* y)
{
	const int ho = 1 + (h - 3 + 2) / stride;
	const int wo = 1 + (w - 3 + 2) / stride;
	float* e = (float*)malloc(sizeof(float) * (size_t)h * w * c_exp);
	float* d = (float*)malloc(sizeof(float) * (size_t)ho * wo * c_exp);
	for(int n = 0; n < batch; ++n) {
		const float* xi = x + (size_t)n * h * w * c_in;
		float* yi = y + (size_t)n * ho * wo * c_out;
		oracle_multiply_matrix_by_transposed_matrix(xi, h * w, c_in, c_in, w_exp, c_exp, c_in, e, c_exp);
		for(size_t i = 0; i < (size_t)h * w; ++i) {
			for(int ch = 0; ch < c_exp; ++ch) {
				float v = e[i * c_exp + ch] + (b_exp != NULL ? b_exp[ch] : 0.f);
				e[i * c_exp + ch] = act_apply(v, act_exp, act_exp_param);
			}
		}
		oracle_blob_channelwise_convolution(1, h, w, c_exp, 3, 3, 1, 1, stride, stride, e, w_dw, b_dw, d);
		for(size_t i = 0; i < (size_t)ho * wo * c_exp; ++i) d[i] = act_apply(d[i], act_dw, act_dw_param);
		for(size_t i = 0; i < (size_t)ho * wo; ++i) {
			for(int o = 0; o < c_out; ++o) {
				double acc = b_down != NULL ? (double)b_down[o] : 0.0;
				for(int ch = 0; ch < c_exp; ++ch) acc += (double)d[i * c_exp + ch] * (double)w_down[(size_t)o * c_exp + ch];
				if(residual) acc += (double)xi[i * c_in + o];
				yi[i * c_out + o] = (float)acc;
			}
		}
	}
	free(e);
	free(d);
}

/* Elementwise family; `op` uses the NB200_VEC_* numbering of include/neoml_b200.h.
   NeoMathEngine/src/CPU/CpuMathEngineVectorMath.cpp and x86/CpuX86MathEngineVectorMath.cpp (one function per op). */
void oracle_vector_op(int op, const float* a, const float* b, float s, float* y, int count)
{
	for(int i = 0; i < count; ++i) {
		const float av = a != NULL ? a[i] : 0.f;
		const float bv = b != NULL ? b[i] : 0.f;
		float r = 0.f;
		switch(op) {
			case 0: r = av; break;
			case 1: case 2: r = s; break;
			case 3: r = av + bv; break;
			case 4: r = av - bv; break;
			case 5: r = av * bv; break;
			case 6: r = av * s; break;
			case 7: r = -av * s; break;
			case 8: r = av + s; break;
			case 9: r = av > 0.f ? av : 0.f; if(s > 0.f && r > s) r = s; break;
			case 10: r = (float)(1.0 / (1.0 + exp(-(double)av))); break;
			case 11: r = (float)sqrt((double)av); break;
			case 12: r = 1.f / av; break;
			case 13: r = (float)tanh((double)av); break;
			case 14: { double t = av; if(t < -87.3365) t = -87.3365; if(t > 88.0) t = 88.0; r = (float)exp(t); break; }
			case 15: r = act_apply(av, ORACLE_ACT_HSWISH, 0.f); break;
			case 16: r = av > bv ? av : bv; break;
			case 17: r = av / bv; break;
			case 18: r = av + bv * s; break;
			default: break;
		}
		y[i] = r;
	}
}

/* NeoMathEngine/src/CPU/CpuMathEngineBlas.cpp (AddVectorToMatrixRows): rows of batch b get v[b*width ...] */
void oracle_add_vector_to_matrix_rows(int batch, const float* x, float* y, int height, int width, const float* v)
{
	for(int b = 0; b < batch; ++b)
		for(int i = 0; i < height; ++i)
			for(int j = 0; j < width; ++j) {
				const size_t o = ((size_t)b * height + i) * width + j;
				y[o] = x[o] + v[(size_t)b * width + j];
			}
}

void oracle_add_vector_to_matrix_columns(const float* x, float* y, int height, int width, const float* v)
{
	for(int i = 0; i < height; ++i)
		for(int j = 0; j < width; ++j) y[(size_t)i * width + j] = x[(size_t)i * width + j] + v[i];
}

/* result[b][w] (+)= sum_h matrix[b][h][w]   (SumMatrixRows / SumMatrixRowsAdd) */
void oracle_sum_matrix_rows(int batch, float* y, const float* x, int height, int width, int add)
{
	for(int b = 0; b < batch; ++b)
		for(int j = 0; j < width; ++j) {
			double acc = add ? (double)y[(size_t)b * width + j] : 0.0;
			for(int i = 0; i < height; ++i) acc += (double)x[((size_t)b * height + i) * width + j];
			y[(size_t)b * width + j] = (float)acc;
		}
}

void oracle_sum_matrix_columns(float* y, const float* x, int height, int width)
{
	for(int i = 0; i < height; ++i) {
		double acc = 0.0;
		for(int j = 0; j < width; ++j) acc += (double)x[(size_t)i * width + j];
		y[i] = (float)acc;
	}
}

void oracle_multiply_diag_matrix_by_matrix(const float* d, int height, const float* x, int width, float* y)
{
	for(int i = 0; i < height; ++i)
		for(int j = 0; j < width; ++j) y[(size_t)i * width + j] = d[i] * x[(size_t)i * width + j];
}

void oracle_multiply_matrix_by_diag_matrix(int batch, const float* x, int height, int width, const float* d,
	int diag_stride, float* y)
{
	for(int b = 0; b < batch; ++b)
		for(int i = 0; i < height; ++i)
			for(int j = 0; j < width; ++j) {
				const size_t o = ((size_t)b * height + i) * width + j;
				y[o] = x[o] * d[(size_t)b * diag_stride + j];
			}
}

/* Row softmax with max subtraction.  NeoMathEngine/src/CPU/CpuMathEngineBlas.cpp:1131-1159 (MlasComputeSoftmax or
   the ExponentFunc loop); naive form in NeoMathEngine/test/src/common/MeTestCommon.h:344-387. */
void oracle_matrix_softmax_by_rows(const float* x, int height, int width, float* y)
{
	for(int i = 0; i < height; ++i) {
		const float* row = x + (size_t)i * width;
		float* out = y + (size_t)i * width;
		float mx = row[0];
		for(int j = 1; j < width; ++j) if(row[j] > mx) mx = row[j];
		double sum = 0.0;
		for(int j = 0; j < width; ++j) sum += exp((double)row[j] - (double)mx);
		for(int j = 0; j < width; ++j) out[j] = (float)(exp((double)row[j] - (double)mx) / sum);
	}
}

/* x[b][h][m][w][c] -> y[b][w][m][h][c].  NeoMathEngine/src/GPU/CUDA/Kernels/CudaBlasKernels.h:982-1004 and
   the CPU twin in CpuMathEngineBlas.cpp (TransposeMatrix). */
void oracle_transpose_matrix(int batch, const float* x, int height, int medium, int width, int channels, float* y)
{
	for(int b = 0; b < batch; ++b)
		for(int hh = 0; hh < height; ++hh)
			for(int m = 0; m < medium; ++m)
				for(int ww = 0; ww < width; ++ww)
					for(int c = 0; c < channels; ++c) {
						const size_t src = ((((size_t)b * height + hh) * medium + m) * width + ww) * channels + c;
						const size_t dst = ((((size_t)b * width + ww) * medium + m) * height + hh) * channels + c;
						y[dst] = x[src];
					}
}

/* First maximum wins.  NeoMathEngine/src/CPU/x86/CpuX86MathEngineBlas.cpp:52-57,191-196 */
void oracle_find_max_value_in_rows(const float* x, int height, int width, float* max_values, int* max_indices)
{
	for(int i = 0; i < height; ++i) {
		const float* row = x + (size_t)i * width;
		int best = 0;
		for(int j = 1; j < width; ++j) if(row[j] > row[best]) best = j;
		max_values[i] = row[best];
		if(max_indices != NULL) max_indices[i] = best;
	}
}

void oracle_find_max_value_in_columns(int batch, const float* x, int height, int width, float* max_values,
	int* row_indices)
{
	for(int b = 0; b < batch; ++b)
		for(int j = 0; j < width; ++j) {
			const float* col = x + (size_t)b * height * width + j;
			int best = 0;
			for(int i = 1; i < height; ++i) if(col[(size_t)i * width] > col[(size_t)best * width]) best = i;
			max_values[(size_t)b * width + j] = col[(size_t)best * width];
			if(row_indices != NULL) row_indices[(size_t)b * width + j] = best;
		}
}

/* No padding; output (h - f)/s + 1.  NeoMathEngine/src/CPU/CpuMathEngineDnnPooling.cpp (BlobMaxPooling):
   indices are offsets inside the input image (pixel * channels + channel). */
void oracle_blob_max_pooling(int batch, int h, int w, int c, int fh, int fw, int sh, int sw, const float* x,
	float* y, int* max_indices)
{
	const int ho = (h - fh) / sh + 1, wo = (w - fw) / sw + 1;
	for(int n = 0; n < batch; ++n)
		for(int oy = 0; oy < ho; ++oy)
			for(int ox = 0; ox < wo; ++ox)
				for(int ch = 0; ch < c; ++ch) {
					float best = -FLT_MAX;
					int bestIdx = 0;
					for(int fy = 0; fy < fh; ++fy)
						for(int fx = 0; fx < fw; ++fx) {
							const int pix = (oy * sh + fy) * w + ox * sw + fx;
							const float v = x[((size_t)n * h * w + pix) * c + ch];
							if((fy == 0 && fx == 0) || v > best) { best = v; bestIdx = pix * c + ch; }
						}
					const size_t o = (((size_t)n * ho + oy) * wo + ox) * c + ch;
					y[o] = best;
					if(max_indices != NULL) max_indices[o] = bestIdx;
				}
}

void oracle_blob_mean_pooling(int batch, int h, int w, int c, int fh, int fw, int sh, int sw, const float* x,
	float* y)
{
	const int ho = (h - fh) / sh + 1, wo = (w - fw) / sw + 1;
	for(int n = 0; n < batch; ++n)
		for(int oy = 0; oy < ho; ++oy)
			for(int ox = 0; ox < wo; ++ox)
				for(int ch = 0; ch < c; ++ch) {
					double acc = 0.0;
					for(int fy = 0; fy < fh; ++fy)
						for(int fx = 0; fx < fw; ++fx)
							acc += (double)x[((size_t)n * h * w + (size_t)(oy * sh + fy) * w + ox * sw + fx) * c + ch];
					y[(((size_t)n * ho + oy) * wo + ox) * c + ch] = (float)(acc / (double)(fh * fw));
				}
}

/* Positive deltas pad, negative crop; padding 0 constant, 1 edge, 2 reflect.
   NeoMathEngine/src/CPU/CpuMathEngineDnnRowwise.cpp:337-356, Rowwise/CpuRowwiseResizeImage.h:104-260 */
void oracle_blob_resize_image(int batch, int h, int w, int c, int dl, int dr, int dt, int db, int padding,
	float default_value, const float* x, float* y)
{
	const int ho = h + dt + db, wo = w + dl + dr;
	for(int n = 0; n < batch; ++n)
		for(int oy = 0; oy < ho; ++oy)
			for(int ox = 0; ox < wo; ++ox) {
				int iy = oy - dt, ix = ox - dl;
				int inside = iy >= 0 && iy < h && ix >= 0 && ix < w;
				if(!inside && padding != 0) {
					if(padding == 1) {
						iy = iy < 0 ? 0 : (iy >= h ? h - 1 : iy);
						ix = ix < 0 ? 0 : (ix >= w ? w - 1 : ix);
					} else {
						if(iy < 0) iy = -iy; else if(iy >= h) iy = 2 * (h - 1) - iy;
						if(ix < 0) ix = -ix; else if(ix >= w) ix = 2 * (w - 1) - ix;
						iy = iy < 0 ? 0 : (iy >= h ? h - 1 : iy);
						ix = ix < 0 ? 0 : (ix >= w ? w - 1 : ix);
					}
					inside = 1;
				}
				float* out = y + (((size_t)n * ho + oy) * wo + ox) * c;
				for(int ch = 0; ch < c; ++ch)
					out[ch] = inside ? x[(((size_t)n * h + iy) * w + ix) * c + ch] : default_value;
			}
}
