// C-ABI entry points for the dense contractions: argument checks, then one description for the shared kernels.
#include "contraction.cuh"
#include "diagnostics.h"

using namespace nb200;

namespace {

void fill_epilogue(ContractionParams& p, const nb200_epilogue* epi)
{
	p.bias = nullptr;
	p.residual = nullptr;
	p.ldr = 0;
	p.act = NB200_ACT_NONE;
	p.act_param = 0.f;
	p.act_param_device = nullptr;
	p.accumulate = 0;
	if(epi != nullptr) {
		p.bias = epi->bias;
		p.residual = epi->residual;
		p.ldr = epi->ld_residual;
		p.act = epi->act;
		p.act_param = epi->act_param;
		p.act_param_device = epi->act_param_device;
		p.accumulate = epi->accumulate;
	}
}

bool vec_ok(const void* base, long long ld, long long batchStride)
{
	return aligned16(base) && (ld % 4) == 0 && (batchStride % 4) == 0;
}

int run(ContractionParams& p, int batch, void* stream, int precision)
{
	if(precision != NB200_PREC_3XTF32 && precision != NB200_PREC_TF32 && precision != NB200_PREC_FP32_SIMT) {
		return NB200_EINVAL;
	}
	if(p.M == 0 || p.N == 0 || batch == 0) return NB200_OK;
	if(p.A == nullptr || p.B == nullptr || p.C == nullptr) return NB200_EINVAL;
	// the kernels index each operand of one batch entry with 32-bit element offsets (NeoML blobs are < 2^31 elements)
	if(static_cast<long long>(p.M) * (p.a_mode == A_ROWS ? p.lda : 1) > 0x7fffffffLL
		|| static_cast<long long>(p.M) * p.ldc > 0x7fffffffLL) {
		return NB200_ETOOBIG;
	}
	p.precision = precision;
	p.stages = 0;
	p.status = device_status_word();
	if(p.status == nullptr) return NB200_ENODEVICE;
	p.c_vec = vec_ok(p.C, p.ldc, p.strideC) && (p.bias == nullptr || aligned16(p.bias))
		&& (p.residual == nullptr || vec_ok(p.residual, p.ldr, p.strideC)) ? 1 : 0;
	if(precision == NB200_PREC_FP32_SIMT) return launch_contraction_simt(p, batch, as_stream(stream));
	return launch_contraction_tc(p, batch, as_stream(stream));
}

} // namespace

// y[pixel][0..cOut) = x[pixel][0..cIn), zero beyond: widens a channels-last blob (or filter) to a multiple of four
// channels so that every filter tap is one aligned 16-byte piece
__global__ void __launch_bounds__(256) pad_channels_kernel(const float* __restrict__ x, float* __restrict__ y,
	long long pixels, int cIn, int cOut)
{
	const long long total = pixels * cOut;
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
		const long long px = i / cOut;
		const int c = static_cast<int>(i - px * cOut);
		y[i] = c < cIn ? __ldg(x + px * cIn + c) : 0.f;
	}
}

// Prepares the filter for the tensor-core kernel once per call, so that no CTA has to convert its B tiles:
// mode 0 (3xTF32): y = x - trunc_tf32(x), the "lo" part of the split (the filter itself serves as "hi");
// mode 1 (TF32):   y = x rounded to the nearest TF32.
__global__ void __launch_bounds__(256) prepare_filter_kernel(const float* __restrict__ x, float* __restrict__ y,
	long long n, int mode)
{
	// the scratch this writes may still be read by the convolution before it in the stream
	dependent_wait();
	dependents_may_start();
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
		const float v = __ldg(x + i);
		y[i] = mode == 0 ? v - __uint_as_float(__float_as_uint(v) & 0xffffe000u) : to_tf32(v);
	}
}

// Room for the partial results of a split-K launch: only launches with few tiles split (at most 74 tiles of 128 x 128
// outputs, cut in as many parts as fill the machine), so the product of parts and outputs is bounded.
constexpr long long SPLIT_TILES_MAX = 74;
// Rows of the first operand (output positions of a convolution) from which preparing the second one pays (8 row tiles:
// every prepared tile is then used eight times).  Attention's per-head products (512 rows) and the late layers of a
// network at batch 1 are faster with the conversion left in the kernel (measured).
constexpr int PREPARE_B_MIN_ROWS = 1024;
constexpr size_t SPLIT_SCRATCH_FLOATS = static_cast<size_t>(148) * 128 * 128;

size_t split_scratch_floats(long long outRows, long long n, long long kk)
{
	const long long tiles = ((outRows + 127) / 128) * ((n + 127) / 128);
	return tiles <= SPLIT_TILES_MAX && kk >= 256 && n % 4 == 0 ? SPLIT_SCRATCH_FLOATS + 8 : 0;
}

// floats of scratch for the prepared filter (rounded up so that what follows stays 16-byte aligned)
size_t prepared_filter_floats(long long k, long long r, long long s, long long c)
{
	return static_cast<size_t>((k * r * s * c + 3) / 4 * 4);
}

// Row-window form of a convolution with few channels (the network stem): the image is copied once with its spatial
// zero padding and its channels widened to a multiple of four, so that the S taps of one filter row are ONE contiguous
// run of at most 32 floats per output position; the filter rows are widened to 32 floats with zeros.
struct WindowPlan {
	int c4, taps, hp, wp; // padded channels, pixels per 128-byte window, padded image height and width
	size_t imageFloats, filterFloats;
};

bool plan_row_window(const nb200_conv_desc* d, WindowPlan* w)
{
	if(d->c <= 0 || d->c >= 32 || d->dil_h != 1 || d->dil_w != 1 || d->wo > 128 || d->wo <= 0 || d->ho <= 0) return false;
	w->c4 = (d->c + 3) / 4 * 4;
	if(d->s * w->c4 > 32 || 32 % w->c4 != 0) return false;
	if(d->r == 1 && d->s == 1) return false; // a pointwise convolution is a plain matrix product already
	w->taps = 32 / w->c4;
	const int needW = (d->wo - 1) * d->stride_w + w->taps, needH = (d->ho - 1) * d->stride_h + d->r;
	w->wp = d->w + 2 * d->pad_w > needW ? d->w + 2 * d->pad_w : needW;
	w->hp = d->h + 2 * d->pad_h > needH ? d->h + 2 * d->pad_h : needH;
	w->imageFloats = static_cast<size_t>(d->batch) * w->hp * w->wp * w->c4;
	w->filterFloats = static_cast<size_t>(d->k) * d->r * 32;
	return w->imageFloats <= 0x7fffffffULL;
}

// y[n][yp][xp][0..c4) = x[n][yp - padH][xp - padW][0..c) inside the image, 0 elsewhere
__global__ void __launch_bounds__(256) pad_image_kernel(const float* __restrict__ x, float* __restrict__ y, int batch,
	int h, int w, int c, int hp, int wp, int c4, int padH, int padW)
{
	const long long total = static_cast<long long>(batch) * hp * wp * (c4 / 4);
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
		const int q = static_cast<int>(i % (c4 / 4));
		long long px = i / (c4 / 4);
		const int xp = static_cast<int>(px % wp); px /= wp;
		const int yp = static_cast<int>(px % hp);
		const int n = static_cast<int>(px / hp);
		const int sy = yp - padH, sx = xp - padW;
		float v[4] = { 0.f, 0.f, 0.f, 0.f };
		if(sy >= 0 && sy < h && sx >= 0 && sx < w) {
			const float* src = x + ((static_cast<long long>(n) * h + sy) * w + sx) * c;
#pragma unroll
			for(int e = 0; e < 4; ++e) if(4 * q + e < c) v[e] = __ldg(src + 4 * q + e);
		}
		reinterpret_cast<float4*>(y)[i] = make_float4(v[0], v[1], v[2], v[3]);
	}
}

// y[k][r][j] for j < 32: tap j / c4, channel j % c4 of filter row r, zero beyond the real taps and channels
__global__ void __launch_bounds__(256) widen_filter_rows_kernel(const float* __restrict__ f, float* __restrict__ y,
	int kCount, int r, int s, int c, int c4)
{
	const int total = kCount * r * 32;
	for(int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
		const int j = i & 31;
		const int row = i >> 5; // k * r + filter row
		const int tap = j / c4, ch = j - tap * c4;
		y[i] = (tap < s && ch < c) ? __ldg(f + (static_cast<long long>(row) * s + tap) * c + ch) : 0.f;
	}
}

// the two filter forms of the row-window path: rows widened to 32 floats, then their lo parts / rounded copies
void prepare_window_filter(void* stream, const nb200_conv_desc* d, const WindowPlan* win, const float* filter, float* out,
	int precision)
{
	widen_filter_rows_kernel<<<grid_for(static_cast<long long>(win->filterFloats), 256, 8), 256, 0, as_stream(stream)>>>(
		filter, out, d->k, d->r, d->s, d->c, win->c4);
	prepare_filter_kernel<<<grid_for(static_cast<long long>(win->filterFloats), 256, 8), 256, 0, as_stream(stream)>>>(
		out, out + win->filterFloats, static_cast<long long>(win->filterFloats), precision == NB200_PREC_3XTF32 ? 0 : 1);
	count_launch(2);
}

bool wants_channel_padding(const nb200_conv_desc* d)
{
	const bool pointwise = d->r == 1 && d->s == 1 && d->pad_h == 0 && d->pad_w == 0 && d->stride_h == 1 && d->stride_w == 1;
	return !pointwise && d->c % 4 != 0;
}

namespace nb200 {

size_t convolution_scratch_floats(const nb200_conv_desc* d, bool withSplitRoom)
{
	if(d == nullptr || d->c <= 0 || d->k <= 0 || d->r <= 0 || d->s <= 0) return 0;
	const size_t c4 = static_cast<size_t>((d->c + 3) / 4 * 4);
	// the prepared filter (always), and for channel counts that are not a multiple of four the widened image and filter
	WindowPlan win;
	if(plan_row_window(d, &win)) return win.imageFloats + 2 * win.filterFloats + 16;
	size_t floats = prepared_filter_floats(d->k, d->r, d->s, static_cast<long long>(c4)) + 8;
	if(wants_channel_padding(d)) floats += (static_cast<size_t>(d->batch) * d->h * d->w + static_cast<size_t>(d->k) * d->r * d->s) * c4 + 8;
	// last, so that a caller with less room loses only the split
	if(withSplitRoom && d->ho > 0 && d->wo > 0) {
		floats += split_scratch_floats(static_cast<long long>(d->batch) * d->ho * d->wo, d->k, static_cast<long long>(d->r) * d->s * c4);
	}
	return floats;
}

} // namespace nb200

extern "C" {

size_t nb200_blob_convolution_scratch_floats(const nb200_conv_desc* d)
{
	return convolution_scratch_floats(d, true);
}

void nb200_debug_set_contraction_trace(void* device_buffer, int steps, int skip_mask)
{
	set_contraction_trace(static_cast<unsigned long long*>(device_buffer), steps, skip_mask);
}

void nb200_debug_time_contractions(int enable)
{
	time_contractions(enable != 0);
}

int nb200_debug_contraction_times(float* ms, int capacity)
{
	if(ms == nullptr || capacity < 0) return NB200_EINVAL;
	return contraction_times(ms, nullptr, capacity);
}

int nb200_debug_contraction_records(float* ms, double* flops, int capacity)
{
	if(ms == nullptr || flops == nullptr || capacity < 0) return NB200_EINVAL;
	return contraction_times(ms, flops, capacity);
}

int nb200_multiply_matrix_by_transposed_matrix(void* stream, const float* a, int m, int k, int lda,
	const float* b, int n, int ldb, float* c, int ldc, const nb200_epilogue* epi, int precision)
{
	if(m < 0 || n < 0 || k <= 0 || lda < k || ldb < k || ldc < n) return NB200_EINVAL;
	set_call_flops(2.0 * m * n * k);
	ContractionParams p = {};
	p.A = a; p.B = b; p.C = c;
	p.M = m; p.N = n; p.K = k;
	p.lda = lda; p.ldb = ldb; p.ldc = ldc;
	p.a_mode = A_ROWS; p.b_mode = B_ROWS;
	fill_epilogue(p, epi);
	if(p.residual == nullptr) p.ldr = ldc;
	p.a_vec = vec_ok(a, lda, 0); p.b_vec = vec_ok(b, ldb, 0);
	return run(p, 1, stream, precision);
}

int nb200_batch_multiply_matrix_by_transposed_matrix(void* stream, int batch, const float* a, int m,
	int k, const float* b, int n, float* c, const nb200_epilogue* epi, int precision)
{
	if(batch < 0 || m < 0 || n < 0 || k <= 0) return NB200_EINVAL;
	set_call_flops(2.0 * batch * m * n * k);
	ContractionParams p = {};
	p.A = a; p.B = b; p.C = c;
	p.M = m; p.N = n; p.K = k;
	p.lda = k; p.ldb = k; p.ldc = n;
	p.strideA = static_cast<long long>(m) * k; p.strideB = static_cast<long long>(n) * k;
	p.strideC = static_cast<long long>(m) * n;
	p.a_mode = A_ROWS; p.b_mode = B_ROWS;
	fill_epilogue(p, epi);
	if(p.residual == nullptr) p.ldr = n;
	p.a_vec = vec_ok(a, k, p.strideA); p.b_vec = vec_ok(b, k, p.strideB);
	return run(p, batch, stream, precision);
}

size_t nb200_matrix_product_scratch_floats(int batch, int m, int n, int k, int ldb)
{
	if(batch <= 0 || m <= 0 || n <= 0 || k <= 0 || ldb < k) return 0;
	size_t floats = 0;
	// the split second operand pays when it is reused by several row tiles
	if(m >= PREPARE_B_MIN_ROWS) floats += (static_cast<size_t>(batch) * n * ldb + 3) / 4 * 4 + 8;
	if(batch == 1) floats += split_scratch_floats(m, n, k);
	return floats;
}

// The product behind the three entry points below.  `prepared` (optional, batch 1): the second operand in the form
// nb200_matrix_product_prepare_second makes, kept by the caller for as long as the operand does not change.
static int matrix_product(void* stream, int batch, const float* a, int m, int k, int lda, const float* b, int n, int ldb,
	float* c, int ldc, float* scratch, const float* prepared, const nb200_epilogue* epi, int precision)
{
	if(batch < 0 || m < 0 || n < 0 || k <= 0 || lda < k || ldb < k || ldc < n) return NB200_EINVAL;
	set_call_flops(2.0 * batch * m * n * k);
	ContractionParams p = {};
	p.A = a; p.B = b; p.C = c;
	p.M = m; p.N = n; p.K = k;
	p.lda = lda; p.ldb = ldb; p.ldc = ldc;
	p.strideA = static_cast<long long>(m) * lda; p.strideB = static_cast<long long>(n) * ldb;
	p.strideC = static_cast<long long>(m) * ldc;
	p.a_mode = A_ROWS; p.b_mode = B_ROWS;
	fill_epilogue(p, epi);
	if(p.residual == nullptr) p.ldr = ldc;
	p.a_vec = vec_ok(a, lda, p.strideA); p.b_vec = vec_ok(b, ldb, p.strideB);
	const bool plain = precision == NB200_PREC_FP32_SIMT || batch == 0 || m == 0 || n == 0 || !p.a_vec || !p.b_vec
		|| static_cast<long long>(batch) * n * ldb > 0x7fffffffLL;
	if(plain || (scratch == nullptr && prepared == nullptr)) return run(p, batch, stream, precision);
	float* rest = scratch != nullptr
		? reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(scratch) + 15) & ~static_cast<uintptr_t>(15)) : nullptr;
	const bool wanted = m >= PREPARE_B_MIN_ROWS;
	const bool given = wanted && prepared != nullptr && batch == 1 && aligned16(prepared);
	const bool prepare = wanted && !given && rest != nullptr;
	if(given) {
		if(precision == NB200_PREC_3XTF32) p.Blo = prepared; else p.B = prepared;
		p.b_ready = 1;
	} else if(prepare) {
		// one pass over the second operand as it lies in memory (the floats between its rows, if any, are carried along)
		if(device_status_word() == nullptr) return NB200_ENODEVICE;
		const long long span = static_cast<long long>(batch - 1) * p.strideB + static_cast<long long>(n - 1) * ldb + k;
		launch_dependent(overlap_launches(), prepare_filter_kernel, dim3(grid_for(span, 256, 8)), dim3(256), 0, as_stream(stream),
			b, rest, span, precision == NB200_PREC_3XTF32 ? 0 : 1);
		count_launch(1);
		const int rc = check_launch();
		if(rc != NB200_OK) return rc;
		if(precision == NB200_PREC_3XTF32) p.Blo = rest; else p.B = rest;
		p.b_ready = 1;
		rest += (static_cast<size_t>(batch) * n * ldb + 3) / 4 * 4;
	}
	if(batch == 1 && rest != nullptr && split_scratch_floats(m, n, k) > 0) {
		p.splitScratch = rest;
		p.splitScratchFloats = static_cast<long long>(SPLIT_SCRATCH_FLOATS);
	}
	const int rc = run(p, batch, stream, precision);
	if(rc != NB200_EINVAL || !(prepare || given)) return rc;
	// the launcher could not describe an operand to TMA after all: in-kernel conversion, unsplit
	p.B = b; p.Blo = nullptr; p.b_ready = 0; p.splitScratch = nullptr;
	return run(p, batch, stream, precision);
}

int nb200_multiply_matrix_by_transposed_matrix_with_scratch(void* stream, int batch, const float* a, int m, int k,
	int lda, const float* b, int n, int ldb, float* c, int ldc, float* scratch, const nb200_epilogue* epi, int precision)
{
	return matrix_product(stream, batch, a, m, k, lda, b, n, ldb, c, ldc, scratch, nullptr, epi, precision);
}

size_t nb200_matrix_product_prepared_floats(int m, int n, int k, int ldb)
{
	if(m < PREPARE_B_MIN_ROWS || n <= 0 || k <= 0 || ldb < k) return 0;
	return (static_cast<size_t>(n - 1) * ldb + k + 3) / 4 * 4;
}

int nb200_matrix_product_prepare_second(void* stream, const float* b, int n, int k, int ldb, float* prepared, int precision)
{
	if(n <= 0 || k <= 0 || ldb < k || b == nullptr || prepared == nullptr || !aligned16(prepared)) return NB200_EINVAL;
	if(precision != NB200_PREC_3XTF32 && precision != NB200_PREC_TF32) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	const long long span = static_cast<long long>(n - 1) * ldb + k;
	prepare_filter_kernel<<<grid_for(span, 256, 8), 256, 0, as_stream(stream)>>>(b, prepared, span,
		precision == NB200_PREC_3XTF32 ? 0 : 1);
	count_launch(1);
	return check_launch();
}

int nb200_multiply_matrix_by_transposed_matrix_prepared(void* stream, const float* a, int m, int k, int lda, const float* b,
	int n, int ldb, float* c, int ldc, const float* prepared_b, float* scratch, const nb200_epilogue* epi, int precision)
{
	return matrix_product(stream, 1, a, m, k, lda, b, n, ldb, c, ldc, scratch, prepared_b, epi, precision);
}

int nb200_multiply_matrix_by_matrix(void* stream, int batch, const float* a, int m, int k,
	const float* b, int n, float* c, const nb200_epilogue* epi, int precision)
{
	if(batch < 0 || m < 0 || n < 0 || k <= 0) return NB200_EINVAL;
	set_call_flops(2.0 * batch * m * n * k);
	ContractionParams p = {};
	p.A = a; p.B = b; p.C = c;
	p.M = m; p.N = n; p.K = k;
	p.lda = k; p.ldb = n; p.ldc = n;
	p.strideA = static_cast<long long>(m) * k; p.strideB = static_cast<long long>(k) * n;
	p.strideC = static_cast<long long>(m) * n;
	p.a_mode = A_ROWS; p.b_mode = B_COLS;
	fill_epilogue(p, epi);
	if(p.residual == nullptr) p.ldr = n;
	p.a_vec = vec_ok(a, k, p.strideA); p.b_vec = 0;
	return run(p, batch, stream, precision);
}

int nb200_blob_convolution(void* stream, const nb200_conv_desc* d, const float* x, const float* filter, float* y,
	float* scratch, const nb200_epilogue* epi, int precision)
{
	if(d != nullptr) set_call_flops(2.0 * d->batch * d->ho * d->wo * d->k * d->r * d->s * d->c);
	return blob_convolution(stream, d, x, filter, y, scratch, scratch != nullptr ? convolution_scratch_floats(d, true) : 0,
		epi, precision, nullptr);
}

size_t nb200_blob_convolution_prepared_filter_floats(const nb200_conv_desc* d)
{
	if(d == nullptr || d->c <= 0 || d->k <= 0 || d->r <= 0 || d->s <= 0 || d->ho <= 0 || d->wo <= 0 || d->batch <= 0) return 0;
	WindowPlan win;
	if(plan_row_window(d, &win)) return 2 * win.filterFloats;
	const bool pointwise = d->r == 1 && d->s == 1 && d->pad_h == 0 && d->pad_w == 0 && d->stride_h == 1 && d->stride_w == 1;
	const long long kk = static_cast<long long>(d->r) * d->s * d->c;
	const bool tmaShape = (pointwise ? d->c % 4 == 0 : d->c % 32 == 0) && kk % 4 == 0;
	if(!tmaShape || static_cast<long long>(d->batch) * d->ho * d->wo < PREPARE_B_MIN_ROWS) return 0;
	return prepared_filter_floats(d->k, d->r, d->s, d->c);
}

int nb200_blob_convolution_prepare_filter(void* stream, const nb200_conv_desc* d, const float* filter, float* prepared,
	int precision)
{
	const size_t floats = nb200_blob_convolution_prepared_filter_floats(d);
	if(floats == 0) return NB200_OK;
	if(filter == nullptr || prepared == nullptr || !aligned16(prepared)
		|| (precision != NB200_PREC_3XTF32 && precision != NB200_PREC_TF32)) {
		return NB200_EINVAL;
	}
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	WindowPlan win;
	if(plan_row_window(d, &win)) {
		prepare_window_filter(stream, d, &win, filter, prepared, precision);
	} else {
		const long long n = static_cast<long long>(d->k) * d->r * d->s * d->c;
		prepare_filter_kernel<<<grid_for(n, 256, 8), 256, 0, as_stream(stream)>>>(filter, prepared, n,
			precision == NB200_PREC_3XTF32 ? 0 : 1);
		count_launch(1);
	}
	return check_launch();
}

int nb200_blob_convolution_with_prepared_filter(void* stream, const nb200_conv_desc* d, const float* x, const float* filter,
	const float* prepared, float* y, float* scratch, const nb200_epilogue* epi, int precision)
{
	if(d != nullptr) set_call_flops(2.0 * d->batch * d->ho * d->wo * d->k * d->r * d->s * d->c);
	return blob_convolution(stream, d, x, filter, y, scratch, scratch != nullptr ? convolution_scratch_floats(d, true) : 0,
		epi, precision, nb200_blob_convolution_prepared_filter_floats(d) > 0 ? prepared : nullptr);
}

} // extern "C"

namespace nb200 {

int blob_convolution(void* stream, const nb200_conv_desc* d, const float* x, const float* filter, float* y,
	float* scratch, size_t scratchFloats, const nb200_epilogue* epi, int precision, const float* prepared)
{
	if(d == nullptr) return NB200_EINVAL;
	WindowPlan win;
	if(scratch != nullptr && precision != NB200_PREC_FP32_SIMT && d->batch > 0 && d->k > 0 && d->r > 0 && d->s > 0
		&& d->h > 0 && d->w > 0 && d->stride_h > 0 && d->stride_w > 0 && d->pad_h >= 0 && d->pad_w >= 0
		&& d->ho == 1 + (d->h - d->r + 2 * d->pad_h) / d->stride_h && d->wo == 1 + (d->w - d->s + 2 * d->pad_w) / d->stride_w
		&& plan_row_window(d, &win) && x != nullptr && filter != nullptr && y != nullptr
		&& scratchFloats >= win.imageFloats + 2 * win.filterFloats + 16 && !gather_forced()) {
		if(device_status_word() == nullptr) return NB200_ENODEVICE;
		float* xs = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(scratch) + 15) & ~static_cast<uintptr_t>(15));
		const float* fs = prepared;
		const float* fprep = prepared != nullptr ? prepared + win.filterFloats : nullptr;
		pad_image_kernel<<<grid_for(static_cast<long long>(win.imageFloats / 4), 256, 16), 256, 0, as_stream(stream)>>>(
			x, xs, d->batch, d->h, d->w, d->c, win.hp, win.wp, win.c4, d->pad_h, d->pad_w);
		count_launch(1);
		if(prepared == nullptr) {
			float* widened = xs + (win.imageFloats + 3) / 4 * 4;
			prepare_window_filter(stream, d, &win, filter, widened, precision);
			fs = widened;
			fprep = widened + win.filterFloats;
		}
		int rc = check_launch();
		if(rc != NB200_OK) return rc;
		ContractionParams p = {};
		p.A = xs; p.B = precision == NB200_PREC_3XTF32 ? fs : fprep; p.C = y;
		p.Blo = precision == NB200_PREC_3XTF32 ? fprep : nullptr;
		p.b_ready = 1;
		p.M = d->batch * d->ho * d->wo; p.N = d->k; p.K = d->r * 32;
		p.lda = 0; p.ldb = p.K; p.ldc = d->k;
		p.a_mode = A_CONV_WINDOW; p.b_mode = B_ROWS; p.a_vec = 1; p.b_vec = 1;
		p.tileM = d->wo;
		p.H = win.hp; p.W = win.wp; p.Cin = win.c4; p.Ho = d->ho; p.Wo = d->wo; p.S = win.taps;
		p.padH = 0; p.padW = 0; p.strH = d->stride_h; p.strW = d->stride_w; p.dilH = 1; p.dilW = 1;
		fill_epilogue(p, epi);
		if(p.residual == nullptr) p.ldr = d->k;
		rc = run(p, 1, stream, precision);
		if(rc != NB200_EINVAL) return rc;
		// the tensor maps could not be built: fall through to the general paths below
	}
	if(scratch != nullptr && d->c > 0 && d->batch > 0 && wants_channel_padding(d) && precision != NB200_PREC_FP32_SIMT) {
		// channel counts that are not a multiple of four (the 3-channel stem) would be gathered element by element;
		// with scratch the image and the filter are first widened to 4-channel pixels (zeros in the new channels add
		// nothing to any sum) and the convolution runs on 16-byte pieces
		if(x == nullptr || filter == nullptr) return NB200_EINVAL;
		if(device_status_word() == nullptr) return NB200_ENODEVICE;
		const int c4 = (d->c + 3) / 4 * 4;
		const long long pixels = static_cast<long long>(d->batch) * d->h * d->w;
		const long long taps = static_cast<long long>(d->k) * d->r * d->s;
		if(pixels * c4 > 0x7fffffffLL) return NB200_ETOOBIG;
		float* xs = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(scratch) + 15) & ~static_cast<uintptr_t>(15));
		float* fs = xs + pixels * c4;
		pad_channels_kernel<<<grid_for(pixels * c4, 256, 16), 256, 0, as_stream(stream)>>>(x, xs, pixels, d->c, c4);
		pad_channels_kernel<<<grid_for(taps * c4, 256, 16), 256, 0, as_stream(stream)>>>(filter, fs, taps, d->c, c4);
		count_launch(2);
		const int rc = check_launch();
		if(rc != NB200_OK) return rc;
		nb200_conv_desc padded = *d;
		padded.c = c4;
		const size_t used = static_cast<size_t>(fs + taps * c4 - scratch);
		return blob_convolution(stream, &padded, xs, fs, y, fs + taps * c4, scratchFloats > used ? scratchFloats - used : 0,
			epi, precision, nullptr);
	}
	if(d->batch < 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->k <= 0 || d->r <= 0 || d->s <= 0
		|| d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 || d->dil_w <= 0 || d->pad_h < 0 || d->pad_w < 0) {
		return NB200_EINVAL;
	}
	// output size rule of the reference (CpuMathEngineDnnConv.cpp:59-62)
	const int ho = 1 + (d->h - (d->r - 1) * d->dil_h - 1 + 2 * d->pad_h) / d->stride_h;
	const int wo = 1 + (d->w - (d->s - 1) * d->dil_w - 1 + 2 * d->pad_w) / d->stride_w;
	if(ho != d->ho || wo != d->wo || ho <= 0 || wo <= 0) return NB200_EINVAL;
	const long long inElems = static_cast<long long>(d->batch) * d->h * d->w * d->c;
	const long long outRows = static_cast<long long>(d->batch) * ho * wo;
	const long long kk = static_cast<long long>(d->r) * d->s * d->c;
	if(inElems > 0x7fffffffLL || outRows * d->k > 0x7fffffffLL || kk > 0x7fffffffLL) return NB200_ETOOBIG;

	ContractionParams p = {};
	p.A = x; p.B = filter; p.C = y;
	p.M = static_cast<int>(outRows); p.N = d->k; p.K = static_cast<int>(kk);
	p.lda = 0; p.ldb = p.K; p.ldc = d->k;
	p.H = d->h; p.W = d->w; p.Cin = d->c; p.Ho = ho; p.Wo = wo; p.S = d->s;
	p.padH = d->pad_h; p.padW = d->pad_w; p.strH = d->stride_h; p.strW = d->stride_w;
	p.dilH = d->dil_h; p.dilW = d->dil_w;
	p.b_mode = B_ROWS;
	fill_epilogue(p, epi);
	if(p.residual == nullptr) p.ldr = d->k;
	p.b_vec = vec_ok(filter, p.K, 0);
	const bool pointwise = d->r == 1 && d->s == 1 && d->pad_h == 0 && d->pad_w == 0 && d->stride_h == 1 && d->stride_w == 1;
	if(pointwise) {
		// a 1x1/stride-1 convolution is the plain product  y[M x K] = x[M x C] * filter[K x C]^T
		p.a_mode = A_ROWS;
		p.lda = d->c;
		p.a_vec = vec_ok(x, d->c, 0);
	} else {
		// gathered rows; 16-byte copies when a chunk of four K indices never straddles a filter tap
		p.a_mode = A_CONV_TAP;
		p.a_vec = d->c % 4 == 0 && aligned16(x) ? 1 : 0;
	}
	// with scratch the filter is prepared once here (one small pass over K*R*S*C floats) instead of being converted
	// tile by tile by every CTA; needs the all-TMA pipeline: 16-byte-aligned operands and 32-channel K blocks
	p.Blo = nullptr;
	p.b_ready = 0;
	const bool tmaShape = aligned16(x) && aligned16(filter) && (pointwise ? d->c % 4 == 0 : d->c % 32 == 0) && kk % 4 == 0;
	if(scratch != nullptr && precision != NB200_PREC_FP32_SIMT && tmaShape && outRows > 0) {
		float* inScratch = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(scratch) + 15) & ~static_cast<uintptr_t>(15));
		// with few output rows (small batches) every filter tile is used by a handful of CTAs at most: the extra launch
		// costs more than converting those tiles in the kernel (ResNet-50 at batch 1: 0.69 -> 0.62 ms per pass)
		const bool prepare = outRows >= PREPARE_B_MIN_ROWS;
		if(prepare) {
			const float* ready = prepared;
			if(ready == nullptr || !aligned16(ready)) {
				const long long n = static_cast<long long>(d->k) * kk;
				launch_dependent(overlap_launches(), prepare_filter_kernel, dim3(grid_for(n, 256, 8)), dim3(256), 0, as_stream(stream),
					filter, inScratch, n, precision == NB200_PREC_3XTF32 ? 0 : 1);
				count_launch(1);
				const int rc = check_launch();
				if(rc != NB200_OK) return rc;
				ready = inScratch;
			}
			if(precision == NB200_PREC_3XTF32) p.Blo = ready; else p.B = ready;
			p.b_ready = 1;
		}
		// whatever the caller's scratch holds beyond the prepared filter is room for split-K partial results
		float* const rest = inScratch + prepared_filter_floats(d->k, d->r, d->s, d->c);
		const size_t used = static_cast<size_t>(rest - scratch);
		if(scratchFloats > used + 4 && split_scratch_floats(outRows, d->k, kk) > 0) {
			p.splitScratch = rest;
			p.splitScratchFloats = static_cast<long long>(scratchFloats - used);
			if(p.splitScratchFloats > static_cast<long long>(SPLIT_SCRATCH_FLOATS)) p.splitScratchFloats = SPLIT_SCRATCH_FLOATS;
		}
		const int rc2 = run(p, 1, stream, precision);
		if(rc2 != NB200_EINVAL) return rc2;
		// the launcher could not describe an operand to TMA after all: fall back to in-kernel conversion
		p.B = filter;
		p.Blo = nullptr;
		p.b_ready = 0;
		p.splitScratch = nullptr;
	}
	return run(p, 1, stream, precision);
}

} // namespace nb200
