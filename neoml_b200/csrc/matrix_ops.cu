// Memory-bound matrix helpers of IBlasEngine used by the inference graphs: broadcast adds, row/column sums,
// diagonal scalings, row softmax, generalised transpose, row/column arg-max.  All are HBM-bound: accesses are
// coalesced along the contiguous dimension, reductions use warp shuffles, 16-byte accesses where alignment allows.
#include "common.cuh"
#include <cooperative_groups.h>
#include <float.h>

namespace nb200 {

namespace {

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
	for(int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
	for(int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
	return v;
}

// y[b][h][w] = x[b][h][w] + v[b][w]
template<bool VEC>
__global__ void __launch_bounds__(256) add_rows_kernel(const float* __restrict__ x, float* __restrict__ y,
	const float* __restrict__ v, long long total, int width, long long perBatch)
{
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
	if(VEC) {
		const long long total4 = total >> 2;
		for(long long i = tid; i < total4; i += stride) {
			const long long e = i << 2;
			const long long b = e / perBatch;
			const int w = static_cast<int>((e - b * perBatch) % width);
			float4 a = reinterpret_cast<const float4*>(x)[i];
			const float4 c = *reinterpret_cast<const float4*>(v + b * width + w);
			a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
			reinterpret_cast<float4*>(y)[i] = a;
		}
	} else {
		for(long long e = tid; e < total; e += stride) {
			const long long b = e / perBatch;
			const int w = static_cast<int>((e - b * perBatch) % width);
			y[e] = x[e] + v[b * width + w];
		}
	}
}

// y[h][w] = x[h][w] + v[h]   /   y[h][w] = x[h][w] * v[h]  (MUL)
template<bool MUL>
__global__ void __launch_bounds__(256) row_scalar_kernel(const float* __restrict__ x, float* __restrict__ y,
	const float* __restrict__ v, long long total, int width)
{
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
		const float s = __ldg(v + e / width);
		y[e] = MUL ? x[e] * s : x[e] + s;
	}
}

// y[b][i][j] = x[b][i][j] * d[b*diagStride + j]
__global__ void __launch_bounds__(256) col_scale_kernel(const float* __restrict__ x, float* __restrict__ y,
	const float* __restrict__ d, long long total, int width, long long perBatch, int diagStride)
{
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
		const long long b = e / perBatch;
		const int j = static_cast<int>((e - b * perBatch) % width);
		y[e] = x[e] * __ldg(d + b * diagStride + j);
	}
}

// y[b][w] (+)= sum_h x[b][h][w]: a block owns 32 columns of one batch entry and a slice of the rows; threads are
// (32 columns) x (8 row lanes); partial sums meet in shared memory.  When the rows are split over several blocks
// (rowSlices > 1) those blocks form one thread-block cluster along y: the block of slice 0 reads the others' sums
// from their shared memory and adds them in slice order, so the result is the same bits on every run (no atomics).
__global__ void __launch_bounds__(256) sum_rows_kernel(float* __restrict__ y, const float* __restrict__ x,
	int height, int width, int rowSlices, int add)
{
	namespace cg = cooperative_groups;
	__shared__ float part[8][33];
	__shared__ float total[32];
	const int b = blockIdx.z;
	const int w = blockIdx.x * 32 + (threadIdx.x & 31);
	const int lane8 = threadIdx.x >> 5;
	const int slice = blockIdx.y;
	const int rowsPerSlice = (height + rowSlices - 1) / rowSlices;
	const int h0 = slice * rowsPerSlice;
	const int h1 = min(height, h0 + rowsPerSlice);
	float acc = 0.f;
	if(w < width) {
		const float* src = x + (static_cast<size_t>(b) * height) * width + w;
		for(int h = h0 + lane8; h < h1; h += 8) acc += src[static_cast<size_t>(h) * width];
	}
	part[lane8][threadIdx.x & 31] = acc;
	__syncthreads();
	float s = 0.f;
	if(lane8 == 0) {
#pragma unroll
		for(int i = 0; i < 8; ++i) s += part[i][threadIdx.x];
		total[threadIdx.x] = s;
	}
	if(rowSlices > 1) {
		cg::cluster_group cluster = cg::this_cluster();
		cluster.sync();
		if(slice == 0 && lane8 == 0) {
			for(int r = 1; r < rowSlices; ++r) s += cluster.map_shared_rank(total, r)[threadIdx.x];
		}
		cluster.sync(); // the other blocks' shared memory stays alive until it has been read
	}
	if(slice == 0 && lane8 == 0 && w < width) {
		float* dst = y + static_cast<size_t>(b) * width + w;
		*dst = add ? *dst + s : s;
	}
}

// The same for widths that are a multiple of four and 16-byte-aligned operands: a block owns 256 columns (64 float4
// lanes) of one batch entry and four row lanes; each warp access is 512 contiguous bytes.
__global__ void __launch_bounds__(256) sum_rows_vec_kernel(float* __restrict__ y, const float* __restrict__ x,
	int height, int width, int rowSlices, int add)
{
	namespace cg = cooperative_groups;
	__shared__ float4 part[4][64];
	__shared__ float4 total[64];
	const int b = blockIdx.z;
	const int q = threadIdx.x & 63;             // float4 lane inside the block's 256 columns
	const int lane4 = threadIdx.x >> 6;         // row lane
	const int w4 = blockIdx.x * 64 + q;         // float4 column
	const int width4 = width >> 2;
	const int slice = blockIdx.y;
	const int rowsPerSlice = (height + rowSlices - 1) / rowSlices;
	const int h0 = slice * rowsPerSlice;
	const int h1 = min(height, h0 + rowsPerSlice);
	float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
	if(w4 < width4) {
		const float4* src = reinterpret_cast<const float4*>(x) + static_cast<size_t>(b) * height * width4 + w4;
		for(int h = h0 + lane4; h < h1; h += 4) {
			const float4 v = __ldg(src + static_cast<size_t>(h) * width4);
			acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
		}
	}
	part[lane4][q] = acc;
	__syncthreads();
	float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
	if(lane4 == 0) {
		s = part[0][q];
#pragma unroll
		for(int i = 1; i < 4; ++i) { s.x += part[i][q].x; s.y += part[i][q].y; s.z += part[i][q].z; s.w += part[i][q].w; }
		total[q] = s;
	}
	if(rowSlices > 1) {
		cg::cluster_group cluster = cg::this_cluster();
		cluster.sync();
		if(slice == 0 && lane4 == 0) {
			for(int r = 1; r < rowSlices; ++r) {
				const float4 o = cluster.map_shared_rank(total, r)[q];
				s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
			}
		}
		cluster.sync();
	}
	if(slice == 0 && lane4 == 0 && w4 < width4) {
		float4* dst = reinterpret_cast<float4*>(y + static_cast<size_t>(b) * width + 4 * w4);
		if(add) {
			const float4 o = *dst;
			s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
		}
		*dst = s;
	}
}

// y[h] = sum_w x[h][w]: one warp per row.  SHIFTED: the element is first moved by the row's own addend and, if
// `square`, multiplied by itself -- every step rounded like the separate calls it stands for -- and the sum runs in
// the same order, so the result is that of AddVectorToMatrixColumns, VectorEltwiseMultiply and SumMatrixColumns.
template<bool SHIFTED>
__global__ void __launch_bounds__(256) sum_cols_kernel(float* __restrict__ y, const float* __restrict__ x,
	int height, int width, const float* __restrict__ rowAdd, int square)
{
	const int warpsPerBlock = blockDim.x >> 5;
	const int lane = threadIdx.x & 31;
	for(int h = blockIdx.x * warpsPerBlock + (threadIdx.x >> 5); h < height; h += gridDim.x * warpsPerBlock) {
		const float* row = x + static_cast<size_t>(h) * width;
		float acc = 0.f;
		if(SHIFTED) {
			const float a = __ldg(rowAdd + h);
			for(int w = lane; w < width; w += 32) {
				float v = __fadd_rn(row[w], a);
				if(square) v = __fmul_rn(v, v);
				acc += v;
			}
		} else {
			for(int w = lane; w < width; w += 32) acc += row[w];
		}
		acc = warp_sum(acc);
		if(lane == 0) y[h] = acc;
	}
}

// y[h][w] = (((x[h][w] + rowAdd[h]) [squared]) * rowMul[h]) * colMul[w] + colAdd[w]; every step optional and rounded
// by itself, in this order: the chain AddVectorToMatrixColumns, [VectorEltwiseMultiply by itself,]
// MultiplyDiagMatrixByMatrix, MultiplyMatrixByDiagMatrix, AddVectorToMatrixRows in one pass.
struct Affine {
	const float* rowAdd;
	const float* rowMul;
	const float* colMul;
	const float* colAdd;
	int square;
};

template<int V>
__global__ void __launch_bounds__(256) affine_kernel(const float* __restrict__ x, float* __restrict__ y, long long total,
	int width, const Affine f)
{
	const int wv = width / V;
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
		const long long h = e / wv;
		const int w = static_cast<int>(e - h * wv) * V;
		float v[V];
		if(V == 4) {
			const float4 t = reinterpret_cast<const float4*>(x)[e];
			v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
		} else {
			v[0] = x[e];
		}
		if(f.rowAdd != nullptr) {
			const float a = __ldg(f.rowAdd + h);
#pragma unroll
			for(int i = 0; i < V; ++i) v[i] = __fadd_rn(v[i], a);
		}
		if(f.square) {
#pragma unroll
			for(int i = 0; i < V; ++i) v[i] = __fmul_rn(v[i], v[i]);
		}
		if(f.rowMul != nullptr) {
			const float m = __ldg(f.rowMul + h);
#pragma unroll
			for(int i = 0; i < V; ++i) v[i] = __fmul_rn(v[i], m);
		}
		if(f.colMul != nullptr) {
#pragma unroll
			for(int i = 0; i < V; ++i) v[i] = __fmul_rn(v[i], __ldg(f.colMul + w + i));
		}
		if(f.colAdd != nullptr) {
#pragma unroll
			for(int i = 0; i < V; ++i) v[i] = __fadd_rn(v[i], __ldg(f.colAdd + w + i));
		}
		if(V == 4) reinterpret_cast<float4*>(y)[e] = make_float4(v[0], v[1], v[2], v[3]);
		else y[e] = v[0];
	}
}

// Row softmax, one warp per row when the row fits 32 registers per lane (width <= 1024), kept in registers between
// the three passes so x is read once and y written once.
// Optional prologue (the attention chain's scale and mask, folded in by the engine): the element becomes
// x * *scale (+) bias[h % biasRows][w], each step rounded to fp32 like the separate VectorMultiply and
// AddVectorToMatrixRows calls it replaces.
template<int PER_LANE>
__global__ void __launch_bounds__(256) softmax_rows_reg_kernel(const float* __restrict__ x, float* __restrict__ y,
	int height, int width, const float* __restrict__ scale, const float* __restrict__ bias, int biasRows)
{
	const int warpsPerBlock = blockDim.x >> 5;
	const int lane = threadIdx.x & 31;
	const float mul = scale != nullptr ? __ldg(scale) : 1.f;
	for(int h = blockIdx.x * warpsPerBlock + (threadIdx.x >> 5); h < height; h += gridDim.x * warpsPerBlock) {
		const float* row = x + static_cast<size_t>(h) * width;
		const float* biasRow = bias != nullptr ? bias + static_cast<size_t>(h % biasRows) * width : nullptr;
		float v[PER_LANE];
		// all loads of the row first, back to back; the optional prologue is applied in loops of its own, each behind ONE
		// branch (a branch per element, even a uniform one, keeps the loads from overlapping: 3x slower, measured)
#pragma unroll
		for(int i = 0; i < PER_LANE; ++i) {
			const int w = lane + 32 * i;
			v[i] = w < width ? row[w] : -FLT_MAX;
		}
		if(scale != nullptr) {
#pragma unroll
			for(int i = 0; i < PER_LANE; ++i) {
				if(lane + 32 * i < width) v[i] = __fmul_rn(v[i], mul);
			}
		}
		if(biasRow != nullptr) {
			float b[PER_LANE];
#pragma unroll
			for(int i = 0; i < PER_LANE; ++i) {
				const int w = lane + 32 * i;
				b[i] = w < width ? __ldg(biasRow + w) : 0.f;
			}
#pragma unroll
			for(int i = 0; i < PER_LANE; ++i) {
				if(lane + 32 * i < width) v[i] = __fadd_rn(v[i], b[i]);
			}
		}
		float mx = -FLT_MAX;
#pragma unroll
		for(int i = 0; i < PER_LANE; ++i) mx = fmaxf(mx, v[i]);
		mx = warp_max(mx);
		float sum = 0.f;
#pragma unroll
		for(int i = 0; i < PER_LANE; ++i) {
			const int w = lane + 32 * i;
			// exponent argument clamped like the reference's ExponentFunc (CpuX86.h:43-62)
			v[i] = w < width ? expf(fmaxf(v[i] - mx, -87.3365f)) : 0.f;
			sum += v[i];
		}
		sum = warp_sum(sum);
		const float inv = 1.f / sum;
		float* out = y + static_cast<size_t>(h) * width;
#pragma unroll
		for(int i = 0; i < PER_LANE; ++i) {
			const int w = lane + 32 * i;
			if(w < width) out[w] = v[i] * inv;
		}
	}
}

// Wide rows: one block per row, three passes through global memory (the row stays in L2).
__global__ void __launch_bounds__(256) softmax_rows_wide_kernel(const float* __restrict__ x, float* __restrict__ y,
	int height, int width)
{
	__shared__ float red[8];
	__shared__ float bcast;
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	for(int h = blockIdx.x; h < height; h += gridDim.x) {
		const float* row = x + static_cast<size_t>(h) * width;
		float* out = y + static_cast<size_t>(h) * width;
		float mx = -FLT_MAX;
		for(int w = threadIdx.x; w < width; w += blockDim.x) mx = fmaxf(mx, row[w]);
		mx = warp_max(mx);
		if(lane == 0) red[warp] = mx;
		__syncthreads();
		if(threadIdx.x == 0) {
			float m = red[0];
			for(int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
			bcast = m;
		}
		__syncthreads();
		mx = bcast;
		float sum = 0.f;
		for(int w = threadIdx.x; w < width; w += blockDim.x) {
			const float e = expf(fmaxf(row[w] - mx, -87.3365f));
			out[w] = e;
			sum += e;
		}
		sum = warp_sum(sum);
		__syncthreads();
		if(lane == 0) red[warp] = sum;
		__syncthreads();
		if(threadIdx.x == 0) {
			float s = 0.f;
			for(int i = 0; i < 8; ++i) s += red[i];
			bcast = 1.f / s;
		}
		__syncthreads();
		const float inv = bcast;
		for(int w = threadIdx.x; w < width; w += blockDim.x) out[w] *= inv;
		__syncthreads();
	}
}

// Generalised transpose  x[b][h][m][w][c] -> y[b][w][m][h][c]  of 4-byte elements.
// channels >= 8 (or tiny h/w): rows of `channels` elements are moved whole, coalesced on both sides.
__global__ void __launch_bounds__(256) transpose_rows_kernel(const uint32_t* __restrict__ x, uint32_t* __restrict__ y,
	int height, int medium, int width, int channels, long long total)
{
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long o = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; o < total; o += stride) {
		// o indexes the output
		long long t = o;
		const int c = static_cast<int>(t % channels); t /= channels;
		const int h = static_cast<int>(t % height); t /= height;
		const int m = static_cast<int>(t % medium); t /= medium;
		const int w = static_cast<int>(t % width); t /= width;
		const long long b = t;
		y[o] = x[(((b * height + h) * medium + m) * width + w) * channels + c];
	}
}

// The same with 16-byte pieces for channel counts that are a multiple of four (attention heads: 64 channels): a
// quarter of the index arithmetic per byte, all of it in 32 bits.
__global__ void __launch_bounds__(256) transpose_rows_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y,
	unsigned height, unsigned medium, unsigned width, unsigned channels4, unsigned total)
{
	for(unsigned o = blockIdx.x * blockDim.x + threadIdx.x; o < total; o += gridDim.x * blockDim.x) {
		unsigned t = o;
		const unsigned c = t % channels4; t /= channels4;
		const unsigned h = t % height; t /= height;
		const unsigned m = t % medium; t /= medium;
		const unsigned w = t % width;
		const unsigned b = t / width;
		y[o] = __ldg(x + ((((static_cast<size_t>(b) * height + h) * medium + m) * width + w) * channels4 + c));
	}
}

// channels == 1, medium == 1: classic 32x32 shared-memory tile transpose of a [height x width] matrix per batch.
__global__ void __launch_bounds__(256) transpose_tile_kernel(const uint32_t* __restrict__ x, uint32_t* __restrict__ y,
	int height, int width)
{
	__shared__ uint32_t tile[32][33];
	const size_t base = static_cast<size_t>(blockIdx.z) * height * width;
	const int w0 = blockIdx.x * 32, h0 = blockIdx.y * 32;
	const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
	for(int i = ty; i < 32; i += 8) {
		const int h = h0 + i, w = w0 + tx;
		if(h < height && w < width) tile[i][tx] = x[base + static_cast<size_t>(h) * width + w];
	}
	__syncthreads();
	for(int i = ty; i < 32; i += 8) {
		const int w = w0 + i, h = h0 + tx;
		if(h < height && w < width) y[base + static_cast<size_t>(w) * height + h] = tile[tx][i];
	}
}

// The same for height and width both a multiple of four and 16-byte-aligned matrices: 64 x 64 tiles moved with
// 16-byte loads and stores (four rows x four columns per thread and direction), 16 KB in flight per block instead
// of 4 KB.  The tile is padded to 65 words per row so that the column-wise reads of the store pass hit 32 banks.
__global__ void __launch_bounds__(256) transpose_tile64_kernel(const uint32_t* __restrict__ x, uint32_t* __restrict__ y,
	int height, int width)
{
	__shared__ uint32_t tile[64][65];
	const size_t base = static_cast<size_t>(blockIdx.z) * height * width;
	const int w0 = blockIdx.x * 64, h0 = blockIdx.y * 64;
	const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // 16 x 16 threads
#pragma unroll
	for(int i = 0; i < 4; ++i) {
		const int r = ty + 16 * i;
		const int h = h0 + r, w = w0 + 4 * tx;
		if(h < height && w < width) {
			const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + base + static_cast<size_t>(h) * width + w));
			tile[r][4 * tx] = v.x; tile[r][4 * tx + 1] = v.y; tile[r][4 * tx + 2] = v.z; tile[r][4 * tx + 3] = v.w;
		}
	}
	__syncthreads();
#pragma unroll
	for(int i = 0; i < 4; ++i) {
		const int c = ty + 16 * i;           // column of the source tile = row of the result
		const int w = w0 + c, h = h0 + 4 * tx;
		if(w < width && h < height) {
			const uint4 v = make_uint4(tile[4 * tx][c], tile[4 * tx + 1][c], tile[4 * tx + 2][c], tile[4 * tx + 3][c]);
			*reinterpret_cast<uint4*>(y + base + static_cast<size_t>(w) * height + h) = v;
		}
	}
}

// Row arg-max: one warp per row, first maximum wins.
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ x, int height, int width,
	float* __restrict__ maxValues, int* __restrict__ maxIndices)
{
	const int warpsPerBlock = blockDim.x >> 5;
	const int lane = threadIdx.x & 31;
	for(int h = blockIdx.x * warpsPerBlock + (threadIdx.x >> 5); h < height; h += gridDim.x * warpsPerBlock) {
		const float* row = x + static_cast<size_t>(h) * width;
		float best = -FLT_MAX;
		int bestIdx = 0x7fffffff;
		for(int w = lane; w < width; w += 32) {
			const float v = row[w];
			if(v > best || bestIdx == 0x7fffffff) { best = v; bestIdx = w; }
		}
#pragma unroll
		for(int o = 16; o > 0; o >>= 1) {
			const float ov = __shfl_xor_sync(0xffffffffu, best, o);
			const int oi = __shfl_xor_sync(0xffffffffu, bestIdx, o);
			if(oi != 0x7fffffff && (bestIdx == 0x7fffffff || ov > best || (ov == best && oi < bestIdx))) { best = ov; bestIdx = oi; }
		}
		if(lane == 0) {
			maxValues[h] = best;
			if(maxIndices != nullptr) maxIndices[h] = bestIdx;
		}
	}
}

// Column arg-max per batch: thread per column, rows walked in order (first maximum wins), coalesced across columns.
__global__ void __launch_bounds__(256) argmax_cols_kernel(const float* __restrict__ x, int height, int width,
	float* __restrict__ maxValues, int* __restrict__ rowIndices, long long totalCols)
{
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < totalCols; t += stride) {
		const long long b = t / width;
		const int w = static_cast<int>(t - b * width);
		const float* col = x + b * height * width + w;
		float best = col[0];
		int bestIdx = 0;
		for(int h = 1; h < height; ++h) {
			const float v = col[static_cast<size_t>(h) * width];
			if(v > best) { best = v; bestIdx = h; }
		}
		maxValues[t] = best;
		if(rowIndices != nullptr) rowIndices[t] = bestIdx;
	}
}

} // namespace
} // namespace nb200

using namespace nb200;

#define NB200_REQUIRE_DEVICE() do { if(device_status_word() == nullptr) return NB200_ENODEVICE; } while(0)

extern "C" {

int nb200_add_vector_to_matrix_rows(void* stream, int batch, const float* x, float* y, int height, int width,
	const float* v)
{
	if(batch < 0 || height < 0 || width < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(batch) * height * width;
	if(total == 0) return NB200_OK;
	if(x == nullptr || y == nullptr || v == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	const long long perBatch = static_cast<long long>(height) * width;
	const bool vec = aligned16(x) && aligned16(y) && aligned16(v) && width % 4 == 0;
	if(vec) {
		add_rows_kernel<true><<<grid_for(total / 4, 256, 16), 256, 0, as_stream(stream)>>>(x, y, v, total, width, perBatch);
	} else {
		add_rows_kernel<false><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(x, y, v, total, width, perBatch);
	}
	count_launch();
	return check_launch();
}

int nb200_add_vector_to_matrix_columns(void* stream, const float* x, float* y, int height, int width, const float* v)
{
	if(height < 0 || width < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(height) * width;
	if(total == 0) return NB200_OK;
	if(x == nullptr || y == nullptr || v == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	row_scalar_kernel<false><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(x, y, v, total, width);
	count_launch();
	return check_launch();
}

int nb200_multiply_diag_matrix_by_matrix(void* stream, const float* d, int height, const float* x, int width, float* y)
{
	if(height < 0 || width < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(height) * width;
	if(total == 0) return NB200_OK;
	if(x == nullptr || y == nullptr || d == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	row_scalar_kernel<true><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(x, y, d, total, width);
	count_launch();
	return check_launch();
}

int nb200_multiply_matrix_by_diag_matrix(void* stream, int batch, const float* x, int height, int width,
	const float* d, int diag_stride, float* y)
{
	if(batch < 0 || height < 0 || width < 0 || diag_stride < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(batch) * height * width;
	if(total == 0) return NB200_OK;
	if(x == nullptr || y == nullptr || d == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	col_scale_kernel<<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(x, y, d, total, width,
		static_cast<long long>(height) * width, diag_stride);
	count_launch();
	return check_launch();
}

int nb200_sum_matrix_rows(void* stream, int batch, float* y, const float* x, int height, int width, int add)
{
	if(batch < 0 || height < 0 || width < 0) return NB200_EINVAL;
	if(batch == 0 || width == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	if(batch > 65535) return NB200_ETOOBIG;
	NB200_REQUIRE_DEVICE();
	const int colBlocks = (width + 31) / 32;
	// split the rows when (columns x batch) alone cannot fill the machine; the slices of one column block form a
	// thread-block cluster (at most 8 blocks, the portable cluster size)
	int rowSlices = 1;
	const long long blocks = static_cast<long long>(colBlocks) * batch;
	const int target = sm_count() * 4;
	if(blocks < target && height >= 256) {
		rowSlices = static_cast<int>((target + blocks - 1) / blocks);
		const int maxSlices = height / 64;
		if(rowSlices > maxSlices) rowSlices = maxSlices;
		if(rowSlices > 8) rowSlices = 8;
		if(rowSlices < 1) rowSlices = 1;
	}
	const int launches = 1;
	if(height == 0) {
		if(!add) cudaMemsetAsync(y, 0, static_cast<size_t>(batch) * width * sizeof(float), as_stream(stream));
		return check_launch();
	}
	cudaLaunchConfig_t config = {};
	config.blockDim = dim3(256);
	config.stream = as_stream(stream);
	cudaLaunchAttribute attribute[1];
	attribute[0].id = cudaLaunchAttributeClusterDimension;
	attribute[0].val.clusterDim.x = 1;
	attribute[0].val.clusterDim.y = rowSlices;
	attribute[0].val.clusterDim.z = 1;
	config.attrs = attribute;
	config.numAttrs = rowSlices > 1 ? 1 : 0;
	if(width % 4 == 0 && aligned16(x) && aligned16(y)) {
		config.gridDim = dim3((width / 4 + 63) / 64, rowSlices, batch);
		cudaLaunchKernelEx(&config, sum_rows_vec_kernel, y, x, height, width, rowSlices, add);
	} else {
		config.gridDim = dim3(colBlocks, rowSlices, batch);
		cudaLaunchKernelEx(&config, sum_rows_kernel, y, x, height, width, rowSlices, add);
	}
	count_launch(launches);
	return check_launch();
}

int nb200_sum_matrix_columns(void* stream, float* y, const float* x, int height, int width)
{
	if(height < 0 || width < 0) return NB200_EINVAL;
	if(height == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	sum_cols_kernel<false><<<grid_for(height, 8, 16), 256, 0, as_stream(stream)>>>(y, x, height, width, nullptr, 0);
	count_launch();
	return check_launch();
}

int nb200_sum_matrix_columns_shifted(void* stream, float* y, const float* x, int height, int width, const float* row_add,
	int square)
{
	if(height < 0 || width < 0) return NB200_EINVAL;
	if(height == 0) return NB200_OK;
	if(x == nullptr || y == nullptr || row_add == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	sum_cols_kernel<true><<<grid_for(height, 8, 16), 256, 0, as_stream(stream)>>>(y, x, height, width, row_add, square);
	count_launch();
	return check_launch();
}

int nb200_matrix_rows_cols_affine(void* stream, const float* x, int height, int width, const float* row_add, int square,
	const float* row_mul, const float* col_mul, const float* col_add, float* y)
{
	if(height < 0 || width < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(height) * width;
	if(total == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	const Affine f = { row_add, row_mul, col_mul, col_add, square };
	if(width % 4 == 0 && aligned16(x) && aligned16(y)) {
		affine_kernel<4><<<grid_for(total / 4, 256, 16), 256, 0, as_stream(stream)>>>(x, y, total / 4, width, f);
	} else {
		affine_kernel<1><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(x, y, total, width, f);
	}
	count_launch();
	return check_launch();
}

int nb200_matrix_softmax_by_rows_fused(void* stream, const float* x, int height, int width, const float* scale_device,
	const float* row_bias, int bias_rows, float* y)
{
	if(height < 0 || width < 0) return NB200_EINVAL;
	if(height == 0 || width == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	cudaStream_t s = as_stream(stream);
	const int grid = grid_for(height, 8, 16);
	if((scale_device != nullptr || row_bias != nullptr) && width > 1024) return NB200_ETOOBIG; // prologue: register kernel only
	if(row_bias != nullptr && bias_rows <= 0) return NB200_EINVAL;
	if(width <= 32) softmax_rows_reg_kernel<1><<<grid, 256, 0, s>>>(x, y, height, width, scale_device, row_bias, bias_rows);
	else if(width <= 64) softmax_rows_reg_kernel<2><<<grid, 256, 0, s>>>(x, y, height, width, scale_device, row_bias, bias_rows);
	else if(width <= 128) softmax_rows_reg_kernel<4><<<grid, 256, 0, s>>>(x, y, height, width, scale_device, row_bias, bias_rows);
	else if(width <= 256) softmax_rows_reg_kernel<8><<<grid, 256, 0, s>>>(x, y, height, width, scale_device, row_bias, bias_rows);
	else if(width <= 512) softmax_rows_reg_kernel<16><<<grid, 256, 0, s>>>(x, y, height, width, scale_device, row_bias, bias_rows);
	else if(width <= 1024) softmax_rows_reg_kernel<32><<<grid, 256, 0, s>>>(x, y, height, width, scale_device, row_bias, bias_rows);
	else softmax_rows_wide_kernel<<<grid_for(height, 1, 16), 256, 0, s>>>(x, y, height, width);
	count_launch();
	return check_launch();
}

int nb200_matrix_softmax_by_rows(void* stream, const float* x, int height, int width, float* y)
{
	return nb200_matrix_softmax_by_rows_fused(stream, x, height, width, nullptr, nullptr, 0, y);
}

int nb200_transpose_matrix(void* stream, int batch, const void* x, int height, int medium, int width, int channels,
	void* y)
{
	if(batch < 0 || height < 0 || medium < 0 || width < 0 || channels < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(batch) * height * medium * width * channels;
	if(total == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	cudaStream_t s = as_stream(stream);
	const uint32_t* src = static_cast<const uint32_t*>(x);
	uint32_t* dst = static_cast<uint32_t*>(y);
	if(channels == 1 && medium == 1 && height > 1 && width > 1 && batch <= 65535 && (height + 31) / 32 <= 65535) {
		if(height % 4 == 0 && width % 4 == 0 && aligned16(x) && aligned16(y)) {
			dim3 grid((width + 63) / 64, (height + 63) / 64, batch);
			transpose_tile64_kernel<<<grid, 256, 0, s>>>(src, dst, height, width);
		} else {
			dim3 grid((width + 31) / 32, (height + 31) / 32, batch);
			transpose_tile_kernel<<<grid, 256, 0, s>>>(src, dst, height, width);
		}
	} else if(channels % 4 == 0 && total / 4 < 0x7fffffffLL && aligned16(x) && aligned16(y)) {
		transpose_rows_vec_kernel<<<grid_for(total / 4, 256, 16), 256, 0, s>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y),
			height, medium, width, channels / 4, static_cast<unsigned>(total / 4));
	} else {
		transpose_rows_kernel<<<grid_for(total, 256, 16), 256, 0, s>>>(src, dst, height, medium, width, channels, total);
	}
	count_launch();
	return check_launch();
}

int nb200_find_max_value_in_rows(void* stream, const float* x, int height, int width, float* max_values, int* max_indices)
{
	if(height < 0 || width <= 0) return NB200_EINVAL;
	if(height == 0) return NB200_OK;
	if(x == nullptr || max_values == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	argmax_rows_kernel<<<grid_for(height, 8, 16), 256, 0, as_stream(stream)>>>(x, height, width, max_values, max_indices);
	count_launch();
	return check_launch();
}

int nb200_find_max_value_in_columns(void* stream, int batch, const float* x, int height, int width, float* max_values,
	int* row_indices)
{
	if(batch < 0 || height <= 0 || width < 0) return NB200_EINVAL;
	const long long totalCols = static_cast<long long>(batch) * width;
	if(totalCols == 0) return NB200_OK;
	if(x == nullptr || max_values == nullptr) return NB200_EINVAL;
	NB200_REQUIRE_DEVICE();
	argmax_cols_kernel<<<grid_for(totalCols, 256, 16), 256, 0, as_stream(stream)>>>(x, height, width, max_values,
		row_indices, totalCols);
	count_launch();
	return check_launch();
}

} // extern "C"
