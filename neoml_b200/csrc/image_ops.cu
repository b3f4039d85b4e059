// Channels-last image ops that are pure data movement or small stencils: 2-D max/mean pooling, image
// resize (pad/crop) and depthwise (channelwise) convolution.  One thread handles 4 consecutive channels of one
// output pixel when channels % 4 == 0 and the buffers are 16-byte aligned, so every access is a coalesced 16-byte
// load/store along the channel dimension; the stencil re-reads hit L1/L2.
#include "common.cuh"
#include <cuda.h>
#include <float.h>
#include <atomic>

namespace nb200 {

namespace {

struct Pool2d {
	int batch, h, w, c, fh, fw, sh, sw, ho, wo;
};

template<bool MAX, int V>
__global__ void __launch_bounds__(256) pool_kernel(const Pool2d p, const float* __restrict__ x, float* __restrict__ y,
	int* __restrict__ maxIndices, long long total)
{
	const int cv = p.c / V;
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
		long long r = t;
		const int c = static_cast<int>(r % cv) * V; r /= cv;
		const int ox = static_cast<int>(r % p.wo); r /= p.wo;
		const int oy = static_cast<int>(r % p.ho); r /= p.ho;
		const long long n = r;
		const float* img = x + n * p.h * p.w * p.c;
		float acc[V];
		int idx[V];
#pragma unroll
		for(int e = 0; e < V; ++e) { acc[e] = MAX ? -FLT_MAX : 0.f; idx[e] = 0; }
		for(int fy = 0; fy < p.fh; ++fy) {
			const int iy = oy * p.sh + fy;
			for(int fx = 0; fx < p.fw; ++fx) {
				const int ix = ox * p.sw + fx;
				const int pix = iy * p.w + ix;
				const float* src = img + static_cast<size_t>(pix) * p.c + c;
				float v[V];
				if(V == 4) {
					const float4 q = __ldg(reinterpret_cast<const float4*>(src));
					v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
				} else {
					v[0] = __ldg(src);
				}
#pragma unroll
				for(int e = 0; e < V; ++e) {
					if(MAX) {
						if(v[e] > acc[e] || (fy == 0 && fx == 0)) { acc[e] = v[e]; idx[e] = pix * p.c + c + e; }
					} else {
						acc[e] += v[e];
					}
				}
			}
		}
		const size_t o = ((static_cast<size_t>(n) * p.ho + oy) * p.wo + ox) * p.c + c;
		if(!MAX) {
			const float inv = 1.f / static_cast<float>(p.fh * p.fw);
#pragma unroll
			for(int e = 0; e < V; ++e) acc[e] *= inv;
		}
		if(V == 4) {
			*reinterpret_cast<float4*>(y + o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
		} else {
			y[o] = acc[0];
		}
		if(MAX && maxIndices != nullptr) {
#pragma unroll
			for(int e = 0; e < V; ++e) maxIndices[o + e] = idx[e];
		}
	}
}

struct Resize {
	int batch, h, w, c, dl, dt, ho, wo, padding;
	float value;
};

template<int V>
__global__ void __launch_bounds__(256) resize_kernel(const Resize p, const float* __restrict__ x, float* __restrict__ y,
	long long total)
{
	const int cv = p.c / V;
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
		long long r = t;
		const int c = static_cast<int>(r % cv) * V; r /= cv;
		const int ox = static_cast<int>(r % p.wo); r /= p.wo;
		const int oy = static_cast<int>(r % p.ho); r /= p.ho;
		const long long n = r;
		int iy = oy - p.dt, ix = ox - p.dl;
		bool inside = iy >= 0 && iy < p.h && ix >= 0 && ix < p.w;
		if(!inside && p.padding != 0) {
			if(p.padding == 1) { // edge
				iy = min(max(iy, 0), p.h - 1);
				ix = min(max(ix, 0), p.w - 1);
			} else { // reflect
				if(iy < 0) iy = -iy; else if(iy >= p.h) iy = 2 * (p.h - 1) - iy;
				if(ix < 0) ix = -ix; else if(ix >= p.w) ix = 2 * (p.w - 1) - ix;
				iy = min(max(iy, 0), p.h - 1);
				ix = min(max(ix, 0), p.w - 1);
			}
			inside = true;
		}
		float* dst = y + t * V;
		if(V == 4) {
			float4 v = make_float4(p.value, p.value, p.value, p.value);
			if(inside) v = __ldg(reinterpret_cast<const float4*>(x + ((n * p.h + iy) * p.w + ix) * p.c + c));
			*reinterpret_cast<float4*>(dst) = v;
		} else {
			*dst = inside ? __ldg(x + ((n * p.h + iy) * p.w + ix) * p.c + c) : p.value;
		}
	}
}

template<int V>
__global__ void __launch_bounds__(256) chconv_kernel(const nb200_chconv_desc p, const float* __restrict__ x,
	const float* __restrict__ filter, const float* __restrict__ freeTerm, float* __restrict__ y, int act,
	float actParam, long long total)
{
	const int cv = p.c / V;
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
		long long r = t;
		const int c = static_cast<int>(r % cv) * V; r /= cv;
		const int ox = static_cast<int>(r % p.wo); r /= p.wo;
		const int oy = static_cast<int>(r % p.ho); r /= p.ho;
		const long long n = r;
		const float* img = x + n * p.h * p.w * p.c;
		float acc[V];
#pragma unroll
		for(int e = 0; e < V; ++e) acc[e] = freeTerm != nullptr ? __ldg(freeTerm + c + e) : 0.f;
		for(int fy = 0; fy < p.r; ++fy) {
			const int iy = oy * p.stride_h - p.pad_h + fy;
			if(static_cast<unsigned>(iy) >= static_cast<unsigned>(p.h)) continue;
			for(int fx = 0; fx < p.s; ++fx) {
				const int ix = ox * p.stride_w - p.pad_w + fx;
				if(static_cast<unsigned>(ix) >= static_cast<unsigned>(p.w)) continue;
				const float* src = img + (static_cast<size_t>(iy) * p.w + ix) * p.c + c;
				const float* wgt = filter + (fy * p.s + fx) * p.c + c;
				if(V == 4) {
					const float4 a = __ldg(reinterpret_cast<const float4*>(src));
					const float4 f = __ldg(reinterpret_cast<const float4*>(wgt));
					acc[0] = fmaf(a.x, f.x, acc[0]); acc[1] = fmaf(a.y, f.y, acc[1]);
					acc[2] = fmaf(a.z, f.z, acc[2]); acc[3] = fmaf(a.w, f.w, acc[3]);
				} else {
					acc[0] = fmaf(__ldg(src), __ldg(wgt), acc[0]);
				}
			}
		}
#pragma unroll
		for(int e = 0; e < V; ++e) acc[e] = apply_act(acc[e], act, actParam);
		float* dst = y + t * V;
		if(V == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
		else *dst = acc[0];
	}
}

// 3x3 depthwise convolution, padding 1, stride 1 or 2, channels a multiple of four: a thread owns four channels of a
// strip of TW neighbouring output columns.  It first loads every input column the strip touches (three rows of four
// channels each; TW + 2 columns for stride 1, 2 TW + 1 for stride 2) -- all independent loads, in flight together --
// and then forms the outputs from registers, so each input column is fetched once per strip instead of three times
// and the index arithmetic is paid once per strip.  Consecutive threads take consecutive channel quads: every load
// and store of a warp is one contiguous run.
template<int STRIDE>
__global__ void __launch_bounds__(256) chconv3x3_kernel(const nb200_chconv_desc p, const float* __restrict__ x,
	const float* __restrict__ filter, const float* __restrict__ freeTerm, float* __restrict__ y, int act,
	float actParam, int strips, unsigned total)
{
	constexpr int TW = STRIDE == 1 ? 4 : 2;
	constexpr int COLS = STRIDE == 1 ? TW + 2 : 2 * TW + 1;
	const unsigned cv = p.c / 4;
	const bool relu = act == NB200_ACT_RELU;
	const float reluHi = actParam > 0.f ? actParam : __int_as_float(0x7f800000);
	for(unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
		unsigned r = t;
		const unsigned cq = r % cv; r /= cv;
		const unsigned sx = r % strips; r /= strips;
		const int oy = static_cast<int>(r % p.ho);
		const unsigned n = r / p.ho;
		const int ox0 = sx * TW;
		const float4* img = reinterpret_cast<const float4*>(x) + static_cast<size_t>(n) * p.h * p.w * cv + cq;
		const int iy0 = oy * STRIDE - 1, ix0 = ox0 * STRIDE - 1;
		float4 col[COLS][3];
#pragma unroll
		for(int k = 0; k < COLS; ++k) {
			const int ix = ix0 + k;
			const bool colOk = static_cast<unsigned>(ix) < static_cast<unsigned>(p.w);
#pragma unroll
			for(int fy = 0; fy < 3; ++fy) {
				const int iy = iy0 + fy;
				col[k][fy] = make_float4(0.f, 0.f, 0.f, 0.f);
				if(colOk && static_cast<unsigned>(iy) < static_cast<unsigned>(p.h)) {
					col[k][fy] = __ldg(img + (static_cast<size_t>(iy) * p.w + ix) * cv);
				}
			}
		}
		const float4* flt = reinterpret_cast<const float4*>(filter) + cq;
		float4 f[9];
#pragma unroll
		for(int i = 0; i < 9; ++i) f[i] = __ldg(flt + i * cv);
		const float4 b = freeTerm != nullptr ? __ldg(reinterpret_cast<const float4*>(freeTerm) + cq) : make_float4(0.f, 0.f, 0.f, 0.f);
		float4* out = reinterpret_cast<float4*>(y) + ((static_cast<size_t>(n) * p.ho + oy) * p.wo + ox0) * cv + cq;
#pragma unroll
		for(int j = 0; j < TW; ++j) {
			if(ox0 + j >= p.wo) break;
			float4 a = b;
#pragma unroll
			for(int fy = 0; fy < 3; ++fy) {
#pragma unroll
				for(int fx = 0; fx < 3; ++fx) {
					const float4 v = col[j * STRIDE + fx][fy];
					const float4 w = f[3 * fy + fx];
					a.x = fmaf(v.x, w.x, a.x); a.y = fmaf(v.y, w.y, a.y); a.z = fmaf(v.z, w.z, a.z); a.w = fmaf(v.w, w.w, a.w);
				}
			}
			if(act == NB200_ACT_HSWISH) {
				a.x = apply_act(a.x, act, actParam); a.y = apply_act(a.y, act, actParam);
				a.z = apply_act(a.z, act, actParam); a.w = apply_act(a.w, act, actParam);
			} else {
				a.x = relu ? fminf(fmaxf(a.x, 0.f), reluHi) : a.x; a.y = relu ? fminf(fmaxf(a.y, 0.f), reluHi) : a.y;
				a.z = relu ? fminf(fmaxf(a.z, 0.f), reluHi) : a.z; a.w = relu ? fminf(fmaxf(a.w, 0.f), reluHi) : a.w;
			}
			out[static_cast<size_t>(j) * cv] = a;
		}
	}
}

// The same convolution for large images: a thread owns four channels of a block of TH output rows by TW output columns
// and walks down the rows with a window of input rows in registers, so every input row of its columns is loaded once
// per block instead of once per output row (stride 1: (TH + 2) * 6 loads for TH * 4 outputs against 18 per 4).  The
// rows of the NEXT output row are requested before the current one is computed (the window holds one output row more
// than it needs), and the filter sits in shared memory, which leaves the registers to the window.  The loop over the
// rows is fully unrolled: the window rotates by renaming, not by moves.  The sums are formed in the order of the strip
// kernel (bias first, filter rows outer, columns inner), so the two kernels agree bit for bit.
template<int STRIDE, int TH>
__global__ void __launch_bounds__(128, 4) chconv3x3_rows_kernel(const nb200_chconv_desc p, const float* __restrict__ x,
	const float* __restrict__ filter, const float* __restrict__ freeTerm, float* __restrict__ y, int act,
	float actParam, int strips, int rowGroups, unsigned total)
{
	constexpr int TW = STRIDE == 1 ? 4 : 2;
	constexpr int COLS = STRIDE == 1 ? TW + 2 : 2 * TW + 1;
	constexpr int WIN = 3; // input rows held
	extern __shared__ float4 filterShared[]; // [9][c / 4]
	const unsigned cv = p.c / 4;
	for(unsigned i = threadIdx.x; i < 9 * cv; i += blockDim.x) filterShared[i] = __ldg(reinterpret_cast<const float4*>(filter) + i);
	__syncthreads();
	const bool relu = act == NB200_ACT_RELU;
	const float reluHi = actParam > 0.f ? actParam : __int_as_float(0x7f800000);
	for(unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
		unsigned r = t;
		const unsigned cq = r % cv; r /= cv;
		const unsigned sx = r % strips; r /= strips;
		const int oy0 = static_cast<int>(r % rowGroups) * TH;
		const unsigned n = r / rowGroups;
		const int ox0 = sx * TW;
		const int ix0 = ox0 * STRIDE - 1;
		const float4* img = reinterpret_cast<const float4*>(x) + static_cast<size_t>(n) * p.h * p.w * cv + cq;
		bool colOk[COLS];
#pragma unroll
		for(int k = 0; k < COLS; ++k) colOk[k] = static_cast<unsigned>(ix0 + k) < static_cast<unsigned>(p.w);
		auto loadRow = [&](int iy, float4 (&row)[COLS]) {
			const bool rowOk = static_cast<unsigned>(iy) < static_cast<unsigned>(p.h);
			const float4* src = img + (static_cast<ptrdiff_t>(iy) * p.w + ix0) * static_cast<ptrdiff_t>(cv);
#pragma unroll
			for(int k = 0; k < COLS; ++k) {
				row[k] = make_float4(0.f, 0.f, 0.f, 0.f);
				if(rowOk && colOk[k]) row[k] = __ldg(src + static_cast<size_t>(k) * cv);
			}
		};
		const float4 b = freeTerm != nullptr ? __ldg(reinterpret_cast<const float4*>(freeTerm) + cq) : make_float4(0.f, 0.f, 0.f, 0.f);
		float4* out = reinterpret_cast<float4*>(y) + ((static_cast<size_t>(n) * p.ho + oy0) * p.wo + ox0) * cv + cq;
		// input row iy sits in slot (iy - first) % WIN, first = the row above the block
		const int first = oy0 * STRIDE - 1;
		float4 win[WIN][COLS];
#pragma unroll
		for(int k = 0; k < 3 - STRIDE; ++k) loadRow(first + k, win[k]);
#pragma unroll
		for(int j = 0; j < TH; ++j) {
			if(oy0 + j >= p.ho) break;
			const int top = STRIDE * j; // offset of this output row's first input row from `first`
#pragma unroll
			for(int k = 3 - STRIDE; k < 3; ++k) loadRow(first + top + k, win[(top + k) % WIN]);
			float4 a[TW];
#pragma unroll
			for(int i = 0; i < TW; ++i) a[i] = b;
#pragma unroll
			for(int fy = 0; fy < 3; ++fy) {
#pragma unroll
				for(int fx = 0; fx < 3; ++fx) {
					const float4 w = filterShared[(3 * fy + fx) * cv + cq];
#pragma unroll
					for(int i = 0; i < TW; ++i) {
						const float4 v = win[(top + fy) % WIN][i * STRIDE + fx];
						a[i].x = fmaf(v.x, w.x, a[i].x); a[i].y = fmaf(v.y, w.y, a[i].y);
						a[i].z = fmaf(v.z, w.z, a[i].z); a[i].w = fmaf(v.w, w.w, a[i].w);
					}
				}
			}
#pragma unroll
			for(int i = 0; i < TW; ++i) {
				if(ox0 + i >= p.wo) break;
				float4 o = a[i];
				if(act == NB200_ACT_HSWISH) {
					o.x = apply_act(o.x, act, actParam); o.y = apply_act(o.y, act, actParam);
					o.z = apply_act(o.z, act, actParam); o.w = apply_act(o.w, act, actParam);
				} else {
					o.x = relu ? fminf(fmaxf(o.x, 0.f), reluHi) : o.x; o.y = relu ? fminf(fmaxf(o.y, 0.f), reluHi) : o.y;
					o.z = relu ? fminf(fmaxf(o.z, 0.f), reluHi) : o.z; o.w = relu ? fminf(fmaxf(o.w, 0.f), reluHi) : o.w;
				}
				out[(static_cast<size_t>(j) * p.wo + i) * cv] = o;
			}
		}
	}
}

// The same convolution for large images with the input staged by TMA: a CTA walks tiles of th output rows x tw output
// columns x 32 channels of one image; one thread issues the bulk copies of the NEXT tiles' input boxes (halo included,
// zeros delivered by the copy engine where the box leaves the image, so the padding costs no test) into the other
// stages of a shared-memory ring (as many stages as fit, up to four) while all threads compute the current tile.
// The bytes in flight per SM are whole input boxes (tens of KB) whatever the register budget of the compute threads.
// A thread owns four channels of DW_RPP output rows x TW output columns and slides a three-row register window down
// its rows; the sums are formed in the order of the other kernels (bias, filter rows outer, columns inner): identical
// results.
constexpr int DW_RPP = 2;  // output rows per thread: two CTAs of eight warps per SM issue better than one CTA with four rows per thread (measured)
constexpr int DW_CC = 32;  // channels per tile: one 128-byte line per pixel
constexpr int DW_MAX_STAGES = 4;
constexpr int SITE_DW_FULL = 0x201;

template<int STRIDE>
__global__ void __launch_bounds__(256, 2) chconv3x3_tma_kernel(const nb200_chconv_desc p, const __grid_constant__ CUtensorMap map,
	const float* __restrict__ filter, const float* __restrict__ freeTerm, float* __restrict__ y, int act, float actParam,
	int strips, int rowParts, int tilesX, int tilesY, int chunks, unsigned numTiles, int stages, int* status)
{
	constexpr int TW = STRIDE == 1 ? 4 : 2;
	constexpr int COLS = STRIDE == 1 ? TW + 2 : 2 * TW + 1;
	constexpr int EXTRA = STRIDE == 1 ? 2 : 1; // input rows / columns beyond STRIDE * outputs
	extern __shared__ uint8_t dwSmemRaw[];
	__shared__ uint64_t fullBar[DW_MAX_STAGES];
	__shared__ int abortFlag;
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dwSmemRaw) + 127) & ~static_cast<uintptr_t>(127));
	const int tid = threadIdx.x;
	const int tw = strips * TW, th = rowParts * DW_RPP;
	const int colsIn = tw * STRIDE + EXTRA, rowsIn = th * STRIDE + EXTRA;
	const uint32_t stageBytes = static_cast<uint32_t>(rowsIn) * colsIn * DW_CC * 4;
	if(tid == 0) {
		for(int i = 0; i < DW_MAX_STAGES; ++i) mbar_init(&fullBar[i], 1);
		abortFlag = 0;
		mbar_init_fence();
		tma_prefetch_descriptor(&map);
	}
	__syncthreads();

	auto issue = [&](unsigned t, int stage) {
		const int chunk = t % chunks; t /= chunks;
		const int tx = t % tilesX; t /= tilesX;
		const int ty = t % tilesY;
		const int n = t / tilesY;
		mbar_arrive_expect_tx(&fullBar[stage], stageBytes);
		tma_load_4d(smem_u32(smem + stage * stageBytes), &map, &fullBar[stage], chunk * DW_CC, tx * tw * STRIDE - 1,
			ty * th * STRIDE - 1, n);
	};

	const int q = tid & 7;
	const int strip = (tid >> 3) % strips;
	const int part = (tid >> 3) / strips;
	const bool active = part < rowParts;
	const bool relu = act == NB200_ACT_RELU;
	const float reluHi = actParam > 0.f ? actParam : __int_as_float(0x7f800000);
	const unsigned cv = p.c / 4;

	if(tid == 0) {
		for(int i = 0; i < stages - 1; ++i) {
			const unsigned long long t = blockIdx.x + static_cast<unsigned long long>(i) * gridDim.x;
			if(t < numTiles) issue(static_cast<unsigned>(t), i);
		}
	}
	int it = 0;
	for(unsigned t = blockIdx.x; t < numTiles; t += gridDim.x, ++it) {
		const int stage = it % stages;
		// the stage this copy fills was read in the previous iteration, which ended with a CTA-wide barrier
		const unsigned long long ahead = t + static_cast<unsigned long long>(stages - 1) * gridDim.x;
		if(tid == 0 && ahead < numTiles) issue(static_cast<unsigned>(ahead), (it + stages - 1) % stages);
		if(!mbar_wait_bounded(&fullBar[stage], (it / stages) & 1, &abortFlag, status, SITE_DW_FULL)) break;
		unsigned r = t;
		const int chunk = r % chunks; r /= chunks;
		const int tx = r % tilesX; r /= tilesX;
		const int ty = r % tilesY;
		const unsigned n = r / tilesY;
		const unsigned cq = chunk * (DW_CC / 4) + q;
		if(active && cq < cv) {
			const float4* flt = reinterpret_cast<const float4*>(filter) + cq;
			float4 f[9];
#pragma unroll
			for(int i = 0; i < 9; ++i) f[i] = __ldg(flt + i * cv);
			const float4 b = freeTerm != nullptr ? __ldg(reinterpret_cast<const float4*>(freeTerm) + cq) : make_float4(0.f, 0.f, 0.f, 0.f);
			const int oy0 = ty * th + part * DW_RPP, ox0 = tx * tw + strip * TW;
			// this thread's corner of the input box, in 16-byte units (a pixel is 8 of them)
			const float4* box = reinterpret_cast<const float4*>(smem + stage * stageBytes)
				+ (static_cast<size_t>(part * DW_RPP * STRIDE) * colsIn + strip * TW * STRIDE) * (DW_CC / 4) + q;
			auto loadRow = [&](int row, float4 (&dst)[COLS]) {
#pragma unroll
				for(int k = 0; k < COLS; ++k) dst[k] = box[(row * colsIn + k) * (DW_CC / 4)];
			};
			float4* out = reinterpret_cast<float4*>(y) + ((static_cast<size_t>(n) * p.ho + oy0) * p.wo + ox0) * cv + cq;
			float4 win[3][COLS];
#pragma unroll
			for(int k = 0; k < 3 - STRIDE; ++k) loadRow(k, win[k]);
#pragma unroll
			for(int j = 0; j < DW_RPP; ++j) {
				if(oy0 + j >= p.ho) break;
				const int top = STRIDE * j;
#pragma unroll
				for(int k = 3 - STRIDE; k < 3; ++k) loadRow(top + k, win[(top + k) % 3]);
				float4 a[TW];
#pragma unroll
				for(int i = 0; i < TW; ++i) a[i] = b;
#pragma unroll
				for(int fy = 0; fy < 3; ++fy) {
#pragma unroll
					for(int fx = 0; fx < 3; ++fx) {
						const float4 w = f[3 * fy + fx];
#pragma unroll
						for(int i = 0; i < TW; ++i) {
							const float4 v = win[(top + fy) % 3][i * STRIDE + fx];
							a[i].x = fmaf(v.x, w.x, a[i].x); a[i].y = fmaf(v.y, w.y, a[i].y);
							a[i].z = fmaf(v.z, w.z, a[i].z); a[i].w = fmaf(v.w, w.w, a[i].w);
						}
					}
				}
#pragma unroll
				for(int i = 0; i < TW; ++i) {
					if(ox0 + i >= p.wo) break;
					float4 o = a[i];
					if(act == NB200_ACT_HSWISH) {
						o.x = apply_act(o.x, act, actParam); o.y = apply_act(o.y, act, actParam);
						o.z = apply_act(o.z, act, actParam); o.w = apply_act(o.w, act, actParam);
					} else {
						o.x = relu ? fminf(fmaxf(o.x, 0.f), reluHi) : o.x; o.y = relu ? fminf(fmaxf(o.y, 0.f), reluHi) : o.y;
						o.z = relu ? fminf(fmaxf(o.z, 0.f), reluHi) : o.z; o.w = relu ? fminf(fmaxf(o.w, 0.f), reluHi) : o.w;
					}
					out[(static_cast<size_t>(j) * p.wo + i) * cv] = o;
				}
			}
		}
		__syncthreads(); // every thread has read this stage: a later copy may overwrite it
	}
}

// 3x3 / stride 2 max pooling without indices (the inference form; ResNet's stem pool), channels a multiple of four:
// a thread owns four channels of a strip of TW output columns and slides along it, so the column shared by two
// neighbouring windows is loaded once.  Window order (rows outer, columns inner) and the `v > best` comparison are those
// of the general kernel, so the results are identical.
constexpr int MP3_TW = 4;

// PADDED: the image the windows slide over is x surrounded by a constant border (`top` rows above, `left` columns to
// the left, p.h x p.w being the padded extent and inH x inW the extent of x itself); positions in the border read as
// `border`.  The result is that of padding into a buffer first and pooling that buffer.
template<bool PADDED>
__global__ void __launch_bounds__(256) maxpool3x3s2_kernel(const Pool2d p, const float* __restrict__ x, float* __restrict__ y,
	int strips, unsigned total, int inH, int inW, int top, int left, float border)
{
	const unsigned cv = p.c / 4;
	for(unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
		unsigned r = t;
		const unsigned cq = r % cv; r /= cv;
		const unsigned sx = r % strips; r /= strips;
		const unsigned oy = r % p.ho;
		const unsigned n = r / p.ho;
		const int ox0 = sx * MP3_TW;
		float4* out = reinterpret_cast<float4*>(y) + ((static_cast<size_t>(n) * p.ho + oy) * p.wo + ox0) * cv + cq;
		const int outs = min(MP3_TW, p.wo - ox0);
		// all columns of the strip first (2 * outs + 1 of them, three rows each): many independent loads in flight
		float4 col[2 * MP3_TW + 1][3];
		if(PADDED) {
			const float4* img = reinterpret_cast<const float4*>(x) + static_cast<size_t>(n) * inH * inW * cv + cq;
			const int iy0 = 2 * static_cast<int>(oy) - top, ix0 = 2 * ox0 - left;
#pragma unroll
			for(int k = 0; k < 2 * MP3_TW + 1; ++k) {
				if(k <= 2 * outs) {
#pragma unroll
					for(int fy = 0; fy < 3; ++fy) {
						const int iy = iy0 + fy, ix = ix0 + k;
						col[k][fy] = iy >= 0 && iy < inH && ix >= 0 && ix < inW
							? __ldg(img + (static_cast<size_t>(iy) * inW + ix) * cv) : make_float4(border, border, border, border);
					}
				}
			}
		} else {
			const float4* img = reinterpret_cast<const float4*>(x) + (static_cast<size_t>(n) * p.h + 2 * oy) * p.w * cv + cq;
#pragma unroll
			for(int k = 0; k < 2 * MP3_TW + 1; ++k) {
				if(k <= 2 * outs) {
#pragma unroll
					for(int fy = 0; fy < 3; ++fy) col[k][fy] = __ldg(img + (static_cast<size_t>(fy) * p.w + 2 * ox0 + k) * cv);
				}
			}
		}
#pragma unroll
		for(int j = 0; j < MP3_TW; ++j) {
			if(j >= outs) break;
			float4 best = col[2 * j][0];
#pragma unroll
			for(int fy = 0; fy < 3; ++fy) {
#pragma unroll
				for(int fx = 0; fx < 3; ++fx) {
					const float4 v = col[2 * j + fx][fy];
					best.x = v.x > best.x ? v.x : best.x; best.y = v.y > best.y ? v.y : best.y;
					best.z = v.z > best.z ? v.z : best.z; best.w = v.w > best.w ? v.w : best.w;
				}
			}
			out[static_cast<size_t>(j) * cv] = best;
		}
	}
}

int pool_common(void* stream, bool isMax, int batch, int h, int w, int c, int fh, int fw, int sh, int sw,
	const float* x, float* y, int* maxIndices)
{
	if(batch < 0 || h <= 0 || w <= 0 || c <= 0 || fh <= 0 || fw <= 0 || sh <= 0 || sw <= 0 || fh > h || fw > w) {
		return NB200_EINVAL;
	}
	Pool2d p = { batch, h, w, c, fh, fw, sh, sw, (h - fh) / sh + 1, (w - fw) / sw + 1 };
	const long long outElems = static_cast<long long>(batch) * p.ho * p.wo * c;
	if(outElems == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	const bool vec = c % 4 == 0 && aligned16(x) && aligned16(y);
	cudaStream_t s = as_stream(stream);
	if(vec && isMax && maxIndices == nullptr && fh == 3 && fw == 3 && sh == 2 && sw == 2 && outElems / 4 < 0x7fffffffLL
		&& static_cast<long long>(batch) * h * w * c < 0x7fffffffLL) {
		const int strips = (p.wo + MP3_TW - 1) / MP3_TW;
		const long long total = static_cast<long long>(batch) * p.ho * strips * (c / 4);
		maxpool3x3s2_kernel<false><<<grid_for(total, 256, 16), 256, 0, s>>>(p, x, y, strips, static_cast<unsigned>(total), h, w, 0, 0, 0.f);
	} else if(vec) {
		const long long total = outElems / 4;
		if(isMax) pool_kernel<true, 4><<<grid_for(total, 256, 16), 256, 0, s>>>(p, x, y, maxIndices, total);
		else pool_kernel<false, 4><<<grid_for(total, 256, 16), 256, 0, s>>>(p, x, y, nullptr, total);
	} else {
		if(isMax) pool_kernel<true, 1><<<grid_for(outElems, 256, 16), 256, 0, s>>>(p, x, y, maxIndices, outElems);
		else pool_kernel<false, 1><<<grid_for(outElems, 256, 16), 256, 0, s>>>(p, x, y, nullptr, outElems);
	}
	count_launch();
	return check_launch();
}

// Launches the TMA-staged kernel when the image is large enough to give every SM several tiles; false = not applicable
// (the register kernels take over).
bool chconv3x3_by_tma(const nb200_chconv_desc* d, const float* x, const float* filter, const float* freeTerm, float* y,
	int act, float actParam, cudaStream_t s)
{
	const int stride = d->stride_h;
	const int tw1 = stride == 1 ? 4 : 2, extra = stride == 1 ? 2 : 1;
	int strips = (d->wo + tw1 - 1) / tw1;
	if(strips > 32) strips = 32;
	// balance the column tiles (57 columns: two tiles of 8 strips, not 14 + 1)
	const int tilesX0 = (d->wo + strips * tw1 - 1) / (strips * tw1);
	strips = ((d->wo + tilesX0 - 1) / tilesX0 + tw1 - 1) / tw1;
	const int tw = strips * tw1;
	const int tilesX = (d->wo + tw - 1) / tw;
	int rowParts = 256 / (8 * strips);
	const int wantParts = (d->ho + DW_RPP - 1) / DW_RPP;
	if(rowParts > wantParts) rowParts = wantParts;
	const int colsIn = tw * stride + extra;
	auto stage_bytes = [&](int parts) { return static_cast<size_t>(parts * DW_RPP * stride + extra) * colsIn * DW_CC * 4; };
	while(rowParts > 1 && stage_bytes(rowParts) > 100 * 1024) --rowParts;
	if(stage_bytes(rowParts) > 100 * 1024) return false;
	const int th = rowParts * DW_RPP;
	const int tilesY = (d->ho + th - 1) / th;
	const int chunks = (d->c + DW_CC - 1) / DW_CC;
	const long long numTiles = static_cast<long long>(d->batch) * tilesY * tilesX * chunks;
	const int sms = sm_count();
	if(numTiles < 8LL * sms || numTiles > 0x7fffffffLL) return false;
	alignas(64) CUtensorMap map;
	if(!make_image_box_map(&map, x, d->c, d->w, d->h, d->batch, DW_CC, colsIn, th * stride + extra)) return false;
	// two CTAs per SM when two stages each fit, else one CTA with as many stages as fit
	int stages = static_cast<int>((112 * 1024) / stage_bytes(rowParts));
	if(stages < 2) stages = static_cast<int>((225 * 1024) / stage_bytes(rowParts));
	if(stages > DW_MAX_STAGES) stages = DW_MAX_STAGES;
	const size_t smemBytes = stages * stage_bytes(rowParts) + 128;
	static std::atomic<bool> attrSet[64];
	int dev = 0;
	if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
	if(!attrSet[dev].load()) {
		if(cudaFuncSetAttribute(chconv3x3_tma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess
			|| cudaFuncSetAttribute(chconv3x3_tma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) {
			cudaGetLastError();
			return false;
		}
		attrSet[dev].store(true);
	}
	const long long perSm = static_cast<long long>(227 * 1024) / static_cast<long long>(smemBytes + 1024);
	long long grid = sms * (perSm < 1 ? 1 : (perSm > 2 ? 2 : perSm));
	if(grid > numTiles) grid = numTiles;
	int* status = device_status_word();
	if(stride == 1) {
		chconv3x3_tma_kernel<1><<<static_cast<unsigned>(grid), 256, smemBytes, s>>>(*d, map, filter, freeTerm, y, act, actParam,
			strips, rowParts, tilesX, tilesY, chunks, static_cast<unsigned>(numTiles), stages, status);
	} else {
		chconv3x3_tma_kernel<2><<<static_cast<unsigned>(grid), 256, smemBytes, s>>>(*d, map, filter, freeTerm, y, act, actParam,
			strips, rowParts, tilesX, tilesY, chunks, static_cast<unsigned>(numTiles), stages, status);
	}
	return true;
}

// y[image][pixel][c] = act(x[image][pixel][c] * scale[image][c]): the squeeze-and-excite gate of a MobileNetV3 block
// applied to the channelwise convolution's output, with the activation that follows it.  V = 4: 16-byte pieces.
template<int V>
__global__ void __launch_bounds__(256) scale_channels_act_kernel(const float* __restrict__ x, const float* __restrict__ scale,
	float* __restrict__ y, long long total, int channelVecs, long long imageVecs, int act, float actParam)
{
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
		const long long image = i / imageVecs;
		const int cv = static_cast<int>(i % channelVecs);
		if(V == 4) {
			float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
			const float4 g = __ldg(reinterpret_cast<const float4*>(scale) + image * channelVecs + cv);
			v.x = apply_act(v.x * g.x, act, actParam); v.y = apply_act(v.y * g.y, act, actParam);
			v.z = apply_act(v.z * g.z, act, actParam); v.w = apply_act(v.w * g.w, act, actParam);
			reinterpret_cast<float4*>(y)[i] = v;
		} else {
			y[i] = apply_act(__ldg(x + i) * __ldg(scale + image * channelVecs + cv), act, actParam);
		}
	}
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_blob_max_pooling(void* stream, int batch, int h, int w, int c, int filter_h, int filter_w, int stride_h,
	int stride_w, const float* x, float* y, int* max_indices)
{
	return pool_common(stream, true, batch, h, w, c, filter_h, filter_w, stride_h, stride_w, x, y, max_indices);
}

int nb200_blob_max_pooling_padded(void* stream, int batch, int h, int w, int c, int pad_left, int pad_right, int pad_top,
	int pad_bottom, float pad_value, int filter_h, int filter_w, int stride_h, int stride_w, const float* x, float* y)
{
	if(batch < 0 || h <= 0 || w <= 0 || c <= 0 || pad_left < 0 || pad_right < 0 || pad_top < 0 || pad_bottom < 0) return NB200_EINVAL;
	const int ph = h + pad_top + pad_bottom, pw = w + pad_left + pad_right;
	// the one form that exists: 3x3 windows, stride 2, whole float4 channel groups (the stem pool of the ResNets)
	if(filter_h != 3 || filter_w != 3 || stride_h != 2 || stride_w != 2 || c % 4 != 0 || ph < 3 || pw < 3) return NB200_EINVAL;
	Pool2d p = { batch, ph, pw, c, 3, 3, 2, 2, (ph - 3) / 2 + 1, (pw - 3) / 2 + 1 };
	const long long outElems = static_cast<long long>(batch) * p.ho * p.wo * c;
	if(outElems == 0) return NB200_OK;
	if(x == nullptr || y == nullptr || !aligned16(x) || !aligned16(y)) return NB200_EINVAL;
	if(outElems / 4 >= 0x7fffffffLL || static_cast<long long>(batch) * h * w * c >= 0x7fffffffLL) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	const int strips = (p.wo + MP3_TW - 1) / MP3_TW;
	const long long total = static_cast<long long>(batch) * p.ho * strips * (c / 4);
	maxpool3x3s2_kernel<true><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p, x, y, strips,
		static_cast<unsigned>(total), h, w, pad_top, pad_left, pad_value);
	count_launch();
	return check_launch();
}

int nb200_blob_mean_pooling(void* stream, int batch, int h, int w, int c, int filter_h, int filter_w, int stride_h,
	int stride_w, const float* x, float* y)
{
	return pool_common(stream, false, batch, h, w, c, filter_h, filter_w, stride_h, stride_w, x, y, nullptr);
}

int nb200_blob_resize_image(void* stream, int batch, int h, int w, int c, int delta_left, int delta_right,
	int delta_top, int delta_bottom, int padding, float default_value, const float* x, float* y)
{
	if(batch < 0 || h <= 0 || w <= 0 || c <= 0 || padding < 0 || padding > 2) return NB200_EINVAL;
	const int ho = h + delta_top + delta_bottom, wo = w + delta_left + delta_right;
	if(ho <= 0 || wo <= 0) return NB200_EINVAL;
	const long long outElems = static_cast<long long>(batch) * ho * wo * c;
	if(outElems == 0) return NB200_OK;
	if(x == nullptr || y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	Resize p = { batch, h, w, c, delta_left, delta_top, ho, wo, padding, default_value };
	cudaStream_t s = as_stream(stream);
	if(c % 4 == 0 && aligned16(x) && aligned16(y)) {
		resize_kernel<4><<<grid_for(outElems / 4, 256, 16), 256, 0, s>>>(p, x, y, outElems / 4);
	} else {
		resize_kernel<1><<<grid_for(outElems, 256, 16), 256, 0, s>>>(p, x, y, outElems);
	}
	count_launch();
	return check_launch();
}

int nb200_scale_channels_activation(void* stream, int batch, int pixels, int channels, const float* x, const float* scale,
	int act, float act_param, float* y)
{
	if(batch < 0 || pixels < 0 || channels < 0) return NB200_EINVAL;
	const long long total = static_cast<long long>(batch) * pixels * channels;
	if(total == 0) return NB200_OK;
	if(x == nullptr || scale == nullptr || y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	cudaStream_t s = as_stream(stream);
	if(channels % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(scale)) {
		scale_channels_act_kernel<4><<<grid_for(total / 4, 256, 16), 256, 0, s>>>(x, scale, y, total / 4, channels / 4,
			static_cast<long long>(pixels) * (channels / 4), act, act_param);
	} else {
		scale_channels_act_kernel<1><<<grid_for(total, 256, 16), 256, 0, s>>>(x, scale, y, total, channels,
			static_cast<long long>(pixels) * channels, act, act_param);
	}
	count_launch();
	return check_launch();
}

int nb200_blob_channelwise_convolution(void* stream, const nb200_chconv_desc* d, const float* x, const float* filter,
	const float* free_term, float* y, int act, float act_param)
{
	if(d == nullptr) return NB200_EINVAL;
	if(d->batch < 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->r <= 0 || d->s <= 0 || d->stride_h <= 0
		|| d->stride_w <= 0 || d->pad_h < 0 || d->pad_w < 0) {
		return NB200_EINVAL;
	}
	const int ho = 1 + (d->h - d->r + 2 * d->pad_h) / d->stride_h;
	const int wo = 1 + (d->w - d->s + 2 * d->pad_w) / d->stride_w;
	if(ho != d->ho || wo != d->wo || ho <= 0 || wo <= 0) return NB200_EINVAL;
	const long long outElems = static_cast<long long>(d->batch) * ho * wo * d->c;
	if(outElems == 0) return NB200_OK;
	if(x == nullptr || filter == nullptr || y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	cudaStream_t s = as_stream(stream);
	const bool vec = d->c % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(filter)
		&& (free_term == nullptr || aligned16(free_term));
	if(vec && d->r == 3 && d->s == 3 && d->pad_h == 1 && d->pad_w == 1 && d->stride_h == d->stride_w && (d->stride_h == 1 || d->stride_h == 2)
		&& static_cast<long long>(d->batch) * d->h * d->w * d->c < 0x7fffffffLL) {
		const int tw = d->stride_h == 1 ? 4 : 2;
		const int strips = (wo + tw - 1) / tw;
		const long long total = static_cast<long long>(d->batch) * ho * strips * (d->c / 4);
		// row blocks when that still gives every SM a few thousand threads
		constexpr int TH = 8;
		const int rowGroups = (ho + TH - 1) / TH;
		const long long totalRows = static_cast<long long>(d->batch) * rowGroups * strips * (d->c / 4);
		if(chconv3x3_by_tma(d, x, filter, free_term, y, act, act_param, s)) {
			count_launch();
			return check_launch();
		}
		const size_t filterBytes = static_cast<size_t>(9) * d->c * sizeof(float);
		if(ho >= TH && totalRows >= 148LL * 1536 && totalRows < 0xffffffffLL && filterBytes <= 40 * 1024) {
			if(d->stride_h == 1) chconv3x3_rows_kernel<1, TH><<<grid_for(totalRows, 128, 24), 128, filterBytes, s>>>(*d, x, filter, free_term, y, act, act_param, strips, rowGroups, static_cast<unsigned>(totalRows));
			else chconv3x3_rows_kernel<2, TH><<<grid_for(totalRows, 128, 24), 128, filterBytes, s>>>(*d, x, filter, free_term, y, act, act_param, strips, rowGroups, static_cast<unsigned>(totalRows));
		} else if(d->stride_h == 1) chconv3x3_kernel<1><<<grid_for(total, 256, 16), 256, 0, s>>>(*d, x, filter, free_term, y, act, act_param, strips, static_cast<unsigned>(total));
		else chconv3x3_kernel<2><<<grid_for(total, 256, 16), 256, 0, s>>>(*d, x, filter, free_term, y, act, act_param, strips, static_cast<unsigned>(total));
	} else if(vec) {
		chconv_kernel<4><<<grid_for(outElems / 4, 256, 16), 256, 0, s>>>(*d, x, filter, free_term, y, act, act_param, outElems / 4);
	} else {
		chconv_kernel<1><<<grid_for(outElems, 256, 16), 256, 0, s>>>(*d, x, filter, free_term, y, act, act_param, outElems);
	}
	count_launch();
	return check_launch();
}

} // extern "C"
