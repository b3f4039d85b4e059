// MobileNetV2 inverted-residual block as ONE kernel (stride 1, 32 input channels, up to 192 expanded channels):
//   y = [x +] W_down * act2( dw3x3( act1( W_exp * x + b_exp ) ) + b_dw ) + b_down
// The expanded activations never leave the SM: algorithmic traffic is the input once (plus its halo), the output once
// and the weights.
//
// A persistent CTA (one per SM) walks output tiles of 8 x 16 pixels.  Per tile:
//   1. TMA brings the 10 x 18 halo patch of x (32 channels = one 128-byte row per pixel, 128-byte swizzle, zeros
//      outside the image) into shared memory; the threads derive the "lo" part of the 3xTF32 split beside it.
//   2. Expand: tcgen05.mma kind::tf32 (A = the patch, 2 x 128 rows; B = W_exp, resident in shared memory; 3 MMAs per
//      product: lo*hi + hi*hi + hi*lo) into tensor memory, all expanded channels at once.  When the MMAs have
//      completed the patch buffer is free and the next tile's TMA load is issued: it lands while this tile is worked on.
//   3. Per chunk of 32 expanded channels: tcgen05.ld -> + bias, activation, zero outside the image (the depthwise
//      convolution pads the EXPANDED image with zeros) -> shared memory; depthwise 3x3 with a warp per output column
//      and a lane per channel (a 10 x 3 register window gives eight outputs) + bias + activation -> written, split in
//      hi / lo, as the K-major A operand of the project product; project: tcgen05.mma accumulates the chunk into the
//      output tile in tensor memory.
//   4. tcgen05.ld of the output tile -> + bias, + residual -> global memory (128 bytes per pixel).
// Every wait is bounded (common.cuh); on a time-out the kernel records it in the status word, frees its tensor memory
// and returns.
#include "contraction.cuh"

#include <cuda.h>

namespace nb200 {

namespace {

constexpr int TH = 8, TW = 16;              // output tile
constexpr int HH = TH + 2, HW = TW + 2;     // halo patch
constexpr int HALO = HH * HW;               // 180 pixels
constexpr int CIN = 32;                     // input channels = K of the expand product = one 128-byte row
constexpr int CHUNK = 32;                   // expanded channels per depthwise / project step
constexpr int E_STRIDE = CHUNK + 1;         // floats per pixel of the expanded chunk in shared memory (no bank conflicts
                                            // for a thread per pixel writing and for a lane per channel reading)
constexpr int THREADS = 256;
constexpr int MAX_CEXP = 192, MAX_COUT = 64;
constexpr int PATCH_BYTES = HALO * 128;     // what one TMA load delivers
constexpr int PATCH_ROOM = (PATCH_BYTES + 1023) / 1024 * 1024;
constexpr int KERNEL_ID = 0x6d;             // in the status word: (KERNEL_ID << 8) | site
enum { SITE_PATCH = 1, SITE_EXPAND = 2, SITE_PROJECT = 3 };

struct FusedParams {
	const float* x;
	float* y;
	const float* wExp; const float* bExp;
	const float* wDw; const float* bDw;
	const float* wDown; const float* bDown;
	int batch, h, w, cExp, cOut;
	int residual;
	int actExp, actDw;
	float actExpParam, actDwParam;
	int tilesX, tilesY, numTiles;
	int* status;
};

// byte offset of element k (0..31) of row r in a K-major tile of 128-byte rows with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t k)
{
	return r * 128u + ((((k >> 2) ^ (r & 7u)) << 4) | ((k & 3u) << 2));
}

__device__ __forceinline__ float lo_part(float v)
{
	return v - __uint_as_float(__float_as_uint(v) & 0xffffe000u);
}

struct SmemLayout {
	uint32_t patchHi, patchLo, wExpHi, wExpLo, wDownHi, wDownLo, e, a2Hi, a2Lo, consts, bars, total;
};

__host__ __device__ inline SmemLayout smem_layout(int cExp, int cOut)
{
	SmemLayout l;
	uint32_t at = 0;
	l.patchHi = at; at += PATCH_ROOM;
	l.patchLo = at; at += PATCH_ROOM;
	// the second 128-row block of the patch operands reaches 256 rows: whatever follows is read as rows that no one uses
	l.wExpHi = at; at += cExp * 128;
	l.wExpLo = at; at += cExp * 128;
	l.wDownHi = at; at += (cExp / CHUNK) * cOut * 128;
	l.wDownLo = at; at += (cExp / CHUNK) * cOut * 128;
	l.a2Hi = at; at += 128 * 128;
	l.a2Lo = at; at += 128 * 128;
	l.e = at; at += (HALO * E_STRIDE * 4 + 15) / 16 * 16;
	l.consts = at; at += (11 * cExp + cOut) * 4;   // bExp, bDw, wDw[9], bDown
	at = (at + 15) / 16 * 16;
	l.bars = at; at += 64;
	l.total = at;
	return l;
}

template<bool THREEX>
__global__ void __launch_bounds__(THREADS, 1) mbv2_fused_kernel(const FusedParams p, const __grid_constant__ CUtensorMap mapX)
{
	extern __shared__ uint8_t smemRaw[];
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
	const SmemLayout L = smem_layout(p.cExp, p.cOut);
	float* const e = reinterpret_cast<float*>(smem + L.e);
	float* const bExp = reinterpret_cast<float*>(smem + L.consts);
	float* const bDw = bExp + p.cExp;
	float* const wDw = bDw + p.cExp;            // [9][cExp]
	float* const bDown = wDw + 9 * p.cExp;
	uint64_t* const patchBar = reinterpret_cast<uint64_t*>(smem + L.bars);
	uint64_t* const expandBar = patchBar + 1;
	uint64_t* const projectBar = patchBar + 2;
	uint32_t* const tmemSlot = reinterpret_cast<uint32_t*>(patchBar + 3);
	volatile int* const abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const int chunks = p.cExp / CHUNK;

	if(tid == 0) {
		mbar_init(patchBar, 1);
		mbar_init(expandBar, 1);
		mbar_init(projectBar, 1);
		*abortFlag = 0;
		mbar_init_fence();
		tma_prefetch_descriptor(&mapX);
	}
	if(warp == 0) {
		tmem_alloc(tmemSlot, 512);
		tmem_relinquish();
	}
	// the weights, once per CTA: expand [cExp][32] and project [cOut][cExp] as swizzled K-major tiles, hi and lo
	for(int i = tid; i < p.cExp * CIN; i += THREADS) {
		const uint32_t n = i >> 5, k = i & 31;
		const float v = __ldg(p.wExp + i);
		const uint32_t off = swz(n, k);
		if(THREEX) {
			*reinterpret_cast<float*>(smem + L.wExpHi + off) = v;
			*reinterpret_cast<float*>(smem + L.wExpLo + off) = lo_part(v);
		} else {
			*reinterpret_cast<float*>(smem + L.wExpHi + off) = to_tf32(v);
		}
	}
	for(int i = tid; i < p.cOut * p.cExp; i += THREADS) {
		const uint32_t n = i / p.cExp, kk = i - n * p.cExp;
		const uint32_t c = kk >> 5, k = kk & 31;
		const float v = __ldg(p.wDown + i);
		const uint32_t off = c * p.cOut * 128 + swz(n, k);
		if(THREEX) {
			*reinterpret_cast<float*>(smem + L.wDownHi + off) = v;
			*reinterpret_cast<float*>(smem + L.wDownLo + off) = lo_part(v);
		} else {
			*reinterpret_cast<float*>(smem + L.wDownHi + off) = to_tf32(v);
		}
	}
	for(int i = tid; i < p.cExp; i += THREADS) {
		bExp[i] = p.bExp != nullptr ? __ldg(p.bExp + i) : 0.f;
		bDw[i] = p.bDw != nullptr ? __ldg(p.bDw + i) : 0.f;
#pragma unroll
		for(int t = 0; t < 9; ++t) wDw[t * p.cExp + i] = __ldg(p.wDw + t * p.cExp + i);
	}
	for(int i = tid; i < p.cOut; i += THREADS) bDown[i] = p.bDown != nullptr ? __ldg(p.bDown + i) : 0.f;
	fence_proxy_async_smem();
	tc_fence_before_sync();
	__syncthreads();
	tc_fence_after_sync();
	const uint32_t tmemBase = *tmemSlot;
	const uint32_t accExpand = tmemBase;                      // two blocks of cExp columns: patch rows 0..127, 128..255
	const uint32_t accProject = tmemBase + 2 * p.cExp;        // cOut columns
	const uint32_t idescExpand = umma_idesc_tf32(128, p.cExp);
	const uint32_t idescProject = umma_idesc_tf32(128, p.cOut);

	auto tile_origin = [&](int tile, int& n, int& y0, int& x0) {
		const int perImage = p.tilesX * p.tilesY;
		n = tile / perImage;
		const int r = tile - n * perImage;
		const int tyi = r / p.tilesX;
		y0 = tyi * TH;
		x0 = (r - tyi * p.tilesX) * TW;
	};
	auto load_patch = [&](int tile) {
		int n, y0, x0;
		tile_origin(tile, n, y0, x0);
		mbar_arrive_expect_tx(patchBar, PATCH_BYTES);
		tma_load_4d(smem_u32(smem + L.patchHi), &mapX, patchBar, 0, x0 - 1, y0 - 1, n);
	};

	bool ok = true;
	uint32_t projectCommits = 0; // project commits issued so far (same count in every thread)
	if(tid == 0 && static_cast<int>(blockIdx.x) < p.numTiles) load_patch(blockIdx.x);
	int local = 0;
	for(int tile = blockIdx.x; tile < p.numTiles && ok; tile += gridDim.x, ++local) {
		int img, y0, x0;
		tile_origin(tile, img, y0, x0);
		// ---- 1. the patch has landed; its lo part (or, in plain TF32, its rounded copy) beside it
		// (every wait is followed by a block-wide vote, so that all threads leave together if one of them gave up)
		ok = mbar_wait_bounded(patchBar, local & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PATCH);
		if(!__syncthreads_and(ok)) { ok = false; break; }
		for(int i = tid; i < HALO * 8; i += THREADS) {
			float4 v = *reinterpret_cast<const float4*>(smem + L.patchHi + i * 16);
			if(THREEX) {
				v.x = lo_part(v.x); v.y = lo_part(v.y); v.z = lo_part(v.z); v.w = lo_part(v.w);
			} else {
				v.x = to_tf32(v.x); v.y = to_tf32(v.y); v.z = to_tf32(v.z); v.w = to_tf32(v.w);
			}
			*reinterpret_cast<float4*>(smem + L.patchLo + i * 16) = v;
		}
		fence_proxy_async_smem();
		tc_fence_before_sync();
		__syncthreads();
		// ---- 2. expand, all channels
		if(tid == 0) {
			tc_fence_after_sync();
			const uint64_t bHi = umma_desc_k128(smem_u32(smem + L.wExpHi));
			const uint64_t bLo = umma_desc_k128(smem_u32(smem + L.wExpLo));
#pragma unroll
			for(int mt = 0; mt < 2; ++mt) {
				const uint64_t aHi = umma_desc_k128(smem_u32(smem + L.patchHi) + mt * 128 * 128);
				const uint64_t aLo = umma_desc_k128(smem_u32(smem + L.patchLo) + mt * 128 * 128);
				const uint32_t d = accExpand + mt * p.cExp;
#pragma unroll
				for(int ks = 0; ks < CIN / 8; ++ks) {
					if(THREEX) {
						umma_tf32_ss(d, aLo + 2 * ks, bHi + 2 * ks, idescExpand, ks > 0 ? 1u : 0u);
						umma_tf32_ss(d, aHi + 2 * ks, bHi + 2 * ks, idescExpand, 1u);
						umma_tf32_ss(d, aHi + 2 * ks, bLo + 2 * ks, idescExpand, 1u);
					} else {
						umma_tf32_ss(d, aLo + 2 * ks, bHi + 2 * ks, idescExpand, ks > 0 ? 1u : 0u); // the rounded copy
					}
				}
			}
			umma_commit(expandBar);
		}
		ok = mbar_wait_bounded(expandBar, local & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_EXPAND);
		if(!__syncthreads_and(ok)) { ok = false; break; }
		tc_fence_after_sync();
		// the patch buffers are free: the next tile's patch travels while this tile is worked on
		if(tid == 0 && tile + static_cast<int>(gridDim.x) < p.numTiles) load_patch(tile + gridDim.x);

		const int quad = warp & 3, half = warp >> 2;
		for(int c = 0; c < chunks && ok; ++c) {
			// ---- 3a. expanded chunk: tensor memory -> + bias, activation, zero outside the image -> shared memory
#pragma unroll
			for(int mt = 0; mt < 2; ++mt) {
				const int rowBase = mt * 128 + quad * 32;
				if(rowBase < HALO) { // warp-uniform
					float v[16];
					tmem_ld16(accExpand + (static_cast<uint32_t>(quad * 32) << 16) + mt * p.cExp + c * CHUNK + half * 16, v);
					const int row = rowBase + lane;
					if(row < HALO) {
						const int hy = row / HW, hx = row - hy * HW;
						const int gy = y0 - 1 + hy, gx = x0 - 1 + hx;
						const bool inside = gy >= 0 && gy < p.h && gx >= 0 && gx < p.w;
						float* dst = e + row * E_STRIDE + half * 16;
						const float* b = bExp + c * CHUNK + half * 16;
#pragma unroll
						for(int j = 0; j < 16; ++j) dst[j] = inside ? apply_act(v[j] + b[j], p.actExp, p.actExpParam) : 0.f;
					}
				}
			}
			// the project MMAs of the chunk before have to be through with the A tile that is overwritten next
			ok = projectCommits == 0
				|| mbar_wait_bounded(projectBar, (projectCommits - 1) & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PROJECT);
			if(!__syncthreads_and(ok)) { ok = false; break; }
			// ---- 3b. depthwise 3x3: a warp per output column, a lane per channel
			{
				const int ch = c * CHUNK + lane;
				float k[9];
#pragma unroll
				for(int t = 0; t < 9; ++t) k[t] = wDw[t * p.cExp + ch];
				const float bias = bDw[ch];
#pragma unroll
				for(int col = 0; col < 2; ++col) {
					const int tx = warp * 2 + col;
					float win[HH][3];
#pragma unroll
					for(int hy = 0; hy < HH; ++hy) {
#pragma unroll
						for(int dx = 0; dx < 3; ++dx) win[hy][dx] = e[(hy * HW + tx + dx) * E_STRIDE + lane];
					}
#pragma unroll
					for(int ty = 0; ty < TH; ++ty) {
						float acc = 0.f;
#pragma unroll
						for(int dy = 0; dy < 3; ++dy) {
#pragma unroll
							for(int dx = 0; dx < 3; ++dx) acc = fmaf(win[ty + dy][dx], k[dy * 3 + dx], acc);
						}
						const float v = apply_act(acc + bias, p.actDw, p.actDwParam);
						const uint32_t off = swz(ty * TW + tx, lane);
						if(THREEX) {
							*reinterpret_cast<float*>(smem + L.a2Hi + off) = v;
							*reinterpret_cast<float*>(smem + L.a2Lo + off) = lo_part(v);
						} else {
							*reinterpret_cast<float*>(smem + L.a2Hi + off) = to_tf32(v);
						}
					}
				}
			}
			fence_proxy_async_smem();
			tc_fence_before_sync();
			__syncthreads();
			// ---- 3c. project: this chunk's 32 channels into the output tile
			if(tid == 0) {
				tc_fence_after_sync();
				const uint64_t aHi = umma_desc_k128(smem_u32(smem + L.a2Hi));
				const uint64_t aLo = umma_desc_k128(smem_u32(smem + L.a2Lo));
				const uint64_t bHi = umma_desc_k128(smem_u32(smem + L.wDownHi) + c * p.cOut * 128);
				const uint64_t bLo = umma_desc_k128(smem_u32(smem + L.wDownLo) + c * p.cOut * 128);
#pragma unroll
				for(int ks = 0; ks < CHUNK / 8; ++ks) {
					const uint32_t first = (c > 0 || ks > 0) ? 1u : 0u;
					if(THREEX) {
						umma_tf32_ss(accProject, aLo + 2 * ks, bHi + 2 * ks, idescProject, first);
						umma_tf32_ss(accProject, aHi + 2 * ks, bHi + 2 * ks, idescProject, 1u);
						umma_tf32_ss(accProject, aHi + 2 * ks, bLo + 2 * ks, idescProject, 1u);
					} else {
						umma_tf32_ss(accProject, aHi + 2 * ks, bHi + 2 * ks, idescProject, first);
					}
				}
				umma_commit(projectBar);
			}
			++projectCommits;
		}
		if(!ok) break;
		// ---- 4. the output tile
		ok = mbar_wait_bounded(projectBar, (projectCommits - 1) & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PROJECT);
		if(!__syncthreads_and(ok)) { ok = false; break; }
		tc_fence_after_sync();
		{
			const int px = quad * 32 + lane;
			const int ty = px / TW, tx = px - ty * TW;
			const int gy = y0 + ty, gx = x0 + tx;
			const bool valid = gy < p.h && gx < p.w;
			const size_t pixel = (static_cast<size_t>(img) * p.h + gy) * p.w + gx;
			for(int piece = half; piece * 16 < p.cOut; piece += 2) {
				float v[16];
				tmem_ld16(accProject + (static_cast<uint32_t>(quad * 32) << 16) + piece * 16, v);
				if(valid) {
					float* dst = p.y + pixel * p.cOut + piece * 16;
					const float* res = p.residual ? p.x + pixel * CIN + piece * 16 : nullptr;
#pragma unroll
					for(int q = 0; q < 4; ++q) {
						float4 o = make_float4(v[4 * q] + bDown[piece * 16 + 4 * q], v[4 * q + 1] + bDown[piece * 16 + 4 * q + 1],
							v[4 * q + 2] + bDown[piece * 16 + 4 * q + 2], v[4 * q + 3] + bDown[piece * 16 + 4 * q + 3]);
						if(res != nullptr) {
							const float4 r = __ldg(reinterpret_cast<const float4*>(res) + q);
							o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
						}
						reinterpret_cast<float4*>(dst)[q] = o;
					}
				}
			}
		}
		// tensor memory and the chunk buffers go back to the next tile
		tc_fence_before_sync();
		__syncthreads();
		tc_fence_after_sync();
	}
	if(!ok) {
		// a wait gave up: let whatever was issued (a TMA load, MMAs) come to rest before tensor memory is freed
		const uint64_t t0 = global_timer_ns();
		while(global_timer_ns() - t0 < 1000000ull) {
		}
	}
	tc_fence_before_sync();
	__syncthreads();
	if(warp == 0) tmem_dealloc(tmemBase, 512);
}

} // namespace

// True when the block was issued as the fused kernel; false when the shape is outside what it covers (the caller then
// runs the three-launch form).  rc receives the launch status.
bool launch_mbv2_fused(void* stream, const nb200_mbv2_desc* d, const float* x, const float* wExp, const float* bExp,
	const float* wDw, const float* bDw, const float* wDown, const float* bDown, float* y, int precision, int* rc)
{
	if(d->stride != 1 || d->c_in != CIN || d->c_exp % CHUNK != 0 || d->c_exp > MAX_CEXP || d->c_exp <= 0
		|| d->c_out % 16 != 0 || d->c_out > MAX_COUT || d->c_out <= 0 || (d->residual && d->c_out != CIN)
		|| (precision != NB200_PREC_3XTF32 && precision != NB200_PREC_TF32) || !aligned16(x) || !aligned16(y)) {
		return false;
	}
	FusedParams p = {};
	p.x = x; p.y = y; p.wExp = wExp; p.bExp = bExp; p.wDw = wDw; p.bDw = bDw; p.wDown = wDown; p.bDown = bDown;
	p.batch = d->batch; p.h = d->h; p.w = d->w; p.cExp = d->c_exp; p.cOut = d->c_out;
	p.residual = d->residual;
	p.actExp = d->act_exp; p.actDw = d->act_dw; p.actExpParam = d->act_exp_param; p.actDwParam = d->act_dw_param;
	p.tilesX = (d->w + TW - 1) / TW;
	p.tilesY = (d->h + TH - 1) / TH;
	const long long tiles = static_cast<long long>(d->batch) * p.tilesX * p.tilesY;
	if(tiles > 0x7fffffffLL) return false;
	p.numTiles = static_cast<int>(tiles);
	p.status = device_status_word();
	if(p.status == nullptr) { *rc = NB200_ENODEVICE; return true; }
	CUtensorMap map;
	if(!make_image_box_map(&map, x, CIN, d->w, d->h, d->batch, CIN, HW, HH, true)) return false;
	const SmemLayout L = smem_layout(d->c_exp, d->c_out);
	const size_t smemBytes = L.total + 1024;
	if(smemBytes > 227 * 1024) return false;
	const int grid = p.numTiles < sm_count() ? p.numTiles : sm_count();
	cudaError_t e;
	if(precision == NB200_PREC_3XTF32) {
		e = cudaFuncSetAttribute(mbv2_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes));
		if(e == cudaSuccess) mbv2_fused_kernel<true><<<grid, THREADS, smemBytes, as_stream(stream)>>>(p, map);
	} else {
		e = cudaFuncSetAttribute(mbv2_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes));
		if(e == cudaSuccess) mbv2_fused_kernel<false><<<grid, THREADS, smemBytes, as_stream(stream)>>>(p, map);
	}
	count_launch(1);
	*rc = check_launch();
	return true;
}

} // namespace nb200
