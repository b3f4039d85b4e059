// MobileNetV2 inverted-residual block as ONE kernel (stride 1, 32 input channels, up to 192 expanded channels):
//   y = [x +] W_down * act2( dw3x3( act1( W_exp * x + b_exp ) ) + b_dw ) + b_down
// The expanded activations never leave the SM: algorithmic traffic is the input once (plus its halo), the output once
// and the weights.
//
// A persistent CTA (one per SM, 16 warps) walks output tiles of 4 x 16 pixels as a three-stage pipeline:
//   expand(t+2)   tensor core   [channels] x [halo pixels] = W_exp (A, resident in shared memory) x patch (B; the
//                               6 x 18 halo patch of x: TMA, 128-byte rows, zeros outside the image), 3 MMAs per
//                               product (lo*hi + hi*hi + hi*lo), into tensor memory -- TRANSPOSED, so that a lane
//                               of tensor memory is a channel and its columns are that channel's halo pixels
//   depthwise(t)  12 warps      a lane owns ONE channel: tcgen05.ld hands it 72 columns (four halo rows), bias +
//                               activation + the zero padding of the EXPANDED image are applied on the way, the nine
//                               taps are FMAs on registers; the result (bias, activation, split in hi / lo) is written
//                               as the K-major A operand of the project product.  No shared-memory round trip.
//   project(t-1)  tensor core   all channel chunks into the output tile in tensor memory; then
//   store(t-1)    4 warps       tcgen05.ld -> + bias, + residual -> global memory (128 bytes per pixel).  The same four
//                               warps first fetch the patch of tile t+2 and derive its lo part, while the others do the
//                               depthwise arithmetic.
// The expand accumulators are double-buffered in tensor memory, so there is ONE block-wide barrier per tile (the A
// operand of tile t is complete): behind it expand(t+2) and project(t) are issued.  Every wait is bounded (common.cuh)
// and the barrier carries a vote: on a time-out the kernel records it in the status word, frees its tensor memory and
// returns.
#include "contraction.cuh"

#include <cuda.h>

namespace nb200 {

namespace {

constexpr int TH = 4, TW = 16;              // output tile (64 pixels)
constexpr int HH = TH + 2, HW = TW + 2;     // halo patch
constexpr int HALO = HH * HW;               // 108 pixels
constexpr int HALO_N = 112;                 // ... as the N extent of the expand product (multiple of 16)
constexpr int CIN = 32;                     // input channels = K of the expand product = one 128-byte row
constexpr int CHUNK = 32;                   // expanded channels per lane quarter = K chunk of the project product
constexpr int THREADS = 512;
constexpr int MAX_CEXP = 192, MAX_COUT = 64;
constexpr int PATCH_BYTES = HALO * 128;     // what one TMA load delivers
constexpr int PATCH_ROOM = HALO_N * 128;    // what the expand product reads (14336, a multiple of 1024)
constexpr int A2_CHUNK_BYTES = TH * TW * 128; // 64 pixel rows of 32 channels
constexpr int TMEM_COLS = 512;
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

// ReLU (optionally with an upper threshold) and "no activation" as one clamp, HSwish apart; decided once per kernel
struct Act {
	bool hswish;
	float lo, hi;
	__device__ __forceinline__ float operator()(float v) const
	{
		return hswish ? v * fminf(fmaxf(v + 3.f, 0.f), 6.f) * (1.f / 6.f) : fminf(fmaxf(v, lo), hi);
	}
};
__device__ __forceinline__ Act make_act(int kind, float param)
{
	Act a;
	a.hswish = kind == NB200_ACT_HSWISH;
	a.lo = kind == NB200_ACT_RELU ? 0.f : -__int_as_float(0x7f800000);
	a.hi = kind == NB200_ACT_RELU && param > 0.f ? param : __int_as_float(0x7f800000);
	return a;
}

// 32 lanes x 32 bit, 8 consecutive columns, issue only (tmem_ld_wait() before the first use)
__device__ __forceinline__ void tmem_ld8_issue_local(uint32_t taddr, uint32_t* r)
{
	asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
		: "r"(taddr));
}

struct SmemLayout {
	uint32_t patchHi, patchLo, wExpHi, wExpLo, wDownHi, wDownLo, a2Hi, a2Lo, consts, bars, total;
};

__host__ __device__ inline SmemLayout smem_layout(int cExp, int cOut)
{
	const uint32_t chunks = cExp / CHUNK;
	SmemLayout l;
	uint32_t at = 0;
	l.patchHi = at; at += PATCH_ROOM;
	l.patchLo = at; at += PATCH_ROOM;
	// a 128-row MMA operand block that starts at row 128 of W_exp reads on into whatever follows (rows nobody uses)
	l.wExpHi = at; at += cExp * 128;
	l.wExpLo = at; at += cExp * 128;
	l.wDownHi = at; at += chunks * cOut * 128;
	l.wDownLo = at; at += chunks * cOut * 128;
	if(at < l.wExpLo + 2 * 128 * 128) at = l.wExpLo + 2 * 128 * 128;
	// The project product's A tiles: a chunk's 64 pixel rows are rows 64..127 of a 128-row block that begins 8 KB
	// earlier (the chunk before, or the weights in front of the first chunk): the output pixels then land in tensor
	// memory lanes 64..127, which the warps that store the tile may read.
	l.a2Hi = at; at += chunks * A2_CHUNK_BYTES;
	l.a2Lo = at; at += chunks * A2_CHUNK_BYTES;
	l.consts = at; at += cOut * 4;                 // bDown
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
	float* const bDown = reinterpret_cast<float*>(smem + L.consts);
	uint64_t* const patchBar = reinterpret_cast<uint64_t*>(smem + L.bars);
	uint64_t* const expandBar = patchBar + 1;   // two: expand(e) completes a phase of expandBar[e & 1] (a waiter is then
	                                            // never more than one phase behind, which parity waits require)
	uint64_t* const projectBar = patchBar + 3;
	uint32_t* const tmemSlot = reinterpret_cast<uint32_t*>(patchBar + 4);
	volatile int* const abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const int chunks = p.cExp / CHUNK;

	if(tid == 0) {
		mbar_init(patchBar, 1);
		mbar_init(&expandBar[0], 1);
		mbar_init(&expandBar[1], 1);
		// one commit per warp that issues project MMAs: two when tensor memory has room for a second output accumulator
		mbar_init(projectBar, (4 * HALO_N + 2 * p.cOut <= TMEM_COLS && p.cExp > CHUNK) ? 2 : 1);
		*abortFlag = 0;
		mbar_init_fence();
		tma_prefetch_descriptor(&mapX);
	}
	if(warp == 0) {
		tmem_alloc(tmemSlot, TMEM_COLS);
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
	for(int i = tid; i < p.cOut; i += THREADS) bDown[i] = p.bDown != nullptr ? __ldg(p.bDown + i) : 0.f;
	fence_proxy_async_smem();
	tc_fence_before_sync();
	__syncthreads();
	tc_fence_after_sync();
	const uint32_t tmemBase = *tmemSlot;
	// expand accumulators, two sets (tile parity) of two blocks of HALO_N columns: channels 0..127, 128..255
	const uint32_t accExpand = tmemBase;
	const uint32_t accProject = tmemBase + 4 * HALO_N;         // cOut columns; lanes 64..127 = the tile's 64 pixels
	const uint32_t idescExpand = umma_idesc_tf32(128, HALO_N);
	const uint32_t idescProject = umma_idesc_tf32(128, p.cOut);
	const Act actExp = make_act(p.actExp, p.actExpParam), actDw = make_act(p.actDw, p.actDwParam);

	// Roles.  The lane quarter a warp may read (warp % 4) holds the 32 channels of chunk `combo`; a chunk has two
	// depthwise warps, one per pair of output rows.  Quarters 2 and 3 exist only in the first 128-channel block: of
	// their other warps, 10 and 11 are the helpers -- they store the finished tile (its pixels sit in lanes 64..127,
	// their quarters) and fetch and split the next patch -- and warps 14 and 15 issue the MMAs (expand / project;
	// issuing costs 50-80 cycles per instruction, so they do nothing else and nothing waits on them but the MMAs).
	const int quad = warp & 3, slot = warp >> 2;
	const bool helper = warp == 10 || warp == 11;
	const bool issuerA = warp == 14;                       // expand, and the even chunks of project
	const bool issuerB = warp == 15;                       // the odd chunks of project, into the second accumulator
	// (the whole warp walks the issue code and one elected lane issues: instructions issued from a lone lane of a
	// diverged warp cost about twice as many cycles each)
	const bool dual = 4 * HALO_N + 2 * p.cOut <= TMEM_COLS && chunks > 1; // room (and use) for two output accumulators
	const int block = quad < 2 ? slot >> 1 : 0;             // which 128-channel block
	const int combo = block * 4 + quad;                     // chunk index = channels [32 * combo, +32)
	const int rowPair = slot & 1;                           // output rows 2 * rowPair, 2 * rowPair + 1
	const bool worker = (quad < 2 || slot < 2) && combo < chunks;
	const int helperIndex = (warp - 10) * 32 + lane;       // 0..63 among the helper threads
	const int ch = combo * CHUNK + lane;
	float k[9], biasExp = 0.f, biasDw = 0.f;
	if(worker) {
#pragma unroll
		for(int t = 0; t < 9; ++t) k[t] = __ldg(p.wDw + t * p.cExp + ch);
		biasExp = p.bExp != nullptr ? __ldg(p.bExp + ch) : 0.f;
		biasDw = p.bDw != nullptr ? __ldg(p.bDw + ch) : 0.f;
	}

	const int myTiles = static_cast<int>(blockIdx.x) < p.numTiles ? (p.numTiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
	auto tile_origin = [&](int j, int& n, int& y0, int& x0) {   // the CTA's j-th tile
		const int tile = blockIdx.x + j * gridDim.x;
		const int perImage = p.tilesX * p.tilesY;
		n = tile / perImage;
		const int r = tile - n * perImage;
		const int tyi = r / p.tilesX;
		y0 = tyi * TH;
		x0 = (r - tyi * p.tilesX) * TW;
	};
	auto load_patch = [&](int j) {
		int n, y0, x0;
		tile_origin(j, n, y0, x0);
		mbar_arrive_expect_tx(patchBar, PATCH_BYTES);
		tma_load_4d(smem_u32(smem + L.patchHi), &mapX, patchBar, 0, x0 - 1, y0 - 1, n);
	};
	// lo part (or, in plain TF32, the rounded copy) of the patch, by `count` threads of which this one is `index`
	auto split_patch = [&](int index, int count) {
		for(int i = index; i < HALO * 8; i += count) {
			float4 v = *reinterpret_cast<const float4*>(smem + L.patchHi + i * 16);
			if(THREEX) {
				v.x = lo_part(v.x); v.y = lo_part(v.y); v.z = lo_part(v.z); v.w = lo_part(v.w);
			} else {
				v.x = to_tf32(v.x); v.y = to_tf32(v.y); v.z = to_tf32(v.z); v.w = to_tf32(v.w);
			}
			*reinterpret_cast<float4*>(smem + L.patchLo + i * 16) = v;
		}
		fence_proxy_async_smem();
	};
	// Issuing an MMA costs the issuing thread 50-80 cycles whatever its size, so the work is split over two warps:
	// one issues expand and the even chunks of project, the other the odd chunks (into a second accumulator).
	auto issue_expand = [&](int e) {
		tc_fence_after_sync();
		const uint64_t bHi = umma_desc_k128(smem_u32(smem + L.patchHi));
		const uint64_t bLo = umma_desc_k128(smem_u32(smem + L.patchLo));
		const int blocks = p.cExp > 128 ? 2 : 1;
		for(int mt = 0; mt < blocks; ++mt) {
			const uint64_t aHi = umma_desc_k128(smem_u32(smem + L.wExpHi) + mt * 128 * 128);
			const uint64_t aLo = umma_desc_k128(smem_u32(smem + L.wExpLo) + mt * 128 * 128);
			const uint32_t d = accExpand + (e & 1) * 2 * HALO_N + mt * HALO_N;
			if(elect_one()) {
#pragma unroll
				for(int ks = 0; ks < CIN / 8; ++ks) {
					if(THREEX) {
						umma_tf32_ss(d, aLo + 2 * ks, bHi + 2 * ks, idescExpand, ks > 0 ? 1u : 0u);
						umma_tf32_ss(d, aHi + 2 * ks, bHi + 2 * ks, idescExpand, 1u);
						umma_tf32_ss(d, aHi + 2 * ks, bLo + 2 * ks, idescExpand, 1u);
					} else {
						umma_tf32_ss(d, aHi + 2 * ks, bLo + 2 * ks, idescExpand, ks > 0 ? 1u : 0u); // rounded weights x rounded patch
					}
				}
			}
			__syncwarp();
		}
		if(elect_one()) umma_commit(&expandBar[e & 1]);
		__syncwarp();
	};
	auto wait_expand = [&](int e) {
		return mbar_wait_bounded(&expandBar[e & 1], (e >> 1) & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_EXPAND);
	};
	// part 0: the even chunks (all chunks when there is one accumulator) into accumulator 0; part 1: the odd chunks
	// into accumulator 1; the store adds the two.  Each part ends with its own commit.
	auto issue_project = [&](int part) {
		tc_fence_after_sync();
		const uint32_t acc = accProject + part * p.cOut;
		const int step = dual ? 2 : 1;
		bool firstMma = true;
		for(int c = part; c < chunks; c += step) {
			// the chunk's pixel rows are rows 64..127 of the block that begins one chunk earlier
			const uint64_t aHi = umma_desc_k128(smem_u32(smem + L.a2Hi) + (c - 1) * A2_CHUNK_BYTES);
			const uint64_t aLo = umma_desc_k128(smem_u32(smem + L.a2Lo) + (c - 1) * A2_CHUNK_BYTES);
			const uint64_t bHi = umma_desc_k128(smem_u32(smem + L.wDownHi) + c * p.cOut * 128);
			const uint64_t bLo = umma_desc_k128(smem_u32(smem + L.wDownLo) + c * p.cOut * 128);
			if(elect_one()) {
#pragma unroll
				for(int ks = 0; ks < CHUNK / 8; ++ks) {
					const uint32_t first = (firstMma && ks == 0) ? 0u : 1u;
					if(THREEX) {
						umma_tf32_ss(acc, aLo + 2 * ks, bHi + 2 * ks, idescProject, first);
						umma_tf32_ss(acc, aHi + 2 * ks, bHi + 2 * ks, idescProject, 1u);
						umma_tf32_ss(acc, aHi + 2 * ks, bLo + 2 * ks, idescProject, 1u);
					} else {
						umma_tf32_ss(acc, aHi + 2 * ks, bHi + 2 * ks, idescProject, first);
					}
				}
			}
			firstMma = false;
			__syncwarp();
		}
		if(elect_one()) umma_commit(projectBar);
		__syncwarp();
	};
	// the finished tile j: tensor memory lanes 64..127 -> + bias, + residual -> global memory (helper warps; one
	// pixel per lane, 16 channels at a time; the residual is in flight together with the tensor-memory loads).
	// `ready` waits for project(j).
	auto store_tile = [&](int j, auto&& ready) -> bool {
		int img, y0, x0;
		tile_origin(j, img, y0, x0);
		const int px = (quad - 2) * 32 + lane;
		const int ty = px / TW, tx = px - ty * TW;
		const int gy = y0 + ty, gx = x0 + tx;
		const bool valid = gy < p.h && gx < p.w;
		const size_t pixel = (static_cast<size_t>(img) * p.h + gy) * p.w + gx;
		if(!ready()) return false;
		tc_fence_after_sync();
		const uint32_t src = accProject + (static_cast<uint32_t>(quad * 32) << 16);
		float* dst = p.y + pixel * p.cOut;
		for(int piece = 0; piece * 16 < p.cOut; ++piece) {
			uint32_t v[16], u[16];
			tmem_ld16_issue(src + piece * 16, v);
			if(dual) tmem_ld16_issue(src + p.cOut + piece * 16, u);
			float4 res[4];
			if(p.residual && valid) { // c_out == 32 = CIN here; in flight together with the tensor-memory loads
#pragma unroll
				for(int q = 0; q < 4; ++q) res[q] = __ldg(reinterpret_cast<const float4*>(p.x + pixel * CIN + piece * 16) + q);
			}
			tmem_ld_wait();
			if(valid) {
#pragma unroll
				for(int q = 0; q < 4; ++q) {
					float o[4];
#pragma unroll
					for(int i = 0; i < 4; ++i) {
						o[i] = __uint_as_float(v[4 * q + i]);
						if(dual) o[i] += __uint_as_float(u[4 * q + i]);
						o[i] += bDown[piece * 16 + 4 * q + i];
					}
					if(p.residual) { o[0] += res[q].x; o[1] += res[q].y; o[2] += res[q].z; o[3] += res[q].w; }
					reinterpret_cast<float4*>(dst + piece * 16)[q] = make_float4(o[0], o[1], o[2], o[3]);
				}
			}
		}
		return true;
	};
	auto project_done = [&](int j) {
		bool done = mbar_wait_bounded(projectBar, j & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PROJECT);
		return static_cast<bool>(__all_sync(0xffffffffu, done));
	};

	// ---- prologue: patch 0 -> expand 0, patch 1 -> expand 1 (every thread helps to split; later the helpers do)
	bool ok = true;
	for(int e = 0; e < 2 && e < myTiles && ok; ++e) {
		if(e > 0) {
			ok = wait_expand(e - 1); // the patch buffers are free
			ok = __syncthreads_and(ok) != 0;
			if(!ok) break;
		}
		if(tid == 0) load_patch(e);
		ok = mbar_wait_bounded(patchBar, e & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PATCH);
		ok = __syncthreads_and(ok) != 0;
		if(!ok) break;
		split_patch(tid, THREADS);
		tc_fence_before_sync();
		__syncthreads();
		if(issuerA) issue_expand(e);
	}
	for(int j = 0; j < myTiles && ok; ++j) {
		int img, y0, x0;
		tile_origin(j, img, y0, x0);
		if(worker) {
			// ---- depthwise(j): expand(j) is in tensor memory (set j & 1)
			ok = wait_expand(j);
			ok = __all_sync(0xffffffffu, ok);
			float out[2][TW];
			if(ok) {
				tc_fence_after_sync();
				const uint32_t src = accExpand + (static_cast<uint32_t>(quad * 32) << 16) + (j & 1) * 2 * HALO_N + block * HALO_N
					+ rowPair * 2 * HW;
				uint32_t raw[56], last[24];
				tmem_ld32_issue(src, raw);
				tmem_ld16_issue(src + 32, raw + 32);
				tmem_ld8_issue_local(src + 48, raw + 48);      // halo rows 0..2 are columns 0..53
				tmem_ld16_issue(src + 54, last);                // halo row 3: columns 54..69 ...
				tmem_ld8_issue_local(src + 64, last + 16);      // ... and 70, 71 (elements 6, 7 of this piece)
				// which halo pixels lie inside the image: bit hx of rowBits[hy] (the same for every lane)
				uint32_t colBits = 0;
#pragma unroll
				for(int hx = 0; hx < HW; ++hx) {
					const int gx = x0 - 1 + hx;
					colBits |= (gx >= 0 && gx < p.w) ? (1u << hx) : 0u;
				}
				uint32_t rowBits[4];
#pragma unroll
				for(int r = 0; r < 4; ++r) {
					const int gy = y0 - 1 + rowPair * 2 + r;
					rowBits[r] = (gy >= 0 && gy < p.h) ? colBits : 0u;
				}
				tmem_ld_wait();
				float win[3][HW];
#pragma unroll
				for(int r = 0; r < 3; ++r) {
#pragma unroll
					for(int hx = 0; hx < HW; ++hx) {
						const float v = actExp(__uint_as_float(raw[r * HW + hx]) + biasExp);
						win[r][hx] = ((rowBits[r] >> hx) & 1u) ? v : 0.f;
					}
				}
#pragma unroll
				for(int t = 0; t < 2; ++t) {
					if(t == 1) {
						// slide down: halo row 3 takes the place of halo row 0 (row index (t + dy) % 3 below)
#pragma unroll
						for(int hx = 0; hx < HW; ++hx) {
							const uint32_t bits = hx < 16 ? last[hx] : last[16 + 6 + (hx - 16)];
							const float v = actExp(__uint_as_float(bits) + biasExp);
							win[0][hx] = ((rowBits[3] >> hx) & 1u) ? v : 0.f;
						}
					}
#pragma unroll
					for(int tx = 0; tx < TW; ++tx) {
						float acc = biasDw;
#pragma unroll
						for(int dy = 0; dy < 3; ++dy) {
#pragma unroll
							for(int dx = 0; dx < 3; ++dx) acc = fmaf(win[(t + dy) % 3][tx + dx], k[dy * 3 + dx], acc);
						}
						out[t][tx] = actDw(acc);
					}
				}
				// project(j-1) still reads the A tiles when this tile's arithmetic is done early: wait, then write
				if(j > 0) {
					ok = mbar_wait_bounded(projectBar, (j - 1) & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PROJECT);
					ok = __all_sync(0xffffffffu, ok);
				}
				if(ok) {
					// pixel ty * 16 + tx of this chunk's A tile; the swizzle phase of its row is (tx & 7)
					uint8_t* const aHi = smem + L.a2Hi + combo * A2_CHUNK_BYTES + ((lane & 3u) << 2);
					uint8_t* const aLo = smem + L.a2Lo + combo * A2_CHUNK_BYTES + ((lane & 3u) << 2);
					const uint32_t kChunk = static_cast<uint32_t>(lane) >> 2;
#pragma unroll
					for(int t = 0; t < 2; ++t) {
#pragma unroll
						for(int tx = 0; tx < TW; ++tx) {
							const float v = out[t][tx];
							const uint32_t off = ((rowPair * 2 + t) * TW + tx) * 128u + ((kChunk ^ (tx & 7u)) << 4);
							if(THREEX) {
								*reinterpret_cast<float*>(aHi + off) = v;
								*reinterpret_cast<float*>(aLo + off) = lo_part(v);
							} else {
								*reinterpret_cast<float*>(aHi + off) = to_tf32(v);
							}
						}
					}
					fence_proxy_async_smem();
				}
			}
		} else if(helper) {
			// ---- patch j+2: its buffers are free once expand(j+1) has completed
			if(j + 2 < myTiles) {
				ok = wait_expand(j + 1);
				ok = __all_sync(0xffffffffu, ok);
				if(ok) {
					if(helperIndex == 0) load_patch(j + 2);
					ok = mbar_wait_bounded(patchBar, (j + 2) & 1, abortFlag, p.status, (KERNEL_ID << 8) | SITE_PATCH);
					ok = __all_sync(0xffffffffu, ok);
					if(ok) split_patch(helperIndex, 64);
				}
			}
			// ---- store(j-1): its project MMAs were issued behind the last barrier
			if(ok && j > 0) {
				ok = store_tile(j - 1, [&] { return project_done(j - 1); });
			}
		}
		// ---- the barrier: tile j's A tiles are written, its expand accumulators read, the output tile of j-1 stored,
		// patch j+2 split
		tc_fence_before_sync();
		if(!__syncthreads_and(ok)) { ok = false; break; }
		if(issuerA) {
			if(j + 2 < myTiles) issue_expand(j + 2);
			issue_project(0);
		} else if(issuerB && dual) {
			issue_project(1);
		}
	}
	if(ok && myTiles > 0 && helper) ok = store_tile(myTiles - 1, [&] { return project_done(myTiles - 1); });
	if(!ok) {
		// a wait gave up: let whatever was issued (a TMA load, MMAs) come to rest before tensor memory is freed
		const uint64_t t0 = global_timer_ns();
		while(global_timer_ns() - t0 < 1000000ull) {
		}
	}
	tc_fence_before_sync();
	__syncthreads();
	if(warp == 0) tmem_dealloc(tmemBase, TMEM_COLS);
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
	const SmemLayout L = smem_layout(d->c_exp, d->c_out);
	const size_t smemBytes = L.total + 1024;
	if(smemBytes > 227 * 1024) return false;
	p.status = device_status_word();
	if(p.status == nullptr) { *rc = NB200_ENODEVICE; return true; }
	CUtensorMap map;
	if(!make_image_box_map(&map, x, CIN, d->w, d->h, d->batch, CIN, HW, HH, 1)) return false;
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
