// The score chain of multi-head attention as ONE kernel:
//   O[b] = softmax_rows( scale * Q[b] * Kt[b] + mask ) * V[b]          b < batch (= sequences x heads)
// with Q [seqQ x 64], Kt [64 x seqTo] (the keys already transposed, as CMultiheadAttentionLayer prepares them,
// NeoML/src/Dnn/Layers/MultiheadAttentionLayer.cpp:145-223), V [seqTo x 64], mask [seqQ x seqTo] shared by every b.
// The scores never reach memory: algorithmic traffic is Q, Kt, V once per 128-row tile of Q and O once.
//
// A persistent CTA (one per SM, 12 warps) walks (b, 128 query rows) items; inside an item the keys come in blocks of 128:
//   QK(g)       tensor core   S = Q * Kt block, 3 MMAs per product (lo*hi + hi*lo + hi*hi, "3xTF32"), 128 x 128 into
//                             tensor memory (two S buffers).  Q: K-major 128-byte rows.  Kt block: rows of 32 keys per
//                             depth index, i.e. an MN-major operand, used as TMA delivers it (32-byte swizzle atoms).
//   softmax(g)  warps 0-3     a thread owns one query row (its lane of tensor memory): block maximum, then
//                             p = exp2( x - m ) with a running reference m that is raised (and O rescaled) only when
//                             the block maximum exceeds it by more than 2^16 -- rare after the first block; p replaces
//                             S in place (the MMA reads the upper 19 bits: that is the hi part), its lo part goes to a
//                             third 128-column region; the row sum is kept in a register.
//   PV(g)       tensor core   O += P * V block, A operand straight from tensor memory (TS form), V block as TMA
//                             delivers it (rows of 32 depth values per key: MN-major), 3 MMAs per product.
//   epilogue    warps 4-7     O * (1 / row sum) -> global memory; the same warps derive the lo parts of Q, Kt, V blocks
//                             in shared memory as the loads land.
// QK(g+1) is issued before PV(g), so the tensor core works on the next block's scores while the softmax of this one
// runs; Kt and V are single-buffered, each being reloaded while the other product runs.  Loads: warp 8 (Q, Kt) and
// warp 9 (V); MMA issue: warp 10 (QK) and warp 11 (PV).  Every wait is bounded (common.cuh): on a time-out the kernel
// records it in the status word, lets its loads land, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>
#include <math.h>

namespace nb200 {

namespace {

constexpr int D = 64;                 // depth of a head
constexpr int BQ = 128, BK = 128;     // query rows per item, keys per block
constexpr int THREADS = 384;
constexpr int TILE_BYTES = 32768;     // every operand buffer: 128 x 64 floats
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_PLO = 256, COL_O = 384;   // S: 2 x 128, P lo: 128, O: 2 x 64
constexpr int KERNEL_ID = 0x6e;       // in the status word: (KERNEL_ID << 8) | site
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RAISE = 16.f;         // log2 of how far a value may exceed the reference before the reference moves
enum { SITE_LOAD = 1, SITE_SPLIT = 2, SITE_QK = 3, SITE_SOFTMAX = 4, SITE_PV = 5, SITE_OUT = 6 };

struct AttnParams {
	float* out;
	const float* scale;   // one float in device memory, or null (1)
	const float* mask;    // seqQ x seqTo, or null
	int seqQ, seqTo, batch;
	int qTiles, numItems, blocks;
	int* status;
};

struct Smem {
	static constexpr uint32_t qHi = 0, qLo = TILE_BYTES, kHi = 2 * TILE_BYTES, kLo = 3 * TILE_BYTES, vHi = 4 * TILE_BYTES,
		vLo = 5 * TILE_BYTES, rowScale = 6 * TILE_BYTES, maskStage = rowScale + 2 * BQ * 4, bars = maskStage + 4 * 32 * 33 * 4,
		total = bars + 256;
};

// barrier indices
enum { B_QFULL, B_QREADY, B_QFREE, B_KFULL, B_KREADY, B_KFREE, B_VFULL, B_VREADY, B_VFREE,
	B_SFULL, B_PREADY = B_SFULL + 2, B_PVDONE = B_PREADY + 2, B_OFULL = B_PVDONE + 2, B_OFREE = B_OFULL + 2,
	B_STATS = B_OFREE + 2, B_COUNT = B_STATS + 2 };

__device__ __forceinline__ float lo_part(float v)
{
	return v - __uint_as_float(__float_as_uint(v) & 0xffffe000u);
}

__device__ __forceinline__ float exp2_fast(float x)
{
	float y;
	asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
	return y;
}

// Shared-memory descriptor of an MN-major tf32 operand tile.  For 32-bit elements the tensor core reads an MN-major
// operand only in the "128-byte swizzle with 32-byte atoms" layout (layout type 1; with the plain 128-byte swizzle the
// product comes out as zeros): a row of 128 bytes holds 32 consecutive M (or N) indices of one K index, its four
// 32-byte units permuted by unit ^= (row & 3) -- what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B; four such
// rows make an atom of 512 bytes, the eight K indices of one MMA are two atoms `stride byte offset` = 512 bytes apart,
// and the next 32 M/N indices lie `groupBytes` further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t groupBytes)
{
	uint64_t d = 0;
	d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
	d |= static_cast<uint64_t>((groupBytes >> 4) & 0x3FFFu) << 16;
	d |= static_cast<uint64_t>(512 >> 4) << 32;
	d |= static_cast<uint64_t>(1) << 46;
	d |= static_cast<uint64_t>(1) << 61;
	return d;
}

constexpr uint32_t B_MN_MAJOR = 1u << 16; // instruction descriptor: B operand is MN-major

__global__ void __launch_bounds__(THREADS, 1) attention_fused_kernel(const AttnParams p, const __grid_constant__ CUtensorMap mapQ,
	const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV)
{
	extern __shared__ uint8_t smemRaw[];
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
	uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + Smem::bars);
	uint32_t* const tmemSlot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
	volatile int* const abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);
	float* const rowScale = reinterpret_cast<float*>(smem + Smem::rowScale);
	const uint32_t smemBase = smem_u32(smem);

	const int tid = threadIdx.x;
	const int warp = tid >> 5, lane = tid & 31;

	if(tid == 0) {
		const uint32_t counts[B_COUNT] = { 1, 128, 1, 1, 128, 1, 1, 128, 1, /*sFull*/ 1, 1, /*pReady*/ 128, 128, /*pvDone*/ 1, 1,
			/*oFull*/ 1, 1, /*oFree*/ 128, 128, /*stats*/ 128, 128 };
		for(int i = 0; i < B_COUNT; ++i) mbar_init(bars + i, counts[i]);
		*abortFlag = 0;
		mbar_init_fence();
	}
	if(warp == 0) {
		tmem_alloc(tmemSlot, TMEM_COLS);
		tmem_relinquish();
	}
	if(warp == 8 && lane == 0) {
		tma_prefetch_descriptor(&mapQ);
		tma_prefetch_descriptor(&mapK);
	}
	if(warp == 9 && lane == 0) tma_prefetch_descriptor(&mapV);
	tc_fence_before_sync();
	__syncthreads();
	tc_fence_after_sync();
	const uint32_t tmemBase = *tmemSlot;

	const int nB = p.blocks;
	int myItems = 0;
	if(static_cast<int>(blockIdx.x) < p.numItems) myItems = (p.numItems - 1 - blockIdx.x) / gridDim.x + 1;
	auto item_of = [&](int it, int& b, int& q0) {
		const int item = blockIdx.x + it * gridDim.x;
		b = item / p.qTiles;
		q0 = (item - b * p.qTiles) * BQ;
	};
	auto wait = [&](int bar, uint32_t parity, int site) {
		return mbar_wait_bounded(bars + bar, parity & 1u, abortFlag, p.status, (KERNEL_ID << 8) | site);
	};
	bool ok = true;

	if(warp < 4) {
		// ================================================= softmax: one query row per thread
		const uint32_t laneBase = tmemBase + (static_cast<uint32_t>(32 * warp) << 16);
		const int row = 32 * warp + lane;
		const float scale2 = (p.scale != nullptr ? __ldg(p.scale) : 1.f) * LOG2E;
		const bool masked = p.mask != nullptr;
		// The mask reaches a thread's row through a per-warp staging square: lane l fetches column l of 32 rows (one
		// 128-byte row segment per instruction), the square is read back row per lane.
		float* const stage = reinterpret_cast<float*>(smem + Smem::maskStage) + warp * (32 * 33);
		int g = 0;
		for(int it = 0; it < myItems && ok; ++it) {
			int b, q0;
			item_of(it, b, q0);
			float m2 = 0.f, sum = 0.f;
			float mk[32];
			auto fetch_mask = [&](int col0) { // rows of this warp x columns col0 .. col0 + 31, as they lie in memory
				const int col = min(col0 + lane, p.seqTo - 1);
#pragma unroll
				for(int i = 0; i < 32; ++i) {
					mk[i] = __ldg(p.mask + static_cast<size_t>(min(q0 + 32 * warp + i, p.seqQ - 1)) * p.seqTo + col);
				}
			};
			for(int j = 0; j < nB && ok; ++j, ++g) {
				const int k0 = j * BK;
				const bool tail = k0 + BK > p.seqTo;
				const uint32_t sAddr = laneBase + COL_S + (g & 1) * BK;
				if(masked) fetch_mask(k0); // in flight while the scores are being computed
				if(!wait(B_SFULL + (g & 1), g >> 1, SITE_SOFTMAX)) { ok = false; break; }
				tc_fence_after_sync();
				// x2 = (scale * s + mask) * log2(e) and the block maximum; with a mask, x2 replaces s in tensor memory
				float bmax = -INFINITY;
#pragma unroll 1
				for(int c = 0; c < BK; c += 32) {
					uint32_t r[32];
					tmem_ld32_issue(sAddr + c, r);
					if(masked) {
#pragma unroll
						for(int i = 0; i < 32; ++i) stage[i * 33 + lane] = mk[i];
						__syncwarp();
					}
					tmem_ld_wait();
#pragma unroll
					for(int i = 0; i < 32; ++i) {
						float x = __uint_as_float(r[i]) * scale2;
						if(masked) x = fmaf(stage[lane * 33 + i], LOG2E, x);
						if(tail && k0 + c + i >= p.seqTo) x = -INFINITY;
						bmax = fmaxf(bmax, x);
						r[i] = __float_as_uint(x);
					}
					if(masked) {
						__syncwarp(); // the square has been read
						if(c + 32 < BK) fetch_mask(k0 + c + 32);
						tmem_st32(sAddr + c, r);
					}
				}
				if(masked) tmem_st_wait();
				if(j == 0) {
					m2 = bmax;
					sum = 0.f;
				}
				const bool raise = j > 0 && bmax > m2 + RAISE;
				if(g > 0) {
					// P lo of the block before (of this item or of the item before) is being read until its P * V has
					// completed; so is O
					if(!wait(B_PVDONE + ((g - 1) & 1), (g - 1) >> 1, SITE_SOFTMAX)) { ok = false; break; }
					tc_fence_after_sync();
					if(__any_sync(0xffffffffu, raise)) {
						const float factor = raise ? exp2_fast(m2 - bmax) : 1.f;
						if(raise) m2 = bmax;
						sum *= factor;
						const uint32_t oAddr = laneBase + COL_O + (it & 1) * D;
#pragma unroll 1
						for(int c = 0; c < D; c += 32) {
							uint32_t r[32];
							tmem_ld32_issue(oAddr + c, r);
							tmem_ld_wait();
#pragma unroll
							for(int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
							tmem_st32(oAddr + c, r);
						}
					}
				}
				// p = 2^(x2 - m2): hi part in place of the scores, lo part beside it
#pragma unroll 1
				for(int c = 0; c < BK; c += 32) {
					uint32_t r[32], lo[32];
					tmem_ld32_issue(sAddr + c, r);
					tmem_ld_wait();
#pragma unroll
					for(int i = 0; i < 32; ++i) {
						float x = __uint_as_float(r[i]);
						if(!masked) {
							x *= scale2;
							if(tail && k0 + c + i >= p.seqTo) x = -INFINITY;
						}
						const float pv = exp2_fast(x - m2);
						sum += pv;
						r[i] = __float_as_uint(pv);
						lo[i] = __float_as_uint(lo_part(pv));
					}
					tmem_st32(sAddr + c, r);
					tmem_st32(laneBase + COL_PLO + c, lo);
				}
				tmem_st_wait();
				if(j == nB - 1) {
					// the row's normaliser for the epilogue warps; the slot is free once the item two back has been stored
					if(it >= 2 && !wait(B_OFREE + (it & 1), (it >> 1) - 1, SITE_SOFTMAX)) { ok = false; break; }
					rowScale[(it & 1) * BQ + row] = 1.f / sum;
					mbar_arrive(bars + B_STATS + (it & 1));
				}
				tc_fence_before_sync();
				mbar_arrive(bars + B_PREADY + (g & 1));
			}
		}
	} else if(warp < 8) {
		// ================================================= lo parts of the operands, and the epilogue
		const int ht = tid - 128;
		auto split = [&](uint32_t hiOff, uint32_t loOff) {
			const float4* hi = reinterpret_cast<const float4*>(smem + hiOff);
			float4* lo = reinterpret_cast<float4*>(smem + loOff);
#pragma unroll 4
			for(int i = ht; i < TILE_BYTES / 16; i += 128) {
				const float4 v = hi[i];
				lo[i] = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
			}
			fence_proxy_async_smem();
		};
		auto split_q = [&](int it) {
			if(!wait(B_QFULL, it, SITE_SPLIT)) return false;
			split(Smem::qHi, Smem::qLo);
			mbar_arrive(bars + B_QREADY);
			return true;
		};
		auto split_k = [&](int g) {
			if(!wait(B_KFULL, g, SITE_SPLIT)) return false;
			split(Smem::kHi, Smem::kLo);
			mbar_arrive(bars + B_KREADY);
			return true;
		};
		auto split_v = [&](int g) {
			if(!wait(B_VFULL, g, SITE_SPLIT)) return false;
			split(Smem::vHi, Smem::vLo);
			mbar_arrive(bars + B_VREADY);
			return true;
		};
		const uint32_t laneBase = tmemBase + (static_cast<uint32_t>(32 * (warp - 4)) << 16);
		const int row = 32 * (warp - 4) + lane;
		if(myItems > 0) ok = split_q(0) && split_k(0);
		int g = 0;
		for(int it = 0; it < myItems && ok; ++it) {
			int b, q0;
			item_of(it, b, q0);
			for(int j = 0; j < nB && ok; ++j, ++g) {
				// what the tensor core needs next comes first: the keys of the next block (and the next item's queries)
				if(j + 1 < nB) {
					ok = split_k(g + 1);
				} else if(it + 1 < myItems) {
					ok = split_q(it + 1) && split_k(g + 1);
				}
				if(ok) ok = split_v(g);
			}
			if(!ok) break;
			// epilogue of this item
			if(!wait(B_OFULL + (it & 1), it >> 1, SITE_OUT) || !wait(B_STATS + (it & 1), it >> 1, SITE_OUT)) { ok = false; break; }
			tc_fence_after_sync();
			const float inv = rowScale[(it & 1) * BQ + row];
			const bool live = q0 + row < p.seqQ;
			float* dst = p.out + (static_cast<size_t>(b) * p.seqQ + q0 + row) * D;
#pragma unroll 1
			for(int c = 0; c < D; c += 32) {
				uint32_t r[32];
				tmem_ld32_issue(laneBase + COL_O + (it & 1) * D + c, r);
				tmem_ld_wait();
				if(live) {
#pragma unroll
					for(int i = 0; i < 32; i += 4) {
						*reinterpret_cast<float4*>(dst + c + i) = make_float4(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
							__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
					}
				}
			}
			tc_fence_before_sync();
			mbar_arrive(bars + B_OFREE + (it & 1));
		}
	} else if(warp == 8) {
		// ================================================= loads: queries and keys
		if(lane == 0) {
			int g = 0, armedQ = -1, armedK = -1;
			for(int it = 0; it < myItems && ok; ++it) {
				int b, q0;
				item_of(it, b, q0);
				if(it > 0 && !wait(B_QFREE, it - 1, SITE_LOAD)) { ok = false; break; }
				mbar_arrive_expect_tx(bars + B_QFULL, TILE_BYTES);
				armedQ = it;
				tma_load_4d(smemBase + Smem::qHi, &mapQ, bars + B_QFULL, 0, q0, b, 0);
				tma_load_4d(smemBase + Smem::qHi + TILE_BYTES / 2, &mapQ, bars + B_QFULL, 32, q0, b, 0);
				for(int j = 0; j < nB; ++j, ++g) {
					if(g > 0 && !wait(B_KFREE, g - 1, SITE_LOAD)) { ok = false; break; }
					mbar_arrive_expect_tx(bars + B_KFULL, TILE_BYTES);
					armedK = g;
#pragma unroll
					for(int i = 0; i < BK / 32; ++i) {
						tma_load_4d(smemBase + Smem::kHi + i * (D * 128), &mapK, bars + B_KFULL, j * BK + 32 * i, 0, b, 0);
					}
				}
			}
			if(!ok) {
				// let what was asked for land before the CTA gives up its shared memory
				volatile int never = 0;
				if(armedQ >= 0) mbar_wait_bounded(bars + B_QFULL, armedQ & 1, &never, nullptr, 0);
				if(armedK >= 0) mbar_wait_bounded(bars + B_KFULL, armedK & 1, &never, nullptr, 0);
			}
		}
	} else if(warp == 9) {
		// ================================================= loads: values
		if(lane == 0) {
			int g = 0, armedV = -1;
			for(int it = 0; it < myItems && ok; ++it) {
				int b, q0;
				item_of(it, b, q0);
				for(int j = 0; j < nB; ++j, ++g) {
					if(g > 0 && !wait(B_VFREE, g - 1, SITE_LOAD)) { ok = false; break; }
					mbar_arrive_expect_tx(bars + B_VFULL, TILE_BYTES);
					armedV = g;
					tma_load_4d(smemBase + Smem::vHi, &mapV, bars + B_VFULL, 0, j * BK, b, 0);
					tma_load_4d(smemBase + Smem::vHi + TILE_BYTES / 2, &mapV, bars + B_VFULL, 32, j * BK, b, 0);
				}
			}
			if(!ok && armedV >= 0) {
				volatile int never = 0;
				mbar_wait_bounded(bars + B_VFULL, armedV & 1, &never, nullptr, 0);
			}
		}
	} else if(warp == 10) {
		// ================================================= MMA issue: S = Q * Kt block
		if(lane == 0) {
			constexpr uint32_t idesc = umma_idesc_tf32(BQ, BK) | B_MN_MAJOR;
			int g = 0;
			for(int it = 0; it < myItems && ok; ++it) {
				for(int j = 0; j < nB; ++j, ++g) {
					if(j == 0 && !wait(B_QREADY, it, SITE_QK)) { ok = false; break; }
					if(!wait(B_KREADY, g, SITE_QK)) { ok = false; break; }
					if(g >= 2 && !wait(B_PVDONE + (g & 1), (g >> 1) - 1, SITE_QK)) { ok = false; break; }
					tc_fence_after_sync();
					const uint32_t acc = tmemBase + COL_S + (g & 1) * BK;
#pragma unroll
					for(int s = 0; s < D / 8; ++s) {
						const uint32_t aOff = (s >> 2) * (TILE_BYTES / 2) + (s & 3) * 32;
						const uint64_t aHi = umma_desc_k128(smemBase + Smem::qHi + aOff);
						const uint64_t aLo = umma_desc_k128(smemBase + Smem::qLo + aOff);
						const uint64_t bHi = umma_desc_mn128(smemBase + Smem::kHi + s * 1024, D * 128);
						const uint64_t bLo = umma_desc_mn128(smemBase + Smem::kLo + s * 1024, D * 128);
						umma_tf32_ss(acc, aLo, bHi, idesc, s > 0 ? 1u : 0u);
						umma_tf32_ss(acc, aHi, bLo, idesc, 1u);
						umma_tf32_ss(acc, aHi, bHi, idesc, 1u);
					}
					umma_commit(bars + B_SFULL + (g & 1));
					umma_commit(bars + B_KFREE);
					if(j == nB - 1) umma_commit(bars + B_QFREE);
				}
			}
		}
	} else if(warp == 11) {
		// ================================================= MMA issue: O += P * V block
		if(lane == 0) {
			constexpr uint32_t idesc = umma_idesc_tf32(BQ, D) | B_MN_MAJOR;
			int g = 0;
			for(int it = 0; it < myItems && ok; ++it) {
				for(int j = 0; j < nB; ++j, ++g) {
					if(!wait(B_VREADY, g, SITE_PV)) { ok = false; break; }
					if(!wait(B_PREADY + (g & 1), g >> 1, SITE_PV)) { ok = false; break; }
					if(j == 0 && it >= 2 && !wait(B_OFREE + (it & 1), (it >> 1) - 1, SITE_PV)) { ok = false; break; }
					tc_fence_after_sync();
					const uint32_t acc = tmemBase + COL_O + (it & 1) * D;
					const uint32_t pHi = tmemBase + COL_S + (g & 1) * BK, pLo = tmemBase + COL_PLO;
#pragma unroll 4
					for(int s = 0; s < BK / 8; ++s) {
						const uint64_t bHi = umma_desc_mn128(smemBase + Smem::vHi + s * 1024, BK * 128);
						const uint64_t bLo = umma_desc_mn128(smemBase + Smem::vLo + s * 1024, BK * 128);
						umma_tf32_ts(acc, pLo + 8 * s, bHi, idesc, (j > 0 || s > 0) ? 1u : 0u);
						umma_tf32_ts(acc, pHi + 8 * s, bLo, idesc, 1u);
						umma_tf32_ts(acc, pHi + 8 * s, bHi, idesc, 1u);
					}
					umma_commit(bars + B_PVDONE + (g & 1));
					umma_commit(bars + B_VFREE);
					if(j == nB - 1) umma_commit(bars + B_OFULL + (it & 1));
				}
			}
		}
	}

	if(!ok || *abortFlag != 0) {
		// a wait gave up: let whatever was issued (MMAs, loads) come to rest before tensor memory is freed
		const uint64_t t0 = global_timer_ns();
		while(global_timer_ns() - t0 < 1000000ull) {
		}
	}
	tc_fence_before_sync();
	__syncthreads();
	if(warp == 0) tmem_dealloc(tmemBase, TMEM_COLS);
}

} // namespace

} // namespace nb200

using namespace nb200;

extern "C" int nb200_attention_scores_values(void* stream, int batch, const float* q, const float* kt, const float* v, int seq_q,
	int depth, int seq_to, const float* scale, const float* mask, float* out, int precision)
{
	if(batch < 0 || seq_q <= 0 || seq_to <= 0 || depth <= 0) return NB200_EINVAL;
	// the one form that exists: heads of depth 64, at least one full tile each way, 3xTF32
	if(depth != D || seq_q < BQ || seq_to < BK || seq_to % 4 != 0 || precision != NB200_PREC_3XTF32) return NB200_EINVAL;
	if(batch == 0) return NB200_OK;
	if(q == nullptr || kt == nullptr || v == nullptr || out == nullptr) return NB200_EINVAL;
	if(!aligned16(q) || !aligned16(kt) || !aligned16(v) || !aligned16(out)) return NB200_EINVAL;
	AttnParams p = {};
	p.out = out; p.scale = scale; p.mask = mask;
	p.seqQ = seq_q; p.seqTo = seq_to; p.batch = batch;
	p.qTiles = (seq_q + BQ - 1) / BQ;
	p.blocks = (seq_to + BK - 1) / BK;
	const long long items = static_cast<long long>(batch) * p.qTiles;
	if(items > 0x7fffffffLL) return NB200_EINVAL;
	p.numItems = static_cast<int>(items);
	p.status = device_status_word();
	if(p.status == nullptr) return NB200_ENODEVICE;
	CUtensorMap mapQ, mapK, mapV;
	if(!make_image_box_map(&mapQ, q, D, seq_q, batch, 1, 32, BQ, 1, 1)
		|| !make_image_box_map(&mapK, kt, seq_to, D, batch, 1, 32, D, 1, 2)
		|| !make_image_box_map(&mapV, v, D, seq_to, batch, 1, 32, BK, 1, 2)) {
		return NB200_EINVAL;
	}
	const size_t smemBytes = Smem::total + 1024;
	const int grid = p.numItems < sm_count() ? p.numItems : sm_count();
	cudaError_t e = cudaFuncSetAttribute(attention_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
		static_cast<int>(smemBytes));
	if(e == cudaSuccess) attention_fused_kernel<<<grid, THREADS, smemBytes, as_stream(stream)>>>(p, mapQ, mapK, mapV);
	count_launch(1);
	return check_launch();
}
