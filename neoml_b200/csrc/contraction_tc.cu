// Implicit-GEMM contraction on the 5th-generation tensor cores (tcgen05.mma kind::tf32, accumulators in TMEM).
//
// Persistent kernel: one CTA per SM walks the 128 x BN output tiles (tile = blockIdx.x + i * gridDim.x, the N tile
// index fastest so that CTAs running together share the same rows of A in L2).  Sixteen warps (four per SM
// sub-partition, so every thread may hold 128 registers), four roles:
//   warp 0      copy (TMA).  Each 32-wide K block of A (128 rows) and B (BN rows) arrives in a ring of "raw"
//               shared-memory slots in the 128-byte-swizzled K-major layout: plain matrices as tiled boxes, a
//               channels-last image with C % 32 == 0 as im2col boxes (no im2col matrix exists anywhere), a padded
//               few-channel image as row windows.  The warp walks its loop as a whole; an elected lane announces the
//               bytes on the slot's barrier and issues the copies.
//   warps 0-1   copy (gather; only in the GATHER instantiation).  Everything TMA cannot describe (4-byte-aligned
//               handles, column-major B, odd channel counts) is gathered by cp.async with zero fill; a slot's
//               completion is signalled by cp.async.mbarrier.arrive.
//   warps 4-7   convert.  Thread = tile row: it reads the row's 32 floats from the raw slot and stores the A operand
//               of the tensor core into one of two stages in tensor memory (tcgen05.st): for 3xTF32 hi = x with the
//               low 13 mantissa bits cleared and lo = x - hi (exact in fp32), for plain TF32 x rounded to nearest.
//               B needs no work when the caller prepared it (lo(B) / rounded B in global memory, fetched by TMA);
//               otherwise these warps also write lo(B) into a 2-slot shared-memory ring (or round B in place).
//   warp 2      allocates TMEM and issues the MMAs (TS form: A from tensor memory, B from shared memory) through an
//               elected lane: per 8-wide K step lo*hi and hi*lo into a "cross" accumulator and hi*hi into the main
//               accumulator for 3xTF32, hi*hi only for plain TF32.  The tensor core truncates on every accumulate,
//               so the small cross terms are kept apart from the large sum; lo*lo is below fp32 resolution.
//   warps 8-15  epilogue: each warp owns 32 rows x BN/2 columns.  It prefetches its residual block into L2 before it
//               waits for the accumulators, then per 16 columns: tcgen05.ld -> shared-memory transpose -> bias /
//               residual (loaded one chunk ahead) / clamp -> coalesced 16-byte stores, free of branches.  Two main
//               accumulators let the epilogue of tile i overlap the MMAs of tile i + 1; where only one cross
//               accumulator fits (BN = 128) the epilogue first folds it into the main one in place.
// Hand-over is by mbarriers: rawFull[r] (TMA bytes [+ 64 cp.async arrivals]), cvtFull[l] (one arrival per converter
// warp after tcgen05.wait::st and the proxy fence), rawEmpty[r] / loEmpty[l] / accFull[b] (tcgen05.commit),
// accEmpty[b] / crossEmpty (one arrival per epilogue warp).  Waits poll with all lanes of a warp and agree by vote:
// divergent single-lane polling and issue cost several hundred cycles per step.  Every wait is bounded; on timeout the
// CTA raises an abort flag, records the site in the device status word and every role falls through to the common
// teardown that frees TMEM.
#include "contraction.cuh"
#include <cuda.h>
#include <string.h>
#include <atomic>
#include <mutex>
#include <utility>
#include <vector>

namespace nb200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 32;                 // floats per K block = one 128-byte swizzle row
constexpr int COPY_WARPS = 2;
constexpr int COPY_THREADS = COPY_WARPS * 32;
constexpr int MMA_WARP = 2;            // warp 3 is a spare that goes straight to the final barrier
constexpr int CVT_WARP0 = 4;
constexpr int WORK_WARPS = 12;         // warps 4..15 are split between converting and the epilogue: 4 + 8 or 8 + 4
constexpr int MAX_EPI_WARPS = 8;
constexpr int THREADS = (CVT_WARP0 + WORK_WARPS) * 32;
constexpr int A_TILE_BYTES = BM * BK * 4; // 16 KB
constexpr int STAGING_BYTES_PER_WARP = 32 * 64; // 32 rows x 16 floats
constexpr int RES_DEPTH = 3;                    // residual chunks (32 rows x 16 floats) an epilogue warp keeps in flight (resident-B kernels)
constexpr int MAX_LO_SLOTS = 4;
// A stages in tensor memory (== B-lo tiles in shared memory when B is converted in the kernel): four where the
// accumulators leave room for them, so that the converters can run further ahead of the tensor core
__host__ __device__ constexpr int lo_slots_for(int bn) { return bn <= 64 ? 4 : 2; }
constexpr int MAX_RAW_SLOTS = 8;

enum {
	SITE_RAW_EMPTY = 0x101, SITE_RAW_FULL = 0x102, SITE_CVT_FULL = 0x103, SITE_LO_EMPTY = 0x104,
	SITE_ACC_FULL = 0x105, SITE_ACC_EMPTY = 0x106
};

__device__ __forceinline__ float4 ldg4(const float* p)
{
	return __ldg(reinterpret_cast<const float4*>(p));
}

// byte offset of 16-byte chunk `chunk` of row `row` inside a 128-byte-swizzled K-major tile
__device__ __forceinline__ uint32_t swz(int row, int chunk)
{
	return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

// debug aid: per-role time stamps of the first traceSteps K-block steps of CTA 0
enum {
	// indexed by K-block step
	TR_COPY_ISSUED = 0, TR_RAW_FULL = 1, TR_CVT_DONE = 2, TR_MMA_ISSUED = 3, TR_COPY_SLOT_FREE = 4, TR_CVT_A_STORED = 5,
	TR_MMA_SAW_STEP = 6, TR_CVT_STAGE_FREE = 15,
	// indexed by tile
	TR_EPI_ACC_FULL = 7, TR_EPI_TMEM_READ = 8, TR_EPI_TILE_DONE = 9, TR_MMA_TILE_COMMITTED = 10, TR_EPI_LD0 = 11, TR_EPI_STS0 = 12,
	TR_EPI_STG0 = 13, TR_EPI_CH1 = 14,
	TR_MMA_TILE_BEGIN = 16, TR_MMA_ACC_EMPTY = 17,
	TR_ROLES = 18
};
__device__ __forceinline__ void trace(const ContractionParams& p, int role, int step)
{
	if(p.trace != nullptr && blockIdx.x == 0 && step < p.traceSteps) p.trace[role * p.traceSteps + step] = clock64();
}

struct TileCoord {
	int m0, n0, batch;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int nTiles, int tilesPerBatch, int bn, int tileM)
{
	TileCoord t;
	t.batch = tile / tilesPerBatch;
	const int r = tile - t.batch * tilesPerBatch;
	const int mTile = r / nTiles;
	t.m0 = mTile * tileM;
	t.n0 = (r - mTile * nTiles) * bn;
	return t;
}

// GATHER = false: both operands arrive by TMA and the cp.async gather code (with its per-row bookkeeping registers) is
// not even compiled in; GATHER = true: the general kernel.
// BRES = true (all-TMA only): the variant for short K loops, where a tile's epilogue outlasts its main loop.  The
// residual comes in through a cp.async ring in shared memory, several column chunks ahead of its use, instead of one
// chunk ahead in registers; and with p.b_resident the whole K range of the CTA's B tile -- every tile of the CTA has
// the same columns -- is loaded once and stays in shared memory while the ring carries A alone (a 128 x 128 tile of
// a K = 64 layer otherwise moves 32 KB of A, 64 KB of B, 64 KB of residual and 64 KB of output through L2).
template<int BN, bool GATHER, bool THREEX, bool BRES>
__global__ void __maxnreg__(128) contraction_tc_kernel(const ContractionParams p, int numTiles, int nTiles,
	int tilesPerBatch, int rawSlots, const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
	const __grid_constant__ CUtensorMap mapBlo)
{
	extern __shared__ uint8_t smem_raw[];
	// once any CTA on this device has given up on a wait, later CTAs do not start: a broken pipeline must not
	// cost two seconds per tile
	if(*reinterpret_cast<volatile int*>(p.status) != 0) return;

	// the swizzle pattern is a function of the absolute shared-memory address: tiles must start on 1024 B
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

	constexpr bool threeX = THREEX; // 3xTF32 split (three MMAs per product) or plain TF32
	constexpr int CVT_WARPS = 4; // eight (the two groups splitting a row's K range) measured no faster: the MMA issue rate bounds a step
	constexpr int CVT_THREADS = CVT_WARPS * 32;
	constexpr int EPI_WARP0 = CVT_WARP0 + CVT_WARPS;
	constexpr int EPI_WARPS = WORK_WARPS - CVT_WARPS;
	constexpr int B_TILE_BYTES = BN * BK * 4;
	// B needs no work in the kernel when the caller prepared it (lo(B) in global memory for 3xTF32, a pre-rounded B for
	// plain TF32); a raw slot then also receives the lo tile by TMA and no lo ring exists
	const bool preB = p.b_ready != 0;
	const bool loByTma = preB && threeX;
	const int B_STEP_BYTES = B_TILE_BYTES + (loByTma ? B_TILE_BYTES : 0); // B of one K block: hi (+ lo)
	const bool bRes = BRES && p.b_resident != 0;
	const int SLOT_BYTES = bRes ? A_TILE_BYTES : A_TILE_BYTES + B_STEP_BYTES;

	// Tensor memory (512 columns): two main accumulators (BN columns each) so that the epilogue of tile i overlaps the
	// MMAs of tile i + 1; for 3xTF32 the cross accumulators, two if they fit, else one that the epilogue folds into
	// the main accumulator first thing (TMEM -> registers -> TMEM) and hands back at once; then two stages of the A
	// operand (32 columns of hi [+ 32 of lo] per stage: row m of the tile in lane m, K index in the column).
	constexpr int LO_SLOTS = lo_slots_for(BN);
	constexpr uint32_t ACC_COLS = BN;
	constexpr uint32_t A_STAGE_COLS = threeX ? 64 : 32;
	// Short-K kernels add the cross products straight into the main accumulator: over at most four K blocks the
	// truncating accumulate costs a few 1e-7 (the separate accumulator exists for the long sums), and the single cross
	// accumulator of BN = 128 would otherwise chain every tile's first MMAs to the previous tile's fold.
	constexpr bool MIX_CROSS = BRES;
	constexpr int CROSS_SETS = (!threeX || MIX_CROSS) ? 0 : (4 * ACC_COLS + LO_SLOTS * A_STAGE_COLS <= 512 ? 2 : 1);
	constexpr bool FOLD = CROSS_SETS == 1;
	constexpr bool SEP_CROSS = CROSS_SETS > 0; // cross products in an accumulator of their own
	constexpr uint32_t CROSS_BASE = 2 * ACC_COLS;
	constexpr uint32_t A_BASE = CROSS_BASE + CROSS_SETS * ACC_COLS;
	constexpr uint32_t TMEM_USED = A_BASE + LO_SLOTS * A_STAGE_COLS;
	static_assert(TMEM_USED <= 512, "tensor memory budget");
	constexpr uint32_t tmemCols = TMEM_USED <= 32 ? 32 : (TMEM_USED <= 64 ? 64 : (TMEM_USED <= 128 ? 128 : (TMEM_USED <= 256 ? 256 : 512)));
	constexpr uint32_t aBaseCol = A_BASE;
	constexpr uint32_t aStageCols = A_STAGE_COLS;
	constexpr int accSets = 2;

	uint8_t* bResident = smem; // BRES: [K block][hi tile, lo tile]
	uint8_t* rawRing = smem + (bRes ? static_cast<size_t>((p.K + BK - 1) / BK) * B_STEP_BYTES : 0);
	uint8_t* loRing = rawRing + static_cast<size_t>(rawSlots) * SLOT_BYTES;
	// residual blocks on their way from global memory (cp.async by the epilogue lanes, each into places of its own)
	uint8_t* resRing = loRing + (threeX && !preB ? LO_SLOTS * B_TILE_BYTES : 0);
	uint8_t* staging = resRing + (BRES && p.residual != nullptr && p.c_vec ? MAX_EPI_WARPS * RES_DEPTH * STAGING_BYTES_PER_WARP : 0);
	uint64_t* rawFullBar = reinterpret_cast<uint64_t*>(staging + MAX_EPI_WARPS * STAGING_BYTES_PER_WARP + MAX_EPI_WARPS * 256);
	uint64_t* rawEmptyBar = rawFullBar + MAX_RAW_SLOTS;
	uint64_t* cvtFullBar = rawEmptyBar + MAX_RAW_SLOTS;
	uint64_t* loEmptyBar = cvtFullBar + MAX_RAW_SLOTS;
	uint64_t* accFullBar = loEmptyBar + MAX_LO_SLOTS;
	uint64_t* accEmptyBar = accFullBar + 2;
	uint64_t* crossEmptyBar = accEmptyBar + 2; // fold scheme only: the single cross accumulator is free again
	uint64_t* bResidentBar = crossEmptyBar + 1; // BRES: the CTA's B tiles have arrived
	uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bResidentBar + 1);
	volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const int numKb = (p.K + BK - 1) / BK;
	const int myTiles = blockIdx.x < numTiles ? (numTiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
	// with split K the unit of work is (tile, K part): `numTiles` counts those, each covers kbPer K blocks
	const int kSplits = GATHER || p.kSplits < 1 ? 1 : p.kSplits;
	const int kbPer = numKb / kSplits;
	const int totalSteps = myTiles * kbPer;
	const bool allTma = !GATHER || (p.a_tma != 0 && p.b_tma != 0);

	if(tid == 0) {
		for(int s = 0; s < MAX_RAW_SLOTS; ++s) {
			// every copy thread's cp.async arrival (only when something is gathered) + the TMA issuer's expect_tx
			mbar_init(&rawFullBar[s], allTma ? 1 : COPY_THREADS + 1);
			mbar_init(&rawEmptyBar[s], 1);
			mbar_init(&cvtFullBar[s], CVT_WARPS);
		}
		for(int s = 0; s < LO_SLOTS; ++s) mbar_init(&loEmptyBar[s], 1);
		for(int b = 0; b < 2; ++b) {
			mbar_init(&accFullBar[b], 1);
			mbar_init(&accEmptyBar[b], EPI_WARPS);
		}
		mbar_init(crossEmptyBar, EPI_WARPS);
		mbar_init(bResidentBar, 1);
		*abortFlag = 0;
		mbar_init_fence();
	}
	if(warp == MMA_WARP) {
		tmem_alloc(tmemSlot, tmemCols);
		tmem_relinquish();
	}
	if(tid == 0) {
		if(p.a_tma) tma_prefetch_descriptor(&mapA);
		if(p.b_tma) tma_prefetch_descriptor(&mapB);
	}
	tc_fence_before_sync();
	__syncthreads();
	tc_fence_after_sync();
	const uint32_t tmemBase = *tmemSlot;
	// everything above touched only this CTA's own state and ran while the previous kernel was finishing; from here on
	// the operands are read and the result is written
	dependent_wait();
	dependents_may_start();

	if(warp < COPY_WARPS && allTma) {
		// ------------------------------------------------------------------ copy, both operands by TMA
		// One thread feeds the ring: wait for the slot, announce the bytes, issue the two tensor copies.  All slot,
		// phase and filter-tap bookkeeping is incremental (no division in the loop).
		if(warp == 0) { // the whole warp walks the loop, one elected lane issues the copies
			int tile = blockIdx.x;
			int slot = 0;
			uint32_t parity = 1; // the first pass over the ring finds every slot free
			int step = 0;
			bool ok = true;
			const int hw = p.Ho * p.Wo;
			if(bRes && myTiles > 0) {
				// all K blocks of this CTA's B columns, once
				const TileCoord first = tile_coord(blockIdx.x, nTiles, tilesPerBatch, BN, p.tileM);
				if(elect_one()) {
					mbar_arrive_expect_tx(bResidentBar, static_cast<uint32_t>(numKb * B_STEP_BYTES));
					for(int kb = 0; kb < numKb; ++kb) {
						const uint32_t dst = smem_u32(bResident + static_cast<size_t>(kb) * B_STEP_BYTES);
						tma_load_3d(dst, &mapB, bResidentBar, kb * BK, first.n0, 0);
						if(loByTma) tma_load_3d(dst + B_TILE_BYTES, &mapBlo, bResidentBar, kb * BK, first.n0, 0);
					}
				}
				__syncwarp();
			}
			for(int local = 0; local < myTiles && ok; ++local, tile += gridDim.x) {
				const int tileIdx = tile / kSplits;
				const int kbBegin = (tile - tileIdx * kSplits) * kbPer;
				const TileCoord tc = tile_coord(tileIdx, nTiles, tilesPerBatch, BN, p.tileM);
				int w0 = 0, h0 = 0, img = 0;
				if(p.a_tma == 3) {
					const int outRow = tc.m0 / p.tileM; // = image * Ho + oy
					img = outRow / p.Ho;
					h0 = outRow - img * p.Ho;
				} else if(p.a_tma == 2) {
					img = tc.m0 / hw;
					const int rem = tc.m0 - img * hw;
					const int oy = rem / p.Wo;
					w0 = (rem - oy * p.Wo) * p.strW - p.padW;
					h0 = oy * p.strH - p.padH;
				}
				int c0 = 0, fs = 0, fr = 0; // channel offset inside the filter tap, tap column, tap row
				if(p.a_tma == 2 && kbBegin > 0) {
					const int tap = kbBegin * BK / p.Cin;
					c0 = kbBegin * BK - tap * p.Cin;
					fr = tap / p.S;
					fs = tap - fr * p.S;
				}
				for(int kb = kbBegin; kb < kbBegin + kbPer; ++kb, ++step) {
					if(!mbar_wait_bounded_warp(&rawEmptyBar[slot], parity, abortFlag, p.status, SITE_RAW_EMPTY)) { ok = false; break; }
					if(lane == 0) trace(p, TR_COPY_SLOT_FREE, step);
					const uint32_t aTile = smem_u32(rawRing + static_cast<size_t>(slot) * SLOT_BYTES);
					if(elect_one()) {
					mbar_arrive_expect_tx(&rawFullBar[slot], SLOT_BYTES);
					if(p.a_tma == 1) {
						tma_load_3d(aTile, &mapA, &rawFullBar[slot], kb * BK, tc.m0, tc.batch);
					} else if(p.a_tma == 3) {
						tma_load_5d(aTile, &mapA, &rawFullBar[slot], 0, 0, kb, h0, img);
					} else {
						tma_load_im2col_4d(aTile, &mapA, &rawFullBar[slot], c0, w0, h0, img,
							static_cast<uint16_t>(fs * p.dilW), static_cast<uint16_t>(fr * p.dilH));
					}
					if(!bRes) {
						tma_load_3d(aTile + A_TILE_BYTES, &mapB, &rawFullBar[slot], kb * BK, tc.n0, tc.batch);
						if(loByTma) tma_load_3d(aTile + A_TILE_BYTES + B_TILE_BYTES, &mapBlo, &rawFullBar[slot], kb * BK, tc.n0, tc.batch);
					}
					}
					__syncwarp();
					if(p.a_tma == 2) {
						c0 += BK;
						if(c0 >= p.Cin) { c0 = 0; if(++fs == p.S) { fs = 0; ++fr; } }
					}
					if(lane == 0) trace(p, TR_COPY_ISSUED, step);
					if(++slot == rawSlots) { slot = 0; parity ^= 1; }
				}
			}
		}
	} else if(GATHER && warp < COPY_WARPS) {
		// ------------------------------------------------------------------ copy, gathered operands
		// piece ownership: chunk tid%8 of rows tid/8 + 8*q.  Column-major B ([k][n]): consecutive lanes take
		// consecutive n so that each 4-byte copy is coalesced: rows tid%32 + 32*(q/4), chunks tid/32 + 2*(q%4).
		constexpr int A_PIECES = BM / 8, B_PIECES = BN / 8;
		const int row0 = tid >> 3, chunk0 = tid & 7;
		const bool bCols = p.b_mode != B_ROWS;
		const bool aVec = p.a_vec != 0, bVec = p.b_vec != 0;
		const bool conv = p.a_mode != A_ROWS;
		int tile = blockIdx.x;
		int step = 0;
		bool ok = true;
		for(int local = 0; local < myTiles && ok; ++local, tile += gridDim.x) {
			const TileCoord tc = tile_coord(tile, nTiles, tilesPerBatch, BN, p.tileM);
			const float* A = p.A + tc.batch * p.strideA;
			const float* B = p.B + tc.batch * p.strideB;
			// where this thread's rows start: an element offset into A (row-major) or the image origin (convolution)
			ConvRow aRow[A_PIECES];
#pragma unroll
			for(int i = 0; i < (p.a_tma ? 0 : A_PIECES); ++i) {
				const int m = tc.m0 + row0 + 8 * i;
				if(conv) {
					aRow[i] = conv_row(p, m);
				} else {
					aRow[i].base = m < p.M ? m * p.lda : -1;
					aRow[i].iy0 = aRow[i].ix0 = 0;
				}
			}
			for(int kb = 0; kb < numKb; ++kb, ++step) {
				const int slot = step % rawSlots;
				const uint32_t parity = ((step / rawSlots) & 1) ^ 1;
				if(!mbar_wait_bounded_warp(&rawEmptyBar[slot], parity, abortFlag, p.status, SITE_RAW_EMPTY)) { ok = false; break; }
				if(tid == 0) trace(p, TR_COPY_SLOT_FREE, step);
				const uint32_t aTile = smem_u32(rawRing + static_cast<size_t>(slot) * SLOT_BYTES);
				const uint32_t bTile = aTile + A_TILE_BYTES;
				if(tid == 0) {
					// operands that are plain boxes of a tensor (or im2col columns of an image) come by TMA: one
					// instruction per tile, zero fill outside the tensor, completion counted in bytes on rawFull
					const uint32_t bytes = (p.a_tma ? A_TILE_BYTES : 0) + (p.b_tma ? B_TILE_BYTES : 0);
					mbar_arrive_expect_tx(&rawFullBar[slot], bytes);
					if(p.a_tma == 1) {
						tma_load_3d(aTile, &mapA, &rawFullBar[slot], kb * BK, tc.m0, tc.batch);
					} else if(p.a_tma == 2) {
						const int k0 = kb * BK;
						const int tap = k0 / p.Cin;
						const int r = tap / p.S;
						const int s = tap - r * p.S;
						const int hw = p.Ho * p.Wo;
						const int n = tc.m0 / hw;
						const int rem = tc.m0 - n * hw;
						const int oy = rem / p.Wo;
						const int ox = rem - oy * p.Wo;
						tma_load_im2col_4d(aTile, &mapA, &rawFullBar[slot], k0 - tap * p.Cin, ox * p.strW - p.padW,
							oy * p.strH - p.padH, n, static_cast<uint16_t>(s * p.dilW), static_cast<uint16_t>(r * p.dilH));
					}
					if(p.b_tma) tma_load_3d(bTile, &mapB, &rawFullBar[slot], kb * BK, tc.n0, tc.batch);
				}
				const int kA = kb * BK + chunk0 * 4;
				const int kLeftA = p.K - kA; // elements of this chunk inside K: >= 4 full, 1..3 partial, <= 0 none
				if(p.a_tma) {
					// nothing to gather
				} else if(!conv) {
#pragma unroll
					for(int i = 0; i < A_PIECES; ++i) {
						const uint32_t dst = aTile + swz(row0 + 8 * i, chunk0);
						const bool rowOk = aRow[i].base >= 0 && kLeftA > 0;
						const float* src = rowOk ? A + aRow[i].base + kA : p.A;
						if(aVec) {
							cp_async16(dst, src, rowOk ? static_cast<uint32_t>(min(kLeftA, 4)) * 4u : 0u);
						} else {
#pragma unroll
							for(int e = 0; e < 4; ++e) {
								const bool eOk = rowOk && e < kLeftA;
								cp_async4(dst + 4 * e, eOk ? src + e : p.A, eOk ? 4u : 0u);
							}
						}
					}
				} else if(aVec) {
					// channels-last image, Cin % 4 == 0: the four K indices of a chunk share one filter tap
					const int tap = kA / p.Cin;
					const int c = kA - tap * p.Cin;
					const int r = tap / p.S;
					const int s = tap - r * p.S;
					const int dy = r * p.dilH, dx = s * p.dilW;
#pragma unroll
					for(int i = 0; i < A_PIECES; ++i) {
						const int iy = aRow[i].iy0 + dy, ix = aRow[i].ix0 + dx;
						const bool pOk = kLeftA > 0 && aRow[i].base >= 0 && static_cast<unsigned>(iy) < static_cast<unsigned>(p.H)
							&& static_cast<unsigned>(ix) < static_cast<unsigned>(p.W);
						const float* src = pOk ? A + aRow[i].base + (iy * p.W + ix) * p.Cin + c : p.A;
						cp_async16(aTile + swz(row0 + 8 * i, chunk0), src, pOk ? 16u : 0u);
					}
				} else {
					// any channel count / alignment: the filter position (r, s, c) of the four K indices depends on k only,
					// so it is decoded once per chunk and stepped; the rows differ in their image origin alone
					int r[4], s[4], c[4];
					{
						const int sc = p.S * p.Cin;
						int rr = kA / sc;
						const int j = kA - rr * sc;
						int ss = j / p.Cin;
						int cc = j - ss * p.Cin;
#pragma unroll
						for(int e = 0; e < 4; ++e) {
							r[e] = rr; s[e] = ss; c[e] = cc;
							if(++cc == p.Cin) { cc = 0; if(++ss == p.S) { ss = 0; ++rr; } }
						}
					}
#pragma unroll
					for(int i = 0; i < A_PIECES; ++i) {
						const uint32_t dst = aTile + swz(row0 + 8 * i, chunk0);
#pragma unroll
						for(int e = 0; e < 4; ++e) {
							const int iy = aRow[i].iy0 + r[e] * p.dilH, ix = aRow[i].ix0 + s[e] * p.dilW;
							const bool eOk = e < kLeftA && aRow[i].base >= 0 && static_cast<unsigned>(iy) < static_cast<unsigned>(p.H)
								&& static_cast<unsigned>(ix) < static_cast<unsigned>(p.W);
							cp_async4(dst + 4 * e, eOk ? A + aRow[i].base + (iy * p.W + ix) * p.Cin + c[e] : p.A, eOk ? 4u : 0u);
						}
					}
				}
#pragma unroll
				for(int j = 0; j < (p.b_tma ? 0 : B_PIECES); ++j) {
					const int row = bCols ? (tid & 31) + 32 * (j >> 2) : row0 + 8 * j;
					const int bChunk = bCols ? (tid >> 5) + 2 * (j & 3) : chunk0;
					const int kB = kb * BK + bChunk * 4;
					const int kLeftB = p.K - kB;
					const uint32_t dst = bTile + swz(row, bChunk);
					const bool rowOk = tc.n0 + row < p.N && kLeftB > 0;
					if(!bCols) {
						const float* src = rowOk ? B + static_cast<size_t>(tc.n0 + row) * p.ldb + kB : p.B;
						if(bVec) {
							cp_async16(dst, src, rowOk ? static_cast<uint32_t>(min(kLeftB, 4)) * 4u : 0u);
						} else {
#pragma unroll
							for(int e = 0; e < 4; ++e) {
								const bool eOk = rowOk && e < kLeftB;
								cp_async4(dst + 4 * e, eOk ? src + e : p.B, eOk ? 4u : 0u);
							}
						}
					} else {
						// B stored [k][n]: four K-consecutive elements of column n are ldb apart
						const float* src = B + static_cast<size_t>(kB) * p.ldb + tc.n0 + row;
#pragma unroll
						for(int e = 0; e < 4; ++e) {
							const bool eOk = rowOk && e < kLeftB;
							cp_async4(dst + 4 * e, eOk ? src + static_cast<size_t>(e) * p.ldb : p.B, eOk ? 4u : 0u);
						}
					}
				}
				if(!allTma) cp_async_arrive_on(&rawFullBar[slot]);
				if(tid == 0) trace(p, TR_COPY_ISSUED, step);
			}
		}
		cp_async_wait<0>();
	} else if(warp >= CVT_WARP0 && warp < EPI_WARP0) {
		// ------------------------------------------------------------------ convert
		// A: thread ct owns row ct of the tile.  It reads the row's 32 floats from the raw slot and stores them as the
		// tensor core's A operand in tensor memory (lane ct): hi = x with the low 13 mantissa bits cleared,
		// lo = x - hi (exact in fp32) for 3xTF32; x rounded to nearest TF32 for plain TF32.  The MMAs then read A from
		// tensor memory, which leaves shared-memory bandwidth to the B operand and the copies.
		// B: 3xTF32 writes lo(B) into a shared-memory lo slot (the raw slot itself serves as hi: the tensor core
		// ignores the low mantissa bits); plain TF32 rounds the raw B tile in place.
		// With eight converter warps the two groups of four split a row's 32 K indices in halves.
		constexpr int K_PER_THREAD = CVT_WARPS == 8 ? 16 : 32;
		constexpr int B_ROWS_PER_PASS = CVT_THREADS / 8;
		constexpr int B_PIECES = BN / B_ROWS_PER_PASS;
		const int ct = tid - CVT_WARP0 * 32;
		const int row0 = ct >> 3, chunk0 = ct & 7;
		const int aRow = (warp & 3) * 32 + lane;                  // the tile row (= tensor-memory lane) of this thread
		const int kHalf = CVT_WARPS == 8 ? (warp - CVT_WARP0) >> 2 : 0; // which 16 K indices (eight warps only)
		const uint32_t aLane = tmemBase + (static_cast<uint32_t>((warp & 3) * 32) << 16) + aBaseCol;
		bool ok = true;
		int slot = 0;
		uint32_t rawParity = 0;
		for(int i = 0; i < totalSteps && ok; ++i) {
			if(!mbar_wait_bounded_warp(&rawFullBar[slot], rawParity, abortFlag, p.status, SITE_RAW_FULL)) { ok = false; break; }
			if(ct == 0) trace(p, TR_RAW_FULL, i);
			const int ls = i % LO_SLOTS;
			// the A stage and the lo slot of step i - 2 are free once that step's MMAs have completed
			if(!mbar_wait_bounded_warp(&loEmptyBar[ls], ((i / LO_SLOTS) & 1) ^ 1, abortFlag, p.status, SITE_LO_EMPTY)) { ok = false; break; }
			tc_fence_after_sync();
			if(ct == 0) trace(p, TR_CVT_STAGE_FREE, i);
			uint8_t* raw = rawRing + static_cast<size_t>(slot) * SLOT_BYTES;
			{
				// two halves of 16 K indices keep the live registers at 32
#pragma unroll
				for(int h2 = 0; h2 < K_PER_THREAD / 16; ++h2) {
					const int half = K_PER_THREAD == 16 ? kHalf : h2;
					uint32_t hi[16], lo[16];
#pragma unroll
					for(int c = 0; c < 4; ++c) {
						const float4 v = *reinterpret_cast<const float4*>(raw + swz(aRow, 4 * half + c));
						const float x[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
						for(int e = 0; e < 4; ++e) {
							if(threeX) {
								hi[4 * c + e] = __float_as_uint(x[e]) & 0xffffe000u;
								lo[4 * c + e] = __float_as_uint(x[e] - __uint_as_float(hi[4 * c + e]));
							} else {
								hi[4 * c + e] = __float_as_uint(to_tf32(x[e]));
							}
						}
					}
					tmem_st16(aLane + ls * aStageCols + 16 * half, hi);
					if(threeX) tmem_st16(aLane + ls * aStageCols + 32 + 16 * half, lo);
				}
				if(ct == 0) trace(p, TR_CVT_A_STORED, i);
				uint8_t* rawB = raw + A_TILE_BYTES;
				uint8_t* loB = loRing + static_cast<size_t>(ls) * B_TILE_BYTES;
#pragma unroll
				for(int q = 0; q < (preB ? 0 : B_PIECES); ++q) {
					const uint32_t off = swz(row0 + B_ROWS_PER_PASS * q, chunk0);
					float4 v = *reinterpret_cast<const float4*>(rawB + off);
					if(threeX) {
						float4 l;
						l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
						l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
						l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
						l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
						*reinterpret_cast<float4*>(loB + off) = l;
					} else {
						v.x = to_tf32(v.x); v.y = to_tf32(v.y); v.z = to_tf32(v.z); v.w = to_tf32(v.w);
						*reinterpret_cast<float4*>(rawB + off) = v;
					}
				}
				tmem_st_wait();
			}
			if(!preB) fence_proxy_async_smem();
			tc_fence_before_sync();
			__syncwarp();
			if(lane == 0) mbar_arrive(&cvtFullBar[ls]);
			if(ct == 0) trace(p, TR_CVT_DONE, i);
			if(++slot == rawSlots) { slot = 0; rawParity ^= 1; }
		}
	} else if(warp == MMA_WARP) {
		// ------------------------------------------------------------------ MMA issuer
		// The whole warp walks the loop (waits are shared by shuffle); one elected lane issues the instructions.
		{
			const uint32_t idesc = umma_idesc_tf32(BM, BN);
			bool ok = true;
			int it = 0;
			int slot = 0;
			if(bRes && myTiles > 0) {
				ok = mbar_wait_bounded_warp(bResidentBar, 0, abortFlag, p.status, SITE_RAW_FULL);
				tc_fence_after_sync();
			}
			for(int local = 0; local < myTiles && ok; ++local) {
				const int set = local & 1;
				const uint32_t accParity = ((local >> 1) & 1) ^ 1;
				if(lane == 0) trace(p, TR_MMA_TILE_BEGIN, local);
				if(!mbar_wait_bounded_warp(&accEmptyBar[set], accParity, abortFlag, p.status, SITE_ACC_EMPTY)) { ok = false; break; }
				if(lane == 0) trace(p, TR_MMA_ACC_EMPTY, local);
				if(FOLD && !mbar_wait_bounded_warp(crossEmptyBar, (local & 1) ^ 1, abortFlag, p.status, SITE_ACC_EMPTY)) { ok = false; break; }
				tc_fence_after_sync();
				const uint32_t accMain = tmemBase + set * ACC_COLS;
				const uint32_t accCross = SEP_CROSS ? tmemBase + CROSS_BASE + (FOLD ? 0 : set * ACC_COLS) : accMain;
				uint32_t acc = 0u; // the first MMA of a tile overwrites the accumulators
				const int work = blockIdx.x + local * gridDim.x;
				const int kbBegin = (work % kSplits) * kbPer;
				for(int kb = kbBegin; kb < kbBegin + kbPer; ++kb, ++it) {
					const int ls = it % LO_SLOTS;
					if(!mbar_wait_bounded_warp(&cvtFullBar[ls], (it / LO_SLOTS) & 1, abortFlag, p.status, SITE_CVT_FULL)) { ok = false; break; }
					tc_fence_after_sync();
					if(lane == 0) trace(p, TR_MMA_SAW_STEP, it);
					const uint32_t aHi = tmemBase + aBaseCol + ls * aStageCols;   // tensor-memory columns of this stage
					const uint32_t aLo = aHi + 32;
					const uint32_t bHi = bRes ? smem_u32(bResident + static_cast<size_t>(kb) * B_STEP_BYTES)
						: smem_u32(rawRing + static_cast<size_t>(slot) * SLOT_BYTES) + A_TILE_BYTES;
					const uint32_t bLo = loByTma ? bHi + B_TILE_BYTES : smem_u32(loRing + static_cast<size_t>(ls) * B_TILE_BYTES);
					// one descriptor per tile and step; the four 8-wide K slices of a 128-byte row are 32 bytes apart, which
					// is +2 in the descriptor's address field (units of 16 bytes)
					const uint64_t dBhi = umma_desc_k128(bHi);
					const uint64_t dBlo = umma_desc_k128(bLo);
					const int kLeft = p.K - kb * BK;
					if(elect_one()) {
						// main between the two cross products: consecutive MMAs never target the same accumulator
						if(kLeft >= BK) {
#pragma unroll
							for(int ks = 0; ks < BK / 8; ++ks) {
								const uint32_t a = ks == 0 ? acc : 1u;
								if(threeX) umma_tf32_ts(accCross, aLo + 8 * ks, dBhi + 2 * ks, idesc, a);
								umma_tf32_ts(accMain, aHi + 8 * ks, dBhi + 2 * ks, idesc, (threeX && !SEP_CROSS) ? 1u : a);
								if(threeX) umma_tf32_ts(accCross, aHi + 8 * ks, dBlo + 2 * ks, idesc, 1u);
							}
						} else {
							const int kSteps = (kLeft + 7) / 8;
							for(int ks = 0; ks < kSteps; ++ks) {
								const uint32_t a = ks == 0 ? acc : 1u;
								if(threeX) umma_tf32_ts(accCross, aLo + 8 * ks, dBhi + 2 * ks, idesc, a);
								umma_tf32_ts(accMain, aHi + 8 * ks, dBhi + 2 * ks, idesc, (threeX && !SEP_CROSS) ? 1u : a);
								if(threeX) umma_tf32_ts(accCross, aHi + 8 * ks, dBlo + 2 * ks, idesc, 1u);
							}
						}
						umma_commit(&rawEmptyBar[slot]);
						umma_commit(&loEmptyBar[ls]);
						if(kb == kbBegin + kbPer - 1) umma_commit(&accFullBar[set]);
					}
					acc = 1u; // every later step of the tile accumulates
					__syncwarp();
					if(lane == 0) trace(p, TR_MMA_ISSUED, it);
					if(++slot == rawSlots) slot = 0;
				}
				if(lane == 0) trace(p, TR_MMA_TILE_COMMITTED, local);
			}
			if(!ok && lane == 0) {
				// something timed out: give whatever was issued time to finish before TMEM is freed
				const uint64_t t0 = global_timer_ns();
				while(global_timer_ns() - t0 < 1000000ull) {
				}
			}
		}
		__syncwarp();
	} else if(warp >= EPI_WARP0) {
		// ------------------------------------------------------------------ epilogue
		constexpr int HALF_COLS = BN / (EPI_WARPS / 4); // columns per warp: half of the tile with eight warps, all with four
		constexpr int CHUNKS = HALF_COLS / 16;
		const int ew = warp - EPI_WARP0;
		const int quad = warp & 3;  // the TMEM lane quarter this warp may read
		const int half = ew >> 2;   // which half of the tile's columns
		uint8_t* stg = staging + ew * STAGING_BYTES_PER_WARP;
		const int rowInGroup = lane >> 2;  // 0..7: which of the 8 rows a warp-wide 16-byte access covers
		const int c4 = lane & 3;           // which 16-byte piece of the 64-byte row slice
		const bool vec = p.c_vec != 0;
		float* biasStrip = reinterpret_cast<float*>(staging + MAX_EPI_WARPS * STAGING_BYTES_PER_WARP) + ew * HALF_COLS;
		int biasCol = -1;
		// uniform epilogue options, decided once: the fast store path has no branch per element
		const bool fastStore = vec && p.accumulate == 0 && p.act != NB200_ACT_HSWISH && p.act != NB200_ACT_SIGMOID_GATE;
		const bool gateStore = vec && p.accumulate == 0 && p.act == NB200_ACT_SIGMOID_GATE;
		const bool clampOn = p.act == NB200_ACT_RELU;
		const float actParam = p.act_param_device != nullptr ? __ldg(p.act_param_device) : p.act_param;
		const float clampHi = actParam > 0.f ? actParam : __int_as_float(0x7f800000);
		bool ok = true;
		for(int local = 0; local < myTiles && ok; ++local) {
			const int work = blockIdx.x + local * gridDim.x;
			const int tile = work / kSplits;
			const TileCoord tc = tile_coord(tile, nTiles, tilesPerBatch, BN, p.tileM);
			// a K part of a split launch stores its partial sums in its own slab
			float* __restrict__ C = p.C + tc.batch * p.strideC + static_cast<size_t>(work - tile * kSplits) * p.M * p.ldc;
			const float* __restrict__ R = p.residual != nullptr ? p.residual + tc.batch * p.strideC : nullptr;
			const int set = local & 1;
			const uint32_t accParity = (local >> 1) & 1;
			const int rowBase = tc.m0 + quad * 32;
			const int colBase = tc.n0 + half * HALF_COLS;
			const bool useRes = vec && R != nullptr;
			const int mEnd = min(p.M, tc.m0 + p.tileM); // rows of this tile that exist and belong to it

			// (BRES kernels) The residual comes in by cp.async, RES_DEPTH column chunks ahead of its use: every lane copies the four
			// 16-byte pieces it will add later into places of its own in the warp's ring (zeros where the tile leaves
			// the matrix), one commit group per chunk, so the global-memory latency is paid while the accumulators are
			// still being computed, folded and transposed -- not once per chunk in the store pass.
			const uint32_t resLane = smem_u32(resRing) + ew * (RES_DEPTH * STAGING_BYTES_PER_WARP) + rowInGroup * 64 + c4 * 16;
			auto issue_res = [&](int ch) {
				if(ch < CHUNKS) {
					const int n = colBase + ch * 16 + c4 * 4;
#pragma unroll
					for(int i = 0; i < 4; ++i) {
						const int m = rowBase + 8 * i + rowInGroup;
						const bool in = m < mEnd && n + 4 <= p.N;
						cp_async16(resLane + (ch % RES_DEPTH) * STAGING_BYTES_PER_WARP + i * 512,
							in ? R + static_cast<size_t>(m) * p.ldr + n : R, in ? 16u : 0u);
					}
				}
				cp_async_commit();
			};
			auto take_res = [&](int ch, float4* dst) {
				cp_async_wait<RES_DEPTH - 1>();
#pragma unroll
				for(int i = 0; i < 4; ++i) {
					asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(dst[i].x), "=f"(dst[i].y), "=f"(dst[i].z), "=f"(dst[i].w)
						: "r"(resLane + (ch % RES_DEPTH) * STAGING_BYTES_PER_WARP + i * 512) : "memory");
				}
			};

			// the bias values of this warp's columns sit in a per-warp shared-memory strip; it is reloaded only when the
			// column range changes (a persistent CTA usually keeps its N tile), before the accumulators are awaited
			if(colBase != biasCol) {
				__syncwarp();
				for(int j = lane; j < HALF_COLS; j += 32) {
					const int n = colBase + j;
					biasStrip[j] = (p.bias != nullptr && n < p.N) ? __ldg(p.bias + n) : 0.f;
				}
				biasCol = colBase;
				__syncwarp();
			}
			float4 res[4];
			float4 resNext[4];
			if(BRES && useRes) {
#pragma unroll
				for(int ch = 0; ch < RES_DEPTH; ++ch) issue_res(ch);
			}
			auto load_res = [&](int ch, float4* dst) {
				const int n = colBase + ch * 16 + c4 * 4;
#pragma unroll
				for(int i = 0; i < 4; ++i) {
					const int m = rowBase + 8 * i + rowInGroup;
					dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
					if(m < mEnd && n + 4 <= p.N) dst[i] = *reinterpret_cast<const float4*>(R + static_cast<size_t>(m) * p.ldr + n);
				}
			};
			if(!BRES && useRes) {
				// pull this warp's residual rows (HALF_COLS * 4 bytes each) towards L2 while the main loop of the tile runs
				const int m = rowBase + lane;
				if(m < p.M && colBase < p.N) {
					const char* line = reinterpret_cast<const char*>(R + static_cast<size_t>(m) * p.ldr + colBase);
					const int bytes = min(HALF_COLS, p.N - colBase) * 4;
					for(int off = 0; off < bytes; off += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(line + off));
				}
			}

			if(!mbar_wait_bounded_warp(&accFullBar[set], accParity, abortFlag, p.status, SITE_ACC_FULL)) { ok = false; break; }
			tc_fence_after_sync();
			if(ew == 0 && lane == 0) trace(p, TR_EPI_ACC_FULL, local);
			const uint32_t laneCol = (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(half * HALF_COLS);
			const uint32_t accMain = tmemBase + set * ACC_COLS + laneCol;
			const uint32_t accCross = tmemBase + CROSS_BASE + (FOLD ? 0 : set * ACC_COLS) + laneCol;
			if(FOLD) {
				// one cross accumulator serves all tiles: add it into the main accumulator in place and hand it back, so
				// that the cross MMAs of the next tile wait for a few hundred cycles instead of for the whole epilogue
#pragma unroll
				for(int g = 0; g < CHUNKS; ++g) {
					uint32_t a[16], b[16];
					tmem_ld16_issue(accMain + g * 16, a);
					tmem_ld16_issue(accCross + g * 16, b);
					tmem_ld_wait();
#pragma unroll
					for(int i = 0; i < 16; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) + __uint_as_float(b[i]));
					tmem_st16(accMain + g * 16, a);
				}
				tmem_st_wait();
				tc_fence_before_sync();
				__syncwarp();
				if(lane == 0) mbar_arrive(crossEmptyBar);
			}
			if(!BRES && useRes) load_res(0, res);

			// accumulators leave TMEM 16 columns at a time (main and cross issued together, one wait); each chunk then
			// goes through the shared-memory transpose and the coalesced store pass
			// The loads of chunk g + 1 are issued as soon as chunk g has been taken out of their registers, and run
			// while chunk g goes through the transpose and the store pass (a tensor-memory load takes several hundred
			// cycles; waited for chunk by chunk it was most of the epilogue).
			uint32_t vm[16], vx[16];
			tmem_ld16_issue(accMain, vm);
			if(SEP_CROSS && !FOLD) tmem_ld16_issue(accCross, vx);
#pragma unroll
			for(int g0 = 0; g0 < CHUNKS; ++g0) {
				tmem_ld_wait();
				if(g0 == 0 && ew == 0 && lane == 0) trace(p, TR_EPI_LD0, local);
				float v[16];
#pragma unroll
				for(int i = 0; i < 16; ++i) {
					v[i] = __uint_as_float(vm[i]);
					if(SEP_CROSS && !FOLD) v[i] += __uint_as_float(vx[i]);
				}
				if(g0 + 1 < CHUNKS) {
					tmem_ld16_issue(accMain + (g0 + 1) * 16, vm);
					if(SEP_CROSS && !FOLD) tmem_ld16_issue(accCross + (g0 + 1) * 16, vx);
				}
				if(g0 + 1 >= CHUNKS) {
					// last TMEM read of this tile: hand the accumulator set back to the MMA warp
					tc_fence_before_sync();
					__syncwarp();
					if(lane == 0) mbar_arrive(&accEmptyBar[set]);
					if(ew == 0 && lane == 0) trace(p, TR_EPI_TMEM_READ, local);
				}
				{
					const int ch = g0;
					const int n = colBase + ch * 16 + c4 * 4; // first of this lane's four columns in the transposed phase
					const bool colsFull = n + 4 <= p.N;
					if(BRES) {
						if(useRes) take_res(ch, res);
					} else if(useRes && ch + 1 < CHUNKS) {
						load_res(ch + 1, resNext);
					}
					// transpose through shared memory: row-per-lane -> 8 rows x 64 B per warp access
#pragma unroll
					for(int q = 0; q < 4; ++q) {
						*reinterpret_cast<float4*>(stg + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) =
							make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
					}
					__syncwarp();
					if(ch == 0 && ew == 0 && lane == 0) trace(p, TR_EPI_STS0, local);
					const float4 bias4 = *reinterpret_cast<const float4*>(biasStrip + ch * 16 + c4 * 4);
					// all four transposed reads first: the stores below are generic-address stores, which the compiler will
					// not move shared-memory loads across
					float4 ov[4];
#pragma unroll
					for(int i = 0; i < 4; ++i) {
						const int r = 8 * i + rowInGroup;
						ov[i] = *reinterpret_cast<const float4*>(stg + r * 64 + ((c4 ^ ((r >> 1) & 3)) << 4));
					}
					if(fastStore && colsFull) {
						// the common case, free of branches: bias, optional residual, clamp by select, predicated 16-byte store
#pragma unroll
						for(int i = 0; i < 4; ++i) {
							const int m = rowBase + 8 * i + rowInGroup;
							float4 o = ov[i];
							o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
							if(useRes) { o.x += res[i].x; o.y += res[i].y; o.z += res[i].z; o.w += res[i].w; }
							o.x = clampOn ? fminf(fmaxf(o.x, 0.f), clampHi) : o.x;
							o.y = clampOn ? fminf(fmaxf(o.y, 0.f), clampHi) : o.y;
							o.z = clampOn ? fminf(fmaxf(o.z, 0.f), clampHi) : o.z;
							o.w = clampOn ? fminf(fmaxf(o.w, 0.f), clampHi) : o.w;
							float* dst = C + static_cast<size_t>(m) * p.ldc + n;
							if(m < mEnd) {
								asm volatile("st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
							}
						}
					} else if(gateStore && colsFull) {
						// the same with the sigmoid gate as activation: a loop of its own, so that the common one above carries
						// none of its code (the short-K layers are bound by that loop)
#pragma unroll
						for(int i = 0; i < 4; ++i) {
							const int m = rowBase + 8 * i + rowInGroup;
							float4 o = ov[i];
							o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
							if(useRes) { o.x += res[i].x; o.y += res[i].y; o.z += res[i].z; o.w += res[i].w; }
							o.x = apply_act(o.x, NB200_ACT_SIGMOID_GATE, actParam); o.y = apply_act(o.y, NB200_ACT_SIGMOID_GATE, actParam);
							o.z = apply_act(o.z, NB200_ACT_SIGMOID_GATE, actParam); o.w = apply_act(o.w, NB200_ACT_SIGMOID_GATE, actParam);
							float* dst = C + static_cast<size_t>(m) * p.ldc + n;
							if(m < mEnd) {
								asm volatile("st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
							}
						}
					} else {
#pragma unroll
						for(int i = 0; i < 4; ++i) {
							const int m = rowBase + 8 * i + rowInGroup;
							const float4 o = ov[i];
							if(m >= mEnd || n >= p.N) continue;
							const float e[4] = { o.x + bias4.x, o.y + bias4.y, o.z + bias4.z, o.w + bias4.w };
							float* dst = C + static_cast<size_t>(m) * p.ldc + n;
#pragma unroll
							for(int t = 0; t < 4; ++t) {
								if(n + t < p.N) {
									float x = e[t];
									if(R != nullptr) x += R[static_cast<size_t>(m) * p.ldr + n + t];
									x = apply_act(x, p.act, actParam);
									if(p.accumulate) x += dst[t];
									dst[t] = x;
								}
							}
						}
					}
					// the places this chunk's residual came from are free again: bring in the chunk RES_DEPTH further on
					if(BRES) {
						if(useRes) issue_res(ch + RES_DEPTH);
					} else {
#pragma unroll
						for(int i = 0; i < 4; ++i) res[i] = resNext[i];
					}
					if(ch == 0 && ew == 0 && lane == 0) trace(p, TR_EPI_STG0, local);
					if(ch == 1 && ew == 0 && lane == 0) trace(p, TR_EPI_CH1, local);
					__syncwarp(); // the staging slice is rewritten by the next column chunk
				}
			}
			if(ew == 0 && lane == 0) trace(p, TR_EPI_TILE_DONE, local);
		}
	}

	tc_fence_before_sync();
	__syncthreads();
	if(warp == MMA_WARP) {
		tc_fence_after_sync();
		tmem_dealloc(tmemBase, tmemCols);
	}
}

// ---- tensor maps ----------------------------------------------------------------------------------------------------
// The driver entry points are fetched through the runtime so that this library does not link libcuda and still loads
// on a machine without a driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
	const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
	CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
	const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
	CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encodeTiled = nullptr;
EncodeIm2colFn g_encodeIm2col = nullptr;
std::once_flag g_encodeOnce;

// Several engines may make their first call at the same moment from different host threads (one thread per replica):
// the lookup runs once, and everybody sees its result.
void lookup_encoders()
{
	std::call_once(g_encodeOnce, [] {
		void* fn = nullptr;
		cudaDriverEntryPointQueryResult q;
		if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess
			&& q == cudaDriverEntryPointSuccess) {
			g_encodeTiled = reinterpret_cast<EncodeTiledFn>(fn);
		}
		fn = nullptr;
		if(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) == cudaSuccess
			&& q == cudaDriverEntryPointSuccess) {
			g_encodeIm2col = reinterpret_cast<EncodeIm2colFn>(fn);
		}
		cudaGetLastError();
	});
}

// Row-addressed operand as a 3-D tensor (k fastest, then rows, then batch); box = 32 k x boxRows rows, 128-byte swizzle.
bool make_rows_map(CUtensorMap* map, const float* base, int k, long long rows, long long ld, int batch,
	long long batchStride, int boxRows)
{
	lookup_encoders();
	if(g_encodeTiled == nullptr) return false;
	if(!aligned16(base) || ld % 4 != 0 || (batch > 1 && batchStride % 4 != 0)) return false;
	const cuuint64_t dims[3] = { static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch) };
	const cuuint64_t strides[2] = { static_cast<cuuint64_t>(ld) * 4,
		static_cast<cuuint64_t>(batch > 1 ? batchStride : rows * ld) * 4 };
	if(strides[0] >= (1ull << 40) || strides[1] >= (1ull << 40)) return false;
	const cuuint32_t box[3] = { BK, static_cast<cuuint32_t>(boxRows), 1 };
	const cuuint32_t elemStrides[3] = { 1, 1, 1 };
	return g_encodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box,
		elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
		CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Channels-last image (C, W, H, N) in im2col mode: a load delivers 128 consecutive output positions x 32 channels of
// one filter tap; the window origins run over [-pad, dim + pad - (filter - 1) * dilation) with the convolution stride.
bool make_im2col_map(CUtensorMap* map, const ContractionParams& p, int batchImages, int filterH)
{
	lookup_encoders();
	if(g_encodeIm2col == nullptr) return false;
	if(!aligned16(p.A) || p.Cin % BK != 0) return false;
	const cuuint64_t dims[4] = { static_cast<cuuint64_t>(p.Cin), static_cast<cuuint64_t>(p.W), static_cast<cuuint64_t>(p.H),
		static_cast<cuuint64_t>(batchImages) };
	const cuuint64_t strides[3] = { static_cast<cuuint64_t>(p.Cin) * 4, static_cast<cuuint64_t>(p.W) * p.Cin * 4,
		static_cast<cuuint64_t>(p.H) * p.W * p.Cin * 4 };
	const int lower[2] = { -p.padW, -p.padH };
	const int upper[2] = { p.padW - (p.S - 1) * p.dilW, p.padH - (filterH - 1) * p.dilH };
	// hardware limits of the im2col descriptor: corners in [-128, 127], tap offsets below 256, strides up to 8
	if(lower[0] < -128 || lower[1] < -128 || upper[0] < -128 || upper[1] < -128 || upper[0] > 127 || upper[1] > 127) return false;
	if((p.S - 1) * p.dilW > 255 || (filterH - 1) * p.dilH > 255 || p.strW > 8 || p.strH > 8) return false;
	const cuuint32_t elemStrides[4] = { 1, static_cast<cuuint32_t>(p.strW), static_cast<cuuint32_t>(p.strH), 1 };
	return g_encodeIm2col(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(p.A), dims, strides, lower, upper,
		BK, BM, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
		CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Padded channels-last image as a 5-D tensor (32 floats of a filter-row window, output column, filter row, output row,
// image): the windows of neighbouring output columns overlap in memory, which a tensor map expresses as a stride
// (strW pixels) smaller than the window.  A load delivers one filter row's windows for all columns of one output row.
bool make_window_map(CUtensorMap* map, const ContractionParams& p, int images, int filterH)
{
	lookup_encoders();
	if(g_encodeTiled == nullptr || !aligned16(p.A) || p.Cin % 4 != 0 || p.Wo > BM) return false;
	const cuuint64_t pixel = static_cast<cuuint64_t>(p.Cin) * 4;
	const cuuint64_t dims[5] = { BK, static_cast<cuuint64_t>(p.Wo), static_cast<cuuint64_t>(filterH),
		static_cast<cuuint64_t>(p.Ho), static_cast<cuuint64_t>(images) };
	const cuuint64_t strides[4] = { p.strW * pixel, p.W * pixel, static_cast<cuuint64_t>(p.strH) * p.W * pixel,
		static_cast<cuuint64_t>(p.H) * p.W * pixel };
	const cuuint32_t box[5] = { BK, BM, 1, 1, 1 };
	const cuuint32_t elemStrides[5] = { 1, 1, 1, 1, 1 };
	return g_encodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(p.A), dims, strides, box,
		elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
		CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

// Channels-last image batch (C, W, H, N) as a plain tiled map without swizzle: a load delivers a box of boxC channels x
// boxW columns x boxH rows of one image, zeros where the box leaves the image (a convolution's padding for free).
bool make_image_box_map(void* map, const float* base, int c, int w, int h, int n, int boxC, int boxW, int boxH, int swizzle)
{
	lookup_encoders();
	if(swizzle != 0 && boxC * 4 != 128) return false;
	if(g_encodeTiled == nullptr || !aligned16(base) || c % 4 != 0 || boxC % 4 != 0 || boxC > 256 || boxW > 256 || boxH > 256) return false;
	const cuuint64_t pixel = static_cast<cuuint64_t>(c) * 4;
	const cuuint64_t dims[4] = { static_cast<cuuint64_t>(c), static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h),
		static_cast<cuuint64_t>(n) };
	const cuuint64_t strides[3] = { pixel, w * pixel, static_cast<cuuint64_t>(h) * w * pixel };
	if(strides[2] >= (1ull << 40)) return false;
	const cuuint32_t box[4] = { static_cast<cuuint32_t>(boxC), static_cast<cuuint32_t>(boxW), static_cast<cuuint32_t>(boxH), 1 };
	const cuuint32_t elemStrides[4] = { 1, 1, 1, 1 };
	return g_encodeTiled(static_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims,
		strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
		swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
		CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
		CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

// Tail of a split-K launch: out = act(part 0 + part 1 + ... (in this order) + bias[n] + residual[m][n]).
struct SplitFinish {
	float* out;
	int parts;
	long long slab; // floats per part
	const float* bias;
	const float* residual;
	int ldr;
	int act;
	float actParam;
	const float* actParamDevice;
};

__global__ void __launch_bounds__(256) split_finish_kernel(const float* __restrict__ partials, int n4, long long quads,
	const SplitFinish f)
{
	dependent_wait();
	dependents_may_start();
	const float param = f.actParamDevice != nullptr ? __ldg(f.actParamDevice) : f.actParam;
	const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
	for(long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < quads; i += stride) {
		const long long row = i / n4;
		const int q = static_cast<int>(i - row * n4);
		float4 v = __ldg(reinterpret_cast<const float4*>(partials) + i);
		for(int part = 1; part < f.parts; ++part) {
			const float4 w = __ldg(reinterpret_cast<const float4*>(partials + part * f.slab) + i);
			v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
		}
		if(f.bias != nullptr) {
			const float4 b = __ldg(reinterpret_cast<const float4*>(f.bias) + q);
			v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
		}
		if(f.residual != nullptr) {
			const float4 r = __ldg(reinterpret_cast<const float4*>(f.residual + row * f.ldr) + q);
			v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
		}
		v.x = apply_act(v.x, f.act, param); v.y = apply_act(v.y, f.act, param);
		v.z = apply_act(v.z, f.act, param); v.w = apply_act(v.w, f.act, param);
		reinterpret_cast<float4*>(f.out)[i] = v;
	}
}

// Optional timing of the contraction launches themselves (benchmarks): a pair of events around every launch, on the
// stream it goes to, so that operand preparation, allocations and the gaps between host calls stay outside.
struct LaunchTiming {
	std::mutex mutex;
	bool enabled = false;
	std::vector<std::pair<cudaEvent_t, cudaEvent_t>> events;
	std::vector<double> flops;   // algorithmic flops of the entry-point call each launch belongs to
	size_t used = 0;
};
LaunchTiming g_timing;
thread_local double t_callFlops = 0.0;

// the next pair of events (created on first use, reused afterwards); false when timing is off
bool timing_events(cudaEvent_t* start, cudaEvent_t* stop)
{
	std::lock_guard<std::mutex> lock(g_timing.mutex);
	if(!g_timing.enabled) return false;
	if(g_timing.used == g_timing.events.size()) {
		cudaEvent_t a = nullptr, b = nullptr;
		if(cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) {
			cudaGetLastError();
			return false;
		}
		g_timing.events.emplace_back(a, b);
		g_timing.flops.push_back(0.0);
	}
	g_timing.flops[g_timing.used] = t_callFlops;
	*start = g_timing.events[g_timing.used].first;
	*stop = g_timing.events[g_timing.used].second;
	++g_timing.used;
	return true;
}

unsigned long long* g_traceBuffer = nullptr;
int g_traceSteps = 0;
int g_traceOptions = 0;

template<int BN>
int launch_bn(const ContractionParams& p0, int batch, cudaStream_t stream)
{
	ContractionParams p = p0;
	p.trace = g_traceBuffer;
	p.traceSteps = g_traceSteps;
	const bool threeX = p.precision == NB200_PREC_3XTF32;
	const bool preB = p.b_ready != 0;
	const int bStepBytes = BN * BK * 4 * (preB && threeX ? 2 : 1);
	int slotBytes = A_TILE_BYTES + bStepBytes;
	int fixedBytes = MAX_EPI_WARPS * STAGING_BYTES_PER_WARP + MAX_EPI_WARPS * 256 /*bias strips*/ + 512 /*barriers*/ + 1024 /*alignment slack*/
		+ (threeX && !preB ? lo_slots_for(BN) * BN * BK * 4 : 0);
	// as many raw slots as fit the 227 KB a CTA may use: the copies run that many K blocks ahead
	int rawSlots = (227 * 1024 - fixedBytes) / slotBytes;
	if(rawSlots > MAX_RAW_SLOTS) rawSlots = MAX_RAW_SLOTS;
	if(p.stages > 1 && p.stages < rawSlots) rawSlots = p.stages;
	if(rawSlots < 2) return NB200_ETOOBIG;
	size_t smemBytes = static_cast<size_t>(rawSlots) * slotBytes + fixedBytes;
	// the attribute is per device; one engine per device may live in this process
	static std::atomic<bool> attrSet[64];
	int dev = 0;
	if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NB200_ENODEVICE;
	if(!attrSet[dev].load()) {
		const int bytes = 227 * 1024;
		const cudaFuncAttribute attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
		if(cudaFuncSetAttribute(contraction_tc_kernel<BN, true, true, false>, attr, bytes) != cudaSuccess
			|| cudaFuncSetAttribute(contraction_tc_kernel<BN, false, true, false>, attr, bytes) != cudaSuccess
			|| cudaFuncSetAttribute(contraction_tc_kernel<BN, true, false, false>, attr, bytes) != cudaSuccess
			|| cudaFuncSetAttribute(contraction_tc_kernel<BN, false, false, false>, attr, bytes) != cudaSuccess
			|| cudaFuncSetAttribute(contraction_tc_kernel<BN, false, true, true>, attr, bytes) != cudaSuccess
			|| cudaFuncSetAttribute(contraction_tc_kernel<BN, false, false, true>, attr, bytes) != cudaSuccess) {
			cudaGetLastError();
			return NB200_ENODEVICE;
		}
		attrSet[dev].store(true);
	}
	if(p.tileM <= 0 || p.tileM > BM || p.a_mode != A_CONV_WINDOW) p.tileM = BM;
	const long long mTiles = (static_cast<long long>(p.M) + p.tileM - 1) / p.tileM;
	const long long nTiles = (p.N + BN - 1) / BN;
	const long long tilesPerBatch = mTiles * nTiles;
	const long long numTiles = tilesPerBatch * batch;
	if(numTiles > 0x7fffffffLL || numTiles * ((p.K + BK - 1) / BK) > 0x7fffffffLL) return NB200_ETOOBIG;
	const int sms = sm_count();
	// operands that TMA can describe are loaded by it; everything else (odd alignment, column-major B, channel counts
	// that do not fill a 32-wide K block) is gathered with cp.async by the copy warps
	alignas(64) CUtensorMap mapA, mapB, mapBlo;
	memset(&mapA, 0, sizeof(mapA));
	memset(&mapB, 0, sizeof(mapB));
	memset(&mapBlo, 0, sizeof(mapBlo));
	p.a_tma = 0;
	p.b_tma = 0;
	if(!(g_traceOptions & 16)) {
		if(p.a_mode == A_ROWS) {
			if(p.a_vec && make_rows_map(&mapA, p.A, p.K, p.M, p.lda, batch, p.strideA, BM)) p.a_tma = 1;
		} else if(p.a_mode == A_CONV_WINDOW) {
			if(batch == 1 && make_window_map(&mapA, p, p.M / (p.Ho * p.Wo), p.K / BK)) p.a_tma = 3;
		} else if(p.a_vec && batch == 1) {
			const int filterH = p.K / (p.S * p.Cin);
			const int images = p.M / (p.Ho * p.Wo);
			if(make_im2col_map(&mapA, p, images, filterH)) p.a_tma = 2;
		}
		if(p.b_mode == B_ROWS && p.b_vec && make_rows_map(&mapB, p.B, p.K, p.N, p.ldb, batch, p.strideB, BN)) p.b_tma = 1;
	}
	if(p.a_mode == A_CONV_WINDOW && (p.a_tma != 3 || !p.b_tma)) return NB200_EINVAL; // no gather form of this mode
	// a prepared B is only usable by the all-TMA pipeline
	if(preB && (!p.a_tma || !p.b_tma || (threeX && !make_rows_map(&mapBlo, p.Blo, p.K, p.N, p.ldb, batch, p.strideB, BN)))) {
		return NB200_EINVAL;
	}
	const bool gather = p.a_tma == 0 || p.b_tma == 0;
	// Few tiles and a long K loop (small batches: a handful of CTAs would walk dozens of K blocks while the other SMs
	// idle): cut every tile's K loop into equal parts that run as separate work items and store their partial sums in
	// slabs of the caller's scratch; a finishing pass sums the slabs in order and applies bias, residual, activation.
	const int numKb = (p.K + BK - 1) / BK;
	int kSplits = 1;
	const long long slab = static_cast<long long>(p.M) * p.N;
	if(!gather && numTiles * 2 <= sms && numKb >= 8 && p.c_vec && !p.accumulate && batch == 1 && p.ldc == p.N
		&& p.splitScratch != nullptr && aligned16(p.splitScratch) && !(g_traceOptions & 32)) {
		const long long room = sms / numTiles;
		// at least four K blocks per part (measured: two is no better, eight is slower at batch 1)
		for(int d = 2; d <= numKb / 4 && d <= room && d * slab <= p.splitScratchFloats; ++d) {
			if(numKb % d == 0) kSplits = d; // the largest divisor of the K-block count that fits the machine and the scratch
		}
	}
	SplitFinish finish = {};
	if(kSplits > 1) {
		finish.bias = p.bias; finish.residual = p.residual; finish.ldr = p.ldr; finish.act = p.act; finish.actParam = p.act_param;
		finish.actParamDevice = p.act_param_device;
		finish.out = p.C; finish.parts = kSplits; finish.slab = slab;
		p.bias = nullptr; p.residual = nullptr; p.act = NB200_ACT_NONE; p.act_param_device = nullptr;
		p.C = p.splitScratch;
	}
	p.kSplits = kSplits;
	const long long numWork = numTiles * kSplits;
	int grid = numWork < sms ? static_cast<int>(numWork) : sms;
	// Short K loops with a prepared B: keep the CTA's B columns (all K blocks, hi + lo) in shared memory for all of its
	// tiles.  Needs every tile of a CTA to have the same columns (grid a multiple of the column tiles), B small enough
	// to leave at least four A slots, and several tiles per CTA to pay for the up-front load.
	// Measured on ResNet-50's stage-1 and stage-2 layers: the residual ring pays up to four K blocks per tile (-8 %),
	// beyond that the shared memory it takes from the operand ring costs more; residency pays for one or two K blocks
	// (-7 %) and loses from eight on.
	bool shortK = false;
	p.b_resident = 0;
	if(!gather && kSplits == 1 && numKb <= 4 && p.a_mode != A_CONV_WINDOW && !(g_traceOptions & 128)) {
		const int resRing = p.residual != nullptr && p.c_vec ? MAX_EPI_WARPS * RES_DEPTH * STAGING_BYTES_PER_WARP : 0;
		const int residentBytes = numKb * bStepBytes;
		const int room = 227 * 1024 - fixedBytes - resRing - residentBytes;
		const int gridRes = static_cast<int>((sms / nTiles) * nTiles);
		if(preB && batch == 1 && numKb <= 2 && room >= 4 * A_TILE_BYTES && nTiles <= sms && gridRes * 10 >= sms * 9 && numTiles >= 4LL * gridRes) {
			shortK = true;
			p.b_resident = 1;
			grid = gridRes;
			slotBytes = A_TILE_BYTES;
			fixedBytes += resRing + residentBytes;
			rawSlots = room / A_TILE_BYTES;
		} else if((227 * 1024 - fixedBytes - resRing) / slotBytes >= 2) {
			shortK = true;
			fixedBytes += resRing;
			rawSlots = (227 * 1024 - fixedBytes) / slotBytes;
		}
		if(shortK) {
			if(rawSlots > MAX_RAW_SLOTS) rawSlots = MAX_RAW_SLOTS;
			if(p.stages > 1 && p.stages < rawSlots) rawSlots = p.stages;
			smemBytes = static_cast<size_t>(rawSlots) * slotBytes + fixedBytes;
		}
	}
	const int nt = static_cast<int>(numWork), nn = static_cast<int>(nTiles), tpb = static_cast<int>(tilesPerBatch);
	cudaEvent_t timedStart = nullptr, timedStop = nullptr;
	const bool timed = timing_events(&timedStart, &timedStop);
	if(timed) cudaEventRecord(timedStart, stream);
	const bool overlap = overlap_launches();
#define NB200_LAUNCH(G, X, R) launch_dependent(overlap, contraction_tc_kernel<BN, G, X, R>, dim3(grid), dim3(THREADS), smemBytes, stream, \
	p, nt, nn, tpb, rawSlots, mapA, mapB, mapBlo)
	if(threeX) {
		if(gather) NB200_LAUNCH(true, true, false); else if(shortK) NB200_LAUNCH(false, true, true); else NB200_LAUNCH(false, true, false);
	} else {
		if(gather) NB200_LAUNCH(true, false, false); else if(shortK) NB200_LAUNCH(false, false, true); else NB200_LAUNCH(false, false, false);
	}
#undef NB200_LAUNCH
	count_launch();
	if(kSplits > 1) {
		const long long quads = slab / 4;
		launch_dependent(overlap, split_finish_kernel, dim3(grid_for(quads, 256, 16)), dim3(256), 0, stream,
			static_cast<const float*>(p.splitScratch), p.N / 4, quads, finish);
		count_launch();
	}
	if(timed) cudaEventRecord(timedStop, stream);
	return check_launch();
}

} // namespace

void time_contractions(bool enable)
{
	std::lock_guard<std::mutex> lock(g_timing.mutex);
	g_timing.enabled = enable;
	if(enable) g_timing.used = 0;
}

void set_call_flops(double flops)
{
	t_callFlops = flops;
}

int contraction_times(float* ms, double* flops, int capacity)
{
	std::lock_guard<std::mutex> lock(g_timing.mutex);
	int n = 0;
	for(size_t i = 0; i < g_timing.used && n < capacity; ++i, ++n) {
		float t = 0.f;
		if(cudaEventSynchronize(g_timing.events[i].second) != cudaSuccess
			|| cudaEventElapsedTime(&t, g_timing.events[i].first, g_timing.events[i].second) != cudaSuccess) {
			cudaGetLastError();
			return -1;
		}
		ms[n] = t;
		if(flops != nullptr) flops[n] = g_timing.flops[i];
	}
	return n;
}

bool overlap_launches()
{
	return !(g_traceOptions & 64);
}

bool gather_forced()
{
	return (g_traceOptions & 16) != 0;
}

void set_contraction_trace(unsigned long long* buffer, int steps, int options)
{
	g_traceBuffer = buffer;
	g_traceSteps = steps;
	g_traceOptions = options;
}

int launch_contraction_tc(const ContractionParams& p, int batch, cudaStream_t stream)
{
	if(p.M <= 0 || p.N <= 0 || batch <= 0) return NB200_OK;
	if(p.K <= 0) return NB200_EINVAL;
	// tile width: least zero-padded columns over all tiles; ties go to the wider tile (fewer re-reads of A)
	const int widths[4] = { 128, 96, 64, 32 };
	int best = 128;
	long long bestPadded = -1;
	for(int i = 0; i < 4; ++i) {
		const long long padded = (static_cast<long long>(p.N) + widths[i] - 1) / widths[i] * widths[i];
		if(bestPadded < 0 || padded < bestPadded) { bestPadded = padded; best = widths[i]; }
	}
	switch(best) {
		case 32: return launch_bn<32>(p, batch, stream);
		case 64: return launch_bn<64>(p, batch, stream);
		case 96: return launch_bn<96>(p, batch, stream);
		default: return launch_bn<128>(p, batch, stream);
	}
}

} // namespace nb200
