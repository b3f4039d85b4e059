// Implicit-GEMM contraction on the 5th-generation tensor cores (tcgen05.mma kind::tf32, accumulators in TMEM).
//
// One CTA computes a 128 x BN tile of C.  Nine warps:
//   warps 0-7  producers: gather 32-wide K blocks of A (128 rows) and B (BN rows) straight from global memory
//              (no im2col matrix exists anywhere), split every value into a TF32 "hi" and a TF32 "lo" part,
//              and store both into the 128-byte-swizzled K-major shared-memory layout the MMA reads.
//              After the main loop the same warps are the epilogue: tcgen05.ld -> bias/residual/activation -> global.
//   warp 8     allocates TMEM, and one elected lane issues the MMAs: per 8-wide K step lo*hi, hi*lo, hi*hi
//              (3xTF32; the lo*lo term is below fp32 resolution) or hi*hi only (plain TF32).
//              The two cross terms go to their own TMEM accumulator: the tensor core truncates on every
//              accumulate, so the main accumulator should take one add per K step, not three; the epilogue adds
//              the small accumulator to the main one in fp32.
// Stage hand-over is by mbarriers: full[s] (256 producer arrivals, after a generic->async proxy fence) and
// empty[s] (tcgen05.commit).  Every wait is bounded; on timeout the CTA raises an abort flag, records the site in
// the device status word and falls through to the common teardown that frees TMEM.
#include "contraction.cuh"

namespace nb200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 32;                 // floats per K block = one 128-byte swizzle row
constexpr int PRODUCER_THREADS = 256;
constexpr int THREADS = PRODUCER_THREADS + 32;
constexpr int A_TILE_BYTES = BM * BK * 4; // 16 KB

enum { SITE_EMPTY = 0x101, SITE_FULL = 0x102, SITE_ACCUM = 0x103, SITE_DRAIN = 0x104 };

template<int BN>
struct Frag {
	float4 a[BM / 32];
	float4 b[BN / 32];
};

__device__ __forceinline__ float4 ldg4(const float* p)
{
	return __ldg(reinterpret_cast<const float4*>(p));
}

// Loads 4 consecutive K elements [k, k+4) of a row-addressed operand (element (row,k) at base + k).
__device__ __forceinline__ float4 load_row4(const float* rowPtr, int k, int K, bool vec)
{
	float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
	if(rowPtr == nullptr || k >= K) return v;
	if(vec && k + 4 <= K) return ldg4(rowPtr + k);
	v.x = __ldg(rowPtr + k);
	if(k + 1 < K) v.y = __ldg(rowPtr + k + 1);
	if(k + 2 < K) v.z = __ldg(rowPtr + k + 2);
	if(k + 3 < K) v.w = __ldg(rowPtr + k + 3);
	return v;
}

__device__ __forceinline__ void split_store(uint8_t* hiTile, uint8_t* loTile, int row, int chunk, float4 v, bool threeX)
{
	const uint32_t off = static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
	float4 hi;
	hi.x = to_tf32(v.x); hi.y = to_tf32(v.y); hi.z = to_tf32(v.z); hi.w = to_tf32(v.w);
	*reinterpret_cast<float4*>(hiTile + off) = hi;
	if(threeX) {
		float4 lo;
		lo.x = to_tf32(v.x - hi.x); lo.y = to_tf32(v.y - hi.y); lo.z = to_tf32(v.z - hi.z); lo.w = to_tf32(v.w - hi.w);
		*reinterpret_cast<float4*>(loTile + off) = lo;
	}
}

template<int BN>
__global__ void __launch_bounds__(THREADS, 1) contraction_tc_kernel(const ContractionParams p)
{
	extern __shared__ uint8_t smem_raw[];
	// the swizzle pattern is a function of the absolute shared-memory address: tiles must start on 1024 B
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

	// once any CTA on this device has given up on a wait, later CTAs do not start: a broken pipeline must not
	// cost two seconds per tile
	if(*reinterpret_cast<volatile int*>(p.status) != 0) return;

	const bool threeX = p.precision == NB200_PREC_3XTF32;
	constexpr int B_TILE_BYTES = BN * BK * 4;
	const int stageBytes = (A_TILE_BYTES + B_TILE_BYTES) * (threeX ? 2 : 1);
	const int stages = p.stages;

	uint64_t* fullBar = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(stages) * stageBytes);
	uint64_t* emptyBar = fullBar + stages;
	uint64_t* accumBar = emptyBar + stages;
	uint64_t* drainBar = accumBar + 1;
	uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(drainBar + 1);
	volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;

	const int nTiles = (p.N + BN - 1) / BN;
	const int tileId = blockIdx.x;
	const int nTile = tileId % nTiles;
	const int mTile = tileId / nTiles;
	const int m0 = mTile * BM;
	const int n0 = nTile * BN;
	const int batch = blockIdx.y;
	const float* __restrict__ A = p.A + batch * p.strideA;
	const float* __restrict__ B = p.B + batch * p.strideB;
	float* __restrict__ C = p.C + batch * p.strideC;
	const float* __restrict__ R = p.residual != nullptr ? p.residual + batch * p.strideC : nullptr;

	const int numKb = (p.K + BK - 1) / BK;
	constexpr uint32_t ACC_COLS = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256)); // power of two
	const uint32_t tmemCols = threeX ? 2 * ACC_COLS : ACC_COLS; // main accumulator [+ cross-term accumulator]

	if(tid == 0) {
		for(int s = 0; s < stages; ++s) {
			mbar_init(&fullBar[s], PRODUCER_THREADS);
			mbar_init(&emptyBar[s], 1);
		}
		mbar_init(accumBar, 1);
		mbar_init(drainBar, 1);
		*abortFlag = 0;
		mbar_init_fence();
	}
	if(warp == 8) {
		tmem_alloc(tmemSlot, tmemCols);
		tmem_relinquish();
	}
	tc_fence_before_sync();
	__syncthreads();
	tc_fence_after_sync();
	const uint32_t tmemBase = *tmemSlot;

	if(warp < 8) {
		// ------------------------------------------------------------------ producers
		// (row, chunk) ownership: a thread always handles 16-byte chunk `chunk` of rows row0, row0+32, ...
		int aRow0, aChunk, bRow0, bChunk;
		aRow0 = tid >> 3; aChunk = tid & 7;
		if(p.b_mode == B_ROWS) { bRow0 = tid >> 3; bChunk = tid & 7; } else { bRow0 = tid & 31; bChunk = tid >> 5; }

		const float* aPtr[BM / 32];
		ConvRow aConv[BM / 32];
#pragma unroll
		for(int i = 0; i < BM / 32; ++i) {
			const int m = m0 + aRow0 + 32 * i;
			aPtr[i] = nullptr;
			aConv[i].base = -1; aConv[i].iy0 = 0; aConv[i].ix0 = 0;
			if(p.a_mode == A_ROWS) {
				if(m < p.M) aPtr[i] = A + static_cast<size_t>(m) * p.lda;
			} else {
				aConv[i] = conv_row(p, m);
			}
		}
		const float* bPtr[BN / 32];
#pragma unroll
		for(int j = 0; j < BN / 32; ++j) {
			const int n = n0 + bRow0 + 32 * j;
			bPtr[j] = nullptr;
			if(n < p.N) bPtr[j] = p.b_mode == B_ROWS ? B + static_cast<size_t>(n) * p.ldb : B + n;
		}

		auto load = [&](int kb, Frag<BN>& f) {
			const int kA = kb * BK + aChunk * 4;
			if(p.a_mode == A_ROWS) {
#pragma unroll
				for(int i = 0; i < BM / 32; ++i) f.a[i] = load_row4(aPtr[i], kA, p.K, p.a_vec != 0);
			} else if(p.a_mode == A_CONV_TAP) {
				const int k0 = kb * BK;
				const int tap = k0 / p.Cin;
				const int c0 = k0 - tap * p.Cin + aChunk * 4;
				const int r = tap / p.S;
				const int s = tap - r * p.S;
				const int dy = r * p.dilH, dx = s * p.dilW;
#pragma unroll
				for(int i = 0; i < BM / 32; ++i) {
					const int iy = aConv[i].iy0 + dy, ix = aConv[i].ix0 + dx;
					const bool ok = aConv[i].base >= 0 && static_cast<unsigned>(iy) < static_cast<unsigned>(p.H)
						&& static_cast<unsigned>(ix) < static_cast<unsigned>(p.W);
					f.a[i] = ok ? ldg4(A + aConv[i].base + (iy * p.W + ix) * p.Cin + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
				}
			} else {
#pragma unroll
				for(int i = 0; i < BM / 32; ++i) {
					const int m = m0 + aRow0 + 32 * i;
					f.a[i].x = gather_a(p, A, aConv[i], m, kA);
					f.a[i].y = gather_a(p, A, aConv[i], m, kA + 1);
					f.a[i].z = gather_a(p, A, aConv[i], m, kA + 2);
					f.a[i].w = gather_a(p, A, aConv[i], m, kA + 3);
				}
			}
			const int kB = kb * BK + bChunk * 4;
			if(p.b_mode == B_ROWS) {
#pragma unroll
				for(int j = 0; j < BN / 32; ++j) f.b[j] = load_row4(bPtr[j], kB, p.K, p.b_vec != 0);
			} else {
#pragma unroll
				for(int j = 0; j < BN / 32; ++j) {
					float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
					if(bPtr[j] != nullptr) {
						const float* q = bPtr[j] + static_cast<size_t>(kB) * p.ldb;
						if(kB < p.K) v.x = __ldg(q);
						if(kB + 1 < p.K) v.y = __ldg(q + p.ldb);
						if(kB + 2 < p.K) v.z = __ldg(q + 2 * static_cast<size_t>(p.ldb));
						if(kB + 3 < p.K) v.w = __ldg(q + 3 * static_cast<size_t>(p.ldb));
					}
					f.b[j] = v;
				}
			}
		};

		auto store = [&](int stage, const Frag<BN>& f) {
			uint8_t* base = smem + static_cast<size_t>(stage) * stageBytes;
			uint8_t* aHi = base;
			uint8_t* aLo = base + A_TILE_BYTES;
			uint8_t* bHi = base + (threeX ? 2 : 1) * A_TILE_BYTES;
			uint8_t* bLo = bHi + B_TILE_BYTES;
#pragma unroll
			for(int i = 0; i < BM / 32; ++i) split_store(aHi, aLo, aRow0 + 32 * i, aChunk, f.a[i], threeX);
#pragma unroll
			for(int j = 0; j < BN / 32; ++j) split_store(bHi, bLo, bRow0 + 32 * j, bChunk, f.b[j], threeX);
		};

		Frag<BN> cur, nxt;
		bool ok = true;
		load(0, cur);
		for(int kb = 0; kb < numKb; ++kb) {
			if(kb + 1 < numKb) load(kb + 1, nxt);
			const int stage = kb % stages;
			const uint32_t parity = ((kb / stages) & 1) ^ 1;
			if(!mbar_wait_bounded(&emptyBar[stage], parity, abortFlag, p.status, SITE_EMPTY)) { ok = false; break; }
			store(stage, cur);
			fence_proxy_async_smem();
			mbar_arrive(&fullBar[stage]);
			cur = nxt;
		}

		// ------------------------------------------------------------------ epilogue
		if(ok) ok = mbar_wait_bounded(accumBar, 0, abortFlag, p.status, SITE_ACCUM);
		if(ok) {
			tc_fence_after_sync();
			const int quad = warp & 3;
			const int half = warp >> 2;
			const int m = m0 + quad * 32 + lane;
			constexpr int COLS_PER_HALF = BN / 2;
			float* cRow = C + static_cast<size_t>(m) * p.ldc;
			const float* rRow = R != nullptr ? R + static_cast<size_t>(m) * p.ldr : nullptr;
#pragma unroll 1
			for(int cc = 0; cc < COLS_PER_HALF; cc += 16) {
				const int col = half * COLS_PER_HALF + cc;
				float v[16];
				// every lane of the warp must take part in the TMEM load, in range or not
				const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(col);
				tmem_ld16(taddr, v);
				if(threeX) {
					float x[16];
					tmem_ld16(taddr + ACC_COLS, x);
#pragma unroll
					for(int i = 0; i < 16; ++i) v[i] += x[i];
				}
				const int n = n0 + col;
				if(m < p.M && n < p.N) {
#pragma unroll
					for(int q = 0; q < 4; ++q) {
						const int nq = n + q * 4;
						if(nq >= p.N) break;
						float o[4] = { v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3] };
						const bool full = nq + 4 <= p.N;
						if(full && p.c_vec) {
							if(p.bias != nullptr) {
								const float4 bv = ldg4(p.bias + nq);
								o[0] += bv.x; o[1] += bv.y; o[2] += bv.z; o[3] += bv.w;
							}
							if(rRow != nullptr) {
								const float4 rv = *reinterpret_cast<const float4*>(rRow + nq);
								o[0] += rv.x; o[1] += rv.y; o[2] += rv.z; o[3] += rv.w;
							}
#pragma unroll
							for(int e = 0; e < 4; ++e) o[e] = apply_act(o[e], p.act, p.act_param);
							if(p.accumulate) {
								const float4 cv = *reinterpret_cast<const float4*>(cRow + nq);
								o[0] += cv.x; o[1] += cv.y; o[2] += cv.z; o[3] += cv.w;
							}
							*reinterpret_cast<float4*>(cRow + nq) = make_float4(o[0], o[1], o[2], o[3]);
						} else {
#pragma unroll
							for(int e = 0; e < 4; ++e) {
								if(nq + e < p.N) {
									float x = o[e];
									if(p.bias != nullptr) x += __ldg(p.bias + nq + e);
									if(rRow != nullptr) x += rRow[nq + e];
									x = apply_act(x, p.act, p.act_param);
									if(p.accumulate) x += cRow[nq + e];
									cRow[nq + e] = x;
								}
							}
						}
					}
				}
			}
		}
	} else {
		// ------------------------------------------------------------------ MMA issuer (warp 8)
		if(lane == 0) {
			const uint32_t idesc = umma_idesc_tf32(BM, BN);
			bool ok = true;
			for(int kb = 0; kb < numKb && ok; ++kb) {
				const int stage = kb % stages;
				const uint32_t parity = (kb / stages) & 1;
				if(!mbar_wait_bounded(&fullBar[stage], parity, abortFlag, p.status, SITE_FULL)) { ok = false; break; }
				tc_fence_after_sync();
				const uint32_t base = smem_u32(smem + static_cast<size_t>(stage) * stageBytes);
				const uint32_t aHi = base;
				const uint32_t aLo = base + A_TILE_BYTES;
				const uint32_t bHi = base + (threeX ? 2 : 1) * A_TILE_BYTES;
				const uint32_t bLo = bHi + B_TILE_BYTES;
				const int kLeft = p.K - kb * BK;
				const int kSteps = kLeft >= BK ? BK / 8 : (kLeft + 7) / 8;
				for(int ks = 0; ks < kSteps; ++ks) {
					const uint32_t kOff = static_cast<uint32_t>(ks) * 32u; // 8 floats inside the 128-byte row
					const uint64_t dAhi = umma_desc_k128(aHi + kOff);
					const uint64_t dBhi = umma_desc_k128(bHi + kOff);
					const uint32_t acc = (kb > 0 || ks > 0) ? 1u : 0u;
					if(threeX) {
						const uint64_t dAlo = umma_desc_k128(aLo + kOff);
						const uint64_t dBlo = umma_desc_k128(bLo + kOff);
						umma_tf32_ss(tmemBase + ACC_COLS, dAlo, dBhi, idesc, acc);
						umma_tf32_ss(tmemBase + ACC_COLS, dAhi, dBlo, idesc, 1u);
					}
					umma_tf32_ss(tmemBase, dAhi, dBhi, idesc, acc);
				}
				umma_commit(&emptyBar[stage]);
			}
			if(ok) {
				umma_commit(accumBar);
			} else {
				// something timed out: let whatever was issued finish before TMEM is freed
				umma_commit(drainBar);
				const uint64_t t0 = global_timer_ns();
				while(!mbar_try_wait(drainBar, 0) && global_timer_ns() - t0 < WAIT_LIMIT_NS) {
				}
			}
		}
		__syncwarp();
	}

	tc_fence_before_sync();
	__syncthreads();
	if(warp == 8) {
		tc_fence_after_sync();
		tmem_dealloc(tmemBase, tmemCols);
	}
}

template<int BN>
int launch_bn(const ContractionParams& p, int batch, cudaStream_t stream)
{
	ContractionParams q = p;
	const bool threeX = p.precision == NB200_PREC_3XTF32;
	const int stageBytes = (A_TILE_BYTES + BN * BK * 4) * (threeX ? 2 : 1);
	const int numKb = (p.K + BK - 1) / BK;
	// as many stages as fit below ~200 KB, at most 6, at least 2, never more than the K blocks there are
	int stages = (200 * 1024) / stageBytes;
	if(stages > 6) stages = 6;
	if(stages > numKb) stages = numKb;
	if(stages < 2) stages = 2;
	if(p.stages > 0) stages = p.stages;
	q.stages = stages;
	const size_t smemBytes = static_cast<size_t>(stages) * stageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
	// the attribute is per device; one engine per device may live in this process
	static bool attrSet[64] = {};
	int dev = 0;
	if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NB200_ENODEVICE;
	if(!attrSet[dev]) {
		if(cudaFuncSetAttribute(contraction_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024)
			!= cudaSuccess) {
			cudaGetLastError();
			return NB200_ENODEVICE;
		}
		attrSet[dev] = true;
	}
	const long long mTiles = (static_cast<long long>(p.M) + BM - 1) / BM;
	const long long nTiles = (p.N + BN - 1) / BN;
	if(mTiles * nTiles > 0x7fffffffLL) return NB200_ETOOBIG;
	for(int b0 = 0; b0 < batch; b0 += 65535) {
		const int nb = batch - b0 < 65535 ? batch - b0 : 65535;
		ContractionParams r = q;
		r.A += b0 * q.strideA; r.B += b0 * q.strideB; r.C += b0 * q.strideC;
		if(r.residual != nullptr) r.residual += b0 * q.strideC;
		dim3 grid(static_cast<unsigned>(mTiles * nTiles), static_cast<unsigned>(nb), 1);
		contraction_tc_kernel<BN><<<grid, THREADS, smemBytes, stream>>>(r);
		count_launch();
	}
	return check_launch();
}

} // namespace

int launch_contraction_tc(const ContractionParams& p, int batch, cudaStream_t stream)
{
	if(p.M <= 0 || p.N <= 0 || batch <= 0) return NB200_OK;
	if(p.K <= 0) return NB200_EINVAL;
	// tile width: least zero-padded columns over all tiles; ties go to the wider tile (fewer re-reads of A)
	const int widths[5] = { 256, 192, 128, 64, 32 };
	int best = 256;
	long long bestPadded = -1;
	for(int i = 0; i < 5; ++i) {
		const long long padded = (static_cast<long long>(p.N) + widths[i] - 1) / widths[i] * widths[i];
		if(bestPadded < 0 || padded < bestPadded) { bestPadded = padded; best = widths[i]; }
	}
	switch(best) {
		case 32: return launch_bn<32>(p, batch, stream);
		case 64: return launch_bn<64>(p, batch, stream);
		case 128: return launch_bn<128>(p, batch, stream);
		case 192: return launch_bn<192>(p, batch, stream);
		default: return launch_bn<256>(p, batch, stream);
	}
}

} // namespace nb200
