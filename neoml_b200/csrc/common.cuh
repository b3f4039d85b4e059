// Shared device/host helpers for the sm_100a kernel library: launch bookkeeping, the per-device status
// word used by bounded waits, and thin wrappers over the PTX this library issues by hand
// (mbarrier, tcgen05 alloc/mma/commit/ld, proxy fences).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/neoml_b200.h"

namespace nb200 {

// ---- host side ---------------------------------------------------------------------------------------------
// Status word (device memory, one per device) that kernels write when a bounded wait gives up.
int* device_status_word();              // nullptr when no device is usable
void count_launch(int n = 1);
int check_launch();                     // maps cudaGetLastError() to NB200_* codes

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid size for grid-stride kernels: a whole number of waves over the SMs of the current device.
int sm_count();
// Tiled tensor map (CUtensorMap behind the void pointer) over a channels-last image batch, zero fill outside the image
// (contraction_tc.cu, where the driver's encoder is looked up).  swizzle 1: the box lands as 128-byte rows with the
// 128-byte swizzle of 16-byte units (boxC * 4 bytes must then be 128), the layout the tensor core reads for K-major
// operands; 2: 128-byte rows whose 32-byte units are permuted (the layout of MN-major tf32 operands); 0: plain.
bool make_image_box_map(void* map, const float* base, int c, int w, int h, int n, int boxC, int boxW, int boxH,
	int swizzle = 0);
// Launch `kernel` so that it may overlap the tail of the kernel before it in `stream` (the kernel itself orders its
// memory accesses with dependent_wait()).  `overlap` false: an ordinary launch.
template<typename... Params, typename... Args>
inline cudaError_t launch_dependent(bool overlap, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smemBytes,
	cudaStream_t stream, Args&&... args)
{
	cudaLaunchConfig_t config = {};
	config.gridDim = grid;
	config.blockDim = block;
	config.dynamicSmemBytes = smemBytes;
	config.stream = stream;
	cudaLaunchAttribute attribute[1];
	attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attribute[0].val.programmaticStreamSerializationAllowed = 1;
	config.attrs = attribute;
	config.numAttrs = overlap ? 1 : 0;
	return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

inline int grid_for(long long work_items, int per_block, int waves_cap = 8)
{
	long long blocks = (work_items + per_block - 1) / per_block;
	long long cap = static_cast<long long>(sm_count()) * waves_cap;
	if(blocks > cap) blocks = cap;
	if(blocks < 1) blocks = 1;
	return static_cast<int>(blocks);
}

// ---- device side -------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
	return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// True in exactly one lane of a fully converged warp.  Code that issues tcgen05 / TMA instructions this way stays
// warp-uniform up to the instruction itself, which lets the compiler keep descriptors and addresses in uniform registers.
// Programmatic dependent launch: a kernel launched with launch_dependent() may start while the kernel before it in
// the stream is still running.  It must call dependent_wait() before it touches global memory that an earlier kernel
// wrote or still reads (the wait returns when every earlier kernel has completed and its writes are visible), and it
// calls dependents_may_start() to let the kernel behind it be scheduled as soon as SMs fall free.  Both are no-ops in
// a kernel that was launched the ordinary way.
__device__ __forceinline__ void dependent_wait()
{
	asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void dependents_may_start()
{
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ bool elect_one()
{
	uint32_t pred = 0;
	asm volatile(
		"{\n\t.reg .pred P;\n\t"
		"elect.sync _|P, 0xffffffff;\n\t"
		"selp.b32 %0, 1, 0, P;\n\t}"
		: "=r"(pred));
	return pred != 0;
}

// -- mbarrier -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence()
{
	asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
	uint32_t done;
	asm volatile(
		"{\n\t.reg .pred P;\n\t"
		"mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
		"selp.b32 %0, 1, 0, P;\n\t}"
		: "=r"(done)
		: "r"(smem_u32(bar)), "r"(parity), "r"(4000u) /* may stay suspended up to 4 us per try: a waiting lane then costs
		                                                    the other warps of its scheduler almost no issue slots */
		: "memory");
	return done != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
	uint64_t t;
	asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
	return t;
}

// Bounded wait: polls until the phase with the given parity completes, the CTA-wide abort flag is raised, or two
// seconds of wall time have passed.  On timeout it raises the abort flag, records `site` in the global status word
// and returns false; the caller must then leave its role loop and go to the common teardown.
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
	int* status, int site, uint64_t limit_ns = WAIT_LIMIT_NS)
{
	if(mbar_try_wait(bar, parity)) return true;
	// the wall clock is looked at only after a few thousand failed polls: reading %globaltimer is slow, and an ordinary
	// wait in a running pipeline ends long before that
	uint64_t t0 = 0;
	for(uint32_t it = 1;; ++it) {
		if(mbar_try_wait(bar, parity)) return true;
		if((it & 4095u) == 0u) {
			if(*abort_flag != 0) return false;
			const uint64_t now = global_timer_ns();
			if(t0 == 0) t0 = now;
			else if(now - t0 > limit_ns) break;
		}
	}
	*abort_flag = 1;
	if(status != nullptr) atomicCAS(status, 0, site);
	return false;
}

// Warp-wide form for a converged warp: every lane polls (one instruction, one broadcast shared-memory access per
// try), so there is no divergent branch and no shuffle on the way out; the lanes agree on the outcome by vote.
__device__ __forceinline__ bool mbar_wait_bounded_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
	int* status, int site)
{
	bool ok = mbar_try_wait(bar, parity);
	if(!__all_sync(0xffffffffu, ok)) {
		uint64_t t0 = 0;
		for(uint32_t it = 1;; ++it) {
			ok = mbar_try_wait(bar, parity);
			if(__all_sync(0xffffffffu, ok)) break;
			if((it & 4095u) == 0u) {
				const bool aborted = *abort_flag != 0;
				const uint64_t now = global_timer_ns();
				if(t0 == 0) t0 = now;
				const bool late = now - t0 > WAIT_LIMIT_NS;
				if(__any_sync(0xffffffffu, aborted || late)) {
					if(late && (threadIdx.x & 31) == 0) {
						*abort_flag = 1;
						if(status != nullptr) atomicCAS(status, 0, site);
					}
					return false;
				}
			}
		}
	}
	return true;
}

// -- proxy / tcgen05 fences --------------------------------------------------------------------------------------
// Makes this thread's generic-proxy shared-memory writes visible to the async proxy (tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem()
{
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync()
{
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync()
{
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// -- tensor memory ---------------------------------------------------------------------------------------------
// Whole-warp calls (.sync.aligned).  `columns` is a power of two >= 32.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t columns)
{
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
		::"r"(smem_u32(dst_smem)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

// 32 lanes x 32 bit, 16 consecutive columns: thread i of warp w reads TMEM lane 32*(w%4)+i.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v)
{
	uint32_t r[16];
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
		  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
		: "r"(taddr));
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
	for(int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Same access pattern, issue only: 16 / 32 columns into r[]; tmem_ld_wait() must precede the first use of r[].
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t* r)
{
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
		  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
		: "r"(taddr));
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r)
{
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
		"%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
		  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
		  "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
		  "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
		: "r"(taddr));
}
// Register -> TMEM: the calling warp writes 32 columns of its 32 lanes (lane quarter = warp index % 4), value r[j] of
// lane l going to (lane base + l, column base + j).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r)
{
	asm volatile(
		"tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
		"%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
		::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
		  "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
		  "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
		  "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
		: "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r)
{
	asm volatile(
		"tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
		::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
		  "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
		: "memory");
}
__device__ __forceinline__ void tmem_st_wait()
{
	asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// -- UMMA descriptors --------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes (32 fp32) with the
// 128-byte swizzle: 16-byte chunk c of row r lives at r*128 + ((c ^ (r & 7)) << 4); 8-row groups are 1024 B apart.
// Field layout (PTX ISA, tcgen05 matrix descriptor): [0,14) start>>4, [16,30) leading byte offset>>4 (unused for
// swizzled K-major, set to 1), [32,46) stride byte offset>>4 (1024 B between 8-row groups), [46,48) version = 1,
// [61,64) layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr)
{
	uint64_t d = 0;
	d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
	d |= static_cast<uint64_t>(1) << 16;
	d |= static_cast<uint64_t>(1024 >> 4) << 32;
	d |= static_cast<uint64_t>(1) << 46;
	d |= static_cast<uint64_t>(2) << 61;
	return d;
}

// Instruction descriptor for kind::tf32, fp32 accumulate, both operands K-major, tile M x N.
// [4,6) D format 1 = F32; [7,10) A format 2 = TF32; [10,13) B format 2 = TF32; [15] A major 0; [16] B major 0;
// [17,23) N>>3; [24,29) M>>4.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n)
{
	return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
		(static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void umma_tf32_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
	uint32_t accumulate)
{
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
		::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
		: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 8 tf32 of K, row m in lane m, element k in column
// tmem_a + k) is read from tensor memory, so only B costs shared-memory bandwidth.
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
	uint32_t accumulate)
{
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
		::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
		: "memory");
}

// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
		::"r"(smem_u32(bar)) : "memory");
}

// -- TMA (bulk tensor copies driven by a CUtensorMap in kernel parameter space) ------------------------------------------
// Arrive + announce `bytes` of pending TMA traffic on the barrier (one thread per phase).
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Tiled load of one box at element coordinates (x, y, z); x * 4 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tmap, uint64_t* bar, int x, int y, int z)
{
	asm volatile(
		"cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
		::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, uint64_t* bar, int c0, int c1, int c2, int c3)
{
	asm volatile(
		"cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
		::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst_smem, const void* tmap, uint64_t* bar, int c0, int c1, int c2,
	int c3, int c4)
{
	asm volatile(
		"cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
		::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
		: "memory");
}
// im2col load from a channels-last image map (C, W, H, N): `pixelsPerColumn` output positions starting at the window
// origin (w, h) of image n, channels [c, c + channelsPerPixel), filter tap offset (off_w, off_h) in input pixels.
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst_smem, const void* tmap, uint64_t* bar, int c, int w,
	int h, int n, uint16_t off_w, uint16_t off_h)
{
	asm volatile(
		"cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
		" [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
		::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n),
		  "h"(off_w), "h"(off_h) : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const void* tmap)
{
	asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// -- Ampere-style asynchronous copies (global -> shared, no registers held while in flight) ------------------------
// 16-byte copy through L2 only; bytes beyond src_bytes (0..16) are written as zero.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, uint32_t src_bytes)
{
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
// 4-byte copy; src_bytes is 4 or 0 (zero fill).
__device__ __forceinline__ void cp_async4(uint32_t dst_smem, const void* src, uint32_t src_bytes)
{
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
	asm volatile("cp.async.commit_group;" ::: "memory");
}
// Arrives on the mbarrier once every cp.async issued so far by this thread has landed; the thread does not wait.
// The arrival is one of the barrier's expected arrivals (.noinc).
__device__ __forceinline__ void cp_async_arrive_on(uint64_t* bar)
{
	asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Named barrier among `threads` threads of the CTA (id 1..15; id 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int threads)
{
	asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
template<int N>
__device__ __forceinline__ void cp_async_wait()
{
	asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float to_tf32(float x)
{
	uint32_t r;
	asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
	return __uint_as_float(r);
}

__device__ __forceinline__ float apply_act(float v, int act, float param)
{
	if(act == NB200_ACT_RELU) {
		v = fmaxf(v, 0.f);
		if(param > 0.f) v = fminf(v, param);
	} else if(act == NB200_ACT_HSWISH) {
		v = v * fminf(fmaxf(v + 3.f, 0.f), 6.f) * (1.f / 6.f);
	} else if(act == NB200_ACT_SIGMOID_GATE) {
		v = __fmul_rn(1.f / (1.f + expf(-__fmul_rn(v, param))), v);
	}
	return v;
}

#endif // __CUDACC__

} // namespace nb200
