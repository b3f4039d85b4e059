// Parameter block shared by the tensor-core (tcgen05) and the CUDA-core contraction kernels.
// One description covers MultiplyMatrixByTransposedMatrix, MultiplyMatrixByMatrix, their batched forms and
// BlobConvolution viewed as an implicit GEMM:  C[M x N] = gatherA[M x K] * gatherB[N x K]^T  (+ epilogue).
#pragma once
#include "common.cuh"

namespace nb200 {

enum { A_ROWS = 0, A_CONV_TAP = 1, A_CONV_WINDOW = 2 };
enum { B_ROWS = 0, B_COLS = 1 };

struct ContractionParams {
	const float* A;
	const float* B;
	float* C;
	const float* bias;
	const float* residual;
	int M, N, K;
	int lda, ldb, ldc, ldr;
	long long strideA, strideB, strideC; // per batch entry (gridDim.y)
	int a_mode; // A_ROWS: element (m,k) at A[m*lda + k]
	            // A_CONV_TAP: channels-last image gather, k = (r*S + s)*Cin + c; a_vec says whether Cin % 4 == 0 and the
	            //             image is 16-byte aligned (then four consecutive k share a filter tap and move as 16 bytes)
	            // A_CONV_WINDOW: tensor-core kernel only.  A is an image already padded in space and channels whose filter
	            //             rows span at most 32 floats: K block kb = filter row kb, and row m's 32 floats are the
	            //             contiguous window that starts at padded pixel (oy*strH + kb, ox*strW).  One tile = the Wo (<= 128)
	            //             positions of one output row (tileM = Wo); H, W are the padded sizes, Cin the padded channels
	int tileM;  // output rows a tile advances by (128 except for A_CONV_WINDOW); rows beyond it are computed but not stored
	int b_mode; // B_ROWS: element (n,k) at B[n*ldb + k];  B_COLS: element (n,k) at B[k*ldb + n]
	int a_vec;  // 16-byte loads are legal for A (base and all row starts 16-byte aligned)
	int b_vec;
	int c_vec;  // 16-byte stores legal for C (and loads for residual)
	int a_tma;  // A arrives by TMA (1: tiled rows, 2: im2col, 3: row windows); the launcher decides, 0 = cp.async gather
	int b_tma;  // B arrives by TMA (tiled rows)
	const float* Blo; // optional: lo(B) = B - trunc_tf32(B) prepared by the caller (same shape and strides as B); with it,
	                  // and for plain TF32 a pre-rounded B passed as B itself, the kernel does no per-step work on B
	int kSplits;      // > 1: every tile's K loop is cut into this many equal parts that run as separate work items (few-tile
	                  // launches: latency at small batch).  Part i stores its partial result at C + i * M * ldc, where C
	                  // is then the caller's split scratch; a finishing pass sums the parts in order (deterministic) and
	                  // applies bias, residual and activation.  Set by the launcher.
	int b_resident;   // set by the launcher (short-K kernels): B stays in shared memory for all tiles of a CTA
	float* splitScratch;          // optional room for those partial results (NULL: never split)
	long long splitScratchFloats;
	int b_ready;      // 1: B needs no conversion in the kernel (Blo given for 3xTF32 / B already rounded for TF32)
	// convolution geometry (a_mode != A_ROWS)
	int H, W, Cin, Ho, Wo, S, padH, padW, strH, strW, dilH, dilW;
	// epilogue
	int act;
	float act_param;
	const float* act_param_device; // optional: the ReLU threshold lives in device memory (one float), read by the kernel
	int accumulate;
	int precision;
	int stages;
	int* status;
	// optional pipeline trace (debug aid): CTA 0 stores clock64() at [role * traceSteps + step]; nullptr = off
	unsigned long long* trace;
	int traceSteps;
};

// Decodes output row m of a convolution into the image base offset and the top-left input coordinate.
struct ConvRow {
	int base; // n * H * W * Cin, or -1 when the row is out of range
	int iy0, ix0;
};

__device__ __forceinline__ ConvRow conv_row(const ContractionParams& p, int m)
{
	ConvRow r;
	if(m >= p.M) {
		r.base = -1;
		r.iy0 = r.ix0 = 0;
		return r;
	}
	const int hw = p.Ho * p.Wo;
	const int n = m / hw;
	const int rem = m - n * hw;
	const int oy = rem / p.Wo;
	const int ox = rem - oy * p.Wo;
	r.base = n * p.H * p.W * p.Cin;
	r.iy0 = oy * p.strH - p.padH;
	r.ix0 = ox * p.strW - p.padW;
	return r;
}

// One element of the gathered A operand (generic, slow path; also used by the CUDA-core kernel).
__device__ __forceinline__ float gather_a(const ContractionParams& p, const float* A, const ConvRow& row, int m, int k)
{
	if(k >= p.K) return 0.f;
	if(p.a_mode == A_ROWS) {
		return m < p.M ? __ldg(A + static_cast<size_t>(m) * p.lda + k) : 0.f;
	}
	if(row.base < 0) return 0.f;
	const int sc = p.S * p.Cin;
	const int r = k / sc;
	const int j = k - r * sc;
	const int s = j / p.Cin;
	const int c = j - s * p.Cin;
	const int iy = row.iy0 + r * p.dilH;
	const int ix = row.ix0 + s * p.dilW;
	if(static_cast<unsigned>(iy) >= static_cast<unsigned>(p.H) || static_cast<unsigned>(ix) >= static_cast<unsigned>(p.W)) {
		return 0.f;
	}
	return __ldg(A + row.base + (iy * p.W + ix) * p.Cin + c);
}

__device__ __forceinline__ float gather_b(const ContractionParams& p, const float* B, int n, int k)
{
	if(k >= p.K || n >= p.N) return 0.f;
	return p.b_mode == B_ROWS ? __ldg(B + static_cast<size_t>(n) * p.ldb + k)
		: __ldg(B + static_cast<size_t>(k) * p.ldb + n);
}

void set_contraction_trace(unsigned long long* buffer, int steps, int options);
int launch_contraction_tc(const ContractionParams& p, int batch, cudaStream_t stream);
int launch_contraction_simt(const ContractionParams& p, int batch, cudaStream_t stream);

// Event timing of the contraction launches (diagnostics.h)
void time_contractions(bool enable);
int contraction_times(float* ms, double* flops, int capacity);
// algorithmic flops of the entry-point call that is about to launch (noted beside each timed launch)
void set_call_flops(double flops);
// true when diagnostic option 16 asks for the cp.async gather kernel even where TMA applies
bool gather_forced();
// false when diagnostic option 64 asks for ordinary launches instead of programmatic dependent ones
bool overlap_launches();
// Scratch floats of a convolution (api_contraction.cu); the room for split-K partial results comes last and is optional.
size_t convolution_scratch_floats(const nb200_conv_desc* d, bool withSplitRoom);
// nb200_blob_convolution with the size of the scratch stated
// `prepared` (optional): the filter forms of nb200_blob_convolution_prepare_filter, made ahead of the call
int blob_convolution(void* stream, const nb200_conv_desc* d, const float* x, const float* filter, float* y,
	float* scratch, size_t scratchFloats, const nb200_epilogue* epi, int precision, const float* prepared = nullptr);

} // namespace nb200
