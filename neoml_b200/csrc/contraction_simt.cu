// Exact-fp32 contraction on the CUDA cores (NB200_PREC_FP32_SIMT): same operand gathers and epilogue as the
// tensor-core kernel, one fused-multiply-add chain per output in ascending K order.  It exists as an on-device
// cross-check of the tcgen05 path (different memory path, different arithmetic units), not for speed.
#include "contraction.cuh"

namespace nb200 {

namespace {

constexpr int TILE = 32;
constexpr int KT = 32;

__global__ void __launch_bounds__(TILE * TILE / 4) contraction_simt_kernel(const ContractionParams p)
{
	__shared__ float sA[KT][TILE + 1];
	__shared__ float sB[KT][TILE + 1];

	const int batch = blockIdx.z;
	const float* A = p.A + batch * p.strideA;
	const float* B = p.B + batch * p.strideB;
	float* C = p.C + batch * p.strideC;
	const float* R = p.residual != nullptr ? p.residual + batch * p.strideC : nullptr;

	const int m0 = blockIdx.x * TILE;
	const int n0 = blockIdx.y * TILE;
	const int tx = threadIdx.x & 31; // n
	const int ty = threadIdx.x >> 5; // 0..7, rows ty*4 .. ty*4+3

	float acc[4] = { 0.f, 0.f, 0.f, 0.f };
	for(int k0 = 0; k0 < p.K; k0 += KT) {
		// each thread fills 4 elements of each staging tile
		for(int i = 0; i < 4; ++i) {
			const int idx = threadIdx.x + i * 256;
			const int kk = idx & 31;
			const int rr = idx >> 5;
			const int m = m0 + rr;
			const ConvRow row = p.a_mode == A_ROWS ? ConvRow{ 0, 0, 0 } : conv_row(p, m);
			sA[kk][rr] = gather_a(p, A, row, m, k0 + kk);
			sB[kk][rr] = gather_b(p, B, n0 + rr, k0 + kk);
		}
		__syncthreads();
		const int kEnd = min(KT, p.K - k0);
		for(int kk = 0; kk < kEnd; ++kk) {
			const float b = sB[kk][tx];
#pragma unroll
			for(int i = 0; i < 4; ++i) acc[i] = fmaf(sA[kk][ty * 4 + i], b, acc[i]);
		}
		__syncthreads();
	}
	const int n = n0 + tx;
	if(n >= p.N) return;
	for(int i = 0; i < 4; ++i) {
		const int m = m0 + ty * 4 + i;
		if(m >= p.M) continue;
		float x = acc[i];
		if(p.bias != nullptr) x += p.bias[n];
		if(R != nullptr) x += R[static_cast<size_t>(m) * p.ldr + n];
		x = apply_act(x, p.act, p.act_param_device != nullptr ? __ldg(p.act_param_device) : p.act_param);
		float* dst = C + static_cast<size_t>(m) * p.ldc + n;
		if(p.accumulate) x += *dst;
		*dst = x;
	}
}

} // namespace

int launch_contraction_simt(const ContractionParams& p, int batch, cudaStream_t stream)
{
	if(p.M <= 0 || p.N <= 0 || batch <= 0) return NB200_OK;
	if(p.K <= 0) return NB200_EINVAL;
	const long long mTiles = (static_cast<long long>(p.M) + TILE - 1) / TILE;
	const int nTiles = (p.N + TILE - 1) / TILE;
	if(nTiles > 65535) return NB200_ETOOBIG;
	for(int b0 = 0; b0 < batch; b0 += 65535) {
		const int nb = batch - b0 < 65535 ? batch - b0 : 65535;
		ContractionParams r = p;
		r.A += b0 * p.strideA; r.B += b0 * p.strideB; r.C += b0 * p.strideC;
		if(r.residual != nullptr) r.residual += b0 * p.strideC;
		dim3 grid(static_cast<unsigned>(mTiles), static_cast<unsigned>(nTiles), static_cast<unsigned>(nb));
		contraction_simt_kernel<<<grid, 256, 0, stream>>>(r);
		count_launch();
	}
	return check_launch();
}

} // namespace nb200
