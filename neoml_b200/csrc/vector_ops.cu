// Elementwise IVectorMathEngine family: one templated grid-stride kernel, 16-byte accesses when every operand is
// 16-byte aligned, scalar accesses otherwise (NeoML handles may start at any 4-byte offset).  HBM-bound.
#include "common.cuh"

namespace nb200 {

namespace {

template<int OP>
__device__ __forceinline__ float vec_apply(float a, float b, float s)
{
	switch(OP) {
		case NB200_VEC_COPY: return a;
		case NB200_VEC_FILL: return s;
		case NB200_VEC_FILL_HANDLE: return s;
		case NB200_VEC_ADD: return a + b;
		case NB200_VEC_SUB: return a - b;
		case NB200_VEC_ELTWISE_MUL: return a * b;
		case NB200_VEC_MULTIPLY: return a * s;
		case NB200_VEC_NEG_MULTIPLY: return -(a * s);
		case NB200_VEC_ADD_VALUE: return a + s;
		case NB200_VEC_RELU: {
			const float r = fmaxf(a, 0.f);
			return s > 0.f ? fminf(r, s) : r;
		}
		case NB200_VEC_SIGMOID: return 1.f / (1.f + expf(-a));
		case NB200_VEC_SQRT: return sqrtf(a);
		case NB200_VEC_INV: return 1.f / a;
		case NB200_VEC_TANH: return tanhf(a);
		case NB200_VEC_EXP: return expf(fminf(fmaxf(a, -87.3365f), 88.f));
		case NB200_VEC_HSWISH: return a <= -3.f ? 0.f : (a >= 3.f ? a : a * (a + 3.f) * (1.f / 6.f));
		case NB200_VEC_ELTWISE_MAX: return fmaxf(a, b);
		case NB200_VEC_ELTWISE_DIV: return a / b;
		case NB200_VEC_MUL_ADD: return a + b * s;
		case NB200_VEC_SIGMOID_MUL: return __fmul_rn(1.f / (1.f + expf(-__fmul_rn(a, s))), a);
	}
	return 0.f;
}

template<int OP> __host__ __device__ constexpr bool uses_a() { return OP != NB200_VEC_FILL && OP != NB200_VEC_FILL_HANDLE; }
template<int OP> __host__ __device__ constexpr bool uses_b()
{
	return OP == NB200_VEC_ADD || OP == NB200_VEC_SUB || OP == NB200_VEC_ELTWISE_MUL || OP == NB200_VEC_ELTWISE_MAX
		|| OP == NB200_VEC_ELTWISE_DIV || OP == NB200_VEC_MUL_ADD;
}

template<int OP, bool VEC>
__global__ void __launch_bounds__(256) vector_kernel(const float* __restrict__ a, const float* __restrict__ b,
	const float* __restrict__ scalar, float value, float* __restrict__ y, int count)
{
	const float s = scalar != nullptr ? __ldg(scalar) : value;
	const int stride = gridDim.x * blockDim.x;
	const int tid = blockIdx.x * blockDim.x + threadIdx.x;
	if(VEC) {
		const int count4 = count >> 2;
		const float4* a4 = reinterpret_cast<const float4*>(a);
		const float4* b4 = reinterpret_cast<const float4*>(b);
		float4* y4 = reinterpret_cast<float4*>(y);
		for(int i = tid; i < count4; i += stride) {
			float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vb = va, r;
			if(uses_a<OP>()) va = a4[i];
			if(uses_b<OP>()) vb = b4[i];
			r.x = vec_apply<OP>(va.x, vb.x, s);
			r.y = vec_apply<OP>(va.y, vb.y, s);
			r.z = vec_apply<OP>(va.z, vb.z, s);
			r.w = vec_apply<OP>(va.w, vb.w, s);
			y4[i] = r;
		}
		for(int i = (count4 << 2) + tid; i < count; i += stride) {
			y[i] = vec_apply<OP>(uses_a<OP>() ? a[i] : 0.f, uses_b<OP>() ? b[i] : 0.f, s);
		}
	} else {
		for(int i = tid; i < count; i += stride) {
			y[i] = vec_apply<OP>(uses_a<OP>() ? a[i] : 0.f, uses_b<OP>() ? b[i] : 0.f, s);
		}
	}
}

template<int OP>
int launch_vec(cudaStream_t stream, const float* a, const float* b, const float* scalar, float value, float* y, int count)
{
	if(uses_a<OP>() && a == nullptr) return NB200_EINVAL;
	if(uses_b<OP>() && b == nullptr) return NB200_EINVAL;
	const bool vec = aligned16(y) && (!uses_a<OP>() || aligned16(a)) && (!uses_b<OP>() || aligned16(b));
	const int grid = grid_for(vec ? (count + 3) / 4 : count, 256, 16);
	if(vec) {
		vector_kernel<OP, true><<<grid, 256, 0, stream>>>(a, b, scalar, value, y, count);
	} else {
		vector_kernel<OP, false><<<grid, 256, 0, stream>>>(a, b, scalar, value, y, count);
	}
	count_launch();
	return check_launch();
}

__global__ void __launch_bounds__(256) copy_int_kernel(const int* __restrict__ a, int* __restrict__ y, int count)
{
	for(int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) y[i] = a[i];
}
__global__ void __launch_bounds__(256) fill_int_kernel(int value, int* __restrict__ y, int count)
{
	for(int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) y[i] = value;
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_vector_op(void* stream, int op, const float* a, const float* b, const float* scalar, float value,
	float* y, int count)
{
	if(count < 0 || op < 0 || op >= NB200_VEC_OP_COUNT) return NB200_EINVAL;
	if(count == 0) return NB200_OK;
	if(y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	cudaStream_t s = as_stream(stream);
	// ops whose scalar NeoML keeps in device memory take it from `scalar`; with scalar == NULL they use `value`
	const bool takesScalar = op == NB200_VEC_FILL_HANDLE || op == NB200_VEC_MULTIPLY || op == NB200_VEC_NEG_MULTIPLY
		|| op == NB200_VEC_ADD_VALUE || op == NB200_VEC_RELU || op == NB200_VEC_MUL_ADD || op == NB200_VEC_SIGMOID_MUL;
	if(op == NB200_VEC_FILL_HANDLE && scalar == nullptr) return NB200_EINVAL;
	if(!takesScalar) scalar = nullptr;
	switch(op) {
#define NB200_CASE(OP) case OP: return launch_vec<OP>(s, a, b, scalar, value, y, count);
		NB200_CASE(NB200_VEC_COPY)
		NB200_CASE(NB200_VEC_FILL)
		NB200_CASE(NB200_VEC_FILL_HANDLE)
		NB200_CASE(NB200_VEC_ADD)
		NB200_CASE(NB200_VEC_SUB)
		NB200_CASE(NB200_VEC_ELTWISE_MUL)
		NB200_CASE(NB200_VEC_MULTIPLY)
		NB200_CASE(NB200_VEC_NEG_MULTIPLY)
		NB200_CASE(NB200_VEC_ADD_VALUE)
		NB200_CASE(NB200_VEC_RELU)
		NB200_CASE(NB200_VEC_SIGMOID)
		NB200_CASE(NB200_VEC_SQRT)
		NB200_CASE(NB200_VEC_INV)
		NB200_CASE(NB200_VEC_TANH)
		NB200_CASE(NB200_VEC_EXP)
		NB200_CASE(NB200_VEC_HSWISH)
		NB200_CASE(NB200_VEC_ELTWISE_MAX)
		NB200_CASE(NB200_VEC_ELTWISE_DIV)
		NB200_CASE(NB200_VEC_MUL_ADD)
		NB200_CASE(NB200_VEC_SIGMOID_MUL)
#undef NB200_CASE
	}
	return NB200_EINVAL;
}

int nb200_vector_copy_int(void* stream, const int* a, int* y, int count)
{
	if(count < 0) return NB200_EINVAL;
	if(count == 0) return NB200_OK;
	if(a == nullptr || y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	copy_int_kernel<<<grid_for(count, 256, 16), 256, 0, as_stream(stream)>>>(a, y, count);
	count_launch();
	return check_launch();
}

int nb200_vector_fill_int(void* stream, int value, int* y, int count)
{
	if(count < 0) return NB200_EINVAL;
	if(count == 0) return NB200_OK;
	if(y == nullptr) return NB200_EINVAL;
	if(device_status_word() == nullptr) return NB200_ENODEVICE;
	fill_int_kernel<<<grid_for(count, 256, 16), 256, 0, as_stream(stream)>>>(value, y, count);
	count_launch();
	return check_launch();
}

} // extern "C"
