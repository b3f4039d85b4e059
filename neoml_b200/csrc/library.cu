// Library-level state of the C ABI: device discovery, the per-device status word, launch accounting.
#include "common.cuh"
#include <atomic>
#include <mutex>

namespace nb200 {

namespace {
constexpr int MAX_DEVICES = 64;
std::atomic<uint64_t> g_launches{ 0 };
std::mutex g_mutex;
int* g_status[MAX_DEVICES] = {};
int g_smCount[MAX_DEVICES] = {};
int g_deviceCount = -1;

// file-scope status words: one per device that loads this library, no allocation needed
__device__ int g_statusWord;

int discover()
{
	std::lock_guard<std::mutex> lock(g_mutex);
	if(g_deviceCount >= 0) return g_deviceCount;
	int n = 0;
	if(cudaGetDeviceCount(&n) != cudaSuccess) {
		cudaGetLastError();
		n = 0;
	}
	int usable = 0;
	for(int i = 0; i < n && i < MAX_DEVICES; ++i) {
		cudaDeviceProp prop;
		if(cudaGetDeviceProperties(&prop, i) == cudaSuccess && prop.major == 10) {
			g_smCount[i] = prop.multiProcessorCount;
			++usable;
		}
	}
	g_deviceCount = usable;
	return usable;
}
} // namespace

int* device_status_word()
{
	if(discover() <= 0) return nullptr;
	int dev = 0;
	if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
	if(g_status[dev] == nullptr) {
		std::lock_guard<std::mutex> lock(g_mutex);
		if(g_status[dev] == nullptr) {
			void* ptr = nullptr;
			if(cudaGetSymbolAddress(&ptr, g_statusWord) != cudaSuccess) {
				cudaGetLastError();
				return nullptr;
			}
			g_status[dev] = static_cast<int*>(ptr);
		}
	}
	return g_status[dev];
}

int sm_count()
{
	if(discover() <= 0) return 148;
	int dev = 0;
	if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || g_smCount[dev] <= 0) return 148;
	return g_smCount[dev];
}

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

thread_local cudaError_t t_lastCudaError = cudaSuccess;

int check_launch()
{
	const cudaError_t e = cudaGetLastError();
	if(e == cudaSuccess) return NB200_OK;
	t_lastCudaError = e;
	return e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ? NB200_ENODEVICE : NB200_ELAUNCH;
}

// One warp waits, with the bounded wait every kernel of the library uses, on a barrier that nothing ever completes.
// After `limit_ns` the wait gives up: the status word receives (0x7e << 8 | 1), the kernel returns normally and the
// context stays usable -- the path a hung pipeline would take, made to happen on purpose and cheaply.
__global__ void __launch_bounds__(32) wait_probe_kernel(int* status, unsigned long long limit_ns)
{
	__shared__ uint64_t bar;
	__shared__ int abortFlag;
	if(threadIdx.x == 0) {
		mbar_init(&bar, 1);
		mbar_init_fence();
		abortFlag = 0;
	}
	__syncthreads();
	if(threadIdx.x == 0) mbar_wait_bounded(&bar, 0, &abortFlag, status, (0x7e << 8) | 1, limit_ns);
	__syncthreads();
}

} // namespace nb200

using namespace nb200;

extern "C" __attribute__((visibility("default"))) int nb200_debug_wait_probe(void* stream, unsigned long long limit_ns)
{
	int* status = device_status_word();
	if(status == nullptr) return NB200_ENODEVICE;
	if(limit_ns == 0 || limit_ns > 1000000000ull) return NB200_EINVAL; // a second at most
	wait_probe_kernel<<<1, 32, 0, as_stream(stream)>>>(status, limit_ns);
	count_launch(1);
	return check_launch();
}

extern "C" {

int nb200_version(void) { return 100; }

int nb200_device_count(void) { return discover(); }

const char* nb200_error_string(int code)
{
	switch(code) {
		case NB200_OK: return "ok";
		case NB200_EINVAL: return "invalid argument";
		case NB200_ENODEVICE: return "no usable sm_100 device";
		case NB200_ELAUNCH: return "kernel launch failed";
		case NB200_EDEVICE: return "a device-side bounded wait timed out";
		case NB200_ETOOBIG: return "request exceeds a fixed capacity";
		default: return "unknown error";
	}
}

int nb200_device_status(void* stream, int reset)
{
	int* word = device_status_word();
	if(word == nullptr) return NB200_ENODEVICE;
	int value = 0;
	if(cudaMemcpyAsync(&value, word, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream)) != cudaSuccess
		|| cudaStreamSynchronize(as_stream(stream)) != cudaSuccess) {
		cudaGetLastError();
		return NB200_ELAUNCH;
	}
	if(reset != 0 && value != 0) {
		const int zero = 0;
		cudaMemcpyAsync(word, &zero, sizeof(int), cudaMemcpyHostToDevice, as_stream(stream));
		cudaStreamSynchronize(as_stream(stream));
	}
	return value;
}

const char* nb200_last_cuda_error(void) { return cudaGetErrorString(t_lastCudaError); }

uint64_t nb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

} // extern "C"
