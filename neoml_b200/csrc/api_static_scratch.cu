// Convolution whose work space belongs to the library itself.
//
// nb200_blob_convolution() prepares its operands (the split filter; for few-channel images a padded copy with
// 4-channel pixels) in scratch memory that the CALLER has to provide.  Some callers have no way to provide it at the moment of the call: a host
// whose device memory has all been handed to a pool of its own, a real-time loop in which cudaMalloc would stall every
// stream of the device, a layer that is called with a fixed memory budget it may not exceed.  For them this file keeps a
// fixed work space inside the module image (a file-scope __device__ array, placed by the driver when the module is
// loaded) and an entry point that uses it.  Neither this call nor anything below it calls cudaMalloc, cudaFree or an
// allocating library routine.
//
// What a user of this entry point has to know:
//  * the first call on a device looks the array's address up (cudaGetSymbolAddress, which may load the module); make
//    one call per device during set-up, with that device current, before any stream capture begins;
//  * the work space holds NB200_STATIC_SCRATCH_FLOATS floats; a convolution that needs more is refused with
//    NB200_ETOOBIG and nothing is launched (use nb200_blob_convolution with scratch of your own for those);
//  * there is ONE work space per device: two calls that are in flight at the same time on one device (different
//    streams, or different threads) race on it.  Calls on one stream are ordered and safe;
//  * nothing in the work space has to be zero beforehand: every float the convolution reads, the zeros of the added
//    channels and of the spatial padding included, is written by the same call first.
#include "contraction.cuh"

#include <mutex>

namespace {

constexpr int MAX_DEVICES = 64;

static __device__ __align__(256) float g_staticScratch[NB200_STATIC_SCRATCH_FLOATS];

std::mutex g_setupMutex;
float* g_scratchOnDevice[MAX_DEVICES] = {};

// the array's address on the current device; looked up once per device
float* static_scratch()
{
	int dev = 0;
	if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
		cudaGetLastError();
		return nullptr;
	}
	std::lock_guard<std::mutex> lock(g_setupMutex);
	if(g_scratchOnDevice[dev] == nullptr) {
		float* ptr = nullptr;
		if(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_staticScratch) != cudaSuccess) {
			cudaGetLastError();
			return nullptr;
		}
		g_scratchOnDevice[dev] = ptr;
	}
	return g_scratchOnDevice[dev];
}

} // namespace

extern "C" int nb200_blob_convolution_static_scratch(void* stream, const nb200_conv_desc* desc, const float* x,
	const float* filter, float* y, const nb200_epilogue* epi, int precision)
{
	if(desc == nullptr) return NB200_EINVAL;
	// the room for split-K partial results is optional: without it a few-tile convolution runs unsplit
	const size_t need = nb200::convolution_scratch_floats(desc, false);
	if(need == 0) {
		// only a descriptor with a non-positive channel, filter-count or filter-size field needs no room: the plain
		// entry point answers it (with NB200_EINVAL) without memory of any kind
		return nb200_blob_convolution(stream, desc, x, filter, y, nullptr, epi, precision);
	}
	if(need > static_cast<size_t>(NB200_STATIC_SCRATCH_FLOATS)) return NB200_ETOOBIG;
	float* scratch = static_scratch();
	if(scratch == nullptr) return NB200_ENODEVICE;
	return nb200::blob_convolution(stream, desc, x, filter, y, scratch, NB200_STATIC_SCRATCH_FLOATS, epi, precision);
}
