// CB200MathEngine: a NeoML::IMathEngine for NVIDIA B200 (sm_100a).
//
// The class is compiled against the unmodified NeoMathEngine public headers of a NeoML checkout and is created
// through a factory with the signature shape of the reference's GPU factory (NeoMathEngine.h:1282-1311).  Every
// compute method is a thin translation of the NeoML call (handles, element counts, descriptors) into one call of the
// C ABI in include/neoml_b200.h; there is no CPU fallback: methods outside the inference hot path raise
// "not implemented" through the process-wide IMathEngineExceptionHandler.
//
// Execution model: one CUDA stream per engine, calls are enqueued in program order of the calling thread(s);
// DataExchangeRaw / GetBuffer / perf-counter reads synchronise, exactly where the reference's blocking memcpy
// (GPU/CUDA/CudaMathEngine.cpp:38-48) made results visible to the host.
#pragma once

#include <NeoMathEngine/NeoMathEngine.h>

#include "neoml_b200.h"

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <thread>
#include <type_traits>
#include <unordered_map>
#include <vector>

namespace NeoML {

// The public handle type keeps its fields protected and befriends a class of this name (MemoryHandle.h:47-50);
// the reference defines it in a private header, an engine living outside that source tree defines its own.
class CMemoryHandleInternal {
public:
	static void* GetRaw( const CMemoryHandle& h ) { return const_cast<char*>( static_cast<const char*>( h.Object ) ) + h.Offset; }
	template<class T> static T* GetRaw( const CTypedMemoryHandle<T>& h ) { return static_cast<T*>( GetRaw( static_cast<const CMemoryHandle&>( h ) ) ); }
	template<class T> static const T* GetRaw( const CTypedMemoryHandle<const T>& h ) { return static_cast<const T*>( GetRaw( static_cast<const CMemoryHandle&>( h ) ) ); }
	static CMemoryHandle Create( IMathEngine* engine, const void* object ) { return CMemoryHandle( engine, object, 0 ); }
	static const void* Base( const CMemoryHandle& h ) { return h.Object; }
	static std::ptrdiff_t Offset( const CMemoryHandle& h ) { return h.Offset; }
};

// Device memory: size-class free lists over cudaMalloc (blocks are recycled, the reference's "reuse mode" is always on
// for GPU engines, MemoryEngineMixin.cpp:38-85) and one growing LIFO stack per host thread.
class CB200Memory {
public:
	CB200Memory( int device, size_t memoryLimit );
	~CB200Memory();

	void* Alloc( size_t bytes );          // nullptr when the limit or the device is exhausted
	void Free( void* ptr );
	void* StackAlloc( size_t bytes );
	void StackFree( void* ptr );
	void CleanUp();                       // releases every cached block and the calling thread's stack
	size_t Current() const { return current; }
	size_t Peak() const { return peak; }
	void ResetPeak() { peak = current; }
	size_t InPools() const { return pooled; }
	size_t FreeOnDevice() const;
	size_t BlockBytes( const void* ptr ) const;  // size of the live heap block that starts at ptr, 0 when unknown
	size_t StackBlockBytes( const void* ptr ) const; // the same for a live stack allocation of the calling thread

private:
	struct CStack {
		std::vector<std::pair<char*, size_t>> slabs; // base, capacity
		struct CMark { int slab; size_t offset; size_t bytes; };
		std::vector<CMark> marks;                     // position before each live allocation and its size
		int slab = 0;
		size_t offset = 0;
	};
	static size_t sizeClass( size_t bytes );
	void* rawAlloc( size_t bytes );

	const int device;
	const size_t limit;
	mutable std::mutex mutex;
	std::map<size_t, std::vector<void*>> freeLists;  // class size -> cached blocks
	std::unordered_map<void*, size_t> live;           // block -> class size
	std::unordered_map<std::thread::id, CStack> stacks;
	size_t current = 0, peak = 0, pooled = 0, reserved = 0;
};

// Descriptor of a channelwise convolution: a plain copy of the geometry, owned by the caller (NeoMathEngine.h:723,750)
struct CB200ChannelwiseDesc : public CChannelwiseConvolutionDesc {
	nb200_chconv_desc d;
};

class CB200MathEngine : public IMathEngine {
public:
	CB200MathEngine( int device, size_t memoryLimit, int flags );
	~CB200MathEngine() override;

	// precision selected by the factory flags: 3xTF32 unless GpuMathEngineCublasUseTensorCoresTF32Flag is given
	int Precision() const { return precision; }
	void* Stream() const { return stream; }
	// for the operation objects of B200Rowwise.cpp: work memory from the block pool (stream-ordered reuse), result
	// check, entry bookkeeping
	float* WorkAlloc( size_t floats ) const;
	void WorkFree( float* ptr ) const;
	void Check( int code, const char* method ) const { check( code, method ); }
	void Enter() const { enter(); }
	template<class T> T* Raw( const CTypedMemoryHandle<T>& h ) const { return raw( h ); }

	// non-pure virtuals of the interface
	CMathEngineDistributedInfo GetDistributedInfo() override { return distributedInfo; }
	void AbortDistributed() override;
	bool IsDistributed() const override { return comm != nullptr; }
	void SetDistributedCommunicator( void* ncclComm, const CMathEngineDistributedInfo& info );
	void ReleaseDistributedCommunicator(); // destroys (or, after an abort, aborts) the NCCL communicator

	// every pure virtual of IVectorMathEngine / IBlasEngine / IDnnEngine / IMathEngine, generated at build time from
	// the NeoMathEngine header this file is compiled against
#include "B200MathEngineDecl.inc"

private:
	void notImplemented( const char* method ) const;
	void check( int code, const char* method ) const;
	void setDevice() const;
	// Entry of every method that reads or writes device data: selects the device and launches a convolution that was
	// held back for fusion (see CPendingConvolution).
	void enter() const;
	void flushPending() const;
	struct CPendingConvolution;
	void launchConvolution( const CPendingConvolution& call ) const;
	bool independentOfPending( const CPendingConvolution& call ) const;
	bool fuseReLU( const float* first, float* result, int size, const float* thresholdOnDevice ) const;
	bool fuseAdd( const float* first, const float* second, float* result, int size ) const;
	// device pointer behind a handle of this engine; a handle that may be written through (non-const element type)
	// ends the life of whatever the engine has prepared from the allocation's earlier contents
	template<class T> T* raw( const CTypedMemoryHandle<T>& h ) const
	{
		if( !h.IsNull() && h.GetMathEngine() != this ) notImplemented( "use of a handle that belongs to another math engine" );
		if( !h.IsNull() ) noteUse( CMemoryHandleInternal::Base( h ) );
		if( lazyCount.load( std::memory_order_relaxed ) != 0 && !h.IsNull() ) {
			touchLazy( CMemoryHandleInternal::Base( h ), CMemoryHandleInternal::GetRaw( h ), !std::is_const<T>::value );
		}
		// last: what was held back for this allocation has now been launched with the prepared form of the old contents
		if( !std::is_const<T>::value && !preparedFilters.empty() ) forgetPreparedFilter( CMemoryHandleInternal::Base( h ) );
		return CMemoryHandleInternal::GetRaw( h );
	}
	// the pointer alone: for a method that first looks whether its operand is a result noted below
	template<class T> T* peek( const CTypedMemoryHandle<T>& h ) const
	{
		if( !h.IsNull() && h.GetMathEngine() != this ) notImplemented( "use of a handle that belongs to another math engine" );
		return CMemoryHandleInternal::GetRaw( h );
	}
	void vectorOp( int op, const float* a, const float* b, const float* scalar, float value, float* y, int n,
		const char* method );

	// Deferred-execution fusion of the calls a CDnn makes for conv -> [eltwise sum ->] ReLU: BlobConvolution records
	// the call instead of launching it; an in-place VectorAdd onto its result becomes the residual of the epilogue, an
	// in-place VectorReLU its activation (threshold read from device memory by the kernel).  Any other call that
	// touches data launches the recorded convolution first, so results are exactly those of the unfused sequence.
	struct CPendingConvolution {
		bool active = false;
		nb200_conv_desc d;
		const float* source = nullptr;
		const float* filter = nullptr;
		const float* freeTerm = nullptr;
		float* result = nullptr;
		const float* residual = nullptr;
		bool relu = false;
		const float* threshold = nullptr;
		long long resultFloats = 0;
		long long sourceFloats = 0, filterFloats = 0;
		const void* filterAllocation = nullptr; // base of the allocation the filter handle points into
	};
	mutable CPendingConvolution pending;
	// The same idea for the score path of attention (and FC bias -> softmax): an in-place VectorMultiply by a device
	// scalar and / or an in-place AddVectorToMatrixRows( batch 1 ) are held back; an in-place MatrixSoftmaxByRows of the
	// same buffer then runs as ONE pass (scale, mask, softmax), anything else launches them as they were called.
	struct CPendingRowOps {
		bool active = false;
		float* data = nullptr;
		long long size = 0;
		const float* scale = nullptr;   // device scalar of the held-back VectorMultiply
		const float* bias = nullptr;    // vector of the held-back AddVectorToMatrixRows
		int biasHeight = 0, biasWidth = 0;
	};
	mutable CPendingRowOps pendingRows;
	void flushRowOps() const;
	// The fully connected layer's pair: MultiplyMatrixByTransposedMatrix is recorded, an in-place AddVectorToMatrixRows
	// of its whole result that follows becomes the bias of the product's epilogue (one pass less over the result).
	struct CPendingProduct {
		bool active = false;
		const float* first = nullptr;
		int firstHeight = 0, firstWidth = 0, firstRowSize = 0;
		const float* second = nullptr;
		int secondHeight = 0, secondRowSize = 0;
		float* result = nullptr;
		int resultRowSize = 0;
	};
	mutable CPendingProduct pendingProduct;
	void flushProduct( const float* bias = nullptr ) const;
	// CGELULayer's fast form: VectorMultiply( x -> y, *scale ), VectorSigmoid( y -> y ), VectorEltwiseMultiply( x, y -> y )
	// are recorded one after the other and, when all three came, run as one pass with the same roundings.
	struct CPendingSigmoidGate {
		bool active = false, sigmoid = false;
		const float* input = nullptr;
		float* output = nullptr;
		int size = 0;
		const float* scale = nullptr;
	};
	mutable CPendingSigmoidGate pendingGate;
	void flushGate() const;
	bool anythingRecorded() const { return pending.active || pendingRows.active || pendingProduct.active || pendingGate.active; }
	// Launches every recorded call.  A note is made, copied or extended only with nothing recorded: a noted result is
	// written when somebody touches it, which may be before the next call's enter(), and a call recorded BEFORE the
	// note may still read what the note will write, or write what it will read.  (A call recorded AFTER a note has
	// resolved its operands through raw(), so it has met the note already.)
	void flushRecorded() const;
	// Results that are noted, not computed.  BlobResizeImage with constant padding, and the score chain of attention
	// (a batched MultiplyMatrixByMatrix, then in place VectorMultiply / AddVectorToMatrixRows / MatrixSoftmaxByRows)
	// only note what they would write.  The consumer that usually follows -- BlobMaxPooling over the padded image,
	// MultiplyMatrixByMatrix of the probabilities by the values -- then runs as ONE kernel over the inputs of the
	// noted calls, and the noted result is never written.  Nobody can observe that: a handle into the result's
	// allocation that reaches raw() has the noted calls launched first, so has a handle that may be written through
	// into an allocation the noted calls read; freeing such an allocation is postponed; freeing the result's own
	// allocation forgets the note.  Only results in heap blocks and stack variables of this engine are noted (their end
	// of life is seen).
	struct CLazyResult {
		enum TKind { K_Resize, K_Scores, K_Affine, K_Product };
		TKind kind = K_Resize;
		const void* resultBase = nullptr;         // allocation the result lies in
		float* result = nullptr;
		long long resultFloats = 0;
		// what the noted calls read: the allocation and where the operand ends in it.  A handle tells where an access
		// starts, not how far it goes, so an access is taken to reach from the handle to the end of its allocation:
		// it meets an operand (or the result) that ends above the handle.
		struct CInput { const void* base; const char* end; };
		std::vector<CInput> inputs;
		template<class THandle> void Reads( const THandle& handle, long long floats )
		{
			inputs.push_back( { CMemoryHandleInternal::Base( handle ),
				static_cast<const char*>( CMemoryHandleInternal::GetRaw( static_cast<const CMemoryHandle&>( handle ) ) ) + floats * sizeof( float ) } );
		}
		// K_Resize: result = from (batch x h x w x c) with a border of `value`
		int batch = 0, h = 0, w = 0, c = 0, left = 0, right = 0, top = 0, bottom = 0;
		float value = 0.f;
		const float* from = nullptr;
		// K_Scores: result[b] = first[b] (seqQ x depth) * second[b] (depth x seqTo), b < batch; then, as noted,
		// * *scale, + mask (maskWidth = seqQ * seqTo values, the same for every b), softmax over each row
		int seqQ = 0, depth = 0, seqTo = 0;
		const float* first = nullptr;
		const float* second = nullptr;
		const float* scale = nullptr;
		const float* mask = nullptr;
		bool softmax = false;
		// K_Affine: result (rows x width) = (((from + rowAdd[row]) [squared]) * rowMul[row]) * colMul[column] + colAdd[column],
		// the steps as noted so far and in this order (CObjectNormalizationLayer's chains)
		int rows = 0, width = 0;
		const float* rowAdd = nullptr;
		bool square = false;
		const float* rowMul = nullptr;
		const float* colMul = nullptr;
		const float* colAdd = nullptr;
		// K_Product: result (rows x width, dense) = first (rows x depth, row size firstRowSize) * second^T (width x depth,
		// row size secondRowSize) -- a fully connected layer's product -- then, as noted: + bias[column]; + residual
		// (CEltwiseSumLayer); or the steps of CGELULayer's fast form: * *gateScale (gate 1), sigmoid (gate 2), * the
		// biased product (gate 3 = complete: x * sigmoid( x * *gateScale ), the product's epilogue does it)
		int firstRowSize = 0, secondRowSize = 0;
		const float* bias = nullptr;
		const float* residual = nullptr;
		const float* gateScale = nullptr;
		int gate = 0;
		const float* gateSource = nullptr; // the buffer the biased product was noted for (the gate's other factor)
	};
	mutable std::vector<CLazyResult> lazy;   // under pendingMutex
	mutable std::atomic<int> lazyCount{ 0 };
	bool noteLazy( const CLazyResult& note ) const;              // false: the result is not in a heap block of this engine
	int findLazy( const void* result, CLazyResult::TKind kind ) const;
	void materializeLazy( size_t index ) const;                  // launches the noted calls, forgets the note
	void materializeAllLazy() const;
	void touchLazy( const void* allocationBase, const void* from, bool mayWrite ) const; // an access starting at `from`
	bool lazyReads( const void* allocationBase ) const;
	bool forgetLazyResultIn( const void* allocationBase ) const; // true if a note was forgotten
	// `result = op( source )` over a noted matrix: the note that describes `result` -- the source's own when the
	// call is in place, a copy bound to the new buffer otherwise; nullptr when `result` cannot carry a note
	CLazyResult* deriveNote( int sourceNote, const CFloatHandle& resultHandle ) const;
	int launchProduct( int batchSize, const float* first, int firstHeight, int firstWidth, const float* second,
		int secondWidth, float* result ) const;
	int productWithScratch( int batchSize, const float* first, int firstHeight, int firstWidth, int firstRowSize,
		const float* second, int secondHeight, int secondRowSize, float* result, int resultRowSize,
		const float* bias = nullptr, const float* residual = nullptr, const float* gateScale = nullptr,
		const void* secondAllocation = nullptr ) const;
	mutable std::recursive_mutex pendingMutex;
	// NeoML frees a layer's input blobs right after its RunOnce (reuse-memory mode), i.e. possibly while a recorded
	// call still refers to them.  Such a heap block goes back to the pool only after the recorded call has been
	// launched: the stream then orders every later user of the block behind it.
	bool pendingRefersTo( const void* begin, size_t bytes ) const;
	void releaseDeferredFrees() const;
	mutable std::vector<void*> deferredFrees;
	// Filters prepared for the tensor core (their split parts / rounded copies, the widened stem filter), kept per
	// filter allocation for as long as nothing writes to it: a network's weights are prepared once, not once per pass.
	// Key: base address of the allocation the filter handle points into.  An entry dies when a method is given a
	// writable handle into that allocation, when host data are copied into it, and when it is freed.
	struct CPreparedFilter {
		const float* filter = nullptr;  // the filter's own address (the handle's, not the allocation's)
		int k = 0, r = 0, s = 0, c = 0;
		float* data = nullptr;
	};
	mutable std::unordered_map<const void*, CPreparedFilter> preparedFilters;
	mutable std::mutex preparedMutex;
	const float* preparedFilterFor( const CPendingConvolution& call ) const;
	// the same for the second operand (the weights) of a fully connected product of `rows` rows
	const float* preparedSecondFor( const void* allocationBase, const float* second, int rows, int secondHeight, int depth,
		int secondRowSize ) const;
	void forgetPreparedFilter( const void* allocationBase ) const;
	void forgetAllPreparedFilters() const;
	// allocation base of every conv filter handle, noted at the call (raw pointers carry no allocation)

	// Host-to-device exchanges that need not wait for the kernels in flight.  Every allocation carries the sequence
	// number of the last call that may touch it (noted when a handle into it is resolved and when it is freed);
	// `completedSeq` is the sequence number reached at the last point where the compute stream was drained.  A large
	// exchange into a heap block whose last use lies at or before that point cannot conflict with anything queued, so
	// it runs on a second stream while the compute stream keeps working; the compute stream then waits for the copy
	// (an event), the host for the copy alone.  Everything else goes in order on the compute stream, as before.
	void noteUse( const void* allocationBase ) const;
	bool idleSinceLastDrain( const void* allocationBase ) const;
	void freeBlock( void* block ) const; // back to the pool, marked as possibly still read by queued kernels
	mutable std::unordered_map<const void*, uint64_t> lastUse;
	mutable std::mutex useMutex;
	mutable uint64_t opSeq = 0, completedSeq = 0;
	void* copyStream = nullptr;
	void* copyDone = nullptr; // cudaEvent_t

	const int device;
	const int precision;
	void* stream = nullptr;
	mutable CB200Memory memory;
	bool initialized = false;
	void* comm = nullptr; // ncclComm_t
	CMathEngineDistributedInfo distributedInfo;
	// pinned staging buffers handed out by GetBuffer, LIFO per engine; released ones are kept for the next call
	// (cudaMallocHost / cudaFreeHost cost milliseconds and synchronise the device, and CDnnBlob maps buffers routinely)
	struct CHostBuffer { void* host; size_t size; size_t capacity; CMemoryHandle handle; size_t pos; };
	std::vector<CHostBuffer> hostBuffers;
	std::vector<std::pair<void*, size_t>> hostCache; // pointer, capacity
	size_t hostCacheBytes = 0;
	void* takeHostBuffer( size_t size, size_t& capacity );
	void keepHostBuffer( void* host, size_t capacity );
	std::mutex hostMutex;
};

// Factory (the reference's signatures, NeoMathEngine.h:1282,1311, under names that do not collide with a
// libNeoMathEngine.so loaded in the same process).
extern "C++" {
IMathEngine* CreateB200MathEngine( int deviceIndex, size_t memoryLimit, int flags );
// The B200 devices of this machine behind the reference's manager interface (NeoMathEngine.h:1286-1305)
IGpuMathEngineManager* CreateB200MathEngineManager();
void CreateDistributedB200MathEngines( IMathEngine** mathEngines, int devsCount, const int* cudaDevs, size_t memoryLimit );
}

} // namespace NeoML
