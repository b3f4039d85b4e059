// CB200MathEngine: lifecycle, memory, host<->device exchange, gauges, timing, factory.
// Compute methods live in B200MathEngineOps.cpp; everything else on the interface is a generated weak stub.
#include "B200MathEngine.h"

#include <neoml_b200.h>

#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>

namespace NeoML {

namespace {

void raiseAssert( const std::string& message )
{
	GetMathEngineExceptionHandler()->OnAssert( message.c_str(), L"B200MathEngine", 0, 0 );
}

// Time-only counter that drains the engine's stream before reading the clock, so that CDnn's per-layer profile
// (NeoML/src/Dnn/BaseLayer.cpp:469-497) measures device work and not launch time.
class CB200PerformanceCounters : public IPerformanceCounters {
public:
	CB200PerformanceCounters( int _device, void* _stream ) : IPerformanceCounters( &counter ), device( _device ), stream( _stream )
	{
		counter.Name = "time ns";
		counter.Value = 0;
		CounterCount() = 1;
		last = now();
	}
	void Synchronise() override
	{
		cudaSetDevice( device );
		cudaStreamSynchronize( static_cast<cudaStream_t>( stream ) );
		const uint64_t t = now();
		counter.Value = t - last;
		last = t;
	}

private:
	static uint64_t now()
	{
		return static_cast<uint64_t>( std::chrono::duration_cast<std::chrono::nanoseconds>(
			std::chrono::steady_clock::now().time_since_epoch() ).count() );
	}
	CCounter counter;
	const int device;
	void* const stream;
	uint64_t last;
};

} // namespace

//---------------------------------------------------------------------------------------------------------------------

CB200MathEngine::CB200MathEngine( int _device, size_t memoryLimit, int flags ) :
	device( _device ),
	precision( ( flags & GpuMathEngineCublasUseTensorCoresTF32Flag ) != 0 ? NB200_PREC_TF32 : NB200_PREC_3XTF32 ),
	memory( _device, memoryLimit )
{
	if( nb200_device_count() <= 0 || cudaSetDevice( device ) != cudaSuccess ) {
		cudaGetLastError();
		return;
	}
	cudaStream_t s = nullptr;
	if( cudaStreamCreateWithFlags( &s, cudaStreamNonBlocking ) != cudaSuccess ) {
		cudaGetLastError();
		return;
	}
	stream = s;
	cudaStream_t c = nullptr;
	cudaEvent_t e = nullptr;
	if( cudaStreamCreateWithFlags( &c, cudaStreamNonBlocking ) == cudaSuccess
		&& cudaEventCreateWithFlags( &e, cudaEventDisableTiming ) == cudaSuccess ) {
		copyStream = c;
		copyDone = e;
	} else {
		cudaGetLastError(); // exchanges then all take the compute stream
		if( c != nullptr ) cudaStreamDestroy( c );
	}
	initialized = true;
}

void CB200MathEngine::noteUse( const void* allocationBase ) const
{
	std::lock_guard<std::mutex> lock( useMutex );
	lastUse[allocationBase] = opSeq + 1;
}

bool CB200MathEngine::idleSinceLastDrain( const void* allocationBase ) const
{
	std::lock_guard<std::mutex> lock( useMutex );
	auto it = lastUse.find( allocationBase );
	return it == lastUse.end() || it->second <= completedSeq;
}

void CB200MathEngine::freeBlock( void* block ) const
{
	if( block == nullptr ) return;
	noteUse( block ); // whoever gets the block next must assume queued kernels still read or write it
	memory.Free( block );
}

CB200MathEngine::~CB200MathEngine()
{
	if( stream != nullptr ) {
		cudaSetDevice( device );
		ReleaseDistributedCommunicator(); // first: after an abort only this lets the stream drain
		cudaStreamSynchronize( static_cast<cudaStream_t>( stream ) );
		forgetAllPreparedFilters();
		lazy.clear(); // nobody is left to read a noted result
		for( void* p : deferredFrees ) memory.Free( p );
		if( copyStream != nullptr ) cudaStreamDestroy( static_cast<cudaStream_t>( copyStream ) );
		if( copyDone != nullptr ) cudaEventDestroy( static_cast<cudaEvent_t>( copyDone ) );
		for( auto& b : hostBuffers ) cudaFreeHost( b.host );
		for( auto& b : hostCache ) cudaFreeHost( b.first );
		cudaStreamDestroy( static_cast<cudaStream_t>( stream ) );
	}
}

bool CB200MathEngine::pendingRefersTo( const void* begin, size_t bytes ) const
{
	const char* lo = static_cast<const char*>( begin );
	const char* hi = lo + bytes;
	auto inside = [&]( const void* p ) { return p != nullptr && static_cast<const char*>( p ) >= lo && static_cast<const char*>( p ) < hi; };
	if( pending.active && ( inside( pending.source ) || inside( pending.filter ) || inside( pending.freeTerm )
		|| inside( pending.result ) || inside( pending.residual ) || inside( pending.threshold ) ) ) {
		return true;
	}
	if( pendingRows.active && ( inside( pendingRows.data ) || inside( pendingRows.scale ) || inside( pendingRows.bias ) ) ) return true;
	if( pendingProduct.active && ( inside( pendingProduct.first ) || inside( pendingProduct.second ) || inside( pendingProduct.result ) ) ) {
		return true;
	}
	return pendingGate.active && ( inside( pendingGate.input ) || inside( pendingGate.output ) || inside( pendingGate.scale ) );
}

void CB200MathEngine::releaseDeferredFrees() const
{
	if( deferredFrees.empty() ) return;
	std::vector<void*> work;
	work.swap( deferredFrees ); // what is called below may come back here
	for( void* p : work ) {
		if( pendingRefersTo( p, memory.BlockBytes( p ) ) || lazyReads( p ) ) {
			deferredFrees.push_back( p );
		} else {
			// a noted call may have prepared an operand from this block after its owner released it
			if( !preparedFilters.empty() ) forgetPreparedFilter( p );
			freeBlock( p );
		}
	}
}

//---------------------------------------------------------------------------------------------------------------------
// noted results (see CLazyResult)

bool CB200MathEngine::noteLazy( const CLazyResult& note ) const
{
	if( note.resultBase == nullptr
		|| ( memory.BlockBytes( note.resultBase ) == 0 && memory.StackBlockBytes( note.resultBase ) == 0 ) ) {
		return false;
	}
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	flushRecorded();
	lazy.push_back( note );
	lazyCount.store( static_cast<int>( lazy.size() ), std::memory_order_relaxed );
	return true;
}

void CB200MathEngine::flushRecorded() const
{
	if( !anythingRecorded() ) return;
	cudaSetDevice( device );
	flushPending();
	flushProduct();
	flushRowOps();
	flushGate();
}

// Whoever finds a note is about to extend it, copy it or consume it: nothing stays recorded across that (see
// flushRecorded; launching recorded calls leaves the notes as they are, so the index stays good).
int CB200MathEngine::findLazy( const void* result, CLazyResult::TKind kind ) const
{
	for( size_t i = 0; i < lazy.size(); ++i ) {
		if( lazy[i].result == result && lazy[i].kind == kind ) {
			flushRecorded();
			return static_cast<int>( i );
		}
	}
	return -1;
}

bool CB200MathEngine::lazyReads( const void* allocationBase ) const
{
	for( const CLazyResult& note : lazy ) {
		for( const CLazyResult::CInput& input : note.inputs ) {
			if( input.base == allocationBase ) return true;
		}
	}
	return false;
}

void CB200MathEngine::materializeLazy( size_t index ) const
{
	CB200MathEngine* self = const_cast<CB200MathEngine*>( this );
	const CLazyResult note = lazy[index];
	lazy.erase( lazy.begin() + index );
	lazyCount.store( static_cast<int>( lazy.size() ), std::memory_order_relaxed );
	cudaSetDevice( device );
	// the kernels launched now read and write these allocations, whenever the calls were noted
	noteUse( note.resultBase );
	for( const CLazyResult::CInput& input : note.inputs ) noteUse( input.base );
	if( note.kind == CLazyResult::K_Resize ) {
		check( nb200_blob_resize_image( stream, note.batch, note.h, note.w, note.c, note.left, note.right, note.top, note.bottom,
			0, note.value, note.from, note.result ), "BlobResizeImage" );
	} else if( note.kind == CLazyResult::K_Product ) {
		// the epilogue carries bias, residual and the complete gate; a gate noted in part runs as the calls it was
		check( productWithScratch( 1, note.first, note.rows, note.depth, note.firstRowSize, note.second, note.width,
			note.secondRowSize, note.result, note.width, note.bias, note.residual, note.gate == 3 ? note.gateScale : nullptr,
			note.inputs.size() > 1 ? note.inputs[1].base : nullptr ), "MultiplyMatrixByTransposedMatrix" );
		if( note.gate == 1 || note.gate == 2 ) {
			check( nb200_vector_op( stream, NB200_VEC_MULTIPLY, note.result, nullptr, note.gateScale, 0.f, note.result,
				static_cast<int>( note.resultFloats ) ), "VectorMultiply" );
		}
		if( note.gate == 2 ) {
			check( nb200_vector_op( stream, NB200_VEC_SIGMOID, note.result, nullptr, nullptr, 0.f, note.result,
				static_cast<int>( note.resultFloats ) ), "VectorSigmoid" );
		}
	} else if( note.kind == CLazyResult::K_Affine ) {
		check( nb200_matrix_rows_cols_affine( stream, note.from, note.rows, note.width, note.rowAdd, note.square ? 1 : 0,
			note.rowMul, note.colMul, note.colAdd, note.result ), "AddVectorToMatrixColumns" );
	} else {
		check( self->launchProduct( note.batch, note.first, note.seqQ, note.depth, note.second, note.seqTo, note.result ),
			"MultiplyMatrixByMatrix" );
		const int rows = note.batch * note.seqQ;
		if( note.softmax && note.seqTo <= 1024 && ( note.scale != nullptr || note.mask != nullptr ) ) {
			check( nb200_matrix_softmax_by_rows_fused( stream, note.result, rows, note.seqTo, note.scale, note.mask,
				note.mask != nullptr ? note.seqQ : 0, note.result ), "MatrixSoftmaxByRows" );
		} else {
			if( note.scale != nullptr ) {
				check( nb200_vector_op( stream, NB200_VEC_MULTIPLY, note.result, nullptr, note.scale, 0.f, note.result,
					static_cast<int>( note.resultFloats ) ), "VectorMultiply" );
			}
			if( note.mask != nullptr ) {
				check( nb200_add_vector_to_matrix_rows( stream, 1, note.result, note.result, note.batch, note.seqQ * note.seqTo,
					note.mask ), "AddVectorToMatrixRows" );
			}
			if( note.softmax ) {
				check( nb200_matrix_softmax_by_rows( stream, note.result, rows, note.seqTo, note.result ), "MatrixSoftmaxByRows" );
			}
		}
	}
	releaseDeferredFrees();
}

void CB200MathEngine::materializeAllLazy() const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	while( !lazy.empty() ) materializeLazy( 0 );
}

void CB200MathEngine::touchLazy( const void* allocationBase, const void* from, bool mayWrite ) const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	const char* const start = static_cast<const char*>( from );
	for( ;; ) {
		int hit = -1;
		for( size_t i = 0; i < lazy.size() && hit < 0; ++i ) {
			if( lazy[i].resultBase == allocationBase
				&& start < reinterpret_cast<const char*>( lazy[i].result + lazy[i].resultFloats ) ) {
				hit = static_cast<int>( i );
			}
			for( size_t k = 0; mayWrite && hit < 0 && k < lazy[i].inputs.size(); ++k ) {
				if( lazy[i].inputs[k].base == allocationBase && start < lazy[i].inputs[k].end ) hit = static_cast<int>( i );
			}
		}
		if( hit < 0 ) return;
		materializeLazy( static_cast<size_t>( hit ) );
	}
}

CB200MathEngine::CLazyResult* CB200MathEngine::deriveNote( int sourceNote, const CFloatHandle& resultHandle ) const
{
	const float* const source = lazy[sourceNote].result;
	if( peek( resultHandle ) == source ) return &lazy[sourceNote];
	CLazyResult copy = lazy[sourceNote];
	// A note made in place reads the buffer it will write, and that buffer is not among its inputs: a copy of it for
	// another buffer would read the source before or after the in-place result lands, whichever is touched first.
	if( copy.kind == CLazyResult::K_Affine && copy.from == copy.result ) return nullptr;
	const void* base = CMemoryHandleInternal::Base( resultHandle );
	if( base == copy.resultBase || ( memory.BlockBytes( base ) == 0 && memory.StackBlockBytes( base ) == 0 ) ) return nullptr;
	for( const CLazyResult::CInput& input : copy.inputs ) {
		if( input.base == base ) return nullptr;
	}
	copy.result = raw( resultHandle ); // whatever was noted for that buffer, or reads it, is carried out first
	copy.resultBase = base;
	if( findLazy( source, copy.kind ) < 0 ) return nullptr; // that included the source
	lazy.push_back( copy );
	lazyCount.store( static_cast<int>( lazy.size() ), std::memory_order_relaxed );
	return &lazy.back();
}

bool CB200MathEngine::forgetLazyResultIn( const void* allocationBase ) const
{
	bool any = false;
	for( size_t i = 0; i < lazy.size(); ) {
		if( lazy[i].resultBase == allocationBase ) {
			lazy.erase( lazy.begin() + i );
			any = true;
		} else {
			++i;
		}
	}
	lazyCount.store( static_cast<int>( lazy.size() ), std::memory_order_relaxed );
	return any;
}

void CB200MathEngine::notImplemented( const char* method ) const
{
	raiseAssert( std::string( "CB200MathEngine::" ) + method + " is not implemented: it lies outside the inference hot path "
		"this engine covers, and the engine has no CPU fallback" );
}

void CB200MathEngine::check( int code, const char* method ) const
{
	if( code == NB200_OK ) return;
	std::string msg = std::string( "CB200MathEngine::" ) + method + ": " + nb200_error_string( code );
	if( code == NB200_ELAUNCH || code == NB200_ENODEVICE ) msg += std::string( " (" ) + nb200_last_cuda_error() + ")";
	raiseAssert( msg );
}

void CB200MathEngine::setDevice() const
{
	// any host thread may call any engine (the reference does the same at the top of every method,
	// GPU/CUDA/CudaMathEngineDnnConv.cu:67)
	cudaSetDevice( device );
}

void CB200MathEngine::enter() const
{
	cudaSetDevice( device );
	{
		std::lock_guard<std::mutex> lock( useMutex );
		++opSeq;
	}
	flushPending();
	flushProduct();
	flushRowOps();
	flushGate();
}

float* CB200MathEngine::WorkAlloc( size_t floats ) const
{
	if( floats == 0 ) return nullptr;
	float* p = static_cast<float*>( memory.Alloc( floats * sizeof( float ) ) );
	if( p == nullptr ) GetMathEngineExceptionHandler()->OnMemoryError();
	return p;
}

void CB200MathEngine::WorkFree( float* ptr ) const
{
	freeBlock( ptr );
}

void CB200MathEngine::flushRowOps() const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( !pendingRows.active ) return;
	const CPendingRowOps p = pendingRows;
	pendingRows = CPendingRowOps();
	if( p.scale != nullptr ) {
		check( nb200_vector_op( stream, NB200_VEC_MULTIPLY, p.data, nullptr, p.scale, 0.f, p.data, static_cast<int>( p.size ) ),
			"VectorMultiply" );
	}
	if( p.bias != nullptr ) {
		check( nb200_add_vector_to_matrix_rows( stream, 1, p.data, p.data, p.biasHeight, p.biasWidth, p.bias ),
			"AddVectorToMatrixRows" );
	}
	releaseDeferredFrees();
}

void CB200MathEngine::flushProduct( const float* bias ) const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( !pendingProduct.active ) return;
	const CPendingProduct p = pendingProduct;
	pendingProduct = CPendingProduct();
	check( productWithScratch( 1, p.first, p.firstHeight, p.firstWidth, p.firstRowSize, p.second, p.secondHeight,
		p.secondRowSize, p.result, p.resultRowSize, bias ), "MultiplyMatrixByTransposedMatrix" );
	releaseDeferredFrees();
}

void CB200MathEngine::flushGate() const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( !pendingGate.active ) return;
	const CPendingSigmoidGate g = pendingGate;
	pendingGate = CPendingSigmoidGate();
	check( nb200_vector_op( stream, NB200_VEC_MULTIPLY, g.input, nullptr, g.scale, 0.f, g.output, g.size ), "VectorMultiply" );
	if( g.sigmoid ) {
		check( nb200_vector_op( stream, NB200_VEC_SIGMOID, g.output, nullptr, nullptr, 0.f, g.output, g.size ), "VectorSigmoid" );
	}
	releaseDeferredFrees();
}

void CB200MathEngine::flushPending() const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( !pending.active ) return;
	pending.active = false;
	launchConvolution( pending );
	releaseDeferredFrees();
}

void CB200MathEngine::launchConvolution( const CPendingConvolution& call ) const
{
	nb200_epilogue epi = {};
	epi.bias = call.freeTerm;
	epi.residual = call.residual;
	epi.ld_residual = call.d.k;
	epi.act = call.relu ? NB200_ACT_RELU : NB200_ACT_NONE;
	epi.act_param_device = call.threshold;
	// scratch (prepared filter, widened pixels) comes from the block pool: the stream orders its reuse
	const size_t scratchFloats = nb200_blob_convolution_scratch_floats( &call.d );
	float* scratch = scratchFloats > 0 ? static_cast<float*>( memory.Alloc( scratchFloats * sizeof( float ) ) ) : nullptr;
	const int rc = nb200_blob_convolution_with_prepared_filter( stream, &call.d, call.source, call.filter,
		preparedFilterFor( call ), call.result, scratch, &epi, precision );
	freeBlock( scratch );
	check( rc, "BlobConvolution" );
}

// The prepared form of the call's filter: made on first use, then found by the filter's allocation.
const float* CB200MathEngine::preparedFilterFor( const CPendingConvolution& call ) const
{
	if( call.filterAllocation == nullptr ) return nullptr;
	const size_t floats = nb200_blob_convolution_prepared_filter_floats( &call.d );
	if( floats == 0 ) return nullptr;
	std::lock_guard<std::mutex> lock( preparedMutex );
	auto it = preparedFilters.find( call.filterAllocation );
	if( it != preparedFilters.end() ) {
		const CPreparedFilter& f = it->second;
		if( f.filter == call.filter && f.k == call.d.k && f.r == call.d.r && f.s == call.d.s && f.c == call.d.c ) return f.data;
		freeBlock( f.data ); // the allocation now serves another filter shape
		preparedFilters.erase( it );
	}
	CPreparedFilter f;
	f.filter = call.filter;
	f.k = call.d.k; f.r = call.d.r; f.s = call.d.s; f.c = call.d.c;
	f.data = static_cast<float*>( memory.Alloc( floats * sizeof( float ) ) );
	if( f.data == nullptr ) return nullptr; // no room: the call prepares into its scratch as before
	if( nb200_blob_convolution_prepare_filter( stream, &call.d, call.filter, f.data, precision ) != NB200_OK ) {
		memory.Free( f.data );
		return nullptr;
	}
	preparedFilters.emplace( call.filterAllocation, f );
	return f.data;
}

const float* CB200MathEngine::preparedSecondFor( const void* allocationBase, const float* second, int rows, int secondHeight,
	int depth, int secondRowSize ) const
{
	if( allocationBase == nullptr || memory.BlockBytes( allocationBase ) == 0 ) return nullptr; // end of life not seen
	const size_t floats = nb200_matrix_product_prepared_floats( rows, secondHeight, depth, secondRowSize );
	if( floats == 0 ) return nullptr;
	std::lock_guard<std::mutex> lock( preparedMutex );
	auto it = preparedFilters.find( allocationBase );
	if( it != preparedFilters.end() ) {
		const CPreparedFilter& f = it->second;
		if( f.filter == second && f.k == secondHeight && f.r == -1 && f.s == secondRowSize && f.c == depth ) return f.data;
		freeBlock( f.data ); // the allocation now serves another operand
		preparedFilters.erase( it );
	}
	CPreparedFilter f;
	f.filter = second;
	f.k = secondHeight; f.r = -1; f.s = secondRowSize; f.c = depth; // r = -1 marks a matrix operand
	f.data = static_cast<float*>( memory.Alloc( floats * sizeof( float ) ) );
	if( f.data == nullptr ) return nullptr; // no room: the call prepares into its scratch as before
	if( nb200_matrix_product_prepare_second( stream, second, secondHeight, depth, secondRowSize, f.data, precision ) != NB200_OK ) {
		memory.Free( f.data );
		return nullptr;
	}
	preparedFilters.emplace( allocationBase, f );
	return f.data;
}

void CB200MathEngine::forgetPreparedFilter( const void* allocationBase ) const
{
	{
		// a recorded convolution that is about to use the prepared form is launched first, with the old contents
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		if( pending.active && pending.filterAllocation == allocationBase ) {
			cudaSetDevice( device );
			flushPending();
		}
	}
	std::lock_guard<std::mutex> lock( preparedMutex );
	auto it = preparedFilters.find( allocationBase );
	if( it == preparedFilters.end() ) return;
	// a recorded convolution may still be about to use it: launch that first (the stream then orders the reuse)
	float* data = it->second.data;
	preparedFilters.erase( it );
	freeBlock( data );
}

void CB200MathEngine::forgetAllPreparedFilters() const
{
	std::lock_guard<std::mutex> lock( preparedMutex );
	for( auto& kv : preparedFilters ) freeBlock( kv.second.data );
	preparedFilters.clear();
}

// True when `call` neither reads what the recorded convolution writes nor writes anything the recorded one reads or
// writes: the two may then run in either order.  A residual block's projection shortcut arrives between the block's
// last convolution and the sum that joins them; launching it at once keeps that last convolution recorded, so the sum
// and the ReLU behind it still ride in its epilogue.
bool CB200MathEngine::independentOfPending( const CPendingConvolution& call ) const
{
	auto overlap = []( const float* a, long long na, const float* b, long long nb ) {
		return a != nullptr && b != nullptr && a < b + nb && b < a + na;
	};
	const CPendingConvolution& p = pending;
	if( p.relu || p.residual != nullptr ) return false;
	// what the new call writes against everything the recorded one touches
	if( overlap( call.result, call.resultFloats, p.result, p.resultFloats ) || overlap( call.result, call.resultFloats, p.source, p.sourceFloats )
		|| overlap( call.result, call.resultFloats, p.filter, p.filterFloats ) || overlap( call.result, call.resultFloats, p.freeTerm, p.d.k ) ) {
		return false;
	}
	// what the new call reads against what the recorded one writes
	return !overlap( call.source, call.sourceFloats, p.result, p.resultFloats ) && !overlap( call.filter, call.filterFloats, p.result, p.resultFloats )
		&& !overlap( call.freeTerm, call.d.k, p.result, p.resultFloats );
}

bool CB200MathEngine::fuseReLU( const float* first, float* result, int size, const float* thresholdOnDevice ) const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( !pending.active || pending.relu || first != pending.result || result != pending.result
		|| size != pending.resultFloats ) {
		return false;
	}
	pending.relu = true;
	pending.threshold = thresholdOnDevice;
	cudaSetDevice( device );
	flushPending(); // nothing fuses behind the activation, and the threshold is read while it certainly still exists
	return true;
}

bool CB200MathEngine::fuseAdd( const float* first, const float* second, float* result, int size ) const
{
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( !pending.active || pending.relu || pending.residual != nullptr || result != pending.result
		|| size != pending.resultFloats || ( first != pending.result && second != pending.result ) || first == second ) {
		return false;
	}
	pending.residual = first == pending.result ? second : first;
	return true;
}

//---------------------------------------------------------------------------------------------------------------------
// identity

TMathEngineType CB200MathEngine::GetType() const { return MET_Cuda; }

void CB200MathEngine::GetMathEngineInfo( CMathEngineInfo& info ) const
{
	info = CMathEngineInfo( MET_Cuda, 0, device );
	cudaDeviceProp prop;
	if( cudaGetDeviceProperties( &prop, device ) == cudaSuccess ) {
		std::snprintf( info.Name, sizeof( info.Name ), "%s (B200 engine)", prop.name );
		info.AvailableMemory = prop.totalGlobalMem;
	} else {
		cudaGetLastError();
	}
}

bool CB200MathEngine::IsInitialized() const { return initialized; }

//---------------------------------------------------------------------------------------------------------------------
// memory

void CB200MathEngine::SetReuseMemoryMode( bool ) {} // blocks are always recycled on this engine
bool CB200MathEngine::GetReuseMemoryMode() const { return true; }
void CB200MathEngine::SetThreadBufferMemoryThreshold( size_t ) {}
size_t CB200MathEngine::GetThreadBufferMemoryThreshold() const { return 0; }

CMemoryHandle CB200MathEngine::HeapAlloc( size_t count )
{
	setDevice();
	void* p = memory.Alloc( count );
	if( p == nullptr ) {
		GetMathEngineExceptionHandler()->OnMemoryError();
		return CMemoryHandle();
	}
	return CMemoryHandleInternal::Create( this, p );
}

void CB200MathEngine::HeapFree( const CMemoryHandle& handle )
{
	if( handle.IsNull() ) return;
	if( handle.GetMathEngine() != this ) { raiseAssert( "HeapFree: the handle belongs to another math engine" ); return; }
	void* block = const_cast<void*>( CMemoryHandleInternal::Base( handle ) );
	if( !preparedFilters.empty() ) forgetPreparedFilter( block );
	{
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const bool forgot = !lazy.empty() && forgetLazyResultIn( block ); // nobody can read the noted result any more
		if( ( anythingRecorded() && pendingRefersTo( block, memory.BlockBytes( block ) ) )
			|| ( !lazy.empty() && lazyReads( block ) ) ) {
			deferredFrees.push_back( block ); // returned to the pool once the recorded call has been launched
			return;
		}
		if( forgot ) releaseDeferredFrees();
	}
	freeBlock( block );
}

void CB200MathEngine::TransferHandleToThisThread( const CMemoryHandle&, size_t ) {} // heap blocks are not thread-bound here

CMemoryHandle CB200MathEngine::StackAlloc( size_t count )
{
	setDevice();
	void* p = memory.StackAlloc( count );
	if( p == nullptr ) {
		GetMathEngineExceptionHandler()->OnMemoryError();
		return CMemoryHandle();
	}
	return CMemoryHandleInternal::Create( this, p );
}

void CB200MathEngine::StackFree( const CMemoryHandle& handle )
{
	if( handle.IsNull() ) return;
	{
		// a recorded call may read a stack variable (NeoML keeps scalars such as a multiplier there): launch it before
		// the variable's memory can be handed out again; the stack is LIFO, so the free itself cannot be postponed
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		if( anythingRecorded() ) enter();
		if( !lazy.empty() ) {
			forgetLazyResultIn( CMemoryHandleInternal::Base( handle ) ); // nobody can read a noted result in this variable any more
			touchLazy( CMemoryHandleInternal::Base( handle ), CMemoryHandleInternal::Base( handle ), true ); // what reads the variable is carried out now
		}
	}
	if( !preparedFilters.empty() ) forgetPreparedFilter( CMemoryHandleInternal::Base( handle ) );
	memory.StackFree( CMemoryHandleInternal::GetRaw( handle ) );
}

size_t CB200MathEngine::GetFreeMemorySize() const { return memory.FreeOnDevice(); }
size_t CB200MathEngine::GetPeakMemoryUsage() const { return memory.Peak(); }
void CB200MathEngine::ResetPeakMemoryUsage() { memory.ResetPeak(); }
size_t CB200MathEngine::GetCurrentMemoryUsage() const { return memory.Current(); }
size_t CB200MathEngine::GetMemoryInPools() const { return memory.InPools(); }

void CB200MathEngine::CleanUp()
{
	enter();
	materializeAllLazy();
	if( stream != nullptr ) cudaStreamSynchronize( static_cast<cudaStream_t>( stream ) );
	forgetAllPreparedFilters();
	memory.CleanUp();
}

void CB200MathEngine::CleanUpSpecial() {}

//---------------------------------------------------------------------------------------------------------------------
// exchange

void CB200MathEngine::DataExchangeRaw( const CMemoryHandle& result, const void* source, size_t size )
{
	if( size == 0 ) return;
	if( result.GetMathEngine() != this ) { raiseAssert( "DataExchangeRaw: the handle belongs to another math engine" ); return; }
	enter();
	const void* base = CMemoryHandleInternal::Base( result );
	if( lazyCount.load( std::memory_order_relaxed ) != 0 ) touchLazy( base, CMemoryHandleInternal::GetRaw( result ), true );
	if( !preparedFilters.empty() ) forgetPreparedFilter( base ); // after whatever still needed the old contents has run
	cudaStream_t s = static_cast<cudaStream_t>( stream );
	void* const destination = CMemoryHandleInternal::GetRaw( result );
	// A large exchange into a heap block that nothing queued can touch overlaps the kernels in flight (see noteUse)
	if( copyStream != nullptr && size >= ( size_t( 1 ) << 20 ) && memory.BlockBytes( base ) > 0 && idleSinceLastDrain( base ) ) {
		cudaStream_t c = static_cast<cudaStream_t>( copyStream );
		cudaEvent_t done = static_cast<cudaEvent_t>( copyDone );
		std::lock_guard<std::mutex> lock( hostMutex ); // one copy at a time owns the event
		if( cudaMemcpyAsync( destination, source, size, cudaMemcpyHostToDevice, c ) != cudaSuccess
			|| cudaEventRecord( done, c ) != cudaSuccess || cudaStreamWaitEvent( s, done, 0 ) != cudaSuccess
			|| cudaStreamSynchronize( c ) != cudaSuccess ) {
			raiseAssert( std::string( "DataExchangeRaw host->device: " ) + cudaGetErrorString( cudaGetLastError() ) );
		}
		noteUse( base );
		return;
	}
	if( cudaMemcpyAsync( destination, source, size, cudaMemcpyHostToDevice, s ) != cudaSuccess
		|| cudaStreamSynchronize( s ) != cudaSuccess ) {
		raiseAssert( std::string( "DataExchangeRaw host->device: " ) + cudaGetErrorString( cudaGetLastError() ) );
	}
	std::lock_guard<std::mutex> lock( useMutex );
	completedSeq = opSeq; // the compute stream has drained
}

void CB200MathEngine::DataExchangeRaw( void* result, const CMemoryHandle& source, size_t size )
{
	if( size == 0 ) return;
	if( source.GetMathEngine() != this ) { raiseAssert( "DataExchangeRaw: the handle belongs to another math engine" ); return; }
	enter();
	if( lazyCount.load( std::memory_order_relaxed ) != 0 ) touchLazy( CMemoryHandleInternal::Base( source ), CMemoryHandleInternal::GetRaw( source ), false );
	cudaStream_t s = static_cast<cudaStream_t>( stream );
	if( cudaMemcpyAsync( result, CMemoryHandleInternal::GetRaw( source ), size, cudaMemcpyDeviceToHost, s ) != cudaSuccess
		|| cudaStreamSynchronize( s ) != cudaSuccess ) {
		raiseAssert( std::string( "DataExchangeRaw device->host: " ) + cudaGetErrorString( cudaGetLastError() ) );
	}
	{
		std::lock_guard<std::mutex> lock( useMutex );
		completedSeq = opSeq; // the compute stream has drained
	}
	// a kernel that gave up on a bounded wait leaves its mark in the status word: surface it at the first sync point
	const int status = nb200_device_status( stream, 1 );
	if( status > 0 ) raiseAssert( "a B200 kernel reported a bounded-wait timeout (status " + std::to_string( status ) + ")" );
}

void* CB200MathEngine::GetBuffer( const CMemoryHandle& handle, size_t pos, size_t size, bool exchange )
{
	setDevice();
	size_t capacity = 0;
	void* host = takeHostBuffer( size, capacity );
	if( host == nullptr ) {
		GetMathEngineExceptionHandler()->OnMemoryError();
		return nullptr;
	}
	if( exchange && size > 0 ) {
		const CMemoryHandle at = CMemoryHandleInternal::Create( this,
			static_cast<const char*>( CMemoryHandleInternal::GetRaw( handle ) ) + pos );
		DataExchangeRaw( host, at, size );
	}
	std::lock_guard<std::mutex> lock( hostMutex );
	hostBuffers.push_back( { host, size, capacity, handle, pos } );
	return host;
}

// Pinned staging memory in power-of-two sizes; released buffers are cached (at most 256 MB in total) and reused.
void* CB200MathEngine::takeHostBuffer( size_t size, size_t& capacity )
{
	capacity = 4096;
	while( capacity < size ) capacity *= 2;
	{
		std::lock_guard<std::mutex> lock( hostMutex );
		for( size_t i = 0; i < hostCache.size(); ++i ) {
			if( hostCache[i].second == capacity ) {
				void* host = hostCache[i].first;
				hostCacheBytes -= capacity;
				hostCache.erase( hostCache.begin() + i );
				return host;
			}
		}
	}
	void* host = nullptr;
	if( cudaMallocHost( &host, capacity ) != cudaSuccess ) {
		cudaGetLastError();
		return nullptr;
	}
	return host;
}

void CB200MathEngine::keepHostBuffer( void* host, size_t capacity )
{
	{
		std::lock_guard<std::mutex> lock( hostMutex );
		if( hostCacheBytes + capacity <= ( size_t( 256 ) << 20 ) ) {
			hostCache.emplace_back( host, capacity );
			hostCacheBytes += capacity;
			return;
		}
	}
	setDevice();
	cudaFreeHost( host );
}

void CB200MathEngine::ReleaseBuffer( const CMemoryHandle& handle, void* ptr, bool exchange )
{
	CHostBuffer buf{};
	{
		std::lock_guard<std::mutex> lock( hostMutex );
		if( hostBuffers.empty() || hostBuffers.back().host != ptr ) { raiseAssert( "ReleaseBuffer: buffers are released in LIFO order" ); return; }
		buf = hostBuffers.back();
		hostBuffers.pop_back();
	}
	if( exchange && buf.size > 0 ) {
		if( !preparedFilters.empty() ) forgetPreparedFilter( CMemoryHandleInternal::Base( handle ) );
		const CMemoryHandle at = CMemoryHandleInternal::Create( this,
			static_cast<const char*>( CMemoryHandleInternal::GetRaw( handle ) ) + buf.pos );
		DataExchangeRaw( at, ptr, buf.size );
	}
	keepHostBuffer( ptr, buf.capacity );
}

CMemoryHandle CB200MathEngine::CopyFrom( const CMemoryHandle& handle, size_t size )
{
	CMemoryHandle result = HeapAlloc( size );
	if( result.IsNull() || size == 0 ) return result;
	IMathEngine* other = handle.GetMathEngine();
	if( other == this ) {
		enter();
		if( lazyCount.load( std::memory_order_relaxed ) != 0 ) touchLazy( CMemoryHandleInternal::Base( handle ), CMemoryHandleInternal::GetRaw( handle ), false );
		noteUse( CMemoryHandleInternal::Base( result ) );
		noteUse( CMemoryHandleInternal::Base( handle ) );
		cudaMemcpyAsync( CMemoryHandleInternal::GetRaw( result ), CMemoryHandleInternal::GetRaw( handle ), size,
			cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>( stream ) );
		return result;
	}
	// through the host, like the reference (MemoryEngineMixin.cpp:218-226)
	std::vector<char> staging( size );
	other->DataExchangeRaw( staging.data(), handle, size );
	DataExchangeRaw( result, staging.data(), size );
	return result;
}

IPerformanceCounters* CB200MathEngine::CreatePerformanceCounters( bool ) const
{
	return new CB200PerformanceCounters( device, stream );
}

//---------------------------------------------------------------------------------------------------------------------
// factory

IMathEngine* CreateB200MathEngine( int deviceIndex, size_t memoryLimit, int flags )
{
	if( nb200_device_count() <= 0 ) return nullptr; // like CreateGpuMathEngine: null when no usable GPU exists
	int count = 0;
	if( cudaGetDeviceCount( &count ) != cudaSuccess ) { cudaGetLastError(); return nullptr; }
	if( deviceIndex < 0 ) deviceIndex = 0;
	if( deviceIndex >= count ) return nullptr;
	CB200MathEngine* engine = new CB200MathEngine( deviceIndex, memoryLimit, flags );
	if( !engine->IsInitialized() ) {
		delete engine;
		return nullptr;
	}
	return engine;
}

// The sm_100 devices as the reference's GPU manager lists them: every entry is MET_Cuda, Id = CUDA device index,
// AvailableMemory = the device's total memory (what the reference reports too, GPU/CUDA/CudaDevice.cpp).
class CB200MathEngineManager : public IGpuMathEngineManager {
public:
	CB200MathEngineManager()
	{
		int count = 0;
		if( nb200_device_count() <= 0 || cudaGetDeviceCount( &count ) != cudaSuccess ) { cudaGetLastError(); return; }
		for( int i = 0; i < count; ++i ) {
			cudaDeviceProp prop;
			if( cudaGetDeviceProperties( &prop, i ) != cudaSuccess ) { cudaGetLastError(); continue; }
			if( prop.major != 10 ) continue;
			CMathEngineInfo info( MET_Cuda, prop.totalGlobalMem, i );
			std::snprintf( info.Name, sizeof( info.Name ), "%s", prop.name );
			devices.push_back( info );
		}
	}

	int GetMathEngineCount() const override { return static_cast<int>( devices.size() ); }

	void GetMathEngineInfo( int index, CMathEngineInfo& info ) const override
	{
		info = index >= 0 && index < GetMathEngineCount() ? devices[index] : CMathEngineInfo();
	}

	IMathEngine* CreateMathEngine( int index, size_t memoryLimit, int flags ) const override
	{
		if( devices.empty() || index >= GetMathEngineCount() ) return nullptr;
		return CreateB200MathEngine( devices[index >= 0 ? index : 0].Id, memoryLimit, flags );
	}

private:
	std::vector<CMathEngineInfo> devices;
};

IGpuMathEngineManager* CreateB200MathEngineManager()
{
	return new CB200MathEngineManager();
}

} // namespace NeoML

// C entry points for hosts that load the engine library dynamically (ctypes, dlopen)
extern "C" __attribute__((visibility("default"))) void* nb200_create_math_engine_manager()
{
	return NeoML::CreateB200MathEngineManager();
}

// Devices the manager lists; with engine != NULL also creates an engine on entry `index` through the manager.
extern "C" __attribute__((visibility("default"))) int nb200_manager_probe( void* manager, int index, void** engine,
	unsigned long long* memory, char* name, int nameSize )
{
	NeoML::IGpuMathEngineManager* m = static_cast<NeoML::IGpuMathEngineManager*>( manager );
	const int count = m->GetMathEngineCount();
	if( index >= 0 && index < count ) {
		NeoML::CMathEngineInfo info;
		m->GetMathEngineInfo( index, info );
		if( memory != nullptr ) *memory = info.AvailableMemory;
		if( name != nullptr && nameSize > 0 ) std::snprintf( name, nameSize, "%s", info.Name );
		if( engine != nullptr ) *engine = m->CreateMathEngine( index, 0, 0 );
	}
	return count;
}

extern "C" __attribute__((visibility("default"))) void nb200_destroy_math_engine_manager( void* manager )
{
	delete static_cast<NeoML::IGpuMathEngineManager*>( manager );
}

extern "C" __attribute__((visibility("default"))) void* nb200_create_math_engine( int device, size_t memoryLimit, int flags )
{
	return NeoML::CreateB200MathEngine( device, memoryLimit, flags );
}

// The CUDA stream an engine made by this library enqueues its work on (NULL for any other IMathEngine): lets a host
// bracket engine calls with its own events.
extern "C" __attribute__((visibility("default"))) void* nb200_engine_stream( void* engine )
{
	NeoML::CB200MathEngine* e = dynamic_cast<NeoML::CB200MathEngine*>( static_cast<NeoML::IMathEngine*>( engine ) );
	if( e == nullptr ) return nullptr;
	e->Enter(); // a recorded call is launched, so that an event recorded next lies behind all work issued so far
	return e->Stream();
}

extern "C" __attribute__((visibility("default"))) void nb200_destroy_math_engine( void* engine )
{
	delete static_cast<NeoML::IMathEngine*>( engine );
}
