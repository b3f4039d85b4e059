// Distributed part of the engine API: CreateDistributedB200MathEngines, AllReduce (mean), Broadcast, AbortDistributed.
// Semantics follow the reference's NCCL communicator (NeoMathEngine/src/GPU/CUDA/CudaMathEngineDnnDistributed.cpp:39-115):
// one communicator per engine inside one process, AllReduce is an in-place fp32 AVERAGE, Broadcast sends from `root`.
// The collectives run on the engine's own stream, so they are ordered with its kernels, and the call returns after the
// stream has drained.  Inference is batch-sharded and uses none of this; the calls exist for the distributed-engine API.
// NCCL is opened with dlopen when the first distributed engine is created (the reference does the same, NcclDll.cpp:17-55),
// so a process that never distributes does not load it.
#include "B200MathEngine.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <atomic>
#include <chrono>
#include <memory>
#include <string>
#include <vector>

namespace NeoML {

namespace {

typedef struct ncclComm* ncclComm_t;
enum { ncclSuccessCode = 0, ncclInProgressCode = 7 };
enum { ncclFloat32 = 7 };
enum { ncclSumOp = 0, ncclAvgOp = 4 };

struct CNccl {
	int ( *CommInitAll )( ncclComm_t*, int, const int* ) = nullptr;
	int ( *CommDestroy )( ncclComm_t ) = nullptr;
	int ( *CommAbort )( ncclComm_t ) = nullptr;
	int ( *AllReduce )( const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t ) = nullptr;
	int ( *Bcast )( const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t ) = nullptr;
	int ( *CommGetAsyncError )( ncclComm_t, int* ) = nullptr;
	void* lib = nullptr;

	bool Load()
	{
		if( lib != nullptr ) return true;
		lib = dlopen( "libnccl.so.2", RTLD_NOW | RTLD_LOCAL );
		if( lib == nullptr ) lib = dlopen( "libnccl.so", RTLD_NOW | RTLD_LOCAL );
		if( lib == nullptr ) return false;
		CommInitAll = reinterpret_cast<decltype( CommInitAll )>( dlsym( lib, "ncclCommInitAll" ) );
		CommDestroy = reinterpret_cast<decltype( CommDestroy )>( dlsym( lib, "ncclCommDestroy" ) );
		CommAbort = reinterpret_cast<decltype( CommAbort )>( dlsym( lib, "ncclCommAbort" ) );
		AllReduce = reinterpret_cast<decltype( AllReduce )>( dlsym( lib, "ncclAllReduce" ) );
		Bcast = reinterpret_cast<decltype( Bcast )>( dlsym( lib, "ncclBroadcast" ) );
		CommGetAsyncError = reinterpret_cast<decltype( CommGetAsyncError )>( dlsym( lib, "ncclCommGetAsyncError" ) );
		return CommInitAll && CommDestroy && CommAbort && AllReduce && Bcast && CommGetAsyncError;
	}
};

CNccl g_nccl;

// shared by the engines of one distributed group: raised by AbortDistributed, seen by every waiting peer
struct CGroupState {
	std::atomic<bool> aborted{ false };
};

struct CCommHolder {
	ncclComm_t comm;
	std::shared_ptr<CGroupState> group;
	std::atomic<bool> commAborted{ false }; // this engine's own communicator has been given to ncclCommAbort

	CCommHolder( ncclComm_t c, std::shared_ptr<CGroupState> g ) : comm( c ), group( std::move( g ) ) {}
	// ends whatever this communicator still has in flight (a collective its peers never joined) -- once
	void AbortOwn();
};

void CCommHolder::AbortOwn()
{
	if( !commAborted.exchange( true ) ) g_nccl.CommAbort( comm );
}

void raise( const std::string& message )
{
	GetMathEngineExceptionHandler()->OnAssert( message.c_str(), L"B200Distributed", 0, 0 );
}

// Waits for the stream like the reference's ncclStreamSynchronize: polls the stream, the communicator's async error
// and the group's abort flag, so a peer that failed on the host cannot leave this rank waiting forever; a peer that
// never arrives at all is given two minutes, after which the communicator is aborted.
void waitCollective( cudaStream_t stream, CCommHolder* holder )
{
	const auto start = std::chrono::steady_clock::now();
	while( true ) {
		const cudaError_t q = cudaStreamQuery( stream );
		if( q == cudaSuccess ) return;
		if( q != cudaErrorNotReady ) { cudaGetLastError(); raise( "collective failed on the stream" ); return; }
		int asyncError = ncclSuccessCode;
		g_nccl.CommGetAsyncError( holder->comm, &asyncError );
		if( asyncError != ncclSuccessCode && asyncError != ncclInProgressCode ) { raise( "NCCL reported an asynchronous error" ); return; }
		if( holder->group->aborted.load() ) {
			holder->AbortOwn(); // the collective on this stream will never complete: take it off the device
			raise( "Stopping due to error in another thread." );
			return;
		}
		if( std::chrono::steady_clock::now() - start > std::chrono::seconds( 120 ) ) {
			holder->group->aborted.store( true );
			holder->AbortOwn();
			raise( "collective timed out: a peer did not join within two minutes" );
			return;
		}
	}
}

} // namespace

void CB200MathEngine::SetDistributedCommunicator( void* holder, const CMathEngineDistributedInfo& info )
{
	comm = holder;
	distributedInfo = info;
}

void CB200MathEngine::ReleaseDistributedCommunicator()
{
	if( comm == nullptr ) return;
	CCommHolder* holder = static_cast<CCommHolder*>( comm );
	comm = nullptr;
	// ncclCommDestroy waits for the communicator's outstanding work: after an abort there may be work that never ends
	if( holder->group->aborted.load() ) holder->AbortOwn(); else g_nccl.CommDestroy( holder->comm );
	delete holder;
}

void CB200MathEngine::AllReduce( const CFloatHandle& handle, int size )
{
	if( comm == nullptr ) return; // a single engine is its own average
	CCommHolder* holder = static_cast<CCommHolder*>( comm );
	enter();
	// a peer that has given up will not join: nothing is launched for it to be waited for
	if( holder->group->aborted.load() ) { raise( "Stopping due to error in another thread." ); return; }
	float* data = raw( handle );
	cudaStream_t s = static_cast<cudaStream_t>( stream );
	if( g_nccl.AllReduce( data, data, static_cast<size_t>( size ), ncclFloat32, ncclAvgOp, holder->comm, s ) != ncclSuccessCode ) {
		raise( "ncclAllReduce failed" );
		return;
	}
	waitCollective( s, holder );
}

void CB200MathEngine::Broadcast( const CFloatHandle& handle, int size, int root )
{
	if( comm == nullptr ) return;
	CCommHolder* holder = static_cast<CCommHolder*>( comm );
	enter();
	if( holder->group->aborted.load() ) { raise( "Stopping due to error in another thread." ); return; }
	float* data = raw( handle );
	cudaStream_t s = static_cast<cudaStream_t>( stream );
	if( g_nccl.Bcast( data, data, static_cast<size_t>( size ), ncclFloat32, root, holder->comm, s ) != ncclSuccessCode ) {
		raise( "ncclBroadcast failed" );
		return;
	}
	waitCollective( s, holder );
}

void CB200MathEngine::AbortDistributed()
{
	if( comm == nullptr ) return;
	CCommHolder* holder = static_cast<CCommHolder*>( comm );
	// The flag reaches every peer: each polls it while it waits for a collective (waitCollective), aborts its own
	// communicator and gives up with the reference's message.  This engine's communicator is aborted here.
	holder->group->aborted.store( true );
	holder->AbortOwn();
}

void CreateDistributedB200MathEngines( IMathEngine** mathEngines, int devsCount, const int* cudaDevs, size_t memoryLimit )
{
	for( int i = 0; i < devsCount; ++i ) mathEngines[i] = nullptr;
	if( devsCount <= 0 ) return;
	if( !g_nccl.Load() ) { raise( "libnccl.so.2 could not be loaded" ); return; }
	std::vector<ncclComm_t> comms( devsCount );
	if( g_nccl.CommInitAll( comms.data(), devsCount, cudaDevs ) != ncclSuccessCode ) { raise( "ncclCommInitAll failed" ); return; }
	std::shared_ptr<CGroupState> group = std::make_shared<CGroupState>();
	for( int i = 0; i < devsCount; ++i ) {
		CB200MathEngine* engine = static_cast<CB200MathEngine*>( CreateB200MathEngine( cudaDevs[i], memoryLimit, 0 ) );
		if( engine == nullptr ) {
			// nothing half-made is left behind: the engines made so far own (and destroy) their communicators
			for( int j = 0; j < i; ++j ) { delete mathEngines[j]; mathEngines[j] = nullptr; }
			for( int j = i; j < devsCount; ++j ) g_nccl.CommDestroy( comms[j] );
			raise( "a distributed B200 engine could not be created" );
			return;
		}
		engine->SetDistributedCommunicator( new CCommHolder( comms[i], group ), CMathEngineDistributedInfo( i, devsCount ) );
		mathEngines[i] = engine;
	}
}

} // namespace NeoML

extern "C" __attribute__((visibility("default"))) int nb200_create_distributed_math_engines( void** engines, int count,
	const int* devices, size_t memoryLimit )
{
	NeoML::CreateDistributedB200MathEngines( reinterpret_cast<NeoML::IMathEngine**>( engines ), count, devices, memoryLimit );
	for( int i = 0; i < count; ++i ) if( engines[i] == nullptr ) return -1;
	return 0;
}

// C entry points for hosts that hold plain device pointers: the collective methods of the engine made on memory the
// caller owns.  Each engine's call comes from its own host thread (the calls are collective), 0 = done.
extern "C" __attribute__((visibility("default"))) int nb200_engine_all_reduce( void* engine, float* data, int size )
{
	NeoML::IMathEngine* e = static_cast<NeoML::IMathEngine*>( engine );
	try {
		e->AllReduce( NeoML::CFloatHandle( NeoML::CMemoryHandleInternal::Create( e, data ) ), size );
	} catch( ... ) {
		return -1;
	}
	return 0;
}

extern "C" __attribute__((visibility("default"))) int nb200_engine_broadcast( void* engine, float* data, int size, int root )
{
	NeoML::IMathEngine* e = static_cast<NeoML::IMathEngine*>( engine );
	try {
		e->Broadcast( NeoML::CFloatHandle( NeoML::CMemoryHandleInternal::Create( e, data ) ), size, root );
	} catch( ... ) {
		return -1;
	}
	return 0;
}
