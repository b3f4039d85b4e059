// The factory translation unit of a libNeoMathEngine.so whose GPU engine is CB200MathEngine.
//
// It takes the place of NeoMathEngine/src/MathEngine.cpp when the library is built from a NeoML checkout together
// with this repository's engine (Makefile of this directory), and defines everything that file defines:
//   - the out-of-line destructors that anchor the vtables of the interface and descriptor classes,
//   - the process-wide exception handler (NeoMathEngineException.h:28-46; default: std::logic_error / std::bad_alloc),
//   - CreateCpuMathEngine: NeoML's own CPU engine, untouched (MathEngine.cpp:224-237),
//   - CreateGpuMathEngine, CreateGpuMathEngineManager, CreateDistributedCudaMathEngines
//     (NeoMathEngine.h:1282,1305,1311; MathEngine.cpp:137-185,242-266): the B200 engine.
// With it NeoML itself (CDnn, CDistributedTraining, the language wrappers) reaches the B200 engine through the calls it
// already makes; nothing in NeoML is changed.
#include <common.h>

#include <NeoMathEngine/NeoMathEngine.h>
#include <CpuMathEngine.h>

#include "B200MathEngine.h"

#include <atomic>
#include <new>
#include <stdexcept>

namespace NeoML {

// ---- vtable anchors -------------------------------------------------------------------------------------------------
#define NB200_ANCHOR( Class ) Class::~Class() = default;
NB200_ANCHOR( IVectorMathEngine )
NB200_ANCHOR( IBlasEngine )
NB200_ANCHOR( IDnnEngine )
NB200_ANCHOR( IMathEngine )
NB200_ANCHOR( IMathEngineExceptionHandler )
NB200_ANCHOR( IGpuMathEngineManager )
NB200_ANCHOR( IThreadPool )
NB200_ANCHOR( CConvolutionDesc )
NB200_ANCHOR( C3dConvolutionDesc )
NB200_ANCHOR( CTimeConvolutionDesc )
NB200_ANCHOR( CRleConvolutionDesc )
NB200_ANCHOR( CChannelwiseConvolutionDesc )
NB200_ANCHOR( CMaxPoolingDesc )
NB200_ANCHOR( CMeanPoolingDesc )
NB200_ANCHOR( C3dMaxPoolingDesc )
NB200_ANCHOR( C3dMeanPoolingDesc )
NB200_ANCHOR( CGlobalMaxPoolingDesc )
NB200_ANCHOR( CMaxOverTimePoolingDesc )
NB200_ANCHOR( CGlobalMaxOverTimePoolingDesc )
NB200_ANCHOR( CDropoutDesc )
NB200_ANCHOR( CLrnDesc )
NB200_ANCHOR( CLstmDesc )
NB200_ANCHOR( CRowwiseOperationDesc )
#undef NB200_ANCHOR

// ---- exception handler ----------------------------------------------------------------------------------------------
namespace {

struct CThrowingHandler : IMathEngineExceptionHandler {
	void OnAssert( const char* message, const wchar_t*, int, int ) override { throw std::logic_error( message ); }
	void OnMemoryError() override { throw std::bad_alloc(); }
};

IMathEngineExceptionHandler* throwingHandler()
{
	static CThrowingHandler handler;
	return &handler;
}

std::atomic<IMathEngineExceptionHandler*> installedHandler{ nullptr };

} // namespace

void SetMathEngineExceptionHandler( IMathEngineExceptionHandler* handler )
{
	installedHandler.store( handler );
}

IMathEngineExceptionHandler* GetMathEngineExceptionHandler()
{
	IMathEngineExceptionHandler* handler = installedHandler.load();
	return handler != nullptr ? handler : throwingHandler();
}

// ---- CPU engine: NeoML's own ----------------------------------------------------------------------------------------
IMathEngine* CreateCpuMathEngine( size_t memoryLimit )
{
	IMathEngine* engine = new CCpuMathEngine( memoryLimit );
	ASSERT_EXPR( engine->IsInitialized() );
	return engine;
}

IMathEngine* CreateCpuMathEngine( int /*threadCount, ignored since NeoML 2.0*/, size_t memoryLimit )
{
	return CreateCpuMathEngine( memoryLimit );
}

// ---- GPU engine: B200 -----------------------------------------------------------------------------------------------
// "The recommended GPU": device 0 of the sm_100 devices the manager lists; null when there is none, as the reference
// returns null on a machine without a usable GPU.
IMathEngine* CreateGpuMathEngine( size_t memoryLimit, int flags )
{
	return CreateB200MathEngine( -1, memoryLimit, flags );
}

IGpuMathEngineManager* CreateGpuMathEngineManager()
{
	return CreateB200MathEngineManager();
}

void CreateDistributedCudaMathEngines( IMathEngine** mathEngines, int devsCount, const int* cudaDevs, size_t memoryLimit )
{
	ASSERT_EXPR( mathEngines != nullptr );
	ASSERT_EXPR( devsCount > 0 );
	ASSERT_EXPR( cudaDevs != nullptr );
	CreateDistributedB200MathEngines( mathEngines, devsCount, cudaDevs, memoryLimit );
}

} // namespace NeoML
