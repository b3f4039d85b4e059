// CDnn graphs of the benchmark configurations behind a C interface (ctypes-friendly): NeoML builds, loads and runs
// the networks; the math engine under them is whatever the NeoMathEngine factory returns --
// CreateCpuMathEngine (NeoML's own CPU engine) or CreateGpuMathEngine / the GPU manager / the distributed factory
// (the B200 engine when libNeoMathEngine.so was built with this repository's factory).
//
// A "model" is an engine-independent NeoML archive in host memory: the network is assembled once on a CPU engine with
// the given weights and serialised (CDnn::Serialize into a CMemoryFile -- the way CDistributedTraining clones a
// network onto its engines, NeoML/src/Dnn/DnnDistributed.cpp:235-243,277-286); a "net" is that archive loaded into a
// CDnn on one engine.  Both engines therefore run bit-identical weights through NeoML's own loading path.
//
//   resnet50     ResNet-50 v1.5: CConvLayer (+ free term = folded BatchNorm) / CReLULayer / CImageResizeLayer +
//                CMaxPoolingLayer (padded pool) / CEltwiseSumLayer / CGlobalMeanPoolingLayer / CFullyConnectedLayer /
//                CSoftmaxLayer / CArgmaxLayer; sinks "probs" (float) and "argmax" (int)
//   transformer  n x CTransformerEncoderLayer (post-norm, GELU, dropout 0) with an optional MT_OneObject mask input
//   conv         one CConvLayer;  mbv2  one CMobileNetV2BlockLayer;  matmul  one CMatrixMultiplicationLayer
//
// Every entry point catches NeoML's exceptions (std::exception-derived in this build) and reports them through
// cdnn_last_error(); a "not implemented" assert of the engine arrives here as such a message.
#include <NeoML/NeoML.h>
#include <NeoML/Dnn/DnnDistributed.h>

#include <dlfcn.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

using namespace NeoML;

#define CDNN_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string lastError;

template<class F> int guarded( F&& f )
{
	try {
		f();
		return 0;
	} catch( const std::exception& e ) {
		lastError = e.what();
	} catch( ... ) {
		lastError = "unknown exception";
	}
	return -1;
}

template<class F> void* guardedPtr( F&& f )
{
	void* result = nullptr;
	return guarded( [&] { result = f(); } ) == 0 ? result : nullptr;
}

struct CModel {
	std::vector<unsigned char> archive;
};

struct CNet {
	IMathEngine* engine = nullptr;
	CRandom random{ 0x5eed };
	std::unique_ptr<CDnn> dnn;
};

// counter-based generator: the same seed gives the same weights wherever the model is built
struct CSplitMix {
	uint64_t state;
	explicit CSplitMix( uint64_t seed ) : state( seed ) {}
	uint64_t next()
	{
		uint64_t z = ( state += 0x9E3779B97F4A7C15ull );
		z = ( z ^ ( z >> 30 ) ) * 0xBF58476D1CE4E5B9ull;
		z = ( z ^ ( z >> 27 ) ) * 0x94D049BB133111EBull;
		return z ^ ( z >> 31 );
	}
	double uniform() { return ( next() >> 11 ) * ( 1.0 / 9007199254740992.0 ); }
	float normal( float sigma )
	{
		const double u1 = 1.0 - uniform(), u2 = uniform();
		return static_cast<float>( sigma * std::sqrt( -2.0 * std::log( u1 ) ) * std::cos( 6.283185307179586 * u2 ) );
	}
};

CPtr<CDnnBlob> blobFrom( IMathEngine& engine, const float* data, std::initializer_list<int> dims7 )
{
	CPtr<CDnnBlob> blob = CDnnBlob::CreateTensor( engine, CT_Float, dims7 );
	blob->CopyFrom( data );
	return blob;
}

void storeModel( CDnn& dnn, CModel& model )
{
	CMemoryFile file;
	{
		CArchive archive( &file, CArchive::SD_Storing );
		dnn.Serialize( archive );
		archive.Close();
	}
	model.archive.resize( static_cast<size_t>( file.GetLength() ) );
	file.SeekToBegin();
	file.Read( model.archive.data(), static_cast<int>( model.archive.size() ) );
}

CPtr<CSourceLayer> addSource( CDnn& dnn, const char* name )
{
	CPtr<CSourceLayer> source = new CSourceLayer( dnn.GetMathEngine() );
	source->SetName( name );
	dnn.AddLayer( *source );
	return source;
}

void addSink( CDnn& dnn, const char* name, CBaseLayer& from, int output = 0 )
{
	CPtr<CSinkLayer> sink = new CSinkLayer( dnn.GetMathEngine() );
	sink->SetName( name );
	sink->Connect( 0, from, output );
	dnn.AddLayer( *sink );
}

CPtr<CConvLayer> addConv( CDnn& dnn, const char* name, CBaseLayer& input, int cin, int cout, int fh, int fw, int strideH,
	int strideW, int padH, int padW, int dilH, int dilW, const float* filter, const float* bias )
{
	IMathEngine& engine = dnn.GetMathEngine();
	CPtr<CConvLayer> conv = new CConvLayer( engine );
	conv->SetName( name );
	conv->SetFilterCount( cout );
	conv->SetFilterHeight( fh );
	conv->SetFilterWidth( fw );
	conv->SetStrideHeight( strideH );
	conv->SetStrideWidth( strideW );
	conv->SetPaddingHeight( padH );
	conv->SetPaddingWidth( padW );
	conv->SetDilationHeight( dilH );
	conv->SetDilationWidth( dilW );
	conv->SetFilterData( blobFrom( engine, filter, { 1, cout, 1, fh, fw, 1, cin } ) );
	if( bias != nullptr ) {
		conv->SetFreeTermData( blobFrom( engine, bias, { 1, 1, 1, 1, 1, 1, cout } ) );
	} else {
		conv->SetZeroFreeTerm( true );
	}
	conv->Connect( input );
	dnn.AddLayer( *conv );
	return conv;
}

CPtr<CBaseLayer> addReLU( CDnn& dnn, const std::string& name, CBaseLayer& input )
{
	CPtr<CReLULayer> relu = new CReLULayer( dnn.GetMathEngine() );
	relu->SetName( name.c_str() );
	relu->Connect( input );
	dnn.AddLayer( *relu );
	return relu.Ptr();
}

// walks a layer graph (composites included) and hands every fully connected layer to `visit`, in name order
template<class F> void forEachFullyConnected( CDnnLayerGraph& graph, const std::string& prefix, F&& visit )
{
	CArray<const char*> names;
	graph.GetLayerList( names );
	std::vector<std::string> sorted;
	for( int i = 0; i < names.Size(); ++i ) sorted.emplace_back( names[i] );
	std::sort( sorted.begin(), sorted.end() );
	for( const std::string& name : sorted ) {
		CPtr<CBaseLayer> layer = graph.GetLayer( name.c_str() );
		const std::string path = prefix + "/" + name;
		if( CFullyConnectedLayer* fc = dynamic_cast<CFullyConnectedLayer*>( layer.Ptr() ) ) {
			visit( path, *fc );
		} else if( CCompositeLayer* composite = dynamic_cast<CCompositeLayer*>( layer.Ptr() ) ) {
			forEachFullyConnected( *composite, path, visit );
		}
	}
}

uint64_t hashName( const std::string& s, uint64_t seed )
{
	uint64_t h = 1469598103934665603ull ^ seed;
	for( unsigned char c : s ) h = ( h ^ c ) * 1099511628211ull;
	return h;
}

} // namespace

//---------------------------------------------------------------------------------------------------------------------

CDNN_API const char* cdnn_last_error() { return lastError.c_str(); }

// kind 0: CreateCpuMathEngine; 1: CreateGpuMathEngine (the recommended GPU); 2: entry `device` of
// CreateGpuMathEngineManager.  Returns NULL (message in cdnn_last_error) when the factory returns none.
CDNN_API void* cdnn_engine_create( int kind, int device, unsigned long long memoryLimit, int flags )
{
	return guardedPtr( [&]() -> void* {
		SetMathEngineExceptionHandler( GetExceptionHandler() ); // what NeoML's own GetRecommendedGpuMathEngine does
		IMathEngine* engine = nullptr;
		if( kind == 0 ) {
			engine = CreateCpuMathEngine( static_cast<size_t>( memoryLimit ) );
		} else if( kind == 1 ) {
			engine = CreateGpuMathEngine( static_cast<size_t>( memoryLimit ), flags );
		} else {
			std::unique_ptr<IGpuMathEngineManager> manager( CreateGpuMathEngineManager() );
			engine = manager->CreateMathEngine( device, static_cast<size_t>( memoryLimit ), flags );
		}
		if( engine == nullptr ) lastError = "the math engine factory returned no engine";
		return engine;
	} );
}

CDNN_API void cdnn_engine_destroy( void* engine )
{
	guarded( [&] { delete static_cast<IMathEngine*>( engine ); } );
}

CDNN_API int cdnn_engine_info( void* engine, int* type, char* name, int nameSize, unsigned long long* peakBytes )
{
	return guarded( [&] {
		IMathEngine* e = static_cast<IMathEngine*>( engine );
		CMathEngineInfo info;
		e->GetMathEngineInfo( info );
		if( type != nullptr ) *type = static_cast<int>( e->GetType() );
		if( name != nullptr && nameSize > 0 ) std::snprintf( name, nameSize, "%s", info.Name );
		if( peakBytes != nullptr ) *peakBytes = e->GetPeakMemoryUsage();
	} );
}

CDNN_API int cdnn_gpu_count()
{
	int count = -1;
	guarded( [&] {
		std::unique_ptr<IGpuMathEngineManager> manager( CreateGpuMathEngineManager() );
		count = manager->GetMathEngineCount();
	} );
	return count;
}

//---------------------------------------------------------------------------------------------------------------------
// models

CDNN_API void cdnn_model_destroy( void* model ) { delete static_cast<CModel*>( model ); }
CDNN_API long long cdnn_model_bytes( void* model ) { return static_cast<long long>( static_cast<CModel*>( model )->archive.size() ); }

// One CConvLayer.  geometry = { cin, cout, fh, fw, strideH, strideW, padH, padW, dilH, dilW }; filter [cout, fh, fw, cin]
CDNN_API void* cdnn_model_conv( const int* g, const float* filter, const float* bias )
{
	return guardedPtr( [&]() -> void* {
		std::unique_ptr<IMathEngine> cpu( CreateCpuMathEngine( 0 ) );
		CRandom random( 1 );
		std::unique_ptr<CModel> model( new CModel );
		{
			CDnn dnn( random, *cpu );
			CPtr<CSourceLayer> in = addSource( dnn, "in" );
			CPtr<CConvLayer> conv = addConv( dnn, "conv", *in, g[0], g[1], g[2], g[3], g[4], g[5], g[6], g[7], g[8], g[9],
				filter, bias );
			addSink( dnn, "out", *conv );
			storeModel( dnn, *model );
		}
		return model.release();
	} );
}

// One CMobileNetV2BlockLayer.  relu thresholds: > 0 ReLU with that upper threshold, 0 plain ReLU, < 0 HSwish.
CDNN_API void* cdnn_model_mbv2( int cin, int cexp, int cout, int stride, int residual, float act1, float act2,
	const float* expandFilter, const float* expandBias, const float* channelwiseFilter, const float* channelwiseBias,
	const float* downFilter, const float* downBias )
{
	return guardedPtr( [&]() -> void* {
		std::unique_ptr<IMathEngine> cpu( CreateCpuMathEngine( 0 ) );
		CRandom random( 1 );
		std::unique_ptr<CModel> model( new CModel );
		{
			CDnn dnn( random, *cpu );
			CPtr<CSourceLayer> in = addSource( dnn, "in" );
			auto activation = []( float v ) {
				return v < 0 ? CActivationDesc( AF_HSwish ) : CActivationDesc( AF_ReLU, CReLUActivationParam{ v } );
			};
			auto optional = [&]( const float* data, int n ) -> CPtr<CDnnBlob> {
				return data == nullptr ? nullptr : blobFrom( *cpu, data, { 1, 1, 1, 1, 1, 1, n } );
			};
			CPtr<CMobileNetV2BlockLayer> block = new CMobileNetV2BlockLayer( *cpu,
				blobFrom( *cpu, expandFilter, { 1, cexp, 1, 1, 1, 1, cin } ), optional( expandBias, cexp ), activation( act1 ),
				stride, blobFrom( *cpu, channelwiseFilter, { 1, 1, 1, 3, 3, 1, cexp } ), optional( channelwiseBias, cexp ),
				activation( act2 ), blobFrom( *cpu, downFilter, { 1, cout, 1, 1, 1, 1, cexp } ), optional( downBias, cout ),
				residual != 0 );
			block->SetName( "block" );
			block->Connect( *in );
			dnn.AddLayer( *block );
			addSink( dnn, "out", *block );
			storeModel( dnn, *model );
		}
		return model.release();
	} );
}

// One CMatrixMultiplicationLayer: inputs "a" [batch, M, K] and "b" [batch, K, N] (as height x channels matrices per
// object), output "out".
CDNN_API void* cdnn_model_matmul()
{
	return guardedPtr( [&]() -> void* {
		std::unique_ptr<IMathEngine> cpu( CreateCpuMathEngine( 0 ) );
		CRandom random( 1 );
		std::unique_ptr<CModel> model( new CModel );
		{
			CDnn dnn( random, *cpu );
			CPtr<CSourceLayer> a = addSource( dnn, "a" );
			CPtr<CSourceLayer> b = addSource( dnn, "b" );
			CPtr<CMatrixMultiplicationLayer> mm = new CMatrixMultiplicationLayer( *cpu );
			mm->SetName( "mm" );
			mm->Connect( 0, *a );
			mm->Connect( 1, *b );
			dnn.AddLayer( *mm );
			addSink( dnn, "out", *mm );
			storeModel( dnn, *model );
		}
		return model.release();
	} );
}

// ResNet-50 v1.5.  `params` holds, in network order (stem; per block: [down], c1, c2, c3 -- `down` first in a
// stage's first block; then the classifier), each convolution's filter [cout, k, k, cin] followed by its cout free
// terms, then the classifier's weights [classes, 2048] and free terms.  v1.5: the stride of a stage sits on the 3x3.
CDNN_API void* cdnn_model_resnet50( const float* params, long long count, int classes )
{
	return guardedPtr( [&]() -> void* {
		std::unique_ptr<IMathEngine> cpu( CreateCpuMathEngine( 0 ) );
		CRandom random( 1 );
		std::unique_ptr<CModel> model( new CModel );
		const float* p = params;
		const float* const end = params + count;
		auto take = [&]( long long n ) {
			const float* at = p;
			p += n;
			if( p > end ) throw std::logic_error( "cdnn_model_resnet50: the parameter array is too short" );
			return at;
		};
		{
			CDnn dnn( random, *cpu );
			auto conv = [&]( const std::string& name, CBaseLayer& input, int cin, int cout, int k, int stride, int pad ) {
				const float* w = take( 1LL * cout * k * k * cin );
				const float* b = take( cout );
				return addConv( dnn, name.c_str(), input, cin, cout, k, k, stride, stride, pad, pad, 1, 1, w, b );
			};
			CPtr<CSourceLayer> in = addSource( dnn, "in" );
			CPtr<CBaseLayer> t = addReLU( dnn, "stem_relu", *conv( "stem", *in, 3, 64, 7, 2, 3 ) );
			// 3x3/2 max pooling with padding 1: NeoML's pooling takes no padding, the image is widened first (what
			// NeoOnnx emits for a padded pool, NeoOnnx/src/Operators/PoolOperator.cpp:66-76); inputs are >= 0 here
			CPtr<CImageResizeLayer> pad = new CImageResizeLayer( *cpu );
			pad->SetName( "pool_pad" );
			for( int side = 0; side < CImageResizeLayer::IS_Count; ++side ) {
				pad->SetDelta( static_cast<CImageResizeLayer::TImageSide>( side ), 1 );
			}
			pad->SetDefaultValue( 0.f );
			pad->Connect( *t );
			dnn.AddLayer( *pad );
			CPtr<CMaxPoolingLayer> pool = new CMaxPoolingLayer( *cpu );
			pool->SetName( "pool" );
			pool->SetFilterHeight( 3 );
			pool->SetFilterWidth( 3 );
			pool->SetStrideHeight( 2 );
			pool->SetStrideWidth( 2 );
			pool->Connect( *pad );
			dnn.AddLayer( *pool );
			t = pool.Ptr();

			const int stages[4][4] = { { 64, 256, 3, 1 }, { 128, 512, 4, 2 }, { 256, 1024, 6, 2 }, { 512, 2048, 3, 2 } };
			int cin = 64;
			for( int si = 0; si < 4; ++si ) {
				const int mid = stages[si][0], out = stages[si][1];
				for( int bi = 0; bi < stages[si][2]; ++bi ) {
					const int stride = bi == 0 ? stages[si][3] : 1;
					const std::string prefix = "s" + std::to_string( si + 1 ) + "b" + std::to_string( bi + 1 );
					CPtr<CBaseLayer> shortcut = t;
					if( bi == 0 ) shortcut = conv( prefix + "_down", *t, cin, out, 1, stride, 0 ).Ptr();
					CPtr<CBaseLayer> u = addReLU( dnn, prefix + "_r1", *conv( prefix + "_c1", *t, cin, mid, 1, 1, 0 ) );
					u = addReLU( dnn, prefix + "_r2", *conv( prefix + "_c2", *u, mid, mid, 3, stride, 1 ) );
					CPtr<CConvLayer> c3 = conv( prefix + "_c3", *u, mid, out, 1, 1, 0 );
					CPtr<CEltwiseSumLayer> sum = new CEltwiseSumLayer( *cpu );
					sum->SetName( ( prefix + "_sum" ).c_str() );
					sum->Connect( 0, *c3 );
					sum->Connect( 1, *shortcut );
					dnn.AddLayer( *sum );
					t = addReLU( dnn, prefix + "_r3", *sum );
					cin = out;
				}
			}
			CPtr<CGlobalMeanPoolingLayer> mean = new CGlobalMeanPoolingLayer( *cpu );
			mean->SetName( "mean" );
			mean->Connect( *t );
			dnn.AddLayer( *mean );
			CPtr<CFullyConnectedLayer> fc = new CFullyConnectedLayer( *cpu );
			fc->SetName( "fc" );
			fc->SetNumberOfElements( classes );
			{
				const float* w = take( 1LL * classes * cin );
				const float* b = take( classes );
				CPtr<CDnnBlob> weights = blobFrom( *cpu, w, { 1, classes, 1, 1, 1, 1, cin } );
				CPtr<CDnnBlob> freeTerms = blobFrom( *cpu, b, { 1, 1, 1, 1, 1, 1, classes } );
				fc->SetWeightsData( weights );
				fc->SetFreeTermData( freeTerms );
			}
			fc->Connect( *mean );
			dnn.AddLayer( *fc );
			CPtr<CSoftmaxLayer> softmax = new CSoftmaxLayer( *cpu );
			softmax->SetName( "softmax" );
			softmax->Connect( *fc );
			dnn.AddLayer( *softmax );
			CPtr<CArgmaxLayer> argmax = new CArgmaxLayer( *cpu );
			argmax->SetName( "argmax_layer" );
			argmax->SetDimension( BD_Channels );
			argmax->Connect( *softmax );
			dnn.AddLayer( *argmax );
			addSink( dnn, "probs", *softmax );
			addSink( dnn, "argmax", *argmax );
			if( p != end ) throw std::logic_error( "cdnn_model_resnet50: the parameter array is too long" );
			storeModel( dnn, *model );
		}
		return model.release();
	} );
}

// `layers` x CTransformerEncoderLayer (post-norm, AF_GELU in its default sigmoid-approximate mode, dropout 0), input
// "in" [1, batch, seq, 1, 1, 1, hidden]; with useMask != 0 a second input "mask" [1, 1, 1, 1, seq, 1, seq] (1 = ignored
// position, MT_OneObject).  Every fully connected layer gets weights and free terms ~ N(0, sigma) from `seed`.
CDNN_API void* cdnn_model_transformer( int layers, int hidden, int heads, int ffn, unsigned long long seed, float sigma,
	int useMask )
{
	return guardedPtr( [&]() -> void* {
		std::unique_ptr<IMathEngine> cpu( CreateCpuMathEngine( 0 ) );
		CRandom random( 1 );
		std::unique_ptr<CModel> model( new CModel );
		{
			CDnn dnn( random, *cpu );
			CPtr<CSourceLayer> in = addSource( dnn, "in" );
			CPtr<CSourceLayer> mask = useMask != 0 ? addSource( dnn, "mask" ) : nullptr;
			CPtr<CBaseLayer> t = in.Ptr();
			for( int i = 0; i < layers; ++i ) {
				CPtr<CTransformerEncoderLayer> layer = new CTransformerEncoderLayer( *cpu );
				layer->SetName( ( "encoder" + std::to_string( i ) ).c_str() );
				layer->SetHeadCount( heads );
				layer->SetHiddenSize( hidden );
				layer->SetFeedForwardSize( ffn );
				layer->SetDropoutRate( 0.f );
				layer->SetActivation( CActivationDesc( AF_GELU ) );
				layer->Connect( 0, *t );
				if( mask != nullptr ) layer->Connect( 1, *mask );
				dnn.AddLayer( *layer );
				t = layer.Ptr();
			}
			addSink( dnn, "out", *t );
			// one pass over a two-token sequence creates the parameter blobs; then they are overwritten
			const int seq = 2;
			std::vector<float> zeros( static_cast<size_t>( seq ) * std::max( hidden, seq ), 0.f );
			in->SetBlob( blobFrom( *cpu, zeros.data(), { 1, 1, seq, 1, 1, 1, hidden } ) );
			if( mask != nullptr ) mask->SetBlob( blobFrom( *cpu, zeros.data(), { 1, 1, 1, 1, seq, 1, seq } ) );
			dnn.RunOnce();
			forEachFullyConnected( dnn, "", [&]( const std::string& path, CFullyConnectedLayer& fc ) {
				CSplitMix rng( hashName( path, seed ) );
				CPtr<CDnnBlob> w = fc.GetWeightsData();
				std::vector<float> values( static_cast<size_t>( w->GetDataSize() ) );
				for( float& v : values ) v = rng.normal( sigma );
				w->CopyFrom( values.data() );
				fc.SetWeightsData( w );
				CPtr<CDnnBlob> b = fc.GetFreeTermData();
				if( b != nullptr ) {
					values.resize( static_cast<size_t>( b->GetDataSize() ) );
					for( float& v : values ) v = rng.normal( sigma );
					b->CopyFrom( values.data() );
					fc.SetFreeTermData( b );
				}
			} );
			storeModel( dnn, *model );
		}
		return model.release();
	} );
}

//---------------------------------------------------------------------------------------------------------------------
// nets

CDNN_API void* cdnn_net_create( void* engine, void* model )
{
	return guardedPtr( [&]() -> void* {
		std::unique_ptr<CNet> net( new CNet );
		net->engine = static_cast<IMathEngine*>( engine );
		net->dnn.reset( new CDnn( net->random, *net->engine ) );
		CModel* m = static_cast<CModel*>( model );
		CMemoryFile file;
		file.Write( m->archive.data(), static_cast<int>( m->archive.size() ) );
		file.SeekToBegin();
		CArchive archive( &file, CArchive::SD_Loading );
		net->dnn->Serialize( archive );
		archive.Close();
		return net.release();
	} );
}

CDNN_API void cdnn_net_destroy( void* net )
{
	guarded( [&] { delete static_cast<CNet*>( net ); } );
}

// Gives source layer `name` a blob of the seven dimensions `dims` (NeoML order: BatchLength, BatchWidth, ListSize,
// Height, Width, Depth, Channels) filled from `host`.  A blob of the same shape is reused: the call is then one
// host-to-device exchange (CDnnBlob::CopyFrom -> IMathEngine::DataExchangeRaw).
CDNN_API int cdnn_net_set_input( void* netPtr, const char* name, const float* host, const int* dims )
{
	return guarded( [&] {
		CNet* net = static_cast<CNet*>( netPtr );
		CPtr<CSourceLayer> source = CheckCast<CSourceLayer>( net->dnn->GetLayer( name ) );
		CPtr<CDnnBlob> blob = source->GetBlob();
		bool same = blob != nullptr && blob->GetDataType() == CT_Float;
		for( int i = 0; same && i < 7; ++i ) same = blob->DimSize( i ) == dims[i];
		if( !same ) {
			blob = CDnnBlob::CreateTensor( *net->engine, CT_Float, { dims[0], dims[1], dims[2], dims[3], dims[4], dims[5], dims[6] } );
		}
		blob->CopyFrom( host );
		if( !same ) source->SetBlob( blob );
	} );
}

CDNN_API int cdnn_net_run( void* net )
{
	return guarded( [&] { static_cast<CNet*>( net )->dnn->RunOnce(); } );
}

// Copies the blob of sink `name` to `host` (device-to-host exchange: results are complete when this returns).
// dims receives the seven dimensions, isInt whether the data are 32-bit integers.  With host == NULL only the shape.
CDNN_API int cdnn_net_get_output( void* netPtr, const char* name, void* host, long long capacityBytes, int* dims, int* isInt )
{
	return guarded( [&] {
		CNet* net = static_cast<CNet*>( netPtr );
		CPtr<CSinkLayer> sink = CheckCast<CSinkLayer>( net->dnn->GetLayer( name ) );
		CPtr<CDnnBlob> blob = sink->GetBlob();
		if( blob == nullptr ) throw std::logic_error( "the sink holds no blob: run the net first" );
		for( int i = 0; dims != nullptr && i < 7; ++i ) dims[i] = blob->DimSize( i );
		if( isInt != nullptr ) *isInt = blob->GetDataType() == CT_Int ? 1 : 0;
		if( host == nullptr ) return;
		if( capacityBytes < static_cast<long long>( blob->GetDataSize() ) * 4 ) throw std::logic_error( "output buffer too small" );
		if( blob->GetDataType() == CT_Int ) {
			blob->CopyTo( static_cast<int*>( host ) );
		} else {
			blob->CopyTo( static_cast<float*>( host ) );
		}
	} );
}

// Wall-clock seconds of `steps` x ( [host -> source blob] RunOnce [sinks -> host] ) on this net.  sinkNames is one
// sink or several separated by commas; their blobs are written to `output` one after the other.  input / output may
// be NULL (then the source keeps its blob / nothing is read back except a final 4-byte read that waits for the device).
static double timeSteps( void* netPtr, int steps, const char* sourceName, const float* input, const char* sinkNames,
	void* output, long long outputBytes, bool twoInputBlobs, long long inputStrideFloats = 0, long long outputStrideBytes = 0 );

CDNN_API double cdnn_net_time_steps( void* netPtr, int steps, const char* sourceName, const float* input, const char* sinkNames,
	void* output, long long outputBytes )
{
	return timeSteps( netPtr, steps, sourceName, input, sinkNames, output, outputBytes, false );
}

// The same work per step -- one host -> device copy of the batch, one RunOnce, the sinks copied to the host -- with
// the input double-buffered by the caller, the way a NeoML user hides the input copy: two blobs alternate as the
// source layer's blob (CSourceLayer::SetBlob), and the batch of step i + 1 is copied into the idle one right after
// RunOnce of step i has been issued, before step i's results are read.  An engine that queues its work asynchronously
// can then overlap that copy with the kernels of step i; on an engine that runs each call to completion nothing changes.
// Step i reads its batch at input + i * inputStrideFloats and writes its results at output + i * outputStrideBytes
// (strides of 0: the same batch and the same result buffer every step).
CDNN_API double cdnn_net_time_steps_double_buffered( void* netPtr, int steps, const char* sourceName, const float* input,
	long long inputStrideFloats, const char* sinkNames, void* output, long long outputStrideBytes, long long outputBytes )
{
	return timeSteps( netPtr, steps, sourceName, input, sinkNames, output, outputBytes, true, inputStrideFloats, outputStrideBytes );
}

static double timeSteps( void* netPtr, int steps, const char* sourceName, const float* input, const char* sinkNames,
	void* output, long long outputBytes, bool twoInputBlobs, long long inputStrideFloats, long long outputStrideBytes )
{
	double seconds = -1;
	guarded( [&] {
		CNet* net = static_cast<CNet*>( netPtr );
		CPtr<CSourceLayer> source = sourceName != nullptr ? CheckCast<CSourceLayer>( net->dnn->GetLayer( sourceName ) ) : nullptr;
		std::vector<CPtr<CSinkLayer>> sinks;
		{
			std::string names( sinkNames );
			size_t at = 0;
			while( at <= names.size() ) {
				const size_t comma = names.find( ',', at );
				const std::string one = names.substr( at, comma == std::string::npos ? std::string::npos : comma - at );
				sinks.push_back( CheckCast<CSinkLayer>( net->dnn->GetLayer( one.c_str() ) ) );
				if( comma == std::string::npos ) break;
				at = comma + 1;
			}
		}
		CPtr<CDnnBlob> inputBlobs[2];
		if( twoInputBlobs && input != nullptr ) {
			inputBlobs[0] = source->GetBlob();
			inputBlobs[1] = CDnnBlob::CreateBlob( *net->engine, CT_Float, inputBlobs[0]->GetDesc() );
		}
		const auto t0 = std::chrono::steady_clock::now();
		if( inputBlobs[1] != nullptr ) inputBlobs[0]->CopyFrom( input );
		for( int i = 0; i < steps; ++i ) {
			if( inputBlobs[1] != nullptr ) {
				source->SetBlob( inputBlobs[i & 1] );
			} else if( input != nullptr ) {
				source->GetBlob()->CopyFrom( input );
			}
			net->dnn->RunOnce();
			if( inputBlobs[1] != nullptr && i + 1 < steps ) inputBlobs[( i + 1 ) & 1]->CopyFrom( input + ( i + 1 ) * inputStrideFloats );
			if( output != nullptr ) {
				char* at = static_cast<char*>( output ) + i * outputStrideBytes;
				for( CPtr<CSinkLayer>& sink : sinks ) {
					CPtr<CDnnBlob> blob = sink->GetBlob();
					const long long bytes = static_cast<long long>( blob->GetDataSize() ) * 4;
					if( at + bytes > static_cast<char*>( output ) + i * outputStrideBytes + outputBytes ) throw std::logic_error( "output buffer too small" );
					if( blob->GetDataType() == CT_Int ) blob->CopyTo( reinterpret_cast<int*>( at ) ); else blob->CopyTo( reinterpret_cast<float*>( at ) );
					at += bytes;
				}
			}
		}
		if( output == nullptr ) {
			// any device-to-host exchange completes the work issued before it
			CPtr<CDnnBlob> blob = sinks[0]->GetBlob();
			int word = 0;
			if( blob->GetDataType() == CT_Int ) {
				net->engine->DataExchangeRaw( &word, blob->GetData<int>(), sizeof( word ) );
			} else {
				net->engine->DataExchangeRaw( &word, blob->GetData<float>(), sizeof( word ) );
			}
		}
		seconds = std::chrono::duration<double>( std::chrono::steady_clock::now() - t0 ).count();
	} );
	return seconds;
}

//---------------------------------------------------------------------------------------------------------------------
// Several replicas of one model, one math engine and one host thread each: the shape of NeoML's
// CDistributedInference / CDistributedTraining (NeoML/src/Dnn/DnnDistributed.cpp:270-296,343-375,551-607), with the
// engines made by the factory's distributed entry points.

namespace {

struct CReplicas {
	std::vector<IMathEngine*> engines;
	std::vector<std::unique_ptr<CNet>> nets;
};

} // namespace

// kind 0: `count` CPU engines (CreateCpuMathEngine each); kind 1: CreateDistributedCudaMathEngines on devices[0..count)
CDNN_API void* cdnn_replicas_create( int kind, int count, const int* devices, void* model )
{
	return guardedPtr( [&]() -> void* {
		SetMathEngineExceptionHandler( GetExceptionHandler() );
		std::unique_ptr<CReplicas> r( new CReplicas );
		r->engines.assign( count, nullptr );
		if( kind == 0 ) {
			for( int i = 0; i < count; ++i ) r->engines[i] = CreateCpuMathEngine( 0 );
		} else {
			CreateDistributedCudaMathEngines( r->engines.data(), count, devices, 0 );
		}
		for( int i = 0; i < count; ++i ) {
			if( r->engines[i] == nullptr ) throw std::logic_error( "the distributed factory returned no engine" );
			r->nets.emplace_back( static_cast<CNet*>( cdnn_net_create( r->engines[i], model ) ) );
			if( r->nets.back() == nullptr ) throw std::logic_error( lastError );
		}
		return r.release();
	} );
}

CDNN_API void cdnn_replicas_destroy( void* replicas )
{
	guarded( [&] {
		CReplicas* r = static_cast<CReplicas*>( replicas );
		r->nets.clear();
		for( IMathEngine* e : r->engines ) delete e;
		delete r;
	} );
}

CDNN_API void* cdnn_replicas_net( void* replicas, int index )
{
	CReplicas* r = static_cast<CReplicas*>( replicas );
	return index >= 0 && index < static_cast<int>( r->nets.size() ) ? r->nets[index].get() : nullptr;
}

// Every replica, on its own host thread, runs `steps` x ( host -> source, RunOnce, sink -> host ) on its slice:
// replica i reads inputs + i * inputFloatsPerReplica and writes outputs + i * outputBytesPerReplica.  All threads
// start together; returns the wall-clock seconds until the last one finished (after `warmup` untimed steps each).
static double replicasTimeSteps( void* replicas, int warmup, int steps, const char* sourceName, const float* inputs,
	long long inputFloatsPerReplica, const char* sinkName, char* outputs, long long outputBytesPerReplica, bool doubleBuffered );

CDNN_API double cdnn_replicas_time_steps( void* replicas, int warmup, int steps, const char* sourceName, const float* inputs,
	long long inputFloatsPerReplica, const char* sinkName, char* outputs, long long outputBytesPerReplica )
{
	return replicasTimeSteps( replicas, warmup, steps, sourceName, inputs, inputFloatsPerReplica, sinkName, outputs,
		outputBytesPerReplica, false );
}

// The same with every replica's input double-buffered (two blobs alternate as the source layer's blob; the copy of
// step i + 1 is issued right after RunOnce of step i): the loop of a caller that hides its input copy.
CDNN_API double cdnn_replicas_time_steps_double_buffered( void* replicas, int warmup, int steps, const char* sourceName,
	const float* inputs, long long inputFloatsPerReplica, const char* sinkName, char* outputs, long long outputBytesPerReplica )
{
	return replicasTimeSteps( replicas, warmup, steps, sourceName, inputs, inputFloatsPerReplica, sinkName, outputs,
		outputBytesPerReplica, true );
}

static double replicasTimeSteps( void* replicas, int warmup, int steps, const char* sourceName, const float* inputs,
	long long inputFloatsPerReplica, const char* sinkName, char* outputs, long long outputBytesPerReplica, bool doubleBuffered )
{
	CReplicas* r = static_cast<CReplicas*>( replicas );
	const int n = static_cast<int>( r->nets.size() );
	std::atomic<int> ready{ 0 };
	std::atomic<bool> go{ false };
	std::vector<std::string> errors( n );
	std::vector<std::thread> threads;
	std::vector<std::chrono::steady_clock::time_point> finished( n );
	for( int i = 0; i < n; ++i ) {
		threads.emplace_back( [&, i] {
			SetMathEngineExceptionHandler( GetExceptionHandler() );
			const float* in = inputs != nullptr ? inputs + i * inputFloatsPerReplica : nullptr;
			char* out = outputs != nullptr ? outputs + i * outputBytesPerReplica : nullptr;
			// the warm-up runs the loop that is timed, so that the engine's pools hold that loop's blocks
			const auto run = [&]( int count ) {
				return doubleBuffered ? cdnn_net_time_steps_double_buffered( r->nets[i].get(), count, sourceName, in, 0, sinkName, out, 0,
					outputBytesPerReplica )
					: cdnn_net_time_steps( r->nets[i].get(), count, sourceName, in, sinkName, out, outputBytesPerReplica );
			};
			if( warmup > 0 && run( warmup ) < 0 ) errors[i] = lastError;
			ready.fetch_add( 1 );
			while( !go.load() ) std::this_thread::yield();
			if( errors[i].empty() && run( steps ) < 0 ) errors[i] = lastError;
			finished[i] = std::chrono::steady_clock::now();
		} );
	}
	while( ready.load() < n ) std::this_thread::yield();
	const auto t0 = std::chrono::steady_clock::now();
	go.store( true );
	for( std::thread& t : threads ) t.join();
	double seconds = 0;
	for( int i = 0; i < n; ++i ) {
		if( !errors[i].empty() ) {
			lastError = errors[i];
			return -1;
		}
		seconds = std::max( seconds, std::chrono::duration<double>( finished[i] - t0 ).count() );
	}
	return seconds;
}

//---------------------------------------------------------------------------------------------------------------------
// Engine checks made of raw IMathEngine calls (what layers do, in orders a test wants to control)

// A convolution whose source blob is freed right after the call, before the in-place ReLU that follows it -- the order
// in which a CDnn in reuse-memory mode releases a layer's inputs (NeoML/src/Dnn/BaseLayer.cpp, setAllocatedBlobs).
// The shape is chosen so that the engine's work memory for the call (the prepared filter: 113 x 3 x 3 x 32 floats)
// falls in the size class of the freed source (32 x 32 x 32 floats).  Writes the largest absolute difference between
// the result with the early free and the result with the source kept alive; 0 is the only right answer.
CDNN_API int cdnn_selftest_free_while_pending( void* enginePtr, float* maxDifference )
{
	return guarded( [&] {
		IMathEngine& e = *static_cast<IMathEngine*>( enginePtr );
		const int h = 32, w = 32, c = 32, k = 113;
		CSplitMix rng( 2718 );
		std::vector<float> x( h * w * c ), f( k * 9 * c ), b( k );
		for( float& v : x ) v = static_cast<float>( rng.uniform() * 2 - 1 );
		for( float& v : f ) v = static_cast<float>( rng.uniform() * 2 - 1 );
		for( float& v : b ) v = static_cast<float>( rng.uniform() * 2 - 1 );
		auto run = [&]( bool earlyFree ) {
			CPtr<CDnnBlob> src = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 1, h, w, c );
			CPtr<CDnnBlob> flt = CDnnBlob::CreateTensor( e, CT_Float, { 1, k, 1, 3, 3, 1, c } );
			CPtr<CDnnBlob> bias = CDnnBlob::CreateVector( e, CT_Float, k );
			CPtr<CDnnBlob> out = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 1, h, w, k );
			CPtr<CDnnBlob> zero = CDnnBlob::CreateVector( e, CT_Float, 1 );
			src->CopyFrom( x.data() );
			flt->CopyFrom( f.data() );
			bias->CopyFrom( b.data() );
			zero->Fill( 0.f );
			std::unique_ptr<CConvolutionDesc> desc( e.InitBlobConvolution( src->GetDesc(), 1, 1, 1, 1, 1, 1, flt->GetDesc(),
				out->GetDesc() ) );
			const CConstFloatHandle freeTerm = bias->GetData();
			e.BlobConvolution( *desc, src->GetData(), flt->GetData(), &freeTerm, out->GetData() );
			if( earlyFree ) src = nullptr;
			e.VectorReLU( out->GetData(), out->GetData(), out->GetDataSize(), zero->GetData() );
			std::vector<float> y( static_cast<size_t>( out->GetDataSize() ) );
			out->CopyTo( y.data() );
			return y;
		};
		const std::vector<float> kept = run( false ), freed = run( true );
		float worst = 0.f;
		for( size_t i = 0; i < kept.size(); ++i ) worst = std::max( worst, std::fabs( kept[i] - freed[i] ) );
		*maxDifference = worst;
	} );
}

// BlobResizeImage (constant border) followed by BlobMaxPooling, the pair behind a padded stem pool, in the orders in
// which a caller may touch the buffers involved.  An engine may hold the padding back and pool the unpadded image in
// one pass; whatever it does, every buffer must read as if each call had run when it was made:
//   0  pad, pool, read the pooled image          1  pad, pool, then read the PADDED image
//   2  pad, free the source, pool                2  (same number) ...
//   3  pad, overwrite the source, read the padded image (it shows the old source)
//   4  pad, free the padded image unread, pad again into a new blob, pool
// Writes the number of values that differ from a host evaluation (0 is the only right answer) and, for case 0, how
// many kernels the pad + pool pair launched (-1 where the engine does not count launches).
CDNN_API int cdnn_selftest_padded_pool( void* enginePtr, int* mismatches, int* launchesOfCase0 )
{
	return guarded( [&] {
		IMathEngine& e = *static_cast<IMathEngine*>( enginePtr );
		const int n = 2, h = 9, w = 11, c = 8, ph = h + 2, pw = w + 2, oh = ( ph - 3 ) / 2 + 1, ow = ( pw - 3 ) / 2 + 1;
		const float border = 0.25f; // above part of the data: the border then decides some maxima
		CSplitMix rng( 31337 );
		std::vector<float> x( static_cast<size_t>( n ) * h * w * c );
		for( float& v : x ) v = static_cast<float>( rng.uniform() * 2 - 1 );
		auto padded = [&]( const std::vector<float>& src ) {
			std::vector<float> y( static_cast<size_t>( n ) * ph * pw * c, border );
			for( int b = 0; b < n; ++b ) for( int i = 0; i < h; ++i ) for( int j = 0; j < w; ++j ) for( int k = 0; k < c; ++k ) {
				y[( ( static_cast<size_t>( b ) * ph + i + 1 ) * pw + j + 1 ) * c + k] = src[( ( static_cast<size_t>( b ) * h + i ) * w + j ) * c + k];
			}
			return y;
		};
		auto pooled = [&]( const std::vector<float>& p ) {
			std::vector<float> y( static_cast<size_t>( n ) * oh * ow * c );
			for( int b = 0; b < n; ++b ) for( int i = 0; i < oh; ++i ) for( int j = 0; j < ow; ++j ) for( int k = 0; k < c; ++k ) {
				float best = -1e30f;
				for( int fy = 0; fy < 3; ++fy ) for( int fx = 0; fx < 3; ++fx ) {
					best = std::max( best, p[( ( static_cast<size_t>( b ) * ph + 2 * i + fy ) * pw + 2 * j + fx ) * c + k] );
				}
				y[( ( static_cast<size_t>( b ) * oh + i ) * ow + j ) * c + k] = best;
			}
			return y;
		};
		const std::vector<float> wantPadded = padded( x ), wantPooled = pooled( wantPadded );
		typedef long long ( *TCount )();
		TCount launchCount = reinterpret_cast<TCount>( dlsym( RTLD_DEFAULT, "nb200_launch_count" ) );
		int wrong = 0;
		auto compare = [&]( const CDnnBlob& blob, const std::vector<float>& want ) {
			std::vector<float> got( static_cast<size_t>( blob.GetDataSize() ) );
			const_cast<CDnnBlob&>( blob ).CopyTo( got.data() );
			if( got.size() != want.size() ) { wrong += 1000000; return; }
			for( size_t i = 0; i < got.size(); ++i ) wrong += got[i] == want[i] ? 0 : 1;
		};
		*launchesOfCase0 = -1;
		for( int scenario = 0; scenario < 5; ++scenario ) {
			CPtr<CDnnBlob> src = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, n, h, w, c );
			CPtr<CDnnBlob> pad = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, n, ph, pw, c );
			CPtr<CDnnBlob> out = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, n, oh, ow, c );
			src->CopyFrom( x.data() );
			pad->Fill( -7.f );
			out->Fill( -7.f );
			std::unique_ptr<CMaxPoolingDesc> desc( e.InitMaxPooling( pad->GetDesc(), 3, 3, 2, 2, out->GetDesc() ) );
			const long long before = launchCount != nullptr ? launchCount() : 0;
			e.BlobResizeImage( src->GetDesc(), src->GetData(), 1, 1, 1, 1, border, pad->GetDesc(), pad->GetData() );
			switch( scenario ) {
				case 0:
					e.BlobMaxPooling( *desc, pad->GetData(), nullptr, out->GetData() );
					if( launchCount != nullptr ) *launchesOfCase0 = static_cast<int>( launchCount() - before );
					compare( *out, wantPooled );
					break;
				case 1:
					e.BlobMaxPooling( *desc, pad->GetData(), nullptr, out->GetData() );
					compare( *pad, wantPadded );
					compare( *out, wantPooled );
					break;
				case 2:
					src = nullptr;
					{ CPtr<CDnnBlob> other = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, n, h, w, c ); other->Fill( 3.f ); }
					e.BlobMaxPooling( *desc, pad->GetData(), nullptr, out->GetData() );
					compare( *out, wantPooled );
					break;
				case 3:
					src->Fill( 9.f );
					compare( *pad, wantPadded );
					break;
				case 4: {
					pad = nullptr;
					CPtr<CDnnBlob> again = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, n, ph, pw, c );
					e.BlobResizeImage( src->GetDesc(), src->GetData(), 1, 1, 1, 1, border, again->GetDesc(), again->GetData() );
					e.BlobMaxPooling( *desc, again->GetData(), nullptr, out->GetData() );
					compare( *out, wantPooled );
					compare( *again, wantPadded );
					break;
				}
			}
		}
		*mismatches = wrong;
	} );
}

// The score chain of CMultiheadAttentionLayer as the layers issue it -- batched MultiplyMatrixByMatrix( Q, Kt ),
// VectorMultiply in place, AddVectorToMatrixRows of the mask into ANOTHER blob (CAddToObjectLayer is not an in-place
// layer), MatrixSoftmaxByRows in place, MultiplyMatrixByMatrix( P, V ) -- in the orders in which a caller may touch the
// buffers.  An engine may run the chain as one kernel and leave scores and probabilities unwritten; whatever it does,
// every buffer must read as if each call had run when it was made:
//   0  the chain, read the result                    1  the chain, then read the probabilities
//   2  blobs released as early as NeoML's reuse mode releases them (Q, Kt after the product; scores after the mask)
//   3  the keys overwritten after the softmax was issued: probabilities and result show the old keys
//   4  no mask: scale and softmax in place
// Writes the largest error of any value read, relative to the RMS of what it is compared with (against a
// double-precision host evaluation), and how many kernels case 0 launched (-1 where launches are not counted).
CDNN_API int cdnn_selftest_attention_chain( void* enginePtr, float* worstError, int* launchesOfCase0 )
{
	return guarded( [&] {
		IMathEngine& e = *static_cast<IMathEngine*>( enginePtr );
		const int heads = 3, seq = 128, depth = 64;
		const float scaleValue = 0.125f;
		CSplitMix rng( 4242 );
		std::vector<float> q( heads * seq * depth ), kt( heads * depth * seq ), v( heads * seq * depth ), mask( seq * seq );
		for( float& x : q ) x = static_cast<float>( rng.uniform() * 2 - 1 );
		for( float& x : kt ) x = static_cast<float>( rng.uniform() * 2 - 1 );
		for( float& x : v ) x = static_cast<float>( rng.uniform() * 2 - 1 );
		for( int i = 0; i < seq; ++i ) for( int j = 0; j < seq; ++j ) mask[i * seq + j] = j > i ? -1e9f : 0.f;
		auto evaluate = [&]( const std::vector<float>& keys, bool withMask, std::vector<double>& probs, std::vector<double>& out ) {
			probs.assign( static_cast<size_t>( heads ) * seq * seq, 0. );
			out.assign( static_cast<size_t>( heads ) * seq * depth, 0. );
			for( int h = 0; h < heads; ++h ) for( int i = 0; i < seq; ++i ) {
				double* row = &probs[( static_cast<size_t>( h ) * seq + i ) * seq];
				double top = -1e300;
				for( int j = 0; j < seq; ++j ) {
					double sum = 0;
					for( int d = 0; d < depth; ++d ) sum += double( q[( h * seq + i ) * depth + d] ) * keys[( h * depth + d ) * seq + j];
					row[j] = sum * scaleValue + ( withMask ? mask[i * seq + j] : 0.f );
					top = std::max( top, row[j] );
				}
				double total = 0;
				for( int j = 0; j < seq; ++j ) { row[j] = std::exp( row[j] - top ); total += row[j]; }
				for( int j = 0; j < seq; ++j ) row[j] /= total;
				for( int d = 0; d < depth; ++d ) {
					double sum = 0;
					for( int j = 0; j < seq; ++j ) sum += row[j] * v[( h * seq + j ) * depth + d];
					out[( static_cast<size_t>( h ) * seq + i ) * depth + d] = sum;
				}
			}
		};
		std::vector<double> wantProbs, wantOut, wantProbsNoMask, wantOutNoMask;
		evaluate( kt, true, wantProbs, wantOut );
		evaluate( kt, false, wantProbsNoMask, wantOutNoMask );
		typedef long long ( *TCount )();
		TCount launchCount = reinterpret_cast<TCount>( dlsym( RTLD_DEFAULT, "nb200_launch_count" ) );
		double worst = 0;
		auto compare = [&]( const CDnnBlob& blob, const std::vector<double>& want ) {
			std::vector<float> got( static_cast<size_t>( blob.GetDataSize() ) );
			const_cast<CDnnBlob&>( blob ).CopyTo( got.data() );
			if( got.size() != want.size() ) { worst = 1e30; return; }
			double square = 0, gap = 0;
			for( size_t i = 0; i < got.size(); ++i ) { square += want[i] * want[i]; gap = std::max( gap, std::fabs( got[i] - want[i] ) ); }
			const double error = gap / std::sqrt( square / got.size() );
			worst = std::max( worst, error == error ? error : 1e30 );
		};
		*launchesOfCase0 = -1;
		for( int scenario = 0; scenario < 5; ++scenario ) {
			const bool withMask = scenario != 4;
			CPtr<CDnnBlob> bq = CDnnBlob::CreateTensor( e, CT_Float, { 1, heads, 1, seq, 1, 1, depth } );
			CPtr<CDnnBlob> bk = CDnnBlob::CreateTensor( e, CT_Float, { 1, heads, 1, depth, 1, 1, seq } );
			CPtr<CDnnBlob> bv = CDnnBlob::CreateTensor( e, CT_Float, { 1, heads, 1, seq, 1, 1, depth } );
			CPtr<CDnnBlob> bm = CDnnBlob::CreateTensor( e, CT_Float, { 1, 1, 1, seq, 1, 1, seq } );
			CPtr<CDnnBlob> scores = CDnnBlob::CreateTensor( e, CT_Float, { 1, heads, 1, seq, 1, 1, seq } );
			CPtr<CDnnBlob> masked = scores;
			if( withMask ) masked = CDnnBlob::CreateTensor( e, CT_Float, { 1, heads, 1, seq, 1, 1, seq } );
			CPtr<CDnnBlob> out = CDnnBlob::CreateTensor( e, CT_Float, { 1, heads, 1, seq, 1, 1, depth } );
			CPtr<CDnnBlob> factor = CDnnBlob::CreateVector( e, CT_Float, 1 );
			bq->CopyFrom( q.data() ); bk->CopyFrom( kt.data() ); bv->CopyFrom( v.data() ); bm->CopyFrom( mask.data() );
			factor->Fill( scaleValue );
			scores->Fill( -7.f ); out->Fill( -7.f );
			if( withMask ) masked->Fill( -7.f );
			const long long before = launchCount != nullptr ? launchCount() : 0;
			e.MultiplyMatrixByMatrix( heads, bq->GetData(), seq, depth, bk->GetData(), seq, scores->GetData(), scores->GetDataSize() );
			if( scenario == 2 ) { bq = nullptr; bk = nullptr; }
			e.VectorMultiply( scores->GetData(), scores->GetData(), scores->GetDataSize(), factor->GetData() );
			if( withMask ) {
				e.AddVectorToMatrixRows( 1, scores->GetData(), masked->GetData(), heads, seq * seq, bm->GetData() );
				if( scenario == 2 ) scores = nullptr;
			}
			e.MatrixSoftmaxByRows( masked->GetData(), heads * seq, seq, masked->GetData() );
			if( scenario == 3 ) bk->Fill( 0.5f );
			e.MultiplyMatrixByMatrix( heads, masked->GetData(), seq, seq, bv->GetData(), depth, out->GetData(), out->GetDataSize() );
			if( scenario == 0 && launchCount != nullptr ) *launchesOfCase0 = static_cast<int>( launchCount() - before );
			compare( *out, withMask ? wantOut : wantOutNoMask );
			if( scenario == 1 || scenario == 3 ) compare( *masked, wantProbs );
		}
		*worstError = static_cast<float>( worst );
	} );
}

// The chains of CObjectNormalizationLayer (ObjectNormalizationLayer.cpp:190-242) on raw engine calls, with its kinds of
// memory (the row vectors in ONE stack variable, the squared differences in another), in the orders in which a caller
// may touch the buffers.  An engine may hold the matrix-sized steps back and run each chain as one pass:
//   0  variance chain: x - mean into a stack matrix, squared in place, row sums; then the stack matrix itself is read
//   1  output chain: x - mean into the output, * 1/std by rows, * scale by columns, + bias by columns; output read
//   2  the output chain, but the row vectors are overwritten before the output is read: it shows the old vectors
//   3  the output chain, the stack variable with the row vectors released before the output is read
//   4  the output chain in place on x (the layer is an in-place layer), output read
// Writes the largest difference from a host evaluation with the same single-precision steps, relative to the
// largest magnitude (0 is expected), and the kernels launched by case 1's four calls plus the read.
CDNN_API int cdnn_selftest_normalization_chain( void* enginePtr, float* worstError, int* launchesOfCase1 )
{
	return guarded( [&] {
		IMathEngine& e = *static_cast<IMathEngine*>( enginePtr );
		const int rows = 37, width = 96;
		CSplitMix rng( 777 );
		std::vector<float> x( rows * width ), negMean( rows ), invStd( rows ), scale( width ), bias( width );
		for( float& v : x ) v = static_cast<float>( rng.uniform() * 4 - 2 );
		for( float& v : negMean ) v = static_cast<float>( rng.uniform() - 0.5 );
		for( float& v : invStd ) v = static_cast<float>( rng.uniform() + 0.5 );
		for( float& v : scale ) v = static_cast<float>( rng.uniform() + 0.5 );
		for( float& v : bias ) v = static_cast<float>( rng.uniform() - 0.5 );
		typedef long long ( *TCount )();
		TCount launchCount = reinterpret_cast<TCount>( dlsym( RTLD_DEFAULT, "nb200_launch_count" ) );
		double worst = 0;
		auto compare = [&]( const std::vector<float>& got, const std::vector<float>& want ) {
			float top = 0;
			for( float v : want ) top = std::max( top, std::fabs( v ) );
			for( size_t i = 0; i < got.size(); ++i ) {
				const double error = std::fabs( got[i] - want[i] ) / top;
				worst = std::max( worst, error == error ? error : 1e30 );
			}
		};
		std::vector<float> wantSquares( rows * width ), wantSums( rows ), wantOut( rows * width );
		for( int r = 0; r < rows; ++r ) {
			for( int c = 0; c < width; ++c ) {
				volatile float d = x[r * width + c] + negMean[r];
				volatile float q = d * d;
				wantSquares[r * width + c] = q;
				volatile float n = d * invStd[r];
				volatile float m = n * scale[c];
				volatile float o = m + bias[c];
				wantOut[r * width + c] = o;
			}
			double sum = 0;
			for( int c = 0; c < width; ++c ) sum += wantSquares[r * width + c];
			wantSums[r] = static_cast<float>( sum );
		}
		*launchesOfCase1 = -1;
		CPtr<CDnnBlob> bx = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
		CPtr<CDnnBlob> bscale = CDnnBlob::CreateVector( e, CT_Float, width );
		CPtr<CDnnBlob> bbias = CDnnBlob::CreateVector( e, CT_Float, width );
		bx->CopyFrom( x.data() ); bscale->CopyFrom( scale.data() ); bbias->CopyFrom( bias.data() );
		for( int scenario = 0; scenario < 5; ++scenario ) {
			CPtr<CDnnBlob> out = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
			out->Fill( -7.f );
			if( scenario == 4 ) out->CopyFrom( x.data() );
			std::vector<float> got( rows * width );
			{
				CFloatHandleStackVar vectors( e, 2 * rows );
				const CFloatHandle mean = vectors.GetHandle(), inv = vectors.GetHandle() + rows;
				e.DataExchangeTyped<float>( mean, negMean.data(), rows );
				e.DataExchangeTyped<float>( inv, invStd.data(), rows );
				if( scenario == 0 ) {
					CFloatHandleStackVar temp( e, rows * width );
					CFloatHandleStackVar sums( e, rows );
					e.AddVectorToMatrixColumns( bx->GetData(), temp.GetHandle(), rows, width, mean );
					e.VectorEltwiseMultiply( temp.GetHandle(), temp.GetHandle(), temp.GetHandle(), rows * width );
					e.SumMatrixColumns( sums.GetHandle(), temp.GetHandle(), rows, width );
					std::vector<float> gotSums( rows );
					e.DataExchangeTyped<float>( gotSums.data(), sums.GetHandle(), rows );
					// sums of 96 values in another order than the host's: compared to that accuracy
					float top = 0;
					for( float v : wantSums ) top = std::max( top, std::fabs( v ) );
					for( int r = 0; r < rows; ++r ) {
						const double error = std::fabs( gotSums[r] - wantSums[r] ) / top;
						worst = std::max( worst, error < 1e-5 ? 0. : error );
					}
					e.DataExchangeTyped<float>( got.data(), temp.GetHandle(), rows * width );
					compare( got, wantSquares );
					continue;
				}
				const long long before = launchCount != nullptr ? launchCount() : 0;
				e.AddVectorToMatrixColumns( scenario == 4 ? out->GetData() : bx->GetData(), out->GetData(), rows, width, mean );
				e.MultiplyDiagMatrixByMatrix( inv, rows, out->GetData(), width, out->GetData(), rows * width );
				e.MultiplyMatrixByDiagMatrix( out->GetData(), rows, width, bscale->GetData(), out->GetData(), rows * width );
				e.AddVectorToMatrixRows( 1, out->GetData(), out->GetData(), rows, width, bbias->GetData() );
				if( scenario == 4 ) {
					out->CopyTo( got.data() );
					compare( got, wantOut );
				} else if( scenario == 1 ) {
					out->CopyTo( got.data() );
					if( launchCount != nullptr ) *launchesOfCase1 = static_cast<int>( launchCount() - before );
					compare( got, wantOut );
				} else if( scenario == 2 ) {
					e.VectorFill( mean, 100.f, 2 * rows );
					out->CopyTo( got.data() );
					compare( got, wantOut );
				}
			}
			if( scenario == 3 ) {
				CFloatHandleStackVar other( e, 2 * rows ); // lands where the row vectors were
				e.VectorFill( other.GetHandle(), 100.f, 2 * rows );
				out->CopyTo( got.data() );
				compare( got, wantOut );
			}
		}
		*worstError = static_cast<float>( worst );
	} );
}

// A fully connected layer's product with what the next layers do to it, on raw engine calls: the free terms added in
// place (CFullyConnectedLayer), then one of
//   0  nothing: the biased product is read            1  CGELULayer's fast form into another blob, that blob read
//   2  the same, then the biased product read as well 3  CEltwiseSumLayer with another tensor into a third blob
//   4  the sum written over the other tensor          5  only the first step of the gate (x * 1.702), then read
//   6  the weights overwritten after the layer ran and before anything was read: the old weights count
// and a 1024-row layer run three times with its weights replaced in between (by a host copy, by a device-side fill).
// An engine may hold the product back and run bias, sum or gate in its epilogue.  Writes the largest error relative
// to the RMS of the expected values (double-precision host evaluation).
CDNN_API int cdnn_selftest_product_chain( void* enginePtr, float* worstError )
{
	return guarded( [&] {
		IMathEngine& e = *static_cast<IMathEngine*>( enginePtr );
		const int rows = 200, depth = 96, width = 160;
		CSplitMix rng( 999 );
		std::vector<float> x( rows * depth ), w( width * depth ), b( width ), other( rows * width );
		for( float& v : x ) v = static_cast<float>( rng.uniform() * 2 - 1 );
		for( float& v : w ) v = static_cast<float>( rng.uniform() * 2 - 1 ) * 0.2f;
		for( float& v : b ) v = static_cast<float>( rng.uniform() - 0.5 );
		for( float& v : other ) v = static_cast<float>( rng.uniform() * 2 - 1 );
		std::vector<double> biased( rows * width ), gated( rows * width ), summed( rows * width ), scaled( rows * width );
		for( int r = 0; r < rows; ++r ) for( int c = 0; c < width; ++c ) {
			double sum = b[c];
			for( int k = 0; k < depth; ++k ) sum += double( x[r * depth + k] ) * w[c * depth + k];
			biased[r * width + c] = sum;
			scaled[r * width + c] = sum * 1.702f;
			gated[r * width + c] = sum / ( 1. + std::exp( -sum * 1.702f ) );
			summed[r * width + c] = sum + other[r * width + c];
		}
		double worst = 0;
		auto compare = [&]( const CDnnBlob& blob, const std::vector<double>& want ) {
			std::vector<float> got( static_cast<size_t>( blob.GetDataSize() ) );
			const_cast<CDnnBlob&>( blob ).CopyTo( got.data() );
			double square = 0, gap = 0;
			for( size_t i = 0; i < got.size(); ++i ) { square += want[i] * want[i]; gap = std::max( gap, std::fabs( got[i] - want[i] ) ); }
			const double error = gap / std::sqrt( square / got.size() );
			worst = std::max( worst, error == error ? error : 1e30 );
		};
		for( int scenario = 0; scenario < 7; ++scenario ) {
			CPtr<CDnnBlob> bx = CDnnBlob::CreateMatrix( e, CT_Float, rows, depth );
			CPtr<CDnnBlob> bw = CDnnBlob::CreateMatrix( e, CT_Float, width, depth );
			CPtr<CDnnBlob> bb = CDnnBlob::CreateVector( e, CT_Float, width );
			CPtr<CDnnBlob> bo = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
			CPtr<CDnnBlob> product = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
			CPtr<CDnnBlob> second = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
			CPtr<CDnnBlob> factor = CDnnBlob::CreateVector( e, CT_Float, 1 );
			bx->CopyFrom( x.data() ); bw->CopyFrom( w.data() ); bb->CopyFrom( b.data() ); bo->CopyFrom( other.data() );
			factor->Fill( 1.702f ); product->Fill( -7.f ); second->Fill( -7.f );
			const int size = rows * width;
			e.MultiplyMatrixByTransposedMatrix( bx->GetData(), rows, depth, depth, bw->GetData(), width, depth, product->GetData(), width, size );
			e.AddVectorToMatrixRows( 1, product->GetData(), product->GetData(), rows, width, bb->GetData() );
			switch( scenario ) {
				case 0:
					compare( *product, biased );
					break;
				case 1: case 2:
					e.VectorMultiply( product->GetData(), second->GetData(), size, factor->GetData() );
					e.VectorSigmoid( second->GetData(), second->GetData(), size );
					e.VectorEltwiseMultiply( product->GetData(), second->GetData(), second->GetData(), size );
					compare( *second, gated );
					if( scenario == 2 ) compare( *product, biased );
					break;
				case 3:
					e.VectorAdd( product->GetData(), bo->GetData(), second->GetData(), size );
					compare( *second, summed );
					break;
				case 4:
					e.VectorAdd( bo->GetData(), product->GetData(), bo->GetData(), size );
					compare( *bo, summed );
					break;
				case 5:
					e.VectorMultiply( product->GetData(), second->GetData(), size, factor->GetData() );
					compare( *second, scaled );
					break;
				case 6:
					bw->Fill( 3.f );
					compare( *product, biased );
					break;
			}
		}
		// A layer of 1024 rows (an engine may keep a prepared form of the weights from pass to pass): three passes, the
		// weights replaced by a host copy before the second and by a device-side fill before the third.
		{
			const int tall = 1024;
			std::vector<float> xs( tall * depth );
			for( float& v : xs ) v = static_cast<float>( rng.uniform() * 2 - 1 );
			CPtr<CDnnBlob> bx = CDnnBlob::CreateMatrix( e, CT_Float, tall, depth );
			CPtr<CDnnBlob> bw = CDnnBlob::CreateMatrix( e, CT_Float, width, depth );
			CPtr<CDnnBlob> bb = CDnnBlob::CreateVector( e, CT_Float, width );
			bx->CopyFrom( xs.data() ); bb->CopyFrom( b.data() );
			std::vector<float> weightsOfPass = w;
			for( int pass = 0; pass < 3; ++pass ) {
				if( pass == 1 ) for( float& v : weightsOfPass ) v = -0.5f * v;
				if( pass == 2 ) {
					for( float& v : weightsOfPass ) v = 0.01f;
					e.VectorFill( bw->GetData(), 0.01f, bw->GetDataSize() );
				} else {
					bw->CopyFrom( weightsOfPass.data() );
				}
				CPtr<CDnnBlob> product = CDnnBlob::CreateMatrix( e, CT_Float, tall, width );
				product->Fill( -7.f );
				e.MultiplyMatrixByTransposedMatrix( bx->GetData(), tall, depth, depth, bw->GetData(), width, depth, product->GetData(),
					width, tall * width );
				e.AddVectorToMatrixRows( 1, product->GetData(), product->GetData(), tall, width, bb->GetData() );
				std::vector<double> want( static_cast<size_t>( tall ) * width );
				for( int r = 0; r < tall; ++r ) for( int c = 0; c < width; ++c ) {
					double sum = b[c];
					for( int k = 0; k < depth; ++k ) sum += double( xs[r * depth + k] ) * weightsOfPass[c * depth + k];
					want[static_cast<size_t>( r ) * width + c] = sum;
				}
				compare( *product, want );
			}
		}
		*worstError = static_cast<float>( worst );
	} );
}

// A seeded random program over a handful of small buffers, made of the calls an engine may hold back, note or fuse
// (the element-wise and row / column broadcast calls, row sums, the fully connected product, copies, fills, frees),
// with operands chosen at random: in place or not, matrices that come back in later calls, row vectors that share
// one allocation, buffers released and allocated again in the middle.  Whatever an engine does between the calls, the
// final contents of every buffer must be those of carrying out each call when it is made; the caller compares the
// state two engines end in.  `state` receives matrices, then vectors, then scalars (stateFloats in all).
CDNN_API int cdnn_selftest_random_program( void* enginePtr, unsigned long long seed, int steps, float* state, int stateFloats )
{
	return guarded( [&] {
		IMathEngine& e = *static_cast<IMathEngine*>( enginePtr );
		// seeds from 5 000 000 on run on 1024-row matrices (from there an engine may keep a prepared form of a product's
		// weights) and draw the steps 0..21, 39 and 40; the state then holds the first 24 rows of everything
		// seeds from 6 000 000 on: small matrices again, all of the above but 39 and 40, and the padded pooling of a
		// network's stem, 41..45
		const bool tall = seed >= 5000000ull && seed < 6000000ull;
		const int seenRows = 24, rows = tall ? 1024 : seenRows, width = 32, size = rows * width;
		const int matrices = 6, rowVectors = 4, colVectors = 3, scalars = 2, weights = 2;
		if( stateFloats != matrices * seenRows * width + rowVectors * seenRows + colVectors * width + scalars ) throw std::logic_error( "state size" );
		CSplitMix rng( seed );
		auto fill = [&]( CDnnBlob& blob, float low, float high ) {
			std::vector<float> v( static_cast<size_t>( blob.GetDataSize() ) );
			for( float& x : v ) x = static_cast<float>( low + ( high - low ) * rng.uniform() );
			blob.CopyFrom( v.data() );
		};
		std::vector<CPtr<CDnnBlob>> m( matrices ), w( weights ), col( colVectors );
		for( auto& b : m ) { b = CDnnBlob::CreateMatrix( e, CT_Float, rows, width ); fill( *b, -1.f, 1.f ); }
		for( auto& b : w ) { b = CDnnBlob::CreateMatrix( e, CT_Float, width, width ); fill( *b, -0.3f, 0.3f ); }
		for( auto& b : col ) { b = CDnnBlob::CreateVector( e, CT_Float, width ); fill( *b, 0.5f, 1.5f ); }
		// the row vectors live two to a blob (as a normalisation keeps its mean and its 1/sigma), the scalars in one blob
		CPtr<CDnnBlob> rowPairs[2] = { CDnnBlob::CreateVector( e, CT_Float, 2 * rows ), CDnnBlob::CreateVector( e, CT_Float, 2 * rows ) };
		fill( *rowPairs[0], 0.5f, 1.5f ); fill( *rowPairs[1], -0.5f, 0.5f );
		CPtr<CDnnBlob> scalarBlob = CDnnBlob::CreateVector( e, CT_Float, scalars );
		fill( *scalarBlob, 0.5f, 1.7f );
		auto rowVec = [&]( int i ) { return rowPairs[i / 2]->GetData() + ( i % 2 ) * rows; };
		auto scalar = [&]( int i ) { return scalarBlob->GetData() + i; };
		auto pick = [&]( int n ) { return static_cast<int>( rng.next() % n ); };
		// attention: 2 heads, 128 queries and keys of depth 64 (the smallest shape an engine may treat as a score chain);
		// what these calls compute reaches the compared state through copies of 24 x 32 pieces into the matrices above
		const int heads = 2, seq = 128, depth = 64, scoreSize = heads * seq * seq, headSize = heads * seq * depth;
		CPtr<CDnnBlob> q, kt, v, mask, attended, scores[2];
		if( seed >= 3000000ull ) {
			q = CDnnBlob::CreateVector( e, CT_Float, headSize ); fill( *q, -1.f, 1.f );
			kt = CDnnBlob::CreateVector( e, CT_Float, headSize ); fill( *kt, -1.f, 1.f );
			v = CDnnBlob::CreateVector( e, CT_Float, headSize ); fill( *v, -1.f, 1.f );
			mask = CDnnBlob::CreateVector( e, CT_Float, seq * seq ); fill( *mask, -0.5f, 0.5f );
			attended = CDnnBlob::CreateVector( e, CT_Float, headSize ); fill( *attended, -1.f, 1.f );
			for( auto& b : scores ) { b = CDnnBlob::CreateVector( e, CT_Float, scoreSize ); fill( *b, -1.f, 1.f ); }
		}
		// convolution: 3 x 3, padding 1, 32 -> 32 channels on 2 x 12 x 12 images, so that any image may follow any other
		const int images = 3, imageSize = 2 * 12 * 12 * 32, filterSize = 32 * 9 * 32;
		CPtr<CDnnBlob> image[3], filter[2], freeTerms[2], zero;
		std::unique_ptr<CConvolutionDesc> convolution;
		if( seed >= 4000000ull ) {
			for( auto& b : image ) { b = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 12, 12, 32 ); fill( *b, -1.f, 1.f ); }
			for( auto& b : filter ) { b = CDnnBlob::CreateTensor( e, CT_Float, { 1, 32, 1, 3, 3, 1, 32 } ); fill( *b, -0.08f, 0.08f ); }
			for( auto& b : freeTerms ) { b = CDnnBlob::CreateVector( e, CT_Float, 32 ); fill( *b, -0.2f, 0.2f ); }
			zero = CDnnBlob::CreateVector( e, CT_Float, 1 );
			zero->Fill( 0.f );
			convolution.reset( e.InitBlobConvolution( image[0]->GetDesc(), 1, 1, 1, 1, 1, 1, filter[0]->GetDesc(), image[1]->GetDesc() ) );
		}
		// padded pooling: an image with a border of one pixel, then 3 x 3 maxima with stride 2
		const int paddedSize = 2 * 14 * 14 * 32, pooledSize = 2 * 6 * 6 * 32;
		const float border = 0.25f; // above part of the data: the border decides some maxima
		CPtr<CDnnBlob> padded[2], pooled;
		std::unique_ptr<CMaxPoolingDesc> pooling;
		if( seed >= 6000000ull ) {
			for( auto& b : padded ) { b = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 14, 14, 32 ); fill( *b, -1.f, 1.f ); }
			pooled = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 6, 6, 32 );
			fill( *pooled, -1.f, 1.f );
			pooling.reset( e.InitMaxPooling( padded[0]->GetDesc(), 3, 3, 2, 2, pooled->GetDesc() ) );
		}
		auto pad = [&]( int from, int to ) {
			e.BlobResizeImage( image[from]->GetDesc(), image[from]->GetData(), 1, 1, 1, 1, border, padded[to]->GetDesc(), padded[to]->GetData() );
		};
		auto convolve = [&]( int from, int to, int which ) {
			const CConstFloatHandle freeTerm = freeTerms[which]->GetData();
			e.BlobConvolution( *convolution, image[from]->GetData(), filter[which]->GetData(), &freeTerm, image[to]->GetData() );
		};
		for( int step = 0; step < steps; ++step ) {
			const int a = pick( matrices ), b = pick( matrices ), c = pick( matrices );
			const int r = pick( rowVectors ), k = pick( colVectors ), s = pick( scalars );
			// seeds from 1 000 000 on also draw the composite steps 15..19, seeds from 2 000 000 on the steps 20 and 21 with
			// temporaries that die early, seeds from 3 000 000 on the calls of attention on buffers of their own, 22..30,
			// seeds from 4 000 000 on the calls around a convolution, 31..38 (smaller seeds keep the programs they always made)
			int op = pick( seed >= 6000000ull ? 44 : tall ? 24 : seed >= 4000000ull ? 39 : seed >= 3000000ull ? 31
				: seed >= 2000000ull ? 22 : seed >= 1000000ull ? 20 : 15 );
			if( tall && op >= 22 ) op += 17;
			if( seed >= 6000000ull && op >= 39 ) op += 2; // 39..43 -> 41..45
			switch( op ) {
				case 0: e.AddVectorToMatrixColumns( m[a]->GetData(), m[b]->GetData(), rows, width, rowVec( r ) ); break;
				case 1: e.VectorEltwiseMultiply( m[a]->GetData(), m[b]->GetData(), m[c]->GetData(), size ); break;
				case 2:
					e.SumMatrixColumns( rowVec( r ), m[a]->GetData(), rows, width );
					e.VectorTanh( rowVec( r ), rowVec( r ), rows );
					break;
				case 3: e.MultiplyDiagMatrixByMatrix( rowVec( r ), rows, m[a]->GetData(), width, m[b]->GetData(), size ); break;
				case 4: e.MultiplyMatrixByDiagMatrix( m[a]->GetData(), rows, width, col[k]->GetData(), m[b]->GetData(), size ); break;
				case 5: e.AddVectorToMatrixRows( 1, m[a]->GetData(), m[b]->GetData(), rows, width, col[k]->GetData() ); break;
				case 6: e.VectorMultiply( m[a]->GetData(), m[b]->GetData(), size, scalar( s ) ); break;
				case 7: e.VectorSigmoid( m[a]->GetData(), m[b]->GetData(), size ); break;
				case 8: e.VectorAdd( m[a]->GetData(), m[b]->GetData(), m[c]->GetData(), size ); break;
				case 9:
					if( a != b ) {
						e.MultiplyMatrixByTransposedMatrix( m[a]->GetData(), rows, width, width, w[pick( weights )]->GetData(), width, width,
							m[b]->GetData(), width, size );
					}
					break;
				case 10: if( a != b ) e.VectorCopy( m[b]->GetData(), m[a]->GetData(), size ); break;
				case 11: // released and allocated again: whatever was held back for the old buffer must not land in the new one
					m[a] = nullptr;
					m[a] = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
					m[a]->Fill( static_cast<float>( rng.uniform() - 0.5 ) );
					break;
				case 12: e.VectorFill( rowVec( r ), static_cast<float>( rng.uniform() + 0.5 ), rows ); break;
				case 13: e.VectorTanh( m[a]->GetData(), m[a]->GetData(), size ); break;
				case 14: fill( *w[pick( weights )], -0.3f, 0.3f ); break; // new weights: a product held back must have used the old ones
				case 15: // a fully connected layer: product, free terms in place, maybe the sum with another tensor
					if( a != b ) {
						e.MultiplyMatrixByTransposedMatrix( m[a]->GetData(), rows, width, width, w[pick( weights )]->GetData(), width, width,
							m[b]->GetData(), width, size );
						e.AddVectorToMatrixRows( 1, m[b]->GetData(), m[b]->GetData(), rows, width, col[k]->GetData() );
						if( pick( 2 ) == 0 ) e.VectorAdd( m[b]->GetData(), m[c]->GetData(), m[pick( matrices )]->GetData(), size );
					}
					break;
				case 16: // the gate x * sigmoid( s * x ), all of it or only its first steps
					if( a != b ) {
						e.VectorMultiply( m[a]->GetData(), m[b]->GetData(), size, scalar( s ) );
						if( pick( 4 ) != 0 ) {
							e.VectorSigmoid( m[b]->GetData(), m[b]->GetData(), size );
							if( pick( 4 ) != 0 ) e.VectorEltwiseMultiply( m[a]->GetData(), m[b]->GetData(), m[b]->GetData(), size );
						}
					}
					break;
				case 17: { // the steps of an object normalisation, in place or not, cut short at random
					const int t = pick( 2 ) == 0 ? a : b;
					e.AddVectorToMatrixColumns( m[a]->GetData(), m[t]->GetData(), rows, width, rowVec( r ) );
					switch( pick( 3 ) ) {
						case 0:
							e.VectorEltwiseMultiply( m[t]->GetData(), m[t]->GetData(), m[t]->GetData(), size );
							if( pick( 2 ) == 0 ) {
								e.SumMatrixColumns( rowVec( ( r + 1 ) % rowVectors ), m[t]->GetData(), rows, width );
								e.VectorTanh( rowVec( ( r + 1 ) % rowVectors ), rowVec( ( r + 1 ) % rowVectors ), rows );
							}
							break;
						case 1: {
							e.MultiplyDiagMatrixByMatrix( rowVec( ( r + 2 ) % rowVectors ), rows, m[t]->GetData(), width, m[t]->GetData(), size );
							const int u = pick( 2 ) == 0 ? t : c;
							if( pick( 3 ) != 0 ) e.MultiplyMatrixByDiagMatrix( m[t]->GetData(), rows, width, col[k]->GetData(), m[u]->GetData(), size );
							if( pick( 3 ) != 0 ) e.AddVectorToMatrixRows( 1, m[u]->GetData(), m[u]->GetData(), rows, width, col[( k + 1 ) % colVectors]->GetData() );
							break;
						}
						default: break;
					}
					break;
				}
				case 18: // scale in place, maybe shift by columns, softmax by rows: attention's row chain without the products
					e.VectorMultiply( m[a]->GetData(), m[a]->GetData(), size, scalar( s ) );
					if( pick( 2 ) == 0 ) e.AddVectorToMatrixRows( 1, m[a]->GetData(), m[a]->GetData(), rows, width, col[k]->GetData() );
					if( pick( 4 ) != 0 ) e.MatrixSoftmaxByRows( m[a]->GetData(), rows, width, pick( 2 ) == 0 ? m[a]->GetData() : m[b]->GetData() );
					break;
				case 19: e.MultiplyDiagMatrixByMatrix( rowVec( r ), rows, m[a]->GetData(), width, m[a]->GetData(), size ); break;
				case 20: { // a normalisation whose row statistics live in ONE stack variable that dies while the matrix is only noted
					CFloatHandleStackVar stats( e, 2 * rows );
					e.SumMatrixColumns( stats.GetHandle(), m[a]->GetData(), rows, width );
					e.VectorTanh( stats.GetHandle(), stats.GetHandle(), rows );
					e.VectorFill( stats.GetHandle() + rows, static_cast<float>( rng.uniform() + 0.5 ), rows );
					const int t = pick( 2 ) == 0 ? a : b;
					e.AddVectorToMatrixColumns( m[a]->GetData(), m[t]->GetData(), rows, width, stats.GetHandle() );
					if( pick( 2 ) == 0 ) e.VectorAddValue( stats.GetHandle() + rows, stats.GetHandle() + rows, rows, scalar( s ) );
					if( pick( 3 ) != 0 ) e.MultiplyDiagMatrixByMatrix( stats.GetHandle() + rows, rows, m[t]->GetData(), width, m[t]->GetData(), size );
					if( pick( 2 ) == 0 ) {
						const int u = pick( 2 ) == 0 ? t : c;
						e.MultiplyMatrixByDiagMatrix( m[t]->GetData(), rows, width, col[k]->GetData(), m[u]->GetData(), size );
					}
					break;
				}
				case 21: // a fully connected layer whose input blob is released right after the call, as reuse-memory mode does
					if( a != b ) {
						CPtr<CDnnBlob> input = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
						e.VectorCopy( input->GetData(), m[a]->GetData(), size );
						e.MultiplyMatrixByTransposedMatrix( input->GetData(), rows, width, width, w[pick( weights )]->GetData(), width, width,
							m[b]->GetData(), width, size );
						if( pick( 2 ) == 0 ) e.AddVectorToMatrixRows( 1, m[b]->GetData(), m[b]->GetData(), rows, width, col[k]->GetData() );
						input = nullptr;
						if( pick( 2 ) == 0 ) { // and the block may come back at once, for something else
							CPtr<CDnnBlob> other = CDnnBlob::CreateMatrix( e, CT_Float, rows, width );
							other->Fill( 3.f );
							e.VectorAdd( m[c]->GetData(), other->GetData(), m[c]->GetData(), size );
							e.VectorTanh( m[c]->GetData(), m[c]->GetData(), size );
						}
					}
					break;
				case 22: // scores = Q * Kt
					e.MultiplyMatrixByMatrix( heads, q->GetData(), seq, depth, kt->GetData(), seq, scores[a % 2]->GetData(), scoreSize );
					break;
				case 23: e.VectorMultiply( scores[a % 2]->GetData(), scores[a % 2]->GetData(), scoreSize, scalar( s ) ); break;
				case 24: // + mask, in place or into the other score buffer
					e.AddVectorToMatrixRows( 1, scores[a % 2]->GetData(), scores[b % 2]->GetData(), heads, seq * seq, mask->GetData() );
					break;
				case 25: e.MatrixSoftmaxByRows( scores[a % 2]->GetData(), heads * seq, seq, scores[b % 2]->GetData() ); break;
				case 26: // out = scores * V; a piece of it goes into the compared state
					e.MultiplyMatrixByMatrix( heads, scores[a % 2]->GetData(), seq, seq, v->GetData(), depth, attended->GetData(), headSize );
					e.VectorCopy( m[c]->GetData(), attended->GetData() + pick( headSize - size ), size );
					e.VectorTanh( m[c]->GetData(), m[c]->GetData(), size );
					break;
				case 27: // somebody reads a score buffer
					e.VectorCopy( m[c]->GetData(), scores[a % 2]->GetData() + pick( scoreSize - size ), size );
					e.VectorTanh( m[c]->GetData(), m[c]->GetData(), size );
					break;
				case 28: { // an operand of the chain changes while scores may still be only noted
					CDnnBlob* operands[4] = { q.Ptr(), kt.Ptr(), v.Ptr(), mask.Ptr() };
					CDnnBlob* chosen = operands[pick( 4 )];
					e.VectorTanh( chosen->GetData(), chosen->GetData(), chosen->GetDataSize() );
					break;
				}
				case 29: { // the whole chain as CMultiheadAttentionLayer issues it, scale and mask at random
					const int x = a % 2, y = pick( 2 ), z = pick( 2 );
					e.MultiplyMatrixByMatrix( heads, q->GetData(), seq, depth, kt->GetData(), seq, scores[x]->GetData(), scoreSize );
					if( pick( 4 ) != 0 ) e.VectorMultiply( scores[x]->GetData(), scores[x]->GetData(), scoreSize, scalar( s ) );
					int at = x;
					if( pick( 2 ) == 0 ) {
						e.AddVectorToMatrixRows( 1, scores[x]->GetData(), scores[y]->GetData(), heads, seq * seq, mask->GetData() );
						at = y;
					}
					e.MatrixSoftmaxByRows( scores[at]->GetData(), heads * seq, seq, scores[z]->GetData() );
					e.MultiplyMatrixByMatrix( heads, scores[z]->GetData(), seq, seq, v->GetData(), depth, attended->GetData(), headSize );
					e.VectorCopy( m[c]->GetData(), attended->GetData() + pick( headSize - size ), size );
					break;
				}
				case 31: if( a % images != b % images ) convolve( a % images, b % images, k % 2 ); break;
				case 32: // another image added in place: the residual sum of a block
					if( a % images != b % images ) {
						e.VectorAdd( image[a % images]->GetData(), image[b % images]->GetData(), image[a % images]->GetData(), imageSize );
					}
					break;
				case 33: e.VectorReLU( image[a % images]->GetData(), image[a % images]->GetData(), imageSize, zero->GetData() ); break;
				case 34: fill( *filter[k % 2], -0.08f, 0.08f ); break; // new weights from the host
				case 35: // the filter written on the device
					e.VectorMultiply( filter[k % 2]->GetData(), filter[k % 2]->GetData(), filterSize, scalar( s ) );
					e.VectorTanh( filter[k % 2]->GetData(), filter[k % 2]->GetData(), filterSize );
					break;
				case 36: // an image is released and allocated again
					image[a % images] = nullptr;
					image[a % images] = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 12, 12, 32 );
					image[a % images]->Fill( static_cast<float>( rng.uniform() - 0.5 ) );
					break;
				case 37: // somebody reads an image; it is also kept bounded
					e.VectorTanh( image[a % images]->GetData(), image[a % images]->GetData(), imageSize );
					e.VectorCopy( m[c]->GetData(), image[a % images]->GetData() + pick( imageSize - size ), size );
					break;
				case 38: { // a residual block's tail: convolution, + shortcut, ReLU; the source may be released at once
					const int from = a % images, to = ( from + 1 + pick( 2 ) ) % images, shortcut = pick( images );
					convolve( from, to, k % 2 );
					const bool early = pick( 2 ) == 0;
					if( early ) image[from] = nullptr;
					if( shortcut != to && ( !early || shortcut != from ) && pick( 4 ) != 0 ) {
						e.VectorAdd( image[to]->GetData(), image[shortcut]->GetData(), image[to]->GetData(), imageSize );
					}
					if( pick( 4 ) != 0 ) e.VectorReLU( image[to]->GetData(), image[to]->GetData(), imageSize, zero->GetData() );
					if( early ) {
						image[from] = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 12, 12, 32 );
						image[from]->Fill( static_cast<float>( rng.uniform() - 0.5 ) );
					}
					e.VectorCopy( m[c]->GetData(), image[to]->GetData() + pick( imageSize - size ), size );
					e.VectorTanh( m[c]->GetData(), m[c]->GetData(), size );
					break;
				}
				case 41: pad( a % images, b % 2 ); break;
				case 42: // pooled = maxima of a padded image; a piece of it goes into the compared state
					e.BlobMaxPooling( *pooling, padded[a % 2]->GetData(), nullptr, pooled->GetData() );
					e.VectorCopy( m[c]->GetData(), pooled->GetData() + pick( pooledSize - size ), size );
					break;
				case 43: // somebody reads a padded image
					e.VectorCopy( m[c]->GetData(), padded[a % 2]->GetData() + pick( paddedSize - size ), size );
					break;
				case 44: { // a stem: convolution, ReLU, border, pooling; the convolution's result may be released at once
					const int from = a % images, to = ( from + 1 + pick( 2 ) ) % images, x = pick( 2 );
					convolve( from, to, k % 2 );
					if( pick( 4 ) != 0 ) e.VectorReLU( image[to]->GetData(), image[to]->GetData(), imageSize, zero->GetData() );
					pad( to, x );
					const bool early = pick( 2 ) == 0;
					if( early ) {
						image[to] = nullptr;
						image[to] = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 12, 12, 32 );
						image[to]->Fill( static_cast<float>( rng.uniform() - 0.5 ) );
					}
					if( pick( 4 ) != 0 ) {
						e.BlobMaxPooling( *pooling, padded[x]->GetData(), nullptr, pooled->GetData() );
						e.VectorCopy( m[c]->GetData(), pooled->GetData() + pick( pooledSize - size ), size );
					}
					break;
				}
				case 45: // a padded image is released and allocated again
					padded[a % 2] = nullptr;
					padded[a % 2] = CDnnBlob::Create2DImageBlob( e, CT_Float, 1, 2, 14, 14, 32 );
					padded[a % 2]->Fill( static_cast<float>( rng.uniform() - 0.5 ) );
					break;
				case 39: { // the weights written on the device
					const int which = pick( weights );
					e.VectorTanh( w[which]->GetData(), w[which]->GetData(), width * width );
					break;
				}
				case 40: { // the weights released and allocated again
					const int which = pick( weights );
					w[which] = nullptr;
					w[which] = CDnnBlob::CreateMatrix( e, CT_Float, width, width );
					fill( *w[which], -0.3f, 0.3f );
					break;
				}
				case 30: // a score buffer is released and allocated again
					scores[a % 2] = nullptr;
					scores[a % 2] = CDnnBlob::CreateVector( e, CT_Float, scoreSize );
					scores[a % 2]->Fill( static_cast<float>( rng.uniform() - 0.5 ) );
					break;
			}
			if( step % 3 == 2 ) e.VectorTanh( m[c]->GetData(), m[c]->GetData(), size ); // keeps magnitudes bounded
		}
		float* out = state;
		std::vector<float> whole( static_cast<size_t>( size ) );
		for( auto& blob : m ) {
			blob->CopyTo( whole.data() );
			std::copy( whole.begin(), whole.begin() + seenRows * width, out );
			out += seenRows * width;
		}
		for( int i = 0; i < 2; ++i ) {
			rowPairs[i]->CopyTo( whole.data() );
			for( int half = 0; half < 2; ++half ) {
				std::copy( whole.begin() + half * rows, whole.begin() + half * rows + seenRows, out );
				out += seenRows;
			}
		}
		for( auto& blob : col ) { blob->CopyTo( out ); out += width; }
		scalarBlob->CopyTo( out );
	} );
}

// Two distributed engines (CreateDistributedCudaMathEngines on devices[0..1]).  First one AllReduce from two host
// threads: every element must come out as the mean.  Then, between steps and with no collective in flight, engine 1
// calls AbortDistributed; the next AllReduce on engine 0 has to end with NeoML's "Stopping due to error in another
// thread." instead of waiting for a peer that will not come.  `message` receives what that call raised.
CDNN_API int cdnn_selftest_abort_distributed( const int* devices, char* message, int messageSize )
{
	return guarded( [&] {
		SetMathEngineExceptionHandler( GetExceptionHandler() );
		IMathEngine* raw[2] = { nullptr, nullptr };
		CreateDistributedCudaMathEngines( raw, 2, devices, 0 );
		std::unique_ptr<IMathEngine> engines[2] = { std::unique_ptr<IMathEngine>( raw[0] ), std::unique_ptr<IMathEngine>( raw[1] ) };
		if( !engines[0] || !engines[1] ) throw std::logic_error( "the distributed factory returned no engines" );
		if( !engines[0]->IsDistributed() || engines[1]->GetDistributedInfo().Threads != 2 ) throw std::logic_error( "distributed info is wrong" );
		const int n = 1000;
		std::string errors[2];
		{
			std::thread workers[2];
			for( int r = 0; r < 2; ++r ) {
				workers[r] = std::thread( [&, r] {
					try {
						CFloatHandleVar data( *engines[r], n );
						std::vector<float> host( n );
						for( int i = 0; i < n; ++i ) host[i] = static_cast<float>( ( r + 1 ) * i );
						engines[r]->DataExchangeTyped<float>( data.GetHandle(), host.data(), n );
						engines[r]->AllReduce( data.GetHandle(), n );
						engines[r]->DataExchangeTyped<float>( host.data(), data.GetHandle(), n );
						for( int i = 0; i < n; ++i ) {
							if( host[i] != 1.5f * i ) throw std::logic_error( "AllReduce did not produce the mean" );
						}
					} catch( const std::exception& ex ) {
						errors[r] = ex.what();
					}
				} );
			}
			for( std::thread& t : workers ) t.join();
		}
		if( !errors[0].empty() || !errors[1].empty() ) throw std::logic_error( "AllReduce: " + errors[0] + " " + errors[1] );
		engines[1]->AbortDistributed();
		std::string raised;
		try {
			CFloatHandleVar data( *engines[0], n );
			engines[0]->VectorFill( data.GetHandle(), 1.f, n );
			engines[0]->AllReduce( data.GetHandle(), n );
		} catch( const std::exception& ex ) {
			raised = ex.what();
		}
		std::snprintf( message, messageSize, "%s", raised.c_str() );
	} );
}
