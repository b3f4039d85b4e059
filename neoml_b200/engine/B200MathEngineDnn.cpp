// CB200MathEngine: the IDnnEngine methods of the inference hot path (convolution, channelwise convolution, pooling,
// image resize, the fused MobileNetV2 block and the rowwise descriptors it needs).
#include "B200MathEngine.h"

#include <neoml_b200.h>

#include <cuda_runtime.h>

namespace NeoML {

namespace {

void raise( const char* message )
{
	GetMathEngineExceptionHandler()->OnAssert( message, L"B200MathEngineDnn", 0, 0 );
}

bool activationOf( TActivationFunction f, int& act )
{
	switch( f ) {
		case AF_Linear: act = NB200_ACT_NONE; return true;
		case AF_ReLU: act = NB200_ACT_RELU; return true;
		case AF_HSwish: act = NB200_ACT_HSWISH; return true;
		default: act = NB200_ACT_NONE; return false;
	}
}

// descriptors: plain copies of the geometry, owned by the caller (deleted with `delete`, NeoMathEngine.h:723,750)
struct CB200ConvolutionDesc : public CConvolutionDesc {
	nb200_conv_desc d;
};
struct CB200ChannelwiseDesc : public CChannelwiseConvolutionDesc {
	nb200_chconv_desc d;
};
struct CB200PoolingGeometry {
	int batch, h, w, c, fh, fw, sh, sw;
};
struct CB200MaxPoolingDesc : public CMaxPoolingDesc {
	CB200PoolingGeometry g;
};
struct CB200MeanPoolingDesc : public CMeanPoolingDesc {
	CB200PoolingGeometry g;
};
// The rowwise MobileNetV2 descriptor captures the weight pointers, as the reference's does
// (GPU/CUDA/Rowwise/CudaRowwiseMobileNetV2.h:94-108)
struct CB200RowwiseMobileNetV2 : public CRowwiseOperationDesc {
	int inputChannels, expandedChannels, outputChannels, stride;
	bool residual;
	int actExpand, actChannelwise;
	float actExpandParam, actChannelwiseParam;
	const float* expandFilter;
	const float* expandFreeTerm;
	const float* channelwiseFilter;
	const float* channelwiseFreeTerm;
	const float* downFilter;
	const float* downFreeTerm;
};

// A blob as a channels-last image batch: objects x height x width x (depth * channels)
CB200PoolingGeometry imageOf( const CBlobDesc& b )
{
	return { b.ObjectCount(), b.Height(), b.Width(), b.Depth() * b.Channels(), 0, 0, 0, 0 };
}

} // namespace

//---------------------------------------------------------------------------------------------------------------------

CConvolutionDesc* CB200MathEngine::InitBlobConvolution( const CBlobDesc& input, int paddingHeight, int paddingWidth,
	int strideHeight, int strideWidth, int dilationHeight, int dilationWidth, const CBlobDesc& filter, const CBlobDesc& output )
{
	if( input.Depth() != 1 || filter.Depth() != 1 ) { notImplemented( "InitBlobConvolution (depth > 1)" ); return nullptr; }
	CB200ConvolutionDesc* desc = new CB200ConvolutionDesc();
	desc->d = { input.ObjectCount(), input.Height(), input.Width(), input.Channels(), filter.ObjectCount(), filter.Height(),
		filter.Width(), paddingHeight, paddingWidth, strideHeight, strideWidth, dilationHeight, dilationWidth,
		output.Height(), output.Width() };
	if( filter.Channels() != input.Channels() || output.Channels() * output.Depth() != filter.ObjectCount()
		|| output.ObjectCount() != input.ObjectCount() ) {
		delete desc;
		raise( "InitBlobConvolution: input, filter and output descriptors do not fit together" );
		return nullptr;
	}
	return desc;
}

void CB200MathEngine::BlobConvolution( const CConvolutionDesc& convDesc, const CConstFloatHandle& source,
	const CConstFloatHandle& filter, const CConstFloatHandle* freeTerm, const CFloatHandle& result )
{
	const nb200_conv_desc& d = static_cast<const CB200ConvolutionDesc&>( convDesc ).d;
	enter(); // launches an earlier convolution that is still held back
	// The call is recorded, not launched: an in-place VectorAdd / VectorReLU that follows rides in its epilogue, any
	// other call launches it first (enter()), so the caller cannot observe the delay.
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	pending = CPendingConvolution();
	pending.d = d;
	pending.source = raw( source );
	pending.filter = raw( filter );
	pending.freeTerm = freeTerm != nullptr ? raw( *freeTerm ) : nullptr;
	pending.result = raw( result );
	pending.resultFloats = static_cast<long long>( d.batch ) * d.ho * d.wo * d.k;
	pending.active = true;
}

CChannelwiseConvolutionDesc* CB200MathEngine::InitBlobChannelwiseConvolution( const CBlobDesc& input, int paddingHeight,
	int paddingWidth, int strideHeight, int strideWidth, const CBlobDesc& filter, const CBlobDesc*, const CBlobDesc& output )
{
	CB200ChannelwiseDesc* desc = new CB200ChannelwiseDesc();
	desc->d = { input.ObjectCount(), input.Height(), input.Width(), input.Depth() * input.Channels(), filter.Height(),
		filter.Width(), paddingHeight, paddingWidth, strideHeight, strideWidth, output.Height(), output.Width() };
	return desc;
}

void CB200MathEngine::BlobChannelwiseConvolution( const CChannelwiseConvolutionDesc& convDesc, const CConstFloatHandle& source,
	const CConstFloatHandle& filter, const CConstFloatHandle* freeTerm, const CFloatHandle& result )
{
	const nb200_chconv_desc& d = static_cast<const CB200ChannelwiseDesc&>( convDesc ).d;
	enter();
	check( nb200_blob_channelwise_convolution( stream, &d, raw( source ), raw( filter ),
		freeTerm != nullptr ? raw( *freeTerm ) : nullptr, raw( result ), NB200_ACT_NONE, 0.f ), "BlobChannelwiseConvolution" );
}

CMaxPoolingDesc* CB200MathEngine::InitMaxPooling( const CBlobDesc& source, int filterHeight, int filterWidth, int strideHeight,
	int strideWidth, const CBlobDesc& )
{
	CB200MaxPoolingDesc* desc = new CB200MaxPoolingDesc();
	desc->g = imageOf( source );
	desc->g.fh = filterHeight; desc->g.fw = filterWidth; desc->g.sh = strideHeight; desc->g.sw = strideWidth;
	return desc;
}

void CB200MathEngine::BlobMaxPooling( const CMaxPoolingDesc& poolDesc, const CConstFloatHandle& source,
	const CIntHandle* maxIndices, const CFloatHandle& result )
{
	const CB200PoolingGeometry& g = static_cast<const CB200MaxPoolingDesc&>( poolDesc ).g;
	enter();
	check( nb200_blob_max_pooling( stream, g.batch, g.h, g.w, g.c, g.fh, g.fw, g.sh, g.sw, raw( source ), raw( result ),
		maxIndices != nullptr ? raw( *maxIndices ) : nullptr ), "BlobMaxPooling" );
}

CMeanPoolingDesc* CB200MathEngine::InitMeanPooling( const CBlobDesc& source, int filterHeight, int filterWidth, int strideHeight,
	int strideWidth, const CBlobDesc& )
{
	CB200MeanPoolingDesc* desc = new CB200MeanPoolingDesc();
	desc->g = imageOf( source );
	desc->g.fh = filterHeight; desc->g.fw = filterWidth; desc->g.sh = strideHeight; desc->g.sw = strideWidth;
	return desc;
}

void CB200MathEngine::BlobMeanPooling( const CMeanPoolingDesc& poolDesc, const CConstFloatHandle& source, const CFloatHandle& result )
{
	const CB200PoolingGeometry& g = static_cast<const CB200MeanPoolingDesc&>( poolDesc ).g;
	enter();
	check( nb200_blob_mean_pooling( stream, g.batch, g.h, g.w, g.c, g.fh, g.fw, g.sh, g.sw, raw( source ), raw( result ) ),
		"BlobMeanPooling" );
}

void CB200MathEngine::BlobResizeImage( const CBlobDesc& from, const CFloatHandle& fromData, int deltaLeft, int deltaRight,
	int deltaTop, int deltaBottom, TBlobResizePadding padding, float defaultValue, const CBlobDesc&, const CFloatHandle& toData )
{
	enter();
	check( nb200_blob_resize_image( stream, from.ObjectCount(), from.Height(), from.Width(), from.Depth() * from.Channels(),
		deltaLeft, deltaRight, deltaTop, deltaBottom, static_cast<int>( padding ), defaultValue, raw( fromData ), raw( toData ) ),
		"BlobResizeImage" );
}

//---------------------------------------------------------------------------------------------------------------------
// fused MobileNetV2 block and the rowwise plumbing CMobileNetV2BlockLayer::Reshape calls
// (NeoML/src/Dnn/Layers/MobileNetV2BlockLayer.cpp:218-251)

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseMobileNetV2( int inputChannels, const CConstFloatHandle& expandFilter,
	const CConstFloatHandle* expandFreeTerm, int expandedChannels, TActivationFunction expandActivation, float expandReluParam,
	const CConstFloatHandle& channelwiseFilter, const CConstFloatHandle* channelwiseFreeTerm, int stride,
	TActivationFunction channelwiseActivation, float channelwiseReluParam, const CConstFloatHandle& downFilter,
	const CConstFloatHandle* downFreeTerm, int outputChannels, bool residual )
{
	int a1 = 0, a2 = 0;
	if( !activationOf( expandActivation, a1 ) || !activationOf( channelwiseActivation, a2 ) ) {
		notImplemented( "InitRowwiseMobileNetV2 (activation other than linear / ReLU / HSwish)" );
		return nullptr;
	}
	CB200RowwiseMobileNetV2* desc = new CB200RowwiseMobileNetV2();
	desc->inputChannels = inputChannels; desc->expandedChannels = expandedChannels; desc->outputChannels = outputChannels;
	desc->stride = stride; desc->residual = residual;
	desc->actExpand = a1; desc->actChannelwise = a2;
	desc->actExpandParam = expandReluParam; desc->actChannelwiseParam = channelwiseReluParam;
	desc->expandFilter = raw( expandFilter );
	desc->expandFreeTerm = expandFreeTerm != nullptr ? raw( *expandFreeTerm ) : nullptr;
	desc->channelwiseFilter = raw( channelwiseFilter );
	desc->channelwiseFreeTerm = channelwiseFreeTerm != nullptr ? raw( *channelwiseFreeTerm ) : nullptr;
	desc->downFilter = raw( downFilter );
	desc->downFreeTerm = downFreeTerm != nullptr ? raw( *downFreeTerm ) : nullptr;
	return desc;
}

CBlobDesc CB200MathEngine::RowwiseReshape( CRowwiseOperationDesc** operations, int operationCount, const CBlobDesc& input )
{
	CBlobDesc output = input;
	for( int i = 0; i < operationCount; ++i ) {
		const CB200RowwiseMobileNetV2* op = dynamic_cast<const CB200RowwiseMobileNetV2*>( operations[i] );
		if( op == nullptr ) { notImplemented( "RowwiseReshape (operation other than MobileNetV2)" ); return output; }
		output.SetDimSize( BD_Height, 1 + ( output.Height() - 1 ) / op->stride );
		output.SetDimSize( BD_Width, 1 + ( output.Width() - 1 ) / op->stride );
		output.SetDimSize( BD_Channels, op->outputChannels );
	}
	return output;
}

void CB200MathEngine::MobileNetV2Block( const CBlobDesc& inputDesc, const CBlobDesc&, const CRowwiseOperationDesc& rowwiseDesc,
	const CChannelwiseConvolutionDesc&, const CConstFloatHandle& inputHandle, const CFloatHandle& outputHandle )
{
	const CB200RowwiseMobileNetV2* op = dynamic_cast<const CB200RowwiseMobileNetV2*>( &rowwiseDesc );
	if( op == nullptr ) { raise( "MobileNetV2Block: the rowwise descriptor was not created by this engine" ); return; }
	nb200_mbv2_desc d = { inputDesc.ObjectCount(), inputDesc.Height(), inputDesc.Width(), op->inputChannels,
		op->expandedChannels, op->outputChannels, op->stride, op->residual ? 1 : 0, op->actExpand, op->actChannelwise,
		op->actExpandParam, op->actChannelwiseParam };
	enter();
	const size_t scratchFloats = nb200_mobilenetv2_scratch_floats( &d );
	CMemoryHandle scratch = StackAlloc( scratchFloats * sizeof( float ) );
	const int rc = nb200_mobilenetv2_block( stream, &d, raw( inputHandle ), op->expandFilter, op->expandFreeTerm,
		op->channelwiseFilter, op->channelwiseFreeTerm, op->downFilter, op->downFreeTerm, raw( outputHandle ),
		static_cast<float*>( CMemoryHandleInternal::GetRaw( scratch ) ), precision );
	StackFree( scratch );
	check( rc, "MobileNetV2Block" );
}

void CB200MathEngine::RowwiseExecute( const CBlobDesc& inputDesc, CRowwiseOperationDesc** operations, int operationCount,
	const CFloatHandle& input, const CFloatHandle& output )
{
	if( operationCount != 1 ) { notImplemented( "RowwiseExecute (chains longer than one MobileNetV2 block)" ); return; }
	const CB200RowwiseMobileNetV2* op = dynamic_cast<const CB200RowwiseMobileNetV2*>( operations[0] );
	if( op == nullptr ) { notImplemented( "RowwiseExecute (operation other than MobileNetV2)" ); return; }
	CB200ChannelwiseDesc unused;
	MobileNetV2Block( inputDesc, inputDesc, *op, unused, input, output );
}

} // namespace NeoML
