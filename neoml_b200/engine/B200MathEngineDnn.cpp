// CB200MathEngine: the IDnnEngine methods of the inference hot path (convolution, channelwise convolution, pooling,
// image resize).  The rowwise operations live in B200Rowwise.cpp.
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
struct CB200PoolingGeometry {
	int batch, h, w, c, fh, fw, sh, sw;
};
struct CB200MaxPoolingDesc : public CMaxPoolingDesc {
	CB200PoolingGeometry g;
};
struct CB200MeanPoolingDesc : public CMeanPoolingDesc {
	CB200PoolingGeometry g;
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
	CPendingConvolution call;
	call.d = d;
	call.source = raw( source );
	call.filter = raw( filter );
	call.freeTerm = freeTerm != nullptr ? raw( *freeTerm ) : nullptr;
	call.result = raw( result );
	call.resultFloats = static_cast<long long>( d.batch ) * d.ho * d.wo * d.k;
	call.sourceFloats = static_cast<long long>( d.batch ) * d.h * d.w * d.c;
	call.filterFloats = static_cast<long long>( d.k ) * d.r * d.s * d.c;
	call.filterAllocation = CMemoryHandleInternal::Base( filter );
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	if( pending.active && !pendingRows.active && independentOfPending( call ) ) {
		// the recorded convolution stays recorded (its sum and activation may still follow); this one runs now
		cudaSetDevice( device );
		launchConvolution( call );
		return;
	}
	enter(); // launches an earlier convolution that is still held back
	// The call is recorded, not launched: an in-place VectorAdd / VectorReLU that follows rides in its epilogue, any
	// other call launches it first (enter()), so the caller cannot observe the delay.
	pending = call;
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
	if( maxIndices == nullptr && lazyCount.load( std::memory_order_relaxed ) != 0 ) {
		// pooling over an image whose padding was only noted (BlobResizeImage): one pass over the unpadded image
		float* const out = raw( result ); // first: a result that overlaps what the note reads has the note carried out
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( source ), CLazyResult::K_Resize );
		if( at >= 0 ) {
			const CLazyResult& note = lazy[at];
			if( note.batch == g.batch && note.h + note.top + note.bottom == g.h && note.w + note.left + note.right == g.w
				&& note.c == g.c && nb200_blob_max_pooling_padded( stream, note.batch, note.h, note.w, note.c, note.left, note.right,
					note.top, note.bottom, note.value, g.fh, g.fw, g.sh, g.sw, note.from, out ) == NB200_OK ) {
				for( const CLazyResult::CInput& input : note.inputs ) noteUse( input.base );
				return;
			}
		}
	}
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
	const int channels = from.Depth() * from.Channels();
	if( static_cast<int>( padding ) == 0 && deltaLeft >= 0 && deltaRight >= 0 && deltaTop >= 0 && deltaBottom >= 0
		&& CMemoryHandleInternal::Base( fromData ) != CMemoryHandleInternal::Base( toData ) ) {
		// a constant border: noted, not written -- the pooling that usually follows reads the unpadded image instead
		// (see CLazyResult); anything else that touches the padded image finds it written
		CLazyResult note;
		note.kind = CLazyResult::K_Resize;
		note.result = raw( toData );
		note.resultBase = CMemoryHandleInternal::Base( toData );
		note.batch = from.ObjectCount(); note.h = from.Height(); note.w = from.Width(); note.c = channels;
		note.left = deltaLeft; note.right = deltaRight; note.top = deltaTop; note.bottom = deltaBottom;
		note.value = defaultValue;
		note.resultFloats = static_cast<long long>( note.batch ) * ( note.h + deltaTop + deltaBottom )
			* ( note.w + deltaLeft + deltaRight ) * channels;
		note.from = raw( CConstFloatHandle( fromData ) );
		note.Reads( fromData, static_cast<long long>( note.batch ) * note.h * note.w * channels );
		if( noteLazy( note ) ) return;
	}
	check( nb200_blob_resize_image( stream, from.ObjectCount(), from.Height(), from.Width(), channels,
		deltaLeft, deltaRight, deltaTop, deltaBottom, static_cast<int>( padding ), defaultValue, raw( fromData ), raw( toData ) ),
		"BlobResizeImage" );
}

} // namespace NeoML
