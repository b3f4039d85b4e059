// Rowwise operations (IDnnEngine::InitRowwise*, RowwiseReshape, RowwiseExecute, MobileNetV2Block, ChannelwiseWith1x1;
// NeoMathEngine.h:1066-1110).  NeoML's optimizer rewrites chains of image layers into these descriptors so that the
// CPU engine can walk them a few rows at a time and keep intermediates in cache.  A GPU gains nothing from row
// blocking, so here every operation works on whole blobs (the reference's CUDA engine does the same,
// GPU/CUDA/Rowwise/CudaRowwiseInterface.h:34-36); what the chain form does buy on this engine is fusion that needs no
// guessing: a convolution (dense or channelwise) directly followed by an activation becomes one launch, and the
// intermediates of a chain live in pool memory that is recycled between operations.
#include "B200MathEngine.h"

#include <neoml_b200.h>

#include <memory>
#include <vector>

namespace NeoML {

namespace {

void raise( const char* message )
{
	GetMathEngineExceptionHandler()->OnAssert( message, L"B200Rowwise", 0, 0 );
}

// activation of a fused tail: what the kernels' epilogues understand
struct CTail {
	int act = NB200_ACT_NONE;
	float param = 0.f;
};

bool tailOf( TActivationFunction f, float reluParam, CTail& tail )
{
	tail.param = 0.f;
	switch( f ) {
		case AF_Linear: tail.act = NB200_ACT_NONE; return true;
		case AF_ReLU: tail.act = NB200_ACT_RELU; tail.param = reluParam; return true;
		case AF_HSwish: tail.act = NB200_ACT_HSWISH; return true;
		default: tail.act = NB200_ACT_NONE; return false;
	}
}

int imageChannels( const CBlobDesc& d ) { return d.Depth() * d.Channels(); }

// One operation of a chain.  Reshape() fixes the geometry, Run() computes whole blobs.
struct CB200RowwiseOp : public CRowwiseOperationDesc {
	virtual CBlobDesc Reshape( const CBlobDesc& input ) = 0;
	// `tail`: an activation of the next operation that this one may absorb (only asked of operations that say so)
	virtual bool AbsorbsActivation() const { return false; }
	virtual void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& tail ) const = 0;
	virtual bool InPlace() const { return false; }
	CBlobDesc inDesc, outDesc;
};

//---------------------------------------------------------------------------------------------------------------------

struct CActivationOp : public CB200RowwiseOp {
	explicit CActivationOp( const CActivationDesc& d ) : desc( d ) {}

	CBlobDesc Reshape( const CBlobDesc& input ) override { inDesc = outDesc = input; return input; }
	bool InPlace() const override { return true; }

	// ReLU and HSwish can ride in the epilogue of the operation before
	bool AsTail( CTail& tail ) const
	{
		if( desc.GetType() == AF_ReLU ) {
			return tailOf( AF_ReLU, desc.HasParam() ? desc.GetParam<CReLUActivationParam>().UpperThreshold : 0.f, tail );
		}
		return desc.GetType() == AF_HSwish && tailOf( AF_HSwish, 0.f, tail );
	}

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& ) const override
	{
		const int n = inDesc.BlobSize();
		void* s = e.Stream();
		switch( desc.GetType() ) {
			case AF_ReLU:
				e.Check( nb200_vector_op( s, NB200_VEC_RELU, in, nullptr, nullptr,
					desc.HasParam() ? desc.GetParam<CReLUActivationParam>().UpperThreshold : 0.f, out, n ), "RowwiseActivation" );
				break;
			case AF_HSwish: e.Check( nb200_vector_op( s, NB200_VEC_HSWISH, in, nullptr, nullptr, 0.f, out, n ), "RowwiseActivation" ); break;
			case AF_Sigmoid: e.Check( nb200_vector_op( s, NB200_VEC_SIGMOID, in, nullptr, nullptr, 0.f, out, n ), "RowwiseActivation" ); break;
			case AF_Tanh: e.Check( nb200_vector_op( s, NB200_VEC_TANH, in, nullptr, nullptr, 0.f, out, n ), "RowwiseActivation" ); break;
			case AF_Exp: e.Check( nb200_vector_op( s, NB200_VEC_EXP, in, nullptr, nullptr, 0.f, out, n ), "RowwiseActivation" ); break;
			case AF_Linear: {
				CLinearActivationParam p;
				if( desc.HasParam() ) p = desc.GetParam<CLinearActivationParam>();
				e.Check( nb200_vector_op( s, NB200_VEC_MULTIPLY, in, nullptr, nullptr, p.Multiplier, out, n ), "RowwiseActivation" );
				if( p.FreeTerm != 0.f ) {
					e.Check( nb200_vector_op( s, NB200_VEC_ADD_VALUE, out, nullptr, nullptr, p.FreeTerm, out, n ), "RowwiseActivation" );
				}
				break;
			}
			default: raise( "rowwise activation: only ReLU, HSwish, sigmoid, tanh, exp and linear are implemented on this engine" );
		}
	}

	CActivationDesc desc;
};

struct CConvOp : public CB200RowwiseOp {
	int padH, padW, strideH, strideW, dilH, dilW, filterCount, filterH, filterW;
	const float* filter;
	const float* freeTerm;
	nb200_conv_desc d;

	CBlobDesc Reshape( const CBlobDesc& input ) override
	{
		inDesc = outDesc = input;
		const int ho = 1 + ( input.Height() - ( filterH - 1 ) * dilH - 1 + 2 * padH ) / strideH;
		const int wo = 1 + ( input.Width() - ( filterW - 1 ) * dilW - 1 + 2 * padW ) / strideW;
		outDesc.SetDimSize( BD_Height, ho );
		outDesc.SetDimSize( BD_Width, wo );
		outDesc.SetDimSize( BD_Depth, 1 );
		outDesc.SetDimSize( BD_Channels, filterCount );
		d = { input.ObjectCount(), input.Height(), input.Width(), imageChannels( input ), filterCount, filterH, filterW,
			padH, padW, strideH, strideW, dilH, dilW, ho, wo };
		return outDesc;
	}
	bool AbsorbsActivation() const override { return true; }

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& tail ) const override
	{
		nb200_epilogue epi = {};
		epi.bias = freeTerm;
		epi.act = tail.act;
		epi.act_param = tail.param;
		float* scratch = e.WorkAlloc( nb200_blob_convolution_scratch_floats( &d ) );
		const int rc = nb200_blob_convolution( e.Stream(), &d, in, filter, out, scratch, &epi, e.Precision() );
		e.WorkFree( scratch );
		e.Check( rc, "RowwiseConv" );
	}
};

struct CChConvOp : public CB200RowwiseOp {
	int padH, padW, strideH, strideW, filterH, filterW;
	const float* filter;
	const float* freeTerm;
	nb200_chconv_desc d;

	CBlobDesc Reshape( const CBlobDesc& input ) override
	{
		inDesc = outDesc = input;
		const int ho = 1 + ( input.Height() - filterH + 2 * padH ) / strideH;
		const int wo = 1 + ( input.Width() - filterW + 2 * padW ) / strideW;
		outDesc.SetDimSize( BD_Height, ho );
		outDesc.SetDimSize( BD_Width, wo );
		d = { input.ObjectCount(), input.Height(), input.Width(), imageChannels( input ), filterH, filterW, padH, padW,
			strideH, strideW, ho, wo };
		return outDesc;
	}
	bool AbsorbsActivation() const override { return true; }

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& tail ) const override
	{
		e.Check( nb200_blob_channelwise_convolution( e.Stream(), &d, in, filter, freeTerm, out, tail.act, tail.param ),
			"RowwiseChConv" );
	}
};

// 3x3 channelwise convolution (padding 1) + activation, then a 1x1 convolution (+ residual): MobileNetV3's tail
struct CChWith1x1Op : public CB200RowwiseOp {
	int stride, outputChannels;
	bool residual;
	CTail activation;
	const float* chFilter;
	const float* chFreeTerm;
	const float* convFilter;
	const float* convFreeTerm;
	nb200_chconv_desc d;

	CBlobDesc Reshape( const CBlobDesc& input ) override
	{
		inDesc = outDesc = input;
		const int ho = 1 + ( input.Height() - 1 ) / stride, wo = 1 + ( input.Width() - 1 ) / stride;
		outDesc.SetDimSize( BD_Height, ho );
		outDesc.SetDimSize( BD_Width, wo );
		outDesc.SetDimSize( BD_Depth, 1 );
		outDesc.SetDimSize( BD_Channels, outputChannels );
		d = { input.ObjectCount(), input.Height(), input.Width(), imageChannels( input ), 3, 3, 1, 1, stride, stride, ho, wo };
		return outDesc;
	}

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& ) const override
	{
		const int rows = d.batch * d.ho * d.wo;
		float* mid = e.WorkAlloc( static_cast<size_t>( rows ) * d.c );
		int rc = nb200_blob_channelwise_convolution( e.Stream(), &d, in, chFilter, chFreeTerm, mid, activation.act, activation.param );
		if( rc == 0 ) {
			nb200_epilogue epi = {};
			epi.bias = convFreeTerm;
			if( residual ) { epi.residual = in; epi.ld_residual = outputChannels; }
			rc = nb200_multiply_matrix_by_transposed_matrix( e.Stream(), mid, rows, d.c, d.c, convFilter, outputChannels, d.c,
				out, outputChannels, &epi, e.Precision() );
		}
		e.WorkFree( mid );
		e.Check( rc, "ChannelwiseWith1x1" );
	}
};

// The weight pointers are captured at Init time, as the reference's descriptor does
// (GPU/CUDA/Rowwise/CudaRowwiseMobileNetV2.h:94-108)
struct CMobileNetV2Op : public CB200RowwiseOp {
	int inputChannels, expandedChannels, outputChannels, stride;
	bool residual;
	CTail expandTail, channelwiseTail;
	const float* expandFilter;
	const float* expandFreeTerm;
	const float* channelwiseFilter;
	const float* channelwiseFreeTerm;
	const float* downFilter;
	const float* downFreeTerm;

	CBlobDesc Reshape( const CBlobDesc& input ) override
	{
		inDesc = outDesc = input;
		outDesc.SetDimSize( BD_Height, 1 + ( input.Height() - 1 ) / stride );
		outDesc.SetDimSize( BD_Width, 1 + ( input.Width() - 1 ) / stride );
		outDesc.SetDimSize( BD_Channels, outputChannels );
		return outDesc;
	}

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& ) const override { RunOn( e, inDesc, in, out ); }

	void RunOn( const CB200MathEngine& e, const CBlobDesc& input, const float* in, float* out ) const
	{
		nb200_mbv2_desc d = { input.ObjectCount(), input.Height(), input.Width(), inputChannels, expandedChannels,
			outputChannels, stride, residual ? 1 : 0, expandTail.act, channelwiseTail.act, expandTail.param, channelwiseTail.param };
		float* scratch = e.WorkAlloc( nb200_mobilenetv2_scratch_floats( &d ) );
		const int rc = nb200_mobilenetv2_block( e.Stream(), &d, in, expandFilter, expandFreeTerm, channelwiseFilter,
			channelwiseFreeTerm, downFilter, downFreeTerm, out, scratch, e.Precision() );
		e.WorkFree( scratch );
		e.Check( rc, "MobileNetV2Block" );
	}
};

struct CPoolingOp : public CB200RowwiseOp {
	bool isMax;
	int filterH, filterW, strideH, strideW;

	CBlobDesc Reshape( const CBlobDesc& input ) override
	{
		inDesc = outDesc = input;
		outDesc.SetDimSize( BD_Height, ( input.Height() - filterH ) / strideH + 1 );
		outDesc.SetDimSize( BD_Width, ( input.Width() - filterW ) / strideW + 1 );
		return outDesc;
	}

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& ) const override
	{
		const int n = inDesc.ObjectCount(), h = inDesc.Height(), w = inDesc.Width(), c = imageChannels( inDesc );
		const int rc = isMax ? nb200_blob_max_pooling( e.Stream(), n, h, w, c, filterH, filterW, strideH, strideW, in, out, nullptr )
			: nb200_blob_mean_pooling( e.Stream(), n, h, w, c, filterH, filterW, strideH, strideW, in, out );
		e.Check( rc, "Rowwise2DPooling" );
	}
};

struct CResizeOp : public CB200RowwiseOp {
	TBlobResizePadding padding;
	float defaultValue;
	int left, right, top, bottom;

	CBlobDesc Reshape( const CBlobDesc& input ) override
	{
		inDesc = outDesc = input;
		outDesc.SetDimSize( BD_Height, input.Height() + top + bottom );
		outDesc.SetDimSize( BD_Width, input.Width() + left + right );
		return outDesc;
	}

	void Run( const CB200MathEngine& e, const float* in, float* out, const CTail& ) const override
	{
		e.Check( nb200_blob_resize_image( e.Stream(), inDesc.ObjectCount(), inDesc.Height(), inDesc.Width(), imageChannels( inDesc ),
			left, right, top, bottom, static_cast<int>( padding ), defaultValue, in, out ), "RowwiseResizeImage" );
	}
};

const float* optional( const CB200MathEngine& e, const CConstFloatHandle* h ) { return h != nullptr ? e.Raw( *h ) : nullptr; }

} // namespace

//---------------------------------------------------------------------------------------------------------------------

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseActivation( const CActivationDesc& desc )
{
	return new CActivationOp( desc );
}

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseConv( int paddingHeight, int paddingWidth, int strideHeight, int strideWidth,
	int dilationHeight, int dilationWidth, const CBlobDesc& filterDesc, const CConstFloatHandle& filter,
	const CConstFloatHandle* freeTerm )
{
	CConvOp* op = new CConvOp();
	op->padH = paddingHeight; op->padW = paddingWidth; op->strideH = strideHeight; op->strideW = strideWidth;
	op->dilH = dilationHeight; op->dilW = dilationWidth;
	op->filterCount = filterDesc.ObjectCount(); op->filterH = filterDesc.Height(); op->filterW = filterDesc.Width();
	op->filter = raw( filter );
	op->freeTerm = optional( *this, freeTerm );
	return op;
}

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseChConv( int paddingHeight, int paddingWidth, int strideHeight, int strideWidth,
	const CBlobDesc& filterDesc, const CConstFloatHandle& filter, const CConstFloatHandle* freeTerm )
{
	CChConvOp* op = new CChConvOp();
	op->padH = paddingHeight; op->padW = paddingWidth; op->strideH = strideHeight; op->strideW = strideWidth;
	op->filterH = filterDesc.Height(); op->filterW = filterDesc.Width();
	op->filter = raw( filter );
	op->freeTerm = optional( *this, freeTerm );
	return op;
}

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseChWith1x1( int stride, const CConstFloatHandle& channelwiseFilter,
	const CConstFloatHandle* channelwiseFreeTerm, TActivationFunction activation, float reluParam,
	const CConstFloatHandle& convFilter, const CConstFloatHandle* convFreeTerm, int outputChannels, bool residual )
{
	CTail tail;
	if( !tailOf( activation, reluParam, tail ) ) {
		notImplemented( "InitRowwiseChWith1x1 (activation other than linear / ReLU / HSwish)" );
		return nullptr;
	}
	CChWith1x1Op* op = new CChWith1x1Op();
	op->stride = stride; op->outputChannels = outputChannels; op->residual = residual; op->activation = tail;
	op->chFilter = raw( channelwiseFilter ); op->chFreeTerm = optional( *this, channelwiseFreeTerm );
	op->convFilter = raw( convFilter ); op->convFreeTerm = optional( *this, convFreeTerm );
	return op;
}

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseMobileNetV2( int inputChannels, const CConstFloatHandle& expandFilter,
	const CConstFloatHandle* expandFreeTerm, int expandedChannels, TActivationFunction expandActivation, float expandReluParam,
	const CConstFloatHandle& channelwiseFilter, const CConstFloatHandle* channelwiseFreeTerm, int stride,
	TActivationFunction channelwiseActivation, float channelwiseReluParam, const CConstFloatHandle& downFilter,
	const CConstFloatHandle* downFreeTerm, int outputChannels, bool residual )
{
	CTail t1, t2;
	if( !tailOf( expandActivation, expandReluParam, t1 ) || !tailOf( channelwiseActivation, channelwiseReluParam, t2 ) ) {
		notImplemented( "InitRowwiseMobileNetV2 (activation other than linear / ReLU / HSwish)" );
		return nullptr;
	}
	CMobileNetV2Op* op = new CMobileNetV2Op();
	op->inputChannels = inputChannels; op->expandedChannels = expandedChannels; op->outputChannels = outputChannels;
	op->stride = stride; op->residual = residual; op->expandTail = t1; op->channelwiseTail = t2;
	op->expandFilter = raw( expandFilter ); op->expandFreeTerm = optional( *this, expandFreeTerm );
	op->channelwiseFilter = raw( channelwiseFilter ); op->channelwiseFreeTerm = optional( *this, channelwiseFreeTerm );
	op->downFilter = raw( downFilter ); op->downFreeTerm = optional( *this, downFreeTerm );
	return op;
}

CRowwiseOperationDesc* CB200MathEngine::InitRowwise2DPooling( bool isMax, int filterHeight, int filterWidth, int strideHeight,
	int strideWidth )
{
	CPoolingOp* op = new CPoolingOp();
	op->isMax = isMax; op->filterH = filterHeight; op->filterW = filterWidth; op->strideH = strideHeight; op->strideW = strideWidth;
	return op;
}

CRowwiseOperationDesc* CB200MathEngine::InitRowwiseResizeImage( TBlobResizePadding padding, float defaultValue, int deltaLeft,
	int deltaRight, int deltaTop, int deltaBottom )
{
	CResizeOp* op = new CResizeOp();
	op->padding = padding; op->defaultValue = defaultValue;
	op->left = deltaLeft; op->right = deltaRight; op->top = deltaTop; op->bottom = deltaBottom;
	return op;
}

CBlobDesc CB200MathEngine::RowwiseReshape( CRowwiseOperationDesc** operations, int operationCount, const CBlobDesc& input )
{
	CBlobDesc desc = input;
	for( int i = 0; i < operationCount; ++i ) {
		CB200RowwiseOp* op = dynamic_cast<CB200RowwiseOp*>( operations[i] );
		if( op == nullptr ) { raise( "RowwiseReshape: an operation was not created by this engine" ); return desc; }
		desc = op->Reshape( desc );
	}
	return desc;
}

void CB200MathEngine::RowwiseExecute( const CBlobDesc& inputDesc, CRowwiseOperationDesc** operations, int operationCount,
	const CFloatHandle& input, const CFloatHandle& output )
{
	enter();
	// the geometry is (re)derived here: the reference allows Execute with the descriptor Reshape was given
	CBlobDesc desc = inputDesc;
	std::vector<CB200RowwiseOp*> ops;
	for( int i = 0; i < operationCount; ++i ) {
		CB200RowwiseOp* op = dynamic_cast<CB200RowwiseOp*>( operations[i] );
		if( op == nullptr ) { raise( "RowwiseExecute: an operation was not created by this engine" ); return; }
		desc = op->Reshape( desc );
		ops.push_back( op );
	}
	const float* current = raw( input );
	float* result = raw( output );
	float* owned = nullptr; // intermediate the chain currently reads, from the pool
	for( size_t i = 0; i < ops.size(); ++i ) {
		CB200RowwiseOp* op = ops[i];
		// an activation right behind a convolution rides in its epilogue
		CTail tail;
		size_t consumed = 1;
		if( op->AbsorbsActivation() && i + 1 < ops.size() ) {
			const CActivationOp* next = dynamic_cast<const CActivationOp*>( ops[i + 1] );
			if( next != nullptr && next->AsTail( tail ) ) consumed = 2; else tail = CTail();
		}
		const bool last = i + consumed >= ops.size();
		float* out = nullptr;
		float* fresh = nullptr;
		if( last ) {
			out = result;
		} else if( op->InPlace() && owned != nullptr ) {
			out = owned; // overwrite the chain's own intermediate
		} else {
			fresh = WorkAlloc( static_cast<size_t>( ops[i + consumed - 1]->outDesc.BlobSize() ) );
			if( fresh == nullptr ) { WorkFree( owned ); return; }
			out = fresh;
		}
		op->Run( *this, current, out, tail );
		if( fresh != nullptr ) {
			WorkFree( owned ); // the stream orders its reuse behind the kernel that just read it
			owned = fresh;
		}
		current = out;
		i += consumed - 1;
	}
	WorkFree( owned );
}

void CB200MathEngine::MobileNetV2Block( const CBlobDesc& inputDesc, const CBlobDesc&, const CRowwiseOperationDesc& rowwiseDesc,
	const CChannelwiseConvolutionDesc&, const CConstFloatHandle& inputHandle, const CFloatHandle& outputHandle )
{
	const CMobileNetV2Op* op = dynamic_cast<const CMobileNetV2Op*>( &rowwiseDesc );
	if( op == nullptr ) { raise( "MobileNetV2Block: the rowwise descriptor was not created by this engine" ); return; }
	enter();
	op->RunOn( *this, inputDesc, raw( inputHandle ), raw( outputHandle ) );
}

// MobileNetV3 block up to its squeeze-and-excite branch (NeoMathEngine.h:1072-1077; CPU
// CpuMathEngineDnnChannelwiseConv.cpp:76-185): output = act2( channelwise( act1( input * expandFilter^T + bias ) ) ).
// The expanded image lives in pool memory; both activations ride in the kernels that produce their inputs.
void CB200MathEngine::MobileNetV3PreSEBlock( const CBlobDesc& inputDesc, const CBlobDesc&,
	const CChannelwiseConvolutionDesc& convDesc, const CConstFloatHandle& inputHandle,
	const CConstFloatHandle& expandFilter, const CConstFloatHandle* expandFreeTerm,
	TActivationFunction expandActivation, float expandReluParam, const CConstFloatHandle& channelwiseFilter,
	const CConstFloatHandle* channelwiseFreeTerm, TActivationFunction channelwiseActivation,
	float channelwiseReluParam, const CFloatHandle& outputHandle )
{
	const nb200_chconv_desc& d = static_cast<const CB200ChannelwiseDesc&>( convDesc ).d;
	CTail expandTail, channelwiseTail;
	if( !tailOf( expandActivation, expandReluParam, expandTail )
		|| !tailOf( channelwiseActivation, channelwiseReluParam, channelwiseTail ) ) {
		notImplemented( "MobileNetV3PreSEBlock (activation other than linear, ReLU, HSwish)" );
		return;
	}
	enter();
	const int rows = inputDesc.ObjectCount() * inputDesc.Height() * inputDesc.Width();
	const int inputChannels = imageChannels( inputDesc );
	if( inputDesc.Height() != d.h || inputDesc.Width() != d.w || inputDesc.ObjectCount() != d.batch ) {
		raise( "MobileNetV3PreSEBlock: the convolution descriptor does not fit the input" );
		return;
	}
	float* expanded = WorkAlloc( static_cast<size_t>( rows ) * d.c );
	const size_t scratchFloats = nb200_matrix_product_scratch_floats( 1, rows, d.c, inputChannels, inputChannels );
	float* scratch = scratchFloats > 0 ? WorkAlloc( scratchFloats ) : nullptr;
	nb200_epilogue epi = {};
	epi.bias = expandFreeTerm != nullptr ? raw( *expandFreeTerm ) : nullptr;
	epi.act = expandTail.act;
	epi.act_param = expandTail.param;
	int rc = nb200_multiply_matrix_by_transposed_matrix_with_scratch( stream, 1, raw( inputHandle ), rows, inputChannels,
		inputChannels, raw( expandFilter ), d.c, inputChannels, expanded, d.c, scratch, &epi, precision );
	if( rc == 0 ) {
		rc = nb200_blob_channelwise_convolution( stream, &d, expanded, raw( channelwiseFilter ),
			channelwiseFreeTerm != nullptr ? raw( *channelwiseFreeTerm ) : nullptr, raw( outputHandle ), channelwiseTail.act,
			channelwiseTail.param );
	}
	if( scratch != nullptr ) WorkFree( scratch );
	WorkFree( expanded );
	check( rc, "MobileNetV3PreSEBlock" );
}

// MobileNetV3 block after its squeeze-and-excite branch (NeoMathEngine.h:1078-1082; CPU
// CpuMathEngineDnnChannelwiseConv.cpp:187-258): output = act( input * se[image][channel] ) * downFilter^T + bias
// (+ residual).  One pass scales and activates into pool memory, the 1x1 convolution adds bias and residual in its
// epilogue.
void CB200MathEngine::MobileNetV3PostSEBlock( const CBlobDesc& channelwiseOutputDesc, int outputChannels,
	const CConstFloatHandle& channelwiseOutputHandle, const CConstFloatHandle& squeezeAndExciteHandle,
	const CConstFloatHandle* residualHandle, TActivationFunction activation, float reluParam,
	const CConstFloatHandle& downFilterHandle, const CConstFloatHandle* downFreeTermHandle,
	const CFloatHandle& outputHandle )
{
	CTail tail;
	if( !tailOf( activation, reluParam, tail ) ) {
		notImplemented( "MobileNetV3PostSEBlock (activation other than linear, ReLU, HSwish)" );
		return;
	}
	enter();
	const int batch = channelwiseOutputDesc.ObjectCount();
	const int pixels = channelwiseOutputDesc.Height() * channelwiseOutputDesc.Width();
	const int channels = imageChannels( channelwiseOutputDesc );
	const int rows = batch * pixels;
	float* scaled = WorkAlloc( static_cast<size_t>( rows ) * channels );
	int rc = nb200_scale_channels_activation( stream, batch, pixels, channels, raw( channelwiseOutputHandle ),
		raw( squeezeAndExciteHandle ), tail.act, tail.param, scaled );
	if( rc == 0 ) {
		const size_t scratchFloats = nb200_matrix_product_scratch_floats( 1, rows, outputChannels, channels, channels );
		float* scratch = scratchFloats > 0 ? WorkAlloc( scratchFloats ) : nullptr;
		nb200_epilogue epi = {};
		epi.bias = downFreeTermHandle != nullptr ? raw( *downFreeTermHandle ) : nullptr;
		if( residualHandle != nullptr ) { epi.residual = raw( *residualHandle ); epi.ld_residual = outputChannels; }
		rc = nb200_multiply_matrix_by_transposed_matrix_with_scratch( stream, 1, scaled, rows, channels, channels,
			raw( downFilterHandle ), outputChannels, channels, raw( outputHandle ), outputChannels, scratch, &epi, precision );
		if( scratch != nullptr ) WorkFree( scratch );
	}
	WorkFree( scaled );
	check( rc, "MobileNetV3PostSEBlock" );
}

void CB200MathEngine::ChannelwiseWith1x1( const CBlobDesc& inputDesc, const CBlobDesc&, const CRowwiseOperationDesc& rowwiseDesc,
	const CChannelwiseConvolutionDesc&, const CConstFloatHandle& inputHandle, const CFloatHandle& outputHandle )
{
	CChWith1x1Op* op = const_cast<CChWith1x1Op*>( dynamic_cast<const CChWith1x1Op*>( &rowwiseDesc ) );
	if( op == nullptr ) { raise( "ChannelwiseWith1x1: the rowwise descriptor was not created by this engine" ); return; }
	enter();
	op->Reshape( inputDesc );
	op->Run( *this, raw( inputHandle ), raw( outputHandle ), CTail() );
}

} // namespace NeoML
