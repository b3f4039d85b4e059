// TEST INFRASTRUCTURE ONLY.  C-ABI shim over the reference's own CPU math engine (libNeoMathEngine.so built by
// oracle/Makefile from the NeoML sources).  It lets Python (ctypes) run IMathEngine calls of the hot path on host
// arrays, to generate golden vectors, to validate oracle/neoml_oracle.c and to time the CPU baseline.
// A CPU-engine memory handle is {engine, base pointer, byte offset} and the engine dereferences base+offset
// (NeoMathEngine/src/MemoryHandleInternal.h:43-54), so host arrays are wrapped in place, without copies.
#include <NeoMathEngine/NeoMathEngine.h>

#include <chrono>
#include <cstring>
#include <memory>
#include <stdexcept>

using namespace NeoML;

namespace {

struct HandleMaker : public CMemoryHandle {
	HandleMaker( IMathEngine* e, const void* p ) : CMemoryHandle( e, p, 0 ) {}
};

CFloatHandle fh( IMathEngine* e, float* p ) { return CFloatHandle( HandleMaker( e, p ) ); }
CConstFloatHandle cfh( IMathEngine* e, const float* p ) { return CConstFloatHandle( HandleMaker( e, p ) ); }
CIntHandle ih( IMathEngine* e, int* p ) { return CIntHandle( HandleMaker( e, p ) ); }

CBlobDesc image_desc( int batch, int h, int w, int c )
{
	CBlobDesc d( CT_Float );
	d.SetDimSize( BD_BatchWidth, batch );
	d.SetDimSize( BD_Height, h );
	d.SetDimSize( BD_Width, w );
	d.SetDimSize( BD_Channels, c );
	return d;
}

TActivationFunction act_of( int a ) { return a == 1 ? AF_ReLU : ( a == 2 ? AF_HSwish : AF_Linear ); }

double now()
{
	return std::chrono::duration<double>( std::chrono::steady_clock::now().time_since_epoch() ).count();
}

} // namespace

#define SHIM_TRY try {
#define SHIM_CATCH } catch( std::exception& ) { return -1; } return 0;

extern "C" {

void* ref_engine_create() { try { return CreateCpuMathEngine( 0 ); } catch( std::exception& ) { return nullptr; } }
void ref_engine_destroy( void* e ) { delete static_cast<IMathEngine*>( e ); }

int ref_multiply_matrix_by_transposed_matrix( void* eng, const float* a, int m, int k, int lda, const float* b, int n,
	int ldb, float* c, int ldc, double* seconds )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	const double t0 = now();
	e->MultiplyMatrixByTransposedMatrix( cfh( e, a ), m, k, lda, cfh( e, b ), n, ldb, fh( e, c ), ldc, m * ldc );
	if( seconds != nullptr ) *seconds = now() - t0;
	SHIM_CATCH
}

int ref_multiply_matrix_by_matrix( void* eng, int batch, const float* a, int m, int k, const float* b, int n, float* c,
	double* seconds )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	const double t0 = now();
	e->MultiplyMatrixByMatrix( batch, cfh( e, a ), m, k, cfh( e, b ), n, fh( e, c ), batch * m * n );
	if( seconds != nullptr ) *seconds = now() - t0;
	SHIM_CATCH
}

int ref_blob_convolution( void* eng, int batch, int h, int w, int c, int k, int r, int s, int padH, int padW, int strH,
	int strW, int dilH, int dilW, const float* x, const float* filter, const float* freeTerm, float* y, double* seconds )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	const int ho = 1 + ( h - ( r - 1 ) * dilH - 1 + 2 * padH ) / strH;
	const int wo = 1 + ( w - ( s - 1 ) * dilW - 1 + 2 * padW ) / strW;
	CBlobDesc in = image_desc( batch, h, w, c ), out = image_desc( batch, ho, wo, k );
	CBlobDesc flt( CT_Float );
	flt.SetDimSize( BD_BatchWidth, k );
	flt.SetDimSize( BD_Height, r );
	flt.SetDimSize( BD_Width, s );
	flt.SetDimSize( BD_Channels, c );
	std::unique_ptr<CConvolutionDesc> desc( e->InitBlobConvolution( in, padH, padW, strH, strW, dilH, dilW, flt, out ) );
	CConstFloatHandle ft = freeTerm != nullptr ? cfh( e, freeTerm ) : CConstFloatHandle();
	const double t0 = now();
	e->BlobConvolution( *desc, cfh( e, x ), cfh( e, filter ), freeTerm != nullptr ? &ft : nullptr, fh( e, y ) );
	if( seconds != nullptr ) *seconds = now() - t0;
	SHIM_CATCH
}

int ref_blob_channelwise_convolution( void* eng, int batch, int h, int w, int c, int r, int s, int padH, int padW,
	int strH, int strW, const float* x, const float* filter, const float* freeTerm, float* y, double* seconds )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	const int ho = 1 + ( h - r + 2 * padH ) / strH;
	const int wo = 1 + ( w - s + 2 * padW ) / strW;
	CBlobDesc in = image_desc( batch, h, w, c ), out = image_desc( batch, ho, wo, c );
	CBlobDesc flt = image_desc( 1, r, s, c );
	CBlobDesc ftDesc = image_desc( 1, 1, 1, c );
	std::unique_ptr<CChannelwiseConvolutionDesc> desc( e->InitBlobChannelwiseConvolution( in, padH, padW, strH, strW,
		flt, freeTerm != nullptr ? &ftDesc : nullptr, out ) );
	CConstFloatHandle ft = freeTerm != nullptr ? cfh( e, freeTerm ) : CConstFloatHandle();
	const double t0 = now();
	e->BlobChannelwiseConvolution( *desc, cfh( e, x ), cfh( e, filter ), freeTerm != nullptr ? &ft : nullptr, fh( e, y ) );
	if( seconds != nullptr ) *seconds = now() - t0;
	SHIM_CATCH
}

int ref_mobilenetv2_block( void* eng, int batch, int h, int w, int cIn, int cExp, int cOut, int stride, int residual,
	int actExp, float actExpParam, int actDw, float actDwParam, const float* x, const float* wExp, const float* bExp,
	const float* wDw, const float* bDw, const float* wDown, const float* bDown, float* y, double* seconds )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	const int ho = 1 + ( h - 3 + 2 ) / stride, wo = 1 + ( w - 3 + 2 ) / stride;
	CBlobDesc in = image_desc( batch, h, w, cIn ), out = image_desc( batch, ho, wo, cOut );
	CBlobDesc chIn = image_desc( batch, h, w, cExp ), chOut = image_desc( batch, ho, wo, cExp );
	CBlobDesc flt = image_desc( 1, 3, 3, cExp ), ftDesc = image_desc( 1, 1, 1, cExp );
	std::unique_ptr<CChannelwiseConvolutionDesc> conv( e->InitBlobChannelwiseConvolution( chIn, 1, 1, stride, stride,
		flt, bDw != nullptr ? &ftDesc : nullptr, chOut ) );
	CConstFloatHandle bE = bExp ? cfh( e, bExp ) : CConstFloatHandle();
	CConstFloatHandle bC = bDw ? cfh( e, bDw ) : CConstFloatHandle();
	CConstFloatHandle bD = bDown ? cfh( e, bDown ) : CConstFloatHandle();
	std::unique_ptr<CRowwiseOperationDesc> row( e->InitRowwiseMobileNetV2( cIn, cfh( e, wExp ), bExp ? &bE : nullptr, cExp,
		act_of( actExp ), actExpParam, cfh( e, wDw ), bDw ? &bC : nullptr, stride, act_of( actDw ), actDwParam,
		cfh( e, wDown ), bDown ? &bD : nullptr, cOut, residual != 0 ) );
	CRowwiseOperationDesc* ops[1] = { row.get() };
	CBlobDesc reshaped = e->RowwiseReshape( ops, 1, in );
	(void)reshaped;
	const double t0 = now();
	e->MobileNetV2Block( in, out, *row, *conv, cfh( e, x ), fh( e, y ) );
	if( seconds != nullptr ) *seconds = now() - t0;
	SHIM_CATCH
}

// op numbering = NB200_VEC_* of include/neoml_b200.h; scalar operands are passed by pointer like the engine wants
int ref_vector_op( void* eng, int op, const float* a, const float* b, const float* scalar, float value, float* y, int n )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	switch( op ) {
		case 0: e->VectorCopy( fh( e, y ), cfh( e, a ), n ); break;
		case 1: e->VectorFill( fh( e, y ), value, n ); break;
		case 2: e->VectorFill( fh( e, y ), n, cfh( e, scalar ) ); break;
		case 3: e->VectorAdd( cfh( e, a ), cfh( e, b ), fh( e, y ), n ); break;
		case 4: e->VectorSub( cfh( e, a ), cfh( e, b ), fh( e, y ), n ); break;
		case 5: e->VectorEltwiseMultiply( cfh( e, a ), cfh( e, b ), fh( e, y ), n ); break;
		case 6: e->VectorMultiply( cfh( e, a ), fh( e, y ), n, cfh( e, scalar ) ); break;
		case 7: e->VectorNegMultiply( cfh( e, a ), fh( e, y ), n, cfh( e, scalar ) ); break;
		case 8: e->VectorAddValue( cfh( e, a ), fh( e, y ), n, cfh( e, scalar ) ); break;
		case 9: e->VectorReLU( cfh( e, a ), fh( e, y ), n, cfh( e, scalar ) ); break;
		case 10: e->VectorSigmoid( cfh( e, a ), fh( e, y ), n ); break;
		case 11: e->VectorSqrt( cfh( e, a ), fh( e, y ), n ); break;
		case 12: e->VectorInv( cfh( e, a ), fh( e, y ), n ); break;
		case 13: e->VectorTanh( cfh( e, a ), fh( e, y ), n ); break;
		case 14: e->VectorExp( cfh( e, a ), fh( e, y ), n ); break;
		case 15: e->VectorHSwish( cfh( e, a ), fh( e, y ), n ); break;
		case 16: e->VectorEltwiseMax( cfh( e, a ), cfh( e, b ), fh( e, y ), n ); break;
		case 17: e->VectorEltwiseDivide( cfh( e, a ), cfh( e, b ), fh( e, y ), n ); break;
		case 18: e->VectorMultiplyAndAdd( cfh( e, a ), cfh( e, b ), fh( e, y ), n, cfh( e, scalar ) ); break;
		default: return -2;
	}
	SHIM_CATCH
}

int ref_add_vector_to_matrix_rows( void* eng, int batch, const float* x, float* y, int height, int width, const float* v )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->AddVectorToMatrixRows( batch, cfh( e, x ), fh( e, y ), height, width, cfh( e, v ) );
	SHIM_CATCH
}

int ref_add_vector_to_matrix_columns( void* eng, const float* x, float* y, int height, int width, const float* v )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->AddVectorToMatrixColumns( cfh( e, x ), fh( e, y ), height, width, cfh( e, v ) );
	SHIM_CATCH
}

int ref_sum_matrix_rows( void* eng, int batch, float* y, const float* x, int height, int width, int add )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	if( add ) e->SumMatrixRowsAdd( batch, fh( e, y ), cfh( e, x ), height, width );
	else e->SumMatrixRows( batch, fh( e, y ), cfh( e, x ), height, width );
	SHIM_CATCH
}

int ref_sum_matrix_columns( void* eng, float* y, const float* x, int height, int width )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->SumMatrixColumns( fh( e, y ), cfh( e, x ), height, width );
	SHIM_CATCH
}

int ref_multiply_diag_matrix_by_matrix( void* eng, const float* d, int height, const float* x, int width, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->MultiplyDiagMatrixByMatrix( cfh( e, d ), height, cfh( e, x ), width, fh( e, y ), height * width );
	SHIM_CATCH
}

int ref_multiply_matrix_by_diag_matrix( void* eng, int batch, const float* x, int height, int width, const float* d,
	int diagStride, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	if( diagStride == 0 && batch == 1 ) {
		e->MultiplyMatrixByDiagMatrix( cfh( e, x ), height, width, cfh( e, d ), fh( e, y ), height * width );
	} else {
		e->BatchMultiplyMatrixByDiagMatrix( batch, cfh( e, x ), height, width, height * width, cfh( e, d ), diagStride,
			fh( e, y ), batch * height * width );
	}
	SHIM_CATCH
}

int ref_matrix_softmax_by_rows( void* eng, const float* x, int height, int width, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->MatrixSoftmaxByRows( cfh( e, x ), height, width, fh( e, y ) );
	SHIM_CATCH
}

int ref_transpose_matrix( void* eng, int batch, const float* x, int height, int medium, int width, int channels, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->TransposeMatrix( batch, cfh( e, x ), height, medium, width, channels, fh( e, y ), batch * height * medium * width * channels );
	SHIM_CATCH
}

int ref_find_max_value_in_rows( void* eng, const float* x, int height, int width, float* maxValues, int* maxIndices )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	if( maxIndices != nullptr ) e->FindMaxValueInRows( cfh( e, x ), height, width, fh( e, maxValues ), ih( e, maxIndices ), height );
	else e->FindMaxValueInRows( cfh( e, x ), height, width, fh( e, maxValues ), height );
	SHIM_CATCH
}

int ref_find_max_value_in_columns( void* eng, int batch, const float* x, int height, int width, float* maxValues, int* rowIndices )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->FindMaxValueInColumns( batch, cfh( e, x ), height, width, fh( e, maxValues ), ih( e, rowIndices ), batch * width );
	SHIM_CATCH
}

int ref_blob_max_pooling( void* eng, int batch, int h, int w, int c, int fh_, int fw, int sh, int sw, const float* x, float* y,
	int* maxIndices )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	CBlobDesc in = image_desc( batch, h, w, c ), out = image_desc( batch, ( h - fh_ ) / sh + 1, ( w - fw ) / sw + 1, c );
	std::unique_ptr<CMaxPoolingDesc> desc( e->InitMaxPooling( in, fh_, fw, sh, sw, out ) );
	CIntHandle idx = maxIndices != nullptr ? ih( e, maxIndices ) : CIntHandle();
	e->BlobMaxPooling( *desc, cfh( e, x ), maxIndices != nullptr ? &idx : nullptr, fh( e, y ) );
	SHIM_CATCH
}

int ref_blob_mean_pooling( void* eng, int batch, int h, int w, int c, int fh_, int fw, int sh, int sw, const float* x, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	CBlobDesc in = image_desc( batch, h, w, c ), out = image_desc( batch, ( h - fh_ ) / sh + 1, ( w - fw ) / sw + 1, c );
	std::unique_ptr<CMeanPoolingDesc> desc( e->InitMeanPooling( in, fh_, fw, sh, sw, out ) );
	e->BlobMeanPooling( *desc, cfh( e, x ), fh( e, y ) );
	SHIM_CATCH
}

int ref_blob_resize_image( void* eng, int batch, int h, int w, int c, int dl, int dr, int dt, int db, int padding,
	float defaultValue, const float* x, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	CBlobDesc in = image_desc( batch, h, w, c ), out = image_desc( batch, h + dt + db, w + dl + dr, c );
	e->BlobResizeImage( in, fh( e, const_cast<float*>( x ) ), dl, dr, dt, db, static_cast<TBlobResizePadding>( padding ),
		defaultValue, out, fh( e, y ) );
	SHIM_CATCH
}

// The way NeoML code really drives an engine: engine-owned memory, typed exchange, a stack variable.
// y = 2 * x + 1 computed on the engine; gauges[0..3] = current / peak / in-pools bytes after the work and the
// in-pools bytes after CleanUp().  Returns 0 on success.
int ref_engine_roundtrip( void* eng, const float* hostIn, float* hostOut, int n, unsigned long long* gauges )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	e->ResetPeakMemoryUsage();
	{
		CFloatHandle x = e->HeapAllocTyped<float>( n );
		e->DataExchangeTyped( x, hostIn, n );
		{
			CFloatHandleStackVar twice( *e, n ), one( *e, 1 );
			one.SetValue( 1.f );
			e->VectorAdd( x, x, twice, n );
			e->VectorAddValue( twice, x, n, one );
		}
		gauges[0] = e->GetCurrentMemoryUsage();
		gauges[1] = e->GetPeakMemoryUsage();
		e->DataExchangeTyped( hostOut, CConstFloatHandle( x ), n );
		e->HeapFree( x );
	}
	gauges[2] = e->GetMemoryInPools();
	e->CleanUp();
	gauges[3] = e->GetMemoryInPools();
	SHIM_CATCH
}

// Makes every result of the calls so far visible, the way NeoML code reads results: a typed exchange of one float.
int ref_engine_sync( void* eng, const float* anyEngineFloat )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	float value = 0.f;
	e->DataExchangeTyped( &value, cfh( e, anyEngineFloat ), 1 );
	SHIM_CATCH
}

// type: TMathEngineType of the engine; returns the device id the engine reports
int ref_engine_info( void* eng, int* type, unsigned long long* availableMemory, char* name, int nameSize )
{
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	CMathEngineInfo info;
	e->GetMathEngineInfo( info );
	*type = static_cast<int>( e->GetType() );
	*availableMemory = info.AvailableMemory;
	std::strncpy( name, info.Name, nameSize - 1 );
	name[nameSize - 1] = 0;
	return info.Id;
}

// Calls a training-only method (outside the inference hot path).  1 = the engine raised through the exception
// handler, 0 = it ran.
int ref_engine_training_method_raises( void* eng, float* x, int n )
{
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	try {
		e->VectorHuberDerivative( cfh( e, x ), fh( e, x ), n );
	} catch( std::exception& ) {
		return 1;
	}
	return 0;
}

// A chain of rowwise operations as NeoML's optimizer builds them (NeoMathEngine.h:1084-1110):
// resize(+1 on every side, zeros) -> max pool 3x3/2 -> conv 3x3 pad 1 (c -> k) -> ReLU(6) -> MobileNetV2 block
// (k -> cexp -> k, stride 1, residual, ReLU6 twice) -> channelwise 3x3 pad 1 -> HSwish -> channelwise 3x3/2 + ReLU +
// 1x1 conv (k -> kout).  outDims receives {objects, height, width, channels} of the result; y must hold it.
int ref_rowwise_chain( void* eng, int batch, int h, int w, int c, int k, int cexp, int kout, const float* x,
	const float* convF, const float* convB, const float* wExp, const float* bExp, const float* wDw, const float* bDw,
	const float* wDown, const float* bDown, const float* chF, const float* chB, const float* ch1F, const float* ch1B,
	const float* c1F, const float* c1B, float* y, int* outDims )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	CBlobDesc input = image_desc( batch, h, w, c );
	CBlobDesc convFilter( CT_Float );
	convFilter.SetDimSize( BD_BatchWidth, k ); convFilter.SetDimSize( BD_Height, 3 ); convFilter.SetDimSize( BD_Width, 3 );
	convFilter.SetDimSize( BD_Channels, c );
	CBlobDesc chFilter( CT_Float );
	chFilter.SetDimSize( BD_Height, 3 ); chFilter.SetDimSize( BD_Width, 3 ); chFilter.SetDimSize( BD_Channels, k );
	CConstFloatHandle hConvB = cfh( e, convB ), hBExp = cfh( e, bExp ), hBDw = cfh( e, bDw ), hBDown = cfh( e, bDown ),
		hChB = cfh( e, chB ), hCh1B = cfh( e, ch1B ), hC1B = cfh( e, c1B );
	std::unique_ptr<CRowwiseOperationDesc> ops[8];
	ops[0].reset( e->InitRowwiseResizeImage( TBlobResizePadding::Constant, 0.f, 1, 1, 1, 1 ) );
	ops[1].reset( e->InitRowwise2DPooling( true, 3, 3, 2, 2 ) );
	ops[2].reset( e->InitRowwiseConv( 1, 1, 1, 1, 1, 1, convFilter, cfh( e, convF ), &hConvB ) );
	ops[3].reset( e->InitRowwiseActivation( CActivationDesc( AF_ReLU, CReLUActivationParam{ 6.f } ) ) );
	ops[4].reset( e->InitRowwiseMobileNetV2( k, cfh( e, wExp ), &hBExp, cexp, AF_ReLU, 6.f, cfh( e, wDw ), &hBDw, 1, AF_ReLU, 6.f,
		cfh( e, wDown ), &hBDown, k, true ) );
	ops[5].reset( e->InitRowwiseChConv( 1, 1, 1, 1, chFilter, cfh( e, chF ), &hChB ) );
	ops[6].reset( e->InitRowwiseActivation( CActivationDesc( AF_HSwish ) ) );
	ops[7].reset( e->InitRowwiseChWith1x1( 2, cfh( e, ch1F ), &hCh1B, AF_ReLU, 0.f, cfh( e, c1F ), &hC1B, kout, false ) );
	CRowwiseOperationDesc* raw[8];
	for( int i = 0; i < 8; ++i ) raw[i] = ops[i].get();
	const CBlobDesc out = e->RowwiseReshape( raw, 8, input );
	outDims[0] = out.ObjectCount(); outDims[1] = out.Height(); outDims[2] = out.Width(); outDims[3] = out.Channels();
	if( y != nullptr ) e->RowwiseExecute( input, raw, 8, fh( e, const_cast<float*>( x ) ), fh( e, y ) );
	SHIM_CATCH
}

// A MobileNetV3 block around a given squeeze-and-excite vector, as CMobileNetV3PreSEBlockLayer / PostSEBlockLayer call
// the engine (NeoMathEngine.h:1072-1082): expand 1x1 (c -> cexp) + act1, channelwise r x r (stride, padding r / 2) +
// act2 -> mid; then mid * se[image][channel] -> act3 -> down 1x1 (cexp -> kout) + bias (+ x when residual).
// Activations: 0 linear, 1 ReLU(param), 2 HSwish.  y must hold batch x ho x wo x kout floats.
int ref_mobilenetv3_block( void* eng, int batch, int h, int w, int c, int cexp, int kout, int r, int stride, int residual,
	int act1, float p1, int act2, float p2, int act3, float p3, const float* x, const float* wExp, const float* bExp,
	const float* wDw, const float* bDw, const float* se, const float* wDown, const float* bDown, float* mid, float* y )
{
	SHIM_TRY
	IMathEngine* e = static_cast<IMathEngine*>( eng );
	const int pad = r / 2;
	const int ho = 1 + ( h - r + 2 * pad ) / stride, wo = 1 + ( w - r + 2 * pad ) / stride;
	CBlobDesc in = image_desc( batch, h, w, c ), expanded = image_desc( batch, h, w, cexp ), out = image_desc( batch, ho, wo, cexp );
	CBlobDesc flt = image_desc( 1, r, r, cexp ), ftDesc = image_desc( 1, 1, 1, cexp );
	std::unique_ptr<CChannelwiseConvolutionDesc> desc( e->InitBlobChannelwiseConvolution( expanded, pad, pad, stride, stride,
		flt, bDw != nullptr ? &ftDesc : nullptr, out ) );
	CConstFloatHandle hBExp = cfh( e, bExp ), hBDw = cfh( e, bDw ), hBDown = cfh( e, bDown ), hRes = cfh( e, x );
	e->MobileNetV3PreSEBlock( in, out, *desc, cfh( e, x ), cfh( e, wExp ), bExp != nullptr ? &hBExp : nullptr, act_of( act1 ), p1,
		cfh( e, wDw ), bDw != nullptr ? &hBDw : nullptr, act_of( act2 ), p2, fh( e, mid ) );
	e->MobileNetV3PostSEBlock( out, kout, cfh( e, mid ), cfh( e, se ), residual ? &hRes : nullptr, act_of( act3 ), p3,
		cfh( e, wDown ), bDown != nullptr ? &hBDown : nullptr, fh( e, y ) );
	SHIM_CATCH
}

} // extern "C"
