// CB200MathEngine compute methods: each translates one IMathEngine call on the inference hot path into one call of the
// C ABI (include/neoml_b200.h) on the engine's stream.  Argument meaning is the reference's
// (NeoMathEngine/include/NeoMathEngine/NeoMathEngine.h); sizes are element counts; optional operands are null pointers.
#include "B200MathEngine.h"

#include <neoml_b200.h>

#include <cuda_runtime.h>


namespace NeoML {

namespace {

void raise( const char* message )
{
	GetMathEngineExceptionHandler()->OnAssert( message, L"B200MathEngineOps", 0, 0 );
}

} // namespace

void CB200MathEngine::vectorOp( int op, const float* a, const float* b, const float* scalar, float value, float* y, int n,
	const char* method )
{
	enter();
	check( nb200_vector_op( stream, op, a, b, scalar, value, y, n ), method );
}

//---------------------------------------------------------------------------------------------------------------------
// IVectorMathEngine

void CB200MathEngine::VectorCopy( const CFloatHandle& first, const CConstFloatHandle& second, int vectorSize )
{
	vectorOp( NB200_VEC_COPY, raw( second ), nullptr, nullptr, 0.f, raw( first ), vectorSize, "VectorCopy" );
}

void CB200MathEngine::VectorCopy( const CIntHandle& first, const CConstIntHandle& second, int vectorSize )
{
	enter();
	check( nb200_vector_copy_int( stream, raw( second ), raw( first ), vectorSize ), "VectorCopy" );
}

void CB200MathEngine::VectorFill( const CFloatHandle& result, float value, int vectorSize )
{
	vectorOp( NB200_VEC_FILL, nullptr, nullptr, nullptr, value, raw( result ), vectorSize, "VectorFill" );
}

void CB200MathEngine::VectorFill( const CIntHandle& result, int value, int vectorSize )
{
	enter();
	check( nb200_vector_fill_int( stream, value, raw( result ), vectorSize ), "VectorFill" );
}

void CB200MathEngine::VectorFill( const CFloatHandle& result, int vectorSize, const CConstFloatHandle& value )
{
	vectorOp( NB200_VEC_FILL_HANDLE, nullptr, nullptr, raw( value ), 0.f, raw( result ), vectorSize, "VectorFill" );
}

void CB200MathEngine::VectorReLU( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize,
	const CConstFloatHandle& upperThresholdHandle )
{
	if( fuseReLU( raw( firstHandle ), raw( resultHandle ), vectorSize, raw( upperThresholdHandle ) ) ) return;
	vectorOp( NB200_VEC_RELU, raw( firstHandle ), nullptr, raw( upperThresholdHandle ), 0.f, raw( resultHandle ), vectorSize, "VectorReLU" );
}

void CB200MathEngine::VectorHSwish( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_HSWISH, raw( firstHandle ), nullptr, nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorHSwish" );
}

void CB200MathEngine::VectorEltwiseMax( const CConstFloatHandle& firstHandle, const CConstFloatHandle& secondHandle,
	const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_ELTWISE_MAX, raw( firstHandle ), raw( secondHandle ), nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorEltwiseMax" );
}

void CB200MathEngine::VectorExp( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_EXP, raw( firstHandle ), nullptr, nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorExp" );
}

void CB200MathEngine::VectorAdd( const CConstFloatHandle& firstHandle, const CConstFloatHandle& secondHandle,
	const CFloatHandle& resultHandle, int vectorSize )
{
	if( fuseAdd( raw( firstHandle ), raw( secondHandle ), raw( resultHandle ), vectorSize ) ) return;
	vectorOp( NB200_VEC_ADD, raw( firstHandle ), raw( secondHandle ), nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorAdd" );
}

void CB200MathEngine::VectorAddValue( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize,
	const CConstFloatHandle& addition )
{
	vectorOp( NB200_VEC_ADD_VALUE, raw( firstHandle ), nullptr, raw( addition ), 0.f, raw( resultHandle ), vectorSize, "VectorAddValue" );
}

void CB200MathEngine::VectorSub( const CConstFloatHandle& firstHandle, const CConstFloatHandle& secondHandle,
	const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_SUB, raw( firstHandle ), raw( secondHandle ), nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorSub" );
}

void CB200MathEngine::VectorMultiplyAndAdd( const CConstFloatHandle& firstHandle, const CConstFloatHandle& secondHandle,
	const CFloatHandle& resultHandle, int vectorSize, const CConstFloatHandle& multHandle )
{
	vectorOp( NB200_VEC_MUL_ADD, raw( firstHandle ), raw( secondHandle ), raw( multHandle ), 0.f, raw( resultHandle ), vectorSize, "VectorMultiplyAndAdd" );
}

void CB200MathEngine::VectorMultiply( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize,
	const CConstFloatHandle& multiplierHandle )
{
	if( raw( firstHandle ) == raw( resultHandle ) && vectorSize > 0 ) {
		// in place: held back, a softmax over the same buffer may absorb it (see CPendingRowOps)
		enter();
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		pendingRows = CPendingRowOps();
		pendingRows.data = raw( resultHandle );
		pendingRows.size = vectorSize;
		pendingRows.scale = raw( multiplierHandle );
		pendingRows.active = true;
		return;
	}
	vectorOp( NB200_VEC_MULTIPLY, raw( firstHandle ), nullptr, raw( multiplierHandle ), 0.f, raw( resultHandle ), vectorSize, "VectorMultiply" );
}

void CB200MathEngine::VectorNegMultiply( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize,
	const CConstFloatHandle& multiplierHandle )
{
	vectorOp( NB200_VEC_NEG_MULTIPLY, raw( firstHandle ), nullptr, raw( multiplierHandle ), 0.f, raw( resultHandle ), vectorSize, "VectorNegMultiply" );
}

void CB200MathEngine::VectorEltwiseMultiply( const CConstFloatHandle& firstHandle, const CConstFloatHandle& secondHandle,
	const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_ELTWISE_MUL, raw( firstHandle ), raw( secondHandle ), nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorEltwiseMultiply" );
}

void CB200MathEngine::VectorEltwiseDivide( const CConstFloatHandle& firstHandle, const CConstFloatHandle& secondHandle,
	const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_ELTWISE_DIV, raw( firstHandle ), raw( secondHandle ), nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorEltwiseDivide" );
}

void CB200MathEngine::VectorSqrt( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_SQRT, raw( firstHandle ), nullptr, nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorSqrt" );
}

void CB200MathEngine::VectorInv( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_INV, raw( firstHandle ), nullptr, nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorInv" );
}

void CB200MathEngine::VectorSigmoid( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_SIGMOID, raw( firstHandle ), nullptr, nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorSigmoid" );
}

void CB200MathEngine::VectorTanh( const CConstFloatHandle& firstHandle, const CFloatHandle& resultHandle, int vectorSize )
{
	vectorOp( NB200_VEC_TANH, raw( firstHandle ), nullptr, nullptr, 0.f, raw( resultHandle ), vectorSize, "VectorTanh" );
}

//---------------------------------------------------------------------------------------------------------------------
// IBlasEngine

void CB200MathEngine::AddVectorToMatrixRows( int batchSize, const CConstFloatHandle& matrixHandle, const CFloatHandle& resultHandle,
	int matrixHeight, int matrixWidth, const CConstFloatHandle& vectorHandle )
{
	const long long size = static_cast<long long>( matrixHeight ) * matrixWidth;
	if( batchSize == 1 && raw( matrixHandle ) == raw( resultHandle ) && size > 0 ) {
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		if( pendingRows.active && pendingRows.data == raw( resultHandle ) && pendingRows.size == size && pendingRows.bias == nullptr ) {
			// joins a held-back VectorMultiply of the same buffer
		} else {
			enter();
			pendingRows = CPendingRowOps();
			pendingRows.data = raw( resultHandle );
			pendingRows.size = size;
			pendingRows.active = true;
		}
		pendingRows.bias = raw( vectorHandle );
		pendingRows.biasHeight = matrixHeight;
		pendingRows.biasWidth = matrixWidth;
		return;
	}
	enter();
	check( nb200_add_vector_to_matrix_rows( stream, batchSize, raw( matrixHandle ), raw( resultHandle ), matrixHeight, matrixWidth,
		raw( vectorHandle ) ), "AddVectorToMatrixRows" );
}

void CB200MathEngine::AddVectorToMatrixColumns( const CConstFloatHandle& matrixHandle, const CFloatHandle& resultHandle,
	int matrixHeight, int matrixWidth, const CConstFloatHandle& vectorHandle )
{
	enter();
	check( nb200_add_vector_to_matrix_columns( stream, raw( matrixHandle ), raw( resultHandle ), matrixHeight, matrixWidth,
		raw( vectorHandle ) ), "AddVectorToMatrixColumns" );
}

void CB200MathEngine::SumMatrixRowsAdd( int batchSize, const CFloatHandle& resultHandle, const CConstFloatHandle& matrixHandle,
	int matrixHeight, int matrixWidth )
{
	enter();
	check( nb200_sum_matrix_rows( stream, batchSize, raw( resultHandle ), raw( matrixHandle ), matrixHeight, matrixWidth, 1 ), "SumMatrixRowsAdd" );
}

void CB200MathEngine::SumMatrixRows( int batchSize, const CFloatHandle& resultHandle, const CConstFloatHandle& matrixHandle,
	int matrixHeight, int matrixWidth )
{
	enter();
	check( nb200_sum_matrix_rows( stream, batchSize, raw( resultHandle ), raw( matrixHandle ), matrixHeight, matrixWidth, 0 ), "SumMatrixRows" );
}

void CB200MathEngine::SumMatrixColumns( const CFloatHandle& resultHandle, const CConstFloatHandle& matrixHandle, int matrixHeight,
	int matrixWidth )
{
	enter();
	check( nb200_sum_matrix_columns( stream, raw( resultHandle ), raw( matrixHandle ), matrixHeight, matrixWidth ), "SumMatrixColumns" );
}

void CB200MathEngine::MatrixSoftmaxByRows( const CConstFloatHandle& matrix, int height, int width, const CFloatHandle& result )
{
	{
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const CPendingRowOps p = pendingRows;
		if( p.active && p.data == raw( result ) && raw( matrix ) == raw( result ) && width > 0 && width <= 1024
			&& p.size == static_cast<long long>( height ) * width && ( p.bias == nullptr || p.biasWidth % width == 0 ) ) {
			// scale, mask and softmax in one pass over the scores
			pendingRows = CPendingRowOps();
			enter();
			check( nb200_matrix_softmax_by_rows_fused( stream, p.data, height, width, p.scale, p.bias,
				p.bias != nullptr ? p.biasWidth / width : 0, p.data ), "MatrixSoftmaxByRows" );
			return;
		}
	}
	enter();
	check( nb200_matrix_softmax_by_rows( stream, raw( matrix ), height, width, raw( result ) ), "MatrixSoftmaxByRows" );
}

void CB200MathEngine::FindMaxValueInRows( const CConstFloatHandle& matrixHandle, int matrixHeight, int matrixWidth,
	const CFloatHandle& resultHandle, const CIntHandle& columnIndices, int vectorSize )
{
	if( vectorSize < matrixHeight ) { raise( "FindMaxValueInRows: result buffer too small" ); return; }
	enter();
	check( nb200_find_max_value_in_rows( stream, raw( matrixHandle ), matrixHeight, matrixWidth, raw( resultHandle ),
		raw( columnIndices ) ), "FindMaxValueInRows" );
}

void CB200MathEngine::FindMaxValueInRows( const CConstFloatHandle& matrixHandle, int matrixHeight, int matrixWidth,
	const CFloatHandle& resultHandle, int vectorSize )
{
	if( vectorSize < matrixHeight ) { raise( "FindMaxValueInRows: result buffer too small" ); return; }
	enter();
	check( nb200_find_max_value_in_rows( stream, raw( matrixHandle ), matrixHeight, matrixWidth, raw( resultHandle ), nullptr ),
		"FindMaxValueInRows" );
}

void CB200MathEngine::FindMaxValueInColumns( int batchSize, const CConstFloatHandle& matrixHandle, int matrixHeight, int matrixWidth,
	const CFloatHandle& resultHandle, const CIntHandle& rowIndices, int vectorSize )
{
	if( vectorSize < batchSize * matrixWidth ) { raise( "FindMaxValueInColumns: result buffer too small" ); return; }
	enter();
	if( matrixWidth == 1 ) {
		// one column per batch entry (CArgmaxLayer over the last dimension): the maximum of each contiguous run of
		// matrixHeight values -- a row maximum, which is what the reference CPU engine forwards this case to
		// (CPU/x86/CpuX86MathEngineBlas.cpp:191-196); first maximum wins in both
		check( nb200_find_max_value_in_rows( stream, raw( matrixHandle ), batchSize, matrixHeight, raw( resultHandle ),
			raw( rowIndices ) ), "FindMaxValueInColumns" );
		return;
	}
	check( nb200_find_max_value_in_columns( stream, batchSize, raw( matrixHandle ), matrixHeight, matrixWidth, raw( resultHandle ),
		raw( rowIndices ) ), "FindMaxValueInColumns" );
}

void CB200MathEngine::MultiplyMatrixByTransposedMatrix( const CConstFloatHandle& firstHandle, int firstHeight, int firstWidth,
	int firstRowSize, const CConstFloatHandle& secondHandle, int secondHeight, int secondRowSize, const CFloatHandle& resultHandle,
	int resultRowSize, int )
{
	enter();
	check( productWithScratch( 1, raw( firstHandle ), firstHeight, firstWidth, firstRowSize, raw( secondHandle ), secondHeight,
		secondRowSize, raw( resultHandle ), resultRowSize ), "MultiplyMatrixByTransposedMatrix" );
}

// first * second^T with work space from the stack allocator: a prepared second operand for tall products, room for
// split-K partial results for products with few output tiles
int CB200MathEngine::productWithScratch( int batchSize, const float* first, int firstHeight, int firstWidth, int firstRowSize,
	const float* second, int secondHeight, int secondRowSize, float* result, int resultRowSize )
{
	const size_t floats = nb200_matrix_product_scratch_floats( batchSize, firstHeight, secondHeight, firstWidth, secondRowSize );
	if( floats == 0 ) {
		return nb200_multiply_matrix_by_transposed_matrix_with_scratch( stream, batchSize, first, firstHeight, firstWidth,
			firstRowSize, second, secondHeight, secondRowSize, result, resultRowSize, nullptr, nullptr, precision );
	}
	CMemoryHandle scratch = StackAlloc( floats * sizeof( float ) );
	const int rc = nb200_multiply_matrix_by_transposed_matrix_with_scratch( stream, batchSize, first, firstHeight, firstWidth,
		firstRowSize, second, secondHeight, secondRowSize, result, resultRowSize,
		static_cast<float*>( CMemoryHandleInternal::GetRaw( scratch ) ), nullptr, precision );
	StackFree( scratch ); // stream order keeps the kernels ahead of the next user of the stack
	return rc;
}

void CB200MathEngine::MultiplyMatrixByTransposedMatrix( int batchSize, const CConstFloatHandle& firstHandle, int firstHeight,
	int firstWidth, const CConstFloatHandle& secondHandle, int secondHeight, const CFloatHandle& resultHandle, int )
{
	enter();
	check( productWithScratch( batchSize, raw( firstHandle ), firstHeight, firstWidth, firstWidth, raw( secondHandle ),
		secondHeight, firstWidth, raw( resultHandle ), secondHeight ), "MultiplyMatrixByTransposedMatrix" );
}

void CB200MathEngine::MultiplyMatrixByMatrix( int batchSize, const CConstFloatHandle& firstHandle, int firstHeight, int firstWidth,
	const CConstFloatHandle& secondHandle, int secondWidth, const CFloatHandle& resultHandle, int )
{
	enter();
	// The second operand is [K x N]: the tensor-core kernel wants both operands K-major.  One transposing pass over it
	// (into stack memory) costs a read and a write of the operand and lets the product run on the TMA-fed path, which
	// is several times faster than gathering a column-major operand element by element.
	const size_t floats = static_cast<size_t>( batchSize ) * firstWidth * secondWidth;
	if( firstWidth >= 4 && secondWidth >= 4 && floats < ( static_cast<size_t>( 1 ) << 31 ) ) {
		CMemoryHandle scratch = StackAlloc( floats * sizeof( float ) );
		float* transposed = static_cast<float*>( CMemoryHandleInternal::GetRaw( scratch ) );
		int rc = nb200_transpose_matrix( stream, batchSize, raw( secondHandle ), firstWidth, 1, secondWidth, 1, transposed );
		if( rc == 0 ) {
			rc = productWithScratch( batchSize, raw( firstHandle ), firstHeight, firstWidth, firstWidth, transposed, secondWidth,
				firstWidth, raw( resultHandle ), secondWidth );
		}
		StackFree( scratch ); // stream order keeps the kernels ahead of the next user of the stack
		check( rc, "MultiplyMatrixByMatrix" );
		return;
	}
	check( nb200_multiply_matrix_by_matrix( stream, batchSize, raw( firstHandle ), firstHeight, firstWidth, raw( secondHandle ),
		secondWidth, raw( resultHandle ), nullptr, precision ), "MultiplyMatrixByMatrix" );
}

void CB200MathEngine::MultiplyDiagMatrixByMatrix( const CConstFloatHandle& firstHandle, int firstSize,
	const CConstFloatHandle& secondHandle, int secondWidth, const CFloatHandle& resultHandle, int )
{
	enter();
	check( nb200_multiply_diag_matrix_by_matrix( stream, raw( firstHandle ), firstSize, raw( secondHandle ), secondWidth,
		raw( resultHandle ) ), "MultiplyDiagMatrixByMatrix" );
}

void CB200MathEngine::BatchMultiplyMatrixByDiagMatrix( int batchSize, const CConstFloatHandle& firstHandle, int height, int width,
	int firstMatrixOffset, const CConstFloatHandle& secondHandle, int secondMatrixOffset, const CFloatHandle& resultHandle, int )
{
	// the kernel assumes densely packed matrices; the reference allows a zero offset to reuse one matrix for all batches
	if( batchSize > 1 && firstMatrixOffset != height * width ) { notImplemented( "BatchMultiplyMatrixByDiagMatrix (strided first operand)" ); return; }
	if( secondMatrixOffset != 0 && secondMatrixOffset != width ) { notImplemented( "BatchMultiplyMatrixByDiagMatrix (strided diagonal)" ); return; }
	enter();
	check( nb200_multiply_matrix_by_diag_matrix( stream, batchSize, raw( firstHandle ), height, width, raw( secondHandle ),
		secondMatrixOffset, raw( resultHandle ) ), "BatchMultiplyMatrixByDiagMatrix" );
}

void CB200MathEngine::TransposeMatrix( int batchSize, const CConstFloatHandle& firstHandle, int height, int medium, int width,
	int channels, const CFloatHandle& resultHandle, int )
{
	enter();
	check( nb200_transpose_matrix( stream, batchSize, raw( firstHandle ), height, medium, width, channels, raw( resultHandle ) ),
		"TransposeMatrix" );
}

void CB200MathEngine::TransposeMatrix( int batchSize, const CConstIntHandle& firstHandle, int height, int medium, int width,
	int channels, const CIntHandle& resultHandle, int )
{
	enter();
	check( nb200_transpose_matrix( stream, batchSize, raw( firstHandle ), height, medium, width, channels, raw( resultHandle ) ),
		"TransposeMatrix" );
}

} // namespace NeoML
