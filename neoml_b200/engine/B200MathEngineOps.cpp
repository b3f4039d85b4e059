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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( firstHandle ) != peek( secondHandle ) ) {
		// a noted fully connected product plus another tensor (CEltwiseSumLayer): the other tensor becomes the residual
		// of the product's epilogue, the sum is noted for the result buffer
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		for( int side = 0; side < 2; ++side ) {
			const CConstFloatHandle& noted = side == 0 ? firstHandle : secondHandle;
			const CConstFloatHandle& other = side == 0 ? secondHandle : firstHandle;
			const int at = findLazy( peek( noted ), CLazyResult::K_Product );
			if( at < 0 || lazy[at].resultFloats != vectorSize || lazy[at].gate != 0 || lazy[at].residual != nullptr
				|| findLazy( peek( other ), CLazyResult::K_Product ) >= 0 ) {
				continue;
			}
			const float* const addend = raw( other ); // whatever is noted for that tensor is carried out first
			if( findLazy( peek( noted ), CLazyResult::K_Product ) != at ) break;
			CLazyResult* note = deriveNote( at, resultHandle );
			if( note == nullptr ) break;
			note->residual = addend;
			// the addend may be the result buffer itself (a sum in place of the other operand): then it is covered by
			// the rule for the result, and reading it is what the epilogue does
			if( peek( other ) != peek( resultHandle ) ) note->Reads( other, vectorSize );
			return;
		}
	}
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( firstHandle ) == peek( resultHandle ) ) {
		// in place on a noted score matrix (see CLazyResult): the factor joins the note
		const float* const factor = raw( multiplierHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( firstHandle ), CLazyResult::K_Scores );
		if( at >= 0 && lazy[at].resultFloats == vectorSize && lazy[at].scale == nullptr && lazy[at].mask == nullptr
			&& !lazy[at].softmax ) {
			lazy[at].scale = factor;
			lazy[at].Reads( multiplierHandle, 1 );
			return;
		}
	}
	if( peek( firstHandle ) == peek( resultHandle ) && vectorSize > 0 ) {
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( firstHandle ) != peek( resultHandle ) ) {
		// a noted product times a device scalar into another buffer: the first step of CGELULayer's gate
		const float* const factor = raw( multiplierHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( firstHandle ), CLazyResult::K_Product );
		if( at >= 0 && lazy[at].resultFloats == vectorSize && lazy[at].gate == 0 && lazy[at].residual == nullptr ) {
			const float* const source = lazy[at].result;
			CLazyResult* note = deriveNote( at, resultHandle );
			if( note != nullptr ) {
				note->gate = 1;
				note->gateScale = factor;
				note->gateSource = source;
				note->Reads( multiplierHandle, 1 );
				return;
			}
		}
	}
	const std::ptrdiff_t apart = peek( resultHandle ) - peek( firstHandle );
	if( vectorSize > 0 && ( apart >= vectorSize || -apart >= vectorSize ) ) {
		// into another buffer: held back, CGELULayer's sigmoid and gate may follow (see CPendingSigmoidGate)
		enter();
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		pendingGate = CPendingSigmoidGate();
		pendingGate.input = raw( firstHandle );
		pendingGate.output = raw( resultHandle );
		pendingGate.size = vectorSize;
		pendingGate.scale = raw( multiplierHandle );
		pendingGate.active = true;
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( firstHandle ) != peek( secondHandle )
		&& ( peek( firstHandle ) == peek( resultHandle ) || peek( secondHandle ) == peek( resultHandle ) ) ) {
		// the sigmoid of a scaled noted product times that product, in place of the sigmoid: CGELULayer's gate is complete
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( resultHandle ), CLazyResult::K_Product );
		const float* const other = peek( firstHandle ) == peek( resultHandle ) ? peek( secondHandle ) : peek( firstHandle );
		// the other factor has to be the biased product itself, still as it was noted: the buffer the gate started from,
		// still described by a note of the same product
		const int source = at >= 0 ? findLazy( other, CLazyResult::K_Product ) : -1;
		if( source >= 0 && lazy[at].gate == 2 && lazy[at].resultFloats == vectorSize && lazy[at].gateSource == other
			&& lazy[source].gate == 0 && lazy[source].residual == nullptr && lazy[source].first == lazy[at].first
			&& lazy[source].second == lazy[at].second && lazy[source].bias == lazy[at].bias ) {
			lazy[at].gate = 3;
			return;
		}
	}
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( firstHandle ) == peek( secondHandle )
		&& peek( firstHandle ) == peek( resultHandle ) ) {
		// a noted matrix multiplied by itself in place: the square joins the note
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( firstHandle ), CLazyResult::K_Affine );
		if( at >= 0 && lazy[at].resultFloats == vectorSize && !lazy[at].square && lazy[at].rowMul == nullptr
			&& lazy[at].colMul == nullptr && lazy[at].colAdd == nullptr ) {
			lazy[at].square = true;
			return;
		}
	}
	{
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const CPendingSigmoidGate g = pendingGate;
		if( g.active && g.sigmoid && raw( resultHandle ) == g.output && vectorSize == g.size
			&& ( ( raw( firstHandle ) == g.input && raw( secondHandle ) == g.output )
				|| ( raw( firstHandle ) == g.output && raw( secondHandle ) == g.input ) ) ) {
			pendingGate = CPendingSigmoidGate();
			enter();
			check( nb200_vector_op( stream, NB200_VEC_SIGMOID_MUL, g.input, nullptr, g.scale, 0.f, g.output, g.size ),
				"VectorEltwiseMultiply" );
			return;
		}
	}
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( firstHandle ) == peek( resultHandle ) ) {
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( firstHandle ), CLazyResult::K_Product );
		if( at >= 0 && lazy[at].gate == 1 && lazy[at].resultFloats == vectorSize ) {
			lazy[at].gate = 2;
			return;
		}
	}
	{
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		if( pendingGate.active && !pendingGate.sigmoid && raw( firstHandle ) == pendingGate.output
			&& raw( resultHandle ) == pendingGate.output && vectorSize == pendingGate.size ) {
			pendingGate.sigmoid = true;
			return;
		}
	}
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && batchSize == 1 ) {
		// the mask of attention added to a noted score matrix (see CLazyResult), in place or into another buffer
		const float* const mask = raw( vectorHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int product = findLazy( peek( matrixHandle ), CLazyResult::K_Product );
		if( product >= 0 && peek( matrixHandle ) == peek( resultHandle ) && lazy[product].rows == matrixHeight
			&& lazy[product].width == matrixWidth && lazy[product].bias == nullptr && lazy[product].residual == nullptr
			&& lazy[product].gate == 0 ) {
			// ... or the free terms of a fully connected layer added to its noted product
			lazy[product].bias = mask;
			lazy[product].Reads( vectorHandle, matrixWidth );
			return;
		}
		const int affine = findLazy( peek( matrixHandle ), CLazyResult::K_Affine );
		if( affine >= 0 && lazy[affine].rows == matrixHeight && lazy[affine].width == matrixWidth && !lazy[affine].square
			&& lazy[affine].colAdd == nullptr ) {
			// ... or the column addends of a noted matrix (the bias of an object normalisation)
			CLazyResult* note = deriveNote( affine, resultHandle );
			if( note != nullptr ) {
				note->colAdd = mask;
				note->Reads( vectorHandle, matrixWidth );
				return;
			}
		}
		const int at = findLazy( peek( matrixHandle ), CLazyResult::K_Scores );
		if( at >= 0 && lazy[at].resultFloats == size && matrixHeight == lazy[at].batch
			&& matrixWidth == lazy[at].seqQ * lazy[at].seqTo && lazy[at].mask == nullptr && !lazy[at].softmax ) {
			CLazyResult* note = deriveNote( at, resultHandle );
			if( note != nullptr ) {
				note->mask = mask;
				note->Reads( vectorHandle, matrixWidth );
				return;
			}
		}
	}
	if( batchSize == 1 && raw( matrixHandle ) == raw( resultHandle ) && size > 0 ) {
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		if( pendingProduct.active && pendingProduct.result == raw( resultHandle ) && pendingProduct.firstHeight == matrixHeight
			&& pendingProduct.secondHeight == matrixWidth && pendingProduct.resultRowSize == matrixWidth ) {
			cudaSetDevice( device );
			flushProduct( raw( vectorHandle ) ); // the product with the vector as its bias
			return;
		}
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
	const long long size = static_cast<long long>( matrixHeight ) * matrixWidth;
	const bool inPlace = peek( matrixHandle ) == peek( resultHandle );
	if( size > 0 && ( inPlace || CMemoryHandleInternal::Base( matrixHandle ) != CMemoryHandleInternal::Base( resultHandle ) )
		&& CMemoryHandleInternal::Base( vectorHandle ) != CMemoryHandleInternal::Base( resultHandle ) ) {
		// noted, not written (see CLazyResult) -- CObjectNormalizationLayer squares and sums this matrix (into a
		// scratch matrix), or scales and shifts it (in place when the layer runs in place); either chain then runs as
		// one pass.  In place the note's source is the result buffer itself: whoever touches it finds it written.
		CLazyResult note;
		note.kind = CLazyResult::K_Affine;
		note.rowAdd = raw( vectorHandle );
		note.result = raw( resultHandle );
		note.from = inPlace ? note.result : raw( matrixHandle );
		note.resultBase = CMemoryHandleInternal::Base( resultHandle );
		note.resultFloats = size;
		note.rows = matrixHeight; note.width = matrixWidth;
		if( !inPlace ) note.Reads( matrixHandle, size );
		note.Reads( vectorHandle, matrixHeight );
		if( noteLazy( note ) ) return;
	}
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 ) {
		// the row sums of a noted matrix (a shifted, maybe squared one): one pass over its source
		float* const sums = raw( resultHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( matrixHandle ), CLazyResult::K_Affine );
		if( at >= 0 && lazy[at].rows == matrixHeight && lazy[at].width == matrixWidth && lazy[at].rowMul == nullptr
			&& lazy[at].colMul == nullptr && lazy[at].colAdd == nullptr ) {
			const CLazyResult& note = lazy[at];
			check( nb200_sum_matrix_columns_shifted( stream, sums, note.from, matrixHeight, matrixWidth, note.rowAdd,
				note.square ? 1 : 0 ), "SumMatrixColumns" );
			for( const CLazyResult::CInput& input : note.inputs ) noteUse( input.base );
			return;
		}
	}
	check( nb200_sum_matrix_columns( stream, raw( resultHandle ), raw( matrixHandle ), matrixHeight, matrixWidth ), "SumMatrixColumns" );
}

void CB200MathEngine::MatrixSoftmaxByRows( const CConstFloatHandle& matrix, int height, int width, const CFloatHandle& result )
{
	if( lazyCount.load( std::memory_order_relaxed ) != 0 ) {
		// over a noted score matrix (see CLazyResult): noted as well
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( matrix ), CLazyResult::K_Scores );
		if( at >= 0 && !lazy[at].softmax && width == lazy[at].seqTo
			&& static_cast<long long>( height ) == static_cast<long long>( lazy[at].batch ) * lazy[at].seqQ ) {
			CLazyResult* note = deriveNote( at, result );
			if( note != nullptr ) {
				note->softmax = true;
				return;
			}
		}
	}
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
	// recorded: the bias that a fully connected layer adds next rides in the epilogue (see CPendingProduct); any other
	// call launches the product first
	std::lock_guard<std::recursive_mutex> lock( pendingMutex );
	const long long size = static_cast<long long>( firstHeight ) * secondHeight;
	if( resultRowSize == secondHeight && size > 0 && size < ( 1ll << 31 )
		&& CMemoryHandleInternal::Base( resultHandle ) != CMemoryHandleInternal::Base( firstHandle )
		&& CMemoryHandleInternal::Base( resultHandle ) != CMemoryHandleInternal::Base( secondHandle ) ) {
		// noted, not launched (see CLazyResult): the bias, the residual sum or the GELU gate that the next layers
		// apply ride in the product's epilogue; whoever else touches the result finds it written
		CLazyResult note;
		note.kind = CLazyResult::K_Product;
		note.first = raw( firstHandle );
		note.second = raw( secondHandle );
		note.result = raw( resultHandle );
		note.resultBase = CMemoryHandleInternal::Base( resultHandle );
		note.resultFloats = size;
		note.rows = firstHeight; note.depth = firstWidth; note.width = secondHeight;
		note.firstRowSize = firstRowSize; note.secondRowSize = secondRowSize;
		note.Reads( firstHandle, static_cast<long long>( firstHeight - 1 ) * firstRowSize + firstWidth );
		note.Reads( secondHandle, static_cast<long long>( secondHeight - 1 ) * secondRowSize + firstWidth );
		if( noteLazy( note ) ) return;
	}
	pendingProduct.first = raw( firstHandle );
	pendingProduct.firstHeight = firstHeight; pendingProduct.firstWidth = firstWidth; pendingProduct.firstRowSize = firstRowSize;
	pendingProduct.second = raw( secondHandle );
	pendingProduct.secondHeight = secondHeight; pendingProduct.secondRowSize = secondRowSize;
	pendingProduct.result = raw( resultHandle );
	pendingProduct.resultRowSize = resultRowSize;
	pendingProduct.active = true;
}

// first * second^T with work space from the stack allocator: a prepared second operand for tall products, room for
// split-K partial results for products with few output tiles
int CB200MathEngine::productWithScratch( int batchSize, const float* first, int firstHeight, int firstWidth, int firstRowSize,
	const float* second, int secondHeight, int secondRowSize, float* result, int resultRowSize, const float* bias,
	const float* residual, const float* gateScale, const void* secondAllocation ) const
{
	CB200MathEngine* self = const_cast<CB200MathEngine*>( this );
	nb200_epilogue withBias = {};
	withBias.bias = bias;
	withBias.residual = residual;
	withBias.ld_residual = resultRowSize;
	if( gateScale != nullptr ) {
		withBias.act = NB200_ACT_SIGMOID_GATE;
		withBias.act_param_device = gateScale;
	}
	const nb200_epilogue* const epi = ( bias != nullptr || residual != nullptr || gateScale != nullptr ) ? &withBias : nullptr;
	// a layer's weights are prepared for the tensor core once and kept for as long as nothing writes to them
	const float* prepared = batchSize == 1 && secondAllocation != nullptr
		? preparedSecondFor( secondAllocation, second, firstHeight, secondHeight, firstWidth, secondRowSize ) : nullptr;
	const size_t floats = nb200_matrix_product_scratch_floats( batchSize, firstHeight, secondHeight, firstWidth, secondRowSize );
	if( floats == 0 ) {
		return nb200_multiply_matrix_by_transposed_matrix_with_scratch( stream, batchSize, first, firstHeight, firstWidth,
			firstRowSize, second, secondHeight, secondRowSize, result, resultRowSize, nullptr, epi, precision );
	}
	CMemoryHandle scratch = self->StackAlloc( floats * sizeof( float ) );
	float* const room = static_cast<float*>( CMemoryHandleInternal::GetRaw( scratch ) );
	const int rc = prepared != nullptr
		? nb200_multiply_matrix_by_transposed_matrix_prepared( stream, first, firstHeight, firstWidth, firstRowSize, second,
			secondHeight, secondRowSize, result, resultRowSize, prepared, room, epi, precision )
		: nb200_multiply_matrix_by_transposed_matrix_with_scratch( stream, batchSize, first, firstHeight, firstWidth,
			firstRowSize, second, secondHeight, secondRowSize, result, resultRowSize, room, epi, precision );
	self->StackFree( scratch ); // stream order keeps the kernels ahead of the next user of the stack
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 ) {
		// probabilities * values, the probabilities being a noted score matrix (see CLazyResult): the whole chain as one
		// kernel over the queries, keys and values; the score matrix stays unwritten
		const float* const values = raw( secondHandle );
		float* const out = raw( resultHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( firstHandle ), CLazyResult::K_Scores );
		if( at >= 0 && lazy[at].softmax && lazy[at].batch == batchSize && lazy[at].seqQ == firstHeight
			&& lazy[at].seqTo == firstWidth && lazy[at].depth == secondWidth ) {
			const CLazyResult& note = lazy[at];
			if( nb200_attention_scores_values( stream, batchSize, note.first, note.second, values, note.seqQ, note.depth,
					note.seqTo, note.scale, note.mask, out, precision ) == NB200_OK ) {
				for( const CLazyResult::CInput& input : note.inputs ) noteUse( input.base );
				return;
			}
		}
	}
	const long long scores = static_cast<long long>( batchSize ) * firstHeight * secondWidth;
	if( precision == NB200_PREC_3XTF32 && batchSize > 0 && firstWidth == 64 && firstHeight >= 128 && secondWidth >= 128
		&& secondWidth % 4 == 0 && scores < ( 1ll << 31 )
		&& CMemoryHandleInternal::Base( resultHandle ) != CMemoryHandleInternal::Base( firstHandle )
		&& CMemoryHandleInternal::Base( resultHandle ) != CMemoryHandleInternal::Base( secondHandle ) ) {
		// the shape of queries * keys in attention: noted, not launched -- scale, mask, softmax and the product with the
		// values may follow and then run as one kernel (see CLazyResult); anything else that touches the result finds
		// it written
		CLazyResult note;
		note.kind = CLazyResult::K_Scores;
		note.first = raw( firstHandle );
		note.second = raw( secondHandle );
		note.result = raw( resultHandle );
		note.resultBase = CMemoryHandleInternal::Base( resultHandle );
		note.resultFloats = scores;
		note.batch = batchSize; note.seqQ = firstHeight; note.depth = firstWidth; note.seqTo = secondWidth;
		note.Reads( firstHandle, static_cast<long long>( batchSize ) * firstHeight * firstWidth );
		note.Reads( secondHandle, static_cast<long long>( batchSize ) * firstWidth * secondWidth );
		if( noteLazy( note ) ) return;
	}
	check( launchProduct( batchSize, raw( firstHandle ), firstHeight, firstWidth, raw( secondHandle ), secondWidth,
		raw( resultHandle ) ), "MultiplyMatrixByMatrix" );
}

int CB200MathEngine::launchProduct( int batchSize, const float* first, int firstHeight, int firstWidth, const float* second,
	int secondWidth, float* result ) const
{
	CB200MathEngine* self = const_cast<CB200MathEngine*>( this );
	// The second operand is [K x N]: the tensor-core kernel wants both operands K-major.  One transposing pass over it
	// (into stack memory) costs a read and a write of the operand and lets the product run on the TMA-fed path, which
	// is several times faster than gathering a column-major operand element by element.
	const size_t floats = static_cast<size_t>( batchSize ) * firstWidth * secondWidth;
	if( firstWidth >= 4 && secondWidth >= 4 && floats < ( static_cast<size_t>( 1 ) << 31 ) ) {
		CMemoryHandle scratch = self->StackAlloc( floats * sizeof( float ) );
		float* transposed = static_cast<float*>( CMemoryHandleInternal::GetRaw( scratch ) );
		int rc = nb200_transpose_matrix( stream, batchSize, second, firstWidth, 1, secondWidth, 1, transposed );
		if( rc == 0 ) {
			rc = productWithScratch( batchSize, first, firstHeight, firstWidth, firstWidth, transposed, secondWidth,
				firstWidth, result, secondWidth );
		}
		self->StackFree( scratch ); // stream order keeps the kernels ahead of the next user of the stack
		return rc;
	}
	return nb200_multiply_matrix_by_matrix( stream, batchSize, first, firstHeight, firstWidth, second, secondWidth, result,
		nullptr, precision );
}

void CB200MathEngine::MultiplyDiagMatrixByMatrix( const CConstFloatHandle& firstHandle, int firstSize,
	const CConstFloatHandle& secondHandle, int secondWidth, const CFloatHandle& resultHandle, int )
{
	enter();
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && peek( secondHandle ) == peek( resultHandle ) ) {
		// in place on a noted matrix: the row factors join the note
		const float* const factors = raw( firstHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( secondHandle ), CLazyResult::K_Affine );
		if( at >= 0 && lazy[at].rows == firstSize && lazy[at].width == secondWidth && !lazy[at].square
			&& lazy[at].rowMul == nullptr && lazy[at].colMul == nullptr && lazy[at].colAdd == nullptr ) {
			lazy[at].rowMul = factors;
			lazy[at].Reads( firstHandle, firstSize );
			return;
		}
	}
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
	if( lazyCount.load( std::memory_order_relaxed ) != 0 && batchSize == 1 ) {
		// a noted matrix times column factors, in place or into another buffer: the factors join the note
		const float* const factors = raw( secondHandle );
		std::lock_guard<std::recursive_mutex> lock( pendingMutex );
		const int at = findLazy( peek( firstHandle ), CLazyResult::K_Affine );
		if( at >= 0 && lazy[at].rows == height && lazy[at].width == width && !lazy[at].square && lazy[at].colMul == nullptr
			&& lazy[at].colAdd == nullptr ) {
			CLazyResult* note = deriveNote( at, resultHandle );
			if( note != nullptr ) {
				note->colMul = factors;
				note->Reads( secondHandle, width );
				return;
			}
		}
	}
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
