// Device memory for CB200MathEngine: a caching allocator (size-class free lists over cudaMalloc) and per-thread LIFO
// stacks.  Behaviour follows the shared memory mixin of the reference (NeoMathEngine/src/MemoryEngineMixin.cpp:27-226,
// MemoryPool.cpp:81-88): memoryLimit 0 means unlimited; freed heap blocks are kept for reuse until CleanUp();
// StackAlloc / StackFree are strictly LIFO per host thread; the gauges count user bytes (current, peak) and cached
// bytes (pools).
#include "B200MathEngine.h"

#include <cuda_runtime.h>

namespace NeoML {

namespace {
constexpr size_t ALIGN = 256;             // every block starts on 256 B: TMA and 16-byte vector paths always apply
constexpr size_t STACK_SLAB = 64u << 20;  // stacks grow in 64 MB slabs (the stem's channel-padding scratch is ~200 MB)

size_t roundUp( size_t v, size_t a ) { return ( v + a - 1 ) / a * a; }
}

CB200Memory::CB200Memory( int _device, size_t memoryLimit ) : device( _device ), limit( memoryLimit ) {}

CB200Memory::~CB200Memory()
{
	cudaSetDevice( device );
	for( auto& kv : freeLists ) for( void* p : kv.second ) cudaFree( p );
	for( auto& kv : live ) cudaFree( kv.first );
	for( auto& kv : stacks ) for( auto& slab : kv.second.slabs ) cudaFree( slab.first );
}

// 1, 1.5, 2, 3, 4, 6, 8 ... x 256 B, like the reference's x1.5 / x2 ladder of pool sizes
size_t CB200Memory::sizeClass( size_t bytes )
{
	size_t c = ALIGN;
	while( c < bytes ) {
		const size_t mid = c + c / 2;
		if( mid >= bytes && mid % ALIGN == 0 ) return mid;
		c *= 2;
	}
	return c;
}

void* CB200Memory::rawAlloc( size_t bytes )
{
	if( limit != 0 && reserved + bytes > limit ) return nullptr;
	void* p = nullptr;
	if( cudaMalloc( &p, bytes ) != cudaSuccess ) {
		cudaGetLastError();
		return nullptr;
	}
	reserved += bytes;
	return p;
}

void* CB200Memory::Alloc( size_t bytes )
{
	if( bytes == 0 ) bytes = 1;
	const size_t cls = sizeClass( bytes );
	std::lock_guard<std::mutex> lock( mutex );
	cudaSetDevice( device );
	void* p = nullptr;
	auto it = freeLists.find( cls );
	if( it != freeLists.end() && !it->second.empty() ) {
		p = it->second.back();
		it->second.pop_back();
		pooled -= cls;
	} else {
		p = rawAlloc( cls );
		if( p == nullptr ) {
			// give cached blocks back to the driver and retry once
			for( auto& kv : freeLists ) {
				for( void* q : kv.second ) { cudaFree( q ); reserved -= kv.first; pooled -= kv.first; }
				kv.second.clear();
			}
			p = rawAlloc( cls );
			if( p == nullptr ) return nullptr;
		}
	}
	live[p] = cls;
	current += cls;
	if( current > peak ) peak = current;
	return p;
}

void CB200Memory::Free( void* ptr )
{
	if( ptr == nullptr ) return;
	std::lock_guard<std::mutex> lock( mutex );
	auto it = live.find( ptr );
	if( it == live.end() ) return;
	const size_t cls = it->second;
	live.erase( it );
	current -= cls;
	// the engine's stream orders every kernel that used the block before any kernel that will use it next
	freeLists[cls].push_back( ptr );
	pooled += cls;
}

void* CB200Memory::StackAlloc( size_t bytes )
{
	bytes = roundUp( bytes == 0 ? 1 : bytes, ALIGN );
	std::lock_guard<std::mutex> lock( mutex );
	cudaSetDevice( device );
	CStack& st = stacks[std::this_thread::get_id()];
	while( true ) {
		if( st.slab < static_cast<int>( st.slabs.size() ) && st.offset + bytes <= st.slabs[st.slab].second ) {
			st.marks.push_back( { st.slab, st.offset, bytes } );
			char* p = st.slabs[st.slab].first + st.offset;
			st.offset += bytes;
			current += bytes;
			if( current > peak ) peak = current;
			return p;
		}
		if( st.slab + 1 < static_cast<int>( st.slabs.size() ) && st.slabs[st.slab + 1].second >= bytes ) {
			++st.slab;
			st.offset = 0;
			continue;
		}
		// a new slab on top (slabs above the current one that are too small are dropped first)
		while( static_cast<int>( st.slabs.size() ) > st.slab + ( st.slabs.empty() ? 0 : 1 ) ) {
			cudaFree( st.slabs.back().first );
			reserved -= st.slabs.back().second;
			st.slabs.pop_back();
		}
		const size_t cap = roundUp( bytes > STACK_SLAB ? bytes : STACK_SLAB, ALIGN );
		void* slab = rawAlloc( cap );
		if( slab == nullptr ) return nullptr;
		st.slabs.emplace_back( static_cast<char*>( slab ), cap );
		st.slab = static_cast<int>( st.slabs.size() ) - 1;
		st.offset = 0;
	}
}

void CB200Memory::StackFree( void* ptr )
{
	std::lock_guard<std::mutex> lock( mutex );
	auto it = stacks.find( std::this_thread::get_id() );
	if( it == stacks.end() || it->second.marks.empty() ) return;
	CStack& st = it->second;
	const CStack::CMark mark = st.marks.back();
	if( st.slabs[mark.slab].first + mark.offset != ptr ) return; // not LIFO: the caller's contract is broken, keep the stack intact
	st.marks.pop_back();
	current -= mark.bytes;
	st.slab = mark.slab;
	st.offset = mark.offset;
}

void CB200Memory::CleanUp()
{
	std::lock_guard<std::mutex> lock( mutex );
	cudaSetDevice( device );
	cudaDeviceSynchronize();
	for( auto& kv : freeLists ) {
		for( void* p : kv.second ) { cudaFree( p ); reserved -= kv.first; }
		kv.second.clear();
	}
	pooled = 0;
	auto it = stacks.find( std::this_thread::get_id() );
	if( it != stacks.end() && it->second.marks.empty() ) {
		for( auto& slab : it->second.slabs ) { cudaFree( slab.first ); reserved -= slab.second; }
		stacks.erase( it );
	}
}

size_t CB200Memory::BlockBytes( const void* ptr ) const
{
	std::lock_guard<std::mutex> lock( mutex );
	auto it = live.find( const_cast<void*>( ptr ) );
	return it == live.end() ? 0 : it->second;
}

size_t CB200Memory::StackBlockBytes( const void* ptr ) const
{
	std::lock_guard<std::mutex> lock( mutex );
	auto it = stacks.find( std::this_thread::get_id() );
	if( it == stacks.end() ) return 0;
	const CStack& st = it->second;
	for( size_t i = st.marks.size(); i-- > 0; ) {
		if( st.slabs[st.marks[i].slab].first + st.marks[i].offset == ptr ) return st.marks[i].bytes;
	}
	return 0;
}

size_t CB200Memory::FreeOnDevice() const
{
	size_t freeBytes = 0, total = 0;
	cudaSetDevice( device );
	if( cudaMemGetInfo( &freeBytes, &total ) != cudaSuccess ) {
		cudaGetLastError();
		return 0;
	}
	if( limit != 0 ) {
		const size_t left = limit > reserved ? limit - reserved : 0;
		return left < freeBytes ? left : freeBytes;
	}
	return freeBytes;
}

} // namespace NeoML
