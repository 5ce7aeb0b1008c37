#include "kv_pool.hh"

#include <algorithm>
#include <numeric>

#include "../../include/glinthawk_attn.h"
#include "gh_driver.hh"

namespace gh {

namespace {

size_t round_up( size_t v, size_t m )
{
  return ( v + m - 1 ) / m * m;
}

} // namespace

KvPool::~KvPool()
{
  destroy();
}

int KvPool::init( const PoolGeometry& g,
                  bool paged,
                  int device,
                  uint64_t page_budget,
                  uint32_t tile_rows,
                  std::string& err )
{
  geo_ = g;
  paged_ = paged;
  device_ = device;
  page_budget_ = page_budget;
  tile_rows_ = std::max<uint32_t>( 1, tile_rows );

  slot_owner_.assign( g.max_contexts, 0 );
  for ( uint32_t s = 0; s < g.max_contexts; s++ )
    free_slots_.push_back( static_cast<int32_t>( s ) );
  slots_.resize( g.max_contexts );

  if ( !paged_ ) {
    // Fully resident slots, like the reference's static Context (one allocation here instead of one per
    // context, src/arch/cuda/llama2/ops.cuh:105-122).
    geo_.page_bytes = 0;
    geo_.slot_stride = round_up( g.slot_bytes, std::lcm<size_t>( g.row_bytes, 256 ) );
    arena_bytes_ = geo_.slot_stride * g.max_contexts;
    void* p = nullptr;
    const cudaError_t e = cudaMalloc( &p, arena_bytes_ );
    if ( e != cudaSuccess ) {
      (void)cudaGetLastError();
      err = std::string( "cudaMalloc of the slot arena (" ) + std::to_string( arena_bytes_ >> 20 )
            + " MiB): " + cudaGetErrorString( e );
      arena_bytes_ = 0;
      return e == cudaErrorMemoryAllocation ? GH_ERR_OOM : GH_ERR_CUDA;
    }
    // Rows past a context's position are read by whole-tile loads (and masked); give them defined contents.
    if ( cudaMemset( p, 0, arena_bytes_ ) != cudaSuccess ) {
      err = "cudaMemset of the slot arena failed";
      cudaFree( p );
      arena_bytes_ = 0;
      return GH_ERR_CUDA;
    }
    arena_ = reinterpret_cast<CUdeviceptr>( p );
    bytes_mapped_ = arena_bytes_;
    return GH_OK;
  }

  const DriverApi* api = driver_api( err );
  if ( api == nullptr )
    return GH_ERR_CUDA;

  prop_ = {};
  prop_.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop_.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop_.location.id = device_;
  access_ = {};
  access_.location = prop_.location;
  access_.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;

  size_t gran = 0;
  CUresult r = api->MemGetAllocationGranularity( &gran, &prop_, CU_MEM_ALLOC_GRANULARITY_MINIMUM );
  if ( r != CUDA_SUCCESS || gran == 0 ) {
    err = "cuMemGetAllocationGranularity: " + driver_error( api, r );
    return GH_ERR_CUDA;
  }
  // 2 MiB blocks, as the reference's DynamicContext commits (context.hh:226), or the device's granularity
  // if that is coarser.
  geo_.page_bytes = round_up( size_t( 2 ) << 20, gran );
  geo_.slot_stride = round_up( g.slot_bytes, std::lcm<size_t>( g.row_bytes, geo_.page_bytes ) );
  arena_bytes_ = geo_.slot_stride * g.max_contexts;

  r = api->MemAddressReserve( &arena_, arena_bytes_, geo_.page_bytes, 0, 0 );
  if ( r != CUDA_SUCCESS ) {
    err = "cuMemAddressReserve(" + std::to_string( arena_bytes_ >> 30 ) + " GiB): " + driver_error( api, r );
    arena_ = 0;
    arena_bytes_ = 0;
    return GH_ERR_OOM;
  }
  arena_is_vmm_ = true;
  const size_t pages_per_slot = geo_.slot_stride / geo_.page_bytes;
  for ( auto& s : slots_ ) {
    s.page_map.assign( pages_per_slot, -1 );
    s.layer_committed.assign( g.n_layers, 0 );
  }
  return GH_OK;
}

void KvPool::destroy()
{
  if ( arena_ == 0 )
    return;
  if ( !arena_is_vmm_ ) {
    cudaFree( reinterpret_cast<void*>( arena_ ) );
  } else {
    std::string err;
    const DriverApi* api = driver_api( err );
    if ( api != nullptr ) {
      for ( int32_t s = 0; s < static_cast<int32_t>( slots_.size() ); s++ )
        reset_slot_locked( s, err );
      for ( auto h : free_pages_ )
        api->MemRelease( h );
      free_pages_.clear();
      api->MemAddressFree( arena_, arena_bytes_ );
    }
  }
  arena_ = 0;
  arena_bytes_ = 0;
  bytes_mapped_ = 0;
}

// ---- id -> slot map -------------------------------------------------------------------------------------

int KvPool::acquire( uint32_t context_id, int32_t* slot )
{
  std::lock_guard<std::mutex> lock( mu_ );
  return acquire_locked( context_id, slot );
}

uint32_t KvPool::slots_free() const
{
  std::lock_guard<std::mutex> lock( mu_ );
  return static_cast<uint32_t>( free_slots_.size() );
}

uint32_t KvPool::slots_allocated() const
{
  std::lock_guard<std::mutex> lock( mu_ );
  return static_cast<uint32_t>( id2slot_.size() );
}

uint64_t KvPool::bytes_mapped() const
{
  std::lock_guard<std::mutex> lock( mu_ );
  return bytes_mapped_;
}

uint64_t KvPool::reset_generation() const
{
  std::lock_guard<std::mutex> lock( mu_ );
  return reset_generation_;
}

int KvPool::acquire_locked( uint32_t context_id, int32_t* slot )
{
  if ( context_id == 0 ) { // NULL_CONTEXT: the empty context
    *slot = -1;
    return GH_OK;
  }
  const auto it = id2slot_.find( context_id );
  if ( it != id2slot_.end() ) {
    *slot = it->second;
    return GH_OK;
  }
  if ( free_slots_.empty() )
    return GH_ERR_NO_SLOT;
  *slot = free_slots_.front();
  free_slots_.pop_front();
  id2slot_.emplace( context_id, *slot );
  slot_owner_[*slot] = context_id;
  return GH_OK;
}

int KvPool::acquire_batch( uint64_t n, const uint32_t* ids, int32_t* slots )
{
  std::lock_guard<std::mutex> lock( mu_ );
  // First make sure every prompt of the batch can be served; bind nothing otherwise.
  size_t need = 0;
  std::vector<uint32_t> fresh;
  for ( uint64_t i = 0; i < n; i++ ) {
    if ( ids[i] != 0 && id2slot_.find( ids[i] ) == id2slot_.end()
         && std::find( fresh.begin(), fresh.end(), ids[i] ) == fresh.end() ) {
      fresh.push_back( ids[i] );
      need++;
    }
  }
  if ( need > free_slots_.size() )
    return GH_ERR_NO_SLOT;
  for ( uint64_t i = 0; i < n; i++ ) {
    const int rc = acquire_locked( ids[i], &slots[i] );
    if ( rc != GH_OK )
      return rc;
  }
  return GH_OK;
}

int KvPool::lookup( uint32_t context_id, int32_t* slot ) const
{
  std::lock_guard<std::mutex> lock( mu_ );
  const auto it = id2slot_.find( context_id );
  if ( it == id2slot_.end() )
    return GH_ERR_NOT_FOUND;
  *slot = it->second;
  return GH_OK;
}

int KvPool::release( uint32_t context_id, std::string& err )
{
  std::lock_guard<std::mutex> lock( mu_ );
  const auto it = id2slot_.find( context_id );
  if ( it == id2slot_.end() )
    return GH_ERR_NOT_FOUND;
  const int32_t slot = it->second;
  id2slot_.erase( it );
  slot_owner_[slot] = 0;
  free_slots_.push_back( slot );
  return reset_slot_locked( slot, err );
}

// ---- storage --------------------------------------------------------------------------------------------

int KvPool::reset_slot( int32_t slot, std::string& err )
{
  std::lock_guard<std::mutex> lock( mu_ );
  return reset_slot_locked( slot, err );
}

int KvPool::reset_slot_locked( int32_t slot, std::string& err )
{
  if ( !valid_slot( slot ) )
    return GH_ERR_INVALID;
  reset_generation_++;
  if ( !paged_ )
    return GH_OK;
  const DriverApi* api = driver_api( err );
  if ( api == nullptr )
    return GH_ERR_CUDA;
  SlotState& s = slots_[slot];
  int rc = GH_OK;
  for ( const Mapping& m : s.mappings ) {
    const CUresult r = api->MemUnmap( m.at, m.bytes );
    if ( r != CUDA_SUCCESS ) {
      err = "cuMemUnmap: " + driver_error( api, r );
      rc = GH_ERR_CUDA;
    }
    if ( m.bytes == geo_.page_bytes && free_pages_.size() < 65536 )
      free_pages_.push_back( m.handle );
    else
      api->MemRelease( m.handle );
    bytes_mapped_ -= m.bytes;
  }
  s.mappings.clear();
  std::fill( s.page_map.begin(), s.page_map.end(), -1 );
  std::fill( s.layer_committed.begin(), s.layer_committed.end(), 0 );
  return rc;
}

int KvPool::commit( int32_t slot, size_t begin, size_t end, std::string& err )
{
  const DriverApi* api = driver_api( err );
  if ( api == nullptr )
    return GH_ERR_CUDA;
  SlotState& s = slots_[slot];
  const size_t page = geo_.page_bytes;
  size_t p = begin / page;
  const size_t p_end = ( end + page - 1 ) / page;
  while ( p < p_end ) {
    if ( s.page_map[p] >= 0 ) {
      p++;
      continue;
    }
    size_t run_end = p + 1;
    while ( run_end < p_end && s.page_map[run_end] < 0 )
      run_end++;
    const size_t bytes = ( run_end - p ) * page;
    if ( page_budget_ != 0 && bytes_mapped_ + bytes > page_budget_ ) {
      err = "page budget exhausted (" + std::to_string( bytes_mapped_ >> 20 ) + " MiB mapped)";
      return GH_ERR_OOM;
    }
    Mapping m {};
    m.bytes = bytes;
    m.at = arena_ + static_cast<size_t>( slot ) * geo_.slot_stride + p * page;
    if ( bytes == page && !free_pages_.empty() ) {
      m.handle = free_pages_.back();
      free_pages_.pop_back();
    } else {
      const CUresult r = api->MemCreate( &m.handle, bytes, &prop_, 0 );
      if ( r != CUDA_SUCCESS ) {
        err = "cuMemCreate(" + std::to_string( bytes >> 20 ) + " MiB): " + driver_error( api, r );
        return r == CUDA_ERROR_OUT_OF_MEMORY ? GH_ERR_OOM : GH_ERR_CUDA;
      }
    }
    CUresult r = api->MemMap( m.at, bytes, 0, m.handle, 0 );
    if ( r == CUDA_SUCCESS )
      r = api->MemSetAccess( m.at, bytes, &access_, 1 );
    if ( r != CUDA_SUCCESS ) {
      err = "cuMemMap/cuMemSetAccess: " + driver_error( api, r );
      api->MemRelease( m.handle );
      return GH_ERR_CUDA;
    }
    const int32_t idx = static_cast<int32_t>( s.mappings.size() );
    s.mappings.push_back( m );
    for ( size_t q = p; q < run_end; q++ )
      s.page_map[q] = idx;
    bytes_mapped_ += bytes;
    p = run_end;
  }
  return GH_OK;
}

int KvPool::prepare( int32_t slot, uint32_t layer, uint32_t pos, bool can_release, std::string& err )
{
  std::lock_guard<std::mutex> lock( mu_ );
  return prepare_locked( slot, layer, pos, can_release, err );
}

int KvPool::prepare_batch( uint64_t n, const int32_t* slots, const uint32_t* pos, uint32_t layer, std::string& err )
{
  if ( !paged_ )
    return GH_OK;
  std::lock_guard<std::mutex> lock( mu_ );
  for ( uint64_t i = 0; i < n; i++ ) {
    if ( slots[i] < 0 )
      continue;
    const int rc = prepare_locked( slots[i], layer, pos[i], false, err );
    if ( rc != GH_OK )
      return rc;
  }
  return GH_OK;
}

int KvPool::prepare_locked( int32_t slot, uint32_t layer, uint32_t pos, bool can_release, std::string& err )
{
  if ( !valid_slot( slot ) || layer >= geo_.n_layers )
    return GH_ERR_INVALID;
  if ( pos >= geo_.seq_len )
    return GH_ERR_CAPACITY;
  if ( !paged_ )
    return GH_OK;
  if ( can_release ) {
    const int rc = reset_slot_locked( slot, err );
    if ( rc != GH_OK )
      return rc;
  }
  // The decode kernel fetches whole tiles of `tile_rows_` tokens, so the mapped region is extended to the end
  // of the tile that holds `pos` (rows past `pos` are fetched but masked).
  const size_t rows = std::min<size_t>( round_up( static_cast<size_t>( pos ) + 1, tile_rows_ ), geo_.seq_len );
  const size_t need = rows * geo_.row_bytes;
  SlotState& s = slots_[slot];
  if ( need <= s.layer_committed[layer] )
    return GH_OK;
  const size_t base = static_cast<size_t>( layer ) * geo_.layer_bytes;
  const int rc = commit( slot, base + s.layer_committed[layer], base + need, err );
  if ( rc != GH_OK )
    return rc;
  // everything up to the end of the last page touched is usable
  const size_t mapped_end = std::min( round_up( base + need, geo_.page_bytes ), base + geo_.layer_bytes );
  s.layer_committed[layer] = mapped_end - base;
  return GH_OK;
}

} // namespace gh
