// Context-slot storage and the context-id -> slot map of the attention stage (host side).
//
// Replaces three reference pieces:
//   * Context / LayerContext / TokenContext address arithmetic  (src/models/llama2/context.hh:61-190)
//   * DynamicContext over VirtualMemoryRegion, 2 MiB demand paging (context.hh:192-249,
//     src/arch/cuda/common/vmem.cuh:11-160)
//   * PreallocatingContextManager, the id -> context map          (src/compute/contextman.hh:57-197)
//
// Unlike the reference, every slot lives in ONE address range ("arena"): slot s starts at
// arena + s * slot_stride, hosted layer l at + l * layer_bytes, token t at + t * row_bytes.  A single TMA
// tensor map over the arena therefore reaches every (slot, layer, token) by row index, and a context is named
// on the device by a byte offset instead of B host-side pointer objects.  With PAGED backing the arena is only
// reserved address space; physical pages are mapped under the rows a context has actually reached and go back
// to a free list (not to the driver) when the context is released.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace gh {

struct PoolGeometry
{
  size_t elem_bytes = 0;
  size_t row_bytes = 0;   // one token of one layer: [K | V]
  size_t layer_bytes = 0; // seq_len rows
  size_t slot_bytes = 0;  // n_layers hosted layers (Context::max_size)
  size_t slot_stride = 0; // distance between slots in the arena (>= slot_bytes, multiple of row and page)
  size_t page_bytes = 0;  // mapping granularity (PAGED) or 0 (STATIC)
  uint32_t seq_len = 0, n_layers = 0, max_contexts = 0;
};

class KvPool
{
public:
  KvPool() = default;
  ~KvPool();
  KvPool( const KvPool& ) = delete;
  KvPool& operator=( const KvPool& ) = delete;

  // status codes are gh_status values; `err` receives a message on failure
  int init( const PoolGeometry& g, bool paged, int device, uint64_t page_budget, uint32_t tile_rows, std::string& err );
  void destroy();

  // Every public member below takes the pool's mutex, as the reference's context manager does around its map
  // (src/compute/contextman.hh:82, 108, 134, 184): a bookkeeping thread may bind and look up contexts while the
  // execution thread prepares rows and launches kernels.

  // ---- id -> slot map ----
  int acquire( uint32_t context_id, int32_t* slot );
  int acquire_batch( uint64_t n, const uint32_t* ids, int32_t* slots );
  int lookup( uint32_t context_id, int32_t* slot ) const;
  int release( uint32_t context_id, std::string& err );
  uint32_t slots_free() const;
  uint32_t slots_allocated() const;

  // ---- storage ----
  // make rows [0, pos] of (slot, layer) usable (rounded up to the tile the kernels read)
  int prepare( int32_t slot, uint32_t layer, uint32_t pos, bool can_release, std::string& err );
  // the same for a whole batch under one lock; slots[i] < 0 = inactive prompt
  int prepare_batch( uint64_t n, const int32_t* slots, const uint32_t* pos, uint32_t layer, std::string& err );
  int reset_slot( int32_t slot, std::string& err );
  // Counts the slot resets so far: rows that were prepared before a reset may be gone after it.
  uint64_t reset_generation() const;
  bool valid_slot( int32_t slot ) const { return slot >= 0 && static_cast<uint32_t>( slot ) < geo_.max_contexts; }

  char* arena() const { return reinterpret_cast<char*>( arena_ ); }
  size_t arena_bytes() const { return arena_bytes_; }
  long long slot_offset( int32_t slot ) const { return static_cast<long long>( slot ) * geo_.slot_stride; }
  long long layer_offset( uint32_t layer ) const { return static_cast<long long>( layer ) * geo_.layer_bytes; }
  const PoolGeometry& geometry() const { return geo_; }
  uint64_t bytes_mapped() const;
  bool paged() const { return paged_; }

private:
  struct Mapping
  {
    CUmemGenericAllocationHandle handle;
    size_t bytes;
    CUdeviceptr at;
  };
  struct SlotState
  {
    std::vector<int32_t> page_map;       // per page of the slot: index into mappings, -1 = unmapped
    std::vector<size_t> layer_committed; // per layer: bytes from the layer start known to be mapped
    std::vector<Mapping> mappings;
  };

  int acquire_locked( uint32_t context_id, int32_t* slot );
  int prepare_locked( int32_t slot, uint32_t layer, uint32_t pos, bool can_release, std::string& err );
  int reset_slot_locked( int32_t slot, std::string& err );
  int commit( int32_t slot, size_t begin, size_t end, std::string& err );

  mutable std::mutex mu_;
  uint64_t reset_generation_ = 0;

  PoolGeometry geo_ {};
  bool paged_ = false;
  int device_ = 0;
  uint32_t tile_rows_ = 1;
  uint64_t page_budget_ = 0;
  uint64_t bytes_mapped_ = 0;
  CUdeviceptr arena_ = 0;
  size_t arena_bytes_ = 0;
  bool arena_is_vmm_ = false;
  CUmemAllocationProp prop_ {};
  CUmemAccessDesc access_ {};
  std::vector<SlotState> slots_;
  std::vector<CUmemGenericAllocationHandle> free_pages_; // single-page handles kept for reuse

  std::unordered_map<uint32_t, int32_t> id2slot_;
  std::vector<uint32_t> slot_owner_;
  std::deque<int32_t> free_slots_;
};

} // namespace gh
