// C ABI of the attention stage (see include/glinthawk_attn.h for the contract of every entry point).
#include "../../include/glinthawk_attn.h"
#include "../../include/glinthawk_attn_aux.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "gh_driver.hh"
#include "gh_kernels.cuh"
#include "kv_pool.hh"
#include "planner.hh"

using namespace gh;

namespace {

constexpr uint32_t kRing = 16;       // batch descriptions that may be in flight at once
constexpr uint32_t kBatchRing = 4;   // of those, the first kBatchRing hold only what gh_attn_batch_begin uploads,
constexpr uint32_t kOpRing = 2;      // the next kOpRing the description the gh_op_* calls of a layer-step share
constexpr uint32_t kHostStages = 4;  // staging sets for the host-buffer entry point
constexpr uint32_t kExtraItems = 1024;
constexpr uint32_t kScratchSets = 4; // decode launches of one handle that may be in flight on different streams

struct DeviceGuard
{
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard( int dev )
  {
    if ( cudaGetDevice( &prev ) != cudaSuccess )
      prev = -1;
    if ( prev != dev )
      ok = cudaSetDevice( dev ) == cudaSuccess;
  }
  ~DeviceGuard()
  {
    if ( prev >= 0 )
      cudaSetDevice( prev );
  }
};

// One uploaded batch description:
// [CtxMeta x max_batch][int32 split list x max_batch][WorkItem x max_items][ptr x max_batch][pos x max_batch]
struct RingEntry
{
  char* host = nullptr; // pinned
  char* dev = nullptr;
  cudaEvent_t last_use = nullptr;
  cudaStream_t streams[4] = {}; // streams that have work referring to this entry
  int n_streams = 0;
  bool many_streams = false;
};

// Scratch of one decode launch: the partial records of contexts cut into several work items.
// A launch owns its set until its kernel has finished, so launches on different streams never share one.
struct ScratchSet
{
  float* part_o = nullptr;
  float* part_ml = nullptr;
  uint32_t* arrivals = nullptr; // [max_batch][n_kv_heads], zero whenever no launch of the set is in flight
  cudaEvent_t done = nullptr;
  cudaStream_t stream = nullptr;
  bool used = false;
  bool done_recorded = false; // `done` marks exactly the end of the set's last launch
};

struct HostStage
{
  char* q = nullptr;
  char* kv = nullptr;
  char* xb = nullptr;
  char* raw = nullptr; // conversion staging, sized for fp32
  cudaEvent_t done = nullptr;
  bool used = false;
};

} // namespace

struct gh_attn
{
  gh_attn_config cfg {};
  Shape sh {};
  size_t elem = 0;
  int device = 0;
  uint32_t sm_count = 148;
  KvPool pool;
  std::string err;
  gh_attn_stats stats {};

  const void* rope_cos = nullptr;
  const void* rope_sin = nullptr;

  // batch descriptions
  uint32_t max_items = 0;
  size_t off_split = 0, off_items = 0, off_ptrs = 0, off_pos = 0, entry_bytes = 0;
  RingEntry ring[kRing];
  uint32_t ring_next = 0;       // next transient entry, counted from kBatchRing + kOpRing
  uint32_t batch_ring_next = 0; // next entry for gh_attn_batch_begin
  uint32_t op_ring_next = 0;    // next entry for the description shared by gh_op_* calls
  // The batch the gh_op_* calls were last made for, when their pointer arrays named rows of this handle's own slots
  // (every layer of a step names the same slots and positions): its uploaded description is reused.
  int op_entry = -1;
  cudaStream_t op_stream = nullptr; // the stream its upload was issued on: only calls on that stream are ordered behind it
  uint32_t op_items = 0, op_split = 0;
  std::vector<int32_t> op_slots, op_slots_tmp;
  std::vector<uint32_t> op_pos, op_pos_tmp;
  int cur = -1; // ring entry of the batch set up last, -1 = none
  uint32_t cur_batch = 0, cur_items = 0, cur_split = 0;
  std::vector<int32_t> cur_slots;
  std::vector<uint32_t> cur_pos;
  std::vector<uint8_t> cur_layer_ready; // per hosted layer: the current batch's rows are known to be mapped
  uint64_t cur_ready_generation = 0;    // pool reset count those marks were taken at
  bool device_error_seen = false;       // a kernel's bounded wait ran out; calls are refused until it is cleared

  // split partials
  ScratchSet scratch[kScratchSets];
  uint32_t scratch_next = 0;
  bool several_streams = false; // decode launches have been seen on more than one stream
  uint32_t* dev_error = nullptr;

  bool use_mma = false;
  CUtensorMap kv_map {};

  HostStage stage[kHostStages];
  uint32_t stage_next = 0;

  // q / kv projection (allocated by the first gh_attn_project_append call)
  void* proj_xb = nullptr;        // rmsnorm output, [max_batch][dim]
  float* proj_ws = nullptr;       // fp32 sums of every piece of every tile
  bool proj_ready = false;
};

namespace {

int fail( gh_attn* h, int status, const std::string& msg )
{
  if ( h != nullptr )
    h->err = msg;
  return status;
}

int cuda_fail( gh_attn* h, const char* what, cudaError_t e )
{
  (void)cudaGetLastError();
  return fail( h, e == cudaErrorMemoryAllocation ? GH_ERR_OOM : GH_ERR_CUDA, std::string( what ) + ": " + cudaGetErrorString( e ) );
}

#define GH_CUDA( h, expr )                                                                                             \
  do {                                                                                                                 \
    const cudaError_t e__ = ( expr );                                                                                  \
    if ( e__ != cudaSuccess )                                                                                          \
      return cuda_fail( ( h ), #expr, e__ );                                                                           \
  } while ( 0 )

size_t dtype_size( uint32_t dt )
{
  return dt == GH_F32 ? 4 : 2;
}

bool dtype_ok( uint32_t dt )
{
  return dt == GH_F16 || dt == GH_F32 || dt == GH_BF16;
}

// Waits (on the host) until everything submitted so far to `st` has finished.  No event is recorded while work is
// being submitted; the wait is paid only when a buffer is about to be recycled, many launches later.
int drain_stream( gh_attn* h, cudaEvent_t ev, cudaStream_t st )
{
  cudaError_t e = cudaEventRecord( ev, st );
  if ( e == cudaSuccess )
    e = cudaEventSynchronize( ev );
  if ( e != cudaSuccess ) { // e.g. the caller destroyed the stream in the meantime
    (void)cudaGetLastError();
    GH_CUDA( h, cudaDeviceSynchronize() );
  }
  return GH_OK;
}

// Claims the next batch-description buffer, waiting (on the host) only if the device may still read it.  The
// description of the current batch (gh_attn_batch_begin) lives in entries of its own, which the transient
// uploads of the other entry points never recycle: it stays valid however many of those follow it.
enum RingKind { RING_TRANSIENT, RING_BATCH, RING_OP };

int ring_claim( gh_attn* h, int* idx, RingKind kind = RING_TRANSIENT )
{
  uint32_t k;
  if ( kind == RING_BATCH ) {
    k = h->batch_ring_next;
    h->batch_ring_next = ( k + 1 ) % kBatchRing;
  } else if ( kind == RING_OP ) {
    k = kBatchRing + h->op_ring_next;
    h->op_ring_next = ( h->op_ring_next + 1 ) % kOpRing;
  } else {
    k = kBatchRing + kOpRing + h->ring_next;
    h->ring_next = ( h->ring_next + 1 ) % ( kRing - kBatchRing - kOpRing );
  }
  RingEntry& r = h->ring[k];
  if ( r.many_streams ) {
    GH_CUDA( h, cudaDeviceSynchronize() );
  } else {
    for ( int i = 0; i < r.n_streams; i++ )
      if ( const int rc = drain_stream( h, r.last_use, r.streams[i] ); rc != GH_OK )
        return rc;
  }
  r.n_streams = 0;
  r.many_streams = false;
  *idx = static_cast<int>( k );
  return GH_OK;
}

// Notes that work referring to ring entry `idx` was submitted to `st` (no CUDA call).
int ring_touch( gh_attn* h, int idx, cudaStream_t st )
{
  RingEntry& r = h->ring[idx];
  for ( int i = 0; i < r.n_streams; i++ )
    if ( r.streams[i] == st )
      return GH_OK;
  if ( r.n_streams < 4 )
    r.streams[r.n_streams++] = st;
  else
    r.many_streams = true;
  return GH_OK;
}

CtxMeta* entry_ctx( gh_attn* h, char* base )
{
  (void)h;
  return reinterpret_cast<CtxMeta*>( base );
}
int32_t* entry_split( gh_attn* h, char* base )
{
  return reinterpret_cast<int32_t*>( base + h->off_split );
}
WorkItem* entry_items( gh_attn* h, char* base )
{
  return reinterpret_cast<WorkItem*>( base + h->off_items );
}
void** entry_ptrs( gh_attn* h, char* base )
{
  return reinterpret_cast<void**>( base + h->off_ptrs );
}
uint32_t* entry_pos( gh_attn* h, char* base )
{
  return reinterpret_cast<uint32_t*>( base + h->off_pos );
}

// Plans `ctx` (kv_off and pos filled in by the caller) and uploads the description into a fresh ring entry.
int plan_and_upload( gh_attn* h, std::vector<CtxMeta>& ctx, cudaStream_t st, int* entry, uint32_t* n_items,
                     uint32_t* n_split, RingKind kind = RING_TRANSIENT )
{
  PlanParams pp;
  pp.n_kv_heads = h->use_mma ? h->sh.n_kv_heads : h->sh.n_heads;
  pp.sm_count = h->sm_count;
  pp.tile = decode_mma_tile_tokens();
  pp.fixed_chunk = h->cfg.decode_chunk;
  pp.max_items = h->max_items;
  pp.blocks_per_sm = h->use_mma ? 4 : 8;
  Plan plan;
  if ( !plan_batch( pp, ctx, plan ) )
    return fail( h, GH_ERR_INVALID, "batch does not fit the work-item buffer" );

  int idx;
  if ( const int rc = ring_claim( h, &idx, kind ); rc != GH_OK )
    return rc;
  RingEntry& r = h->ring[idx];
  std::memcpy( entry_ctx( h, r.host ), ctx.data(), ctx.size() * sizeof( CtxMeta ) );
  std::memcpy( entry_split( h, r.host ), plan.split_ctx.data(), plan.split_ctx.size() * sizeof( int32_t ) );
  std::memcpy( entry_items( h, r.host ), plan.items.data(), plan.items.size() * sizeof( WorkItem ) );
  // one copy covers the context records, the split list and the items (adjacent, up to the items actually used)
  const size_t bytes = h->off_items + plan.items.size() * sizeof( WorkItem );
  GH_CUDA( h, cudaMemcpyAsync( r.dev, r.host, bytes, cudaMemcpyHostToDevice, st ) );
  if ( const int rc = ring_touch( h, idx, st ); rc != GH_OK )
    return rc;
  *entry = idx;
  *n_items = static_cast<uint32_t>( plan.items.size() );
  *n_split = static_cast<uint32_t>( plan.split_ctx.size() );
  h->stats.last_items = *n_items;
  h->stats.last_split_contexts = *n_split;
  h->stats.batch_plans++;
  h->stats.last_chunk = plan.chunk;
  return GH_OK;
}

// Hands out the next scratch set.  If its previous launch ran on another stream, the new stream is made to wait
// for it on the device; the host never blocks here.
int scratch_claim( gh_attn* h, cudaStream_t st, ScratchSet** out )
{
  ScratchSet& s = h->scratch[h->scratch_next];
  h->scratch_next = ( h->scratch_next + 1 ) % kScratchSets;
  if ( s.used && s.stream != st ) {
    // From now on the end of every launch is marked, so that streams wait for exactly what they must.  This
    // first time, everything submitted to the set's previous stream so far stands in for its last launch.
    h->several_streams = true;
    cudaError_t e = s.done_recorded ? cudaSuccess : cudaEventRecord( s.done, s.stream );
    if ( e == cudaSuccess )
      e = cudaStreamWaitEvent( st, s.done, 0 );
    if ( e != cudaSuccess ) {
      (void)cudaGetLastError();
      GH_CUDA( h, cudaDeviceSynchronize() );
    }
  }
  *out = &s;
  return GH_OK;
}

int scratch_release( gh_attn* h, ScratchSet* s, cudaStream_t st )
{
  s->used = true;
  s->stream = st;
  s->done_recorded = false;
  if ( h->several_streams ) { // single-stream callers never pay for this
    GH_CUDA( h, cudaEventRecord( s->done, st ) );
    s->done_recorded = true;
  }
  return GH_OK;
}

DecodeArgs decode_args( gh_attn* h, int entry, uint32_t n_items, uint32_t n_split, long long layer_off, const void* q,
                        void* xb )
{
  DecodeArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.ctx = entry_ctx( h, h->ring[entry].dev );
  a.items = entry_items( h, h->ring[entry].dev );
  a.n_items = n_items;
  a.split_ctx = entry_split( h, h->ring[entry].dev );
  a.n_split_ctx = n_split;
  a.arena = h->pool.arena();
  a.layer_off = layer_off;
  a.q = q;
  a.xb = xb;
  a.dev_error = h->dev_error;
  a.sm_count = h->sm_count;
  // (the CUDA-core kernel is followed by a merge launch when contexts are cut, which has to wait for all of it)
  a.trigger_early = ( h->use_mma || n_split == 0 ) ? 1u : 0u;
  return a;
}

int run_decode( gh_attn* h, DecodeArgs a, bool allow_mma, cudaStream_t st )
{
  ScratchSet* set = nullptr;
  if ( const int rc = scratch_claim( h, st, &set ); rc != GH_OK )
    return rc;
  a.part_o = set->part_o;
  a.part_ml = set->part_ml;
  a.arrivals = set->arrivals;
  cudaError_t e;
  if ( h->use_mma && allow_mma ) {
    e = launch_decode_mma( a, &h->kv_map, st, &h->stats.kernel_launches );
    h->stats.last_kernel = 1;
  } else {
    e = launch_decode_generic( a, st, &h->stats.kernel_launches );
    h->stats.last_kernel = 0;
  }
  if ( e != cudaSuccess )
    return cuda_fail( h, "decode kernel launch", e );
  return scratch_release( h, set, st );
}

// Once a kernel has reported that one of its bounded waits ran out, its outputs cannot be trusted: every compute
// entry point refuses to go on until gh_attn_clear_device_error has been called.
int check_device_ok( gh_attn* h )
{
  if ( h->device_error_seen )
    return fail( h, GH_ERR_CUDA,
                 "a kernel reported a timed-out wait (gh_attn_stats.device_error = " + std::to_string( h->stats.device_error )
                   + "); call gh_attn_clear_device_error" );
  return GH_OK;
}

int check_batch_ready( gh_attn* h, uint32_t layer )
{
  if ( const int rc = check_device_ok( h ); rc != GH_OK )
    return rc;
  if ( h->cur < 0 )
    return fail( h, GH_ERR_STATE, "no batch: call gh_attn_batch_begin first" );
  if ( layer >= h->sh.n_layers )
    return fail( h, GH_ERR_INVALID, "layer " + std::to_string( layer ) + " is not hosted" );
  return GH_OK;
}

// Context::prepare for every active prompt of the current batch (src/models/llama2/model.hh:617-621).
// The batch is walked once per (batch, layer): the append and decode calls of a layer-step share the result, which
// stays valid until a slot is reset.
int prepare_layer( gh_attn* h, uint32_t layer )
{
  if ( !h->pool.paged() )
    return GH_OK;
  const uint64_t generation = h->pool.reset_generation();
  if ( generation != h->cur_ready_generation ) {
    std::fill( h->cur_layer_ready.begin(), h->cur_layer_ready.end(), 0 );
    h->cur_ready_generation = generation;
  }
  if ( h->cur_layer_ready[layer] )
    return GH_OK;
  const int rc = h->pool.prepare_batch( h->cur_batch, h->cur_slots.data(), h->cur_pos.data(), layer, h->err );
  if ( rc == GH_OK )
    h->cur_layer_ready[layer] = 1;
  return rc;
}

} // namespace

// ---------------------------------------------------------------------------------------------------------

extern "C" {

const char* gh_status_string( int status )
{
  switch ( status ) {
    case GH_OK: return "ok";
    case GH_ERR_INVALID: return "invalid argument";
    case GH_ERR_CUDA: return "CUDA error";
    case GH_ERR_NO_SLOT: return "no free context slot";
    case GH_ERR_CAPACITY: return "token position beyond slot capacity";
    case GH_ERR_OOM: return "out of device memory";
    case GH_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case GH_ERR_STATE: return "call out of order";
    case GH_ERR_NOT_FOUND: return "unknown context id";
    default: return "unknown status";
  }
}

int gh_attn_create( const gh_attn_config* cfg, gh_attn_t* out )
{
  if ( cfg == nullptr || out == nullptr || cfg->struct_size != sizeof( gh_attn_config ) )
    return GH_ERR_INVALID;
  *out = nullptr;
  if ( cfg->n_heads == 0 || cfg->n_kv_heads == 0 || cfg->n_heads % cfg->n_kv_heads != 0
       || cfg->n_heads / cfg->n_kv_heads > (uint32_t)kMaxGroup || cfg->head_size == 0 || cfg->head_size % 8 != 0
       || cfg->head_size > (uint32_t)kMaxHeadSize || cfg->seq_len == 0 || cfg->n_layers_hosted == 0
       || !dtype_ok( cfg->dtype ) || cfg->max_batch == 0 || cfg->max_batch > (uint32_t)kMaxBatch
       || cfg->max_contexts == 0 || cfg->backing > GH_BACKING_PAGED )
    return GH_ERR_INVALID;

  int n_dev = 0;
  if ( cudaGetDeviceCount( &n_dev ) != cudaSuccess || cfg->device < 0 || cfg->device >= n_dev ) {
    (void)cudaGetLastError();
    return GH_ERR_CUDA; // no CPU path exists: without a usable device the stage cannot be created
  }

  // every early return below releases whatever has been allocated so far
  struct Destroyer
  {
    void operator()( gh_attn* p ) const { gh_attn_destroy( p ); }
  };
  std::unique_ptr<gh_attn, Destroyer> h( new gh_attn() );
  h->cfg = *cfg;
  h->device = cfg->device;
  DeviceGuard guard( h->device );
  if ( !guard.ok )
    return GH_ERR_CUDA;
  GH_CUDA( h.get(), cudaFree( nullptr ) );

  cudaDeviceProp prop {};
  GH_CUDA( h.get(), cudaGetDeviceProperties( &prop, h->device ) );
  h->sm_count = static_cast<uint32_t>( prop.multiProcessorCount );

  Shape& sh = h->sh;
  sh.n_heads = cfg->n_heads;
  sh.n_kv_heads = cfg->n_kv_heads;
  sh.group = cfg->n_heads / cfg->n_kv_heads;
  sh.head_size = cfg->head_size;
  sh.kv_dim = cfg->n_kv_heads * cfg->head_size;
  sh.seq_len = cfg->seq_len;
  sh.n_layers = cfg->n_layers_hosted;
  sh.row_elems = 2 * sh.kv_dim;
  h->elem = dtype_size( cfg->dtype );

  h->use_mma = !cfg->force_generic && decode_mma_supported( sh, cfg->dtype );

  PoolGeometry g;
  g.elem_bytes = h->elem;
  g.row_bytes = static_cast<size_t>( sh.row_elems ) * h->elem;
  g.layer_bytes = g.row_bytes * sh.seq_len;
  g.slot_bytes = g.layer_bytes * sh.n_layers;
  g.seq_len = sh.seq_len;
  g.n_layers = sh.n_layers;
  g.max_contexts = cfg->max_contexts;
  const uint32_t tile = h->use_mma ? decode_mma_tile_tokens() : 1;
  int rc = h->pool.init( g, cfg->backing == GH_BACKING_PAGED, h->device, cfg->page_budget, tile, h->err );
  if ( rc != GH_OK ) {
    std::fprintf( stderr, "gh_attn_create: %s\n", h->err.c_str() );
    return rc;
  }

  // batch-description ring
  h->max_items = cfg->max_batch + kExtraItems;
  h->off_split = sizeof( CtxMeta ) * cfg->max_batch;
  h->off_items = h->off_split + ( sizeof( int32_t ) * cfg->max_batch + 15 ) / 16 * 16;
  h->off_ptrs = h->off_items + sizeof( WorkItem ) * h->max_items;
  h->off_pos = h->off_ptrs + sizeof( void* ) * cfg->max_batch;
  h->entry_bytes = ( h->off_pos + sizeof( uint32_t ) * cfg->max_batch + 255 ) / 256 * 256;
  GH_CUDA( h.get(), cudaMallocHost( reinterpret_cast<void**>( &h->ring[0].host ), h->entry_bytes * kRing ) );
  GH_CUDA( h.get(), cudaMalloc( reinterpret_cast<void**>( &h->ring[0].dev ), h->entry_bytes * kRing ) );
  char* host_all = h->ring[0].host;
  char* dev_all = h->ring[0].dev;
  for ( uint32_t k = 0; k < kRing; k++ ) {
    h->ring[k].host = host_all + k * h->entry_bytes;
    h->ring[k].dev = dev_all + k * h->entry_bytes;
    GH_CUDA( h.get(), cudaEventCreateWithFlags( &h->ring[k].last_use, cudaEventDisableTiming ) );
  }

  // split partial records: one per (work item, query head)
  const size_t recs = static_cast<size_t>( h->max_items ) * sh.n_heads;
  for ( auto& set : h->scratch ) {
    GH_CUDA( h.get(), cudaMalloc( reinterpret_cast<void**>( &set.part_o ), recs * sh.head_size * sizeof( float ) ) );
    GH_CUDA( h.get(), cudaMalloc( reinterpret_cast<void**>( &set.part_ml ), recs * 2 * sizeof( float ) ) );
    const size_t counts = static_cast<size_t>( cfg->max_batch ) * sh.n_kv_heads * sizeof( uint32_t );
    GH_CUDA( h.get(), cudaMalloc( reinterpret_cast<void**>( &set.arrivals ), counts ) );
    GH_CUDA( h.get(), cudaMemset( set.arrivals, 0, counts ) );
    GH_CUDA( h.get(), cudaEventCreateWithFlags( &set.done, cudaEventDisableTiming ) );
  }
  GH_CUDA( h.get(), cudaMalloc( reinterpret_cast<void**>( &h->dev_error ), sizeof( uint32_t ) ) );
  GH_CUDA( h.get(), cudaMemset( h->dev_error, 0, sizeof( uint32_t ) ) );
  h->stats.scratch_bytes = kScratchSets * ( recs * ( sh.head_size + 2 ) * sizeof( float ) )
                           + 2 * h->entry_bytes * kRing;

  if ( h->use_mma ) {
    const DriverApi* api = driver_api( h->err );
    if ( api == nullptr )
      return GH_ERR_CUDA;
    const uint64_t total_rows = h->pool.arena_bytes() / g.row_bytes;
    if ( total_rows >= ( 1ull << 31 ) ) { // TMA coordinates are signed 32-bit
      h->use_mma = false; // arena too large for one descriptor; the CUDA-core kernel has no such limit
    } else {
      const cuuint64_t dims[2] = { sh.row_elems, total_rows };
      const cuuint64_t strides[1] = { g.row_bytes };
      const cuuint32_t box[2] = { 64, decode_mma_box_rows() };
      const cuuint32_t estr[2] = { 1, 1 };
      const CUresult r = api->TensorMapEncodeTiled(
        &h->kv_map, cfg->dtype == GH_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
        h->pool.arena(), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE );
      if ( r != CUDA_SUCCESS ) {
        h->err = "cuTensorMapEncodeTiled: " + driver_error( api, r );
        std::fprintf( stderr, "gh_attn_create: %s\n", h->err.c_str() );
        return GH_ERR_CUDA;
      }
      GH_CUDA( h.get(), decode_mma_prepare() );
      GH_CUDA( h.get(), prefill_umma_prepare() );
    }
  }

  h->cur_slots.reserve( cfg->max_batch );
  h->cur_pos.reserve( cfg->max_batch );
  *out = h.release();
  return GH_OK;
}

int gh_attn_destroy( gh_attn_t h )
{
  if ( h == nullptr )
    return GH_ERR_INVALID;
  DeviceGuard guard( h->device );
  cudaDeviceSynchronize();
  for ( auto& s : h->stage ) {
    cudaFree( s.q );
    cudaFree( s.kv );
    cudaFree( s.xb );
    cudaFree( s.raw );
    if ( s.done )
      cudaEventDestroy( s.done );
  }
  for ( auto& r : h->ring )
    if ( r.last_use )
      cudaEventDestroy( r.last_use );
  if ( h->ring[0].host )
    cudaFreeHost( h->ring[0].host );
  cudaFree( h->ring[0].dev );
  for ( auto& set : h->scratch ) {
    cudaFree( set.part_o );
    cudaFree( set.part_ml );
    cudaFree( set.arrivals );
    if ( set.done )
      cudaEventDestroy( set.done );
  }
  cudaFree( h->dev_error );
  cudaFree( h->proj_xb );
  cudaFree( h->proj_ws );
  h->pool.destroy();
  (void)cudaGetLastError();
  delete h;
  return GH_OK;
}

const char* gh_attn_last_error( gh_attn_t h )
{
  return h != nullptr ? h->err.c_str() : "null handle";
}

int gh_attn_get_stats( gh_attn_t h, gh_attn_stats* out )
{
  if ( h == nullptr || out == nullptr )
    return GH_ERR_INVALID;
  DeviceGuard guard( h->device );
  h->stats.bytes_mapped = h->pool.bytes_mapped();
  h->stats.bytes_reserved = h->pool.arena_bytes();
  h->stats.slots_free = h->pool.slots_free();
  h->stats.slots_allocated = h->pool.slots_allocated();
  uint32_t flag = 0;
  GH_CUDA( h, cudaMemcpy( &flag, h->dev_error, sizeof( flag ), cudaMemcpyDeviceToHost ) );
  h->stats.device_error = flag;
  h->device_error_seen = flag != 0;
  *out = h->stats;
  return GH_OK;
}

int gh_attn_synchronize( gh_attn_t h, void* stream )
{
  if ( h == nullptr )
    return GH_ERR_INVALID;
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  uint32_t flag = 0; // the kernels' error word rides along: the caller learns of a timed-out wait where it waits anyway
  GH_CUDA( h, cudaMemcpyAsync( &flag, h->dev_error, sizeof( flag ), cudaMemcpyDeviceToHost, st ) );
  GH_CUDA( h, cudaStreamSynchronize( st ) );
  if ( flag != 0 ) {
    h->stats.device_error = flag;
    h->device_error_seen = true;
    return check_device_ok( h );
  }
  return GH_OK;
}

int gh_attn_inject_device_error( gh_attn_t h, uint32_t bits )
{
  if ( h == nullptr )
    return GH_ERR_INVALID;
  DeviceGuard guard( h->device );
  uint32_t flag = 0;
  GH_CUDA( h, cudaDeviceSynchronize() );
  GH_CUDA( h, cudaMemcpy( &flag, h->dev_error, sizeof( flag ), cudaMemcpyDeviceToHost ) );
  flag |= bits;
  GH_CUDA( h, cudaMemcpy( h->dev_error, &flag, sizeof( flag ), cudaMemcpyHostToDevice ) );
  return GH_OK;
}

int gh_attn_clear_device_error( gh_attn_t h )
{
  if ( h == nullptr )
    return GH_ERR_INVALID;
  DeviceGuard guard( h->device );
  GH_CUDA( h, cudaDeviceSynchronize() );
  GH_CUDA( h, cudaMemset( h->dev_error, 0, sizeof( uint32_t ) ) );
  for ( auto& set : h->scratch ) // a launch that gave up may have left arrival counts behind
    GH_CUDA( h, cudaMemset( set.arrivals, 0, static_cast<size_t>( h->cfg.max_batch ) * h->sh.n_kv_heads * sizeof( uint32_t ) ) );
  h->stats.device_error = 0;
  h->device_error_seen = false;
  return GH_OK;
}

int gh_attn_set_rope_tables( gh_attn_t h, const void* freq_cis_real, const void* freq_cis_imag )
{
  if ( h == nullptr || freq_cis_real == nullptr || freq_cis_imag == nullptr )
    return GH_ERR_INVALID;
  h->rope_cos = freq_cis_real;
  h->rope_sin = freq_cis_imag;
  return GH_OK;
}

// ---- slot pool ------------------------------------------------------------------------------------------

int gh_slot_acquire( gh_attn_t h, uint32_t context_id, int32_t* slot )
{
  if ( h == nullptr || slot == nullptr )
    return GH_ERR_INVALID;
  return h->pool.acquire( context_id, slot ); // status only: may run beside the thread that owns the handle
}

int gh_slots_acquire_batch( gh_attn_t h, uint64_t batch, const uint32_t* context_ids, int32_t* slots )
{
  if ( h == nullptr || ( batch > 0 && ( context_ids == nullptr || slots == nullptr ) ) )
    return GH_ERR_INVALID;
  return h->pool.acquire_batch( batch, context_ids, slots ); // status only, as above
}

int gh_slot_lookup( gh_attn_t h, uint32_t context_id, int32_t* slot )
{
  if ( h == nullptr || slot == nullptr )
    return GH_ERR_INVALID;
  return h->pool.lookup( context_id, slot );
}

int gh_slot_release( gh_attn_t h, uint32_t context_id )
{
  if ( h == nullptr )
    return GH_ERR_INVALID;
  DeviceGuard guard( h->device );
  return h->pool.release( context_id, h->err );
}

int gh_slot_prepare( gh_attn_t h, int32_t slot, uint32_t layer, uint32_t pos, int can_release )
{
  if ( h == nullptr )
    return GH_ERR_INVALID;
  if ( slot == -1 )
    return GH_OK; // the empty context prepares trivially (context.hh:223-225)
  DeviceGuard guard( h->device );
  const int rc = h->pool.prepare( slot, layer, pos, can_release != 0, h->err );
  if ( rc == GH_ERR_INVALID )
    h->err = "slot or layer out of range";
  else if ( rc == GH_ERR_CAPACITY )
    h->err = "token position " + std::to_string( pos ) + " >= slot capacity " + std::to_string( h->sh.seq_len );
  return rc;
}

int gh_slot_layer_ptr( gh_attn_t h, int32_t slot, uint32_t layer, void** ptr )
{
  if ( h == nullptr || ptr == nullptr )
    return GH_ERR_INVALID;
  if ( slot == -1 ) { // empty context -> empty layer view (context.hh:117-118)
    *ptr = nullptr;
    return GH_OK;
  }
  if ( !h->pool.valid_slot( slot ) || layer >= h->sh.n_layers )
    return fail( h, GH_ERR_INVALID, "slot or layer out of range" );
  *ptr = h->pool.arena() + h->pool.slot_offset( slot ) + h->pool.layer_offset( layer );
  return GH_OK;
}

int gh_slot_token_ptr( gh_attn_t h, int32_t slot, uint32_t layer, uint32_t token, void** ptr )
{
  if ( h != nullptr && token >= h->sh.seq_len )
    return fail( h, GH_ERR_CAPACITY, "token beyond slot capacity" );
  const int rc = gh_slot_layer_ptr( h, slot, layer, ptr );
  if ( rc == GH_OK && *ptr != nullptr )
    *ptr = static_cast<char*>( *ptr ) + static_cast<size_t>( token ) * h->pool.geometry().row_bytes;
  return rc;
}

size_t gh_slot_bytes( gh_attn_t h )
{
  return h != nullptr ? h->pool.geometry().slot_bytes : 0;
}

// ---- fused hot path -------------------------------------------------------------------------------------

int gh_attn_batch_begin( gh_attn_t h, uint64_t batch, const int32_t* slots, const uint32_t* pos, void* stream )
{
  if ( h == nullptr || batch == 0 || batch > h->cfg.max_batch || slots == nullptr || pos == nullptr )
    return fail( h, GH_ERR_INVALID, "bad batch arguments" );
  DeviceGuard guard( h->device );
  std::vector<CtxMeta> ctx( batch );
  for ( uint64_t i = 0; i < batch; i++ ) {
    CtxMeta& c = ctx[i];
    c = CtxMeta {};
    c.pos = pos[i];
    if ( slots[i] == -1 ) {
      c.kv_off = kInactive;
      continue;
    }
    if ( !h->pool.valid_slot( slots[i] ) )
      return fail( h, GH_ERR_INVALID, "slot out of range at batch index " + std::to_string( i ) );
    if ( pos[i] >= h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY,
                   "token position " + std::to_string( pos[i] ) + " >= slot capacity at batch index " + std::to_string( i ) );
    c.kv_off = h->pool.slot_offset( slots[i] );
  }
  h->cur = -1;
  int entry;
  uint32_t n_items, n_split;
  if ( const int rc = plan_and_upload( h, ctx, static_cast<cudaStream_t>( stream ), &entry, &n_items, &n_split, RING_BATCH );
       rc != GH_OK )
    return rc;
  h->cur = entry;
  h->cur_layer_ready.assign( h->sh.n_layers, 0 );
  h->cur_batch = static_cast<uint32_t>( batch );
  h->cur_items = n_items;
  h->cur_split = n_split;
  h->cur_slots.assign( slots, slots + batch );
  h->cur_pos.assign( pos, pos + batch );
  return GH_OK;
}

// The kernels move q, new K/V rows, cache rows and outputs in 16-byte pieces.  cudaMalloc'ed buffers and rows of the
// model's sizes always satisfy this; anything else is turned away here instead of faulting on the device.
static bool aligned16( const void* p )
{
  return ( reinterpret_cast<uintptr_t>( p ) & 15 ) == 0;
}
static int misaligned( gh_attn* h )
{
  return fail( h, GH_ERR_INVALID, "device buffers must be 16-byte aligned" );
}
static bool rows_aligned16( void* const* rows, uint64_t batch )
{
  for ( uint64_t i = 0; rows != nullptr && i < batch; i++ )
    if ( !aligned16( rows[i] ) )
      return false;
  return true;
}

int gh_attn_append( gh_attn_t h, uint32_t layer, void* q_inout, const void* kv_new, void* stream )
{
  if ( h == nullptr || kv_new == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( q_inout ) || !aligned16( kv_new ) )
    return misaligned( h );
  if ( const int rc = check_batch_ready( h, layer ); rc != GH_OK )
    return rc;
  if ( h->rope_cos == nullptr )
    return fail( h, GH_ERR_STATE, "RoPE tables not set" );
  DeviceGuard guard( h->device );
  if ( const int rc = prepare_layer( h, layer ); rc != GH_OK )
    return rc;
  AppendArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.batch = h->cur_batch;
  a.ctx = entry_ctx( h, h->ring[h->cur].dev );
  a.arena = h->pool.arena();
  a.layer_off = h->pool.layer_offset( layer );
  a.q = q_inout;
  a.kv_new = kv_new;
  a.rope_cos = h->rope_cos;
  a.rope_sin = h->rope_sin;
  a.dependent_launch = h->cfg.pipeline_steps != 0 ? 2u : 1u;
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  if ( const cudaError_t e = launch_append( a, st, &h->stats.kernel_launches ); e != cudaSuccess )
    return cuda_fail( h, "append kernel launch", e );
  return ring_touch( h, h->cur, st );
}

// rmsnorm + projections + RoPE + append.  Destination rows either come from the current batch's slots (ctx != nullptr)
// or are given as device pointers with their positions (token_rows / pos_dev, the reference's token contexts).
static int project_common( gh_attn* h,
                           uint32_t batch,
                           const void* x,
                           const void* rms_weight,
                           const void* wq,
                           const void* wkv,
                           void* q_out,
                           const void* rope_cos,
                           const void* rope_sin,
                           const CtxMeta* ctx,
                           long long layer_off,
                           void* const* token_rows,
                           const uint32_t* pos_dev,
                           cudaStream_t st )
{
  if ( !h->use_mma || !project_supported( h->sh, h->cfg.dtype ) )
    return fail( h, GH_ERR_UNSUPPORTED,
                 "the fused projection needs fp16 or bf16 storage and dim, kv_dim that are multiples of 128" );
  const DriverApi* api = driver_api( h->err );
  if ( api == nullptr )
    return GH_ERR_CUDA;
  const uint32_t dim = h->sh.n_heads * h->sh.head_size;
  ProjectArgs a {};
  uint32_t grid = 0;
  project_plan( h->sh, h->sm_count, &a, &grid );
  if ( !h->proj_ready ) { // first call: scratch for the normalised activations and the stream-K pieces
    GH_CUDA( h, project_prepare() );
    GH_CUDA( h, cudaMalloc( &h->proj_xb, static_cast<size_t>( h->cfg.max_batch ) * dim * h->elem ) );
    GH_CUDA( h, cudaMalloc( reinterpret_cast<void**>( &h->proj_ws ), project_workspace_bytes( a ) ) );
    h->stats.scratch_bytes += static_cast<size_t>( h->cfg.max_batch ) * dim * h->elem + project_workspace_bytes( a );
    h->proj_ready = true;
  }

  // rmsnorm for the whole batch (src/models/llama2/model.hh:331-335)
  if ( const cudaError_t e = launch_rmsnorm( h->proj_xb, x, rms_weight, batch, dim, h->cfg.dtype, st, &h->stats.kernel_launches );
       e != cudaSuccess )
    return cuda_fail( h, "rmsnorm launch", e );

  const CUtensorMapDataType dt = h->cfg.dtype == GH_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  auto encode = [&]( CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows ) -> int {
    const cuuint64_t dims[2] = { dim, rows };
    const cuuint64_t strides[1] = { static_cast<cuuint64_t>( dim ) * h->elem };
    const cuuint32_t box[2] = { 64, box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = api->TensorMapEncodeTiled( map, dt, 2, const_cast<void*>( base ), dims, strides, box, estr,
                                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE );
    if ( r != CUDA_SUCCESS )
      return fail( h, GH_ERR_CUDA, "cuTensorMapEncodeTiled (projection): " + driver_error( api, r ) );
    return GH_OK;
  };
  CUtensorMap wq_map {}, wkv_map {}, xb_map {};
  if ( const int rc = encode( &wq_map, wq, dim, 128 ); rc != GH_OK )
    return rc;
  if ( const int rc = encode( &wkv_map, wkv, 2ull * h->sh.kv_dim, 128 ); rc != GH_OK )
    return rc;

  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.ctx = ctx;
  a.token_rows = token_rows;
  a.pos = pos_dev;
  a.arena = h->pool.arena();
  a.layer_off = layer_off;
  a.q_out = q_out;
  a.rope_cos = rope_cos;
  a.rope_sin = rope_sin;
  a.ws = h->proj_ws;
  a.dev_error = h->dev_error;
  // the MMA's N takes at most project_max_rows() batch rows: larger batches go in slices (the weights are then
  // streamed once per slice)
  for ( uint32_t b0 = 0; b0 < batch; b0 += project_max_rows() ) {
    a.batch0 = b0;
    a.batch = std::min( project_max_rows(), batch - b0 );
    a.nb = ( a.batch + 15 ) / 16 * 16;
    if ( const int rc = encode( &xb_map, h->proj_xb, batch, a.nb ); rc != GH_OK )
      return rc;
    if ( const cudaError_t e = launch_project( a, grid, &wq_map, &wkv_map, &xb_map, st, &h->stats.kernel_launches );
         e != cudaSuccess )
      return cuda_fail( h, "projection launch", e );
  }
  return GH_OK;
}

int gh_attn_project_append( gh_attn_t h,
                            uint32_t layer,
                            const void* x,
                            const void* rms_weight,
                            const void* wq,
                            const void* wkv,
                            void* q_out,
                            void* stream )
{
  if ( h == nullptr || x == nullptr || rms_weight == nullptr || wq == nullptr || wkv == nullptr || q_out == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( x ) || !aligned16( rms_weight ) || !aligned16( wq ) || !aligned16( wkv ) || !aligned16( q_out ) )
    return misaligned( h );
  if ( const int rc = check_batch_ready( h, layer ); rc != GH_OK )
    return rc;
  if ( h->rope_cos == nullptr )
    return fail( h, GH_ERR_STATE, "RoPE tables not set" );
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  if ( const int rc = prepare_layer( h, layer ); rc != GH_OK )
    return rc;
  if ( const int rc = project_common( h, h->cur_batch, x, rms_weight, wq, wkv, q_out, h->rope_cos, h->rope_sin,
                                      entry_ctx( h, h->ring[h->cur].dev ), h->pool.layer_offset( layer ), nullptr, nullptr, st );
       rc != GH_OK )
    return rc;
  return ring_touch( h, h->cur, st );
}

int gh_attn_decode( gh_attn_t h, uint32_t layer, const void* q, void* xb, void* stream )
{
  if ( h == nullptr || q == nullptr || xb == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( q ) || !aligned16( xb ) )
    return misaligned( h );
  if ( const int rc = check_batch_ready( h, layer ); rc != GH_OK )
    return rc;
  DeviceGuard guard( h->device );
  if ( const int rc = prepare_layer( h, layer ); rc != GH_OK )
    return rc;
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  DecodeArgs a = decode_args( h, h->cur, h->cur_items, h->cur_split, h->pool.layer_offset( layer ), q, xb );
  // Between gh_attn_batch_begin (whose upload orders everything before it) and this launch the library's kernels
  // write row `pos` of the batch's contexts and nothing else of their K/V.
  a.stream_old_rows_early = 1;
  if ( const int rc = run_decode( h, a, true, st ); rc != GH_OK )
    return rc;
  return ring_touch( h, h->cur, st );
}

int gh_attn_step( gh_attn_t h, uint32_t layer, void* q_inout, const void* kv_new, void* xb, void* stream )
{
  if ( const int rc = gh_attn_append( h, layer, q_inout, kv_new, stream ); rc != GH_OK )
    return rc;
  return gh_attn_decode( h, layer, q_inout, xb, stream );
}

int gh_attn_prefill_chunk( gh_attn_t h,
                           uint32_t layer,
                           uint64_t n_ctx,
                           const int32_t* slots,
                           const uint32_t* pos0,
                           uint32_t n_tokens,
                           void* q_inout,
                           const void* kv_new,
                           void* xb,
                           void* stream )
{
  if ( h == nullptr || slots == nullptr || pos0 == nullptr || q_inout == nullptr || kv_new == nullptr || xb == nullptr
       || n_ctx == 0 || n_ctx > h->cfg.max_batch || n_tokens == 0 )
    return fail( h, GH_ERR_INVALID, "bad prefill arguments" );
  if ( !aligned16( q_inout ) || !aligned16( kv_new ) || !aligned16( xb ) )
    return misaligned( h );
  if ( layer >= h->sh.n_layers )
    return fail( h, GH_ERR_INVALID, "layer is not hosted" );
  if ( h->rope_cos == nullptr )
    return fail( h, GH_ERR_STATE, "RoPE tables not set" );
  if ( const int rc = check_device_ok( h ); rc != GH_OK )
    return rc;
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );

  // the chunk's rows must fit the slots; map pages up to the chunk's last token
  std::vector<CtxMeta> base( n_ctx );
  for ( uint64_t i = 0; i < n_ctx; i++ ) {
    base[i] = CtxMeta {};
    base[i].pos = pos0[i];
    if ( slots[i] == -1 ) {
      base[i].kv_off = kInactive;
      continue;
    }
    if ( !h->pool.valid_slot( slots[i] ) )
      return fail( h, GH_ERR_INVALID, "slot out of range at index " + std::to_string( i ) );
    if ( static_cast<uint64_t>( pos0[i] ) + n_tokens > h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY, "chunk runs past the slot capacity at index " + std::to_string( i ) );
    base[i].kv_off = h->pool.slot_offset( slots[i] );
    if ( const int rc = h->pool.prepare( slots[i], layer, pos0[i] + n_tokens - 1, false, h->err ); rc != GH_OK )
      return rc;
  }

  // 1. one append launch for every (context, token) of the chunk
  {
    int idx;
    if ( const int rc = ring_claim( h, &idx ); rc != GH_OK )
      return rc;
    RingEntry& r = h->ring[idx];
    std::memcpy( entry_ctx( h, r.host ), base.data(), n_ctx * sizeof( CtxMeta ) );
    GH_CUDA( h, cudaMemcpyAsync( r.dev, r.host, n_ctx * sizeof( CtxMeta ), cudaMemcpyHostToDevice, st ) );
    AppendArgs a {};
    a.sh = h->sh;
    a.dtype = h->cfg.dtype;
    a.batch = static_cast<uint32_t>( n_ctx );
    a.tokens_per_ctx = n_tokens;
    a.ctx = entry_ctx( h, r.dev );
    a.arena = h->pool.arena();
    a.layer_off = h->pool.layer_offset( layer );
    a.q = q_inout;
    a.kv_new = kv_new;
    a.rope_cos = h->rope_cos;
    a.rope_sin = h->rope_sin;
    if ( const cudaError_t e = launch_append( a, st, &h->stats.kernel_launches ); e != cudaSuccess )
      return cuda_fail( h, "prefill append launch", e );
    if ( const int rc = ring_touch( h, idx, st ); rc != GH_OK )
      return rc;
  }

  // 2a. tensor-core kernels: consecutive tokens of a context share one block per kv head, so they share every K/V
  //     fetch.  Work item = (context, token group), never cut.  The tcgen05 kernel packs
  //     128 / group tokens into a block; the warp-level kernel in chunk mode packs 16 / group (groups the tcgen05
  //     kernel does not take).
  const bool umma = h->use_mma && prefill_umma_supported( h->sh, h->cfg.dtype );
  CUtensorMap q_map {}, xb_map {};
  if ( umma ) {
    const DriverApi* api = driver_api( h->err );
    if ( api == nullptr )
      return GH_ERR_CUDA;
    // [contexts][chunk tokens][heads][head_size], innermost first; one box = half the head dims of one kv head's
    // query heads for one query block
    const uint64_t hb = static_cast<uint64_t>( h->sh.head_size ) * h->elem;
    const cuuint64_t dims[4] = { h->sh.head_size, h->sh.n_heads, n_tokens, n_ctx };
    const cuuint64_t strides[3] = { hb, hb * h->sh.n_heads, hb * h->sh.n_heads * n_tokens };
    const cuuint32_t box[4] = { 64, h->sh.group, prefill_umma_tokens_per_item( h->sh ), 1 };
    const cuuint32_t estr[4] = { 1, 1, 1, 1 };
    const CUtensorMapDataType dt = h->cfg.dtype == GH_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    for ( int which = 0; which < 2; which++ ) {
      const CUresult r = api->TensorMapEncodeTiled( which == 0 ? &q_map : &xb_map, dt, 4, which == 0 ? q_inout : xb, dims,
                                                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE );
      if ( r != CUDA_SUCCESS ) {
        h->err = "cuTensorMapEncodeTiled (prompt chunk): " + driver_error( api, r );
        return GH_ERR_CUDA;
      }
    }
  }
  if ( umma || ( h->use_mma && decode_mma_chunk_supported( h->sh ) ) ) {
    const uint32_t per_item = umma ? prefill_umma_tokens_per_item( h->sh ) : 16 / h->sh.group;
    std::vector<WorkItem> items;
    for ( uint64_t i = 0; i < n_ctx; i++ ) {
      if ( base[i].kv_off == kInactive )
        continue;
      for ( uint32_t g = 0; g * per_item < n_tokens; g++ ) {
        WorkItem w;
        w.ctx = static_cast<int32_t>( i );
        // (tcgen05 kernel: the arena row where the context's layer 0 starts; the chunk mode of the decode kernel: 0)
        w.t_begin = umma ? static_cast<int32_t>( base[i].kv_off / static_cast<long long>( h->pool.geometry().row_bytes ) ) : 0;
        w.t_end = static_cast<int32_t>( pos0[i] + std::min( n_tokens, ( g + 1 ) * per_item ) ); // last token's prefix
        w.split = static_cast<int32_t>( g );
        items.push_back( w );
      }
    }
    // Contexts with the longest prefix first, and the query blocks of one context next to each other (longest
    // first): blocks that run at the same time then read the same few contexts' K/V rows, which stay in L2.
    std::stable_sort( items.begin(), items.end(), [&]( const WorkItem& x, const WorkItem& y ) {
      if ( x.ctx != y.ctx ) {
        const uint32_t px = pos0[x.ctx], py = pos0[y.ctx];
        return px != py ? px > py : x.ctx < y.ctx;
      }
      return x.t_end > y.t_end;
    } );
    for ( auto& c : base )
      c.nsplits = 1;
    for ( size_t i0 = 0; i0 < items.size(); i0 += h->max_items ) {
      const size_t n = std::min<size_t>( h->max_items, items.size() - i0 );
      int idx;
      if ( const int rc = ring_claim( h, &idx ); rc != GH_OK )
        return rc;
      RingEntry& r = h->ring[idx];
      std::memcpy( entry_ctx( h, r.host ), base.data(), n_ctx * sizeof( CtxMeta ) );
      std::memcpy( entry_items( h, r.host ), items.data() + i0, n * sizeof( WorkItem ) );
      GH_CUDA( h, cudaMemcpyAsync( r.dev, r.host, h->off_items + n * sizeof( WorkItem ), cudaMemcpyHostToDevice, st ) );
      DecodeArgs a = decode_args( h, idx, static_cast<uint32_t>( n ), 0, h->pool.layer_offset( layer ), q_inout, xb );
      a.chunk_tokens = n_tokens;
      a.layer_row = static_cast<int32_t>( h->pool.layer_offset( layer ) / static_cast<long long>( h->pool.geometry().row_bytes ) );
      if ( umma ) {
        if ( const cudaError_t e = launch_prefill_umma( a, &h->kv_map, &q_map, &xb_map, st, &h->stats.kernel_launches ); e != cudaSuccess )
          return cuda_fail( h, "prefill kernel launch", e );
        h->stats.last_kernel = 2;
      } else if ( const int rc = run_decode( h, a, true, st ); rc != GH_OK ) {
        return rc;
      }
      if ( const int rc = ring_touch( h, idx, st ); rc != GH_OK )
        return rc;
    }
    return GH_OK;
  }

  // 2b. otherwise every (context, token) is a decode problem over its own prefix, launched in slices of at
  //    most max_batch problems
  const size_t q_row_bytes = static_cast<size_t>( h->sh.n_heads ) * h->sh.head_size * h->elem;
  const uint64_t total = n_ctx * n_tokens;
  std::vector<CtxMeta> slice;
  for ( uint64_t v0 = 0; v0 < total; v0 += h->cfg.max_batch ) {
    const uint64_t v1 = std::min<uint64_t>( total, v0 + h->cfg.max_batch );
    slice.assign( v1 - v0, CtxMeta {} );
    for ( uint64_t v = v0; v < v1; v++ ) {
      const uint64_t i = v / n_tokens, t = v - i * n_tokens;
      slice[v - v0] = base[i];
      slice[v - v0].pos = base[i].pos + static_cast<uint32_t>( t );
    }
    int entry;
    uint32_t n_items, n_split;
    if ( const int rc = plan_and_upload( h, slice, st, &entry, &n_items, &n_split ); rc != GH_OK )
      return rc;
    const DecodeArgs a = decode_args( h, entry, n_items, n_split, h->pool.layer_offset( layer ),
                                      static_cast<const char*>( q_inout ) + v0 * q_row_bytes,
                                      static_cast<char*>( xb ) + v0 * q_row_bytes );
    if ( const int rc = run_decode( h, a, true, st ); rc != GH_OK )
      return rc;
    if ( const int rc = ring_touch( h, entry, st ); rc != GH_OK )
      return rc;
  }
  return GH_OK;
}

int gh_attn_forward_attention_host( gh_attn_t h,
                                    uint32_t layer,
                                    uint32_t io_dtype,
                                    const void* q_host,
                                    const void* kv_host,
                                    void* xb_host,
                                    void* stream )
{
  if ( h == nullptr || q_host == nullptr || kv_host == nullptr || xb_host == nullptr || !dtype_ok( io_dtype ) )
    return fail( h, GH_ERR_INVALID, "bad argument" );
  if ( const int rc = check_batch_ready( h, layer ); rc != GH_OK )
    return rc;
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  const size_t B = h->cur_batch;
  const size_t q_elems = B * h->sh.n_heads * h->sh.head_size;
  const size_t kv_elems = B * h->sh.row_elems;

  HostStage& s = h->stage[h->stage_next];
  h->stage_next = ( h->stage_next + 1 ) % kHostStages;
  if ( s.q == nullptr ) {
    const size_t mb = h->cfg.max_batch;
    GH_CUDA( h, cudaMalloc( reinterpret_cast<void**>( &s.q ), mb * h->sh.n_heads * h->sh.head_size * h->elem ) );
    GH_CUDA( h, cudaMalloc( reinterpret_cast<void**>( &s.kv ), mb * h->sh.row_elems * h->elem ) );
    GH_CUDA( h, cudaMalloc( reinterpret_cast<void**>( &s.xb ), mb * h->sh.n_heads * h->sh.head_size * h->elem ) );
    GH_CUDA( h, cudaMalloc( reinterpret_cast<void**>( &s.raw ),
                            mb * ( h->sh.n_heads * h->sh.head_size + h->sh.row_elems ) * sizeof( float ) ) );
    GH_CUDA( h, cudaEventCreateWithFlags( &s.done, cudaEventDisableTiming ) );
  }
  if ( s.used ) // the staging set may still be in use by an earlier layer on another stream: order on the device
    GH_CUDA( h, cudaStreamWaitEvent( st, s.done, 0 ) );
  s.used = true;

  const size_t io = dtype_size( io_dtype );
  if ( io_dtype == h->cfg.dtype ) {
    GH_CUDA( h, cudaMemcpyAsync( s.q, q_host, q_elems * io, cudaMemcpyHostToDevice, st ) );
    GH_CUDA( h, cudaMemcpyAsync( s.kv, kv_host, kv_elems * io, cudaMemcpyHostToDevice, st ) );
  } else {
    char* raw_q = s.raw;
    char* raw_kv = s.raw + q_elems * io;
    GH_CUDA( h, cudaMemcpyAsync( raw_q, q_host, q_elems * io, cudaMemcpyHostToDevice, st ) );
    GH_CUDA( h, cudaMemcpyAsync( raw_kv, kv_host, kv_elems * io, cudaMemcpyHostToDevice, st ) );
    GH_CUDA( h, launch_convert( s.q, h->cfg.dtype, raw_q, io_dtype, q_elems, st, &h->stats.kernel_launches ) );
    GH_CUDA( h, launch_convert( s.kv, h->cfg.dtype, raw_kv, io_dtype, kv_elems, st, &h->stats.kernel_launches ) );
  }
  if ( const int rc = gh_attn_step( h, layer, s.q, s.kv, s.xb, stream ); rc != GH_OK )
    return rc;
  if ( io_dtype == h->cfg.dtype ) {
    GH_CUDA( h, cudaMemcpyAsync( xb_host, s.xb, q_elems * io, cudaMemcpyDeviceToHost, st ) );
  } else {
    GH_CUDA( h, launch_convert( s.raw, io_dtype, s.xb, h->cfg.dtype, q_elems, st, &h->stats.kernel_launches ) );
    GH_CUDA( h, cudaMemcpyAsync( xb_host, s.raw, q_elems * io, cudaMemcpyDeviceToHost, st ) );
  }
  GH_CUDA( h, cudaEventRecord( s.done, st ) );
  return GH_OK;
}

static_assert( sizeof( gh_wire_metadata ) == 32 && sizeof( gh_wire_prompt ) == 57, "wire structs must stay packed" );

int gh_attn_forward_attention_state( gh_attn_t h, uint32_t first_layer_hosted, void* state, size_t state_bytes, void* stream )
{
  if ( h == nullptr || state == nullptr || state_bytes < sizeof( gh_wire_metadata ) )
    return fail( h, GH_ERR_INVALID, "no state, or too short for its metadata" );
  char* bytes = static_cast<char*>( state );
  gh_wire_metadata md;
  std::memcpy( &md, bytes, sizeof( md ) );
  if ( md.batch_size == 0 || md.batch_size > h->cfg.max_batch || !dtype_ok( md.dtype ) )
    return fail( h, GH_ERR_INVALID, "state with a batch size or dtype this stage does not take" );
  if ( md.next_stage != GH_STAGE_ATTENTION )
    return fail( h, GH_ERR_STATE, "the state's next stage is not attention" );
  if ( md.has_queries == 0 || md.has_kvs == 0 )
    return fail( h, GH_ERR_UNSUPPORTED, "the state carries no queries or no key-values" );
  if ( md.next_layer < first_layer_hosted || md.next_layer - first_layer_hosted >= h->sh.n_layers )
    return fail( h, GH_ERR_INVALID, "layer " + std::to_string( md.next_layer ) + " is not hosted" );
  const uint32_t layer = md.next_layer - first_layer_hosted;
  const size_t B = md.batch_size, sz = dtype_size( md.dtype );
  const size_t dim = static_cast<size_t>( h->sh.n_heads ) * h->sh.head_size;
  const size_t off_prompts = sizeof( gh_wire_metadata );
  const size_t off_act = off_prompts + B * sizeof( gh_wire_prompt );
  const size_t off_q = off_act + ( md.has_activations != 0 ? B * dim * sz : 0 );
  const size_t off_kv = off_q + B * dim * sz;
  if ( off_kv + B * h->sh.row_elems * sz != state_bytes )
    return fail( h, GH_ERR_INVALID, "state of " + std::to_string( state_bytes ) + " bytes, its metadata describes "
                                      + std::to_string( off_kv + B * h->sh.row_elems * sz ) );

  // get_contexts: every active prompt's slot, all or nothing (contextman.hh:127-171)
  std::vector<uint32_t> ids( B ), pos( B );
  std::vector<int32_t> slots( B );
  for ( size_t i = 0; i < B; i++ ) {
    gh_wire_prompt pr;
    std::memcpy( &pr, bytes + off_prompts + i * sizeof( gh_wire_prompt ), sizeof( pr ) );
    ids[i] = pr.active != 0 ? pr.context_id : 0u;
    pos[i] = pr.token_pos;
  }
  if ( const int rc = h->pool.acquire_batch( B, ids.data(), slots.data() ); rc != GH_OK )
    return fail( h, rc, "not enough free context slots for the state's prompts" );
  DeviceGuard guard( h->device );
  for ( size_t i = 0; i < B; i++ ) {
    if ( slots[i] < 0 )
      continue;
    // Context::prepare( next_layer, token_pos, token_pos == 0 && first_layer_served == next_layer ), model.hh:617-621
    const int rc = h->pool.prepare( slots[i], layer, pos[i], pos[i] == 0 && layer == 0, h->err );
    if ( rc != GH_OK )
      return rc == GH_ERR_CAPACITY ? fail( h, rc, "token position beyond slot capacity in the state" ) : rc;
  }
  if ( const int rc = gh_attn_batch_begin( h, B, slots.data(), pos.data(), stream ); rc != GH_OK )
    return rc;
  // q in, new [K,V] rows in, attention output back over the queries buffer (model.hh:697-722)
  if ( const int rc = gh_attn_forward_attention_host( h, layer, md.dtype, bytes + off_q, bytes + off_kv, bytes + off_q, stream );
       rc != GH_OK )
    return rc;
  if ( const int rc = gh_attn_synchronize( h, stream ); rc != GH_OK )
    return rc;
  md.next_stage = GH_STAGE_POST_ATTENTION;
  std::memcpy( bytes, &md, sizeof( md ) );
  return GH_OK;
}

// ---- the reference's operations, argument for argument -------------------------------------------------

namespace {

// Uploads a host array of device pointers (and optionally positions) into a fresh ring entry.
int upload_ptrs( gh_attn* h, uint64_t batch, const void* const* ptrs, const uint32_t* pos, cudaStream_t st, int* entry )
{
  if ( batch == 0 || batch > h->cfg.max_batch || ptrs == nullptr )
    return fail( h, GH_ERR_INVALID, "bad batch arguments" );
  int idx;
  if ( const int rc = ring_claim( h, &idx ); rc != GH_OK )
    return rc;
  RingEntry& r = h->ring[idx];
  std::memcpy( entry_ptrs( h, r.host ), ptrs, batch * sizeof( void* ) );
  if ( pos != nullptr )
    std::memcpy( entry_pos( h, r.host ), pos, batch * sizeof( uint32_t ) );
  GH_CUDA( h, cudaMemcpyAsync( r.dev + h->off_ptrs, r.host + h->off_ptrs, h->entry_bytes - h->off_ptrs,
                               cudaMemcpyHostToDevice, st ) );
  if ( const int rc = ring_touch( h, idx, st ); rc != GH_OK )
    return rc;
  *entry = idx;
  return GH_OK;
}

// The reference hands its operations host arrays of row pointers (src/models/llama2/base.hh:197-202).  When every
// non-null pointer names a row of this handle's own slots, all in one hosted layer, the call can run on the same
// kernels and the same kind of batch description as gh_attn_append / gh_attn_decode, and nothing but the first call
// of a step has to upload anything.  `token_rows`: the pointers are token rows (their position is part of the address;
// it must agree with pos[] where that is given); otherwise they are layer bases and pos[] gives the positions.
// Fills h->op_slots_tmp / op_pos_tmp and *layer; false = some pointer is foreign memory (or nothing is active).
bool resolve_own_rows( gh_attn* h, uint64_t batch, const void* const* ptrs, const uint32_t* pos, bool token_rows,
                       uint32_t* layer )
{
  const PoolGeometry& g = h->pool.geometry();
  const char* arena = h->pool.arena();
  const size_t arena_bytes = h->pool.arena_bytes();
  h->op_slots_tmp.resize( batch );
  h->op_pos_tmp.resize( batch );
  long long the_layer = -1;
  for ( uint64_t i = 0; i < batch; i++ ) {
    if ( ptrs[i] == nullptr ) {
      h->op_slots_tmp[i] = -1;
      h->op_pos_tmp[i] = 0; // an inactive prompt's position means nothing (copy_kv_cache does not even receive it)
      continue;
    }
    const char* p = static_cast<const char*>( ptrs[i] );
    if ( p < arena || p >= arena + arena_bytes )
      return false;
    const size_t off = static_cast<size_t>( p - arena );
    const size_t slot = off / g.slot_stride, within = off % g.slot_stride;
    if ( within >= g.slot_bytes )
      return false;
    const size_t l = within / g.layer_bytes, rem = within % g.layer_bytes;
    if ( rem % g.row_bytes != 0 || ( the_layer >= 0 && static_cast<long long>( l ) != the_layer ) )
      return false;
    const uint32_t row = static_cast<uint32_t>( rem / g.row_bytes );
    if ( token_rows ? ( pos != nullptr && pos[i] != row ) : ( row != 0 ) )
      return false;
    the_layer = static_cast<long long>( l );
    h->op_slots_tmp[i] = static_cast<int32_t>( slot );
    h->op_pos_tmp[i] = token_rows ? row : pos[i];
  }
  if ( the_layer < 0 )
    return false;
  *layer = static_cast<uint32_t>( the_layer );
  return true;
}

// The uploaded description for (op_slots_tmp, op_pos_tmp): the one already on the device when they equal the last
// call's, else a fresh plan and upload.
int op_batch_entry( gh_attn* h, uint64_t batch, cudaStream_t st )
{
  if ( h->op_entry >= 0 && h->op_stream == st && h->op_slots == h->op_slots_tmp && h->op_pos == h->op_pos_tmp )
    return GH_OK;
  h->op_entry = -1;
  std::vector<CtxMeta> ctx( batch );
  for ( uint64_t i = 0; i < batch; i++ ) {
    ctx[i] = CtxMeta {};
    ctx[i].pos = h->op_pos_tmp[i];
    ctx[i].kv_off = h->op_slots_tmp[i] < 0 ? kInactive : h->pool.slot_offset( h->op_slots_tmp[i] );
  }
  int entry;
  if ( const int rc = plan_and_upload( h, ctx, st, &entry, &h->op_items, &h->op_split, RING_OP ); rc != GH_OK )
    return rc;
  h->op_entry = entry;
  h->op_stream = st;
  h->op_slots.swap( h->op_slots_tmp );
  h->op_pos.swap( h->op_pos_tmp );
  return GH_OK;
}

// copy_kv_cache and / or apply_rope on rows of the handle's own slots: the append kernels driven by the shared
// description, no pointer array on the device.
int append_own_rows( gh_attn* h, uint64_t batch, uint32_t layer, void* q, const void* kv_new, const void* rope_cos,
                     const void* rope_sin, cudaStream_t st )
{
  if ( const int rc = op_batch_entry( h, batch, st ); rc != GH_OK )
    return rc;
  AppendArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.batch = static_cast<uint32_t>( batch );
  a.ctx = entry_ctx( h, h->ring[h->op_entry].dev );
  a.arena = h->pool.arena();
  a.layer_off = h->pool.layer_offset( layer );
  a.q = q;
  a.kv_new = kv_new;
  a.rope_cos = rope_cos;
  a.rope_sin = rope_sin;
  a.dependent_launch = h->cfg.pipeline_steps != 0 ? 2u : 1u;
  if ( const cudaError_t e = launch_append( a, st, &h->stats.kernel_launches ); e != cudaSuccess )
    return cuda_fail( h, "append kernel launch", e );
  return ring_touch( h, h->op_entry, st );
}

ScoreArgs score_args( gh_attn* h, int entry, uint64_t batch, const void* q, void* att, void* xb )
{
  ScoreArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.batch = static_cast<uint32_t>( batch );
  a.layer_bases = reinterpret_cast<const void* const*>( entry_ptrs( h, h->ring[entry].dev ) );
  a.pos = entry_pos( h, h->ring[entry].dev );
  a.q = q;
  a.att = att;
  a.xb = xb;
  return a;
}

} // namespace

int gh_op_copy_kv_cache( gh_attn_t h, void* const* token_rows, const void* state_kv, uint64_t batch, void* stream )
{
  if ( h == nullptr || state_kv == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( state_kv ) || ( batch <= h->cfg.max_batch && !rows_aligned16( token_rows, batch ) ) )
    return misaligned( h );
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  uint32_t layer;
  if ( batch > 0 && batch <= h->cfg.max_batch && token_rows != nullptr
       && resolve_own_rows( h, batch, const_cast<const void* const*>( token_rows ), nullptr, true, &layer ) )
    return append_own_rows( h, batch, layer, nullptr, state_kv, nullptr, nullptr, st );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, const_cast<const void* const*>( token_rows ), nullptr, st, &entry ); rc != GH_OK )
    return rc;
  AppendArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.batch = static_cast<uint32_t>( batch );
  a.token_rows = entry_ptrs( h, h->ring[entry].dev );
  a.kv_new = state_kv;
  if ( const cudaError_t e = launch_append( a, st, &h->stats.kernel_launches ); e != cudaSuccess )
    return cuda_fail( h, "copy_kv_cache launch", e );
  return ring_touch( h, entry, st );
}

int gh_op_apply_rope( gh_attn_t h,
                      uint64_t batch,
                      const uint32_t* pos,
                      const void* freq_cis_real,
                      const void* freq_cis_imag,
                      void* state_q,
                      void* const* token_rows,
                      void* stream )
{
  if ( h == nullptr || pos == nullptr || freq_cis_real == nullptr || freq_cis_imag == nullptr || state_q == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( state_q ) || !aligned16( freq_cis_real ) || !aligned16( freq_cis_imag )
       || ( batch <= h->cfg.max_batch && !rows_aligned16( token_rows, batch ) ) )
    return misaligned( h );
  for ( uint64_t i = 0; i < batch && i < h->cfg.max_batch; i++ )
    if ( token_rows != nullptr && token_rows[i] != nullptr && pos[i] >= h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY, "token position beyond the RoPE tables" );
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  uint32_t layer;
  if ( batch > 0 && batch <= h->cfg.max_batch && token_rows != nullptr
       && resolve_own_rows( h, batch, const_cast<const void* const*>( token_rows ), pos, true, &layer ) )
    return append_own_rows( h, batch, layer, state_q, nullptr, freq_cis_real, freq_cis_imag, st );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, const_cast<const void* const*>( token_rows ), pos, st, &entry ); rc != GH_OK )
    return rc;
  AppendArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.batch = static_cast<uint32_t>( batch );
  a.token_rows = entry_ptrs( h, h->ring[entry].dev );
  a.pos = entry_pos( h, h->ring[entry].dev );
  a.q = state_q;
  a.rope_cos = freq_cis_real;
  a.rope_sin = freq_cis_imag;
  if ( const cudaError_t e = launch_append( a, st, &h->stats.kernel_launches ); e != cudaSuccess )
    return cuda_fail( h, "apply_rope launch", e );
  return ring_touch( h, entry, st );
}

int gh_op_copy_kv_cache_apply_rope( gh_attn_t h,
                                    uint64_t batch,
                                    const uint32_t* pos,
                                    const void* freq_cis_real,
                                    const void* freq_cis_imag,
                                    void* state_q,
                                    void* const* token_rows,
                                    const void* state_kv,
                                    void* stream )
{
  if ( h == nullptr || pos == nullptr || freq_cis_real == nullptr || freq_cis_imag == nullptr || state_q == nullptr
       || state_kv == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( state_q ) || !aligned16( state_kv ) || !aligned16( freq_cis_real ) || !aligned16( freq_cis_imag )
       || ( batch <= h->cfg.max_batch && !rows_aligned16( token_rows, batch ) ) )
    return misaligned( h );
  for ( uint64_t i = 0; i < batch && i < h->cfg.max_batch; i++ )
    if ( token_rows != nullptr && token_rows[i] != nullptr && pos[i] >= h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY, "token position beyond the RoPE tables" );
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  uint32_t layer;
  if ( batch > 0 && batch <= h->cfg.max_batch && token_rows != nullptr
       && resolve_own_rows( h, batch, const_cast<const void* const*>( token_rows ), pos, true, &layer ) )
    return append_own_rows( h, batch, layer, state_q, state_kv, freq_cis_real, freq_cis_imag, st );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, const_cast<const void* const*>( token_rows ), pos, st, &entry ); rc != GH_OK )
    return rc;
  AppendArgs a {};
  a.sh = h->sh;
  a.dtype = h->cfg.dtype;
  a.batch = static_cast<uint32_t>( batch );
  a.token_rows = entry_ptrs( h, h->ring[entry].dev );
  a.pos = entry_pos( h, h->ring[entry].dev );
  a.q = state_q;
  a.kv_new = state_kv;
  a.rope_cos = freq_cis_real;
  a.rope_sin = freq_cis_imag;
  if ( const cudaError_t e = launch_append( a, st, &h->stats.kernel_launches ); e != cudaSuccess )
    return cuda_fail( h, "copy_kv_cache + apply_rope launch", e );
  return ring_touch( h, entry, st );
}

int gh_op_project_append( gh_attn_t h,
                          uint64_t batch,
                          const void* x,
                          const void* rms_weight,
                          const void* wq,
                          const void* wkv,
                          void* state_q,
                          const uint32_t* pos,
                          const void* freq_cis_real,
                          const void* freq_cis_imag,
                          void* const* token_rows,
                          void* stream )
{
  if ( h == nullptr || x == nullptr || rms_weight == nullptr || wq == nullptr || wkv == nullptr || state_q == nullptr
       || pos == nullptr || freq_cis_real == nullptr || freq_cis_imag == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( !aligned16( x ) || !aligned16( rms_weight ) || !aligned16( wq ) || !aligned16( wkv ) || !aligned16( state_q )
       || ( batch <= h->cfg.max_batch && !rows_aligned16( token_rows, batch ) ) )
    return misaligned( h );
  for ( uint64_t i = 0; i < batch && i < h->cfg.max_batch; i++ )
    if ( token_rows != nullptr && token_rows[i] != nullptr && pos[i] >= h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY, "token position beyond the RoPE tables" );
  if ( const int rc = check_device_ok( h ); rc != GH_OK )
    return rc;
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, const_cast<const void* const*>( token_rows ), pos, st, &entry ); rc != GH_OK )
    return rc;
  if ( const int rc = project_common( h, static_cast<uint32_t>( batch ), x, rms_weight, wq, wkv, state_q, freq_cis_real,
                                      freq_cis_imag, nullptr, 0, entry_ptrs( h, h->ring[entry].dev ),
                                      entry_pos( h, h->ring[entry].dev ), st );
       rc != GH_OK )
    return rc;
  return ring_touch( h, entry, st );
}

static int check_positions( gh_attn* h, uint64_t batch, const void* const* bases, const uint32_t* pos )
{
  if ( pos == nullptr || bases == nullptr || batch == 0 || batch > h->cfg.max_batch )
    return fail( h, GH_ERR_INVALID, "bad batch arguments" );
  for ( uint64_t i = 0; i < batch; i++ )
    if ( bases[i] != nullptr && pos[i] >= h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY, "token position beyond slot capacity at batch index " + std::to_string( i ) );
  return GH_OK;
}

int gh_op_attention_0_gemm( gh_attn_t h,
                            const void* query,
                            const void* const* layer_bases,
                            void* att,
                            uint64_t batch,
                            const uint32_t* pos,
                            void* stream )
{
  if ( h == nullptr || query == nullptr || att == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( const int rc = check_positions( h, batch, layer_bases, pos ); rc != GH_OK )
    return rc;
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, layer_bases, pos, st, &entry ); rc != GH_OK )
    return rc;
  if ( const cudaError_t e = launch_scores( score_args( h, entry, batch, query, att, nullptr ), st, &h->stats.kernel_launches );
       e != cudaSuccess )
    return cuda_fail( h, "attention_0_gemm launch", e );
  return ring_touch( h, entry, st );
}

int gh_op_attention_softmax( gh_attn_t h, void* att, const uint32_t* pos, void* temp_buffer, uint64_t batch, void* stream )
{
  (void)temp_buffer;
  if ( h == nullptr || att == nullptr || pos == nullptr || batch == 0 || batch > h->cfg.max_batch )
    return fail( h, GH_ERR_INVALID, "bad argument" );
  for ( uint64_t i = 0; i < batch; i++ )
    if ( pos[i] >= h->sh.seq_len )
      return fail( h, GH_ERR_CAPACITY, "token position beyond slot capacity" );
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  std::vector<const void*> none( batch, nullptr );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, none.data(), pos, st, &entry ); rc != GH_OK )
    return rc;
  if ( const cudaError_t e = launch_softmax( score_args( h, entry, batch, nullptr, att, nullptr ), st, &h->stats.kernel_launches );
       e != cudaSuccess )
    return cuda_fail( h, "attention_softmax launch", e );
  return ring_touch( h, entry, st );
}

int gh_op_attention_2_gemm( gh_attn_t h,
                            const void* att,
                            const void* const* layer_bases,
                            void* xb,
                            uint64_t batch,
                            const uint32_t* pos,
                            void* stream )
{
  if ( h == nullptr || att == nullptr || xb == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( const int rc = check_positions( h, batch, layer_bases, pos ); rc != GH_OK )
    return rc;
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  int entry;
  if ( const int rc = upload_ptrs( h, batch, layer_bases, pos, st, &entry ); rc != GH_OK )
    return rc;
  if ( const cudaError_t e = launch_values( score_args( h, entry, batch, nullptr, const_cast<void*>( att ), xb ), st,
                                            &h->stats.kernel_launches );
       e != cudaSuccess )
    return cuda_fail( h, "attention_2_gemm launch", e );
  return ring_touch( h, entry, st );
}

int gh_op_attention_fused( gh_attn_t h,
                           const void* query,
                           const void* const* layer_bases,
                           void* xb,
                           uint64_t batch,
                           const uint32_t* pos,
                           void* stream )
{
  if ( h == nullptr || query == nullptr || xb == nullptr )
    return fail( h, GH_ERR_INVALID, "null argument" );
  if ( const int rc = check_positions( h, batch, layer_bases, pos ); rc != GH_OK )
    return rc;
  if ( const int rc = check_device_ok( h ); rc != GH_OK )
    return rc;
  if ( !aligned16( query ) || !aligned16( xb ) || !rows_aligned16( const_cast<void* const*>( layer_bases ), batch ) )
    return misaligned( h );
  DeviceGuard guard( h->device );
  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  uint32_t own_layer;
  if ( resolve_own_rows( h, batch, layer_bases, pos, false, &own_layer ) ) {
    // every layer of a step names the same slots and positions: one plan and one upload serve them all
    if ( const int rc = op_batch_entry( h, batch, st ); rc != GH_OK )
      return rc;
    DecodeArgs a = decode_args( h, h->op_entry, h->op_items, h->op_split, h->pool.layer_offset( own_layer ), query, xb );
    a.stream_old_rows_early = 1; // (the shared description is only reused while the operations name the same rows)
    if ( const int rc = run_decode( h, a, true, st ); rc != GH_OK )
      return rc;
    return ring_touch( h, h->op_entry, st );
  }
  const char* arena = h->pool.arena();
  const size_t row_bytes = h->pool.geometry().row_bytes;
  bool in_arena = true;
  std::vector<CtxMeta> ctx( batch );
  for ( uint64_t i = 0; i < batch; i++ ) {
    CtxMeta& c = ctx[i];
    c = CtxMeta {};
    c.pos = pos[i];
    if ( layer_bases[i] == nullptr ) {
      c.kv_off = kInactive;
      continue;
    }
    const char* p = static_cast<const char*>( layer_bases[i] );
    c.kv_off = p - arena;
    if ( p < arena || p >= arena + h->pool.arena_bytes() || ( c.kv_off % static_cast<long long>( row_bytes ) ) != 0 )
      in_arena = false; // foreign memory: the TMA descriptor does not cover it, use plain loads
  }
  int entry;
  uint32_t n_items, n_split;
  if ( const int rc = plan_and_upload( h, ctx, st, &entry, &n_items, &n_split ); rc != GH_OK )
    return rc;
  const DecodeArgs a = decode_args( h, entry, n_items, n_split, 0, query, xb );
  if ( const int rc = run_decode( h, a, in_arena, st ); rc != GH_OK )
    return rc;
  return ring_touch( h, entry, st );
}

int gh_op_convert_and_copy( gh_attn_t h,
                            void* dst,
                            uint32_t dst_dtype,
                            const void* src,
                            uint32_t src_dtype,
                            uint64_t n,
                            uint32_t copy_type )
{
  if ( h == nullptr || dst == nullptr || src == nullptr || !dtype_ok( dst_dtype ) || !dtype_ok( src_dtype ) )
    return fail( h, GH_ERR_INVALID, "bad argument" );
  if ( n == 0 )
    return GH_OK;
  DeviceGuard guard( h->device );
  const size_t db = dtype_size( dst_dtype ), sb = dtype_size( src_dtype );
  if ( copy_type == GH_COPY_DEVICE_TO_DEVICE ) {
    if ( dst_dtype == src_dtype )
      GH_CUDA( h, cudaMemcpy( dst, src, n * db, cudaMemcpyDeviceToDevice ) );
    else
      GH_CUDA( h, launch_convert( dst, dst_dtype, src, src_dtype, n, nullptr, &h->stats.kernel_launches ) );
    GH_CUDA( h, cudaStreamSynchronize( nullptr ) );
    return GH_OK;
  }
  if ( copy_type != GH_COPY_HOST_TO_DEVICE && copy_type != GH_COPY_DEVICE_TO_HOST )
    return fail( h, GH_ERR_INVALID, "invalid copy type" );
  const bool h2d = copy_type == GH_COPY_HOST_TO_DEVICE;
  if ( dst_dtype == src_dtype ) {
    GH_CUDA( h, cudaMemcpy( dst, src, n * db, h2d ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost ) );
    return GH_OK;
  }
  // The element conversion runs on the device (the reference converts on the host through a temporary array,
  // src/arch/cuda/llama2/ops.cuh:463-486); the result is the same static_cast per element.
  void* tmp = nullptr;
  GH_CUDA( h, cudaMalloc( &tmp, n * ( h2d ? sb : db ) ) );
  cudaError_t e;
  if ( h2d ) {
    e = cudaMemcpy( tmp, src, n * sb, cudaMemcpyHostToDevice );
    if ( e == cudaSuccess )
      e = launch_convert( dst, dst_dtype, tmp, src_dtype, n, nullptr, &h->stats.kernel_launches );
    if ( e == cudaSuccess )
      e = cudaStreamSynchronize( nullptr );
  } else {
    e = launch_convert( tmp, dst_dtype, src, src_dtype, n, nullptr, &h->stats.kernel_launches );
    if ( e == cudaSuccess )
      e = cudaMemcpy( dst, tmp, n * db, cudaMemcpyDeviceToHost );
  }
  cudaFree( tmp );
  if ( e != cudaSuccess )
    return cuda_fail( h, "convert_and_copy", e );
  return GH_OK;
}

int gh_plan_batch( uint32_t blocks_per_item,
                   uint32_t sm_count,
                   uint32_t tile,
                   uint32_t fixed_chunk,
                   uint32_t max_items,
                   uint64_t batch,
                   const uint32_t* pos,
                   int32_t* items_out,
                   uint32_t* n_items,
                   uint32_t* chunk )
{
  if ( pos == nullptr || items_out == nullptr || n_items == nullptr || chunk == nullptr || blocks_per_item == 0
       || sm_count == 0 || tile == 0 || max_items == 0 )
    return GH_ERR_INVALID;
  std::vector<CtxMeta> ctx( batch );
  for ( uint64_t i = 0; i < batch; i++ ) {
    ctx[i] = CtxMeta {};
    ctx[i].pos = pos[i];
    ctx[i].kv_off = pos[i] == 0xffffffffu ? kInactive : 0;
  }
  PlanParams pp;
  pp.n_kv_heads = blocks_per_item;
  pp.sm_count = sm_count;
  pp.tile = tile;
  pp.fixed_chunk = fixed_chunk;
  pp.max_items = max_items;
  pp.blocks_per_sm = 4; // what the tensor-core decode kernel keeps resident
  Plan plan;
  if ( !plan_batch( pp, ctx, plan ) )
    return GH_ERR_INVALID;
  std::memcpy( items_out, plan.items.data(), plan.items.size() * sizeof( WorkItem ) );
  *n_items = static_cast<uint32_t>( plan.items.size() );
  *chunk = plan.chunk;
  return GH_OK;
}

int gh_plan_projection( uint32_t n_heads,
                        uint32_t head_size,
                        uint32_t kv_dim,
                        uint32_t sm_count,
                        uint32_t* plan_out,
                        int32_t* pieces_out,
                        uint32_t max_pieces,
                        uint32_t* n_pieces )
{
  if ( plan_out == nullptr || pieces_out == nullptr || n_pieces == nullptr || n_heads == 0 || head_size == 0 || sm_count == 0 )
    return GH_ERR_INVALID;
  Shape sh {};
  sh.n_heads = n_heads;
  sh.head_size = head_size;
  sh.kv_dim = kv_dim;
  if ( !project_supported( sh, DT_F16 ) )
    return GH_ERR_UNSUPPORTED;
  ProjectArgs a {};
  uint32_t grid = 0;
  project_plan( sh, sm_count, &a, &grid );
  plan_out[0] = grid, plan_out[1] = a.units_per_cta, plan_out[2] = a.max_segs, plan_out[3] = a.n_tiles, plan_out[4] = a.kblocks;
  uint32_t n = 0;
  std::vector<int32_t> tmp( 5 * ( a.n_tiles + 2 ) ); // a CTA touches every tile at most once
  for ( uint32_t c = 0; c < grid; c++ ) {
    const uint32_t k = project_pieces( a, c, tmp.data(), a.n_tiles + 2 );
    for ( uint32_t i = 0; i < k; i++, n++ )
      if ( n < max_pieces ) {
        pieces_out[6 * n] = static_cast<int32_t>( c );
        std::memcpy( pieces_out + 6 * n + 1, tmp.data() + 5 * i, 5 * sizeof( int32_t ) );
      }
  }
  *n_pieces = n;
  return n <= max_pieces ? GH_OK : GH_ERR_CAPACITY;
}

int gh_fill_normal( gh_attn_t h, void* dst, uint64_t n, uint32_t dtype, uint64_t seed, uint64_t offset, void* stream )
{
  if ( h == nullptr || dst == nullptr || !dtype_ok( dtype ) )
    return fail( h, GH_ERR_INVALID, "bad argument" );
  DeviceGuard guard( h->device );
  if ( const cudaError_t e = launch_fill_normal( dst, n, dtype, seed, offset, static_cast<cudaStream_t>( stream ),
                                                 &h->stats.kernel_launches );
       e != cudaSuccess )
    return cuda_fail( h, "fill kernel launch", e );
  return GH_OK;
}

} // extern "C"
