// gh_decode_noalloc: fused decode attention for callers that must not allocate device memory.
//
// Who needs this.  A Glinthawk worker hands out its GPU memory once, at start-up: weights, the activation
// scratchpad and every context slot are allocated before the first prompt arrives, and from then on the process
// treats a failed device allocation as fatal.  Code that runs inside such a process after start-up — or inside a
// serving loop that cannot afford the device-wide synchronisation cudaMalloc and cudaFree imply — has no safe way to
// obtain the scratch memory that split-K decode attention needs (partial results of contexts cut into several
// work items and the batch description).  This entry point needs no handle and never calls
// cudaMalloc, cudaFree or any allocating library routine: its scratch is a fixed array that is part of the library
// image, so every GPU that loads the library holds GH_NOALLOC_SCRATCH_BYTES of it until the process exits.
//
// The kernel is the CUDA-core decode kernel (one query head per thread block, plain loads, any fp32/fp16/bf16
// layout the reference uses) with its scratch pointed at that array.
//
// Rules for callers:
//   * Sizes are bounded (see the GH_NOALLOC_MAX_* constants); larger requests are refused with GH_ERR_INVALID and a
//     message from gh_decode_noalloc_error().
//   * The first call on each device looks up the device address of the array.  Make that first call during
//     set-up, before any stream capture begins on that device.
//   * Do not call it while `stream` is being captured: the batch description is uploaded from arrays on the
//     caller's stack, which are gone when the call returns.  Such a call is refused with GH_ERR_STATE.
//   * All calls on a device share the one array, which still holds whatever the previous call left there.
//     Nothing in it has to start at zero: the batch description is uploaded on `stream` before the launch, and
//     every partial record that is read was written earlier in the same call.  Two calls whose kernels could
//     overlap on the GPU (different streams, no dependency between them) race on the array: serialise them.
#include "../../include/glinthawk_attn.h"

#include <cstdio>
#include <mutex>

#include "gh_kernels.cuh"
#include "gh_merge.cuh"

using namespace gh;

namespace {

constexpr uint32_t kNaMaxBatch = GH_NOALLOC_MAX_BATCH;
constexpr uint32_t kNaMaxItems = GH_NOALLOC_MAX_ITEMS;
constexpr uint32_t kNaMaxHeads = GH_NOALLOC_MAX_HEADS;
constexpr uint32_t kNaMaxQElems = GH_NOALLOC_MAX_Q_ELEMS;

// Layout of the scratch array (byte offsets).
constexpr size_t kOffCtx = 0;                                                     // CtxMeta[kNaMaxBatch]
constexpr size_t kOffItems = kOffCtx + sizeof( CtxMeta ) * kNaMaxBatch;             // WorkItem[kNaMaxItems]
constexpr size_t kOffSplit = kOffItems + sizeof( WorkItem ) * kNaMaxItems;          // int32[kNaMaxBatch] cut contexts
constexpr size_t kOffPartMl = kOffSplit + sizeof( int32_t ) * kNaMaxBatch;          // float[kNaMaxItems*kNaMaxHeads*2]
constexpr size_t kOffPartO = 256 * 1024;                                          // float[kNaMaxItems * kNaMaxQElems]
constexpr size_t kScratchBytes = kOffPartO + sizeof( float ) * kNaMaxItems * kNaMaxQElems;
static_assert( kOffPartMl + sizeof( float ) * kNaMaxItems * kNaMaxHeads * 2 <= kOffPartO, "scratch layout overlaps" );
static_assert( kScratchBytes == GH_NOALLOC_SCRATCH_BYTES, "header and implementation disagree on the scratch size" );

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__( 256 ) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int refuse( const char* fmt, unsigned long long a = 0, unsigned long long b = 0 )
{
  std::snprintf( g_error, sizeof( g_error ), fmt, a, b );
  return GH_ERR_INVALID;
}

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

// Same algorithm as the CUDA-core decode kernel: 4 warps share one (work item, query head); warp w takes every 4th
// token, lanes split the head dimension, online softmax in fp32 (log2 domain), states combined through shared
// memory, then the result is written or a partial record is left for the merge kernel that follows.
template<typename T, int DPL>
__global__ void __launch_bounds__( kThreads ) decode_noalloc_kernel( const DecodeArgs a )
{
  __shared__ float sm_o[kWarps][DPL * 32];
  __shared__ float sm_m[kWarps];
  __shared__ float sm_l[kWarps];
  __shared__ float sm_fo[DPL * 32];
  __shared__ float sm_fm[1];
  __shared__ float sm_fl[1];

  const Shape& sh = a.sh;
  const WorkItem it = a.items[blockIdx.x];
  const CtxMeta c = a.ctx[it.ctx];
  const int head = blockIdx.y;
  const int kvh = head / sh.group;
  const int hs = sh.head_size;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const float scale_log2 = ( 1.0f / sqrtf( (float)hs ) ) * 1.4426950408889634f;

  const T* base = reinterpret_cast<const T*>( a.arena + c.kv_off + a.layer_off );
  const T* qh = static_cast<const T*>( a.q ) + (size_t)it.ctx * sh.n_heads * hs + (size_t)head * hs;

  float qr[DPL], acc[DPL];
#pragma unroll
  for ( int k = 0; k < DPL; k++ ) {
    const int d = lane + 32 * k;
    qr[k] = d < hs ? Conv<T>::to_f32( qh[d] ) : 0.f;
    acc[k] = 0.f;
  }
  float m = -INFINITY, l = 0.f;

  for ( int t = it.t_begin + warp; t < it.t_end; t += kWarps ) {
    const T* krow = base + (size_t)t * sh.row_elems + kvh * hs;
    const T* vrow = krow + sh.kv_dim;
    float part = 0.f;
    float v[DPL];
#pragma unroll
    for ( int k = 0; k < DPL; k++ ) {
      const int d = lane + 32 * k;
      const bool in = d < hs;
      part += in ? Conv<T>::to_f32( krow[d] ) * qr[k] : 0.f;
      v[k] = in ? Conv<T>::to_f32( vrow[d] ) : 0.f;
    }
    const float s = warp_sum( part ) * scale_log2;
    const float mn = fmaxf( m, s );
    const float corr = exp2f( m - mn );
    const float p = exp2f( s - mn );
    l = l * corr + p;
#pragma unroll
    for ( int k = 0; k < DPL; k++ )
      acc[k] = acc[k] * corr + p * v[k];
    m = mn;
  }

#pragma unroll
  for ( int k = 0; k < DPL; k++ )
    sm_o[warp][lane + 32 * k] = acc[k];
  if ( lane == 0 ) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
  __syncthreads();

  float M = -INFINITY;
#pragma unroll
  for ( int w = 0; w < kWarps; w++ )
    M = fmaxf( M, sm_m[w] );
  float wgt[kWarps], L = 0.f;
#pragma unroll
  for ( int w = 0; w < kWarps; w++ ) {
    wgt[w] = sm_m[w] == -INFINITY ? 0.f : exp2f( sm_m[w] - M );
    L += wgt[w] * sm_l[w];
  }
  for ( int d = threadIdx.x; d < hs; d += kThreads ) {
    float o = 0.f;
#pragma unroll
    for ( int w = 0; w < kWarps; w++ )
      o += wgt[w] * sm_o[w][d];
    sm_fo[d] = o;
  }
  if ( threadIdx.x == 0 ) {
    sm_fm[0] = M;
    sm_fl[0] = L;
  }
  __syncthreads();

  store_item<T>( sh, c, it, head, 1, sm_fo, sm_fm, sm_fl, static_cast<T*>( a.xb ), a.part_o, a.part_ml, threadIdx.x,
                 kThreads );
}

template<typename T>
cudaError_t launch_t( const DecodeArgs& a, cudaStream_t st )
{
  const dim3 grid( a.n_items, a.sh.n_heads );
  if ( a.sh.head_size <= 64 )
    decode_noalloc_kernel<T, 2><<<grid, kThreads, 0, st>>>( a );
  else if ( a.sh.head_size <= 128 )
    decode_noalloc_kernel<T, 4><<<grid, kThreads, 0, st>>>( a );
  else
    decode_noalloc_kernel<T, 8><<<grid, kThreads, 0, st>>>( a );
  cudaError_t e = cudaGetLastError();
  if ( e == cudaSuccess && a.n_split_ctx > 0 ) // combine the records of the contexts that were cut
    e = launch_merge_partials<T>( a.sh, a.ctx, a.split_ctx, a.n_split_ctx, a.part_o, a.part_ml, static_cast<T*>( a.xb ), st );
  return e;
}

// Device address of the scratch array on the current device, looked up once per device with that device current.
int scratch_address( unsigned char** out )
{
  int dev = -1;
  cudaError_t e = cudaGetDevice( &dev );
  if ( e != cudaSuccess || dev < 0 || dev >= kMaxDevices ) {
    (void)cudaGetLastError();
    std::snprintf( g_error, sizeof( g_error ), "no usable current CUDA device (%s)", cudaGetErrorString( e ) );
    return GH_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock( g_setup_mutex );
  if ( g_scratch_addr[dev] == nullptr ) {
    unsigned char* ptr = nullptr;
    e = cudaGetSymbolAddress( reinterpret_cast<void**>( &ptr ), g_noalloc_scratch );
    if ( e != cudaSuccess || ptr == nullptr ) {
      (void)cudaGetLastError();
      std::snprintf( g_error, sizeof( g_error ), "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev,
                     cudaGetErrorString( e ) );
      return GH_ERR_CUDA;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return GH_OK;
}

} // namespace

extern "C" {

const char* gh_decode_noalloc_error( void )
{
  return g_error;
}

int gh_decode_noalloc( const gh_noalloc_shape* shape,
                       uint64_t batch,
                       const void* const* layer_bases,
                       const uint32_t* pos,
                       const void* q,
                       void* xb,
                       void* stream )
{
  g_error[0] = '\0';
  if ( shape == nullptr || shape->struct_size != sizeof( gh_noalloc_shape ) || layer_bases == nullptr
       || pos == nullptr || q == nullptr || xb == nullptr )
    return refuse( "null argument or gh_noalloc_shape of the wrong size" );
  if ( shape->n_heads == 0 || shape->n_kv_heads == 0 || shape->n_heads % shape->n_kv_heads != 0
       || shape->head_size == 0 || shape->head_size % 8 != 0 || shape->head_size > (uint32_t)kMaxHeadSize
       || shape->dtype > GH_BF16 )
    return refuse( "unsupported shape or dtype" );
  if ( batch == 0 || batch > kNaMaxBatch )
    return refuse( "batch of %llu contexts is outside 1..%llu (GH_NOALLOC_MAX_BATCH)", batch, kNaMaxBatch );
  if ( shape->n_heads > kNaMaxHeads )
    return refuse( "%llu query heads exceed GH_NOALLOC_MAX_HEADS = %llu", shape->n_heads, kNaMaxHeads );
  if ( (uint64_t)shape->n_heads * shape->head_size > kNaMaxQElems )
    return refuse( "n_heads * head_size = %llu exceeds GH_NOALLOC_MAX_Q_ELEMS = %llu",
                   (uint64_t)shape->n_heads * shape->head_size, kNaMaxQElems );

  // ---- plan on the stack: cut long contexts so that about 16 blocks per SM exist, within kNaMaxItems items ----
  CtxMeta ctx[kNaMaxBatch];
  WorkItem items[kNaMaxItems];
  uint64_t total = 0;
  uint32_t active = 0;
  for ( uint64_t i = 0; i < batch; i++ ) {
    ctx[i] = CtxMeta {};
    ctx[i].pos = pos[i];
    if ( layer_bases[i] == nullptr ) {
      ctx[i].kv_off = kInactive;
      continue;
    }
    if ( pos[i] >= ( 1u << 24 ) )
      return refuse( "token position %llu at batch index %llu is not plausible", pos[i], i );
    ctx[i].kv_off = static_cast<long long>( reinterpret_cast<uintptr_t>( layer_bases[i] ) ); // arena base is null
    total += (uint64_t)pos[i] + 1;
    active++;
  }
  if ( active == 0 )
    return GH_OK;
  uint64_t chunk = ( total * shape->n_heads + 148 * 16 - 1 ) / ( 148 * 16 );
  chunk = ( ( chunk < 256 ? 256 : chunk ) + 63 ) / 64 * 64;
  for ( ;; ) {
    uint64_t n = 0, most = 0;
    for ( uint64_t i = 0; i < batch; i++ )
      if ( ctx[i].kv_off != kInactive ) {
        const uint64_t k = ( (uint64_t)ctx[i].pos + chunk ) / chunk;
        n += k;
        most = k > most ? k : most;
      }
    if ( n <= kNaMaxItems && most <= (uint64_t)kMaxSplits )
      break;
    chunk *= 2;
  }
  int32_t split_ctx[kNaMaxBatch];
  uint32_t n_items = 0, records = 0, n_split = 0;
  for ( uint64_t i = 0; i < batch; i++ ) {
    if ( ctx[i].kv_off == kInactive )
      continue;
    const uint64_t len = (uint64_t)ctx[i].pos + 1;
    const uint64_t nsplits = ( len + chunk - 1 ) / chunk;
    const uint64_t step = ( ( len + nsplits - 1 ) / nsplits + 63 ) / 64 * 64;
    int32_t made = 0;
    for ( uint64_t b = 0; b < len; b += step ) {
      WorkItem& w = items[n_items++];
      w.ctx = static_cast<int32_t>( i );
      w.t_begin = static_cast<int32_t>( b );
      w.t_end = static_cast<int32_t>( b + step < len ? b + step : len );
      w.split = made++;
    }
    ctx[i].nsplits = made;
    ctx[i].partial_base = static_cast<int32_t>( records );
    if ( made > 1 ) {
      records += made;
      split_ctx[n_split++] = static_cast<int32_t>( i );
    }
  }

  unsigned char* scratch = nullptr;
  if ( const int rc = scratch_address( &scratch ); rc != GH_OK )
    return rc;

  const cudaStream_t st = static_cast<cudaStream_t>( stream );
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if ( cudaStreamIsCapturing( st, &capturing ) != cudaSuccess )
    (void)cudaGetLastError();
  else if ( capturing != cudaStreamCaptureStatusNone ) {
    std::snprintf( g_error, sizeof( g_error ), "called during stream capture: the batch description is uploaded from the stack" );
    return GH_ERR_STATE;
  }
  cudaError_t e = cudaMemcpyAsync( scratch + kOffCtx, ctx, sizeof( CtxMeta ) * batch, cudaMemcpyHostToDevice, st );
  if ( e == cudaSuccess )
    e = cudaMemcpyAsync( scratch + kOffItems, items, sizeof( WorkItem ) * n_items, cudaMemcpyHostToDevice, st );
  if ( e == cudaSuccess && n_split > 0 )
    e = cudaMemcpyAsync( scratch + kOffSplit, split_ctx, sizeof( int32_t ) * n_split, cudaMemcpyHostToDevice, st );
  if ( e != cudaSuccess ) {
    (void)cudaGetLastError();
    std::snprintf( g_error, sizeof( g_error ), "uploading the batch description failed: %s", cudaGetErrorString( e ) );
    return GH_ERR_CUDA;
  }

  DecodeArgs a {};
  a.sh.n_heads = shape->n_heads;
  a.sh.n_kv_heads = shape->n_kv_heads;
  a.sh.group = shape->n_heads / shape->n_kv_heads;
  a.sh.head_size = shape->head_size;
  a.sh.kv_dim = shape->n_kv_heads * shape->head_size;
  a.sh.row_elems = 2 * a.sh.kv_dim;
  a.dtype = shape->dtype;
  a.ctx = reinterpret_cast<const CtxMeta*>( scratch + kOffCtx );
  a.items = reinterpret_cast<const WorkItem*>( scratch + kOffItems );
  a.n_items = n_items;
  a.arena = nullptr;
  a.layer_off = 0;
  a.q = q;
  a.xb = xb;
  a.part_o = reinterpret_cast<float*>( scratch + kOffPartO );
  a.part_ml = reinterpret_cast<float*>( scratch + kOffPartMl );
  a.split_ctx = reinterpret_cast<const int32_t*>( scratch + kOffSplit );
  a.n_split_ctx = n_split;

  switch ( shape->dtype ) {
    case GH_F32: e = launch_t<float>( a, st ); break;
    case GH_F16: e = launch_t<__half>( a, st ); break;
    default: e = launch_t<__nv_bfloat16>( a, st ); break;
  }
  if ( e != cudaSuccess ) {
    (void)cudaGetLastError();
    std::snprintf( g_error, sizeof( g_error ), "kernel launch failed: %s", cudaGetErrorString( e ) );
    return GH_ERR_CUDA;
  }
  return GH_OK;
}

} // extern "C"
