// Fused RoPE + K/V append for a whole batch in one launch.
//
// Replaces, per layer-step, the reference's B cudaMemcpyAsync calls (copy_kv_cache,
// src/arch/cuda/llama2/ops.cuh:435-453) and B do_rope launches (apply_rope, :413-433, kernel :190-220).
// Arithmetic follows the amd64 backend, which is the parity target (src/arch/amd64/llama2/ops.hh:150-162):
// table values and operands are loaded from the storage type into fp32, the rotation is computed in fp32 and
// rounded once.  V is never converted: it moves as 16-byte chunks, bit for bit.
//
// Tiny (a few MiB per launch) and therefore latency-bound: the grid is (context, slice) with one 16-byte chunk
// per thread, so every load of the launch is in flight at once.  The kernel lets the kernel behind it in the
// stream start its prologue early (programmatic dependent launch); that kernel must wait for this one before it
// touches q or the slot rows.
#include "gh_kernels.cuh"

namespace gh {

namespace {

template<typename T>
__device__ __forceinline__ Vec16<T> rotate_chunk( const Vec16<T>& x, const T* __restrict__ cs, const T* __restrict__ sn )
{
  Vec16<T> r;
#pragma unroll
  for ( int p = 0; p < Vec16<T>::N / 2; p++ ) {
    const float c = Conv<T>::to_f32( cs[p] );
    const float s = Conv<T>::to_f32( sn[p] );
    const float x0 = Conv<T>::to_f32( x.v[2 * p] );
    const float x1 = Conv<T>::to_f32( x.v[2 * p + 1] );
    // Products are rounded separately (no fused multiply-add), like `k0 * fcr - k1 * fci` evaluated by the
    // reference; the final rounding to the storage type is the only other one.
    r.v[2 * p] = Conv<T>::from_f32( __fsub_rn( __fmul_rn( x0, c ), __fmul_rn( x1, s ) ) );
    r.v[2 * p + 1] = Conv<T>::from_f32( __fadd_rn( __fmul_rn( x0, s ), __fmul_rn( x1, c ) ) );
  }
  return r;
}

template<typename T>
__global__ void __launch_bounds__( 256 ) append_kernel( const AppendArgs a )
{
  constexpr int N = Vec16<T>::N;
  const int i = blockIdx.x / a.tokens_per_ctx;   // context
  const int tk = blockIdx.x - i * a.tokens_per_ctx; // token of a prefill chunk (0 for a decode step)
  const int in_row = blockIdx.x;                  // row of q and kv_new: [context][token]
  const Shape& sh = a.sh;
  asm volatile( "griddepcontrol.launch_dependents;" ::: "memory" );

  T* row;
  uint32_t pos;
  if ( a.token_rows != nullptr ) {
    row = static_cast<T*>( a.token_rows[i] );
    pos = a.pos != nullptr ? a.pos[i] : 0u;
    if ( row == nullptr )
      return;
  } else {
    const CtxMeta c = a.ctx[i];
    if ( c.kv_off == kInactive )
      return;
    pos = c.pos + tk;
    row = reinterpret_cast<T*>( a.arena + c.kv_off + a.layer_off ) + (size_t)pos * sh.row_elems;
  }

  const T* src = a.kv_new != nullptr ? static_cast<const T*>( a.kv_new ) + (size_t)in_row * sh.row_elems : nullptr;
  T* q = a.q != nullptr ? static_cast<T*>( a.q ) + (size_t)in_row * sh.n_heads * sh.head_size : nullptr;
  const bool rotate = a.rope_cos != nullptr;
  const T* cs_row = rotate ? static_cast<const T*>( a.rope_cos ) + (size_t)pos * ( sh.head_size / 2 ) : nullptr;
  const T* sn_row = rotate ? static_cast<const T*>( a.rope_sin ) + (size_t)pos * ( sh.head_size / 2 ) : nullptr;

  const int k_chunks = sh.kv_dim / N;
  const int per_chunk = 1 + ( ( rotate && q != nullptr ) ? (int)sh.group : 0 );
  const int k_units = k_chunks * per_chunk;
  const int v_units = src != nullptr ? k_chunks : 0;

  for ( int u = blockIdx.y * blockDim.x + threadIdx.x; u < k_units + v_units; u += gridDim.y * blockDim.x ) {
    if ( u >= k_units ) { // V: plain copy
      const int e = ( u - k_units ) * N;
      st16( row + sh.kv_dim + e, ld16( src + sh.kv_dim + e ) );
      continue;
    }
    const int chunk = u / per_chunk;
    const int which = u - chunk * per_chunk; // 0 = the K chunk, 1.. = the query heads sharing this kv head
    const int e = chunk * N;                 // element offset inside the K half of the row
    const int kvh = e / sh.head_size;
    const int d = e - kvh * sh.head_size;    // first dimension of the chunk, even
    if ( which == 0 ) {
      if ( src == nullptr && !rotate )
        continue;
      Vec16<T> x = ld16( src != nullptr ? src + e : row + e );
      if ( rotate )
        x = rotate_chunk( x, cs_row + d / 2, sn_row + d / 2 );
      st16( row + e, x );
    } else {
      T* qp = q + (size_t)( kvh * sh.group + ( which - 1 ) ) * sh.head_size + d;
      st16( qp, rotate_chunk( ld16( qp ), cs_row + d / 2, sn_row + d / 2 ) );
    }
  }
}

// The same arithmetic with the units of a token taken in address order (a warp reads and writes 512 consecutive
// bytes); one thread carries its unit through TB consecutive tokens of a context with their loads in flight together.
// Used for decode steps (TB = 1) and prompt chunks (TB = 2: hundreds of MB, bandwidth-bound) whenever the rows go to
// the arena's own slots; append_kernel above stays for the reference's pointer-array operations.
template<typename T, int TB>
__global__ void __launch_bounds__( 256, 6 ) append_ordered_kernel( const AppendArgs a )
{
  constexpr int N = Vec16<T>::N;
  const Shape& sh = a.sh;
  const int blocks_per_ctx = ( a.tokens_per_ctx + TB - 1 ) / TB;
  const int i = blockIdx.x / blocks_per_ctx;                 // context
  const int tk0 = ( blockIdx.x - i * blocks_per_ctx ) * TB;  // first token of the chunk this block handles
  asm volatile( "griddepcontrol.launch_dependents;" ::: "memory" );
  // Launched as a programmatic dependent of the kernel before it in the stream (normally the previous layer-step's
  // decode kernel), so that this kernel's launch latency hides behind that kernel's tail.  Unless the caller declared
  // consecutive calls independent, q and the new rows are not read, and nothing is written, before that kernel has
  // completed (the waits below); the batch description and the rotation tables, which no kernel writes, are
  // fetched ahead of the wait.
  const bool wait_first = a.dependent_launch == 1;
  const CtxMeta c = a.ctx[i];
  if ( c.kv_off == kInactive )
    return;
  const int n_tok = min( TB, (int)a.tokens_per_ctx - tk0 );

  // units of a token, each a 16-byte chunk, in address order so that a warp touches consecutive bytes:
  // K chunks | q chunks (every head) | V chunks
  const int k_chunks = sh.kv_dim / N;
  const int q_chunks = a.q != nullptr ? (int)( sh.n_heads * sh.head_size ) / N : 0;
  const int u = blockIdx.y * blockDim.x + threadIdx.x;
  if ( u >= 2 * k_chunks + q_chunks )
    return;

  const size_t in_row0 = (size_t)i * a.tokens_per_ctx + tk0; // row of q and kv_new: [context][token]
  const uint32_t pos0 = c.pos + tk0;
  T* row0 = reinterpret_cast<T*>( a.arena + c.kv_off + a.layer_off ) + (size_t)pos0 * sh.row_elems;
  const T* src0 = static_cast<const T*>( a.kv_new ) + in_row0 * sh.row_elems;

  if ( u >= k_chunks + q_chunks ) { // V: plain copy
    const int e = sh.kv_dim + ( u - k_chunks - q_chunks ) * N;
    if ( wait_first )
      asm volatile( "griddepcontrol.wait;" ::: "memory" );
    Vec16<T> x[TB];
#pragma unroll
    for ( int t = 0; t < TB; t++ )
      if ( t < n_tok )
        x[t] = ld16( src0 + (size_t)t * sh.row_elems + e );
#pragma unroll
    for ( int t = 0; t < TB; t++ )
      if ( t < n_tok )
        st16( row0 + (size_t)t * sh.row_elems + e, x[t] );
    return;
  }
  const size_t q_row = (size_t)sh.n_heads * sh.head_size;
  const T* from;  // token t's chunk is at from + t * from_stride, and goes to to + t * to_stride
  T* to;
  size_t from_stride, to_stride;
  int e; // element offset inside the K half of the row, or inside the token's q
  if ( u < k_chunks ) {
    e = u * N;
    from = src0 + e, from_stride = sh.row_elems;
    to = row0 + e, to_stride = sh.row_elems;
  } else {
    e = ( u - k_chunks ) * N;
    to = static_cast<T*>( a.q ) + in_row0 * q_row + e;
    from = to, from_stride = to_stride = q_row;
  }
  const int d = e % (int)sh.head_size; // first dimension of the chunk within its head, even
  const T* cs0 = static_cast<const T*>( a.rope_cos ) + (size_t)pos0 * ( sh.head_size / 2 ) + d / 2;
  const T* sn0 = static_cast<const T*>( a.rope_sin ) + (size_t)pos0 * ( sh.head_size / 2 ) + d / 2;
  Vec16<T> x[TB];
  uint2 cs[TB], sn[TB]; // the chunk's N / 2 rotation pairs: 8 bytes of each table
#pragma unroll
  for ( int t = 0; t < TB; t++ )
    if ( t < n_tok ) {
      cs[t] = *reinterpret_cast<const uint2*>( cs0 + (size_t)t * ( sh.head_size / 2 ) );
      sn[t] = *reinterpret_cast<const uint2*>( sn0 + (size_t)t * ( sh.head_size / 2 ) );
    }
  if ( wait_first )
    asm volatile( "griddepcontrol.wait;" ::: "memory" );
#pragma unroll
  for ( int t = 0; t < TB; t++ )
    if ( t < n_tok )
      x[t] = ld16( from + (size_t)t * from_stride );
#pragma unroll
  for ( int t = 0; t < TB; t++ )
    if ( t < n_tok )
      st16( to + (size_t)t * to_stride,
            rotate_chunk( x[t], reinterpret_cast<const T*>( &cs[t] ), reinterpret_cast<const T*>( &sn[t] ) ) );
}

} // namespace

cudaError_t launch_append( const AppendArgs& args, cudaStream_t st, uint64_t* launches )
{
  if ( args.batch == 0 )
    return cudaSuccess;
  AppendArgs a = args;
  if ( a.tokens_per_ctx == 0 )
    a.tokens_per_ctx = 1;
  // chunk operations per context: K chunks (each with the group's q chunks) + V chunks
  const unsigned n16 = a.dtype == DT_F32 ? 4 : 8;
  const unsigned units = ( a.sh.kv_dim / n16 ) * ( 2 + a.sh.group );
  const unsigned tokens = a.tokens_per_ctx > 0 ? a.tokens_per_ctx : 1;
  // Rotation + new rows + the arena's own slots (what gh_attn_append and the chunk entry point pass): the kernel
  // that walks a token's units in address order.  Two tokens per thread measured best for prompt chunks on B200
  // (1, 2, 3, 4, 8, 16 tried: more tokens per thread cost more in occupancy than they gain in loads in flight); a
  // decode step has one token per context, and the address order alone shortens its launch by about a fifth.
  if ( a.token_rows == nullptr && a.kv_new != nullptr && a.rope_cos != nullptr ) {
    const unsigned cunits = 2 * ( a.sh.kv_dim / n16 ) + ( a.q != nullptr ? a.sh.n_heads * a.sh.head_size / n16 : 0 );
    const unsigned tb = tokens >= 2 ? 2 : 1;
    const dim3 cgrid( a.batch * ( ( tokens + tb - 1 ) / tb ), ( cunits + 255 ) / 256 );
    if ( a.dependent_launch != 0 && tb == 1 ) {
      // A programmatic dependent of the kernel before it in the stream: its blocks are placed while that kernel's
      // last blocks still run (the decode kernel releases its dependents as soon as its last block has started).
      // dependent_launch == 1: the kernel then waits for that kernel to complete; == 2: it goes ahead.
      cudaLaunchConfig_t cfg {};
      cfg.gridDim = cgrid;
      cfg.blockDim = dim3( 256 );
      cfg.stream = st;
      cudaLaunchAttribute attr {};
      attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr.val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      cudaError_t e;
      switch ( a.dtype ) {
        case DT_F32: e = cudaLaunchKernelEx( &cfg, append_ordered_kernel<float, 1>, a ); break;
        case DT_F16: e = cudaLaunchKernelEx( &cfg, append_ordered_kernel<__half, 1>, a ); break;
        case DT_BF16: e = cudaLaunchKernelEx( &cfg, append_ordered_kernel<__nv_bfloat16, 1>, a ); break;
        default: return cudaErrorInvalidValue;
      }
      ( *launches )++;
      return e;
    }
    if ( tb == 2 ) {
      switch ( a.dtype ) {
        case DT_F32: append_ordered_kernel<float, 2><<<cgrid, 256, 0, st>>>( a ); break;
        case DT_F16: append_ordered_kernel<__half, 2><<<cgrid, 256, 0, st>>>( a ); break;
        case DT_BF16: append_ordered_kernel<__nv_bfloat16, 2><<<cgrid, 256, 0, st>>>( a ); break;
        default: return cudaErrorInvalidValue;
      }
    } else {
      switch ( a.dtype ) {
        case DT_F32: append_ordered_kernel<float, 1><<<cgrid, 256, 0, st>>>( a ); break;
        case DT_F16: append_ordered_kernel<__half, 1><<<cgrid, 256, 0, st>>>( a ); break;
        case DT_BF16: append_ordered_kernel<__nv_bfloat16, 1><<<cgrid, 256, 0, st>>>( a ); break;
        default: return cudaErrorInvalidValue;
      }
    }
    ( *launches )++;
    return cudaGetLastError();
  }
  const dim3 grid( a.batch * tokens, ( units + 255 ) / 256 );
  switch ( a.dtype ) {
    case DT_F32: append_kernel<float><<<grid, 256, 0, st>>>( a ); break;
    case DT_F16: append_kernel<__half><<<grid, 256, 0, st>>>( a ); break;
    case DT_BF16: append_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>( a ); break;
    default: return cudaErrorInvalidValue;
  }
  ( *launches )++;
  return cudaGetLastError();
}

} // namespace gh
