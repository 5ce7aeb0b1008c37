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
