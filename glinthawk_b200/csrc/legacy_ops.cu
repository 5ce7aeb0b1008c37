// The reference's three attention operations as separate kernels that materialise the score matrix, plus the
// dtype-converting copy and a data generator.  These exist so that a caller holding the reference's argument
// lists gets the reference's observable behaviour op by op (including the contents of `att` and every
// intermediate rounding, src/arch/amd64/llama2/ops.hh:110-132,216,277); the fused kernels are the fast path.
#include "gh_kernels.cuh"

namespace gh {

namespace {

// attention_0_gemm (ops.hh:170-223): att[i][head][t] = RN( scale * <K[t][kvh], q[head]> ), fp32 accumulation.
template<typename T>
__global__ void __launch_bounds__( 128 ) scores_kernel( const ScoreArgs a )
{
  const Shape& sh = a.sh;
  const int i = blockIdx.z, head = blockIdx.y;
  const T* base = static_cast<const T*>( a.layer_bases[i] );
  if ( base == nullptr )
    return;
  const int n = (int)a.pos[i] + 1;
  const int t0 = blockIdx.x * 64;
  if ( t0 >= n )
    return;
  const int hs = sh.head_size, kvh = head / sh.group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = 1.0f / sqrtf( (float)hs );
  const T* qh = static_cast<const T*>( a.q ) + (size_t)i * sh.n_heads * hs + (size_t)head * hs;
  T* att = static_cast<T*>( a.att ) + ( (size_t)i * sh.n_heads + head ) * sh.seq_len;
  for ( int t = t0 + warp; t < min( t0 + 64, n ); t += 4 ) {
    const T* krow = base + (size_t)t * sh.row_elems + kvh * hs;
    float part = 0.f;
    for ( int d = lane; d < hs; d += 32 )
      part += Conv<T>::to_f32( krow[d] ) * Conv<T>::to_f32( qh[d] );
    const float sum = warp_sum( part );
    if ( lane == 0 )
      att[t] = Conv<T>::from_f32( scale * sum );
  }
}

__device__ __forceinline__ float block_reduce( float v, bool is_max, float* sm )
{
  v = is_max ? warp_max( v ) : warp_sum( v );
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if ( lane == 0 )
    sm[warp] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for ( int w = 0; w < nw; w++ )
    r = is_max ? fmaxf( r, sm[w] ) : r + sm[w];
  return r;
}

// attention_softmax (ops.hh:110-132, 283-298): max over storage values; x - max formed in the storage type;
// expf in fp32; each exponential rounded to the storage type before it enters the fp32 sum; one rounding after
// the division.  Like the reference, rows of inactive prompts are processed too (ops.hh:292-296).
template<typename T>
__global__ void __launch_bounds__( 256 ) softmax_kernel( const ScoreArgs a )
{
  __shared__ float sm[8];
  const Shape& sh = a.sh;
  const int i = blockIdx.y, head = blockIdx.x;
  const int n = (int)a.pos[i] + 1;
  T* x = static_cast<T*>( a.att ) + ( (size_t)i * sh.n_heads + head ) * sh.seq_len;
  float mx = -INFINITY;
  for ( int t = threadIdx.x; t < n; t += blockDim.x )
    mx = fmaxf( mx, Conv<T>::to_f32( x[t] ) );
  mx = block_reduce( mx, true, sm );
  float sum = 0.f;
  for ( int t = threadIdx.x; t < n; t += blockDim.x ) {
    const T d = Conv<T>::from_f32( Conv<T>::to_f32( x[t] ) - mx );
    const T e = Conv<T>::from_f32( expf( Conv<T>::to_f32( d ) ) );
    x[t] = e;
    sum += Conv<T>::to_f32( e );
  }
  sum = block_reduce( sum, false, sm );
  for ( int t = threadIdx.x; t < n; t += blockDim.x )
    x[t] = Conv<T>::from_f32( Conv<T>::to_f32( x[t] ) / sum );
}

// attention_2_gemm (ops.hh:225-281): xb[i][head][d] = RN( sum_t att[head][t] * V[t][kvh][d] ), fp32, t ascending.
template<typename T>
__global__ void __launch_bounds__( 128 ) values_kernel( const ScoreArgs a )
{
  const Shape& sh = a.sh;
  const int i = blockIdx.y, head = blockIdx.x;
  const T* base = static_cast<const T*>( a.layer_bases[i] );
  if ( base == nullptr )
    return;
  const int n = (int)a.pos[i] + 1;
  const int hs = sh.head_size, kvh = head / sh.group;
  const T* att = static_cast<const T*>( a.att ) + ( (size_t)i * sh.n_heads + head ) * sh.seq_len;
  T* out = static_cast<T*>( a.xb ) + (size_t)i * sh.n_heads * hs + (size_t)head * hs;
  for ( int d = threadIdx.x; d < hs; d += blockDim.x ) {
    const T* v = base + sh.kv_dim + kvh * hs + d;
    float acc = 0.f;
    for ( int t = 0; t < n; t++ )
      acc += Conv<T>::to_f32( v[(size_t)t * sh.row_elems] ) * Conv<T>::to_f32( att[t] );
    out[d] = Conv<T>::from_f32( acc );
  }
}

template<typename D, typename S>
__global__ void convert_kernel( D* dst, const S* src, uint64_t n )
{
  for ( uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x )
    dst[i] = Conv<D>::from_f32( Conv<S>::to_f32( src[i] ) );
}

__device__ __forceinline__ uint64_t mix64( uint64_t z )
{
  z = ( z ^ ( z >> 30 ) ) * 0xbf58476d1ce4e5b9ull;
  z = ( z ^ ( z >> 27 ) ) * 0x94d049bb133111ebull;
  return z ^ ( z >> 31 );
}

// Counter-based N(0,1): element pair k draws two 32-bit uniforms from a 64-bit hash of (seed, k) and applies
// the Box-Muller transform.  Independent of launch geometry.
template<typename T>
__global__ void fill_normal_kernel( T* dst, uint64_t n, uint64_t seed, uint64_t offset )
{
  const uint64_t pairs = ( n + 1 ) / 2;
  for ( uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; p < pairs; p += (uint64_t)gridDim.x * blockDim.x ) {
    const uint64_t hsh = mix64( seed * 0x9e3779b97f4a7c15ull + ( offset / 2 + p ) + 0x632be59bd9b4e019ull );
    const float u1 = ( (float)( (uint32_t)hsh >> 8 ) + 0.5f ) * ( 1.0f / 16777216.0f );
    const float u2 = ( (float)( (uint32_t)( hsh >> 32 ) >> 8 ) + 0.5f ) * ( 1.0f / 16777216.0f );
    const float r = sqrtf( -2.0f * __logf( u1 ) );
    float sn, cs;
    __sincosf( 6.283185307179586f * u2, &sn, &cs );
    dst[2 * p] = Conv<T>::from_f32( r * cs );
    if ( 2 * p + 1 < n )
      dst[2 * p + 1] = Conv<T>::from_f32( r * sn );
  }
}

template<typename D>
cudaError_t convert_from( D* dst, const void* src, uint32_t src_dtype, uint64_t n, cudaStream_t st )
{
  const int blocks = (int)( ( n + 255 ) / 256 < 1184 ? ( n + 255 ) / 256 : 1184 );
  switch ( src_dtype ) {
    case DT_F32: convert_kernel<<<blocks, 256, 0, st>>>( dst, static_cast<const float*>( src ), n ); break;
    case DT_F16: convert_kernel<<<blocks, 256, 0, st>>>( dst, static_cast<const __half*>( src ), n ); break;
    case DT_BF16: convert_kernel<<<blocks, 256, 0, st>>>( dst, static_cast<const __nv_bfloat16*>( src ), n ); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

#define GH_DISPATCH_T( dtype, EXPR )                                                                                   \
  switch ( dtype ) {                                                                                                   \
    case DT_F32: { using T = float; EXPR; } break;                                                                     \
    case DT_F16: { using T = __half; EXPR; } break;                                                                    \
    case DT_BF16: { using T = __nv_bfloat16; EXPR; } break;                                                            \
    default: return cudaErrorInvalidValue;                                                                             \
  }

} // namespace

cudaError_t launch_scores( const ScoreArgs& a, cudaStream_t st, uint64_t* launches )
{
  if ( a.batch == 0 )
    return cudaSuccess;
  const dim3 grid( ( a.sh.seq_len + 63 ) / 64, a.sh.n_heads, a.batch );
  GH_DISPATCH_T( a.dtype, ( scores_kernel<T><<<grid, 128, 0, st>>>( a ) ) );
  ( *launches )++;
  return cudaGetLastError();
}

cudaError_t launch_softmax( const ScoreArgs& a, cudaStream_t st, uint64_t* launches )
{
  if ( a.batch == 0 )
    return cudaSuccess;
  const dim3 grid( a.sh.n_heads, a.batch );
  GH_DISPATCH_T( a.dtype, ( softmax_kernel<T><<<grid, 256, 0, st>>>( a ) ) );
  ( *launches )++;
  return cudaGetLastError();
}

cudaError_t launch_values( const ScoreArgs& a, cudaStream_t st, uint64_t* launches )
{
  if ( a.batch == 0 )
    return cudaSuccess;
  const dim3 grid( a.sh.n_heads, a.batch );
  GH_DISPATCH_T( a.dtype, ( values_kernel<T><<<grid, 128, 0, st>>>( a ) ) );
  ( *launches )++;
  return cudaGetLastError();
}

cudaError_t launch_convert( void* dst, uint32_t dst_dtype, const void* src, uint32_t src_dtype, uint64_t n,
                            cudaStream_t st, uint64_t* launches )
{
  if ( n == 0 )
    return cudaSuccess;
  cudaError_t e;
  switch ( dst_dtype ) {
    case DT_F32: e = convert_from( static_cast<float*>( dst ), src, src_dtype, n, st ); break;
    case DT_F16: e = convert_from( static_cast<__half*>( dst ), src, src_dtype, n, st ); break;
    case DT_BF16: e = convert_from( static_cast<__nv_bfloat16*>( dst ), src, src_dtype, n, st ); break;
    default: return cudaErrorInvalidValue;
  }
  ( *launches )++;
  return e;
}

cudaError_t launch_fill_normal( void* dst, uint64_t n, uint32_t dtype, uint64_t seed, uint64_t offset,
                                cudaStream_t st, uint64_t* launches )
{
  if ( n == 0 )
    return cudaSuccess;
  const uint64_t pairs = ( n + 1 ) / 2;
  const int blocks = (int)( ( pairs + 255 ) / 256 < 2368 ? ( pairs + 255 ) / 256 : 2368 );
  GH_DISPATCH_T( dtype, ( fill_normal_kernel<T><<<blocks, 256, 0, st>>>( static_cast<T*>( dst ), n, seed, offset ) ) );
  ( *launches )++;
  return cudaGetLastError();
}

} // namespace gh
