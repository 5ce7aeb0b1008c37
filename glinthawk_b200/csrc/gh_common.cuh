// Shared device-side types and helpers of the attention-stage library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gh {

// Storage-type codes: the reference's DataType values (src/models/types.hh:20-25).
enum : uint32_t
{
  DT_F16 = 0,
  DT_F32 = 1,
  DT_BF16 = 2
};

constexpr int kMaxGroup = 16;     // query heads per kv head (Llama3-405B has 16, src/models/llama2/variants.hh:62)
constexpr int kMaxHeadSize = 256; // elements
constexpr int kMaxBatch = 1024;   // MAX_BATCH_SIZE, src/models/llama2/base.hh:26

// One prompt of the current batch, as the kernels see it.
struct CtxMeta
{
  long long kv_off;     // byte offset of the context's KV for layer 0 from the arena base; kInactive = skip
  uint32_t pos;         // position of the token being appended / attended from; attends over pos+1 tokens
  int32_t nsplits;      // work items this context was cut into
  int32_t partial_base; // first partial-result record of this context (meaningful when nsplits > 1)
  int32_t pad;
};
constexpr long long kInactive = -0x7fffffffffffffffLL - 1;

// One unit of decode work: tokens [t_begin, t_end) of one context, for every kv head.
struct WorkItem
{
  int32_t ctx;
  int32_t t_begin;
  int32_t t_end;
  int32_t split;
};

// Shape constants passed by value to every kernel.
struct Shape
{
  uint32_t n_heads, n_kv_heads, group, head_size, kv_dim, seq_len, n_layers;
  uint32_t row_elems; // 2 * kv_dim
};

template<typename T>
struct Conv;

template<>
struct Conv<float>
{
  static __device__ __forceinline__ float to_f32( float v ) { return v; }
  static __device__ __forceinline__ float from_f32( float v ) { return v; }
};
template<>
struct Conv<__half>
{
  static __device__ __forceinline__ float to_f32( __half v ) { return __half2float( v ); }
  static __device__ __forceinline__ __half from_f32( float v ) { return __float2half_rn( v ); }
};
template<>
struct Conv<__nv_bfloat16>
{
  static __device__ __forceinline__ float to_f32( __nv_bfloat16 v ) { return __bfloat162float( v ); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32( float v ) { return __float2bfloat16_rn( v ); }
};

// A 16-byte chunk of storage elements.
template<typename T>
struct alignas( 16 ) Vec16
{
  static constexpr int N = 16 / sizeof( T );
  T v[N];
};

template<typename T>
__device__ __forceinline__ Vec16<T> ld16( const T* p )
{
  Vec16<T> r;
  *reinterpret_cast<uint4*>( &r ) = *reinterpret_cast<const uint4*>( p );
  return r;
}

template<typename T>
__device__ __forceinline__ void st16( T* p, const Vec16<T>& r )
{
  *reinterpret_cast<uint4*>( p ) = *reinterpret_cast<const uint4*>( &r );
}

__device__ __forceinline__ float warp_sum( float v )
{
#pragma unroll
  for ( int o = 16; o > 0; o >>= 1 )
    v += __shfl_xor_sync( 0xffffffffu, v, o );
  return v;
}

__device__ __forceinline__ float warp_max( float v )
{
#pragma unroll
  for ( int o = 16; o > 0; o >>= 1 )
    v = fmaxf( v, __shfl_xor_sync( 0xffffffffu, v, o ) );
  return v;
}

} // namespace gh
