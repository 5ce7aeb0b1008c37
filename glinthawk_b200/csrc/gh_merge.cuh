// Epilogue shared by the decode kernels, and the two ways the pieces of contexts that were cut are combined.
//
// A context that fits one work item is finished by the block that processed it.  A context cut into several items
// leaves one partial record per (item, query head).  The CUDA-core kernels leave the records to a second, tiny,
// massively parallel kernel, launched only when the batch has cut contexts, as a programmatic dependent of the decode
// kernel.  The tensor-core kernel counts the arrivals of a context's blocks and lets the block that arrives last
// combine the records (combine_records below): with few contexts per GPU, where contexts are cut to fill the SMs,
// the extra launch cost a fifth of the layer-step.  Nothing waits on another block either way: no spinning.
#pragma once

#include "gh_common.cuh"

namespace gh {

constexpr int kMaxSplits = 64; // a context is never cut into more work items than this

// Partial record r = ( partial_base + split ) * n_heads + head:
//   part_o[r][head_size]  sum_t 2^(s_t - m) * V_t   (fp32, not normalised)
//   part_ml[r][2]         m (running maximum of the log2-scaled scores), l = sum_t 2^(s_t - m)
//
// `sm_o` [nrows][head_size], `sm_m` [nrows], `sm_l` [nrows] hold the calling block's result for query heads
// head0 .. head0+nrows-1 in shared memory; threads tid, tid + nthreads, ... of the calling group take part.
// HS: the head size when it is known at compile time (indices then need no division), 0 = take it from the shape.
template<typename T, int HS = 0>
__device__ __forceinline__ void store_item( const Shape& sh,
                                            const CtxMeta& c,
                                            const WorkItem& it,
                                            const int head0,
                                            const int nrows,
                                            const float* sm_o,
                                            const float* sm_m,
                                            const float* sm_l,
                                            T* __restrict__ xb,
                                            float* __restrict__ part_o,
                                            float* __restrict__ part_ml,
                                            const int tid,
                                            const int nthreads )
{
  const int hs = HS != 0 ? HS : (int)sh.head_size;
  if ( c.nsplits == 1 ) {
    T* out = xb + (size_t)it.ctx * sh.n_heads * hs + (size_t)head0 * hs;
    for ( int e = tid; e < nrows * hs; e += nthreads )
      out[e] = Conv<T>::from_f32( sm_o[e] / sm_l[e / hs] );
    return;
  }
  const size_t rec0 = ( (size_t)( c.partial_base + it.split ) * sh.n_heads + head0 );
  for ( int e = tid; e < nrows * hs; e += nthreads )
    part_o[rec0 * hs + e] = sm_o[e];
  for ( int r = tid; r < nrows; r += nthreads ) {
    part_ml[( rec0 + r ) * 2 + 0] = sm_m[r];
    part_ml[( rec0 + r ) * 2 + 1] = sm_l[r];
  }
}

// For the block of a cut context that arrived last (every record of the context is visible to it): combines the
// records of query heads head0 .. head0+nrows-1 and writes xb.  `scratch` is shared memory for
// nrows * (2 * nsplits + 1) floats; barrier `bar_id` is met by all `nthreads` calling threads.
template<typename T, int HS = 0>
__device__ __forceinline__ void combine_records( const Shape& sh,
                                                 const CtxMeta& c,
                                                 const int ctx_index,
                                                 const int head0,
                                                 const int nrows,
                                                 T* __restrict__ xb,
                                                 const float* part_o,
                                                 const float* part_ml,
                                                 float* scratch,
                                                 const int tid,
                                                 const int nthreads )
{
  const int hs = HS != 0 ? HS : (int)sh.head_size, ns = c.nsplits;
  float* sm_ml = scratch;                 // [nrows][ns][2], then the weights in place of m
  float* sm_L = scratch + nrows * ns * 2; // [nrows]
  const size_t rec0 = (size_t)c.partial_base * sh.n_heads + head0;
  // The combining block sits at the tail of the launch, and its latency is what the launch pays: a thread finishes
  // kU outputs at a time with the loads of kS records for all of them in flight together, and the first such round
  // of loads is issued before the records' (m, l) are fetched and turned into weights, so that those two round trips
  // to memory overlap.
  constexpr int kU = 8, kS = 4;
  T* out = xb + (size_t)ctx_index * sh.n_heads * hs + (size_t)head0 * hs;
  const int n_out = nrows * hs;
  const size_t rec_stride = (size_t)sh.n_heads * hs;
  auto load_round = [&]( float ( &v )[kS][kU], const int e0, const int s0 ) {
#pragma unroll
    for ( int ds = 0; ds < kS; ds++ )
#pragma unroll
      for ( int u = 0; u < kU; u++ ) {
        const int e = e0 + u * nthreads;
        v[ds][u] = ( s0 + ds < ns && e < n_out ) ? __ldcg( part_o + rec0 * hs + (size_t)( s0 + ds ) * rec_stride + e ) : 0.f;
      }
  };
  float v[kS][kU];
  load_round( v, tid, 0 );
  for ( int i = tid; i < nrows * ns; i += nthreads ) {
    const int r = i / ns, sp = i - r * ns;
    const float2 ml = __ldcg( reinterpret_cast<const float2*>( part_ml + ( rec0 + (size_t)sp * sh.n_heads + r ) * 2 ) );
    sm_ml[i * 2] = ml.x;
    sm_ml[i * 2 + 1] = ml.y;
  }
  asm volatile( "bar.sync 1, %0;" ::"r"( nthreads ) : "memory" );
  for ( int r = tid; r < nrows; r += nthreads ) {
    float M = -INFINITY;
    for ( int sp = 0; sp < ns; sp++ )
      M = fmaxf( M, sm_ml[( r * ns + sp ) * 2] );
    float L = 0.f;
    for ( int sp = 0; sp < ns; sp++ ) {
      const float w = exp2f( sm_ml[( r * ns + sp ) * 2] - M );
      L += w * sm_ml[( r * ns + sp ) * 2 + 1];
      sm_ml[( r * ns + sp ) * 2] = w;
    }
    sm_L[r] = L;
  }
  asm volatile( "bar.sync 1, %0;" ::"r"( nthreads ) : "memory" );
  for ( int e0 = tid; e0 < n_out; e0 += nthreads * kU ) {
    float O[kU];
    int row[kU];
#pragma unroll
    for ( int u = 0; u < kU; u++ ) {
      O[u] = 0.f;
      row[u] = min( e0 + u * nthreads, n_out - 1 ) / hs;
    }
    for ( int s0 = 0; s0 < ns; s0 += kS ) {
      if ( e0 != tid || s0 != 0 ) // (the first round is already here)
        load_round( v, e0, s0 );
#pragma unroll
      for ( int ds = 0; ds < kS; ds++ ) // records in their order: the same bits whichever block combines
        if ( s0 + ds < ns ) {
#pragma unroll
          for ( int u = 0; u < kU; u++ )
            O[u] += sm_ml[( row[u] * ns + s0 + ds ) * 2] * v[ds][u];
        }
    }
#pragma unroll
    for ( int u = 0; u < kU; u++ ) {
      const int e = e0 + u * nthreads;
      if ( e < n_out )
        out[e] = Conv<T>::from_f32( O[u] / sm_L[row[u]] );
    }
  }
}

// Combines the partial records of cut contexts: block (x, y) = (entry of split_ctx, query head), one thread per
// head dimension (looping when head_size > blockDim.x).  Every thread's loads are independent of each other.
template<typename T>
__global__ void __launch_bounds__( 128 ) merge_partials_kernel( const Shape sh,
                                                                const CtxMeta* __restrict__ ctx,
                                                                const int32_t* __restrict__ split_ctx,
                                                                const float* __restrict__ part_o,
                                                                const float* __restrict__ part_ml,
                                                                T* __restrict__ xb )
{
  __shared__ float sm_w[kMaxSplits];
  __shared__ float sm_L;
  asm volatile( "griddepcontrol.wait;" ::: "memory" ); // the records come from the kernel before this one
  const int ci = split_ctx[blockIdx.x];
  const CtxMeta c = ctx[ci];
  const int head = blockIdx.y;
  const int ns = c.nsplits;
  const int hs = sh.head_size;
  const size_t rec0 = (size_t)c.partial_base * sh.n_heads + head;
  const size_t rec_stride = sh.n_heads;

  if ( threadIdx.x < 32 ) { // one warp turns the records' (m, l) into weights and the total
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int s0 = threadIdx.x, s1 = threadIdx.x + 32;
    if ( s0 < ns ) {
      m0 = part_ml[( rec0 + s0 * rec_stride ) * 2];
      l0 = part_ml[( rec0 + s0 * rec_stride ) * 2 + 1];
    }
    if ( s1 < ns ) {
      m1 = part_ml[( rec0 + s1 * rec_stride ) * 2];
      l1 = part_ml[( rec0 + s1 * rec_stride ) * 2 + 1];
    }
    const float M = warp_max( fmaxf( m0, m1 ) );
    const float w0 = s0 < ns ? exp2f( m0 - M ) : 0.f;
    const float w1 = s1 < ns ? exp2f( m1 - M ) : 0.f;
    const float L = warp_sum( w0 * l0 + w1 * l1 );
    if ( s0 < ns )
      sm_w[s0] = w0;
    if ( s1 < ns )
      sm_w[s1] = w1;
    if ( threadIdx.x == 0 )
      sm_L = L;
  }
  __syncthreads();

  T* out = xb + (size_t)ci * sh.n_heads * hs + (size_t)head * hs;
  for ( int d = threadIdx.x; d < hs; d += blockDim.x ) {
    const float* src = part_o + rec0 * hs + d;
    float O = 0.f;
#pragma unroll 8
    for ( int sp = 0; sp < ns; sp++ )
      O += sm_w[sp] * src[(size_t)sp * rec_stride * hs];
    out[d] = Conv<T>::from_f32( O / sm_L );
  }
}

// Launches merge_partials_kernel behind the kernel that wrote the records (same stream).
template<typename T>
inline cudaError_t launch_merge_partials( const Shape& sh,
                                          const CtxMeta* ctx,
                                          const int32_t* split_ctx,
                                          uint32_t n_split_ctx,
                                          const float* part_o,
                                          const float* part_ml,
                                          T* xb,
                                          cudaStream_t st )
{
  cudaLaunchConfig_t cfg {};
  cfg.gridDim = dim3( n_split_ctx, sh.n_heads );
  cfg.blockDim = dim3( 128 );
  cfg.stream = st;
  cudaLaunchAttribute attr {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx( &cfg, merge_partials_kernel<T>, sh, ctx, split_ctx, part_o, part_ml, xb );
}

} // namespace gh
