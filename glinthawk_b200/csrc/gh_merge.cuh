// Epilogue shared by the decode kernels: write the result of a work item, or, for a context that was cut into
// several items, store a partial record and let whichever thread block finishes last combine the records.
// Nothing here waits on another block: the last arriver is found with one atomic increment
// (fence -> atomic -> fence), so there is no spin loop that could hang.
#pragma once

#include "gh_common.cuh"

namespace gh {

// Partial record r = ( partial_base + split ) * n_heads + head:
//   part_o[r][head_size]  sum_t 2^(s_t - m) * V_t   (fp32, not normalised)
//   part_ml[r][2]         m (running maximum of the log2-scaled scores), l = sum_t 2^(s_t - m)
//
// `sm_o` [nrows][head_size], `sm_m` [nrows], `sm_l` [nrows] hold this block's result for query heads
// head0 .. head0+nrows-1 in shared memory.  All `nthreads` threads of the calling group take part; `bar_id`
// names the hardware barrier that group synchronises on (0 = the whole block).
template<typename T>
__device__ __forceinline__ void finish_item( const Shape& sh,
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
                                             int* __restrict__ counters,
                                             const int counter_idx,
                                             int* sm_flag,
                                             const int tid,
                                             const int nthreads,
                                             const int bar_id )
{
  const int hs = sh.head_size;
  T* out = xb + (size_t)it.ctx * sh.n_heads * hs + (size_t)head0 * hs;

  if ( c.nsplits == 1 ) {
    for ( int e = tid; e < nrows * hs; e += nthreads ) {
      const int r = e / hs;
      out[e] = Conv<T>::from_f32( sm_o[e] / sm_l[r] );
    }
    return;
  }

  const size_t rec0 = ( (size_t)( c.partial_base + it.split ) * sh.n_heads + head0 );
  for ( int e = tid; e < nrows * hs; e += nthreads )
    part_o[rec0 * hs + e] = sm_o[e];
  for ( int r = tid; r < nrows; r += nthreads ) {
    part_ml[( rec0 + r ) * 2 + 0] = sm_m[r];
    part_ml[( rec0 + r ) * 2 + 1] = sm_l[r];
  }
  __threadfence();
  asm volatile( "bar.sync %0, %1;" ::"r"( bar_id ), "r"( nthreads ) : "memory" );
  if ( tid == 0 ) {
    const int prev = atomicAdd( &counters[counter_idx], 1 );
    *sm_flag = ( prev == c.nsplits - 1 ) ? 1 : 0;
  }
  asm volatile( "bar.sync %0, %1;" ::"r"( bar_id ), "r"( nthreads ) : "memory" );
  if ( *sm_flag == 0 )
    return;
  __threadfence();

  // This block arrived last: every record of the context is visible.  Combine them.
  for ( int e = tid; e < nrows * hs; e += nthreads ) {
    const int r = e / hs;
    float M = -INFINITY;
    for ( int s = 0; s < c.nsplits; s++ ) {
      const size_t rec = (size_t)( c.partial_base + s ) * sh.n_heads + head0 + r;
      M = fmaxf( M, __ldcg( &part_ml[rec * 2] ) );
    }
    float L = 0.f, O = 0.f;
    for ( int s = 0; s < c.nsplits; s++ ) {
      const size_t rec = (size_t)( c.partial_base + s ) * sh.n_heads + head0 + r;
      const float w = exp2f( __ldcg( &part_ml[rec * 2] ) - M );
      L += w * __ldcg( &part_ml[rec * 2 + 1] );
      O += w * __ldcg( &part_o[rec * hs + ( e - r * hs )] );
    }
    out[e] = Conv<T>::from_f32( O / L );
  }
  if ( tid == 0 )
    counters[counter_idx] = 0; // leave the counter ready for the next launch
}

} // namespace gh
