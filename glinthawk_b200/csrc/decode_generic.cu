// Fused decode attention on CUDA cores: any head size up to 256, any group size, fp32 / fp16 / bf16 storage.
//
// One launch for the whole ragged batch replaces attention_0_gemm + attention_softmax + attention_2_gemm
// (src/arch/amd64/llama2/ops.hh:170-223, 283-298, 225-281): scores are never written to memory, the softmax is
// computed online in fp32 and the weighted sum of V is accumulated in fp32.  This is the kernel for fp32
// storage (where tensor cores would cost precision) and for head sizes the tensor-core kernel does not cover;
// it handles one query head per thread block and therefore re-reads K/V once per head of a group.
//
// Block = 4 warps working on one (work item, query head).  Warp w takes tokens t_begin + w, + 4, ...; its lanes
// split the head dimension; a dot product costs one warp reduction.  The four running softmax states are
// combined through shared memory, then store_item() writes the result or the partial record.
#include "gh_kernels.cuh"
#include "gh_merge.cuh"

namespace gh {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

template<typename T, int DPL> // DPL = head dimensions per lane
__global__ void __launch_bounds__( kThreads ) decode_generic_kernel( const DecodeArgs a )
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
    decode_generic_kernel<T, 2><<<grid, kThreads, 0, st>>>( a );
  else if ( a.sh.head_size <= 128 )
    decode_generic_kernel<T, 4><<<grid, kThreads, 0, st>>>( a );
  else
    decode_generic_kernel<T, 8><<<grid, kThreads, 0, st>>>( a );
  cudaError_t e = cudaGetLastError();
  if ( e == cudaSuccess && a.n_split_ctx > 0 )
    e = launch_merge_partials<T>( a.sh, a.ctx, a.split_ctx, a.n_split_ctx, a.part_o, a.part_ml, static_cast<T*>( a.xb ), st );
  return e;
}

} // namespace

cudaError_t launch_decode_generic( const DecodeArgs& a, cudaStream_t st, uint64_t* launches )
{
  if ( a.n_items == 0 )
    return cudaSuccess;
  cudaError_t e;
  switch ( a.dtype ) {
    case DT_F32: e = launch_t<float>( a, st ); break;
    case DT_F16: e = launch_t<__half>( a, st ); break;
    case DT_BF16: e = launch_t<__nv_bfloat16>( a, st ); break;
    default: return cudaErrorInvalidValue;
  }
  *launches += a.n_split_ctx > 0 ? 2 : 1;
  return e;
}

} // namespace gh
