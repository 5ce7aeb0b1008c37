// tcgen05 / TMA / mbarrier building blocks shared by the kernels that run on the 5th-generation tensor cores
// (prompt-chunk attention, the q/kv projection).  Inline PTX only; every wait is bounded.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace gh {
namespace umma {

constexpr uint32_t kWaitLimit = 1u << 16;     // attempts per wait ...
constexpr uint32_t kWaitHintNs = 20000;     // ... of up to 20 us each: a wait gives up after about a second

__device__ __forceinline__ uint32_t smem_u32( const void* p )
{
  return static_cast<uint32_t>( __cvta_generic_to_shared( p ) );
}

// Bounded wait on an mbarrier phase.  Gives up when the limit is reached or another role of the block has
// raised `fail`.
__device__ __forceinline__ bool mbar_wait( uint64_t* bar, uint32_t parity, volatile int* fail )
{
  const uint32_t addr = smem_u32( bar );
  for ( uint32_t it = 0; it < kWaitLimit; it++ ) {
    uint32_t done;
    // the hint lets a waiting thread sleep up to that many nanoseconds per attempt instead of taking issue slots
    // from the warps that have work; it wakes as soon as the phase completes
    asm volatile( "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                  : "=r"( done )
                  : "r"( addr ), "r"( parity ), "r"( kWaitHintNs )
                  : "memory" );
    if ( done )
      return true;
    if ( ( it & 15u ) == 15u && *fail != 0 )
      return false;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d( void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar )
{
  asm volatile( "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"( smem_u32( dst ) ),
                "l"( reinterpret_cast<uint64_t>( map ) ), "r"( x ), "r"( y ), "r"( smem_u32( bar ) )
                : "memory" );
}

// The same with an L2 eviction policy (from createpolicy) for the fetched lines.
__device__ __forceinline__ void tma_load_2d_hint( void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t policy )
{
  asm volatile( "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                ::"r"( smem_u32( dst ) ),
                "l"( reinterpret_cast<uint64_t>( map ) ), "r"( x ), "r"( y ), "r"( smem_u32( bar ) ), "l"( policy )
                : "memory" );
}

__device__ __forceinline__ void tma_load_4d( void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar )
{
  asm volatile( "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                ::"r"( smem_u32( dst ) ),
                "l"( reinterpret_cast<uint64_t>( map ) ), "r"( c0 ), "r"( c1 ), "r"( c2 ), "r"( c3 ), "r"( smem_u32( bar ) )
                : "memory" );
}

// Shared -> global; the part of the box outside the tensor is not written.
__device__ __forceinline__ void tma_store_4d( const CUtensorMap* map, int c0, int c1, int c2, int c3, const void* src )
{
  asm volatile( "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                ::"l"( reinterpret_cast<uint64_t>( map ) ), "r"( c0 ), "r"( c1 ), "r"( c2 ), "r"( c3 ), "r"( smem_u32( src ) )
                : "memory" );
}

// Shared-memory matrix descriptors (sm_100 format): start address, leading / stride byte offsets (all >> 4),
// version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc( uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes )
{
  uint64_t d = 0;
  d |= static_cast<uint64_t>( ( saddr & 0x3FFFF ) >> 4 );
  d |= static_cast<uint64_t>( lbo_bytes >> 4 ) << 16;
  d |= static_cast<uint64_t>( sbo_bytes >> 4 ) << 32;
  d |= static_cast<uint64_t>( 1 ) << 46;
  d |= static_cast<uint64_t>( 2 ) << 61;
  return d;
}
// K-major operand ([rows][64 elements] regions): 8-row groups are 1024 B apart; the leading offset is unused.
__device__ __forceinline__ uint64_t desc_kmajor( uint32_t saddr )
{
  return umma_desc( saddr, 16, 1024 );
}
__device__ __forceinline__ void umma_f16( uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate )
{
  asm volatile( "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                ::"r"( tmem_d ), "l"( da ), "l"( db ), "r"( idesc ), "r"( accumulate )
                : "memory" );
}

// The same with the A operand in tensor memory: row i of A in lane i, two 16-bit elements per 32-bit column.
__device__ __forceinline__ void umma_f16_ts( uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate )
{
  asm volatile( "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                ::"r"( tmem_d ), "r"( tmem_a ), "l"( db ), "r"( idesc ), "r"( accumulate )
                : "memory" );
}

__device__ __forceinline__ void umma_commit( uint64_t* bar )
{
  asm volatile( "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"( smem_u32( bar ) )
                : "memory" );
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32( uint32_t taddr, float ( &v )[32] )
{
  uint32_t r[32];
  asm volatile( "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                : "=r"( r[0] ), "=r"( r[1] ), "=r"( r[2] ), "=r"( r[3] ), "=r"( r[4] ), "=r"( r[5] ), "=r"( r[6] ), "=r"( r[7] ),
                  "=r"( r[8] ), "=r"( r[9] ), "=r"( r[10] ), "=r"( r[11] ), "=r"( r[12] ), "=r"( r[13] ), "=r"( r[14] ), "=r"( r[15] ),
                  "=r"( r[16] ), "=r"( r[17] ), "=r"( r[18] ), "=r"( r[19] ), "=r"( r[20] ), "=r"( r[21] ), "=r"( r[22] ), "=r"( r[23] ),
                  "=r"( r[24] ), "=r"( r[25] ), "=r"( r[26] ), "=r"( r[27] ), "=r"( r[28] ), "=r"( r[29] ), "=r"( r[30] ), "=r"( r[31] )
                : "r"( taddr ) );
  asm volatile( "tcgen05.wait::ld.sync.aligned;" ::: "memory" );
#pragma unroll
  for ( int i = 0; i < 32; i++ )
    v[i] = __uint_as_float( r[i] );
}

// 64 consecutive fp32 columns of this thread's TMEM lane, one load and one wait.
__device__ __forceinline__ void tmem_ld64( uint32_t taddr, float ( &v )[64] )
{
  uint32_t r[64];
  asm volatile( "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
                : "=r"( r[0] ), "=r"( r[1] ), "=r"( r[2] ), "=r"( r[3] ), "=r"( r[4] ), "=r"( r[5] ), "=r"( r[6] ), "=r"( r[7] ), "=r"( r[8] ), "=r"( r[9] ), "=r"( r[10] ), "=r"( r[11] ), "=r"( r[12] ), "=r"( r[13] ), "=r"( r[14] ), "=r"( r[15] ), "=r"( r[16] ), "=r"( r[17] ), "=r"( r[18] ), "=r"( r[19] ), "=r"( r[20] ), "=r"( r[21] ), "=r"( r[22] ), "=r"( r[23] ), "=r"( r[24] ), "=r"( r[25] ), "=r"( r[26] ), "=r"( r[27] ), "=r"( r[28] ), "=r"( r[29] ), "=r"( r[30] ), "=r"( r[31] ), "=r"( r[32] ), "=r"( r[33] ), "=r"( r[34] ), "=r"( r[35] ), "=r"( r[36] ), "=r"( r[37] ), "=r"( r[38] ), "=r"( r[39] ), "=r"( r[40] ), "=r"( r[41] ), "=r"( r[42] ), "=r"( r[43] ), "=r"( r[44] ), "=r"( r[45] ), "=r"( r[46] ), "=r"( r[47] ), "=r"( r[48] ), "=r"( r[49] ), "=r"( r[50] ), "=r"( r[51] ), "=r"( r[52] ), "=r"( r[53] ), "=r"( r[54] ), "=r"( r[55] ), "=r"( r[56] ), "=r"( r[57] ), "=r"( r[58] ), "=r"( r[59] ), "=r"( r[60] ), "=r"( r[61] ), "=r"( r[62] ), "=r"( r[63] )
                : "r"( taddr ) );
  asm volatile( "tcgen05.wait::ld.sync.aligned;" ::: "memory" );
#pragma unroll
  for ( int i = 0; i < 64; i++ )
    v[i] = __uint_as_float( r[i] );
}

// Write 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st32( uint32_t taddr, const float ( &v )[32] )
{
  uint32_t r[32];
#pragma unroll
  for ( int i = 0; i < 32; i++ )
    r[i] = __float_as_uint( v[i] );
  asm volatile( "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                ::"r"( taddr ),
                "r"( r[0] ), "r"( r[1] ), "r"( r[2] ), "r"( r[3] ), "r"( r[4] ), "r"( r[5] ), "r"( r[6] ), "r"( r[7] ), "r"( r[8] ),
                "r"( r[9] ), "r"( r[10] ), "r"( r[11] ), "r"( r[12] ), "r"( r[13] ), "r"( r[14] ), "r"( r[15] ), "r"( r[16] ),
                "r"( r[17] ), "r"( r[18] ), "r"( r[19] ), "r"( r[20] ), "r"( r[21] ), "r"( r[22] ), "r"( r[23] ), "r"( r[24] ),
                "r"( r[25] ), "r"( r[26] ), "r"( r[27] ), "r"( r[28] ), "r"( r[29] ), "r"( r[30] ), "r"( r[31] )
                : "memory" );
  asm volatile( "tcgen05.wait::st.sync.aligned;" ::: "memory" );
}

__device__ __forceinline__ void tmem_st32_bits( uint32_t taddr, const uint32_t ( &r )[32] )
{
  asm volatile( "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                ::"r"( taddr ),
                "r"( r[0] ), "r"( r[1] ), "r"( r[2] ), "r"( r[3] ), "r"( r[4] ), "r"( r[5] ), "r"( r[6] ), "r"( r[7] ), "r"( r[8] ),
                "r"( r[9] ), "r"( r[10] ), "r"( r[11] ), "r"( r[12] ), "r"( r[13] ), "r"( r[14] ), "r"( r[15] ), "r"( r[16] ),
                "r"( r[17] ), "r"( r[18] ), "r"( r[19] ), "r"( r[20] ), "r"( r[21] ), "r"( r[22] ), "r"( r[23] ), "r"( r[24] ),
                "r"( r[25] ), "r"( r[26] ), "r"( r[27] ), "r"( r[28] ), "r"( r[29] ), "r"( r[30] ), "r"( r[31] )
                : "memory" );
  asm volatile( "tcgen05.wait::st.sync.aligned;" ::: "memory" );
}

template<typename T>
__device__ __forceinline__ uint32_t pack2( float lo, float hi );
template<>
__device__ __forceinline__ uint32_t pack2<__half>( float lo, float hi )
{
  const __half2 h = __floats2half2_rn( lo, hi );
  return *reinterpret_cast<const uint32_t*>( &h );
}
template<>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>( float lo, float hi )
{
  const __nv_bfloat162 h = __floats2bfloat162_rn( lo, hi );
  return *reinterpret_cast<const uint32_t*>( &h );
}

__device__ __forceinline__ float fast_exp2( float x )
{
  float y;
  asm( "ex2.approx.ftz.f32 %0, %1;" : "=f"( y ) : "f"( x ) );
  return y;
}

} // namespace umma
} // namespace gh
