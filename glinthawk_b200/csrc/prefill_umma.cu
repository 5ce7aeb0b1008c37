// Causal attention for a multi-token prompt chunk on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The reference has no multi-token operation: it feeds a prompt one token per forward pass
// (src/worker/worker.hh:789-796, src/frontend/infer.cc:124-126), i.e. n_tokens x (attention_0_gemm, attention_softmax,
// attention_2_gemm) per context (src/arch/amd64/llama2/ops.hh:170-298).  This kernel computes the same thing for a
// whole chunk after the append kernel has written (and rotated) the chunk's K/V rows into the slots.
//
// One thread block = (context, kv head, query block).  A query block is 128 rows of the score matrix: 128 / group
// consecutive prompt tokens x the group's query heads, so every K/V byte fetched serves 128 rows.  Keys are walked in
// tiles of 64 tokens, staged by TMA (same arena descriptor and 128-byte swizzle as the decode kernel):
//
//   S[128 x 64]   = Q[128 x 128 dims] . K_tile^T      tcgen05.mma, both operands K-major in shared memory -> TMEM
//   P             = 2^(S * scale - m), causal mask    one thread per row (tcgen05.ld), no shuffles; written to shared
//                                                     memory as the next MMA's A operand
//   O[128 x 128] += P[128 x 64 keys] . V_tile         tcgen05.mma, V is the MN-major B operand straight from the tile
//
// Two passes over the keys: the first only finds each row's maximum m, the second accumulates with that final
// maximum, so O in TMEM never has to be rescaled.  Tensor work doubles for S, which costs little here; K is read
// twice, through L2.  fp32 accumulation throughout; P is rounded to the storage type (as in the decode kernel).
// 96 KiB of shared memory and 256 TMEM columns per block: two blocks per SM overlap each other's phases.
//
// Every wait is bounded; on expiry the kernel raises the sticky error word, frees its TMEM and leaves.
#include <type_traits>

#include "gh_kernels.cuh"

namespace gh {

namespace {

constexpr int kHS = 128;
constexpr int kRows = 128;                 // rows of a query block = TMEM lanes
constexpr int kKeys = 64;                  // keys per tile
constexpr int kBoxRows = 32;               // token rows per TMA box of the arena descriptor
constexpr int kQRegion = kRows * 128;      // [128 rows x 128 B] swizzled region (Q: two of them, P: one) = 16 KiB
constexpr int kKRegion = kKeys * 128;      // [64 keys x 128 B] swizzled region (K and V tiles: two each) = 8 KiB
constexpr int kKTile = 2 * kKRegion;       // 16 KiB
constexpr int kOffP = 2 * kQRegion;        // shared-memory map: Q | P | K stage 0 | K stage 1 | V
constexpr int kOffK = kOffP + kQRegion;
constexpr int kOffV = kOffK + 2 * kKTile;
constexpr int kSmemBytes = kOffV + kKTile + 1024; // 96 KiB + alignment slack: two blocks per SM
constexpr int kTmemCols = 256;             // S: columns 0..63, O: columns 128..255 (two blocks fill the SM's 512)
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32( const void* p )
{
  return static_cast<uint32_t>( __cvta_generic_to_shared( p ) );
}

__device__ __forceinline__ bool mbar_wait( uint64_t* bar, uint32_t parity )
{
  const uint32_t addr = smem_u32( bar );
  for ( uint32_t it = 0; it < kWaitLimit; it++ ) {
    uint32_t done;
    asm volatile( "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                  : "=r"( done )
                  : "r"( addr ), "r"( parity )
                  : "memory" );
    if ( done )
      return true;
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
// MN-major operand (V: [keys][64 dims] regions): the next 64 dims are one region further, the next 8 keys 1024 B.
__device__ __forceinline__ uint64_t desc_mnmajor( uint32_t saddr )
{
  return umma_desc( saddr, kKRegion, 1024 );
}

__device__ __forceinline__ void umma_f16( uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate )
{
  asm volatile( "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                ::"r"( tmem_d ), "l"( da ), "l"( db ), "r"( idesc ), "r"( accumulate )
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


// One work item = (context, query block): `split` is the query block's index, t_end the number of keys its last
// token sees.  Thread r of the block owns row r = (token r / group, head r % group) of the query block.
template<typename T>
__global__ void __launch_bounds__( kRows, 2 )
  prefill_umma_kernel( const DecodeArgs a, const __grid_constant__ CUtensorMap kv_map )
{
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_k[2]; // K tile landed in stage s
  __shared__ uint64_t bar_v;    // V tile landed
  __shared__ uint64_t bar_s;    // S = Q K^T of the current tile is in TMEM
  __shared__ uint64_t bar_pv;   // O += P V of the current tile has finished (P, V and S may be reused)
  __shared__ uint32_t tmem_base;
  __shared__ int sm_fail;

  uint8_t* base = reinterpret_cast<uint8_t*>( ( reinterpret_cast<uintptr_t>( smem_raw ) + 1023 ) & ~uintptr_t( 1023 ) );
  uint8_t* sQ = base;
  uint8_t* sP = base + kOffP;
  uint8_t* sK = base + kOffK; // two stages
  uint8_t* sV = base + kOffV;

  const Shape& sh = a.sh;
  const int group = sh.group;
  const int item_idx = blockIdx.x / sh.n_kv_heads;
  const int kvh = blockIdx.x - item_idx * sh.n_kv_heads;
  const WorkItem it = a.items[item_idx];
  const CtxMeta c = a.ctx[it.ctx];
  const int r = threadIdx.x;
  const int warp = r >> 5;

  const int tok_per_block = kRows / group;
  const int tok0 = it.split * tok_per_block;                                // first chunk token of the query block
  const int n_tok = min( tok_per_block, (int)a.chunk_tokens - tok0 );       // tokens the block really has
  const int row_tok = r / group, row_head = r - row_tok * group;
  const bool row_live = row_tok < n_tok;
  const int n_keys = it.t_end;                                              // keys seen by the block's last token
  const int row_limit = row_live ? n_keys - ( n_tok - 1 - row_tok ) : 0;    // keys seen by this row's token
  const int n_tiles = ( n_keys + kKeys - 1 ) / kKeys;
  const float scale_log2 = 0.08838834764831845f * 1.4426950408889634f;      // 1/sqrt(128) * log2(e)

  if ( r == 0 ) {
    sm_fail = 0;
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"( smem_u32( &bar_k[0] ) ) );
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"( smem_u32( &bar_k[1] ) ) );
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"( smem_u32( &bar_v ) ) );
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"( smem_u32( &bar_s ) ) );
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"( smem_u32( &bar_pv ) ) );
    asm volatile( "fence.mbarrier_init.release.cluster;" ::: "memory" );
    asm volatile( "prefetch.tensormap [%0];" ::"l"( reinterpret_cast<uint64_t>( &kv_map ) ) : "memory" );
  }
  if ( warp == 0 ) {
    asm volatile( "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"( smem_u32( &tmem_base ) ),
                  "r"( kTmemCols ) );
    asm volatile( "tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" );
  }
  // the append kernel (the kernel before this one in the stream) rotated q and wrote the chunk's K/V rows
  asm volatile( "griddepcontrol.wait;" ::: "memory" );

  // ---- Q block into shared memory, K-major with the 128-byte swizzle the MMA descriptors expect
  {
    const T* qrow = static_cast<const T*>( a.q )
                    + ( ( (size_t)it.ctx * a.chunk_tokens + tok0 + row_tok ) * sh.n_heads + (size_t)kvh * group + row_head ) * kHS;
#pragma unroll
    for ( int ch = 0; ch < 16; ch++ ) { // 16 chunks of 8 elements
      uint4 v = make_uint4( 0, 0, 0, 0 );
      if ( row_live )
        v = *reinterpret_cast<const uint4*>( qrow + ch * 8 );
      *reinterpret_cast<uint4*>( sQ + ( ch >> 3 ) * kQRegion + r * 128 + ( ( ( ch & 7 ) ^ ( r & 7 ) ) << 4 ) ) = v;
    }
  }
  asm volatile( "fence.proxy.async.shared::cta;" ::: "memory" );
  asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
  __syncthreads();
  asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;
  const uint32_t lane_off = static_cast<uint32_t>( warp * 32 ) << 16; // this warp's quarter of the TMEM lanes

  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  // instruction descriptors: fp32 accumulate, A/B format, M = 128; S has N = 64 keys, O has N = 128 dims with V as
  // the MN-major B operand
  const uint32_t idesc_s = ( 1u << 4 ) | ( fmt << 7 ) | ( fmt << 10 ) | ( ( (uint32_t)kKeys >> 3 ) << 17 ) | ( ( 128u >> 4 ) << 24 );
  const uint32_t idesc_pv = ( 1u << 4 ) | ( fmt << 7 ) | ( fmt << 10 ) | ( 1u << 16 ) | ( ( 128u >> 3 ) << 17 ) | ( ( 128u >> 4 ) << 24 );

  const long long row_bytes = (long long)sh.row_elems * (long long)sizeof( T );
  const int arena_row0 = static_cast<int>( ( c.kv_off + a.layer_off ) / row_bytes );
  const int xk = kvh * kHS, xv = (int)sh.kv_dim + kvh * kHS;

  // TMA loads of key tile t (thread 0 only).  Only boxes holding at least one live key are fetched: rows beyond may
  // lie in pages that are not mapped.
  auto load_tile = [&]( int t, uint8_t* dst, int x, uint64_t* bar ) {
    const int live = min( kKeys, n_keys - t * kKeys );
    const int boxes = ( live + kBoxRows - 1 ) / kBoxRows;
    asm volatile( "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"( smem_u32( bar ) ),
                  "r"( (uint32_t)boxes * kBoxRows * 128 * 2 )
                  : "memory" );
    for ( int j = 0; j < boxes; j++ ) {
      const int y = arena_row0 + t * kKeys + j * kBoxRows;
      tma_load_2d( dst + j * kBoxRows * 128, &kv_map, x, y, bar );
      tma_load_2d( dst + kKRegion + j * kBoxRows * 128, &kv_map, x + 64, y, bar );
    }
  };
  auto load_k = [&]( int t ) { load_tile( t, sK + ( t & 1 ) * kKTile, xk, &bar_k[t & 1] ); };
  auto load_v = [&]( int t ) { load_tile( t, sV, xv, &bar_v ); };
  // S = Q K_tile^T: 8 MMAs of 16 dims each (thread 0 only)
  auto issue_s = [&]( int s ) {
#pragma unroll
    for ( int k = 0; k < 8; k++ ) {
      const uint64_t da = desc_kmajor( smem_u32( sQ + ( k >> 2 ) * kQRegion + ( k & 3 ) * 32 ) );
      const uint64_t db = desc_kmajor( smem_u32( sK + s * kKTile + ( k >> 2 ) * kKRegion + ( k & 3 ) * 32 ) );
      umma_f16( tmem_s, da, db, idesc_s, k > 0 ? 1u : 0u );
    }
    umma_commit( &bar_s );
  };
  // thread 0: wait for K tile t, then S; on a timeout raise the flag and release the waiters
  auto k_then_s = [&]( int t, uint32_t parity ) {
    if ( mbar_wait( &bar_k[t & 1], parity ) ) {
      asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
      issue_s( t & 1 );
    } else {
      sm_fail = 1;
      asm volatile( "mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"( smem_u32( &bar_s ) ) : "memory" );
    }
  };

  uint32_t k_uses[2] = { 0, 0 }; // completed phases of the barriers, tracked identically by every thread
  uint32_t v_uses = 0, s_phase = 0, pv_phase = 0;
  bool ok = true;

  // ================= pass 1: row maxima =================
  float m = -INFINITY;
  if ( r == 0 )
    load_k( 0 );
  for ( int t = 0; t < n_tiles && ok; t++ ) {
    const int s = t & 1;
    if ( r == 0 ) {
      if ( t + 1 < n_tiles )
        load_k( t + 1 ); // its stage was last read by tile t-1's MMAs, which have completed
      k_then_s( t, k_uses[s] & 1 );
    }
    k_uses[s]++;
    ok = mbar_wait( &bar_s, s_phase & 1 );
    s_phase++;
    asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
    if ( __all_sync( 0xffffffffu, ok && sm_fail == 0 ) ) {
      const int lim = row_limit - t * kKeys; // keys of this tile the row sees
      // tcgen05.ld is a warp-wide instruction: the decision to load a column block is made per warp
      const int warp_lim = __reduce_max_sync( 0xffffffffu, lim );
#pragma unroll 1
      for ( int cb = 0; cb < kKeys / 32; cb++ ) {
        if ( cb * 32 >= warp_lim )
          break;
        float v[32];
        tmem_ld32( tmem_s + lane_off + cb * 32, v );
#pragma unroll
        for ( int j = 0; j < 32; j++ )
          m = fmaxf( m, ( cb * 32 + j < lim ) ? v[j] * scale_log2 : -INFINITY );
      }
    }
    asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
    ok = __syncthreads_and( ok && sm_fail == 0 ) != 0; // everyone has read S before the next MMA overwrites it
  }

  // ================= pass 2: P and O =================
  const float m_use = ( m == -INFINITY ) ? 0.f : m; // a row that sees nothing carries zeros, not NaNs
  float l = 0.f;
  if ( ok && r == 0 )
    load_k( 0 );
  for ( int t = 0; t < n_tiles && ok; t++ ) {
    const int s = t & 1;
    // P, V and S are free once tile t-1's P.V has finished
    if ( t > 0 ) {
      ok = mbar_wait( &bar_pv, pv_phase & 1 );
      pv_phase++;
      asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
    }
    if ( r == 0 && ok ) {
      load_v( t );
      if ( t + 1 < n_tiles )
        load_k( t + 1 );
      k_then_s( t, k_uses[s] & 1 );
    }
    k_uses[s]++;
    if ( ok ) {
      ok = mbar_wait( &bar_s, s_phase & 1 );
      s_phase++;
    }
    asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
    if ( __all_sync( 0xffffffffu, ok && sm_fail == 0 ) ) {
      const int lim = row_limit - t * kKeys;
      const int warp_lim = __reduce_max_sync( 0xffffffffu, lim );
#pragma unroll 1
      for ( int cb = 0; cb < kKeys / 32; cb++ ) {
        float v[32];
        if ( cb * 32 < warp_lim ) {
          tmem_ld32( tmem_s + lane_off + cb * 32, v );
        } else {
#pragma unroll
          for ( int j = 0; j < 32; j++ )
            v[j] = 0.f;
        }
        uint32_t pk[16];
#pragma unroll
        for ( int j = 0; j < 32; j += 2 ) {
          const float p0 = ( cb * 32 + j < lim ) ? fast_exp2( v[j] * scale_log2 - m_use ) : 0.f;
          const float p1 = ( cb * 32 + j + 1 < lim ) ? fast_exp2( v[j + 1] * scale_log2 - m_use ) : 0.f;
          l += p0 + p1;
          pk[j >> 1] = pack2<T>( p0, p1 );
        }
        // 32 keys = 4 chunks of 8 keys (16 B) of row r in P's K-major swizzled layout
#pragma unroll
        for ( int q4 = 0; q4 < 4; q4++ ) {
          const int ch = cb * 4 + q4; // chunk index 0..7 along the 64 keys
          *reinterpret_cast<uint4*>( sP + r * 128 + ( ( ch ^ ( r & 7 ) ) << 4 ) )
            = make_uint4( pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3] );
        }
      }
      // V rows past the last key hold stale or foreign data: clear them so that 0 * garbage cannot make a NaN
      ok = mbar_wait( &bar_v, v_uses & 1 );
      const int live = min( kKeys, n_keys - t * kKeys ); // keys of this tile that exist at all
      if ( ok && r >= live && r < kKeys ) {
        uint8_t* v0 = sV + r * 128;
#pragma unroll
        for ( int ch = 0; ch < 8; ch++ ) {
          *reinterpret_cast<uint4*>( v0 + ch * 16 ) = make_uint4( 0, 0, 0, 0 );
          *reinterpret_cast<uint4*>( v0 + kKRegion + ch * 16 ) = make_uint4( 0, 0, 0, 0 );
        }
      }
    }
    v_uses++;
    asm volatile( "fence.proxy.async.shared::cta;" ::: "memory" ); // P and the cleared V rows -> tensor-core proxy
    asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
    ok = __syncthreads_and( ok && sm_fail == 0 ) != 0;
    if ( ok && r == 0 ) {
      asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
#pragma unroll
      for ( int k = 0; k < kKeys / 16; k++ ) { // 16 keys per MMA
        const uint64_t da = desc_kmajor( smem_u32( sP + k * 32 ) );
        const uint64_t db = desc_mnmajor( smem_u32( sV + k * 16 * 128 ) );
        umma_f16( tmem_o, da, db, idesc_pv, ( t > 0 || k > 0 ) ? 1u : 0u );
      }
      umma_commit( &bar_pv );
    }
  }

  // ================= epilogue: O / l -> xb =================
  if ( ok && n_tiles > 0 ) {
    ok = mbar_wait( &bar_pv, pv_phase & 1 );
    asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
  }
  ok = __all_sync( 0xffffffffu, ok );
  if ( ok ) { // warp-uniform: the TMEM loads below are warp-wide; only the stores depend on the row
    T* out = static_cast<T*>( a.xb )
             + ( ( (size_t)it.ctx * a.chunk_tokens + tok0 + row_tok ) * sh.n_heads + (size_t)kvh * group + row_head ) * kHS;
    const float inv = 1.0f / l;
#pragma unroll 1
    for ( int cb = 0; cb < 4; cb++ ) {
      float v[32];
      tmem_ld32( tmem_o + lane_off + cb * 32, v );
#pragma unroll
      for ( int q4 = 0; q4 < 4; q4++ ) {
        uint32_t w[4];
#pragma unroll
        for ( int j = 0; j < 4; j++ )
          w[j] = pack2<T>( v[q4 * 8 + 2 * j] * inv, v[q4 * 8 + 2 * j + 1] * inv );
        if ( row_live )
          *reinterpret_cast<uint4*>( out + cb * 32 + q4 * 8 ) = make_uint4( w[0], w[1], w[2], w[3] );
      }
    }
  }
  if ( !ok && r == 0 )
    atomicOr( a.dev_error, 4u );
  asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
  __syncthreads();
  if ( warp == 0 )
    asm volatile( "tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"( tmem_base ), "r"( kTmemCols ) );
}

} // namespace

bool prefill_umma_supported( const Shape& sh, uint32_t dtype )
{
  return ( dtype == DT_F16 || dtype == DT_BF16 ) && sh.head_size == kHS && sh.group <= 16 && kRows % sh.group == 0
         && sh.seq_len % 64 == 0;
}

uint32_t prefill_umma_tokens_per_item( const Shape& sh )
{
  return kRows / sh.group;
}

cudaError_t prefill_umma_prepare()
{
  cudaError_t e = cudaFuncSetAttribute( prefill_umma_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes );
  if ( e == cudaSuccess )
    e = cudaFuncSetAttribute( prefill_umma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes );
  return e;
}

cudaError_t launch_prefill_umma( const DecodeArgs& a, const CUtensorMap* kv_map, cudaStream_t st, uint64_t* launches )
{
  if ( a.n_items == 0 )
    return cudaSuccess;
  cudaLaunchConfig_t cfg {};
  cfg.gridDim = dim3( a.n_items * a.sh.n_kv_heads );
  cfg.blockDim = dim3( kRows );
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if ( a.dtype == DT_F16 )
    e = cudaLaunchKernelEx( &cfg, prefill_umma_kernel<__half>, a, *kv_map );
  else if ( a.dtype == DT_BF16 )
    e = cudaLaunchKernelEx( &cfg, prefill_umma_kernel<__nv_bfloat16>, a, *kv_map );
  else
    return cudaErrorInvalidValue;
  ( *launches )++;
  return e;
}

} // namespace gh
