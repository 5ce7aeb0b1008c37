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
//   P             = 2^(S * scale - m), causal mask    one thread per row (tcgen05.ld), no shuffles; stored back over
//                                                     S in TMEM (tcgen05.st), 16 bits per key
//   O[128 x 128] += P[128 x 64 keys] . V_tile         tcgen05.mma with A = P from TMEM, V the MN-major B operand
//                                                     straight from the tile
//
// Three roles: warps 0..3 own one score row per thread; one lane of warp 4 feeds the K/V stages (and the Q block)
// by TMA; one lane of warp 5 issues the MMAs.  They meet only on mbarriers.
//
// One pass over the keys with a running row maximum m.  O lives in TMEM, so raising m means rescaling O there
// (tcgen05.ld, multiply, tcgen05.st); that is done lazily, only when some row of a warp has outgrown its m by more
// than 2^8, so P stays below 256 (exact enough in fp16 and bf16, harmless in the fp32 accumulator) and on typical data
// only the first tiles rescale.  K and V tiles are double-buffered and S has two TMEM buffers: S of tile t+1 is
// issued before the row owners start on tile t, and the P.V MMAs of tile t run while they work on tile t+1.  Keeping
// P out of shared memory matters: the MMAs' operand reads, not their arithmetic, are what fills the SM here.
// fp32 accumulation throughout; P is rounded to the storage type (as in the decode kernel).  The finished O block
// leaves through the Q block's shared memory and a TMA store.
// 96 KiB of shared memory and 256 TMEM columns per block: two blocks per SM overlap each other's phases.
//
// Every wait is bounded; on expiry the kernel raises the sticky error word, frees its TMEM and leaves.
#include <type_traits>

#include "gh_kernels.cuh"
#include "gh_umma.cuh"

namespace gh {

namespace {

constexpr int kHS = 128;
constexpr int kRows = 128;                 // rows of a query block = TMEM lanes = row-owner threads
constexpr int kThreads = kRows + 64;       // + the TMA warp and the MMA warp
constexpr int kKeys = 64;                  // keys per tile
constexpr int kBoxRows = 32;               // token rows per TMA box of the arena descriptor
constexpr int kQRegion = kRows * 128;      // [128 rows x 128 B] swizzled region (Q: two of them) = 16 KiB
constexpr int kKRegion = kKeys * 128;      // [64 keys x 128 B] swizzled region (K and V tiles: two each) = 8 KiB
constexpr int kKTile = 2 * kKRegion;       // 16 KiB
constexpr int kOffK = 2 * kQRegion;        // shared-memory map: Q | K stages 0, 1 | V stages 0, 1 | barriers
constexpr int kOffV = kOffK + 2 * kKTile;
constexpr int kOffBar = kOffV + 2 * kKTile;
constexpr int kSmemBytes = kOffBar + 128;  // 96 KiB + barriers; two blocks per SM
constexpr int kTmemCols = 256;             // S buffers: columns 0..63 and 64..127, O: columns 128..255
constexpr float kGrowLog2 = 8.f;           // a row's maximum may lag its true maximum by this much (log2 units)
using namespace umma;

// Two fp32 values in one 64-bit register for the packed fp32 instructions of sm_100 (fma.rn.f32x2, add.rn.f32x2):
// the row owners are short of issue slots, and these halve the scale-and-shift and the row-sum instructions.
__device__ __forceinline__ unsigned long long pack_f2( float lo, float hi )
{
  unsigned long long r;
  asm( "mov.b64 %0, {%1, %2};" : "=l"( r ) : "f"( lo ), "f"( hi ) );
  return r;
}
__device__ __forceinline__ void unpack_f2( unsigned long long v, float& lo, float& hi )
{
  asm( "mov.b64 {%0, %1}, %2;" : "=f"( lo ), "=f"( hi ) : "l"( v ) );
}
__device__ __forceinline__ unsigned long long fma_f2( unsigned long long a, unsigned long long b, unsigned long long c )
{
  unsigned long long r;
  asm( "fma.rn.f32x2 %0, %1, %2, %3;" : "=l"( r ) : "l"( a ), "l"( b ), "l"( c ) );
  return r;
}
__device__ __forceinline__ unsigned long long add_f2( unsigned long long a, unsigned long long b )
{
  unsigned long long r;
  asm( "add.rn.f32x2 %0, %1, %2;" : "=l"( r ) : "l"( a ), "l"( b ) );
  return r;
}
__device__ __forceinline__ float max3( float a, float b, float c )
{
  float r;
  asm( "max.f32 %0, %1, %2, %3;" : "=f"( r ) : "f"( a ), "f"( b ), "f"( c ) );
  return r;
}

// MN-major operand (V: [keys][64 dims] regions): the next 64 dims are one region further, the next 8 keys 1024 B.
__device__ __forceinline__ uint64_t desc_mnmajor( uint32_t saddr )
{
  return umma_desc( saddr, kKRegion, 1024 );
}



// One work item = (context, query block): `split` is the query block's index, t_end the number of keys its last
// token sees.  Warps 0..3: thread r owns row r = (token r / group, head r % group) of the query block and does its
// softmax; warp 4: one lane feeds the K/V stages by TMA; warp 5: one lane issues the MMAs.
template<typename T>
__global__ void __launch_bounds__( kThreads, 2 )
  prefill_umma_kernel( const DecodeArgs a, const __grid_constant__ CUtensorMap kv_map,
                       const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap xb_map )
{
  extern __shared__ __align__( 1024 ) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kOffK; // two stages
  uint8_t* sV = smem + kOffV; // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>( smem + kOffBar );
  uint64_t* bar_k = bars;          // [2] K tile landed in stage s                      (TMA -> MMA lane)
  uint64_t* bar_v = bars + 2;      // [2] V tile landed in stage s                      (TMA -> MMA lane, row owners)
  uint64_t* bar_s = bars + 4;      // [2] S = Q K^T complete in TMEM buffer b           (MMA -> row owners)
  uint64_t* bar_kfree = bars + 6;  // [2] the MMAs reading K stage s have completed     (MMA -> TMA lane)
  uint64_t* bar_vfree = bars + 8;  // [2] the MMAs reading V stage s have completed     (MMA -> TMA lane)
  uint64_t* bar_pv = bars + 10;    // O += P V of a tile has completed: O may be rescaled (MMA -> row owners)
  uint64_t* bar_p = bars + 11;     // all 128 row owners have put P in place of S       (row owners -> MMA lane)
  uint64_t* bar_q = bars + 12;     // Q block has landed                                (TMA -> MMA lane)
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>( bars + 13 );
  volatile int* fail = reinterpret_cast<volatile int*>( bars + 14 );

  const int r = threadIdx.x;
  const int warp = r >> 5;
  // the swizzled tiles need a 1024-byte aligned base; with no static shared memory the dynamic region starts on one
  if ( ( smem_u32( smem ) & 1023u ) != 0 ) {
    if ( r == 0 )
      atomicOr( a.dev_error, 8u );
    return;
  }

  const Shape& sh = a.sh;
  const int group = sh.group;
  const int item_idx = blockIdx.x / sh.n_kv_heads;
  const int kvh = blockIdx.x - item_idx * sh.n_kv_heads;
  const WorkItem it = a.items[item_idx];

  const int tok_per_block = kRows / group;
  const int tok0 = it.split * tok_per_block;                          // first chunk token of the query block
  const int n_tok = min( tok_per_block, (int)a.chunk_tokens - tok0 ); // tokens the block really has
  const int n_keys = it.t_end;                                        // keys seen by the block's last token
  const int n_tiles = ( n_keys + kKeys - 1 ) / kKeys;

  // The TMA lane sets the barriers up and has the Q block and the first tiles on their way before the rest of the
  // block has finished its own set-up; warp 5 gets the tensor memory.
  const int arena_row0 = it.t_begin + a.layer_row; // (the host put the context's first arena row into the item)
  const int xk = kvh * kHS, xv = (int)sh.kv_dim + kvh * kHS;
  // Only boxes holding at least one live key are fetched: rows beyond may lie in pages that are not mapped.
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
  auto load_v = [&]( int t ) { load_tile( t, sV + ( t & 1 ) * kKTile, xv, &bar_v[t & 1] ); };
  if ( r == 4 * 32 ) {
    *fail = 0;
#pragma unroll
    for ( int i = 0; i < 13; i++ )
      asm volatile( "mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"( smem_u32( &bars[i] ) ), "r"( i == 11 ? kRows : 1 ) );
    asm volatile( "fence.mbarrier_init.release.cluster;" ::: "memory" );
    // the append kernel (the kernel before this one in the stream) rotated q and wrote the chunk's K/V rows
    asm volatile( "griddepcontrol.wait;" ::: "memory" );
    // The query block: box = [64 dims][group heads][128 / group tokens] of q viewed as
    // [contexts][chunk tokens][heads][128], twice (dims 0..63, 64..127).  Its rows land in (token, head) order
    // with the 128-byte swizzle the MMA descriptors expect; tokens past the chunk's end arrive as zeros.
    asm volatile( "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"( smem_u32( bar_q ) ), "r"( 2 * kQRegion )
                  : "memory" );
    tma_load_4d( sQ, &q_map, 0, kvh * group, tok0, it.ctx, bar_q );
    tma_load_4d( sQ + kQRegion, &q_map, 64, kvh * group, tok0, it.ctx, bar_q );
    load_k( 0 );
    if ( n_tiles > 1 )
      load_k( 1 );
    load_v( 0 );
  }
  if ( warp == 5 ) {
    asm volatile( "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"( smem_u32( tmem_base_p ) ),
                  "r"( kTmemCols ) );
    asm volatile( "tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" );
  }
  asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
  __syncthreads();
  asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
  const uint32_t tmem_base = *tmem_base_p;
  asm volatile( "griddepcontrol.wait;" ::: "memory" );

  constexpr unsigned kFull = 0xffffffffu;

  if ( warp == 4 ) {
    // =========================== TMA lane: the remaining K/V tiles, as their stages fall free ===========================
    if ( r == 4 * 32 ) {
      // in the order the MMA lane needs them: K(t+2) once S(t) has completed, V(t+1) once P.V(t-1) has
      bool ok = true;
      for ( int t = 0; t < n_tiles && ok; t++ ) {
        if ( t + 2 < n_tiles ) {
          ok = mbar_wait( &bar_kfree[t & 1], ( t >> 1 ) & 1, fail );
          if ( ok )
            load_k( t + 2 );
        }
        if ( ok && t + 1 < n_tiles ) {
          if ( t >= 1 )
            ok = mbar_wait( &bar_vfree[( t + 1 ) & 1], ( ( t - 1 ) >> 1 ) & 1, fail );
          if ( ok )
            load_v( t + 1 );
        }
      }
      if ( !ok )
        *fail = 1;
    }
  } else if ( warp == 5 ) {
    // =========================== MMA lane ===========================
    if ( r == 5 * 32 ) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      // instruction descriptors: fp32 accumulate, A/B format, M = 128; S has N = 64 keys, O has N = 128 dims with V
      // as the MN-major B operand
      const uint32_t idesc_s = ( 1u << 4 ) | ( fmt << 7 ) | ( fmt << 10 ) | ( ( (uint32_t)kKeys >> 3 ) << 17 ) | ( ( 128u >> 4 ) << 24 );
      const uint32_t idesc_pv = ( 1u << 4 ) | ( fmt << 7 ) | ( fmt << 10 ) | ( 1u << 16 ) | ( ( 128u >> 3 ) << 17 ) | ( ( 128u >> 4 ) << 24 );
      // S(t) = Q K_tile^T into S buffer t & 1: 8 MMAs of 16 dims each
      auto issue_s = [&]( int t ) {
        const int b = t & 1;
#pragma unroll
        for ( int k = 0; k < 8; k++ ) {
          const uint64_t da = desc_kmajor( smem_u32( sQ + ( k >> 2 ) * kQRegion + ( k & 3 ) * 32 ) );
          const uint64_t db = desc_kmajor( smem_u32( sK + b * kKTile + ( k >> 2 ) * kKRegion + ( k & 3 ) * 32 ) );
          umma_f16( tmem_base + b * kKeys, da, db, idesc_s, k > 0 ? 1u : 0u );
        }
        umma_commit( &bar_s[b] );
        umma_commit( &bar_kfree[b] );
      };
      bool ok = mbar_wait( bar_q, 0, fail );
      ok = ok && mbar_wait( &bar_k[0], 0, fail );
      if ( ok ) {
        asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
        issue_s( 0 );
      }
      for ( int t = 0; t < n_tiles && ok; t++ ) {
        const int b = t & 1;
        // S of the next tile first, so that the row owners find it ready; its TMEM buffer was read during tile
        // t-1, which bar_p of that tile (waited for below, one iteration ago) covers
        if ( t + 1 < n_tiles ) {
          ok = mbar_wait( &bar_k[b ^ 1], ( ( t + 1 ) >> 1 ) & 1, fail );
          if ( !ok )
            break;
          issue_s( t + 1 );
        }
        ok = mbar_wait( bar_p, t & 1, fail );
        ok = ok && mbar_wait( &bar_v[b], ( t >> 1 ) & 1, fail );
        if ( !ok )
          break;
        asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
#pragma unroll
        for ( int k = 0; k < kKeys / 16; k++ ) { // 16 keys per MMA
          const uint64_t db = desc_mnmajor( smem_u32( sV + b * kKTile + k * 16 * 128 ) );
          umma_f16_ts( tmem_base + 128, tmem_base + b * kKeys + k * 8, db, idesc_pv, ( t > 0 || k > 0 ) ? 1u : 0u );
        }
        umma_commit( bar_pv );
        umma_commit( &bar_vfree[b] );
      }
      if ( !ok )
        *fail = 1;
    }
  } else {
    // =========================== row owners (warps 0..3) ===========================
    const int row_tok = r / group;
    const bool row_live = row_tok < n_tok;
    const int row_limit = row_live ? n_keys - ( n_tok - 1 - row_tok ) : 0; // keys seen by this row's token
    const float scale_log2 = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
    const uint32_t lane_off = static_cast<uint32_t>( warp * 32 ) << 16; // this warp's quarter of the TMEM lanes
    const uint32_t tmem_s = tmem_base + lane_off;                       // + 64 for the second buffer
    const uint32_t tmem_o = tmem_base + lane_off + 128;

    float m = -INFINITY; // the maximum the row's exponentials are taken against (log2 units); may lag the true one
    float l = 0.f;       // row sum of P
    bool ok = true;
#pragma unroll 1
    for ( int t = 0; t < n_tiles; t++ ) {
      const int b = t & 1;
      const uint32_t ph = ( t >> 1 ) & 1;
      ok = __all_sync( kFull, mbar_wait( &bar_s[b], ph, fail ) );
      if ( !ok )
        break;
      asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );

      // ---- scores of this thread's row; tcgen05.ld is warp-wide, so whether to load a column block is decided per
      //      warp
      const int lim = row_limit - t * kKeys; // keys of this tile the row sees
      const int warp_lim = __reduce_max_sync( kFull, lim );
      const bool full_tile = __all_sync( kFull, lim >= kKeys );
      float sc[64];
      if ( warp_lim > 0 ) {
        tmem_ld64( tmem_s + b * kKeys, sc );
      } else {
#pragma unroll
        for ( int j = 0; j < 64; j++ )
          sc[j] = 0.f;
      }
      float tmax = -INFINITY;
      if ( full_tile ) {
        // four chains of eight three-input maxima each instead of one chain of 32: the row owners have only two
        // warps per scheduler to hide a chain's latency behind
        float t4[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };
#pragma unroll
        for ( int j = 0; j < 32; j++ )
          t4[j & 3] = max3( t4[j & 3], sc[j], sc[32 + j] );
        tmax = fmaxf( max3( t4[0], t4[1], t4[2] ), t4[3] );
      } else {
#pragma unroll
        for ( int j = 0; j < 32; j++ ) {
          tmax = fmaxf( tmax, j < lim ? sc[j] : -INFINITY );
          tmax = fmaxf( tmax, 32 + j < lim ? sc[32 + j] : -INFINITY );
        }
      }
      // raise m only when some row of the warp has outgrown it by more than 2^kGrowLog2: then every row of the warp
      // adopts its true maximum and O is rescaled below
      const float m_new = fmaxf( m, tmax * scale_log2 );
      const bool warp_grow = __any_sync( kFull, m_new > m + kGrowLog2 );
      float f = 1.f;
      if ( warp_grow ) {
        if ( m_new > m )
          f = fast_exp2( m - m_new ); // 0 for a row that had seen nothing
        m = m_new;
        l *= f;
      }
      const float neg_m = ( m == -INFINITY ) ? 0.f : -m; // a row that sees nothing carries zeros, not NaNs
      uint32_t pk[32];
      if ( full_tile ) {
        const unsigned long long scale2 = pack_f2( scale_log2, scale_log2 ), shift2 = pack_f2( neg_m, neg_m );
        unsigned long long l2 = pack_f2( 0.f, 0.f );
#pragma unroll
        for ( int j = 0; j < 32; j += 2 ) {
          float xa0, xa1, xb0, xb1;
          unpack_f2( fma_f2( pack_f2( sc[j], sc[j + 1] ), scale2, shift2 ), xa0, xa1 );
          unpack_f2( fma_f2( pack_f2( sc[32 + j], sc[33 + j] ), scale2, shift2 ), xb0, xb1 );
          const float a0 = fast_exp2( xa0 ), a1 = fast_exp2( xa1 ), b0 = fast_exp2( xb0 ), b1 = fast_exp2( xb1 );
          l2 = add_f2( l2, add_f2( pack_f2( a0, a1 ), pack_f2( b0, b1 ) ) );
          pk[j >> 1] = pack2<T>( a0, a1 );
          pk[16 + ( j >> 1 )] = pack2<T>( b0, b1 );
        }
        float l_lo, l_hi;
        unpack_f2( l2, l_lo, l_hi );
        l += l_lo + l_hi;
      } else {
#pragma unroll
        for ( int j = 0; j < 32; j += 2 ) {
          const float a0 = j < lim ? fast_exp2( fmaf( sc[j], scale_log2, neg_m ) ) : 0.f;
          const float a1 = j + 1 < lim ? fast_exp2( fmaf( sc[j + 1], scale_log2, neg_m ) ) : 0.f;
          const float b0 = 32 + j < lim ? fast_exp2( fmaf( sc[32 + j], scale_log2, neg_m ) ) : 0.f;
          const float b1 = 33 + j < lim ? fast_exp2( fmaf( sc[33 + j], scale_log2, neg_m ) ) : 0.f;
          l += ( a0 + a1 ) + ( b0 + b1 );
          pk[j >> 1] = pack2<T>( a0, a1 );
          pk[16 + ( j >> 1 )] = pack2<T>( b0, b1 );
        }
      }

      // ---- O may be rescaled once the previous tile's P.V has completed
      if ( t > 0 && warp_grow ) {
        ok = __all_sync( kFull, mbar_wait( bar_pv, ( t - 1 ) & 1, fail ) );
        if ( !ok )
          break;
        asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
#pragma unroll 1
        for ( int cb = 0; cb < 4; cb++ ) {
          float o[32];
          tmem_ld32( tmem_o + cb * 32, o );
#pragma unroll
          for ( int j = 0; j < 32; j++ )
            o[j] *= f;
          tmem_st32( tmem_o + cb * 32, o );
        }
      }
      // ---- P replaces S in tensor memory: 64 keys of 16 bits = the first 32 columns of this tile's S buffer, from
      //      where the P.V MMAs take it as their A operand.  (Tile 0 has nothing to rescale: its first MMA
      //      overwrites O.)
      tmem_st32_bits( tmem_s + b * kKeys, pk );
      // V rows past the last key hold stale or foreign data: clear them so that 0 * garbage cannot make a NaN
      const int live = min( kKeys, n_keys - t * kKeys ); // keys of this tile that exist at all
      if ( live < kKeys ) {
        ok = __all_sync( kFull, mbar_wait( &bar_v[b], ph, fail ) );
        if ( !ok )
          break;
        if ( r >= live && r < kKeys ) {
          uint8_t* v0 = sV + b * kKTile + r * 128;
#pragma unroll
          for ( int ch = 0; ch < 8; ch++ ) {
            *reinterpret_cast<uint4*>( v0 + ch * 16 ) = make_uint4( 0, 0, 0, 0 );
            *reinterpret_cast<uint4*>( v0 + kKRegion + ch * 16 ) = make_uint4( 0, 0, 0, 0 );
          }
        }
      }
      asm volatile( "fence.proxy.async.shared::cta;" ::: "memory" ); // the cleared V rows -> tensor-core proxy
      asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
      asm volatile( "mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"( smem_u32( bar_p ) ) : "memory" );
    }

    // ---- epilogue: O / l -> xb
    if ( ok )
      ok = __all_sync( kFull, mbar_wait( bar_pv, ( n_tiles - 1 ) & 1, fail ) );
    if ( ok ) {
      asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
      // O / l goes through the Q block's shared memory (free since the last S completed), in the same row-major
      // swizzled layout, and leaves by TMA: rows of tokens past the chunk's end are clipped by the tensor map
      const float inv = row_live ? 1.0f / l : 0.f;
#pragma unroll 1
      for ( int half = 0; half < 2; half++ ) { // 64 dims = one swizzled region of the staging buffer
        float v[64];
        tmem_ld64( tmem_o + half * 64, v );
#pragma unroll
        for ( int ch = 0; ch < 8; ch++ ) { // 16-byte chunks of the row
          uint32_t w[4];
#pragma unroll
          for ( int j = 0; j < 4; j++ )
            w[j] = pack2<T>( v[ch * 8 + 2 * j] * inv, v[ch * 8 + 2 * j + 1] * inv );
          *reinterpret_cast<uint4*>( sQ + half * kQRegion + r * 128 + ( ( ch ^ ( r & 7 ) ) << 4 ) )
            = make_uint4( w[0], w[1], w[2], w[3] );
        }
      }
      asm volatile( "fence.proxy.async.shared::cta;" ::: "memory" );
      asm volatile( "bar.sync 1, %0;" ::"n"( kRows ) : "memory" ); // the four row-owner warps only
      if ( r == 0 ) {
        tma_store_4d( &xb_map, 0, kvh * group, tok0, it.ctx, sQ );
        tma_store_4d( &xb_map, 64, kvh * group, tok0, it.ctx, sQ + kQRegion );
        asm volatile( "cp.async.bulk.commit_group;" ::: "memory" );
        asm volatile( "cp.async.bulk.wait_group.read 0;" ::: "memory" ); // shared memory is read out before the block ends
      }
    } else {
      *fail = 1;
    }
  }

  asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
  __syncthreads();
  if ( r == 0 && *fail != 0 )
    atomicOr( a.dev_error, 4u );
  if ( warp == 5 ) {
    __syncwarp();
    asm volatile( "tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"( tmem_base ), "r"( kTmemCols ) );
  }
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
  // two blocks of 112 KiB each need the largest shared-memory carve-out
  if ( e == cudaSuccess )
    e = cudaFuncSetAttribute( prefill_umma_kernel<__half>, cudaFuncAttributePreferredSharedMemoryCarveout,
                              cudaSharedmemCarveoutMaxShared );
  if ( e == cudaSuccess )
    e = cudaFuncSetAttribute( prefill_umma_kernel<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                              cudaSharedmemCarveoutMaxShared );
  return e;
}

cudaError_t launch_prefill_umma( const DecodeArgs& a, const CUtensorMap* kv_map, const CUtensorMap* q_map,
                                 const CUtensorMap* xb_map, cudaStream_t st, uint64_t* launches )
{
  if ( a.n_items == 0 )
    return cudaSuccess;
  cudaLaunchConfig_t cfg {};
  cfg.gridDim = dim3( a.n_items * a.sh.n_kv_heads );
  cfg.blockDim = dim3( kThreads );
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if ( a.dtype == DT_F16 )
    e = cudaLaunchKernelEx( &cfg, prefill_umma_kernel<__half>, a, *kv_map, *q_map, *xb_map );
  else if ( a.dtype == DT_BF16 )
    e = cudaLaunchKernelEx( &cfg, prefill_umma_kernel<__nv_bfloat16>, a, *kv_map, *q_map, *xb_map );
  else
    return cudaErrorInvalidValue;
  ( *launches )++;
  return e;
}

} // namespace gh

