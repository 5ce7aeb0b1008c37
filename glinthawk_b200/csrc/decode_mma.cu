// Fused ragged-batch decode attention for 16-bit KV with head size 128: TMA-staged K/V tiles, warp-level
// tensor-core products with fp32 accumulation, online softmax, GQA sharing, split-K with a warp-level merge inside a
// block and, across the blocks of a cut context, a merge by whichever of them finishes last.
//
// One launch per layer-step replaces, for the whole batch, the reference's per-context cuBLAS QK^T call, four
// softmax kernels and cuBLAS AV call (src/arch/cuda/llama2/ops.cuh:272-411) and the `att` score matrix between
// them.  The arithmetic it must agree with is the amd64 backend's (src/arch/amd64/llama2/ops.hh:170-298).
//
// Decomposition.  A work item is a run of tokens [t_begin, t_end) of one context (t_begin a multiple of the
// 64-token tile); one thread block handles one (work item, kv head), so all query heads of a GQA group share
// every K/V byte that is fetched.  A block is NW consumer warps + 1 producer warp (NW = 2 by default):
//   * The producer's elected lane walks the item tile by tile (a tile is 16*NW tokens) and issues four TMA tile
//     loads per 32 tokens (K dims 0-63, K dims 64-127, V dims 0-63, V dims 64-127; each a [32 tokens x 128 B] box,
//     128-byte swizzle) into a ring of shared-memory stages, completion signalled on an mbarrier per stage.  The KV arena is ONE
//     2-D tensor [rows][2*kv_dim], so a context/layer/token is just a row coordinate.  No multicast: every block
//     fetches its own tiles.
//   * Consumer warp w owns tokens 16w..16w+15 of every tile: S = Q K^T with mma.m16n8k16 (query heads of the group
//     are the M rows, padded to 16), online softmax in the log2 domain with quad shuffles, O += P V with the
//     probabilities re-used from registers.  The warps keep independent (m, l, O) states that are combined
//     through shared memory at the end ("warp-level merge"); the blocks of a context cut into several items leave
//     partial records and count their arrivals, and the last one to arrive combines the records (gh_merge.cuh).
// The path is HBM-bound: 512 B of K+V per (token, kv head) against 2 x 16 x 128 x 2 tensor flops.
//
// Every wait on an mbarrier is bounded; when a bound is hit the kernel raises a sticky error word and leaves.
#include "gh_kernels.cuh"
#include "gh_merge.cuh"

namespace gh {

namespace {

constexpr int kHS = 128;
constexpr int kPlanTile = 64; // work items start on multiples of this many tokens
constexpr int kBoxRows = 32;  // token rows per TMA box (every variant's tile is a multiple)
constexpr uint32_t kWaitLimit = 1u << 22;

// Compile-time geometry of one kernel variant: NW consumer warps (each owns 16 tokens of a tile), ST ring stages,
// MINB thread blocks per SM the register budget is sized for.
template<int NW, int ST, int MINB>
struct Geo
{
  static constexpr int kConsumerWarps = NW;
  static constexpr int kTile = NW * 16;               // tokens per stage
  static constexpr int kConsumers = NW * 32;
  static constexpr int kThreads = kConsumers + 32;    // + producer warp
  static constexpr int kBoxBytes = kTile * 128;       // one [kTile tokens x 64 elements] box
  static constexpr int kStageBytes = 4 * kBoxBytes;   // K lo, K hi, V lo, V hi
  static constexpr int kStages = ST;
  static constexpr int kSmemBytes = ST * kStageBytes + 1024; // + slack to align the ring to 1024 B
  static constexpr int kMinBlocks = MINB;
};

__device__ __forceinline__ uint32_t smem_u32( const void* p )
{
  return static_cast<uint32_t>( __cvta_generic_to_shared( p ) );
}

__device__ __forceinline__ void mbar_init( uint64_t* bar, uint32_t count )
{
  asm volatile( "mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"( smem_u32( bar ) ), "r"( count ) );
}

__device__ __forceinline__ void mbar_expect_tx( uint64_t* bar, uint32_t bytes )
{
  asm volatile( "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"( smem_u32( bar ) ), "r"( bytes )
                : "memory" );
}

__device__ __forceinline__ void mbar_arrive( uint64_t* bar )
{
  asm volatile( "mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"( smem_u32( bar ) ) : "memory" );
}

// Bounded wait: false when the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait( uint64_t* bar, uint32_t parity )
{
  const uint32_t addr = smem_u32( bar );
  for ( uint32_t it = 0; it < kWaitLimit; it++ ) {
    uint32_t done;
    asm volatile( "{\n"
                  ".reg .pred p;\n"
                  "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                  "selp.u32 %0, 1, 0, p;\n"
                  "}\n"
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

__device__ __forceinline__ void ldmatrix_x4( uint32_t ( &r )[4], uint32_t addr )
{
  asm volatile( "ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                : "=r"( r[0] ), "=r"( r[1] ), "=r"( r[2] ), "=r"( r[3] )
                : "r"( addr ) );
}

__device__ __forceinline__ void ldmatrix_x4_trans( uint32_t ( &r )[4], uint32_t addr )
{
  asm volatile( "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                : "=r"( r[0] ), "=r"( r[1] ), "=r"( r[2] ), "=r"( r[3] )
                : "r"( addr ) );
}

template<typename T>
__device__ __forceinline__ void mma_16816( float ( &c )[4], const uint32_t ( &a )[4], uint32_t b0, uint32_t b1 );

template<>
__device__ __forceinline__ void mma_16816<__half>( float ( &c )[4], const uint32_t ( &a )[4], uint32_t b0, uint32_t b1 )
{
  asm volatile( "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+f"( c[0] ), "+f"( c[1] ), "+f"( c[2] ), "+f"( c[3] )
                : "r"( a[0] ), "r"( a[1] ), "r"( a[2] ), "r"( a[3] ), "r"( b0 ), "r"( b1 ) );
}

template<>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>( float ( &c )[4],
                                                          const uint32_t ( &a )[4],
                                                          uint32_t b0,
                                                          uint32_t b1 )
{
  asm volatile( "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+f"( c[0] ), "+f"( c[1] ), "+f"( c[2] ), "+f"( c[3] )
                : "r"( a[0] ), "r"( a[1] ), "r"( a[2] ), "r"( a[3] ), "r"( b0 ), "r"( b1 ) );
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

// G16: the group has more than 8 query heads, so rows 8..15 of the M=16 tile are live too.
//
// CHUNK: prefill-chunk mode.  The 16 rows of the tile are (token, head) pairs of 16/group consecutive prompt tokens
// of one context instead of up to 16 heads of one token, so the tokens of a group share every K/V fetch.  A work
// item is then (context, token group): `split` is the group's index, t_end the prefix length of the group's last
// token; row r attends causally over the prefix of ITS token, which is shorter by (last token - its token).
template<typename T, bool G16, typename G, bool CHUNK>
__global__ void __launch_bounds__( G::kThreads, G::kMinBlocks )
  decode_mma_kernel( const DecodeArgs a, const __grid_constant__ CUtensorMap kv_map )
{
  constexpr bool ROWS16 = G16 || CHUNK;
  constexpr int kTile = G::kTile, kConsumerWarps = G::kConsumerWarps, kConsumers = G::kConsumers;
  constexpr int kBoxBytes = G::kBoxBytes, kStageBytes = G::kStageBytes, kStages = G::kStages;
  // The kernel behind this one in the stream may be placed on the SMs once every block of this launch has started
  // (so it never takes a block slot from this launch); if it is one of this library's kernels it waits there for this
  // launch to complete, unless the caller declared the two independent.
  if ( a.trigger_early )
    asm volatile( "griddepcontrol.launch_dependents;" ::: "memory" );
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kStages];
  __shared__ uint64_t bar_empty[kStages];
  __shared__ float sm_wm[kConsumerWarps][16];
  __shared__ float sm_wl[kConsumerWarps][16];
  __shared__ float sm_m[16];
  __shared__ float sm_l[16];

  uint8_t* ring = reinterpret_cast<uint8_t*>( ( reinterpret_cast<uintptr_t>( smem_raw ) + 1023 ) & ~uintptr_t( 1023 ) );

  const Shape& sh = a.sh;
  const int item_idx = blockIdx.x / sh.n_kv_heads;
  const int kvh = blockIdx.x - item_idx * sh.n_kv_heads;
  const WorkItem it = a.items[item_idx];
  const CtxMeta c = a.ctx[it.ctx];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = ( it.t_end - it.t_begin + kTile - 1 ) / kTile;

  if ( threadIdx.x == 0 ) {
    for ( int s = 0; s < kStages; s++ ) {
      mbar_init( &bar_full[s], 1 );
      mbar_init( &bar_empty[s], kConsumerWarps );
    }
    asm volatile( "fence.mbarrier_init.release.cluster;" ::: "memory" );
  }
  __syncthreads();

  if ( warp == kConsumerWarps ) {
    // ---------------- producer ----------------
    if ( lane == 0 ) {
      asm volatile( "prefetch.tensormap [%0];" ::"l"( reinterpret_cast<uint64_t>( &kv_map ) ) : "memory" );
      // Launched as a programmatic dependent of the kernel before it in the stream (normally the append kernel), so
      // this block may be running while that kernel still is.  In a decode step that kernel writes one row of the
      // context, the one at the context's position; every row before it was written at least one step earlier.  The
      // tiles that end before that row are therefore fetched without waiting for that kernel: the stream of old rows
      // starts while the append (and the tail of the launch before it) still runs.  The wait comes before the first
      // tile that reaches the new row, and before anything in chunk mode, where that kernel wrote the whole chunk.
      const size_t row_bytes = (size_t)sh.row_elems * sizeof( T );
      const int row0 = static_cast<int>( ( c.kv_off + a.layer_off ) / (long long)row_bytes ) + it.t_begin;
      const int xk = kvh * kHS;
      const int xv = (int)sh.kv_dim + kvh * kHS;
      bool waited = false;
      if ( CHUNK || a.stream_old_rows_early == 0 ) {
        asm volatile( "griddepcontrol.wait;" ::: "memory" );
        waited = true;
      }
      for ( int t = 0; t < n_tiles; t++ ) {
        const int s = t % kStages;
        if ( t >= kStages && !mbar_wait( &bar_empty[s], ( ( t / kStages ) - 1 ) & 1 ) ) {
          atomicOr( a.dev_error, 1u );
          break;
        }
        if ( !waited && it.t_begin + ( t + 1 ) * kTile > (int)c.pos ) {
          asm volatile( "griddepcontrol.wait;" ::: "memory" );
          waited = true;
        }
        uint8_t* st = ring + s * kStageBytes;
        mbar_expect_tx( &bar_full[s], kStageBytes );
        const int y = row0 + t * kTile;
#pragma unroll
        for ( int j = 0; j < kTile / kBoxRows; j++ ) { // the descriptor's box is kBoxRows tokens x 128 B
          uint8_t* sub = st + j * kBoxRows * 128;
          tma_load_2d( sub + 0 * kBoxBytes, &kv_map, xk, y + j * kBoxRows, &bar_full[s] );
          tma_load_2d( sub + 1 * kBoxBytes, &kv_map, xk + 64, y + j * kBoxRows, &bar_full[s] );
          tma_load_2d( sub + 2 * kBoxBytes, &kv_map, xv, y + j * kBoxRows, &bar_full[s] );
          tma_load_2d( sub + 3 * kBoxBytes, &kv_map, xv + 64, y + j * kBoxRows, &bar_full[s] );
        }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int quad_row = lane >> 2;       // row of the M=16 tile this thread holds (and row + 8)
  const int quad_col = ( lane & 3 ) * 2; // first of its two columns inside an 8-wide tile
  const int group = sh.group;
  const float scale_log2 = 0.08838834764831845f * 1.4426950408889634f; // 1/sqrt(128) * log2(e)

  // Q fragments (A operand), 8 k-steps of 16 dims; rows that stand for no (token, head) are zero.
  uint32_t qf[8][4];
  // chunk mode: which prompt token and head each of this thread's two rows stands for
  const int tok_per_item = CHUNK ? 16 / group : 1;
  const int tok0 = CHUNK ? it.split * tok_per_item : 0;                          // first token of the group
  const int n_tok = CHUNK ? min( tok_per_item, (int)a.chunk_tokens - tok0 ) : 1; // tokens the group really has
  const int row_tok[2] = { CHUNK ? quad_row / group : 0, CHUNK ? ( quad_row + 8 ) / group : 0 };
  const int row_head[2] = { CHUNK ? quad_row % group : quad_row, CHUNK ? ( quad_row + 8 ) % group : quad_row + 8 };
  // tokens by which a row's prefix is shorter than the item's (the last token's) prefix
  const int row_short[2] = { CHUNK ? max( 0, n_tok - 1 - row_tok[0] ) : 0, CHUNK ? max( 0, n_tok - 1 - row_tok[1] ) : 0 };
  asm volatile( "griddepcontrol.wait;" ::: "memory" ); // q was rotated by the kernel before this one
  {
    const size_t q_ctx_row = CHUNK ? (size_t)it.ctx * a.chunk_tokens + tok0 : (size_t)it.ctx;
    const T* qbase = static_cast<const T*>( a.q ) + q_ctx_row * sh.n_heads * kHS + (size_t)kvh * group * kHS;
    const bool live[2] = { CHUNK ? row_tok[0] < n_tok : quad_row < group,
                           CHUNK ? row_tok[1] < n_tok : ( G16 && quad_row + 8 < group ) };
    const T* rowp[2] = { qbase + ( (size_t)row_tok[0] * sh.n_heads + row_head[0] ) * kHS,
                         qbase + ( (size_t)row_tok[1] * sh.n_heads + row_head[1] ) * kHS };
#pragma unroll
    for ( int ks = 0; ks < 8; ks++ ) {
      const int d = ks * 16 + quad_col;
      qf[ks][0] = live[0] ? *reinterpret_cast<const uint32_t*>( rowp[0] + d ) : 0u;
      qf[ks][2] = live[0] ? *reinterpret_cast<const uint32_t*>( rowp[0] + d + 8 ) : 0u;
      qf[ks][1] = live[1] ? *reinterpret_cast<const uint32_t*>( rowp[1] + d ) : 0u;
      qf[ks][3] = live[1] ? *reinterpret_cast<const uint32_t*>( rowp[1] + d + 8 ) : 0u;
    }
  }

  float o[16][4];
#pragma unroll
  for ( int n = 0; n < 16; n++ )
    o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = { -INFINITY, -INFINITY };
  float l_run[2] = { 0.f, 0.f };

  // ldmatrix lane addressing (see the header comment): matrix index lane/8, row lane%8
  const int lm = lane >> 3, lr = lane & 7;
  const int k_tok = warp * 16 + ( lm >> 1 ) * 8 + lr; // K: matrices 0,1 -> tokens 0-7, matrices 2,3 -> tokens 8-15
  const int k_chunk_sel = lm & 1;                     //    matrices 0,2 -> dims +0..7, 1,3 -> dims +8..15
  const int v_tok = warp * 16 + ( lm & 1 ) * 8 + lr;  // V: matrices 0,2 -> tokens 0-7, 1,3 -> tokens 8-15
  const int v_chunk_sel = lm >> 1;                    //    matrices 0,1 -> dims +0..7, 2,3 -> dims +8..15

  // Whether some block has already given up on a wait: read here, where the load's latency hides behind the first
  // tile's, and used after the loop.
  const uint32_t seen_error = threadIdx.x == 0 ? *reinterpret_cast<volatile uint32_t*>( a.dev_error ) : 0u;
  bool ok = true;
  for ( int t = 0; t < n_tiles; t++ ) {
    const int s = t % kStages;
    // every lane waits (each needs the acquire); the verdict is made warp-uniform before branching on it
    if ( !__all_sync( 0xffffffffu, mbar_wait( &bar_full[s], ( t / kStages ) & 1 ) ) ) {
      if ( lane == 0 )
        atomicOr( a.dev_error, 2u );
      ok = false;
      break;
    }
    const uint32_t st = smem_u32( ring + s * kStageBytes );
    const int remaining = it.t_end - it.t_begin - t * kTile; // tokens of the item from this tile's start on
    const int valid = min( kTile, remaining );               // live tokens in this tile
    const int w0 = warp * 16;

    if ( w0 < valid ) {
      if ( valid < w0 + 16 ) {
        // Ragged end: rows past the context's last token hold whatever the slot had before.  Their scores are
        // masked below; their V rows are cleared here so that 0 * garbage cannot produce a NaN.
        for ( int e = lane; e < 16 * 16; e += 32 ) {
          const int row = w0 + ( e >> 4 ), ch = e & 15;
          if ( row >= valid ) {
            uint8_t* p = ring + s * kStageBytes + ( 2 + ( ch >> 3 ) ) * kBoxBytes + row * 128 + ( ch & 7 ) * 16;
            *reinterpret_cast<uint4*>( p ) = make_uint4( 0, 0, 0, 0 );
          }
        }
        __syncwarp();
      }

      // ---- S = Q K^T for this warp's 16 tokens: two 16x8 accumulator tiles
      float sacc[2][4] = { { 0.f, 0.f, 0.f, 0.f }, { 0.f, 0.f, 0.f, 0.f } };
#pragma unroll
      for ( int ks = 0; ks < 8; ks++ ) {
        const int chunk = ( ( ks & 3 ) * 2 + k_chunk_sel ) ^ ( k_tok & 7 );
        uint32_t b[4];
        ldmatrix_x4( b, st + ( ks >> 2 ) * kBoxBytes + k_tok * 128 + chunk * 16 );
        mma_16816<T>( sacc[0], qf[ks], b[0], b[1] );
        mma_16816<T>( sacc[1], qf[ks], b[2], b[3] );
      }

      // ---- online softmax (log2 domain).  Thread holds, for row quad_row (and +8): columns quad_col, +1 of
      // each 8-token tile.
      float p[2][4];
#pragma unroll
      for ( int half = 0; half < ( ROWS16 ? 2 : 1 ); half++ ) {
        const int lim = remaining - row_short[half]; // this row's own causal limit, counted from the tile's start
        float sv[4];
#pragma unroll
        for ( int nt = 0; nt < 2; nt++ )
#pragma unroll
          for ( int j = 0; j < 2; j++ ) {
            const int tok = w0 + nt * 8 + quad_col + j;
            const float v = sacc[nt][half * 2 + j] * scale_log2;
            sv[nt * 2 + j] = tok < lim ? v : -INFINITY;
          }
        float mx = fmaxf( fmaxf( sv[0], sv[1] ), fmaxf( sv[2], sv[3] ) );
        mx = fmaxf( mx, __shfl_xor_sync( 0xffffffffu, mx, 1 ) );
        mx = fmaxf( mx, __shfl_xor_sync( 0xffffffffu, mx, 2 ) );
        const float m_new = fmaxf( m_run[half], mx );
        // In chunk mode a row can have no visible token among THIS warp's 16 (its prefix ends earlier): keep the
        // exponent arguments finite so that such a row carries zeros, not NaNs, until the warps are combined.
        const float m_use = ( CHUNK && m_new == -INFINITY ) ? 0.f : m_new;
        const float corr = fast_exp2( m_run[half] - m_use );
        float psum = 0.f;
#pragma unroll
        for ( int e = 0; e < 4; e++ ) {
          const float pe = fast_exp2( sv[e] - m_use );
          p[half][e] = pe;
          psum += pe;
        }
        l_run[half] = l_run[half] * corr + psum;
        m_run[half] = m_new;
        if ( __any_sync( 0xffffffffu, corr != 1.0f ) ) {
#pragma unroll
          for ( int n = 0; n < 16; n++ ) {
            o[n][half * 2 + 0] *= corr;
            o[n][half * 2 + 1] *= corr;
          }
        }
      }
      uint32_t pf[4];
      pf[0] = pack2<T>( p[0][0], p[0][1] );
      pf[2] = pack2<T>( p[0][2], p[0][3] );
      pf[1] = ROWS16 ? pack2<T>( p[1][0], p[1][1] ) : 0u;
      pf[3] = ROWS16 ? pack2<T>( p[1][2], p[1][3] ) : 0u;

      // ---- O += P V
#pragma unroll
      for ( int dp = 0; dp < 8; dp++ ) {
        const int chunk = ( ( dp & 3 ) * 2 + v_chunk_sel ) ^ ( v_tok & 7 );
        uint32_t b[4];
        ldmatrix_x4_trans( b, st + ( 2 + ( dp >> 2 ) ) * kBoxBytes + v_tok * 128 + chunk * 16 );
        mma_16816<T>( o[2 * dp], pf, b[0], b[1] );
        mma_16816<T>( o[2 * dp + 1], pf, b[2], b[3] );
      }
    }

    if ( valid < kTile )
      asm volatile( "fence.proxy.async.shared::cta;" ::: "memory" );
    __syncwarp();
    if ( lane == 0 )
      mbar_arrive( &bar_empty[s] );
  }

  // ---- combine the warps' states through shared memory (the ring is free once every warp is here)
  // The consumers meet at two more barriers below, so they must all stay or all leave: the barrier itself ORs every
  // thread's verdict (its own waits and, for one thread, the error word as it was when the block started) into one
  // that is the same for the whole block.
  uint32_t bad = ok ? 0u : 1u;
  if ( seen_error != 0 )
    bad = 1u;
  asm volatile( "{\n"
                ".reg .pred p, q;\n"
                "setp.ne.u32 p, %0, 0;\n"
                "barrier.cta.red.or.pred q, 1, %1, p;\n"
                "selp.u32 %0, 1, 0, q;\n"
                "}\n"
                : "+r"( bad )
                : "n"( kConsumers )
                : "memory" );
  if ( bad ) {
    // A wait ran out somewhere in this block or another: give any copy still in flight time to land, then leave.
    __nanosleep( 1000000 );
    return;
  }
  constexpr int kRows = ROWS16 ? 16 : 8;
  static_assert( ( kConsumerWarps + 1 ) * kRows * kHS * 4 <= kStages * kStageBytes, "merge scratch must fit the ring" );
  float* sm_wo = reinterpret_cast<float*>( ring );                 // [warp][kRows][128]
  float* sm_o = sm_wo + kConsumerWarps * kRows * kHS;               // [kRows][128] merged
#pragma unroll
  for ( int half = 0; half < ( ROWS16 ? 2 : 1 ); half++ ) {
    float l = l_run[half];
    l += __shfl_xor_sync( 0xffffffffu, l, 1 );
    l += __shfl_xor_sync( 0xffffffffu, l, 2 );
    const int row = quad_row + half * 8;
    if ( ( lane & 3 ) == 0 ) {
      sm_wm[warp][row] = m_run[half];
      sm_wl[warp][row] = l;
    }
#pragma unroll
    for ( int n = 0; n < 16; n++ )
      *reinterpret_cast<float2*>( &sm_wo[( warp * kRows + row ) * kHS + n * 8 + quad_col] )
        = make_float2( o[n][half * 2], o[n][half * 2 + 1] );
  }
  asm volatile( "bar.sync 1, %0;" ::"n"( kConsumers ) : "memory" );

  const int live_rows = CHUNK ? n_tok * group : group;
  for ( int d = threadIdx.x; d < kHS; d += kConsumers ) {
    for ( int r = 0; r < live_rows; r++ ) {
      float M = -INFINITY;
#pragma unroll
      for ( int w = 0; w < kConsumerWarps; w++ )
        M = fmaxf( M, sm_wm[w][r] );
      float L = 0.f, O = 0.f;
#pragma unroll
      for ( int w = 0; w < kConsumerWarps; w++ ) {
        const float wgt = fast_exp2( sm_wm[w][r] - M );
        L += wgt * sm_wl[w][r];
        O += wgt * sm_wo[( w * kRows + r ) * kHS + d];
      }
      sm_o[r * kHS + d] = O;
      if ( d == 0 ) {
        sm_m[r] = M;
        sm_l[r] = L;
      }
    }
  }
  asm volatile( "bar.sync 1, %0;" ::"n"( kConsumers ) : "memory" );

  if constexpr ( CHUNK ) {
    // row r = (token r / group, head r % group) of the group; a chunk item is never cut, so this is the result
    T* out = static_cast<T*>( a.xb ) + ( (size_t)it.ctx * a.chunk_tokens + tok0 ) * sh.n_heads * kHS + (size_t)kvh * group * kHS;
    for ( int e = threadIdx.x; e < live_rows * kHS; e += kConsumers ) {
      const int r = e / kHS, d = e - r * kHS;
      out[( (size_t)( r / group ) * sh.n_heads + ( r % group ) ) * kHS + d] = Conv<T>::from_f32( sm_o[e] / sm_l[r] );
    }
  } else {
    store_item<T, kHS>( sh, c, it, kvh * group, group, sm_o, sm_m, sm_l, static_cast<T*>( a.xb ), a.part_o, a.part_ml,
                   threadIdx.x, kConsumers );
#ifndef GH_DECODE_MERGE_KERNEL // (defined only in comparison builds: the records then go to merge_partials_kernel)
    if ( c.nsplits > 1 ) {
      // This block left a partial record.  Count it; whichever block of the (context, kv head) arrives last finds
      // every record of the context in memory and combines them.  No block waits for another.
      __threadfence();
      asm volatile( "bar.sync 1, %0;" ::"n"( kConsumers ) : "memory" );
      int* sm_last = reinterpret_cast<int*>( &sm_wm[0][0] ); // (the warps' states were consumed above)
      if ( threadIdx.x == 0 ) {
        uint32_t* count = a.arrivals + (size_t)it.ctx * sh.n_kv_heads + kvh;
        const bool last = atomicAdd( count, 1u ) + 1u == (uint32_t)c.nsplits;
        if ( last )
          *count = 0; // nobody else touches it in this launch: it is zero again for the next one
        *sm_last = last ? 1 : 0;
      }
      asm volatile( "bar.sync 1, %0;" ::"n"( kConsumers ) : "memory" );
      if ( *sm_last != 0 ) {
        __threadfence();
        static_assert( 16 * ( 2 * kMaxSplits + 1 ) * 4 <= kStages * kStageBytes, "combine scratch must fit the ring" );
        combine_records<T, kHS>( sh, c, it.ctx, kvh * group, group, static_cast<T*>( a.xb ), a.part_o, a.part_ml,
                            reinterpret_cast<float*>( ring ), threadIdx.x, kConsumers );
      }
    }
#endif
  }
}

template<typename T, typename G>
cudaError_t launch_g( const DecodeArgs& a, const CUtensorMap* map, cudaStream_t st )
{
  cudaLaunchConfig_t cfg {};
  cfg.gridDim = dim3( a.n_items * a.sh.n_kv_heads );
  cfg.blockDim = dim3( G::kThreads );
  cfg.dynamicSmemBytes = G::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization; // start while the previous kernel drains
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if ( a.chunk_tokens > 0 )
    return cudaLaunchKernelEx( &cfg, decode_mma_kernel<T, true, G, true>, a, *map );
  cudaError_t e = a.sh.group > 8 ? cudaLaunchKernelEx( &cfg, decode_mma_kernel<T, true, G, false>, a, *map )
                                 : cudaLaunchKernelEx( &cfg, decode_mma_kernel<T, false, G, false>, a, *map );
#ifdef GH_DECODE_MERGE_KERNEL
  if ( e == cudaSuccess && a.n_split_ctx > 0 )
    e = launch_merge_partials<T>( a.sh, a.ctx, a.split_ctx, a.n_split_ctx, a.part_o, a.part_ml, static_cast<T*>( a.xb ), st );
#endif
  return e;
}

// The geometry that is built: four small blocks per SM overlap one block's fill and drain with three others'
// streaming, the fastest of the geometries measured on B200 (64-token tiles with a 96 KiB ring and two blocks per
// SM, 32-token tiles with 64 KiB and three blocks, and with 96 KiB and two blocks were all slower).
using Geo0 = Geo<2, 3, 4>; // 32-token tiles, 48 KiB ring, 4 blocks per SM

template<typename T>
cudaError_t launch_t( const DecodeArgs& a, const CUtensorMap* map, cudaStream_t st )
{
  return launch_g<T, Geo0>( a, map, st );
}

template<typename T, bool G16, typename G>
cudaError_t allow_smem()
{
  cudaError_t e = cudaFuncSetAttribute( decode_mma_kernel<T, G16, G, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        G::kSmemBytes );
  if ( e == cudaSuccess && G16 )
    e = cudaFuncSetAttribute( decode_mma_kernel<T, true, G, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              G::kSmemBytes );
  return e;
}

template<typename G>
cudaError_t allow_smem_all()
{
  cudaError_t e = allow_smem<__half, false, G>();
  if ( e == cudaSuccess )
    e = allow_smem<__half, true, G>();
  if ( e == cudaSuccess )
    e = allow_smem<__nv_bfloat16, false, G>();
  if ( e == cudaSuccess )
    e = allow_smem<__nv_bfloat16, true, G>();
  return e;
}

} // namespace

uint32_t decode_mma_tile_tokens()
{
  return kPlanTile;
}

uint32_t decode_mma_box_rows()
{
  return kBoxRows;
}

bool decode_mma_supported( const Shape& sh, uint32_t dtype )
{
  return ( dtype == DT_F16 || dtype == DT_BF16 ) && sh.head_size == kHS && sh.group <= 16
         && sh.seq_len % kPlanTile == 0;
}

bool decode_mma_chunk_supported( const Shape& sh )
{
  return sh.group == 1 || sh.group == 2 || sh.group == 4 || sh.group == 8;
}

cudaError_t decode_mma_prepare()
{
  return allow_smem_all<Geo0>();
}

cudaError_t launch_decode_mma( const DecodeArgs& a, const CUtensorMap* kv_map, cudaStream_t st, uint64_t* launches )
{
  if ( a.n_items == 0 )
    return cudaSuccess;
  cudaError_t e;
  switch ( a.dtype ) {
    case DT_F16: e = launch_t<__half>( a, kv_map, st ); break;
    case DT_BF16: e = launch_t<__nv_bfloat16>( a, kv_map, st ); break;
    default: return cudaErrorInvalidValue;
  }
  *launches += 1;
  return e;
}

} // namespace gh
