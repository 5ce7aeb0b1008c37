// The producer of the attention stage fused to it: rmsnorm, the q and kv projections on the 5th-generation tensor
// cores (tcgen05 + TMEM), and RoPE + K/V append from the fp32 sums.
//
// Replaces, per layer-step, the reference's
//   rmsnorm( xb, x, rms_att_weight ); matmul( q, xb, wq ); matmul( kv, xb, wkv );   src/models/llama2/model.hh:326-343
//   copy_kv_cache( token_contexts, kv ); apply_rope( pos, fcr, fci, q, token_contexts )            model.hh:345-360
// (operations: src/arch/amd64/common/ops.hh:141-170, 212-229; src/arch/amd64/llama2/ops.hh:138-164, 300-352).  The
// kv scratch buffer in the storage type disappears: K and V go from the fp32 sums into the slot rows.  Rounding points
// are the reference's: xb, q and kv are rounded to the storage type, the rotation is done in fp32 on those rounded
// values with separately rounded products and rounded once more.
//
// The GEMM is skinny (a decode batch of at most a few hundred rows against [dim + 2 kv_dim] x [dim] weights), so the
// weight stream is what has to be kept flowing and the weights take the MMA's M side:
//   D[128 features x Nb batch rows] += W[128 x 64] . XB[Nb x 64]^T     tcgen05.mma M = 128, N = Nb <= 256, fp32 in TMEM
// Work unit = (tile of 128 output features, block of 64 k).  The units are dealt to the CTAs (one per SM) as equal
// contiguous runs, so a CTA works through the tail of one tile, some whole tiles and the head of another
// ("stream-K"): all SMs stream weights for the same time whatever the number of tiles.  Every piece leaves its fp32
// sums in a workspace slot of its own, and a second, wide kernel adds the pieces of each tile in a fixed order, rounds,
// rotates and stores: no counters, no waiting, the same bits on every run.  (Finishing tiles inside the GEMM kernel,
// by whichever CTA delivered the last piece, was measured first: with only the four read-out warps per SM doing the
// rotation it cost 70 us of tail at 256 rows; the wide kernel costs a few.)
//
// Roles per CTA: warps 0..3 = read-out (thread r owns feature r of the tile = TMEM lane r), one lane of warp 4 = TMA
// producer (ring of W and XB tiles, 4 to 10 stages deep, 128-byte swizzle), one lane of warp 5 = MMA issuer.  Two TMEM
// accumulators so that the next piece is multiplied while the previous one is written out.  Every wait is bounded.
#include <algorithm>
#include <type_traits>

#include "gh_kernels.cuh"
#include "gh_umma.cuh"

namespace gh {

namespace {

using namespace umma;

constexpr int kTileF = 128;                   // output features per tile = MMA M = TMEM lanes
constexpr int kBK = 64;                       // k elements per stage: one 128-byte swizzled row
constexpr int kMaxNb = 256;                   // batch rows per launch = MMA N
constexpr int kATile = kTileF * 128;          // 16 KiB of weights per stage
constexpr int kRing = 4 * ( kATile + kMaxNb * 128 ); // 192 KiB of stages: 4 at 256 batch rows, more when the
constexpr int kMaxStages = 10;                //   activation tile is smaller (a stage is 16 KiB + nb * 128 B)
constexpr int kOffBar = kRing;                // then the barriers: ( 2 * kMaxStages + 6 ) words of 8 bytes
constexpr int kSmemBytes = kOffBar + 256;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;                // two accumulators of up to 256 columns

// One block per row; the row is read once, in 16-byte pieces, and kept in registers between the two passes
// (up to kNormPieces pieces per thread: dim <= 256 * kNormPieces * elements per piece).
constexpr int kNormPieces = 8;

template<typename T>
__global__ void __launch_bounds__( 256 ) rmsnorm_kernel( T* __restrict__ out, const T* __restrict__ x,
                                                          const T* __restrict__ weight, uint32_t dim )
{
  constexpr int N = Vec16<T>::N;
  asm volatile( "griddepcontrol.launch_dependents;" ::: "memory" );
  const T* X = x + (size_t)blockIdx.x * dim;
  T* O = out + (size_t)blockIdx.x * dim;
  const uint32_t pieces = dim / N; // dim is a multiple of 128
  // the norm weights are model weights: nothing in the stream writes them, so they are fetched ahead of the wait
  Vec16<T> wrow[kNormPieces];
#pragma unroll
  for ( int k = 0; k < kNormPieces; k++ ) {
    const uint32_t p = threadIdx.x + k * 256;
    if ( p < pieces )
      wrow[k] = ld16( weight + (size_t)p * N );
  }
  // launched as a programmatic dependent of the kernel before it in the stream (its launch latency hides behind
  // that kernel's tail); x and the scratch row may still be in use until that kernel has completed
  asm volatile( "griddepcontrol.wait;" ::: "memory" );
  Vec16<T> row[kNormPieces];
  float ss = 0.f;
#pragma unroll
  for ( int k = 0; k < kNormPieces; k++ ) {
    const uint32_t p = threadIdx.x + k * 256;
    if ( p < pieces ) {
      row[k] = ld16( X + (size_t)p * N );
#pragma unroll
      for ( int e = 0; e < N; e++ ) {
        const float v = Conv<T>::to_f32( row[k].v[e] );
        ss += v * v;
      }
    }
  }
  __shared__ float part[8];
  ss = warp_sum( ss );
  if ( ( threadIdx.x & 31 ) == 0 )
    part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for ( int w = 0; w < 8; w++ )
    tot += part[w];
  // src/arch/amd64/common/ops.hh:158-161
  tot /= dim;
  tot += 1e-5f;
  tot = 1.0f / sqrtf( tot );
#pragma unroll
  for ( int k = 0; k < kNormPieces; k++ ) {
    const uint32_t p = threadIdx.x + k * 256;
    if ( p < pieces ) {
      Vec16<T> o;
#pragma unroll
      for ( int e = 0; e < N; e++ )
        o.v[e] = Conv<T>::from_f32( __fmul_rn( Conv<T>::to_f32( wrow[k].v[e] ), __fmul_rn( tot, Conv<T>::to_f32( row[k].v[e] ) ) ) );
      st16( O + (size_t)p * N, o );
    }
  }
}

// The run of work units CTA `c` owns, and the pieces (tile, k-block range) it falls into.
struct Piece
{
  int tile, k0, k1; // k-blocks [k0, k1) of the tile
  int seg, nsegs;   // index of this piece among the tile's pieces, and how many there are
};

__host__ __device__ __forceinline__ Piece piece_at( int u, int u_end, int kblocks, int upc )
{
  Piece p;
  p.tile = u / kblocks;
  p.k0 = u - p.tile * kblocks;
  p.k1 = p.k0 + ( u_end - u ) < kblocks ? p.k0 + ( u_end - u ) : kblocks;
  const int first = p.tile * kblocks, last = first + kblocks - 1; // the tile's units; cuts fall on multiples of upc
  p.seg = u / upc - first / upc;
  p.nsegs = last / upc - first / upc + 1;
  return p;
}

template<typename T>
__global__ void __launch_bounds__( kThreads, 1 )
  project_kernel( const ProjectArgs a, const __grid_constant__ CUtensorMap wq_map,
                  const __grid_constant__ CUtensorMap wkv_map, const __grid_constant__ CUtensorMap xb_map )
{
  extern __shared__ __align__( 1024 ) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>( smem + kOffBar );
  uint64_t* bar_full = bars;                    // [stages] tiles of a stage have landed          (TMA -> MMA lane)
  uint64_t* bar_empty = bars + kMaxStages;      // [stages] the MMAs reading a stage have completed (MMA -> TMA lane)
  uint64_t* bar_acc_full = bars + 2 * kMaxStages;     // [2] a piece's accumulator is complete     (MMA -> epilogue)
  uint64_t* bar_acc_free = bars + 2 * kMaxStages + 2; // [2] the accumulator has been read out     (epilogue -> MMA lane)
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>( bars + 2 * kMaxStages + 4 );
  volatile int* fail = reinterpret_cast<volatile int*>( bars + 2 * kMaxStages + 5 );

  const int r = threadIdx.x;
  const int warp = r >> 5;
  if ( ( smem_u32( smem ) & 1023u ) != 0 ) { // the swizzled tiles need a 1024-byte aligned base
    if ( r == 0 )
      atomicOr( a.dev_error, 8u );
    return;
  }
  asm volatile( "griddepcontrol.launch_dependents;" ::: "memory" );

  const int kblocks = a.kblocks, upc = a.units_per_cta;
  const int u_begin = blockIdx.x * upc;
  const int u_end = min( (int)( a.n_tiles * a.kblocks ), u_begin + upc );
  const int nb = a.nb;
  const int stage_bytes = kATile + ( ( nb * 128 + 1023 ) & ~1023 ); // both tiles 1024-byte aligned
  const int n_stages = min( kMaxStages, kRing / stage_bytes );

  if ( r == 0 ) {
    *fail = 0;
    for ( int i = 0; i < 2 * kMaxStages + 2; i++ )
      asm volatile( "mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"( smem_u32( &bars[i] ) ) );
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"( smem_u32( &bar_acc_free[0] ) ), "r"( kTileF ) );
    asm volatile( "mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"( smem_u32( &bar_acc_free[1] ) ), "r"( kTileF ) );
    asm volatile( "fence.mbarrier_init.release.cluster;" ::: "memory" );
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

  constexpr unsigned kFull = 0xffffffffu;

  if ( warp == 4 ) {
    // =========================== TMA lane ===========================
    if ( r == 4 * 32 ) {
      bool ok = true;
      uint32_t n = 0; // stages filled so far
      uint64_t stream_policy;
      asm volatile( "createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"( stream_policy ) );
      // The weights do not depend on the kernel before this one in the stream (rmsnorm): the weight tiles of the first
      // ring of stages are on their way before this lane waits for that kernel, the activation tiles follow after.
      // Nothing else in the block touches anything that kernel or its predecessors write: the other roles only see
      // what these loads bring.
      const int first_units = min( n_stages, u_end - u_begin );
      for ( int pass = 0; pass < 2; pass++ ) {
        if ( pass == 1 )
          asm volatile( "griddepcontrol.wait;" ::: "memory" );
        for ( int i = 0; i < first_units; i++ ) {
          const Piece p = piece_at( u_begin + i, u_end, kblocks, upc );
          uint8_t* sA = smem + i * stage_bytes;
          if ( pass == 0 ) {
            const bool is_q = p.tile < (int)a.q_tiles;
            asm volatile( "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"( smem_u32( &bar_full[i] ) ),
                          "r"( (uint32_t)( kATile + nb * 128 ) )
                          : "memory" );
            tma_load_2d_hint( sA, is_q ? &wq_map : &wkv_map, p.k0 * kBK,
                              ( is_q ? p.tile : p.tile - (int)a.q_tiles ) * kTileF, &bar_full[i], stream_policy );
          } else {
            tma_load_2d( sA + kATile, &xb_map, p.k0 * kBK, (int)a.batch0, &bar_full[i] );
          }
        }
      }
      n = static_cast<uint32_t>( first_units );
      for ( int u = u_begin + first_units; u < u_end && ok; ) {
        const Piece p = piece_at( u, u_end, kblocks, upc );
        const bool is_q = p.tile < (int)a.q_tiles;
        const CUtensorMap* wmap = is_q ? &wq_map : &wkv_map;
        const int wrow = ( is_q ? p.tile : p.tile - (int)a.q_tiles ) * kTileF;
        for ( int kb = p.k0; kb < p.k1 && ok; kb++, n++ ) {
          const int s = n % n_stages;
          if ( n >= (uint32_t)n_stages )
            ok = mbar_wait( &bar_empty[s], ( n / n_stages - 1 ) & 1, fail );
          if ( !ok )
            break;
          uint8_t* sA = smem + s * stage_bytes;
          asm volatile( "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"( smem_u32( &bar_full[s] ) ),
                        "r"( (uint32_t)( kATile + nb * 128 ) )
                        : "memory" );
          tma_load_2d_hint( sA, wmap, kb * kBK, wrow, &bar_full[s], stream_policy ); // read once: do not keep in L2
          tma_load_2d( sA + kATile, &xb_map, kb * kBK, (int)a.batch0, &bar_full[s] ); // rows past the batch arrive as zeros
        }
        u += p.k1 - p.k0;
      }
      if ( !ok )
        *fail = 1;
    }
  } else if ( warp == 5 ) {
    // =========================== MMA lane ===========================
    if ( r == 5 * 32 ) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      // fp32 accumulate, A/B format, both operands K-major, N = nb, M = 128
      const uint32_t idesc = ( 1u << 4 ) | ( fmt << 7 ) | ( fmt << 10 ) | ( ( (uint32_t)nb >> 3 ) << 17 ) | ( ( 128u >> 4 ) << 24 );
      bool ok = true;
      uint32_t n = 0, piece_i = 0;
      for ( int u = u_begin; u < u_end && ok; piece_i++ ) {
        const Piece p = piece_at( u, u_end, kblocks, upc );
        const int ab = piece_i & 1;
        if ( piece_i >= 2 ) { // the accumulator was used two pieces ago: wait until it has been read out
          ok = mbar_wait( &bar_acc_free[ab], ( piece_i / 2 - 1 ) & 1, fail );
          asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
        }
        for ( int kb = p.k0; kb < p.k1 && ok; kb++, n++ ) {
          const int s = n % n_stages;
          ok = mbar_wait( &bar_full[s], ( n / n_stages ) & 1, fail );
          if ( !ok )
            break;
          asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
          const uint32_t sA = smem_u32( smem + s * stage_bytes );
#pragma unroll
          for ( int k = 0; k < kBK / 16; k++ )
            umma_f16( tmem_base + ab * kMaxNb, desc_kmajor( sA + k * 32 ), desc_kmajor( sA + kATile + k * 32 ), idesc,
                      ( kb > p.k0 || k > 0 ) ? 1u : 0u );
          umma_commit( &bar_empty[s] );
        }
        if ( ok )
          umma_commit( &bar_acc_full[ab] );
        u += p.k1 - p.k0;
      }
      if ( !ok )
        *fail = 1;
    }
  } else {
    // =========================== accumulator read-out (warps 0..3): thread r owns feature r of the tile ===========================
    // Every piece leaves its fp32 sums in its own workspace slot, [batch row][feature]; project_finish_kernel adds
    // the pieces of a tile in their fixed order and does the rest.  Nobody counts arrivals or waits for anybody.
    const uint32_t lane_off = static_cast<uint32_t>( warp * 32 ) << 16; // this warp's quarter of the TMEM lanes
    const int batch = a.batch;
    const int n_chunks = ( batch + 31 ) / 32;
    const size_t slot_floats = (size_t)n_chunks * 32 * kTileF;
    bool ok = true;
    uint32_t piece_i = 0;
    for ( int u = u_begin; u < u_end; piece_i++ ) {
      const Piece p = piece_at( u, u_end, kblocks, upc );
      const int ab = piece_i & 1;
      ok = __all_sync( kFull, mbar_wait( &bar_acc_full[ab], ( piece_i / 2 ) & 1, fail ) );
      if ( !ok )
        break;
      asm volatile( "tcgen05.fence::after_thread_sync;" ::: "memory" );
      const uint32_t tacc = tmem_base + ab * kMaxNb + lane_off;
      float* slot = a.ws + ( (size_t)p.tile * a.max_segs + p.seg ) * slot_floats;
      for ( int cb = 0; cb < n_chunks; cb++ ) {
        float v[32];
        tmem_ld32( tacc + cb * 32, v );
#pragma unroll
        for ( int j = 0; j < 32; j++ ) // (columns past the batch are never read back)
          slot[(size_t)( cb * 32 + j ) * kTileF + r] = v[j];
      }
      asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
      asm volatile( "mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"( smem_u32( &bar_acc_free[ab] ) ) : "memory" );
      u += p.k1 - p.k0;
    }
    if ( !ok )
      *fail = 1;
  }

  asm volatile( "tcgen05.fence::before_thread_sync;" ::: "memory" );
  __syncthreads();
  if ( r == 0 && *fail != 0 )
    atomicOr( a.dev_error, 16u );
  if ( warp == 5 ) {
    __syncwarp();
    asm volatile( "tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"( tmem_base ), "r"( kTmemCols ) );
  }
}

constexpr int kFinishRows = 16; // batch rows per block of the finishing kernel
constexpr int kFinishSegs = 3;  // pieces of a tile whose loads are in flight together

// Second step of the projection: one block = (tile of 128 features, 16 batch rows); a thread owns one (even, odd)
// feature pair and walks 4 of the rows.  It adds the tile's pieces in their fixed order (deterministic), rounds to the
// storage type (the reference stores q and kv there), rotates q and K pairs by the row's position with separately
// rounded products (src/arch/amd64/llama2/ops.hh:150-162) and writes q, or K/V straight into the slot row.
template<typename T>
__global__ void __launch_bounds__( 256, 3 ) project_finish_kernel( const ProjectArgs a )
{
  asm volatile( "griddepcontrol.launch_dependents;" ::: "memory" );
  const int tile = blockIdx.x;
  const int pair = threadIdx.x & 63; // features 2 * pair, 2 * pair + 1 of the tile
  const int sub = threadIdx.x >> 6;  // rows sub, sub + 4, ... of the block's kFinishRows
  const int hs = a.sh.head_size;
  const int dim = a.dim, kv_dim = a.sh.kv_dim, batch = a.batch;
  const int f = tile * kTileF + 2 * pair;
  const bool rotate = f < dim + kv_dim;
  const int d2 = ( f % hs ) >> 1;
  const int first = tile * (int)a.kblocks, last = first + (int)a.kblocks - 1;
  const int nsegs = last / (int)a.units_per_cta - first / (int)a.units_per_cta + 1;
  const size_t slot_floats = (size_t)( ( batch + 31 ) / 32 ) * 32 * kTileF;
  const float* tile_ws = a.ws + (size_t)tile * a.max_segs * slot_floats;
  const T* __restrict__ cos_t = static_cast<const T*>( a.rope_cos );
  const T* __restrict__ sin_t = static_cast<const T*>( a.rope_sin );
  constexpr int R = kFinishRows / 4;
  // First what the kernels before this one in the stream do not write (the batch description and the tables come
  // from copies, which programmatic launches do not overtake): positions and row pointers, then the table values.
  // Blocks that become resident while the projection still runs have these two rounds of loads behind them when it
  // completes.
  uint32_t pos[R];
  T* row[R]; // the prompt's slot row at its position; nullptr = inactive prompt
#pragma unroll
  for ( int k = 0; k < R; k++ ) {
    const int i = blockIdx.y * kFinishRows + sub + 4 * k;
    pos[k] = 0;
    row[k] = nullptr;
    if ( i < batch ) {
      if ( a.token_rows != nullptr ) {
        pos[k] = a.pos[a.batch0 + i];
        row[k] = static_cast<T*>( a.token_rows[a.batch0 + i] );
      } else {
        const CtxMeta c = a.ctx[a.batch0 + i];
        pos[k] = c.pos;
        if ( c.kv_off != kInactive )
          row[k] = reinterpret_cast<T*>( a.arena + c.kv_off + a.layer_off ) + (size_t)c.pos * a.sh.row_elems;
      }
    }
  }
  float cs[R], sn[R];
#pragma unroll
  for ( int k = 0; k < R; k++ ) {
    const int i = blockIdx.y * kFinishRows + sub + 4 * k;
    // An inactive prompt's position is not checked by the host (it may be any value): its q is don't-care and its
    // K goes nowhere, so nothing of the tables is read for it.
    cs[k] = 1.f, sn[k] = 0.f;
    if ( rotate && i < batch && row[k] != nullptr ) {
      const size_t ti = (size_t)pos[k] * ( hs / 2 ) + d2;
      cs[k] = Conv<T>::to_f32( __ldg( cos_t + ti ) );
      sn[k] = Conv<T>::to_f32( __ldg( sin_t + ti ) );
    }
  }
  // the partial sums come from the projection kernel, the kernel before this one in the stream
  asm volatile( "griddepcontrol.wait;" ::: "memory" );
  // pieces three at a time, all of their rows' loads in flight, added in their fixed order (the same bits on every
  // run; a missing piece adds +0, which changes no bit of a sum that started from +0)
  float2 acc[R];
#pragma unroll
  for ( int k = 0; k < R; k++ )
    acc[k] = make_float2( 0.f, 0.f );
  for ( int s0 = 0; s0 < nsegs; s0 += kFinishSegs ) {
    float2 part[kFinishSegs][R];
#pragma unroll
    for ( int ds = 0; ds < kFinishSegs; ds++ )
#pragma unroll
      for ( int k = 0; k < R; k++ ) {
        const int i = blockIdx.y * kFinishRows + sub + 4 * k;
        part[ds][k] = make_float2( 0.f, 0.f );
        if ( s0 + ds < nsegs && i < batch )
          part[ds][k] = __ldcg( reinterpret_cast<const float2*>( tile_ws + (size_t)( s0 + ds ) * slot_floats + (size_t)i * kTileF
                                                                 + 2 * pair ) );
      }
#pragma unroll
    for ( int ds = 0; ds < kFinishSegs; ds++ )
#pragma unroll
      for ( int k = 0; k < R; k++ ) {
        acc[k].x += part[ds][k].x;
        acc[k].y += part[ds][k].y;
      }
  }
#pragma unroll
  for ( int k = 0; k < R; k++ ) {
    const int i = blockIdx.y * kFinishRows + sub + 4 * k;
    if ( i >= batch )
      continue;
    float x0 = Conv<T>::to_f32( Conv<T>::from_f32( acc[k].x ) ), x1 = Conv<T>::to_f32( Conv<T>::from_f32( acc[k].y ) );
    if ( rotate ) {
      const float y0 = __fsub_rn( __fmul_rn( x0, cs[k] ), __fmul_rn( x1, sn[k] ) );
      const float y1 = __fadd_rn( __fmul_rn( x0, sn[k] ), __fmul_rn( x1, cs[k] ) );
      x0 = y0, x1 = y1;
    }
    const T o0 = Conv<T>::from_f32( x0 ), o1 = Conv<T>::from_f32( x1 );
    const uint32_t bits = static_cast<uint32_t>( *reinterpret_cast<const uint16_t*>( &o0 ) )
                          | ( static_cast<uint32_t>( *reinterpret_cast<const uint16_t*>( &o1 ) ) << 16 );
    T* dst = nullptr;
    if ( f < dim )
      dst = static_cast<T*>( a.q_out ) + (size_t)( a.batch0 + i ) * dim + f;
    else if ( row[k] != nullptr )
      dst = row[k] + ( f - dim );
    if ( dst != nullptr )
      *reinterpret_cast<uint32_t*>( dst ) = bits;
  }
}

} // namespace

bool project_supported( const Shape& sh, uint32_t dtype )
{
  const uint32_t dim = sh.n_heads * sh.head_size;
  return ( dtype == DT_F16 || dtype == DT_BF16 ) && dim % kTileF == 0 && sh.kv_dim % kTileF == 0 && sh.head_size % 2 == 0
         && kTileF % sh.head_size == 0;
}

uint32_t project_max_rows()
{
  return kMaxNb;
}

cudaError_t project_prepare()
{
  cudaError_t e = cudaFuncSetAttribute( project_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes );
  if ( e == cudaSuccess )
    e = cudaFuncSetAttribute( project_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes );
  return e;
}

void project_plan( const Shape& sh, uint32_t sm_count, ProjectArgs* a, uint32_t* grid )
{
  const uint32_t dim = sh.n_heads * sh.head_size;
  a->dim = dim;
  a->q_tiles = dim / kTileF;
  a->n_tiles = ( dim + 2 * sh.kv_dim ) / kTileF;
  a->kblocks = dim / kBK;
  const uint32_t units = a->n_tiles * a->kblocks;
  // one CTA per SM, but no piece shorter than four k-blocks unless the whole problem is that small
  const uint32_t ctas = std::max( 1u, std::min( sm_count, units / 4 ) );
  a->units_per_cta = ( units + ctas - 1 ) / ctas;
  *grid = ( units + a->units_per_cta - 1 ) / a->units_per_cta;
  a->max_segs = ( a->kblocks + a->units_per_cta - 1 ) / a->units_per_cta + 1;
}

uint32_t project_pieces( const ProjectArgs& a, uint32_t cta, int32_t* out, uint32_t cap )
{
  const int upc = a.units_per_cta, kblocks = a.kblocks;
  const int u_begin = cta * upc, u_end = std::min<int>( a.n_tiles * a.kblocks, u_begin + upc );
  uint32_t n = 0;
  for ( int u = u_begin; u < u_end; ) {
    const Piece p = piece_at( u, u_end, kblocks, upc );
    if ( n < cap ) {
      int32_t* rec = out + 5 * n;
      rec[0] = p.tile, rec[1] = p.k0, rec[2] = p.k1, rec[3] = p.seg, rec[4] = p.nsegs;
    }
    n++;
    u += p.k1 - p.k0;
  }
  return n;
}

size_t project_workspace_bytes( const ProjectArgs& a )
{
  return (size_t)a.n_tiles * a.max_segs * kMaxNb * kTileF * sizeof( float );
}

cudaError_t launch_rmsnorm( void* out, const void* x, const void* weight, uint32_t rows, uint32_t dim, uint32_t dtype,
                            cudaStream_t st, uint64_t* launches )
{
  if ( rows == 0 )
    return cudaSuccess;
  const uint32_t per_piece = dtype == DT_F32 ? 4 : 8;
  if ( dim % per_piece != 0 || dim > 256u * kNormPieces * per_piece )
    return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg {};
  cfg.gridDim = dim3( rows );
  cfg.blockDim = dim3( 256 );
  cfg.stream = st;
  cudaLaunchAttribute attr {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  switch ( dtype ) {
    case DT_F32:
      e = cudaLaunchKernelEx( &cfg, rmsnorm_kernel<float>, static_cast<float*>( out ), static_cast<const float*>( x ),
                              static_cast<const float*>( weight ), dim );
      break;
    case DT_F16:
      e = cudaLaunchKernelEx( &cfg, rmsnorm_kernel<__half>, static_cast<__half*>( out ), static_cast<const __half*>( x ),
                              static_cast<const __half*>( weight ), dim );
      break;
    case DT_BF16:
      e = cudaLaunchKernelEx( &cfg, rmsnorm_kernel<__nv_bfloat16>, static_cast<__nv_bfloat16*>( out ),
                              static_cast<const __nv_bfloat16*>( x ), static_cast<const __nv_bfloat16*>( weight ), dim );
      break;
    default: return cudaErrorInvalidValue;
  }
  ( *launches )++;
  return e;
}

cudaError_t launch_project( const ProjectArgs& a, uint32_t grid, const CUtensorMap* wq_map, const CUtensorMap* wkv_map,
                            const CUtensorMap* xb_map, cudaStream_t st, uint64_t* launches )
{
  if ( a.batch == 0 )
    return cudaSuccess;
  cudaLaunchConfig_t cfg {};
  cfg.gridDim = dim3( grid );
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
    e = cudaLaunchKernelEx( &cfg, project_kernel<__half>, a, *wq_map, *wkv_map, *xb_map );
  else if ( a.dtype == DT_BF16 )
    e = cudaLaunchKernelEx( &cfg, project_kernel<__nv_bfloat16>, a, *wq_map, *wkv_map, *xb_map );
  else
    return cudaErrorInvalidValue;
  ( *launches )++;
  if ( e != cudaSuccess )
    return e;
  cfg.gridDim = dim3( a.n_tiles, ( a.batch + kFinishRows - 1 ) / kFinishRows );
  cfg.blockDim = dim3( 256 );
  cfg.dynamicSmemBytes = 0;
  if ( a.dtype == DT_F16 )
    e = cudaLaunchKernelEx( &cfg, project_finish_kernel<__half>, a );
  else
    e = cudaLaunchKernelEx( &cfg, project_finish_kernel<__nv_bfloat16>, a );
  ( *launches )++;
  return e;
}

} // namespace gh
