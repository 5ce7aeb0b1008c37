// Host-side work planning for the fused decode kernels (pure host code, no CUDA calls).
//
// A batch is ragged: context i attends over pos[i] + 1 tokens.  Work items are ordered longest-first so that the
// hardware block scheduler approximates longest-processing-time-first, and long contexts are cut along the token
// axis only as far as that pays: every extra item costs a pipeline fill and drain (about 2 us on B200), and an item
// of a cut context also writes a partial record that is read back when the records are combined.  The blocks that
// run at the same time share the HBM bandwidth equally: with every block slot of the GPU busy a block takes about
// 40 ns per token (one "token-time"), with fewer blocks running each gets more, down to about 20 ns per token, where
// a block is bound by the latency of its own loads.  So a long context is the critical path of a launch even when
// the GPU is saturated, and how far cutting pays depends on how many other contexts there are to fill the slots.
// The split length is chosen by simulating this sharing for a dozen candidate lengths (an event-driven simulation,
// one event per work item) and keeping the shortest launch; the model's constants were fitted to launch times
// measured on B200 for 32 to 256 contexts per GPU and reproduce them to within 3 %.  The
// reference has no counterpart: it loops over the batch on the host and launches per context
// (src/arch/cuda/llama2/ops.cuh:272-453).
#pragma once

#include <algorithm>
#include <cstdint>
#include <functional>
#include <queue>
#include <vector>

#include "gh_common.cuh"
#include "gh_merge.cuh"

namespace gh {

struct PlanParams
{
  uint32_t n_kv_heads = 1;      // blocks per work item
  uint32_t sm_count = 148;
  uint32_t tile = 64;           // split boundaries are multiples of this many tokens
  uint32_t fixed_chunk = 0;     // non-zero: use exactly this split length
  uint32_t max_items = 0;       // capacity of the item and partial-record buffers
  uint32_t blocks_per_sm = 2;       // thread blocks resident per SM
  uint32_t min_chunk = 256;
  uint32_t whole_overhead = 100;    // cost of an uncut context's item beyond its tokens, in token-times
  uint32_t piece_overhead = 250;    // the same for an item of a cut context (partial record, arrival count, combining)
  uint32_t alone_rate_pct = 50;     // time per token of a block that runs latency-bound, in percent of a token-time
                                    // (a token-time = time per token of a block when all block slots stream together)
};

struct Plan
{
  std::vector<WorkItem> items;
  std::vector<int32_t> split_ctx; // batch indices of the contexts that were cut
  uint32_t chunk = 0;
  uint32_t partial_records = 0;
};

inline uint32_t round_up_u32( uint64_t v, uint32_t m )
{
  return static_cast<uint32_t>( ( v + m - 1 ) / m * m );
}

// `ctx[i].kv_off` and `ctx[i].pos` must be filled in; nsplits / partial_base are written here.
// Returns false if the batch cannot be described within max_items even with unsplit contexts.
inline bool plan_batch( const PlanParams& p, std::vector<CtxMeta>& ctx, Plan& out )
{
  uint64_t total = 0;
  uint32_t active = 0;
  for ( const auto& c : ctx ) {
    if ( c.kv_off != kInactive ) {
      total += static_cast<uint64_t>( c.pos ) + 1;
      active++;
    }
  }
  out.items.clear();
  out.split_ctx.clear();
  out.partial_records = 0;
  out.chunk = 0;
  if ( active == 0 )
    return true;
  if ( active > p.max_items )
    return false;

  uint32_t max_len = 0;
  for ( const auto& c : ctx )
    if ( c.kv_off != kInactive )
      max_len = std::max( max_len, c.pos + 1 );

  // number of work items for a split length; "too many" when a context would be cut into more than kMaxSplits
  auto item_count = [&]( uint32_t chunk ) -> uint64_t {
    uint64_t n = 0;
    for ( const auto& c : ctx )
      if ( c.kv_off != kInactive )
        n += ( static_cast<uint64_t>( c.pos ) + chunk ) / chunk; // ceil( (pos+1) / chunk )
    if ( ( static_cast<uint64_t>( max_len ) + chunk - 1 ) / chunk > static_cast<uint64_t>( kMaxSplits ) )
      return ~uint64_t( 0 );
    return n;
  };

  // Predicted duration, in token-times, of the launch with split length `chunk`.  Items (each fanning out to
  // n_kv_heads blocks at once) start longest-first while item slots are free; the n items running at any moment each
  // progress at min( 1 / alone_rate, slots / n ) tokens per token-time.  Because all running items progress at the
  // same rate, progress is tracked in one shared coordinate: an item of length L that starts at progress v ends at
  // v + L, and the elapsed time between two ends is the progress made divided by the rate in force.
  const uint32_t machines = std::max<uint32_t>( 1, p.sm_count * p.blocks_per_sm / std::max<uint32_t>( 1, p.n_kv_heads ) );
  const double top_rate = 100.0 / std::max<uint32_t>( 1, p.alone_rate_pct );
  std::vector<uint32_t> costs;
  auto makespan = [&]( uint32_t chunk ) {
    costs.clear();
    for ( const auto& c : ctx ) {
      if ( c.kv_off == kInactive )
        continue;
      const uint32_t len = c.pos + 1;
      const uint32_t n = ( len + chunk - 1 ) / chunk;
      const uint32_t step = round_up_u32( ( len + n - 1 ) / n, p.tile );
      const uint32_t overhead = n > 1 ? p.piece_overhead : p.whole_overhead;
      for ( uint32_t b = 0; b < len; b += step )
        costs.push_back( std::min( step, len - b ) + overhead );
    }
    std::sort( costs.begin(), costs.end(), std::greater<uint32_t>() );
    std::priority_queue<double, std::vector<double>, std::greater<double>> ends; // progress at which running items end
    size_t next = 0;
    double progress = 0.0, elapsed = 0.0;
    while ( next < costs.size() && ends.size() < machines )
      ends.push( progress + costs[next++] );
    while ( !ends.empty() ) {
      const double rate = std::min( top_rate, static_cast<double>( machines ) / static_cast<double>( ends.size() ) );
      const double end = ends.top();
      ends.pop();
      elapsed += ( end - progress ) / rate;
      progress = end;
      if ( next < costs.size() )
        ends.push( progress + costs[next++] );
    }
    return static_cast<uint64_t>( elapsed + 0.5 );
  };

  uint32_t chunk = p.fixed_chunk;
  if ( chunk != 0 ) {
    chunk = round_up_u32( chunk, p.tile );
    while ( item_count( chunk ) > p.max_items )
      chunk *= 2;
  } else {
    // candidates: no cut at all, then three quarters and halves of that, and so on down to the minimum split
    // length; of equally good ones the longest wins (fewest items)
    const uint32_t top = round_up_u32( max_len, p.tile );
    const uint32_t floor_len = std::max( p.min_chunk, p.tile );
    uint64_t best = ~0ull;
    auto consider = [&]( uint32_t cand ) {
      if ( ( cand < floor_len && cand != top ) || item_count( cand ) > p.max_items )
        return;
      const uint64_t ms = makespan( cand );
      if ( ms < best ) {
        best = ms;
        chunk = cand;
      }
    };
    for ( uint32_t cand = top;; cand = round_up_u32( cand / 2, p.tile ) ) {
      consider( cand );
      if ( cand <= floor_len )
        break;
      consider( round_up_u32( static_cast<uint64_t>( cand ) * 3 / 4, p.tile ) );
    }
    if ( chunk == 0 )
      return false;
  }
  out.chunk = chunk;

  for ( size_t i = 0; i < ctx.size(); i++ ) {
    CtxMeta& c = ctx[i];
    if ( c.kv_off == kInactive ) {
      c.nsplits = 0;
      c.partial_base = 0;
      continue;
    }
    const uint32_t len = c.pos + 1;
    const uint32_t nsplits = ( len + chunk - 1 ) / chunk;
    // equal-sized splits, boundaries on tile multiples
    const uint32_t step = round_up_u32( ( len + nsplits - 1 ) / nsplits, p.tile );
    uint32_t made = 0;
    for ( uint32_t b = 0; b < len; b += step ) {
      WorkItem w;
      w.ctx = static_cast<int32_t>( i );
      w.t_begin = static_cast<int32_t>( b );
      w.t_end = static_cast<int32_t>( std::min( len, b + step ) );
      w.split = static_cast<int32_t>( made++ );
      out.items.push_back( w );
    }
    c.nsplits = static_cast<int32_t>( made );
    c.partial_base = static_cast<int32_t>( out.partial_records );
    if ( made > 1 ) {
      out.partial_records += made;
      out.split_ctx.push_back( static_cast<int32_t>( i ) );
    }
  }

  std::stable_sort( out.items.begin(), out.items.end(), []( const WorkItem& a, const WorkItem& b ) {
    return ( a.t_end - a.t_begin ) > ( b.t_end - b.t_begin );
  } );
  return true;
}

} // namespace gh
