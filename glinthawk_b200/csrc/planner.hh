// Host-side work planning for the fused decode kernels (pure host code, no CUDA calls).
//
// A batch is ragged: context i attends over pos[i] + 1 tokens.  Long contexts are cut along the token axis
// into work items of similar size so that every SM streams KV for the whole launch, and the items are ordered
// longest-first so the hardware block scheduler approximates longest-processing-time-first.  The reference has
// no counterpart: it loops over the batch on the host and launches per context
// (src/arch/cuda/llama2/ops.cuh:272-453).
#pragma once

#include <algorithm>
#include <cstdint>
#include <vector>

#include "gh_common.cuh"

namespace gh {

struct PlanParams
{
  uint32_t n_kv_heads = 1;      // blocks per work item
  uint32_t sm_count = 148;
  uint32_t tile = 64;           // split boundaries are multiples of this many tokens
  uint32_t fixed_chunk = 0;     // non-zero: use exactly this split length
  uint32_t max_items = 0;       // capacity of the item and partial-record buffers
  uint32_t blocks_per_sm_target = 16; // aim for about this many blocks per SM over the launch
  uint32_t min_chunk = 256;
};

struct Plan
{
  std::vector<WorkItem> items;
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
  out.partial_records = 0;
  out.chunk = 0;
  if ( active == 0 )
    return true;
  if ( active > p.max_items )
    return false;

  uint32_t chunk = p.fixed_chunk;
  if ( chunk == 0 ) {
    const uint64_t blocks_target = static_cast<uint64_t>( p.sm_count ) * p.blocks_per_sm_target;
    const uint64_t per_block = ( total * p.n_kv_heads + blocks_target - 1 ) / blocks_target;
    chunk = std::max( round_up_u32( per_block, p.tile ), round_up_u32( p.min_chunk, p.tile ) );
  } else {
    chunk = round_up_u32( chunk, p.tile );
  }

  for ( ;; ) {
    uint64_t n_items = 0;
    for ( const auto& c : ctx )
      if ( c.kv_off != kInactive )
        n_items += ( static_cast<uint64_t>( c.pos ) + chunk ) / chunk; // ceil( (pos+1) / chunk )
    if ( n_items <= p.max_items )
      break;
    chunk *= 2;
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
    if ( made > 1 )
      out.partial_records += made;
  }

  std::stable_sort( out.items.begin(), out.items.end(), []( const WorkItem& a, const WorkItem& b ) {
    return ( a.t_end - a.t_begin ) > ( b.t_end - b.t_begin );
  } );
  return true;
}

} // namespace gh
