// Request -> GPU assignment for the attention stage of one box: which rank's slot pool a prompt's KV lives in.
//
// Restates, for the GPUs of one box, what the reference's tier router does for the attention stage:
//   ParentTierRouter::assign_ranks         src/compute/routerman.hh:311-331   prompt i of a batch -> (tier, rank), once;
//                                                                             the prompt keeps it for life
//   ParentTierRouter::is_context_available src/compute/routerman.hh:295-307   room for one more full batch everywhere?
//   SliceConcurrency::tier_rank / cutting_plan  src/compute/common.hh:44-104  batch index -> rank by equal slices
// with two things the reference does not have: contexts are released again, and a policy that balances cached tokens
// (what a decode step streams) instead of prompt counts.  Host-only, deterministic: processes that make the same calls
// hold the same table, so the ranks of a box need no communication to agree.
#pragma once

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <numeric>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace gh {

enum class RoutePolicy : uint32_t
{
  Position = 0, // the reference's: prompt i of the batch goes to rank i / per_rank_batch
  Balanced = 1  // longest prompt first onto the rank with the fewest cached tokens that still has room in its slice
};

class ContextRouter
{
public:
  enum class Status
  {
    Ok,
    Invalid,
    NoSlot,
    NotFound
  };

  ContextRouter( uint32_t n_ranks, uint32_t per_rank_batch, uint32_t slots_per_rank, RoutePolicy policy )
    : per_rank_batch_( per_rank_batch )
    , policy_( policy )
    , free_( n_ranks, slots_per_rank )
    , tokens_( n_ranks, 0 )
  {
  }

  uint32_t n_ranks() const { return static_cast<uint32_t>( free_.size() ); }
  uint32_t full_batch() const { return n_ranks() * per_rank_batch_; }

  // Every rank still has a slot for each prompt of its slice of a full batch.
  bool is_context_available() const
  {
    std::lock_guard lock { mu_ };
    return std::all_of( free_.begin(), free_.end(), [this]( uint32_t f ) { return f >= per_rank_batch_; } );
  }

  // Ranks for the prompts of one batch (at most a full batch).  A prompt that already has a rank keeps it; the others
  // get one and take a slot there.  All or nothing: when a new prompt finds no room, nothing is changed.
  Status assign( uint32_t n, const uint64_t* ids, const uint32_t* expected_tokens, uint32_t* ranks_out )
  {
    if ( n > full_batch() || ( n != 0 && ( ids == nullptr || ranks_out == nullptr ) ) )
      return Status::Invalid;
    std::lock_guard lock { mu_ };
    std::unordered_set<uint64_t> seen;
    std::vector<uint32_t> fresh;                 // batch indices of the prompts without a rank
    std::vector<uint32_t> quota( n_ranks(), per_rank_batch_ ); // room left in each rank's slice of this batch
    for ( uint32_t i = 0; i < n; i++ ) {
      if ( !seen.insert( ids[i] ).second )
        return Status::Invalid; // the same prompt twice in one batch
      const auto it = owner_.find( ids[i] );
      if ( it == owner_.end() ) {
        fresh.push_back( i );
      } else {
        ranks_out[i] = it->second.rank;
        if ( quota[it->second.rank] > 0 )
          quota[it->second.rank]--;
      }
    }
    std::vector<uint32_t> free_left = free_;
    std::vector<uint64_t> load = tokens_;
    auto tokens_of = [&]( uint32_t i ) { return expected_tokens != nullptr ? expected_tokens[i] : 0u; };
    if ( policy_ == RoutePolicy::Position ) {
      for ( const uint32_t i : fresh ) {
        const uint32_t rank = i / per_rank_batch_;
        if ( free_left[rank] == 0 )
          return Status::NoSlot;
        free_left[rank]--;
        ranks_out[i] = rank;
      }
    } else {
      std::stable_sort( fresh.begin(), fresh.end(), [&]( uint32_t a, uint32_t b ) { return tokens_of( a ) > tokens_of( b ); } );
      for ( const uint32_t i : fresh ) {
        int best = -1;
        for ( uint32_t r = 0; r < n_ranks(); r++ )
          if ( quota[r] > 0 && free_left[r] > 0 && ( best < 0 || load[r] < load[best] ) )
            best = static_cast<int>( r );
        if ( best < 0 )
          return Status::NoSlot;
        quota[best]--;
        free_left[best]--;
        load[best] += tokens_of( i );
        ranks_out[i] = static_cast<uint32_t>( best );
      }
    }
    for ( const uint32_t i : fresh ) {
      owner_[ids[i]] = Entry { ranks_out[i], tokens_of( i ) };
      tokens_[ranks_out[i]] += tokens_of( i );
    }
    free_ = free_left;
    return Status::Ok;
  }

  Status lookup( uint64_t id, uint32_t* rank_out ) const
  {
    std::lock_guard lock { mu_ };
    const auto it = owner_.find( id );
    if ( it == owner_.end() )
      return Status::NotFound;
    *rank_out = it->second.rank;
    return Status::Ok;
  }

  // The prompts' cached tokens as they are now (they grow by one per step): what the balanced policy weighs.
  Status note_tokens( uint32_t n, const uint64_t* ids, const uint32_t* cached_tokens )
  {
    std::lock_guard lock { mu_ };
    for ( uint32_t i = 0; i < n; i++ )
      if ( owner_.find( ids[i] ) == owner_.end() )
        return Status::NotFound;
    for ( uint32_t i = 0; i < n; i++ ) {
      Entry& e = owner_[ids[i]];
      tokens_[e.rank] += cached_tokens[i];
      tokens_[e.rank] -= e.tokens;
      e.tokens = cached_tokens[i];
    }
    return Status::Ok;
  }

  // Finished prompts give their slots back (the reference never does).  Unknown ids are an error and change nothing.
  Status release( uint32_t n, const uint64_t* ids )
  {
    std::lock_guard lock { mu_ };
    std::unordered_set<uint64_t> seen;
    for ( uint32_t i = 0; i < n; i++ )
      if ( owner_.find( ids[i] ) == owner_.end() || !seen.insert( ids[i] ).second )
        return Status::NotFound;
    for ( uint32_t i = 0; i < n; i++ ) {
      const auto it = owner_.find( ids[i] );
      free_[it->second.rank]++;
      tokens_[it->second.rank] -= it->second.tokens;
      owner_.erase( it );
    }
    return Status::Ok;
  }

  void loads( uint32_t* free_slots_out, uint64_t* tokens_out ) const
  {
    std::lock_guard lock { mu_ };
    for ( uint32_t r = 0; r < n_ranks(); r++ ) {
      if ( free_slots_out != nullptr )
        free_slots_out[r] = free_[r];
      if ( tokens_out != nullptr )
        tokens_out[r] = tokens_[r];
    }
  }

  // The batch cut into per-rank shards (the reference's cutting plan, src/compute/common.hh:95-98, for ranks that
  // were not assigned by position): indices grouped by rank, in batch order within a rank, and how many each rank has.
  static Status cut( uint32_t n_ranks, uint32_t n, const uint32_t* ranks, uint32_t* order_out, uint32_t* counts_out )
  {
    std::fill( counts_out, counts_out + n_ranks, 0u );
    for ( uint32_t i = 0; i < n; i++ ) {
      if ( ranks[i] >= n_ranks )
        return Status::Invalid;
      counts_out[ranks[i]]++;
    }
    std::vector<uint32_t> at( n_ranks, 0 );
    std::partial_sum( counts_out, counts_out + n_ranks - 1, at.begin() + 1 );
    for ( uint32_t i = 0; i < n; i++ )
      order_out[at[ranks[i]]++] = i;
    return Status::Ok;
  }

private:
  struct Entry
  {
    uint32_t rank;
    uint32_t tokens;
  };
  const uint32_t per_rank_batch_;
  const RoutePolicy policy_;
  mutable std::mutex mu_; // the reference guards its free-context counts the same way (ctx_mutex_)
  std::vector<uint32_t> free_;   // free slots per rank
  std::vector<uint64_t> tokens_; // cached tokens per rank, as last told
  std::unordered_map<uint64_t, Entry> owner_;
};

} // namespace gh
