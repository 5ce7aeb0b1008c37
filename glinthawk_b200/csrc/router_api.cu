// C ABI of the request -> GPU router (include/glinthawk_router.h).  Host code only.
#include "../../include/glinthawk_router.h"
#include "router.hh"

#include <new>

struct gh_router
{
  gh::ContextRouter impl;
};

namespace {

int code( gh::ContextRouter::Status s )
{
  switch ( s ) {
    case gh::ContextRouter::Status::Ok: return GH_OK;
    case gh::ContextRouter::Status::NoSlot: return GH_ERR_NO_SLOT;
    case gh::ContextRouter::Status::NotFound: return GH_ERR_NOT_FOUND;
    default: return GH_ERR_INVALID;
  }
}

} // namespace

extern "C" {

int gh_router_create( gh_router_t* out, uint32_t n_ranks, uint32_t per_rank_batch, uint32_t slots_per_rank, uint32_t policy )
{
  if ( out == nullptr || n_ranks == 0 || per_rank_batch == 0 || policy > GH_ROUTE_BALANCED
       || static_cast<uint64_t>( n_ranks ) * per_rank_batch > 0x7fffffffull )
    return GH_ERR_INVALID;
  gh_router* r = new ( std::nothrow )
    gh_router { gh::ContextRouter( n_ranks, per_rank_batch, slots_per_rank, static_cast<gh::RoutePolicy>( policy ) ) };
  if ( r == nullptr )
    return GH_ERR_OOM;
  *out = r;
  return GH_OK;
}

void gh_router_destroy( gh_router_t r )
{
  delete r;
}

int gh_router_is_context_available( gh_router_t r )
{
  if ( r == nullptr )
    return -GH_ERR_INVALID;
  return r->impl.is_context_available() ? 1 : 0;
}

int gh_router_assign_ranks( gh_router_t r, uint32_t n, const uint64_t* prompt_ids, const uint32_t* expected_tokens,
                            uint32_t* ranks_out )
{
  if ( r == nullptr )
    return GH_ERR_INVALID;
  try {
    return code( r->impl.assign( n, prompt_ids, expected_tokens, ranks_out ) );
  } catch ( const std::bad_alloc& ) {
    return GH_ERR_OOM;
  }
}

int gh_router_lookup( gh_router_t r, uint64_t prompt_id, uint32_t* rank_out )
{
  if ( r == nullptr || rank_out == nullptr )
    return GH_ERR_INVALID;
  return code( r->impl.lookup( prompt_id, rank_out ) );
}

int gh_router_note_tokens( gh_router_t r, uint32_t n, const uint64_t* prompt_ids, const uint32_t* cached_tokens )
{
  if ( r == nullptr || ( n != 0 && ( prompt_ids == nullptr || cached_tokens == nullptr ) ) )
    return GH_ERR_INVALID;
  return code( r->impl.note_tokens( n, prompt_ids, cached_tokens ) );
}

int gh_router_release( gh_router_t r, uint32_t n, const uint64_t* prompt_ids )
{
  if ( r == nullptr || ( n != 0 && prompt_ids == nullptr ) )
    return GH_ERR_INVALID;
  try {
    return code( r->impl.release( n, prompt_ids ) );
  } catch ( const std::bad_alloc& ) {
    return GH_ERR_OOM;
  }
}

int gh_router_loads( gh_router_t r, uint32_t* free_slots_out, uint64_t* tokens_out )
{
  if ( r == nullptr )
    return GH_ERR_INVALID;
  r->impl.loads( free_slots_out, tokens_out );
  return GH_OK;
}

int gh_router_cut( uint32_t n_ranks, uint32_t n, const uint32_t* ranks, uint32_t* order_out, uint32_t* counts_out )
{
  if ( n_ranks == 0 || counts_out == nullptr || ( n != 0 && ( ranks == nullptr || order_out == nullptr ) ) )
    return GH_ERR_INVALID;
  try {
    return code( gh::ContextRouter::cut( n_ranks, n, ranks, order_out, counts_out ) );
  } catch ( const std::bad_alloc& ) {
    return GH_ERR_OOM;
  }
}

} // extern "C"
