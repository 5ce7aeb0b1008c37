/*
 * glinthawk_router.h — request -> GPU assignment for the attention stage on the GPUs of one box: which rank's slot
 * pool (gh_slot_acquire, glinthawk_attn.h) holds a prompt's KV.  Host-only: no entry point here touches a device.
 *
 * Replaces, for the attention stage, the bookkeeping of the reference's tier router:
 *   ParentTierRouter::assign_ranks          src/compute/routerman.hh:311-331
 *   ParentTierRouter::is_context_available  src/compute/routerman.hh:295-307
 *   SliceConcurrency::tier_rank / cutting_plan  src/compute/common.hh:44-104
 * A prompt is given a rank once and keeps it (its KV never moves).  Unlike the reference, prompts can be released,
 * and besides the reference's assignment by batch position there is one that balances cached tokens.  The table is
 * a deterministic function of the calls made, so processes that make the same calls agree without communicating.
 * Calls on one router may come from several threads (one mutex, like the reference's ctx_mutex_).
 */
#ifndef GLINTHAWK_ROUTER_H
#define GLINTHAWK_ROUTER_H

#include "glinthawk_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gh_router* gh_router_t;

typedef enum gh_route_policy
{
  GH_ROUTE_POSITION = 0, /* the reference's: prompt i of a batch goes to rank i / per_rank_batch */
  GH_ROUTE_BALANCED = 1  /* longest prompt first onto the rank with the fewest cached tokens; every rank still gets
                            at most per_rank_batch prompts of a batch */
} gh_route_policy;

/* n_ranks GPUs, each serving per_rank_batch prompts of a full batch (the reference's attention concurrency of a
 * node, src/compute/common.hh:27-41) out of slots_per_rank context slots. */
int gh_router_create( gh_router_t* out, uint32_t n_ranks, uint32_t per_rank_batch, uint32_t slots_per_rank, uint32_t policy );
void gh_router_destroy( gh_router_t r );

/* 1 when every rank has free slots for its share of one more full batch, 0 when not, negative on a null router
 * (routerman.hh:295-307: the worker only admits a new batch of prompts when this holds). */
int gh_router_is_context_available( gh_router_t r );

/* Ranks for the n <= n_ranks * per_rank_batch prompts of one batch.  A prompt that already has a rank keeps it;
 * every other prompt gets one and takes a slot there.  expected_tokens (may be NULL = all equal) is what the
 * balanced policy weighs: the prompt's length if known, else 0.  All or nothing: GH_ERR_NO_SLOT leaves the
 * router unchanged.  GH_ERR_INVALID: null argument, n too large, or the same id twice. */
int gh_router_assign_ranks( gh_router_t r, uint32_t n, const uint64_t* prompt_ids, const uint32_t* expected_tokens,
                            uint32_t* ranks_out );

/* The rank of a prompt; GH_ERR_NOT_FOUND when it has none. */
int gh_router_lookup( gh_router_t r, uint64_t prompt_id, uint32_t* rank_out );

/* Tells the router how many tokens the prompts have cached by now.  GH_ERR_NOT_FOUND (nothing changed) when one
 * of them has no rank.  No reference counterpart. */
int gh_router_note_tokens( gh_router_t r, uint32_t n, const uint64_t* prompt_ids, const uint32_t* cached_tokens );

/* Finished prompts: their slots become free again and their tokens leave the ranks' loads.  GH_ERR_NOT_FOUND
 * (nothing changed) when an id is unknown or listed twice.  No reference counterpart: the reference's contexts are
 * never handed back (src/compute/contextman.hh:82-184). */
int gh_router_release( gh_router_t r, uint32_t n, const uint64_t* prompt_ids );

/* Free slots and cached tokens per rank (either pointer may be NULL), n_ranks entries each. */
int gh_router_loads( gh_router_t r, uint32_t* free_slots_out, uint64_t* tokens_out );

/* Cuts a batch into per-rank shards: order_out receives the batch indices grouped by rank (batch order within a
 * rank), counts_out the number per rank — the reference's cutting plan (src/compute/common.hh:95-98) for ranks
 * that were not assigned by position. */
int gh_router_cut( uint32_t n_ranks, uint32_t n, const uint32_t* ranks, uint32_t* order_out, uint32_t* counts_out );

#ifdef __cplusplus
}
#endif
#endif
