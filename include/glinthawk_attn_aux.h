/*
 * glinthawk_attn_aux.h — entry points of libglinthawk_attn.so that are NOT part of the drop-in for Glinthawk's
 * attention stage: helpers for benchmarks and tests (device-side random fill, host-side views of the work plans,
 * host-side injection of the kernels' error word).  A binding of the reference needs none of them; the drop-in
 * interface is glinthawk_attn.h.
 */
#ifndef GLINTHAWK_ATTN_AUX_H
#define GLINTHAWK_ATTN_AUX_H

#include "glinthawk_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Fills n elements of `dtype` at device pointer `dst` with N(0,1) values from a counter-based generator
 * keyed by (seed, element index + offset).  No reference counterpart (the reference's profiler fills its
 * contexts with uniform noise, src/profile/profiler.hh:79-93). */
int gh_fill_normal( gh_attn_t h, void* dst, uint64_t n, uint32_t dtype, uint64_t seed, uint64_t offset, void* stream );

/* Host-side fault injection for tests of the error path: ORs `bits` into the kernels' error word as if a bounded
 * wait had run out.  Nothing on the GPU is made to wait or fail.  No reference counterpart. */
int gh_attn_inject_device_error( gh_attn_t h, uint32_t bits );

/* Host-only (touches no device): the split plan gh_attn_batch_begin makes for token positions `pos`
 * (UINT32_MAX marks an inactive prompt).  `blocks_per_item` is the number of thread blocks a work item fans out
 * to (kv heads for the tensor-core kernel).  Writes n_items records {context, t_begin, t_end, split} to
 * items_out (room for max_items) and the split length to *chunk.  No reference counterpart: the reference
 * loops over the batch on the host and launches per context (src/arch/cuda/llama2/ops.cuh:272-453). */
int gh_plan_batch( uint32_t blocks_per_item,
                   uint32_t sm_count,
                   uint32_t tile,
                   uint32_t fixed_chunk,
                   uint32_t max_items,
                   uint64_t batch,
                   const uint32_t* pos,
                   int32_t* items_out,
                   uint32_t* n_items,
                   uint32_t* chunk );


/* Host-only (touches no device): how gh_attn_project_append deals its work to the SMs.  plan_out receives
 * {CTAs, work units per CTA, most pieces a tile is cut into, feature tiles, k-blocks per tile}; pieces_out receives
 * one record {CTA, tile, first k-block, end k-block, index of the piece within its tile, pieces of that tile} per
 * piece, CTA by CTA in processing order.  No reference counterpart (the reference calls cuBLAS,
 * src/arch/cuda/common/ops.cuh:616-693). */
int gh_plan_projection( uint32_t n_heads,
                        uint32_t head_size,
                        uint32_t kv_dim,
                        uint32_t sm_count,
                        uint32_t* plan_out,
                        int32_t* pieces_out,
                        uint32_t max_pieces,
                        uint32_t* n_pieces );

#ifdef __cplusplus
}
#endif

#endif /* GLINTHAWK_ATTN_AUX_H */
