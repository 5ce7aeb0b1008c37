/*
 * glinthawk_attn.h — C ABI of the B200 (sm_100a) KV-cache attention stage.
 *
 * A drop-in for the attention-stage part of Glinthawk's `Operations` interface and its per-context KV
 * storage.  Every entry point names the reference interface it replaces (paths are relative to the
 * reference project).  Plain pointers and sizes only; every function returns a gh_status code and never
 * aborts the process.  There is no CPU fallback: every compute entry point launches CUDA kernels.
 *
 * Conventions
 *   - "device pointer" = CUDA device memory on the handle's device; "host array" = ordinary host memory.
 *   - dtype codes are the reference's DataType values (src/models/types.hh:20-25).
 *   - KV layout is the reference's (src/models/llama2/context.hh:79-89,115-127,177-189): a context slot is
 *     [hosted layer][token][K: kv_head x head_size | V: kv_head x head_size], token t of a layer at
 *     layer_base + t * 2 * kv_dim elements.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  All compute calls are
 *     asynchronous with respect to the host unless stated otherwise.
 *   - A handle is used by one host thread at a time (the reference calls its operations from one execution
 *     thread per model instance, src/compute/kernel.hh:103-136), with one exception that the reference has too
 *     (src/compute/kernel.hh:139-170 looks contexts up on a bookkeeping thread, under the context manager's mutex,
 *     src/compute/contextman.hh:82-184): gh_slot_acquire, gh_slots_acquire_batch and gh_slot_lookup may be called
 *     from another thread while the owning thread submits work.  Those three report through their status code only
 *     and never change the text gh_attn_last_error returns.
 */
#ifndef GLINTHAWK_ATTN_H
#define GLINTHAWK_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gh_attn* gh_attn_t;

typedef enum gh_status
{
  GH_OK = 0,
  GH_ERR_INVALID = 1,     /* bad argument (null pointer, size out of range, unknown code) */
  GH_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed; see gh_attn_last_error */
  GH_ERR_NO_SLOT = 3,     /* the slot pool has no free context left */
  GH_ERR_CAPACITY = 4,    /* token position >= slot capacity (seq_len) */
  GH_ERR_OOM = 5,         /* device memory (or the configured page budget) exhausted */
  GH_ERR_UNSUPPORTED = 6, /* shape / dtype combination has no kernel */
  GH_ERR_STATE = 7,       /* call out of order (e.g. a layer call before gh_attn_batch_begin) */
  GH_ERR_NOT_FOUND = 8    /* unknown context id */
} gh_status;

/* Reference DataType codes (src/models/types.hh:20-25). */
typedef enum gh_dtype
{
  GH_F16 = 0,
  GH_F32 = 1,
  GH_BF16 = 2
} gh_dtype;

/* Reference CopyType values (src/models/types.hh:132-138). */
typedef enum gh_copy_type
{
  GH_COPY_HOST_TO_DEVICE = 0,
  GH_COPY_DEVICE_TO_HOST = 1,
  GH_COPY_DEVICE_TO_DEVICE = 2,
  GH_COPY_HOST_TO_HOST = 3 /* rejected, as in the reference's CUDA backend (ops.cuh:490) */
} gh_copy_type;

/* How context slots are backed.  STATIC = every slot fully resident, like the reference's `Context`
 * (src/arch/cuda/llama2/ops.cuh:105-122); PAGED = address space reserved per slot and 2 MiB physical pages
 * mapped on demand, like `DynamicContext` (src/models/llama2/context.hh:192-249 over
 * src/arch/cuda/common/vmem.cuh:77-160). */
typedef enum gh_backing
{
  GH_BACKING_STATIC = 0,
  GH_BACKING_PAGED = 1
} gh_backing;

/* Shape and sizing.  Replaces the compile-time `ModelConfig` constants (src/models/llama2/variants.hh:9-33)
 * and the parts of `ConfigRuntime` the attention stage reads (src/models/llama2/base.hh:28-70):
 * concurrency_limit -> max_batch, max_context_count -> max_contexts, num_attention_layers_hosted ->
 * n_layers_hosted. */
typedef struct gh_attn_config
{
  uint32_t struct_size;     /* sizeof(gh_attn_config), for forward compatibility */
  uint32_t n_heads;         /* query heads */
  uint32_t n_kv_heads;      /* key/value heads; n_heads % n_kv_heads == 0, group size <= 16 */
  uint32_t head_size;       /* multiple of 8, <= 256 */
  uint32_t seq_len;         /* slot capacity in tokens */
  uint32_t n_layers_hosted; /* attention layers whose KV lives in every slot */
  uint32_t dtype;           /* gh_dtype of KV, q, xb and the RoPE tables */
  uint32_t max_batch;       /* <= 1024 (MAX_BATCH_SIZE, src/models/llama2/base.hh:26) */
  uint32_t max_contexts;    /* number of slots in the pool */
  uint32_t backing;         /* gh_backing */
  int32_t device;           /* CUDA device ordinal */
  uint32_t decode_chunk;    /* tokens per split of a long context; 0 = chosen per batch */
  uint64_t page_budget;     /* PAGED only: upper bound on mapped bytes, 0 = no bound */
  uint32_t force_generic;   /* 1 = always use the CUDA-core decode kernel (testing) */
  uint32_t pipeline_steps;  /* 1 = the append launch of a gh_attn_append / gh_attn_step call may start while the decode
                             * launch of the call before it on the same stream is still running (programmatic
                             * dependent launch).  For callers whose consecutive calls are independent of each other:
                             * another layer or another batch, and q / kv_new / xb buffers that the previous call
                             * neither reads nor writes.  0 (default) = calls execute strictly one after the other. */
} gh_attn_config;

typedef struct gh_attn_stats
{
  uint64_t kernel_launches; /* kernels this handle has launched since creation */
  uint64_t bytes_mapped;    /* device bytes currently backing slots */
  uint64_t bytes_reserved;  /* address space reserved for slots */
  uint64_t scratch_bytes;   /* split partials + batch metadata */
  uint32_t slots_free;
  uint32_t slots_allocated;
  uint32_t last_items;      /* work items (context splits) of the most recent batch */
  uint32_t last_chunk;      /* split length used by the most recent batch */
  uint32_t last_kernel;     /* 0 = CUDA-core decode kernel, 1 = TMA + warp tensor-core kernel, 2 = tcgen05 prefill kernel */
  uint32_t device_error;    /* sticky flag written by kernels whose bounded waits ran out */
  uint32_t last_split_contexts; /* contexts of the most recent batch that were cut into several work items */
  uint32_t pad;
  uint64_t batch_plans;     /* batch descriptions planned and uploaded since creation */
} gh_attn_stats;

/* ---- lifetime ------------------------------------------------------------------------------------- */

/* Replaces the `LlamaOperations( const ConfigRuntime& )` constructor (src/arch/cuda/llama2/ops.cuh:226-269)
 * plus the slot pre-allocation of `PreallocatingContextManager` (src/compute/contextman.hh:90-102). */
int gh_attn_create( const gh_attn_config* cfg, gh_attn_t* out );
int gh_attn_destroy( gh_attn_t h );
/* Text of the most recent failure on this handle (valid until the next call on it). */
const char* gh_attn_last_error( gh_attn_t h );
const char* gh_status_string( int status );
int gh_attn_get_stats( gh_attn_t h, gh_attn_stats* out );

/* Blocks the host until everything submitted to `stream` has finished (cudaStreamSynchronize).  For callers whose
 * other operations run on the host and are therefore not ordered by the stream; the reference's CUDA backend gets
 * the same effect from its blocking cudaMemcpy calls (src/arch/cuda/llama2/ops.cuh:455-492).  Returns GH_ERR_CUDA
 * when a kernel of this handle has reported a timed-out wait (see gh_attn_clear_device_error). */
int gh_attn_synchronize( gh_attn_t h, void* stream );

/* Every wait inside the kernels is bounded.  A kernel whose wait ran out raises gh_attn_stats.device_error and skips
 * its stores, so the outputs of that launch (and of launches that were already queued behind it) are not valid.
 * Once the host has seen the flag (gh_attn_synchronize or gh_attn_get_stats) every compute entry point of the handle
 * returns GH_ERR_CUDA until this call: it waits for the device to drain and clears the flag.  No reference
 * counterpart (the reference aborts the process on any CUDA error, src/arch/cuda/common/ops.cu:5-19). */
int gh_attn_clear_device_error( gh_attn_t h );

/* RoPE tables [seq_len][head_size/2] of the handle's dtype, device pointers, not owned.  They are what
 * `apply_rope` receives as freq_cis_real / freq_cis_imag (src/models/llama2/base.hh:110-112). */
int gh_attn_set_rope_tables( gh_attn_t h, const void* freq_cis_real, const void* freq_cis_imag );

/* ---- slot pool: PreallocatingContextManager (src/compute/contextman.hh:57-197) -------------------- */

/* get_context (contextman.hh:104-124): the slot already bound to context_id, else bind a free one. */
int gh_slot_acquire( gh_attn_t h, uint32_t context_id, int32_t* slot );
/* get_contexts (contextman.hh:127-171): all-or-nothing for a batch; context id 0 (NULL_CONTEXT,
 * src/models/types.hh:18) marks an inactive prompt and yields slot -1 (the "empty context"). */
int gh_slots_acquire_batch( gh_attn_t h, uint64_t batch, const uint32_t* context_ids, int32_t* slots );
int gh_slot_lookup( gh_attn_t h, uint32_t context_id, int32_t* slot );
/* release_context (contextman.hh:180-196; fatal in the reference, supported here): unbinds the id and, for
 * PAGED backing, unmaps the slot's pages at once and returns them to the pool.  Every kernel that reads or writes
 * the slot must have FINISHED (not merely been submitted) before this call: synchronize the streams that carry
 * them first, e.g. with gh_attn_synchronize.  Call it from the thread that owns the handle. */
int gh_slot_release( gh_attn_t h, uint32_t context_id );

/* ---- context views: Context / LayerContext / TokenContext (src/models/llama2/context.hh:61-190) ---- */

/* Context::prepare( layer, token_pos, can_release ) (context.hh:164-169, 221-248): make sure the slot can
 * hold token `pos` of hosted layer `layer`; can_release drops what the slot held before (its pages are unmapped
 * at once, so, as for gh_slot_release, all work on the slot must have finished). */
int gh_slot_prepare( gh_attn_t h, int32_t slot, uint32_t layer, uint32_t pos, int can_release );
/* Context::layer( l ) -> LayerContext (context.hh:171): device pointer of the layer's first token row. */
int gh_slot_layer_ptr( gh_attn_t h, int32_t slot, uint32_t layer, void** ptr );
/* LayerContext::token( t ).key() (context.hh:115-120, 79): device pointer of one token row. */
int gh_slot_token_ptr( gh_attn_t h, int32_t slot, uint32_t layer, uint32_t token, void** ptr );
/* Context::max_size( n_layers_hosted ) (context.hh:173). */
size_t gh_slot_bytes( gh_attn_t h );

/* ---- fused hot path -------------------------------------------------------------------------------- */

/* Alignment: q, the new K/V rows, xb and every cache row handed to the entry points of this and the next section
 * must be 16-byte aligned device pointers; a call with a misaligned one returns GH_ERR_INVALID and launches nothing.
 * Buffers from cudaMalloc and the rows of any model shape (row sizes are multiples of 16 bytes) always are. */

/* Per-batch set-up, the attention-relevant part of Llama2::forward_prelude / forward_attention
 * (src/models/llama2/model.hh:446-477, 611-628): records slot and token position of every prompt of the
 * batch (host arrays, as the reference's ScratchPad keeps them, src/models/llama2/base.hh:197-202), plans
 * the splits of long contexts and uploads the batch description on `stream`.  slot -1 = inactive prompt.
 * The per-layer calls below refer to the batch set up last; a per-layer call on another stream than `stream` must
 * be ordered behind the upload by the caller (an event recorded on `stream` after this call). */
int gh_attn_batch_begin( gh_attn_t h, uint64_t batch, const int32_t* slots, const uint32_t* pos, void* stream );

/* copy_kv_cache + apply_rope in one kernel (src/arch/amd64/llama2/ops.hh:335-352 and :300-333; order of
 * src/models/llama2/model.hh:345-364): row i of kv_new ([K,V], 2*kv_dim elements) goes to token pos[i] of
 * hosted layer `layer` of slot[i], K rotated on the way (fp32 arithmetic from the stored tables, one
 * rounding); V is copied bit for bit; q [batch][n_heads*head_size] is rotated in place. */
int gh_attn_append( gh_attn_t h, uint32_t layer, void* q_inout, const void* kv_new, void* stream );

/* attention_0_gemm + attention_softmax + attention_2_gemm in one kernel (src/arch/amd64/llama2/ops.hh:
 * 170-223, 283-298, 225-281): xb[i][head] = softmax_t( q.K_t / sqrt(head_size) ) . V over t <= pos[i], fp32
 * accumulation, no score matrix in memory.  Rows of inactive prompts are left untouched.
 * The kernel starts fetching the rows BEFORE each context's position while the library's kernels in front of it in
 * the stream (the append of this step, the tail of the previous layer's launch) are still running; it waits for them
 * before it touches the row at the position, q or xb.  So the cached rows before the position have to be in place
 * when gh_attn_batch_begin is called for the batch, which is the case for rows written by earlier steps, by
 * gh_attn_prefill_chunk calls issued before that gh_attn_batch_begin, by copies, or by kernels of the caller's. */
int gh_attn_decode( gh_attn_t h, uint32_t layer, const void* q, void* xb, void* stream );

/* gh_attn_append then gh_attn_decode: Llama2::attention_ops with the cache update of pre_attention_ops
 * (src/models/llama2/model.hh:345-387). */
int gh_attn_step( gh_attn_t h, uint32_t layer, void* q_inout, const void* kv_new, void* xb, void* stream );

/* The producer of the stage's inputs fused to the append, for the batch set up by gh_attn_batch_begin:
 *   xb = rmsnorm( x, rms_weight );  q = xb . wq^T;  kv = xb . wkv^T        Llama2::pre_attention_ops,
 *                                                                           src/models/llama2/model.hh:326-343
 *   copy_kv_cache( kv ) and apply_rope( q, K )                              model.hh:345-360
 * x is [batch][dim], rms_weight [dim], wq [dim][dim], wkv [2*kv_dim][dim] (row r = output feature r, as the
 * reference stores them: src/models/llama2/base.hh:477-499), q_out [batch][dim]: device pointers of the handle's
 * dtype.  On return (stream order) q_out holds the rotated queries and every active prompt's slot row at its
 * position holds the rotated K and the V; follow with gh_attn_decode.  The intermediate kv buffer of the reference does
 * not exist: K and V go from the tensor cores' accumulators into the slots.  Values are rounded to the storage type
 * where the reference rounds them (xb, q, kv before the rotation, and after it).
 * fp16 / bf16 with dim and kv_dim multiples of 128 only (GH_ERR_UNSUPPORTED otherwise).  The first call allocates
 * scratch (batch x dim activations and a few tens of MB of partial sums), which every later call of the handle
 * reuses: calls on different streams must not overlap (decode launches may, they have scratch sets of their own).
 * Batches of more than 256 prompts are processed in slices of 256, each streaming the weights once. */
int gh_attn_project_append( gh_attn_t h,
                            uint32_t layer,
                            const void* x,
                            const void* rms_weight,
                            const void* wq,
                            const void* wkv,
                            void* q_out,
                            void* stream );

/* A chunk of n_tokens consecutive prompt tokens per context in one call: token t of context i is appended at
 * position pos0[i] + t and attends causally over positions 0 .. pos0[i] + t.  q_inout and xb are
 * [n_ctx][n_tokens][n_heads*head_size], kv_new is [n_ctx][n_tokens][2*kv_dim] (device pointers); slots and pos0 are
 * host arrays.  The result equals n_tokens consecutive gh_attn_step calls.  The reference has no multi-token
 * operation: it feeds prompts one token per forward pass (src/worker/worker.hh:789-796,
 * src/frontend/infer.cc:124-126).  Does not disturb the batch set up by gh_attn_batch_begin.
 * fp16/bf16 with head size 128 runs on the tcgen05 tensor-core kernel (gh_attn_stats.last_kernel == 2); every other
 * case takes a slower kernel with the same result. */
int gh_attn_prefill_chunk( gh_attn_t h,
                           uint32_t layer,
                           uint64_t n_ctx,
                           const int32_t* slots,
                           const uint32_t* pos0,
                           uint32_t n_tokens,
                           void* q_inout,
                           const void* kv_new,
                           void* xb,
                           void* stream );

/* Llama2::forward_attention for one layer with HOST buffers (src/models/llama2/model.hh:630-722): q_host
 * [batch][n_heads*head_size] and kv_host [batch][2*kv_dim] of dtype `io_dtype` are converted and copied in
 * (convert_and_copy, src/arch/cuda/llama2/ops.cuh:455-492), the stage runs, and xb is converted and copied
 * back into xb_host.  Asynchronous: xb_host is valid once `stream` has drained.  Host buffers should be
 * pinned for the copies to overlap. */
int gh_attn_forward_attention_host( gh_attn_t h,
                                    uint32_t layer,
                                    uint32_t io_dtype,
                                    const void* q_host,
                                    const void* kv_host,
                                    void* xb_host,
                                    void* stream );

/* ---- the wire format: a serialized BatchedInferenceState ------------------------------------------- */

/* What travels between Glinthawk's workers: BatchedInferenceState::serialize() (src/models/common/state.hh:561-594)
 * = StateMetadata, then batch_size x PromptData, then the activations, queries and key-values buffers that the
 * metadata says are present, each [batch_size][row] of the state's dtype.  The two structs below restate the
 * reference's packed structs field for field (state.hh:17-50; PromptID is a 32-byte SHA-256, src/util/digest.hh:15-18;
 * stage codes are InferenceStage, src/models/types.hh:29-38). */
#pragma pack( push, 1 )
typedef struct gh_wire_metadata
{
  uint64_t id;
  uint32_t batch_size;
  uint8_t dtype; /* gh_dtype */
  uint32_t route_id;
  uint32_t model_id;
  uint32_t next_layer;
  uint8_t next_stage; /* gh_stage */
  int8_t next_tier;
  uint8_t next_rank;
  uint8_t has_activations;
  uint8_t has_queries;
  uint8_t has_kvs;
  uint8_t is_sharded;
} gh_wire_metadata; /* 32 bytes */

typedef struct gh_wire_prompt
{
  uint8_t active;
  uint8_t prompt_id[32];
  uint32_t context_id;
  uint32_t token;
  uint32_t token_pos;
  uint8_t temperature;
  uint32_t prompt_length;
  uint32_t max_completion_length;
  uint8_t finished;
  int8_t kv_tier;
  uint8_t kv_rank;
} gh_wire_prompt; /* 57 bytes */
#pragma pack( pop )

typedef enum gh_stage
{
  GH_STAGE_PRE_ATTENTION = 0,
  GH_STAGE_ATTENTION = 1,
  GH_STAGE_POST_ATTENTION = 2,
  GH_STAGE_CLASSIFICATION = 3
} gh_stage;

/* Llama2::forward_attention( states, contexts ) on the serialized state itself (src/models/llama2/model.hh:611-725,
 * with the context look-up of PreallocatingContextManager::get_contexts, src/compute/contextman.hh:127-171, done
 * here): `state` holds state_bytes of BatchedInferenceState::serialize() output with next_stage == Attention,
 * queries and key-values present.  For every active prompt the slot bound to its context_id is looked up (bound on
 * first use), prepared for token_pos (a prompt at position 0 of the first hosted layer starts its slot afresh,
 * model.hh:617-621), its new [K,V] row is appended and the attention output computed; inactive prompts are skipped.
 * The result is written where the reference writes it: over the queries buffer (model.hh:697-722), and next_stage
 * becomes PostAttention; everything else in `state` is left as it is, so the bytes are again a valid serialized
 * state.  `first_layer_hosted` is the model layer that hosted layer 0 stands for (next_layer is a model layer).
 * Blocking, like the reference's (it copies with cudaMemcpy); replaces the batch set up by gh_attn_batch_begin.
 * The state's dtype may differ from the handle's (the reference mixes fp16 pre-/post-attention with fp32 attention). */
int gh_attn_forward_attention_state( gh_attn_t h, uint32_t first_layer_hosted, void* state, size_t state_bytes, void* stream );

/* ---- the reference's five operations, argument for argument --------------------------------------- */
/* `token_rows` / `layer_bases` are HOST arrays of device pointers (what TokenContext::key() and
 * LayerContext::token(0).key() return); a null entry means "inactive, skip" (ops.hh:195,250,314,344).
 * `pos` is a host array.  These materialise the score matrix `att` [batch][n_heads][seq_len] exactly as the
 * reference does and round where it rounds.
 * When the pointers name rows of the handle's own slots (what the adapter's Context hands out), copy_kv_cache,
 * apply_rope and the fused attention call run on the kernels of gh_attn_append / gh_attn_decode, and the batch
 * description they share is planned and uploaded once per step, by the first call that names new slots or positions;
 * pointers into other device memory take a slower path that uploads the pointer array with every call. */

/* copy_kv_cache( token_contexts[], state_kv, batch ) — src/arch/cuda/llama2/ops.cuh:435-453. */
int gh_op_copy_kv_cache( gh_attn_t h, void* const* token_rows, const void* state_kv, uint64_t batch, void* stream );
/* apply_rope( batch, token_positions, freq_cis_real, freq_cis_imag, state_q, token_contexts[] ) —
 * src/arch/cuda/llama2/ops.cuh:413-433; arithmetic follows the amd64 rule (ops.hh:150-162). */
int gh_op_apply_rope( gh_attn_t h,
                      uint64_t batch,
                      const uint32_t* pos,
                      const void* freq_cis_real,
                      const void* freq_cis_imag,
                      void* state_q,
                      void* const* token_rows,
                      void* stream );
/* copy_kv_cache followed by apply_rope on the same token rows, as Llama2::pre_attention_ops and attention_ops issue
 * them back to back (src/models/llama2/model.hh:345-364), in one kernel launch: row i of state_kv goes to
 * token_rows[i] with K rotated on the way, state_q is rotated in place.  Same result as the two calls above. */
int gh_op_copy_kv_cache_apply_rope( gh_attn_t h,
                                    uint64_t batch,
                                    const uint32_t* pos,
                                    const void* freq_cis_real,
                                    const void* freq_cis_imag,
                                    void* state_q,
                                    void* const* token_rows,
                                    const void* state_kv,
                                    void* stream );
/* attention_0_gemm( query, layer_contexts[], att, batch, token_positions ) — ops.cuh:272-324. */
int gh_op_attention_0_gemm( gh_attn_t h,
                            const void* query,
                            const void* const* layer_bases,
                            void* att,
                            uint64_t batch,
                            const uint32_t* pos,
                            void* stream );
/* attention_softmax( att, token_positions, temp_buffer, batch ) — ops.cuh:385-411. temp_buffer is unused. */
int gh_op_attention_softmax( gh_attn_t h, void* att, const uint32_t* pos, void* temp_buffer, uint64_t batch, void* stream );
/* attention_2_gemm( att, layer_contexts[], xb, batch, token_positions ) — ops.cuh:326-383. */
int gh_op_attention_2_gemm( gh_attn_t h,
                            const void* att,
                            const void* const* layer_bases,
                            void* xb,
                            uint64_t batch,
                            const uint32_t* pos,
                            void* stream );
/* Fused stand-in for the three calls above with the same inputs: reads q and the layer contexts, writes xb,
 * never touches `att`.  What an adapter calls from attention_0_gemm when it does not need `att`. */
int gh_op_attention_fused( gh_attn_t h,
                           const void* query,
                           const void* const* layer_bases,
                           void* xb,
                           uint64_t batch,
                           const uint32_t* pos,
                           void* stream );
/* convert_and_copy<Dst,Src>( dst, src, n, CopyType ) — ops.cuh:455-492.  Blocking, like the reference's. */
int gh_op_convert_and_copy( gh_attn_t h,
                            void* dst,
                            uint32_t dst_dtype,
                            const void* src,
                            uint32_t src_dtype,
                            uint64_t n,
                            uint32_t copy_type );

/* Llama2::pre_attention_ops with the cache update, followed by apply_rope, argument for argument
 * (src/models/llama2/model.hh:326-360): the same fused producer as gh_attn_project_append, with the destination rows
 * given the way copy_kv_cache and apply_rope receive them (`token_rows`, null = inactive prompt; `pos`; the RoPE
 * tables).  state_q receives the rotated queries. */
int gh_op_project_append( gh_attn_t h,
                          uint64_t batch,
                          const void* x,
                          const void* rms_weight,
                          const void* wq,
                          const void* wkv,
                          void* state_q,
                          const uint32_t* pos,
                          const void* freq_cis_real,
                          const void* freq_cis_imag,
                          void* const* token_rows,
                          void* stream );

/* ---- decode attention without any allocation ------------------------------------------------------ */

/* Limits of gh_decode_noalloc; requests beyond them are refused. */
#define GH_NOALLOC_MAX_BATCH 64u       /* contexts per call */
#define GH_NOALLOC_MAX_ITEMS 128u      /* work items after cutting long contexts (the call adapts the cut to fit) */
#define GH_NOALLOC_MAX_HEADS 128u      /* query heads */
#define GH_NOALLOC_MAX_Q_ELEMS 8192u   /* n_heads * head_size */
#define GH_NOALLOC_SCRATCH_BYTES 4456448u /* size of the built-in scratch array, held per GPU */

typedef struct gh_noalloc_shape
{
  uint32_t struct_size; /* sizeof(gh_noalloc_shape) */
  uint32_t n_heads;
  uint32_t n_kv_heads;
  uint32_t head_size;
  uint32_t dtype;       /* gh_dtype of the KV rows, q and xb */
} gh_noalloc_shape;

/* This entry point has no counterpart in the reference.  It computes what gh_op_attention_fused computes — xb from
 * q and the layer contexts, for t <= pos[i] — but needs no handle and allocates nothing: not with cudaMalloc, not
 * through any library.  It is for code that runs where device allocation is off the table: inside a worker that
 * gave all of its GPU memory to weights and context slots at start-up and treats a failed allocation as fatal, or
 * inside a serving loop that must not trigger the device-wide synchronisation an allocation implies.  The scratch it
 * needs (split partial results and the batch description) lives in a fixed array of
 * GH_NOALLOC_SCRATCH_BYTES inside the library image; every GPU the library is used on holds that array until the
 * process exits.
 *
 * `layer_bases` is a host array of device pointers to the first token row of each context's layer (null = skip),
 * `pos` a host array, q and xb device pointers, exactly as for gh_op_attention_fused; the current CUDA device is
 * used.  The first call on a device resolves the array's device address; make it before any stream capture on
 * that device.  Do not call this entry point while a stream capture is in progress (it returns GH_ERR_STATE then):
 * each call uploads its batch description from the caller's stack.  Every call reuses the same array (nothing in
 * it needs clearing: all that a call reads it has written first), so calls whose kernels could run concurrently on
 * one GPU race with each other and must be ordered by the caller.
 * Returns GH_ERR_INVALID when a limit above is exceeded; gh_decode_noalloc_error() then names the limit. */
int gh_decode_noalloc( const gh_noalloc_shape* shape,
                       uint64_t batch,
                       const void* const* layer_bases,
                       const uint32_t* pos,
                       const void* q,
                       void* xb,
                       void* stream );
/* Message of the calling thread's most recent gh_decode_noalloc failure ("" after a success). */
const char* gh_decode_noalloc_error( void );

#ifdef __cplusplus
}
#endif

#endif /* GLINTHAWK_ATTN_H */
