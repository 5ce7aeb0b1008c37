// Host-side launch interface of the attention-stage kernels.  Each launcher returns the cudaError_t of the
// launch (cudaSuccess when the batch is empty and nothing was launched) and adds the number of kernels it
// launched to *launches.
#pragma once

#include <cuda.h>

#include "gh_common.cuh"

namespace gh {

struct AppendArgs
{
  Shape sh;
  uint32_t dtype;
  uint32_t batch;
  uint32_t tokens_per_ctx; // 1 for a decode step; T for a prefill chunk (token t of context i goes to pos + t)
  const CtxMeta* ctx;   // device, [batch]; used when token_rows == nullptr
  void* const* token_rows; // device array of row pointers (the reference's token contexts), or nullptr
  const uint32_t* pos;  // device, [batch]; used together with token_rows
  char* arena;
  long long layer_off;  // byte offset of the hosted layer inside a slot
  void* q;              // [batch][n_heads * head_size], rotated in place; may be nullptr (K/V only)
  const void* kv_new;   // [batch][2 * kv_dim]; nullptr = rotate the row already in the slot (apply_rope alone)
  const void* rope_cos; // [seq_len][head_size / 2]; nullptr = copy without rotation (copy_kv_cache alone)
  const void* rope_sin;
  uint32_t dependent_launch; // 0 = ordinary launch; 1 = programmatic dependent of the kernel before it in the stream that
                             // waits for that kernel to complete before it touches anything; 2 = the same without the
                             // wait (gh_attn_config.pipeline_steps: the caller declared consecutive calls independent)
};

struct DecodeArgs
{
  Shape sh;
  uint32_t dtype;
  const CtxMeta* ctx;
  const WorkItem* items;
  uint32_t n_items;
  const char* arena;
  long long layer_off;
  const void* q;
  void* xb;
  float* part_o;
  float* part_ml;
  uint32_t* arrivals;       // [batch][n_kv_heads] arrival counts of the blocks of cut contexts, all zero between
                            // launches (tensor-core kernel: the last block to arrive combines the records itself)
  const int32_t* split_ctx; // batch indices of the contexts that were cut into several items
  uint32_t n_split_ctx;
  uint32_t* dev_error;
  uint32_t sm_count;
  uint32_t chunk_tokens; // 0 = decode step; T = prefill chunk of T tokens per context (tensor-core kernel only)
  int32_t layer_row;     // tcgen05 prompt-chunk kernel: layer_off in rows; its items carry the arena row of their
                         // context's layer 0 in t_begin, so that a block needs no second look-up before its first copy
  uint32_t trigger_early; // 1 = release the next programmatic dependent launch as soon as every block has started
  uint32_t stream_old_rows_early; // 1 = the kernels before this one in the stream write, of the contexts' K/V, only the
                                  // row at each context's position (a decode step's append): the tensor-core kernel
                                  // then fetches the rows before it without waiting for those kernels
};

struct ScoreArgs // the reference's three unfused operations
{
  Shape sh;
  uint32_t dtype;
  uint32_t batch;
  const void* const* layer_bases; // device array [batch] of layer base pointers, null = skip
  const uint32_t* pos;            // device [batch]
  const void* q;
  void* att; // [batch][n_heads][seq_len]
  void* xb;
};

cudaError_t launch_append( const AppendArgs& a, cudaStream_t st, uint64_t* launches );
cudaError_t launch_decode_generic( const DecodeArgs& a, cudaStream_t st, uint64_t* launches );
// TMA + tensor-core decode kernel; `kv_map` describes the whole arena as [rows][2 * kv_dim].
bool decode_mma_supported( const Shape& sh, uint32_t dtype );
bool decode_mma_chunk_supported( const Shape& sh ); // prefill-chunk mode packs 16 / group tokens into a tile
cudaError_t decode_mma_prepare(); // one-time function attributes
cudaError_t launch_decode_mma( const DecodeArgs& a, const CUtensorMap* kv_map, cudaStream_t st, uint64_t* launches );
uint32_t decode_mma_tile_tokens(); // work items start on multiples of this
uint32_t decode_mma_box_rows();    // token rows of the TMA box the descriptor must be encoded with

// tcgen05 kernel for prompt chunks: work item = (context, query block of 128 / group tokens).  q_map and xb_map
// describe the chunk's q and xb buffers as [contexts][chunk tokens][heads][128] with the box
// [1][128 / group][group][64] and the 128-byte swizzle.
bool prefill_umma_supported( const Shape& sh, uint32_t dtype );
uint32_t prefill_umma_tokens_per_item( const Shape& sh );
cudaError_t prefill_umma_prepare();
cudaError_t launch_prefill_umma( const DecodeArgs& a, const CUtensorMap* kv_map, const CUtensorMap* q_map,
                                 const CUtensorMap* xb_map, cudaStream_t st, uint64_t* launches );

// The stage's producer (rmsnorm + q / kv projection) with the RoPE + append epilogue, on tcgen05.
struct ProjectArgs
{
  Shape sh;
  uint32_t dtype;
  uint32_t batch;  // batch rows covered by this launch (at most project_max_rows())
  uint32_t batch0; // index of the first of them in the whole batch
  uint32_t nb;     // batch rounded up to a multiple of 16: the MMA's N
  uint32_t dim, n_tiles, q_tiles, kblocks, units_per_cta, max_segs; // set by project_plan()
  const CtxMeta* ctx;      // device, whole batch; used when token_rows == nullptr
  void* const* token_rows; // device array of destination row pointers (the reference's token contexts), or nullptr
  const uint32_t* pos;     // device, [batch]; used together with token_rows
  char* arena;
  long long layer_off;
  void* q_out;          // [whole batch][dim]
  const void* rope_cos; // [seq_len][head_size / 2]
  const void* rope_sin;
  float* ws;           // project_workspace_bytes()
  uint32_t* dev_error;
};
bool project_supported( const Shape& sh, uint32_t dtype );
uint32_t project_max_rows();
cudaError_t project_prepare();
void project_plan( const Shape& sh, uint32_t sm_count, ProjectArgs* a, uint32_t* grid );
size_t project_workspace_bytes( const ProjectArgs& a );
// host copy of the walk every role of CTA `cta` does: records {tile, k0, k1, piece index, pieces of the tile}
uint32_t project_pieces( const ProjectArgs& a, uint32_t cta, int32_t* out, uint32_t cap );
cudaError_t launch_rmsnorm( void* out, const void* x, const void* weight, uint32_t rows, uint32_t dim, uint32_t dtype,
                            cudaStream_t st, uint64_t* launches );
// wq_map / wkv_map: the weight matrices as [rows][dim] with box [128][64]; xb_map: the normalised activations as
// [batch][dim] with box [nb][64]; all with the 128-byte swizzle.
cudaError_t launch_project( const ProjectArgs& a, uint32_t grid, const CUtensorMap* wq_map, const CUtensorMap* wkv_map,
                            const CUtensorMap* xb_map, cudaStream_t st, uint64_t* launches );

cudaError_t launch_scores( const ScoreArgs& a, cudaStream_t st, uint64_t* launches );  // attention_0_gemm
cudaError_t launch_softmax( const ScoreArgs& a, cudaStream_t st, uint64_t* launches ); // attention_softmax
cudaError_t launch_values( const ScoreArgs& a, cudaStream_t st, uint64_t* launches );  // attention_2_gemm

cudaError_t launch_convert( void* dst, uint32_t dst_dtype, const void* src, uint32_t src_dtype, uint64_t n,
                            cudaStream_t st, uint64_t* launches );
cudaError_t launch_fill_normal( void* dst, uint64_t n, uint32_t dtype, uint64_t seed, uint64_t offset,
                                cudaStream_t st, uint64_t* launches );

} // namespace gh
