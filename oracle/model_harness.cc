/*
 * TEST INFRASTRUCTURE ONLY.  Runs the reference project's OWN model class, `Llama2<Config, DType, Ops, Context>`
 * (src/models/llama2/model.hh), end to end on a tiny Llama-2 shape, twice:
 *
 *   impl "ref"   Ops = the reference's amd64 operations, Context = the reference's amd64 context (all CPU)
 *   impl "b200"  Ops = the adapter of glinthawk_b200/cpp/glinthawk_b200_ops.hh, Context = the adapter's context:
 *                the attention stage (copy_kv_cache, apply_rope, the three attention operations, the KV slots)
 *                runs on the GPU through the C ABI; every other operation (matmul, rmsnorm, ...) is still the
 *                reference's amd64 code, working on CUDA managed memory so that both sides see the same buffers.
 *
 * Both are driven exactly like the reference's `infer` front end drives a batch (src/frontend/infer.cc:93-153):
 * prompts are fed one token per forward pass, then tokens are generated greedily.  The program writes, per
 * forward pass, the logits of every prompt and the chosen tokens, and at the end the KV cache of every context.
 * tests/test_gpu_model.py compares the two runs.
 */
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "arch/amd64/llama2/ops.hh"
#include "glinthawk_b200_ops.hh"
#include "models/llama2/model.hh"

namespace gl = glinthawk;
namespace ref = glinthawk::models::llama2;

struct Tiny15M : public ref::configs::Llama2 // the stories15M shape
{
  constexpr static uint64_t dim = 288;
  constexpr static uint64_t kv_dim = 288;
  constexpr static uint64_t hidden_dim = 768;
  constexpr static uint64_t n_layers = 6;
  constexpr static uint64_t head_size = 48;
  constexpr static uint64_t n_heads = 6;
  constexpr static uint64_t n_kv_heads = 6;
  constexpr static uint64_t gqa_size = 1;
  constexpr static uint64_t seq_len = 256;
  constexpr static bool wcls_present = false;
  constexpr static uint64_t attention_rounds = 1;
};

using DType = gl::float32_t;

// The reference's CPU operations on memory the GPU can also touch.
template<typename T>
class ManagedHostOperations : public gl::models::common::amd64::Operations<T>
{
public:
  struct Deleter
  {
    void operator()( T* p ) const { cudaFree( p ); }
  };
  using DeviceUniquePtr = std::unique_ptr<T, Deleter>;

  DeviceUniquePtr device_allocate( const uint64_t size_bytes ) const
  {
    void* p = nullptr;
    CHECK_EQ( cudaMallocManaged( &p, size_bytes ), cudaSuccess ) << "cudaMallocManaged failed";
    std::memset( p, 0, size_bytes );
    return DeviceUniquePtr { static_cast<T*>( p ) };
  }
};

using RefOps = ref::amd64::LlamaOperations<Tiny15M, DType>;
using RefCtx = ref::amd64::Context<Tiny15M, DType>;
using B200Ops = ref::b200::LlamaOperations<Tiny15M, DType, ManagedHostOperations<DType>>;
using B200Ctx = ref::b200::Context<Tiny15M, DType>;

template<typename Ops, typename Ctx>
class Model : public ref::Llama2<Tiny15M, DType, Ops, Ctx>
{
public:
  using ref::Llama2<Tiny15M, DType, Ops, Ctx>::Llama2;
  const DType* logits() const { return this->scratchpad_.logits; }
};

template<typename Ops, typename Ctx>
int run( const std::string& model_dir, const std::string& prompts_path, const int n_generate, const std::string& out_path )
{
  // prompts: [B u32] then per context [len u32][tokens u32 x len]
  std::ifstream pf { prompts_path, std::ios::binary };
  uint32_t B = 0;
  pf.read( reinterpret_cast<char*>( &B ), 4 );
  std::vector<std::vector<uint32_t>> prompts( B );
  uint32_t max_len = 0;
  for ( auto& p : prompts ) {
    uint32_t len = 0;
    pf.read( reinterpret_cast<char*>( &len ), 4 );
    p.resize( len );
    pf.read( reinterpret_cast<char*>( p.data() ), 4 * len );
    max_len = std::max( max_len, len );
  }

  std::array<std::array<bool, 4>, Tiny15M::n_layers> hosting {};
  for ( auto& row : hosting )
    row.fill( true );
  Model<Ops, Ctx> model { model_dir, hosting, B, B, false };
  if constexpr ( std::is_same_v<Ops, B200Ops> )
    model.ops().set_blocking( true ); // the CPU operations read what the GPU wrote

  using State = gl::models::BatchedInferenceState<Tiny15M>;
  State state { B, gl::DataType::Float32, {}, {} };
  state.set_next_layer( 0 );
  state.set_next_stage( gl::models::InferenceStage::PreAttention );
  std::vector<std::shared_ptr<Ctx>> contexts;
  for ( uint32_t i = 0; i < B; i++ ) {
    contexts.push_back( std::make_shared<Ctx>( model.settings() ) );
    state.set_prompt( i, {}, gl::ContextID { i + 1 }, prompts[i][0], 0, 0.0f, prompts[i].size(), n_generate, 0, 0 );
  }

  FILE* out = std::fopen( out_path.c_str(), "wb" );
  const uint32_t steps = max_len + n_generate - 1;
  std::fwrite( &steps, 4, 1, out );
  for ( uint32_t step = 0; step < steps; step++ ) {
    model.forward( state, contexts );
    if constexpr ( std::is_same_v<Ops, B200Ops> )
      cudaDeviceSynchronize();
    std::fwrite( model.logits(), sizeof( DType ), static_cast<size_t>( B ) * Tiny15M::vocab_size, out );
    for ( uint32_t i = 0; i < B; i++ ) {
      // feed the next prompt token while the prompt lasts, else keep the generated one (infer.cc:124-128)
      if ( state.token_pos( i ) < prompts[i].size() )
        state.set_token( i, prompts[i][state.token_pos( i )] );
      const uint32_t tok = state.token( i ), pos = state.token_pos( i );
      std::fwrite( &tok, 4, 1, out );
      std::fwrite( &pos, 4, 1, out );
    }
  }

  // KV cache: per context, per layer, the rows written so far
  const size_t row = Tiny15M::kv_dim * 2;
  std::vector<DType> host( row * Tiny15M::seq_len );
  for ( uint32_t i = 0; i < B; i++ ) {
    const uint32_t rows = state.token_pos( i );
    std::fwrite( &rows, 4, 1, out );
    for ( uint32_t l = 0; l < Tiny15M::n_layers; l++ ) {
      const DType* src = contexts[i]->layer( l ).token( 0 ).key();
      if constexpr ( std::is_same_v<Ops, B200Ops> )
        cudaMemcpy( host.data(), src, rows * row * sizeof( DType ), cudaMemcpyDeviceToHost );
      else
        std::memcpy( host.data(), src, rows * row * sizeof( DType ) );
      std::fwrite( host.data(), sizeof( DType ), rows * row, out );
    }
  }
  std::fclose( out );
  std::printf( "%u contexts, %u forward passes\n", B, steps );
  return 0;
}

// The wire format of gh_attn_forward_attention_state is the reference's own: the restated structs must match the
// reference's packed structs byte for byte (src/models/common/state.hh:17-50).
namespace wire = glinthawk::models;
static_assert( sizeof( gh_wire_metadata ) == sizeof( wire::StateMetadata ) && sizeof( gh_wire_prompt ) == sizeof( wire::PromptData ) );
static_assert( offsetof( gh_wire_metadata, dtype ) == offsetof( wire::StateMetadata, dtype )
               && offsetof( gh_wire_metadata, next_layer ) == offsetof( wire::StateMetadata, next_layer )
               && offsetof( gh_wire_metadata, next_stage ) == offsetof( wire::StateMetadata, next_stage )
               && offsetof( gh_wire_metadata, has_queries ) == offsetof( wire::StateMetadata, has_queries )
               && offsetof( gh_wire_metadata, is_sharded ) == offsetof( wire::StateMetadata, is_sharded ) );
static_assert( offsetof( gh_wire_prompt, context_id ) == offsetof( wire::PromptData, context_id )
               && offsetof( gh_wire_prompt, token_pos ) == offsetof( wire::PromptData, token_pos )
               && offsetof( gh_wire_prompt, kv_rank ) == offsetof( wire::PromptData, kv_rank ) );
static_assert( GH_STAGE_ATTENTION == static_cast<int>( wire::InferenceStage::Attention )
               && GH_STAGE_POST_ATTENTION == static_cast<int>( wire::InferenceStage::PostAttention ) );

int main( int argc, char** argv )
{
  if ( argc != 6 ) {
    std::fprintf( stderr, "usage: %s <ref|b200> <model_dir> <prompts.bin> <n_generate> <out.bin>\n", argv[0] );
    return 2;
  }
  const std::string impl = argv[1];
  const int n_generate = std::atoi( argv[4] );
  if ( impl == "ref" )
    return run<RefOps, RefCtx>( argv[2], argv[3], n_generate, argv[5] );
  if ( impl == "b200" )
    return run<B200Ops, B200Ctx>( argv[2], argv[3], n_generate, argv[5] );
  return 2;
}
