/*
 * TEST INFRASTRUCTURE ONLY.  Compiles the adapter header (glinthawk_b200/cpp/glinthawk_b200_ops.hh) against the
 * reference tree and asserts, at compile time, that it satisfies the reference's own interface concepts
 * (src/models/llama2/ops/concept.hh:15-42, src/models/llama2/context.hh:17-45) — the same static_asserts the
 * reference places after its own backends (src/arch/amd64/llama2/ops.hh:79-85).  The non-attention operations
 * come from the reference's amd64 common operations here, because that base class is host-only and therefore
 * compiles without the reference's CUDA sources.
 *
 * When run (on a machine with a GPU) it drives one layer-step through the reference's view types and the adapter
 * and prints the attention output, which tests/test_gpu_adapter.py compares with the oracle.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_runtime_api.h>

#include "arch/amd64/common/ops.hh"
#include "glinthawk_b200_ops.hh"

namespace ref = glinthawk::models::llama2;

struct MiniG8 : public ref::configs::Llama2
{
  constexpr static uint64_t dim = 2048;
  constexpr static uint64_t kv_dim = 256;
  constexpr static uint64_t hidden_dim = 8192;
  constexpr static uint64_t n_layers = 2;
  constexpr static uint64_t head_size = 128;
  constexpr static uint64_t n_heads = 16;
  constexpr static uint64_t n_kv_heads = 2;
  constexpr static uint64_t gqa_size = 8;
  constexpr static uint64_t seq_len = 512;
  constexpr static bool wcls_present = false;
  constexpr static uint64_t attention_rounds = 1;
};

using DType = glinthawk::float16_t;
using Base = glinthawk::models::common::amd64::Operations<DType>;
using Ctx = ref::b200::Context<MiniG8, DType>;
using Ops = ref::b200::LlamaOperations<MiniG8, DType, Base>;

static_assert( ref::ContextConcept<Ctx, DType> );
static_assert( ref::LlamaOperationsConcept<Ops, DType, ref::ConfigRuntime<MiniG8>> );

// Reads one binary blob written by the test: [B u32][pos u32 x B][q][kv_new][fcr][fci][cache_0]...[cache_B-1]
int main( int argc, char** argv )
{
  if ( argc != 3 ) {
    std::fprintf( stderr, "usage: %s <case.bin> <out.bin>\n", argv[0] );
    return 2;
  }
  FILE* f = std::fopen( argv[1], "rb" );
  if ( !f )
    return 2;
  uint32_t B = 0;
  if ( std::fread( &B, 4, 1, f ) != 1 )
    return 2;
  std::vector<uint32_t> pos( B );
  if ( std::fread( pos.data(), 4, B, f ) != B )
    return 2;
  auto read_dev = [&]( size_t elems ) {
    std::vector<DType> host( elems );
    if ( std::fread( host.data(), sizeof( DType ), elems, f ) != elems )
      std::abort();
    DType* d = nullptr;
    if ( cudaMalloc( reinterpret_cast<void**>( &d ), elems * sizeof( DType ) ) != cudaSuccess )
      std::abort();
    cudaMemcpy( d, host.data(), elems * sizeof( DType ), cudaMemcpyHostToDevice );
    return d;
  };
  DType* q = read_dev( B * MiniG8::dim );
  DType* kv = read_dev( B * MiniG8::kv_dim * 2 );
  DType* fcr = read_dev( MiniG8::seq_len * MiniG8::head_size / 2 );
  DType* fci = read_dev( MiniG8::seq_len * MiniG8::head_size / 2 );

  // settings as the reference would build them: every stage of both layers hosted here
  alignas( ref::ConfigRuntime<MiniG8> ) static unsigned char raw[sizeof( ref::ConfigRuntime<MiniG8> )] {};
  auto& settings = *reinterpret_cast<ref::ConfigRuntime<MiniG8>*>( raw );
  auto& table = const_cast<std::remove_const_t<decltype( settings.hosting_table_ )>&>( settings.hosting_table_ );
  for ( auto& row : table )
    row.fill( true );
  const_cast<uint64_t&>( settings.concurrency_limit ) = B;
  const_cast<uint64_t&>( settings.max_context_count ) = B;
  settings.num_attention_layers_hosted_ = MiniG8::n_layers;

  Ops ops { settings };
  std::vector<std::unique_ptr<Ctx>> contexts;
  std::vector<Ctx::LayerContextType> layers( B );
  std::vector<Ctx::TokenContextType> tokens( B );
  const int layer = 1;
  for ( uint32_t i = 0; i < B; i++ ) {
    contexts.emplace_back( std::make_unique<Ctx>( settings ) );
    if ( !contexts[i]->prepare( layer, pos[i], false ) )
      return 3;
    layers[i] = contexts[i]->layer( layer );
    tokens[i] = layers[i].token( static_cast<int>( pos[i] ) );
    const size_t elems = static_cast<size_t>( pos[i] + 1 ) * MiniG8::kv_dim * 2;
    std::vector<DType> host( elems );
    if ( std::fread( host.data(), sizeof( DType ), elems, f ) != elems )
      return 2;
    cudaMemcpy( layers[i].token( 0 ).key(), host.data(), elems * sizeof( DType ), cudaMemcpyHostToDevice );
  }
  std::fclose( f );

  DType* xb = nullptr;
  cudaMalloc( reinterpret_cast<void**>( &xb ), B * MiniG8::dim * sizeof( DType ) );
  // the order Llama2 fixes (src/models/llama2/model.hh:345-387)
  ops.copy_kv_cache( tokens.data(), kv, B );
  ops.apply_rope( B, pos.data(), fcr, fci, q, tokens.data() );
  ops.attention_0_gemm( q, layers.data(), nullptr, B, pos.data() );
  ops.attention_softmax( nullptr, pos.data(), nullptr, B );
  ops.attention_2_gemm( nullptr, layers.data(), xb, B, pos.data() );
  if ( cudaDeviceSynchronize() != cudaSuccess )
    return 4;

  std::vector<DType> out( B * MiniG8::dim );
  cudaMemcpy( out.data(), xb, out.size() * sizeof( DType ), cudaMemcpyDeviceToHost );
  FILE* o = std::fopen( argv[2], "wb" );
  std::fwrite( out.data(), sizeof( DType ), out.size(), o );
  std::fclose( o );
  std::printf( "adapter layer-step done: %u contexts\n", B );
  return 0;
}
