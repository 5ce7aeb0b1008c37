/*
 * TEST INFRASTRUCTURE ONLY — never linked into, imported by, or called from the product path.
 *
 * C-callable harness around the reference project's OWN amd64/OpenMP attention operations
 * (glinthawk::models::llama2::amd64::LlamaOperations, src/arch/amd64/llama2/ops.hh:170-368) and its KV views
 * (src/models/llama2/context.hh:61-132).  It is compiled against the reference tree where it lies (see
 * oracle/build.py); no reference source is copied into this repository.  The operations are templates over a
 * compile-time `Config`, so this file defines Config structs for the shapes the parity tests and the CPU
 * baseline use (the reference's own variant list, src/models/llama2/variants.hh:37-186, lacks most of them)
 * and instantiates each for fp32 and fp16 (the amd64 backend has no bf16, src/arch/float.hh:13).
 *
 * Exports:
 *   ghref_shape_count / ghref_shape_name / ghref_shape_dims   the shape table
 *   ghref_op          one reference operation on caller buffers
 *   ghref_layer_step  the five operations in model order (src/models/llama2/model.hh:345-387)
 *   ghref_pre_attention  rmsnorm + the q and kv projections that feed the stage (model.hh:326-343)
 *   ghref_threads     omp_get_max_threads()
 */
#include <cstdint>
#include <cstring>
#include <omp.h>
#include <vector>

#include "arch/amd64/llama2/ops.hh"

namespace ref = glinthawk::models::llama2;

namespace {

template<uint64_t DIM, uint64_t HQ, uint64_t HKV, uint64_t S, uint64_t L>
struct Shape : public ref::configs::Llama2
{
  constexpr static uint64_t dim = DIM;
  constexpr static uint64_t n_heads = HQ;
  constexpr static uint64_t n_kv_heads = HKV;
  constexpr static uint64_t gqa_size = HQ / HKV;
  constexpr static uint64_t kv_dim = DIM / gqa_size;
  constexpr static uint64_t head_size = DIM / HQ;
  constexpr static uint64_t hidden_dim = 4 * DIM;
  constexpr static uint64_t n_layers = L;
  constexpr static uint64_t seq_len = S;
  constexpr static bool wcls_present = false;
  constexpr static uint64_t attention_rounds = 1;
};

// name, dim, query heads, kv heads, slot capacity (seq_len), layers
#define GHREF_SHAPES( X )                                                                                              \
  X( tiny15m, 288, 6, 6, 256, 6 )                                                                                      \
  X( s110m, 768, 12, 12, 1024, 12 )                                                                                    \
  X( l7b_4k, 4096, 32, 32, 4096, 32 )                                                                                  \
  X( l13b_4k, 5120, 40, 40, 4096, 40 )                                                                                 \
  X( l70b_4k, 8192, 64, 8, 4096, 80 )                                                                                  \
  X( l3_8b_8k, 4096, 32, 8, 8192, 32 )                                                                                 \
  X( l3_405b, 16384, 128, 8, 2048, 126 )                                                                               \
  X( mini_mha, 512, 4, 4, 512, 2 )                                                                                     \
  X( mini_g4, 1024, 8, 2, 512, 2 )                                                                                     \
  X( mini_g8, 2048, 16, 2, 512, 2 )                                                                                    \
  X( mini_g16, 4096, 32, 2, 512, 2 )

struct ShapeInfo
{
  const char* name;
  uint64_t dim, n_heads, n_kv_heads, head_size, seq_len, n_layers;
};

#define X_INFO( n, d, hq, hkv, s, l ) { #n, d, hq, hkv, d / hq, s, l },
const ShapeInfo kShapes[] = { GHREF_SHAPES( X_INFO ) };
#undef X_INFO
constexpr int kShapeCount = sizeof( kShapes ) / sizeof( kShapes[0] );

// The non-empty constructors of the reference's views are protected (only Context may build them); a derived
// type may call them, and slicing back to the base gives exactly the object the operations expect.
template<typename Config, typename DType>
struct LayerView : public ref::LayerContext<Config, DType>
{
  explicit LayerView( DType* p )
    : ref::LayerContext<Config, DType>( p )
  {
  }
};

enum Op : int
{
  OP_COPY_KV_CACHE = 0,
  OP_APPLY_ROPE = 1,
  OP_ATTENTION_0_GEMM = 2,
  OP_ATTENTION_SOFTMAX = 3,
  OP_ATTENTION_2_GEMM = 4,
  OP_LAYER_STEP = 5,
};

template<typename Config, typename DType>
int run( int op,
         uint64_t B,
         const uint32_t* pos,
         void* const* layer_bases,
         const void* fcr,
         const void* fci,
         void* q,
         const void* kv_new,
         void* att,
         void* xb )
{
  using Ops = ref::amd64::LlamaOperations<Config, DType>;
  using Layer = ref::LayerContext<Config, DType>;
  using Token = ref::TokenContext<Config, DType>;

  // The operations' constructor takes the runtime settings by reference and ignores them
  // (src/arch/amd64/llama2/ops.hh:32).  GCC 13 refuses the settings' default constructor (a const member
  // without initialiser), and the other constructor wants a CONFIG file on disk, so hand it zeroed storage.
  alignas( ref::ConfigRuntime<Config> ) static unsigned char settings_storage[sizeof( ref::ConfigRuntime<Config> )] {};
  Ops ops { *reinterpret_cast<const ref::ConfigRuntime<Config>*>( settings_storage ) };

  std::vector<Layer> layers( B );
  std::vector<Token> tokens( B );
  for ( uint64_t i = 0; i < B; i++ ) {
    layers[i] = LayerView<Config, DType>( static_cast<DType*>( layer_bases[i] ) );
    tokens[i] = layers[i].token( static_cast<int>( pos[i] ) );
  }

  auto Q = static_cast<DType*>( q );
  auto ATT = static_cast<DType*>( att );
  auto XB = static_cast<DType*>( xb );

  if ( op == OP_COPY_KV_CACHE or op == OP_LAYER_STEP )
    ops.copy_kv_cache( tokens.data(), static_cast<const DType*>( kv_new ), B );
  if ( op == OP_APPLY_ROPE or op == OP_LAYER_STEP )
    ops.apply_rope( B, pos, static_cast<const DType*>( fcr ), static_cast<const DType*>( fci ), Q, tokens.data() );
  if ( op == OP_ATTENTION_0_GEMM or op == OP_LAYER_STEP )
    ops.attention_0_gemm( Q, layers.data(), ATT, B, pos );
  if ( op == OP_ATTENTION_SOFTMAX or op == OP_LAYER_STEP )
    ops.attention_softmax( ATT, pos, nullptr, B );
  if ( op == OP_ATTENTION_2_GEMM or op == OP_LAYER_STEP )
    ops.attention_2_gemm( ATT, layers.data(), XB, B, pos );
  return 0;
}

template<typename Config>
int run_dtype( int dtype,
               int op,
               uint64_t B,
               const uint32_t* pos,
               void* const* layer_bases,
               const void* fcr,
               const void* fci,
               void* q,
               const void* kv_new,
               void* att,
               void* xb )
{
  switch ( dtype ) { // reference DataType codes, src/models/types.hh:20-25
    case 0: return run<Config, glinthawk::float16_t>( op, B, pos, layer_bases, fcr, fci, q, kv_new, att, xb );
    case 1: return run<Config, glinthawk::float32_t>( op, B, pos, layer_bases, fcr, fci, q, kv_new, att, xb );
    default: return -2;
  }
}

// pre_attention_ops without the cache update (src/models/llama2/model.hh:326-343): the reference's own rmsnorm and
// matmul templates (src/arch/amd64/common/ops.hh:141-170, 212-229).
template<typename Config, typename DType>
int run_pre_attention( uint64_t B, const void* x, const void* rms_w, const void* wq, const void* wkv, void* xb, void* q, void* kv )
{
  using Ops = ref::amd64::LlamaOperations<Config, DType>;
  alignas( ref::ConfigRuntime<Config> ) static unsigned char settings_storage[sizeof( ref::ConfigRuntime<Config> )] {};
  Ops ops { *reinterpret_cast<const ref::ConfigRuntime<Config>*>( settings_storage ) };
  ops.template rmsnorm<Config::dim>(
    static_cast<DType*>( xb ), static_cast<const DType*>( x ), nullptr, static_cast<const DType*>( rms_w ), B );
  ops.template matmul<Config::dim, Config::dim>(
    static_cast<DType*>( q ), static_cast<const DType*>( xb ), static_cast<const DType*>( wq ), B );
  ops.template matmul<Config::dim, Config::kv_dim * 2>(
    static_cast<DType*>( kv ), static_cast<const DType*>( xb ), static_cast<const DType*>( wkv ), B );
  return 0;
}

template<typename Config>
int run_pre_attention_dtype( int dtype, uint64_t B, const void* x, const void* rms_w, const void* wq, const void* wkv, void* xb,
                             void* q, void* kv )
{
  switch ( dtype ) {
    case 0: return run_pre_attention<Config, glinthawk::float16_t>( B, x, rms_w, wq, wkv, xb, q, kv );
    case 1: return run_pre_attention<Config, glinthawk::float32_t>( B, x, rms_w, wq, wkv, xb, q, kv );
    default: return -2;
  }
}

} // namespace

extern "C" {

int ghref_shape_count()
{
  return kShapeCount;
}

const char* ghref_shape_name( int idx )
{
  return ( idx >= 0 and idx < kShapeCount ) ? kShapes[idx].name : nullptr;
}

// out[6] = dim, n_heads, n_kv_heads, head_size, seq_len, n_layers
int ghref_shape_dims( int idx, uint64_t* out )
{
  if ( idx < 0 or idx >= kShapeCount )
    return -1;
  const auto& s = kShapes[idx];
  out[0] = s.dim, out[1] = s.n_heads, out[2] = s.n_kv_heads, out[3] = s.head_size, out[4] = s.seq_len,
  out[5] = s.n_layers;
  return 0;
}

int ghref_threads()
{
  return omp_get_max_threads();
}

// Runs one reference operation (op 0..4) or the whole layer-step (op 5) for shape `idx`.
// Buffers an operation does not touch may be null.  `att` holds B * n_heads * seq_len elements.
int ghref_op( int idx,
              int dtype,
              int op,
              uint64_t B,
              const uint32_t* pos,
              void* const* layer_bases,
              const void* fcr,
              const void* fci,
              void* q,
              const void* kv_new,
              void* att,
              void* xb )
{
  int i = 0;
#define X_RUN( n, d, hq, hkv, s, l )                                                                                   \
  if ( idx == i++ )                                                                                                    \
    return run_dtype<Shape<d, hq, hkv, s, l>>( dtype, op, B, pos, layer_bases, fcr, fci, q, kv_new, att, xb );
  GHREF_SHAPES( X_RUN )
#undef X_RUN
  return -1;
}

int ghref_pre_attention( int idx,
                         int dtype,
                         uint64_t B,
                         const void* x,
                         const void* rms_w,
                         const void* wq,
                         const void* wkv,
                         void* xb,
                         void* q,
                         void* kv )
{
  int i = 0;
#define X_RUN( n, d, hq, hkv, s, l )                                                                                   \
  if ( idx == i++ )                                                                                                    \
    return run_pre_attention_dtype<Shape<d, hq, hkv, s, l>>( dtype, B, x, rms_w, wq, wkv, xb, q, kv );
  GHREF_SHAPES( X_RUN )
#undef X_RUN
  return -1;
}

int ghref_layer_step( int idx,
                      int dtype,
                      uint64_t B,
                      const uint32_t* pos,
                      void* const* layer_bases,
                      const void* fcr,
                      const void* fci,
                      void* q,
                      const void* kv_new,
                      void* att,
                      void* xb )
{
  return ghref_op( idx, dtype, OP_LAYER_STEP, B, pos, layer_bases, fcr, fci, q, kv_new, att, xb );
}

} // extern "C"
