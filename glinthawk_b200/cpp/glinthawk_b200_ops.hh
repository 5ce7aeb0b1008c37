// Adapter that lets Glinthawk's own model code use the B200 attention stage.
//
// A maintainer drops this header into the reference tree (e.g. as src/arch/b200/llama2/ops.hh), links
// libglinthawk_attn.so, and instantiates
//
//     Llama2<Config, DType, b200::LlamaOperations<Config, DType, common::cuda::Operations<DType>>,
//            b200::Context<Config, DType>>
//
// exactly where the CUDA backend is instantiated today (DECLARE_MODEL, src/models/llama2/model.hh:810-877).
// `Base` supplies the non-attention operations (matmul, rmsnorm, ...), which this adapter does not replace;
// the six attention-stage operations and the context type below forward to the C ABI of glinthawk_attn.h.
//
//   reference interface                                   -> what it calls
//   LlamaOperations::copy_kv_cache       (ops.cuh:435-453)    held back until apply_rope names the same rows, then
//   LlamaOperations::apply_rope          (ops.cuh:413-433)    gh_op_copy_kv_cache_apply_rope (one kernel for both); each
//                                                             on its own: gh_op_copy_kv_cache / gh_op_apply_rope
//   LlamaOperations::attention_0_gemm    (ops.cuh:272-324)    remembered; see attention_2_gemm
//   LlamaOperations::attention_softmax   (ops.cuh:385-411)    nothing (fused) / gh_op_attention_softmax
//   LlamaOperations::attention_2_gemm    (ops.cuh:326-383)    gh_op_attention_fused / gh_op_attention_2_gemm
//   LlamaOperations::convert_and_copy    (ops.cuh:455-492)    gh_op_convert_and_copy
//   Context ctor / prepare / layer()     (context.hh:134-190) gh_slot_acquire / gh_slot_prepare / gh_slot_layer_ptr
//
// Error convention: the C ABI returns status codes; the reference aborts on any CUDA failure
// (CHECK_CUDA -> LOG(FATAL), src/arch/cuda/common/ops.cu:5-19), so a non-zero status is turned into LOG(FATAL).
#pragma once

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <mutex>
#include <type_traits>
#include <vector>

#include <glog/logging.h>

#include "glinthawk_attn.h"
#include "models/llama2/base.hh"
#include "models/llama2/context.hh"
#include "models/llama2/ops/concept.hh"

namespace glinthawk::models::llama2::b200 {

template<typename DType>
constexpr uint32_t dtype_code()
{
  // gh_dtype uses the reference's DataType values (src/models/types.hh:20-25)
  if constexpr ( std::is_same_v<DType, glinthawk::float32_t> )
    return GH_F32;
  else if constexpr ( sizeof( DType ) == 2 && std::is_same_v<DType, glinthawk::float16_t> )
    return GH_F16;
  else
    return GH_BF16;
}

#define GH_B200_CHECK( h, expr )                                                                                       \
  do {                                                                                                                 \
    const int gh_rc__ = ( expr );                                                                                      \
    if ( gh_rc__ != GH_OK )                                                                                            \
      LOG( FATAL ) << #expr << " failed: " << gh_status_string( gh_rc__ ) << ": " << gh_attn_last_error( h );          \
  } while ( 0 )

// One attention stage per (Config, DType) and process: the slot pool the contexts draw from and the handle
// the operations launch through.  Created on first use from the model's runtime settings.
template<typename Config, typename DType>
class Stage
{
public:
  static gh_attn_t get( const ConfigRuntime<Config>& settings )
  {
    static std::mutex mu;
    std::lock_guard lock { mu };
    gh_attn_t& h = handle();
    if ( h == nullptr ) {
      gh_attn_config cfg {};
      cfg.struct_size = sizeof( cfg );
      cfg.n_heads = Config::n_heads;
      cfg.n_kv_heads = Config::n_kv_heads;
      cfg.head_size = Config::head_size;
      cfg.seq_len = Config::seq_len;
      cfg.n_layers_hosted = static_cast<uint32_t>( settings.num_attention_layers_hosted() );
      cfg.dtype = dtype_code<DType>();
      cfg.max_batch = static_cast<uint32_t>( settings.concurrency_limit );
      cfg.max_contexts = static_cast<uint32_t>( settings.max_context_count );
      cfg.backing = paged() ? GH_BACKING_PAGED : GH_BACKING_STATIC;
      cfg.device = device(); // 0 unless set: the reference's CUDA backend uses device 0 implicitly (vmem.cuh:29,92)
      const int rc = gh_attn_create( &cfg, &h );
      if ( rc != GH_OK )
        LOG( FATAL ) << "gh_attn_create failed: " << gh_status_string( rc );
    }
    return h;
  }

  static gh_attn_t get()
  {
    CHECK( handle() != nullptr ) << "attention stage used before it was created";
    return handle();
  }

  // `profile-stage (paged|static)` in the reference picks DynamicContext or Context; here it is a switch.
  static bool& paged()
  {
    static bool p = false;
    return p;
  }

  // The CUDA device the stage is created on; set it before the first model or context is constructed.
  static int& device()
  {
    static int d = 0;
    return d;
  }

  static uint32_t next_context_id()
  {
    static std::atomic<uint32_t> next { 1 };
    return next.fetch_add( 1 );
  }

private:
  static gh_attn_t& handle()
  {
    static gh_attn_t h = nullptr;
    return h;
  }
};

// The reference's views are kept as they are: llama2::LayerContext / TokenContext are 8-byte wrappers around a
// device pointer (context.hh:68,102), and a slot of the arena has exactly the layout llama2::Context::set_buffer
// lays out (context.hh:177-189), so the base class does all the address arithmetic.
template<typename Config, typename DType>
class Context : public llama2::Context<Config, DType>
{
private:
  gh_attn_t h_ { nullptr };
  int32_t slot_ { -1 };
  uint32_t context_id_ { 0 };
  int32_t hosted_index_[Config::n_layers] {};

public:
  using llama2::Context<Config, DType>::Context;

  Context( const ConfigRuntime<Config>& settings, const bool make_empty = false )
    : llama2::Context<Config, DType>()
  {
    int32_t next = 0;
    for ( size_t i = 0; i < Config::n_layers; i++ )
      hosted_index_[i] = settings.hosts( i, InferenceStage::Attention ) ? next++ : -1;
    if ( make_empty )
      return;
    h_ = Stage<Config, DType>::get( settings );
    context_id_ = Stage<Config, DType>::next_context_id();
    GH_B200_CHECK( h_, gh_slot_acquire( h_, context_id_, &slot_ ) );
    void* base = nullptr;
    GH_B200_CHECK( h_, gh_slot_layer_ptr( h_, slot_, 0, &base ) );
    llama2::Context<Config, DType>::set_buffer( settings, static_cast<DType*>( base ) );
  }

  ~Context()
  {
    if ( h_ != nullptr && context_id_ != 0 )
      gh_slot_release( h_, context_id_ );
  }

  Context( const Context& ) = delete;
  Context& operator=( const Context& ) = delete;

  bool prepare( const size_t layer_num, const size_t token_pos, const bool can_release )
  {
    if ( llama2::Context<Config, DType>::empty() )
      return true;
    if ( hosted_index_[layer_num] < 0 )
      return false;
    return gh_slot_prepare( h_, slot_, static_cast<uint32_t>( hosted_index_[layer_num] ),
                            static_cast<uint32_t>( token_pos ), can_release ? 1 : 0 )
           == GH_OK;
  }

  int32_t slot() const { return slot_; }
};

template<typename Config, typename DType, typename Base, typename Ctx = Context<Config, DType>>
requires ModelConfig<Config> && ContextConcept<Ctx, DType>
class LlamaOperations : public Base
{
private:
  gh_attn_t h_;
  bool fused_ { true };
  bool blocking_ { false };
  mutable const DType* pending_query_ { nullptr };
  mutable std::vector<void*> ptrs_;
  // copy_kv_cache is the last operation of pre_attention_ops and apply_rope the first of attention_ops
  // (src/models/llama2/model.hh:345-364): the copy is held back so that the two run as one kernel launch.
  mutable std::vector<void*> pending_copy_rows_;
  mutable const DType* pending_copy_kv_ { nullptr };

  template<typename View>
  void* const* pointers( const View views[], const uint64_t n, const bool token_rows ) const
  {
    ptrs_.resize( n );
    for ( uint64_t i = 0; i < n; i++ ) {
      if constexpr ( requires( View v ) { v.key(); } ) {
        (void)token_rows;
        ptrs_[i] = const_cast<DType*>( views[i].key() ); // null for an inactive prompt
      } else {
        ptrs_[i] = views[i].empty() ? nullptr : const_cast<DType*>( views[i].token( 0 ).key() );
      }
    }
    return ptrs_.data();
  }

public:
  using typename Base::DeviceUniquePtr;
  using ContextType = Ctx;

  template<typename... BaseArgs>
  explicit LlamaOperations( const ConfigRuntime<Config>& settings, BaseArgs&&... base_args )
    : Base( std::forward<BaseArgs>( base_args )... )
    , h_( Stage<Config, DType>::get( settings ) )
  {
  }

  // false = run the three attention operations one by one and materialise `att`, exactly like the reference
  void set_fused( const bool fused ) { fused_ = fused; }

  // true = every attention-stage operation returns only after the GPU has finished it.  Needed when `Base`'s
  // operations run on the host (on managed or mapped memory) and therefore are not ordered by the CUDA stream.
  void set_blocking( const bool blocking ) { blocking_ = blocking; }

  ~LlamaOperations() { flush_copy(); }

private:
  void done() const
  {
    if ( blocking_ )
      GH_B200_CHECK( h_, gh_attn_synchronize( h_, nullptr ) );
  }

  // issues a copy_kv_cache that no apply_rope picked up
  void flush_copy() const
  {
    if ( pending_copy_kv_ == nullptr )
      return;
    GH_B200_CHECK( h_, gh_op_copy_kv_cache( h_, pending_copy_rows_.data(), pending_copy_kv_, pending_copy_rows_.size(),
                                            nullptr ) );
    pending_copy_kv_ = nullptr;
  }

public:

  void attention_0_gemm( const DType* query,
                         const typename ContextType::LayerContextType layer_contexts[],
                         DType* att,
                         const uint64_t batch_size,
                         const uint32_t* token_positions ) const
  {
    flush_copy();
    if ( fused_ ) {
      pending_query_ = query; // consumed by attention_2_gemm, which has every other argument
      return;
    }
    GH_B200_CHECK( h_, gh_op_attention_0_gemm( h_, query, pointers( layer_contexts, batch_size, false ), att,
                                               batch_size, token_positions, nullptr ) );
    done();
  }

  void attention_softmax( DType* att, const uint32_t* token_positions, DType* temp_buffer, const uint64_t batch_size )
    const
  {
    flush_copy();
    if ( fused_ )
      return;
    GH_B200_CHECK( h_, gh_op_attention_softmax( h_, att, token_positions, temp_buffer, batch_size, nullptr ) );
    done();
  }

  void attention_2_gemm( const DType* att,
                         const typename ContextType::LayerContextType layer_contexts[],
                         DType* xb,
                         const uint64_t batch_size,
                         const uint32_t* token_positions ) const
  {
    flush_copy();
    if ( fused_ ) {
      CHECK( pending_query_ != nullptr ) << "attention_2_gemm without a preceding attention_0_gemm";
      GH_B200_CHECK( h_, gh_op_attention_fused( h_, pending_query_, pointers( layer_contexts, batch_size, false ), xb,
                                                batch_size, token_positions, nullptr ) );
      pending_query_ = nullptr;
      done();
      return;
    }
    GH_B200_CHECK( h_, gh_op_attention_2_gemm( h_, att, pointers( layer_contexts, batch_size, false ), xb, batch_size,
                                               token_positions, nullptr ) );
    done();
  }

  void apply_rope( const uint64_t curr_batch_size,
                   const uint32_t* token_positions,
                   const DType* freq_cis_real,
                   const DType* freq_cis_imag,
                   DType* state_q,
                   typename ContextType::TokenContextType token_contexts[] ) const
  {
    void* const* rows = pointers( token_contexts, curr_batch_size, true );
    if ( pending_copy_kv_ != nullptr && pending_copy_rows_.size() == curr_batch_size
         && std::equal( pending_copy_rows_.begin(), pending_copy_rows_.end(), rows ) ) {
      const DType* state_kv = pending_copy_kv_;
      pending_copy_kv_ = nullptr;
      GH_B200_CHECK( h_, gh_op_copy_kv_cache_apply_rope( h_, curr_batch_size, token_positions, freq_cis_real,
                                                         freq_cis_imag, state_q, rows, state_kv, nullptr ) );
      done();
      return;
    }
    flush_copy();
    GH_B200_CHECK( h_, gh_op_apply_rope( h_, curr_batch_size, token_positions, freq_cis_real, freq_cis_imag, state_q,
                                         rows, nullptr ) );
    done();
  }

  void copy_kv_cache( typename ContextType::TokenContextType token_contexts[],
                      const DType* state_kv,
                      const uint64_t batch_size ) const
  {
    flush_copy();
    void* const* rows = pointers( token_contexts, batch_size, true );
    if ( blocking_ ) { // the caller may read the rows on the host right away
      GH_B200_CHECK( h_, gh_op_copy_kv_cache( h_, rows, state_kv, batch_size, nullptr ) );
      done();
      return;
    }
    pending_copy_rows_.assign( rows, rows + batch_size );
    pending_copy_kv_ = state_kv;
  }

  // Not a reference operation: Llama2::pre_attention_ops with the cache update followed by apply_rope
  // (src/models/llama2/model.hh:326-360) as one call, for a model that wants the q / kv projections on the tcgen05
  // path with K and V written straight into the contexts (no `kv` scratch).  fp16 / bf16, dim and kv_dim multiples of
  // 128.
  void pre_attention_rope_append( const uint64_t curr_batch_size,
                                  const DType* x,
                                  const DType* rms_att_weight,
                                  const DType* wq,
                                  const DType* wkv,
                                  DType* state_q,
                                  const uint32_t* token_positions,
                                  const DType* freq_cis_real,
                                  const DType* freq_cis_imag,
                                  typename ContextType::TokenContextType token_contexts[] ) const
  {
    flush_copy();
    GH_B200_CHECK( h_, gh_op_project_append( h_, curr_batch_size, x, rms_att_weight, wq, wkv, state_q, token_positions,
                                             freq_cis_real, freq_cis_imag, pointers( token_contexts, curr_batch_size, true ),
                                             nullptr ) );
    done();
  }

  template<typename DTypeDst, typename DTypeSrc>
  void convert_and_copy( DTypeDst* dst, const DTypeSrc* src, const uint64_t size, const CopyType type ) const
  {
    flush_copy();
    if constexpr ( std::is_void_v<DTypeDst> || std::is_void_v<DTypeSrc> ) {
      LOG( FATAL ) << "convert_and_copy needs concrete element types";
    } else {
      GH_B200_CHECK( h_, gh_op_convert_and_copy( h_, dst, dtype_code<DTypeDst>(), src, dtype_code<DTypeSrc>(), size,
                                                 static_cast<uint32_t>( type ) ) );
    }
  }
};

} // namespace glinthawk::models::llama2::b200
