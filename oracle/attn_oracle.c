/*
 * TEST INFRASTRUCTURE ONLY — never linked into, imported by, or called from the product path.
 *
 * Plain-C restatement of the attention-stage operations of Glinthawk's amd64 backend
 * (src/arch/amd64/llama2/ops.hh; rmsnorm and matmul of src/arch/amd64/common/ops.hh for the stage's producer) over Glinthawk's KV layout (src/models/llama2/context.hh:79-89,
 * 115-127: per layer, token t lives at base + t * 2 * kv_dim elements, K heads first, then V heads).
 * It is the checker the CUDA path is compared with; it is itself pinned against the reference's own
 * amd64 code compiled from the reference tree (oracle/ref_harness.cc) through the fixtures in
 * tests/golden/.  The reference project ships no tests or golden vectors of its own.
 *
 * Storage type codes follow the reference's DataType enum (src/models/types.hh:20-25):
 *   0 = Float16, 1 = Float32, 2 = BFloat16.
 * The reference has no working bf16 on amd64 (src/arch/float.hh:13); code 2 here applies the same
 * algorithm with bf16 round-to-nearest-even storage.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC oracle/attn_oracle.c -o oracle/libattn_oracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 gho_f16;
typedef struct
{
  uint16_t bits;
} gho_bf16;

static inline float bf16_to_f32( gho_bf16 v )
{
  uint32_t u = (uint32_t)v.bits << 16;
  float f;
  memcpy( &f, &u, 4 );
  return f;
}

static inline gho_bf16 f32_to_bf16( float f )
{
  uint32_t u;
  memcpy( &u, &f, 4 );
  gho_bf16 r;
  if ( ( u & 0x7fffffffu ) > 0x7f800000u ) { /* NaN: keep it quiet */
    r.bits = (uint16_t)( ( u >> 16 ) | 0x0040u );
    return r;
  }
  u += 0x7fffu + ( ( u >> 16 ) & 1u );
  r.bits = (uint16_t)( u >> 16 );
  return r;
}

/* ---- fp32 ---- */
#define T float
#define LD( x ) ( x )
#define RN( f ) ( (float)( f ) )
#define SFX f32
#include "attn_oracle_impl.inc"
#undef T
#undef LD
#undef RN
#undef SFX

/* ---- fp16 ---- */
#define T gho_f16
#define LD( x ) ( (float)( x ) )
#define RN( f ) ( (gho_f16)( f ) )
#define SFX f16
#include "attn_oracle_impl.inc"
#undef T
#undef LD
#undef RN
#undef SFX

/* ---- bf16 ---- */
#define T gho_bf16
#define LD( x ) bf16_to_f32( x )
#define RN( f ) f32_to_bf16( (float)( f ) )
#define SFX bf16
#include "attn_oracle_impl.inc"
#undef T
#undef LD
#undef RN
#undef SFX

enum
{
  GHO_F16 = 0,
  GHO_F32 = 1,
  GHO_BF16 = 2
};

#define DISPATCH( dtype, call_f32, call_f16, call_bf16 )                                                               \
  switch ( dtype ) {                                                                                                   \
    case GHO_F32: call_f32; return 0;                                                                                  \
    case GHO_F16: call_f16; return 0;                                                                                  \
    case GHO_BF16: call_bf16; return 0;                                                                                \
    default: return -1;                                                                                                \
  }

int gho_copy_kv_cache( int dtype, void* const* token_rows, const void* state_kv, uint64_t B, uint64_t kv_dim )
{
  DISPATCH( dtype,
            copy_kv_cache_f32( token_rows, (const float*)state_kv, B, kv_dim ),
            copy_kv_cache_f16( token_rows, (const gho_f16*)state_kv, B, kv_dim ),
            copy_kv_cache_bf16( token_rows, (const gho_bf16*)state_kv, B, kv_dim ) )
}

int gho_apply_rope( int dtype,
                    uint64_t B,
                    const uint32_t* pos,
                    const void* fcr,
                    const void* fci,
                    void* state_q,
                    void* const* token_rows,
                    uint64_t n_kv_heads,
                    uint64_t gqa,
                    uint64_t hs )
{
  DISPATCH(
    dtype,
    apply_rope_f32( B, pos, (const float*)fcr, (const float*)fci, (float*)state_q, token_rows, n_kv_heads, gqa, hs ),
    apply_rope_f16(
      B, pos, (const gho_f16*)fcr, (const gho_f16*)fci, (gho_f16*)state_q, token_rows, n_kv_heads, gqa, hs ),
    apply_rope_bf16(
      B, pos, (const gho_bf16*)fcr, (const gho_bf16*)fci, (gho_bf16*)state_q, token_rows, n_kv_heads, gqa, hs ) )
}

int gho_attention_0_gemm( int dtype,
                          const void* query,
                          const void* const* layer_bases,
                          void* att,
                          uint64_t B,
                          const uint32_t* pos,
                          uint64_t n_kv_heads,
                          uint64_t gqa,
                          uint64_t hs,
                          uint64_t seq_len )
{
  DISPATCH(
    dtype,
    attention_0_gemm_f32( (const float*)query, layer_bases, (float*)att, B, pos, n_kv_heads, gqa, hs, seq_len ),
    attention_0_gemm_f16( (const gho_f16*)query, layer_bases, (gho_f16*)att, B, pos, n_kv_heads, gqa, hs, seq_len ),
    attention_0_gemm_bf16(
      (const gho_bf16*)query, layer_bases, (gho_bf16*)att, B, pos, n_kv_heads, gqa, hs, seq_len ) )
}

int gho_attention_softmax( int dtype, void* att, const uint32_t* pos, uint64_t B, uint64_t n_heads, uint64_t seq_len )
{
  DISPATCH( dtype,
            attention_softmax_f32( (float*)att, pos, B, n_heads, seq_len ),
            attention_softmax_f16( (gho_f16*)att, pos, B, n_heads, seq_len ),
            attention_softmax_bf16( (gho_bf16*)att, pos, B, n_heads, seq_len ) )
}

int gho_attention_2_gemm( int dtype,
                          const void* att,
                          const void* const* layer_bases,
                          void* xb,
                          uint64_t B,
                          const uint32_t* pos,
                          uint64_t n_kv_heads,
                          uint64_t gqa,
                          uint64_t hs,
                          uint64_t seq_len )
{
  DISPATCH(
    dtype,
    attention_2_gemm_f32( (const float*)att, layer_bases, (float*)xb, B, pos, n_kv_heads, gqa, hs, seq_len ),
    attention_2_gemm_f16( (const gho_f16*)att, layer_bases, (gho_f16*)xb, B, pos, n_kv_heads, gqa, hs, seq_len ),
    attention_2_gemm_bf16( (const gho_bf16*)att, layer_bases, (gho_bf16*)xb, B, pos, n_kv_heads, gqa, hs, seq_len ) )
}

int gho_rmsnorm( int dtype, void* out, const void* x, const void* weight, uint64_t B, uint64_t size )
{
  DISPATCH( dtype,
            rmsnorm_f32( (float*)out, (const float*)x, (const float*)weight, B, size ),
            rmsnorm_f16( (gho_f16*)out, (const gho_f16*)x, (const gho_f16*)weight, B, size ),
            rmsnorm_bf16( (gho_bf16*)out, (const gho_bf16*)x, (const gho_bf16*)weight, B, size ) )
}

int gho_matmul( int dtype, void* xout, const void* x, const void* w, uint64_t B, uint64_t s, uint64_t r )
{
  DISPATCH( dtype,
            matmul_f32( (float*)xout, (const float*)x, (const float*)w, B, s, r ),
            matmul_f16( (gho_f16*)xout, (const gho_f16*)x, (const gho_f16*)w, B, s, r ),
            matmul_bf16( (gho_bf16*)xout, (const gho_bf16*)x, (const gho_bf16*)w, B, s, r ) )
}

/* The producer of the attention stage's inputs, src/models/llama2/model.hh:326-351 (pre_attention_ops without the
 * cache update): xb = rmsnorm(x, rms_att_weight); q = xb . wq^T; kv = xb . wkv^T.  wq is [dim][dim], wkv
 * [2*kv_dim][dim], both row-major. */
int gho_pre_attention( int dtype,
                       uint64_t B,
                       const void* x,
                       const void* rms_w,
                       const void* wq,
                       const void* wkv,
                       void* xb,
                       void* q,
                       void* kv,
                       uint64_t dim,
                       uint64_t kv_dim )
{
  if ( gho_rmsnorm( dtype, xb, x, rms_w, B, dim ) != 0 )
    return -1;
  gho_matmul( dtype, q, xb, wq, B, dim, dim );
  gho_matmul( dtype, kv, xb, wkv, B, dim, 2 * kv_dim );
  return 0;
}

static size_t elem_size( int dtype )
{
  return dtype == GHO_F32 ? 4 : 2;
}

static float load_as_f32( int dtype, const void* p, uint64_t i )
{
  switch ( dtype ) {
    case GHO_F32: return ( (const float*)p )[i];
    case GHO_F16: return (float)( (const gho_f16*)p )[i];
    default: return bf16_to_f32( ( (const gho_bf16*)p )[i] );
  }
}

/* src/arch/amd64/llama2/ops.hh:354-368 (convert_and_copy): memcpy when the types agree, else an element-wise
 * static_cast.  A cast between two 16-bit formats passes through fp32 here (the reference has no such pair). */
int gho_convert_and_copy( int dst_dtype, void* dst, int src_dtype, const void* src, uint64_t n )
{
  if ( dst_dtype < 0 || dst_dtype > 2 || src_dtype < 0 || src_dtype > 2 )
    return -1;
  if ( dst_dtype == src_dtype ) {
    memcpy( dst, src, n * elem_size( dst_dtype ) );
    return 0;
  }
  for ( uint64_t i = 0; i < n; i++ ) {
    const float v = load_as_f32( src_dtype, src, i );
    switch ( dst_dtype ) {
      case GHO_F32: ( (float*)dst )[i] = v; break;
      case GHO_F16: ( (gho_f16*)dst )[i] = (gho_f16)v; break;
      default: ( (gho_bf16*)dst )[i] = f32_to_bf16( v ); break;
    }
  }
  return 0;
}

/* One layer-step of the attention stage for a batch, in the order the model fixes
 * (src/models/llama2/model.hh:345-350 then :354-387): append the raw [K,V] row, rotate K in the slot and Q in
 * place, scores, softmax, weighted sum of V.  `att` is caller scratch of B * n_heads * seq_len elements. */
int gho_layer_step( int dtype,
                    uint64_t B,
                    const uint32_t* pos,
                    void* const* layer_bases,
                    const void* fcr,
                    const void* fci,
                    void* q_inout,
                    const void* kv_new,
                    void* att,
                    void* xb,
                    uint64_t n_kv_heads,
                    uint64_t gqa,
                    uint64_t hs,
                    uint64_t seq_len )
{
  if ( dtype < 0 || dtype > 2 )
    return -1;
  const uint64_t kvd = n_kv_heads * hs;
  void** rows = (void**)malloc( B * sizeof( void* ) );
  for ( uint64_t i = 0; i < B; i++ )
    rows[i] = layer_bases[i] ? (char*)layer_bases[i] + (uint64_t)pos[i] * 2 * kvd * elem_size( dtype ) : NULL;
  gho_copy_kv_cache( dtype, rows, kv_new, B, kvd );
  gho_apply_rope( dtype, B, pos, fcr, fci, q_inout, rows, n_kv_heads, gqa, hs );
  gho_attention_0_gemm( dtype, q_inout, (const void* const*)layer_bases, att, B, pos, n_kv_heads, gqa, hs, seq_len );
  gho_attention_softmax( dtype, att, pos, B, n_kv_heads * gqa, seq_len );
  gho_attention_2_gemm( dtype, att, (const void* const*)layer_bases, xb, B, pos, n_kv_heads, gqa, hs, seq_len );
  free( rows );
  return 0;
}
