// Launch prototypes shared between the kernel translation units and the C ABI.
// All shapes are in elements; `dtype` uses the SVODB_* codes of svodb.h.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace svodb {

// ---- rows.cu: LayerNorm / RMSNorm (+ fused residual) ------------------------
struct NormArgs {
  const void* x;
  const void* residual;  // nullable
  const void* w;
  const void* b;  // nullable
  void* out;
  void* sum;  // nullable, with residual
  int64_t rows;
  int d;
  float eps;
  int layer;  // 1 = LayerNorm, 0 = RMSNorm
  int dtype;
};
// Returns 1 when the warp-per-row kernel ran, 0 when the generic one did.
int launch_norm(const NormArgs& a, cudaStream_t s);

// ---- heads.cu ---------------------------------------------------------------
struct HeadsArgs {
  const void* qkv;
  const void* q_w;  // nullable
  const void* k_w;  // nullable
  const void* cos;  // nullable
  const void* sin;
  void* q;
  void* k;
  void* v;
  int64_t batch, t;
  int heads, kv_heads, d;
  float eps;
  int per_batch_tables;
  int dtype;
  int in_place;  // write each head back where it was read (q, k, v unused)
};
int launch_heads(const HeadsArgs& a, cudaStream_t s);

// ---- glue.cu ----------------------------------------------------------------
struct EmbedArgs {
  const void* ids;
  int ids_i64;
  const void* table;
  const void* pos_table;  // nullable
  const void* type_row;   // nullable
  int64_t pad_id;         // < 0: no position ids
  void* out;
  int64_t batch, t;
  int d;
  int64_t vocab, max_pos;
  int dtype;
};
void launch_embed(const EmbedArgs& a, cudaStream_t s);

// The send half of the peer-memory all-gather (peer.cu) for a kernel that produces
// the rows itself: block r stores its row into stage[step & 1][rank][r] of every
// peer, fences at system scope and counts itself; the block that counts last writes
// step + 1 into flags[rank] of every peer. world <= 1: nothing to send.
struct PeerPush {
  int world, rank;
  float* stage[8];
  uint32_t* flags[8];
  uint32_t* local;  // {steps completed, rows pushed, peers unstaged}
};

struct PoolArgs {
  const PeerPush* push;  // nullable: the rows also go to the peers' stages (fused norm + pool kernel only)
  const void* hidden;
  const void* aux;  // mask [B,L] (u8 or i32) or lengths [B] i32
  int aux_i32;
  int mode;  // 0 cls, 1 mean, 2 last, 3 gather `slots` tokens per row (aux = [B, slots] i32)
  int slots;
  int normalize;
  float* out;
  int64_t out_row_stride;
  int64_t batch, l;
  int d;
  int dtype;
};
void launch_pool(const PoolArgs& a, cudaStream_t s);

// A norm fused with the lookup before it or the pooling after it: weight
// (null = no norm, pooling only), bias (nullable), LayerNorm or RMSNorm.
struct EmbedNormArgs {
  const void* w;
  const void* b;
  float eps;
  int layer;  // 1 = LayerNorm, 0 = RMSNorm
};
// Both return 1 when the fused kernel ran, 0 (nothing launched) when the shape,
// dtype or alignment is outside it: 16-bit rows of 256..2048 elements in
// multiples of 256 on 16-byte boundaries.
int launch_embed_norm(const EmbedArgs& a, const EmbedNormArgs& n, cudaStream_t s);
int launch_norm_pool(const PoolArgs& a, const EmbedNormArgs& n, cudaStream_t s);

void launch_rope_table(double theta, const int32_t* positions, int64_t n_pos, int head_dim, void* cos, void* sin,
                       int dtype, cudaStream_t s);

// ---- attention ----------------------------------------------------------------
struct AttnArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  // element strides
  int64_t q_sb, q_st, q_sh;
  int64_t k_sb, k_st, k_sh;
  int64_t v_sb, v_st, v_sh;
  int64_t o_sb, o_st, o_sh;
  int64_t batch, t, tk;
  int heads, kv_heads, d;
  int dtype;
  float scale;
  int causal;
  const int32_t* key_lens;   // [B] or null
  const void* key_mask;      // [B,Tk] or null
  int key_mask_i32;          // element width of key_mask: 1 = i32, 0 = u8
  int has_window;
  int64_t win_left, win_right;
  int has_chunk;
  int64_t chunk_size, chunk_left, chunk_right;
  const int32_t* seg_start;  // [B,T] or null
  const void* bias;          // [B|1,H,T,Tk] stream dtype, or null
  int bias_per_batch;
  float* lse;                // [B,H,T] or null
  int splits;                // >= 1
  float* o_part;             // splits > 1: [S,B,T,H,D]
  float* m_part;             // [S,B,T,H]
  float* l_part;
  uint32_t* status;
  int packed;                // q,k,v are views of one fused projection
  // `ops::Cache`: k, v point at the first head this attention reads of cache
  // row 0; batch lane b reads row row_map[b] (b without a map) of kv_rows.
  int64_t kv_rows;
  const int32_t* row_map;    // [B] or null
  const void* k_app;         // [B, n_app, kv_heads, D] contiguous, or null
  const void* v_app;
  int n_app;
  const int32_t* app_lens;   // [B] or null
};
// Exact CUDA-core path (any float dtype, any D <= 256, every mask, bias, splits).
int launch_attention_generic(const AttnArgs& a, cudaStream_t s);
// tcgen05 path; returns 0 when it ran, nonzero (and launches nothing) when the
// shape is outside what it covers.
int launch_attention_tc(const AttnArgs& a, cudaStream_t s, char* cfg, size_t cfg_len);
bool attention_tc_covers(const AttnArgs& a);
// The persistent form (one CTA per SM over a work queue); same contract.
int launch_attention_tc_p(const AttnArgs& a, cudaStream_t s, char* cfg, size_t cfg_len);
bool attention_tc_p_covers(const AttnArgs& a);

// The split count an attention over `keys` keys (cached + appended) really runs
// with: a request is capped at the number of 32-key tiles, so no split is empty
// by construction.
inline int capped_splits(int64_t keys, int requested) {
  if (requested <= 1) return 1;
  const int64_t tiles = (keys + 31) / 32;
  return (int)(requested > tiles ? (tiles > 1 ? tiles : 1) : requested);
}

struct CombineArgs {
  const float* o_part;
  const float* m_part;
  const float* l_part;
  void* o;
  int64_t rows;  // B*T*H
  int d;
  int splits;
  int dtype;
};
void launch_combine(const CombineArgs& a, cudaStream_t s);

// ---- GEMM ---------------------------------------------------------------------
struct GemmArgs {
  const void* a;  // [M,K], row stride lda
  const void* w;  // [N,K] ([2N,K] gated), row stride ldw
  const void* bias;      // nullable
  const void* residual;  // nullable, row stride ldr
  void* c;               // [M,N], row stride ldc
  int64_t m;
  int n, k;
  int64_t lda, ldw, ldr, ldc;
  int act;
  int gated;
  int has_scale;
  float scale;
  const void* rope_cos;  // [seq, head_dim/2] stream dtype, nullable
  const void* rope_sin;
  int rope_heads, rope_head_dim;
  int64_t rope_seq;
  // Per-head RMSNorm in the store (tensor-core path only): weight [head_dim] for
  // the first norm_q_heads heads, another for the next norm_k_heads; the head
  // size is rope_head_dim. Nullable.
  const void* norm_q;
  const void* norm_k;
  int norm_q_heads, norm_k_heads;
  float norm_eps;
  int dtype;
  uint32_t* status;
  int force_bn;  // 0 = the launcher's choice; 64/128/256 = that tile width on one CTA; 512 = the CTA-pair kernel
  // Split-K on the CTA-pair kernel (tk/src/kernels/gemm.rs:454-466,750-808): > 1 =
  // that many splits of the k loop, f32 blocks and tile counters in `workspace`.
  int k_splits;
  void* workspace;
  size_t workspace_bytes;
};
// Workspace bytes of a split-K GEMM: [tiles][2] counters, then [tiles][splits][2][128][256] f32.
size_t gemm_splitk_workspace_bytes(int64_t m, int64_t n, int k_splits);
// Whether the split-K instantiation takes the call (plain epilogue: bias, activation,
// scale, residual; no gate, no rotation, no per-head store), workspace included.
bool gemm_tc2_splitk_covers(const GemmArgs& a);
int launch_gemm_tc2_splitk(const GemmArgs& a, cudaStream_t s, char* cfg, size_t cfg_len);
int launch_gemm_generic(const GemmArgs& a, cudaStream_t s);
int launch_gemm_tc(const GemmArgs& a, cudaStream_t s, char* cfg, size_t cfg_len);
bool gemm_tc_covers(const GemmArgs& a);
// The same GEMM on CTA pairs (cta_group::2, 256 x 256 tiles): the large
// projections without per-head stores.
int launch_gemm_tc2(const GemmArgs& a, cudaStream_t s, char* cfg, size_t cfg_len);
bool gemm_tc2_covers(const GemmArgs& a);
bool gemm_tc2_preferred(const GemmArgs& a);

// Sets the calling thread's `svodb_last_error` text (printf-style).
void set_last_error(const char* fmt, ...);

// The device status word bounded waits report into (one per device).
uint32_t* device_status_word();

}  // namespace svodb
