/* svodb — C ABI of the B200 (sm_100a) replacement for svod's `tk` encoder hot path.
 *
 * Every entry point is `extern "C"`, takes plain pointers / sizes / POD structs,
 * launches on the caller's CUDA stream and returns an `int` status
 * (SVODB_OK = 0). The caller owns all device memory: inputs, outputs and any
 * workspace. Nothing here allocates device memory unless its comment says so.
 *
 * The op-level functions mirror `svod_tk::ops` (tk/src/ops/mod.rs:30-38): same
 * operand meaning, same validation order and the same error classes
 * (`ops::Error`, tk/src/ops/mod.rs:132-159). Where the reference would take its
 * "graph" path for lack of a tile kernel (f32 operands, odd shapes), this
 * library runs an exact generic CUDA kernel instead; `svodb_last_chosen` reports
 * which ran, as `ops::chosen()` does (tk/src/ops/mod.rs:83-118).
 *
 * The device-level functions (`svodb_module_*`, `svodb_program_launch`,
 * `svodb_graph_*`, `svodb_alloc`...) mirror the `device` crate seam a Rust host
 * binds: `Program::execute` (device/src/device.rs:42-121), `CudaProgram::load`
 * (device/src/cuda/program.rs:116-219), `Graph::replay` (device/src/device.rs:144-171),
 * the allocator (device/src/cuda/allocator.rs).
 */
#ifndef SVODB_H_
#define SVODB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: `ops::Error` variants (tk/src/ops/mod.rs:132-159) ---- */
enum {
  SVODB_OK = 0,
  SVODB_ERR_SHAPE = 1,      /* Error::Shape */
  SVODB_ERR_DTYPE = 2,      /* Error::Dtype */
  SVODB_ERR_HEADS = 3,      /* Error::Heads */
  SVODB_ERR_GRAPH = 4,      /* Error::Graph: what the graph op would reject */
  SVODB_ERR_LAUNCH = 5,     /* Error::Launch: CUDA launch / driver failure */
  SVODB_ERR_UNREALIZED = 6, /* Error::Unrealized: null data pointer */
  SVODB_ERR_ALIAS = 7,      /* launch::aliasing (tk/src/launch.rs:227-246) */
  SVODB_ERR_TIMEOUT = 8,    /* a bounded device-side wait ran out */
  SVODB_ERR_POISONED = 9,   /* a sticky CUDA error latched (device/src/cuda/sys.rs:78-96) */
  SVODB_ERR_WORKSPACE = 10, /* workspace missing or too small */
  SVODB_ERR_UNSUPPORTED = 11
};

/* ---- element types (dtype/src: Float32, Float16, BFloat16, Int32, Int64, Bool) ---- */
enum { SVODB_F32 = 0, SVODB_F16 = 1, SVODB_BF16 = 2, SVODB_I32 = 3, SVODB_I64 = 4, SVODB_U8 = 5 };

/* ---- `kernels::Act` (tk/src/kernels/mod.rs:272-280); GELU_TANH is the extra
 * `Tensor::gelu` form (tensor/src/activation.rs:198-230). GELU is the exact (erf)
 * form: the reference evaluates erf by Abramowitz-Stegun 7.1.26 (mod.rs:304-335),
 * this library as x*Phi(x) = max(x,0) - a*2^P(a); both sit within 1e-6 of erf. ---- */
enum { SVODB_ACT_NONE = 0, SVODB_ACT_GELU = 1, SVODB_ACT_SILU = 2, SVODB_ACT_GELU_TANH = 3 };

#define SVODB_MAX_RANK 5

/* A realized, dense device tensor: `stride` in elements, innermost stride 1. */
typedef struct svodb_tensor {
  void* data;
  int32_t dtype;
  int32_t rank;
  int64_t shape[SVODB_MAX_RANK];
  int64_t stride[SVODB_MAX_RANK];
} svodb_tensor;

/* ---- library / device ---------------------------------------------------- */

/* Library version string. */
const char* svodb_version(void);

/* Thread-local message of the last failing call on this thread
 * (the `Display` text of `ops::Error`). */
const char* svodb_last_error(void);

/* `ops::supported(&DeviceSpec)` (tk/src/ops/mod.rs:161-166): 1 when CUDA device
 * `device` has the tcgen05 kernels (compute capability 10.x), else 0. */
int svodb_supported(int device);

/* `ops::chosen()` (tk/src/ops/mod.rs:101-118): what the last op on this thread
 * ran, e.g. "linear: kernel gemm {bm:128,bn:256,bk:64,stages:4}" or
 * "attention: graph dtype" (generic kernel and why). */
const char* svodb_last_chosen(void);

/* Shape-keyed config choice, the seam of a tune store (tk/src/tune.rs: a
 * measured config per shape, kept in the process and on disk). The library keeps
 * the process map; the host owns measurement and the file.
 * `svodb_last_config_key`: the key of the last `svodb_linear` on this thread that
 * reached the tensor-core kernel, "gemm|<dtype>|<m>|<n>|<k>|<epilogue>" ("" when
 * none did). `svodb_config_set(key, bn)`: later calls with that key use tile
 * width bn (64, 128 or 256 on one CTA, 512 = the CTA-pair kernel; a choice the
 * shape or epilogue cannot take is ignored); bn = 0 forgets the key. The key
 * "attention|one_item" (value 1) keeps attention on the one-item-per-CTA kernel,
 * "attention|exact" (value 1) on the exact CUDA-core kernel (for A/B timings).
 * `svodb_config_get` returns 0 when the key is unset. */
const char* svodb_last_config_key(void);
int svodb_config_set(const char* key, int32_t value);
int32_t svodb_config_get(const char* key);
void svodb_config_clear(void);

/* Reads and clears the device status word bounded waits report into
 * (0 = ok). Synchronises `stream`. Returns SVODB_ERR_TIMEOUT when a wait ran
 * out since the last call. */
int svodb_device_status(void* stream);

/* Self-tests of the failure paths; none of them hangs or faults the device.
 * `svodb_selftest_wait_timeout`: launches a one-warp kernel whose bounded wait
 * (on a barrier nothing arrives on) gives up after `polls` tries (1..2^20) and
 * returns normally; `svodb_device_status` then reports SVODB_ERR_TIMEOUT once,
 * as it would for a production kernel (device/src/cuda/sys.rs has no
 * counterpart: the reference has no device-side waits).
 * `svodb_selftest_latch_error`: feeds a `cudaError_t` value through the
 * classification a failed launch gets; a sticky code (device/src/cuda/sys.rs:78-96)
 * latches the library into SVODB_ERR_POISONED for every later call until
 * `svodb_selftest_clear_latch`. */
int svodb_selftest_wait_timeout(uint32_t polls, void* stream);
int svodb_selftest_latch_error(int32_t code);
void svodb_selftest_clear_latch(void);

/* ---- op layer: `svod_tk::ops` --------------------------------------------- */

struct svodb_qkv_opts;

/* `ops::Linear` + `ops::Rotary` (tk/src/ops/linear.rs:24-56). */
typedef struct svodb_linear_opts {
  const svodb_tensor* bias;     /* [N] ([2N] gated) or NULL */
  int32_t act;                  /* SVODB_ACT_* */
  int32_t gated;                /* w is [2N,K], gate rows over up rows */
  const svodb_tensor* residual; /* [lead..., N] or NULL, added last */
  int32_t has_scale;
  float scale;                  /* multiplies the activated value before the residual */
  const svodb_tensor* rope_cos; /* [1,T,1,head_dim/2] or NULL */
  const svodb_tensor* rope_sin;
  int32_t rope_heads;
  int32_t rope_head_dim;
  int64_t into_at;              /* y is channels [at, at+N) of a wider buffer: pass
                                   `y` as that view (data offset, wide row stride) */
  /* No counterpart in the reference's `Linear`: the attention prologue of
   * `ops::heads` (tk/src/ops/heads.rs:37-102) applied in this projection's
   * store. x is [B,T,K], N = (heads + 2*kv_heads)*head_dim; q and k heads are
   * RMS-normalised and rotated from the f32 accumulator (no rounding between
   * the projection and the prologue), v heads pass through, and y stays the
   * packed [B,T,N] projection that `svodb_attention_packed` reads in place.
   * Excludes rope_*, gated, act, scale and residual. NULL = off. */
  const struct svodb_qkv_opts* qkv;
  /* Split-K (the reference's `gemm_tail` + `split_merge`, tk/src/kernels/gemm.rs:454-466,
   * 750-808: f32 partials of a k loop cut into pieces, merged by one pass that applies the
   * epilogue once; never with a gate or a rotation). 0 or 1 = the k loop in one piece;
   * > 1 = that many pieces on the CTA-pair kernel, for problems of few 256 x 256 tiles and
   * a long k loop, with `workspace` of `svodb_linear_workspace_bytes` bytes (256-byte
   * aligned). Here the CTA that brings a tile's last piece merges them in piece order
   * inside the same launch. A call the split kernel does not cover runs unsplit. */
  int32_t k_splits;
  void* workspace;
  size_t workspace_bytes;
} svodb_linear_opts;

/* Bytes of `workspace` a split-K linear of m rows, n columns needs (0 for k_splits <= 1). */
size_t svodb_linear_workspace_bytes(int64_t m, int64_t n, int32_t k_splits);

/* `ops::linear(x, w, opts)` (tk/src/ops/linear.rs:63-191):
 * y[lead..., N] = scale*act(x[lead..., K] . w[N,K]^T + bias) + residual. */
int svodb_linear(const svodb_tensor* x, const svodb_tensor* w, const svodb_linear_opts* opts, svodb_tensor* y,
                 void* stream);

/* `ops::Attn` (tk/src/ops/attention.rs:59-86) flattened. */
typedef struct svodb_attn_opts {
  int32_t causal;
  const svodb_tensor* key_lens; /* KeyMask::Lens: [B] i32/i64, or NULL */
  const svodb_tensor* key_mask; /* KeyMask::Bool: [B,Tk] u8/i32 (nonzero = attended), or NULL */
  int32_t has_window;
  int64_t window_left, window_right;
  int32_t has_chunk;            /* `Chunk{size,left,right}` */
  int64_t chunk_size, chunk_left /* -1 = every earlier chunk */, chunk_right;
  const svodb_tensor* seg_start; /* [B,T] i32 or NULL */
  int32_t splits;               /* 0 or 1 = the keys in one pass; >1 = that many key splits (capped at
                                   the number of 32-key tiles), which need `workspace` */
  int32_t has_scale;
  float scale;                  /* default 1/sqrt(D) */
  const svodb_tensor* bias;     /* [B|1,H,T,Tk] in the stream dtype, or NULL */
  svodb_tensor* lse;            /* optional out: [B,H,T] f32, ln-sum-exp of the masked scaled scores */
  void* workspace;              /* device scratch for key splits (f32 partials) */
  size_t workspace_bytes;
  /* `ops::Cache` (tk/src/ops/attention.rs:39-55): k and v are caches
   * [rows, Tk, H_all, D] holding several layers' heads; this attention reads
   * heads [head_start, head_start + kv_heads) of cache row row_map[b] (row b
   * without a map), then the appended keys. The masks apply to cached keys; an
   * appended key is hidden only past app_lens[b]. */
  int32_t has_cache;
  int32_t cache_head_start;
  int32_t cache_kv_heads;
  const svodb_tensor* cache_row_map;  /* [B] i32 or NULL */
  const svodb_tensor* cache_app_k;    /* [B, n, kv_heads, D] keys scored after the cached prefix
                                         (needs key_lens), or NULL */
  const svodb_tensor* cache_app_v;
  const svodb_tensor* cache_app_lens; /* [B] i32 visible appended rows, or NULL = all */
} svodb_attn_opts;

/* Bytes of `workspace` a split attention of this shape needs
 * (`o_part`, `m_part`, `l_part`: tk/src/ops/attention.rs:285-292). */
size_t svodb_attention_workspace_bytes(int64_t batch, int64_t t, int64_t heads, int64_t d, int32_t splits);

/* `ops::attention(q,k,v,opts)` (tk/src/ops/attention.rs:100-102):
 * q [B,T,H,D], k,v [B,Tk,Hkv,D] sequence-major -> o [B,T,H,D].
 * Calls with more work items (256 query rows x head x batch lane) than the
 * device has SMs run a persistent kernel that hands the items out through a
 * counter inside the library, one counter per (device, stream) pair, zeroed on
 * the stream before each launch (a memset node under capture). Launches on one
 * stream follow one another, so they may share it; a captured graph keeps the
 * counter of the stream it was captured on, so two graphs captured on the SAME
 * stream must not be replayed at the same time on different streams. Config key
 * "attention|one_item" = 1 (`svodb_config_set`) turns the persistent kernel off. */
int svodb_attention(const svodb_tensor* q, const svodb_tensor* k, const svodb_tensor* v, const svodb_attn_opts* opts,
                    svodb_tensor* o, void* stream);

/* Bytes of the scratch array built into the library for
 * `svodb_attention_splits_noalloc`; every GPU that loads the library holds this
 * much until the process exits. */
#define SVODB_NOALLOC_SCRATCH_BYTES (8u << 20)

/* No counterpart in the reference. `svodb_attention` with key splits, for
 * callers that may not allocate device memory when they call (inside a stream
 * capture or a plan replay, where memory was laid out ahead of time and
 * cudaMalloc is not allowed): the f32 partials live in a fixed
 * SVODB_NOALLOC_SCRATCH_BYTES array inside the library instead of
 * `opts->workspace`, which is ignored. Allocates nothing. Shapes whose partials
 * (`svodb_attention_workspace_bytes`) exceed the array return
 * SVODB_ERR_WORKSPACE. The array is shared by every call on a device: calls
 * that overlap on the GPU race, so issue them on one stream; nothing in it
 * needs clearing between calls. The first call on a device looks up the
 * array's address; make it before starting a stream capture. */
int svodb_attention_splits_noalloc(const svodb_tensor* q, const svodb_tensor* k, const svodb_tensor* v,
                                   const svodb_attn_opts* opts, svodb_tensor* o, void* stream);

/* `ops::attention_packed(qkv, heads, kv_heads, opts)` (tk/src/ops/attention.rs:107-122):
 * qkv [B,T,(H+2Hkv)*D] read in place -> o [B,T,H,D]. */
int svodb_attention_packed(const svodb_tensor* qkv, int32_t heads, int32_t kv_heads, const svodb_attn_opts* opts,
                           svodb_tensor* o, void* stream);

/* `kernels::attention::combine` (tk/src/kernels/attention.rs:984-1014): merges
 * f32 partials o_part [S,B,T,H,D], m_part/l_part [S,B,T,H] (m in log2 units). */
int svodb_combine_splits(const svodb_tensor* o_part, const svodb_tensor* m_part, const svodb_tensor* l_part,
                         svodb_tensor* o, void* stream);

/* `ops::Qkv` (tk/src/ops/heads.rs:18-32). */
typedef struct svodb_qkv_opts {
  int32_t heads, kv_heads, head_dim;
  const svodb_tensor* q_norm; /* [head_dim] or NULL */
  const svodb_tensor* k_norm;
  double eps;
  const svodb_tensor* rope_cos; /* [1|B, T, 1, head_dim/2] or NULL */
  const svodb_tensor* rope_sin;
} svodb_qkv_opts;

/* `ops::heads(qkv, opts)` (tk/src/ops/heads.rs:37-102). */
int svodb_heads(const svodb_tensor* qkv, const svodb_qkv_opts* opts, svodb_tensor* q, svodb_tensor* k,
                svodb_tensor* v, void* stream);

/* `ops::layer_norm` / `add_layer_norm` / `rms_norm` / `add_rms_norm`
 * (tk/src/ops/norm.rs:17-41). `b` may be NULL. The fused forms write
 * `sum = round(x + residual)` and normalise the rounded sum. */
int svodb_layer_norm(const svodb_tensor* x, const svodb_tensor* w, const svodb_tensor* b, double eps,
                     svodb_tensor* out, void* stream);
int svodb_add_layer_norm(const svodb_tensor* x, const svodb_tensor* residual, const svodb_tensor* w,
                         const svodb_tensor* b, double eps, svodb_tensor* sum, svodb_tensor* out, void* stream);
int svodb_rms_norm(const svodb_tensor* x, const svodb_tensor* w, double eps, svodb_tensor* out, void* stream);
int svodb_add_rms_norm(const svodb_tensor* x, const svodb_tensor* residual, const svodb_tensor* w, double eps,
                       svodb_tensor* sum, svodb_tensor* out, void* stream);

/* ---- glue the encoder callers need around the ops -------------------------- */

/* Token embedding lookup `out[b,t,:] = table[ids[b,t],:]`
 * (`Embedding::forward`, lowered as a gather: tensor/src/transformer.rs:33-64).
 * XLM-R form adds position and token-type rows: ids i32/i64 [B,T];
 * `pos_table`/`type_row` may be NULL; position ids follow
 * model/src/xlm_roberta/position_ids.rs:27-32 when `pad_id >= 0`. */
int svodb_embed(const svodb_tensor* ids, const svodb_tensor* table, const svodb_tensor* pos_table,
                const svodb_tensor* type_row, int64_t pad_id, svodb_tensor* out, void* stream);

/* The same lookup with the embedding norm applied before the store, one kernel
 * instead of a gather pass and a norm pass over [B, T, D]
 * (`Embeddings::forward`: word + position + type rows, then LayerNorm,
 * model/src/xlm_roberta/embeddings.rs:53-63; ModernBERT: table row, then LayerNorm
 * without bias). `norm_w` [D] is required, `norm_b` [D] may be NULL; `layer` != 0
 * = LayerNorm, 0 = RMSNorm. Rows outside the fused kernel (D not a multiple of
 * 256 in 256..2048, operands off the 16-byte boundary) run the lookup and then
 * the norm in place; `svodb_last_chosen` says which. */
int svodb_embed_norm(const svodb_tensor* ids, const svodb_tensor* table, const svodb_tensor* pos_table,
                     const svodb_tensor* type_row, int64_t pad_id, const svodb_tensor* norm_w,
                     const svodb_tensor* norm_b, double eps, int32_t layer, svodb_tensor* out, void* stream);

/* `encoder_head::pool` + `lp_normalize` (model/src/encoder_head.rs:280-286;
 * tensor/src/nn/norm.rs:205-213) and Qwen3's last-token gather
 * (model/src/qwen3/model.rs:77-99): hidden [B,L,D] -> out [B,D] f32 rows of an
 * `out` that may be a slice of a wider gather buffer.
 * mode 0 = CLS, 1 = masked mean (mask [B,L] u8/i32), 2 = last token (lengths [B] i32),
 * 3 = gather: token indices [B,S] i32 -> out [B*S, D], the pooled slots of packed rows
 * (model/src/qwen3/embed.rs:119-136, embedder.rs:37-52). */
int svodb_pool(const svodb_tensor* hidden, const svodb_tensor* mask_or_lengths, int32_t mode, int32_t normalize,
               svodb_tensor* out, void* stream);

/* The stack's final norm, the pooling and the L2 normalisation as ONE kernel
 * (model/src/encoder_head.rs:280-286 applied to the last norm's output;
 * model/src/qwen3/model.rs:77-99): `hidden` [B,L,D] is the stack's output BEFORE
 * its final norm. CLS, last-token and gather modes normalise only the tokens
 * they pool; the masked mean normalises the row's real tokens as it sums them.
 * `norm_w` NULL = no norm (a post-LN stack): pooling + L2 in one launch. Modes,
 * mask / lengths / indices and `out` as in `svodb_pool`. Rows outside the fused
 * kernel (D not a multiple of 256 in 256..2048, operands off the 16-byte
 * boundary) take the unfused sequence, which writes the normalised hidden
 * states into `scratch` (the shape and dtype of `hidden`; may be NULL when the
 * fused kernel applies or there is no norm) - SVODB_ERR_WORKSPACE without it. */
int svodb_norm_pool(const svodb_tensor* hidden, const svodb_tensor* norm_w, const svodb_tensor* norm_b, double eps,
                    int32_t layer, svodb_tensor* scratch, const svodb_tensor* mask_or_lengths, int32_t mode,
                    int32_t normalize, svodb_tensor* out, void* stream);

/* RoPE tables `Tensor::rope_table` (tensor/src/transformer.rs:130-164): angles
 * and cos/sin in f32, cast last; positions [P] i32 (NULL = 0..P-1);
 * cos,sin [P, head_dim/2]. */
int svodb_rope_table(double theta, const svodb_tensor* positions, int32_t head_dim, svodb_tensor* cos,
                     svodb_tensor* sin, void* stream);

/* ---- native model runners ------------------------------------------------------
 * The three encoder stacks driven from compiled code, for hosts without a Python
 * layer: what the model structs + `HeadPlans` do in the reference
 * (model/src/{qwen3,xlm_roberta,modernbert}/...; model/src/encoder_head.rs:384-500).
 * A model borrows the caller's device weights (dense row-major, all of one 16-bit
 * dtype); a plan owns one arena of activations, the RoPE tables and one captured
 * CUDA graph for a `(rows, len)` shape on its own stream. */
typedef struct svodb_model svodb_model;
typedef struct svodb_plan svodb_plan;

/* Qwen3 embedding decoder (model/src/qwen3/config.rs:62-81). */
typedef struct svodb_qwen3_config {
  int32_t vocab, hidden, layers, heads, kv_heads, head_dim, ffn;
  int32_t dtype;    /* SVODB_BF16 / SVODB_F16 of every weight */
  double eps;       /* RMSNorm epsilon */
  double rope_theta;
} svodb_qwen3_config;

/* in_w [hidden], qkv_w [(heads+2*kv_heads)*head_dim, hidden], qn_w, kn_w [head_dim],
 * o_w [hidden, heads*head_dim], post_w [hidden], gu_w [2*ffn, hidden] (gate rows
 * first), down_w [hidden, ffn]. */
typedef struct svodb_qwen3_layer {
  const void *in_w, *qkv_w, *qn_w, *kn_w, *o_w, *post_w, *gu_w, *down_w;
} svodb_qwen3_layer;

typedef struct svodb_qwen3_weights {
  const void* embed;               /* [vocab, hidden] */
  const svodb_qwen3_layer* layers; /* [cfg.layers] */
  const void* norm_w;              /* [hidden] */
} svodb_qwen3_weights;

/* XLM-RoBERTa / BGE-M3 encoder (model/src/xlm_roberta/config.rs:119-136). */
typedef struct svodb_xlmr_config {
  int32_t vocab, hidden, layers, heads, ffn, max_positions;
  int32_t pad_id;   /* position ids count the tokens that differ from it */
  int32_t dtype;
  int32_t pooling;  /* 0 = CLS, 1 = masked mean */
  double eps;       /* LayerNorm epsilon */
} svodb_xlmr_config;

/* qkv_w [3*hidden, hidden] = the reference's q, k, v weights stacked (rows q, then
 * k, then v), qkv_b [3*hidden] likewise; o_w [hidden, hidden]; fi_w [ffn, hidden];
 * fo_w [hidden, ffn]; biases and LayerNorm weights [hidden] ([ffn] for fi_b). */
typedef struct svodb_xlmr_layer {
  const void *qkv_w, *qkv_b, *o_w, *o_b, *ln1_w, *ln1_b, *fi_w, *fi_b, *fo_w, *fo_b, *ln2_w, *ln2_b;
} svodb_xlmr_layer;

typedef struct svodb_xlmr_weights {
  const void *word, *pos, *type;   /* [vocab, hidden], [max_positions, hidden], [hidden] (type row 0) */
  const void *emb_ln_w, *emb_ln_b; /* [hidden] */
  const svodb_xlmr_layer* layers;  /* [cfg.layers] */
} svodb_xlmr_weights;

/* ModernBERT encoder (model/src/modernbert/config.rs:72-92). */
typedef struct svodb_modernbert_config {
  int32_t vocab, hidden, layers, heads, ffn;
  int32_t global_every;  /* layer l attends globally when l % global_every == 0 */
  int32_t local_window;  /* total width of the local layers' window (half to each side) */
  int32_t dtype;
  int32_t pooling;       /* 0 = CLS, 1 = masked mean */
  double eps, global_theta, local_theta;
} svodb_modernbert_config;

/* attn_ln_w [hidden] or NULL (layer 0 has none), qkv_w [3*hidden, hidden],
 * o_w [hidden, hidden], mlp_ln_w [hidden], wi_w [2*ffn, hidden] (gate rows first),
 * wo_w [hidden, ffn]. */
typedef struct svodb_modernbert_layer {
  const void *attn_ln_w, *qkv_w, *o_w, *mlp_ln_w, *wi_w, *wo_w;
} svodb_modernbert_layer;

typedef struct svodb_modernbert_weights {
  const void *embed, *emb_ln_w;         /* [vocab, hidden], [hidden] */
  const svodb_modernbert_layer* layers; /* [cfg.layers] */
  const void* final_ln_w;               /* [hidden] */
} svodb_modernbert_weights;

int svodb_qwen3_create(const svodb_qwen3_config* cfg, const svodb_qwen3_weights* weights, svodb_model** out);
int svodb_xlmr_create(const svodb_xlmr_config* cfg, const svodb_xlmr_weights* weights, svodb_model** out);
int svodb_modernbert_create(const svodb_modernbert_config* cfg, const svodb_modernbert_weights* weights,
                            svodb_model** out);
void svodb_model_free(svodb_model* model);
/* Prepares the plan of one shape: allocates, runs once eagerly, captures.
 * reference_ops != 0 (Qwen3 only) keeps the reference's op sequence (projection,
 * heads kernel, attention) instead of the prologue fused into the projection's store. */
int svodb_model_plan(svodb_model* model, int64_t rows, int64_t len, int32_t reference_ops, svodb_plan** out);
/* One batch from host memory: ids [rows, len] i32 and `host_aux` = lengths [rows]
 * i32 (Qwen3) or the padding mask [rows, len] bytes, nonzero = real token (XLM-R,
 * ModernBERT); NULL keeps what the plan holds. Graph replay, then the pooled
 * unit-norm rows [rows, hidden] f32 to host memory (NULL = leave them on the
 * device and do not wait). With host_out the call waits for the replay and
 * returns SVODB_ERR_TIMEOUT if a bounded device-side wait ran out during it;
 * without, call `svodb_device_status(svodb_plan_stream(plan))` before trusting
 * the rows. */
int svodb_plan_run(svodb_plan* plan, const int32_t* host_ids, const void* host_aux, float* host_out);
void* svodb_plan_stream(svodb_plan* plan);   /* the plan's CUstream */
float* svodb_plan_output(svodb_plan* plan);  /* device [rows, hidden] f32 */
void svodb_plan_free(svodb_plan* plan);

/* ---- device seam: what the `device` crate binds ----------------------------- */

typedef struct svodb_program svodb_program;
typedef struct svodb_graph svodb_graph;

/* One kernel parameter: `AbiParamDescriptor{slot,kind}` (device/src/device.rs:366-381). */
typedef struct svodb_abi_param {
  int32_t slot;
  int32_t kind; /* 0 = Storage (8-byte device pointer), 1 = Scalar (4-byte i32) */
} svodb_abi_param;

/* `CudaProgram::load` (device/src/cuda/program.rs:116-219): loads a cubin or PTX
 * image, resolves `entry`. */
int svodb_module_load(const void* image, size_t bytes, const char* entry, const svodb_abi_param* params, int32_t n,
                      svodb_program** out);
/* `Program::execute` (device/src/device.rs:42-66): kernarg = pointers then i32
 * scalars in ascending slot order (device/src/cuda/program.rs:1-5,264-274). */
int svodb_program_launch(svodb_program* p, void* stream, void* const* bufs, int32_t n_bufs, const int32_t* vals,
                         int32_t n_vals, const uint32_t grid[3], const uint32_t block[3], uint32_t dyn_smem);
int svodb_program_free(svodb_program* p);

/* `CudaGraph::capture` / `Graph::replay` (device/src/cuda/graph.rs:127-173,375-391),
 * stream-capture based. */
int svodb_graph_begin(void* stream);
int svodb_graph_end(void* stream, svodb_graph** out);
int svodb_graph_replay(svodb_graph* g, void* stream);
int svodb_graph_free(svodb_graph* g);

/* `Allocator` (device/src/cuda/allocator.rs): kind 0 = device, 1 = pinned host. */
int svodb_alloc(size_t bytes, int32_t kind, void** out);
int svodb_free(void* ptr, int32_t kind);
int svodb_copy_h2d(void* dst, const void* src, size_t bytes, void* stream);
int svodb_copy_d2h(void* dst, const void* src, size_t bytes, void* stream);
int svodb_stream_sync(void* stream);
int svodb_memset(void* ptr, int32_t value, size_t bytes, void* stream);

/* ---- the path's one collective over NVLink peer memory ----
 * No counterpart in the reference (it runs on one GPU): the all-gather of pooled
 * rows that follows `svodb_norm_pool` when the batch is dealt over several GPUs,
 * as kernels of this library instead of a collective library's. One process per
 * GPU. Every rank allocates (`svodb_alloc`, zeroed) a stage of
 * `svodb_peer_stage_bytes` bytes, 256 bytes of flags and 256 bytes of local
 * counters, exports stage and flags (`svodb_ipc_export`), the host exchanges the
 * 64-byte handles by whatever channel it has, and each rank maps the others'
 * (`svodb_ipc_open`; its own pointers go in at its own index). `svodb_peer_all_gather`
 * then puts rank r's `[rows, d]` f32 block into slot r of every rank's `gathered`
 * [world*rows, d]: a push kernel (plain stores into the peers' stages, a
 * system-scope fence, a flag per peer) and an unstage kernel that waits for each
 * peer's flag — `wait_polls` polls of about 256 ns (0 = a few seconds), after which
 * the step reports SVODB_ERR_TIMEOUT through `svodb_device_status` — and copies
 * its rows in. `mine` is normally slot `rank` of `gathered`. Both launches can be
 * captured in a CUDA graph; ranks must reach the same step count. */
typedef struct svodb_peer_gather {
  int32_t world, rank;  /* world <= 8 */
  void* stage[8];       /* rank p's stage as mapped in this process */
  void* flags[8];       /* rank p's flags as mapped in this process */
  void* local;          /* this rank's private counters (256 bytes, zeroed) */
  uint32_t wait_polls;
  int32_t phases;       /* 0 = the whole step; 1 = the push alone, 2 = the unstage alone (a host may put
                           other work between them; every step needs both, in this order) */
} svodb_peer_gather;
size_t svodb_peer_stage_bytes(int32_t world, int64_t rows, int64_t d);
int svodb_ipc_export(const void* dev_ptr, uint8_t handle[64]);
int svodb_ipc_open(const uint8_t handle[64], void** out);
int svodb_ipc_close(void* ptr);
int svodb_peer_all_gather(const svodb_peer_gather* pg, const float* mine, float* gathered, int64_t rows, int64_t d,
                          void* stream);
/* `svodb_norm_pool` writing this rank's rows into slot `rank` of `gathered` [world*rows, D] f32
 * and gathering the others': where the fused norm + pool kernel takes the call, that kernel
 * itself stores each pooled row into every peer's stage and raises the flags (compute and send
 * in one launch), and only the unstage follows; otherwise the whole gather follows. */
int svodb_norm_pool_gather(const svodb_tensor* hidden, const svodb_tensor* norm_w, const svodb_tensor* norm_b, double eps,
                           int32_t layer, svodb_tensor* scratch, const svodb_tensor* mask_or_lengths, int32_t mode,
                           int32_t normalize, const svodb_peer_gather* pg, svodb_tensor* gathered, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SVODB_H_ */
