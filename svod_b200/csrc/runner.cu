// Native runners of the three encoder stacks: the host side a compiled caller
// links instead of a Python one. A runner owns what `HeadPlans` owns in the
// reference (model/src/encoder_head.rs:384-500): per plan shape `(rows, len)` one
// arena of activations, the RoPE tables, and one captured CUDA graph of the whole
// stack; a run is two host-to-device copies, a graph launch and one
// device-to-host copy of the pooled rows.
//
// The op sequences are the reference's, issued through this library's own C
// entry points:
//   Qwen3       model/src/qwen3/{decoder_layer.rs:55-65, attention.rs:69-113,
//               feed_forward.rs:38-42, model.rs:77-99}; the attention prologue in
//               the QKV projection's store unless `reference_ops` asks for
//               linear -> heads -> attention
//   XLM-R       model/src/xlm_roberta/{embeddings.rs:53-63, attention.rs:63-77,
//               feed_forward.rs:40-45, encoder_layer.rs:45-49}; one fused [3D, D]
//               projection computes the columns of the reference's three
//   ModernBERT  model/src/modernbert/{attention.rs:52-68, mlp.rs:41-46,
//               encoder_layer.rs:52-60, encoder.rs:33-54}
// with the embedding norm fused into the lookup and the final norm, pooling and
// L2 normalisation as one kernel (model/src/encoder_head.rs:280-286).
#include <cuda_runtime.h>
#include <string.h>

#include <vector>

#include "kernels.h"
#include "svodb.h"

enum { kQwen3 = 0, kXlmr = 1, kModernBert = 2 };

struct svodb_model {
  int kind;
  svodb_qwen3_config q;
  svodb_xlmr_config x;
  svodb_modernbert_config m;
  std::vector<svodb_qwen3_layer> q_layers;
  std::vector<svodb_xlmr_layer> x_layers;
  std::vector<svodb_modernbert_layer> m_layers;
  svodb_qwen3_weights qw;
  svodb_xlmr_weights xw;
  svodb_modernbert_weights mw;
  int dtype() const { return kind == kQwen3 ? q.dtype : kind == kXlmr ? x.dtype : m.dtype; }
  int64_t hidden() const { return kind == kQwen3 ? q.hidden : kind == kXlmr ? x.hidden : m.hidden; }
};

struct svodb_plan {
  const svodb_model* model;
  int64_t rows, len;
  char* arena;        // every device buffer of the plan, one allocation
  size_t arena_bytes;
  int32_t* ids;       // [rows, len]
  void* aux;          // Qwen3: lengths [rows] i32; the others: padding mask [rows, len] bytes
  size_t aux_bytes;
  float* pooled;      // [rows, D]
  svodb_graph* graph;
  cudaStream_t stream;
};

namespace {

size_t esize_of(int dtype) { return dtype == SVODB_F32 ? 4 : 2; }

svodb_tensor tensor(const void* data, int dtype, std::initializer_list<int64_t> shape) {
  svodb_tensor t{};
  t.data = const_cast<void*>(data);
  t.dtype = dtype;
  t.rank = (int32_t)shape.size();
  int i = 0;
  for (int64_t s : shape) t.shape[i++] = s;
  int64_t stride = 1;
  for (int d = t.rank - 1; d >= 0; --d) {
    t.stride[d] = stride;
    stride *= t.shape[d];
  }
  return t;
}

struct Bump {
  char* base;
  size_t at;
  void* take(size_t bytes) {
    void* p = base != nullptr ? base + at : nullptr;
    at += (bytes + 255) & ~size_t(255);
    return p;
  }
};

#define RUN(call)                 \
  do {                            \
    int rc_ = (call);             \
    if (rc_ != SVODB_OK) return rc_; \
  } while (0)

// The activations of one plan, carved from its arena. Not every stack uses
// every buffer.
struct Acts {
  void *x, *xn, *qkv, *q, *k, *v, *attn, *h, *hn, *g;
  void *cos, *sin;    // Qwen3 / ModernBERT global tables [len, head_dim/2]
  void *cos2, *sin2;  // ModernBERT local tables
};

Acts carve(Bump& b, const svodb_model& m, int64_t B, int64_t L, int reference_ops) {
  const size_t e = esize_of(m.dtype());
  const size_t tok = (size_t)B * L;
  Acts a{};
  if (m.kind == kQwen3) {
    const svodb_qwen3_config& c = m.q;
    const size_t qkv = (size_t)(c.heads + 2 * c.kv_heads) * c.head_dim;
    a.x = b.take(tok * c.hidden * e);
    a.xn = b.take(tok * c.hidden * e);
    a.qkv = b.take(tok * qkv * e);
    if (reference_ops) {
      a.q = b.take(tok * c.heads * c.head_dim * e);
      a.k = b.take(tok * c.kv_heads * c.head_dim * e);
      a.v = b.take(tok * c.kv_heads * c.head_dim * e);
    }
    a.attn = b.take(tok * c.heads * c.head_dim * e);
    a.h = b.take(tok * c.hidden * e);
    a.hn = b.take(tok * c.hidden * e);
    a.g = b.take(tok * c.ffn * e);
    a.cos = b.take((size_t)L * (c.head_dim / 2) * e);
    a.sin = b.take((size_t)L * (c.head_dim / 2) * e);
  } else if (m.kind == kXlmr) {
    const svodb_xlmr_config& c = m.x;
    a.x = b.take(tok * c.hidden * e);
    a.qkv = b.take(tok * 3 * c.hidden * e);
    a.attn = b.take(tok * c.hidden * e);
    a.h = b.take(tok * c.hidden * e);    // the projections' outputs before each norm
    a.hn = b.take(tok * c.hidden * e);   // the hidden states after the first norm
    a.g = b.take(tok * c.ffn * e);
  } else {
    const svodb_modernbert_config& c = m.m;
    const size_t hd = (size_t)c.hidden / c.heads;
    a.x = b.take(tok * c.hidden * e);
    a.xn = b.take(tok * c.hidden * e);
    a.qkv = b.take(tok * 3 * c.hidden * e);
    a.attn = b.take(tok * c.hidden * e);
    a.h = b.take(tok * c.hidden * e);
    a.hn = b.take(tok * c.hidden * e);
    a.g = b.take(tok * c.ffn * e);
    a.cos = b.take((size_t)L * (hd / 2) * e);
    a.sin = b.take((size_t)L * (hd / 2) * e);
    a.cos2 = b.take((size_t)L * (hd / 2) * e);
    a.sin2 = b.take((size_t)L * (hd / 2) * e);
  }
  return a;
}

int forward_qwen3(const svodb_plan* p, const Acts& a, int reference_ops) {
  const svodb_model& m = *p->model;
  const svodb_qwen3_config& c = m.q;
  const int dt = c.dtype;
  const int64_t B = p->rows, L = p->len, D = c.hidden, H = c.heads, Hkv = c.kv_heads, hd = c.head_dim, F = c.ffn;
  const int64_t QKV = (H + 2 * Hkv) * hd;
  void* s = p->stream;
  svodb_tensor ids = tensor(p->ids, SVODB_I32, {B, L});
  svodb_tensor table = tensor(m.qw.embed, dt, {c.vocab, D});
  svodb_tensor x = tensor(a.x, dt, {B, L, D});
  svodb_tensor xn = tensor(a.xn, dt, {B, L, D});
  svodb_tensor qkv = tensor(a.qkv, dt, {B, L, QKV});
  svodb_tensor attn4 = tensor(a.attn, dt, {B, L, H, hd});
  svodb_tensor attn3 = tensor(a.attn, dt, {B, L, H * hd});
  svodb_tensor h = tensor(a.h, dt, {B, L, D});
  svodb_tensor hn = tensor(a.hn, dt, {B, L, D});
  svodb_tensor g = tensor(a.g, dt, {B, L, F});
  svodb_tensor cos = tensor(a.cos, dt, {1, L, 1, hd / 2});
  svodb_tensor sin = tensor(a.sin, dt, {1, L, 1, hd / 2});
  RUN(svodb_embed(&ids, &table, nullptr, nullptr, -1, &x, s));
  svodb_attn_opts causal{};
  causal.causal = 1;
  for (const svodb_qwen3_layer& lw : m.q_layers) {
    svodb_tensor in_w = tensor(lw.in_w, dt, {D});
    svodb_tensor post_w = tensor(lw.post_w, dt, {D});
    svodb_tensor qkv_w = tensor(lw.qkv_w, dt, {QKV, D});
    svodb_tensor o_w = tensor(lw.o_w, dt, {D, H * hd});
    svodb_tensor gu_w = tensor(lw.gu_w, dt, {2 * F, D});
    svodb_tensor down_w = tensor(lw.down_w, dt, {D, F});
    svodb_tensor qn_w = tensor(lw.qn_w, dt, {hd});
    svodb_tensor kn_w = tensor(lw.kn_w, dt, {hd});
    svodb_qkv_opts pro{};
    pro.heads = (int32_t)H, pro.kv_heads = (int32_t)Hkv, pro.head_dim = (int32_t)hd;
    pro.q_norm = &qn_w, pro.k_norm = &kn_w;
    pro.eps = c.eps;
    pro.rope_cos = &cos, pro.rope_sin = &sin;
    RUN(svodb_rms_norm(&x, &in_w, c.eps, &xn, s));
    if (!reference_ops) {
      svodb_linear_opts lo{};
      lo.qkv = &pro;
      RUN(svodb_linear(&xn, &qkv_w, &lo, &qkv, s));
      RUN(svodb_attention_packed(&qkv, (int32_t)H, (int32_t)Hkv, &causal, &attn4, s));
    } else {
      svodb_tensor q = tensor(a.q, dt, {B, L, H, hd});
      svodb_tensor k = tensor(a.k, dt, {B, L, Hkv, hd});
      svodb_tensor v = tensor(a.v, dt, {B, L, Hkv, hd});
      RUN(svodb_linear(&xn, &qkv_w, nullptr, &qkv, s));
      RUN(svodb_heads(&qkv, &pro, &q, &k, &v, s));
      RUN(svodb_attention(&q, &k, &v, &causal, &attn4, s));
    }
    svodb_linear_opts oo{};
    oo.residual = &x;
    RUN(svodb_linear(&attn3, &o_w, &oo, &h, s));
    RUN(svodb_rms_norm(&h, &post_w, c.eps, &hn, s));
    svodb_linear_opts go{};
    go.act = SVODB_ACT_SILU;
    go.gated = 1;
    RUN(svodb_linear(&hn, &gu_w, &go, &g, s));
    svodb_linear_opts dn{};
    dn.residual = &h;
    RUN(svodb_linear(&g, &down_w, &dn, &x, s));
  }
  // final RMSNorm of the pooled (last real) tokens, pooling, L2: one kernel
  svodb_tensor norm_w = tensor(m.qw.norm_w, dt, {D});
  svodb_tensor lens = tensor(p->aux, SVODB_I32, {B});
  svodb_tensor pooled = tensor(p->pooled, SVODB_F32, {B, D});
  RUN(svodb_norm_pool(&x, &norm_w, nullptr, c.eps, 0, &xn, &lens, 2, 1, &pooled, s));
  return SVODB_OK;
}

int forward_xlmr(const svodb_plan* p, const Acts& a) {
  const svodb_model& m = *p->model;
  const svodb_xlmr_config& c = m.x;
  const int dt = c.dtype;
  const int64_t B = p->rows, L = p->len, D = c.hidden, H = c.heads, F = c.ffn;
  void* s = p->stream;
  svodb_tensor ids = tensor(p->ids, SVODB_I32, {B, L});
  svodb_tensor mask = tensor(p->aux, SVODB_U8, {B, L});
  svodb_tensor word = tensor(m.xw.word, dt, {c.vocab, D});
  svodb_tensor pos = tensor(m.xw.pos, dt, {c.max_positions, D});
  svodb_tensor type = tensor(m.xw.type, dt, {D});
  svodb_tensor eln_w = tensor(m.xw.emb_ln_w, dt, {D});
  svodb_tensor eln_b = tensor(m.xw.emb_ln_b, dt, {D});
  svodb_tensor x = tensor(a.x, dt, {B, L, D});
  svodb_tensor qkv = tensor(a.qkv, dt, {B, L, 3 * D});
  svodb_tensor attn4 = tensor(a.attn, dt, {B, L, H, D / H});
  svodb_tensor attn3 = tensor(a.attn, dt, {B, L, D});
  svodb_tensor y = tensor(a.h, dt, {B, L, D});
  svodb_tensor x1 = tensor(a.hn, dt, {B, L, D});
  svodb_tensor f = tensor(a.g, dt, {B, L, F});
  RUN(svodb_embed_norm(&ids, &word, &pos, &type, c.pad_id, &eln_w, &eln_b, c.eps, 1, &x, s));
  svodb_attn_opts keys{};
  keys.key_mask = &mask;
  for (const svodb_xlmr_layer& lw : m.x_layers) {
    svodb_tensor qkv_w = tensor(lw.qkv_w, dt, {3 * D, D}), qkv_b = tensor(lw.qkv_b, dt, {3 * D});
    svodb_tensor o_w = tensor(lw.o_w, dt, {D, D}), o_b = tensor(lw.o_b, dt, {D});
    svodb_tensor ln1_w = tensor(lw.ln1_w, dt, {D}), ln1_b = tensor(lw.ln1_b, dt, {D});
    svodb_tensor fi_w = tensor(lw.fi_w, dt, {F, D}), fi_b = tensor(lw.fi_b, dt, {F});
    svodb_tensor fo_w = tensor(lw.fo_w, dt, {D, F}), fo_b = tensor(lw.fo_b, dt, {D});
    svodb_tensor ln2_w = tensor(lw.ln2_w, dt, {D}), ln2_b = tensor(lw.ln2_b, dt, {D});
    svodb_linear_opts po{};
    po.bias = &qkv_b;
    RUN(svodb_linear(&x, &qkv_w, &po, &qkv, s));
    RUN(svodb_attention_packed(&qkv, (int32_t)H, (int32_t)H, &keys, &attn4, s));
    svodb_linear_opts oo{};
    oo.bias = &o_b, oo.residual = &x;
    RUN(svodb_linear(&attn3, &o_w, &oo, &y, s));
    RUN(svodb_layer_norm(&y, &ln1_w, &ln1_b, c.eps, &x1, s));
    svodb_linear_opts fi{};
    fi.bias = &fi_b, fi.act = SVODB_ACT_GELU;
    RUN(svodb_linear(&x1, &fi_w, &fi, &f, s));
    svodb_linear_opts fo{};
    fo.bias = &fo_b, fo.residual = &x1;
    RUN(svodb_linear(&f, &fo_w, &fo, &y, s));
    RUN(svodb_layer_norm(&y, &ln2_w, &ln2_b, c.eps, &x, s));
  }
  // post-LN: the last layer's norm is the final one; pooling + L2 in one kernel
  svodb_tensor pooled = tensor(p->pooled, SVODB_F32, {B, D});
  const int mode = c.pooling == 1 ? 1 : 0;
  RUN(svodb_norm_pool(&x, nullptr, nullptr, c.eps, 1, nullptr, mode == 1 ? &mask : nullptr, mode, 1, &pooled, s));
  return SVODB_OK;
}

int forward_modernbert(const svodb_plan* p, const Acts& a) {
  const svodb_model& m = *p->model;
  const svodb_modernbert_config& c = m.m;
  const int dt = c.dtype;
  const int64_t B = p->rows, L = p->len, D = c.hidden, H = c.heads, F = c.ffn, hd = D / H;
  void* s = p->stream;
  svodb_tensor ids = tensor(p->ids, SVODB_I32, {B, L});
  svodb_tensor mask = tensor(p->aux, SVODB_U8, {B, L});
  svodb_tensor table = tensor(m.mw.embed, dt, {c.vocab, D});
  svodb_tensor eln_w = tensor(m.mw.emb_ln_w, dt, {D});
  svodb_tensor x = tensor(a.x, dt, {B, L, D});
  svodb_tensor xn = tensor(a.xn, dt, {B, L, D});
  svodb_tensor qkv = tensor(a.qkv, dt, {B, L, 3 * D});
  svodb_tensor attn4 = tensor(a.attn, dt, {B, L, H, hd});
  svodb_tensor attn3 = tensor(a.attn, dt, {B, L, D});
  svodb_tensor h = tensor(a.h, dt, {B, L, D});
  svodb_tensor hn = tensor(a.hn, dt, {B, L, D});
  svodb_tensor g = tensor(a.g, dt, {B, L, F});
  svodb_tensor cos_g = tensor(a.cos, dt, {1, L, 1, hd / 2}), sin_g = tensor(a.sin, dt, {1, L, 1, hd / 2});
  svodb_tensor cos_l = tensor(a.cos2, dt, {1, L, 1, hd / 2}), sin_l = tensor(a.sin2, dt, {1, L, 1, hd / 2});
  RUN(svodb_embed_norm(&ids, &table, nullptr, nullptr, -1, &eln_w, nullptr, c.eps, 1, &x, s));
  int li = 0;
  for (const svodb_modernbert_layer& lw : m.m_layers) {
    const bool global = li % c.global_every == 0;
    ++li;
    svodb_tensor qkv_w = tensor(lw.qkv_w, dt, {3 * D, D});
    svodb_tensor o_w = tensor(lw.o_w, dt, {D, D});
    svodb_tensor mlp_w = tensor(lw.mlp_ln_w, dt, {D});
    svodb_tensor wi_w = tensor(lw.wi_w, dt, {2 * F, D});
    svodb_tensor wo_w = tensor(lw.wo_w, dt, {D, F});
    const svodb_tensor* src = &x;
    svodb_tensor aw;
    if (lw.attn_ln_w != nullptr) {  // layer 0 has no attention norm
      aw = tensor(lw.attn_ln_w, dt, {D});
      RUN(svodb_layer_norm(&x, &aw, nullptr, c.eps, &xn, s));
      src = &xn;
    }
    svodb_linear_opts po{};
    po.rope_cos = global ? &cos_g : &cos_l;
    po.rope_sin = global ? &sin_g : &sin_l;
    po.rope_heads = (int32_t)(2 * H);
    po.rope_head_dim = (int32_t)hd;
    RUN(svodb_linear(src, &qkv_w, &po, &qkv, s));
    svodb_attn_opts ao{};
    ao.key_mask = &mask;
    if (!global) {
      ao.has_window = 1;
      ao.window_left = ao.window_right = c.local_window / 2;
    }
    RUN(svodb_attention_packed(&qkv, (int32_t)H, (int32_t)H, &ao, &attn4, s));
    svodb_linear_opts oo{};
    oo.residual = &x;
    RUN(svodb_linear(&attn3, &o_w, &oo, &h, s));
    RUN(svodb_layer_norm(&h, &mlp_w, nullptr, c.eps, &hn, s));
    svodb_linear_opts go{};
    go.act = SVODB_ACT_GELU;
    go.gated = 1;
    RUN(svodb_linear(&hn, &wi_w, &go, &g, s));
    svodb_linear_opts dn{};
    dn.residual = &h;
    RUN(svodb_linear(&g, &wo_w, &dn, &x, s));
  }
  // final LayerNorm of the pooled tokens, pooling, L2: one kernel
  svodb_tensor fln = tensor(m.mw.final_ln_w, dt, {D});
  svodb_tensor pooled = tensor(p->pooled, SVODB_F32, {B, D});
  const int mode = c.pooling == 0 ? 0 : 1;
  RUN(svodb_norm_pool(&x, &fln, nullptr, c.eps, 1, &xn, mode == 1 ? &mask : nullptr, mode, 1, &pooled, s));
  return SVODB_OK;
}

int forward(const svodb_plan* p, const Acts& a, int reference_ops) {
  switch (p->model->kind) {
    case kQwen3: return forward_qwen3(p, a, reference_ops);
    case kXlmr: return forward_xlmr(p, a);
    default: return forward_modernbert(p, a);
  }
}

int bad(int code, const char* msg) {
  svodb::set_last_error("%s", msg);
  return code;
}

bool half_type(int dt) { return dt == SVODB_BF16 || dt == SVODB_F16; }

}  // namespace

extern "C" {

int svodb_qwen3_create(const svodb_qwen3_config* cfg, const svodb_qwen3_weights* w, svodb_model** out) {
  if (cfg == nullptr || w == nullptr || out == nullptr || w->layers == nullptr || w->embed == nullptr ||
      w->norm_w == nullptr)
    return bad(SVODB_ERR_UNREALIZED, "qwen3_create: null argument");
  if (!(cfg->kv_heads > 0 && cfg->heads % cfg->kv_heads == 0)) {
    svodb::set_last_error("qwen3_create: %d query heads are not a multiple of %d key/value heads", cfg->heads,
                          cfg->kv_heads);
    return SVODB_ERR_HEADS;
  }
  // the embedding lookup is a 16-bit kernel: an f32 model would only fail later, at plan time
  if (!half_type(cfg->dtype)) return bad(SVODB_ERR_DTYPE, "qwen3_create: weights must be bf16 or f16");
  svodb_model* m = new svodb_model();
  m->kind = kQwen3;
  m->q = *cfg;
  m->q_layers.assign(w->layers, w->layers + cfg->layers);
  m->qw = *w;
  m->qw.layers = m->q_layers.data();
  *out = m;
  return SVODB_OK;
}

int svodb_xlmr_create(const svodb_xlmr_config* cfg, const svodb_xlmr_weights* w, svodb_model** out) {
  if (cfg == nullptr || w == nullptr || out == nullptr || w->layers == nullptr || w->word == nullptr ||
      w->pos == nullptr || w->type == nullptr || w->emb_ln_w == nullptr || w->emb_ln_b == nullptr)
    return bad(SVODB_ERR_UNREALIZED, "xlmr_create: null argument");
  if (!(cfg->heads > 0 && cfg->hidden % cfg->heads == 0))
    return bad(SVODB_ERR_HEADS, "xlmr_create: the hidden size is not a multiple of the head count");
  if (!half_type(cfg->dtype)) return bad(SVODB_ERR_DTYPE, "xlmr_create: weights must be bf16 or f16");
  svodb_model* m = new svodb_model();
  m->kind = kXlmr;
  m->x = *cfg;
  m->x_layers.assign(w->layers, w->layers + cfg->layers);
  m->xw = *w;
  m->xw.layers = m->x_layers.data();
  *out = m;
  return SVODB_OK;
}

int svodb_modernbert_create(const svodb_modernbert_config* cfg, const svodb_modernbert_weights* w,
                            svodb_model** out) {
  if (cfg == nullptr || w == nullptr || out == nullptr || w->layers == nullptr || w->embed == nullptr ||
      w->emb_ln_w == nullptr || w->final_ln_w == nullptr)
    return bad(SVODB_ERR_UNREALIZED, "modernbert_create: null argument");
  if (!(cfg->heads > 0 && cfg->hidden % cfg->heads == 0))
    return bad(SVODB_ERR_HEADS, "modernbert_create: the hidden size is not a multiple of the head count");
  if (cfg->global_every <= 0) return bad(SVODB_ERR_SHAPE, "modernbert_create: global_every must be positive");
  if (!half_type(cfg->dtype)) return bad(SVODB_ERR_DTYPE, "modernbert_create: weights must be bf16 or f16");
  svodb_model* m = new svodb_model();
  m->kind = kModernBert;
  m->m = *cfg;
  m->m_layers.assign(w->layers, w->layers + cfg->layers);
  m->mw = *w;
  m->mw.layers = m->m_layers.data();
  *out = m;
  return SVODB_OK;
}

void svodb_model_free(svodb_model* m) { delete m; }

int svodb_model_plan(svodb_model* m, int64_t rows, int64_t len, int32_t reference_ops, svodb_plan** out) {
  if (m == nullptr || out == nullptr || rows <= 0 || len <= 0)
    return bad(SVODB_ERR_SHAPE, "model_plan: a plan needs a model and a positive shape");
  if (m->kind != kQwen3) reference_ops = 0;
  svodb_plan* p = new svodb_plan();
  p->model = m;
  p->rows = rows, p->len = len;
  p->graph = nullptr;
  p->arena = nullptr;
  p->aux_bytes = m->kind == kQwen3 ? (size_t)rows * 4 : (size_t)rows * len;
  const size_t D = (size_t)m->hidden();
  // size the arena with a dry carve, then carve for real
  Bump dry{nullptr, 0};
  dry.take((size_t)rows * len * 4);
  dry.take(p->aux_bytes);
  dry.take((size_t)rows * D * 4);
  carve(dry, *m, rows, len, reference_ops);
  p->arena_bytes = dry.at;
  if (cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete p;
    return bad(SVODB_ERR_LAUNCH, "model_plan: no stream");
  }
  int rc = svodb_alloc(p->arena_bytes, 0, (void**)&p->arena);
  if (rc != SVODB_OK) {
    cudaStreamDestroy(p->stream);
    delete p;
    return rc;
  }
  Bump b{p->arena, 0};
  p->ids = (int32_t*)b.take((size_t)rows * len * 4);
  p->aux = b.take(p->aux_bytes);
  p->pooled = (float*)b.take((size_t)rows * D * 4);
  Acts a = carve(b, *m, rows, len, reference_ops);
  // inputs until the first run: token 0 everywhere, full-length rows
  cudaMemsetAsync(p->ids, 0, (size_t)rows * len * 4, p->stream);
  if (m->kind == kQwen3) {
    std::vector<int32_t> full((size_t)rows, (int32_t)len);
    cudaMemcpyAsync(p->aux, full.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, p->stream);
    cudaStreamSynchronize(p->stream);  // `full` leaves scope below
    svodb_tensor cos = tensor(a.cos, m->q.dtype, {len, m->q.head_dim / 2});
    svodb_tensor sin = tensor(a.sin, m->q.dtype, {len, m->q.head_dim / 2});
    rc = svodb_rope_table(m->q.rope_theta, nullptr, m->q.head_dim, &cos, &sin, p->stream);
  } else {
    cudaMemsetAsync(p->aux, 1, p->aux_bytes, p->stream);
    if (m->kind == kModernBert) {
      const int32_t hd = m->m.hidden / m->m.heads;
      svodb_tensor cg = tensor(a.cos, m->m.dtype, {len, hd / 2}), sg = tensor(a.sin, m->m.dtype, {len, hd / 2});
      svodb_tensor cl = tensor(a.cos2, m->m.dtype, {len, hd / 2}), sl = tensor(a.sin2, m->m.dtype, {len, hd / 2});
      rc = svodb_rope_table(m->m.global_theta, nullptr, hd, &cg, &sg, p->stream);
      if (rc == SVODB_OK) rc = svodb_rope_table(m->m.local_theta, nullptr, hd, &cl, &sl, p->stream);
    }
  }
  // One eager pass first: first-use work (kernel attributes) happens outside the capture.
  if (rc == SVODB_OK) rc = forward(p, a, reference_ops);
  if (rc == SVODB_OK) rc = svodb_device_status(p->stream);
  if (rc == SVODB_OK) rc = svodb_graph_begin(p->stream);
  if (rc == SVODB_OK) {
    rc = forward(p, a, reference_ops);
    svodb_graph* g = nullptr;
    int rc_end = svodb_graph_end(p->stream, &g);
    if (rc == SVODB_OK) rc = rc_end;
    p->graph = g;
  }
  if (rc != SVODB_OK) {
    svodb_plan_free(p);
    return rc;
  }
  *out = p;
  return SVODB_OK;
}

int svodb_plan_run(svodb_plan* p, const int32_t* host_ids, const void* host_aux, float* host_out) {
  if (p == nullptr || p->graph == nullptr) return bad(SVODB_ERR_UNREALIZED, "plan_run: the plan was not prepared");
  const size_t D = (size_t)p->model->hidden();
  if (host_ids != nullptr) RUN(svodb_copy_h2d(p->ids, host_ids, (size_t)p->rows * p->len * 4, p->stream));
  if (host_aux != nullptr) RUN(svodb_copy_h2d(p->aux, host_aux, p->aux_bytes, p->stream));
  RUN(svodb_graph_replay(p->graph, p->stream));
  if (host_out != nullptr) {
    RUN(svodb_copy_d2h(host_out, p->pooled, (size_t)p->rows * D * 4, p->stream));
    // waits for the stream and reads (and clears) the status word: a bounded wait
    // that ran out during this replay is this call's error, never a later launch's
    RUN(svodb_device_status(p->stream));
  }
  return SVODB_OK;
}

void* svodb_plan_stream(svodb_plan* p) { return p != nullptr ? (void*)p->stream : nullptr; }
float* svodb_plan_output(svodb_plan* p) { return p != nullptr ? p->pooled : nullptr; }

void svodb_plan_free(svodb_plan* p) {
  if (p == nullptr) return;
  if (p->stream != nullptr) cudaStreamSynchronize(p->stream);
  svodb_graph_free(p->graph);
  svodb_free(p->arena, 0);
  if (p->stream != nullptr) cudaStreamDestroy(p->stream);
  delete p;
}

}  // extern "C"
