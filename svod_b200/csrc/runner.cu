// Native runner of the Qwen3 embedding stack: the host side a compiled caller
// links instead of a Python one. It owns what `HeadPlans` owns in the reference
// (model/src/encoder_head.rs:384-500): per plan shape `(rows, len)` one arena of
// activations, the RoPE tables, and one captured CUDA graph of the whole stack;
// a run is two host-to-device copies, a graph launch and one device-to-host copy
// of the pooled rows.
//
// The op sequence is the reference's (model/src/qwen3/decoder_layer.rs:55-65,
// attention.rs:69-113, feed_forward.rs:38-42, model.rs:77-99), issued through
// this library's own C entry points, with the attention prologue in the QKV
// projection's store unless `reference_ops` asks for linear -> heads -> attention.
#include <cuda_runtime.h>
#include <string.h>

#include <vector>

#include "kernels.h"
#include "svodb.h"

struct svodb_qwen3 {
  svodb_qwen3_config cfg;
  std::vector<svodb_qwen3_layer> layers;
  const void* embed;
  const void* norm_w;
};

struct svodb_plan {
  const svodb_qwen3* model;
  int64_t rows, len;
  char* arena;        // every device buffer of the plan, one allocation
  size_t arena_bytes;
  int32_t* ids;       // [rows, len]
  int32_t* lengths;   // [rows]
  float* pooled;      // [rows, D]
  svodb_graph* graph;
  cudaStream_t stream;
};

namespace {

size_t esize_of(int dtype) { return dtype == SVODB_F32 ? 4 : 2; }

svodb_tensor tensor(void* data, int dtype, std::initializer_list<int64_t> shape) {
  svodb_tensor t{};
  t.data = data;
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

// The whole stack on `stream`, reading plan->ids / plan->lengths and writing
// plan->pooled. `bufs` are the activations carved from the arena.
struct Acts {
  void *x, *xn, *qkv, *q, *k, *v, *attn, *h, *hn, *g, *cos, *sin;
};

int forward(const svodb_plan* p, const Acts& a, int reference_ops) {
  const svodb_qwen3_config& c = p->model->cfg;
  const int dt = c.dtype;
  const int64_t B = p->rows, L = p->len, D = c.hidden, H = c.heads, Hkv = c.kv_heads, hd = c.head_dim, F = c.ffn;
  const int64_t QKV = (H + 2 * Hkv) * hd;
  void* s = p->stream;
  svodb_tensor ids = tensor(p->ids, SVODB_I32, {B, L});
  svodb_tensor table = tensor(const_cast<void*>(p->model->embed), dt, {c.vocab, D});
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
  for (const svodb_qwen3_layer& lw : p->model->layers) {
    svodb_tensor in_w = tensor(const_cast<void*>(lw.in_w), dt, {D});
    svodb_tensor post_w = tensor(const_cast<void*>(lw.post_w), dt, {D});
    svodb_tensor qkv_w = tensor(const_cast<void*>(lw.qkv_w), dt, {QKV, D});
    svodb_tensor o_w = tensor(const_cast<void*>(lw.o_w), dt, {D, H * hd});
    svodb_tensor gu_w = tensor(const_cast<void*>(lw.gu_w), dt, {2 * F, D});
    svodb_tensor down_w = tensor(const_cast<void*>(lw.down_w), dt, {D, F});
    svodb_tensor qn_w = tensor(const_cast<void*>(lw.qn_w), dt, {hd});
    svodb_tensor kn_w = tensor(const_cast<void*>(lw.kn_w), dt, {hd});
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
  svodb_tensor norm_w = tensor(const_cast<void*>(p->model->norm_w), dt, {D});
  RUN(svodb_rms_norm(&x, &norm_w, c.eps, &xn, s));
  svodb_tensor lens = tensor(p->lengths, SVODB_I32, {B});
  svodb_tensor pooled = tensor(p->pooled, SVODB_F32, {B, D});
  RUN(svodb_pool(&xn, &lens, 2, 1, &pooled, s));
  return SVODB_OK;
}

Acts carve(Bump& b, const svodb_qwen3_config& c, int64_t B, int64_t L, int reference_ops) {
  const size_t e = esize_of(c.dtype);
  const size_t tok = (size_t)B * L;
  const size_t qkv = (size_t)(c.heads + 2 * c.kv_heads) * c.head_dim;
  Acts a{};
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
  return a;
}

}  // namespace

extern "C" {

int svodb_qwen3_create(const svodb_qwen3_config* cfg, const svodb_qwen3_weights* w, svodb_qwen3** out) {
  if (cfg == nullptr || w == nullptr || out == nullptr || w->layers == nullptr || w->embed == nullptr ||
      w->norm_w == nullptr) {
    svodb::set_last_error("qwen3_create: null argument");
    return SVODB_ERR_UNREALIZED;
  }
  if (!(cfg->kv_heads > 0 && cfg->heads % cfg->kv_heads == 0)) {
    svodb::set_last_error("qwen3_create: %d query heads are not a multiple of %d key/value heads", cfg->heads,
                          cfg->kv_heads);
    return SVODB_ERR_HEADS;
  }
  if (cfg->dtype != SVODB_BF16 && cfg->dtype != SVODB_F16 && cfg->dtype != SVODB_F32) {
    svodb::set_last_error("qwen3_create: weights must be a float type");
    return SVODB_ERR_DTYPE;
  }
  svodb_qwen3* m = new svodb_qwen3();
  m->cfg = *cfg;
  m->layers.assign(w->layers, w->layers + cfg->layers);
  m->embed = w->embed;
  m->norm_w = w->norm_w;
  *out = m;
  return SVODB_OK;
}

void svodb_qwen3_free(svodb_qwen3* m) { delete m; }

int svodb_qwen3_plan(svodb_qwen3* m, int64_t rows, int64_t len, int32_t reference_ops, svodb_plan** out) {
  if (m == nullptr || out == nullptr || rows <= 0 || len <= 0) {
    svodb::set_last_error("qwen3_plan: a plan needs a model and a positive shape");
    return SVODB_ERR_SHAPE;
  }
  svodb_plan* p = new svodb_plan();
  p->model = m;
  p->rows = rows, p->len = len;
  p->graph = nullptr;
  p->arena = nullptr;
  // size the arena with a dry carve, then carve for real
  Bump dry{nullptr, 0};
  dry.take((size_t)rows * len * 4);
  dry.take((size_t)rows * 4);
  dry.take((size_t)rows * m->cfg.hidden * 4);
  carve(dry, m->cfg, rows, len, reference_ops);
  p->arena_bytes = dry.at;
  if (cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete p;
    svodb::set_last_error("qwen3_plan: no stream");
    return SVODB_ERR_LAUNCH;
  }
  int rc = svodb_alloc(p->arena_bytes, 0, (void**)&p->arena);
  if (rc != SVODB_OK) {
    cudaStreamDestroy(p->stream);
    delete p;
    return rc;
  }
  Bump b{p->arena, 0};
  p->ids = (int32_t*)b.take((size_t)rows * len * 4);
  p->lengths = (int32_t*)b.take((size_t)rows * 4);
  p->pooled = (float*)b.take((size_t)rows * m->cfg.hidden * 4);
  Acts a = carve(b, m->cfg, rows, len, reference_ops);
  cudaMemsetAsync(p->ids, 0, (size_t)rows * len * 4, p->stream);
  std::vector<int32_t> full((size_t)rows, (int32_t)len);
  cudaMemcpyAsync(p->lengths, full.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, p->stream);
  svodb_tensor cos = tensor(a.cos, m->cfg.dtype, {len, m->cfg.head_dim / 2});
  svodb_tensor sin = tensor(a.sin, m->cfg.dtype, {len, m->cfg.head_dim / 2});
  rc = svodb_rope_table(m->cfg.rope_theta, nullptr, m->cfg.head_dim, &cos, &sin, p->stream);
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

int svodb_plan_run(svodb_plan* p, const int32_t* host_ids, const int32_t* host_lengths, float* host_out) {
  if (p == nullptr || p->graph == nullptr) {
    svodb::set_last_error("plan_run: the plan was not prepared");
    return SVODB_ERR_UNREALIZED;
  }
  const size_t D = (size_t)p->model->cfg.hidden;
  if (host_ids != nullptr) RUN(svodb_copy_h2d(p->ids, host_ids, (size_t)p->rows * p->len * 4, p->stream));
  if (host_lengths != nullptr) RUN(svodb_copy_h2d(p->lengths, host_lengths, (size_t)p->rows * 4, p->stream));
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
