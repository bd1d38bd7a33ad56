// The C ABI: validation in the order and with the error classes of svod's
// `tk::ops` (tk/src/ops/{linear,attention,heads,norm}.rs), kernel-vs-generic
// dispatch (the reference's kernel-vs-graph `Plan`, tk/src/ops/shape.rs:92-231),
// the `chosen()` report, and the device seam (module load / launch, graph
// capture / replay, allocator).
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "svodb.h"

using namespace svodb;

namespace {

thread_local char g_error[512] = "";
thread_local char g_chosen[256] = "";
bool g_poisoned = false;

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

void chose_kernel(const char* op, const char* family, const char* cfg) {
  snprintf(g_chosen, sizeof g_chosen, "%s: kernel %s %s", op, family, cfg);
}
void chose_graph(const char* op, const char* why) { snprintf(g_chosen, sizeof g_chosen, "%s: graph %s", op, why); }

// Sticky CUDA errors poison the device: every later call fails fast
// (device/src/cuda/sys.rs:78-96).
bool sticky(cudaError_t e) {
  switch (e) {
    case cudaErrorIllegalAddress:
    case cudaErrorLaunchFailure:
    case cudaErrorIllegalInstruction:
    case cudaErrorMisalignedAddress:
    case cudaErrorHardwareStackError:
    case cudaErrorInvalidAddressSpace:
    case cudaErrorInvalidPc:
    case cudaErrorAssert:
    case cudaErrorECCUncorrectable:
      return true;
    default:
      return false;
  }
}

int check_launch(const char* op) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return SVODB_OK;
  if (sticky(e)) g_poisoned = true;
  return fail(SVODB_ERR_LAUNCH, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
}

#define GUARD(op)                                                                       \
  do {                                                                                  \
    if (g_poisoned) return fail(SVODB_ERR_POISONED, "%s: the device is poisoned", op); \
  } while (0)

bool is_float(int dt) { return dt == SVODB_F32 || dt == SVODB_F16 || dt == SVODB_BF16; }
bool is_half(int dt) { return dt == SVODB_F16 || dt == SVODB_BF16; }
const char* dtype_name(int dt) {
  static const char* names[] = {"Float32", "Float16", "BFloat16", "Int32", "Int64", "UInt8"};
  return dt >= 0 && dt <= 5 ? names[dt] : "?";
}
size_t esize(int dt) {
  switch (dt) {
    case SVODB_F32: case SVODB_I32: return 4;
    case SVODB_I64: return 8;
    case SVODB_U8: return 1;
    default: return 2;
  }
}

void fmt_shape(const svodb_tensor* t, char* buf, size_t n) {
  size_t at = (size_t)snprintf(buf, n, "[");
  for (int i = 0; i < t->rank && at < n; ++i)
    at += (size_t)snprintf(buf + at, n - at, i ? ", %lld" : "%lld", (long long)t->shape[i]);
  if (at < n) snprintf(buf + at, n - at, "]");
}

int shape_err(const char* op, const char* operand, const svodb_tensor* got, const char* expected) {
  char buf[128];
  fmt_shape(got, buf, sizeof buf);
  return fail(SVODB_ERR_SHAPE, "%s: %s has shape %s, expected %s", op, operand, buf, expected);
}
int dtype_err(const char* op, const char* operand, int got, int want) {
  return fail(SVODB_ERR_DTYPE, "%s: %s is %s, the input is %s", op, operand, dtype_name(got), dtype_name(want));
}

int64_t numel(const svodb_tensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->rank; ++i) n *= t->shape[i];
  return n;
}

// Dense row-major in every dim but an optionally wider stride of dim `rank-2`
// (a channel window of a wider buffer).
bool rows_dense(const svodb_tensor* t) {
  if (t->rank == 0) return true;
  if (t->stride[t->rank - 1] != 1) return false;
  if (t->rank == 1) return true;
  int64_t ld = t->stride[t->rank - 2];
  if (ld < t->shape[t->rank - 1]) return false;
  int64_t expect = ld * t->shape[t->rank - 2];
  for (int i = t->rank - 3; i >= 0; --i) {
    if (t->stride[i] != expect) return false;
    expect *= t->shape[i];
  }
  return true;
}
bool contiguous(const svodb_tensor* t) {
  int64_t expect = 1;
  for (int i = t->rank - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->stride[i] != expect) return false;
    expect *= t->shape[i];
  }
  return true;
}

int realized(const char* op, const char* operand, const svodb_tensor* t) {
  if (t == nullptr) return fail(SVODB_ERR_UNREALIZED, "%s: %s is missing", op, operand);
  if (t->rank < 0 || t->rank > SVODB_MAX_RANK) return shape_err(op, operand, t, "rank <= 5");
  if (t->data == nullptr && numel(t) != 0)
    return fail(SVODB_ERR_UNREALIZED, "%s: %s is not a realized buffer", op, operand);
  return SVODB_OK;
}

// `launch::aliasing` (tk/src/launch.rs:227-246): a written parameter may not
// share storage with another parameter.
struct Span {
  const char* lo;
  const char* hi;
};
Span span_of(const svodb_tensor* t) {
  int64_t last = 0;
  for (int i = 0; i < t->rank; ++i)
    if (t->shape[i] > 0) last += (t->shape[i] - 1) * t->stride[i];
  const char* lo = (const char*)t->data;
  return Span{lo, lo + (size_t)(last + 1) * esize(t->dtype)};
}
int no_alias(const char* op, const svodb_tensor* out, std::initializer_list<const svodb_tensor*> others) {
  if (out == nullptr || out->data == nullptr) return SVODB_OK;
  Span o = span_of(out);
  for (const svodb_tensor* t : others) {
    if (t == nullptr || t->data == nullptr || t == out) continue;
    Span s = span_of(t);
    if (o.lo < s.hi && s.lo < o.hi) return fail(SVODB_ERR_ALIAS, "%s: an output shares storage with an input", op);
  }
  return SVODB_OK;
}

bool same_shape(const svodb_tensor* a, const svodb_tensor* b) {
  if (a->rank != b->rank) return false;
  for (int i = 0; i < a->rank; ++i)
    if (a->shape[i] != b->shape[i]) return false;
  return true;
}

#define TRY(expr)                  \
  do {                             \
    int rc_ = (expr);              \
    if (rc_ != SVODB_OK) return rc_; \
  } while (0)

}  // namespace

// The status word bounded device waits report into: a module-scope device
// variable (one instance per device that loads the library), so the op layer
// allocates nothing.
__device__ uint32_t g_status_word = 0;

namespace svodb {
void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}

uint32_t* device_status_word() {
  static std::mutex mu;
  static std::vector<uint32_t*> words(64, nullptr);
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 0 || dev >= (int)words.size()) return nullptr;
  if (words[dev] == nullptr) {
    void* w = nullptr;
    if (cudaGetSymbolAddress(&w, g_status_word) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    words[dev] = (uint32_t*)w;
  }
  return words[dev];
}
}  // namespace svodb

extern "C" {

const char* svodb_version(void) { return "svodb 0.1 (sm_100a)"; }
const char* svodb_last_error(void) { return g_error; }
const char* svodb_last_chosen(void) { return g_chosen; }

// ---------------------------------------------------------------------------
// shape-keyed configs (the process half of a tune store)
// ---------------------------------------------------------------------------
namespace {
thread_local char g_config_key[160] = "";
std::mutex g_config_mutex;
std::unordered_map<std::string, int32_t>& config_map() {
  static std::unordered_map<std::string, int32_t> m;
  return m;
}
int32_t config_lookup(const char* key) {
  std::lock_guard<std::mutex> lock(g_config_mutex);
  auto it = config_map().find(key);
  return it == config_map().end() ? 0 : it->second;
}
}  // namespace

const char* svodb_last_config_key(void) { return g_config_key; }
int svodb_config_set(const char* key, int32_t value) {
  if (key == nullptr || key[0] == 0) return fail(SVODB_ERR_GRAPH, "config: an empty key");
  std::lock_guard<std::mutex> lock(g_config_mutex);
  if (value == 0) config_map().erase(key);
  else config_map()[key] = value;
  return SVODB_OK;
}
int32_t svodb_config_get(const char* key) { return key == nullptr ? 0 : config_lookup(key); }
void svodb_config_clear(void) {
  std::lock_guard<std::mutex> lock(g_config_mutex);
  config_map().clear();
}

int svodb_supported(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

int svodb_device_status(void* stream) {
  GUARD("device_status");
  uint32_t* w = device_status_word();
  if (w == nullptr) return fail(SVODB_ERR_LAUNCH, "device_status: no status word");
  uint32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, w, sizeof host, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) {
    if (sticky(e)) g_poisoned = true;
    return fail(SVODB_ERR_LAUNCH, "device_status: %s", cudaGetErrorString(e));
  }
  if (host != 0) {
    cudaMemsetAsync(w, 0, sizeof host, (cudaStream_t)stream);
    cudaStreamSynchronize((cudaStream_t)stream);
    if (host == kStatusBadIndex)
      return fail(SVODB_ERR_SHAPE, "a device-side index was out of range (a cache row map entry)");
    return fail(SVODB_ERR_TIMEOUT, "a bounded device wait ran out (code %u)", host);
  }
  return SVODB_OK;
}

// The error latch, exercised without a device fault: `code` (a cudaError_t value)
// goes through the same classification as the result of a failed launch; a
// sticky code poisons the library exactly as a real one would.
int svodb_selftest_latch_error(int32_t code) {
  GUARD("selftest_latch_error");
  const cudaError_t e = (cudaError_t)code;
  if (e == cudaSuccess) return SVODB_OK;
  if (sticky(e)) g_poisoned = true;
  return fail(SVODB_ERR_LAUNCH, "selftest_latch_error: %s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
}

// Clears the latch a self-test set. A latch set by a real sticky error must not
// be cleared: that context is gone and the process has to restart.
void svodb_selftest_clear_latch(void) { g_poisoned = false; }

// ---------------------------------------------------------------------------
// linear
// ---------------------------------------------------------------------------
namespace {
// The attention prologue over a packed projection y [B,T,(H+2Hkv)*D], each head
// rewritten where it lies.
void heads_in_place(const svodb_qkv_opts* qo, svodb_tensor* y, int per_batch, cudaStream_t s) {
  if (qo->q_norm == nullptr && qo->k_norm == nullptr && qo->rope_cos == nullptr) return;
  HeadsArgs h{};
  h.qkv = y->data;
  h.q_w = qo->q_norm ? qo->q_norm->data : nullptr;
  h.k_w = qo->k_norm ? qo->k_norm->data : nullptr;
  h.cos = qo->rope_cos ? qo->rope_cos->data : nullptr;
  h.sin = qo->rope_sin ? qo->rope_sin->data : nullptr;
  h.batch = y->shape[0], h.t = y->shape[1];
  h.heads = qo->heads, h.kv_heads = qo->kv_heads, h.d = qo->head_dim;
  h.eps = (float)qo->eps;
  h.per_batch_tables = per_batch;
  h.dtype = y->dtype;
  h.in_place = 1;
  launch_heads(h, s);
}
}  // namespace

int svodb_linear(const svodb_tensor* x, const svodb_tensor* w, const svodb_linear_opts* opts, svodb_tensor* y,
                 void* stream) {
  static const char* OP = "linear";
  GUARD(OP);
  svodb_linear_opts none{};
  if (opts == nullptr) opts = &none;
  TRY(realized(OP, "x", x));
  TRY(realized(OP, "w", w));
  TRY(realized(OP, "y", y));
  if (x->rank < 1) return shape_err(OP, "x", x, "[..., K]");
  const int64_t k = x->shape[x->rank - 1];
  if (w->rank != 2 || w->shape[1] != k) return shape_err(OP, "w", w, "[N, K]");
  if (!is_float(x->dtype)) return fail(SVODB_ERR_GRAPH, "%s: x is %s, not a float type", OP, dtype_name(x->dtype));
  if (w->dtype != x->dtype) return dtype_err(OP, "w", w->dtype, x->dtype);
  int64_t n = w->shape[0];
  if (opts->gated) {
    if (n % 2 != 0) return shape_err(OP, "w", w, "[2N, K]");
    n /= 2;
  }
  if (opts->bias != nullptr) {
    TRY(realized(OP, "bias", opts->bias));
    if (opts->bias->rank != 1 || opts->bias->shape[0] != w->shape[0]) return shape_err(OP, "bias", opts->bias, "[N]");
    if (opts->bias->dtype != x->dtype) return dtype_err(OP, "bias", opts->bias->dtype, x->dtype);
  }
  // out shape = lead..., N
  if (y->rank != x->rank) return shape_err(OP, "y", y, "[lead..., N]");
  for (int i = 0; i < x->rank - 1; ++i)
    if (y->shape[i] != x->shape[i]) return shape_err(OP, "y", y, "[lead..., N]");
  if (y->shape[y->rank - 1] != n) return shape_err(OP, "y", y, "[lead..., N]");
  if (y->dtype != x->dtype) return dtype_err(OP, "y", y->dtype, x->dtype);
  if (opts->residual != nullptr) {
    TRY(realized(OP, "residual", opts->residual));
    if (!same_shape(opts->residual, y)) return shape_err(OP, "residual", opts->residual, "[lead..., N]");
    if (opts->residual->dtype != x->dtype) return dtype_err(OP, "residual", opts->residual->dtype, x->dtype);
  }
  const bool rope = opts->rope_cos != nullptr;
  int64_t seq = 0;
  const svodb_qkv_opts* qo = opts->qkv;
  int qkv_per_batch = 0;
  if (qo != nullptr) {
    // The `ops::heads` prologue in the store: same checks as `svodb_heads`.
    if (rope || opts->gated || opts->act != SVODB_ACT_NONE || opts->has_scale || opts->residual != nullptr)
      return fail(SVODB_ERR_GRAPH, "%s: the qkv prologue excludes rope, gate, activation, scale and residual", OP);
    const int H = qo->heads, Hkv = qo->kv_heads, d = qo->head_dim;
    if (!(Hkv > 0 && H > 0 && H % Hkv == 0))
      return fail(SVODB_ERR_HEADS, "%s: %d query heads are not a multiple of %d key/value heads", OP, H, Hkv);
    if (x->rank != 3) return shape_err(OP, "x", x, "[B, T, K] under the qkv prologue");
    if (d <= 0 || n != (int64_t)(H + 2 * Hkv) * d) return shape_err(OP, "w", w, "[(heads + 2*kv_heads)*head_dim, K]");
    const svodb_tensor* norms[2] = {qo->q_norm, qo->k_norm};
    const char* nnames[2] = {"q norm", "k norm"};
    for (int i = 0; i < 2; ++i) {
      if (norms[i] == nullptr) continue;
      TRY(realized(OP, nnames[i], norms[i]));
      if (norms[i]->rank != 1 || norms[i]->shape[0] != d || !contiguous(norms[i]))
        return shape_err(OP, nnames[i], norms[i], "[head_dim]");
      if (norms[i]->dtype != x->dtype) return dtype_err(OP, nnames[i], norms[i]->dtype, x->dtype);
    }
    if (qo->rope_cos != nullptr) {
      if (d % 2 != 0) return shape_err(OP, "w", w, "an even head_dim under a rotation");
      TRY(realized(OP, "cos", qo->rope_cos));
      TRY(realized(OP, "sin", qo->rope_sin));
      const svodb_tensor* c = qo->rope_cos;
      const int64_t B = x->shape[0], T = x->shape[1];
      const bool fits = c->rank == 4 && (c->shape[0] == 1 || c->shape[0] == B) && c->shape[1] == T &&
                        c->shape[2] == 1 && c->shape[3] == d / 2 && contiguous(c);
      if (!fits) return shape_err(OP, "cos", c, "[1 | B, T, 1, head_dim/2]");
      if (!same_shape(qo->rope_sin, c) || !contiguous(qo->rope_sin)) return shape_err(OP, "sin", qo->rope_sin, "the shape of cos");
      if (c->dtype != x->dtype) return dtype_err(OP, "cos", c->dtype, x->dtype);
      if (qo->rope_sin->dtype != x->dtype) return dtype_err(OP, "sin", qo->rope_sin->dtype, x->dtype);
      qkv_per_batch = c->shape[0] != 1;
    }
  }
  if (rope) {
    const int hd = opts->rope_head_dim, nh = opts->rope_heads;
    if (x->rank != 3 || opts->gated) return shape_err(OP, "x", x, "[B, T, K] under a plain weight");
    if (!(hd > 0 && hd % 2 == 0 && (int64_t)nh * hd <= n)) return shape_err(OP, "w", w, "[>= heads*head_dim, K] of even heads");
    seq = x->shape[1];
    const svodb_tensor* tabs[2] = {opts->rope_cos, opts->rope_sin};
    const char* names[2] = {"cos", "sin"};
    for (int i = 0; i < 2; ++i) {
      TRY(realized(OP, names[i], tabs[i]));
      const svodb_tensor* t = tabs[i];
      const bool fits = t->rank == 4 && t->shape[0] == 1 && t->shape[1] == seq && t->shape[2] == 1 &&
                        t->shape[3] == hd / 2 && contiguous(t);
      if (!fits) return shape_err(OP, names[i], t, "[1, T, 1, head_dim/2]");
    }
  }
  if (!rows_dense(x) || !rows_dense(y) || !contiguous(w) ||
      (opts->residual != nullptr && !rows_dense(opts->residual)))
    return fail(SVODB_ERR_GRAPH, "%s: operands must be dense rows (innermost stride 1)", OP);
  TRY(no_alias(OP, y, {x, w, opts->bias, opts->residual, opts->rope_cos, opts->rope_sin}));
  if (qo != nullptr) TRY(no_alias(OP, y, {qo->q_norm, qo->k_norm, qo->rope_cos, qo->rope_sin}));

  GemmArgs a{};
  a.a = x->data;
  a.w = w->data;
  a.bias = opts->bias ? opts->bias->data : nullptr;
  a.residual = opts->residual ? opts->residual->data : nullptr;
  a.c = y->data;
  a.k = (int)k;
  a.n = (int)n;
  a.m = k == 0 ? 0 : numel(x) / (k ? k : 1);
  a.lda = x->rank >= 2 ? x->stride[x->rank - 2] : k;
  a.ldw = k;
  a.ldc = y->rank >= 2 ? y->stride[y->rank - 2] : n;
  a.ldr = opts->residual ? (opts->residual->rank >= 2 ? opts->residual->stride[opts->residual->rank - 2] : n) : 0;
  a.act = opts->act;
  a.gated = opts->gated;
  a.has_scale = opts->has_scale;
  a.scale = opts->scale;
  a.dtype = x->dtype;
  a.status = device_status_word();
  if (a.m == 0 || n == 0) {
    chose_graph(OP, "shape");
    return SVODB_OK;
  }
  // The tables ride the stream dtype or the rotation runs after a plain GEMM,
  // and a turn runs alone after the bias (tk/src/ops/linear.rs:132-164).
  bool rope_in_store = rope && opts->rope_cos->dtype == x->dtype && opts->rope_sin->dtype == x->dtype;
  if (rope && !rope_in_store)
    return dtype_err(OP, "cos", opts->rope_cos->dtype, x->dtype);
  if (rope) {
    a.rope_cos = opts->rope_cos->data;
    a.rope_sin = opts->rope_sin->data;
    a.rope_heads = opts->rope_heads;
    a.rope_head_dim = opts->rope_head_dim;
    a.rope_seq = seq;
  }
  cudaStream_t s = (cudaStream_t)stream;
  char cfg[128];
  // The config store's key of this call and the tile width it holds for it.
  g_config_key[0] = 0;
  {
    const char* epi = qo != nullptr ? "qkv" : rope ? "rope" : opts->gated ? "gated" : "plain";
    char key[160];
    snprintf(key, sizeof key, "gemm|%s|%lld|%lld|%lld|%s%s%s", dtype_name(x->dtype), (long long)a.m, (long long)n,
             (long long)k, epi, opts->residual != nullptr ? "+res" : "", opts->act != SVODB_ACT_NONE ? "+act" : "");
    a.force_bn = config_lookup(key);
    if (gemm_tc_covers(a)) snprintf(g_config_key, sizeof g_config_key, "%s", key);
  }
  if (qo != nullptr) {
    // In the store when the tensor-core kernel covers it (dense y rows of 128-
    // column heads); else a plain projection and the prologue over y in place.
    GemmArgs f = a;
    f.rope_head_dim = qo->head_dim;
    f.rope_heads = qo->heads + qo->kv_heads;
    if (qo->rope_cos != nullptr) {
      f.rope_cos = qo->rope_cos->data;
      f.rope_sin = qo->rope_sin->data;
      f.rope_seq = qkv_per_batch ? a.m : x->shape[1];
    }
    f.norm_q = qo->q_norm ? qo->q_norm->data : nullptr;
    f.norm_k = qo->k_norm ? qo->k_norm->data : nullptr;
    f.norm_q_heads = qo->heads;
    f.norm_k_heads = qo->kv_heads;
    f.norm_eps = (float)qo->eps;
    const bool any = f.rope_cos != nullptr || f.norm_q != nullptr || f.norm_k != nullptr;
    if (any && (f.force_bn == 512 ? gemm_tc2_covers(f) : (f.force_bn == 0 && gemm_tc2_preferred(f)))) {
      int rc = launch_gemm_tc2(f, s, cfg, sizeof cfg);
      if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
      if (rc == 0) {
        chose_kernel(OP, "gemm", cfg);
        return check_launch(OP);
      }
    }
    if (any && gemm_tc_covers(f)) {
      int rc = launch_gemm_tc(f, s, cfg, sizeof cfg);
      if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
      if (rc == 0) {
        chose_kernel(OP, "gemm", cfg);
        return check_launch(OP);
      }
    }
    if (any && !contiguous(y))
      return fail(SVODB_ERR_GRAPH, "%s: the qkv prologue outside the kernel needs a contiguous y", OP);
  }
  if (qo == nullptr && opts->k_splits > 1) {
    // split-K where the caller asked for it and the split kernel covers the call;
    // everything else runs its k loop in one piece
    GemmArgs sk = a;
    sk.k_splits = opts->k_splits;
    sk.workspace = opts->workspace;
    sk.workspace_bytes = opts->workspace_bytes;
    const size_t need = gemm_splitk_workspace_bytes(a.m, a.n, opts->k_splits);
    if (opts->workspace == nullptr || opts->workspace_bytes < need)
      return fail(SVODB_ERR_WORKSPACE, "%s: %d k splits need %zu workspace bytes", OP, opts->k_splits, need);
    if (gemm_tc2_splitk_covers(sk)) {
      int rc = launch_gemm_tc2_splitk(sk, s, cfg, sizeof cfg);
      if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
      if (rc == 0) {
        chose_kernel(OP, "gemm", cfg);
        return check_launch(OP);
      }
    }
  }
  if (a.force_bn == 512 ? gemm_tc2_covers(a) : (a.force_bn == 0 && gemm_tc2_preferred(a))) {
    int rc = launch_gemm_tc2(a, s, cfg, sizeof cfg);
    if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
    if (rc == 0) {
      chose_kernel(OP, "gemm", cfg);
      if (qo != nullptr) heads_in_place(qo, y, qkv_per_batch, s);
      return check_launch(OP);
    }
  }
  if (gemm_tc_covers(a)) {
    int rc = launch_gemm_tc(a, s, cfg, sizeof cfg);
    if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
    if (rc == 0) {
      chose_kernel(OP, "gemm", cfg);
      if (qo != nullptr) heads_in_place(qo, y, qkv_per_batch, s);
      return check_launch(OP);
    }
  }
  const char* why = !is_half(a.dtype) ? "dtype" : (n % 8 != 0 || k % 16 != 0) ? "shape" : "config";
  launch_gemm_generic(a, s);
  if (qo != nullptr) heads_in_place(qo, y, qkv_per_batch, s);
  chose_graph(OP, why);
  return check_launch(OP);
}

// ---------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------
namespace {

int attend(const char* OP, const svodb_tensor* q, const svodb_tensor* k, const svodb_tensor* v, bool packed,
           const svodb_attn_opts* opts, svodb_tensor* o, void* stream) {
  svodb_attn_opts none{};
  if (opts == nullptr) opts = &none;
  if (q->rank != 4) return shape_err(OP, "q", q, "[B, T, H, D]");
  const bool cached = opts->has_cache != 0;
  const bool mapped = cached && opts->cache_row_map != nullptr;
  if (cached && packed) return fail(SVODB_ERR_GRAPH, "%s: a packed projection is not a cache", OP);
  if (!(k->rank == 4 && (k->shape[0] == q->shape[0] || mapped) && k->shape[3] == q->shape[3]))
    return shape_err(OP, "k", k, mapped ? "[rows, Tk, H_kv, D]" : "[B, Tk, H_kv, D]");
  if (!same_shape(v, k)) return shape_err(OP, "v", v, "the shape of k");
  if (!is_float(q->dtype)) return fail(SVODB_ERR_GRAPH, "%s: q is %s, not a float type", OP, dtype_name(q->dtype));
  if (k->dtype != q->dtype) return dtype_err(OP, "k", k->dtype, q->dtype);
  if (v->dtype != q->dtype) return dtype_err(OP, "v", v->dtype, q->dtype);
  const int64_t B = q->shape[0], T = q->shape[1], H = q->shape[2], D = q->shape[3];
  const int64_t Tk = k->shape[1], Hkv = cached ? opts->cache_kv_heads : k->shape[2];
  if (!(Hkv > 0 && H % Hkv == 0))
    return fail(SVODB_ERR_HEADS, "%s: %lld query heads are not a multiple of %lld key/value heads", OP, (long long)H,
                (long long)Hkv);
  // `ops::Cache` (tk/src/ops/attention.rs:148-170)
  int64_t n_app = 0;
  if (cached) {
    if (opts->cache_head_start < 0 || opts->cache_head_start + Hkv > k->shape[2])
      return shape_err(OP, "k", k, "[rows, Tk, >= head_start + kv_heads, D]");
    if (mapped) {
      TRY(realized(OP, "row map", opts->cache_row_map));
      const svodb_tensor* m = opts->cache_row_map;
      if (m->rank != 1 || m->shape[0] != B) return shape_err(OP, "row map", m, "[B]");
      if (m->dtype != SVODB_I32) return dtype_err(OP, "row map", m->dtype, SVODB_I32);
    }
    if ((opts->cache_app_k != nullptr) != (opts->cache_app_v != nullptr))
      return fail(SVODB_ERR_GRAPH, "%s: appended keys and values come together", OP);
    if (opts->cache_app_k != nullptr) {
      const svodb_tensor* ap[2] = {opts->cache_app_k, opts->cache_app_v};
      const char* names[2] = {"appended k", "appended v"};
      for (int i = 0; i < 2; ++i) {
        TRY(realized(OP, names[i], ap[i]));
        const svodb_tensor* t = ap[i];
        const bool fits = t->rank == 4 && t->shape[0] == B && t->shape[1] > 0 && t->shape[1] == ap[0]->shape[1] &&
                          t->shape[2] == Hkv && t->shape[3] == D && contiguous(t);
        if (!fits) return shape_err(OP, names[i], t, "[B, n, kv_heads, D]");
        if (t->dtype != q->dtype) return dtype_err(OP, names[i], t->dtype, q->dtype);
      }
      if (opts->key_lens == nullptr) return fail(SVODB_ERR_SHAPE, "%s: key lens has shape [], expected [B] with appended rows", OP);
      n_app = opts->cache_app_k->shape[1];
    }
    if (opts->cache_app_lens != nullptr) {
      TRY(realized(OP, "appended lens", opts->cache_app_lens));
      const svodb_tensor* t = opts->cache_app_lens;
      if (n_app == 0 || t->rank != 1 || t->shape[0] != B) return shape_err(OP, "appended lens", t, "[B] with appended rows");
      if (t->dtype != SVODB_I32) return dtype_err(OP, "appended lens", t->dtype, SVODB_I32);
    }
  }
  if (opts->key_lens != nullptr && opts->key_mask != nullptr)
    return fail(SVODB_ERR_GRAPH, "%s: key lengths and a key mask are alternatives (KeyMask)", OP);
  if (opts->key_lens != nullptr) {
    TRY(realized(OP, "key lens", opts->key_lens));
    if (opts->key_lens->rank != 1 || opts->key_lens->shape[0] != B) return shape_err(OP, "key lens", opts->key_lens, "[B]");
    if (opts->key_lens->dtype != SVODB_I32) return dtype_err(OP, "key lens", opts->key_lens->dtype, SVODB_I32);
  }
  if (opts->key_mask != nullptr) {
    TRY(realized(OP, "key mask", opts->key_mask));
    const svodb_tensor* m = opts->key_mask;
    if (m->rank != 2 || m->shape[0] != B || m->shape[1] != Tk || !contiguous(m))
      return shape_err(OP, "key mask", m, "[B, Tk]");
    if (m->dtype != SVODB_U8 && m->dtype != SVODB_I32) return dtype_err(OP, "key mask", m->dtype, SVODB_U8);
  }
  if (opts->seg_start != nullptr) {
    TRY(realized(OP, "seg start", opts->seg_start));
    const svodb_tensor* sg = opts->seg_start;
    if (sg->rank != 2 || sg->shape[0] != B || sg->shape[1] != T || !contiguous(sg))
      return shape_err(OP, "seg start", sg, "[B, T]");
    if (sg->dtype != SVODB_I32) return dtype_err(OP, "seg start", sg->dtype, SVODB_I32);
  }
  int bias_per_batch = 0;
  if (opts->bias != nullptr) {
    TRY(realized(OP, "bias", opts->bias));
    const svodb_tensor* bs = opts->bias;
    const bool fits = bs->rank == 4 && (bs->shape[0] == B || bs->shape[0] == 1) && bs->shape[1] == H &&
                      bs->shape[2] == T && bs->shape[3] == Tk + n_app && contiguous(bs);
    if (!fits) return shape_err(OP, "bias", bs, "[B | 1, H, T, Tk (+ appended)]");
    if (bs->dtype != q->dtype) return dtype_err(OP, "bias", bs->dtype, q->dtype);
    bias_per_batch = bs->shape[0] != 1 || B == 1;
  }
  if (!(o->rank == 4 && same_shape(o, q))) return shape_err(OP, "o", o, "[B, T, H, D]");
  if (o->dtype != q->dtype) return dtype_err(OP, "o", o->dtype, q->dtype);
  if (opts->lse != nullptr) {
    TRY(realized(OP, "lse", opts->lse));
    const svodb_tensor* l = opts->lse;
    if (l->rank != 3 || l->shape[0] != B || l->shape[1] != H || l->shape[2] != T || !contiguous(l))
      return shape_err(OP, "lse", l, "[B, H, T]");
    if (l->dtype != SVODB_F32) return dtype_err(OP, "lse", l->dtype, SVODB_F32);
  }
  const svodb_tensor* all[4] = {q, k, v, o};
  for (const svodb_tensor* t : all)
    if (t->stride[3] != 1) return fail(SVODB_ERR_GRAPH, "%s: the head dim must be contiguous", OP);
  if (packed) TRY(no_alias(OP, o, {q}));
  else TRY(no_alias(OP, o, {q, k, v}));
  if (opts->has_chunk && opts->chunk_size <= 0) return fail(SVODB_ERR_GRAPH, "%s: a chunk of size 0", OP);

  AttnArgs a{};
  a.q = q->data, a.k = k->data, a.v = v->data, a.o = o->data;
  a.kv_rows = k->shape[0];
  if (cached) {
    // the first head this attention reads
    a.k = (const char*)k->data + (size_t)opts->cache_head_start * k->stride[2] * esize(k->dtype);
    a.v = (const char*)v->data + (size_t)opts->cache_head_start * v->stride[2] * esize(v->dtype);
    a.row_map = mapped ? (const int32_t*)opts->cache_row_map->data : nullptr;
    if (n_app > 0) {
      a.k_app = opts->cache_app_k->data;
      a.v_app = opts->cache_app_v->data;
      a.n_app = (int)n_app;
      a.app_lens = opts->cache_app_lens ? (const int32_t*)opts->cache_app_lens->data : nullptr;
    }
  }
  a.q_sb = q->stride[0], a.q_st = q->stride[1], a.q_sh = q->stride[2];
  a.k_sb = k->stride[0], a.k_st = k->stride[1], a.k_sh = k->stride[2];
  a.v_sb = v->stride[0], a.v_st = v->stride[1], a.v_sh = v->stride[2];
  a.o_sb = o->stride[0], a.o_st = o->stride[1], a.o_sh = o->stride[2];
  a.batch = B, a.t = T, a.tk = Tk;
  a.heads = (int)H, a.kv_heads = (int)Hkv, a.d = (int)D;
  a.dtype = q->dtype;
  a.scale = opts->has_scale ? opts->scale : 1.0f / sqrtf((float)D);
  a.causal = opts->causal;
  a.key_lens = opts->key_lens ? (const int32_t*)opts->key_lens->data : nullptr;
  a.key_mask = opts->key_mask ? opts->key_mask->data : nullptr;
  a.key_mask_i32 = opts->key_mask ? opts->key_mask->dtype == SVODB_I32 : 0;
  a.has_window = opts->has_window;
  a.win_left = opts->window_left, a.win_right = opts->window_right;
  a.has_chunk = opts->has_chunk;
  a.chunk_size = opts->chunk_size, a.chunk_left = opts->chunk_left, a.chunk_right = opts->chunk_right;
  a.seg_start = opts->seg_start ? (const int32_t*)opts->seg_start->data : nullptr;
  a.bias = opts->bias ? opts->bias->data : nullptr;
  a.bias_per_batch = bias_per_batch;
  a.lse = opts->lse ? (float*)opts->lse->data : nullptr;
  a.splits = opts->splits > 1 ? opts->splits : 1;
  a.status = device_status_word();
  a.packed = packed;
  if (B * T * H == 0 || D == 0) {
    chose_graph(OP, "shape");
    return SVODB_OK;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (Tk + n_app == 0) {
    // No key at all: every row attends to nothing (zeros), as the graph writes it.
    for (int64_t b = 0; b < B; ++b)
      for (int64_t t = 0; t < T; ++t)
        cudaMemsetAsync((char*)o->data + (b * o->stride[0] + t * o->stride[1]) * esize(o->dtype), 0,
                        (size_t)(H * D) * esize(o->dtype), s);
    chose_graph(OP, "shape");
    return check_launch(OP);
  }
  a.splits = capped_splits(Tk + n_app, a.splits);  // capped at the key tile count
  if (a.splits > 1) {
    const size_t need = svodb_attention_workspace_bytes(B, T, H, D, a.splits);
    if (opts->workspace == nullptr || opts->workspace_bytes < need)
      return fail(SVODB_ERR_WORKSPACE, "%s: %d key splits need %zu workspace bytes", OP, a.splits, need);
    if (opts->lse != nullptr) return fail(SVODB_ERR_UNSUPPORTED, "%s: lse is not produced under key splits", OP);
    const int64_t rows = B * T * H;
    a.o_part = (float*)opts->workspace;
    a.m_part = a.o_part + (size_t)a.splits * rows * D;
    a.l_part = a.m_part + (size_t)a.splits * rows;
    if (!(o->stride[2] == D && o->stride[1] == H * D && o->stride[0] == T * H * D))
      return fail(SVODB_ERR_GRAPH, "%s: a split attention writes a contiguous output", OP);
  }
  char cfg[128];
  auto merge_splits = [&]() {
    if (a.splits <= 1) return;
    CombineArgs c{};
    c.o_part = a.o_part, c.m_part = a.m_part, c.l_part = a.l_part;
    c.o = o->data;
    c.rows = B * T * H;
    c.d = (int)D;
    c.splits = a.splits;
    c.dtype = a.dtype;
    launch_combine(c, s);
  };
  const bool exact_only = config_lookup("attention|exact") != 0;
  if (!exact_only && attention_tc_p_covers(a) && config_lookup("attention|one_item") == 0) {
    int rc = launch_attention_tc_p(a, s, cfg, sizeof cfg);
    if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
    if (rc == 0) {
      merge_splits();
      chose_kernel(OP, packed ? "flash_attention_packed" : "flash_attention", cfg);
      return check_launch(OP);
    }
  }
  if (!exact_only && attention_tc_covers(a)) {
    int rc = launch_attention_tc(a, s, cfg, sizeof cfg);
    if (rc < 0) return fail(SVODB_ERR_LAUNCH, "%s: the tensor map or kernel attributes were rejected", OP);
    if (rc == 0) {
      chose_kernel(OP, packed ? "flash_attention_packed" : "flash_attention", cfg);
      return check_launch(OP);
    }
  }
  if (D > 256) return fail(SVODB_ERR_UNSUPPORTED, "%s: head dim %lld is above 256", OP, (long long)D);
  const char* why = !is_half(a.dtype) ? "dtype" : "shape";
  int rc = launch_attention_generic(a, s);
  if (rc != 0) return fail(SVODB_ERR_LAUNCH, "%s: kernel attributes were rejected (%d)", OP, rc);
  merge_splits();
  chose_graph(OP, why);
  return check_launch(OP);
}

}  // namespace

size_t svodb_linear_workspace_bytes(int64_t m, int64_t n, int32_t k_splits) {
  return gemm_splitk_workspace_bytes(m, n, k_splits);
}

size_t svodb_attention_workspace_bytes(int64_t batch, int64_t t, int64_t heads, int64_t d, int32_t splits) {
  if (splits <= 1) return 0;
  const size_t rows = (size_t)batch * (size_t)t * (size_t)heads;
  return sizeof(float) * (size_t)splits * rows * ((size_t)d + 2);
}

int svodb_attention(const svodb_tensor* q, const svodb_tensor* k, const svodb_tensor* v, const svodb_attn_opts* opts,
                    svodb_tensor* o, void* stream) {
  static const char* OP = "attention";
  GUARD(OP);
  TRY(realized(OP, "q", q));
  TRY(realized(OP, "k", k));
  TRY(realized(OP, "v", v));
  TRY(realized(OP, "o", o));
  return attend(OP, q, k, v, false, opts, o, stream);
}

int svodb_attention_packed(const svodb_tensor* qkv, int32_t heads, int32_t kv_heads, const svodb_attn_opts* opts,
                           svodb_tensor* o, void* stream) {
  static const char* OP = "attention";
  GUARD(OP);
  TRY(realized(OP, "qkv", qkv));
  TRY(realized(OP, "o", o));
  if (!(kv_heads > 0 && heads % kv_heads == 0))
    return fail(SVODB_ERR_HEADS, "%s: %d query heads are not a multiple of %d key/value heads", OP, heads, kv_heads);
  const int slots = heads + 2 * kv_heads;
  if (qkv->rank != 3 || qkv->shape[2] <= 0 || qkv->shape[2] % slots != 0 || !contiguous(qkv))
    return shape_err(OP, "qkv", qkv, "[B, T, slots*D]");
  const int64_t d = qkv->shape[2] / slots;
  const int64_t B = qkv->shape[0], T = qkv->shape[1], W = qkv->shape[2];
  auto view = [&](int64_t head0, int64_t nheads) {
    svodb_tensor t{};
    t.data = (char*)qkv->data + (size_t)(head0 * d) * esize(qkv->dtype);
    t.dtype = qkv->dtype;
    t.rank = 4;
    t.shape[0] = B, t.shape[1] = T, t.shape[2] = nheads, t.shape[3] = d;
    t.stride[0] = T * W, t.stride[1] = W, t.stride[2] = d, t.stride[3] = 1;
    return t;
  };
  svodb_tensor q = view(0, heads), k = view(heads, kv_heads), v = view(heads + kv_heads, kv_heads);
  return attend(OP, &q, &k, &v, true, opts, o, stream);
}

int svodb_combine_splits(const svodb_tensor* o_part, const svodb_tensor* m_part, const svodb_tensor* l_part,
                         svodb_tensor* o, void* stream) {
  static const char* OP = "combine_splits";
  GUARD(OP);
  TRY(realized(OP, "o_part", o_part));
  TRY(realized(OP, "m_part", m_part));
  TRY(realized(OP, "l_part", l_part));
  TRY(realized(OP, "o", o));
  if (o_part->rank != 5 || !contiguous(o_part)) return shape_err(OP, "o_part", o_part, "[S, B, T, H, D]");
  if (m_part->rank != 4 || !contiguous(m_part)) return shape_err(OP, "m_part", m_part, "[S, B, T, H]");
  if (!same_shape(l_part, m_part) || !contiguous(l_part)) return shape_err(OP, "l_part", l_part, "[S, B, T, H]");
  for (int i = 0; i < 4; ++i)
    if (m_part->shape[i] != o_part->shape[i]) return shape_err(OP, "m_part", m_part, "[S, B, T, H]");
  if (o->rank != 4 || !contiguous(o)) return shape_err(OP, "o", o, "[B, T, H, D]");
  for (int i = 0; i < 4; ++i)
    if (o->shape[i] != o_part->shape[i + 1]) return shape_err(OP, "o", o, "[B, T, H, D]");
  if (o_part->dtype != SVODB_F32 || m_part->dtype != SVODB_F32 || l_part->dtype != SVODB_F32)
    return dtype_err(OP, "partials", o_part->dtype, SVODB_F32);
  if (!is_float(o->dtype)) return dtype_err(OP, "o", o->dtype, SVODB_BF16);
  CombineArgs c{};
  c.o_part = (const float*)o_part->data;
  c.m_part = (const float*)m_part->data;
  c.l_part = (const float*)l_part->data;
  c.o = o->data;
  c.rows = o->shape[0] * o->shape[1] * o->shape[2];
  c.d = (int)o->shape[3];
  c.splits = (int)o_part->shape[0];
  c.dtype = o->dtype;
  launch_combine(c, (cudaStream_t)stream);
  chose_kernel(OP, "combine_splits", "{br:4}");
  return check_launch(OP);
}

// ---------------------------------------------------------------------------
// heads
// ---------------------------------------------------------------------------
int svodb_heads(const svodb_tensor* qkv, const svodb_qkv_opts* opts, svodb_tensor* q, svodb_tensor* k,
                svodb_tensor* v, void* stream) {
  static const char* OP = "heads";
  GUARD(OP);
  if (opts == nullptr) return fail(SVODB_ERR_GRAPH, "%s: options are required", OP);
  TRY(realized(OP, "qkv", qkv));
  TRY(realized(OP, "q", q));
  TRY(realized(OP, "k", k));
  TRY(realized(OP, "v", v));
  const int H = opts->heads, Hkv = opts->kv_heads, d = opts->head_dim;
  if (!(Hkv > 0 && H % Hkv == 0))
    return fail(SVODB_ERR_HEADS, "%s: %d query heads are not a multiple of %d key/value heads", OP, H, Hkv);
  const int slots = H + 2 * Hkv;
  if (qkv->rank != 3 || qkv->shape[2] != (int64_t)slots * d || !contiguous(qkv))
    return shape_err(OP, "qkv", qkv, "[B, T, slots*head_dim]");
  if (!is_float(qkv->dtype)) return fail(SVODB_ERR_GRAPH, "%s: qkv is not a float type", OP);
  const svodb_tensor* norms[2] = {opts->q_norm, opts->k_norm};
  const char* nnames[2] = {"q norm", "k norm"};
  for (int i = 0; i < 2; ++i) {
    if (norms[i] == nullptr) continue;
    TRY(realized(OP, nnames[i], norms[i]));
    if (norms[i]->rank != 1 || norms[i]->shape[0] != d) return shape_err(OP, nnames[i], norms[i], "[head_dim]");
    if (norms[i]->dtype != qkv->dtype) return dtype_err(OP, nnames[i], norms[i]->dtype, qkv->dtype);
  }
  const int64_t B = qkv->shape[0], T = qkv->shape[1];
  int per_batch = 0;
  if (opts->rope_cos != nullptr) {
    if (d % 2 != 0) return shape_err(OP, "qkv", qkv, "an even head_dim under a rotation");
    TRY(realized(OP, "cos", opts->rope_cos));
    TRY(realized(OP, "sin", opts->rope_sin));
    const svodb_tensor* c = opts->rope_cos;
    const bool fits = c->rank == 4 && (c->shape[0] == 1 || c->shape[0] == B) && c->shape[1] == T &&
                      c->shape[2] == 1 && c->shape[3] == d / 2 && contiguous(c);
    if (!fits) return shape_err(OP, "cos", c, "[1 | B, T, 1, head_dim/2]");
    if (!same_shape(opts->rope_sin, c) || !contiguous(opts->rope_sin)) return shape_err(OP, "sin", opts->rope_sin, "the shape of cos");
    if (c->dtype != qkv->dtype) return dtype_err(OP, "cos", c->dtype, qkv->dtype);
    if (opts->rope_sin->dtype != qkv->dtype) return dtype_err(OP, "sin", opts->rope_sin->dtype, qkv->dtype);
    per_batch = c->shape[0] != 1;
  }
  auto out_ok = [&](const svodb_tensor* t, int heads) {
    return t->rank == 4 && t->shape[0] == B && t->shape[1] == T && t->shape[2] == heads && t->shape[3] == d &&
           contiguous(t) && t->dtype == qkv->dtype;
  };
  if (!out_ok(q, H)) return shape_err(OP, "q", q, "[B, T, heads, head_dim]");
  if (!out_ok(k, Hkv)) return shape_err(OP, "k", k, "[B, T, kv_heads, head_dim]");
  if (!out_ok(v, Hkv)) return shape_err(OP, "v", v, "[B, T, kv_heads, head_dim]");
  TRY(no_alias(OP, q, {qkv, k, v}));
  TRY(no_alias(OP, k, {qkv, v}));
  TRY(no_alias(OP, v, {qkv}));
  HeadsArgs a{};
  a.qkv = qkv->data;
  a.q_w = opts->q_norm ? opts->q_norm->data : nullptr;
  a.k_w = opts->k_norm ? opts->k_norm->data : nullptr;
  a.cos = opts->rope_cos ? opts->rope_cos->data : nullptr;
  a.sin = opts->rope_sin ? opts->rope_sin->data : nullptr;
  a.q = q->data, a.k = k->data, a.v = v->data;
  a.batch = B, a.t = T;
  a.heads = H, a.kv_heads = Hkv, a.d = d;
  a.eps = (float)opts->eps;
  a.per_batch_tables = per_batch;
  a.dtype = qkv->dtype;
  if (launch_heads(a, (cudaStream_t)stream)) chose_kernel(OP, "heads", "{lanes_per_head:d/16}");
  else chose_graph(OP, is_half(a.dtype) ? "shape" : "dtype");
  return check_launch(OP);
}

// ---------------------------------------------------------------------------
// norms
// ---------------------------------------------------------------------------
namespace {
int norm_op(const char* OP, int layer, const svodb_tensor* x, const svodb_tensor* residual, const svodb_tensor* w,
            const svodb_tensor* b, double eps, svodb_tensor* sum, svodb_tensor* out, void* stream) {
  GUARD(OP);
  TRY(realized(OP, "x", x));
  TRY(realized(OP, "w", w));
  TRY(realized(OP, "out", out));
  if (x->rank < 1) return shape_err(OP, "x", x, "[..., D]");
  const int64_t d = x->shape[x->rank - 1];
  if (!is_float(x->dtype)) return fail(SVODB_ERR_GRAPH, "%s: x is not a float type", OP);
  if (w->rank != 1 || w->shape[0] != d) return shape_err(OP, "w", w, "[D]");
  if (w->dtype != x->dtype) return dtype_err(OP, "w", w->dtype, x->dtype);
  if (b != nullptr) {
    TRY(realized(OP, "b", b));
    if (b->rank != 1 || b->shape[0] != d) return shape_err(OP, "b", b, "[D]");
    if (b->dtype != x->dtype) return dtype_err(OP, "b", b->dtype, x->dtype);
  }
  if (residual != nullptr) {
    TRY(realized(OP, "residual", residual));
    TRY(realized(OP, "sum", sum));
    if (!same_shape(residual, x)) return shape_err(OP, "residual", residual, "the shape of x");
    if (residual->dtype != x->dtype) return dtype_err(OP, "residual", residual->dtype, x->dtype);
    if (!same_shape(sum, x) || !contiguous(sum) || sum->dtype != x->dtype) return shape_err(OP, "sum", sum, "the shape of x");
    if (!contiguous(residual)) return fail(SVODB_ERR_GRAPH, "%s: residual must be contiguous", OP);
  }
  if (!same_shape(out, x) || out->dtype != x->dtype) return shape_err(OP, "out", out, "the shape of x");
  if (!contiguous(x) || !contiguous(out)) return fail(SVODB_ERR_GRAPH, "%s: x and out must be contiguous", OP);
  TRY(no_alias(OP, out, {x, residual, w, b, sum}));
  if (sum != nullptr) TRY(no_alias(OP, sum, {x, residual, w, b}));
  NormArgs a{};
  a.x = x->data;
  a.residual = residual ? residual->data : nullptr;
  a.w = w->data;
  a.b = b ? b->data : nullptr;
  a.out = out->data;
  a.sum = sum ? sum->data : nullptr;
  a.d = (int)d;
  a.rows = d == 0 ? 0 : numel(x) / d;
  a.eps = (float)eps;
  a.layer = layer;
  a.dtype = x->dtype;
  if (a.rows == 0) {
    chose_graph(OP, "shape");
    return SVODB_OK;
  }
  if (launch_norm(a, (cudaStream_t)stream)) chose_kernel(OP, OP, "{br:8}");
  else chose_graph(OP, is_half(a.dtype) ? "shape" : "dtype");
  return check_launch(OP);
}
}  // namespace

int svodb_layer_norm(const svodb_tensor* x, const svodb_tensor* w, const svodb_tensor* b, double eps,
                     svodb_tensor* out, void* stream) {
  return norm_op("layer_norm", 1, x, nullptr, w, b, eps, nullptr, out, stream);
}
int svodb_add_layer_norm(const svodb_tensor* x, const svodb_tensor* residual, const svodb_tensor* w,
                         const svodb_tensor* b, double eps, svodb_tensor* sum, svodb_tensor* out, void* stream) {
  if (residual == nullptr) return fail(SVODB_ERR_UNREALIZED, "layer_norm: residual is missing");
  return norm_op("layer_norm", 1, x, residual, w, b, eps, sum, out, stream);
}
int svodb_rms_norm(const svodb_tensor* x, const svodb_tensor* w, double eps, svodb_tensor* out, void* stream) {
  return norm_op("rms_norm", 0, x, nullptr, w, nullptr, eps, nullptr, out, stream);
}
int svodb_add_rms_norm(const svodb_tensor* x, const svodb_tensor* residual, const svodb_tensor* w, double eps,
                       svodb_tensor* sum, svodb_tensor* out, void* stream) {
  if (residual == nullptr) return fail(SVODB_ERR_UNREALIZED, "rms_norm: residual is missing");
  return norm_op("rms_norm", 0, x, residual, w, nullptr, eps, sum, out, stream);
}

// ---------------------------------------------------------------------------
// glue
// ---------------------------------------------------------------------------
namespace {
// A fused norm's operands: weight [D] (required), bias [D] or null, both of the row dtype.
int norm_operands(const char* op, const svodb_tensor* w, const svodb_tensor* b, int64_t d, int dtype) {
  TRY(realized(op, "norm weight", w));
  if (numel(w) != d || !contiguous(w)) return shape_err(op, "norm weight", w, "[D]");
  if (w->dtype != dtype) return dtype_err(op, "norm weight", w->dtype, dtype);
  if (b != nullptr) {
    TRY(realized(op, "norm bias", b));
    if (numel(b) != d || !contiguous(b)) return shape_err(op, "norm bias", b, "[D]");
    if (b->dtype != dtype) return dtype_err(op, "norm bias", b->dtype, dtype);
  }
  return SVODB_OK;
}

int embed_impl(const char* OP, const svodb_tensor* ids, const svodb_tensor* table, const svodb_tensor* pos_table,
               const svodb_tensor* type_row, int64_t pad_id, const svodb_tensor* norm_w, const svodb_tensor* norm_b,
               double eps, int layer, svodb_tensor* out, void* stream) {
  GUARD(OP);
  TRY(realized(OP, "ids", ids));
  TRY(realized(OP, "table", table));
  TRY(realized(OP, "out", out));
  if (ids->rank != 2 || !contiguous(ids)) return shape_err(OP, "ids", ids, "[B, T]");
  if (ids->dtype != SVODB_I32 && ids->dtype != SVODB_I64) return dtype_err(OP, "ids", ids->dtype, SVODB_I32);
  if (table->rank != 2 || !contiguous(table)) return shape_err(OP, "table", table, "[V, D]");
  if (!is_half(table->dtype)) return dtype_err(OP, "table", table->dtype, SVODB_BF16);
  const int64_t d = table->shape[1];
  if (d % 8 != 0) return shape_err(OP, "table", table, "[V, D] with D a multiple of 8");
  if (out->rank != 3 || out->shape[0] != ids->shape[0] || out->shape[1] != ids->shape[1] || out->shape[2] != d ||
      !contiguous(out) || out->dtype != table->dtype)
    return shape_err(OP, "out", out, "[B, T, D]");
  if (pos_table != nullptr) {
    TRY(realized(OP, "pos_table", pos_table));
    if (pos_table->rank != 2 || pos_table->shape[1] != d || !contiguous(pos_table) || pos_table->dtype != table->dtype)
      return shape_err(OP, "pos_table", pos_table, "[P, D]");
  }
  if (type_row != nullptr) {
    TRY(realized(OP, "type_row", type_row));
    if (numel(type_row) < d || type_row->dtype != table->dtype) return shape_err(OP, "type_row", type_row, "[D]");
  }
  EmbedArgs a{};
  a.ids = ids->data;
  a.ids_i64 = ids->dtype == SVODB_I64;
  a.table = table->data;
  a.pos_table = pos_table ? pos_table->data : nullptr;
  a.type_row = type_row ? type_row->data : nullptr;
  a.pad_id = pad_id;
  a.out = out->data;
  a.batch = ids->shape[0], a.t = ids->shape[1];
  a.d = (int)d;
  a.vocab = table->shape[0];
  a.max_pos = pos_table ? pos_table->shape[0] : 1;
  a.dtype = table->dtype;
  if (norm_w == nullptr) {
    launch_embed(a, (cudaStream_t)stream);
    return check_launch(OP);
  }
  TRY(norm_operands(OP, norm_w, norm_b, d, table->dtype));
  EmbedNormArgs n{norm_w->data, norm_b ? norm_b->data : nullptr, (float)eps, layer};
  if (launch_embed_norm(a, n, (cudaStream_t)stream)) {
    chose_kernel(OP, "embed_norm", "{tokens_per_block:8}");
    return check_launch(OP);
  }
  // outside the fused kernel's rows: the lookup, then the norm over it in place
  launch_embed(a, (cudaStream_t)stream);
  NormArgs r{};
  r.x = out->data, r.w = norm_w->data, r.b = n.b, r.out = out->data;
  r.rows = a.batch * a.t, r.d = a.d, r.eps = n.eps, r.layer = layer, r.dtype = a.dtype;
  launch_norm(r, (cudaStream_t)stream);
  chose_graph(OP, "shape");
  return check_launch(OP);
}
}  // namespace

int svodb_embed(const svodb_tensor* ids, const svodb_tensor* table, const svodb_tensor* pos_table,
                const svodb_tensor* type_row, int64_t pad_id, svodb_tensor* out, void* stream) {
  return embed_impl("embed", ids, table, pos_table, type_row, pad_id, nullptr, nullptr, 0.0, 1, out, stream);
}

int svodb_embed_norm(const svodb_tensor* ids, const svodb_tensor* table, const svodb_tensor* pos_table,
                     const svodb_tensor* type_row, int64_t pad_id, const svodb_tensor* norm_w,
                     const svodb_tensor* norm_b, double eps, int32_t layer, svodb_tensor* out, void* stream) {
  if (norm_w == nullptr) return fail(SVODB_ERR_UNREALIZED, "embed_norm: norm weight is missing");
  return embed_impl("embed_norm", ids, table, pos_table, type_row, pad_id, norm_w, norm_b, eps, layer ? 1 : 0, out,
                    stream);
}

namespace {
int pool_impl(const char* OP, const svodb_tensor* hidden, const svodb_tensor* norm_w, const svodb_tensor* norm_b,
              double eps, int layer, svodb_tensor* scratch, const svodb_tensor* mask_or_lengths, int32_t mode,
              int32_t normalize, svodb_tensor* out, void* stream, bool fused, const PeerPush* push = nullptr,
              bool* pushed = nullptr) {
  GUARD(OP);
  TRY(realized(OP, "hidden", hidden));
  TRY(realized(OP, "out", out));
  if (hidden->rank != 3 || !contiguous(hidden) || !is_float(hidden->dtype)) return shape_err(OP, "hidden", hidden, "[B, L, D]");
  const int64_t B = hidden->shape[0], L = hidden->shape[1], D = hidden->shape[2];
  if (mode < 0 || mode > 3) return fail(SVODB_ERR_GRAPH, "%s: mode %d", OP, mode);
  const svodb_tensor* aux = mask_or_lengths;
  int64_t slots = 1;
  if (mode == 3) {
    TRY(realized(OP, "token index", aux));
    if (aux->rank != 2 || aux->shape[0] != B || !contiguous(aux)) return shape_err(OP, "token index", aux, "[B, S]");
    if (aux->dtype != SVODB_I32) return dtype_err(OP, "token index", aux->dtype, SVODB_I32);
    slots = aux->shape[1];
  }
  if (out->rank != 2 || out->shape[0] != B * slots || out->shape[1] != D || out->stride[1] != 1 ||
      out->dtype != SVODB_F32)
    return shape_err(OP, "out", out, "[B (x S), D] f32");
  if (mode == 1) {
    TRY(realized(OP, "mask", aux));
    if (aux->rank != 2 || aux->shape[0] != B || aux->shape[1] != L || !contiguous(aux)) return shape_err(OP, "mask", aux, "[B, L]");
    if (aux->dtype != SVODB_U8 && aux->dtype != SVODB_I32) return dtype_err(OP, "mask", aux->dtype, SVODB_U8);
  } else if (mode == 2) {
    TRY(realized(OP, "lengths", aux));
    if (aux->rank != 1 || aux->shape[0] != B) return shape_err(OP, "lengths", aux, "[B]");
    if (aux->dtype != SVODB_I32) return dtype_err(OP, "lengths", aux->dtype, SVODB_I32);
  }
  if (L == 0) return shape_err(OP, "hidden", hidden, "[B, L >= 1, D]");
  PoolArgs a{};
  a.push = push;
  a.hidden = hidden->data;
  a.aux = aux ? aux->data : nullptr;
  a.aux_i32 = aux ? aux->dtype == SVODB_I32 : 0;
  a.mode = mode;
  a.slots = (int)slots;
  a.normalize = normalize;
  a.out = (float*)out->data;
  a.out_row_stride = out->stride[0];
  a.batch = B, a.l = L;
  a.d = (int)D;
  a.dtype = hidden->dtype;
  if (!fused) {
    launch_pool(a, (cudaStream_t)stream);
    return check_launch(OP);
  }
  if (norm_w != nullptr) TRY(norm_operands(OP, norm_w, norm_b, D, hidden->dtype));
  EmbedNormArgs n{norm_w ? norm_w->data : nullptr, norm_b ? norm_b->data : nullptr, (float)eps, layer};
  if (launch_norm_pool(a, n, (cudaStream_t)stream)) {
    if (pushed != nullptr) *pushed = push != nullptr && push->world > 1;
    chose_kernel(OP, "norm_pool", norm_w ? (push != nullptr && push->world > 1 ? "{norm:fused,push:peers}" : "{norm:fused}")
                                         : (push != nullptr && push->world > 1 ? "{norm:none,push:peers}" : "{norm:none}"));
    return check_launch(OP);
  }
  a.push = nullptr;  // the unfused kernels below do not send
  // outside the fused kernel's rows: the norm into the caller's scratch, then the two pooling kernels
  if (norm_w != nullptr) {
    if (scratch == nullptr || scratch->data == nullptr || !same_shape(scratch, hidden) || !contiguous(scratch) ||
        scratch->dtype != hidden->dtype)
      return fail(SVODB_ERR_WORKSPACE, "%s: rows of %lld elements take the unfused path, which needs a scratch tensor "
                  "of the hidden states' shape", OP, (long long)D);
    NormArgs r{};
    r.x = hidden->data, r.w = norm_w->data, r.b = n.b, r.out = scratch->data;
    r.rows = B * L, r.d = (int)D, r.eps = n.eps, r.layer = layer, r.dtype = hidden->dtype;
    launch_norm(r, (cudaStream_t)stream);
    a.hidden = scratch->data;
  }
  launch_pool(a, (cudaStream_t)stream);
  chose_graph(OP, "shape");
  return check_launch(OP);
}
}  // namespace

int svodb_pool(const svodb_tensor* hidden, const svodb_tensor* mask_or_lengths, int32_t mode, int32_t normalize,
               svodb_tensor* out, void* stream) {
  return pool_impl("pool", hidden, nullptr, nullptr, 0.0, 1, nullptr, mask_or_lengths, mode, normalize, out, stream,
                   false);
}

int svodb_norm_pool(const svodb_tensor* hidden, const svodb_tensor* norm_w, const svodb_tensor* norm_b, double eps,
                    int32_t layer, svodb_tensor* scratch, const svodb_tensor* mask_or_lengths, int32_t mode,
                    int32_t normalize, svodb_tensor* out, void* stream) {
  return pool_impl("norm_pool", hidden, norm_w, norm_b, eps, layer ? 1 : 0, scratch, mask_or_lengths, mode, normalize,
                   out, stream, true);
}

int svodb_norm_pool_gather(const svodb_tensor* hidden, const svodb_tensor* norm_w, const svodb_tensor* norm_b, double eps,
                           int32_t layer, svodb_tensor* scratch, const svodb_tensor* mask_or_lengths, int32_t mode,
                           int32_t normalize, const svodb_peer_gather* pg, svodb_tensor* gathered, void* stream) {
  static const char* OP = "norm_pool_gather";
  if (pg == nullptr || gathered == nullptr || gathered->data == nullptr)
    return fail(SVODB_ERR_SHAPE, "%s: no peer context or gathered buffer", OP);
  if (pg->world < 1 || pg->world > 8 || pg->rank < 0 || pg->rank >= pg->world)
    return fail(SVODB_ERR_SHAPE, "%s: world %d rank %d", OP, pg->world, pg->rank);
  if (gathered->rank != 2 || gathered->dtype != SVODB_F32 || !contiguous(gathered) || gathered->shape[0] % pg->world != 0)
    return shape_err(OP, "gathered", gathered, "[world * rows, D] f32");
  const int64_t rows = gathered->shape[0] / pg->world, D = gathered->shape[1];
  // this rank's slot of the gathered buffer is the pooling's output
  svodb_tensor mine = *gathered;
  mine.data = (float*)gathered->data + (int64_t)pg->rank * rows * D;
  mine.shape[0] = rows;
  PeerPush push{};
  push.world = pg->world, push.rank = pg->rank;
  if (pg->world > 1) {
    for (int i = 0; i < pg->world; ++i) {
      if (pg->stage[i] == nullptr || pg->flags[i] == nullptr)
        return fail(SVODB_ERR_SHAPE, "%s: rank %d's buffers are not mapped", OP, i);
      push.stage[i] = (float*)pg->stage[i];
      push.flags[i] = (uint32_t*)pg->flags[i];
    }
    if (pg->local == nullptr) return fail(SVODB_ERR_SHAPE, "%s: no local counters", OP);
    push.local = (uint32_t*)pg->local;
  }
  bool pushed = false;
  const int rc = pool_impl(OP, hidden, norm_w, norm_b, eps, layer ? 1 : 0, scratch, mask_or_lengths, mode, normalize,
                           &mine, stream, true, &push, &pushed);
  if (rc != SVODB_OK || pg->world == 1) return rc;
  // the rows are on their way (sent by the pooling kernel itself), or still to be sent
  svodb_peer_gather step = *pg;
  step.phases = pushed ? 2 : 0;
  return svodb_peer_all_gather(&step, (const float*)mine.data, (float*)gathered->data, rows, D, stream);
}

int svodb_rope_table(double theta, const svodb_tensor* positions, int32_t head_dim, svodb_tensor* cos,
                     svodb_tensor* sin, void* stream) {
  static const char* OP = "rope_table";
  GUARD(OP);
  TRY(realized(OP, "cos", cos));
  TRY(realized(OP, "sin", sin));
  if (head_dim < 2 || head_dim % 2 != 0) return fail(SVODB_ERR_GRAPH, "%s: head_dim %d is not an even number >= 2", OP, head_dim);
  if (cos->rank != 2 || cos->shape[1] != head_dim / 2 || !contiguous(cos) || !is_float(cos->dtype))
    return shape_err(OP, "cos", cos, "[P, head_dim/2]");
  if (!same_shape(sin, cos) || !contiguous(sin) || sin->dtype != cos->dtype) return shape_err(OP, "sin", sin, "the shape of cos");
  const int32_t* pos = nullptr;
  if (positions != nullptr) {
    TRY(realized(OP, "positions", positions));
    if (numel(positions) != cos->shape[0] || positions->dtype != SVODB_I32 || !contiguous(positions))
      return shape_err(OP, "positions", positions, "[P] i32");
    pos = (const int32_t*)positions->data;
  }
  launch_rope_table(theta, pos, cos->shape[0], head_dim, cos->data, sin->data, cos->dtype, (cudaStream_t)stream);
  return check_launch(OP);
}

// ---------------------------------------------------------------------------
// device seam
// ---------------------------------------------------------------------------
struct svodb_program {
  CUmodule module;
  CUfunction function;
  std::vector<svodb_abi_param> params;
};
struct svodb_graph {
  cudaGraph_t graph;
  cudaGraphExec_t exec;
};

namespace {
struct Driver {
  CUresult (*module_load_data)(CUmodule*, const void*) = nullptr;
  CUresult (*module_get_function)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*module_unload)(CUmodule) = nullptr;
  CUresult (*launch_kernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                            void**, void**) = nullptr;
  CUresult (*func_set_attribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  bool ok = false;
};
const Driver& driver() {
  static Driver d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    cudaFree(nullptr);  // make sure the primary context exists
    auto get = [](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult q;
      return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess;
    };
    d.ok = get("cuModuleLoadData", (void**)&d.module_load_data) &&
           get("cuModuleGetFunction", (void**)&d.module_get_function) &&
           get("cuModuleUnload", (void**)&d.module_unload) && get("cuLaunchKernel", (void**)&d.launch_kernel) &&
           get("cuFuncSetAttribute", (void**)&d.func_set_attribute);
  }
  return d;
}
}  // namespace

int svodb_module_load(const void* image, size_t bytes, const char* entry, const svodb_abi_param* params, int32_t n,
                      svodb_program** out) {
  static const char* OP = "module_load";
  GUARD(OP);
  (void)bytes;
  if (image == nullptr || entry == nullptr || out == nullptr) return fail(SVODB_ERR_UNREALIZED, "%s: null argument", OP);
  const Driver& d = driver();
  if (!d.ok) return fail(SVODB_ERR_LAUNCH, "%s: the CUDA driver entry points are unavailable", OP);
  svodb_program* p = new svodb_program();
  CUresult r = d.module_load_data(&p->module, image);
  if (r != CUDA_SUCCESS) {
    delete p;
    return fail(SVODB_ERR_LAUNCH, "%s: cuModuleLoadData failed (%d)", OP, (int)r);
  }
  r = d.module_get_function(&p->function, p->module, entry);
  if (r != CUDA_SUCCESS) {
    d.module_unload(p->module);
    delete p;
    return fail(SVODB_ERR_LAUNCH, "%s: no entry `%s` (%d)", OP, entry, (int)r);
  }
  for (int i = 0; i < n; ++i) p->params.push_back(params[i]);
  *out = p;
  return SVODB_OK;
}

int svodb_program_launch(svodb_program* p, void* stream, void* const* bufs, int32_t n_bufs, const int32_t* vals,
                         int32_t n_vals, const uint32_t grid[3], const uint32_t block[3], uint32_t dyn_smem) {
  static const char* OP = "program_launch";
  GUARD(OP);
  if (p == nullptr) return fail(SVODB_ERR_UNREALIZED, "%s: null program", OP);
  const Driver& d = driver();
  // The reference packs the kernarg blob as 8-byte pointers then 4-byte scalars
  // in ascending slot order (device/src/cuda/program.rs:264-274); the same
  // parameter order is handed to cuLaunchKernel by address here.
  std::vector<void*> argv;
  std::vector<void*> ptrs(bufs, bufs + n_bufs);
  std::vector<int32_t> ints(vals, vals + n_vals);
  for (int i = 0; i < n_bufs; ++i) argv.push_back(&ptrs[i]);
  for (int i = 0; i < n_vals; ++i) argv.push_back(&ints[i]);
  if (dyn_smem > 48 * 1024) d.func_set_attribute(p->function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)dyn_smem);
  CUresult r = d.launch_kernel(p->function, grid[0], grid[1], grid[2], block[0], block[1], block[2], dyn_smem,
                               (CUstream)stream, argv.data(), nullptr);
  if (r != CUDA_SUCCESS) return fail(SVODB_ERR_LAUNCH, "%s: cuLaunchKernel failed (%d)", OP, (int)r);
  return SVODB_OK;
}

int svodb_program_free(svodb_program* p) {
  if (p == nullptr) return SVODB_OK;
  const Driver& d = driver();
  if (d.ok) d.module_unload(p->module);
  delete p;
  return SVODB_OK;
}

int svodb_graph_begin(void* stream) {
  GUARD("graph_begin");
  cudaError_t e = cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) return fail(SVODB_ERR_LAUNCH, "graph_begin: %s", cudaGetErrorString(e));
  return SVODB_OK;
}
int svodb_graph_end(void* stream, svodb_graph** out) {
  GUARD("graph_end");
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture((cudaStream_t)stream, &g);
  if (e != cudaSuccess || g == nullptr) {
    cudaGetLastError();
    return fail(SVODB_ERR_LAUNCH, "graph_end: %s", cudaGetErrorString(e));
  }
  cudaGraphExec_t x = nullptr;
  e = cudaGraphInstantiate(&x, g, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g);
    return fail(SVODB_ERR_LAUNCH, "graph_end: instantiate: %s", cudaGetErrorString(e));
  }
  *out = new svodb_graph{g, x};
  return SVODB_OK;
}
int svodb_graph_replay(svodb_graph* g, void* stream) {
  GUARD("graph_replay");
  if (g == nullptr) return fail(SVODB_ERR_UNREALIZED, "graph_replay: null graph");
  cudaError_t e = cudaGraphLaunch(g->exec, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    if (sticky(e)) g_poisoned = true;
    return fail(SVODB_ERR_LAUNCH, "graph_replay: %s", cudaGetErrorString(e));
  }
  return SVODB_OK;
}
int svodb_graph_free(svodb_graph* g) {
  if (g == nullptr) return SVODB_OK;
  cudaGraphExecDestroy(g->exec);
  cudaGraphDestroy(g->graph);
  delete g;
  return SVODB_OK;
}

int svodb_alloc(size_t bytes, int32_t kind, void** out) {
  GUARD("alloc");
  if (out == nullptr) return fail(SVODB_ERR_UNREALIZED, "alloc: null out");
  cudaError_t e = kind == 1 ? cudaMallocHost(out, bytes) : cudaMalloc(out, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SVODB_ERR_LAUNCH, "alloc: %s", cudaGetErrorString(e));
  }
  return SVODB_OK;
}
int svodb_free(void* ptr, int32_t kind) {
  if (ptr == nullptr) return SVODB_OK;
  cudaError_t e = kind == 1 ? cudaFreeHost(ptr) : cudaFree(ptr);
  if (e != cudaSuccess) return fail(SVODB_ERR_LAUNCH, "free: %s", cudaGetErrorString(e));
  return SVODB_OK;
}
int svodb_copy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
  GUARD("copy_h2d");
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(SVODB_ERR_LAUNCH, "copy_h2d: %s", cudaGetErrorString(e));
  return SVODB_OK;
}
int svodb_copy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
  GUARD("copy_d2h");
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(SVODB_ERR_LAUNCH, "copy_d2h: %s", cudaGetErrorString(e));
  return SVODB_OK;
}
int svodb_stream_sync(void* stream) {
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) {
    if (sticky(e)) g_poisoned = true;
    return fail(SVODB_ERR_LAUNCH, "stream_sync: %s", cudaGetErrorString(e));
  }
  return SVODB_OK;
}

}  // extern "C"
