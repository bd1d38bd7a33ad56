/*
 * CPU restatement (C11 + OpenMP, f32) of the reference's tile-kernel operators.
 *
 * TEST INFRASTRUCTURE ONLY: tests, the smoke check and the benchmark's CPU legs
 * may load this; the product never does.
 *
 * It restates, in plain loops, what the reference's graph fallbacks compute on its
 * CPU device (f32 arithmetic over 16-bit-rounded tensors, one rounding at each
 * operator's store):
 *   linear      tk/src/ops/linear.rs:306-355, order of the epilogue tk/src/kernels/gemm.rs:605-651
 *   activations tk/src/kernels/mod.rs:304-335 (erf by Abramowitz-Stegun 7.1.26, silu by exp2)
 *   attention   tensor/src/transformer.rs:358-531, masks as tk/src/kernels/attention.rs:381-450,
 *               empty rows -> 0 (:974-980)
 *   heads       tk/src/ops/heads.rs:115-134, tk/src/kernels/heads.rs:73-110
 *   norms       tensor/src/nn/norm.rs:333-358, fused sum tk/src/kernels/rows.rs:76-114
 *   rope table  tensor/src/transformer.rs:130-164
 *   rounding    tk/src/interp.rs:37-71 (nearest even)
 * and the layer wiring of the three callers:
 *   Qwen3       model/src/qwen3/{attention.rs:69-113, feed_forward.rs:38-42, decoder_layer.rs:55-65}
 *   XLM-R       model/src/xlm_roberta/{attention.rs:63-77, feed_forward.rs:40-45, encoder_layer.rs:45-49}
 *   ModernBERT  model/src/modernbert/{attention.rs:52-68, mlp.rs:41-46, encoder_layer.rs:52-60, encoder.rs:33-54}
 *
 * Tensors are f32 arrays that hold values already rounded to the 16-bit type
 * (`dtype`: 0 = bf16, 1 = f16, 2 = f32 keeps every bit). The numpy float64
 * restatement is the pinned checker; this file is validated against it on CPU
 * and exists so that the timed CPU baseline is compiled, threaded f32 code.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { SO_BF16 = 0, SO_F16 = 1, SO_F32 = 2 };
enum { SO_ACT_NONE = 0, SO_ACT_GELU = 1, SO_ACT_SILU = 2, SO_ACT_GELU_TANH = 3 };

static inline float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* nearest-even rounding to bf16, kept as f32 (tk/src/interp.rs:37-50) */
static inline float round_bf16(float x) {
  uint32_t u = f32_bits(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return x; /* inf / nan */
  u += 0x7fffu + ((u >> 16) & 1u);
  return bits_f32(u & 0xffff0000u);
}

/* nearest-even rounding to IEEE half, kept as f32 (tk/src/interp.rs:52-71) */
static inline float round_f16(float x) {
  if (!isfinite(x)) return x;
  float a = fabsf(x);
  if (a >= 65520.0f) return copysignf(INFINITY, x);
  if (a < 6.103515625e-05f) { /* subnormal halves: multiples of 2^-24 */
    float q = rintf(a * 16777216.0f);
    return copysignf(q / 16777216.0f, x);
  }
  uint32_t u = f32_bits(a);
  u += 0xfffu + ((u >> 13) & 1u);
  u &= 0xffffe000u;
  return copysignf(bits_f32(u), x);
}

static inline float round_to(int dtype, float x) {
  return dtype == SO_BF16 ? round_bf16(x) : dtype == SO_F16 ? round_f16(x) : x;
}

int so_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the team size of the loops below, whatever OMP_NUM_THREADS said at start-up. */
void so_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void so_round(float* x, int64_t n, int dtype) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) x[i] = round_to(dtype, x[i]);
}

/* ---- activations (tk/src/kernels/mod.rs:272-335) ---- */
static inline float gelu_as(float x) {
  /* 0.5 (x + |x| erf(|x|/sqrt2)), erf by Abramowitz-Stegun 7.1.26 */
  const float p = 0.3275911f, a1 = 0.254829592f, a2 = -0.284496736f, a3 = 1.421413741f, a4 = -1.453152027f,
              a5 = 1.061405429f;
  float ax = fabsf(x);
  float z = ax * 0.70710678118654752f;
  float t = 1.0f / (1.0f + p * z);
  float poly = ((((a5 * t + a4) * t + a3) * t + a2) * t + a1) * t;
  float e = exp2f(-z * z * 1.4426950408889634f);
  float erf_abs = 1.0f - poly * e;
  return 0.5f * (x + ax * erf_abs);
}
static inline float silu_f(float x) { return x / (1.0f + exp2f(-x * 1.4426950408889634f)); }
static inline float gelu_tanh_f(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
static inline float activate(int act, float x) {
  switch (act) {
    case SO_ACT_GELU: return gelu_as(x);
    case SO_ACT_SILU: return silu_f(x);
    case SO_ACT_GELU_TANH: return gelu_tanh_f(x);
    default: return x;
  }
}

/* ---- linear: scale * act(x w^T + bias) [* (up + bias_up)] + residual, one rounding ---- */
typedef float v8 __attribute__((vector_size(32), aligned(4)));

static inline float hsum8(v8 v) { return ((v[0] + v[4]) + (v[1] + v[5])) + ((v[2] + v[6]) + (v[3] + v[7])); }

/* 4 x 4 block of dot products over k (both operands k-contiguous), two rows at a
 * time: 8 accumulators + 2 + 4 operand vectors fit the 16 vector registers */
static void dot_4x4(const float* a, int64_t lda, const float* w, int64_t ldw, int64_t k, float out[4][4]) {
  for (int i0 = 0; i0 < 4; i0 += 2) {
    v8 acc[2][4];
    for (int i = 0; i < 2; ++i)
      for (int j = 0; j < 4; ++j) acc[i][j] = (v8){0, 0, 0, 0, 0, 0, 0, 0};
    const float* a0 = a + (int64_t)i0 * lda;
    int64_t kk = 0;
    for (; kk + 8 <= k; kk += 8) {
      v8 av[2], wv[4];
      for (int i = 0; i < 2; ++i) memcpy(&av[i], a0 + i * lda + kk, 32);
      for (int j = 0; j < 4; ++j) memcpy(&wv[j], w + j * ldw + kk, 32);
      for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * wv[j];
    }
    for (int i = 0; i < 2; ++i)
      for (int j = 0; j < 4; ++j) {
        float s = hsum8(acc[i][j]);
        for (int64_t r = kk; r < k; ++r) s += a0[i * lda + r] * w[j * ldw + r];
        out[i0 + i][j] = s;
      }
  }
}

static float dot_1(const float* a, const float* w, int64_t k) {
  v8 acc = (v8){0, 0, 0, 0, 0, 0, 0, 0};
  int64_t kk = 0;
  for (; kk + 8 <= k; kk += 8) {
    v8 av, wv;
    memcpy(&av, a + kk, 32);
    memcpy(&wv, w + kk, 32);
    acc += av * wv;
  }
  float s = hsum8(acc);
  for (; kk < k; ++kk) s += a[kk] * w[kk];
  return s;
}

static inline float finish(float acc, float up, int gated, const float* bias, int64_t n_out, int64_t col, int act,
                           int has_scale, float scale, const float* residual, int64_t row, int dtype) {
  float g = acc + (bias ? bias[col] : 0.0f);
  float y = activate(act, g);
  if (gated) y *= up + (bias ? bias[n_out + col] : 0.0f);
  if (has_scale) y *= scale;
  if (residual) y += residual[row * n_out + col];
  return round_to(dtype, y);
}

/* x [m,k], w [n,k] ([2n,k] gated: gate rows then up rows), bias [n] / [2n], residual [m,n], out [m,n] */
void so_linear(const float* x, const float* w, const float* bias, const float* residual, float* out, int64_t m,
               int64_t n, int64_t k, int act, int gated, int has_scale, float scale, int dtype) {
  const int64_t nb = 32; /* weight rows per block: 32 x k floats stay in L2 while the rows stream */
  const int64_t n_blocks = (n + nb - 1) / nb, m_blocks = (m + 63) / 64;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t bn = 0; bn < n_blocks; ++bn)
    for (int64_t bm = 0; bm < m_blocks; ++bm) {
      const int64_t n0 = bn * nb, n1 = n0 + nb < n ? n0 + nb : n;
      const int64_t m0 = bm * 64, m1 = m0 + 64 < m ? m0 + 64 : m;
      for (int64_t i = m0; i < m1; i += 4)
        for (int64_t j = n0; j < n1; j += 4) {
          if (i + 4 <= m1 && j + 4 <= n1) {
            float g[4][4], u[4][4];
            dot_4x4(x + i * k, k, w + j * k, k, k, g);
            if (gated) dot_4x4(x + i * k, k, w + (n + j) * k, k, k, u);
            for (int a = 0; a < 4; ++a)
              for (int b = 0; b < 4; ++b)
                out[(i + a) * n + j + b] = finish(g[a][b], gated ? u[a][b] : 0.0f, gated, bias, n, j + b, act,
                                                  has_scale, scale, residual, i + a, dtype);
          } else {
            for (int64_t a = i; a < i + 4 && a < m1; ++a)
              for (int64_t b = j; b < j + 4 && b < n1; ++b) {
                float g = dot_1(x + a * k, w + b * k, k);
                float u = gated ? dot_1(x + a * k, w + (n + b) * k, k) : 0.0f;
                out[a * n + b] = finish(g, u, gated, bias, n, b, act, has_scale, scale, residual, a, dtype);
              }
          }
        }
    }
}

/* ---- row norms (tensor/src/nn/norm.rs:333-358; fused sum tk/src/kernels/rows.rs:76-114) ---- */
/* kind 0 = layer norm (biased variance), 1 = rms norm. residual != NULL: sum_out = round(x + residual),
 * and the ROUNDED sum is what gets normalised. */
void so_norm_rows(int kind, const float* x, const float* w, const float* b, const float* residual, float* out,
                  float* sum_out, int64_t rows, int64_t d, float eps, int dtype) {
#pragma omp parallel
  {
    float* row = (float*)malloc((size_t)d * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      for (int64_t c = 0; c < d; ++c) {
        float v = x[r * d + c];
        if (residual) {
          v = round_to(dtype, v + residual[r * d + c]);
          if (sum_out) sum_out[r * d + c] = v;
        }
        row[c] = v;
      }
      float mean = 0.0f;
      if (kind == 0) {
        for (int64_t c = 0; c < d; ++c) mean += row[c];
        mean /= (float)d;
      }
      float var = 0.0f;
      for (int64_t c = 0; c < d; ++c) var += (row[c] - mean) * (row[c] - mean);
      const float inv = 1.0f / sqrtf(var / (float)d + eps);
      for (int64_t c = 0; c < d; ++c) {
        float y = (row[c] - mean) * inv * (w ? w[c] : 1.0f) + (b ? b[c] : 0.0f);
        out[r * d + c] = round_to(dtype, y);
      }
    }
    free(row);
  }
}

/* ---- rope table (tensor/src/transformer.rs:130-164): f32 angles, cast last ---- */
void so_rope_table(float theta, const int32_t* positions, int64_t n_pos, int head_dim, float* cos_out,
                   float* sin_out, int dtype) {
  const int half = head_dim / 2;
  for (int64_t p = 0; p < n_pos; ++p)
    for (int i = 0; i < half; ++i) {
      const float inv_freq = powf(theta, -(float)(2 * i) / (float)head_dim);
      const float ang = (float)positions[p] * inv_freq;
      cos_out[p * half + i] = round_to(dtype, cosf(ang));
      sin_out[p * half + i] = round_to(dtype, sinf(ang));
    }
}

/* ---- heads (tk/src/kernels/heads.rs:73-110): split, per-head RMSNorm of q/k, split-half rotation ---- */
/* qkv [b,t,(h+2hkv)*d] -> q [b,t,h,d], k,v [b,t,hkv,d]; tables [t, d/2] (shared over the batch) */
void so_heads(const float* qkv, const float* q_w, const float* k_w, const float* cos_t, const float* sin_t,
              float* q, float* k, float* v, int64_t b, int64_t t, int h, int hkv, int d, float eps, int dtype) {
  const int total = h + 2 * hkv, half = d / 2;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < b; ++bi)
    for (int64_t ti = 0; ti < t; ++ti) {
      const float* src = qkv + (bi * t + ti) * (int64_t)total * d;
      for (int hh = 0; hh < total; ++hh) {
        const float* x = src + (int64_t)hh * d;
        if (hh >= h + hkv) {
          memcpy(v + ((bi * t + ti) * hkv + (hh - h - hkv)) * (int64_t)d, x, (size_t)d * sizeof(float));
          continue;
        }
        const float* wn = hh < h ? q_w : k_w;
        float* dst = hh < h ? q + ((bi * t + ti) * h + hh) * (int64_t)d : k + ((bi * t + ti) * hkv + (hh - h)) * (int64_t)d;
        float inv = 1.0f;
        if (wn) {
          float ss = 0.0f;
          for (int c = 0; c < d; ++c) ss += x[c] * x[c];
          inv = 1.0f / sqrtf(ss / (float)d + eps);
        }
        for (int c = 0; c < half; ++c) {
          float y1 = wn ? x[c] * inv * wn[c] : x[c];
          float y2 = wn ? x[c + half] * inv * wn[c + half] : x[c + half];
          if (cos_t) {
            const float cs = cos_t[ti * half + c], sn = sin_t[ti * half + c];
            const float r1 = y1 * cs - y2 * sn, r2 = y1 * sn + y2 * cs;
            y1 = r1, y2 = r2;
          }
          dst[c] = round_to(dtype, y1);
          dst[c + half] = round_to(dtype, y2);
        }
      }
    }
}

/* e^x for x <= 0 in plain arithmetic the compiler can vectorise: 2^(x log2 e) with the
 * fraction by a degree-6 polynomial (relative error below 3e-7, far inside the 16-bit
 * rounding the weights get); inputs below -87 give 0. */
static inline float exp_neg(float x) {
  float y = x * 1.4426950408889634f;
  if (y < -126.0f) y = -126.0f;
  const float n = __builtin_rintf(y);
  const float f = y - n; /* [-0.5, 0.5] */
  float p = 1.530151e-4f;
  p = p * f + 1.339887e-3f;
  p = p * f + 9.618437e-3f;
  p = p * f + 5.550357e-2f;
  p = p * f + 2.402265e-1f;
  p = p * f + 6.931472e-1f;
  p = p * f + 1.0f;
  const int32_t e = (int32_t)n;
  return x < -87.0f ? 0.0f : bits_f32(f32_bits(p) + ((uint32_t)e << 23));
}

/* ---- attention (tensor/src/transformer.rs:358-531): f32 scores and softmax, weights cast to the
 * tensor dtype before @V (:526-530), hidden keys excluded, a row with no visible key -> 0 ---- */
/* q [b,t,h,d], k,v [b,tk,hkv,d], o [b,t,h,d]; key_lens [b] or NULL; key_mask [b,tk] bytes (nonzero = visible,
 * `KeyMask::Bool`) or NULL; window (left,right) when has_window */
void so_attention(const float* q, const float* k, const float* v, float* o, int64_t b, int64_t t, int64_t tk, int h,
                  int hkv, int d, int causal, const int32_t* key_lens, const uint8_t* key_mask, int has_window,
                  int win_left, int win_right, float scale, int dtype) {
  const int group = h / hkv;
  const int64_t row_blocks = (t + 3) / 4;
  const int64_t ldq = (int64_t)h * d, ldk = (int64_t)hkv * d;
#pragma omp parallel
  {
    /* four query rows at a time: their scores, then their weights, over the union of their key ranges */
    float* s = (float*)malloc((size_t)(4 * tk) * sizeof(float));
#pragma omp for collapse(3) schedule(dynamic, 4)
    for (int64_t bi = 0; bi < b; ++bi)
      for (int hh = 0; hh < h; ++hh)
        for (int64_t ib = 0; ib < row_blocks; ++ib) {
          const int kh = hh / group;
          const int64_t i0 = ib * 4;
          const int nr = (int)(t - i0 < 4 ? t - i0 : 4);
          int64_t lo[4], hi[4], blo = tk, bhi = 0;
          for (int r = 0; r < nr; ++r) {
            const int64_t i = i0 + r;
            lo[r] = 0, hi[r] = tk;
            if (key_lens && key_lens[bi] < hi[r]) hi[r] = key_lens[bi] < 0 ? 0 : key_lens[bi];
            if (causal && i + 1 < hi[r]) hi[r] = i + 1;
            if (has_window) {
              if (i - win_left > lo[r]) lo[r] = i - win_left;
              if (i + win_right + 1 < hi[r]) hi[r] = i + win_right + 1;
            }
            if (hi[r] > lo[r]) {
              if (lo[r] < blo) blo = lo[r];
              if (hi[r] > bhi) bhi = hi[r];
            }
          }
          const float* q0 = q + ((bi * t + i0) * h + hh) * (int64_t)d;
          const float* k0 = k + (bi * tk * hkv + kh) * (int64_t)d;
          const float* v0 = v + (bi * tk * hkv + kh) * (int64_t)d;
          /* scores */
          int64_t j = blo;
          if (nr == 4)
            for (; j + 4 <= bhi; j += 4) {
              float blk[4][4];
              dot_4x4(q0, ldq, k0 + j * ldk, ldk, d, blk);
              for (int r = 0; r < 4; ++r)
                for (int c = 0; c < 4; ++c) s[r * tk + j + c] = blk[r][c] * scale;
            }
          for (; j < bhi; ++j)
            for (int r = 0; r < nr; ++r) s[r * tk + j] = dot_1(q0 + r * ldq, k0 + j * ldk, d) * scale;
          /* weights: softmax over each row's own range, rounded to the tensor type, zero outside it */
          for (int r = 0; r < nr; ++r) {
            float* sr = s + r * tk;
            float mx = -INFINITY, sum = 0.0f;
            if (key_mask)
              for (int64_t jj = lo[r]; jj < hi[r]; ++jj)
                if (!key_mask[bi * tk + jj]) sr[jj] = -INFINITY;
            for (int64_t jj = lo[r]; jj < hi[r]; ++jj) mx = sr[jj] > mx ? sr[jj] : mx;
            const int empty = !(mx > -INFINITY); /* no visible key (also the empty range) */
            for (int64_t jj = lo[r]; jj < hi[r]; ++jj) {
              sr[jj] = empty ? 0.0f : exp_neg(sr[jj] - mx);
              sum += sr[jj];
            }
            const float inv = empty ? 0.0f : 1.0f / sum;
            for (int64_t jj = blo; jj < bhi; ++jj)
              sr[jj] = (jj >= lo[r] && jj < hi[r]) ? round_to(dtype, sr[jj] * inv) : 0.0f;
          }
          /* o = weights . v, 16 output columns of the four rows at a time held in registers */
          for (int c0 = 0; c0 < d; c0 += 16) {
            if (d - c0 >= 16) {
              v8 acc[4][2];
              for (int r = 0; r < 4; ++r) acc[r][0] = acc[r][1] = (v8){0, 0, 0, 0, 0, 0, 0, 0};
              for (int64_t jj = blo; jj < bhi; ++jj) {
                v8 va, vb;
                memcpy(&va, v0 + jj * ldk + c0, 32);
                memcpy(&vb, v0 + jj * ldk + c0 + 8, 32);
                for (int r = 0; r < nr; ++r) {
                  const float pw = s[r * tk + jj];
                  acc[r][0] += pw * va;
                  acc[r][1] += pw * vb;
                }
              }
              for (int r = 0; r < nr; ++r) {
                float* orow = o + ((bi * t + i0 + r) * h + hh) * (int64_t)d + c0;
                for (int c = 0; c < 8; ++c) orow[c] = round_to(dtype, acc[r][0][c]);
                for (int c = 0; c < 8; ++c) orow[8 + c] = round_to(dtype, acc[r][1][c]);
              }
            } else {
              for (int r = 0; r < nr; ++r)
                for (int c = 0; c < d - c0; ++c) {
                  float a = 0.0f;
                  for (int64_t jj = blo; jj < bhi; ++jj) a += s[r * tk + jj] * v0[jj * ldk + c0 + c];
                  o[((bi * t + i0 + r) * h + hh) * (int64_t)d + c0 + c] = round_to(dtype, a);
                }
            }
          }
        }
    free(s);
  }
}

/* ---- Qwen3 layers (model/src/qwen3/decoder_layer.rs:55-65): h [b,t,dm] in place ---- */
/* weights per layer, in this order: in_w [dm], qkv_w [(h+2hkv)d, dm], qn_w [d], kn_w [d], o_w [dm, h d],
 * post_w [dm], gu_w [2f, dm], down_w [dm, f]. Returns 0, or -1 when scratch cannot be allocated. */
int so_qwen3_layers(float* hid, const float* const* weights, int n_layers, int64_t b, int64_t t, int dm, int h,
                    int hkv, int d, int f, float theta, float eps, int dtype) {
  const int64_t rows = b * t, total = (int64_t)(h + 2 * hkv) * d;
  float* xn = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* qkv = (float*)malloc((size_t)(rows * total) * sizeof(float));
  float* q = (float*)malloc((size_t)(rows * h * d) * sizeof(float));
  float* k = (float*)malloc((size_t)(rows * hkv * d) * sizeof(float));
  float* v = (float*)malloc((size_t)(rows * hkv * d) * sizeof(float));
  float* a = (float*)malloc((size_t)(rows * h * d) * sizeof(float));
  float* g = (float*)malloc((size_t)(rows * f) * sizeof(float));
  float* h2 = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* cs = (float*)malloc((size_t)(t * d / 2) * sizeof(float));
  float* sn = (float*)malloc((size_t)(t * d / 2) * sizeof(float));
  int32_t* pos = (int32_t*)malloc((size_t)t * sizeof(int32_t));
  int rc = -1;
  if (xn && qkv && q && k && v && a && g && h2 && cs && sn && pos) {
    for (int64_t i = 0; i < t; ++i) pos[i] = (int32_t)i;
    so_rope_table(theta, pos, t, d, cs, sn, dtype);
    const float scale = 1.0f / sqrtf((float)d);
    for (int l = 0; l < n_layers; ++l) {
      const float* const* w = weights + (int64_t)l * 8;
      so_norm_rows(1, hid, w[0], NULL, NULL, xn, NULL, rows, dm, eps, dtype);
      so_linear(xn, w[1], NULL, NULL, qkv, rows, total, dm, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_heads(qkv, w[2], w[3], cs, sn, q, k, v, b, t, h, hkv, d, eps, dtype);
      so_attention(q, k, v, a, b, t, t, h, hkv, d, 1, NULL, NULL, 0, 0, 0, scale, dtype);
      so_linear(a, w[4], NULL, hid, h2, rows, dm, (int64_t)h * d, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_norm_rows(1, h2, w[5], NULL, NULL, xn, NULL, rows, dm, eps, dtype);
      so_linear(xn, w[6], NULL, NULL, g, rows, f, dm, SO_ACT_SILU, 1, 0, 1.0f, dtype);
      so_linear(g, w[7], NULL, h2, hid, rows, dm, f, SO_ACT_NONE, 0, 0, 1.0f, dtype);
    }
    rc = 0;
  }
  free(xn), free(qkv), free(q), free(k), free(v), free(a), free(g), free(h2), free(cs), free(sn), free(pos);
  return rc;
}

/* ---- RoPE in the projection's store (tk/src/kernels/gemm.rs:670-718): x.w^T + bias, then the first
 * heads*hd output columns turned by split halves, row r at position r % t, then the one rounding ---- */
void so_linear_rope(const float* x, const float* w, const float* bias, float* out, int64_t m, int64_t n, int64_t k,
                    int64_t t, const float* cos_t, const float* sin_t, int heads, int hd, int dtype) {
  so_linear(x, w, bias, NULL, out, m, n, k, SO_ACT_NONE, 0, 0, 1.0f, SO_F32);
  const int half = hd / 2;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    float* y = out + r * n;
    const int64_t pos = r % t;
    for (int hh = 0; hh < heads; ++hh)
      for (int c = 0; c < half; ++c) {
        const float cs = cos_t[pos * half + c], sn = sin_t[pos * half + c];
        const float y1 = y[hh * hd + c], y2 = y[hh * hd + c + half];
        y[hh * hd + c] = y1 * cs - y2 * sn;
        y[hh * hd + c + half] = y1 * sn + y2 * cs;
      }
    for (int64_t c = 0; c < n; ++c) y[c] = round_to(dtype, y[c]);
  }
}

/* ---- XLM-R layers (model/src/xlm_roberta/encoder_layer.rs:45-49): post-LN, h [b,t,dm] in place ---- */
/* weights per layer, in this order (16): q_w [dm,dm], q_b, k_w, k_b, v_w, v_b, o_w, o_b, ln1_w, ln1_b,
 * fi_w [f,dm], fi_b, fo_w [dm,f], fo_b, ln2_w, ln2_b. key_mask [b,t] bytes (nonzero = visible). */
int so_xlmr_layers(float* hid, const float* const* weights, int n_layers, int64_t b, int64_t t, int dm, int h, int f,
                   const uint8_t* key_mask, float eps, int dtype) {
  const int64_t rows = b * t;
  const int d = dm / h;
  float* q = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* k = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* v = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* a = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* x = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* y = (float*)malloc((size_t)(rows * f) * sizeof(float));
  int rc = -1;
  if (q && k && v && a && x && y) {
    const float scale = 1.0f / sqrtf((float)d);
    for (int l = 0; l < n_layers; ++l) {
      const float* const* w = weights + (int64_t)l * 16;
      so_linear(hid, w[0], w[1], NULL, q, rows, dm, dm, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_linear(hid, w[2], w[3], NULL, k, rows, dm, dm, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_linear(hid, w[4], w[5], NULL, v, rows, dm, dm, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_attention(q, k, v, a, b, t, t, h, h, d, 0, NULL, key_mask, 0, 0, 0, scale, dtype);
      so_linear(a, w[6], w[7], hid, x, rows, dm, dm, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_norm_rows(0, x, w[8], w[9], NULL, hid, NULL, rows, dm, eps, dtype);
      so_linear(hid, w[10], w[11], NULL, y, rows, f, dm, SO_ACT_GELU, 0, 0, 1.0f, dtype);
      so_linear(y, w[12], w[13], hid, x, rows, dm, f, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_norm_rows(0, x, w[14], w[15], NULL, hid, NULL, rows, dm, eps, dtype);
    }
    rc = 0;
  }
  free(q), free(k), free(v), free(a), free(x), free(y);
  return rc;
}

/* ---- ModernBERT layers (model/src/modernbert/encoder_layer.rs:52-60): pre-LN without bias, h in place ---- */
/* weights per layer, in this order (6): attn_ln_w [dm] or NULL (layer 0 has none), qkv_w [3dm,dm], o_w [dm,dm],
 * mlp_ln_w [dm], wi_w [2f,dm] (gate rows first), wo_w [dm,f]. Layer `first_layer + l` is global (no window,
 * global_theta) when its index is a multiple of `global_every`, else local (window, local_theta)
 * (model/src/modernbert/encoder.rs:33-54, config.rs:78-92). */
int so_modernbert_layers(float* hid, const float* const* weights, int n_layers, int first_layer, int64_t b, int64_t t,
                         int dm, int h, int f, const uint8_t* key_mask, int global_every, float global_theta,
                         float local_theta, int win_left, int win_right, float eps, int dtype) {
  const int64_t rows = b * t;
  const int d = dm / h, half = d / 2;
  float* xn = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* qkv = (float*)malloc((size_t)(rows * 3 * dm) * sizeof(float));
  float* q = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* k = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* v = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* a = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* h2 = (float*)malloc((size_t)(rows * dm) * sizeof(float));
  float* g = (float*)malloc((size_t)(rows * f) * sizeof(float));
  float* tab = (float*)malloc((size_t)(4 * t * half) * sizeof(float)); /* cos, sin global; cos, sin local */
  int32_t* pos = (int32_t*)malloc((size_t)t * sizeof(int32_t));
  int rc = -1;
  if (xn && qkv && q && k && v && a && h2 && g && tab && pos) {
    for (int64_t i = 0; i < t; ++i) pos[i] = (int32_t)i;
    so_rope_table(global_theta, pos, t, d, tab, tab + t * half, dtype);
    so_rope_table(local_theta, pos, t, d, tab + 2 * t * half, tab + 3 * t * half, dtype);
    const float scale = 1.0f / sqrtf((float)d);
    for (int l = 0; l < n_layers; ++l) {
      const float* const* w = weights + (int64_t)l * 6;
      const int is_global = (first_layer + l) % global_every == 0;
      const float* cs = is_global ? tab : tab + 2 * t * half;
      const float* sn = cs + t * half;
      const float* src = hid;
      if (w[0]) {
        so_norm_rows(0, hid, w[0], NULL, NULL, xn, NULL, rows, dm, eps, dtype);
        src = xn;
      }
      so_linear_rope(src, w[1], NULL, qkv, rows, 3 * (int64_t)dm, dm, t, cs, sn, 2 * h, d, dtype);
      /* the packed projection read in place = three column windows (tk/src/ops/attention.rs:107-122) */
#pragma omp parallel for schedule(static)
      for (int64_t r = 0; r < rows; ++r) {
        memcpy(q + r * dm, qkv + r * 3 * dm, (size_t)dm * sizeof(float));
        memcpy(k + r * dm, qkv + r * 3 * dm + dm, (size_t)dm * sizeof(float));
        memcpy(v + r * dm, qkv + r * 3 * dm + 2 * dm, (size_t)dm * sizeof(float));
      }
      so_attention(q, k, v, a, b, t, t, h, h, d, 0, NULL, key_mask, !is_global, win_left, win_right, scale, dtype);
      so_linear(a, w[2], NULL, hid, h2, rows, dm, dm, SO_ACT_NONE, 0, 0, 1.0f, dtype);
      so_norm_rows(0, h2, w[3], NULL, NULL, xn, NULL, rows, dm, eps, dtype);
      so_linear(xn, w[4], NULL, NULL, g, rows, f, dm, SO_ACT_GELU, 1, 0, 1.0f, dtype);
      so_linear(g, w[5], NULL, h2, hid, rows, dm, f, SO_ACT_NONE, 0, 0, 1.0f, dtype);
    }
    rc = 0;
  }
  free(xn), free(qkv), free(q), free(k), free(v), free(a), free(h2), free(g), free(tab), free(pos);
  return rc;
}
