// Small kernels around the op layer that the encoder callers need: token
// embedding lookup (with XLM-R position ids), pooling + L2 normalisation, and
// RoPE tables. All HBM-bound or negligible; written for coalesced access.
#include "common.cuh"
#include "kernels.h"
#include "rows_parts.cuh"
#include "svodb.h"

namespace svodb {

namespace {

// out[b,t,:] = table[ids[b,t]] (+ pos_table[pos_id] + type_row), each add
// rounded to the element type as the graph's 16-bit adds are
// (model/src/xlm_roberta/embeddings.rs:53-63). Position ids:
// `cumsum(ids != pad) * (ids != pad) + pad` (position_ids.rs:27-32).
// One block per (batch row, group of kTok tokens).
constexpr int kTok = 8;

template <typename T, typename I>
__global__ void __launch_bounds__(256)
    embed_kernel(const I* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ pos_table,
                 const T* __restrict__ type_row, int64_t pad_id, T* __restrict__ out, int64_t t_len, int d,
                 int64_t vocab, int64_t max_pos, int vec16) {
  __shared__ int red[8];
  __shared__ int64_t tok_id[kTok];
  __shared__ int64_t tok_pos[kTok];
  const int64_t b = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kTok;
  const I* row = ids + b * t_len;
  const int tid = threadIdx.x;
  int before = 0;
  if (pos_table != nullptr && pad_id >= 0) {
    int cnt = 0;
    for (int64_t i = tid; i < t0; i += 256) cnt += (int64_t)row[i] != pad_id;
    cnt = (int)warp_sum((float)cnt);  // counts stay below 2^24: exact in f32
    if ((tid & 31) == 0) red[tid >> 5] = cnt;
    __syncthreads();
    for (int i = 0; i < 8; ++i) before += red[i];
  }
  if (tid == 0) {
    int run = before;
    for (int j = 0; j < kTok; ++j) {
      const int64_t t = t0 + j;
      if (t >= t_len) break;
      int64_t id = (int64_t)row[t];
      const bool real = id != pad_id;
      run += real ? 1 : 0;
      tok_pos[j] = pad_id >= 0 ? (real ? run : 0) + pad_id : t;
      tok_id[j] = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    }
  }
  __syncthreads();
  const int vec = d / 8;
  for (int j = 0; j < kTok; ++j) {
    const int64_t t = t0 + j;
    if (t >= t_len) break;
    const T* src = table + tok_id[j] * d;
    int64_t p = tok_pos[j];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    const T* psrc = pos_table != nullptr ? pos_table + p * d : nullptr;
    T* dst = out + (b * t_len + t) * d;
    if (!vec16) {
      // an operand off the 16-byte boundary: element by element, same roundings
      for (int c = tid; c < d; c += 256) {
        float v = Elem<T>::to_f(src[c]);
        if (psrc != nullptr) v = Elem<T>::to_f(Elem<T>::from_f(v + Elem<T>::to_f(psrc[c])));
        if (type_row != nullptr) v = Elem<T>::to_f(Elem<T>::from_f(v + Elem<T>::to_f(type_row[c])));
        dst[c] = Elem<T>::from_f(v);
      }
      continue;
    }
    for (int c = tid; c < vec; c += 256) {
      uint4 u = ldg128(src + c * 8);
      if (psrc != nullptr || type_row != nullptr) {
        uint32_t uu[4] = {u.x, u.y, u.z, u.w};
        if (psrc != nullptr) {
          uint4 pu = ldg128(psrc + c * 8);
          const uint32_t pp[4] = {pu.x, pu.y, pu.z, pu.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 a = Elem<T>::unpack(uu[i]), q = Elem<T>::unpack(pp[i]);
            uu[i] = Elem<T>::pack(a.x + q.x, a.y + q.y);
          }
        }
        if (type_row != nullptr) {
          uint4 tu = ldg128(type_row + c * 8);
          const uint32_t tt[4] = {tu.x, tu.y, tu.z, tu.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 a = Elem<T>::unpack(uu[i]), q = Elem<T>::unpack(tt[i]);
            uu[i] = Elem<T>::pack(a.x + q.x, a.y + q.y);
          }
        }
        u = make_uint4(uu[0], uu[1], uu[2], uu[3]);
      }
      stg128(dst + c * 8, u);
    }
  }
}

// The same lookup with the embedding LayerNorm applied before the store
// (model/src/xlm_roberta/embeddings.rs:53-63: word + position + type, then LN):
// one kernel instead of a gather pass and a norm pass over [B, T, D]. A block
// takes kTok tokens of one row; its warps each gather one token's row into
// registers (every add rounded to the element type, as above), normalise the
// rounded sum and store it. d = SPANS * 256.
template <typename T, typename I, int SPANS>
__global__ void __launch_bounds__(kTok * 32)
    embed_norm_kernel(const I* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ pos_table,
                      const T* __restrict__ type_row, int64_t pad_id, const T* __restrict__ w,
                      const T* __restrict__ b, float eps, int layer, T* __restrict__ out, int64_t t_len,
                      int64_t vocab, int64_t max_pos) {
  constexpr int D = SPANS * 256;
  __shared__ int red[kTok];
  __shared__ int64_t tok_id[kTok];
  __shared__ int64_t tok_pos[kTok];
  const int64_t bi = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kTok;
  const I* row = ids + bi * t_len;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int before = 0;
  if (pos_table != nullptr && pad_id >= 0) {
    int cnt = 0;
    for (int64_t i = tid; i < t0; i += kTok * 32) cnt += (int64_t)row[i] != pad_id;
    cnt = (int)warp_sum((float)cnt);  // counts stay below 2^24: exact in f32
    if (lane == 0) red[warp] = cnt;
    __syncthreads();
    for (int i = 0; i < kTok; ++i) before += red[i];
  }
  if (tid == 0) {
    int run = before;
    for (int j = 0; j < kTok; ++j) {
      const int64_t t = t0 + j;
      if (t >= t_len) break;
      int64_t id = (int64_t)row[t];
      const bool real = id != pad_id;
      run += real ? 1 : 0;
      tok_pos[j] = pad_id >= 0 ? (real ? run : 0) + pad_id : t;
      tok_id[j] = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    }
  }
  __syncthreads();
  const int64_t t = t0 + warp;
  if (t >= t_len) return;
  const T* src = table + tok_id[warp] * D;
  int64_t pp = tok_pos[warp];
  pp = pp < 0 ? 0 : (pp >= max_pos ? max_pos - 1 : pp);
  const T* psrc = pos_table != nullptr ? pos_table + pp * D : nullptr;
  float v[SPANS][8];
#pragma unroll
  for (int s = 0; s < SPANS; ++s) {
    const int off = s * 256 + lane * 8;
    rows_parts::unpack8<T>(ldg128(src + off), v[s]);
    if (psrc != nullptr) {
      float q[8];
      rows_parts::unpack8<T>(ldg128(psrc + off), q);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[s][i] += q[i];
      rows_parts::unpack8<T>(rows_parts::pack8<T>(v[s]), v[s]);
    }
    if (type_row != nullptr) {
      float q[8];
      rows_parts::unpack8<T>(ldg128(type_row + off), q);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[s][i] += q[i];
      rows_parts::unpack8<T>(rows_parts::pack8<T>(v[s]), v[s]);
    }
  }
  const float inv = rows_parts::centre_and_scale<SPANS>(v, eps, layer);
  T* dst = out + (bi * t_len + t) * D;
#pragma unroll
  for (int s = 0; s < SPANS; ++s) {
    const int off = s * 256 + lane * 8;
    float y[8];
    rows_parts::affine8<T>(v[s], inv, ldg128(w + off), b != nullptr ? ldg128(b + off) : make_uint4(0, 0, 0, 0),
                           b != nullptr, y);
    stg128(dst + off, rows_parts::pack8<T>(y));
  }
}

// Final norm + pooling + L2 in one kernel (model/src/encoder_head.rs:280-286 after
// the stack's last norm): one block per output row. CLS, last-token and gather
// modes normalise the ONE token they pool (the other rows of the hidden states
// never need their final norm); the masked mean walks the row's real tokens,
// normalising each, and sums them in f32. The normalised values are rounded to
// the element type before they are pooled, as the unfused sequence stores them.
// w == nullptr: the hidden states are pooled as they are. d = SPANS * 256.
template <typename T, int SPANS>
__global__ void __launch_bounds__(256)
    norm_pool_kernel(const T* __restrict__ hidden, const T* __restrict__ w, const T* __restrict__ b, float eps,
                     int layer, const void* __restrict__ aux, int aux_i32, int mode, int slots, int normalize,
                     float* __restrict__ out, int64_t out_row_stride, int64_t l_len, const PeerPush pp) {
  constexpr int D = SPANS * 256;
  __shared__ float part[8192];  // [warps][D], warps * D <= 8192
  __shared__ float cnts[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int64_t bi = mode == 3 ? blockIdx.x / slots : blockIdx.x;
  const T* h = hidden + bi * l_len * D;
  float acc[SPANS][8];
#pragma unroll
  for (int s = 0; s < SPANS; ++s)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[s][i] = 0.f;
  float cnt = 0.f;
  int64_t first = 0, last = 1;  // the token range this block walks
  if (mode == 1) {
    last = l_len;
  } else if (mode == 2) {
    first = (int64_t)((const int32_t*)aux)[bi] - 1;
  } else if (mode == 3) {
    first = (int64_t)((const int32_t*)aux)[blockIdx.x];
  }
  if (mode != 1) {
    first = first < 0 ? 0 : (first > l_len - 1 ? l_len - 1 : first);
    last = first + 1;
  }
  for (int64_t t = first + warp; t < last; t += warps) {
    if (mode == 1) {
      const int m = aux_i32 ? ((const int32_t*)aux)[bi * l_len + t] : (int)((const uint8_t*)aux)[bi * l_len + t];
      if (m == 0) continue;
      cnt += 1.f;
    }
    float v[SPANS][8];
#pragma unroll
    for (int s = 0; s < SPANS; ++s) rows_parts::unpack8<T>(ldg128(h + t * D + s * 256 + lane * 8), v[s]);
    if (w != nullptr) {
      const float inv = rows_parts::centre_and_scale<SPANS>(v, eps, layer);
#pragma unroll
      for (int s = 0; s < SPANS; ++s) {
        const int off = s * 256 + lane * 8;
        float y[8];
        rows_parts::affine8<T>(v[s], inv, ldg128(w + off), b != nullptr ? ldg128(b + off) : make_uint4(0, 0, 0, 0),
                               b != nullptr, y);
        rows_parts::unpack8<T>(rows_parts::pack8<T>(y), v[s]);  // the 16-bit value the norm would store
      }
    }
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[s][i] += v[s][i];
  }
  if (warps > 1) {
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) part[warp * D + s * 256 + lane * 8 + i] = acc[s][i];
    if (lane == 0) cnts[warp] = cnt;
    __syncthreads();
    if (warp != 0) return;
    cnt = 0.f;
    for (int k = 0; k < warps; ++k) cnt += cnts[k];
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = 0.f;
        for (int k = 0; k < warps; ++k) t += part[k * D + s * 256 + lane * 8 + i];  // fixed order: reproducible
        acc[s][i] = t;
      }
  }
  if (mode == 1) {
    const float invc = 1.0f / fmaxf(cnt, 1e-9f);
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[s][i] *= invc;
  }
  if (normalize) {
    float sq = 0.f;
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = fmaf(acc[s][i], acc[s][i], sq);
    const float inv = 1.0f / (sqrtf(warp_sum(sq)) + 1.17549435e-38f);
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[s][i] *= inv;
  }
  float* dst = out + (int64_t)blockIdx.x * out_row_stride;
#pragma unroll
  for (int s = 0; s < SPANS; ++s) {
    float4* d4 = reinterpret_cast<float4*>(dst + s * 256 + lane * 8);
    d4[0] = make_float4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]);
    d4[1] = make_float4(acc[s][4], acc[s][5], acc[s][6], acc[s][7]);
  }
  // Several GPUs: the row also goes straight into every peer's staging buffer (plain
  // stores over NVLink) — the send half of the all-gather, in the kernel that made the row.
  if (pp.world > 1) {
    const uint32_t step = *reinterpret_cast<volatile uint32_t*>(pp.local);
    const size_t slot = (((size_t)(step & 1u) * pp.world + pp.rank) * gridDim.x + blockIdx.x) * D;
    for (int p = 0; p < pp.world; ++p) {
      if (p == pp.rank) continue;
      float* pd = pp.stage[p] + slot;
#pragma unroll
      for (int s = 0; s < SPANS; ++s) {
        float4* d4 = reinterpret_cast<float4*>(pd + s * 256 + lane * 8);
        d4[0] = make_float4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]);
        d4[1] = make_float4(acc[s][4], acc[s][5], acc[s][6], acc[s][7]);
      }
    }
    __threadfence_system();
    __syncwarp();
    if (lane == 0 && atomicAdd(&pp.local[1], 1u) == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < pp.world; ++p)
        if (p != pp.rank) *reinterpret_cast<volatile uint32_t*>(pp.flags[p] + pp.rank) = step + 1u;
      pp.local[1] = 0u;
    }
  }
}

// Pooling, pass 1: out[b, c] = pooled value in f32 (un-normalised).
// grid (ceil(D/128), B), 256 threads: thread = (token lane 0..1, column 0..127).
template <typename T>
__global__ void __launch_bounds__(256)
    pool_kernel(const T* __restrict__ hidden, const void* __restrict__ aux, int aux_i32, int mode,
                float* __restrict__ out, int64_t out_row_stride, int64_t l_len, int d, int slots) {
  __shared__ float part[2][128];
  // mode 3 gathers `slots` tokens per row: output row y = (b, slot)
  const int64_t b = mode == 3 ? blockIdx.y / slots : blockIdx.y;
  const int col = blockIdx.x * 128 + (threadIdx.x & 127);
  const int tl = threadIdx.x >> 7;
  const T* h = hidden + b * l_len * d;
  float acc = 0.f, cnt = 0.f;
  if (mode == 1) {
    for (int64_t t = tl; t < l_len; t += 2) {
      const int m = aux_i32 ? ((const int32_t*)aux)[b * l_len + t] : (int)((const uint8_t*)aux)[b * l_len + t];
      if (m != 0) {
        cnt += 1.f;
        if (col < d) acc += Elem<T>::to_f(h[t * d + col]);
      }
    }
  } else if (tl == 0 && col < d) {
    int64_t t = 0;
    if (mode == 2) {
      t = (int64_t)((const int32_t*)aux)[b] - 1;
      t = t < 0 ? 0 : (t > l_len - 1 ? l_len - 1 : t);
    } else if (mode == 3) {
      t = (int64_t)((const int32_t*)aux)[blockIdx.y];
      t = t < 0 ? 0 : (t > l_len - 1 ? l_len - 1 : t);
    }
    acc = Elem<T>::to_f(h[t * d + col]);
  }
  __shared__ float cnts[2];
  part[tl][threadIdx.x & 127] = acc;
  if ((threadIdx.x & 127) == 0) cnts[tl] = cnt;
  __syncthreads();
  if (tl == 0 && col < d) {
    float v = part[0][threadIdx.x] + part[1][threadIdx.x];
    if (mode == 1) v = v / fmaxf(cnts[0] + cnts[1], 1e-9f);
    out[(int64_t)blockIdx.y * out_row_stride + col] = v;
  }
}

// Pass 2: x / (||x||_2 + f32::MIN_POSITIVE) in place, one block per row.
__global__ void __launch_bounds__(256) l2_kernel(float* __restrict__ out, int64_t out_row_stride, int d) {
  __shared__ float red[8];
  float* row = out + (int64_t)blockIdx.x * out_row_stride;
  float sq = 0.f;
  for (int i = threadIdx.x; i < d; i += 256) sq = fmaf(row[i], row[i], sq);
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = 1.0f / (sqrtf(tot) + 1.17549435e-38f);
  for (int i = threadIdx.x; i < d; i += 256) row[i] *= inv;
}

// cos/sin of position * theta^(-2i/D), angles and functions in f32, cast last
// (tensor/src/transformer.rs:130-164).
template <typename T>
__global__ void rope_table_kernel(float theta, const int32_t* __restrict__ positions, int64_t n_pos, int half,
                                  float expo_step, T* __restrict__ cos, T* __restrict__ sin) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pos * half) return;
  const int64_t p = idx / half;
  const int i = (int)(idx % half);
  const float pos = positions != nullptr ? (float)positions[p] : (float)p;
  const float inv_freq = powf(theta, (float)i * expo_step);
  const float ang = pos * inv_freq;
  cos[idx] = Elem<T>::from_f(cosf(ang));
  sin[idx] = Elem<T>::from_f(sinf(ang));
}

}  // namespace

void launch_embed(const EmbedArgs& a, cudaStream_t s) {
  if (a.batch * a.t == 0) return;
  dim3 grid((unsigned)((a.t + kTok - 1) / kTok), (unsigned)a.batch);
  const int vec16 = aligned16(a.table) && aligned16(a.pos_table) && aligned16(a.type_row) && aligned16(a.out) ? 1 : 0;
#define SVODB_EMBED(T, I)                                                                                         \
  embed_kernel<T, I><<<grid, 256, 0, s>>>((const I*)a.ids, (const T*)a.table, (const T*)a.pos_table,              \
                                          (const T*)a.type_row, a.pad_id, (T*)a.out, a.t, a.d, a.vocab, a.max_pos, \
                                          vec16)
  if (a.dtype == SVODB_BF16) {
    if (a.ids_i64) SVODB_EMBED(__nv_bfloat16, int64_t);
    else SVODB_EMBED(__nv_bfloat16, int32_t);
  } else {
    if (a.ids_i64) SVODB_EMBED(__half, int64_t);
    else SVODB_EMBED(__half, int32_t);
  }
#undef SVODB_EMBED
}

namespace {
template <typename T, typename I>
bool embed_norm_dispatch(const EmbedArgs& a, const EmbedNormArgs& n, cudaStream_t s) {
  dim3 grid((unsigned)((a.t + kTok - 1) / kTok), (unsigned)a.batch);
#define SVODB_EN(SP)                                                                                                \
  case SP:                                                                                                          \
    embed_norm_kernel<T, I, SP><<<grid, kTok * 32, 0, s>>>((const I*)a.ids, (const T*)a.table, (const T*)a.pos_table, \
                                                           (const T*)a.type_row, a.pad_id, (const T*)n.w,             \
                                                           (const T*)n.b, n.eps, n.layer, (T*)a.out, a.t, a.vocab,   \
                                                           a.max_pos);                                               \
    return true
  switch (a.d / 256) {
    SVODB_EN(1); SVODB_EN(2); SVODB_EN(3); SVODB_EN(4); SVODB_EN(5); SVODB_EN(6); SVODB_EN(7); SVODB_EN(8);
    default: return false;
  }
#undef SVODB_EN
}

template <typename T>
bool norm_pool_dispatch(const PoolArgs& a, const EmbedNormArgs& n, cudaStream_t s) {
  const int64_t out_rows = a.mode == 3 ? a.batch * a.slots : a.batch;
  // the masked mean walks a whole row with as many warps as the partial sums leave room for
  const int spans = a.d / 256;
  int warps = 1;
  if (a.mode == 1) warps = spans <= 4 ? 8 : (spans <= 8 ? 4 : 1);
  const PeerPush pp = a.push != nullptr ? *a.push : PeerPush{};
#define SVODB_NP(SP)                                                                                               \
  case SP:                                                                                                         \
    norm_pool_kernel<T, SP><<<(unsigned)out_rows, warps * 32, 0, s>>>((const T*)a.hidden, (const T*)n.w,           \
                                                                      (const T*)n.b, n.eps, n.layer, a.aux,         \
                                                                      a.aux_i32, a.mode, a.slots, a.normalize,      \
                                                                      a.out, a.out_row_stride, a.l, pp);            \
    return true
  switch (spans) {
    SVODB_NP(1); SVODB_NP(2); SVODB_NP(3); SVODB_NP(4); SVODB_NP(5); SVODB_NP(6); SVODB_NP(7); SVODB_NP(8);
    default: return false;
  }
#undef SVODB_NP
}
}  // namespace

int launch_embed_norm(const EmbedArgs& a, const EmbedNormArgs& n, cudaStream_t s) {
  if (a.batch * a.t == 0) return 1;
  const bool fits = a.d % 256 == 0 && a.d >= 256 && a.d <= 2048 && aligned16(a.table) && aligned16(a.pos_table) &&
                    aligned16(a.type_row) && aligned16(a.out) && aligned16(n.w) && aligned16(n.b);
  if (!fits) return 0;
  if (a.dtype == SVODB_BF16)
    return (a.ids_i64 ? embed_norm_dispatch<__nv_bfloat16, int64_t>(a, n, s)
                      : embed_norm_dispatch<__nv_bfloat16, int32_t>(a, n, s)) ? 1 : 0;
  if (a.dtype == SVODB_F16)
    return (a.ids_i64 ? embed_norm_dispatch<__half, int64_t>(a, n, s) : embed_norm_dispatch<__half, int32_t>(a, n, s)) ? 1 : 0;
  return 0;
}

int launch_norm_pool(const PoolArgs& a, const EmbedNormArgs& n, cudaStream_t s) {
  if (a.batch == 0) return 1;
  const bool fits = a.d % 256 == 0 && a.d >= 256 && a.d <= 2048 && aligned16(a.hidden) && aligned16(n.w) &&
                    aligned16(n.b) && aligned16(a.out) && a.out_row_stride % 4 == 0;
  if (!fits) return 0;
  if (a.dtype == SVODB_BF16) return norm_pool_dispatch<__nv_bfloat16>(a, n, s) ? 1 : 0;
  if (a.dtype == SVODB_F16) return norm_pool_dispatch<__half>(a, n, s) ? 1 : 0;
  return 0;
}

void launch_pool(const PoolArgs& a, cudaStream_t s) {
  if (a.batch == 0) return;
  const int64_t out_rows = a.mode == 3 ? a.batch * a.slots : a.batch;
  dim3 grid((unsigned)((a.d + 127) / 128), (unsigned)out_rows);
  if (a.dtype == SVODB_BF16)
    pool_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)a.hidden, a.aux, a.aux_i32, a.mode, a.out,
                                                    a.out_row_stride, a.l, a.d, a.slots);
  else if (a.dtype == SVODB_F16)
    pool_kernel<__half><<<grid, 256, 0, s>>>((const __half*)a.hidden, a.aux, a.aux_i32, a.mode, a.out,
                                             a.out_row_stride, a.l, a.d, a.slots);
  else
    pool_kernel<float><<<grid, 256, 0, s>>>((const float*)a.hidden, a.aux, a.aux_i32, a.mode, a.out,
                                            a.out_row_stride, a.l, a.d, a.slots);
  if (a.normalize) l2_kernel<<<(unsigned)out_rows, 256, 0, s>>>(a.out, a.out_row_stride, a.d);
}

void launch_rope_table(double theta, const int32_t* positions, int64_t n_pos, int head_dim, void* cos, void* sin,
                       int dtype, cudaStream_t s) {
  const int half = head_dim / 2;
  const int64_t n = n_pos * half;
  if (n == 0) return;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  const float step = (float)(-2.0 / head_dim);
  if (dtype == SVODB_BF16)
    rope_table_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((float)theta, positions, n_pos, half, step,
                                                            (__nv_bfloat16*)cos, (__nv_bfloat16*)sin);
  else if (dtype == SVODB_F16)
    rope_table_kernel<__half><<<blocks, 256, 0, s>>>((float)theta, positions, n_pos, half, step, (__half*)cos,
                                                     (__half*)sin);
  else
    rope_table_kernel<float><<<blocks, 256, 0, s>>>((float)theta, positions, n_pos, half, step, (float*)cos,
                                                    (float*)sin);
}

}  // namespace svodb
