// Exact CUDA-core attention: the path ops take where the reference would build
// its graph (f32 operands, head dims the tensor-core kernel does not tile,
// additive bias, key splits). Any float dtype, D <= 256, every mask of
// `ops::Attn`, f32 arithmetic throughout.
//
// Semantics follow tk/src/kernels/attention.rs:381-450 and the f64 mirror in
// tk/src/test/unit/attention.rs:102-178: scores scaled, bias added, masks to
// -inf, base-2 online softmax, a row with no visible key yields zeros
// (kernels/attention.rs:971-980). Split runs write the unnormalised f32
// accumulator with `(m, l)` in log2 units (kernels/attention.rs:910-920) for
// `combine_splits`.
#include <math.h>

#include "common.cuh"
#include "kernels.h"
#include "svodb.h"

namespace svodb {

namespace {

constexpr int BQ = 32;   // queries per block
constexpr int BKV = 32;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ bool key_hidden(const AttnArgs& a, int64_t b, int64_t i, int64_t j, int64_t len) {
  if (j >= len) return true;
  if (a.causal && j > i) return true;
  if (a.has_window && (j + a.win_left < i || j > i + a.win_right)) return true;
  if (a.has_chunk) {
    const int64_t cj = j / a.chunk_size, ci = i / a.chunk_size;
    if (cj > ci + a.chunk_right) return true;
    if (a.chunk_left >= 0 && cj + a.chunk_left < ci) return true;
  }
  if (a.key_mask != nullptr) {
    const int64_t at = b * a.tk + j;
    const int m = a.key_mask_i32 ? ((const int32_t*)a.key_mask)[at] : (int)((const uint8_t*)a.key_mask)[at];
    if (m == 0) return true;
  }
  if (a.seg_start != nullptr && j < (int64_t)a.seg_start[b * a.t + i]) return true;
  return false;
}

// grid: (ceil(T/BQ) * splits, H, B); 256 threads.
template <typename T>
__global__ void __launch_bounds__(256) attention_generic_kernel(const AttnArgs a) {
  extern __shared__ float smem[];
  const int D = a.d;
  const int DP = D + 1;
  float* Qs = smem;               // [BQ][DP]
  float* Ks = Qs + BQ * DP;       // [BKV][DP]
  float* Vs = Ks + BKV * DP;      // [BKV][D]
  float* Ss = Vs + BKV * D;       // [BQ][BKV+1]
  float* corr_s = Ss + BQ * (BKV + 1);  // [BQ]
  float* m_s = corr_s + BQ;             // [BQ]
  float* l_s = m_s + BQ;                // [BQ]

  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int splits = a.splits;
  const int64_t qt = blockIdx.x / splits;
  const int split = blockIdx.x % splits;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int hk = h / (a.heads / a.kv_heads);
  const int64_t i0 = qt * BQ;
  const T* q = (const T*)a.q + b * a.q_sb + h * a.q_sh;
  // `ops::Cache`: lane b reads cache row row_map[b]; keys tk .. tk+n_app-1 are
  // the appended rows, hidden only past app_lens[b].
  int64_t kv_row = a.row_map != nullptr ? (int64_t)a.row_map[b] : b;
  // A map entry outside the cache: nothing is read through it; the lane sees no
  // key at all (zeros) and the status word reports it.
  const bool bad_row = kv_row < 0 || kv_row >= a.kv_rows;
  if (bad_row) {
    kv_row = 0;
    if (tid == 0 && a.status != nullptr) atomicExch(a.status, (uint32_t)kStatusBadIndex);
  }
  const T* k = (const T*)a.k + kv_row * a.k_sb + hk * a.k_sh;
  const T* v = (const T*)a.v + kv_row * a.v_sb + hk * a.v_sh;
  const int64_t keys = a.tk + a.n_app;
  const T* k_app = a.n_app > 0 ? (const T*)a.k_app + (b * a.n_app * a.kv_heads + hk) * (int64_t)a.d : nullptr;
  const T* v_app = a.n_app > 0 ? (const T*)a.v_app + (b * a.n_app * a.kv_heads + hk) * (int64_t)a.d : nullptr;
  const int64_t app_seen = bad_row ? 0 : (a.app_lens != nullptr ? (int64_t)a.app_lens[b] : a.n_app);
  const float sc = a.scale * kLog2e;
  int64_t len = a.tk;
  if (a.key_lens != nullptr) {
    int64_t kl = a.key_lens[b];
    len = kl < 0 ? 0 : (kl < len ? kl : len);
  }
  if (bad_row) len = 0;

  for (int e = tid; e < BQ * D; e += 256) {
    const int r = e / D, c = e % D;
    const int64_t i = i0 + r;
    Qs[r * DP + c] = i < a.t ? Elem<T>::to_f(q[i * a.q_st + c]) : 0.f;
  }
  if (tid < BQ) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  // Output ownership: row = tid/8, columns (tid%8) + 8*c.
  const int orow = tid >> 3, ocol0 = tid & 7;
  float oacc[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) oacc[c] = 0.f;

  // This split's share of the key tiles.
  const int64_t tiles = (keys + BKV - 1) / BKV;
  const int64_t per = (tiles + splits - 1) / splits;
  const int64_t tile_lo = split * per;
  const int64_t tile_hi = tile_lo + per < tiles ? tile_lo + per : tiles;

  for (int64_t kt = tile_lo; kt < tile_hi; ++kt) {
    const int64_t j0 = kt * BKV;
    __syncthreads();
    for (int e = tid; e < BKV * D; e += 256) {
      const int r = e / D, c = e % D;
      const int64_t j = j0 + r;
      float kf = 0.f, vf = 0.f;
      if (j < a.tk) {
        kf = Elem<T>::to_f(k[j * a.k_st + c]);
        vf = Elem<T>::to_f(v[j * a.v_st + c]);
      } else if (j < keys) {
        const int64_t at = (j - a.tk) * a.kv_heads * D + c;
        kf = Elem<T>::to_f(k_app[at]);
        vf = Elem<T>::to_f(v_app[at]);
      }
      Ks[r * DP + c] = kf;
      Vs[r * D + c] = vf;
    }
    __syncthreads();
    // Scores: thread -> row tid/8, keys (tid%8) + 8*jj.
    {
      const int r = tid >> 3;
      const int64_t i = i0 + r;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int c = (tid & 7) + 8 * jj;
        const int64_t j = j0 + c;
        float s = -INFINITY;
        const bool visible = j < a.tk ? !key_hidden(a, b, i, j, len) : (j < keys && j - a.tk < app_seen);
        if (i < a.t && visible) {
          float dot = 0.f;
          for (int dd = 0; dd < D; ++dd) dot = fmaf(Qs[r * DP + dd], Ks[c * DP + dd], dot);
          s = dot * sc;
          if (a.bias != nullptr) {
            const int64_t bb = a.bias_per_batch ? b : 0;
            s = fmaf(Elem<T>::to_f(((const T*)a.bias)[((bb * a.heads + h) * a.t + i) * keys + j]), kLog2e, s);
          }
        }
        Ss[r * (BKV + 1) + c] = s;
      }
    }
    __syncthreads();
    // Row statistics: warp w owns rows 4w .. 4w+3, lane = key.
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int r = wid * 4 + rr;
      const float s = Ss[r * (BKV + 1) + lane];
      const float m_old = m_s[r];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float p = (s == -INFINITY) ? 0.f : exp2f(s - m_new);
      const float corr = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m_new);
      const float psum = warp_sum(p);
      Ss[r * (BKV + 1) + lane] = p;
      if (lane == 0) {
        corr_s[r] = corr;
        m_s[r] = m_new;
        l_s[r] = l_s[r] * corr + psum;
      }
    }
    __syncthreads();
    {
      const float corr = corr_s[orow];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int col = ocol0 + 8 * c;
        if (col < D) {
          float acc = oacc[c] * corr;
          for (int j = 0; j < BKV; ++j) acc = fmaf(Ss[orow * (BKV + 1) + j], Vs[j * D + col], acc);
          oacc[c] = acc;
        }
      }
    }
  }
  __syncthreads();
  const int64_t i = i0 + orow;
  if (i >= a.t) return;
  const float m = m_s[orow], l = l_s[orow];
  if (splits == 1) {
    const float inv = l == 0.f ? 0.f : 1.0f / l;
    T* o = (T*)a.o + b * a.o_sb + i * a.o_st + h * a.o_sh;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const int col = ocol0 + 8 * c;
      if (col < D) o[col] = Elem<T>::from_f(oacc[c] * inv);
    }
    if (a.lse != nullptr && ocol0 == 0)
      a.lse[(b * a.heads + h) * a.t + i] = l == 0.f ? -INFINITY : kLn2 * (m + log2f(l));
  } else {
    const int64_t row = ((int64_t)split * a.batch + b) * a.t * a.heads + i * a.heads + h;
    float* op = a.o_part + row * D;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const int col = ocol0 + 8 * c;
      if (col < D) op[col] = oacc[c];
    }
    if (ocol0 == 0) {
      // An empty share keeps a finite sentinel maximum, as the reference's
      // m0 = -1e30 (kernels/attention.rs:616), so the merge never sees inf - inf.
      a.m_part[row] = m == -INFINITY ? -1e30f : m;
      a.l_part[row] = l;
    }
  }
}

// One warp per output row of D elements.
template <typename T>
__global__ void __launch_bounds__(128) combine_kernel(const CombineArgs a) {
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int lane = threadIdx.x & 31;
  float m = -INFINITY;
  for (int s = 0; s < a.splits; ++s) m = fmaxf(m, a.m_part[(int64_t)s * a.rows + row]);
  float l = 0.f;
  for (int s = 0; s < a.splits; ++s) {
    const int64_t r = (int64_t)s * a.rows + row;
    l = fmaf(a.l_part[r], exp2f(a.m_part[r] - m), l);
  }
  const float inv = l == 0.f ? 1.f : 1.0f / l;
  T* o = (T*)a.o + row * a.d;
  for (int c = lane; c < a.d; c += 32) {
    float acc = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      const int64_t r = (int64_t)s * a.rows + row;
      acc = fmaf(a.o_part[r * a.d + c], exp2f(a.m_part[r] - m), acc);
    }
    o[c] = Elem<T>::from_f(acc * inv);
  }
}

template <typename T>
int run(const AttnArgs& a, cudaStream_t s) {
  const size_t smem =
      sizeof(float) * (size_t)(BQ * (a.d + 1) + BKV * (a.d + 1) + BKV * a.d + BQ * (BKV + 1) + 3 * BQ);
  cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((unsigned)(((a.t + BQ - 1) / BQ) * a.splits), (unsigned)a.heads, (unsigned)a.batch);
  attention_generic_kernel<T><<<grid, 256, smem, s>>>(a);
  return 0;
}

}  // namespace

int launch_attention_generic(const AttnArgs& a, cudaStream_t s) {
  if (a.batch * a.t * a.heads == 0) return 0;
  if (a.dtype == SVODB_BF16) return run<__nv_bfloat16>(a, s);
  if (a.dtype == SVODB_F16) return run<__half>(a, s);
  return run<float>(a, s);
}

void launch_combine(const CombineArgs& a, cudaStream_t s) {
  if (a.rows == 0) return;
  const unsigned blocks = (unsigned)((a.rows + 3) / 4);
  if (a.dtype == SVODB_BF16) combine_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(a);
  else if (a.dtype == SVODB_F16) combine_kernel<__half><<<blocks, 128, 0, s>>>(a);
  else combine_kernel<float><<<blocks, 128, 0, s>>>(a);
}

}  // namespace svodb
