// Attention prologue: a fused `[q | k | v]` projection `[B,T,(H+2Hkv)*D]` split
// into sequence-major heads, q and k RMS-normalised over D and rotated.
//
// Semantics follow tk/src/kernels/heads.rs:36-125: per head row
// `inv = rsqrt(mean(x^2) + eps)`, `y = x*inv*w` (q, k only, weight in f32), then
// the half-split rotation `y1' = y1*c - y2*s`, `y2' = y1*s + y2*c` with tables of
// `[1|B, T, D/2]`; v is a pure copy; one rounding at the store.
//
// HBM-bound: every element is read once and written once with 128-bit accesses.
// A head row is owned by D/16 adjacent lanes: each lane holds 8 elements of the
// head's first half and the 8 partner elements of its second half.
#include "common.cuh"
#include "kernels.h"
#include "svodb.h"

namespace svodb {

namespace {

template <typename T>
__device__ __forceinline__ void unpack8(uint4 u, float (&f)[8]) {
  const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 p = Elem<T>::unpack(uu[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(Elem<T>::pack(f[0], f[1]), Elem<T>::pack(f[2], f[3]), Elem<T>::pack(f[4], f[5]),
                    Elem<T>::pack(f[6], f[7]));
}

// LPH = lanes per head row = D/16.
template <typename T, int LPH>
__global__ void __launch_bounds__(256)
    heads_kernel(const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
                 const T* __restrict__ cos, const T* __restrict__ sin, T* __restrict__ q, T* __restrict__ k,
                 T* __restrict__ v, int64_t tokens, int64_t t_len, int heads, int kv_heads, float eps,
                 int per_batch_tables, int in_place) {
  constexpr int D = LPH * 16;
  constexpr int HALF = D / 2;
  const int slots = heads + 2 * kv_heads;
  const int64_t total = tokens * slots;
  const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t head_row = gthread / LPH;
  const int sub = (int)(gthread % LPH);
  const bool live = head_row < total;
  const int64_t hr = live ? head_row : total - 1;
  const int64_t token = hr / slots;
  const int slot = (int)(hr % slots);
  const T* src = qkv + hr * D;
  float x1[8], x2[8];
  unpack8<T>(ldg128(src + sub * 8), x1);
  unpack8<T>(ldg128(src + HALF + sub * 8), x2);

  const int which = slot < heads ? 0 : (slot < heads + kv_heads ? 1 : 2);
  const T* w = which == 0 ? q_w : (which == 1 ? k_w : nullptr);
  // The sum of squares is reduced over the LPH lanes of the head row; every lane
  // of the warp takes part in the shuffles.
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) sq = fmaf(x1[i], x1[i], fmaf(x2[i], x2[i], sq));
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if (w != nullptr) {
    const float inv = rsqrtf(sq * (1.0f / D) + eps);
    float w1[8], w2[8];
    unpack8<T>(ldg128(w + sub * 8), w1);
    unpack8<T>(ldg128(w + HALF + sub * 8), w2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x1[i] = x1[i] * inv * w1[i];
      x2[i] = x2[i] * inv * w2[i];
    }
  }
  if (cos != nullptr && which < 2) {
    const int64_t trow = per_batch_tables ? token : token % t_len;
    float c[8], s[8];
    unpack8<T>(ldg128(cos + trow * HALF + sub * 8), c);
    unpack8<T>(ldg128(sin + trow * HALF + sub * 8), s);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = x1[i], b = x2[i];
      x1[i] = a * c[i] - b * s[i];
      x2[i] = a * s[i] + b * c[i];
    }
  }
  if (!live) return;
  T* dst;
  // In place: the head goes back where it came from (every element is read by
  // the one thread that rewrites it, before it does).
  if (in_place) dst = const_cast<T*>(src);
  else if (which == 0) dst = q + (token * heads + slot) * D;
  else if (which == 1) dst = k + (token * kv_heads + (slot - heads)) * D;
  else dst = v + (token * kv_heads + (slot - heads - kv_heads)) * D;
  stg128(dst + sub * 8, pack8<T>(x1));
  stg128(dst + HALF + sub * 8, pack8<T>(x2));
}

// Any even D and any float type: one thread per rotation pair, one warp-sized
// loop per head row.
template <typename T>
__global__ void __launch_bounds__(128)
    heads_generic_kernel(const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
                         const T* __restrict__ cos, const T* __restrict__ sin, T* __restrict__ q, T* __restrict__ k,
                         T* __restrict__ v, int64_t tokens, int64_t t_len, int heads, int kv_heads, int d, float eps,
                         int per_batch_tables, int in_place) {
  const int slots = heads + 2 * kv_heads;
  const int64_t head_row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (head_row >= tokens * slots) return;
  const int lane = threadIdx.x & 31;
  const int64_t token = head_row / slots;
  const int slot = (int)(head_row % slots);
  const int half = d / 2;
  const T* src = qkv + head_row * d;
  const int which = slot < heads ? 0 : (slot < heads + kv_heads ? 1 : 2);
  const T* w = which == 0 ? q_w : (which == 1 ? k_w : nullptr);
  float inv = 1.f;
  if (w != nullptr) {
    float sq = 0.f;
    for (int i = lane; i < d; i += 32) {
      float f = Elem<T>::to_f(src[i]);
      sq = fmaf(f, f, sq);
    }
    inv = rsqrtf(warp_sum(sq) / d + eps);
  }
  T* dst;
  if (in_place) dst = const_cast<T*>(src);
  else if (which == 0) dst = q + (token * heads + slot) * d;
  else if (which == 1) dst = k + (token * kv_heads + (slot - heads)) * d;
  else dst = v + (token * kv_heads + (slot - heads - kv_heads)) * d;
  const int64_t trow = per_batch_tables ? token : token % t_len;
  for (int i = lane; i < half; i += 32) {
    float a = Elem<T>::to_f(src[i]), b = Elem<T>::to_f(src[i + half]);
    if (w != nullptr) {
      a = a * inv * Elem<T>::to_f(w[i]);
      b = b * inv * Elem<T>::to_f(w[i + half]);
    }
    if (cos != nullptr && which < 2) {
      const float c = Elem<T>::to_f(cos[trow * half + i]), s = Elem<T>::to_f(sin[trow * half + i]);
      const float a2 = a * c - b * s, b2 = a * s + b * c;
      a = a2, b = b2;
    }
    dst[i] = Elem<T>::from_f(a);
    dst[i + half] = Elem<T>::from_f(b);
  }
}

template <typename T, int LPH>
void run(const HeadsArgs& a, cudaStream_t s) {
  const int64_t tokens = a.batch * a.t;
  const int64_t threads = tokens * (a.heads + 2 * a.kv_heads) * LPH;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  heads_kernel<T, LPH><<<blocks, 256, 0, s>>>((const T*)a.qkv, (const T*)a.q_w, (const T*)a.k_w, (const T*)a.cos,
                                              (const T*)a.sin, (T*)a.q, (T*)a.k, (T*)a.v, tokens, a.t, a.heads,
                                              a.kv_heads, a.eps, a.per_batch_tables, a.in_place);
}

template <typename T>
bool dispatch(const HeadsArgs& a, cudaStream_t s) {
  switch (a.d) {
    case 16: run<T, 1>(a, s); return true;
    case 32: run<T, 2>(a, s); return true;
    case 64: run<T, 4>(a, s); return true;
    case 128: run<T, 8>(a, s); return true;
    case 256: run<T, 16>(a, s); return true;
    default: return false;
  }
}

template <typename T>
void run_generic(const HeadsArgs& a, cudaStream_t s) {
  const int64_t tokens = a.batch * a.t;
  const int64_t head_rows = tokens * (a.heads + 2 * a.kv_heads);
  heads_generic_kernel<T><<<(unsigned)((head_rows + 3) / 4), 128, 0, s>>>(
      (const T*)a.qkv, (const T*)a.q_w, (const T*)a.k_w, (const T*)a.cos, (const T*)a.sin, (T*)a.q, (T*)a.k, (T*)a.v,
      tokens, a.t, a.heads, a.kv_heads, a.d, a.eps, a.per_batch_tables, a.in_place);
}

}  // namespace

int launch_heads(const HeadsArgs& a, cudaStream_t s) {
  if (a.batch * a.t == 0) return 1;
  // Vector kernel: 16-bit, D a power of two in 16..256 (tk/src/ops/heads.rs; the
  // reference's kernel has the same bound).
  // Its 128-bit accesses need every operand on a 16-byte boundary; a view that
  // starts at an odd element takes the generic kernel.
  const bool aligned = aligned16(a.qkv) && aligned16(a.q_w) && aligned16(a.k_w) && aligned16(a.cos) &&
                       aligned16(a.sin) && aligned16(a.q) && aligned16(a.k) && aligned16(a.v);
  if (aligned && a.dtype == SVODB_BF16 && dispatch<__nv_bfloat16>(a, s)) return 1;
  if (aligned && a.dtype == SVODB_F16 && dispatch<__half>(a, s)) return 1;
  if (a.dtype == SVODB_BF16) run_generic<__nv_bfloat16>(a, s);
  else if (a.dtype == SVODB_F16) run_generic<__half>(a, s);
  else run_generic<float>(a, s);
  return 0;
}

}  // namespace svodb
