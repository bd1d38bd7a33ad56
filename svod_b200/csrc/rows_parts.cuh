// Row arithmetic shared by the norm kernel and the kernels that fuse a norm with
// what precedes or follows it (embedding lookup, pooling): one warp holds a row
// of d = SPANS * 256 elements in registers, lane l owning elements
// [span*256 + l*8, +8) of every span. Semantics as tk/src/kernels/rows.rs:41-115:
// f32 reductions, biased variance from the centred values, rsqrt(var + eps),
// weight (and bias) in f32, one rounding at the store.
#pragma once

#include "common.cuh"

namespace svodb {
namespace rows_parts {

template <typename T>
__device__ __forceinline__ void unpack8(uint4 u, float (&v)[8]) {
  const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = Elem<T>::unpack(uu[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(Elem<T>::pack(v[0], v[1]), Elem<T>::pack(v[2], v[3]), Elem<T>::pack(v[4], v[5]),
                    Elem<T>::pack(v[6], v[7]));
}

// v <- (v - mean) * 1: centres the row (layer norm) and returns rsqrt(var + eps).
template <int SPANS>
__device__ __forceinline__ float centre_and_scale(float (&v)[SPANS][8], float eps, int layer) {
  constexpr int D = SPANS * 256;
  float mean = 0.f;
  if (layer) {
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < SPANS; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += v[s][i];
    mean = warp_sum(acc) * (1.0f / D);
  }
  float sq = 0.f;
#pragma unroll
  for (int s = 0; s < SPANS; ++s)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[s][i] -= mean;
      sq = fmaf(v[s][i], v[s][i], sq);
    }
  return rsqrtf(warp_sum(sq) * (1.0f / D) + eps);
}

// y = v * inv * w (+ b), the values of one span for this lane, before the rounding.
template <typename T>
__device__ __forceinline__ void affine8(const float (&v)[8], float inv, uint4 wreg, uint4 breg, bool has_b,
                                        float (&y)[8]) {
  float wf[8], bf[8];
  unpack8<T>(wreg, wf);
  unpack8<T>(breg, bf);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    y[i] = v[i] * inv * wf[i];
    if (has_b) y[i] += bf[i];
  }
}

}  // namespace rows_parts
}  // namespace svodb
