// Pieces shared by the one-CTA and the CTA-pair tcgen05 GEMM kernels: the tile
// raster and the accumulator -> f32 helpers of the epilogue.
#pragma once

#include "common.cuh"

namespace svodb {
namespace gemm_parts {

// Tiles are walked in groups of 8 tile rows, column by column inside a group, so
// that the CTAs running at one time share W tiles and a band of A rows in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mt, int& nt) {
  const int per_group = 8 * tiles_n;
  const int group = t / per_group;
  const int first = group * 8;
  const int gsize = tiles_m - first < 8 ? tiles_m - first : 8;
  const int r = t - group * per_group;
  mt = first + r % gsize;
  nt = r / gsize;
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, bool ok, float (&f)[8]) {
  if (ok) {
    uint4 u = ldg128(p);
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 v = Elem<T>::unpack(uu[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 0.f;
  }
}

__device__ __forceinline__ void act32(float (&x)[32], int act) {
  switch (act) {
    case kActGelu:
#pragma unroll
      for (int i = 0; i < 32; i += 2) gelu2_f(x[i], x[i + 1]);
      break;
    case kActSilu:
#pragma unroll
      for (int i = 0; i < 32; ++i) x[i] = silu_f(x[i]);
      break;
    case kActGeluTanh:
#pragma unroll
      for (int i = 0; i < 32; ++i) x[i] = gelu_tanh_f(x[i]);
      break;
    default: break;
  }
}

// Loads 32 accumulator columns starting at `col` of this warp's lane quarter
// and adds the bias of output columns `n_at ..`.
template <typename T>
__device__ __forceinline__ void acc32(uint32_t taddr, const T* bias, int n_at, int n_lim, float (&x)[32]) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
  // the bias chunk is requested while the accumulator load is in flight: the two
  // latencies overlap instead of following one another
  uint4 bu[4];
  if (bias != nullptr) {
#pragma unroll
    for (int v = 0; v < 4; ++v)
      bu[v] = n_at + v * 8 < n_lim ? ldg128(bias + n_at + v * 8) : make_uint4(0, 0, 0, 0);
  }
  tmem_ld_wait_for(r);
#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(r[i]);
  if (bias != nullptr) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const uint32_t uu[4] = {bu[v].x, bu[v].y, bu[v].z, bu[v].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 b = Elem<T>::unpack(uu[i]);
        x[v * 8 + 2 * i] += b.x;
        x[v * 8 + 2 * i + 1] += b.y;
      }
    }
  }
}

}  // namespace gemm_parts
}  // namespace svodb
