// LayerNorm / RMSNorm over the last dim, optionally after a residual add whose
// rounded sum is written out and is what gets normalised.
//
// Semantics follow tk/src/kernels/rows.rs:41-115: f32 reductions, biased
// variance from the centred values, `rsqrt(var + eps)`, weight (and bias) in
// f32, one rounding at the store; the fused sum is rounded to the element type
// first (rows.rs:77-85).
//
// HBM-bound: one warp per row, 128-bit loads/stores, the whole row held in
// registers so x (and the residual) are read exactly once.
#include "common.cuh"
#include "kernels.h"
#include "rows_parts.cuh"
#include "svodb.h"

namespace svodb {

namespace {

constexpr int kWarpsPerBlock = 8;

// d = SPANS * 256: lane l owns elements [span*256 + l*8, +8).
template <typename T, int SPANS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    norm_rows_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                     const T* __restrict__ b, T* __restrict__ out, T* __restrict__ sum, int64_t rows, float eps,
                     int layer) {
  const int lane = threadIdx.x & 31;
  constexpr int D = SPANS * 256;
  // The weights (and bias) stay in registers across the rows a warp walks: read
  // per row they would cost the load path as much as the row itself.
  uint4 wreg[SPANS], breg[SPANS];
#pragma unroll
  for (int s = 0; s < SPANS; ++s) {
    wreg[s] = ldg128(w + s * 256 + lane * 8);
    breg[s] = b != nullptr ? ldg128(b + s * 256 + lane * 8) : make_uint4(0, 0, 0, 0);
  }
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  for (int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); row < rows; row += stride) {
    const T* xr = x + row * D;
    float v[SPANS][8];
#pragma unroll
    for (int s = 0; s < SPANS; ++s) {
      const int off = s * 256 + lane * 8;
      rows_parts::unpack8<T>(ldg128(xr + off), v[s]);
      if (res != nullptr) {
        float r[8];
        rows_parts::unpack8<T>(ldg128(res + row * D + off), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[s][i] += r[i];
        const uint4 packed = rows_parts::pack8<T>(v[s]);  // the rounded sum is what gets normalised
        rows_parts::unpack8<T>(packed, v[s]);
        stg128(sum + row * D + off, packed);
      }
    }
    const float inv = rows_parts::centre_and_scale<SPANS>(v, eps, layer);
#pragma unroll
    for (int s = 0; s < SPANS; ++s) {
      float y[8];
      rows_parts::affine8<T>(v[s], inv, wreg[s], breg[s], b != nullptr, y);
      stg128(out + row * D + s * 256 + lane * 8, rows_parts::pack8<T>(y));
    }
  }
}

// Any d, any float type: one block per row, three passes served by L1/L2.
template <typename T>
__global__ void __launch_bounds__(256)
    norm_rows_generic_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                             const T* __restrict__ b, T* __restrict__ out, T* __restrict__ sum, int d, float eps,
                             int layer) {
  __shared__ float red[8];
  __shared__ float bcast;
  const int64_t row = blockIdx.x;
  const T* xr = x + row * d;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  auto value = [&](int i) -> float {
    float f = Elem<T>::to_f(xr[i]);
    if (res != nullptr) f = Elem<T>::to_f(Elem<T>::from_f(f + Elem<T>::to_f(res[row * d + i])));
    return f;
  };
  auto block_sum = [&](float v) -> float {
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
      float t = lane < 8 ? red[lane] : 0.f;
      t = warp_sum(t);
      if (lane == 0) bcast = t;
    }
    __syncthreads();
    return bcast;
  };
  float acc = 0.f;
  for (int i = tid; i < d; i += 256) {
    float f = value(i);
    if (res != nullptr) sum[row * d + i] = Elem<T>::from_f(f);
    acc += f;
  }
  const float mean = layer ? block_sum(acc) / d : 0.f;
  float sq = 0.f;
  for (int i = tid; i < d; i += 256) {
    float c = value(i) - mean;
    sq = fmaf(c, c, sq);
  }
  const float inv = rsqrtf(block_sum(sq) / d + eps);
  for (int i = tid; i < d; i += 256) {
    float y = (value(i) - mean) * inv * Elem<T>::to_f(w[i]);
    if (b != nullptr) y += Elem<T>::to_f(b[i]);
    out[row * d + i] = Elem<T>::from_f(y);
  }
}

template <typename T, int SPANS>
void run_rows(const NormArgs& a, cudaStream_t s) {
  // A few resident blocks per SM walk the rows with a grid stride.
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int64_t want = (a.rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const unsigned blocks = (unsigned)(want < (int64_t)sms * 6 ? want : (int64_t)sms * 6);
  norm_rows_kernel<T, SPANS><<<blocks, kWarpsPerBlock * 32, 0, s>>>(
      (const T*)a.x, (const T*)a.residual, (const T*)a.w, (const T*)a.b, (T*)a.out, (T*)a.sum, a.rows, a.eps, a.layer);
}

template <typename T>
bool run_rows_dispatch(const NormArgs& a, cudaStream_t s) {
  switch (a.d / 256) {
    case 1: run_rows<T, 1>(a, s); return true;
    case 2: run_rows<T, 2>(a, s); return true;
    case 3: run_rows<T, 3>(a, s); return true;
    case 4: run_rows<T, 4>(a, s); return true;
    case 5: run_rows<T, 5>(a, s); return true;
    case 6: run_rows<T, 6>(a, s); return true;
    case 7: run_rows<T, 7>(a, s); return true;
    case 8: run_rows<T, 8>(a, s); return true;
    default: return false;
  }
}

template <typename T>
void run_generic(const NormArgs& a, cudaStream_t s) {
  norm_rows_generic_kernel<T><<<(unsigned)a.rows, 256, 0, s>>>((const T*)a.x, (const T*)a.residual, (const T*)a.w,
                                                                 (const T*)a.b, (T*)a.out, (T*)a.sum, a.d, a.eps,
                                                                 a.layer);
}

}  // namespace

int launch_norm(const NormArgs& a, cudaStream_t s) {
  if (a.rows == 0) return 1;
  // The warp-per-row kernel covers what the reference's kernel covers: 16-bit
  // rows of 256..2048 elements in multiples of 256 (tk/src/ops/config/norm.rs:19-24).
  // Its 128-bit accesses need every operand on a 16-byte boundary (a view that
  // starts at an odd element does not); such rows take the generic kernel.
  const bool fits = a.d % 256 == 0 && a.d >= 256 && a.d <= 2048 && aligned16(a.x) && aligned16(a.residual) &&
                    aligned16(a.w) && aligned16(a.b) && aligned16(a.out) && aligned16(a.sum);
  if (fits && a.dtype == SVODB_BF16 && run_rows_dispatch<__nv_bfloat16>(a, s)) return 1;
  if (fits && a.dtype == SVODB_F16 && run_rows_dispatch<__half>(a, s)) return 1;
  if (a.dtype == SVODB_BF16) run_generic<__nv_bfloat16>(a, s);
  else if (a.dtype == SVODB_F16) run_generic<__half>(a, s);
  else run_generic<float>(a, s);
  return 0;
}

}  // namespace svodb
