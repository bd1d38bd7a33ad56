// Exact CUDA-core linear: the path `linear` takes where the reference would
// build its graph (f32 operands, N not a multiple of 8, K not a multiple of 16).
// f32 accumulation and the same epilogue order as the tensor-core kernel
// (tk/src/kernels/gemm.rs:605-651): +bias -> act -> *up (gated) -> *scale ->
// RoPE turn -> +residual -> one rounding.
#include "common.cuh"
#include "kernels.h"
#include "svodb.h"

namespace svodb {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

// grid (ceil(N/TN), ceil(M/TM)); 256 threads, each a 4x4 patch.
template <typename T>
__global__ void __launch_bounds__(256) gemm_generic_kernel(const GemmArgs a) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bg[TK][TN + 1];  // gate (or the only) half
  __shared__ float Bu[TK][TN + 1];  // up half when gated
  const int tid = threadIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * TM;
  const int n0 = blockIdx.x * TN;
  const T* A = (const T*)a.a;
  const T* W = (const T*)a.w;
  const int tr = tid / 16, tc = tid % 16;
  float accg[4][4] = {}, accu[4][4] = {};
  for (int k0 = 0; k0 < a.k; k0 += TK) {
    for (int e = tid; e < TM * TK; e += 256) {
      const int r = e / TK, c = e % TK;
      const int64_t mm = m0 + r;
      const int kk = k0 + c;
      As[c][r] = (mm < a.m && kk < a.k) ? Elem<T>::to_f(A[mm * a.lda + kk]) : 0.f;
      const int nn = n0 + r;
      const bool in = nn < a.n && kk < a.k;
      Bg[c][r] = in ? Elem<T>::to_f(W[(int64_t)nn * a.ldw + kk]) : 0.f;
      if (a.gated) Bu[c][r] = in ? Elem<T>::to_f(W[(int64_t)(nn + a.n) * a.ldw + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[4], bg[4], bu[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][tr * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bg[j] = Bg[kk][tc * 4 + j];
        bu[j] = a.gated ? Bu[kk][tc * 4 + j] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          accg[i][j] = fmaf(av[i], bg[j], accg[i][j]);
          accu[i][j] = fmaf(av[i], bu[j], accu[i][j]);
        }
    }
    __syncthreads();
  }
  const T* bias = (const T*)a.bias;
  // Without RoPE the residual joins before the single rounding; with RoPE the
  // rotation partner lives in another thread's patch, so the turn and the
  // residual run as passes over the stored output (below).
  const bool fuse_res = a.residual != nullptr && a.rope_cos == nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t mm = m0 + tr * 4 + i;
    if (mm >= a.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nn = n0 + tc * 4 + j;
      if (nn >= a.n) continue;
      float y = accg[i][j];
      if (bias != nullptr) y += Elem<T>::to_f(bias[nn]);
      y = activate_rt(y, a.act);
      if (a.gated) {
        float u = accu[i][j];
        if (bias != nullptr) u += Elem<T>::to_f(bias[nn + a.n]);
        y *= u;
      }
      if (a.has_scale) y *= a.scale;
      if (fuse_res) y += Elem<T>::to_f(((const T*)a.residual)[mm * a.ldr + nn]);
      ((T*)a.c)[mm * a.ldc + nn] = Elem<T>::from_f(y);
    }
  }
}

// RoPE turn as a pass over the stored output. The reference's own graph path
// rounds between the linear and the rotation as well (tk/src/ops/linear.rs:306-331).
template <typename T>
__global__ void __launch_bounds__(256) rope_residual_kernel(const GemmArgs a) {
  const int half = a.rope_head_dim / 2;
  const int pairs = a.rope_heads * half;
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= a.m * pairs) return;
  const int64_t mm = idx / pairs;
  const int p = (int)(idx % pairs);
  const int head = p / half, i = p % half;
  const int64_t pos = mm % a.rope_seq;
  T* row = (T*)a.c + mm * a.ldc + head * a.rope_head_dim;
  const float c = Elem<T>::to_f(((const T*)a.rope_cos)[pos * half + i]);
  const float s = Elem<T>::to_f(((const T*)a.rope_sin)[pos * half + i]);
  const float x1 = Elem<T>::to_f(row[i]), x2 = Elem<T>::to_f(row[i + half]);
  row[i] = Elem<T>::from_f(x1 * c - x2 * s);
  row[i + half] = Elem<T>::from_f(x1 * s + x2 * c);
}

template <typename T>
__global__ void __launch_bounds__(256) add_residual_kernel(const GemmArgs a) {
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= a.m * a.n) return;
  const int64_t mm = idx / a.n;
  const int nn = (int)(idx % a.n);
  T* c = (T*)a.c + mm * a.ldc + nn;
  *c = Elem<T>::from_f(Elem<T>::to_f(*c) + Elem<T>::to_f(((const T*)a.residual)[mm * a.ldr + nn]));
}

template <typename T>
int run(const GemmArgs& a0, cudaStream_t s) {
  GemmArgs a = a0;
  dim3 grid((unsigned)((a.n + TN - 1) / TN), (unsigned)((a.m + TM - 1) / TM));
  const bool rope = a.rope_cos != nullptr;
  gemm_generic_kernel<T><<<grid, 256, 0, s>>>(a);
  if (rope) {
    const int64_t n = a.m * a.rope_heads * (a.rope_head_dim / 2);
    rope_residual_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a);
    if (a.residual != nullptr)
      add_residual_kernel<T><<<(unsigned)((a.m * a.n + 255) / 256), 256, 0, s>>>(a);
  }
  return 0;
}

}  // namespace

int launch_gemm_generic(const GemmArgs& a, cudaStream_t s) {
  if (a.m == 0 || a.n == 0) return 0;
  if (a.dtype == SVODB_BF16) return run<__nv_bfloat16>(a, s);
  if (a.dtype == SVODB_F16) return run<__half>(a, s);
  return run<float>(a, s);
}

}  // namespace svodb
