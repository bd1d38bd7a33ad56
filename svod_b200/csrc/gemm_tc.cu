// tcgen05 GEMM with the fused epilogue of `ops::linear`:
//   C[M,N] = scale * act(A[M,K] . W[N,K]^T + bias) (* up) -> RoPE turn -> + residual
// (order of tk/src/kernels/gemm.rs:605-651; gated weights are `[2N,K]`, gate rows
// over up rows, gemm.rs:21-23,547-559; in-store RoPE, gemm.rs:670-718).
//
// Blackwell design (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: A tile 128x64 and W tile BNx64 per k-block into a
//               128B-swizzled shared-memory ring (non-multicast TMA, OOB rows and
//               the K tail zero-filled by the hardware).
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma 128xBNx16
//               (kind::f16, f32 accumulate) into one of two TMEM accumulators;
//               tcgen05.commit releases ring slots and publishes the accumulator.
//   warps 2..9  epilogue: tcgen05.ld 32 columns at a time (one output row per
//               thread), bias / activation / gate / scale / RoPE / residual in
//               f32, one rounding, 64-byte contiguous stores per row. The second
//               accumulator lets the epilogue of tile i overlap the MMAs of i+1.
// A gated tile loads gate rows and up rows into one BN-row B tile, so a single
// MMA produces [gate | up] side by side in TMEM.
//
// Tiles are walked in groups of 8 tile-rows (the reference's TileOrder::DEFAULT,
// gemm.rs:164,198-213) so concurrently running CTAs share W tiles in L2.
//
// Every mbarrier wait is bounded: on timeout the kernel records a status code,
// drains and frees its TMEM.
#include <cuda.h>
#include <stdio.h>

#include "common.cuh"
#include "gemm_parts.cuh"
#include "kernels.h"
#include "svodb.h"
#include "tensormap.h"

namespace svodb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 16-bit elements = one 128-byte swizzle row
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (2 + kEpiWarps);

template <int BN>
struct Cfg {
  static constexpr int kStageBytes = (BM + BN) * BK * 2;
  static constexpr int kStages = (192 * 1024) / kStageBytes > 8 ? 8 : (192 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  // Output staging for the TMA-store epilogue: one 128-row x 64-column sub-tile
  // (16 KiB, 128-byte swizzle) per column half of the tile.
  static constexpr int kStagingBytes = 2 * 128 * 128;
  static constexpr size_t kSmemBytes =
      (size_t)kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/ + 1024 /*head norm weights*/;
};

struct Params {
  int64_t m;
  int n, k;
  int tiles_m, tiles_n;
  int out_bn;        // output columns per tile: BN, or BN/2 when gated
  int gated;
  int act;
  int has_scale;
  float scale;
  const void* bias;
  const void* residual;
  void* c;
  int64_t ldr, ldc;
  const void* rope_cos;
  const void* rope_sin;
  int rope_width;     // heads * head_dim turned columns (0 = none)
  int rope_head_dim;
  int64_t rope_seq;
  int tma_epilogue;   // stage the output through shared memory and TMA-store it
  // Attention prologue in the store (the tile's column half is one 128-wide
  // head): RMSNorm over the head with `norm_q` for columns below norm_q_cols,
  // `norm_k` below norm_cols, none above; then the rotation for columns below
  // rope_width; staged and TMA-stored like the plain epilogue.
  int head_epilogue;
  int head64_epilogue;  // the same for 64-wide heads: one head per 64-column sub-tile
  const void* norm_q;
  const void* norm_k;
  int norm_q_cols, norm_cols;
  float norm_eps;
  uint32_t* status;
};

using namespace gemm_parts;

template <typename T>
__device__ __forceinline__ void store32(const Params& p, int64_t row, bool row_ok, int n_at, float (&x)[32]) {
  const T* res = (const T*)p.residual;
  T* c = (T*)p.c;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const int n = n_at + v * 8;
    const bool ok = row_ok && n < p.n;
    if (res != nullptr) {
      float r[8];
      load8<T>(res + row * p.ldr + n, ok, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[v * 8 + i] += r[i];
    }
    if (ok) {
      stg128(c + row * p.ldc + n,
             make_uint4(Elem<T>::pack(x[v * 8 + 0], x[v * 8 + 1]), Elem<T>::pack(x[v * 8 + 2], x[v * 8 + 3]),
                        Elem<T>::pack(x[v * 8 + 4], x[v * 8 + 5]), Elem<T>::pack(x[v * 8 + 6], x[v * 8 + 7])));
    }
  }
}


template <typename T, int BN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_r,
                   const Params p) {
  using C = Cfg<BN>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  // The swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + (size_t)S * C::kStageBytes;  // [2 halves][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::kStagingBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* acc_full = bars + 2 * S;
  uint64_t* acc_empty = bars + 2 * S + 2;
  uint64_t* res_full = bars + 2 * S + 4;  // [2 halves]: residual sub-tile landed in staging
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 6);
  float* head_w = reinterpret_cast<float*>(bars + 32);  // [2][128]: q and k head-norm weights as f32

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.k + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kEpiWarps);
      mbar_init(&res_full[i], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  if ((p.head_epilogue || p.head64_epilogue) && threadIdx.x < 256) {
    const T* wsrc = (const T*)(threadIdx.x < 128 ? p.norm_q : p.norm_k);
    const int at = threadIdx.x & 127;
    head_w[threadIdx.x] = (wsrc != nullptr && at < p.rope_head_dim) ? Elem<T>::to_f(wsrc[at]) : 1.0f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      uint32_t issued = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mt, nt;
        tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
        const int m0 = mt * BM;
        const int n0 = nt * p.out_bn;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, p.status)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + (size_t)s * C::kStageBytes;
          uint8_t* b_dst = a_dst + BM * BK * 2;
          mbar_expect_tx(&full[s], (uint32_t)C::kStageBytes);
          tma_load_2d(a_dst, &tmap_a, &full[s], kb * BK, m0);
          if (p.gated) {
            tma_load_2d(b_dst, &tmap_w, &full[s], kb * BK, n0);
            tma_load_2d(b_dst + (BN / 2) * BK * 2, &tmap_w, &full[s], kb * BK, p.n + n0);
          } else {
            tma_load_2d(b_dst, &tmap_w, &full[s], kb * BK, n0);
          }
          ++issued;
          if (++s == S) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (!ok) {
        // Error path: let the copies already in flight land before the CTA's
        // shared memory is released (bounded).
        const uint32_t back = issued < (uint32_t)S ? issued : (uint32_t)S;
        int ss = s;
        uint32_t pp = ph;
        for (uint32_t i = 0; i < back; ++i) {
          if (--ss < 0) {
            ss = S - 1;
            pp ^= 1;
          }
          for (uint32_t it = 0; it < (1u << 16); ++it)
            if (mbar_try_wait(&full[ss], pp)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the schedule so that addresses and descriptors stay
    // warp-uniform values; one elected lane issues the MMAs and the commits.
    {
      constexpr uint32_t idesc = umma_idesc(Elem<T>::kUmmaFormat, BM, BN, 0, 0);
      const bool leader = elect_one();
      const uint64_t desc0 = umma_desc_sw128(smem_u32(smem), 16, 1024);
      int s = 0;
      uint32_t ph = 0;
      int as = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[as], aph ^ 1, p.status)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[s], ph, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_desc = desc0 + (uint64_t)((s * C::kStageBytes) >> 4);
          const uint64_t b_desc = a_desc + (uint64_t)((BM * BK * 2) >> 4);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)  // 16 columns = 32 bytes inside the 128-byte swizzle row
            if (leader) umma_ss(d_tmem, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
          if (leader) tc_commit(&empty[s]);
          if (++s == S) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok && leader) tc_commit(&acc_full[as]);
        __syncwarp();
        if (++as == 2) {
          as = 0;
          aph ^= 1;
        }
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;  // TMEM lanes this warp may touch: 32*(warp%4) ..
    const int chalf = ew >> 2;     // which half of the tile's output columns
    const T* bias = (const T*)p.bias;
    int as = 0;
    uint32_t aph = 0;
    uint32_t res_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mt, nt;
      tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
      const int64_t row = (int64_t)mt * BM + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      const int n0 = nt * p.out_bn;
      const int cols = p.out_bn / 2;  // output columns this warp covers
      const int c_lo = chalf * cols;
      // Head epilogue: this row's rotation tables are requested before the wait
      // for the accumulator, so their L2 latency passes while the tile's MMAs
      // finish (the second half of each 128-byte table row then hits L1).
      uint4 cs4[4], sn4[4];
      const bool head_turned = p.head_epilogue && n0 + c_lo < p.rope_width;
      const int64_t rope_pos = row_ok ? row % p.rope_seq : 0;
      if (head_turned) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          cs4[v] = ldg128((const T*)p.rope_cos + rope_pos * 64 + v * 8);
          sn4[v] = ldg128((const T*)p.rope_sin + rope_pos * 64 + v * 8);
        }
      }
      // Staged epilogue with a residual: the first sub-tile's residual is fetched
      // into the staging buffer while the tile is still being accumulated (the
      // buffer is free once the previous tile's store has read it).
      const bool res_ahead = p.tma_epilogue && p.residual != nullptr && n0 + c_lo < p.n;
      if (res_ahead && (ew & 3) == 0 && lane == 0) {
        tma_store_wait_read();
        mbar_expect_tx(&res_full[chalf], 128 * 128);
        tma_load_2d(staging + chalf * (128 * 128), &tmap_r, &res_full[chalf], n0 + c_lo, mt * BM);
      }
      if (!mbar_wait(&acc_full[as], aph, p.status)) {
        if (res_ahead) mbar_wait(&res_full[chalf], res_phase, p.status);  // the copy in flight lands or times out
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (uint32_t)(as * BN) + ((uint32_t)(quarter * 32) << 16);
      if (p.tma_epilogue) {
        // Staged epilogue: each column half (4 warps, 128 rows) builds 64-column
        // sub-tiles in swizzled shared memory; one thread TMA-loads the residual
        // sub-tile into the same buffer beforehand and TMA-stores the result, so
        // global memory sees whole 128-byte rows instead of per-thread 16-byte
        // pieces (which would compete with the operand loads of the next tile).
        uint8_t* stg = staging + chalf * (128 * 128);
        const bool chief = (ew & 3) == 0 && lane == 0;
        const int r_tile = quarter * 32 + lane;  // this thread's row of the tile
        const int m0 = mt * BM;
        for (int sub = 0; sub < cols / 64; ++sub) {
          const int c0 = c_lo + sub * 64;
          const int n_at = n0 + c0;
          // the previous store out of this buffer must have read it
          if (chief) tma_store_wait_read();
          named_barrier(1 + chalf, 128);
          if (sub > 0 && p.residual != nullptr && chief && n_at < p.n) {  // the first was fetched ahead
            mbar_expect_tx(&res_full[chalf], 128 * 128);
            tma_load_2d(stg, &tmap_r, &res_full[chalf], n_at, m0);
          }
          // 32 columns at a time: accumulator -> epilogue math -> (+ residual) ->
          // four 16-byte chunks of the swizzled staging row.
          uint8_t* srow = stg + r_tile * 128;
          const bool with_res = p.residual != nullptr && n_at < p.n;
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            float xs[32];
            acc32<T>(t_acc + (uint32_t)(c0 + 32 * hc), bias, n_at + 32 * hc, p.n, xs);
            act32(xs, p.act);
            if (p.gated) {
              float u[32];
              acc32<T>(t_acc + (uint32_t)(BN / 2 + c0 + 32 * hc), bias != nullptr ? bias + p.n : nullptr,
                       n_at + 32 * hc, p.n, u);
#pragma unroll
              for (int i = 0; i < 32; ++i) xs[i] *= u[i];
            }
            if (p.has_scale) {
#pragma unroll
              for (int i = 0; i < 32; ++i) xs[i] *= p.scale;
            }
            if (hc == 0 && with_res) {
              // A timed-out wait is only recorded here: every thread of the half
              // still walks both named barriers below, then leaves the tile loop.
              if (!mbar_wait(&res_full[chalf], res_phase, p.status)) ok = false;
              res_phase ^= 1;
            }
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              const int c = hc * 4 + c4;  // chunk c of row r sits at (c ^ (r & 7))
              uint4* slot = reinterpret_cast<uint4*>(srow + ((c ^ (r_tile & 7)) << 4));
              if (with_res) {
                const uint4 rv = *slot;
                const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = Elem<T>::unpack(rr[i]);
                  xs[c4 * 8 + 2 * i] += f.x;
                  xs[c4 * 8 + 2 * i + 1] += f.y;
                }
              }
              *slot = make_uint4(Elem<T>::pack(xs[c4 * 8 + 0], xs[c4 * 8 + 1]), Elem<T>::pack(xs[c4 * 8 + 2], xs[c4 * 8 + 3]),
                                 Elem<T>::pack(xs[c4 * 8 + 4], xs[c4 * 8 + 5]), Elem<T>::pack(xs[c4 * 8 + 6], xs[c4 * 8 + 7]));
            }
          }
          fence_proxy_async_smem();
          named_barrier(1 + chalf, 128);
          if (chief && n_at < p.n) {
            tma_store_2d(&tmap_c, stg, n_at, m0);
            tma_store_commit();
          }
        }
        if (!ok) break;
      } else if (p.head64_epilogue) {
        // 64-wide heads: every 64-column sub-tile is one head with both rotation
        // halves in it; norm and rotation from the accumulator, staged, TMA-stored.
        uint8_t* stg = staging + chalf * (128 * 128);
        const bool chief = (ew & 3) == 0 && lane == 0;
        const int r_tile = quarter * 32 + lane;
        const int m0 = mt * BM;
        const T* cos = (const T*)p.rope_cos;
        const T* sin = (const T*)p.rope_sin;
        const int64_t pos = row_ok ? row % p.rope_seq : 0;
        for (int sub = 0; sub < cols / 64; ++sub) {
          const int c0 = c_lo + sub * 64;
          const int h_col = n0 + c0;
          const bool turned = h_col < p.rope_width;
          const float* nw = h_col < p.norm_q_cols ? head_w : (h_col < p.norm_cols ? head_w + 128 : nullptr);
          float a[32], b[32];
          acc32<T>(t_acc + (uint32_t)c0, bias, h_col, p.n, a);
          acc32<T>(t_acc + (uint32_t)(c0 + 32), bias, h_col + 32, p.n, b);
          uint4 cs4[4], sn4[4];
          if (turned) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              cs4[v] = ldg128(cos + pos * 32 + v * 8);
              sn4[v] = ldg128(sin + pos * 32 + v * 8);
            }
          }
          if (nw != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) ss = fmaf(a[i], a[i], fmaf(b[i], b[i], ss));
            const float inv = rsqrtf(ss * (1.0f / 64.0f) + p.norm_eps);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              a[i] = a[i] * inv * nw[i];
              b[i] = b[i] * inv * nw[32 + i];
            }
          }
          if (turned) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint32_t cu[4] = {cs4[v].x, cs4[v].y, cs4[v].z, cs4[v].w};
              const uint32_t su[4] = {sn4[v].x, sn4[v].y, sn4[v].z, sn4[v].w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 c2 = Elem<T>::unpack(cu[i]), s2 = Elem<T>::unpack(su[i]);
                const int e = v * 8 + 2 * i;
                const float a0 = a[e], a1 = a[e + 1], b0 = b[e], b1 = b[e + 1];
                a[e] = a0 * c2.x - b0 * s2.x;
                b[e] = a0 * s2.x + b0 * c2.x;
                a[e + 1] = a1 * c2.y - b1 * s2.y;
                b[e + 1] = a1 * s2.y + b1 * c2.y;
              }
            }
          }
          // the previous store out of this buffer must have read it
          if (chief) tma_store_wait_read();
          named_barrier(1 + chalf, 128);
          uint8_t* srow = stg + r_tile * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            *reinterpret_cast<uint4*>(srow + ((c ^ (r_tile & 7)) << 4)) =
                make_uint4(Elem<T>::pack(a[c * 8 + 0], a[c * 8 + 1]), Elem<T>::pack(a[c * 8 + 2], a[c * 8 + 3]),
                           Elem<T>::pack(a[c * 8 + 4], a[c * 8 + 5]), Elem<T>::pack(a[c * 8 + 6], a[c * 8 + 7]));
            *reinterpret_cast<uint4*>(srow + (((c + 4) ^ (r_tile & 7)) << 4)) =
                make_uint4(Elem<T>::pack(b[c * 8 + 0], b[c * 8 + 1]), Elem<T>::pack(b[c * 8 + 2], b[c * 8 + 3]),
                           Elem<T>::pack(b[c * 8 + 4], b[c * 8 + 5]), Elem<T>::pack(b[c * 8 + 6], b[c * 8 + 7]));
          }
          fence_proxy_async_smem();
          named_barrier(1 + chalf, 128);
          if (chief && h_col < p.n) {
            tma_store_2d(&tmap_c, stg, h_col, m0);
            tma_store_commit();
          }
        }
      } else if (p.head_epilogue) {
        // One 128-column head per column half. A first pass over the accumulator
        // takes the sum of squares; the second forms both halves of the head at
        // once (a rotated column needs its partner 64 columns away): the first
        // half goes to the staging buffer, the second waits packed in registers
        // until the first sub-tile's TMA store has read the buffer.
        uint8_t* stg = staging + chalf * (128 * 128);
        const bool chief = (ew & 3) == 0 && lane == 0;
        const int r_tile = quarter * 32 + lane;
        const int m0 = mt * BM;
        const int h_col = n0 + c_lo;  // first output column of this head
        const bool turned = head_turned;
        const float* nw = h_col < p.norm_q_cols ? head_w : (h_col < p.norm_cols ? head_w + 128 : nullptr);
        const T* cos = (const T*)p.rope_cos;
        const T* sin = (const T*)p.rope_sin;
        const int64_t pos = rope_pos;
        const uint32_t t_head = t_acc + (uint32_t)c_lo;
        float inv = 1.f;
        if (nw != nullptr) {
          float ss0 = 0.f, ss1 = 0.f;
#pragma unroll 1
          for (int c = 0; c < 128; c += 64) {
            uint32_t r0[32], r1[32];
            tmem_ld32(t_head + (uint32_t)c, r0);
            tmem_ld32(t_head + (uint32_t)(c + 32), r1);
            tmem_ld_wait();
            if (bias != nullptr) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float b0[8], b1[8];
                load8<T>(bias + h_col + c + v * 8, true, b0);
                load8<T>(bias + h_col + c + 32 + v * 8, true, b1);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  r0[v * 8 + i] = __float_as_uint(__uint_as_float(r0[v * 8 + i]) + b0[i]);
                  r1[v * 8 + i] = __float_as_uint(__uint_as_float(r1[v * 8 + i]) + b1[i]);
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              ss0 = fmaf(__uint_as_float(r0[i]), __uint_as_float(r0[i]), ss0);
              ss1 = fmaf(__uint_as_float(r1[i]), __uint_as_float(r1[i]), ss1);
            }
          }
          inv = rsqrtf((ss0 + ss1) * (1.0f / 128.0f) + p.norm_eps);
        }
        // the previous store out of this buffer must have read it
        if (chief) tma_store_wait_read();
        named_barrier(1 + chalf, 128);
        uint8_t* srow = stg + r_tile * 128;
        uint32_t keep[32];  // second half of the head, packed
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          uint32_t ra[32], rb[32];
          tmem_ld32(t_head + (uint32_t)(32 * hc), ra);
          tmem_ld32(t_head + (uint32_t)(64 + 32 * hc), rb);
          if (turned && hc == 1) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              cs4[v] = ldg128(cos + pos * 64 + 32 + v * 8);
              sn4[v] = ldg128(sin + pos * 64 + 32 + v * 8);
            }
          }
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float a[8], b[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              a[i] = __uint_as_float(ra[v * 8 + i]);
              b[i] = __uint_as_float(rb[v * 8 + i]);
            }
            if (bias != nullptr) {
              float b0[8], b1[8];
              load8<T>(bias + h_col + 32 * hc + v * 8, true, b0);
              load8<T>(bias + h_col + 64 + 32 * hc + v * 8, true, b1);
#pragma unroll
              for (int i = 0; i < 8; ++i) a[i] += b0[i], b[i] += b1[i];
            }
            if (nw != nullptr) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                a[i] = a[i] * inv * nw[32 * hc + v * 8 + i];
                b[i] = b[i] * inv * nw[64 + 32 * hc + v * 8 + i];
              }
            }
            if (turned) {
              const uint32_t cu[4] = {cs4[v].x, cs4[v].y, cs4[v].z, cs4[v].w};
              const uint32_t su[4] = {sn4[v].x, sn4[v].y, sn4[v].z, sn4[v].w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 c2 = Elem<T>::unpack(cu[i]), s2 = Elem<T>::unpack(su[i]);
                const float a0 = a[2 * i], a1 = a[2 * i + 1], b0 = b[2 * i], b1 = b[2 * i + 1];
                a[2 * i] = a0 * c2.x - b0 * s2.x;
                b[2 * i] = a0 * s2.x + b0 * c2.x;
                a[2 * i + 1] = a1 * c2.y - b1 * s2.y;
                b[2 * i + 1] = a1 * s2.y + b1 * c2.y;
              }
            }
            const int chunk = hc * 4 + v;  // 16-byte chunk of the 64-column sub-tile row
            *reinterpret_cast<uint4*>(srow + ((chunk ^ (r_tile & 7)) << 4)) =
                make_uint4(Elem<T>::pack(a[0], a[1]), Elem<T>::pack(a[2], a[3]), Elem<T>::pack(a[4], a[5]),
                           Elem<T>::pack(a[6], a[7]));
#pragma unroll
            for (int i = 0; i < 4; ++i) keep[chunk * 4 + i] = Elem<T>::pack(b[2 * i], b[2 * i + 1]);
          }
        }
        fence_proxy_async_smem();
        named_barrier(1 + chalf, 128);
        if (chief && h_col < p.n) {
          tma_store_2d(&tmap_c, stg, h_col, m0);
          tma_store_commit();
          tma_store_wait_read();
        }
        named_barrier(1 + chalf, 128);
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(srow + ((c ^ (r_tile & 7)) << 4)) =
              make_uint4(keep[c * 4], keep[c * 4 + 1], keep[c * 4 + 2], keep[c * 4 + 3]);
        fence_proxy_async_smem();
        named_barrier(1 + chalf, 128);
        if (chief && h_col + 64 < p.n) {
          tma_store_2d(&tmap_c, stg, h_col + 64, m0);
          tma_store_commit();
        }
      } else if (p.rope_width > 0 && n0 + c_lo < p.rope_width) {
        // In-store RoPE: whole heads, pairs (c, c + head_dim/2) from two chunks.
        const int hd = p.rope_head_dim, half = hd / 2;
        const T* cos = (const T*)p.rope_cos;
        const T* sin = (const T*)p.rope_sin;
        const int64_t pos = row_ok ? row % p.rope_seq : 0;
        for (int h0 = c_lo; h0 < c_lo + cols; h0 += hd) {
          const bool turned = n0 + h0 < p.rope_width;
          for (int j = 0; j < half; j += 32) {
            float x1[32], x2[32];
            acc32<T>(t_acc + (uint32_t)(h0 + j), bias, n0 + h0 + j, p.n, x1);
            acc32<T>(t_acc + (uint32_t)(h0 + half + j), bias, n0 + h0 + half + j, p.n, x2);
            if (turned) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float cs[8], sn[8];
                load8<T>(cos + pos * half + j + v * 8, true, cs);
                load8<T>(sin + pos * half + j + v * 8, true, sn);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float a = x1[v * 8 + i], b = x2[v * 8 + i];
                  x1[v * 8 + i] = a * cs[i] - b * sn[i];
                  x2[v * 8 + i] = a * sn[i] + b * cs[i];
                }
              }
            }
            store32<T>(p, row, row_ok, n0 + h0 + j, x1);
            store32<T>(p, row, row_ok, n0 + h0 + half + j, x2);
          }
        }
      } else {
        for (int c0 = c_lo; c0 < c_lo + cols; c0 += 32) {
          float x[32];
          acc32<T>(t_acc + (uint32_t)c0, bias, n0 + c0, p.n, x);
          act32(x, p.act);
          if (p.gated) {
            float u[32];
            acc32<T>(t_acc + (uint32_t)(BN / 2 + c0), bias != nullptr ? bias + p.n : nullptr, n0 + c0, p.n, u);
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] *= u[i];
          }
          if (p.has_scale) {
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] *= p.scale;
          }
          store32<T>(p, row, row_ok, n0 + c0, x);
        }
      }
      // All of this warp's TMEM reads of the tile have completed (wait::ld in acc32).
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
      if (++as == 2) {
        as = 0;
        aph ^= 1;
      }
    }
  }

  if ((p.tma_epilogue || p.head_epilogue || p.head64_epilogue) && warp >= 2 && ((warp - 2) & 3) == 0 && lane == 0) tma_store_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T, int BN>
int run(const GemmArgs& a, const Params& p0, int sms, cudaStream_t s, char* cfg, size_t cfg_len) {
  using C = Cfg<BN>;
  Params p = p0;
  p.out_bn = a.gated ? BN / 2 : BN;
  p.tiles_m = (int)((a.m + BM - 1) / BM);
  p.tiles_n = (a.n + p.out_bn - 1) / p.out_bn;
  CUtensorMap ta, tw;
  const int dt = a.dtype;
  if (!make_tmap_2d(&ta, a.a, dt, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM)) return -1;
  const uint64_t w_rows = (uint64_t)(a.gated ? 2 * a.n : a.n);
  if (!make_tmap_2d(&tw, a.w, dt, (uint64_t)a.k, w_rows, (uint64_t)a.ldw, BK, a.gated ? BN / 2 : BN)) return -1;
  // The staged epilogue needs whole 64-column sub-tiles per column half and
  // plain (non-rotating) stores; small tiles and RoPE keep the direct stores.
  const bool per_head = a.rope_cos != nullptr || a.norm_q != nullptr || a.norm_k != nullptr;
  p.tma_epilogue = (p.out_bn >= 128 && !per_head) ? 1 : 0;
  // Heads of 128 columns are one column half of a 256-wide tile: staged too.
  p.head_epilogue = (per_head && a.rope_head_dim == 128 && p.out_bn == 256) ? 1 : 0;
  // Heads of 64 columns are one sub-tile each (the tile's column halves hold 1 or 2 of them).
  p.head64_epilogue = (per_head && a.rope_head_dim == 64 && p.out_bn >= 128) ? 1 : 0;
  CUtensorMap tc = ta, tr = ta;
  if (p.tma_epilogue || p.head_epilogue || p.head64_epilogue) {
    if (!make_tmap_2d(&tc, a.c, dt, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, 64, BM)) return -1;
    tr = tc;
    if (a.residual != nullptr &&
        !make_tmap_2d(&tr, a.residual, dt, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldr, 64, BM))
      return -1;
  }
  // the attribute belongs to the device's copy of the kernel: once per device
  static bool attr_seen[64] = {};
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_seen[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)C::kSmemBytes) != cudaSuccess)
      return -1;
    attr_set = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sms ? tiles : sms;
  gemm_tc_kernel<T, BN><<<grid, kThreads, C::kSmemBytes, s>>>(ta, tw, tc, tr, p);
  if (cfg != nullptr)
    snprintf(cfg, cfg_len, "{bm:%d,bn:%d,bk:%d,stages:%d,gated:%d,grid:%d}", BM, BN, BK, C::kStages, a.gated, grid);
  return 0;
}


int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

}  // namespace

bool gemm_tc_covers(const GemmArgs& a) {
  // The reference's kernel gate (tk/src/ops/shape.rs:120-139): 16-bit operands,
  // N a multiple of 8, K a multiple of 16. Plus what TMA and the 128-bit
  // epilogue accesses need: 16-byte aligned bases and row strides.
  if (a.dtype != SVODB_BF16 && a.dtype != SVODB_F16) return false;
  if (a.n % 8 != 0 || a.k % 16 != 0 || a.m <= 0 || a.n <= 0 || a.k <= 0) return false;
  if (a.m > 0x7fffffffLL) return false;
  if (a.lda % 8 != 0 || a.ldw % 8 != 0 || a.ldc % 8 != 0) return false;
  if (!aligned16(a.a) || !aligned16(a.w) || !aligned16(a.c)) return false;
  if (a.bias != nullptr && !aligned16(a.bias)) return false;
  if (a.residual != nullptr && (!aligned16(a.residual) || a.ldr % 8 != 0)) return false;
  if (a.rope_cos != nullptr) {
    // A tile turns whole heads: pairs must sit in two 32-column chunks of one
    // warp's column range.
    const int hd = a.rope_head_dim;
    if (hd != 64 && hd != 128) return false;
    if (a.gated || a.act != kActNone || a.residual != nullptr || a.has_scale) return false;
    if (!aligned16(a.rope_cos) || !aligned16(a.rope_sin)) return false;
  }
  if (a.norm_q != nullptr || a.norm_k != nullptr) {
    // The per-head norm lives in the staged head epilogues: 64- or 128-column heads.
    if (a.rope_head_dim != 128 && a.rope_head_dim != 64) return false;
    if (a.gated || a.act != kActNone || a.residual != nullptr || a.has_scale) return false;
    if ((a.norm_q != nullptr && !aligned16(a.norm_q)) || (a.norm_k != nullptr && !aligned16(a.norm_k))) return false;
  }
  return true;
}

int launch_gemm_tc(const GemmArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  if (!gemm_tc_covers(a)) return 1;
  Params p{};
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.gated = a.gated;
  p.act = a.act;
  p.has_scale = a.has_scale;
  p.scale = a.scale;
  p.bias = a.bias;
  p.residual = a.residual;
  p.c = a.c;
  p.ldr = a.ldr;
  p.ldc = a.ldc;
  p.rope_cos = a.rope_cos;
  p.rope_sin = a.rope_sin;
  p.rope_width = a.rope_cos != nullptr ? a.rope_heads * a.rope_head_dim : 0;
  p.rope_head_dim = a.rope_head_dim;
  p.rope_seq = a.rope_seq > 0 ? a.rope_seq : 1;
  p.norm_q = a.norm_q;
  p.norm_k = a.norm_k;
  p.norm_q_cols = a.norm_q != nullptr ? a.norm_q_heads * a.rope_head_dim : 0;
  p.norm_cols = a.norm_k != nullptr ? (a.norm_q_heads + a.norm_k_heads) * a.rope_head_dim : p.norm_q_cols;
  p.norm_eps = a.norm_eps;
  p.status = a.status;
  const int sms = sm_count();
  // Tile width: the widest MMA whose tile count still fills the SMs. A gated
  // tile spends half its MMA width on the up rows; a turned tile must hold
  // whole heads per epilogue warp (64 columns at least).
  const int64_t tiles_m = (a.m + BM - 1) / BM;
  auto tiles = [&](int bn) { return tiles_m * ((a.n + (a.gated ? bn / 2 : bn) - 1) / (a.gated ? bn / 2 : bn)); };
  int bn = 256;
  const bool per_head = a.rope_cos != nullptr || a.norm_q != nullptr || a.norm_k != nullptr;
  const int min_bn = a.gated ? 128 : (per_head ? 2 * a.rope_head_dim : 64);
  // Tile width by a small cost model (cycles): waves x (the longer of the tile's MMAs and the time
  // its operands take to arrive from L2 at ~52 bytes per clock and SM, plus a fixed per-tile cost of
  // prologue, first-load latency and epilogue). Narrow tiles fill more SMs but move more bytes per
  // flop; the widest of equally cheap widths wins.
  {
    double best = 0;
    for (int cand = 256; cand >= min_bn; cand /= 2) {
      const double waves = (double)((tiles(cand) + sms - 1) / sms);
      const double mma = 2.0 * cand * (a.k / BK);
      const double feed = (double)(BM + cand) * a.k * 2.0 / 52.0;
      const double cost = waves * ((mma > feed ? mma : feed) + 6000.0);
      if (cand == 256 || cost < best * 0.97) best = cost, bn = cand;
    }
  }
  if (bn < min_bn) bn = min_bn;
  if ((a.force_bn == 64 || a.force_bn == 128 || a.force_bn == 256) && a.force_bn >= min_bn) bn = a.force_bn;
  if (bn > 256) return 1;
  int rc;
  if (a.dtype == SVODB_BF16) {
    rc = bn == 256 ? run<__nv_bfloat16, 256>(a, p, sms, s, cfg, cfg_len)
       : bn == 128 ? run<__nv_bfloat16, 128>(a, p, sms, s, cfg, cfg_len)
                   : run<__nv_bfloat16, 64>(a, p, sms, s, cfg, cfg_len);
  } else {
    rc = bn == 256 ? run<__half, 256>(a, p, sms, s, cfg, cfg_len)
       : bn == 128 ? run<__half, 128>(a, p, sms, s, cfg, cfg_len)
                   : run<__half, 64>(a, p, sms, s, cfg, cfg_len);
  }
  return rc;
}

}  // namespace svodb
