// Split-K form of the CTA-pair tcgen05 GEMM (gemm_tc2.cu): the reference's tail
// split + merge (tk/src/kernels/gemm.rs:454-466,750-808 — the k loop cut into
// pieces whose f32 partials a second pass merges, applying the epilogue once;
// never with a gate or a rotation) for problems of few 256 x 256 tiles and a
// long k loop.
//
// A work item is (tile, piece). The loader and the MMA warp are those of the
// pair kernel over the piece's k-blocks (same barriers, same bounded waits).
// Each CTA of the pair leaves its 128 x 256 f32 block in the caller's workspace
// — in the order the epilogue warps hold it, so every access is 512 contiguous
// bytes per warp — and counts it on the tile's counter; the CTA that counts a
// tile's last block merges the blocks in piece order (the sum never depends on
// who came last), applies bias -> activation -> scale -> residual, and stores
// through per-warp 32-row slabs by TMA. Nobody waits for anybody: a CTA that is
// not last goes on to its next item. A kernel of its own rather than an
// instantiation of the pair kernel's template, so the pair kernel stays as it is.
#include <cuda.h>
#include <stdio.h>

#include "common.cuh"
#include "gemm_parts.cuh"
#include "kernels.h"
#include "svodb.h"
#include "tensormap.h"

namespace svodb {

namespace {

constexpr int BM = 128;  // rows per CTA (the pair's tile has 256)
constexpr int BN = 256;  // accumulator columns
constexpr int BK = 64;
constexpr int kStages = 6;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kStageBytes = (BM + BN / 2) * BK * 2;  // A 16 KiB + this CTA's half of W 16 KiB
constexpr int kStagingBytes = kEpiWarps * 32 * 128;  // a 32-row x 64-column slab per epilogue warp
constexpr int kTmemCols = 512;
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;

struct ParamsSk {
  int64_t m;
  int n, k;
  int tiles_m, tiles_n;
  int act;
  int has_scale;
  float scale;
  const void* bias;
  const void* residual;
  int64_t ldr;
  uint32_t* status;
  int k_splits;     // piece s accumulates k-blocks [s*num_kb/S, (s+1)*num_kb/S)
  float* partials;  // [tile][piece][cta][128 x 256] f32
  int* counters;    // [tile][cta]: blocks landed
};

using namespace gemm_parts;

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tc2_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                           const __grid_constant__ CUtensorMap tmap_c, const ParamsSk p) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + (size_t)S * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  uint64_t* full = bars;                   // [S]  used in the even CTA
  uint64_t* empty = bars + S;              // [S]  in both CTAs
  uint64_t* acc_full = bars + 2 * S;       // [2]  in both CTAs
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2]  used in the even CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = the CTA that issues the MMAs
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int num_kb = (p.k + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int splits = p.k_splits;
  const int num_items = num_tiles * splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 2 * kEpiWarps);  // the epilogue warps of both CTAs
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  // The partner's barriers must exist before anything signals them.
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int it = pair; it < num_items && ok; it += pairs) {
        const int t = it / splits;
        const int split = it - t * splits;
        const int kb0 = split * num_kb / splits;
        const int kb1 = (split + 1) * num_kb / splits;
        int mt, nt;
        tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
        const int m0 = mt * 2 * BM + (int)rank * BM;
        const int n0 = nt * BN;
        // this CTA's 128 rows of the W tile: the lower / upper half of the tile's 256 rows
        const int w_row = n0 + (int)rank * (BN / 2);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, p.status)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + (size_t)s * kStageBytes;
          uint8_t* b_dst = a_dst + BM * BK * 2;
          const uint32_t full_addr = cluster_map(&full[s], 0);
          if (rank == 0) mbar_expect_tx(&full[s], (uint32_t)(2 * kStageBytes));
          tma_load_2d_pair(a_dst, &tmap_a, full_addr, kb * BK, m0);
          tma_load_2d_pair(b_dst, &tmap_w, full_addr, kb * BK, w_row);
          if (++s == S) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      // Error path: a bounded pause lets copies already in flight land before
      // the CTA's shared memory is released.
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (rank == 0) {
      constexpr uint32_t idesc = umma_idesc(Elem<T>::kUmmaFormat, 2 * BM, BN, 0, 0);
      const bool leader = elect_one();
      const uint64_t desc0 = umma_desc_sw128(smem_u32(smem), 16, 1024);
      int s = 0;
      uint32_t ph = 0;
      int as = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int it = pair; it < num_items && ok; it += pairs) {
        const int split = it % splits;
        const int kb0 = split * num_kb / splits;
        const int kb1 = (split + 1) * num_kb / splits;
        if (!mbar_wait(&acc_empty[as], aph ^ 1, p.status)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_desc = desc0 + (uint64_t)((s * kStageBytes) >> 4);
          const uint64_t b_desc = a_desc + (uint64_t)((BM * BK * 2) >> 4);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            if (leader)
              umma_ss_pair(d_tmem, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)(k4 * 2), idesc,
                           ((kb - kb0) | k4) != 0 ? 1u : 0u);
          // the stage is free in both CTAs once these MMAs have read it
          if (leader) {
            tc_commit_pair(cluster_map(&empty[s], 0));
            tc_commit_pair(cluster_map(&empty[s], 1));
          }
          if (++s == S) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok && leader) {
          tc_commit_pair(cluster_map(&acc_full[as], 0));
          tc_commit_pair(cluster_map(&acc_full[as], 1));
        }
        __syncwarp();
        if (++as == 2) {
          as = 0;
          aph ^= 1;
        }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, each its 128 rows) ----------------
    // Every item leaves this CTA's f32 block in the workspace and counts it; the
    // CTA that counts the last block of a tile merges the blocks in split order
    // (so the sum does not depend on who came last), applies the epilogue once and
    // stores. Nobody waits for anybody: a CTA that is not last simply goes on.
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int group = ew >> 2;  // which 128 of the tile's 256 columns
    const T* bias = (const T*)p.bias;
    volatile uint32_t* landed = tmem_slot + 1;
    uint8_t* slab = staging + ew * (32 * 128);
    uint8_t* srow = slab + lane * 128;
    int as = 0;
    uint32_t aph = 0;
    for (int it = pair; it < num_items; it += pairs) {
      const int t = it / splits;
      const int split = it - t * splits;
      int mt, nt;
      tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
      const int m_at = mt * 2 * BM + (int)rank * BM + quarter * 32;
      const int n0 = nt * BN + group * 128;
      if (!mbar_wait(&acc_full[as], aph, p.status)) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (uint32_t)(as * BN + group * 128) + ((uint32_t)(quarter * 32) << 16);
      // A block is kept in the order the warps hold it, not row-major: 32 chunks of
      // (lane quarter, 32 columns), each [8 column quads][32 lanes][4 floats], so that
      // every store and every load of the merge is 512 contiguous bytes per warp.
      const size_t block = (size_t)BM * BN;
      float* mine = p.partials + (((size_t)t * splits + split) * 2 + rank) * block +
                    (size_t)(quarter * 8 + group * 4) * 1024 + lane * 4;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(t_acc + (uint32_t)(c * 32), r);
        tmem_ld_wait_for(r);
#pragma unroll
        for (int v = 0; v < 8; ++v)
          __stcg(reinterpret_cast<uint4*>(mine + c * 1024 + v * 128),
                 make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_map(&acc_empty[as], 0));
      if (++as == 2) {
        as = 0;
        aph ^= 1;
      }
      __threadfence();
      named_barrier(1, 32 * kEpiWarps);
      if (ew == 0 && lane == 0) *landed = (uint32_t)atomicAdd(&p.counters[t * 2 + (int)rank], 1);
      named_barrier(1, 32 * kEpiWarps);
      if ((int)*landed != splits - 1) continue;
      __threadfence();
      const float* first = p.partials + (((size_t)t * splits) * 2 + rank) * block +
                           (size_t)(quarter * 8 + group * 4) * 1024 + lane * 4;
      const int64_t row = (int64_t)m_at + lane;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        const int n_at = n0 + half * 64;
        const bool live = m_at < p.m && n_at < p.n;
        if (lane == 0) tma_store_wait_read();  // this warp's previous store has read the slab
        __syncwarp();
        // the 64 columns of every piece, sixteen 16-byte loads in flight per piece
        float x0[32], x1[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) x0[i] = 0.f, x1[i] = 0.f;
#pragma unroll 1
        for (int sp = 0; sp < splits; ++sp) {
          const float* src = first + (size_t)sp * 2 * block + half * 2048;
          float4 f0[8], f1[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            f0[v] = __ldcg(reinterpret_cast<const float4*>(src + v * 128));
            f1[v] = __ldcg(reinterpret_cast<const float4*>(src + 1024 + v * 128));
          }
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            x0[4 * v] += f0[v].x, x0[4 * v + 1] += f0[v].y, x0[4 * v + 2] += f0[v].z, x0[4 * v + 3] += f0[v].w;
            x1[4 * v] += f1[v].x, x1[4 * v + 1] += f1[v].y, x1[4 * v + 2] += f1[v].z, x1[4 * v + 3] += f1[v].w;
          }
        }
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          float(&xs)[32] = hc == 0 ? x0 : x1;
          const int n_c = n_at + hc * 32;
          if (bias != nullptr) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float b8[8];
              load8<T>(bias + n_c + v * 8, n_c + v * 8 < p.n, b8);
#pragma unroll
              for (int i = 0; i < 8; ++i) xs[v * 8 + i] += b8[i];
            }
          }
          act32(xs, p.act);
          if (p.has_scale) {
#pragma unroll
            for (int i = 0; i < 32; ++i) xs[i] *= p.scale;
          }
          if (p.residual != nullptr) {
            const T* rrow = (const T*)p.residual + row * p.ldr + n_c;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float r8[8];
              load8<T>(rrow + v * 8, row < p.m && n_c + v * 8 < p.n, r8);
#pragma unroll
              for (int i = 0; i < 8; ++i) xs[v * 8 + i] += r8[i];
            }
          }
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int c = hc * 4 + c4;  // chunk c of row r sits at (c ^ (r & 7))
            *reinterpret_cast<uint4*>(srow + ((c ^ (lane & 7)) << 4)) =
                make_uint4(Elem<T>::pack(xs[c4 * 8 + 0], xs[c4 * 8 + 1]), Elem<T>::pack(xs[c4 * 8 + 2], xs[c4 * 8 + 3]),
                           Elem<T>::pack(xs[c4 * 8 + 4], xs[c4 * 8 + 5]), Elem<T>::pack(xs[c4 * 8 + 6], xs[c4 * 8 + 7]));
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && live) {
          tma_store_2d(&tmap_c, slab, n_at, m_at);
          tma_store_commit();
        }
      }
    }
  }

  if (warp >= 2 && lane == 0) tma_store_wait_all();
  tc_fence_before();
  __syncthreads();
  // Neither CTA may leave while the other can still signal its barriers or the
  // pair MMAs can still read its shared memory.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <typename T>
int run_sk(const GemmArgs& a, int sms, cudaStream_t s, char* cfg, size_t cfg_len) {
  ParamsSk p{};
  p.m = a.m, p.n = a.n, p.k = a.k;
  p.act = a.act, p.has_scale = a.has_scale, p.scale = a.scale;
  p.bias = a.bias, p.residual = a.residual, p.ldr = a.ldr, p.status = a.status;
  p.tiles_m = (int)((a.m + 2 * BM - 1) / (2 * BM));
  p.tiles_n = (a.n + BN - 1) / BN;
  CUtensorMap ta, tw, tc;
  const int dt = a.dtype;
  if (!make_tmap_2d(&ta, a.a, dt, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM)) return -1;
  if (!make_tmap_2d(&tw, a.w, dt, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldw, BK, BN / 2)) return -1;
  // the output as 32-row x 64-column boxes, one per epilogue warp and store
  if (!make_tmap_2d(&tc, a.c, dt, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, 64, 32)) return -1;
  // the attribute belongs to the device's copy of the kernel: once per device
  static bool attr_seen[64] = {};
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_seen[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tc2_splitk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) !=
        cudaSuccess)
      return -1;
    attr_set = true;
  }
  // workspace: [tiles][2] counters (zeroed on the stream before the launch), then
  // the f32 blocks from the next 256-byte boundary
  const int tiles = p.tiles_m * p.tiles_n;
  p.k_splits = a.k_splits;
  p.counters = (int*)a.workspace;
  const size_t head = ((size_t)tiles * 2 * sizeof(int) + 255) & ~(size_t)255;
  p.partials = (float*)((uint8_t*)a.workspace + head);
  if (cudaMemsetAsync(a.workspace, 0, (size_t)tiles * 2 * sizeof(int), s) != cudaSuccess) return -1;
  const int items = tiles * a.k_splits;
  const int pairs = items < sms / 2 ? items : sms / 2;
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  lc.blockDim = dim3(kThreads, 1, 1);
  lc.dynamicSmemBytes = kSmemBytes;
  lc.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  if (cudaLaunchKernelEx(&lc, gemm_tc2_splitk_kernel<T>, ta, tw, tc, p) != cudaSuccess) return -1;
  if (cfg != nullptr)
    snprintf(cfg, cfg_len, "{bm:%d,bn:%d,bk:%d,stages:%d,gated:0,grid:%d,cta_pair:1,epi_warps:%d,k_splits:%d}", 2 * BM, BN,
             BK, kStages, 2 * pairs, kEpiWarps, a.k_splits);
  return 0;
}

}  // namespace

size_t gemm_splitk_workspace_bytes(int64_t m, int64_t n, int k_splits) {
  if (k_splits <= 1 || m <= 0 || n <= 0) return 0;
  const size_t tiles = (size_t)((m + 2 * BM - 1) / (2 * BM)) * (size_t)((n + BN - 1) / BN);
  const size_t head = (tiles * 2 * sizeof(int) + 255) & ~(size_t)255;
  return head + tiles * (size_t)k_splits * 2 * BM * BN * sizeof(float);
}

// Split-K takes a plain epilogue on tiles of 256 x 256 whose k loop has at least
// one k-block per piece (the reference never splits a gated or rotated GEMM:
// tk/src/kernels/gemm.rs:459-462).
bool gemm_tc2_splitk_covers(const GemmArgs& a) {
  if (a.k_splits <= 1 || a.k_splits > 16) return false;
  if (!gemm_tc_covers(a)) return false;
  if (a.gated || a.rope_cos != nullptr || a.norm_q != nullptr || a.norm_k != nullptr) return false;
  if (a.n < BN || a.m < 2 * BM) return false;
  if ((a.k + BK - 1) / BK < a.k_splits) return false;
  if (a.workspace == nullptr || (reinterpret_cast<uintptr_t>(a.workspace) & 255) != 0) return false;
  return a.workspace_bytes >= gemm_splitk_workspace_bytes(a.m, a.n, a.k_splits);
}

int launch_gemm_tc2_splitk(const GemmArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  if (!gemm_tc2_splitk_covers(a)) return 1;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  return a.dtype == SVODB_BF16 ? run_sk<__nv_bfloat16>(a, sms, s, cfg, cfg_len) : run_sk<__half>(a, sms, s, cfg, cfg_len);
}

}  // namespace svodb
