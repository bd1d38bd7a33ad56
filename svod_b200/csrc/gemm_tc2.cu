// tcgen05 GEMM on CTA pairs (cta_group::2): y = epilogue(x . w^T) for the large
// projections. Same contract and epilogue order as gemm_tc.cu
// (tk/src/kernels/gemm.rs:605-651: +bias -> act -> *up -> *scale -> +residual ->
// one rounding); what changes is who loads what:
//
//   cluster of 2 CTAs = one 256-row x 256-column accumulator tile. Each CTA
//   loads its own 128 rows of A and HALF of the W tile (128 of its 256 rows), so
//   a k-block costs each SM 32 KiB of operand traffic from L2 instead of 48 KiB;
//   the even CTA's MMA warp issues `tcgen05.mma.cta_group::2` (M = 256), which
//   reads both CTAs' shared memory and writes 128 accumulator rows into each
//   CTA's tensor memory. Both CTAs run the staged TMA-store epilogue on their
//   own rows.
//
// Barriers: `full` lives in the even CTA and counts the bytes of both CTAs'
// loads (the loads are plain, non-multicast TMA with the pair qualifier, which
// lets their completion be counted on the partner's barrier); `empty` and
// `acc_full` exist in both CTAs and are signalled by one tcgen05.commit each;
// `acc_empty` lives in the even CTA and collects the epilogue warps of both.
// Every mbarrier wait is bounded; the two cluster barriers are reached by every
// thread of both CTAs on every path.
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
// Epilogue warps per CTA: 8 (two groups of four, 128 accumulator columns each)
// or, where the epilogue math is heavy (an activation on a plain projection), 16
// (four groups, 64 columns each) so that it stays shorter than the k loop.
constexpr int kStageBytes = (BM + BN / 2) * BK * 2;  // A 16 KiB + this CTA's half of W 16 KiB
constexpr int kGroupStaging = 128 * 128;  // one 128-row x 64-column sub-tile per epilogue group
constexpr int kTableBytes = 2 * 128 * 128;  // head variant: this CTA's 128 rows of cos and of sin
constexpr int kTmemCols = 512;
// The head variant (attention prologue in the store) gives one pipeline stage up
// for the rotation tables.
template <bool HEADS, int EW>
struct Cfg2 {
  static constexpr int kGroups = EW / 4;
  static constexpr int kThreads = 32 * (2 + EW);
  static constexpr int kStagingBytes = kGroups * kGroupStaging;
  static constexpr int kStages = (HEADS || EW == 16) ? 5 : 6;
  // sixteen-warp variant: the bias of a group's 64 columns, three tiles deep
  static constexpr int kBiasBytes = EW == 16 ? 3 * kGroups * 128 : 0;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + kStagingBytes + (HEADS ? kTableBytes : 0) +
                                       1024 /*align*/ + 256 /*barriers*/ + (HEADS ? 1024 : 0) /*norm weights*/ +
                                       kBiasBytes;
  static_assert(kSmemBytes <= 232448, "beyond the 227 KiB a CTA may hold");
};

struct Params2 {
  int64_t m;
  int n, k;
  int tiles_m, tiles_n;  // pair tiles: 256 rows x out_bn columns
  int out_bn;            // 256, or 128 when gated
  int gated;
  int act;
  int has_scale;
  float scale;
  const void* bias;
  const void* residual;
  uint32_t* status;
  // head variant: per-head RMSNorm (weights norm_q below norm_q_cols, norm_k
  // below norm_cols) and rotation (columns below rope_width) of 128-wide heads
  const void* norm_q;
  const void* norm_k;
  int norm_q_cols, norm_cols;
  float norm_eps;
  int rope_width;
  int head_dim;      // 128 (norm and/or rotation), or 64 (rotation only)
  int64_t rope_seq;  // table rows; a tile's 128 rows never wrap around it
};

using namespace gemm_parts;

template <typename T, bool HEADS, int EW>
__global__ void __launch_bounds__(32 * (2 + EW), 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_r,
                    const __grid_constant__ CUtensorMap tmap_cos, const __grid_constant__ CUtensorMap tmap_sin,
                    const Params2 p) {
  using C = Cfg2<HEADS, EW>;
  constexpr int S = C::kStages;
  constexpr int kEpiWarps = EW;
  constexpr int kStagingBytes = C::kStagingBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + (size_t)S * kStageBytes;  // [2 halves][128 rows][128 B]
  uint8_t* tables = staging + kStagingBytes;          // head variant: [cos | sin][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(tables + (HEADS ? kTableBytes : 0));
  uint64_t* full = bars;                   // [S]  used in the even CTA
  uint64_t* empty = bars + S;              // [S]  in both CTAs
  uint64_t* acc_full = bars + 2 * S;       // [2]  in both CTAs
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2]  used in the even CTA
  uint64_t* res_full = bars + 2 * S + 4;   // [4 groups] local: residual sub-tile landed in staging
  uint64_t* tab_full = bars + 2 * S + 8;   // local: this tile's table rows landed
  uint64_t* tab_empty = bars + 2 * S + 9;  // local: every epilogue warp has read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 10);
  float* head_w = reinterpret_cast<float*>(bars + 32);  // head variant: [2][128] norm weights as f32

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = the CTA that issues the MMAs
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int num_kb = (p.k + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 2 * kEpiWarps);  // the epilogue warps of both CTAs
    }
    for (int i = 0; i < 4; ++i) mbar_init(&res_full[i], 1);
    mbar_init(tab_full, 1);
    mbar_init(tab_empty, kEpiWarps);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  if (HEADS && threadIdx.x < 256) {
    const T* wsrc = (const T*)(threadIdx.x < 128 ? p.norm_q : p.norm_k);
    head_w[threadIdx.x] = wsrc != nullptr ? Elem<T>::to_f(wsrc[threadIdx.x & 127]) : 1.0f;
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
      uint32_t tab_ph = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += pairs) {
        int mt, nt;
        tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
        const int m0 = mt * 2 * BM + (int)rank * BM;
        const int n0 = nt * p.out_bn;
        // this CTA's 128 rows of the W tile: the lower / upper half of a plain
        // tile's 256 rows; the gate rows / the up rows of a gated tile
        const int w_row = p.gated ? (rank == 0 ? n0 : p.n + n0) : n0 + (int)rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
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
        if (HEADS && ok && n0 < p.rope_width) {
          // The rotation tables of this CTA's 128 rows, whole 128-byte rows by TMA
          // (per-row 16-byte reads of them would compete with the operand stream).
          // Issued after the tile's operands: the previous tile's epilogue has had
          // the whole k loop to finish with the buffer.
          if (!mbar_wait(tab_empty, tab_ph ^ 1, p.status)) {
            ok = false;
            break;
          }
          tab_ph ^= 1;
          const int row0 = (int)((int64_t)m0 % p.rope_seq);
          mbar_expect_tx(tab_full, (uint32_t)(p.head_dim == 64 ? kTableBytes / 2 : kTableBytes));
          const int tab_row = p.head_dim == 64 ? row0 / 2 : row0;  // 64-wide heads: two positions per map row
          tma_load_2d(tables, &tmap_cos, tab_full, 0, tab_row);
          tma_load_2d(tables + kTableBytes / 2, &tmap_sin, tab_full, 0, tab_row);
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
      for (int t = pair; t < num_tiles && ok; t += pairs) {
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
          const uint64_t a_desc = desc0 + (uint64_t)((s * kStageBytes) >> 4);
          const uint64_t b_desc = a_desc + (uint64_t)((BM * BK * 2) >> 4);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            if (leader)
              umma_ss_pair(d_tmem, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)(k4 * 2), idesc,
                           (kb | k4) != 0 ? 1u : 0u);
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
  } else if constexpr (EW == 16) {
    // ---------------- epilogue, sixteen warps (both CTAs, each its 128 rows) ----------------
    // Bias -> activation -> scale, no residual, no gate. Each warp owns 32 rows x 64
    // columns of the tile and shares nothing with the others but the accumulator:
    // it reads both 32-column halves from tensor memory at once, hands the
    // accumulator back to the MMA warp as soon as they are in registers, and stores
    // its own 32-row slab by TMA, so no warp waits for a slower one.
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int group = ew >> 2;
    const T* bias = (const T*)p.bias;
    uint8_t* bias_slots = reinterpret_cast<uint8_t*>(bars) + 256;  // [3 tiles][4 groups][128 B]
    uint8_t* slab = staging + group * kGroupStaging + quarter * (32 * 128);
    uint8_t* srow = slab + lane * 128;
    int as = 0;
    uint32_t aph = 0;
    int slot = 0;
    for (int t = pair; t < num_tiles; t += pairs) {
      int mt, nt;
      tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
      const int m_at = mt * 2 * BM + (int)rank * BM + quarter * 32;
      const int n_at = nt * BN + group * 64;
      const bool live = m_at < p.m && n_at < p.n;
      // The group's 64 bias values go to shared memory before the accumulator is
      // waited for (their latency hides behind the wait). The four warps of a
      // group write the same bytes; a slot is reused every third tile, which the
      // accumulator hand-over below keeps apart from any warp still reading it.
      uint8_t* bslot = bias_slots + (slot * 4 + group) * 128;
      if (bias != nullptr) {
        const int c = n_at + 2 * lane;
        *reinterpret_cast<uint32_t*>(bslot + 4 * lane) =
            (live && c < p.n) ? __ldg(reinterpret_cast<const uint32_t*>(bias + c)) : 0u;
      }
      if (!mbar_wait(&acc_full[as], aph, p.status)) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (uint32_t)(as * BN + group * 64) + ((uint32_t)(quarter * 32) << 16);
      uint32_t r0[32], r1[32];
      tmem_ld32(t_acc, r0);
      tmem_ld32(t_acc + 32u, r1);
      tmem_ld_wait_for(r0);
      tmem_ld_wait_for(r1);
      __syncwarp();  // the slot's bytes are visible to every lane
      float x0[32], x1[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) x0[i] = __uint_as_float(r0[i]), x1[i] = __uint_as_float(r1[i]);
      if (bias != nullptr) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 b0 = *reinterpret_cast<const uint4*>(bslot + v * 16);
          const uint4 b1 = *reinterpret_cast<const uint4*>(bslot + 64 + v * 16);
          const uint32_t u0[4] = {b0.x, b0.y, b0.z, b0.w};
          const uint32_t u1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f0 = Elem<T>::unpack(u0[i]);
            const float2 f1 = Elem<T>::unpack(u1[i]);
            x0[v * 8 + 2 * i] += f0.x, x0[v * 8 + 2 * i + 1] += f0.y;
            x1[v * 8 + 2 * i] += f1.x, x1[v * 8 + 2 * i + 1] += f1.y;
          }
        }
      }
      // This warp has read the accumulator and the bias slot: one arrival on the
      // even CTA's barrier, from either CTA.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(cluster_map(&acc_empty[as], 0));
        tma_store_wait_read();  // this warp's previous store has read the slab
      }
      __syncwarp();
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        float(&xs)[32] = hc == 0 ? x0 : x1;
        act32(xs, p.act);
        if (p.has_scale) {
#pragma unroll
          for (int i = 0; i < 32; ++i) xs[i] *= p.scale;
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
        tma_store_2d(&tmap_r, slab, n_at, m_at);  // the 32-row view of the output
        tma_store_commit();
      }
      if (++as == 2) {
        as = 0;
        aph ^= 1;
      }
      if (++slot == 3) slot = 0;
    }
  } else {
    // ---------------- epilogue (both CTAs, each its 128 rows) ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int chalf = ew >> 2;  // epilogue group: which slice of the tile's output columns
    const T* bias = (const T*)p.bias;
    int as = 0;
    uint32_t aph = 0;
    uint32_t res_phase = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += pairs) {
      int mt, nt;
      tile_coords(t, p.tiles_m, p.tiles_n, mt, nt);
      const int n0 = nt * p.out_bn;
      const int cols = p.out_bn / C::kGroups;
      const int c_lo = chalf * cols;
      uint8_t* stg = staging + chalf * kGroupStaging;
      const bool chief = (ew & 3) == 0 && lane == 0;
      const int m0 = mt * 2 * BM + (int)rank * BM;
      const bool rows_live = m0 < p.m;  // a ragged last tile may leave the odd CTA no row
      if constexpr (!HEADS) {
        // The residual of the group's first sub-tile is fetched into the staging
        // buffer while the tile is still being accumulated (the buffer is free as
        // soon as the previous tile's store has read it), so that its latency
        // does not sit between the accumulator and the store.
        const int n_first = rows_live ? n0 + c_lo : p.n;
        if (p.residual != nullptr && chief && n_first < p.n) {
          tma_store_wait_read();
          mbar_expect_tx(&res_full[chalf], 128 * 128);
          tma_load_2d(stg, &tmap_r, &res_full[chalf], n_first, m0);
        }
      }
      if (!mbar_wait(&acc_full[as], aph, p.status)) {
        // leave only after the residual copy in flight (if any) has landed or timed out
        if constexpr (!HEADS) {
          if (p.residual != nullptr && rows_live && n0 + c_lo < p.n) mbar_wait(&res_full[chalf], res_phase, p.status);
        }
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (uint32_t)(as * BN) + ((uint32_t)(quarter * 32) << 16);
      const int r_tile = quarter * 32 + lane;
      if constexpr (HEADS) {
       if (p.head_dim == 64) {
        // 64-wide heads, rotation only: a head is one 64-column sub-tile, its two
        // 32-column halves are partners. Table rows are 64 bytes here, two to a
        // 128-byte line of the slab (128-byte swizzle over those lines).
        const bool tile_tables = n0 < p.rope_width;
        if (tile_tables) {
          if (!mbar_wait(tab_full, res_phase, p.status)) ok = false;
          res_phase ^= 1;
        }
        const uint8_t* cline = tables + (r_tile >> 1) * 128;
        const uint8_t* nline = cline + kTableBytes / 2;
        const int half_sel = (r_tile & 1) << 2, line_x = (r_tile >> 1) & 7;
        uint8_t* srow = stg + r_tile * 128;
        for (int sub = 0; sub < 2; ++sub) {
          const int h_col = n0 + c_lo + sub * 64;
          const bool turned = h_col < p.rope_width;
          const uint32_t t_head = t_acc + (uint32_t)(c_lo + sub * 64);
          if (chief) tma_store_wait_read();
          named_barrier(1 + chalf, 128);
          uint32_t ra[32], rb[32];
          tmem_ld32(t_head, ra);
          tmem_ld32(t_head + 32u, rb);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float a[8], b[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              a[i] = __uint_as_float(ra[v * 8 + i]);
              b[i] = __uint_as_float(rb[v * 8 + i]);
            }
            if (turned) {
              const int at = ((half_sel | v) ^ line_x) << 4;
              const uint4 c4 = *reinterpret_cast<const uint4*>(cline + at);
              const uint4 s4 = *reinterpret_cast<const uint4*>(nline + at);
              const uint32_t cu[4] = {c4.x, c4.y, c4.z, c4.w};
              const uint32_t su[4] = {s4.x, s4.y, s4.z, s4.w};
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
            *reinterpret_cast<uint4*>(srow + ((v ^ (r_tile & 7)) << 4)) =
                make_uint4(Elem<T>::pack(a[0], a[1]), Elem<T>::pack(a[2], a[3]), Elem<T>::pack(a[4], a[5]),
                           Elem<T>::pack(a[6], a[7]));
            *reinterpret_cast<uint4*>(srow + (((4 + v) ^ (r_tile & 7)) << 4)) =
                make_uint4(Elem<T>::pack(b[0], b[1]), Elem<T>::pack(b[2], b[3]), Elem<T>::pack(b[4], b[5]),
                           Elem<T>::pack(b[6], b[7]));
          }
          fence_proxy_async_smem();
          named_barrier(1 + chalf, 128);
          if (chief && rows_live && h_col < p.n) {
            tma_store_2d(&tmap_c, stg, h_col, m0);
            tma_store_commit();
          }
        }
        if (tile_tables) {
          // this warp has read its table rows
          __syncwarp();
          if (lane == 0) mbar_arrive(tab_empty);
        }
       } else {
        // One 128-column head per column half: sum of squares over the head, then
        // both halves of the head at once (a rotated column needs its partner 64
        // columns away); the first half goes to the staging buffer, the second
        // waits packed in registers until the first sub-tile's store has read it.
        const int h_col = n0 + c_lo;
        const bool tile_tables = n0 < p.rope_width;
        const bool turned = h_col < p.rope_width;
        const float* nw = h_col < p.norm_q_cols ? head_w : (h_col < p.norm_cols ? head_w + 128 : nullptr);
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
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              ss0 = fmaf(__uint_as_float(r0[i]), __uint_as_float(r0[i]), ss0);
              ss1 = fmaf(__uint_as_float(r1[i]), __uint_as_float(r1[i]), ss1);
            }
          }
          inv = rsqrtf((ss0 + ss1) * (1.0f / 128.0f) + p.norm_eps);
        }
        if (tile_tables) {
          if (!mbar_wait(tab_full, res_phase, p.status)) ok = false;
          res_phase ^= 1;  // the head variant has no residual: the phase bit serves the tables
        }
        if (chief) tma_store_wait_read();
        named_barrier(1 + chalf, 128);
        uint8_t* srow = stg + r_tile * 128;
        const uint8_t* crow = tables + r_tile * 128;
        const uint8_t* nrow = crow + kTableBytes / 2;
        uint32_t keep[32];
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          uint32_t ra[32], rb[32];
          tmem_ld32(t_head + (uint32_t)(32 * hc), ra);
          tmem_ld32(t_head + (uint32_t)(64 + 32 * hc), rb);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int chunk = hc * 4 + v;  // 16-byte chunk of a 64-column row
            float a[8], b[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              a[i] = __uint_as_float(ra[v * 8 + i]);
              b[i] = __uint_as_float(rb[v * 8 + i]);
            }
            if (nw != nullptr) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                a[i] = a[i] * inv * nw[32 * hc + v * 8 + i];
                b[i] = b[i] * inv * nw[64 + 32 * hc + v * 8 + i];
              }
            }
            if (turned) {
              const uint4 c4 = *reinterpret_cast<const uint4*>(crow + ((chunk ^ (r_tile & 7)) << 4));
              const uint4 s4 = *reinterpret_cast<const uint4*>(nrow + ((chunk ^ (r_tile & 7)) << 4));
              const uint32_t cu[4] = {c4.x, c4.y, c4.z, c4.w};
              const uint32_t su[4] = {s4.x, s4.y, s4.z, s4.w};
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
            *reinterpret_cast<uint4*>(srow + ((chunk ^ (r_tile & 7)) << 4)) =
                make_uint4(Elem<T>::pack(a[0], a[1]), Elem<T>::pack(a[2], a[3]), Elem<T>::pack(a[4], a[5]),
                           Elem<T>::pack(a[6], a[7]));
#pragma unroll
            for (int i = 0; i < 4; ++i) keep[chunk * 4 + i] = Elem<T>::pack(b[2 * i], b[2 * i + 1]);
          }
        }
        if (tile_tables) {
          // this warp has read its table rows
          __syncwarp();
          if (lane == 0) mbar_arrive(tab_empty);
        }
        fence_proxy_async_smem();
        named_barrier(1 + chalf, 128);
        const bool live = rows_live && h_col < p.n;
        if (chief && live) {
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
        if (chief && live && h_col + 64 < p.n) {
          tma_store_2d(&tmap_c, stg, h_col + 64, m0);
          tma_store_commit();
        }
       }
      } else
      for (int sub = 0; sub < cols / 64; ++sub) {
        const int c0 = c_lo + sub * 64;
        const int n_at = rows_live ? n0 + c0 : p.n;  // past N: nothing is loaded or stored
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
      // This warp's TMEM reads of the tile are complete: one arrival on the even
      // CTA's barrier, from either CTA.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_map(&acc_empty[as], 0));
      if (++as == 2) {
        as = 0;
        aph ^= 1;
      }
    }
  }

  if (warp >= 2 && lane == 0) tma_store_wait_all();  // whoever issued stores; a no-op for the others
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

template <typename T, bool HEADS, int EW>
int run2(const GemmArgs& a, int sms, cudaStream_t s, char* cfg, size_t cfg_len) {
  using C = Cfg2<HEADS, EW>;
  Params2 p{};
  p.m = a.m, p.n = a.n, p.k = a.k;
  p.gated = a.gated, p.act = a.act, p.has_scale = a.has_scale, p.scale = a.scale;
  p.bias = a.bias, p.residual = a.residual, p.status = a.status;
  p.out_bn = a.gated ? BN / 2 : BN;
  p.tiles_m = (int)((a.m + 2 * BM - 1) / (2 * BM));
  p.tiles_n = (a.n + p.out_bn - 1) / p.out_bn;
  CUtensorMap ta, tw, tc, tr;
  const int dt = a.dtype;
  if (!make_tmap_2d(&ta, a.a, dt, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM)) return -1;
  const uint64_t w_rows = (uint64_t)(a.gated ? 2 * a.n : a.n);
  if (!make_tmap_2d(&tw, a.w, dt, (uint64_t)a.k, w_rows, (uint64_t)a.ldw, BK, BN / 2)) return -1;
  if (!make_tmap_2d(&tc, a.c, dt, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, 64, BM)) return -1;
  tr = tc;
  // sixteen epilogue warps: the residual's slot carries the output again, as 32-row boxes
  if (EW == 16 && !make_tmap_2d(&tr, a.c, dt, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, 64, 32)) return -1;
  if (EW != 16 && a.residual != nullptr && !make_tmap_2d(&tr, a.residual, dt, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldr, 64, BM))
    return -1;
  CUtensorMap tcos = tc, tsin = tc;
  if (HEADS) {
    p.norm_q = a.norm_q, p.norm_k = a.norm_k;
    p.norm_q_cols = a.norm_q != nullptr ? a.norm_q_heads * 128 : 0;
    p.norm_cols = a.norm_k != nullptr ? (a.norm_q_heads + a.norm_k_heads) * 128 : p.norm_q_cols;
    p.norm_eps = a.norm_eps;
    p.head_dim = a.rope_cos != nullptr && a.rope_head_dim == 64 ? 64 : 128;
    p.rope_width = a.rope_cos != nullptr ? a.rope_heads * p.head_dim : 0;
    p.rope_seq = a.rope_seq > 0 ? a.rope_seq : 1;
    if (a.rope_cos != nullptr) {
      // [rope_seq rows, head_dim/2 columns] tables, one 128-position slab per CTA and
      // tile. 64-wide heads have 64-byte table rows: the map views two positions as
      // one 128-byte row, so the slab keeps the 128-byte-row swizzle.
      const uint64_t per_row = p.head_dim == 64 ? 2 : 1;
      if (!make_tmap_2d(&tcos, a.rope_cos, dt, 64, (uint64_t)p.rope_seq / per_row, 64, 64, BM / (uint32_t)per_row)) return -1;
      if (!make_tmap_2d(&tsin, a.rope_sin, dt, 64, (uint64_t)p.rope_seq / per_row, 64, 64, BM / (uint32_t)per_row)) return -1;
    }
  }
  // the attribute belongs to the device's copy of the kernel: once per device
  static bool attr_seen[64] = {};
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_seen[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tc2_kernel<T, HEADS, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)C::kSmemBytes) != cudaSuccess)
      return -1;
    attr_set = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  lc.blockDim = dim3(C::kThreads, 1, 1);
  lc.dynamicSmemBytes = C::kSmemBytes;
  lc.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  if (cudaLaunchKernelEx(&lc, gemm_tc2_kernel<T, HEADS, EW>, ta, tw, tc, tr, tcos, tsin, p) != cudaSuccess) return -1;
  if (cfg != nullptr)
    snprintf(cfg, cfg_len, "{bm:%d,bn:%d,bk:%d,stages:%d,gated:%d,grid:%d,cta_pair:1,epi_warps:%d}", 2 * BM, BN, BK,
             C::kStages, a.gated, 2 * pairs, EW);
  return 0;
}

int sm_count2() {
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

// The pair kernel takes what the one-CTA kernel covers once the problem has at
// least one 256 x 256 tile per CTA pair; per-head stores only for 128-wide heads
// without a bias whose table rows never wrap inside a tile (the rest stays on the
// one-CTA kernel).
bool gemm_tc2_covers(const GemmArgs& a) {
  if (!gemm_tc_covers(a)) return false;
  const bool heads = a.rope_cos != nullptr || a.norm_q != nullptr || a.norm_k != nullptr;
  if (heads) {
    // 128-wide heads (norm and/or rotation), or 64-wide heads with a rotation only
    const bool wide64 = a.rope_head_dim == 64 && a.rope_cos != nullptr && a.norm_q == nullptr && a.norm_k == nullptr;
    if ((a.rope_head_dim != 128 && !wide64) || a.bias != nullptr) return false;
    if (a.rope_cos != nullptr && (a.rope_seq <= 0 || a.rope_seq % BM != 0)) return false;
  }
  const int out_bn = a.gated ? BN / 2 : BN;
  if (a.n < out_bn || a.m < 2 * BM) return false;
  const int64_t tiles = ((a.m + 2 * BM - 1) / (2 * BM)) * ((a.n + out_bn - 1) / out_bn);
  return tiles >= sm_count2() / 2;
}

// Where the pair kernel is the default: from K = 512 on (measured at K = 512 /
// 768: plain 980 vs 740 and 1446 vs 1167 TFLOP/s, gated 1425 vs 1240); a config
// store may still choose either kernel per shape.
bool gemm_tc2_preferred(const GemmArgs& a) {
  if (!gemm_tc2_covers(a)) return false;
  return a.k >= 512;
}

int launch_gemm_tc2(const GemmArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  if (!gemm_tc2_covers(a)) return 1;
  const int sms = sm_count2();
  const bool heads = a.rope_cos != nullptr || a.norm_q != nullptr || a.norm_k != nullptr;
  // sixteen epilogue warps where each output value costs an activation
  // (long k loops hide the epilogue anyway and prefer the deeper ring of the eight-warp variant;
  // measured: a residual alone does not pay for them)
  const bool wide = !heads && !a.gated && a.act != kActNone && a.residual == nullptr && a.k <= 2048;
  if (a.dtype == SVODB_BF16)
    return heads  ? run2<__nv_bfloat16, true, 8>(a, sms, s, cfg, cfg_len)
           : wide ? run2<__nv_bfloat16, false, 16>(a, sms, s, cfg, cfg_len)
                  : run2<__nv_bfloat16, false, 8>(a, sms, s, cfg, cfg_len);
  return heads  ? run2<__half, true, 8>(a, sms, s, cfg, cfg_len)
         : wide ? run2<__half, false, 16>(a, sms, s, cfg, cfg_len)
                : run2<__half, false, 8>(a, sms, s, cfg, cfg_len);
}

}  // namespace svodb
