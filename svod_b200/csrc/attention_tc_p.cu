// Persistent form of the tcgen05 flash-attention forward (attention_tc.cu): one
// CTA per SM walks a queue of (256 query rows, head, batch) work items instead
// of one item per CTA, so that an item's fixed costs — launch, barrier and TMEM
// set-up, the first Q/K/V round trip, the pipeline ramp, the O read-out and
// store — overlap the neighbouring items' work instead of adding to it. With
// one CTA per SM (shared memory and tensor memory are both full) nothing else
// can overlap them: at 4096 keys they are about a fifth of a causal item.
//
// Same math, same roles and the same TMEM / shared-memory layout as the
// one-item kernel (see its header). What changes:
//   * a work queue: the loader takes the next item off an atomic counter and
//     publishes it through a two-slot ring (`item_full` / `item_empty`); items
//     are ordered so that CTAs running together share K/V in L2 (batch, KV head,
//     then query tiles from the heaviest) and the light tiles come last;
//   * every barrier phase comes from running counters (blocks loaded, blocks
//     per tile, tail commits, live items per tile) instead of the block index
//     inside one item;
//   * `q_empty` (the issuer's last QK of an item frees the Q tile for the
//     loader) and `o_empty` (the softmax warps have read O out, the next item's
//     first P.V may overwrite it): the loader and the issuers run into the next
//     item while the softmax warps still finish the last one.
// A bool key mask needs no CTA-wide scan here: the loader warp scans the mask row
// of its item's batch lane (once per change of lane); the softmax gathers the
// bits of a block's keys with a ballot. The loader also works out each item's
// key-block ranges (`Work`) once and publishes them with the item, so that the
// issuers and the softmax warps start an item by reading 80 bytes.
#include <cuda.h>
#include <math.h>
#include <stdio.h>

#include <map>
#include <mutex>
#include <utility>

#include "attention_parts.cuh"
#include "common.cuh"
#include "kernels.h"
#include "svodb.h"
#include "tensormap.h"

namespace svodb {

namespace {

using namespace fa_parts;

// Queue heads: items handed out so far by a running launch, one per (device,
// stream) pair, zeroed on the stream just before each launch.
constexpr int kQueueSlots = 256;
// Output staging of the softmax warps: a 32-row x 64-column slab each, stored by TMA.
constexpr int kOutStageBytes = 8 * 32 * 128;
template <int D>
constexpr size_t smem_bytes_p() {
  using C = FaCfg<D>;
  return 1024 + (size_t)2 * C::kQTileBytes + (size_t)2 * C::kStages * C::kKvBytes + kOutStageBytes + 512;
}
__device__ int g_next_item[kQueueSlots];

struct Item {
  int qt, h, b, valid;
  int split;  // key split of this item (0 without splits)
};

// Work item w in queue order: batch, KV head, query head of the group (or head
// pair, when an item is one tile of two heads: `heads` then counts pairs), then
// query tile pairs from the last (the heaviest under a causal mask) to the first,
// so that the items in flight at one time share few KV heads and their keys stay
// in L2. The last `tail_groups` (batch, KV head) groups are interleaved instead:
// tile pair first (heaviest first), then group, then query head. The queue then
// ends on the lightest items of many groups rather than starting the heaviest
// items of the last group when everything else is done.
__device__ __forceinline__ Item decode_item(int w, int n_items, int n_qt, int heads, int kv_heads, int tail_groups,
                                            int splits) {
  Item it{0, 0, 0, 0, 0};
  if (w >= n_items) return it;
  // the splits of one (tile pair, head, batch) follow one another in the queue
  it.split = w % splits;
  w /= splits;
  n_items /= splits;
  const int group = heads / kv_heads;
  const int per_kv = group * n_qt;
  const int head_groups = n_items / per_kv - tail_groups;
  int kvb, r, q;
  if (w < head_groups * per_kv) {
    kvb = w / per_kv;  // (batch, kv head)
    r = w - kvb * per_kv;
    q = r / group;
    r -= q * group;
  } else {
    const int t = w - head_groups * per_kv;
    const int per_qt = tail_groups * group;
    q = t / per_qt;
    const int r2 = t - q * per_qt;
    kvb = head_groups + r2 / group;
    r = r2 % group;
  }
  it.qt = n_qt - 1 - q;
  it.h = (kvb % kv_heads) * group + r;
  it.b = kvb / kv_heads;
  it.valid = 1;
  return it;
}

// What a bool key mask row says about a batch lane: the keys past `len` are all
// hidden; `general` when hidden keys also lie before it (then the softmax reads
// the row's bits block by block). The loader warp scans the row, all lanes taking
// part, when its item's batch lane changes.
struct MaskRow {
  int64_t b;
  int len;
  int general;
};

__device__ __forceinline__ void scan_mask_row(const FaParams& p, int64_t b, int lane, MaskRow& row) {
  if (row.b == b) return;
  int first_zero = 0x7fffffff, last_set = 0;
  const int64_t base = b * p.tk;
  if (!p.key_mask_i32 && (p.tk & 15) == 0 && (reinterpret_cast<uintptr_t>(p.key_mask) & 15) == 0) {
    // byte masks in 16-byte pieces: per 4-byte word, 0xff for every nonzero byte
    const uint4* row = reinterpret_cast<const uint4*>((const uint8_t*)p.key_mask + base);
    const int pieces = (int)(p.tk >> 4);
    for (int c = lane; c < pieces; c += 32) {
      const uint4 u = __ldg(row + c);
      const uint32_t wd[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t set = __vcmpne4(wd[q], 0u);
        const int at = c * 16 + q * 4;
        if (set != 0u) last_set = max(last_set, at + ((31 - __clz((int)set)) >> 3) + 1);
        if (set != 0xffffffffu) first_zero = min(first_zero, at + ((__ffs((int)~set) - 1) >> 3));
      }
    }
  } else {
    for (int64_t j = lane; j < p.tk; j += 32) {
      const int m = p.key_mask_i32 ? ((const int32_t*)p.key_mask)[base + j] : (int)((const uint8_t*)p.key_mask)[base + j];
      if (m != 0) last_set = (int)j + 1;
      else if ((int)j < first_zero) first_zero = (int)j;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    first_zero = min(first_zero, __shfl_xor_sync(0xffffffffu, first_zero, o));
    last_set = max(last_set, __shfl_xor_sync(0xffffffffu, last_set, o));
  }
  row.b = b;
  row.len = last_set;
  row.general = first_zero < last_set ? 1 : 0;
}

// What every role derives from an item: the key-block ranges of its two tiles.
// The loader works it out once per item and publishes it with the item.
struct Work {
  int valid;
  int h, hk, split;
  int b, i0;         // batch lane, first query row of the item (both below 2^31); tile i covers rows
                     // i0 + i*128 of head h, or with paired heads rows i0 of head h + i
  int len, general;  // the mask context (`Ctx`): visible key bound, whether to consult the bitmask
  Range r0, r1;
  int u_lo, u_hi;    // the union of the two ranges: the blocks the loader brings
};

// The read-out of one tile's O by one softmax warp (32 rows): 64 columns at a time
// through the warp's slab — both 32-column halves read from tensor memory at once,
// scaled by 1/l, packed into the swizzled rows (16-byte chunk c of row r at
// c ^ (r & 7)) — and one TMA store per 64 columns, which writes whole 128-byte
// lines and cuts rows past T and columns past the real head dim by itself. Not
// inlined: the block loop's registers and schedule stay what they are without it.
template <typename T, int D>
__device__ __noinline__ void store_o_slab(uint32_t o_tmem, float inv, uint8_t* slab, int lane, const CUtensorMap* tmap_o,
                                          int h, int row0, int b, int d_real, bool rows_live) {
  uint8_t* srow = slab + lane * 128;
#pragma unroll 1
  for (int c = 0; c < D; c += 64) {
    uint32_t oa[32], ob[32];
    tmem_ld32(o_tmem + c, oa);
    tmem_ld32(o_tmem + c + 32, ob);
    if (lane == 0) tma_store_wait_read();  // the slab's previous store has read it
    __syncwarp();
    tmem_ld_wait_for(oa);
    tmem_ld_wait_for(ob);
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      uint32_t wv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = (v & 3) * 8 + 2 * e;
        wv[e] = v < 4 ? Elem<T>::pack(__uint_as_float(oa[k]) * inv, __uint_as_float(oa[k + 1]) * inv)
                      : Elem<T>::pack(__uint_as_float(ob[k]) * inv, __uint_as_float(ob[k + 1]) * inv);
      }
      *reinterpret_cast<uint4*>(srow + ((v ^ (lane & 7)) << 4)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && rows_live && c < d_real) {
      tma_store_4d(tmap_o, slab, c, h, row0, b);
      tma_store_commit();
    }
  }
}

// EXTRAS = key splits and / or an additive bias: a separate instantiation, so that
// the plain kernel's inner loop carries neither their registers nor their branches.
template <typename T, int D, bool EXTRAS>
__global__ void __launch_bounds__(kThreadsFa, 1)
    attention_tc_p_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                          const FaParams p, const int n_items,
                          const int tail_groups, int* const queue) {
  using C = FaCfg<D>;
  constexpr int S = C::kStages;
  constexpr int QB = C::kQTileBytes;
  constexpr int KB = C::kKvBytes;
  constexpr int KBOX = kBKV * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                         // [2][QB]
  uint8_t* k_s = q_s + 2 * QB;                 // [S][KB]
  uint8_t* v_s = k_s + S * KB;                 // [S][KB]
  uint8_t* o_stage = v_s + S * KB;             // [8 softmax warps][32 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(o_stage + kOutStageBytes);
  uint64_t* q_full = bars;                     // [2]
  uint64_t* q_empty = bars + 2;                // [2]
  uint64_t* k_full = bars + 4;                 // [S]
  uint64_t* k_empty = k_full + S;
  uint64_t* v_full = k_empty + S;
  uint64_t* v_empty = v_full + S;
  uint64_t* s_full = v_empty + S;              // [2 tiles][2 buffers]
  uint64_t* p_full = s_full + 4;               // [2 tiles][2 buffers]
  uint64_t* tail_done = p_full + 4;            // [2 tiles]
  uint64_t* o_empty = tail_done + 2;           // [2 tiles]
  uint64_t* item_full = o_empty + 2;           // [2 slots]
  uint64_t* item_empty = item_full + 2;        // [2 slots]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(item_empty + 2);
  Work* item_ring = reinterpret_cast<Work*>(tmem_slot + 4);  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&tail_done[i], 1);
      mbar_init(&o_empty[i], 4);      // the tile's four softmax warps
      mbar_init(&item_full[i], 1);
      mbar_init(&item_empty[i], 10);  // two issuers + eight softmax warps
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    for (int i = 0; i < S; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto plan = [&](const Item& it, const MaskRow& mrow) -> Work {
    Work w;
    w.valid = it.valid;
    w.h = p.pair_heads ? 2 * it.h : it.h;
    w.hk = w.h / (p.heads / p.kv_heads);
    w.b = it.b;
    w.i0 = it.qt * (p.pair_heads ? kBQ : 2 * kBQ);
    Ctx ctx;
    ctx.len = p.tk;
    ctx.general_mask = 0;
    if (p.key_lens != nullptr) {
      const int64_t kl = p.key_lens[it.b];
      ctx.len = kl < 0 ? 0 : (kl < ctx.len ? kl : ctx.len);
    }
    if (p.key_mask != nullptr) {
      ctx.general_mask = mrow.general;
      if (mrow.len < ctx.len) ctx.len = mrow.len;
    }
    w.len = (int)ctx.len;
    w.general = ctx.general_mask;
    w.r0 = tile_range(p, ctx, w.b, w.i0);
    w.r1 = tile_range(p, ctx, w.b, (int64_t)w.i0 + (p.pair_heads ? 0 : kBQ));
    w.split = it.split;
    if (EXTRAS && p.splits > 1) {
      // this split's share of the key blocks
      const int total = (int)((p.tk + kBKV - 1) / kBKV);
      const int per = (total + p.splits - 1) / p.splits;
      const int s_lo = it.split * per, s_hi = s_lo + per;
      w.r0.lo = max(w.r0.lo, s_lo), w.r0.hi = min(w.r0.hi, s_hi);
      w.r1.lo = max(w.r1.lo, s_lo), w.r1.hi = min(w.r1.hi, s_hi);
      if (w.r0.hi <= w.r0.lo) w.r0 = Range{0, 0};
      if (w.r1.hi <= w.r1.lo) w.r1 = Range{0, 0};
    }
    const bool live0 = w.r0.hi > w.r0.lo, live1 = w.r1.hi > w.r1.lo;
    w.u_lo = 0, w.u_hi = 0;
    if (live0 && live1) {
      w.u_lo = w.r0.lo < w.r1.lo ? w.r0.lo : w.r1.lo;
      w.u_hi = w.r0.hi > w.r1.hi ? w.r0.hi : w.r1.hi;
    } else if (live0) {
      w.u_lo = w.r0.lo, w.u_hi = w.r0.hi;
    } else if (live1) {
      w.u_lo = w.r1.lo, w.u_hi = w.r1.hi;
    }
    return w;
  };

  if (warp < 4) {
    // 4 warps x 72 + 8 warps x 216 registers = the 384 x 168 the CTA was launched
    // with: a larger request here would leave the softmax warps' increase waiting
    // for registers that never come.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0) {
      // ---------------- scheduler + TMA loader ----------------
      // The whole warp walks the queue (a key mask row is scanned by all lanes);
      // lane 0 takes the items, publishes them and issues the copies.
      {
        int s = 0;
        uint32_t ph = 0;
        uint32_t q_items[2] = {0, 0};  // live items so far, per tile
        bool ok = true;
        MaskRow mrow{-1, 0, 0};
        for (uint32_t n_it = 0; ok; ++n_it) {
          const int slot = (int)(n_it & 1);
          int wi = -1;
          if (lane == 0 && mbar_wait(&item_empty[slot], ((n_it >> 1) & 1) ^ 1, p.status)) wi = atomicAdd(queue, 1);
          wi = __shfl_sync(0xffffffffu, wi, 0);
          if (wi < 0) break;  // the wait ran out
          Item it = decode_item(wi, n_items, p.n_qt, p.pair_heads ? p.heads / 2 : p.heads, p.kv_heads, tail_groups,
                                EXTRAS ? p.splits : 1);
          // The loader alone scans a bool key mask row (all its lanes, once per change
          // of batch lane, while it runs ahead of the other warps) and hands what it
          // found to them with the item.
          if (it.valid && p.key_mask != nullptr) scan_mask_row(p, it.b, lane, mrow);
          Work w{};
          if (it.valid) w = plan(it, mrow);
          if (lane == 0) {
            item_ring[slot] = w;
            __threadfence_block();
            mbar_arrive(&item_full[slot]);
          }
          if (!it.valid) break;
          if (w.u_hi <= w.u_lo) continue;
          if (lane == 0) {
          for (int i = 0; i < 2; ++i) {
            if (i == 0 ? w.r0.hi > w.r0.lo : w.r1.hi > w.r1.lo) {
              // the issuer's last QK of the tile's previous live item has read this Q tile
              if (!mbar_wait(&q_empty[i], (q_items[i] & 1) ^ 1, p.status)) {
                ok = false;
                break;
              }
              ++q_items[i];
              mbar_expect_tx(&q_full[i], QB);
              for (int c = 0; c < D / 64; ++c)
                tma_load_4d(q_s + i * QB + c * (128 * 128), &tmap_q, &q_full[i], c * 64, w.h + (p.pair_heads ? i : 0),
                            w.i0 + (p.pair_heads ? 0 : i * kBQ), w.b);
            }
          }
          const int kv_b = p.row_map != nullptr ? p.row_map[w.b] : w.b;
          for (int j = w.u_lo; j < w.u_hi && ok; ++j) {
            if (!mbar_wait(&k_empty[s], ph ^ 1, p.status)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&k_full[s], KB);
            for (int c = 0; c < D / 64; ++c)
              tma_load_4d(k_s + s * KB + c * KBOX, &tmap_k, &k_full[s], c * 64, w.hk, j * kBKV, kv_b);
            if (!mbar_wait(&v_empty[s], ph ^ 1, p.status)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&v_full[s], KB);
            for (int c = 0; c < D / 64; ++c)
              tma_load_4d(v_s + s * KB + c * KBOX, &tmap_v, &v_full[s], c * 64, w.hk, j * kBKV, kv_b);
            if (++s == S) {
              s = 0;
              ph ^= 1;
            }
          }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (!ok) {
          // Error path: give copies in flight a bounded time to land.
          for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
      }
    } else if (warp == 1 || warp == 3) {
      // ---------------- MMA issuers: warp 1 drives tile 0, warp 3 tile 1 ----------------
      const int i = warp == 1 ? 0 : 1;
      const bool leader = elect_one();
      constexpr uint32_t idesc_qk = umma_idesc(Elem<T>::kUmmaFormat, 128, kBKV, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(Elem<T>::kUmmaFormat, 128, D, 0, 1);
      const uint64_t qa = umma_desc_sw128(smem_u32(q_s) + i * QB, 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(k_s), 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(v_s), KBOX, 1024);
      uint32_t kv_blocks = 0;  // K/V blocks of all earlier items (ring position)
      uint32_t my_blocks = 0;  // blocks of this tile in all earlier items (S/P buffer and phase)
      uint32_t my_items = 0;   // live items of this tile so far
      bool ok = true;
      for (uint32_t n_it = 0; ok; ++n_it) {
        const int slot = (int)(n_it & 1);
        if (!mbar_wait(&item_full[slot], (n_it >> 1) & 1, p.status)) break;
        const Work w = item_ring[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(&item_empty[slot]);
        if (!w.valid) break;
        if (w.u_hi <= w.u_lo) continue;
        const Range r = i == 0 ? w.r0 : w.r1;
        const int nblk = r.hi - r.lo;
        const bool live = nblk > 0;
        bool q_ready = false;
        for (int t = w.u_lo - 1; t <= w.u_hi && ok; ++t) {
          const int jq = t + 1;
          const int jp = t - 1;
          const bool have_k = jq >= w.u_lo && jq < w.u_hi;
          const bool have_v = jp >= w.u_lo && jp < w.u_hi;
          const uint32_t kpos = kv_blocks + (uint32_t)(have_k ? jq - w.u_lo : 0);
          const uint32_t vpos = kv_blocks + (uint32_t)(have_v ? jp - w.u_lo : 0);
          const int ks_slot = (int)(kpos % S), vs_slot = (int)(vpos % S);
          const bool do_pv = have_v && jp >= r.lo && jp < r.hi;
          const bool do_qk = have_k && jq >= r.lo && jq < r.hi;
          // Every slot is waited for and released by both issuers, used or not.
          if ((have_k && !mbar_wait(&k_full[ks_slot], (kpos / S) & 1, p.status)) ||
              (have_v && !mbar_wait(&v_full[vs_slot], (vpos / S) & 1, p.status))) {
            ok = false;
            break;
          }
          if (do_pv) {
            const uint32_t n = (uint32_t)(jp - r.lo);
            const uint32_t N = my_blocks + n;  // this tile's running block counter
            if (n == 0 && !mbar_wait(&o_empty[i], (my_items & 1) ^ 1, p.status)) {
              ok = false;  // the previous item's O has not been read out
              break;
            }
            if (!mbar_wait(&p_full[i * 2 + (N & 1)], (N >> 1) & 1, p.status)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + 256 + i * D;
            const uint32_t a_tmem = tmem_base + (uint32_t)((i * 2 + (N & 1)) * kBKV);
            const uint64_t vb = v_desc0 + (uint64_t)((vs_slot * KB) >> 4);
            const uint32_t first = n != 0 ? 1u : 0u;
#pragma unroll
            for (int ks = 0; ks < kBKV / 16; ++ks)
              if (leader)
                umma_ts(d_tmem, a_tmem + ks * 8, vb + (uint64_t)(ks * (2048 >> 4)), idesc_pv,
                        (first | (uint32_t)ks) != 0 ? 1u : 0u);
            if (leader && (int)n + 2 >= nblk) tc_commit(&tail_done[i]);
          }
          if (do_qk) {
            if (!q_ready) {
              if (!mbar_wait(&q_full[i], my_items & 1, p.status)) {
                ok = false;
                break;
              }
              q_ready = true;
            }
            tc_fence_after();
            const uint32_t N = my_blocks + (uint32_t)(jq - r.lo);
            const uint32_t d_tmem = tmem_base + (uint32_t)((i * 2 + (N & 1)) * kBKV);
            const uint64_t kb = k_desc0 + (uint64_t)((ks_slot * KB) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint64_t qoff = (uint64_t)((ks >> 2) * ((128 * 128) >> 4) + (ks & 3) * 2);
              const uint64_t koff = (uint64_t)((ks >> 2) * (KBOX >> 4) + (ks & 3) * 2);
              if (leader) umma_ss(d_tmem, qa + qoff, kb + koff, idesc_qk, ks != 0 ? 1u : 0u);
            }
            if (leader) tc_commit(&s_full[i * 2 + (N & 1)]);
            // the item's last QK has read the Q tile: the loader may bring the next one
            if (leader && jq == r.hi - 1) tc_commit(&q_empty[i]);
          }
          if (leader && have_v) tc_commit(&v_empty[vs_slot]);
          if (leader && have_k) tc_commit(&k_empty[ks_slot]);
          __syncwarp();
        }
        kv_blocks += (uint32_t)(w.u_hi - w.u_lo);
        if (live) {
          my_blocks += (uint32_t)nblk;
          ++my_items;
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ---------------- softmax + epilogue ----------------
    const int i = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t o_tmem = tmem_base + 256 + i * D + lane_addr;
    const float sl2 = p.scale_log2;
    const int my_turn = 1 + i * 4 + quarter;
    const int other_turn = 1 + (1 - i) * 4 + quarter;
    uint32_t my_blocks = 0;   // blocks of this tile in all earlier items
    uint32_t tail_count = 0;  // tail commits of this tile in all earlier items
    // A warp whose bounded wait ran out stops computing but keeps walking the
    // queue and, for every later item, arrives on its partner's barrier at each
    // turn the partner may take (`ok` stays false): the partner, which sees the
    // same items, is never left waiting, and the warp that gave up never waits
    // on a named barrier (they have no limit) again. Both leave when the queue
    // ends or stops being fed.
    bool ok = true;
    for (uint32_t n_it = 0;; ++n_it) {
      const int slot = (int)(n_it & 1);
      // Both warps of a MUFU pair must take the same items: this wait ignores a
      // status word that is already set (it would let one partner leave while the
      // other still receives the item and then waits on a named barrier for good)
      // and ends only with the item or with its own limit, which both reach together.
      if (!mbar_wait_patient(&item_full[slot], (n_it >> 1) & 1, p.status)) {
        // No item within the limit: the queue is dead. Should the partner have
        // caught an item in the instant between the two limits (the loader can be
        // at most two items ahead), it is released through every turn it may take.
        for (int64_t m = 0; m < 2 * (p.tk / kBKV + 2); ++m) named_barrier_arrive(other_turn, 64);
        break;
      }
      const Work w = item_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&item_empty[slot]);
      if (!w.valid) break;
      if (!ok) {
        const int pairs = min(w.r0.hi - w.r0.lo, w.r1.hi - w.r1.lo);
        // arrivals only: a partner still computing is released at each of its
        // turns, and this warp never waits on a barrier without a limit again
        for (int m = 0; m < pairs; ++m)
          if (i == 0 || m + 1 < pairs) named_barrier_arrive(other_turn, 64);
        continue;
      }
      const Range r = i == 0 ? w.r0 : w.r1;
      const int h = w.h + (p.pair_heads ? i : 0);
      const int64_t b = w.b;
      const int64_t i_first = (int64_t)w.i0 + (p.pair_heads ? 0 : (int64_t)i * kBQ);
      const int64_t row = i_first + quarter * 32 + lane;
      const bool row_ok = row < p.t;
      const int64_t i_last = (i_first + kBQ - 1 < p.t - 1) ? i_first + kBQ - 1 : p.t - 1;
      int64_t seg_me = 0, seg_last = 0;
      if (p.seg_start != nullptr && i_first < p.t) {
        seg_me = p.seg_start[b * p.t + (row_ok ? row : i_last)];
        seg_last = p.seg_start[b * p.t + i_last];
      }
      int64_t vis_lo64 = 0, vis_hi64 = w.len;
      if (p.causal && row + 1 < vis_hi64) vis_hi64 = row + 1;
      if (p.has_window) {
        if (row - p.win_left > vis_lo64) vis_lo64 = row - p.win_left;
        if (row + p.win_right + 1 < vis_hi64) vis_hi64 = row + p.win_right + 1;
      }
      if (p.has_chunk) {
        const int64_t ci = row / p.chunk_size;
        if ((ci + p.chunk_right + 1) * p.chunk_size < vis_hi64) vis_hi64 = (ci + p.chunk_right + 1) * p.chunk_size;
        if (p.chunk_left >= 0 && (ci - p.chunk_left) * p.chunk_size > vis_lo64) vis_lo64 = (ci - p.chunk_left) * p.chunk_size;
      }
      if (p.seg_start != nullptr && seg_me > vis_lo64) vis_lo64 = seg_me;
      const int vis_lo = (int)vis_lo64, vis_hi = (int)(vis_hi64 < vis_lo64 ? vis_lo64 : vis_hi64);
      auto vis_word = [&](int base) -> uint32_t {
        int a = vis_lo - base, bnd = vis_hi - base;
        a = a < 0 ? 0 : a;
        bnd = bnd > 32 ? 32 : bnd;
        uint32_t wd = 0;
        if (bnd > a) wd = (bnd == 32 ? 0xffffffffu : ((1u << bnd) - 1u)) & ~((1u << a) - 1u);
        return wd;
      };
      float m_run = -INFINITY;
      float l_run = 0.f;
      const int nblk = r.hi - r.lo;
      // The hand-over of the MUFU unit between the two tiles (see the one-item
      // kernel): a named barrier per (tile, quarter); a warp that gave up still
      // walks the rest of the item's sequence.
      const int n_paired = min(w.r0.hi - w.r0.lo, w.r1.hi - w.r1.lo);
      int turns_done = 0;
      uint32_t sr[2][32];
      bool requested = false;
      for (int j = r.lo; j < r.hi && ok; ++j) {
        const int n = j - r.lo;
        const uint32_t N = my_blocks + (uint32_t)n;
        const int buf = (int)(N & 1);
        turns_done = n;
        const uint32_t s_tmem = tmem_base + (uint32_t)((i * 2 + buf) * kBKV) + lane_addr;
        if (!requested) {
          if (!mbar_wait(&s_full[i * 2 + buf], (N >> 1) & 1, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          tmem_ld32(s_tmem, sr[0]);
          tmem_ld32(s_tmem + 32, sr[1]);
        }
        const int64_t j0 = (int64_t)j * kBKV, j1 = j0 + kBKV - 1;
        bool need_mask = j1 >= w.len || p.has_chunk || w.general;
        if (p.causal && j1 > i_first) need_mask = true;
        if (p.has_window && (j0 + p.win_left < i_last || j1 > i_first + p.win_right)) need_mask = true;
        if (p.seg_start != nullptr && j0 < seg_last) need_mask = true;
        tmem_ld_wait_for(sr[0]);
        tmem_ld_wait_for(sr[1]);
        if (EXTRAS && p.bias != nullptr && row_ok) {
          // + bias / scale in raw-score units: (s + bias/scale) * scale = s*scale + bias, before the masks
          const T* brow = (const T*)p.bias + (((p.bias_per_batch ? b : 0) * p.heads + h) * p.t + row) * p.tk + j0;
          const bool vec = ((reinterpret_cast<uintptr_t>(brow) & 15) == 0) && j1 < p.tk;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float bv[8];
            if (vec) {
              const uint4 u = ldg128(brow + c * 8);
              const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = Elem<T>::unpack(uu[e]);
                bv[2 * e] = f.x, bv[2 * e + 1] = f.y;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) bv[e] = j0 + c * 8 + e < p.tk ? Elem<T>::to_f(brow[c * 8 + e]) : 0.f;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int k = c * 8 + e;
              sr[k >> 5][k & 31] = __float_as_uint(fmaf(bv[e], p.inv_scale, __uint_as_float(sr[k >> 5][k & 31])));
            }
          }
        }
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t vw = vis_word((int)j0 + 32 * c);
            if (w.general) {
              // the mask bits of these 32 keys: one key per lane, gathered by a ballot
              const int64_t jk = j0 + 32 * c + lane;
              int m = 0;
              if (jk < p.tk)
                m = p.key_mask_i32 ? ((const int32_t*)p.key_mask)[b * p.tk + jk]
                                   : (int)((const uint8_t*)p.key_mask)[b * p.tk + jk];
              vw &= __ballot_sync(0xffffffffu, m != 0);
            }
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (((vw >> e) & 1u) == 0) sr[c][e] = 0xff800000u;
          }
        }
        float mx;
        {
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              m0 = max3(m0, __uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
              m1 = max3(m1, __uint_as_float(sr[c][e + 2]), __uint_as_float(sr[c][e + 3]));
              m2 = max3(m2, __uint_as_float(sr[c][e + 4]), __uint_as_float(sr[c][e + 5]));
              m3 = max3(m3, __uint_as_float(sr[c][e + 6]), __uint_as_float(sr[c][e + 7]));
            }
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        }
        const float mx_t = mx * sl2;
        float m_new = m_run;
        if (mx_t > m_run + kRescaleAbove || m_run == -INFINITY) m_new = fmaxf(m_run, mx_t);
        bool tail0_seen = false;
        const bool moved = m_new != m_run && m_run != -INFINITY;
        const float corr = moved ? ex2_approx(m_run - m_new) : 1.0f;
        if (__any_sync(0xffffffffu, moved)) {
          // the previous block's P.V has landed once the next block's S is
          // complete (issue order); the tile's last block reads the tail barrier
          const uint32_t Nn = N + 1;
          const bool landed = n + 1 < nblk ? mbar_wait(&s_full[i * 2 + (int)(Nn & 1)], (Nn >> 1) & 1, p.status)
                                           : mbar_wait(&tail_done[i], tail_count & 1, p.status);
          if (!landed) {
            ok = false;
            break;
          }
          tail0_seen = n + 1 == nblk;
          tc_fence_after();
          l_run *= corr;
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t orr[32];
            tmem_ld32(o_tmem + c, orr);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) orr[e] = __float_as_uint(__uint_as_float(orr[e]) * corr);
            tmem_st32(o_tmem + c, orr);
          }
          tmem_st_wait();
        }
        m_run = m_new;
        float m_use = m_run == -INFINITY ? 0.f : m_run;
        if (n < n_paired && (i == 1 || n > 0)) {
          named_barrier(my_turn, 64);
          asm volatile("" : "+f"(m_use));
        }
        const float2 sl2_2 = make_float2(sl2, sl2), nm_2 = make_float2(-m_use, -m_use);
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
        uint32_t pk[32];
        constexpr int kLag = 6;
        float2 xs[32];
#pragma unroll
        for (int k = 0; k < 32; ++k)
          xs[k] = __ffma2_rn(make_float2(__uint_as_float(sr[k >> 4][2 * (k & 15)]),
                                         __uint_as_float(sr[k >> 4][2 * (k & 15) + 1])),
                             sl2_2, nm_2);
#pragma unroll
        for (int k = 0; k < 32 + kLag; ++k) {
          if (k < 32) {
            xs[k].x = ex2_approx(xs[k].x);
            xs[k].y = ex2_approx(xs[k].y);
          }
          if (k >= kLag) {
            const int d = k - kLag;
            if (d & 1) lb = __fadd2_rn(lb, xs[d]);
            else la = __fadd2_rn(la, xs[d]);
            pk[d] = Elem<T>::pack(xs[d].x, xs[d].y);
          }
        }
        tmem_st32(s_tmem, pk);
        if (n < n_paired && (i == 0 || n + 1 < n_paired)) named_barrier_arrive(other_turn, 64);
        turns_done = n + 1;
        l_run += (la.x + la.y) + (lb.x + lb.y);
        requested = false;
        if (n + 1 < nblk) {
          const uint32_t Nn = N + 1;
          if (mbar_test_wait(&s_full[i * 2 + (int)(Nn & 1)], (Nn >> 1) & 1)) {
            tc_fence_after();
            const uint32_t next_tmem = tmem_base + (uint32_t)((i * 2 + (int)(Nn & 1)) * kBKV) + lane_addr;
            tmem_ld32(next_tmem, sr[0]);
            tmem_ld32(next_tmem + 32, sr[1]);
            requested = true;
          }
        }
        tmem_st_wait();
        // the first of the tile's two tail commits is observed before the last P
        // (which lets the second happen) is published
        if (n + 1 == nblk && nblk >= 2 && !tail0_seen && !mbar_wait(&tail_done[i], tail_count & 1, p.status)) {
          ok = false;
          break;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[i * 2 + buf]);
      }
      if (!ok) {
        for (int m = turns_done; m < n_paired; ++m)
          if (i == 0 || m + 1 < n_paired) named_barrier_arrive(other_turn, 64);
        continue;
      }
      // ---- epilogue: O / l, or this split's unnormalised state ----
      T* orow = (T*)p.o + b * p.o_sb + row * p.o_st + (int64_t)h * p.o_sh;
      const int64_t prow = (((int64_t)w.split * p.batch + b) * p.t + row) * p.heads + h;  // partial-state row
      float* oprow = EXTRAS && p.splits > 1 ? p.o_part + prow * p.d_real : nullptr;
      if (nblk > 0) {
        // the last P.V: the item's second tail commit (its only one for a one-block tile)
        const uint32_t last = tail_count + (nblk >= 2 ? 1u : 0u);
        if (!mbar_wait(&tail_done[i], last & 1, p.status)) {
          ok = false;  // the item's hand-over sequence is complete: drain from the next item on
          continue;
        }
        tc_fence_after();
        const float inv = l_run == 0.f ? 0.f : 1.0f / l_run;
        if (EXTRAS && oprow != nullptr) {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t orr[32];
            tmem_ld32(o_tmem + c, orr);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                if (c + v * 4 >= p.d_real) break;
                *reinterpret_cast<uint4*>(oprow + c + v * 4) =
                    make_uint4(orr[v * 4], orr[v * 4 + 1], orr[v * 4 + 2], orr[v * 4 + 3]);
              }
            }
          }
        } else {
          const int64_t row0 = i_first + quarter * 32;
          store_o_slab<T, D>(o_tmem, inv, o_stage + (warp - 4) * (32 * 128), lane, &tmap_o, h, (int)row0, (int)b,
                             p.d_real, row0 < p.t);
        }
        // O is read out: the next live item's first P.V may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[i]);
        my_blocks += (uint32_t)nblk;
        tail_count += nblk >= 2 ? 2u : 1u;
      } else if (EXTRAS && row_ok && oprow != nullptr) {
        for (int c = 0; c < p.d_real; c += 4) *reinterpret_cast<uint4*>(oprow + c) = make_uint4(0, 0, 0, 0);
      } else if (row_ok) {
        // No key block reaches this tile: zeros (attention.rs:971-980).
        for (int c = 0; c < p.d_real; c += 8) stg128(orow + c, make_uint4(0, 0, 0, 0));
      }
      if (EXTRAS && oprow != nullptr && row_ok) {
        // an empty share keeps a finite sentinel maximum, so the merge never sees inf - inf
        p.m_part[prow] = m_run == -INFINITY ? -1e30f : m_run;
        p.l_part[prow] = l_run;
      }
      if (p.lse != nullptr && row_ok)
        p.lse[(b * p.heads + h) * p.t + row] = l_run == 0.f ? -INFINITY : kLn2F * (m_run + log2f(l_run));
    }
    if (lane == 0) tma_store_wait_all();  // the slab stays put until its last store has read it
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// The queue head of a launch on `stream`: launches on one stream run one after
// the other and share a head; every other (device, stream) pair gets a head of
// its own, so launches that overlap on different streams never share one. A
// graph replays with the head of the stream it was captured on. Returns nullptr
// once kQueueSlots pairs have been seen: the caller then takes the one-item kernel.
int* queue_head(cudaStream_t stream) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, int> slots;
  static int* base[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (base[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_next_item) != cudaSuccess) return nullptr;
    base[dev] = (int*)p;
  }
  const auto key = std::make_pair(dev, stream);
  auto it = slots.find(key);
  if (it == slots.end()) {
    int used = 0;
    for (const auto& kv : slots) used += kv.first.first == dev ? 1 : 0;
    if (used >= kQueueSlots) return nullptr;
    it = slots.emplace(key, used).first;
  }
  return base[dev] + it->second;
}

// An item is one 128-row tile of two query heads (instead of two tiles of one head)
// whenever grouped-query attention gives every KV head an even number of query heads.
bool pairs_heads(const AttnArgs& a) {
  const int group = a.kv_heads > 0 ? a.heads / a.kv_heads : 0;
  return group >= 2 && group % 2 == 0;
}

int64_t item_count(const AttnArgs& a, int splits) {
  if (pairs_heads(a)) return ((a.t + kBQ - 1) / kBQ) * (int64_t)(a.heads / 2) * a.batch * splits;
  return ((a.t + 2 * kBQ - 1) / (2 * kBQ)) * (int64_t)a.heads * a.batch * splits;
}

template <typename T, int D, bool EXTRAS>
int run_p(const AttnArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  using C = FaCfg<D>;
  CUtensorMap tq, tk, tv;
  const uint32_t box[4] = {64, 1, 128, 1};
  const uint32_t kvbox[4] = {64, 1, kBKV, 1};
  {
    const uint64_t dims[4] = {(uint64_t)a.d, (uint64_t)a.heads, (uint64_t)a.t, (uint64_t)a.batch};
    const uint64_t st[3] = {(uint64_t)a.q_sh, (uint64_t)a.q_st, (uint64_t)a.q_sb};
    if (!make_tmap(&tq, a.q, a.dtype, 4, dims, st, box)) return -1;
  }
  {
    const uint64_t dims[4] = {(uint64_t)a.d, (uint64_t)a.kv_heads, (uint64_t)a.tk, (uint64_t)a.kv_rows};
    const uint64_t stk[3] = {(uint64_t)a.k_sh, (uint64_t)a.k_st, (uint64_t)a.k_sb};
    const uint64_t stv[3] = {(uint64_t)a.v_sh, (uint64_t)a.v_st, (uint64_t)a.v_sb};
    if (!make_tmap(&tk, a.k, a.dtype, 4, dims, stk, kvbox)) return -1;
    if (!make_tmap(&tv, a.v, a.dtype, 4, dims, stv, kvbox)) return -1;
  }
  CUtensorMap to = tq;
  if (a.o != nullptr) {
    // the output as 32-row x 64-column boxes, one per softmax warp and store
    const uint32_t obox[4] = {64, 1, 32, 1};
    const uint64_t dims[4] = {(uint64_t)a.d, (uint64_t)a.heads, (uint64_t)a.t, (uint64_t)a.batch};
    const uint64_t st[3] = {(uint64_t)a.o_sh, (uint64_t)a.o_st, (uint64_t)a.o_sb};
    if (!make_tmap(&to, a.o, a.dtype, 4, dims, st, obox)) return -1;
  }
  // the attribute belongs to the device's copy of the kernel: once per device
  static bool attr_seen[64] = {};
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_seen[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_tc_p_kernel<T, D, EXTRAS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes_p<D>()) != cudaSuccess)
      return -1;
    attr_set = true;
  }
  int* head = queue_head(s);
  if (head == nullptr) return 1;  // no queue head left for this stream: the one-item kernel takes the call
  FaParams p{};
  p.o = a.o;
  p.o_sb = a.o_sb, p.o_st = a.o_st, p.o_sh = a.o_sh;
  p.t = a.t, p.tk = a.tk;
  p.heads = a.heads, p.kv_heads = a.kv_heads;
  p.scale_log2 = a.scale * kLog2eF;
  p.causal = a.causal;
  p.key_lens = a.key_lens;
  p.key_mask = a.key_mask;
  p.key_mask_i32 = a.key_mask_i32;
  p.has_window = a.has_window;
  p.win_left = a.win_left, p.win_right = a.win_right;
  p.has_chunk = a.has_chunk;
  p.chunk_size = a.chunk_size, p.chunk_left = a.chunk_left, p.chunk_right = a.chunk_right;
  p.seg_start = a.seg_start;
  p.row_map = a.row_map;
  p.lse = a.lse;
  p.pair_heads = pairs_heads(a) ? 1 : 0;
  p.n_qt = (int)(p.pair_heads ? (a.t + kBQ - 1) / kBQ : (a.t + 2 * kBQ - 1) / (2 * kBQ));
  p.d_real = a.d;
  p.splits = a.splits > 1 ? a.splits : 1;
  p.batch = a.batch;
  p.o_part = a.o_part, p.m_part = a.m_part, p.l_part = a.l_part;
  p.bias = a.bias;
  p.bias_per_batch = a.bias_per_batch;
  p.inv_scale = 1.0f / a.scale;
  p.status = a.status;
  const int item_heads = p.pair_heads ? a.heads / 2 : a.heads;
  const int64_t items = (int64_t)p.n_qt * item_heads * a.batch * p.splits;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int grid = (int)(items < sms ? items : sms);
  // Under a causal mask the items differ in length: interleave enough of the last
  // groups that their work is several times (SMs x longest item).
  int tail_groups = 0;
  if (a.causal) {
    const int64_t groups = (int64_t)a.batch * a.kv_heads;
    const int64_t per_kv = (int64_t)(item_heads / a.kv_heads) * p.n_qt;
    const int64_t want = (6 * (int64_t)sms + per_kv - 1) / per_kv;
    tail_groups = (int)(want < groups ? want : groups);
  }
  if (cudaMemsetAsync(head, 0, sizeof(int), s) != cudaSuccess) return -1;
  attention_tc_p_kernel<T, D, EXTRAS><<<grid, kThreadsFa, smem_bytes_p<D>(), s>>>(tq, tk, tv, to, p, (int)items,
                                                                                  tail_groups, head);
  if (cfg != nullptr)
    snprintf(cfg, cfg_len, p.pair_heads ? "{bq:%d,bkv:%d,d:%d,stages:%d,splits:%d,persistent:%d,head_pairs:1}"
                                        : "{bq:%d,bkv:%d,d:%d,stages:%d,splits:%d,persistent:%d}",
             2 * kBQ, kBKV, a.d, C::kStages,
             p.splits, grid);
  return 0;
}

}  // namespace

// The persistent kernel takes what the one-item kernel takes once there are more
// items than SMs (otherwise nothing would overlap), and it alone takes key
// splits and an additive bias, whatever the item count.
bool attention_tc_p_covers(const AttnArgs& a) {
  AttnArgs plain = a;
  plain.splits = 1;
  plain.bias = nullptr;
  if (!attention_tc_covers(plain)) return false;
  const int splits = a.splits > 1 ? a.splits : 1;
  const int64_t items = item_count(a, splits);
  if (items >= 0x7fffffffLL) return false;
  if (a.splits > 1 || a.bias != nullptr) {
    // partial rows are written 16 bytes at a time; the score rows of the bias are read per thread
    if (a.splits > 1 && (a.o_part == nullptr || (reinterpret_cast<uintptr_t>(a.o_part) & 15) != 0 || a.d % 4 != 0))
      return false;
    return true;
  }
  return items > 148;
}

int launch_attention_tc_p(const AttnArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  if (!attention_tc_p_covers(a)) return 1;
  const bool extras = a.splits > 1 || a.bias != nullptr;
  if (a.dtype == SVODB_BF16) {
    if (extras)
      return a.d > 64 ? run_p<__nv_bfloat16, 128, true>(a, s, cfg, cfg_len)
                      : run_p<__nv_bfloat16, 64, true>(a, s, cfg, cfg_len);
    return a.d > 64 ? run_p<__nv_bfloat16, 128, false>(a, s, cfg, cfg_len)
                    : run_p<__nv_bfloat16, 64, false>(a, s, cfg, cfg_len);
  }
  if (extras) return a.d > 64 ? run_p<__half, 128, true>(a, s, cfg, cfg_len) : run_p<__half, 64, true>(a, s, cfg, cfg_len);
  return a.d > 64 ? run_p<__half, 128, false>(a, s, cfg, cfg_len) : run_p<__half, 64, false>(a, s, cfg, cfg_len);
}

}  // namespace svodb
