// tcgen05 flash-attention forward: o = softmax(q.k^T*scale + masks) . v over
// sequence-major q [B,T,H,D], k/v [B,Tk,Hkv,D] (or one packed projection),
// 16-bit operands, D in {64,128}.
//
// Semantics follow tk/src/kernels/attention.rs:381-450: scores in f32, base-2
// online softmax with the lazy rescale (a row adopts a new maximum only when it
// grew by more than 8 in log2 units, attention.rs:373-379,418-431),
// probabilities rounded to the stream type before P.V while the row sum is
// taken from the f32 values (attention.rs:434-444), `O/l` at the end with rows
// no key reached written as zeros (attention.rs:971-980). Masks: causal, key
// lengths, bool key mask, window, chunk, segment starts (attention.rs:641-697);
// key blocks no query of a tile can see are skipped and only blocks a mask edge
// crosses pay for the mask (attention.rs:586-612,698-733).
//
// Blackwell design — one CTA per (256 query rows, head, batch), 384 threads:
//   warp 0        TMA loader: two 128-row Q tiles once, then K and V blocks of
//                 64 keys through two 4-stage shared-memory rings (non-multicast
//                 TMA, 128B swizzle; ragged T / Tk tails zero-filled).
//   warps 1, 3    MMA issuers, one per query tile (the whole warp walks the
//                 schedule so descriptors stay warp-uniform; an elected lane
//                 issues). Step t: O_i += P_i(t-1).V(t-1) with P read from TMEM
//                 (TS form) and V as the MN-major shared-memory operand, then
//                 S_i(t+1) = Q_i.K(t+1)^T (SS form) into the score buffer that
//                 P_i(t-1) just vacated: scores run one block ahead of the
//                 softmax. Completion is in issue order, so "S(t+1) complete"
//                 also tells the softmax that P.V(t-1) has landed; only the last
//                 two P.V of a tile need a barrier of their own (tail_done).
//   warp 2        TMEM allocation; warps 2-3 turn a bool key mask into a prefix
//                 length or a bitmask before the main loop.
//   warps 4-7     softmax of tile 0: one query row per thread, S read from TMEM
//   warps 8-11    softmax of tile 1  (tcgen05.ld), P written back over S as
//                 packed 16-bit (tcgen05.st), O rescaled in TMEM when a row's
//                 maximum moves, final O/l -> global. The two warps that share
//                 a scheduler (same lane quarter, different tile) take turns on
//                 the MUFU unit through a named barrier, and a warp requests the
//                 next block's scores before it publishes P.
// Registers: setmaxnreg moves the loader/issuer warpgroup down to 64 and the
// softmax warpgroups up to 216 inside the CTA's launch-time pool (384 x 168).
// TMEM (512 columns): per tile two 64-column score buffers, S_i[buf] at
// (2i+buf)*64; O_i at 256 + i*D; P aliases the first 32 columns of its S buffer.
//
// Every mbarrier wait is bounded; a timeout records a status code and the CTA
// drains and frees its TMEM. Named barriers have no timeout, so a warp that
// gave up never waits on one again: it only arrives, once per remaining turn of
// its partner, which is thereby released whether or not it gave up too.
#include <cuda.h>
#include <math.h>
#include <stdio.h>

#include "attention_parts.cuh"
#include "common.cuh"
#include "kernels.h"
#include "svodb.h"
#include "tensormap.h"

namespace svodb {

namespace {

using namespace fa_parts;


template <typename T, int D>
__global__ void __launch_bounds__(kThreadsFa, 1)
    attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using C = FaCfg<D>;
  constexpr int S = C::kStages;
  constexpr int QB = C::kQTileBytes;   // one 128-row Q tile
  constexpr int KB = C::kKvBytes;      // one 64-key K or V block
  constexpr int KBOX = kBKV * 128;     // bytes of one 64-column box of a K/V block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                         // [2][QB]
  uint8_t* k_s = q_s + 2 * QB;                 // [S][KB]
  uint8_t* v_s = k_s + S * KB;                 // [S][KB]
  uint32_t* mask_bits = reinterpret_cast<uint32_t*>(v_s + S * KB);  // [kMaxMaskWords]
  uint64_t* bars = reinterpret_cast<uint64_t*>(mask_bits + kMaxMaskWords);
  uint64_t* q_full = bars;                     // [2]
  uint64_t* k_full = bars + 2;                 // [S]
  uint64_t* k_empty = k_full + S;
  uint64_t* v_full = k_empty + S;
  uint64_t* v_empty = v_full + S;
  uint64_t* s_full = v_empty + S;              // [2 tiles][2 buffers]
  uint64_t* p_full = s_full + 4;               // [2 tiles][2 buffers]
  uint64_t* tail_done = p_full + 4;            // [2 tiles]: the last two P.V of a tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail_done + 2);
  int* scan = reinterpret_cast<int*>(tmem_slot + 1);  // [0] first zero, [1] last nonzero + 1

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Heavier (later, under a causal mask) query tiles are scheduled first.
  const int qt = p.n_qt - 1 - (int)blockIdx.x;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int hk = h / (p.heads / p.kv_heads);
  const int64_t i0 = (int64_t)qt * 2 * kBQ;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&tail_done[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp
    }
    for (int i = 0; i < S; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);  // released by both tiles' issuers
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
    }
    scan[0] = 0x7fffffff;
    scan[1] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  __syncthreads();
  // ---- key mask scan (warps 2-3): prefix length, or a bitmask -----------------
  if (p.key_mask != nullptr && (warp == 2 || warp == 3)) {
    const int tid = threadIdx.x - 64;
    int first_zero = 0x7fffffff, last_set = 0;
    const int words = (int)((p.tk + 31) / 32);
    for (int wd = tid; wd < words; wd += 64) {
      uint32_t bits = 0;
      const int64_t base = (int64_t)wd * 32;
      for (int e = 0; e < 32; ++e) {
        const int64_t j = base + e;
        if (j < p.tk) {
          const int64_t at = b * p.tk + j;
          const int m = p.key_mask_i32 ? ((const int32_t*)p.key_mask)[at] : (int)((const uint8_t*)p.key_mask)[at];
          if (m != 0) {
            bits |= 1u << e;
            last_set = (int)j + 1;
          } else if ((int)j < first_zero) {
            first_zero = (int)j;
          }
        }
      }
      if (wd < kMaxMaskWords) mask_bits[wd] = bits;
    }
    atomicMin(&scan[0], first_zero);
    atomicMax(&scan[1], last_set);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  Ctx ctx;
  ctx.len = p.tk;
  ctx.general_mask = 0;
  if (p.key_lens != nullptr) {
    const int64_t kl = p.key_lens[b];
    ctx.len = kl < 0 ? 0 : (kl < ctx.len ? kl : ctx.len);
  }
  if (p.key_mask != nullptr) {
    const int first_zero = scan[0], last_set = scan[1];
    if (first_zero < last_set) ctx.general_mask = 1;  // not a prefix: consult the bitmask
    if (last_set < ctx.len) ctx.len = last_set;
  }
  const Range r0 = tile_range(p, ctx, b, i0);
  const Range r1 = tile_range(p, ctx, b, i0 + kBQ);
  const bool live0 = r0.hi > r0.lo, live1 = r1.hi > r1.lo;
  int u_lo = 0, u_hi = 0;
  if (live0 && live1) {
    u_lo = r0.lo < r1.lo ? r0.lo : r1.lo;
    u_hi = r0.hi > r1.hi ? r0.hi : r1.hi;
  } else if (live0) {
    u_lo = r0.lo, u_hi = r0.hi;
  } else if (live1) {
    u_lo = r1.lo, u_hi = r1.hi;
  }

  // Registers: the loader / MMA / mask warpgroup gives registers back to
  // the two softmax warpgroups.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 0) {
      // ---------------- TMA loader ----------------
      if (lane == 0 && u_hi > u_lo) {
        for (int i = 0; i < 2; ++i) {
          if (i == 0 ? live0 : live1) {
            mbar_expect_tx(&q_full[i], QB);
            for (int c = 0; c < D / 64; ++c)
              tma_load_4d(q_s + i * QB + c * (128 * 128), &tmap_q, &q_full[i], c * 64, h, (int)(i0 + i * kBQ),
                          (int)b);
          }
        }
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        const int kv_b = p.row_map != nullptr ? p.row_map[b] : (int)b;
        for (int j = u_lo; j < u_hi; ++j) {
          if (!mbar_wait(&k_empty[s], ph ^ 1, p.status)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&k_full[s], KB);
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(k_s + s * KB + c * KBOX, &tmap_k, &k_full[s], c * 64, hk, j * kBKV, kv_b);
          if (!mbar_wait(&v_empty[s], ph ^ 1, p.status)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&v_full[s], KB);
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(v_s + s * KB + c * KBOX, &tmap_v, &v_full[s], c * 64, hk, j * kBKV, kv_b);
          if (++s == S) {
            s = 0;
            ph ^= 1;
          }
        }
        if (!ok) {
          // Error path: give copies in flight a bounded time to land.
          for (uint32_t it = 0; it < (1u << 18); ++it) {
            bool all = true;
            for (int i = 0; i < S; ++i) all = all && mbar_try_wait(&k_full[i], ph) && mbar_try_wait(&v_full[i], ph);
            if (all) break;
          }
        }
      }
    } else if (warp == 1 || warp == 3) {
      // ---------------- MMA issuers: warp 1 drives tile 0, warp 3 tile 1 ----------------
      // Each query tile has its own issuing warp, so the barrier round trips of
      // one tile's schedule overlap the other's MMAs. The whole warp walks the
      // schedule (addresses and descriptors stay warp-uniform values); one
      // elected lane issues the MMAs and commits.
      const int i = warp == 1 ? 0 : 1;
      const Range r = i == 0 ? r0 : r1;
      const bool leader = elect_one();
      if (u_hi > u_lo) {
        constexpr uint32_t idesc_qk = umma_idesc(Elem<T>::kUmmaFormat, 128, kBKV, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc(Elem<T>::kUmmaFormat, 128, D, 0, 1);
        const uint64_t qa = umma_desc_sw128(smem_u32(q_s) + i * QB, 16, 1024);
        const uint64_t k_desc0 = umma_desc_sw128(smem_u32(k_s), 16, 1024);
        // V block: [keys][D]; 64-column boxes KBOX apart (LBO), 8-key groups 1 KiB apart (SBO).
        const uint64_t v_desc0 = umma_desc_sw128(smem_u32(v_s), KBOX, 1024);
        const int nblk = r.hi - r.lo;
        bool ok = true;
        bool q_ready = false;
        // Step t issues O += P(t-1).V(t-1) and then S(t+1) = Q.K(t+1)^T into the
        // score buffer that P(t-1) just vacated: S runs one block ahead of the
        // softmax. Both issuers walk the union of the two tiles' key ranges and
        // each releases every K/V slot (the ring barriers count two arrivals).
        for (int t = u_lo - 1; t <= u_hi && ok; ++t) {
          const int jq = t + 1;  // block whose scores are issued this step
          const int jp = t - 1;  // block whose P.V is issued this step
          const bool have_k = jq >= u_lo && jq < u_hi;
          const bool have_v = jp >= u_lo && jp < u_hi;
          const int ks_slot = have_k ? (jq - u_lo) % S : 0;
          const int vs_slot = have_v ? (jp - u_lo) % S : 0;
          const bool do_pv = have_v && jp >= r.lo && jp < r.hi;
          const bool do_qk = have_k && jq >= r.lo && jq < r.hi;
          // Every slot is waited for and released by both issuers, used or not:
          // an issuer can then never arrive twice on one phase of a ring barrier.
          if ((have_k && !mbar_wait(&k_full[ks_slot], (uint32_t)(((jq - u_lo) / S) & 1), p.status)) ||
              (have_v && !mbar_wait(&v_full[vs_slot], (uint32_t)(((jp - u_lo) / S) & 1), p.status))) {
            ok = false;
            break;
          }
          if (do_pv) {
            const int n = jp - r.lo;  // this tile's block counter
            if (!mbar_wait(&p_full[i * 2 + (n & 1)], (uint32_t)((n >> 1) & 1), p.status)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + 256 + i * D;
            const uint32_t a_tmem = tmem_base + (uint32_t)((i * 2 + (n & 1)) * kBKV);
            const uint64_t vb = v_desc0 + (uint64_t)((vs_slot * KB) >> 4);
            const uint32_t first = n != 0 ? 1u : 0u;
#pragma unroll
            for (int ks = 0; ks < kBKV / 16; ++ks)  // 16 keys per step = 2 KiB of V, 8 packed P columns
              if (leader)
                umma_ts(d_tmem, a_tmem + ks * 8, vb + (uint64_t)(ks * (2048 >> 4)), idesc_pv,
                        (first | (uint32_t)ks) != 0 ? 1u : 0u);
            // The last two P.V of a tile have no later S to announce them: they
            // are published on tail_done (phase 0: block N-2, phase 1: block N-1;
            // a one-block tile uses phase 0 only).
            if (leader && n + 2 >= nblk) tc_commit(&tail_done[i]);
          }
          if (do_qk) {
            if (!q_ready) {
              if (!mbar_wait(&q_full[i], 0, p.status)) {
                ok = false;
                break;
              }
              q_ready = true;
            }
            tc_fence_after();
            const int n = jq - r.lo;
            const uint32_t d_tmem = tmem_base + (uint32_t)((i * 2 + (n & 1)) * kBKV);
            const uint64_t kb = k_desc0 + (uint64_t)((ks_slot * KB) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              // 16 columns = 32 bytes inside a 64-column box
              const uint64_t qoff = (uint64_t)((ks >> 2) * ((128 * 128) >> 4) + (ks & 3) * 2);
              const uint64_t koff = (uint64_t)((ks >> 2) * (KBOX >> 4) + (ks & 3) * 2);
              if (leader) umma_ss(d_tmem, qa + qoff, kb + koff, idesc_qk, ks != 0 ? 1u : 0u);
            }
            // In-order completion: S(t+1) complete implies P.V(t-1) complete.
            if (leader) tc_commit(&s_full[i * 2 + (n & 1)]);
          }
          if (leader && have_v) tc_commit(&v_empty[vs_slot]);
          if (leader && have_k) tc_commit(&k_empty[ks_slot]);
          __syncwarp();
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ---------------- softmax + epilogue ----------------
    const int i = (warp - 4) >> 2;                 // query tile
    const int quarter = warp & 3;                  // TMEM lane quarter
    const Range r = i == 0 ? r0 : r1;
    const int64_t i_first = i0 + (int64_t)i * kBQ;
    const int64_t row = i_first + quarter * 32 + lane;
    const bool row_ok = row < p.t;
    const int64_t i_last = (i_first + kBQ - 1 < p.t - 1) ? i_first + kBQ - 1 : p.t - 1;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t o_tmem = tmem_base + 256 + i * D + lane_addr;
    const float sl2 = p.scale_log2;
    int64_t seg_me = 0, seg_last = 0;
    if (p.seg_start != nullptr && i_first < p.t) {
      seg_me = p.seg_start[b * p.t + (row_ok ? row : i_last)];
      seg_last = p.seg_start[b * p.t + i_last];
    }
    // Every mask but the bool key mask is an interval of keys per query row:
    // this row sees keys [vis_lo, vis_hi) (and, under a general key mask, the set
    // bits of the bitmask among them).
    int64_t vis_lo64 = 0, vis_hi64 = ctx.len;
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
    // Visibility of keys base .. base+31 as a bit word.
    auto vis_word = [&](int base) -> uint32_t {
      int a = vis_lo - base, bnd = vis_hi - base;
      a = a < 0 ? 0 : a;
      bnd = bnd > 32 ? 32 : bnd;
      uint32_t w = 0;
      if (bnd > a) w = (bnd == 32 ? 0xffffffffu : ((1u << bnd) - 1u)) & ~((1u << a) - 1u);
      if (ctx.general_mask) w &= mask_bits[base >> 5];
      return w;
    };
    float m_run = -INFINITY;  // running maximum, scaled log2 units
    float l_run = 0.f;
    bool ok = true;
    const int nblk = r.hi - r.lo;
    // The two tiles' warps of one quarter share a scheduler and its MUFU unit.
    // Left alone they fall into step, their exponential bursts collide and the
    // unit idles while both read scores and take maxima. They take turns
    // instead: tile 0 runs the exponentials of its block n, then tile 1 those
    // of its block n, then tile 0 block n+1, ... for the blocks both tiles have,
    // so one tile's TMEM reads and maxima overlap the other's exponentials.
    // The hand-over is a named barrier per (tile, quarter) over the two warps
    // (64 threads): the waiting warp is descheduled and polls nothing, so it
    // takes neither issue slots nor MIO queue entries from the warp that runs.
    // A named barrier has no timeout, so a warp that gives up (a bounded wait
    // ran out) still walks the rest of the hand-over sequence below the loop
    // and its partner is never left waiting.
    const int n_paired = min(r0.hi - r0.lo, r1.hi - r1.lo);
    const int my_turn = 1 + i * 4 + quarter;
    const int other_turn = 1 + (1 - i) * 4 + quarter;
    int turns_done = 0;  // hand-over steps this warp has completed
    // The 64-column score row of this thread. The read of block n+1 is issued
    // at the end of block n whenever those scores are already complete (they
    // usually are: S runs a block ahead), so its latency and the barrier probe
    // hide behind the publication of P(n).
    uint32_t sr[2][32];
    bool requested = false;
    for (int j = r.lo; j < r.hi; ++j) {
      const int n = j - r.lo;
      const int buf = n & 1;
      turns_done = n;
      const uint32_t s_tmem = tmem_base + (uint32_t)((i * 2 + buf) * kBKV) + lane_addr;
      if (!requested) {
        if (!mbar_wait(&s_full[i * 2 + buf], (uint32_t)((n >> 1) & 1), p.status)) {
          ok = false;
          break;
        }
        tc_fence_after();
        tmem_ld32(s_tmem, sr[0]);
        tmem_ld32(s_tmem + 32, sr[1]);
      }
      const int64_t j0 = (int64_t)j * kBKV, j1 = j0 + kBKV - 1;
      bool need_mask = j1 >= ctx.len || ctx.general_mask || p.has_chunk;
      if (p.causal && j1 > i_first) need_mask = true;
      if (p.has_window && (j0 + p.win_left < i_last || j1 > i_first + p.win_right)) need_mask = true;
      if (p.seg_start != nullptr && j0 < seg_last) need_mask = true;

      tmem_ld_wait_for(sr[0]);
      tmem_ld_wait_for(sr[1]);
      if (need_mask) {
        // Hidden scores become -inf: they drop out of the maximum and their
        // probability is 2^(-inf) = 0 (the scale is positive on this path).
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t vw = vis_word((int)j0 + 32 * c);
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (((vw >> e) & 1u) == 0) sr[c][e] = 0xff800000u;
        }
      }
      // row maximum of the raw scores, two new values per instruction
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
      const float mx_t = mx * sl2;  // scale > 0 on this path
      // Lazy rescale: adopt the new maximum only when it grew by more than 2^8.
      float m_new = m_run;
      if (mx_t > m_run + kRescaleAbove || m_run == -INFINITY) m_new = fmaxf(m_run, mx_t);
      // The accumulator is rescaled by warp-wide TMEM accesses, so the branch is
      // taken by the whole warp when any of its rows moved; rows that kept their
      // maximum scale by exactly 1.
      bool tail0_seen = false;
      const bool moved = m_new != m_run && m_run != -INFINITY;
      const float corr = moved ? ex2_approx(m_run - m_new) : 1.0f;
      if (__any_sync(0xffffffffu, moved)) {
        // S runs ahead of P.V: the previous block's P.V may still be in flight.
        // Completion is in issue order, so it has landed once S of the next
        // block is complete (that wait does not consume the phase: the regular
        // wait of block n+1 passes at once afterwards); the tile's last block
        // has no next S and reads the tail barrier's first phase instead.
        const bool landed = n + 1 < nblk
                                ? mbar_wait(&s_full[i * 2 + ((n + 1) & 1)], (uint32_t)(((n + 1) >> 1) & 1), p.status)
                                : mbar_wait(&tail_done[i], 0, p.status);
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
        // tile 1 follows tile 0's block n; tile 0 follows tile 1's block n-1
        named_barrier(my_turn, 64);
        asm volatile("" : "+f"(m_use));  // keeps the exponentials below the barrier
      }
      // p = 2^(s*scale - m) with the scale and the subtraction as packed f32x2
      // FMAs; the row sum is taken from the f32 values, P is rounded to the
      // stream type and written over S.
      const float2 sl2_2 = make_float2(sl2, sl2), nm_2 = make_float2(-m_use, -m_use);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
      uint32_t pk[32];
      // The MUFU unit takes one warp instruction every 8 cycles and returns its
      // result some tens of cycles later. All scaled scores are formed first,
      // then the 64 exponentials are issued back to back while the sums and the
      // 16-bit packing of pair k - kLag run in their shadow, so nothing waits
      // on a result that was only just requested.
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
      // tile 0 waits for tile 1's block n only if it has a paired block n+1
      if (n < n_paired && (i == 0 || n + 1 < n_paired))
        named_barrier_arrive(other_turn, 64);
      turns_done = n + 1;
      l_run += (la.x + la.y) + (lb.x + lb.y);
      requested = false;
      if (n + 1 < nblk &&
          mbar_test_wait(&s_full[i * 2 + (buf ^ 1)], (uint32_t)(((n + 1) >> 1) & 1))) {
        tc_fence_after();
        const uint32_t next_tmem = tmem_base + (uint32_t)((i * 2 + (buf ^ 1)) * kBKV) + lane_addr;
        tmem_ld32(next_tmem, sr[0]);
        tmem_ld32(next_tmem + 32, sr[1]);
        requested = true;
      }
      // Every lane's P stores have completed (wait::st is warp-wide); one lane
      // per warp then publishes the tile to the MMA issuer.
      tmem_st_wait();
      // The tail barrier sees two commits (P.V of blocks N-2 and N-1); a parity
      // wait tells only adjacent phases apart, so the first is observed before
      // the last P — which lets the second happen — is published.
      if (n + 1 == nblk && nblk >= 2 && !tail0_seen && !mbar_wait(&tail_done[i], 0, p.status)) {
        ok = false;
        break;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i * 2 + buf]);
    }
    if (!ok) {
      for (int m = turns_done; m < n_paired; ++m) {
        // arrivals only: the partner is released at each of its remaining turns and
        // this warp never waits on a barrier without a limit again
        if (i == 0 || m + 1 < n_paired) named_barrier_arrive(other_turn, 64);
      }
    }
    // ---- epilogue: O / l ----
    T* orow = (T*)p.o + b * p.o_sb + row * p.o_st + (int64_t)h * p.o_sh;
    if (r.hi > r.lo && ok) {
      // the last P.V: the tail barrier's second phase (its only one for a one-block tile)
      if (mbar_wait(&tail_done[i], nblk >= 2 ? 1u : 0u, p.status)) {
        tc_fence_after();
        const float inv = l_run == 0.f ? 0.f : 1.0f / l_run;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t orr[32];
          tmem_ld32(o_tmem + c, orr);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (c + v * 8 >= p.d_real) break;  // padded head dim: nothing past the real columns
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = Elem<T>::pack(__uint_as_float(orr[v * 8 + 2 * e]) * inv,
                                     __uint_as_float(orr[v * 8 + 2 * e + 1]) * inv);
              stg128(orow + c + v * 8, make_uint4(w[0], w[1], w[2], w[3]));
            }
          }
        }
      }
    } else if (row_ok && ok) {
      // No key block reaches this tile: zeros (attention.rs:971-980).
      for (int c = 0; c < p.d_real; c += 8) stg128(orow + c, make_uint4(0, 0, 0, 0));
    }
    if (p.lse != nullptr && row_ok && ok)
      p.lse[(b * p.heads + h) * p.t + row] = l_run == 0.f ? -INFINITY : kLn2F * (m_run + log2f(l_run));
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


bool aligned16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, int D>
int run(const AttnArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  using C = FaCfg<D>;
  CUtensorMap tq, tk, tv;
  const uint32_t box[4] = {64, 1, 128, 1};     // Q tile rows
  const uint32_t kvbox[4] = {64, 1, kBKV, 1};  // K/V block rows
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
  // the attribute belongs to the device's copy of the kernel: once per device
  static bool attr_seen[64] = {};
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_seen[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_tc_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)C::kSmemBytes) != cudaSuccess)
      return -1;
    attr_set = true;
  }
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
  p.n_qt = (int)((a.t + 2 * kBQ - 1) / (2 * kBQ));
  p.d_real = a.d;
  p.status = a.status;
  dim3 grid((unsigned)p.n_qt, (unsigned)a.heads, (unsigned)a.batch);
  attention_tc_kernel<T, D><<<grid, kThreadsFa, C::kSmemBytes, s>>>(tq, tk, tv, p);
  if (cfg != nullptr)
    snprintf(cfg, cfg_len, "{bq:%d,bkv:%d,d:%d,stages:%d,splits:1}", 2 * kBQ, kBKV, a.d, C::kStages);
  return 0;
}

}  // namespace

bool attention_tc_covers(const AttnArgs& a) {
  // The reference's kernel gate (tk/src/ops/shape.rs:92-99,189-206): one 16-bit
  // dtype. This kernel tiles head dims 64 and 128; every other multiple of 8 up
  // to 128 (the reference plans 32, 48, 64, 128: website/docs/tile-kernels/op-layer.md)
  // runs on the next of the two with the missing columns zero-filled by the TMA
  // loads and never stored. It takes no additive bias and no key splits (the
  // exact kernel serves those), and needs a positive scale because the running
  // maximum is kept in raw-score units.
  if (a.dtype != SVODB_BF16 && a.dtype != SVODB_F16) return false;
  if (a.d < 8 || a.d > 128 || a.d % 8 != 0) return false;
  if (a.bias != nullptr || a.splits > 1 || a.n_app > 0) return false;
  if (!(a.scale > 0.f)) return false;
  if (a.batch <= 0 || a.t <= 0 || a.tk <= 0 || a.batch > 65535 || a.heads > 65535) return false;
  if (a.t > 0x7fffff00LL || a.tk > 0x7fffff00LL) return false;
  if (a.key_mask != nullptr && a.tk > (int64_t)kMaxMaskWords * 32) return false;
  if (a.has_chunk && a.chunk_size <= 0) return false;
  const int64_t strides[] = {a.q_sb, a.q_st, a.q_sh, a.k_sb, a.k_st, a.k_sh, a.v_sb, a.v_st, a.v_sh,
                             a.o_sb, a.o_st, a.o_sh};
  for (int64_t st : strides)
    if (st % 8 != 0) return false;
  if (!aligned16p(a.q) || !aligned16p(a.k) || !aligned16p(a.v) || !aligned16p(a.o)) return false;
  return true;
}

int launch_attention_tc(const AttnArgs& a, cudaStream_t s, char* cfg, size_t cfg_len) {
  if (!attention_tc_covers(a)) return 1;
  if (a.dtype == SVODB_BF16)
    return a.d > 64 ? run<__nv_bfloat16, 128>(a, s, cfg, cfg_len) : run<__nv_bfloat16, 64>(a, s, cfg, cfg_len);
  return a.d > 64 ? run<__half, 128>(a, s, cfg, cfg_len) : run<__half, 64>(a, s, cfg, cfg_len);
}

}  // namespace svodb
