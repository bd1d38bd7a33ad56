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
//                 128 keys through separate shared-memory rings (non-multicast
//                 TMA, 128B swizzle; ragged T / Tk tails zero-filled).
//   warp 1        MMA issuer (one thread): S_i = Q_i.K^T (SS, both K-major) into
//                 TMEM, then O_i += P_i.V with P read from TMEM (TS) and V as the
//                 MN-major shared-memory operand. The two query tiles alternate
//                 (PV_0, QK_0, PV_1, QK_1) so the tensor core works on one tile
//                 while the other tile's softmax runs.
//   warps 2-3     turn a bool key mask into a prefix length or a bitmask.
//   warps 4-7     softmax of tile 0: one query row per thread, S read from TMEM
//   warps 8-11    softmax of tile 1  (tcgen05.ld), P written back over S as
//                 packed 16-bit (tcgen05.st), O rescaled in TMEM when a row's
//                 maximum moves, final O/l -> global.
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D);
// P_i aliases the first 64 columns of S_i.
//
// Every mbarrier wait is bounded; a timeout records a status code and the CTA
// drains and frees its TMEM.
#include <cuda.h>
#include <math.h>
#include <stdio.h>

#include "common.cuh"
#include "kernels.h"
#include "svodb.h"
#include "tensormap.h"

namespace svodb {

namespace {

constexpr int kBQ = 128;   // rows per query tile (two tiles per CTA)
constexpr int kBKV = 128;  // keys per block
constexpr int kThreadsFa = 384;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;
constexpr float kRescaleAbove = 8.0f;
constexpr int kMaxMaskWords = 2048;  // general key mask: up to 65536 keys

template <int D>
struct FaCfg {
  static constexpr int kTileBytes = 128 * D * 2;  // one Q tile / one K block / one V block
  static constexpr int kStages = D == 128 ? 2 : 4;
  static constexpr size_t kSmemBytes =
      1024 + (size_t)(2 + 2 * kStages) * kTileBytes + (size_t)kMaxMaskWords * 4 + 512;
};

struct FaParams {
  void* o;
  int64_t o_sb, o_st, o_sh;
  int64_t t, tk;
  int heads, kv_heads;
  float scale_log2;
  int causal;
  const int32_t* key_lens;
  const void* key_mask;
  int key_mask_i32;
  int has_window;
  int64_t win_left, win_right;
  int has_chunk;
  int64_t chunk_size, chunk_left, chunk_right;
  const int32_t* seg_start;
  float* lse;
  int n_qt;  // query tile pairs per (head, batch)
  uint32_t* status;
};

struct Range {
  int lo, hi;  // key blocks [lo, hi)
};

// The mask context shared by every role of a CTA.
struct Ctx {
  int64_t len;       // visible key count bound: min(Tk, key_lens[b] or the prefix mask's length)
  int general_mask;  // the key mask is not a prefix: consult the bitmask
};

__device__ __forceinline__ Range tile_range(const FaParams& p, const Ctx& c, int64_t b, int64_t i_first) {
  Range r{0, 0};
  if (i_first >= p.t) return r;
  const int64_t i_last = (i_first + kBQ - 1 < p.t - 1) ? i_first + kBQ - 1 : p.t - 1;
  int64_t lo = 0, hi = c.len;
  if (p.causal && i_last + 1 < hi) hi = i_last + 1;
  if (p.has_window) {
    if (i_first - p.win_left > lo) lo = i_first - p.win_left;
    if (i_last + p.win_right + 1 < hi) hi = i_last + p.win_right + 1;
  }
  if (p.has_chunk) {
    const int64_t h2 = (i_last / p.chunk_size + p.chunk_right + 1) * p.chunk_size;
    if (h2 < hi) hi = h2;
    if (p.chunk_left >= 0) {
      const int64_t l2 = (i_first / p.chunk_size - p.chunk_left) * p.chunk_size;
      if (l2 > lo) lo = l2;
    }
  }
  if (p.seg_start != nullptr) {
    const int64_t s = p.seg_start[b * p.t + i_first];
    if (s > lo) lo = s;
  }
  if (hi <= lo) return r;
  r.lo = (int)(lo / kBKV);
  r.hi = (int)((hi + kBKV - 1) / kBKV);
  return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreadsFa, 1)
    attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using C = FaCfg<D>;
  constexpr int S = C::kStages;
  constexpr int TB = C::kTileBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                         // [2][TB]
  uint8_t* k_s = q_s + 2 * TB;                 // [S][TB]
  uint8_t* v_s = k_s + S * TB;                 // [S][TB]
  uint32_t* mask_bits = reinterpret_cast<uint32_t*>(v_s + S * TB);  // [kMaxMaskWords]
  uint64_t* bars = reinterpret_cast<uint64_t*>(mask_bits + kMaxMaskWords);
  uint64_t* q_full = bars;                     // [2]
  uint64_t* k_full = bars + 2;                 // [S]
  uint64_t* k_empty = k_full + S;
  uint64_t* v_full = k_empty + S;
  uint64_t* v_empty = v_full + S;
  uint64_t* s_full = v_empty + S;              // [2]
  uint64_t* p_full = s_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_full + 2);
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
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp
    }
    for (int i = 0; i < S; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
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
    if (first_zero >= last_set) {
      // Set bits form a prefix [0, last_set).
      if (last_set < ctx.len) ctx.len = last_set;
    } else {
      ctx.general_mask = 1;
      if (last_set < ctx.len) ctx.len = last_set;
    }
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

  // Register budget: the loader / MMA / mask warpgroup gives registers back so
  // the two softmax warpgroups can hold a whole 128-column score row each.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
  if (warp == 0) {
    // ---------------- TMA loader ----------------
    if (lane == 0 && u_hi > u_lo) {
      for (int i = 0; i < 2; ++i) {
        if (i == 0 ? live0 : live1) {
          mbar_expect_tx(&q_full[i], TB);
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(q_s + i * TB + c * (128 * 128), &tmap_q, &q_full[i], c * 64, h, (int)(i0 + i * kBQ), (int)b);
        }
      }
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int issued = 0;
      for (int j = u_lo; j < u_hi; ++j) {
        if (!mbar_wait(&k_empty[s], ph ^ 1, p.status)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&k_full[s], TB);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(k_s + s * TB + c * (128 * 128), &tmap_k, &k_full[s], c * 64, hk, j * kBKV, (int)b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, p.status)) {
          ok = false;
          // the K copy just issued is drained below
          ++issued;
          break;
        }
        mbar_expect_tx(&v_full[s], TB);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(v_s + s * TB + c * (128 * 128), &tmap_v, &v_full[s], c * 64, hk, j * kBKV, (int)b);
        ++issued;
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
        (void)issued;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && u_hi > u_lo) {
      constexpr uint32_t idesc_qk = umma_idesc(Elem<T>::kUmmaFormat, 128, kBKV, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(Elem<T>::kUmmaFormat, 128, D, 0, 1);
      const uint64_t q_desc0 = umma_desc_sw128(smem_u32(q_s), 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(k_s), 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(v_s), 128 * 128, 1024);
      bool ok = true;
      bool q_ready[2] = {false, false};
      bool pending[2] = {false, false};   // a P.V of the previous block is owed
      bool o_started[2] = {false, false};
      uint32_t p_phase[2] = {0, 0};
      int s = 0;            // ring slot of block j
      uint32_t ph = 0;
      int s_prev = 0;       // ring slot of block j-1
      for (int j = u_lo; j <= u_hi && ok; ++j) {
        const bool have_block = j < u_hi;
        if (have_block) {
          if (!mbar_wait(&k_full[s], ph, p.status)) {
            ok = false;
            break;
          }
        }
        bool v_waited = false;
        for (int i = 0; i < 2 && ok; ++i) {
          const Range& r = i == 0 ? r0 : r1;
          if (pending[i]) {
            // O_i += P_i(j-1) . V(j-1)
            if (!v_waited) {
              // V of block j-1 sits in slot s_prev; its phase is that block's lap of the ring.
              if (!mbar_wait(&v_full[s_prev], (uint32_t)(((j - 1 - u_lo) / S) & 1), p.status)) {
                ok = false;
                break;
              }
              v_waited = true;
            }
            if (!mbar_wait(&p_full[i], p_phase[i], p.status)) {
              ok = false;
              break;
            }
            p_phase[i] ^= 1;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + 256 + i * D;
            const uint32_t a_tmem = tmem_base + i * 128;
            // V block: [keys][D] with 64-wide column boxes 16 KiB apart (LBO),
            // 8-key groups 1 KiB apart (SBO); 16 keys per step = 2 KiB. Descriptors
            // are formed per step from one base.
            const uint64_t v_base = v_desc0 + (uint64_t)((s_prev * TB) >> 4);
            const uint32_t first = o_started[i] ? 1u : 0u;
#pragma unroll
            for (int ks = 0; ks < kBKV / 16; ++ks)
              umma_ts(d_tmem, a_tmem + ks * 8, v_base + (uint64_t)(ks * (2048 >> 4)), idesc_pv, (first | (uint32_t)ks) != 0 ? 1u : 0u);
            o_started[i] = true;
            pending[i] = false;
          }
          if (have_block && j >= r.lo && j < r.hi) {
            if (!q_ready[i]) {
              if (!mbar_wait(&q_full[i], 0, p.status)) {
                ok = false;
                break;
              }
              q_ready[i] = true;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + i * 128;
            const uint64_t qa = q_desc0 + (uint64_t)((i * TB) >> 4);
            const uint64_t kb = k_desc0 + (uint64_t)((s * TB) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              // 16 columns = 32 bytes inside a 64-column box; boxes are 16 KiB apart
              const uint64_t off = (uint64_t)((ks >> 2) * ((128 * 128) >> 4) + (ks & 3) * 2);
              umma_ss(d_tmem, qa + off, kb + off, idesc_qk, ks != 0 ? 1u : 0u);
            }
            tc_commit(&s_full[i]);
            pending[i] = true;
          } else if (j > r.lo && j == r.hi && r.hi > r.lo) {
            // Tile i's last P.V was just issued: publish its finished O.
            tc_commit(&s_full[i]);
          }
        }
        if (!ok) break;
        if (j > u_lo) tc_commit(&v_empty[s_prev]);  // both tiles' P.V of block j-1 are issued
        if (have_block) {
          tc_commit(&k_empty[s]);
          s_prev = s;
          if (++s == S) {
            s = 0;
            ph ^= 1;
          }
        }
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
    const uint32_t s_tmem = tmem_base + i * 128 + lane_addr;
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
    uint32_t s_phase = 0;
    bool ok = true;
    for (int j = r.lo; j < r.hi; ++j) {
      if (!mbar_wait(&s_full[i], s_phase, p.status)) {
        ok = false;
        break;
      }
      s_phase ^= 1;
      tc_fence_after();
      const int64_t j0 = (int64_t)j * kBKV, j1 = j0 + kBKV - 1;
      bool need_mask = j1 >= ctx.len || ctx.general_mask || p.has_chunk;
      if (p.causal && j1 > i_first) need_mask = true;
      if (p.has_window && (j0 + p.win_left < i_last || j1 > i_first + p.win_right)) need_mask = true;
      if (p.seg_start != nullptr && j0 < seg_last) need_mask = true;

      // The whole 128-column score row of this thread is read once, with the
      // four loads in flight together.
      uint32_t sr[4][32];
      tmem_ld32(s_tmem, sr[0]);
      tmem_ld32(s_tmem + 32, sr[1]);
      tmem_ld32(s_tmem + 64, sr[2]);
      tmem_ld32(s_tmem + 96, sr[3]);
      tmem_ld_wait();
      if (need_mask) {
        // Hidden scores become -inf: they drop out of the maximum and their
        // probability is 2^(-inf) = 0 (the scale is positive on this path).
#pragma unroll
        for (int c = 0; c < 4; ++c) {
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
        for (int c = 0; c < 4; ++c) {
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
      const bool moved = m_new != m_run && m_run != -INFINITY;
      const float corr = moved ? ex2_approx(m_run - m_new) : 1.0f;
      if (__any_sync(0xffffffffu, moved)) {
        l_run *= corr;
        // O_i holds the sum over earlier blocks; its last P.V completed before
        // this block's S was published.
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
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      // p = 2^(s*scale - m) with the scale and the subtraction as packed f32x2
      // FMAs; the row sum is taken from the f32 values, P is rounded to the
      // stream type and written over S.
      const float2 sl2_2 = make_float2(sl2, sl2), nm_2 = make_float2(-m_use, -m_use);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float2 x0 = __ffma2_rn(make_float2(__uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1])), sl2_2, nm_2);
          float2 x1 = __ffma2_rn(make_float2(__uint_as_float(sr[c][e + 2]), __uint_as_float(sr[c][e + 3])), sl2_2, nm_2);
          x0.x = ex2_approx(x0.x);
          x0.y = ex2_approx(x0.y);
          x1.x = ex2_approx(x1.x);
          x1.y = ex2_approx(x1.y);
          la = __fadd2_rn(la, x0);
          lb = __fadd2_rn(lb, x1);
          pk[e / 2] = Elem<T>::pack(x0.x, x0.y);
          pk[e / 2 + 1] = Elem<T>::pack(x1.x, x1.y);
        }
        tmem_st16(s_tmem + 16 * c, pk);
      }
      const float l0 = la.x + la.y, l1 = lb.x + lb.y, l2 = 0.f, l3 = 0.f;
      l_run += (l0 + l1) + (l2 + l3);
      // Every lane's P stores have completed (wait::st is warp-wide); one lane
      // per warp then publishes the tile to the MMA issuer.
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i]);
    }
    // ---- epilogue: O / l ----
    T* orow = (T*)p.o + b * p.o_sb + row * p.o_st + (int64_t)h * p.o_sh;
    if (r.hi > r.lo && ok) {
      if (mbar_wait(&s_full[i], s_phase, p.status)) {
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
      for (int c = 0; c < D; c += 8) stg128(orow + c, make_uint4(0, 0, 0, 0));
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
  const uint32_t box[4] = {64, 1, 128, 1};
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)a.heads, (uint64_t)a.t, (uint64_t)a.batch};
    const uint64_t st[3] = {(uint64_t)a.q_sh, (uint64_t)a.q_st, (uint64_t)a.q_sb};
    if (!make_tmap(&tq, a.q, a.dtype, 4, dims, st, box)) return -1;
  }
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)a.kv_heads, (uint64_t)a.tk, (uint64_t)a.batch};
    const uint64_t stk[3] = {(uint64_t)a.k_sh, (uint64_t)a.k_st, (uint64_t)a.k_sb};
    const uint64_t stv[3] = {(uint64_t)a.v_sh, (uint64_t)a.v_st, (uint64_t)a.v_sb};
    if (!make_tmap(&tk, a.k, a.dtype, 4, dims, stk, box)) return -1;
    if (!make_tmap(&tv, a.v, a.dtype, 4, dims, stv, box)) return -1;
  }
  static bool attr_set = false;
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
  p.lse = a.lse;
  p.n_qt = (int)((a.t + 2 * kBQ - 1) / (2 * kBQ));
  p.status = a.status;
  dim3 grid((unsigned)p.n_qt, (unsigned)a.heads, (unsigned)a.batch);
  attention_tc_kernel<T, D><<<grid, kThreadsFa, C::kSmemBytes, s>>>(tq, tk, tv, p);
  if (cfg != nullptr)
    snprintf(cfg, cfg_len, "{bq:%d,bkv:%d,d:%d,stages:%d,splits:1}", 2 * kBQ, kBKV, D, C::kStages);
  return 0;
}

}  // namespace

bool attention_tc_covers(const AttnArgs& a) {
  // The reference's kernel gate (tk/src/ops/shape.rs:92-99,189-206): one 16-bit
  // dtype. This kernel tiles head dims 64 and 128, takes no additive bias and no
  // key splits (the exact kernel serves those), and needs a positive scale
  // because the running maximum is kept in raw-score units.
  if (a.dtype != SVODB_BF16 && a.dtype != SVODB_F16) return false;
  if (a.d != 64 && a.d != 128) return false;
  if (a.bias != nullptr || a.splits > 1) return false;
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
    return a.d == 128 ? run<__nv_bfloat16, 128>(a, s, cfg, cfg_len) : run<__nv_bfloat16, 64>(a, s, cfg, cfg_len);
  return a.d == 128 ? run<__half, 128>(a, s, cfg, cfg_len) : run<__half, 64>(a, s, cfg, cfg_len);
}

}  // namespace svodb
