// Pieces shared by the tcgen05 flash-attention kernels: tile constants, the
// parameter block, the per-tile key-block range under the masks.
#pragma once

#include <stdint.h>

#include "common.cuh"

namespace svodb {
namespace fa_parts {

constexpr int kBQ = 128;   // rows per query tile (two tiles per CTA)
constexpr int kBKV = 64;   // keys per block
constexpr int kThreadsFa = 384;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;
constexpr float kRescaleAbove = 8.0f;
constexpr int kMaxMaskWords = 2048;  // general key mask: up to 65536 keys

template <int D>
struct FaCfg {
  static constexpr int kQTileBytes = 128 * D * 2;   // one 128-row Q tile
  static constexpr int kKvBytes = kBKV * D * 2;     // one K or V block
  static constexpr int kStages = 4;
  static constexpr size_t kSmemBytes =
      1024 + (size_t)2 * kQTileBytes + (size_t)2 * kStages * kKvBytes + (size_t)kMaxMaskWords * 4 + 512;
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
  const int32_t* row_map;  // `ops::Cache`: cache row of batch lane b, or null
  float* lse;
  int n_qt;  // work items per (head or head pair, batch): pairs of 128-row tiles, or 128-row tiles when pair_heads
  // How an item's two query tiles are chosen (persistent kernel): 0 = two consecutive
  // 128-row tiles of one head; 1 = the SAME 128-row tile of two consecutive query
  // heads that share a KV head (grouped-query attention with an even group), so that
  // under a causal mask or a window both tiles walk the same key blocks and end together.
  int pair_heads;
  int d_real;  // the tensors' head dim (a multiple of 8, <= D): columns past it are TMA zero fill and never stored
  // Key splits (persistent kernel): split s of `splits` takes an equal share of the
  // key blocks and writes its unnormalised state instead of the output:
  // o_part [S,B,T,H,d] f32, m_part / l_part [S,B,T,H] (m in scaled log2 units,
  // -1e30 for a share no key reached: tk/src/kernels/attention.rs:616,910-920).
  int splits;
  int64_t batch;
  float* o_part;
  float* m_part;
  float* l_part;
  // Additive bias [B|1, H, T, Tk] in the stream dtype (persistent kernel), added to
  // the scaled score before the masks (attention.rs:405-407).
  const void* bias;
  int bias_per_batch;
  float inv_scale;  // 1 / scale: the bias in raw-score units
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

}  // namespace fa_parts
}  // namespace svodb
