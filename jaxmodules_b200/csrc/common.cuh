// Shared helpers for the blockwise masked attention kernels: status handling, the device
// form of the mask predicate, and small numeric utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bma.h"

namespace bma {

// ---- host-side error plumbing ----------------------------------------------------------
void set_last_cuda_error(cudaError_t e, const char* where);

#define BMA_CUDA_TRY(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      ::bma::set_last_cuda_error(_e, #expr);                 \
      return BMA_ERR_CUDA;                                   \
    }                                                        \
  } while (0)

#define BMA_REQUIRE(cond, code) \
  do {                          \
    if (!(cond)) return (code); \
  } while (0)

// Device-side status word (one per device, lives for the lifetime of the module).  Kernels
// get its address as an argument and record a non-zero code with atomicCAS when a bounded
// wait or a bounds check gives up.  Returns nullptr (and records the CUDA error) on failure.
int* device_status_ptr();

// Host-side count of kernels launched by this library in this process (diagnostics).
void count_launches(int n);

__device__ __forceinline__ void report_device_error(int* status, int code) { atomicCAS(status, 0, code); }

// Terms of the mask that are looked up (segment ids, bit table, tile bits) rather than computed from the indices.
constexpr int kTableTerms = BMA_MASK_SEGMENT | BMA_MASK_BITMAP | BMA_MASK_TILES;

// ---- mask predicate --------------------------------------------------------------------
// Device copy of bma_mask_spec with the per-(b,h) row pointers resolved once per CTA.
struct MaskView {
  int flags;
  int q_valid, k_valid;
  int q_offset, k_offset;
  int band_left, band_right;
  int win_block, win_left, win_right, win_nblk;
  const int32_t* seg_q_row;     // &seg_q[b*stride]
  const int32_t* seg_k_row;
  const uint32_t* bitmap_bh;    // &bitmap[((b%BB)*BH + h%BH) * bitmap_q * words]
  int bitmap_words;
  const uint8_t* tile_class_bh; // TILES: &tile_class[((b%TB)*TH + h%TH) * tiles_q * tiles_k], likewise tile_slot_bh
  const int32_t* tile_slot_bh;
  const uint32_t* tile_bits;
  int tiles_k;
};

__device__ __forceinline__ MaskView make_mask_view(const bma_mask_spec& s, int b, int h) {
  MaskView m;
  m.flags = s.flags;
  m.q_valid = s.q_valid; m.k_valid = s.k_valid;
  m.q_offset = s.q_offset; m.k_offset = s.k_offset;
  m.band_left = s.band_left; m.band_right = s.band_right;
  m.win_block = s.win_block; m.win_left = s.win_left; m.win_right = s.win_right; m.win_nblk = s.win_nblk;
  m.seg_q_row = (s.flags & BMA_MASK_SEGMENT) ? s.seg_q + (int64_t)b * s.seg_q_stride : nullptr;
  m.seg_k_row = (s.flags & BMA_MASK_SEGMENT) ? s.seg_k + (int64_t)b * s.seg_k_stride : nullptr;
  m.bitmap_words = s.bitmap_words;
  m.bitmap_bh = nullptr;
  if (s.flags & BMA_MASK_BITMAP) {
    int64_t bh = (int64_t)(b % s.bitmap_B) * s.bitmap_H + (h % s.bitmap_H);
    m.bitmap_bh = s.bitmap + bh * (int64_t)s.bitmap_q * s.bitmap_words;
  }
  m.tile_class_bh = nullptr; m.tile_slot_bh = nullptr; m.tile_bits = nullptr; m.tiles_k = 0;
  if (s.flags & BMA_MASK_TILES) {
    const int64_t bh = ((int64_t)(b % s.tiles_B) * s.tiles_H + (h % s.tiles_H)) * s.tiles_q * s.tiles_k;
    m.tile_class_bh = s.tile_class + bh;
    m.tile_slot_bh = s.tile_slot + bh;
    m.tile_bits = s.tile_bits;
    m.tiles_k = s.tiles_k;
  }
  return m;
}

// TILES term: the 32 keys [gk32, gk32 + 32) (gk32 a multiple of 32) of global query gq as a bit word.
__device__ __forceinline__ uint32_t tiles_word(const MaskView& m, int gq, int gk32) {
  const int64_t t = (int64_t)(gq >> 7) * m.tiles_k + (gk32 >> 7);
  const int c = __ldg(m.tile_class_bh + t);
  if (c != 1) return c == 2 ? 0xffffffffu : 0u;
  const int slot = __ldg(m.tile_slot_bh + t);
  if (slot < 0) return 0u;   // a cut tile that was not stored (the builder ran out of room): nothing is read
  return __ldg(m.tile_bits + ((int64_t)slot * 256 + (gq & 127)) * 4 + ((gk32 & 127) >> 5));
}
// The transposed copy: the 32 queries [gq32, gq32 + 32) (gq32 a multiple of 32) of global key gk.
__device__ __forceinline__ uint32_t tiles_word_t(const MaskView& m, int gk, int gq32) {
  const int64_t t = (int64_t)(gq32 >> 7) * m.tiles_k + (gk >> 7);
  const int c = __ldg(m.tile_class_bh + t);
  if (c != 1) return c == 2 ? 0xffffffffu : 0u;
  const int slot = __ldg(m.tile_slot_bh + t);
  if (slot < 0) return 0u;
  return __ldg(m.tile_bits + ((int64_t)slot * 256 + 128 + (gk & 127)) * 4 + ((gq32 & 127) >> 5));
}

// First key index and one-past-last key index of the reference's block window for the
// query at global index gq (start clamped like XLA's dynamic_slice).
__device__ __forceinline__ void block_window_range(const MaskView& m, int gq, int& k_lo, int& k_hi) {
  int i = gq / m.win_block;
  int total = m.win_left + m.win_right;
  int s = max(0, i - m.win_left);
  s = min(s, m.win_nblk - total);
  k_lo = s * m.win_block;
  k_hi = (s + total) * m.win_block;
}

// mask_fn(b, h, q, k) for local indices q, k (tile offset + lane offset).
__device__ __forceinline__ bool mask_allowed(const MaskView& m, int q, int k) {
  bool ok = (q < m.q_valid) & (k < m.k_valid);
  const int gq = q + m.q_offset, gk = k + m.k_offset;
  if (m.flags & BMA_MASK_CAUSAL) ok &= (gk <= gq);
  if (m.flags & BMA_MASK_BAND) ok &= (gk >= gq - m.band_left) & (gk <= gq + m.band_right);
  if (m.flags & BMA_MASK_BLOCK_WINDOW) {
    int lo, hi;
    block_window_range(m, gq, lo, hi);
    ok &= (gk >= lo) & (gk < hi);
  }
  if ((m.flags & BMA_MASK_SEGMENT) && ok) ok = (__ldg(m.seg_q_row + gq) == __ldg(m.seg_k_row + gk));
  if ((m.flags & BMA_MASK_BITMAP) && ok)
    ok = (__ldg(m.bitmap_bh + (int64_t)gq * m.bitmap_words + (gk >> 5)) >> (gk & 31)) & 1u;
  if ((m.flags & BMA_MASK_TILES) && ok) ok = (tiles_word(m, gq, gk & ~31) >> (gk & 31)) & 1u;
  return ok;
}

// Bit j of the result: ids[j] == ref for j in [0, n) (n <= 32), 0 for j >= n.  `ids` is a run of
// segment ids in global memory; the common aligned full run is read with four-wide loads.
__device__ __forceinline__ uint32_t seg_equal_bits32(const int32_t* ids, int n, int ref) {
  uint32_t w = 0;
  if (n >= 32 && (reinterpret_cast<uintptr_t>(ids) & 15) == 0) {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
      const int4 v = __ldg(reinterpret_cast<const int4*>(ids) + j4);
      w |= (uint32_t)(v.x == ref) << (j4 * 4);
      w |= (uint32_t)(v.y == ref) << (j4 * 4 + 1);
      w |= (uint32_t)(v.z == ref) << (j4 * 4 + 2);
      w |= (uint32_t)(v.w == ref) << (j4 * 4 + 3);
    }
  } else {
    for (int j = 0; j < 32; ++j)
      if (j < n && __ldg(ids + j) == ref) w |= 1u << j;
  }
  return w;
}

// Bits of the segment and bit-table terms of query row q (local) for the 32 keys starting at local
// key k_start: bit j set = key k_start + j passes both terms.  The interval terms (valid box,
// causal, band, block window) are NOT included; callers AND this with their interval bits.
__device__ __forceinline__ uint32_t table_bits_row32(const MaskView& m, int q, int k_start) {
  uint32_t w = 0xffffffffu;
  if (q >= m.q_valid) return 0u;
  const int gq = q + m.q_offset, gk = k_start + m.k_offset;
  const int n = min(32, m.k_valid - k_start);
  if (n <= 0) return 0u;
  if (m.flags & BMA_MASK_SEGMENT) w &= seg_equal_bits32(m.seg_k_row + gk, n, __ldg(m.seg_q_row + gq));
  if (m.flags & BMA_MASK_BITMAP) {
    const uint32_t* rowp = m.bitmap_bh + (int64_t)gq * m.bitmap_words;
    const int word = gk >> 5, sh = gk & 31;
    uint32_t v = __ldg(rowp + word) >> sh;
    if (sh && word + 1 < m.bitmap_words) v |= __ldg(rowp + word + 1) << (32 - sh);
    w &= v;
  }
  if (m.flags & BMA_MASK_TILES) {   // keys past k_valid fall outside the interval bits the caller ANDs with
    const int sh = gk & 31;
    uint32_t v = tiles_word(m, gq, gk - sh) >> sh;
    if (sh && ((gk - sh + 32) >> 7) < m.tiles_k) v |= tiles_word(m, gq, gk - sh + 32) << (32 - sh);
    w &= v;
  }
  return w;
}

// The same for key row k (local) and the 32 queries starting at local query q_start (bit j =
// query q_start + j).  The bit table is stored by query row, so that term is gathered bit by bit.
__device__ __forceinline__ uint32_t table_bits_col32(const MaskView& m, int k, int q_start) {
  uint32_t w = 0xffffffffu;
  if (k >= m.k_valid) return 0u;
  const int gk = k + m.k_offset, gq = q_start + m.q_offset;
  const int n = min(32, m.q_valid - q_start);
  if (n <= 0) return 0u;
  if (m.flags & BMA_MASK_SEGMENT) w &= seg_equal_bits32(m.seg_q_row + gq, n, __ldg(m.seg_k_row + gk));
  if (m.flags & BMA_MASK_BITMAP) {
    uint32_t v = 0;
    for (int j = 0; j < n; ++j)
      v |= ((__ldg(m.bitmap_bh + (int64_t)(gq + j) * m.bitmap_words + (gk >> 5)) >> (gk & 31)) & 1u) << j;
    w &= v;
  }
  if (m.flags & BMA_MASK_TILES) {   // every cut tile is stored by key row as well: one word per 32 queries
    const int sh = gq & 31;
    uint32_t v = tiles_word_t(m, gk, gq - sh) >> sh;
    if (sh && n > 32 - sh) v |= tiles_word_t(m, gk, gq - sh + 32) << (32 - sh);
    w &= v;             // queries past q_valid fall outside the interval bits the caller ANDs with
  }
  return w;
}

// ---- numeric helpers -------------------------------------------------------------------
__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Host-side dispatchers implemented in the individual .cu files.
int simt_fwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st);
int simt_bwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st);
int sm100_fwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st);
int sm100_bwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, void* ws,
              size_t ws_bytes, const int64_t* visited_host, cudaEvent_t mark, cudaStream_t st);
size_t sm100_bwd_workspace_bytes(const bma_attn_args& a);
size_t sm100_bwd_scratch_bytes(const bma_attn_args& a, const bma_block_lists& lists, const int64_t* visited_host);
size_t sm100_bwd_scratch_min_bytes(const bma_attn_args& a, const bma_block_lists& lists, const int64_t* visited_host);
bool sm100_supported(const bma_attn_args& a);
bool sm100_bwd_supported(const bma_attn_args& a);

// Compact slot addressing of the backward scratch (bwd_slots.cu): tables at the front of the workspace.
struct SlotTables {
  int64_t* head_base;   // [B*Hq + 1] exclusive prefix of visited blocks over (b, h), row-major
  int64_t* head_total;  // [lists.B * lists.H]
  int32_t* row_base;    // [lists.B, lists.H, NQ] exclusive prefix inside a list head
  int32_t* rank;        // [lists.B, lists.H, NQ, NKV] position of kj among the row's visited tiles, -1 = not visited
  size_t bytes;         // size of the tables (a multiple of 1024); the slots follow
};
SlotTables slot_tables_layout(const bma_attn_args& a, const bma_block_lists& l, void* ws);
int slot_tables_build(const bma_attn_args& a, const bma_block_lists& l, const SlotTables& t, cudaStream_t st);
int block_lists_visited(const bma_block_lists& l, int64_t* visited, cudaStream_t st);

constexpr int kSimtTile = 64;
constexpr int kSm100Tile = 128;

}  // namespace bma
