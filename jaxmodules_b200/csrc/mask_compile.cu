// Block-mask compilation (integer work, HBM-write bound).
//
// Produces the arrays of the reference's BlockMask (jaxmodules/block_mask.py:17-42) for a
// device-evaluable mask description, bit-exact with what create_block_mask
// (jaxmodules/block_mask.py:454-498) followed by BlockMask.from_blocks (:227-275) and
// get_sparse_{kv,q}_data_from_blocks (:411-451) returns:
//   pass 0 (only for segment masks)  per-block min/max of the segment ids
//   pass 1 classify                  one flag byte per block: 0 empty, 1 partial (any ^ all), 2 full (all)
//   pass 2 compact                   per row: count + [set indices ascending, unset indices ascending]
//                                    (== stable argsort(-blocks)), once along kv and once along q.
// The reference evaluates the dense B*H*Q*KV mask twice; here structured masks are classified
// from interval arithmetic on the block corners, and only blocks that a segment boundary or a
// bitmap touches are scanned element by element.  Masks that do not depend on b or h are
// classified once and the rows are replicated on the way out, so the cost is writing the
// int32 lists.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace bma {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxRowWidth = 16384;  // widest index row kept in shared memory (2 rows * 4 B * width)

__host__ __device__ inline bool depends_on_b(const bma_mask_spec& s) {
  return (s.flags & BMA_MASK_SEGMENT) || ((s.flags & BMA_MASK_BITMAP) && s.bitmap_B > 1) ||
         ((s.flags & BMA_MASK_TILES) && s.tiles_B > 1);
}
__host__ __device__ inline bool depends_on_h(const bma_mask_spec& s) {
  return ((s.flags & BMA_MASK_BITMAP) && s.bitmap_H > 1) || ((s.flags & BMA_MASK_TILES) && s.tiles_H > 1);
}

struct SegSummary {  // workspace views, each [B, nblocks]
  int32_t* qmin; int32_t* qmax; int32_t* kmin; int32_t* kmax;
};

// pass 0: min / max segment id of every q block and every kv block (valid part only).
__global__ void seg_summary_kernel(bma_mask_spec spec, int B, int NQ, int NKV, int QB, int KVB, SegSummary out) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int64_t total = (int64_t)B * (NQ + NKV);
  for (int64_t w = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); w < total;
       w += (int64_t)gridDim.x * warps_per_cta) {
    const int b = (int)(w / (NQ + NKV));
    const int r = (int)(w % (NQ + NKV));
    const bool is_q = r < NQ;
    const int blk = is_q ? r : r - NQ;
    const int bs = is_q ? QB : KVB;
    const int valid = is_q ? spec.q_valid : spec.k_valid;
    const int off = is_q ? spec.q_offset : spec.k_offset;
    const int32_t* row = is_q ? spec.seg_q + (int64_t)b * spec.seg_q_stride : spec.seg_k + (int64_t)b * spec.seg_k_stride;
    const int lo = blk * bs, hi = min(lo + bs, valid);
    int mn = INT32_MAX, mx = INT32_MIN;
    for (int i = lo + lane; i < hi; i += 32) {
      int v = __ldg(row + off + i);
      mn = min(mn, v);
      mx = max(mx, v);
    }
    for (int o = 16; o; o >>= 1) {
      mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
      if (is_q) { out.qmin[(int64_t)b * NQ + blk] = mn; out.qmax[(int64_t)b * NQ + blk] = mx; }
      else      { out.kmin[(int64_t)b * NKV + blk] = mn; out.kmax[(int64_t)b * NKV + blk] = mx; }
    }
  }
}

// Exact any/all of the interval terms (valid box, causal, band, block window) on one block.
// Returns false when the block window changes inside the q block, in which case the caller
// has to scan.  any/all are only meaningful when true is returned.
__device__ __forceinline__ bool interval_classify(const bma_mask_spec& s, int q0, int k0, int QB, int KVB,
                                                  bool& any, bool& all) {
  const int qa = q0, qb = min(q0 + QB, s.q_valid) - 1;
  const int ka = k0, kb = min(k0 + KVB, s.k_valid) - 1;
  any = false; all = false;
  if (qb < qa || kb < ka) return true;
  const bool whole = (q0 + QB <= s.q_valid) && (k0 + KVB <= s.k_valid);
  const int64_t gqa = (int64_t)qa + s.q_offset, gqb = (int64_t)qb + s.q_offset;
  int64_t gka = (int64_t)ka + s.k_offset, gkb = (int64_t)kb + s.k_offset;
  int64_t lo = INT64_MIN / 4, hi = INT64_MAX / 4;
  if (s.flags & BMA_MASK_CAUSAL) hi = min(hi, (int64_t)0);
  if (s.flags & BMA_MASK_BAND) { lo = max(lo, -(int64_t)s.band_left); hi = min(hi, (int64_t)s.band_right); }
  bool window_covers = true;
  int64_t aka = gka, akb = gkb;  // key range after intersecting with the window (for "any")
  if (s.flags & BMA_MASK_BLOCK_WINDOW) {
    if (gqa / s.win_block != gqb / s.win_block) return false;
    const int total = s.win_left + s.win_right;
    int64_t st = max((int64_t)0, gqa / s.win_block - s.win_left);
    st = min(st, (int64_t)s.win_nblk - total);
    const int64_t wlo = st * s.win_block, whi = (st + total) * s.win_block;
    window_covers = (gka >= wlo) && (gkb < whi);
    aka = max(gka, wlo);
    akb = min(gkb, whi - 1);
  }
  // k - q takes every integer value in [aka - gqb, akb - gqa] on the box
  any = (aka <= akb) && (max(lo, aka - gqb) <= min(hi, akb - gqa));
  all = whole && window_covers && (gka - gqb >= lo) && (gkb - gqa <= hi);
  return true;
}

// pass 1a: one THREAD per block.  Interval terms and the per-block segment-id ranges decide almost every
// block in closed form; flags leave as coalesced bytes.  The few blocks that stay open (a segment boundary,
// a bit table or a change of the block window inside the block) are appended to a work list for pass 1b.
// The list and its counter live in output arrays that pass 2 overwrites afterwards (`todo` = kv_idx, one
// int32 per block at least; `todo_count` = kv_num[0]), so the scratch stays at one byte per block.
struct BlockCoord { int cb, ch, qi, kj; };
__device__ __forceinline__ BlockCoord block_coord(int64_t w, int CH, int NQ, int NKV) {
  BlockCoord c;
  const int64_t row = w / NKV;
  c.kj = (int)(w - row * NKV);
  uint32_t r = (uint32_t)row;
  c.qi = (int)(r % (uint32_t)NQ);
  r /= (uint32_t)NQ;
  c.ch = (int)(r % (uint32_t)CH);
  c.cb = (int)(r / (uint32_t)CH);
  return c;
}

__global__ void classify_kernel(bma_mask_spec spec, int CB, int CH, int NQ, int NKV, int QB, int KVB,
                                SegSummary seg, uint8_t* __restrict__ flags, int32_t* __restrict__ todo,
                                int32_t* __restrict__ todo_count) {
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)CB * CH * NQ * NKV;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // `base` is the warp's first block: uniform across the warp, so the ballot below sees all 32 lanes
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31); base < total; base += stride) {
    const int64_t w = base + lane;
    const bool valid = w < total;
    bool any = false, all = false, scan = false;
    if (valid) {
      const BlockCoord c = block_coord(w, CH, NQ, NKV);
      const bool decided = interval_classify(spec, c.qi * QB, c.kj * KVB, QB, KVB, any, all);
      scan = !decided;
      if (decided && any && (spec.flags & BMA_MASK_SEGMENT)) {
        const int qmn = seg.qmin[(int64_t)c.cb * NQ + c.qi], qmx = seg.qmax[(int64_t)c.cb * NQ + c.qi];
        const int kmn = seg.kmin[(int64_t)c.cb * NKV + c.kj], kmx = seg.kmax[(int64_t)c.cb * NKV + c.kj];
        if (qmx < kmn || qmn > kmx) { any = false; all = false; }          // ids never meet
        else if (!(qmn == qmx && kmn == kmx && qmn == kmn)) {                 // a boundary crosses the block
          if (spec.flags & BMA_MASK_COMPILE_CONSERVATIVE) all = false;        // "partial" without looking closer
          else scan = true;
        }
      }
      if (decided && any && (spec.flags & BMA_MASK_BITMAP)) scan = true;
      if (decided && any && (spec.flags & BMA_MASK_TILES)) {
        // a block that IS a stored tile takes the tile's class (exactly, when no other term cuts the block); any other
        // block geometry is scanned element by element
        const bool is_tile = QB == 128 && KVB == 128 && (spec.q_offset & 127) == 0 && (spec.k_offset & 127) == 0;
        if (!is_tile) scan = true;
        else {
          const int64_t t = (((int64_t)(c.cb % spec.tiles_B) * spec.tiles_H + (c.ch % spec.tiles_H)) * spec.tiles_q +
                             ((c.qi * QB + spec.q_offset) >> 7)) * spec.tiles_k + ((c.kj * KVB + spec.k_offset) >> 7);
          const int tc = spec.tile_class[t];
          if (tc == 0) { any = false; all = false; }
          else if (tc == 1) {
            if (all || (spec.flags & BMA_MASK_COMPILE_CONSERVATIVE)) all = false;   // cut by the tile alone: partial
            else scan = true;                                                        // cut by two terms: may be empty
          }
        }
      }
      flags[w] = all ? 2 : (any ? 1 : 0);   // rewritten by pass 1b when `scan`
    }
    const unsigned m = __ballot_sync(0xffffffffu, scan);
    if (m != 0u) {  // one atomic per warp
      const int leader = __ffs(m) - 1;
      int pos = 0;
      if (lane == leader) pos = atomicAdd(todo_count, __popc(m));
      pos = __shfl_sync(0xffffffffu, pos, leader);
      if (scan) todo[pos + __popc(m & ((1u << lane) - 1u))] = (int32_t)w;
    }
  }
}

// pass 1b: one WARP per listed block: exact any/all by evaluating the mask on every element
// (stops as soon as the block is known to be partial).
__global__ void scan_kernel(bma_mask_spec spec, int CH, int NQ, int NKV, int QB, int KVB, uint8_t* __restrict__ flags,
                            const int32_t* __restrict__ todo, const int32_t* __restrict__ todo_count) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int count = *todo_count;
  for (int i = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); i < count; i += gridDim.x * warps_per_cta) {
    const int64_t w = todo[i];
    const BlockCoord c = block_coord(w, CH, NQ, NKV);
    const MaskView m = make_mask_view(spec, c.cb, c.ch);
    const int q0 = c.qi * QB, k0 = c.kj * KVB;
    const int qb_end = min(q0 + QB, spec.q_valid), kb_end = min(k0 + KVB, spec.k_valid);
    bool any = false;
    bool all = (q0 + QB <= spec.q_valid) && (k0 + KVB <= spec.k_valid);
    for (int q = q0; q < qb_end && !(any && !all); ++q) {
      for (int kb = k0; kb < kb_end; kb += 32) {
        const int k = kb + lane;
        const bool in = k < kb_end;
        const bool ok = in && mask_allowed(m, q, k);
        const unsigned okb = __ballot_sync(0xffffffffu, ok);
        const unsigned inb = __ballot_sync(0xffffffffu, in);
        any |= (okb != 0u);
        all &= (okb == inb);
      }
    }
    if (lane == 0) flags[w] = all ? 2 : (any ? 1 : 0);
  }
}

// pass 2: one CTA per (classification row, replica chunk).  TRANSPOSED = q-side lists.
// Shared memory: 2 index rows of `NC` int32, the row's `NC` flag bytes, + scan scratch.
template <bool TRANSPOSED>
__device__ __forceinline__ void compact_row(const uint8_t* __restrict__ flags, int CB, int CH, int NQ, int NKV, int out_B,
                                            int out_H, int32_t* __restrict__ part_num, int32_t* __restrict__ part_idx,
                                            int32_t* __restrict__ full_num, int32_t* __restrict__ full_idx) {
  extern __shared__ int32_t smem[];
  const int NR = TRANSPOSED ? NKV : NQ;   // rows of the output
  const int NC = TRANSPOSED ? NQ : NKV;   // row width
  int32_t* row_p = smem;
  int32_t* row_f = smem + NC;
  __shared__ int warp_p[kThreads / 32], warp_f[kThreads / 32];
  __shared__ int tot_p, tot_f;

  const int r = blockIdx.x % NR;
  const int ch = (blockIdx.x / NR) % CH;
  const int cb = blockIdx.x / (NR * CH);
  const uint8_t* fbase = flags + (int64_t)(cb * CH + ch) * NQ * NKV;
  // the row's flags go to shared memory first: all loads of a thread are in flight together (a column of the
  // flag grid, for the q-side lists, is one byte per 32-byte sector), and both passes below read them twice
  uint8_t* fl = reinterpret_cast<uint8_t*>(smem + 2 * NC);
  for (int c = threadIdx.x; c < NC; c += kThreads) fl[c] = TRANSPOSED ? fbase[(int64_t)c * NKV + r] : fbase[(int64_t)r * NKV + c];
  __syncthreads();
  auto flag_at = [&](int c) -> int { return fl[c]; };

  const int per = (NC + kThreads - 1) / kThreads;
  const int c0 = min(NC, (int)threadIdx.x * per), c1 = min(NC, c0 + per);
  int np = 0, nf = 0;
  for (int c = c0; c < c1; ++c) {
    const int f = flag_at(c);
    np += (f == 1);
    nf += (f == 2);
  }
  // exclusive block scan of (np, nf)
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int sp = np, sf = nf;
  for (int o = 1; o < 32; o <<= 1) {
    int tp = __shfl_up_sync(0xffffffffu, sp, o), tf = __shfl_up_sync(0xffffffffu, sf, o);
    if (lane >= o) { sp += tp; sf += tf; }
  }
  if (lane == 31) { warp_p[wid] = sp; warp_f[wid] = sf; }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ap = 0, af = 0;
    for (int i = 0; i < kThreads / 32; ++i) {
      int tp = warp_p[i], tf = warp_f[i];
      warp_p[i] = ap; warp_f[i] = af;
      ap += tp; af += tf;
    }
    tot_p = ap; tot_f = af;
  }
  __syncthreads();
  int before_p = warp_p[wid] + sp - np, before_f = warp_f[wid] + sf - nf;
  const int total_p = tot_p, total_f = tot_f;
  for (int c = c0; c < c1; ++c) {
    const int f = flag_at(c);
    if (f == 1) row_p[before_p++] = c; else row_p[total_p + (c - before_p)] = c;
    if (f == 2) row_f[before_f++] = c; else row_f[total_f + (c - before_f)] = c;
  }
  __syncthreads();

  // replicate to every (b, h) of the output that this classification row stands for
  const int rep_b = (CB == out_B) ? 1 : out_B, rep_h = (CH == out_H) ? 1 : out_H;
  const int reps = rep_b * rep_h;
  for (int rep = blockIdx.y; rep < reps; rep += gridDim.y) {
    const int b = (CB == out_B) ? cb : rep / rep_h;
    const int h = (CH == out_H) ? ch : rep % rep_h;
    const int64_t row = ((int64_t)b * out_H + h) * NR + r;
    if (threadIdx.x == 0) { part_num[row] = total_p; full_num[row] = total_f; }
    int32_t* dp = part_idx + row * NC;
    int32_t* df = full_idx + row * NC;
    if ((NC & 3) == 0 && (((uintptr_t)part_idx | (uintptr_t)full_idx) & 15) == 0) {
      const int4* sp4 = reinterpret_cast<const int4*>(row_p);
      const int4* sf4 = reinterpret_cast<const int4*>(row_f);
      for (int i = threadIdx.x; i < NC / 4; i += kThreads) {
        reinterpret_cast<int4*>(dp)[i] = sp4[i];
        reinterpret_cast<int4*>(df)[i] = sf4[i];
      }
    } else {
      for (int i = threadIdx.x; i < NC; i += kThreads) { dp[i] = row_p[i]; df[i] = row_f[i]; }
    }
  }
}

template <bool TRANSPOSED>
__global__ void compact_kernel(const uint8_t* __restrict__ flags, int CB, int CH, int NQ, int NKV, int out_B,
                               int out_H, int32_t* __restrict__ part_num, int32_t* __restrict__ part_idx,
                               int32_t* __restrict__ full_num, int32_t* __restrict__ full_idx) {
  compact_row<TRANSPOSED>(flags, CB, CH, NQ, NKV, out_B, out_H, part_num, part_idx, full_num, full_idx);
}

// Both list sides in ONE launch (blockIdx.z = 0: kv side, 1: q side): no launch gap between them, and the tail of one
// side fills with the other's rows.  The builder is bound by the HBM writes of the index arrays.
__global__ void compact_both_kernel(const uint8_t* __restrict__ flags, int CB, int CH, int NQ, int NKV, int out_B, int out_H,
                                    bma_block_lists l) {
  if (blockIdx.z == 0) {
    if ((int)blockIdx.x < CB * CH * NQ)
      compact_row<false>(flags, CB, CH, NQ, NKV, out_B, out_H, l.kv_num, l.kv_idx, l.full_kv_num, l.full_kv_idx);
  } else {
    if ((int)blockIdx.x < CB * CH * NKV)
      compact_row<true>(flags, CB, CH, NQ, NKV, out_B, out_H, l.q_num, l.q_idx, l.full_q_num, l.full_q_idx);
  }
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspacePlan {
  size_t flags_off, seg_off, total;
  int CB, CH;
};

WorkspacePlan plan_workspace(const bma_mask_spec& s, int B, int H, int NQ, int NKV) {
  WorkspacePlan p;
  p.CB = depends_on_b(s) ? B : 1;
  p.CH = depends_on_h(s) ? H : 1;
  p.flags_off = 0;
  size_t flags_bytes = (size_t)p.CB * p.CH * NQ * NKV;
  p.seg_off = align_up(flags_bytes, 256);
  size_t seg_bytes = (s.flags & BMA_MASK_SEGMENT) ? sizeof(int32_t) * 2 * (size_t)B * (NQ + NKV) : 0;
  p.total = p.seg_off + align_up(seg_bytes, 256);
  return p;
}

}  // namespace

size_t mask_compile_workspace_bytes(const bma_mask_spec& spec, int B, int H, int NQ, int NKV) {
  return plan_workspace(spec, B, H, NQ, NKV).total;
}

int mask_compile_validate(const bma_mask_spec& s, int B, int H, const bma_block_lists& l) {
  BMA_REQUIRE(B > 0 && H > 0 && l.NQ > 0 && l.NKV > 0 && l.q_block > 0 && l.kv_block > 0, BMA_ERR_ARG);
  BMA_REQUIRE(l.kv_num && l.kv_idx && l.full_kv_num && l.full_kv_idx, BMA_ERR_ARG);
  const bool any_q = l.q_num || l.q_idx || l.full_q_num || l.full_q_idx;
  const bool all_q = l.q_num && l.q_idx && l.full_q_num && l.full_q_idx;
  BMA_REQUIRE(!any_q || all_q, BMA_ERR_ARG);
  BMA_REQUIRE((l.B == B || (l.B == 1 && !depends_on_b(s))) && (l.H == H || (l.H == 1 && !depends_on_h(s))), BMA_ERR_ARG);
  BMA_REQUIRE(s.q_valid >= 0 && s.k_valid >= 0, BMA_ERR_ARG);
  BMA_REQUIRE((int64_t)l.NQ * l.q_block >= s.q_valid && (int64_t)l.NKV * l.kv_block >= s.k_valid, BMA_ERR_ARG);
  if (s.flags & BMA_MASK_SEGMENT) BMA_REQUIRE(s.seg_q && s.seg_k, BMA_ERR_ARG);
  if (s.flags & BMA_MASK_BITMAP)
    BMA_REQUIRE(s.bitmap && s.bitmap_B > 0 && s.bitmap_H > 0 && s.bitmap_words > 0 && s.bitmap_q > 0, BMA_ERR_ARG);
  if (s.flags & BMA_MASK_TILES) {
    BMA_REQUIRE(s.tile_class && s.tile_slot && s.tiles_B > 0 && s.tiles_H > 0 && s.tiles_q > 0 && s.tiles_k > 0, BMA_ERR_ARG);
    BMA_REQUIRE((int64_t)s.tiles_q * 128 >= (int64_t)s.q_valid + s.q_offset && (int64_t)s.tiles_k * 128 >= (int64_t)s.k_valid + s.k_offset,
                BMA_ERR_ARG);
  }
  if (s.flags & BMA_MASK_BLOCK_WINDOW)
    BMA_REQUIRE(s.win_block > 0 && s.win_left >= 0 && s.win_right >= 0 && s.win_left + s.win_right <= s.win_nblk,
                BMA_ERR_ARG);
  if (s.flags & BMA_MASK_BAND) BMA_REQUIRE(s.band_left >= 0 && s.band_right >= 0, BMA_ERR_ARG);
  BMA_REQUIRE(l.NQ <= kMaxRowWidth && l.NKV <= kMaxRowWidth, BMA_ERR_LIMIT);
  return BMA_OK;
}

// Launches the three passes with `workspace` as scratch (flags, then segment summaries).
int mask_compile_launch(const bma_mask_spec& spec, int B, int H, const bma_block_lists& l, void* workspace,
                        cudaStream_t st) {
  const WorkspacePlan p = plan_workspace(spec, B, H, l.NQ, l.NKV);
  uint8_t* flags = static_cast<uint8_t*>(workspace) + p.flags_off;
  SegSummary seg{nullptr, nullptr, nullptr, nullptr};
  int sm_count = 148;
  {
    int dev = 0;
    BMA_CUDA_TRY(cudaGetDevice(&dev));
    BMA_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  if (spec.flags & BMA_MASK_SEGMENT) {
    int32_t* base = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + p.seg_off);
    seg.qmin = base;
    seg.qmax = seg.qmin + (size_t)B * l.NQ;
    seg.kmin = seg.qmax + (size_t)B * l.NQ;
    seg.kmax = seg.kmin + (size_t)B * l.NKV;
    const int64_t warps = (int64_t)B * (l.NQ + l.NKV);
    const int grid = (int)std::min<int64_t>((warps + 7) / 8, (int64_t)sm_count * 8);
    seg_summary_kernel<<<grid, kThreads, 0, st>>>(spec, B, l.NQ, l.NKV, l.q_block, l.kv_block, seg);
    count_launches(1);
  }
  {
    const int64_t blocks = (int64_t)p.CB * p.CH * l.NQ * l.NKV;
    const int grid = (int)std::min<int64_t>((blocks + kThreads - 1) / kThreads, (int64_t)sm_count * 16);
    // blocks that closed forms cannot decide exist only with these terms; without them pass 1b is not launched
    const bool may_scan = (spec.flags & (BMA_MASK_BITMAP | BMA_MASK_BLOCK_WINDOW | BMA_MASK_TILES)) ||
                          ((spec.flags & BMA_MASK_SEGMENT) && !(spec.flags & BMA_MASK_COMPILE_CONSERVATIVE));
    if (may_scan) BMA_CUDA_TRY(cudaMemsetAsync(l.kv_num, 0, sizeof(int32_t), st));
    classify_kernel<<<grid, kThreads, 0, st>>>(spec, p.CB, p.CH, l.NQ, l.NKV, l.q_block, l.kv_block, seg, flags, l.kv_idx, l.kv_num);
    count_launches(1);
    if (may_scan) {
      scan_kernel<<<sm_count * 8, kThreads, 0, st>>>(spec, p.CH, l.NQ, l.NKV, l.q_block, l.kv_block, flags, l.kv_idx, l.kv_num);
      count_launches(1);
    }
  }
  auto launch_compact = [&](bool transposed) -> int {
    const int NR = transposed ? l.NKV : l.NQ, NC = transposed ? l.NQ : l.NKV;
    const int rows = p.CB * p.CH * NR;
    const int reps = ((p.CB == l.B) ? 1 : l.B) * ((p.CH == l.H) ? 1 : l.H);
    int gy = std::max(1, std::min(reps, (sm_count * 4 + rows - 1) / rows));
    gy = std::min(gy, 65535);
    const size_t smem = sizeof(int32_t) * 2 * (size_t)NC + align_up((size_t)NC, 16);
    dim3 grid(rows, gy);
    if (transposed) {
      if (smem > 48 * 1024)
        BMA_CUDA_TRY(cudaFuncSetAttribute(compact_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      compact_kernel<true><<<grid, kThreads, smem, st>>>(flags, p.CB, p.CH, l.NQ, l.NKV, l.B, l.H, l.q_num, l.q_idx,
                                                         l.full_q_num, l.full_q_idx);
    } else {
      if (smem > 48 * 1024)
        BMA_CUDA_TRY(cudaFuncSetAttribute(compact_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      compact_kernel<false><<<grid, kThreads, smem, st>>>(flags, p.CB, p.CH, l.NQ, l.NKV, l.B, l.H, l.kv_num, l.kv_idx,
                                                          l.full_kv_num, l.full_kv_idx);
    }
    count_launches(1);
    return BMA_OK;
  };
  int rc = BMA_OK;
  if (l.q_num) {   // both sides: one launch
    const int rows = p.CB * p.CH * std::max(l.NQ, l.NKV);
    const int reps = ((p.CB == l.B) ? 1 : l.B) * ((p.CH == l.H) ? 1 : l.H);
    int gy = std::max(1, std::min(reps, (sm_count * 4 + rows - 1) / rows));
    gy = std::min(gy, 65535);
    const int NC = std::max(l.NQ, l.NKV);
    const size_t smem = sizeof(int32_t) * 2 * (size_t)NC + align_up((size_t)NC, 16);
    if (smem > 48 * 1024)
      BMA_CUDA_TRY(cudaFuncSetAttribute(compact_both_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    compact_both_kernel<<<dim3(rows, gy, 2), kThreads, smem, st>>>(flags, p.CB, p.CH, l.NQ, l.NKV, l.B, l.H, l);
    count_launches(1);
  } else {
    rc = launch_compact(false);
    if (rc != BMA_OK) return rc;
  }
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that must not allocate: the scratch lives in the module image.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;  // 4 MiB per GPU that loads the library

// Block flags and segment summaries of bma_mask_compile_static.  Every call on a device uses this
// one array, so two calls whose kernels overlap on the GPU race on it.  Nothing in it has to start
// at zero: the classify pass writes every flag and the summary pass every summary before they are
// read, so no clearing is needed between calls.
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevicesStatic = 64;
void* g_static_scratch_ptr[kMaxDevicesStatic] = {};
std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device.  In host code the symbol name is only
// a handle, not an address a kernel may dereference; the address comes from the runtime, once per
// device, with that device current.
int static_scratch_address(void** out) {
  int dev = 0;
  BMA_CUDA_TRY(cudaGetDevice(&dev));
  BMA_REQUIRE(dev >= 0 && dev < kMaxDevicesStatic, BMA_ERR_LIMIT);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void* ptr = nullptr;
    BMA_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
    BMA_REQUIRE(ptr != nullptr, BMA_ERR_CUDA);
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return BMA_OK;
}

}  // namespace

size_t mask_compile_static_limit() { return kStaticScratchBytes; }

int mask_compile_static(const bma_mask_spec& spec, int B, int H, const bma_block_lists& l, cudaStream_t st) {
  int rc = mask_compile_validate(spec, B, H, l);
  if (rc != BMA_OK) return rc;
  if (mask_compile_workspace_bytes(spec, B, H, l.NQ, l.NKV) > kStaticScratchBytes) return BMA_ERR_LIMIT;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != BMA_OK) return rc;
  return mask_compile_launch(spec, B, H, l, scratch, st);
}

}  // namespace bma
