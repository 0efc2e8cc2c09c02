// Compact addressing of the backward scratch (the bf16 dS tiles that the dK/dV kernel hands to the dQ replay
// kernel): one 32 KB slot per VISITED block instead of one per block of the dense [B, Hq, NQ, NKV] grid.
//
//   slot(b, h, qi, kj) = head_base[b * Hq + h] + row_base[b', h', qi] + rank[b', h', qi, kj]
//
// with (b', h') the list head that (b, h) reads (the lists broadcast over B and / or H), rank = the number of
// visited kv tiles of row qi below kj (the order in which the query-major replay kernel walks the row, so it
// needs no table: its running count IS the rank), row_base = exclusive prefix of the row counts inside a list
// head, head_base = exclusive prefix over (b, h) in row-major order of the list heads' totals.  A launch over a
// range of (batch, head) units subtracts the head_base of its first head.
//
// Three small launches per backward call build the tables from the kv-side lists into the front of the caller's
// workspace: ranks (one warp per list row), row bases (one CTA per list head), head bases (one CTA).
#include <algorithm>

#include "common.cuh"

namespace bma {

namespace {

constexpr int kMaxKvTilesBwd = 1024;  // the tensor-core backward takes L <= 131072

// rank[row][kj] = number of visited kv tiles below kj, or -1 when (row, kj) is not visited; row_count[row].
__global__ void __launch_bounds__(256) slot_rank_kernel(bma_block_lists l, int32_t* __restrict__ rank, int32_t* __restrict__ row_count) {
  __shared__ uint32_t bits[8][kMaxKvTilesBwd / 32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t rows = (int64_t)l.B * l.H * l.NQ;
  const int64_t row = (int64_t)blockIdx.x * 8 + w;
  if (row >= rows) return;
  const int words = (l.NKV + 31) / 32;
  bits[w][lane] = 0u;
  __syncwarp();
  const int nfull = min(max(l.full_kv_num[row], 0), l.NKV), npart = min(max(l.kv_num[row], 0), l.NKV);
  const int32_t* full_idx = l.full_kv_idx + row * l.NKV;
  const int32_t* part_idx = l.kv_idx + row * l.NKV;
  for (int i = lane; i < nfull; i += 32) {
    const int j = full_idx[i];
    if (j >= 0 && j < l.NKV) atomicOr(&bits[w][j >> 5], 1u << (j & 31));
  }
  for (int i = lane; i < npart; i += 32) {
    const int j = part_idx[i];
    if (j >= 0 && j < l.NKV) atomicOr(&bits[w][j >> 5], 1u << (j & 31));
  }
  __syncwarp();
  const uint32_t mine = lane < words ? bits[w][lane] : 0u;
  int prefix = __popc(mine);   // inclusive scan over the lanes' word counts
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, prefix, off);
    if (lane >= off) prefix += v;
  }
  const int total = __shfl_sync(0xffffffffu, prefix, 31);
  const int below = prefix - __popc(mine);
  if (lane < words) {
    int32_t* out = rank + row * l.NKV + lane * 32;
    for (int bit = 0; bit < 32 && lane * 32 + bit < l.NKV; ++bit)
      out[bit] = (mine >> bit) & 1u ? below + __popc(mine & ((1u << bit) - 1u)) : -1;
  }
  if (lane == 0) row_count[row] = total;
}

// One CTA per list head: row_base = exclusive prefix of row_count over its NQ rows (in place), head_total.
__global__ void __launch_bounds__(1024) slot_row_base_kernel(int NQ, int32_t* __restrict__ row_count_to_base, int64_t* __restrict__ head_total) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  int32_t* rc = row_count_to_base + (int64_t)blockIdx.x * NQ;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < NQ; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < NQ ? rc[i] : 0;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) warp_sums[w] = incl;
    __syncthreads();
    if (w == 0) {
      int s = warp_sums[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, s, off);
        if (lane >= off) s += t;
      }
      warp_sums[lane] = s;   // inclusive over warps
    }
    __syncthreads();
    const int carry = carry_s;
    const int before = carry + (w > 0 ? warp_sums[w - 1] : 0) + incl - v;
    if (i < NQ) rc[i] = before;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) head_total[blockIdx.x] = carry_s;
}

// One CTA: head_base[i] for i in [0, B*Hq] = exclusive prefix over (b, h) of head_total[b', h'].
__global__ void __launch_bounds__(1024) slot_head_base_kernel(int B, int Hq, int LB, int LH, const int64_t* __restrict__ head_total,
                                                              int64_t* __restrict__ head_base) {
  __shared__ long long warp_sums[32];
  __shared__ long long carry_s;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t n = (int64_t)B * Hq;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += 1024) {
    const int64_t i = base + threadIdx.x;
    long long v = 0;
    if (i < n) {
      const int b = (int)(i / Hq), h = (int)(i % Hq);
      v = head_total[(int64_t)(LB == 1 ? 0 : b) * LH + (LH == 1 ? 0 : h)];
    }
    long long incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const long long t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) warp_sums[w] = incl;
    __syncthreads();
    if (w == 0) {
      long long s = warp_sums[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const long long t = __shfl_up_sync(0xffffffffu, s, off);
        if (lane >= off) s += t;
      }
      warp_sums[lane] = s;
    }
    __syncthreads();
    const long long carry = carry_s;
    if (i < n) head_base[i] = carry + (w > 0 ? warp_sums[w - 1] : 0) + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) head_base[n] = carry_s;
}

// visited[b', h'] = sum over the rows of a list head of (kv_num + full_kv_num)
__global__ void __launch_bounds__(256) visited_kernel(bma_block_lists l, int64_t* __restrict__ visited) {
  __shared__ long long part[8];
  const int64_t row0 = (int64_t)blockIdx.x * l.NQ;
  long long s = 0;
  for (int i = threadIdx.x; i < l.NQ; i += blockDim.x) s += (long long)l.kv_num[row0 + i] + l.full_kv_num[row0 + i];
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    long long t = 0;
    for (int i = 0; i < 8; ++i) t += part[i];
    visited[blockIdx.x] = t;
  }
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

// Layout of the tables at the front of the backward workspace.
SlotTables slot_tables_layout(const bma_attn_args& a, const bma_block_lists& l, void* ws) {
  SlotTables t;
  uint8_t* p = static_cast<uint8_t*>(ws);
  size_t off = 0;
  t.head_base = reinterpret_cast<int64_t*>(p + off);
  off = align_up(off + sizeof(int64_t) * ((size_t)a.B * a.Hq + 1), 256);
  t.head_total = reinterpret_cast<int64_t*>(p + off);
  off = align_up(off + sizeof(int64_t) * (size_t)l.B * l.H, 256);
  t.row_base = reinterpret_cast<int32_t*>(p + off);
  off = align_up(off + sizeof(int32_t) * (size_t)l.B * l.H * l.NQ, 256);
  t.rank = reinterpret_cast<int32_t*>(p + off);
  off = align_up(off + sizeof(int32_t) * (size_t)l.B * l.H * l.NQ * l.NKV, 1024);
  t.bytes = off;
  return t;
}

int slot_tables_build(const bma_attn_args& a, const bma_block_lists& l, const SlotTables& t, cudaStream_t st) {
  BMA_REQUIRE(l.NKV <= kMaxKvTilesBwd, BMA_ERR_LIMIT);
  const int64_t rows = (int64_t)l.B * l.H * l.NQ;
  slot_rank_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(l, t.rank, t.row_base);
  slot_row_base_kernel<<<(unsigned)(l.B * l.H), 1024, 0, st>>>(l.NQ, t.row_base, t.head_total);
  slot_head_base_kernel<<<1, 1024, 0, st>>>(a.B, a.Hq, l.B, l.H, t.head_total, t.head_base);
  count_launches(3);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

int block_lists_visited(const bma_block_lists& l, int64_t* visited, cudaStream_t st) {
  visited_kernel<<<(unsigned)(l.B * l.H), 256, 0, st>>>(l, visited);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

}  // namespace bma
