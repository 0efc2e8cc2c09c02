// Backward dQ from stored dS tiles, bf16, head dim 128 / 64, sm_100a (tcgen05 + TMEM + TMA).
//
// The dK/dV kernel (attn_bwd_sm100.cu) can leave the bf16 dSt tile of every visited block in a
// scratch buffer: 32 KB per block, the raw shared-memory image of a [128 keys x 128 queries] operand
// in the 128-byte-swizzled layout (two boxes of 64 query columns).  Read back into shared memory
// at a 1024-byte boundary, the same bytes are dS as an MN-major A operand (M = query, contiguous;
// K = key), so
//     dQ += dS K             A = dS (shared, MN-major),  B = K (shared, MN-major)  -> TMEM
// is the only MMA left for dQ: S and dP are not recomputed.  The kernel is bound by the HBM
// stream of the dS tiles (32 KB per 4.2 MFLOP), not by the tensor core.
//
// One CTA per SM on a PAIR of 128-query tiles (2p, 2p+1) of one (batch, query head) walking the
// union of their kv lists: a K tile is fetched once for both.  warp 8: producer (K through the
// tensor map, two stages; dS tiles as untiled bulk copies, four stages); warp 9: tcgen05.mma issue
// on a converged warp; warpgroups 0 / 1: epilogue of tile A / B (dQ * scale -> bf16 -> TMA store).
// The block lists must name the same blocks on the q side (walked by the dK/dV kernel) and on the
// kv side (walked here): a slot is read only if it was written during the same backward call.
// Every mbarrier wait is bounded; on a timeout the thread records an error code and unwinds.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace bma {
namespace {

using namespace ptx;

constexpr int BM = kSm100Tile, BN = kSm100Tile;
constexpr int kThreads = 320;  // two epilogue warpgroups + producer warp + MMA warp
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kHalfTile = BM * 64 * 2;
template <int HD> constexpr uint32_t kTileBytesOf = (HD / 64) * kHalfTile;
constexpr uint32_t kDsBytes = 2 * kHalfTile;
constexpr int kDsStages = 4;
constexpr int kMaxKvTiles = 1024;

enum {
  BAR_K_FULL0 = 0, BAR_K_FULL1, BAR_K_FREE0, BAR_K_FREE1,
  BAR_DS_FULL0, BAR_DS_FREE0 = BAR_DS_FULL0 + kDsStages,
  BAR_DONE = BAR_DS_FREE0 + kDsStages, BAR_EPI0, BAR_EPI1,
  NUM_BARS
};

template <int HD>
struct __align__(1024) ReplaySmem {
  uint8_t ds[kDsStages][kDsBytes];
  uint8_t k[2][kTileBytesOf<HD>];
  uint16_t merged[kMaxKvTiles];  // kv tile | (tile A listed) << 12 | (tile B listed) << 14
  uint8_t cls[2][kMaxKvTiles];
  uint64_t bar[NUM_BARS];
  uint32_t tmem_base;
  int n_merged;
  int n_blocks[2];  // blocks of tile A / B
};

struct ReplayParams {
  bma_attn_args a;
  bma_block_lists l;
  const uint8_t* ds;  // slots of kDsBytes, addressed compactly: head_base[b, h] - head_base[first head of the launch]
                      // + row_base[q tile] + (number of the row's visited kv tiles before this one)
  const int64_t* head_base;
  const int32_t* row_base;
  int64_t capacity;
  int b0, h0, nh;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_replay_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_dq, const ReplayParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t kTileBytes = kTileBytesOf<HD>;
  ReplaySmem<HD>& sm = *reinterpret_cast<ReplaySmem<HD>*>(smem_raw);

  const bma_attn_args& a = p.a;
  const int pair = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest causal tiles first
  const int h = blockIdx.y + p.h0, b = blockIdx.z + p.b0;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int wg = warp >> 2;
  const int NQ = p.l.NQ, NKV = p.l.NKV;

  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0) report_device_error(p.status, 501);
    return;
  }

  // ---- merged kv list of the two query tiles ------------------------------------------------
  const int lb = p.l.B == 1 ? 0 : b, lh = p.l.H == 1 ? 0 : h;
  for (int i = threadIdx.x; i < NKV; i += kThreads) { sm.cls[0][i] = 0; sm.cls[1][i] = 0; }
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(&sm.bar[i], (i == BAR_EPI0 || i == BAR_EPI1) ? 128 : 1);
    fence_barrier_init();
  }
  __syncthreads();
  for (int x = 0; x < 2; ++x) {
    const int qi = pair * 2 + x;
    if (qi >= NQ) break;
    const int64_t lrow = ((int64_t)lb * p.l.H + lh) * NQ + qi;
    const int nfull = p.l.full_kv_num[lrow], npart = p.l.kv_num[lrow];
    const int32_t* full_idx = p.l.full_kv_idx + lrow * NKV;
    const int32_t* part_idx = p.l.kv_idx + lrow * NKV;
    for (int i = threadIdx.x; i < nfull; i += kThreads) sm.cls[x][full_idx[i]] = 1;
    for (int i = threadIdx.x; i < npart; i += kThreads) sm.cls[x][part_idx[i]] = 1;
  }
  __syncthreads();
  if (warp == 0) {
    int count = 0, n0 = 0, n1 = 0;
    for (int base = 0; base < NKV; base += 32) {
      const int j = base + lane;
      const uint32_t ca = j < NKV ? sm.cls[0][j] : 0, cb = j < NKV ? sm.cls[1][j] : 0;
      const unsigned m = __ballot_sync(0xffffffffu, (ca | cb) != 0);
      if (ca | cb) sm.merged[count + __popc(m & ((1u << lane) - 1))] = (uint16_t)((uint32_t)j | (ca << 12) | (cb << 14));
      count += __popc(m);
      n0 += __popc(__ballot_sync(0xffffffffu, ca != 0));
      n1 += __popc(__ballot_sync(0xffffffffu, cb != 0));
    }
    if (lane == 0) { sm.n_merged = count; sm.n_blocks[0] = n0; sm.n_blocks[1] = n1; }
  }
  if (warp == 8) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const int T = sm.n_merged;

  if (wg == 2) {
    if (warp == 8 && lane == 0 && T > 0) {
      // ---------------------------------------------------------------- producer
      prefetch_tensormap(&map_k);
      const uint64_t policy = l2_evict_first();  // every dS tile is read exactly once
      // first slot of each of the two query rows; the walk below visits a row's kv tiles in ascending order, which is
      // the order the slots were numbered in
      const int64_t head0 = __ldg(p.head_base + (int64_t)b * a.Hq + h) - __ldg(p.head_base + (int64_t)p.b0 * a.Hq + p.h0);
      int64_t next_slot[2];
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int qi = min(pair * 2 + x, NQ - 1);
        next_slot[x] = head0 + __ldg(p.row_base + ((int64_t)lb * p.l.H + lh) * NQ + qi);
      }
      bool ok = true;
      int s = 0;  // dS tiles requested so far
      for (int n = 0; n < T && ok; ++n) {
        const int st = n & 1;
        const uint32_t e = sm.merged[n];
        const int kj = (int)(e & 0x3ffu);
        // the dS tiles first: they come from HBM, the K tile mostly from L2
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!((e >> (12 + 2 * x)) & 3u)) continue;
          const int slot = s % kDsStages;
          if (s >= kDsStages) ok = mbar_wait(&sm.bar[BAR_DS_FREE0 + slot], ((s / kDsStages) - 1) & 1);
          if (!ok) break;
          // (an index outside the buffer cannot come from consistent lists; it is clamped and reported, never read)
          int64_t gslot = next_slot[x]++;
          if (gslot < 0 || gslot >= p.capacity) { gslot = 0; report_device_error(p.status, 511); }
          mbar_expect_tx(&sm.bar[BAR_DS_FULL0 + slot], kDsBytes);
          bulk_load_1d(sm.ds[slot], p.ds + gslot * (int64_t)kDsBytes, kDsBytes, &sm.bar[BAR_DS_FULL0 + slot], policy);
          ++s;
        }
        if (!ok) break;
        if (n >= 2) ok = mbar_wait(&sm.bar[BAR_K_FREE0 + st], ((n >> 1) - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_K_FULL0 + st], kTileBytes);
#pragma unroll
        for (int box = 0; box < HD / 64; ++box)
          tma_load_4d(sm.k[st] + box * kHalfTile, &map_k, &sm.bar[BAR_K_FULL0 + st], box * 64, hk, kj * BN, b);
      }
      if (!ok) report_device_error(p.status, 510);
    } else if (warp == 9 && T > 0) {
      // ---------------------------------------------------------------- MMA issuer (converged warp, one elected lane)
      const bool leader = elect_one();
      constexpr uint32_t idesc_nn = make_idesc_bf16(BM, HD, 1, 1);  // both operands MN-major
      const uint64_t dds0 = make_smem_desc(smem_u32(sm.ds[0]), kHalfTile, 1024);
      const uint64_t dkm0 = make_smem_desc(smem_u32(sm.k[0]), kHalfTile, 1024);
      constexpr uint32_t kStageUnits = kTileBytes >> 4, kDsUnits = kDsBytes >> 4;
      bool ok = true;
      int s = 0, cnt0 = 0, cnt1 = 0;
      for (int n = 0; n < T && ok; ++n) {
        const int st = n & 1;
        const uint32_t e = sm.merged[n];
        ok = mbar_wait(&sm.bar[BAR_K_FULL0 + st], (n >> 1) & 1);
        if (!ok) break;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!((e >> (12 + 2 * x)) & 3u)) continue;
          const int slot = s % kDsStages;
          ok = mbar_wait(&sm.bar[BAR_DS_FULL0 + slot], (s / kDsStages) & 1);
          if (!ok) break;
          tc_fence_after();
          int& cnt = x == 0 ? cnt0 : cnt1;
          // 16 keys per MMA = 16 rows of 128 bytes in both images
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)
            if (leader)
              mma_ss(tmem + x * 128, dds0 + (uint32_t)(slot * kDsUnits + ks * (2048 >> 4)),
                     dkm0 + (uint32_t)(st * kStageUnits + ks * (2048 >> 4)), idesc_nn, (cnt > 0) || (ks > 0));
          if (leader) mma_commit(&sm.bar[BAR_DS_FREE0 + slot]);
          ++cnt;
          ++s;
        }
        if (!ok) break;
        if (leader) mma_commit(&sm.bar[BAR_K_FREE0 + st]);
      }
      if (ok && leader) mma_commit(&sm.bar[BAR_DONE]);
      if (!ok && leader) report_device_error(p.status, 520);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warpgroups: dQ * scale
    const int x = wg;
    const int qi = pair * 2 + x;
    const int row = threadIdx.x & 127;  // TMEM lane == query row of the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_dq = tmem + x * 128 + lane_base;
    const int cnt = sm.n_blocks[x];
    // all MMAs of the CTA are complete after BAR_DONE, so every dS stage is free for staging
    bool ok = T > 0 ? mbar_wait(&sm.bar[BAR_DONE], 0) : true;
    if (!ok) {
      report_device_error(p.status, 530 + warp);
    } else if (qi < NQ) {
      tc_fence_after();
      uint8_t* q_row = sm.ds[x] + row * 128;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        if (cnt > 0) {
          tmem_ld32(tmem_dq + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = u * 8;
          uint4 v4;
          v4.x = pack_bf16(__uint_as_float(r[j]) * a.scale, __uint_as_float(r[j + 1]) * a.scale);
          v4.y = pack_bf16(__uint_as_float(r[j + 2]) * a.scale, __uint_as_float(r[j + 3]) * a.scale);
          v4.z = pack_bf16(__uint_as_float(r[j + 4]) * a.scale, __uint_as_float(r[j + 5]) * a.scale);
          v4.w = pack_bf16(__uint_as_float(r[j + 6]) * a.scale, __uint_as_float(r[j + 7]) * a.scale);
          const int chunk = ((c & 1) * 4 + u) ^ (row & 7);  // 32 columns = four 16-byte chunks of a box row
          *reinterpret_cast<uint4*>(q_row + (c >> 1) * kHalfTile + chunk * 16) = v4;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the TMA engine reads the staged tile through the async proxy
      mbar_arrive(&sm.bar[BAR_EPI0 + x]);
      ok = mbar_wait(&sm.bar[BAR_EPI0 + x], 0);
      if (!ok) {
        report_device_error(p.status, 550 + warp);
      } else if (row == 0) {
#pragma unroll
        for (int box = 0; box < HD / 64; ++box) tma_store_4d(&map_dq, sm.ds[x] + box * kHalfTile, box * 64, h, qi * BM, b);
        bulk_commit();
        bulk_wait_read0();  // shared memory must stay intact until the stores have read it
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

int sm100_bwd_dq_from_ds(const bma_attn_args& a, const bma_block_lists& lists, const void* ds, const SlotTables& tables,
                         int64_t capacity, int b0, int nb, int hk0, int nhk, cudaStream_t st) {
  BMA_REQUIRE(lists.NKV <= kMaxKvTiles, BMA_ERR_LIMIT);
  BMA_REQUIRE(ds != nullptr, BMA_ERR_ARG);
  CUtensorMap mk, mdq;
  int rc;
  if ((rc = make_tile_map_bf16(&mk, a.k.ptr, a.B, a.L, a.Hkv, a.d, a.k.stride_b, a.k.stride_l, a.k.stride_h, BN))) return rc;
  if ((rc = make_tile_map_bf16(&mdq, a.dq.ptr, a.B, a.N, a.Hq, a.d, a.dq.stride_b, a.dq.stride_l, a.dq.stride_h, BM))) return rc;
  ReplayParams p;
  p.a = a; p.l = lists;
  p.ds = static_cast<const uint8_t*>(ds);
  p.head_base = tables.head_base; p.row_base = tables.row_base; p.capacity = capacity;
  const int G = a.Hq / a.Hkv;
  p.b0 = b0; p.h0 = hk0 * G; p.nh = nhk * G;
  p.status = device_status_ptr();
  BMA_REQUIRE(p.status != nullptr, BMA_ERR_CUDA);

  dim3 grid(ceil_div(ceil_div(a.N, BM), 2), p.nh, nb);
  auto launch = [&](auto kernel, size_t smem) -> int {
    BMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kThreads, smem, st>>>(mk, mdq, p);
    return BMA_OK;
  };
  rc = a.d == 128 ? launch(bwd_dq_replay_kernel<128>, sizeof(ReplaySmem<128>)) : launch(bwd_dq_replay_kernel<64>, sizeof(ReplaySmem<64>));
  if (rc) return rc;
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

}  // namespace bma
