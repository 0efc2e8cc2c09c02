// Backward for bf16, head dim 128, on the sm_100a tensor core (tcgen05 + TMEM + TMA).
//
// One CTA per (kv tile of 128 keys, kv head, batch), one CTA per SM (all 512 TMEM columns).  K and
// V of the tile stay in shared memory; the CTA walks the q tiles named by the q-side block lists of
// every query head of the group (full tiles first, then partial ones) and per q tile runs five
// 128x128x128 MMAs:
//     St  = K Q^T            A = K (K-major),  B = Q  (K-major)      -> TMEM [256,384)
//     dPt = V dO^T           A = V (K-major),  B = dO (K-major)      -> TMEM [384,512)
//     dV += Pt dO            A = Pt (bf16 in TMEM, over dPt),  B = dO (MN-major) -> TMEM [0,128)
//     dK += dSt Q            A = dSt (shared, K-major),        B = Q  (MN-major) -> TMEM [128,256)
//     dQ  = dS K             A = dSt (same bytes, MN-major),   B = K  (MN-major) -> TMEM [384,512)
// with Pt = exp2(St*scale*log2e - lse*log2e) and dSt = Pt * (dPt - delta) computed by eight warps
// (thread = key row; warps w and w+4 split the 128 query columns).
//
// Pipelining: the consumers pull St into registers and release its columns at once, so the next
// tile's K Q^T runs under the element-wise math, and they compute the exponentials of tile n+1
// while the MMAs of tile n run.  Pt is written over the dPt columns once every consumer has read
// them; dQ reuses the same columns after Pt has been consumed, and the next V dO^T waits until the
// dQ tile has been pulled into registers.
// dQ tiles leave through shared memory (the dSt buffer and the dO stage that just became free) and
// a TMA reduce-add into a float32 accumulator in global memory: several kv tiles contribute to
// one q tile, so the summation order is not fixed.  A second small kernel scales and casts the
// accumulator.  dK and dV are accumulated in TMEM in float32 and written once.
// Every mbarrier wait is bounded; on a timeout the thread records an error code and unwinds.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace bma {
namespace {

using namespace ptx;

constexpr int BT = kSm100Tile, HD = 128;
constexpr int kConsumers = 256;
constexpr int kThreads = kConsumers + 128;  // + one warpgroup: warp 8 TMA, warp 9 MMA issue
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kHalfTile = BT * 64 * 2;
constexpr uint32_t kTileBytes = 2 * kHalfTile;
constexpr uint32_t kDqBox = BT * 32 * 4;  // one [128 rows x 32 float] box of the dQ tile
constexpr uint32_t COL_DV = 0, COL_DK = 128, COL_ST = 256, COL_DPT = 384, COL_PT = 384, COL_DQ = 384;

enum {
  BAR_KV = 0, BAR_FULLQ0, BAR_FULLQ1, BAR_FULLDO0, BAR_FULLDO1,
  BAR_S1, BAR_S2, BAR_LS, BAR_P, BAR_X, BAR_D, BAR_DQ, BAR_STG,
  BAR_SYNC1, BAR_SYNC2, BAR_SYNC3,  // consumer-wide rendezvous points (bounded, unlike bar.sync)
  NUM_BARS
};

struct __align__(1024) BwdSmem {
  uint8_t k[kTileBytes];
  uint8_t v[kTileBytes];
  uint8_t ds[kTileBytes];        // dSt (bf16) for the MMAs; between tiles: dQ columns 0..63 (float32)
  uint8_t q[2][kTileBytes];
  uint8_t d_o[2][kTileBytes];    // dO stages; a stage that was just consumed stages dQ columns 64..127
  float lse2[2][BT];
  float delta[2][BT];
  uint64_t bar[NUM_BARS];
  uint32_t tmem_base;
};

struct BwdParams {
  bma_attn_args a;
  bma_mask_spec spec;
  bma_block_lists l;
  float scale_log2;
  int interval_mask;
  int* status;
};

// Rendezvous of the 256 consumer threads on an mbarrier: arrive, then a bounded wait (a plain
// bar.sync would wait forever for a thread that gave up on an earlier wait).
__device__ __forceinline__ bool consumer_sync(uint64_t* bar, uint32_t parity) {
  mbar_arrive(bar);
  return mbar_wait(bar, parity);
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void setmaxnreg_inc_208() { asm volatile("setmaxnreg.inc.sync.aligned.u32 208;"); }
__device__ __forceinline__ void setmaxnreg_dec_80() { asm volatile("setmaxnreg.dec.sync.aligned.u32 80;"); }
// TMA reduce-add of one box from shared memory into the float32 tensor described by `m`
// (rows outside the tensor are clipped); completion is tracked by the bulk async-group.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Allowed query interval [jlo, jhi] (tile-local columns, inclusive) of key row k for masks made of
// interval terms (the block window is constant over the q tile; the host checks that).
__device__ __forceinline__ void col_interval(const MaskView& m, int k, int q0, int& jlo, int& jhi) {
  jlo = 0;
  jhi = min(BT, m.q_valid - q0) - 1;
  if (k >= m.k_valid) { jlo = 1; jhi = 0; return; }
  const int gk = k + m.k_offset;
  const int base = m.q_offset + q0;  // global index of column 0
  if (m.flags & BMA_MASK_CAUSAL) jlo = max(jlo, gk - base);
  if (m.flags & BMA_MASK_BAND) {  // gq - left <= gk <= gq + right  <=>  gk - right <= gq <= gk + left
    jlo = max(jlo, gk - m.band_right - base);
    jhi = min(jhi, gk + m.band_left - base);
  }
  if (m.flags & BMA_MASK_BLOCK_WINDOW) {
    int wlo, whi;
    block_window_range(m, base, wlo, whi);
    if (gk < wlo || gk >= whi) { jlo = 1; jhi = 0; }
  }
}

struct QTileIter {  // flattened walk over (group head, listed q tile)
  const bma_block_lists& l;
  int b, hk, G, kj;
  int g, it, nfull, npart;
  const int32_t* full_idx;
  const int32_t* part_idx;
  __device__ QTileIter(const bma_block_lists& l_, int b_, int hk_, int G_, int kj_)
      : l(l_), b(b_), hk(hk_), G(G_), kj(kj_), g(-1), it(0), nfull(0), npart(0), full_idx(nullptr), part_idx(nullptr) {}
  __device__ void load_head() {
    const int h = hk * G + g;
    const int lb = l.B == 1 ? 0 : b, lh = l.H == 1 ? 0 : h;
    const int64_t row = ((int64_t)lb * l.H + lh) * l.NKV + kj;
    nfull = l.full_q_num[row];
    npart = l.q_num[row];
    full_idx = l.full_q_idx + row * l.NQ;
    part_idx = l.q_idx + row * l.NQ;
    it = 0;
  }
  __device__ bool next(int& h, int& qi, bool& partial) {
    if (g < 0) { g = 0; load_head(); }
    while (it >= nfull + npart) {
      if (++g >= G) return false;
      load_head();
    }
    h = hk * G + g;
    partial = it >= nfull;
    qi = partial ? part_idx[it - nfull] : full_idx[it];
    ++it;
    return true;
  }
};

__global__ void __launch_bounds__(kThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
           const __grid_constant__ CUtensorMap map_dq, const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);

  const bma_attn_args& a = p.a;
  const int kj = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int k0 = kj * BT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if ((smem_u32(smem_raw) & 1023u) != 0u) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) report_device_error(p.status, 301);
    return;
  }

  int total = 0;  // q tiles this CTA visits
  for (int g = 0; g < G; ++g) {
    const int h = hk * G + g;
    const int lb = p.l.B == 1 ? 0 : b, lh = p.l.H == 1 ? 0 : h;
    const int64_t row = ((int64_t)lb * p.l.H + lh) * p.l.NKV + kj;
    total += p.l.full_q_num[row] + p.l.q_num[row];
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i)
      mbar_init(&sm.bar[i], (i == BAR_LS || i == BAR_P || i == BAR_DQ || i >= BAR_SYNC1) ? kConsumers : 1);
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp >= 8) {
    setmaxnreg_dec_80();
    if (warp == 8 && lane == 0 && total > 0) {
      // ---------------------------------------------------------------- TMA producer
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      prefetch_tensormap(&map_do);
      auto load_tile = [&](const CUtensorMap* m, uint8_t* dst, uint64_t* bar, int head, int row0) {
        tma_load_4d(dst, m, bar, 0, head, row0, b);
        tma_load_4d(dst + kHalfTile, m, bar, 64, head, row0, b);
      };
      mbar_expect_tx(&sm.bar[BAR_KV], 2 * kTileBytes);
      load_tile(&map_k, sm.k, &sm.bar[BAR_KV], hk, k0);
      load_tile(&map_v, sm.v, &sm.bar[BAR_KV], hk, k0);
      QTileIter loader(p.l, b, hk, G, kj);
      bool ok = true;
      for (int n = 0; n < total && ok; ++n) {
        int h, qi; bool partial;
        loader.next(h, qi, partial);
        const int st = n & 1;
        // Q stage: free once tile n-2 has been multiplied (BAR_D of n-2 has the parity of n)
        if (n >= 2) ok = mbar_wait(&sm.bar[BAR_D], n & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_FULLQ0 + st], kTileBytes);
        load_tile(&map_q, sm.q[st], &sm.bar[BAR_FULLQ0 + st], h, qi * BT);
        // dO stage: after tile n-2 it staged half of that tile's dQ; free once the reduce has read it
        if (n >= 2) ok = mbar_wait(&sm.bar[BAR_STG], n & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_FULLDO0 + st], kTileBytes);
        load_tile(&map_do, sm.d_o[st], &sm.bar[BAR_FULLDO0 + st], h, qi * BT);
      }
      if (!ok) report_device_error(p.status, 305);
    } else if (warp == 9 && lane == 0 && total > 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_kk = make_idesc_bf16(BT, BT, 0, 0);  // both operands K-major
      constexpr uint32_t idesc_kn = make_idesc_bf16(BT, HD, 0, 1);  // B MN-major
      constexpr uint32_t idesc_nn = make_idesc_bf16(BT, HD, 1, 1);  // A and B MN-major
      const uint32_t k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), ds_addr = smem_u32(sm.ds);
      auto gemm_st = [&](uint32_t q_addr) {  // St = K Q^T
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfTile + (ks & 3) * 32;
          mma_ss(tmem + COL_ST, make_smem_desc(k_addr + off, 16, 1024), make_smem_desc(q_addr + off, 16, 1024), idesc_kk, ks > 0);
        }
        mma_commit(&sm.bar[BAR_S1]);
      };
      auto gemm_dpt = [&](uint32_t do_addr) {  // dPt = V dO^T
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfTile + (ks & 3) * 32;
          mma_ss(tmem + COL_DPT, make_smem_desc(v_addr + off, 16, 1024), make_smem_desc(do_addr + off, 16, 1024), idesc_kk, ks > 0);
        }
        mma_commit(&sm.bar[BAR_S2]);
      };
      bool ok = mbar_wait(&sm.bar[BAR_KV], 0) && mbar_wait(&sm.bar[BAR_FULLQ0], 0);
      if (ok) {
        tc_fence_after();
        gemm_st(smem_u32(sm.q[0]));
        ok = mbar_wait(&sm.bar[BAR_FULLDO0], 0);
        if (ok) { tc_fence_after(); gemm_dpt(smem_u32(sm.d_o[0])); }
      }
      for (int n = 0; n < total && ok; ++n) {
        const int st = n & 1;
        const uint32_t ph = n & 1;
        const uint32_t q_addr = smem_u32(sm.q[st]), do_addr = smem_u32(sm.d_o[st]);
        const uint32_t q_next = smem_u32(sm.q[st ^ 1]), do_next = smem_u32(sm.d_o[st ^ 1]);
        // St columns are free as soon as the consumers hold them in registers
        ok = mbar_wait(&sm.bar[BAR_LS], ph);
        if (ok && n + 1 < total) {
          ok = mbar_wait(&sm.bar[BAR_FULLQ0 + (st ^ 1)], ((n + 1) >> 1) & 1);
          if (ok) { tc_fence_after(); gemm_st(q_next); }
        }
        if (ok) ok = mbar_wait(&sm.bar[BAR_P], ph);
        if (!ok) break;
        tc_fence_after();
        // dV += Pt dO      (A from TMEM, 8 columns per 16-query k-step; B = dO rows as K)
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks)
          mma_ts(tmem + COL_DV, tmem + COL_PT + ks * 8, make_smem_desc(do_addr + ks * 2048, kHalfTile, 1024), idesc_kn, (n > 0) || (ks > 0));
        mma_commit(&sm.bar[BAR_X]);
        // dK += dSt Q      (A = dSt in shared memory, K-major over queries)
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfTile + (ks & 3) * 32;
          mma_ss(tmem + COL_DK, make_smem_desc(ds_addr + off, 16, 1024), make_smem_desc(q_addr + ks * 2048, kHalfTile, 1024), idesc_kn, (n > 0) || (ks > 0));
        }
        // dQ overwrites the columns Pt was read from: wait for dV to finish (dK keeps the pipe busy meanwhile)
        ok = mbar_wait(&sm.bar[BAR_X], ph);
        if (!ok) break;
        // dQ = dS K        (A = the same bytes read MN-major: M = query, K = key rows)
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks)
          mma_ss(tmem + COL_DQ, make_smem_desc(ds_addr + ks * 2048, kHalfTile, 1024), make_smem_desc(k_addr + ks * 2048, kHalfTile, 1024), idesc_nn, ks > 0);
        mma_commit(&sm.bar[BAR_D]);
        // the next dPt lands in the dQ columns: wait until the consumers hold the dQ tile in registers
        if (n + 1 < total) {
          ok = mbar_wait(&sm.bar[BAR_DQ], ph) && mbar_wait(&sm.bar[BAR_FULLDO0 + (st ^ 1)], ((n + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          gemm_dpt(do_next);
        }
      }
      if (!ok) report_device_error(p.status, 310);
    }
  } else {
    // ------------------------------------------------------------------ softmax-gradient warps
    setmaxnreg_inc_208();
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;  // TMEM lane: key row while computing dS, query row while draining dQ
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int k = k0 + row;
    bool ok = true;
    QTileIter walker(p.l, b, hk, G, kj);
    int h = 0, qi = 0;
    bool partial = false;
    float pr[64];  // Pt of the current tile (this thread's key row, its 64 query columns)

    // exponentials of one tile: stage the row statistics, pull St out of TMEM, release its columns
    auto exp_phase = [&](int n, int h_, int qi_, bool partial_) -> bool {
      const int st = n & 1;
      const int q0 = qi_ * BT;
      {  // lse*log2e (+inf for rows that attend nothing / lie outside) and delta of the q tile
        const int idx = threadIdx.x & (BT - 1);
        const int q = q0 + idx;
        const int64_t off = ((int64_t)b * a.Hq + h_) * a.N + q;
        if (threadIdx.x < BT) {
          const float lv = q < a.N ? a.lse[off] : -INFINITY;
          sm.lse2[st][idx] = (lv == -INFINITY) ? INFINITY : lv * kLog2e;
        } else {
          sm.delta[st][idx] = q < a.N ? a.delta[off] : 0.f;
        }
      }
      if (!consumer_sync(&sm.bar[BAR_SYNC1], n & 1)) return false;
      uint32_t bits[2] = {0xffffffffu, 0xffffffffu};
      if (partial_) {
        const MaskView mv = make_mask_view(p.spec, b, h_);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int cg = half * 2 + c;
          if (p.interval_mask) {
            int jlo, jhi;
            col_interval(mv, k, q0, jlo, jhi);
            const int lo = max(jlo - cg * 32, 0), hi = min(jhi - cg * 32, 31);
            bits[c] = (lo <= hi) ? ((0xffffffffu >> (31 - hi)) & (0xffffffffu << lo)) : 0u;
          } else {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) w |= (mask_allowed(mv, q0 + cg * 32 + j, k) ? 1u : 0u) << j;
            bits[c] = w;
          }
        }
      }
      if (!mbar_wait(&sm.bar[BAR_S1], n & 1)) return false;
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld32(tmem + COL_ST + lane_base + (half * 2) * 32, s0);
      tmem_ld32(tmem + COL_ST + lane_base + (half * 2 + 1) * 32, s1);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm.bar[BAR_LS]);
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 la = *reinterpret_cast<const float4*>(&sm.lse2[st][(half * 2) * 32 + j4 * 4]);
        const float4 lb = *reinterpret_cast<const float4*>(&sm.lse2[st][(half * 2 + 1) * 32 + j4 * 4]);
        const float lav[4] = {la.x, la.y, la.z, la.w}, lbv[4] = {lb.x, lb.y, lb.z, lb.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j4 * 4 + e;
          pr[j] = ex2(fmaf(__uint_as_float(s0[j]), p.scale_log2, -lav[e]));
          pr[32 + j] = ex2(fmaf(__uint_as_float(s1[j]), p.scale_log2, -lbv[e]));
        }
      }
      if (partial_) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          pr[j] = (bits[0] >> j) & 1u ? pr[j] : 0.f;
          pr[32 + j] = (bits[1] >> j) & 1u ? pr[32 + j] : 0.f;
        }
      }
      return true;
    };

    if (total > 0) {
      walker.next(h, qi, partial);
      ok = exp_phase(0, h, qi, partial);
    }
    for (int n = 0; n < total && ok; ++n) {
      const int st = n & 1;
      const uint32_t ph = n & 1;
      const int q0 = qi * BT;
      const int h_cur = h;

      // ---- dSt = Pt * (dPt - delta)
      ok = mbar_wait(&sm.bar[BAR_S2], ph);
      if (!ok) break;
      tc_fence_after();
      uint32_t pk[32], dsp[32];
      {
        uint32_t d0[32], d1[32];
        tmem_ld32(tmem + COL_DPT + lane_base + (half * 2) * 32, d0);
        tmem_ld32(tmem + COL_DPT + lane_base + (half * 2 + 1) * 32, d1);
        tmem_wait_ld();
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          const float4 da = *reinterpret_cast<const float4*>(&sm.delta[st][(half * 2) * 32 + j4 * 4]);
          const float4 db = *reinterpret_cast<const float4*>(&sm.delta[st][(half * 2 + 1) * 32 + j4 * 4]);
          const float dav[4] = {da.x, da.y, da.z, da.w}, dbv[4] = {db.x, db.y, db.z, db.w};
          float x0[4], x1[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = j4 * 4 + e;
            x0[e] = pr[j] * (__uint_as_float(d0[j]) - dav[e]);
            x1[e] = pr[32 + j] * (__uint_as_float(d1[j]) - dbv[e]);
          }
          pk[j4 * 2] = pack_bf16(pr[j4 * 4], pr[j4 * 4 + 1]);
          pk[j4 * 2 + 1] = pack_bf16(pr[j4 * 4 + 2], pr[j4 * 4 + 3]);
          pk[16 + j4 * 2] = pack_bf16(pr[32 + j4 * 4], pr[32 + j4 * 4 + 1]);
          pk[16 + j4 * 2 + 1] = pack_bf16(pr[32 + j4 * 4 + 2], pr[32 + j4 * 4 + 3]);
          dsp[j4 * 2] = pack_bf16(x0[0], x0[1]);
          dsp[j4 * 2 + 1] = pack_bf16(x0[2], x0[3]);
          dsp[16 + j4 * 2] = pack_bf16(x1[0], x1[1]);
          dsp[16 + j4 * 2 + 1] = pack_bf16(x1[2], x1[3]);
        }
      }
      // The dSt buffer and the other dO stage still hold the previous tile's dQ until the reduce
      // has read them; the thread that issued the reduce waits for that and frees the dO stage.
      if (threadIdx.x == 0 && n > 0) {
        bulk_wait_read0();
        mbar_arrive(&sm.bar[BAR_STG]);
      }
      // every consumer holds its dPt values: Pt may now overwrite those columns
      ok = consumer_sync(&sm.bar[BAR_SYNC2], ph);
      if (!ok) break;
      tmem_st32(tmem + COL_PT + lane_base + half * 32, pk);  // 64 queries = 32 packed columns per half
      {
        // dSt row `row`, query columns [64*half, 64*half+64): eight 16-byte chunks of the 128-byte-swizzled
        // [128 keys x 64 queries] box `half`
        uint8_t* ds_row = sm.ds + half * kHalfTile + row * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int chunk = u ^ (row & 7);
          *reinterpret_cast<uint4*>(ds_row + chunk * 16) = make_uint4(dsp[u * 4], dsp[u * 4 + 1], dsp[u * 4 + 2], dsp[u * 4 + 3]);
        }
      }
      tmem_wait_st();
      fence_proxy_async();  // dSt was written with ordinary stores; the MMA reads it through the async proxy
      tc_fence_before();
      mbar_arrive(&sm.bar[BAR_P]);

      // ---- exponentials of the next tile while the MMAs of this one run
      if (n + 1 < total) {
        walker.next(h, qi, partial);
        ok = exp_phase(n + 1, h, qi, partial);
        if (!ok) break;
      }

      // ---- dQ tile: TMEM -> registers -> shared memory -> TMA reduce-add into the float32 accumulator
      ok = mbar_wait(&sm.bar[BAR_D], ph);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem + COL_DQ + lane_base + half * 64, r0);
        tmem_ld32(tmem + COL_DQ + lane_base + half * 64 + 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&sm.bar[BAR_DQ]);
        // two [128 rows x 32 float] boxes per half, 128-byte swizzle; lane = query row
        uint8_t* stage = half == 0 ? sm.ds : sm.d_o[st];
        uint8_t* row0 = stage + row * 128;
        uint8_t* row1 = stage + kDqBox + row * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int chunk = u ^ (row & 7);
          *reinterpret_cast<uint4*>(row0 + chunk * 16) = make_uint4(r0[u * 4], r0[u * 4 + 1], r0[u * 4 + 2], r0[u * 4 + 3]);
          *reinterpret_cast<uint4*>(row1 + chunk * 16) = make_uint4(r1[u * 4], r1[u * 4 + 1], r1[u * 4 + 2], r1[u * 4 + 3]);
        }
      }
      fence_proxy_async();
      ok = consumer_sync(&sm.bar[BAR_SYNC3], ph);
      if (!ok) break;
      if (threadIdx.x == 0) {
        tma_reduce_add_4d(&map_dq, sm.ds, 0, h_cur, q0, b);
        tma_reduce_add_4d(&map_dq, sm.ds + kDqBox, 32, h_cur, q0, b);
        tma_reduce_add_4d(&map_dq, sm.d_o[st], 64, h_cur, q0, b);
        tma_reduce_add_4d(&map_dq, sm.d_o[st] + kDqBox, 96, h_cur, q0, b);
        bulk_commit();
      }
    }
    if (threadIdx.x == 0 && total > 0) bulk_wait0();  // the last reduce must be complete before the CTA retires

    // ---- epilogue: dK (scaled) and dV of this kv tile
    if (!ok) {
      report_device_error(p.status, 320 + warp);
    } else {
      // every lane takes part in the collective TMEM loads; only rows inside the tensor store
      const bool store = k < a.L;
      const int ks = store ? k : 0;
      __nv_bfloat16* dk = static_cast<__nv_bfloat16*>(a.dk.ptr) + (int64_t)b * a.dk.stride_b + (int64_t)ks * a.dk.stride_l + (int64_t)hk * a.dk.stride_h + half * 64;
      __nv_bfloat16* dv = static_cast<__nv_bfloat16*>(a.dv.ptr) + (int64_t)b * a.dv.stride_b + (int64_t)ks * a.dv.stride_l + (int64_t)hk * a.dv.stride_h + half * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rk[32], rv[32];
        if (total > 0) {
          tmem_ld32(tmem + COL_DK + lane_base + half * 64 + c * 32, rk);
          tmem_ld32(tmem + COL_DV + lane_base + half * 64 + c * 32, rv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) { rk[j] = 0u; rv[j] = 0u; }
        }
        if (store) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 ok4, ov4;
            ok4.x = pack_bf16(__uint_as_float(rk[j]) * a.scale, __uint_as_float(rk[j + 1]) * a.scale);
            ok4.y = pack_bf16(__uint_as_float(rk[j + 2]) * a.scale, __uint_as_float(rk[j + 3]) * a.scale);
            ok4.z = pack_bf16(__uint_as_float(rk[j + 4]) * a.scale, __uint_as_float(rk[j + 5]) * a.scale);
            ok4.w = pack_bf16(__uint_as_float(rk[j + 6]) * a.scale, __uint_as_float(rk[j + 7]) * a.scale);
            ov4.x = pack_bf16(__uint_as_float(rv[j]), __uint_as_float(rv[j + 1]));
            ov4.y = pack_bf16(__uint_as_float(rv[j + 2]), __uint_as_float(rv[j + 3]));
            ov4.z = pack_bf16(__uint_as_float(rv[j + 4]), __uint_as_float(rv[j + 5]));
            ov4.w = pack_bf16(__uint_as_float(rv[j + 6]), __uint_as_float(rv[j + 7]));
            *reinterpret_cast<uint4*>(dk + c * 32 + j) = ok4;
            *reinterpret_cast<uint4*>(dv + c * 32 + j) = ov4;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemCols);
}

// dq = bf16(dq_accum * scale)
__global__ void dq_convert_kernel(const float* __restrict__ acc, bma_tensor dq, int B, int N, int H, float scale) {
  const int64_t total = (int64_t)B * N * H * (HD / 8);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % (HD / 8));
    const int h = (int)((i / (HD / 8)) % H);
    const int n = (int)((i / ((int64_t)(HD / 8) * H)) % N);
    const int b = (int)(i / ((int64_t)(HD / 8) * H * N));
    const float4 x = *reinterpret_cast<const float4*>(acc + i * 8);
    const float4 y = *reinterpret_cast<const float4*>(acc + i * 8 + 4);
    uint4 o;
    o.x = ptx::pack_bf16(x.x * scale, x.y * scale);
    o.y = ptx::pack_bf16(x.z * scale, x.w * scale);
    o.z = ptx::pack_bf16(y.x * scale, y.y * scale);
    o.w = ptx::pack_bf16(y.z * scale, y.w * scale);
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(dq.ptr) + (int64_t)b * dq.stride_b + (int64_t)n * dq.stride_l + (int64_t)h * dq.stride_h + c8 * 8;
    *reinterpret_cast<uint4*>(dst) = o;
  }
}

bool aligned16(const bma_tensor& t) {
  return t.ptr && (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && t.stride_b % 8 == 0 && t.stride_l % 8 == 0 && t.stride_h % 8 == 0;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 4-D float32 map over the contiguous [B, N, H, 128] dQ accumulator, box = [128 rows x 32 floats], 128-byte swizzle.
int make_dq_map(CUtensorMap* out, float* base, int B, int N, int H) {
  void* fnp = nullptr;
  cudaDriverEntryPointQueryResult qr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fnp, cudaEnableDefault, &qr) != cudaSuccess ||
      qr != cudaDriverEntryPointSuccess) {
    set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    return BMA_ERR_CUDA;
  }
  const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)N, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)HD * 4, (cuuint64_t)H * HD * 4, (cuuint64_t)N * H * HD * 4};
  const cuuint32_t box[4] = {32, 1, (cuuint32_t)BT, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(fnp)(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr,
                                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(dq)"); return BMA_ERR_CUDA; }
  return BMA_OK;
}

}  // namespace

bool sm100_bwd_supported(const bma_attn_args& a) { return sm100_supported(a); }

size_t sm100_bwd_workspace_bytes(const bma_attn_args& a) { return sizeof(float) * (size_t)a.B * a.N * a.Hq * a.d; }

int sm100_bwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, void* ws, size_t ws_bytes,
              cudaStream_t st) {
  BMA_REQUIRE(lists.q_block == BT && lists.kv_block == BT && lists.q_num, BMA_ERR_ARG);
  BMA_REQUIRE(a.d_o.dtype == BMA_DTYPE_BF16, BMA_ERR_UNSUPPORTED);  // bma_attn_bwd_preprocess provides the bf16 copy
  BMA_REQUIRE(aligned16(a.d_o) && aligned16(a.dq) && aligned16(a.dk) && aligned16(a.dv), BMA_ERR_UNSUPPORTED);
  BMA_REQUIRE(ws && ws_bytes >= sm100_bwd_workspace_bytes(a) && (reinterpret_cast<uintptr_t>(ws) & 127) == 0, BMA_ERR_WORKSPACE);
  // the per-row form of the block window needs the window to be constant over a 128-query tile
  int interval = (spec.flags & (BMA_MASK_SEGMENT | BMA_MASK_BITMAP)) ? 0 : 1;
  if ((spec.flags & BMA_MASK_BLOCK_WINDOW) && !(spec.win_block % BT == 0 && spec.q_offset % BT == 0)) interval = 0;

  CUtensorMap mq, mk, mv, mdo, mdq;
  int rc;
  if ((rc = make_tile_map_bf16(&mq, a.q.ptr, a.B, a.N, a.Hq, a.d, a.q.stride_b, a.q.stride_l, a.q.stride_h, BT))) return rc;
  if ((rc = make_tile_map_bf16(&mk, a.k.ptr, a.B, a.L, a.Hkv, a.d, a.k.stride_b, a.k.stride_l, a.k.stride_h, BT))) return rc;
  if ((rc = make_tile_map_bf16(&mv, a.v.ptr, a.B, a.L, a.Hkv, a.d, a.v.stride_b, a.v.stride_l, a.v.stride_h, BT))) return rc;
  if ((rc = make_tile_map_bf16(&mdo, a.d_o.ptr, a.B, a.N, a.Hq, a.d, a.d_o.stride_b, a.d_o.stride_l, a.d_o.stride_h, BT))) return rc;
  if ((rc = make_dq_map(&mdq, static_cast<float*>(ws), a.B, a.N, a.Hq))) return rc;

  BwdParams p;
  p.a = a; p.spec = spec; p.l = lists;
  p.scale_log2 = a.scale * kLog2e;
  p.interval_mask = interval;
  p.status = device_status_ptr();
  BMA_REQUIRE(p.status != nullptr, BMA_ERR_CUDA);
  BMA_CUDA_TRY(cudaMemsetAsync(ws, 0, sm100_bwd_workspace_bytes(a), st));
  const size_t smem = sizeof(BwdSmem);
  BMA_CUDA_TRY(cudaFuncSetAttribute(bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(ceil_div(a.L, BT), a.Hkv, a.B);
  bwd_kernel<<<grid, kThreads, smem, st>>>(mq, mk, mv, mdo, mdq, p);
  const int64_t n8 = (int64_t)a.B * a.N * a.Hq * (HD / 8);
  const int cgrid = (int)std::min<int64_t>((n8 + 255) / 256, 148 * 16);
  dq_convert_kernel<<<cgrid, 256, 0, st>>>(static_cast<float*>(ws), a.dq, a.B, a.N, a.Hq, a.scale);
  count_launches(2);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

}  // namespace bma
