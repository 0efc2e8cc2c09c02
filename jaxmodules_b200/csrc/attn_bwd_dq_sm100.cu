// Backward dQ for bf16, head dim 128 / 64, on the sm_100a tensor core (tcgen05 + TMEM + TMA): the
// variant that recomputes S and dP.  It runs when the caller gives bma_attn_bwd no scratch buffer
// (or one smaller than a single (batch, kv head) unit); otherwise attn_bwd_dq_replay_sm100.cu
// computes dQ from the dS tiles that the dK/dV kernel stored.
//
// Query-major, the mirror image of the forward kernel: one CTA per SM works on a PAIR of 128-query
// tiles (2p, 2p+1) of one (batch, query head) and walks the union of the kv tiles their block
// lists name; the dQ accumulators stay in tensor memory for the whole walk, so nothing is
// reduced through global memory and the summation order is fixed.  Per (query tile, kv tile):
//     S  = Q K^T             A = Q  (K-major),  B = K (K-major)      -> TMEM SD_x [x*128, +128)
//     dP = dO V^T            A = dO (K-major),  B = V (K-major)      -> the same columns, once S is in registers
//     dQ += dS K             A = dS (bf16 in TMEM over dP),  B = K (MN-major) -> TMEM [256 + x*128, +128)
// with P = exp2(S*scale*log2e - lse*log2e) and dS = P * (dP - delta) computed by the warpgroup of
// the tile (thread = query row, so lse and delta are per-thread scalars).  The exponentials run
// while dO V^T executes, and the two query tiles alternate on the tensor core.
//
//   warpgroup 0 / 1: element-wise math of tile A / B;  warp 8: TMA (Q, dO once; K two stages,
//   V one stage);  warp 9: tcgen05.mma issue.
// Every mbarrier wait is bounded; on a timeout the thread records an error code and unwinds.
#include "common.cuh"
#include "ptx_sm100.cuh"

// Element-wise math: 0 = scalar arithmetic; 1 = the packed two-wide FP32 instructions of sm_100 for the scale-and-shift
// and for dS = P * (dP - delta), with a quarter of the exponentials as a packed polynomial on the FMA pipe.
#ifndef BMA_DQ_MATH
#define BMA_DQ_MATH 1
#endif
#ifndef BMA_DQ_POLY
#define BMA_DQ_POLY 0  // measured: 3.84 ms against 3.78 ms for the whole backward on the config-2 shape, so off
#endif

namespace bma {
namespace {

using namespace ptx;

constexpr int BM = kSm100Tile, BN = kSm100Tile;  // the head dimension HD (64 or 128) is a template parameter
constexpr int kThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kHalfTile = BM * 64 * 2;
template <int HD> constexpr uint32_t kTileBytesOf = (HD / 64) * kHalfTile;  // a [128 x HD] operand tile
constexpr int kMaxKvTiles = 1024;  // merged kv list (16-bit entries) kept in shared memory: L <= 131072

enum {
  BAR_Q = 0,
  BAR_K_FULL0, BAR_K_FULL1, BAR_K_FREE0, BAR_K_FREE1, BAR_V_FULL, BAR_V_FREE,
  BAR_S0, BAR_S1, BAR_LS0, BAR_LS1, BAR_DP0, BAR_DP1, BAR_DS0, BAR_DS1, BAR_DQ0, BAR_DQ1, BAR_EPI0, BAR_EPI1,
  NUM_BARS
};

template <int HD>
struct __align__(1024) DqSmem {
  uint8_t q[2][kTileBytesOf<HD>];
  uint8_t d_o[2][kTileBytesOf<HD>];
  uint8_t k[2][kTileBytesOf<HD>];
  uint8_t v[kTileBytesOf<HD>];
  uint16_t merged[kMaxKvTiles];  // kv tile | class for tile A << 12 | class for tile B << 14  (1 partial, 2 full)
  uint64_t bar[NUM_BARS];
  uint32_t tmem_base;
  int n_merged;
};

struct DqParams {
  bma_attn_args a;
  bma_mask_spec spec;
  bma_block_lists l;
  float scale_log2;
  int interval_mask;
  int* status;
};

__device__ __forceinline__ void setmaxnreg_inc_200() { asm volatile("setmaxnreg.inc.sync.aligned.u32 200;"); }
__device__ __forceinline__ void setmaxnreg_dec_96() { asm volatile("setmaxnreg.dec.sync.aligned.u32 96;"); }

// Allowed key interval [jlo, jhi] (tile-local, inclusive) of query row q for interval-only masks.
__device__ __forceinline__ void row_interval(const MaskView& m, int q, int k0, int& jlo, int& jhi) {
  if (q >= m.q_valid) { jlo = 1; jhi = 0; return; }
  const int gq = q + m.q_offset;
  int lo = 0, hi = INT32_MAX;
  if (m.flags & BMA_MASK_CAUSAL) hi = min(hi, gq);
  if (m.flags & BMA_MASK_BAND) { lo = max(lo, gq - m.band_left); hi = min(hi, gq + m.band_right); }
  if (m.flags & BMA_MASK_BLOCK_WINDOW) {
    int wlo, whi;
    block_window_range(m, gq, wlo, whi);
    lo = max(lo, wlo);
    hi = min(hi, whi - 1);
  }
  jlo = lo - m.k_offset - k0;
  jhi = min(hi - m.k_offset, m.k_valid - 1) - k0;
}

template <int HD, bool KB>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
              const __grid_constant__ CUtensorMap map_dq, const DqParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t kTileBytes = kTileBytesOf<HD>;
  DqSmem<HD>& sm = *reinterpret_cast<DqSmem<HD>*>(smem_raw);

  const bma_attn_args& a = p.a;
  const int pair = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;  // provably warp-uniform
  const int wg = warp >> 2;
  const int NQ = p.l.NQ, NKV = p.l.NKV;

  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0) report_device_error(p.status, 401);
    return;
  }

  // ---- merged kv list of the two query tiles ------------------------------------------------
  const int lb = p.l.B == 1 ? 0 : b, lh = p.l.H == 1 ? 0 : h;
  uint8_t* cls0 = sm.v;                 // scratch: the V stage is not loaded before the list is built
  uint8_t* cls1 = sm.v + kMaxKvTiles;
  for (int i = threadIdx.x; i < NKV; i += kThreads) { cls0[i] = 0; cls1[i] = 0; }
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      const bool wide = i == BAR_LS0 || i == BAR_LS1 || i == BAR_DS0 || i == BAR_DS1 || i == BAR_EPI0 || i == BAR_EPI1;
      mbar_init(&sm.bar[i], wide ? 128 : 1);
    }
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 8 && lane == 0) {
    // Q and dO of the two query tiles do not depend on the block lists: their loads run under the
    // list build.  (Rows past the end are zero-filled by TMA.)
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_do);
    mbar_expect_tx(&sm.bar[BAR_Q], 4 * kTileBytes);
#pragma unroll
    for (int x = 0; x < 2; ++x)
#pragma unroll
      for (int box = 0; box < HD / 64; ++box) {
        tma_load_4d(sm.q[x] + box * kHalfTile, &map_q, &sm.bar[BAR_Q], box * 64, h, (pair * 2 + x) * BM, b);
        tma_load_4d(sm.d_o[x] + box * kHalfTile, &map_do, &sm.bar[BAR_Q], box * 64, h, (pair * 2 + x) * BM, b);
      }
  }
  for (int x = 0; x < 2; ++x) {
    const int qi = pair * 2 + x;
    if (qi >= NQ) break;
    const int64_t lrow = ((int64_t)lb * p.l.H + lh) * NQ + qi;
    const int nfull = p.l.full_kv_num[lrow], npart = p.l.kv_num[lrow];
    const int32_t* full_idx = p.l.full_kv_idx + lrow * NKV;
    const int32_t* part_idx = p.l.kv_idx + lrow * NKV;
    uint8_t* cls = x ? cls1 : cls0;
    for (int i = threadIdx.x; i < nfull; i += kThreads) cls[full_idx[i]] = 2;
    for (int i = threadIdx.x; i < npart; i += kThreads) cls[part_idx[i]] = 1;
  }
  __syncthreads();
  if (warp == 0) {
    int count = 0;
    for (int base = 0; base < NKV; base += 32) {
      const int j = base + lane;
      const uint32_t ca = j < NKV ? cls0[j] : 0, cb = j < NKV ? cls1[j] : 0;
      const unsigned m = __ballot_sync(0xffffffffu, (ca | cb) != 0);
      if (ca | cb) sm.merged[count + __popc(m & ((1u << lane) - 1))] = (uint16_t)((uint32_t)j | (ca << 12) | (cb << 14));
      count += __popc(m);
    }
    if (lane == 0) sm.n_merged = count;
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
    setmaxnreg_dec_96();
    if (warp == 8 && lane == 0 && T > 0) {
      // ---------------------------------------------------------------- TMA producer
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      auto load_tile = [&](const CUtensorMap* m, uint8_t* dst, uint64_t* bar, int head, int row0) {
#pragma unroll
        for (int box = 0; box < HD / 64; ++box) tma_load_4d(dst + box * kHalfTile, m, bar, box * 64, head, row0, b);
      };
      bool ok = true;
      for (int n = 0; n < T && ok; ++n) {
        const int st = n & 1;
        const int row0 = (int)(sm.merged[n] & 0x3ffu) * BN;
        if (n >= 2) ok = mbar_wait(&sm.bar[BAR_K_FREE0 + st], ((n >> 1) - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_K_FULL0 + st], kTileBytes);
        load_tile(&map_k, sm.k[st], &sm.bar[BAR_K_FULL0 + st], hk, row0);
        if (n >= 1) ok = mbar_wait(&sm.bar[BAR_V_FREE], (n - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_V_FULL], kTileBytes);
        load_tile(&map_v, sm.v, &sm.bar[BAR_V_FULL], hk, row0);
      }
      if (!ok) report_device_error(p.status, 410);
    } else if (warp == 9 && T > 0) {
      // ---------------------------------------------------------------- MMA issuer: the whole warp runs the loop
      // (warp-uniform control flow and descriptors), one elected lane issues the tcgen05 instructions.  A loop run
      // by lane 0 alone costs ~60-70 cycles of issue per MMA under load — no slack against the 64 cycles an MMA takes.
      const bool leader = elect_one();
      constexpr uint32_t idesc_kk = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_kn = make_idesc_bf16(BM, HD, 0, 1);
      // descriptors are built once; per MMA only the 16-byte-unit start address moves
      const uint64_t dq0 = make_smem_desc(smem_u32(sm.q[0]), 16, 1024), dq1 = make_smem_desc(smem_u32(sm.q[1]), 16, 1024);
      const uint64_t ddo0 = make_smem_desc(smem_u32(sm.d_o[0]), 16, 1024), ddo1 = make_smem_desc(smem_u32(sm.d_o[1]), 16, 1024);
      const uint64_t dk0 = make_smem_desc(smem_u32(sm.k[0]), 16, 1024);            // K-major (S = Q K^T)
      const uint64_t dkm0 = make_smem_desc(smem_u32(sm.k[0]), kHalfTile, 1024);    // MN-major (dQ += dS K)
      const uint64_t dv = make_smem_desc(smem_u32(sm.v), 16, 1024);
      constexpr uint32_t kStageUnits = kTileBytes >> 4;
      int cnt0 = 0, cnt1 = 0;  // tiles of x already folded into dQ_x (phase counter of the per-tile barriers)
      bool ok = mbar_wait(&sm.bar[BAR_Q], 0);

      auto issue_s = [&](int x, int st) {  // S_x = Q_x K^T
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfTile + (ks & 3) * 32) >> 4;
          if (leader) mma_ss(tmem + x * 128, (x == 0 ? dq0 : dq1) + off, dk0 + (uint32_t)(st * kStageUnits + off), idesc_kk, ks > 0);
        }
        if (leader) mma_commit(&sm.bar[BAR_S0 + x]);
      };
      if (ok) ok = mbar_wait(&sm.bar[BAR_K_FULL0], 0);
      if (ok) {
        tc_fence_after();
        const uint32_t e = sm.merged[0];
        if ((e >> 12) & 3u) issue_s(0, 0);
        if ((e >> 14) & 3u) issue_s(1, 0);
      }
      for (int n = 0; n < T && ok; ++n) {
        const int st = n & 1;
        const uint32_t e = sm.merged[n];
        const uint32_t e_next = (n + 1 < T) ? sm.merged[n + 1] : 0u;
        ok = mbar_wait(&sm.bar[BAR_V_FULL], n & 1);
        if (!ok) break;
        // dP_x = dO_x V^T into the S columns, as soon as the warpgroup holds S in registers
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!((e >> (12 + 2 * x)) & 3u)) continue;
          ok = mbar_wait(&sm.bar[BAR_LS0 + x], (x == 0 ? cnt0 : cnt1) & 1);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = ((ks >> 2) * kHalfTile + (ks & 3) * 32) >> 4;
            if (leader) mma_ss(tmem + x * 128, (x == 0 ? ddo0 : ddo1) + off, dv + off, idesc_kk, ks > 0);
          }
          if (leader) mma_commit(&sm.bar[BAR_DP0 + x]);
        }
        if (!ok) break;
        if (leader) mma_commit(&sm.bar[BAR_V_FREE]);
        if (n + 1 < T) {
          ok = mbar_wait(&sm.bar[BAR_K_FULL0 + (st ^ 1)], ((n + 1) >> 1) & 1);
          if (!ok) break;
        }
        // dQ_x += dS_x K, then the next S_x into the same columns (in-order execution keeps dS intact)
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if ((e >> (12 + 2 * x)) & 3u) {
            int& cnt = x == 0 ? cnt0 : cnt1;
            ok = mbar_wait(&sm.bar[BAR_DS0 + x], cnt & 1);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              if (leader)
                mma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8, dkm0 + (uint32_t)(st * kStageUnits + ks * (2048 >> 4)),
                       idesc_kn, (cnt > 0) || (ks > 0));
            if (leader) mma_commit(&sm.bar[BAR_DQ0 + x]);
            ++cnt;
          }
          if ((e_next >> (12 + 2 * x)) & 3u) { tc_fence_after(); issue_s(x, st ^ 1); }
        }
        if (!ok) break;
        if (leader) mma_commit(&sm.bar[BAR_K_FREE0 + st]);
      }
      if (!ok && leader) report_device_error(p.status, 420);
    }
  } else {
    // ------------------------------------------------------------------ element-wise warpgroups
    setmaxnreg_inc_200();
    const int x = wg;
    const int qi = pair * 2 + x;
    const int row = threadIdx.x & 127;  // TMEM lane == query row of the tile
    const int q = qi * BM + row;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_sd = tmem + x * 128 + lane_base, tmem_dq = tmem + 256 + x * 128 + lane_base;
    const MaskView mv = make_mask_view(p.spec, b, h);
    const float kb2 = KB ? __ldg(a.key_bias + h) * kLog2e : 0.f;  // per-head key bias, log2 units
    float lse2 = INFINITY, delta = 0.f;  // +inf: rows outside the tensor or without any key get P = 0
    if (qi < NQ && q < a.N) {
      const int64_t off = ((int64_t)b * a.Hq + h) * a.N + q;
      const float lv = a.lse[off];
      lse2 = (lv == -INFINITY) ? INFINITY : lv * kLog2e;
      delta = a.delta[off];
    }
    bool ok = true;
    int cnt = 0;

    for (int n = 0; n < T; ++n) {
      const uint32_t e = sm.merged[n];
      const uint32_t cls = (e >> (12 + 2 * x)) & 3u;
      if (cls == 0) continue;
      const int k0 = (int)(e & 0x3ffu) * BN;
      ok = mbar_wait(&sm.bar[BAR_S0 + x], cnt & 1);
      if (!ok) break;
      tc_fence_after();
      float pr[BN];
      {
        uint32_t r0[32], r1[32], r2[32], r3[32];
        tmem_ld32(tmem_sd + 0, r0);
        tmem_ld32(tmem_sd + 32, r1);
        tmem_ld32(tmem_sd + 64, r2);
        tmem_ld32(tmem_sd + 96, r3);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&sm.bar[BAR_LS0 + x]);  // dO V^T may overwrite the columns now
if constexpr (KB) {  // key bias: + kb2 * (global key index) on every column
          const float base = fmaf(kb2, (float)(mv.k_offset + k0), -lse2);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            pr[j] = ex2(fmaf(__uint_as_float(r0[j]), p.scale_log2, fmaf((float)j, kb2, base)));
            pr[32 + j] = ex2(fmaf(__uint_as_float(r1[j]), p.scale_log2, fmaf((float)(32 + j), kb2, base)));
            pr[64 + j] = ex2(fmaf(__uint_as_float(r2[j]), p.scale_log2, fmaf((float)(64 + j), kb2, base)));
            pr[96 + j] = ex2(fmaf(__uint_as_float(r3[j]), p.scale_log2, fmaf((float)(96 + j), kb2, base)));
          }
        } else {
#if BMA_DQ_MATH == 0
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          pr[j] = ex2(fmaf(__uint_as_float(r0[j]), p.scale_log2, -lse2));
          pr[32 + j] = ex2(fmaf(__uint_as_float(r1[j]), p.scale_log2, -lse2));
          pr[64 + j] = ex2(fmaf(__uint_as_float(r2[j]), p.scale_log2, -lse2));
#if BMA_DQ_POLY
          pr[96 + j] = exp2_fma(fmaf(__uint_as_float(r3[j]), p.scale_log2, -lse2));  // a quarter of the exponentials on the FMA pipe
#else
          pr[96 + j] = ex2(fmaf(__uint_as_float(r3[j]), p.scale_log2, -lse2));
#endif
        }
#else     // packed two-wide FP32 arithmetic; a quarter of the exponentials as a packed polynomial on the FMA pipe
        {
          const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1])), sc2, nl2);
            const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1])), sc2, nl2);
            const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(r2[j]), __uint_as_float(r2[j + 1])), sc2, nl2);
            const float2 x3 = __ffma2_rn(make_float2(__uint_as_float(r3[j]), __uint_as_float(r3[j + 1])), sc2, nl2);
            pr[j] = ex2(x0.x); pr[j + 1] = ex2(x0.y);
            pr[32 + j] = ex2(x1.x); pr[32 + j + 1] = ex2(x1.y);
            pr[64 + j] = ex2(x2.x); pr[64 + j + 1] = ex2(x2.y);
            const float2 e3 = exp2_fma2(x3);
            pr[96 + j] = e3.x; pr[96 + j + 1] = e3.y;
          }
        }
#endif
        }
      }
      if (cls == 1) {
        uint32_t bits[4];
        {
          int jlo, jhi;
          row_interval(mv, q, k0, jlo, jhi);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int lo = max(jlo - c * 32, 0), hi = min(jhi - c * 32, 31);
            bits[c] = (lo <= hi) ? ((0xffffffffu >> (31 - hi)) & (0xffffffffu << lo)) : 0u;
          }
          if (mv.flags & kTableTerms) {  // segment ids / bit table: 32 keys per word
#pragma unroll
            for (int c = 0; c < 4; ++c)
              if (bits[c]) bits[c] &= table_bits_row32(mv, q, k0 + c * 32);
          }
        }
#pragma unroll
        for (int j = 0; j < BN; ++j) pr[j] = (bits[j >> 5] >> (j & 31)) & 1u ? pr[j] : 0.f;
      }
      // dS = P * (dP - delta), bf16, back into the first 64 columns
      ok = mbar_wait(&sm.bar[BAR_DP0 + x], cnt & 1);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_sd + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
#if BMA_DQ_MATH == 0
          const float d0 = pr[c * 32 + 2 * j] * (__uint_as_float(r[2 * j]) - delta);
          const float d1 = pr[c * 32 + 2 * j + 1] * (__uint_as_float(r[2 * j + 1]) - delta);
          pk[j] = pack_bf16(d0, d1);
#else
          const float2 t = __fadd2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), make_float2(-delta, -delta));
          const float2 ds = __fmul2_rn(make_float2(pr[c * 32 + 2 * j], pr[c * 32 + 2 * j + 1]), t);
          pk[j] = pack_bf16(ds.x, ds.y);
#endif
        }
        tmem_st16(tmem_sd + c * 16, pk);  // columns [16c, 16c+16) lie inside chunks already read
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.bar[BAR_DS0 + x]);
      ++cnt;
    }

    // ---- epilogue: dQ * scale
    if (ok && cnt > 0) ok = mbar_wait(&sm.bar[BAR_DQ0 + x], (cnt - 1) & 1);
    if (!ok) {
      report_device_error(p.status, 430 + warp);
    } else if (qi < NQ) {
      // dQ goes through shared memory — the tile's own Q buffer, which no MMA reads any more — in the
      // 128-byte-swizzled box layout and leaves as TMA stores of whole lines (rows past the end of the
      // tensor are clipped by the tensor map).  A tile without any key block must first let the Q load land.
      if (cnt == 0) ok = mbar_wait(&sm.bar[BAR_Q], 0);
      tc_fence_after();
      uint8_t* q_row = sm.q[x] + row * 128;
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
          const int chunk = ((c & 1) * 4 + u) ^ (row & 7);            // 32 columns = four 16-byte chunks of a box row
          *reinterpret_cast<uint4*>(q_row + (c >> 1) * kHalfTile + chunk * 16) = v4;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the TMA engine reads the staged tile through the async proxy
      mbar_arrive(&sm.bar[BAR_EPI0 + x]);
      ok = ok && mbar_wait(&sm.bar[BAR_EPI0 + x], 0);
      if (!ok) {
        report_device_error(p.status, 450 + warp);
      } else if (row == 0) {
#pragma unroll
        for (int box = 0; box < HD / 64; ++box) tma_store_4d(&map_dq, sm.q[x] + box * kHalfTile, box * 64, h, qi * BM, b);
        bulk_commit();
        bulk_wait_read0();  // shared memory must stay intact until the stores have read it
      }
    }
  }

  if (T == 0 && warp == 8 && lane == 0 && !mbar_wait(&sm.bar[BAR_Q], 0))   // nobody consumed Q / dO: let the loads land before the CTA ends
    report_device_error(p.status, 440);
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

int sm100_bwd_dq(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st) {
  BMA_REQUIRE(lists.NKV <= kMaxKvTiles, BMA_ERR_LIMIT);
  CUtensorMap mq, mk, mv, mdo, mdq;
  int rc;
  if ((rc = make_tile_map_bf16(&mq, a.q.ptr, a.B, a.N, a.Hq, a.d, a.q.stride_b, a.q.stride_l, a.q.stride_h, BM))) return rc;
  if ((rc = make_tile_map_bf16(&mk, a.k.ptr, a.B, a.L, a.Hkv, a.d, a.k.stride_b, a.k.stride_l, a.k.stride_h, BN))) return rc;
  if ((rc = make_tile_map_bf16(&mv, a.v.ptr, a.B, a.L, a.Hkv, a.d, a.v.stride_b, a.v.stride_l, a.v.stride_h, BN))) return rc;
  if ((rc = make_tile_map_bf16(&mdo, a.d_o.ptr, a.B, a.N, a.Hq, a.d, a.d_o.stride_b, a.d_o.stride_l, a.d_o.stride_h, BM))) return rc;
  if ((rc = make_tile_map_bf16(&mdq, a.dq.ptr, a.B, a.N, a.Hq, a.d, a.dq.stride_b, a.dq.stride_l, a.dq.stride_h, BM))) return rc;
  DqParams p;
  p.a = a; p.spec = spec; p.l = lists;
  p.scale_log2 = a.scale * kLog2e;
  p.interval_mask = (spec.flags & kTableTerms) ? 0 : 1;
  p.status = device_status_ptr();
  BMA_REQUIRE(p.status != nullptr, BMA_ERR_CUDA);

  dim3 grid(ceil_div(ceil_div(a.N, BM), 2), a.Hq, a.B);
  auto launch = [&](auto kernel, size_t smem) -> int {
    BMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kThreads, smem, st>>>(mq, mk, mv, mdo, mdq, p);
    return BMA_OK;
  };
  if (a.d == 128) rc = a.key_bias ? launch(bwd_dq_kernel<128, true>, sizeof(DqSmem<128>)) : launch(bwd_dq_kernel<128, false>, sizeof(DqSmem<128>));
  else rc = a.key_bias ? launch(bwd_dq_kernel<64, true>, sizeof(DqSmem<64>)) : launch(bwd_dq_kernel<64, false>, sizeof(DqSmem<64>));
  if (rc) return rc;
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

}  // namespace bma
