// Flash-style forward for bf16, head dim 128, on the sm_100a tensor core (tcgen05) with TMEM
// accumulators and TMA-staged operands.
//
// One CTA per SM works on a PAIR of 128-query tiles (2p, 2p+1) of one (batch, query head) and
// walks the union of the kv tiles their block lists name; each K / V tile is fetched once for both.
// The two query tiles ping-pong on the tensor core: while one tile's softmax runs, the other
// tile's MMAs execute.
//
//   warpgroup 0 / 1 (thread = query row of tile A / B): read S from TMEM, fp32 online softmax
//       (exp2 with the scale folded in, running max with lazy rescale of O), write P as bf16 over
//       the S columns, final O / l and the log-sum-exp.  The element predicate is evaluated only
//       on partial tiles (a per-row bit mask); full tiles take a mask-free path.
//   warp 8  (one lane): TMA loads, Q once, K and V through two-stage rings (128-byte swizzle,
//       K-major boxes of [128 rows x 64 columns]).
//   warp 9  (one lane): tcgen05.mma issue:  S_x = Q_x K^T  (A, B from shared memory),
//       O_x (+)= P_x V  (A = P from tensor memory, B = V read MN-major).
//
// TMEM (512 columns): S_A [0,128) (P_A bf16 in [0,64)), S_B [128,256), O_A [256,384), O_B [384,512).
// MMAs issued by one thread execute in issue order, so P_x V (reads P_x) followed by the next
// S_x (overwrites it) needs no extra barrier.  Every mbarrier wait is bounded; on a timeout the
// thread records an error code and unwinds to the common exit where TMEM is released.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace bma {
namespace {

using namespace ptx;

constexpr int BM = kSm100Tile, BN = kSm100Tile;  // the head dimension HD (64 or 128) is a template parameter
constexpr int kThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kHalfTile = BM * 64 * 2;     // one [128 x 64] bf16 box
template <int HD> constexpr uint32_t kTileBytesOf = (HD / 64) * kHalfTile;  // a [128 x HD] operand tile: HD/64 boxes
constexpr float kRescaleThreshold = 8.0f;       // log2 units: rescale O only when the max grew by > 2^8
constexpr int kMaxKvTiles = 4096;               // merged kv list kept in shared memory
// P goes from the softmax warps to the MMA warp in two parts, each with its own barrier, so that the first k-steps of
// P V run under the remaining exponentials.  The exponentials are taken in four chunks of 32 keys (two k-steps) whose
// TMEM stores are issued as they become ready; the first part is kSplitChunks chunks long.
// Measured (same box, forward TFLOP/s on config 2 / L=8192 / config 5): four parts of one chunk 1037 / 1065 / 1192 against
// 1091 / 1129 / 1258 for two even parts -- each hand-over costs a TMEM store wait, a fence and 128 barrier arrivals; a
// 96 + 32 split (fewer k-steps of P V behind the last exponential) 1069 / 1122 / 1242 against 1067 / 1131 / 1248 for
// 64 + 64: the tail of P V is not what the next S waits for -- it queues behind the other tile's MMAs.
#ifndef BMA_FWD_P_SPLIT
#define BMA_FWD_P_SPLIT 2
#endif
constexpr int kPParts = 2;
constexpr int kSplitChunks = BMA_FWD_P_SPLIT;   // 2: 64 + 64 keys, 3: 96 + 32 keys

enum {
  BAR_Q = 0,
  BAR_K_FULL0, BAR_K_FULL1, BAR_K_FREE0, BAR_K_FREE1,
  BAR_V_FULL0, BAR_V_FULL1, BAR_V_FREE0, BAR_V_FREE1,
  BAR_S0, BAR_S1, BAR_PART, BAR_PART_LAST = BAR_PART + 2 * kPParts - 1, BAR_O0, BAR_O1, BAR_EPI0, BAR_EPI1,
  NUM_BARS
};

template <int HD>
struct __align__(1024) FwdSmem {
  uint8_t q[2][kTileBytesOf<HD>];
  uint8_t k[2][kTileBytesOf<HD>];
  uint8_t v[2][kTileBytesOf<HD>];
  uint32_t merged[kMaxKvTiles];  // kv tile | class for tile A << 16 | class for tile B << 18  (1 partial, 2 full)
  uint8_t cls[2][kMaxKvTiles];
  uint64_t bar[NUM_BARS];
  uint32_t tmem_base;
  int n_merged;
};

struct FwdParams {
  bma_attn_args a;
  bma_mask_spec spec;
  bma_block_lists l;
  float scale_log2;
  int interval_mask;  // 1: the mask has only interval terms (no segment ids / bit table)
  int* status;
};

__device__ __forceinline__ void setmaxnreg_inc_208() { asm volatile("setmaxnreg.inc.sync.aligned.u32 208;"); }
__device__ __forceinline__ void setmaxnreg_dec_80() { asm volatile("setmaxnreg.dec.sync.aligned.u32 80;"); }
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Exponentials of 2 * WORDS scores of one row against the reference maximum: p = 2^(s * sc - m), packed to bf16 pairs in pk,
// returns their sum.  MUFU is the narrowest pipe of the softmax (8 issue cycles per warp instruction, shared by the two
// warpgroups whose exponential phases overlap), so a share of the exponentials is a polynomial on the FMA pipe, and the
// scale / subtract, the polynomial and the row sum use the packed two-wide FP32 instructions of sm_100:
//   BMA_FWD_EXP_MODE 0: scalar arithmetic, a quarter of the exponentials on the FMA pipe
//   BMA_FWD_EXP_MODE 1: packed arithmetic, half of them on the FMA pipe
//   BMA_FWD_EXP_MODE 2: packed arithmetic, a quarter on the FMA pipe
//   BMA_FWD_EXP_MODE 3: packed arithmetic, three eighths on the FMA pipe
#ifndef BMA_FWD_EXP_MODE
#define BMA_FWD_EXP_MODE 2
#endif
template <int WORDS>
__device__ __forceinline__ float exp_part(const float* s, float sc, float m_sub, uint32_t (&pk)[WORDS]) {
#if BMA_FWD_EXP_MODE == 0
  float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll
  for (int j = 0; j < WORDS; j += 2) {
    const float e0 = ex2(fmaf(s[2 * j], sc, -m_sub));
    const float e1 = ex2(fmaf(s[2 * j + 1], sc, -m_sub));
    const float e2 = ex2(fmaf(s[2 * j + 2], sc, -m_sub));
    const float e3 = exp2_fma(fmaf(s[2 * j + 3], sc, -m_sub));
    rs0 += e0; rs1 += e1; rs2 += e2; rs3 += e3;
    pk[j] = pack_bf16(e0, e1);
    pk[j + 1] = pack_bf16(e2, e3);
  }
  return (rs0 + rs1) + (rs2 + rs3);
#else
  const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(-m_sub, -m_sub);
  float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);
#if BMA_FWD_EXP_MODE == 1
#pragma unroll
  for (int j = 0; j < WORDS; j += 2) {
    const float2 xa = __ffma2_rn(make_float2(s[2 * j], s[2 * j + 1]), sc2, nm2);
    const float2 xb = __ffma2_rn(make_float2(s[2 * j + 2], s[2 * j + 3]), sc2, nm2);
    const float2 ea = make_float2(ex2(xa.x), ex2(xa.y));
    const float2 eb = exp2_fma2(xb);
    ra = __fadd2_rn(ra, ea);
    rb = __fadd2_rn(rb, eb);
    pk[j] = pack_bf16(ea.x, ea.y);
    pk[j + 1] = pack_bf16(eb.x, eb.y);
  }
#elif BMA_FWD_EXP_MODE == 3
#pragma unroll
  for (int j = 0; j < WORDS; j += 8) {
    float2 e[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float2 x = __ffma2_rn(make_float2(s[2 * (j + u)], s[2 * (j + u) + 1]), sc2, nm2);
      e[u] = (u == 2 || u == 5 || u == 7) ? exp2_fma2(x) : make_float2(ex2(x.x), ex2(x.y));
      pk[j + u] = pack_bf16(e[u].x, e[u].y);
    }
    ra = __fadd2_rn(ra, __fadd2_rn(__fadd2_rn(e[0], e[1]), __fadd2_rn(e[2], e[3])));
    rb = __fadd2_rn(rb, __fadd2_rn(__fadd2_rn(e[4], e[5]), __fadd2_rn(e[6], e[7])));
  }
#else
#pragma unroll
  for (int j = 0; j < WORDS; j += 4) {
    const float2 x0 = __ffma2_rn(make_float2(s[2 * j], s[2 * j + 1]), sc2, nm2);
    const float2 x1 = __ffma2_rn(make_float2(s[2 * j + 2], s[2 * j + 3]), sc2, nm2);
    const float2 x2 = __ffma2_rn(make_float2(s[2 * j + 4], s[2 * j + 5]), sc2, nm2);
    const float2 x3 = __ffma2_rn(make_float2(s[2 * j + 6], s[2 * j + 7]), sc2, nm2);
    const float2 e0 = make_float2(ex2(x0.x), ex2(x0.y));
    const float2 e1 = make_float2(ex2(x1.x), ex2(x1.y));
    const float2 e2 = make_float2(ex2(x2.x), ex2(x2.y));
    const float2 e3 = exp2_fma2(x3);
    ra = __fadd2_rn(ra, __fadd2_rn(e0, e1));
    rb = __fadd2_rn(rb, __fadd2_rn(e2, e3));
    pk[j] = pack_bf16(e0.x, e0.y);
    pk[j + 1] = pack_bf16(e1.x, e1.y);
    pk[j + 2] = pack_bf16(e2.x, e2.y);
    pk[j + 3] = pack_bf16(e3.x, e3.y);
  }
#endif
  return (ra.x + ra.y) + (rb.x + rb.y);
#endif
}

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

// KB: the variant that folds the scale (and the per-head key bias, bma_attn_args.key_bias, when there is one)
// into the scores BEFORE the running maximum is taken.  Compiled in only where it is needed: a key bias, or a
// negative scale, for which max(raw score) * scale is the MINIMUM of the scaled scores and the exponentials
// taken against it would overflow.
template <int HD, bool KB>
__global__ void __launch_bounds__(kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t kTileBytes = kTileBytesOf<HD>;
  FwdSmem<HD>& sm = *reinterpret_cast<FwdSmem<HD>*>(smem_raw);

  const bma_attn_args& a = p.a;
  const int pair = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;  // provably warp-uniform
  const int wg = warp >> 2;
  const int NQ = p.l.NQ, NKV = p.l.NKV;

  if ((smem_u32(smem_raw) & 1023u) != 0u) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) report_device_error(p.status, 101);
    return;
  }

  // ---- merged kv list of the two query tiles ------------------------------------------------
  const int lb = p.l.B == 1 ? 0 : b, lh = p.l.H == 1 ? 0 : h;
  for (int i = threadIdx.x; i < NKV; i += kThreads) { sm.cls[0][i] = 0; sm.cls[1][i] = 0; }
  if (threadIdx.x == 0) {
    mbar_init(&sm.bar[BAR_Q], 1);
    for (int i = BAR_K_FULL0; i < NUM_BARS; ++i)
      mbar_init(&sm.bar[i], ((i >= BAR_PART && i <= BAR_PART_LAST) || i == BAR_EPI0 || i == BAR_EPI1) ? 128 : 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 8 && lane == 0) {
    // The two Q tiles do not depend on the block lists: their loads run under the list build.
    // (A tile past the end is zero-filled by TMA.)
    prefetch_tensormap(&map_q);
    mbar_expect_tx(&sm.bar[BAR_Q], 2 * kTileBytes);
#pragma unroll
    for (int x = 0; x < 2; ++x)
#pragma unroll
      for (int box = 0; box < HD / 64; ++box)
        tma_load_4d(sm.q[x] + box * kHalfTile, &map_q, &sm.bar[BAR_Q], box * 64, h, (pair * 2 + x) * BM, b);
  }
  for (int x = 0; x < 2; ++x) {
    const int qi = pair * 2 + x;
    if (qi >= NQ) break;
    const int64_t lrow = ((int64_t)lb * p.l.H + lh) * NQ + qi;
    const int nfull = p.l.full_kv_num[lrow], npart = p.l.kv_num[lrow];
    const int32_t* full_idx = p.l.full_kv_idx + lrow * NKV;
    const int32_t* part_idx = p.l.kv_idx + lrow * NKV;
    for (int i = threadIdx.x; i < nfull; i += kThreads) sm.cls[x][full_idx[i]] = 2;
    for (int i = threadIdx.x; i < npart; i += kThreads) sm.cls[x][part_idx[i]] = 1;
  }
  __syncthreads();
  if (warp == 0) {
    int count = 0;
    for (int base = 0; base < NKV; base += 32) {
      const int j = base + lane;
      const uint32_t ca = j < NKV ? sm.cls[0][j] : 0, cb = j < NKV ? sm.cls[1][j] : 0;
      const unsigned m = __ballot_sync(0xffffffffu, (ca | cb) != 0);
      if (ca | cb) sm.merged[count + __popc(m & ((1u << lane) - 1))] = (uint32_t)j | (ca << 16) | (cb << 18);
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
    setmaxnreg_dec_80();
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
        const int row0 = (int)(sm.merged[n] & 0xffffu) * BN;
        if (n >= 2) ok = mbar_wait(&sm.bar[BAR_K_FREE0 + st], ((n >> 1) - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_K_FULL0 + st], kTileBytes);
        load_tile(&map_k, sm.k[st], &sm.bar[BAR_K_FULL0 + st], hk, row0);
        if (n >= 2) ok = mbar_wait(&sm.bar[BAR_V_FREE0 + st], ((n >> 1) - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(&sm.bar[BAR_V_FULL0 + st], kTileBytes);
        load_tile(&map_v, sm.v[st], &sm.bar[BAR_V_FULL0 + st], hk, row0);
      }
      if (!ok) report_device_error(p.status, 110);
    } else if (warp == 9 && T > 0) {
      // ---------------------------------------------------------------- MMA issuer (whole warp, one elected lane issues)
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, HD, 0, 1);
      // Descriptors are built once; per MMA only the 16-byte-unit start address in the low bits moves
      // (tiles are 1024-byte aligned and below 256 KB, so the sum never leaves the address field).
      // Everything is kept in scalars: an array indexed by the stage would live in local memory and
      // every MMA would wait on a load — the issuing thread must stay ahead of the tensor core.
      const uint64_t dq0 = make_smem_desc(smem_u32(sm.q[0]), 16, 1024), dq1 = make_smem_desc(smem_u32(sm.q[1]), 16, 1024);
      const uint64_t dk0 = make_smem_desc(smem_u32(sm.k[0]), 16, 1024);
      const uint64_t dv0 = make_smem_desc(smem_u32(sm.v[0]), kHalfTile, 1024);
      constexpr uint32_t kStageUnits = kTileBytes >> 4;
      int cnt0 = 0, cnt1 = 0;  // tiles already multiplied into O_x (also the phase counter of BAR_PH / BAR_P)
      bool ok = mbar_wait(&sm.bar[BAR_Q], 0);

      auto issue_s = [&](int x, int st) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfTile + (ks & 3) * 32) >> 4;  // 64-column box, then 32 B per k-step
          if (leader) mma_ss(tmem + x * 128, (x == 0 ? dq0 : dq1) + off, dk0 + (uint32_t)(st * kStageUnits + off), idesc_s, ks > 0);
        }
        if (leader) mma_commit(&sm.bar[BAR_S0 + x]);
      };
      if (ok) ok = mbar_wait(&sm.bar[BAR_K_FULL0], 0);
      if (ok) {
        tc_fence_after();
        const uint32_t e = sm.merged[0];
        if ((e >> 16) & 3u) issue_s(0, 0);
        if ((e >> 18) & 3u) issue_s(1, 0);
        if (leader) mma_commit(&sm.bar[BAR_K_FREE0]);
      }
      for (int n = 0; n < T && ok; ++n) {
        const int st = n & 1;
        const uint32_t e = sm.merged[n];
        const uint32_t e_next = (n + 1 < T) ? sm.merged[n + 1] : 0u;
        ok = mbar_wait(&sm.bar[BAR_V_FULL0 + st], (n >> 1) & 1);
        if (ok && n + 1 < T) ok = mbar_wait(&sm.bar[BAR_K_FULL0 + (st ^ 1)], ((n + 1) >> 1) & 1);
        if (!ok) break;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if ((e >> (16 + 2 * x)) & 3u) {
            int& cnt = x == 0 ? cnt0 : cnt1;
            // P arrives in two halves (keys 0..63, then 64..127) so that the first k-steps run under
            // the second half of the exponentials
#pragma unroll
            for (int hf = 0; hf < kPParts; ++hf) {
              ok = mbar_wait(&sm.bar[BAR_PART + 2 * hf + x], cnt & 1);
              if (!ok) break;
              tc_fence_after();
#pragma unroll
              for (int ks = (hf == 0 ? 0 : 2 * kSplitChunks); ks < (hf == 0 ? 2 * kSplitChunks : 8); ++ks) {
                // B = V[kv rows][d] read MN-major: 16 kv rows per k-step = 2048 B; the two 64-column boxes are kHalfTile apart
                if (leader)
                  mma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8, dv0 + (uint32_t)(st * kStageUnits + ks * (2048 >> 4)),
                         idesc_o, (cnt > 0) || (ks > 0));
              }
            }
            if (!ok) break;
            if (leader) mma_commit(&sm.bar[BAR_O0 + x]);
            ++cnt;
          }
          if ((e_next >> (16 + 2 * x)) & 3u) issue_s(x, st ^ 1);
        }
        if (!ok) break;
        if (leader) {
          mma_commit(&sm.bar[BAR_V_FREE0 + st]);
          if (n + 1 < T) mma_commit(&sm.bar[BAR_K_FREE0 + (st ^ 1)]);
        }
      }
      if (!ok && leader) report_device_error(p.status, 120);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc_208();
    const int x = wg;                         // which query tile of the pair
    const int qi = pair * 2 + x;
    const int row = threadIdx.x & 127;        // TMEM lane == query row of the tile
    const int q = qi * BM + row;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem + x * 128 + lane_base, tmem_o = tmem + 256 + x * 128 + lane_base;
    const float kb2 = (KB && a.key_bias) ? __ldg(a.key_bias + h) * kLog2e : 0.f;  // per-head key bias, log2 units
    float m_ref = -INFINITY;  // reference max (log2 domain) the exponentials are taken against
    float l = 0.f;
    bool ok = true;
    int cnt = 0;

    for (int n = 0; n < T; ++n) {
      const uint32_t e = sm.merged[n];
      const uint32_t cls = (e >> (16 + 2 * x)) & 3u;
      if (cls == 0) continue;
      const int k0 = (int)(e & 0xffffu) * BN;
      ok = mbar_wait(&sm.bar[BAR_S0 + x], cnt & 1);
      if (!ok) break;
      tc_fence_after();
      float s[BN];
      {
        uint32_t r0[32], r1[32], r2[32], r3[32];
        tmem_ld32(tmem_s + 0, r0);
        tmem_ld32(tmem_s + 32, r1);
        tmem_ld32(tmem_s + 64, r2);
        tmem_ld32(tmem_s + 96, r3);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          s[j] = __uint_as_float(r0[j]);
          s[32 + j] = __uint_as_float(r1[j]);
          s[64 + j] = __uint_as_float(r2[j]);
          s[96 + j] = __uint_as_float(r3[j]);
        }
      }
      const float sc = KB ? 1.f : p.scale_log2;
      if constexpr (KB) {  // key bias: fold the scale and kb2 * (global key index) into the scores once
        const float base = kb2 * (float)(p.spec.k_offset + k0);
#pragma unroll
        for (int j = 0; j < BN; ++j) s[j] = fmaf(s[j], p.scale_log2, fmaf((float)j, kb2, base));
      }
      if (cls == 1) {  // partial tile: masked scores become -inf (their exponential is exactly 0)
        uint32_t bits[4];
        {
          // the mask description is rebuilt from the kernel parameters here rather than carried in registers through the full tiles
          const MaskView mv = make_mask_view(p.spec, b, h);
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
        for (int j = 0; j < BN; ++j) s[j] = (bits[j >> 5] >> (j & 31)) & 1u ? s[j] : -INFINITY;
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int j = 0; j < BN; j += 8) {
        mx0 = max3(mx0, s[j], s[j + 1]);
        mx1 = max3(mx1, s[j + 2], s[j + 3]);
        mx2 = max3(mx2, s[j + 4], s[j + 5]);
        mx3 = max3(mx3, s[j + 6], s[j + 7]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_cand = fmaxf(m_ref, mx * sc);
      // lazy rescale: keep the old reference unless the maximum grew by more than 2^threshold
      const bool grow = (m_cand - m_ref) > kRescaleThreshold;  // also true when m_ref == -inf and m_cand is finite
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m_ref - m_cand);  // 0 when m_ref == -inf
        m_ref = m_cand;
      }
      if (cnt > 0 && __any_sync(0xffffffffu, grow)) {
        // O_x must be quiescent: the previous P V of this tile has to be complete
        ok = mbar_wait(&sm.bar[BAR_O0 + x], (cnt - 1) & 1);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_o + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
          tmem_st32(tmem_o + c * 32, r);
        }
      }
      const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
      float row_sum = 0.f;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
        row_sum += exp_part<16>(&s[ch * 32], sc, m_sub, pk);
        tmem_st16(tmem_s + ch * 16, pk);
        if (ch == kSplitChunks - 1 || ch == 3) {   // end of a part: its stores have landed, the MMA warp may read it
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&sm.bar[BAR_PART + 2 * (ch == 3 ? 1 : 0) + x]);
        }
      }
      l = l * alpha + row_sum;
      ++cnt;
    }

    // ---- epilogue: O / l and the log-sum-exp
    if (ok && cnt > 0) ok = mbar_wait(&sm.bar[BAR_O0 + x], (cnt - 1) & 1);
    if (!ok) {
      report_device_error(p.status, 200 + warp);
    } else if (qi < NQ) {
      // O goes through shared memory — the tile's own Q buffer, which no MMA reads any more — in the
      // 128-byte-swizzled box layout and leaves as TMA stores of whole lines (rows past the end of the
      // tensor are clipped by the tensor map).  The buffer holds a bf16 tile of HD columns, i.e. HD/2 float32
      // columns at a time (two passes).  A tile without any key block must first let the Q load land.
      if (cnt == 0) ok = mbar_wait(&sm.bar[BAR_Q], 0);
      tc_fence_after();
      // A row whose reference maximum never became finite has seen no allowed key: O = 0 and lse = -inf.  (Its l is
      // not exactly 0: the polynomial exponential clamps its argument and returns 2^-126 for a masked score.)
      const bool dead = (m_ref == -INFINITY);
      const float inv = (l > 0.f && !dead) ? 1.f / l : 0.f;
      uint8_t* q_row = sm.q[x] + row * 128;
      uint32_t syncs = 0;
      auto rendezvous = [&]() {  // the 128 threads of this tile
        mbar_arrive(&sm.bar[BAR_EPI0 + x]);
        ok = ok && mbar_wait(&sm.bar[BAR_EPI0 + x], syncs & 1);
        ++syncs;
      };
      if (a.o.dtype == BMA_DTYPE_F32) {
        constexpr int kBoxes = HD / 64;    // boxes of [128 rows x 32 floats] the buffer holds
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
          for (int cc = 0; cc < kBoxes; ++cc) {
            uint32_t r[32];
            if (cnt > 0) {
              tmem_ld32(tmem_o + (pass * kBoxes + cc) * 32, r);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float4 v4 = make_float4(__uint_as_float(r[u * 4]) * inv, __uint_as_float(r[u * 4 + 1]) * inv,
                                            __uint_as_float(r[u * 4 + 2]) * inv, __uint_as_float(r[u * 4 + 3]) * inv);
              *reinterpret_cast<float4*>(q_row + cc * kHalfTile + ((u ^ (row & 7)) * 16)) = v4;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the TMA engine reads through the async proxy
          rendezvous();
          if (ok && row == 0) {
#pragma unroll
            for (int cc = 0; cc < kBoxes; ++cc) tma_store_4d(&map_o, sm.q[x] + cc * kHalfTile, (pass * kBoxes + cc) * 32, h, qi * BM, b);
            bulk_commit();
            bulk_wait_read0();  // the buffer is reused by the next pass / must outlive the reads
          }
          if (pass == 0) rendezvous();  // nobody overwrites the buffer before the stores have read it
        }
      } else {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          if (cnt > 0) {
            tmem_ld32(tmem_o + c * 32, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = u * 8;
            uint4 v4;
            v4.x = pack_bf16(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            v4.y = pack_bf16(__uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
            v4.z = pack_bf16(__uint_as_float(r[j + 4]) * inv, __uint_as_float(r[j + 5]) * inv);
            v4.w = pack_bf16(__uint_as_float(r[j + 6]) * inv, __uint_as_float(r[j + 7]) * inv);
            const int chunk = ((c & 1) * 4 + u) ^ (row & 7);
            *reinterpret_cast<uint4*>(q_row + (c >> 1) * kHalfTile + chunk * 16) = v4;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        rendezvous();
        if (ok && row == 0) {
#pragma unroll
          for (int box = 0; box < HD / 64; ++box) tma_store_4d(&map_o, sm.q[x] + box * kHalfTile, box * 64, h, qi * BM, b);
          bulk_commit();
          bulk_wait_read0();
        }
      }
      if (!ok) report_device_error(p.status, 230 + warp);
      if (q < a.N && a.lse)
        a.lse[((int64_t)b * a.Hq + h) * a.N + q] = (l > 0.f && !dead) ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
  }

  // ---- teardown: every thread arrives here (all waits above are bounded)
  if (T == 0 && warp == 8 && lane == 0 && !mbar_wait(&sm.bar[BAR_Q], 0))   // nobody consumed Q: let its load land before the CTA ends
    report_device_error(p.status, 130);
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemCols);
}


// =================================================================================================
// Persistent variant: one CTA per SM for the whole launch.  Work items — a PAIR of q tiles of one
// (batch, query head) — are handed out by an atomic counter, heaviest pairs of a group of heads first
// (causal: the last pair walks the most kv tiles), so that set-up, pipeline fill and epilogue of one
// item overlap the main loop of the next:
//   * barriers and tensor memory are set up once per CTA;
//   * warp 10 takes the next item from the counter and merges its kv lists into the other of two list
//     slots while the current item computes;
//   * the TMA producer's K/V ring simply continues into the next item (its first two tiles are in
//     flight before the current item has finished), and the next Q tile is fetched as soon as the
//     epilogue has let go of the Q buffer (it doubles as the staging buffer of the O store);
//   * the two q tiles of a pair still move through the kv list together (one MMA-issuing warp alternating
//     between them): letting each tile run at its own pace was measured slower — the tile that gets ahead
//     holds the two-stage K/V ring, so the loads of the next tile can no longer be issued a whole tile early.
// =================================================================================================
enum {
  PB_LIST_FULL0 = 0, PB_LIST_FULL1, PB_LIST_FREE0, PB_LIST_FREE1,
  PB_Q_FULL0, PB_Q_FULL1, PB_Q_FREE0, PB_Q_FREE1,
  PB_K_FULL0, PB_K_FULL1, PB_K_FREE0, PB_K_FREE1,
  PB_V_FULL0, PB_V_FULL1, PB_V_FREE0, PB_V_FREE1,
  PB_S0, PB_S1, PB_PART, PB_PART_LAST = PB_PART + 2 * kPParts - 1, PB_O0, PB_O1, PB_EPI0, PB_EPI1,
  PB_NUM
};
constexpr int kListConsumers = 2 + 256;  // producer, MMA warp (one lane each), every softmax thread

template <int HD>
struct __align__(1024) FwdPersistentSmem {
  uint8_t q[2][kTileBytesOf<HD>];
  uint8_t k[2][kTileBytesOf<HD>];
  uint8_t v[2][kTileBytesOf<HD>];
  uint16_t merged[2][kMaxKvTiles];  // kv tile | class for tile A << 12 | class for tile B << 14  (1 partial, 2 full)
  uint8_t cls[kMaxKvTiles];         // scratch of the list builder: class A | class B << 2
  uint64_t bar[PB_NUM];
  int4 item[2];                     // (pair, h, b, number of merged kv tiles; -1 = no more work)
  uint32_t tmem_base;
};

struct FwdPersistentParams {
  FwdParams f;
  int* counter;      // zeroed before the launch
  int n_pairs;       // ceil(NQ / 2)
  int group_heads;   // heads (b * Hq + h, flattened) per scheduling group
};

// item index -> (pair, h, b): groups of `group_heads` consecutive heads, inside a group the heaviest
// (last) pair of every head first.  Heads of a group share their K/V in L2 while they run side by side.
__device__ __forceinline__ void decode_item(const FwdPersistentParams& p, int w, int& pair, int& h, int& b) {
  const int BH = p.f.a.B * p.f.a.Hq, NP = p.n_pairs;
  const int per_group = p.group_heads * NP;
  const int full_groups = BH / p.group_heads;
  int g = w / per_group;
  int gh = p.group_heads;
  if (g >= full_groups) { g = full_groups; gh = BH - full_groups * p.group_heads; }
  const int r = w - g * per_group;
  pair = NP - 1 - r / gh;
  const int bh = g * p.group_heads + r % gh;
  h = bh % p.f.a.Hq;
  b = bh / p.f.a.Hq;
}

template <int HD, bool KB>
__global__ void __launch_bounds__(kThreads, 1)
fwd_persistent_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                      const FwdPersistentParams pp) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t kTileBytes = kTileBytesOf<HD>;
  FwdPersistentSmem<HD>& sm = *reinterpret_cast<FwdPersistentSmem<HD>*>(smem_raw);
  const FwdParams& p = pp.f;
  const bma_attn_args& a = p.a;
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int wg = warp >> 2;
  const int NQ = p.l.NQ, NKV = p.l.NKV;
  const int n_items = pp.n_pairs * a.Hq * a.B;
  const int G = a.Hq / a.Hkv;

  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0) report_device_error(p.status, 101);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < PB_NUM; ++i) {
      uint32_t count = 1;
      if (i == PB_LIST_FREE0 || i == PB_LIST_FREE1) count = kListConsumers;
      else if (i >= PB_PART && i <= PB_PART_LAST) count = 128;
      else if (i == PB_EPI0 || i == PB_EPI1) count = 128;
      mbar_init(&sm.bar[i], count);
    }
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

  if (wg == 2) {
    setmaxnreg_dec_80();
    if (warp == 10) {
      // ------------------------------------------------------------ scheduler + kv list merge (whole warp)
      bool ok = true;
      for (int it = 0; ok; ++it) {
        const int slot = it & 1;
        if (it >= 2) ok = mbar_wait_relaxed(&sm.bar[PB_LIST_FREE0 + slot], ((it >> 1) - 1) & 1);
        if (!ok) break;
        int w = 0;
        if (lane == 0) w = atomicAdd(pp.counter, 1);
        w = __shfl_sync(0xffffffffu, w, 0);
        if (w >= n_items) {
          if (lane == 0) {
            sm.item[slot] = make_int4(0, 0, 0, -1);
            mbar_arrive(&sm.bar[PB_LIST_FULL0 + slot]);
          }
          break;
        }
        int pair, h, b;
        decode_item(pp, w, pair, h, b);
        const int lb = p.l.B == 1 ? 0 : b, lh = p.l.H == 1 ? 0 : h;
        for (int i = lane * 16; i < NKV; i += 32 * 16) *reinterpret_cast<uint4*>(&sm.cls[i]) = make_uint4(0, 0, 0, 0);
        __syncwarp();
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int qi = pair * 2 + x;
          if (qi < NQ) {
            const int64_t lrow = ((int64_t)lb * p.l.H + lh) * NQ + qi;
            const int nfull = p.l.full_kv_num[lrow], npart = p.l.kv_num[lrow];
            const int32_t* full_idx = p.l.full_kv_idx + lrow * NKV;
            const int32_t* part_idx = p.l.kv_idx + lrow * NKV;
            for (int i = lane; i < nfull; i += 32) sm.cls[full_idx[i]] |= (uint8_t)(2u << (2 * x));
            for (int i = lane; i < npart; i += 32) sm.cls[part_idx[i]] |= (uint8_t)(1u << (2 * x));
          }
          __syncwarp();
        }
        int count = 0;
        for (int base = 0; base < NKV; base += 32) {
          const int j = base + lane;
          const uint32_t c = j < NKV ? sm.cls[j] : 0u;
          const unsigned m = __ballot_sync(0xffffffffu, c != 0u);
          if (c) sm.merged[slot][count + __popc(m & ((1u << lane) - 1))] = (uint16_t)((uint32_t)j | (c << 12));
          count += __popc(m);
        }
        __syncwarp();
        if (lane == 0) {
          sm.item[slot] = make_int4(pair, h, b, count);
          mbar_arrive(&sm.bar[PB_LIST_FULL0 + slot]);   // release: the list and the header are visible to whoever acquires
        }
      }
      if (!ok && lane == 0) report_device_error(p.status, 140);
    } else if (warp == 8 && lane == 0) {
      // ------------------------------------------------------------ TMA producer
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      bool ok = true;
      uint32_t g = 0;   // K/V tiles fetched so far: the ring runs on across items
      for (int it = 0; ok; ++it) {
        const int slot = it & 1;
        ok = mbar_wait(&sm.bar[PB_LIST_FULL0 + slot], (it >> 1) & 1);
        if (!ok) break;
        const int4 item = sm.item[slot];
        const int T = item.w;
        if (T < 0) break;
        const int pair = item.x, h = item.y, b = item.z, hk = h / G;
        auto load_q = [&]() {
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            if (it >= 1) ok = ok && mbar_wait(&sm.bar[PB_Q_FREE0 + x], (it - 1) & 1);   // the previous item's O store has read the buffer
            if (!ok) return;
            mbar_expect_tx(&sm.bar[PB_Q_FULL0 + x], kTileBytes);
#pragma unroll
            for (int box = 0; box < HD / 64; ++box)
              tma_load_4d(sm.q[x] + box * kHalfTile, &map_q, &sm.bar[PB_Q_FULL0 + x], box * 64, h, (pair * 2 + x) * BM, b);
          }
        };
        bool q_loaded = false;
        for (int n = 0; n < T && ok; ++n, ++g) {
          if (n == 2) { load_q(); q_loaded = true; if (!ok) break; }   // after the first two K/V tiles: those can fly while the previous item still stores
          const int st = g & 1;
          const int row0 = (int)(sm.merged[slot][n] & 0xfffu) * BN;
          if (g >= 2) ok = mbar_wait(&sm.bar[PB_K_FREE0 + st], ((g >> 1) - 1) & 1);
          if (!ok) break;
          mbar_expect_tx(&sm.bar[PB_K_FULL0 + st], kTileBytes);
#pragma unroll
          for (int box = 0; box < HD / 64; ++box) tma_load_4d(sm.k[st] + box * kHalfTile, &map_k, &sm.bar[PB_K_FULL0 + st], box * 64, hk, row0, b);
          if (g >= 2) ok = mbar_wait(&sm.bar[PB_V_FREE0 + st], ((g >> 1) - 1) & 1);
          if (!ok) break;
          mbar_expect_tx(&sm.bar[PB_V_FULL0 + st], kTileBytes);
#pragma unroll
          for (int box = 0; box < HD / 64; ++box) tma_load_4d(sm.v[st] + box * kHalfTile, &map_v, &sm.bar[PB_V_FULL0 + st], box * 64, hk, row0, b);
        }
        if (ok && !q_loaded) load_q();
        if (!ok) break;
        mbar_arrive(&sm.bar[PB_LIST_FREE0 + slot]);
      }
      if (!ok) report_device_error(p.status, 110);
    } else if (warp == 9) {
      // ------------------------------------------------------------ MMA issuer (whole warp, one elected lane issues)
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, HD, 0, 1);
      const uint64_t dq0 = make_smem_desc(smem_u32(sm.q[0]), 16, 1024), dq1 = make_smem_desc(smem_u32(sm.q[1]), 16, 1024);
      const uint64_t dk0 = make_smem_desc(smem_u32(sm.k[0]), 16, 1024);
      const uint64_t dv0 = make_smem_desc(smem_u32(sm.v[0]), kHalfTile, 1024);
      constexpr uint32_t kStageUnits = kTileBytes >> 4;
      auto issue_s = [&](int x, int st) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfTile + (ks & 3) * 32) >> 4;
          if (leader) mma_ss(tmem + x * 128, (x == 0 ? dq0 : dq1) + off, dk0 + (uint32_t)(st * kStageUnits + off), idesc_s, ks > 0);
        }
        if (leader) mma_commit(&sm.bar[PB_S0 + x]);
      };
      bool ok = true;
      uint32_t g0 = 0;                 // ring index of the item's first K/V tile
      uint32_t done0 = 0, done1 = 0;   // tiles multiplied so far per q tile, over all items (phase counters of PH / P)
      for (int it = 0; ok; ++it) {
        const int slot = it & 1;
        ok = mbar_wait(&sm.bar[PB_LIST_FULL0 + slot], (it >> 1) & 1);
        if (!ok) break;
        const int T = sm.item[slot].w;
        if (T < 0) break;
        bool have_q0 = false, have_q1 = false;
        auto need_q = [&](int x) {   // the item's Q tile has landed (asked once, before the first S of that tile)
          bool& have = x == 0 ? have_q0 : have_q1;
          if (!have) { ok = ok && mbar_wait(&sm.bar[PB_Q_FULL0 + x], it & 1); have = true; }
        };
        int cnt0 = 0, cnt1 = 0;        // tiles accumulated into O_x within this item
        if (T > 0) {
          const int st = g0 & 1;
          ok = mbar_wait(&sm.bar[PB_K_FULL0 + st], (g0 >> 1) & 1);
          const uint32_t e = sm.merged[slot][0];
          if (ok && ((e >> 12) & 3u)) { need_q(0); if (ok) { tc_fence_after(); issue_s(0, st); } }
          if (ok && ((e >> 14) & 3u)) { need_q(1); if (ok) { tc_fence_after(); issue_s(1, st); } }
          if (ok && leader) mma_commit(&sm.bar[PB_K_FREE0 + st]);
        }
        for (int n = 0; n < T && ok; ++n) {
          const uint32_t g = g0 + (uint32_t)n;
          const int st = g & 1;
          const uint32_t e = sm.merged[slot][n];
          const uint32_t e_next = (n + 1 < T) ? (uint32_t)sm.merged[slot][n + 1] : 0u;
          ok = mbar_wait(&sm.bar[PB_V_FULL0 + st], (g >> 1) & 1);
          if (ok && n + 1 < T) ok = mbar_wait(&sm.bar[PB_K_FULL0 + (st ^ 1)], ((g + 1) >> 1) & 1);
          if (!ok) break;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            if ((e >> (12 + 2 * x)) & 3u) {
              int& cnt = x == 0 ? cnt0 : cnt1;
              uint32_t& done = x == 0 ? done0 : done1;
#pragma unroll
              for (int hf = 0; hf < kPParts; ++hf) {
                ok = mbar_wait(&sm.bar[PB_PART + 2 * hf + x], done & 1);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = (hf == 0 ? 0 : 2 * kSplitChunks); ks < (hf == 0 ? 2 * kSplitChunks : 8); ++ks)
                  if (leader)
                    mma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8, dv0 + (uint32_t)(st * kStageUnits + ks * (2048 >> 4)),
                           idesc_o, (cnt > 0) || (ks > 0));
              }
              if (!ok) break;
              if (leader) mma_commit(&sm.bar[PB_O0 + x]);
              ++cnt;
              ++done;
            }
            if ((e_next >> (12 + 2 * x)) & 3u) {
              need_q(x);
              if (!ok) break;
              tc_fence_after();
              issue_s(x, st ^ 1);
            }
          }
          if (!ok) break;
          if (leader) {
            mma_commit(&sm.bar[PB_V_FREE0 + st]);
            if (n + 1 < T) mma_commit(&sm.bar[PB_K_FREE0 + (st ^ 1)]);
          }
        }
        if (!ok) break;
        g0 += (uint32_t)T;
        if (leader) mbar_arrive(&sm.bar[PB_LIST_FREE0 + slot]);
      }
      if (!ok && leader) report_device_error(p.status, 120);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc_208();
    const int x = wg;
    const int row = threadIdx.x & 127;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem + x * 128 + lane_base, tmem_o = tmem + 256 + x * 128 + lane_base;
    const int sh = 12 + 2 * x;
    bool ok = true;
    uint32_t done = 0;    // tiles of this q tile processed over all items (phase counter of S / PH / P / O)
    uint32_t syncs = 0;   // rendezvous of this tile's 128 threads so far
    for (int it = 0; ok; ++it) {
      const int slot = it & 1;
      ok = mbar_wait(&sm.bar[PB_LIST_FULL0 + slot], (it >> 1) & 1);
      if (!ok) break;
      const int4 item = sm.item[slot];
      const int T = item.w;
      if (T < 0) break;
      const int pair = item.x, h = item.y, b = item.z;
      const int qi = pair * 2 + x;
      const int q = qi * BM + row;
      const float kb2 = (KB && a.key_bias) ? __ldg(a.key_bias + h) * kLog2e : 0.f;
      float m_ref = -INFINITY;
      float l = 0.f;
      int cnt = 0;

      for (int n = 0; n < T; ++n) {
        const uint32_t e = sm.merged[slot][n];
        const uint32_t cls = (e >> sh) & 3u;
        if (cls == 0) continue;
        const int k0 = (int)(e & 0xfffu) * BN;
        ok = mbar_wait(&sm.bar[PB_S0 + x], done & 1);
        if (!ok) break;
        tc_fence_after();
        float s[BN];
        {
          uint32_t r0[32], r1[32], r2[32], r3[32];
          tmem_ld32(tmem_s + 0, r0);
          tmem_ld32(tmem_s + 32, r1);
          tmem_ld32(tmem_s + 64, r2);
          tmem_ld32(tmem_s + 96, r3);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            s[j] = __uint_as_float(r0[j]);
            s[32 + j] = __uint_as_float(r1[j]);
            s[64 + j] = __uint_as_float(r2[j]);
            s[96 + j] = __uint_as_float(r3[j]);
          }
        }
        const float sc = KB ? 1.f : p.scale_log2;
        if constexpr (KB) {
          const float base = kb2 * (float)(p.spec.k_offset + k0);
#pragma unroll
          for (int j = 0; j < BN; ++j) s[j] = fmaf(s[j], p.scale_log2, fmaf((float)j, kb2, base));
        }
        if (cls == 1) {
          uint32_t bits[4];
          {
            // the mask description is rebuilt from the kernel parameters here rather than carried in registers through the full tiles
            const MaskView mv = make_mask_view(p.spec, b, h);
            int jlo, jhi;
            row_interval(mv, q, k0, jlo, jhi);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int lo = max(jlo - c * 32, 0), hi = min(jhi - c * 32, 31);
              bits[c] = (lo <= hi) ? ((0xffffffffu >> (31 - hi)) & (0xffffffffu << lo)) : 0u;
            }
            if (mv.flags & kTableTerms) {
#pragma unroll
              for (int c = 0; c < 4; ++c)
                if (bits[c]) bits[c] &= table_bits_row32(mv, q, k0 + c * 32);
            }
          }
#pragma unroll
          for (int j = 0; j < BN; ++j) s[j] = (bits[j >> 5] >> (j & 31)) & 1u ? s[j] : -INFINITY;
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int j = 0; j < BN; j += 8) {
          mx0 = max3(mx0, s[j], s[j + 1]);
          mx1 = max3(mx1, s[j + 2], s[j + 3]);
          mx2 = max3(mx2, s[j + 4], s[j + 5]);
          mx3 = max3(mx3, s[j + 6], s[j + 7]);
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float m_cand = fmaxf(m_ref, mx * sc);
        const bool grow = (m_cand - m_ref) > kRescaleThreshold;
        float alpha = 1.f;
        if (grow) {
          alpha = ex2(m_ref - m_cand);
          m_ref = m_cand;
        }
        if (cnt > 0 && __any_sync(0xffffffffu, grow)) {
          ok = mbar_wait(&sm.bar[PB_O0 + x], (done - 1) & 1);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_o + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
            tmem_st32(tmem_o + c * 32, r);
          }
        }
        const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
        float row_sum = 0.f;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t pk[16];
          row_sum += exp_part<16>(&s[ch * 32], sc, m_sub, pk);
          tmem_st16(tmem_s + ch * 16, pk);
          if (ch == kSplitChunks - 1 || ch == 3) {   // end of a part: its stores have landed, the MMA warp may read it
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sm.bar[PB_PART + 2 * (ch == 3 ? 1 : 0) + x]);
          }
        }
        l = l * alpha + row_sum;
        ++cnt;
        ++done;
      }
      if (!ok) break;
      mbar_arrive(&sm.bar[PB_LIST_FREE0 + slot]);   // this thread has read the last list entry it needs

      // ---- epilogue of the item: O / l and the log-sum-exp.  O is staged in the tile's own Q buffer (every S MMA that
      // read it has completed once the last P V has) and leaves as TMA stores; the buffer goes back to the producer after.
      if (cnt > 0) ok = mbar_wait(&sm.bar[PB_O0 + x], (done - 1) & 1);
      else ok = mbar_wait(&sm.bar[PB_Q_FULL0 + x], it & 1);   // nobody consumed Q: let its load land before the buffer is written
      if (!ok) break;
      tc_fence_after();
      const bool dead = (m_ref == -INFINITY);
      const float inv = (l > 0.f && !dead) ? 1.f / l : 0.f;
      uint8_t* q_row = sm.q[x] + row * 128;
      auto rendezvous = [&]() {
        mbar_arrive(&sm.bar[PB_EPI0 + x]);
        ok = ok && mbar_wait(&sm.bar[PB_EPI0 + x], syncs & 1);
        ++syncs;
      };
      if (a.o.dtype == BMA_DTYPE_F32) {
        constexpr int kBoxes = HD / 64;
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
          for (int cc = 0; cc < kBoxes; ++cc) {
            uint32_t r[32];
            if (cnt > 0) {
              tmem_ld32(tmem_o + (pass * kBoxes + cc) * 32, r);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float4 v4 = make_float4(__uint_as_float(r[u * 4]) * inv, __uint_as_float(r[u * 4 + 1]) * inv,
                                            __uint_as_float(r[u * 4 + 2]) * inv, __uint_as_float(r[u * 4 + 3]) * inv);
              *reinterpret_cast<float4*>(q_row + cc * kHalfTile + ((u ^ (row & 7)) * 16)) = v4;
            }
          }
          if (pass == 1) tc_fence_before();   // the O columns are free for the next item's first P V (ordered by this tile's next P arrival)
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          rendezvous();
          if (ok && row == 0) {
            if (qi < NQ) {
#pragma unroll
              for (int cc = 0; cc < kBoxes; ++cc) tma_store_4d(&map_o, sm.q[x] + cc * kHalfTile, (pass * kBoxes + cc) * 32, h, qi * BM, b);
              bulk_commit();
              bulk_wait_read0();
            }
            if (pass == 1) mbar_arrive(&sm.bar[PB_Q_FREE0 + x]);
          }
          if (pass == 0) rendezvous();
        }
      } else {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          if (cnt > 0) {
            tmem_ld32(tmem_o + c * 32, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = u * 8;
            uint4 v4;
            v4.x = pack_bf16(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            v4.y = pack_bf16(__uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
            v4.z = pack_bf16(__uint_as_float(r[j + 4]) * inv, __uint_as_float(r[j + 5]) * inv);
            v4.w = pack_bf16(__uint_as_float(r[j + 6]) * inv, __uint_as_float(r[j + 7]) * inv);
            const int chunk = ((c & 1) * 4 + u) ^ (row & 7);
            *reinterpret_cast<uint4*>(q_row + (c >> 1) * kHalfTile + chunk * 16) = v4;
          }
        }
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        rendezvous();
        if (ok && row == 0) {
          if (qi < NQ) {
#pragma unroll
            for (int box = 0; box < HD / 64; ++box) tma_store_4d(&map_o, sm.q[x] + box * kHalfTile, box * 64, h, qi * BM, b);
            bulk_commit();
            bulk_wait_read0();
          }
          mbar_arrive(&sm.bar[PB_Q_FREE0 + x]);
        }
      }
      if (!ok) break;
      if (qi < NQ && q < a.N && a.lse)
        a.lse[((int64_t)b * a.Hq + h) * a.N + q] = (l > 0.f && !dead) ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
    if (!ok) report_device_error(p.status, 200 + warp);
  }

  // ---- teardown: every thread arrives here (all waits above are bounded)
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

// ---- host ------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tile_map_bf16(CUtensorMap* out, const void* base, int B, int L, int H, int d, int64_t stride_b,
                       int64_t stride_l, int64_t stride_h, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point"); return BMA_ERR_CUDA; }
  const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_l * 2, (cuuint64_t)stride_b * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled"); return BMA_ERR_CUDA; }
  return BMA_OK;
}

// Same for a float32 tensor: boxes of [box_rows x 32 columns] (128 bytes per row).
static int make_tile_map_f32(CUtensorMap* out, const void* base, int B, int L, int H, int d, int64_t stride_b,
                             int64_t stride_l, int64_t stride_h, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_last_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point"); return BMA_ERR_CUDA; }
  const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)stride_h * 4, (cuuint64_t)stride_l * 4, (cuuint64_t)stride_b * 4};
  const cuuint32_t box[4] = {32, 1, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled"); return BMA_ERR_CUDA; }
  return BMA_OK;
}

static bool tma_compatible(const bma_tensor& t) {
  return t.ptr && t.dtype == BMA_DTYPE_BF16 && (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 &&
         t.stride_b % 8 == 0 && t.stride_l % 8 == 0 && t.stride_h % 8 == 0 && t.stride_b > 0 && t.stride_l > 0 &&
         t.stride_h > 0;
}

// Work counters of the persistent kernels: a small pool inside the library image (nothing is allocated), handed out
// round robin and zeroed on the launch's stream before each launch.  Two launches share a counter only if more than
// kWorkCounters persistent launches are in flight at once on different streams of one device.
namespace {
constexpr int kWorkCounters = 256;
__device__ int g_work_counters[kWorkCounters];
}  // namespace
int* work_counter_slot() {
  static std::mutex mu;
  static int* base[64] = {};
  static unsigned next = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_work_counters);
    if (e != cudaSuccess) { set_last_cuda_error(e, "cudaGetSymbolAddress(work counters)"); return nullptr; }
    base[dev] = static_cast<int*>(ptr);
  }
  return base[dev] + (next++ % kWorkCounters);
}

// Which forward kernel: the persistent one wins where a row of the mask has few kv tiles (a sliding window: set-up,
// pipeline fill and the output store are a large share of such an item and overlap the next item there; measured
// +15 % on a +-256-token window at L = 8192) and loses a few per cent on long rows (its main loop is 3-4 % slower per
// tile than the one-item-per-CTA kernel's, which the saved set-up no longer outweighs at 17 tiles per item).
// BMA_FWD_PERSISTENT=0 / 1 forces one of the two (A/B measurements).
static bool fwd_persistent_enabled(const bma_mask_spec& spec) {
  const char* e = getenv("BMA_FWD_PERSISTENT");   // read per call, so that a test can switch it
  if (e && e[0]) return e[0] != '0';
  int64_t width = INT64_MAX;   // upper bound of the keys a query row can see
  if (spec.flags & BMA_MASK_BAND) width = std::min<int64_t>(width, (int64_t)spec.band_left + spec.band_right + 1);
  if (spec.flags & BMA_MASK_BLOCK_WINDOW) width = std::min<int64_t>(width, (int64_t)(spec.win_left + spec.win_right) * spec.win_block);
  return width <= 10 * BN;
}

bool sm100_supported(const bma_attn_args& a) {
  static int cc_major = -1;
  if (cc_major < 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess)
      cc_major = v;
    else { (void)cudaGetLastError(); return false; }
  }
  if (cc_major != 10) return false;
  return (a.d == 128 || a.d == 64) && tma_compatible(a.q) && tma_compatible(a.k) && tma_compatible(a.v) &&
         ceil_div(a.L, BN) <= kMaxKvTiles;
}

int sm100_fwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st) {
  BMA_REQUIRE(lists.q_block == BM && lists.kv_block == BN, BMA_ERR_ARG);
  BMA_REQUIRE(lists.NKV <= kMaxKvTiles, BMA_ERR_LIMIT);
  BMA_REQUIRE(a.o.dtype == BMA_DTYPE_F32 || a.o.dtype == BMA_DTYPE_BF16, BMA_ERR_UNSUPPORTED);
  BMA_REQUIRE((reinterpret_cast<uintptr_t>(a.o.ptr) & 15) == 0 && a.o.stride_b % 8 == 0 && a.o.stride_l % 8 == 0 &&
                  a.o.stride_h % 8 == 0,
              BMA_ERR_UNSUPPORTED);
  CUtensorMap mq, mk, mv, mo;
  int rc;
  if ((rc = make_tile_map_bf16(&mq, a.q.ptr, a.B, a.N, a.Hq, a.d, a.q.stride_b, a.q.stride_l, a.q.stride_h, BM))) return rc;
  if ((rc = make_tile_map_bf16(&mk, a.k.ptr, a.B, a.L, a.Hkv, a.d, a.k.stride_b, a.k.stride_l, a.k.stride_h, BN))) return rc;
  if ((rc = make_tile_map_bf16(&mv, a.v.ptr, a.B, a.L, a.Hkv, a.d, a.v.stride_b, a.v.stride_l, a.v.stride_h, BN))) return rc;
  if (a.o.dtype == BMA_DTYPE_F32)
    rc = make_tile_map_f32(&mo, a.o.ptr, a.B, a.N, a.Hq, a.d, a.o.stride_b, a.o.stride_l, a.o.stride_h, BM);
  else
    rc = make_tile_map_bf16(&mo, a.o.ptr, a.B, a.N, a.Hq, a.d, a.o.stride_b, a.o.stride_l, a.o.stride_h, BM);
  if (rc) return rc;
  FwdParams p;
  p.a = a; p.spec = spec; p.l = lists;
  p.scale_log2 = a.scale * kLog2e;
  p.interval_mask = (spec.flags & kTableTerms) ? 0 : 1;
  p.status = device_status_ptr();
  BMA_REQUIRE(p.status != nullptr, BMA_ERR_CUDA);
  const bool kb = a.key_bias != nullptr || a.scale < 0.f;
  if (fwd_persistent_enabled(spec)) {
    // One CTA per SM for the whole launch; items are drawn from a counter that is zeroed on the stream first.
    int dev = 0, sms = 148;
    BMA_CUDA_TRY(cudaGetDevice(&dev));
    BMA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    FwdPersistentParams pp;
    pp.f = p;
    pp.n_pairs = ceil_div(ceil_div(a.N, BM), 2);
    const int64_t n_items = (int64_t)pp.n_pairs * a.Hq * a.B;
    BMA_REQUIRE(n_items < (int64_t)INT32_MAX - sms - 1, BMA_ERR_LIMIT);
    pp.group_heads = std::max(1, std::min(a.B * a.Hq, ceil_div(2 * sms, pp.n_pairs)));
    pp.counter = work_counter_slot();
    BMA_REQUIRE(pp.counter != nullptr, BMA_ERR_CUDA);
    BMA_CUDA_TRY(cudaMemsetAsync(pp.counter, 0, sizeof(int), st));
    const dim3 pgrid((unsigned)std::min<int64_t>(n_items, sms));
    auto plaunch = [&](auto kernel, size_t smem) -> int {
      BMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      kernel<<<pgrid, kThreads, smem, st>>>(mq, mk, mv, mo, pp);
      return BMA_OK;
    };
    if (a.d == 128) rc = kb ? plaunch(fwd_persistent_kernel<128, true>, sizeof(FwdPersistentSmem<128>)) : plaunch(fwd_persistent_kernel<128, false>, sizeof(FwdPersistentSmem<128>));
    else rc = kb ? plaunch(fwd_persistent_kernel<64, true>, sizeof(FwdPersistentSmem<64>)) : plaunch(fwd_persistent_kernel<64, false>, sizeof(FwdPersistentSmem<64>));
    if (rc) return rc;
    count_launches(1);
    BMA_CUDA_TRY(cudaGetLastError());
    return BMA_OK;
  }
  dim3 grid(ceil_div(ceil_div(a.N, BM), 2), a.Hq, a.B);
  auto launch = [&](auto kernel, size_t smem) -> int {
    BMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kThreads, smem, st>>>(mq, mk, mv, mo, p);
    return BMA_OK;
  };
  if (a.d == 128) rc = kb ? launch(fwd_kernel<128, true>, sizeof(FwdSmem<128>)) : launch(fwd_kernel<128, false>, sizeof(FwdSmem<128>));
  else rc = kb ? launch(fwd_kernel<64, true>, sizeof(FwdSmem<64>)) : launch(fwd_kernel<64, false>, sizeof(FwdSmem<64>));
  if (rc) return rc;
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

}  // namespace bma
