// Flash-style forward for bf16, head dim 128, on the sm_100a tensor core (tcgen05) with TMEM
// accumulators and TMA-staged operands.
//
// One CTA = one 128-query tile of one (batch, query head); two CTAs are resident per SM so that
// one CTA's softmax overlaps the other's MMAs.  The CTA walks only the kv tiles named in the block
// lists (full tiles first, then partial ones); the element predicate is evaluated only on partial
// tiles.
//
//   warp 4 (one elected lane)  TMA loads of Q / K / V tiles (128-byte swizzle, K-major boxes of
//                              [128 rows x 64 columns]) and tcgen05.mma issue:
//                                S = Q K^T          (A, B from shared memory, 128x128x128)
//                                O (+)= P V         (A = P from tensor memory, B = V MN-major)
//   warps 0-3 (thread = row)   read S from TMEM, online softmax in FP32 (exp2 with the scale folded
//                              in, running max with lazy rescale of O), write P as bf16 back into
//                              the S columns, final O / l and log-sum-exp.
//
// TMEM columns (256 per CTA): [0,128) S fp32, reused as P bf16 in [0,64); [128,256) O fp32.
// Every mbarrier wait is bounded; on a timeout the CTA records an error code and unwinds.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace bma {
namespace {

using namespace ptx;

constexpr int BM = kSm100Tile, BN = kSm100Tile, HD = 128;
constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = kSoftmaxThreads + 32;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kHalfTile = BM * 64 * 2;     // one [128 x 64] bf16 box
constexpr uint32_t kTileBytes = 2 * kHalfTile;  // a [128 x 128] operand tile
constexpr float kRescaleThreshold = 8.0f;       // log2 units: rescale O only when the max grew by > 2^8

enum { BAR_Q = 0, BAR_K, BAR_V, BAR_S, BAR_P, BAR_O, NUM_BARS };

struct __align__(1024) FwdSmem {
  uint8_t q[kTileBytes];
  uint8_t k[kTileBytes];
  uint8_t v[kTileBytes];
  uint64_t bar[NUM_BARS];
  uint32_t tmem_base;
  int abort;
};

struct FwdParams {
  bma_attn_args a;
  bma_mask_spec spec;
  bma_block_lists l;
  float scale_log2;
  int interval_mask;  // 1: the mask has only interval terms (no segment ids / bit table)
  int* status;
};

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
  // to tile-local key indices
  jlo = lo - m.k_offset - k0;
  jhi = min(hi - m.k_offset, m.k_valid - 1) - k0;
}

// Compiled for 256 threads x 2 CTAs per SM (128 registers); launched with kThreads.
__global__ void __launch_bounds__(256, 2)
fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const bma_attn_args& a = p.a;
  const int qi = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int q0 = qi * BM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // block lists of this q tile
  const int lb = p.l.B == 1 ? 0 : b, lh = p.l.H == 1 ? 0 : h;
  const int64_t lrow = ((int64_t)lb * p.l.H + lh) * p.l.NQ + qi;
  const int nfull = p.l.full_kv_num[lrow], npart = p.l.kv_num[lrow];
  const int32_t* full_idx = p.l.full_kv_idx + lrow * p.l.NKV;
  const int32_t* part_idx = p.l.kv_idx + lrow * p.l.NKV;
  const int ntiles = nfull + npart;

  if (threadIdx.x == 0) {
    mbar_init(&sm.bar[BAR_Q], 1);
    mbar_init(&sm.bar[BAR_K], 1);
    mbar_init(&sm.bar[BAR_V], 1);
    mbar_init(&sm.bar[BAR_S], 1);
    mbar_init(&sm.bar[BAR_P], kSoftmaxThreads);
    mbar_init(&sm.bar[BAR_O], 1);
    sm.abort = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tmem_s = tmem, tmem_p = tmem, tmem_o = tmem + 128;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer / MMA issuer
    if (lane == 0 && ntiles > 0) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, HD, 0, 1);
      const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v);
      bool ok = true;

      auto load_tile = [&](const CUtensorMap* m, uint8_t* dst, uint64_t* bar, int head, int row0) {
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(dst, m, bar, 0, head, row0, b);
        tma_load_4d(dst + kHalfTile, m, bar, 64, head, row0, b);
      };
      auto tile_of = [&](int it) { return it < nfull ? full_idx[it] : part_idx[it - nfull]; };

      load_tile(&map_q, sm.q, &sm.bar[BAR_Q], h, q0);
      load_tile(&map_k, sm.k, &sm.bar[BAR_K], hk, tile_of(0) * BN);
      load_tile(&map_v, sm.v, &sm.bar[BAR_V], hk, tile_of(0) * BN);
      ok = mbar_wait(&sm.bar[BAR_Q], 0);

      for (int it = 0; it < ntiles && ok; ++it) {
        const uint32_t ph = it & 1;
        // ---- S = Q K^T
        ok = ok && mbar_wait(&sm.bar[BAR_K], ph);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfTile + (ks & 3) * 32;  // 64-column box, then 32 B per k-step
          mma_ss(tmem_s, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024), idesc_s, ks > 0);
        }
        mma_commit(&sm.bar[BAR_S]);
        // K buffer is free once S is done: prefetch the next K tile
        ok = mbar_wait(&sm.bar[BAR_S], ph);
        if (!ok) break;
        if (it + 1 < ntiles) load_tile(&map_k, sm.k, &sm.bar[BAR_K], hk, tile_of(it + 1) * BN);
        // ---- O (+)= P V
        ok = mbar_wait(&sm.bar[BAR_P], ph) && mbar_wait(&sm.bar[BAR_V], ph);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          // B = V[kv rows][d]: MN-major; 16 kv rows per k-step = 2048 B; the two 64-column boxes are kHalfTile apart
          mma_ts(tmem_o, tmem_p + ks * 8, make_smem_desc(v_addr + ks * 2048, kHalfTile, 1024), idesc_o, (it > 0) || (ks > 0));
        }
        mma_commit(&sm.bar[BAR_O]);
        ok = mbar_wait(&sm.bar[BAR_O], ph);
        if (!ok) break;
        if (it + 1 < ntiles) load_tile(&map_v, sm.v, &sm.bar[BAR_V], hk, tile_of(it + 1) * BN);
      }
      if (!ok) {
        report_device_error(p.status, 100 + BAR_S);
        atomicExch(&sm.abort, 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int row = threadIdx.x;  // TMEM lane == query row of the tile
    const int q = q0 + row;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const MaskView mv = make_mask_view(p.spec, b, h);
    float m_ref = -INFINITY;  // reference max (log2 domain) the exponentials are taken against
    float l = 0.f;
    bool ok = true;

    for (int it = 0; it < ntiles; ++it) {
      const uint32_t ph = it & 1;
      const bool partial = it >= nfull;
      const int k0 = (partial ? part_idx[it - nfull] : full_idx[it]) * BN;
      ok = mbar_wait(&sm.bar[BAR_S], ph);
      if (!ok) break;
      tc_fence_after();
      // allowed-key bits of this row for the four 32-column chunks (all ones on full tiles)
      uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (partial) {
        if (p.interval_mask) {
          int jlo, jhi;
          row_interval(mv, q, k0, jlo, jhi);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int lo = max(jlo - c * 32, 0), hi = min(jhi - c * 32, 31);  // chunk-local inclusive range
            bits[c] = (lo <= hi) ? ((0xffffffffu >> (31 - hi)) & (0xffffffffu << lo)) : 0u;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) w |= (mask_allowed(mv, q, k0 + c * 32 + j) ? 1u : 0u) << j;
            bits[c] = w;
          }
        }
      }
      // pass 1: row maximum of the allowed scores
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_s + lane_base + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float v = (bits[c] >> j) & 1u ? __uint_as_float(r[j]) : -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      const float m_cand = fmaxf(m_ref, mx * p.scale_log2);
      // lazy rescale: keep the old reference unless the maximum grew by more than 2^threshold
      const bool grow = (m_cand - m_ref) > kRescaleThreshold;  // also true when m_ref == -inf and m_cand is finite
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m_ref - m_cand);  // 0 when m_ref == -inf
        m_ref = m_cand;
      }
      if (it > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_o + lane_base + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
          tmem_st32(tmem_o + lane_base + c * 32, r);
        }
      }
      // keep the compiler from carrying 128 per-element predicates from pass 1 into pass 2
#pragma unroll
      for (int c = 0; c < 4; ++c) asm volatile("" : "+r"(bits[c]));
      // pass 2: exponentials, row sum, P as bf16 into the S columns already consumed
      const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_s + lane_base + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float e0 = ex2(fmaf(__uint_as_float(r[2 * j]), p.scale_log2, -m_sub));
          float e1 = ex2(fmaf(__uint_as_float(r[2 * j + 1]), p.scale_log2, -m_sub));
          e0 = (bits[c] >> (2 * j)) & 1u ? e0 : 0.f;
          e1 = (bits[c] >> (2 * j + 1)) & 1u ? e1 : 0.f;
          rs += e0 + e1;
          pk[j] = pack_bf16(e0, e1);
        }
        tmem_st16(tmem_p + lane_base + c * 16, pk);
      }
      l = l * alpha + rs;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.bar[BAR_P]);
    }

    // ---- epilogue: O / l and the log-sum-exp
    if (ok && ntiles > 0) ok = mbar_wait(&sm.bar[BAR_O], (ntiles - 1) & 1);
    if (!ok) {
      report_device_error(p.status, 200 + warp);
    } else {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool store = q < a.N;
      float* of = nullptr;
      __nv_bfloat16* ob = nullptr;
      if (a.o.dtype == BMA_DTYPE_F32)
        of = static_cast<float*>(a.o.ptr) + (int64_t)b * a.o.stride_b + (int64_t)q * a.o.stride_l + (int64_t)h * a.o.stride_h;
      else
        ob = static_cast<__nv_bfloat16*>(a.o.ptr) + (int64_t)b * a.o.stride_b + (int64_t)q * a.o.stride_l + (int64_t)h * a.o.stride_h;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (ntiles > 0) {
          tmem_ld32(tmem_o + lane_base + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (store) {
          if (of) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v4 = make_float4(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv,
                                      __uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
              *reinterpret_cast<float4*>(of + c * 32 + j) = v4;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v4;
              v4.x = pack_bf16(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
              v4.y = pack_bf16(__uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
              v4.z = pack_bf16(__uint_as_float(r[j + 4]) * inv, __uint_as_float(r[j + 5]) * inv);
              v4.w = pack_bf16(__uint_as_float(r[j + 6]) * inv, __uint_as_float(r[j + 7]) * inv);
              *reinterpret_cast<uint4*>(ob + c * 32 + j) = v4;
            }
          }
        }
      }
      if (store && a.lse)
        a.lse[((int64_t)b * a.Hq + h) * a.N + q] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
  }

  // ---- teardown: every thread arrives here (all waits above are bounded)
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, kTmemCols);
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

static bool tma_compatible(const bma_tensor& t) {
  return t.ptr && t.dtype == BMA_DTYPE_BF16 && (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 &&
         t.stride_b % 8 == 0 && t.stride_l % 8 == 0 && t.stride_h % 8 == 0 && t.stride_b > 0 && t.stride_l > 0 &&
         t.stride_h > 0;
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
  return a.d == HD && tma_compatible(a.q) && tma_compatible(a.k) && tma_compatible(a.v);
}

int sm100_fwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st) {
  BMA_REQUIRE(lists.q_block == BM && lists.kv_block == BN, BMA_ERR_ARG);
  BMA_REQUIRE(a.o.dtype == BMA_DTYPE_F32 || a.o.dtype == BMA_DTYPE_BF16, BMA_ERR_UNSUPPORTED);
  BMA_REQUIRE((reinterpret_cast<uintptr_t>(a.o.ptr) & 15) == 0 && a.o.stride_b % 8 == 0 && a.o.stride_l % 8 == 0 &&
                  a.o.stride_h % 8 == 0,
              BMA_ERR_UNSUPPORTED);
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_tile_map_bf16(&mq, a.q.ptr, a.B, a.N, a.Hq, a.d, a.q.stride_b, a.q.stride_l, a.q.stride_h, BM))) return rc;
  if ((rc = make_tile_map_bf16(&mk, a.k.ptr, a.B, a.L, a.Hkv, a.d, a.k.stride_b, a.k.stride_l, a.k.stride_h, BN))) return rc;
  if ((rc = make_tile_map_bf16(&mv, a.v.ptr, a.B, a.L, a.Hkv, a.d, a.v.stride_b, a.v.stride_l, a.v.stride_h, BN))) return rc;
  FwdParams p;
  p.a = a; p.spec = spec; p.l = lists;
  p.scale_log2 = a.scale * kLog2e;
  p.interval_mask = (spec.flags & (BMA_MASK_SEGMENT | BMA_MASK_BITMAP)) ? 0 : 1;
  p.status = device_status_ptr();
  BMA_REQUIRE(p.status != nullptr, BMA_ERR_CUDA);
  const size_t smem = sizeof(FwdSmem) + 1024;
  BMA_CUDA_TRY(cudaFuncSetAttribute(fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(ceil_div(a.N, BM), a.Hq, a.B);
  fwd_kernel<<<grid, kThreads, smem, st>>>(mq, mk, mv, p);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

}  // namespace bma
