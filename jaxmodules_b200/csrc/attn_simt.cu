// FP32 SIMT attention kernels (forward, dK/dV, dQ) driven by the block lists.
//
// These cover everything the tensor-core kernels do not: float32 inputs (whose 1e-4
// tolerance a single-pass reduced-precision MMA cannot meet), head dims other than 128,
// and they are the exact-arithmetic cross-check for the tcgen05 path.  All arithmetic is
// FP32 FMA; inputs may be float32 or bfloat16 and are widened when a tile is staged.
//
// Semantics follow jaxmodules/attention.py:52-105 (scores exp(q.k/sqrt(d)) times mask, rows
// without an allowed key give 0) with a max-subtracted online softmax, which is the same
// function.  Empty blocks are never visited, full blocks skip the element predicate.
//
// Tile: 64 queries x 64 keys per CTA of 256 threads; thread (ty, tx) = (tid/16, tid%16) owns
// score rows 4*ty..4*ty+3, score columns 4*tx..4*tx+3, and output columns tx + 16*c.
#include <algorithm>

#include "common.cuh"

namespace bma {
namespace {

constexpr int TQ = kSimtTile, TK = kSimtTile;
constexpr int NT = 256;
constexpr int PS = TK + 4;  // padded row stride of the transposed / probability tiles

struct SimtParams {
  bma_attn_args a;
  bma_mask_spec spec;
  bma_block_lists l;
  float scale_log2;  // scale * log2(e)
};

template <typename T>
__device__ __forceinline__ const T* row_ptr(const bma_tensor& t, int b, int l, int h) {
  return static_cast<const T*>(t.ptr) + (int64_t)b * t.stride_b + (int64_t)l * t.stride_l + (int64_t)h * t.stride_h;
}
template <typename T>
__device__ __forceinline__ T* row_ptr_mut(const bma_tensor& t, int b, int l, int h) {
  return static_cast<T*>(t.ptr) + (int64_t)b * t.stride_b + (int64_t)l * t.stride_l + (int64_t)h * t.stride_h;
}

// Stage a [rows x d] tile (row-major, zero padded to DP columns / TQ rows) into shared memory.
template <typename T, int DP>
__device__ __forceinline__ void stage_natural(float* dst, const bma_tensor& t, int b, int l0, int h, int lmax, int d) {
  for (int idx = threadIdx.x; idx < TQ * DP; idx += NT) {
    const int r = idx / DP, c = idx % DP;
    float v = 0.f;
    if (l0 + r < lmax && c < d) v = to_float(row_ptr<T>(t, b, l0 + r, h)[c]);
    dst[r * DP + c] = v;
  }
}
// Stage a tile transposed: dst[c][r], row stride PS.
template <typename T, int DP>
__device__ __forceinline__ void stage_transposed(float* dst, const bma_tensor& t, int b, int l0, int h, int lmax, int d) {
  for (int idx = threadIdx.x; idx < TK * DP; idx += NT) {
    const int r = idx / DP, c = idx % DP;
    float v = 0.f;
    if (l0 + r < lmax && c < d) v = to_float(row_ptr<T>(t, b, l0 + r, h)[c]);
    dst[c * PS + r] = v;
  }
}

// acc[i][j] += sum_c A[4*ty+i][c] * Bt[c][4*tx+j]   (A natural with stride DP, Bt transposed with stride PS)
template <int DP>
__device__ __forceinline__ void tile_dot(const float* A, const float* Bt, int ty, int tx, float acc[4][4]) {
#pragma unroll 4
  for (int c = 0; c < DP; c += 4) {
    float4 a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(A + (ty * 4 + i) * DP + c);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 bv = *reinterpret_cast<const float4*>(Bt + (c + e) * PS + tx * 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float av = e == 0 ? a[i].x : e == 1 ? a[i].y : e == 2 ? a[i].z : a[i].w;
        acc[i][0] = fmaf(av, bv.x, acc[i][0]);
        acc[i][1] = fmaf(av, bv.y, acc[i][1]);
        acc[i][2] = fmaf(av, bv.z, acc[i][2]);
        acc[i][3] = fmaf(av, bv.w, acc[i][3]);
      }
    }
  }
}

__device__ __forceinline__ float group16_max(float v) {
  for (int o = 8; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float group16_sum(float v) {
  for (int o = 8; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct ListRow {
  const int32_t* full_idx; const int32_t* part_idx;
  int nfull, npart;
};
// kv-side lists of q-tile `qi` (TRANSPOSED = false) or q-side lists of kv-tile `kj` (true)
template <bool QSIDE>
__device__ __forceinline__ ListRow list_row(const bma_block_lists& l, int b, int h, int r) {
  const int lb = l.B == 1 ? 0 : b, lh = l.H == 1 ? 0 : h;
  const int NR = QSIDE ? l.NKV : l.NQ, NC = QSIDE ? l.NQ : l.NKV;
  const int64_t row = ((int64_t)lb * l.H + lh) * NR + r;
  ListRow o;
  o.nfull = (QSIDE ? l.full_q_num : l.full_kv_num)[row];
  o.npart = (QSIDE ? l.q_num : l.kv_num)[row];
  o.full_idx = (QSIDE ? l.full_q_idx : l.full_kv_idx) + row * NC;
  o.part_idx = (QSIDE ? l.q_idx : l.kv_idx) + row * NC;
  return o;
}

// ---------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------
template <typename T, int DC>
__global__ void __launch_bounds__(NT) simt_fwd_kernel(const SimtParams p) {
  constexpr int DP = 16 * DC;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                  // [TQ][DP]
  float* Kt = Qs + TQ * DP;        // [DP][PS]
  float* Vs = Kt + DP * PS;        // [TK][DP]
  float* Ps = Vs + TK * DP;        // [TQ][PS]

  const bma_attn_args& a = p.a;
  const int qi = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int q0 = qi * TQ;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const MaskView mv = make_mask_view(p.spec, b, h);
  const float kb2 = p.a.key_bias ? __ldg(p.a.key_bias + h) * kLog2e : 0.f;  // per-head key bias in log2 units
  const ListRow lr = list_row<false>(p.l, b, h, qi);

  stage_natural<T, DP>(Qs, a.q, b, q0, h, a.N, a.d);

  float m[4], lsum[4], o[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY; lsum[i] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) o[i][c] = 0.f;
  }

  const int ntiles = lr.nfull + lr.npart;
  for (int it = 0; it < ntiles; ++it) {
    const bool partial = it >= lr.nfull;
    const int kj = partial ? lr.part_idx[it - lr.nfull] : lr.full_idx[it];
    const int k0 = kj * TK;
    __syncthreads();  // previous tile fully consumed (also orders the Q staging on the first trip)
    stage_transposed<T, DP>(Kt, a.k, b, k0, hk, a.L, a.d);
    stage_natural<T, DP>(Vs, a.v, b, k0, hk, a.L, a.d);
    __syncthreads();

    float s[4][4] = {};
    tile_dot<DP>(Qs, Kt, ty, tx, s);
    float mx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      mx[i] = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = fmaf(s[i][j], p.scale_log2, kb2 * (float)(mv.k_offset + k0 + tx * 4 + j));
        if (partial && !mask_allowed(mv, q0 + ty * 4 + i, k0 + tx * 4 + j)) v = -INFINITY;
        s[i][j] = v;
        mx[i] = fmaxf(mx[i], v);
      }
      mx[i] = group16_max(mx[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float m_new = fmaxf(m[i], mx[i]);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m[i] - m_safe);
      float rs = 0.f;
      float4 pv;
      float* pvp = &pv.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[i][j] - m_safe);
        pvp[j] = e;
        rs += e;
      }
      rs = group16_sum(rs);
      lsum[i] = lsum[i] * alpha + rs;
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < DC; ++c) o[i][c] *= alpha;
      *reinterpret_cast<float4*>(Ps + (ty * 4 + i) * PS + tx * 4) = pv;
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < TK; ++kk) {
      float pr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pr[i] = Ps[(ty * 4 + i) * PS + kk];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const float vv = Vs[kk * DP + c * 16 + tx];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i][c] = fmaf(pr[i], vv, o[i][c]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int q = q0 + ty * 4 + i;
    if (q >= a.N) continue;
    const float inv = lsum[i] > 0.f ? 1.f / lsum[i] : 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int col = c * 16 + tx;
      if (col < a.d) {
        const float val = o[i][c] * inv;
        if (a.o.dtype == BMA_DTYPE_F32) row_ptr_mut<float>(a.o, b, q, h)[col] = val;
        else row_ptr_mut<__nv_bfloat16>(a.o, b, q, h)[col] = __float2bfloat16_rn(val);
      }
    }
    if (tx == 0 && a.lse)
      a.lse[((int64_t)b * a.Hq + h) * a.N + q] = lsum[i] > 0.f ? (m[i] + log2f(lsum[i])) * kLn2 : -INFINITY;
  }
}

// Shared by both backward kernels: p and ds of one 64x64 tile into registers.
// s[i][j] holds q.k on entry and p on exit; dp[i][j] holds dO.v on entry and ds on exit.
__device__ __forceinline__ void softmax_grad_tile(float s[4][4], float dp[4][4], const float* lse2, const float* delta,
                                                  int ty, int tx, bool partial, const MaskView& mv, int q0, int k0,
                                                  float scale_log2, float kb2) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float l2 = lse2[ty * 4 + i], dl = delta[ty * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      bool ok = l2 != -INFINITY;
      if (partial) ok = ok && mask_allowed(mv, q0 + ty * 4 + i, k0 + tx * 4 + j);
      const float pr = ok ? exp2f(fmaf(s[i][j], scale_log2, kb2 * (float)(mv.k_offset + k0 + tx * 4 + j)) - l2) : 0.f;
      s[i][j] = pr;
      dp[i][j] = pr * (dp[i][j] - dl);
    }
  }
}

template <typename TD>
__device__ __forceinline__ void stage_rowstats(float* lse2, float* delta, const bma_attn_args& a, int b, int h, int q0) {
  for (int r = threadIdx.x; r < TQ; r += NT) {
    const int q = q0 + r;
    float l = -INFINITY, dl = 0.f;
    if (q < a.N) {
      l = a.lse[((int64_t)b * a.Hq + h) * a.N + q];
      dl = a.delta[((int64_t)b * a.Hq + h) * a.N + q];
    }
    lse2[r] = l * kLog2e;  // -inf stays -inf
    delta[r] = dl;
  }
}

// ---------------------------------------------------------------------------------------
// dK / dV: one CTA per (kv tile, kv head, batch); loops the query heads of the group and the
// q tiles of the q-side lists.  No atomics, fixed summation order.
// ---------------------------------------------------------------------------------------
template <typename T, typename TDO, int DC>
__global__ void __launch_bounds__(NT) simt_bwd_dkdv_kernel(const SimtParams p) {
  constexpr int DP = 16 * DC;
  extern __shared__ __align__(16) float sm[];
  float* Kt = sm;                   // [DP][PS]
  float* Vt = Kt + DP * PS;         // [DP][PS]
  float* Qs = Vt + DP * PS;         // [TQ][DP]
  float* dOs = Qs + TQ * DP;        // [TQ][DP]
  float* Ps = dOs + TQ * DP;        // [TQ][PS]
  float* dSs = Ps + TQ * PS;        // [TQ][PS]
  float* lse2 = dSs + TQ * PS;      // [TQ]
  float* dlt = lse2 + TQ;           // [TQ]

  const bma_attn_args& a = p.a;
  const int kj = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int k0 = kj * TK;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;

  stage_transposed<T, DP>(Kt, a.k, b, k0, hk, a.L, a.d);
  stage_transposed<T, DP>(Vt, a.v, b, k0, hk, a.L, a.d);

  float dk[4][DC], dv[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DC; ++c) { dk[i][c] = 0.f; dv[i][c] = 0.f; }

  for (int g = 0; g < G; ++g) {
    const int h = hk * G + g;
    const MaskView mv = make_mask_view(p.spec, b, h);
    const float kb2 = p.a.key_bias ? __ldg(p.a.key_bias + h) * kLog2e : 0.f;  // per-head key bias in log2 units
    const ListRow lr = list_row<true>(p.l, b, h, kj);
    const int ntiles = lr.nfull + lr.npart;
    for (int it = 0; it < ntiles; ++it) {
      const bool partial = it >= lr.nfull;
      const int qi = partial ? lr.part_idx[it - lr.nfull] : lr.full_idx[it];
      const int q0 = qi * TQ;
      __syncthreads();
      stage_natural<T, DP>(Qs, a.q, b, q0, h, a.N, a.d);
      stage_natural<TDO, DP>(dOs, a.d_o, b, q0, h, a.N, a.d);
      stage_rowstats<T>(lse2, dlt, a, b, h, q0);
      __syncthreads();
      float s[4][4] = {}, dp[4][4] = {};
      tile_dot<DP>(Qs, Kt, ty, tx, s);
      tile_dot<DP>(dOs, Vt, ty, tx, dp);
      softmax_grad_tile(s, dp, lse2, dlt, ty, tx, partial, mv, q0, k0, p.scale_log2, kb2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        *reinterpret_cast<float4*>(Ps + (ty * 4 + i) * PS + tx * 4) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
        *reinterpret_cast<float4*>(dSs + (ty * 4 + i) * PS + tx * 4) = make_float4(dp[i][0], dp[i][1], dp[i][2], dp[i][3]);
      }
      __syncthreads();
      // dV[k][c] += sum_q P[q][k] dO[q][c];  dK[k][c] += sum_q dS[q][k] Q[q][c]   (k = 4*ty+i)
#pragma unroll 2
      for (int q = 0; q < TQ; ++q) {
        const float4 pk = *reinterpret_cast<const float4*>(Ps + q * PS + ty * 4);
        const float4 dsk = *reinterpret_cast<const float4*>(dSs + q * PS + ty * 4);
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const float dov = dOs[q * DP + c * 16 + tx];
          const float qv = Qs[q * DP + c * 16 + tx];
          dv[0][c] = fmaf(pk.x, dov, dv[0][c]); dv[1][c] = fmaf(pk.y, dov, dv[1][c]);
          dv[2][c] = fmaf(pk.z, dov, dv[2][c]); dv[3][c] = fmaf(pk.w, dov, dv[3][c]);
          dk[0][c] = fmaf(dsk.x, qv, dk[0][c]); dk[1][c] = fmaf(dsk.y, qv, dk[1][c]);
          dk[2][c] = fmaf(dsk.z, qv, dk[2][c]); dk[3][c] = fmaf(dsk.w, qv, dk[3][c]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int k = k0 + ty * 4 + i;
    if (k >= a.L) continue;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int col = c * 16 + tx;
      if (col < a.d) {
        row_ptr_mut<T>(a.dk, b, k, hk)[col] = from_float<T>(dk[i][c] * a.scale);
        row_ptr_mut<T>(a.dv, b, k, hk)[col] = from_float<T>(dv[i][c]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// dQ: one CTA per (q tile, query head, batch); loops the kv tiles of the kv-side lists.
// ---------------------------------------------------------------------------------------
template <typename T, typename TDO, int DC>
__global__ void __launch_bounds__(NT) simt_bwd_dq_kernel(const SimtParams p) {
  constexpr int DP = 16 * DC;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                   // [TQ][DP]
  float* dOs = Qs + TQ * DP;        // [TQ][DP]
  float* Kt = dOs + TQ * DP;        // [DP][PS]
  float* Vt = Kt + DP * PS;         // [DP][PS]
  float* Ks = Vt + DP * PS;         // [TK][DP]
  float* dSs = Ks + TK * DP;        // [TQ][PS]
  float* lse2 = dSs + TQ * PS;
  float* dlt = lse2 + TQ;

  const bma_attn_args& a = p.a;
  const int qi = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int q0 = qi * TQ;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const MaskView mv = make_mask_view(p.spec, b, h);
  const float kb2 = p.a.key_bias ? __ldg(p.a.key_bias + h) * kLog2e : 0.f;  // per-head key bias in log2 units
  const ListRow lr = list_row<false>(p.l, b, h, qi);

  stage_natural<T, DP>(Qs, a.q, b, q0, h, a.N, a.d);
  stage_natural<TDO, DP>(dOs, a.d_o, b, q0, h, a.N, a.d);
  stage_rowstats<T>(lse2, dlt, a, b, h, q0);

  float dq[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DC; ++c) dq[i][c] = 0.f;

  const int ntiles = lr.nfull + lr.npart;
  for (int it = 0; it < ntiles; ++it) {
    const bool partial = it >= lr.nfull;
    const int kj = partial ? lr.part_idx[it - lr.nfull] : lr.full_idx[it];
    const int k0 = kj * TK;
    __syncthreads();
    stage_transposed<T, DP>(Kt, a.k, b, k0, hk, a.L, a.d);
    stage_transposed<T, DP>(Vt, a.v, b, k0, hk, a.L, a.d);
    stage_natural<T, DP>(Ks, a.k, b, k0, hk, a.L, a.d);
    __syncthreads();
    float s[4][4] = {}, dp[4][4] = {};
    tile_dot<DP>(Qs, Kt, ty, tx, s);
    tile_dot<DP>(dOs, Vt, ty, tx, dp);
    softmax_grad_tile(s, dp, lse2, dlt, ty, tx, partial, mv, q0, k0, p.scale_log2, kb2);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<float4*>(dSs + (ty * 4 + i) * PS + tx * 4) = make_float4(dp[i][0], dp[i][1], dp[i][2], dp[i][3]);
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < TK; ++kk) {
      float dsr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dsr[i] = dSs[(ty * 4 + i) * PS + kk];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const float kv = Ks[kk * DP + c * 16 + tx];
#pragma unroll
        for (int i = 0; i < 4; ++i) dq[i][c] = fmaf(dsr[i], kv, dq[i][c]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int q = q0 + ty * 4 + i;
    if (q >= a.N) continue;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int col = c * 16 + tx;
      if (col < a.d) row_ptr_mut<T>(a.dq, b, q, h)[col] = from_float<T>(dq[i][c] * a.scale);
    }
  }
}

template <int DC> constexpr size_t fwd_smem() { return sizeof(float) * (TQ * 16 * DC + 16 * DC * PS + TK * 16 * DC + TQ * PS); }
template <int DC> constexpr size_t dkdv_smem() { return sizeof(float) * (2 * 16 * DC * PS + 2 * TQ * 16 * DC + 2 * TQ * PS + 2 * TQ); }
template <int DC> constexpr size_t dq_smem() { return sizeof(float) * (2 * TQ * 16 * DC + 2 * 16 * DC * PS + TK * 16 * DC + TQ * PS + 2 * TQ); }

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) BMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return BMA_OK;
}

template <typename T, int DC>
int launch_fwd(const SimtParams& p, cudaStream_t st) {
  int rc = set_smem(simt_fwd_kernel<T, DC>, fwd_smem<DC>());
  if (rc) return rc;
  dim3 grid(ceil_div(p.a.N, TQ), p.a.Hq, p.a.B);
  simt_fwd_kernel<T, DC><<<grid, NT, fwd_smem<DC>(), st>>>(p);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

template <typename T, typename TDO, int DC>
int launch_bwd(const SimtParams& p, cudaStream_t st) {
  int rc = set_smem(simt_bwd_dkdv_kernel<T, TDO, DC>, dkdv_smem<DC>());
  if (rc) return rc;
  rc = set_smem(simt_bwd_dq_kernel<T, TDO, DC>, dq_smem<DC>());
  if (rc) return rc;
  dim3 gkv(ceil_div(p.a.L, TK), p.a.Hkv, p.a.B);
  simt_bwd_dkdv_kernel<T, TDO, DC><<<gkv, NT, dkdv_smem<DC>(), st>>>(p);
  dim3 gq(ceil_div(p.a.N, TQ), p.a.Hq, p.a.B);
  simt_bwd_dq_kernel<T, TDO, DC><<<gq, NT, dq_smem<DC>(), st>>>(p);
  count_launches(2);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

template <typename T>
int dispatch_fwd(const SimtParams& p, cudaStream_t st) {
  const int d = p.a.d;
  if (d <= 16) return launch_fwd<T, 1>(p, st);
  if (d <= 32) return launch_fwd<T, 2>(p, st);
  if (d <= 64) return launch_fwd<T, 4>(p, st);
  if (d <= 128) return launch_fwd<T, 8>(p, st);
  return BMA_ERR_UNSUPPORTED;
}
template <typename T, typename TDO>
int dispatch_bwd(const SimtParams& p, cudaStream_t st) {
  const int d = p.a.d;
  if (d <= 16) return launch_bwd<T, TDO, 1>(p, st);
  if (d <= 32) return launch_bwd<T, TDO, 2>(p, st);
  if (d <= 64) return launch_bwd<T, TDO, 4>(p, st);
  if (d <= 128) return launch_bwd<T, TDO, 8>(p, st);
  return BMA_ERR_UNSUPPORTED;
}

SimtParams make_params(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& l) {
  SimtParams p;
  p.a = a; p.spec = spec; p.l = l;
  p.scale_log2 = a.scale * kLog2e;
  return p;
}

}  // namespace

int simt_fwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st) {
  BMA_REQUIRE(lists.q_block == TQ && lists.kv_block == TK, BMA_ERR_ARG);
  const SimtParams p = make_params(a, spec, lists);
  if (a.q.dtype == BMA_DTYPE_F32) return dispatch_fwd<float>(p, st);
  return dispatch_fwd<__nv_bfloat16>(p, st);
}

int simt_bwd(const bma_attn_args& a, const bma_mask_spec& spec, const bma_block_lists& lists, cudaStream_t st) {
  BMA_REQUIRE(lists.q_block == TQ && lists.kv_block == TK && lists.q_num, BMA_ERR_ARG);
  const SimtParams p = make_params(a, spec, lists);
  const bool f32 = a.q.dtype == BMA_DTYPE_F32, do_f32 = a.d_o.dtype == BMA_DTYPE_F32;
  if (f32 && do_f32) return dispatch_bwd<float, float>(p, st);
  if (f32) return dispatch_bwd<float, __nv_bfloat16>(p, st);
  if (do_f32) return dispatch_bwd<__nv_bfloat16, float>(p, st);
  return dispatch_bwd<__nv_bfloat16, __nv_bfloat16>(p, st);
}

}  // namespace bma
