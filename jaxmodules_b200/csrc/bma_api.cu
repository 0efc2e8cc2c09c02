// extern "C" entry points of libbma.so: argument validation, backend choice, and the two
// small HBM-bound kernels (backward preprocess, partial-result merge).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace bma {

// implemented in mask_compile.cu
size_t mask_compile_workspace_bytes(const bma_mask_spec& spec, int B, int H, int NQ, int NKV);
int mask_compile_validate(const bma_mask_spec& s, int B, int H, const bma_block_lists& l);
int mask_compile_launch(const bma_mask_spec& spec, int B, int H, const bma_block_lists& l, void* workspace,
                        cudaStream_t st);
size_t mask_compile_static_limit();
int mask_compile_static(const bma_mask_spec& spec, int B, int H, const bma_block_lists& l, cudaStream_t st);

namespace {
thread_local char g_err_text[512] = "";
__device__ int g_device_status_word = 0;
constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {};
std::mutex g_status_mutex;
std::atomic<unsigned long long> g_launches{0};
}  // namespace

void count_launches(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

void set_last_cuda_error(cudaError_t e, const char* where) {
  std::snprintf(g_err_text, sizeof(g_err_text), "CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), where);
  (void)cudaGetLastError();  // clear the sticky-less error so that later calls start clean
}

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_device_status_word);
    if (e != cudaSuccess) { set_last_cuda_error(e, "cudaGetSymbolAddress(status)"); return nullptr; }
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

namespace {

// ---- backward preprocess: delta = rowsum(dO * O), optional bf16 copy of dO ---------------
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
  v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
}

// Streaming form for d <= 128 with vector accesses: one warp takes FOUR consecutive queries of one
// (batch, head), issues all eight 16-byte loads per lane before it uses any of them, and writes the four
// delta values as one 16-byte line, so that the [B, Hq, N] delta array is written in whole sectors
// (one warp per row wrote 4 bytes per 32-byte sector).  Bound by HBM: reads |O| + |dO|, writes the bf16
// copy of dO and delta.
template <typename TO, typename TDO>
__global__ void __launch_bounds__(256) bwd_preprocess_rows4_kernel(bma_attn_args a, __nv_bfloat16* __restrict__ do_bf16) {
  const int lane = threadIdx.x & 31;
  const int warps = (blockDim.x >> 5);
  const int64_t nq4 = (a.N + 3) / 4;
  const int64_t units = (int64_t)a.B * a.Hq * nq4;
  const int c = lane * 4;
  const bool act = c < a.d;
  for (int64_t u = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); u < units; u += (int64_t)gridDim.x * warps) {
    const int q0 = (int)(u % nq4) * 4;
    const int h = (int)((u / nq4) % a.Hq);
    const int b = (int)(u / (nq4 * a.Hq));
    float gv[4][4], ov[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int q = q0 + i;
      if (act && q < a.N) {
        load4(static_cast<const TDO*>(a.d_o.ptr) + (int64_t)b * a.d_o.stride_b + (int64_t)q * a.d_o.stride_l + (int64_t)h * a.d_o.stride_h + c, gv[i]);
        load4(static_cast<const TO*>(a.o.ptr) + (int64_t)b * a.o.stride_b + (int64_t)q * a.o.stride_l + (int64_t)h * a.o.stride_h + c, ov[i]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) { gv[i][e] = 0.f; ov[i][e] = 0.f; }
      }
    }
    // With a bf16 copy, delta is taken from the ROUNDED cotangent -- the values the dP = dO V^T product of the backward
    // kernels sees -- so that dP - delta cancels where it should (a row that attends one key has dS = 0 exactly; with
    // the float32 cotangent in delta and the bf16 one in dP the difference of the two roundings would survive).
    float acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int q = q0 + i;
      if (do_bf16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(gv[i][0], gv[i][1]), hi = __floats2bfloat162_rn(gv[i][2], gv[i][3]);
        uint2 w;
        w.x = *reinterpret_cast<uint32_t*>(&lo);
        w.y = *reinterpret_cast<uint32_t*>(&hi);
        gv[i][0] = __uint_as_float(w.x << 16); gv[i][1] = __uint_as_float(w.x & 0xffff0000u);
        gv[i][2] = __uint_as_float(w.y << 16); gv[i][3] = __uint_as_float(w.y & 0xffff0000u);
        if (act && q < a.N) *reinterpret_cast<uint2*>(do_bf16 + (((int64_t)b * a.N + q) * a.Hq + h) * a.d + c) = w;
      }
      acc[i] = fmaf(gv[i][0], ov[i][0], fmaf(gv[i][1], ov[i][1], fmaf(gv[i][2], ov[i][2], gv[i][3] * ov[i][3])));
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }
    float* dst = a.delta + ((int64_t)b * a.Hq + h) * a.N + q0;
    if (lane == 0) {
      if (q0 + 3 < a.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (q0 + i < a.N) dst[i] = acc[i];
      }
    }
  }
}

// One warp per (b, q, h) row.  VEC: 4-element vector accesses (d % 4 == 0, 16-byte aligned rows).
template <typename TO, typename TDO, bool VEC>
__global__ void bwd_preprocess_kernel(bma_attn_args a, __nv_bfloat16* __restrict__ do_bf16) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)a.B * a.N * a.Hq;
  const int warps = (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * warps) {
    const int h = (int)(r % a.Hq);
    const int q = (int)((r / a.Hq) % a.N);
    const int b = (int)(r / ((int64_t)a.Hq * a.N));
    const TO* o = static_cast<const TO*>(a.o.ptr) + (int64_t)b * a.o.stride_b + (int64_t)q * a.o.stride_l + (int64_t)h * a.o.stride_h;
    const TDO* g = static_cast<const TDO*>(a.d_o.ptr) + (int64_t)b * a.d_o.stride_b + (int64_t)q * a.d_o.stride_l + (int64_t)h * a.d_o.stride_h;
    float acc = 0.f;
    if (VEC) {
      for (int c = lane * 4; c < a.d; c += 128) {
        float gv[4], ov[4];
        load4(g + c, gv);
        load4(o + c, ov);
        if (do_bf16) {   // delta from the rounded cotangent, see bwd_preprocess_rows4_kernel
          __nv_bfloat162 lo = __floats2bfloat162_rn(gv[0], gv[1]), hi = __floats2bfloat162_rn(gv[2], gv[3]);
          uint2 w;
          w.x = *reinterpret_cast<uint32_t*>(&lo);
          w.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(do_bf16 + r * a.d + c) = w;
          gv[0] = __uint_as_float(w.x << 16); gv[1] = __uint_as_float(w.x & 0xffff0000u);
          gv[2] = __uint_as_float(w.y << 16); gv[3] = __uint_as_float(w.y & 0xffff0000u);
        }
        acc = fmaf(gv[0], ov[0], acc); acc = fmaf(gv[1], ov[1], acc);
        acc = fmaf(gv[2], ov[2], acc); acc = fmaf(gv[3], ov[3], acc);
      }
    } else {
      for (int c = lane; c < a.d; c += 32) {
        float gv = to_float(g[c]);
        if (do_bf16) {
          const __nv_bfloat16 gb = __float2bfloat16_rn(gv);
          do_bf16[r * a.d + c] = gb;
          gv = __bfloat162float(gb);
        }
        acc = fmaf(gv, to_float(o[c]), acc);
      }
    }
    for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) a.delta[((int64_t)b * a.Hq + h) * a.N + q] = acc;
  }
}

// ---- merge of two partial results over disjoint key sets ---------------------------------
__global__ void merge_kernel(bma_attn_args a) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)a.B * a.N * a.Hq;
  const int warps = (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * warps) {
    const int h = (int)(r % a.Hq);
    const int q = (int)((r / a.Hq) % a.N);
    const int b = (int)(r / ((int64_t)a.Hq * a.N));
    float* oa = static_cast<float*>(a.o.ptr) + (int64_t)b * a.o.stride_b + (int64_t)q * a.o.stride_l + (int64_t)h * a.o.stride_h;
    const float* ob = static_cast<const float*>(a.d_o.ptr) + (int64_t)b * a.d_o.stride_b + (int64_t)q * a.d_o.stride_l + (int64_t)h * a.d_o.stride_h;
    const int64_t li = ((int64_t)b * a.Hq + h) * a.N + q;
    const float la = a.lse[li], lb = a.delta[li];
    const float mx = fmaxf(la, lb);
    float wa = 0.f, wb = 0.f, l = -INFINITY;
    if (mx != -INFINITY) {
      const float ea = expf(la - mx), eb = expf(lb - mx);
      l = mx + logf(ea + eb);
      wa = ea / (ea + eb);
      wb = eb / (ea + eb);
    }
    for (int c = lane; c < a.d; c += 32) oa[c] = wa * oa[c] + wb * ob[c];
    if (lane == 0) a.lse[li] = l;
  }
}

// ---- self-test of the bounded waits ------------------------------------------------------------
// One CTA waits on an mbarrier that nobody arrives at, with the same polling scheme as the attention kernels but a
// caller-chosen time limit; when the limit passes it records `code` in the status word and returns.  Nothing
// faults, traps or hangs: this is how a host learns of a lost producer without losing the context.
__global__ void expire_wait_kernel(int* status, unsigned long long limit_ns, int code) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_barrier_init();
    const uint64_t t0 = ptx::global_timer_ns();
    bool done = false;
    for (uint32_t i = 0; i < (1u << 26) && !done; ++i) {
      if (ptx::mbar_try_wait(&bar, 0)) done = true;
      else if ((i & 63u) == 63u && ptx::global_timer_ns() - t0 > limit_ns) break;
    }
    if (!done) report_device_error(status, code);
  }
}

int validate_tensor(const bma_tensor& t, bool required) {
  if (!t.ptr) return required ? BMA_ERR_ARG : BMA_OK;
  BMA_REQUIRE(t.dtype == BMA_DTYPE_F32 || t.dtype == BMA_DTYPE_BF16, BMA_ERR_UNSUPPORTED);
  return BMA_OK;
}

int validate_common(const bma_attn_args* a) {
  BMA_REQUIRE(a != nullptr, BMA_ERR_ARG);
  BMA_REQUIRE(a->B > 0 && a->N > 0 && a->L > 0 && a->Hq > 0 && a->Hkv > 0 && a->d > 0, BMA_ERR_ARG);
  BMA_REQUIRE(a->Hq % a->Hkv == 0, BMA_ERR_ARG);
  BMA_REQUIRE(a->d <= 128, BMA_ERR_UNSUPPORTED);
  BMA_REQUIRE(a->Hq <= 65535 && a->B <= 65535, BMA_ERR_LIMIT);
  return BMA_OK;
}

int validate_lists(const bma_attn_args* a, const bma_block_lists* l, int tile, bool need_q_side) {
  BMA_REQUIRE(l != nullptr, BMA_ERR_ARG);
  BMA_REQUIRE(l->kv_num && l->kv_idx && l->full_kv_num && l->full_kv_idx, BMA_ERR_ARG);
  BMA_REQUIRE(!need_q_side || (l->q_num && l->q_idx && l->full_q_num && l->full_q_idx), BMA_ERR_ARG);
  BMA_REQUIRE(l->q_block == tile && l->kv_block == tile, BMA_ERR_ARG);
  BMA_REQUIRE(l->NQ == ceil_div(a->N, tile) && l->NKV == ceil_div(a->L, tile), BMA_ERR_ARG);
  BMA_REQUIRE((l->B == 1 || l->B == a->B) && (l->H == 1 || l->H == a->Hq), BMA_ERR_ARG);
  return BMA_OK;
}

int pick_backend(const bma_attn_args* a) {
  if (a->backend == BMA_BACKEND_SIMT) return BMA_BACKEND_SIMT;
  if (sm100_supported(*a)) return BMA_BACKEND_TCGEN05;
  if (a->backend == BMA_BACKEND_TCGEN05) return -1;
  return BMA_BACKEND_SIMT;
}

int pick_backend_bwd(const bma_attn_args* a) {
  if (a->backend == BMA_BACKEND_SIMT) return BMA_BACKEND_SIMT;
  if (sm100_bwd_supported(*a)) return BMA_BACKEND_TCGEN05;
  if (a->backend == BMA_BACKEND_TCGEN05) return -1;
  return BMA_BACKEND_SIMT;
}

int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

}  // namespace
}  // namespace bma

using namespace bma;

extern "C" {

int bma_version(void) { return 1000; }

unsigned long long bma_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* bma_error_string(int status) {
  switch (status) {
    case BMA_OK: return "ok";
    case BMA_ERR_ARG: return "invalid argument (null pointer, bad size or inconsistent shapes)";
    case BMA_ERR_UNSUPPORTED: return "request not covered by any kernel (dtype / head dim / backend)";
    case BMA_ERR_WORKSPACE: return "workspace missing or too small";
    case BMA_ERR_CUDA: return g_err_text[0] ? g_err_text : "CUDA call failed";
    case BMA_ERR_LIMIT: return "size beyond a fixed limit of the library";
    case BMA_ERR_DEVICE_CHECK: return "a device-side bounded wait or bounds check gave up";
    default: return "unknown status";
  }
}

size_t bma_mask_compile_workspace_bytes(const bma_mask_spec* spec, int32_t B, int32_t H, int32_t NQ, int32_t NKV) {
  if (!spec || B <= 0 || H <= 0 || NQ <= 0 || NKV <= 0) return 0;
  return mask_compile_workspace_bytes(*spec, B, H, NQ, NKV);
}

int bma_mask_compile(const bma_mask_spec* spec, int32_t B, int32_t H, const bma_block_lists* lists, void* workspace,
                     size_t workspace_bytes, bma_stream_t stream) {
  BMA_REQUIRE(spec && lists, BMA_ERR_ARG);
  int rc = mask_compile_validate(*spec, B, H, *lists);
  if (rc != BMA_OK) return rc;
  const size_t need = mask_compile_workspace_bytes(*spec, B, H, lists->NQ, lists->NKV);
  BMA_REQUIRE(workspace != nullptr && workspace_bytes >= need, BMA_ERR_WORKSPACE);
  return mask_compile_launch(*spec, B, H, *lists, workspace, static_cast<cudaStream_t>(stream));
}

size_t bma_mask_compile_static_limit(void) { return mask_compile_static_limit(); }

int bma_mask_compile_static(const bma_mask_spec* spec, int32_t B, int32_t H, const bma_block_lists* lists,
                            bma_stream_t stream) {
  BMA_REQUIRE(spec && lists, BMA_ERR_ARG);
  return mask_compile_static(*spec, B, H, *lists, static_cast<cudaStream_t>(stream));
}

int bma_attn_plan(const bma_attn_args* args, int32_t* backend, int32_t* q_tile, int32_t* kv_tile) {
  int rc = validate_common(args);
  if (rc != BMA_OK) return rc;
  const int be = pick_backend(args);
  BMA_REQUIRE(be > 0, BMA_ERR_UNSUPPORTED);
  const int tile = be == BMA_BACKEND_TCGEN05 ? kSm100Tile : kSimtTile;
  if (backend) *backend = be;
  if (q_tile) *q_tile = tile;
  if (kv_tile) *kv_tile = tile;
  return BMA_OK;
}

int bma_attn_bwd_plan(const bma_attn_args* args, int32_t* backend, int32_t* q_tile, int32_t* kv_tile) {
  int rc = validate_common(args);
  if (rc != BMA_OK) return rc;
  const int be = pick_backend_bwd(args);
  BMA_REQUIRE(be > 0, BMA_ERR_UNSUPPORTED);
  const int tile = be == BMA_BACKEND_TCGEN05 ? kSm100Tile : kSimtTile;
  if (backend) *backend = be;
  if (q_tile) *q_tile = tile;
  if (kv_tile) *kv_tile = tile;
  return BMA_OK;
}

int bma_attn_fwd(const bma_attn_args* args, const bma_mask_spec* spec, const bma_block_lists* lists,
                 bma_stream_t stream) {
  int rc = validate_common(args);
  if (rc != BMA_OK) return rc;
  BMA_REQUIRE(spec != nullptr, BMA_ERR_ARG);
  if ((rc = validate_tensor(args->q, true)) || (rc = validate_tensor(args->k, true)) ||
      (rc = validate_tensor(args->v, true)) || (rc = validate_tensor(args->o, true)))
    return rc;
  BMA_REQUIRE(args->q.dtype == args->k.dtype && args->k.dtype == args->v.dtype, BMA_ERR_UNSUPPORTED);
  const int be = pick_backend(args);
  BMA_REQUIRE(be > 0, BMA_ERR_UNSUPPORTED);
  const int tile = be == BMA_BACKEND_TCGEN05 ? kSm100Tile : kSimtTile;
  if ((rc = validate_lists(args, lists, tile, false))) return rc;
  BMA_REQUIRE(spec->q_valid <= args->N && spec->k_valid <= args->L, BMA_ERR_ARG);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return be == BMA_BACKEND_TCGEN05 ? sm100_fwd(*args, *spec, *lists, st) : simt_fwd(*args, *spec, *lists, st);
}

int bma_attn_bwd_preprocess(const bma_attn_args* args, void* d_o_bf16, bma_stream_t stream) {
  int rc = validate_common(args);
  if (rc != BMA_OK) return rc;
  if ((rc = validate_tensor(args->o, true)) || (rc = validate_tensor(args->d_o, true))) return rc;
  BMA_REQUIRE(args->delta != nullptr, BMA_ERR_ARG);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = (int64_t)args->B * args->N * args->Hq;
  const int grid = (int)std::min<int64_t>((rows + 7) / 8, (int64_t)sm_count() * 16);
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(d_o_bf16);
  const bool of = args->o.dtype == BMA_DTYPE_F32, gf = args->d_o.dtype == BMA_DTYPE_F32;
  auto vec_ok = [&](const bma_tensor& t) {
    return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && t.stride_b % 4 == 0 && t.stride_l % 4 == 0 && t.stride_h % 4 == 0;
  };
  const bool vec = args->d % 4 == 0 && vec_ok(args->o) && vec_ok(args->d_o) && (reinterpret_cast<uintptr_t>(out) & 7) == 0;
  const int64_t units4 = (int64_t)args->B * args->Hq * ((args->N + 3) / 4);
  const int grid4 = (int)std::min<int64_t>((units4 + 7) / 8, (int64_t)sm_count() * 32);
#define BMA_PRE(TO, TDO)                                                                   \
  do {                                                                                     \
    if (vec && args->d <= 128) bwd_preprocess_rows4_kernel<TO, TDO><<<grid4, 256, 0, st>>>(*args, out); \
    else if (vec) bwd_preprocess_kernel<TO, TDO, true><<<grid, 256, 0, st>>>(*args, out);  \
    else bwd_preprocess_kernel<TO, TDO, false><<<grid, 256, 0, st>>>(*args, out);          \
  } while (0)
  if (of && gf) BMA_PRE(float, float);
  else if (of) BMA_PRE(float, __nv_bfloat16);
  else if (gf) BMA_PRE(__nv_bfloat16, float);
  else BMA_PRE(__nv_bfloat16, __nv_bfloat16);
#undef BMA_PRE
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

size_t bma_attn_bwd_workspace_bytes(const bma_attn_args* args) {
  if (validate_common(args) != BMA_OK) return 0;
  return pick_backend_bwd(args) == BMA_BACKEND_TCGEN05 ? sm100_bwd_workspace_bytes(*args) : 0;
}

size_t bma_attn_bwd_scratch_bytes(const bma_attn_args* args, const bma_block_lists* lists, const int64_t* visited_host) {
  if (validate_common(args) != BMA_OK || !lists) return 0;
  return pick_backend_bwd(args) == BMA_BACKEND_TCGEN05 ? sm100_bwd_scratch_bytes(*args, *lists, visited_host) : 0;
}

size_t bma_attn_bwd_scratch_min_bytes(const bma_attn_args* args, const bma_block_lists* lists, const int64_t* visited_host) {
  if (validate_common(args) != BMA_OK || !lists) return 0;
  return pick_backend_bwd(args) == BMA_BACKEND_TCGEN05 ? sm100_bwd_scratch_min_bytes(*args, *lists, visited_host) : 0;
}

int bma_block_lists_visited(const bma_block_lists* lists, int64_t* visited, bma_stream_t stream) {
  BMA_REQUIRE(lists && visited, BMA_ERR_ARG);
  BMA_REQUIRE(lists->B > 0 && lists->H > 0 && lists->NQ > 0 && lists->kv_num && lists->full_kv_num, BMA_ERR_ARG);
  return block_lists_visited(*lists, visited, static_cast<cudaStream_t>(stream));
}

int bma_debug_expire_wait(uint64_t limit_ns, int32_t code, bma_stream_t stream) {
  BMA_REQUIRE(limit_ns > 0 && limit_ns <= 1000000000ull && code > 0, BMA_ERR_ARG);   // at most one second
  int* status = device_status_ptr();
  BMA_REQUIRE(status != nullptr, BMA_ERR_CUDA);
  expire_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_ns, code);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

int bma_attn_bwd(const bma_attn_args* args, const bma_mask_spec* spec, const bma_block_lists* lists, void* workspace,
                 size_t workspace_bytes, const int64_t* visited_host, void* mid_event, bma_stream_t stream) {
  cudaEvent_t mark = static_cast<cudaEvent_t>(mid_event);
  int rc = validate_common(args);
  if (rc != BMA_OK) return rc;
  BMA_REQUIRE(spec != nullptr, BMA_ERR_ARG);
  if ((rc = validate_tensor(args->q, true)) || (rc = validate_tensor(args->k, true)) ||
      (rc = validate_tensor(args->v, true)) || (rc = validate_tensor(args->d_o, true)) ||
      (rc = validate_tensor(args->dq, true)) || (rc = validate_tensor(args->dk, true)) ||
      (rc = validate_tensor(args->dv, true)))
    return rc;
  BMA_REQUIRE(args->lse && args->delta, BMA_ERR_ARG);
  BMA_REQUIRE(args->q.dtype == args->k.dtype && args->k.dtype == args->v.dtype, BMA_ERR_UNSUPPORTED);
  BMA_REQUIRE(args->dq.dtype == args->q.dtype && args->dk.dtype == args->q.dtype && args->dv.dtype == args->q.dtype,
              BMA_ERR_UNSUPPORTED);
  const int be = pick_backend_bwd(args);
  BMA_REQUIRE(be > 0, BMA_ERR_UNSUPPORTED);
  const int tile = be == BMA_BACKEND_TCGEN05 ? kSm100Tile : kSimtTile;
  if ((rc = validate_lists(args, lists, tile, true))) return rc;
  BMA_REQUIRE(spec->q_valid <= args->N && spec->k_valid <= args->L, BMA_ERR_ARG);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (be == BMA_BACKEND_TCGEN05) {
    const size_t need = sm100_bwd_workspace_bytes(*args);
    BMA_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), BMA_ERR_WORKSPACE);
    return sm100_bwd(*args, *spec, *lists, workspace, workspace_bytes, visited_host, mark, st);
  }
  return simt_bwd(*args, *spec, *lists, st);
}

int bma_attn_merge(const bma_attn_args* args, bma_stream_t stream) {
  int rc = validate_common(args);
  if (rc != BMA_OK) return rc;
  BMA_REQUIRE(args->o.ptr && args->d_o.ptr && args->lse && args->delta, BMA_ERR_ARG);
  BMA_REQUIRE(args->o.dtype == BMA_DTYPE_F32 && args->d_o.dtype == BMA_DTYPE_F32, BMA_ERR_UNSUPPORTED);
  const int64_t rows = (int64_t)args->B * args->N * args->Hq;
  const int grid = (int)std::min<int64_t>((rows + 7) / 8, (int64_t)sm_count() * 16);
  merge_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(*args);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

int bma_device_status(bma_stream_t stream, int32_t* detail) {
  int* p = device_status_ptr();
  BMA_REQUIRE(p != nullptr, BMA_ERR_CUDA);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int v = 0;
  BMA_CUDA_TRY(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, st));
  BMA_CUDA_TRY(cudaStreamSynchronize(st));
  if (v != 0) BMA_CUDA_TRY(cudaMemsetAsync(p, 0, sizeof(int), st));
  if (detail) *detail = v;
  return v == 0 ? BMA_OK : BMA_ERR_DEVICE_CHECK;
}

}  // extern "C"
