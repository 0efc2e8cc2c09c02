// Mask programs: an arbitrary integer predicate of (b, h, q, k), given as straight-line
// three-address code, evaluated for a whole [B, H, N, L] box into the bit table the mask
// description takes.  One thread produces one 32-key word; the program (a few hundred bytes)
// travels in the kernel parameters, the value file sits in local memory.  The work is integer ALU
// plus one coalesced 4-byte store per 32 predicates, so the kernel is bound by instruction issue,
// not by HBM: 2^32 predicates of ~10 instructions take a few milliseconds.
#include "common.cuh"

namespace bma {
namespace {

__device__ __forceinline__ int32_t floor_div(int32_t a, int32_t b) {
  if (b == 0) return 0;
  int32_t q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}
__device__ __forceinline__ int32_t floor_mod(int32_t a, int32_t b) {
  if (b == 0) return 0;
  int32_t r = a % b;
  if (r != 0 && ((r < 0) != (b < 0))) r += b;
  return r;
}
__device__ __forceinline__ int64_t clamp_index(int32_t i, int64_t n) {
  return i < 0 ? 0 : (i >= n ? n - 1 : (int64_t)i);
}

__device__ int32_t run_program(const bma_mask_program& p, int32_t b, int32_t h, int32_t q, int32_t k) {
  int32_t v[4 + BMA_PROGRAM_MAX_INSTR];
  v[0] = b; v[1] = h; v[2] = q; v[3] = k;
  for (int i = 0; i < p.n_instr; ++i) {
    const int32_t op = p.code[4 * i], x = p.code[4 * i + 1], y = p.code[4 * i + 2], z = p.code[4 * i + 3];
    int32_t r = 0;
    switch (op) {
      case BMA_OP_CONST: r = x; break;
      case BMA_OP_NEG: r = -v[x]; break;
      case BMA_OP_ABS: r = v[x] < 0 ? -v[x] : v[x]; break;
      case BMA_OP_NOT: r = v[x] == 0; break;
      case BMA_OP_INV: r = ~v[x]; break;
      case BMA_OP_ADD: r = v[x] + v[y]; break;
      case BMA_OP_SUB: r = v[x] - v[y]; break;
      case BMA_OP_MUL: r = v[x] * v[y]; break;
      case BMA_OP_FLOORDIV: r = floor_div(v[x], v[y]); break;
      case BMA_OP_MOD: r = floor_mod(v[x], v[y]); break;
      case BMA_OP_MIN: r = min(v[x], v[y]); break;
      case BMA_OP_MAX: r = max(v[x], v[y]); break;
      case BMA_OP_LT: r = v[x] < v[y]; break;
      case BMA_OP_LE: r = v[x] <= v[y]; break;
      case BMA_OP_GT: r = v[x] > v[y]; break;
      case BMA_OP_GE: r = v[x] >= v[y]; break;
      case BMA_OP_EQ: r = v[x] == v[y]; break;
      case BMA_OP_NE: r = v[x] != v[y]; break;
      case BMA_OP_AND: r = v[x] & v[y]; break;
      case BMA_OP_OR: r = v[x] | v[y]; break;
      case BMA_OP_XOR: r = v[x] ^ v[y]; break;
      case BMA_OP_SHL: r = (int32_t)((uint32_t)v[x] << (v[y] & 31)); break;
      case BMA_OP_SHR: r = v[x] >> (v[y] & 31); break;
      case BMA_OP_SELECT: r = v[x] ? v[y] : v[z]; break;
      case BMA_OP_LOAD1: r = __ldg(p.tables[x] + clamp_index(v[y], p.table_cols[x])); break;
      case BMA_OP_LOAD2:
        r = __ldg(p.tables[x] + clamp_index(v[y], p.table_rows[x]) * p.table_stride[x] + clamp_index(v[z], p.table_cols[x]));
        break;
      default: break;
    }
    v[4 + i] = r;
  }
  return v[3 + p.n_instr];
}

struct TableParams {
  bma_mask_program prog;
  int32_t B, H, N, L, words, q_offset, k_offset;
  int32_t* bits;
};

__global__ void __launch_bounds__(256) mask_table_kernel(const __grid_constant__ TableParams p) {
  const int64_t total = (int64_t)p.B * p.H * p.N * p.words;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int w = (int)(idx % p.words);
    int64_t rest = idx / p.words;
    const int q = (int)(rest % p.N);
    rest /= p.N;
    const int h = (int)(rest % p.H), b = (int)(rest / p.H);
    uint32_t word = 0;
    for (int j = 0; j < 32; ++j) {
      const int k = w * 32 + j;
      if (k < p.L && run_program(p.prog, b, h, q + p.q_offset, k + p.k_offset) != 0) word |= 1u << j;
    }
    p.bits[idx] = (int32_t)word;
  }
}

// The TILES form: one CTA of 128 threads per 128 x 128 tile, thread = query row.  Every thread evaluates its row's 128
// keys into four words; the CTA reduces "some pair allowed" / "every valid pair allowed"; a cut tile takes the next
// slot from a counter and stores its bits twice, by query row and by key row (4 KB).  Slots are handed out in completion order: they differ from run to
// run, the predicate they encode does not.
struct TilesParams {
  bma_mask_program prog;
  int32_t B, H, N, L, TQ, TK, q_offset, k_offset, capacity;
  uint8_t* tile_class;
  int32_t* tile_slot;
  uint32_t* tile_bits;
  int32_t* counter;
};

__global__ void __launch_bounds__(128) mask_tiles_kernel(const __grid_constant__ TilesParams p) {
  __shared__ int s_any, s_open, s_slot;
  __shared__ uint32_t s_cols[128][4];   // the tile by key row: word w of key j = the ballot of warp w (query rows 32w ..)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t tiles = (int64_t)p.B * p.H * p.TQ * p.TK;
  for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int tk = (int)(t % p.TK);
    int64_t rest = t / p.TK;
    const int tq = (int)(rest % p.TQ);
    rest /= p.TQ;
    const int h = (int)(rest % p.H), b = (int)(rest / p.H);
    if (threadIdx.x == 0) { s_any = 0; s_open = 0; }
    __syncthreads();
    // tile (tq, tk) of the GLOBAL grid holds local rows / keys [tq*128 - q_offset, ...): offsets are multiples of 128
    const int q = tq * 128 + (int)threadIdx.x - p.q_offset;
    const bool row_valid = q >= 0 && q < p.N;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    bool any = false, open = false;   // open: a valid pair of this row is NOT allowed
    for (int j = 0; j < 128; ++j) {   // the whole warp walks the keys together: the ballot is the key's column word
      const int k = tk * 128 + j - p.k_offset;
      const bool valid = row_valid && k >= 0 && k < p.L;
      const bool ok = valid && run_program(p.prog, b, h, q + p.q_offset, k + p.k_offset) != 0;
      if (ok) { w[j >> 5] |= 1u << (j & 31); any = true; }
      else if (valid) open = true;
      const uint32_t col = __ballot_sync(0xffffffffu, ok);
      if (lane == 0) s_cols[j][warp] = col;
    }
    if (any) atomicOr(&s_any, 1);
    if (open) atomicOr(&s_open, 1);
    __syncthreads();
    const int cls = !s_any ? 0 : (s_open ? 1 : 2);
    if (threadIdx.x == 0) {
      p.tile_class[t] = (uint8_t)cls;
      int slot = -1;
      if (cls == 1) slot = atomicAdd(p.counter, 1);
      p.tile_slot[t] = (slot >= 0 && slot < p.capacity) ? slot : -1;
      s_slot = slot;
    }
    __syncthreads();
    const int slot = s_slot;
    if (cls == 1 && slot >= 0 && slot < p.capacity) {
      uint32_t* out = p.tile_bits + (int64_t)slot * 256 * 4;
      *reinterpret_cast<uint4*>(out + threadIdx.x * 4) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(out + (128 + threadIdx.x) * 4) =
          make_uint4(s_cols[threadIdx.x][0], s_cols[threadIdx.x][1], s_cols[threadIdx.x][2], s_cols[threadIdx.x][3]);
    }
    __syncthreads();
  }
}

}  // namespace

// every operand must name an earlier value, every table an existing one: checked on the host, once, so that the
// kernels need no bounds checks of their own
int validate_program(const bma_mask_program* program) {
  BMA_REQUIRE(program->n_instr >= 1 && program->n_instr <= BMA_PROGRAM_MAX_INSTR, BMA_ERR_ARG);
  BMA_REQUIRE(program->n_tables >= 0 && program->n_tables <= BMA_PROGRAM_MAX_TABLES, BMA_ERR_ARG);
  for (int i = 0; i < program->n_instr; ++i) {
    const int32_t op = program->code[4 * i], x = program->code[4 * i + 1], y = program->code[4 * i + 2], z = program->code[4 * i + 3];
    const int32_t defined = 4 + i;
    auto val = [&](int32_t r) { return r >= 0 && r < defined; };
    BMA_REQUIRE(op >= 0 && op < BMA_OP_COUNT, BMA_ERR_ARG);
    if (op == BMA_OP_CONST) continue;
    if (op == BMA_OP_LOAD1 || op == BMA_OP_LOAD2) {
      BMA_REQUIRE(x >= 0 && x < program->n_tables && program->tables[x] != nullptr, BMA_ERR_ARG);
      BMA_REQUIRE(program->table_cols[x] > 0 && program->table_rows[x] > 0, BMA_ERR_ARG);
      BMA_REQUIRE(val(y) && (op == BMA_OP_LOAD1 || val(z)), BMA_ERR_ARG);
      continue;
    }
    BMA_REQUIRE(val(x), BMA_ERR_ARG);
    if (op >= BMA_OP_ADD) BMA_REQUIRE(val(y), BMA_ERR_ARG);
    if (op == BMA_OP_SELECT) BMA_REQUIRE(val(z), BMA_ERR_ARG);
  }
  return BMA_OK;
}

}  // namespace bma

extern "C" int bma_mask_tiles_build(const bma_mask_program* program, int32_t B, int32_t H, int32_t N, int32_t L,
                                    int32_t q_offset, int32_t k_offset, uint8_t* tile_class, int32_t* tile_slot,
                                    uint32_t* tile_bits, int32_t capacity, int32_t* counter, bma_stream_t stream) {
  using namespace bma;
  BMA_REQUIRE(program != nullptr && tile_class != nullptr && tile_slot != nullptr && counter != nullptr, BMA_ERR_ARG);
  BMA_REQUIRE(B > 0 && H > 0 && N > 0 && L > 0 && capacity >= 0 && (capacity == 0 || tile_bits != nullptr), BMA_ERR_ARG);
  BMA_REQUIRE(q_offset >= 0 && k_offset >= 0 && q_offset % 128 == 0 && k_offset % 128 == 0, BMA_ERR_ARG);
  int rc = validate_program(program);
  if (rc != BMA_OK) return rc;
  TilesParams p;
  p.prog = *program;
  p.B = B; p.H = H; p.N = N; p.L = L;
  p.TQ = (N + q_offset + 127) / 128; p.TK = (L + k_offset + 127) / 128;
  p.q_offset = q_offset; p.k_offset = k_offset; p.capacity = capacity;
  p.tile_class = tile_class; p.tile_slot = tile_slot; p.tile_bits = tile_bits; p.counter = counter;
  const int64_t tiles = (int64_t)B * H * p.TQ * p.TK;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)(tiles < (int64_t)sms * 16 ? tiles : (int64_t)sms * 16);
  mask_tiles_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}

extern "C" int bma_mask_table_build(const bma_mask_program* program, int32_t B, int32_t H, int32_t N, int32_t L,
                                    int32_t q_offset, int32_t k_offset, int32_t* bits, bma_stream_t stream) {
  using namespace bma;
  BMA_REQUIRE(program != nullptr && bits != nullptr, BMA_ERR_ARG);
  BMA_REQUIRE(B > 0 && H > 0 && N > 0 && L > 0, BMA_ERR_ARG);
  int rc = validate_program(program);
  if (rc != BMA_OK) return rc;
  TableParams p;
  p.prog = *program;
  p.B = B; p.H = H; p.N = N; p.L = L; p.words = (L + 31) / 32;
  p.q_offset = q_offset; p.k_offset = k_offset;
  p.bits = bits;
  const int64_t total = (int64_t)B * H * N * p.words;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (total + 255) / 256;
  const int grid = (int)(want < (int64_t)sms * 16 ? want : (int64_t)sms * 16);  // grid-stride beyond 16 CTAs per SM
  mask_table_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launches(1);
  BMA_CUDA_TRY(cudaGetLastError());
  return BMA_OK;
}
