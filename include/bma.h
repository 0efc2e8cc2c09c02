/*
 * bma.h — C ABI of the B200-native blockwise masked attention library (libbma.so).
 *
 * The reference (acutkosky/jaxmodules) is pure Python on JAX and has no native boundary of
 * its own; the seam this ABI replaces is the body of the custom_vjp triple
 *   _masked_attention_via_map       jaxmodules/attention.py:180-241   (primal)
 *   _masked_attention_via_map_fwd   jaxmodules/attention.py:244-264   (vjp forward rule)
 *   _masked_attention_via_map_bwd   jaxmodules/attention.py:266-342   (vjp backward rule)
 * and the array builder behind create_block_mask, jaxmodules/block_mask.py:411-498.
 * Each entry point below names the reference code it stands in for.
 *
 * Conventions
 *   - plain C types only; every function returns an int status (BMA_OK == 0, negative =
 *     rejected arguments / host-side failure, positive = a device-side check tripped) and
 *     never throws, exits or synchronises the device;
 *   - the caller owns every buffer (inputs, outputs, workspace); all pointers are device
 *     pointers on the current device unless stated otherwise; the mask/args structs
 *     themselves are host memory and are copied at call time;
 *   - work is enqueued on the stream that is passed (a cudaStream_t cast to void*);
 *   - tensors are [B, L, H, d] with d contiguous and explicit element strides for B, L, H.
 */
#ifndef BMA_H_
#define BMA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* bma_stream_t; /* cudaStream_t */

/* ---- status codes ------------------------------------------------------------------ */
enum {
  BMA_OK = 0,
  BMA_ERR_ARG = -1,         /* null pointer, negative size, inconsistent shapes           */
  BMA_ERR_UNSUPPORTED = -2, /* valid request that no kernel covers (dtype, head dim ...)   */
  BMA_ERR_WORKSPACE = -3,   /* workspace missing or smaller than *_workspace_bytes()       */
  BMA_ERR_CUDA = -4,        /* a CUDA runtime / driver call failed; see bma_error_string   */
  BMA_ERR_LIMIT = -5,       /* size beyond a documented fixed limit                        */
  BMA_ERR_DEVICE_CHECK = 1  /* a bounded wait or bounds check inside a kernel gave up      */
};

enum { BMA_DTYPE_F32 = 0, BMA_DTYPE_BF16 = 1 };

/* ---- mask description ----------------------------------------------------------------
 * Device-evaluable form of the reference's mask_fn(b, h, q, k) (jaxmodules/attention.py:
 * 368-372, 404-419, 437).  The predicate is the AND of every enabled term; with flags == 0
 * every (q, k) inside the valid box is allowed.
 *   gq = q + q_offset, gk = k + k_offset          (offsets are 0 except for sequence shards)
 *   always      : q < q_valid  &&  k < k_valid                       (attention.py:437)
 *   CAUSAL      : gk <= gq                                           (attention.py:414)
 *   BAND        : gq - band_left <= gk <= gq + band_right
 *   BLOCK_WINDOW: the key-block window of window_size (attention.py:161-167, 199-204):
 *                 i = gq / win_block, s = min(max(0, i - win_left), win_nblk - win_left - win_right),
 *                 s*win_block <= gk < (s + win_left + win_right)*win_block
 *   SEGMENT     : seg_q[b*seg_q_stride + gq] == seg_k[b*seg_k_stride + gk]
 *   BITMAP      : bit (gk & 31) of bitmap[((b%bitmap_B)*bitmap_H + h%bitmap_H)*bitmap_q + gq)*bitmap_words + gk/32]
 *                 (an arbitrary host-evaluated mask_fn; h is the QUERY head, attention.py:72-73)
 *   TILES       : the same arbitrary predicate stored per 128 x 128 tile of the global (gq, gk) grid, so that its
 *                 memory grows with the tiles the mask CUTS, not with N*L (bma_mask_tiles_build makes it from a mask
 *                 program).  t = ((b%tiles_B)*tiles_H + h%tiles_H)*tiles_q + gq/128)*tiles_k + gk/128:
 *                 tile_class[t] = 0 no pair of the tile is allowed, 2 every pair is, 1 some are -- and then bit (gk & 31)
 *                 of tile_bits[(tile_slot[t]*256 + gq%128)*4 + (gk%128)/32] decides.  A cut tile is stored twice, by
 *                 query row and (second 2 KB) by key row -- bit (gq & 31) of
 *                 tile_bits[(tile_slot[t]*256 + 128 + gk%128)*4 + (gq%128)/32] -- for the kernels that walk keys.
 */
enum {
  BMA_MASK_CAUSAL = 1,
  BMA_MASK_BAND = 2,
  BMA_MASK_BLOCK_WINDOW = 4,
  BMA_MASK_SEGMENT = 8,
  BMA_MASK_BITMAP = 16,
  BMA_MASK_TILES = 32,
  /* Not a mask term but a request to bma_mask_compile: segment-id blocks that the per-block id ranges
   * cannot decide are reported PARTIAL without scanning their elements.  The lists then may name a block
   * whose exact class is empty (never the reverse, and full blocks stay exact), which is harmless for the
   * attention kernels -- they evaluate the predicate on every partial block -- and saves the scan.
   * create_block_mask never sets it: its arrays are exact (jaxmodules/block_mask.py:471-481). */
  BMA_MASK_COMPILE_CONSERVATIVE = 256
};

typedef struct bma_mask_spec {
  int32_t flags;
  int32_t q_valid, k_valid;
  int32_t q_offset, k_offset;
  int32_t band_left, band_right;
  int32_t win_block, win_left, win_right, win_nblk;
  int32_t bitmap_B, bitmap_H, bitmap_q, bitmap_words;
  int32_t reserved_;
  const int32_t* seg_q;
  const int32_t* seg_k;
  int64_t seg_q_stride, seg_k_stride;
  const uint32_t* bitmap;
  int32_t tiles_B, tiles_H, tiles_q, tiles_k; /* TILES: extents of the tile grid (tiles_q = ceil(rows / 128) ...) */
  const uint8_t* tile_class;                   /* [tiles_B, tiles_H, tiles_q, tiles_k]            */
  const int32_t* tile_slot;                    /* same shape; meaningful where tile_class == 1     */
  const uint32_t* tile_bits;                   /* [slots, 2, 128, 4]: by query row, by key row     */
} bma_mask_spec;

/* ---- block lists ---------------------------------------------------------------------
 * The arrays of the reference's BlockMask (jaxmodules/block_mask.py:17-42): per q-block row
 * the number and the indices of PARTIAL kv blocks (kv_*), of FULL kv blocks (full_kv_*), and
 * the same per kv-block column (q_*, full_q_*).  Index rows have full width (NKV resp. NQ):
 * set blocks ascending, then unset blocks ascending, exactly what
 * argsort(-blocks) yields (block_mask.py:428-430).  B and H may be 1 to broadcast
 * (attention.py:521-522).  All int32.
 */
typedef struct bma_block_lists {
  int32_t B, H, NQ, NKV;
  int32_t q_block, kv_block;
  int32_t* kv_num;       /* [B,H,NQ]      */
  int32_t* kv_idx;       /* [B,H,NQ,NKV]  */
  int32_t* full_kv_num;  /* [B,H,NQ]      */
  int32_t* full_kv_idx;  /* [B,H,NQ,NKV]  */
  int32_t* q_num;        /* [B,H,NKV]     may be NULL together with the next three */
  int32_t* q_idx;        /* [B,H,NKV,NQ]  */
  int32_t* full_q_num;   /* [B,H,NKV]     */
  int32_t* full_q_idx;   /* [B,H,NKV,NQ]  */
} bma_block_lists;

/* ---- tensors ------------------------------------------------------------------------- */
typedef struct bma_tensor {
  void* ptr;
  int64_t stride_b, stride_l, stride_h; /* in elements; innermost (d) stride is 1 */
  int32_t dtype;                        /* BMA_DTYPE_* */
  int32_t reserved_;
} bma_tensor;

typedef struct bma_attn_args {
  int32_t B, N, L, Hq, Hkv, d;
  float scale;      /* 1/sqrt(d) for default_kernel, jaxmodules/attention.py:50 */
  int32_t backend;  /* BMA_BACKEND_AUTO or a forced backend (tests) */
  bma_tensor q, k, v;      /* inputs                                             */
  bma_tensor o;            /* [B,N,Hq,d] output (fwd) / input (bwd)               */
  float* lse;              /* [B,Hq,N] natural-log sum of exp; -inf for empty rows */
  bma_tensor d_o;          /* cotangent of o (bwd)                               */
  float* delta;            /* [B,Hq,N] rowsum(dO*O) (bwd)                        */
  bma_tensor dq, dk, dv;   /* outputs (bwd), dtype of q/k/v                      */
  const float* key_bias;   /* [Hq] or null: logits get + key_bias[h] * k (k = global key index incl. the mask's
                              k_offset) before the softmax -- the part of an affine score_mod
                              (jaxmodules/attention.py:543-554), e.g. ALiBi, that does not cancel in the softmax. */
} bma_attn_args;

enum { BMA_BACKEND_AUTO = 0, BMA_BACKEND_SIMT = 1, BMA_BACKEND_TCGEN05 = 2 };

/* ---- entry points -------------------------------------------------------------------- */

/* Library / ABI version (major*1000 + minor). */
int bma_version(void);

/* Number of CUDA kernels this library has launched in the calling process (diagnostics for
 * benchmarks; no counterpart in the reference). */
unsigned long long bma_launch_count(void);

/* Static text for a status code; for BMA_ERR_CUDA the text of the last CUDA error seen by
 * the calling thread is appended. */
const char* bma_error_string(int status);

/* Scratch bytes bma_mask_compile needs for a mask of B x H x NQ x NKV blocks. */
size_t bma_mask_compile_workspace_bytes(const bma_mask_spec* spec, int32_t B, int32_t H,
                                        int32_t NQ, int32_t NKV);

/* Block-mask compilation: classifies every (q-block, kv-block) of the mask as empty /
 * partial / full (partial = any ^ all, full = all) and writes the BlockMask arrays.
 * Replaces create_block_mask + BlockMask.from_blocks + get_sparse_{kv,q}_data_from_blocks,
 * jaxmodules/block_mask.py:454-498, 227-275, 411-451.  `B`,`H` are the mask's logical batch
 * and query-head counts; lists->B / lists->H are the extents actually written (1 only if
 * the spec does not depend on that index).  NQ = ceil(q_valid / q_block) etc. are taken
 * from `lists`; elements outside the valid box count as masked.  The output arrays double as
 * scratch during the call (the list of blocks that need an element scan sits in kv_idx until
 * the lists are written): they must not alias the inputs and hold no meaningful data until the
 * call's work has completed on `stream`. */
int bma_mask_compile(const bma_mask_spec* spec, int32_t B, int32_t H,
                     const bma_block_lists* lists, void* workspace, size_t workspace_bytes,
                     bma_stream_t stream);

/* bma_mask_compile without a caller-provided workspace and without any allocation.  This entry
 * point has no counterpart in the reference.  It exists for callers that are not allowed to
 * allocate device memory at call time -- for example a custom-call handler running inside a
 * compiled program whose buffers were all planned ahead of time, or a serving loop that froze its
 * memory pool at start-up -- where a cudaMalloc would stall the device or break that plan.  The
 * scratch (block flags, segment summaries) is a fixed 4 MiB array inside the library image, held
 * by every GPU that loads the library until the process exits; bma_mask_compile_static_limit()
 * returns that size.  A mask whose bma_mask_compile_workspace_bytes() exceeds it is rejected with
 * BMA_ERR_LIMIT (use bma_mask_compile with your own workspace).  Neither this call nor anything
 * it runs calls cudaMalloc, cudaFree or an allocating library routine; inputs and outputs are
 * still the caller's buffers.
 *   - The first call on each device looks up the array's device address; make that first call
 *     outside of any stream capture, with the device current.
 *   - All calls on one device share the array: calls whose kernels may overlap on the GPU
 *     (different streams, no ordering between them) race on it.  Calls ordered on one stream
 *     are safe; nothing has to be cleared between them because every byte that is read was
 *     written earlier in the same call. */
size_t bma_mask_compile_static_limit(void);
int bma_mask_compile_static(const bma_mask_spec* spec, int32_t B, int32_t H,
                            const bma_block_lists* lists, bma_stream_t stream);

/* ---- mask programs: an arbitrary integer predicate of (b, h, q, k) evaluated on the device --------
 * Replaces the fancy_vmap evaluation of a Python mask_fn over index grids
 * (jaxmodules/attention.py:70-73, jaxmodules/vectorize.py:407-527) for predicates outside the
 * bma_mask_spec family.  A program is straight-line three-address code over 32-bit integers:
 * values 0..3 are b, h, q, k (global indices, offsets already added), instruction i defines value
 * 4+i, the last value is the predicate (non-zero = attend).  code[4*i..4*i+3] = {op, x, y, z}:
 *   CONST        value = x (immediate)
 *   unary        NEG ABS NOT(value == 0) INV(bitwise ~)                          operand value x
 *   binary       ADD SUB MUL FLOORDIV MOD (Python floor semantics; divisor 0 gives 0) MIN MAX
 *                LT LE GT GE EQ NE (0 / 1) AND OR XOR SHL SHR                    operand values x, y
 *   SELECT       value = x ? y : z
 *   LOAD1        value = tables[x][clamp(value y)]                               (z unused)
 *   LOAD2        value = tables[x][clamp(value y) * table_stride[x] + clamp(value z)]
 * Table reads clamp their indices into range, so no program can read outside its tables.
 * bma_mask_table_build evaluates the program for every (b, h, q, k) of the box and packs the
 * result along k into the bit table a bma_mask_spec takes (BMA_MASK_BITMAP: bit k%32 of word
 * k/32, [B, H, N, ceil(L/32)] int32, padding bits zero); B or H may be 1 when the program does
 * not read that index. */
enum {
  BMA_OP_CONST = 0, BMA_OP_NEG, BMA_OP_ABS, BMA_OP_NOT, BMA_OP_INV,
  BMA_OP_ADD, BMA_OP_SUB, BMA_OP_MUL, BMA_OP_FLOORDIV, BMA_OP_MOD, BMA_OP_MIN, BMA_OP_MAX,
  BMA_OP_LT, BMA_OP_LE, BMA_OP_GT, BMA_OP_GE, BMA_OP_EQ, BMA_OP_NE,
  BMA_OP_AND, BMA_OP_OR, BMA_OP_XOR, BMA_OP_SHL, BMA_OP_SHR,
  BMA_OP_SELECT, BMA_OP_LOAD1, BMA_OP_LOAD2, BMA_OP_COUNT
};
#define BMA_PROGRAM_MAX_INSTR 60
#define BMA_PROGRAM_MAX_TABLES 4

typedef struct bma_mask_program {
  int32_t n_instr;                                  /* 1 .. BMA_PROGRAM_MAX_INSTR */
  int32_t n_tables;                                 /* 0 .. BMA_PROGRAM_MAX_TABLES */
  int32_t code[4 * BMA_PROGRAM_MAX_INSTR];
  const int32_t* tables[BMA_PROGRAM_MAX_TABLES];    /* device pointers */
  int64_t table_rows[BMA_PROGRAM_MAX_TABLES];       /* LOAD2: rows; LOAD1: 1 */
  int64_t table_cols[BMA_PROGRAM_MAX_TABLES];       /* elements per row */
  int64_t table_stride[BMA_PROGRAM_MAX_TABLES];     /* elements between rows */
} bma_mask_program;

int bma_mask_table_build(const bma_mask_program* program, int32_t B, int32_t H, int32_t N, int32_t L,
                         int32_t q_offset, int32_t k_offset, int32_t* bits, bma_stream_t stream);

/* The same evaluation into the TILES form of the mask description: classifies every 128 x 128 tile of the
 * [B, H, N, L] box (global indices q + q_offset, k + k_offset must be tile-aligned: both offsets multiples of 128)
 * and stores the bits of the tiles that are cut.  tile_class / tile_slot: [B, H, ceil(N/128), ceil(L/128)];
 * tile_bits: room for `capacity` tiles of 4 KB (may be NULL with capacity 0 to count only); *counter (device int32,
 * zeroed by the caller) receives the number of cut tiles -- when it exceeds `capacity` the surplus tiles were not
 * stored and the call has to be repeated with more room.  Elements outside N x L count as not allowed in the bits
 * and are ignored by the class.  B or H may be 1 when the program does not read that index. */
int bma_mask_tiles_build(const bma_mask_program* program, int32_t B, int32_t H, int32_t N, int32_t L,
                         int32_t q_offset, int32_t k_offset, uint8_t* tile_class, int32_t* tile_slot,
                         uint32_t* tile_bits, int32_t capacity, int32_t* counter, bma_stream_t stream);

/* Which backend and tile sizes bma_attn_fwd (bma_attn_plan) and bma_attn_bwd
 * (bma_attn_bwd_plan) will use for these arguments; the block lists passed to each must be
 * compiled at exactly those block sizes.  (The reference has one block_size for both passes,
 * jaxmodules/attention.py:195-196, 280-281; results do not depend on it.) */
int bma_attn_plan(const bma_attn_args* args, int32_t* backend, int32_t* q_tile, int32_t* kv_tile);
int bma_attn_bwd_plan(const bma_attn_args* args, int32_t* backend, int32_t* q_tile, int32_t* kv_tile);

/* Forward: O = softmax_masked(Q K^T * scale) V and lse, visiting only listed blocks and
 * applying the element predicate only on partial ones.  Replaces the lax.map/lax.scan
 * nest of jaxmodules/attention.py:52-177, 219-241. */
int bma_attn_fwd(const bma_attn_args* args, const bma_mask_spec* spec,
                 const bma_block_lists* lists, bma_stream_t stream);

/* Backward preprocess: delta = rowsum(dO * O); when d_o_bf16 is non-NULL also writes a
 * bf16 copy of dO there (and takes delta from that rounded copy, the values the backward's
 * dO V^T product sees, so that dP - delta cancels exactly where it should) as a DENSE
 * [B, N, Hq, d] array (the caller allocates B*N*Hq*d bf16
 * elements and describes it to bma_attn_bwd with strides N*Hq*d, Hq*d, d -- whatever the
 * strides of args->o and args->d_o are).  The cotangent arrives in float32 because the
 * reference returns O in float32, jaxmodules/attention.py:173.  Part of what jax.vjp
 * derives at jaxmodules/attention.py:320-321. */
int bma_attn_bwd_preprocess(const bma_attn_args* args, void* d_o_bf16, bma_stream_t stream);

/* Scratch bytes bma_attn_bwd needs.  Currently 0 for every backend (all gradients are
 * accumulated on chip); the query stays so that a backend with scratch can be added. */
size_t bma_attn_bwd_workspace_bytes(const bma_attn_args* args);

/* Number of visited (full + partial) blocks per list head: visited[b' * lists->H + h'] = sum over the rows of
 * (kv_num + full_kv_num), int64 on the device, [lists->B * lists->H].  One small kernel; the caller copies the result
 * to the host once per mask and hands it to bma_attn_bwd_scratch_bytes / bma_attn_bwd, which size the backward
 * scratch by it.  No counterpart in the reference (its backward recomputes everything, jaxmodules/attention.py:266-342). */
int bma_block_lists_visited(const bma_block_lists* lists, int64_t* visited, bma_stream_t stream);

/* Optional scratch of bma_attn_bwd (0 when the backend has no use for it).  Given a workspace of
 * at least this size, the tensor-core backward hands every bf16 dS tile (32 KB per VISITED
 * 128x128 block; the slots are addressed compactly -- a prefix over the block lists, built into
 * the front of the workspace by three small launches per call) from the dK/dV kernel to the dQ
 * kernel through that buffer instead of recomputing S and dP there: 5 instead of 7 MMAs per
 * block, for 32 KB of HBM traffic each way.
 *   visited_host: HOST array [lists->B * lists->H] of visited-block counts per list head (from
 *     bma_block_lists_visited), or NULL; without it every size is the dense bound N/128 * L/128
 *     blocks per query head.
 * Only valid when the q-side and kv-side arrays of `lists` name the same blocks (they do when both
 * come from one bma_mask_compile call): a slot is read only if it was written during the same call,
 * and a block that only one side names is reported through the status word, never written.
 * A workspace that holds the tables plus at least the largest (batch, kv head) unit still takes this
 * path: the backward then runs as consecutive launches over ranges of units that reuse the slots.
 * With a smaller or NULL workspace the dQ kernel recomputes S and dP; results agree to the bf16
 * rounding of dS either way.  The workspace must be 256-byte aligned. */
size_t bma_attn_bwd_scratch_bytes(const bma_attn_args* args, const bma_block_lists* lists,
                                  const int64_t* visited_host);
/* The smallest workspace that still takes the hand-over path: the tables plus the largest unit. */
size_t bma_attn_bwd_scratch_min_bytes(const bma_attn_args* args, const bma_block_lists* lists,
                                      const int64_t* visited_host);

/* Backward: dQ, dK, dV from (Q, K, V, O, dO, lse, delta).  Replaces
 * _masked_attention_via_map_bwd, jaxmodules/attention.py:266-342.  `lists` must carry the
 * q-side arrays.  `workspace` must hold bma_attn_bwd_workspace_bytes(); one of
 * bma_attn_bwd_scratch_bytes() selects the hand-over variant described above (pass the same
 * visited_host).  mid_event: NULL, or a cudaEvent_t (created with timing enabled) that is recorded
 * on `stream` between the dK/dV pass and the dQ pass when the backward runs as one range, so that
 * the two kernels can be timed separately; ignored by the SIMT backend. */
int bma_attn_bwd(const bma_attn_args* args, const bma_mask_spec* spec,
                 const bma_block_lists* lists, void* workspace, size_t workspace_bytes,
                 const int64_t* visited_host, void* mid_event, bma_stream_t stream);

/* Self-test of the bounded waits (no counterpart in the reference): launches one CTA that waits on a
 * barrier nobody arrives at, gives up after limit_ns (at most 1e9) exactly like the waits inside the
 * attention kernels, records `code` (> 0) in the device status word and returns.  The context stays
 * usable; bma_device_status then returns BMA_ERR_DEVICE_CHECK with *detail == code. */
int bma_debug_expire_wait(uint64_t limit_ns, int32_t code, bma_stream_t stream);

/* Merge of two partial attention results over disjoint key sets (sequence-sharded
 * execution; no counterpart in the reference, which is single-device):
 *   lse = log(exp(lse_a) + exp(lse_b)),  o = exp(lse_a - lse) o_a + exp(lse_b - lse) o_b,
 * written in place into (o_a, lse_a).  o_* are float32 [B,N,Hq,d] described by args->o
 * (a) and args->d_o (b); lse_* by args->lse (a) and args->delta (b). */
int bma_attn_merge(const bma_attn_args* args, bma_stream_t stream);

/* Reads and clears the device-side status word that bounded waits / bounds checks write.
 * Synchronises `stream`.  Returns BMA_OK or BMA_ERR_DEVICE_CHECK; *detail gets the code. */
int bma_device_status(bma_stream_t stream, int32_t* detail);

#ifdef __cplusplus
}
#endif
#endif /* BMA_H_ */
