// XLA-FFI handlers over the C ABI of include/bma.h: the custom calls that jaxmodules_b200/jax_binding.py registers
// with jax.ffi and wraps in the jax.custom_vjp triple of the reference (jaxmodules/attention.py:180, 244-273, 345).
// No logic lives here: buffers and attributes are copied into the bma_* structs, the stream comes from the call
// frame, workspaces and the backward scratch are extra RESULT buffers (XLA plans them; nothing is allocated), and a
// non-zero status becomes an ffi::Error.
//
// NOT compiled or tested where this library is developed (no jax / XLA headers there); build.py compiles it only when
// jax.ffi.include_dir() exists:   g++ -shared -fPIC -std=c++17 -I$(python -c "import jax; print(jax.ffi.include_dir())")
//                                     -Iinclude bma_jax.cc -L.. -lbma -o libbma_jax.so
#include <cstdint>
#include <cstring>

#include <cuda_runtime_api.h>

#include "../../include/bma.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;
using I32 = ffi::Buffer<ffi::S32>;
using F32 = ffi::Buffer<ffi::F32>;

namespace {

ffi::Error Status(int rc, const char* what) {
  if (rc == BMA_OK) return ffi::Error::Success();
  return ffi::Error(rc < 0 ? ffi::ErrorCode::kInvalidArgument : ffi::ErrorCode::kInternal,
                    std::string(what) + ": " + bma_error_string(rc));
}

// [B, L, H, d] dense buffer -> bma_tensor
bma_tensor Tensor(void* ptr, ffi::Span<const int64_t> dims, ffi::DataType dt) {
  bma_tensor t{};
  t.ptr = ptr;
  t.stride_h = dims[3];
  t.stride_l = dims[2] * dims[3];
  t.stride_b = dims[1] * t.stride_l;
  t.dtype = dt == ffi::DataType::BF16 ? BMA_DTYPE_BF16 : BMA_DTYPE_F32;
  return t;
}

// mask attribute: the eleven leading int32 fields of bma_mask_spec in declaration order; seg: [B, L] ids or empty
bma_mask_spec Spec(ffi::Span<const int32_t> m, const I32& seg) {
  bma_mask_spec s{};
  std::memcpy(&s, m.begin(), sizeof(int32_t) * 11);
  if (s.flags & BMA_MASK_SEGMENT) {
    s.seg_q = s.seg_k = seg.typed_data();
    s.seg_q_stride = s.seg_k_stride = seg.dimensions()[1];
  }
  return s;
}

bma_attn_args Args(ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, float scale) {
  bma_attn_args a{};
  auto qd = q.dimensions(), kd = k.dimensions();
  a.B = (int32_t)qd[0]; a.N = (int32_t)qd[1]; a.Hq = (int32_t)qd[2]; a.d = (int32_t)qd[3];
  a.L = (int32_t)kd[1]; a.Hkv = (int32_t)kd[2];
  a.scale = scale;
  a.backend = BMA_BACKEND_AUTO;
  a.q = Tensor(q.untyped_data(), qd, q.element_type());
  a.k = Tensor(k.untyped_data(), kd, k.element_type());
  a.v = Tensor(v.untyped_data(), kd, v.element_type());
  return a;
}

// the eight BlockMask arrays, kv side then q side ([B', H', NQ] counts, [B', H', NQ, NKV] indices)
bma_block_lists Lists(int32_t tile, I32* n, I32* i, I32* fn, I32* fi, I32* qn, I32* qi, I32* fqn, I32* fqi) {
  bma_block_lists l{};
  auto d = i->dimensions();
  l.B = (int32_t)d[0]; l.H = (int32_t)d[1]; l.NQ = (int32_t)d[2]; l.NKV = (int32_t)d[3];
  l.q_block = l.kv_block = tile;
  l.kv_num = n->typed_data(); l.kv_idx = i->typed_data(); l.full_kv_num = fn->typed_data(); l.full_kv_idx = fi->typed_data();
  if (qn) { l.q_num = qn->typed_data(); l.q_idx = qi->typed_data(); l.full_q_num = fqn->typed_data(); l.full_q_idx = fqi->typed_data(); }
  return l;
}

ffi::Error MaskCompileImpl(cudaStream_t st, I32 seg, ffi::Result<I32> n, ffi::Result<I32> i, ffi::Result<I32> fn, ffi::Result<I32> fi,
                           ffi::Result<I32> qn, ffi::Result<I32> qi, ffi::Result<I32> fqn, ffi::Result<I32> fqi,
                           ffi::Result<ffi::Buffer<ffi::U8>> ws, ffi::Span<const int32_t> mask, int32_t B, int32_t H, int32_t tile) {
  bma_mask_spec s = Spec(mask, seg);
  bma_block_lists l = Lists(tile, &*n, &*i, &*fn, &*fi, &*qn, &*qi, &*fqn, &*fqi);
  return Status(bma_mask_compile(&s, B, H, &l, ws->typed_data(), ws->size_bytes(), st), "bma_mask_compile");
}

ffi::Error FwdImpl(cudaStream_t st, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, I32 seg, I32 n, I32 i, I32 fn, I32 fi,
                   ffi::Result<F32> o, ffi::Result<F32> lse, ffi::Span<const int32_t> mask, float scale, int32_t tile) {
  bma_attn_args a = Args(q, k, v, scale);
  a.o = Tensor(o->typed_data(), q.dimensions(), ffi::DataType::F32);   // float32 like the reference (jaxmodules/attention.py:173)
  a.lse = lse->typed_data();
  bma_mask_spec s = Spec(mask, seg);
  bma_block_lists l = Lists(tile, &n, &i, &fn, &fi, nullptr, nullptr, nullptr, nullptr);
  return Status(bma_attn_fwd(&a, &s, &l, st), "bma_attn_fwd");
}

ffi::Error BwdImpl(cudaStream_t st, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, F32 o, F32 lse, F32 d_o, I32 seg,
                   I32 n, I32 i, I32 fn, I32 fi, I32 qn, I32 qi, I32 fqn, I32 fqi,
                   ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv,
                   ffi::Result<F32> delta, ffi::Result<ffi::Buffer<ffi::BF16>> do16, ffi::Result<ffi::Buffer<ffi::U8>> scratch,
                   ffi::Span<const int32_t> mask, ffi::Span<const int64_t> visited, float scale, int32_t tile) {
  bma_attn_args a = Args(q, k, v, scale);
  a.o = Tensor(o.typed_data(), q.dimensions(), ffi::DataType::F32);
  a.lse = lse.typed_data();
  a.d_o = Tensor(d_o.typed_data(), q.dimensions(), ffi::DataType::F32);
  a.delta = delta->typed_data();
  if (int rc = bma_attn_bwd_preprocess(&a, do16->typed_data(), st)) return Status(rc, "bma_attn_bwd_preprocess");
  a.d_o = Tensor(do16->typed_data(), q.dimensions(), ffi::DataType::BF16);   // the dense bf16 copy the preprocess wrote
  a.dq = Tensor(dq->untyped_data(), q.dimensions(), q.element_type());
  a.dk = Tensor(dk->untyped_data(), k.dimensions(), k.element_type());
  a.dv = Tensor(dv->untyped_data(), k.dimensions(), k.element_type());
  bma_mask_spec s = Spec(mask, seg);
  bma_block_lists l = Lists(tile, &n, &i, &fn, &fi, &qn, &qi, &fqn, &fqi);
  const int64_t* counts = visited.size() ? visited.begin() : nullptr;   // host attribute: per-list-head visited blocks
  return Status(bma_attn_bwd(&a, &s, &l, scratch->typed_data(), scratch->size_bytes(), counts, nullptr, st), "bma_attn_bwd");
}

}  // namespace

#define STREAM .Ctx<ffi::PlatformStream<cudaStream_t>>()
XLA_FFI_DEFINE_HANDLER_SYMBOL(BmaMaskCompile, MaskCompileImpl,
    ffi::Ffi::Bind() STREAM.Arg<I32>().Ret<I32>().Ret<I32>().Ret<I32>().Ret<I32>().Ret<I32>().Ret<I32>().Ret<I32>().Ret<I32>()
        .Ret<ffi::Buffer<ffi::U8>>().Attr<ffi::Span<const int32_t>>("mask").Attr<int32_t>("B").Attr<int32_t>("H").Attr<int32_t>("tile"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(BmaAttnFwd, FwdImpl,
    ffi::Ffi::Bind() STREAM.Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>()
        .Ret<F32>().Ret<F32>().Attr<ffi::Span<const int32_t>>("mask").Attr<float>("scale").Attr<int32_t>("tile"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(BmaAttnBwd, BwdImpl,
    ffi::Ffi::Bind() STREAM.Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<F32>().Arg<F32>().Arg<F32>().Arg<I32>()
        .Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>().Arg<I32>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<F32>().Ret<ffi::Buffer<ffi::BF16>>().Ret<ffi::Buffer<ffi::U8>>()
        .Attr<ffi::Span<const int32_t>>("mask").Attr<ffi::Span<const int64_t>>("visited").Attr<float>("scale").Attr<int32_t>("tile"));
