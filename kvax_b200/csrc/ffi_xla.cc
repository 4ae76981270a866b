// XLA FFI handlers over the C ABI of include/kvax_b200.h: what a JAX host binds in place of the
// `jt.triton_call(...)` custom calls of the reference (kvax/ops/mask_creator.py:280, 296 and
// kvax/ops/flash_attention_triton.py:1517, 1692, 1740, 1778, 1819).
//
// One handler per operation, exported as a C symbol with XLA_FFI_DEFINE_HANDLER_SYMBOL:
//   kvax_b200_ffi_mask_build      create_attention_mask: 4 int32 inputs -> 4 int32 arrays per mask (+ workspace)
//   kvax_b200_ffi_permute_tokens  chunk permutation of one array
//   kvax_b200_ffi_attn_fwd        forward: out, lse2 (+ workspace, status)
//   kvax_b200_ffi_attn_bwd        backward: dq, dk, dv (+ workspace, status)
// Conventions: XLA owns every buffer; scratch memory and the status word are extra *results* the Python
// side declares and drops (so the handlers allocate nothing and can run under XLA's command buffers);
// buffers are dense row-major in the public (batch, seq, heads, dim) layout, strides follow from
// `dimensions()`; tile sizes, flags and the scale are attributes; the handler runs on XLA's stream
// (`PlatformStream<cudaStream_t>`), only enqueues work and returns.  A rejected call becomes an
// `ffi::Error`; a device-side wait that gave up shows in the status result, never as a trap.
// Handlers keep no mutable global state, so XLA may call them from several threads.
//
// This file needs the XLA FFI headers (`xla/ffi/api/ffi.h`, shipped inside jaxlib:
// `jax.ffi.include_dir()`).  kvax_b200/build.py compiles it into libkvax_b200_xla_ffi.so only when
// that directory is given (XLA_FFI_INCLUDE_DIR) or jaxlib is importable; the image this repository is
// developed in has no jaxlib, so the file is written against the published API and has not been
// compiled here.  Python twin: kvax_b200/jax_binding/.
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/kvax_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error to_error(int rc, const char* what) {
  if (rc == KVAX_B200_OK) return ffi::Error::Success();
  const std::string msg = std::string(what) + ": " + kvax_b200_error_string(rc);
  if (rc == KVAX_B200_EINVAL || rc == KVAX_B200_EUNSUPPORTED) return ffi::Error::InvalidArgument(msg);
  return ffi::Error::Internal(msg);
}

// element strides (batch, seq, heads) of a dense (batch, seq, heads, dim) buffer
void dense_strides(ffi::Span<const int64_t> d, int64_t out[3]) {
  out[2] = d[3];
  out[1] = d[2] * d[3];
  out[0] = d[1] * d[2] * d[3];
}

kvax_b200_stream_t as_stream(cudaStream_t s) { return reinterpret_cast<kvax_b200_stream_t>(s); }

// ---------------------------------------------------------------------------------------------
// mask_build: up to three masks per call; masks beyond n_masks get zero-sized results on the Python side
// ---------------------------------------------------------------------------------------------
ffi::Error MaskBuild(cudaStream_t stream, ffi::Buffer<ffi::S32> q_pos, ffi::Buffer<ffi::S32> q_seg,
                     ffi::Buffer<ffi::S32> kv_pos, ffi::Buffer<ffi::S32> kv_seg,
                     ffi::ResultBuffer<ffi::S32> fwd_bounds,    // (4, B, 1, n_q_blocks): lower, upper, lower_full, upper_full
                     ffi::ResultBuffer<ffi::S32> dq_bounds,     // (4, B, 1, n) or zero-sized
                     ffi::ResultBuffer<ffi::S32> dkdv_bounds,   // (4, B, 1, n) or zero-sized
                     ffi::ResultBuffer<ffi::U8> workspace, int32_t fwd_q_block, int32_t fwd_kv_block,
                     int32_t bwd_q_block, int32_t bwd_kv_block, bool calc_bwd_mask, bool skip_pad_tokens) {
  const auto qd = q_pos.dimensions(), kd = kv_pos.dimensions();
  if (qd.size() != 2 || kd.size() != 2 || qd[0] != kd[0]) return ffi::Error::InvalidArgument("positions must be (batch, seq)");
  kvax_b200_mask_params p = {};
  p.q_positions = q_pos.typed_data();
  p.q_segment_ids = q_seg.typed_data();
  p.kv_positions = kv_pos.typed_data();
  p.kv_segment_ids = kv_seg.typed_data();
  p.batch = int32_t(qd[0]);
  p.q_len = int32_t(qd[1]);
  p.kv_len = int32_t(kd[1]);
  p.skip_pad_tokens = skip_pad_tokens ? 1 : 0;
  p.n_masks = calc_bwd_mask ? 3 : 1;
  auto fill = [&](int i, ffi::ResultBuffer<ffi::S32>& r, int32_t qb, int32_t kb, int32_t kv_outer) {
    const int64_t per = int64_t(r->element_count()) / 4;
    int32_t* base = r->typed_data();
    p.masks[i].q_block = qb;
    p.masks[i].kv_block = kb;
    p.masks[i].kv_outer = kv_outer;
    p.masks[i].lower = base;
    p.masks[i].upper = base + per;
    p.masks[i].lower_full = base + 2 * per;
    p.masks[i].upper_full = base + 3 * per;
  };
  fill(0, fwd_bounds, fwd_q_block, fwd_kv_block, 0);
  if (calc_bwd_mask) {
    fill(1, dq_bounds, bwd_kv_block, bwd_q_block, 0);      // dq mask: block sizes swapped (mask_creator.py:457-460)
    fill(2, dkdv_bounds, bwd_q_block, bwd_kv_block, 1);
  }
  if (workspace->size_bytes() < kvax_b200_mask_workspace_bytes(&p)) return ffi::Error::InvalidArgument("mask workspace too small");
  return to_error(kvax_b200_mask_build(&p, workspace->untyped_data(), workspace->size_bytes(), as_stream(stream)),
                  "kvax_b200_mask_build");
}

// ---------------------------------------------------------------------------------------------
// permute_tokens: (B, S, ...) any dtype
// ---------------------------------------------------------------------------------------------
ffi::Error PermuteTokens(cudaStream_t stream, ffi::AnyBuffer src, ffi::Result<ffi::AnyBuffer> dst, int32_t cp, bool reverse) {
  const auto d = src.dimensions();
  if (d.size() < 2) return ffi::Error::InvalidArgument("permute_tokens needs (batch, seq, ...)");
  const int64_t row_bytes = int64_t(src.size_bytes()) / (d[0] * d[1]);
  return to_error(kvax_b200_permute_tokens(src.untyped_data(), dst->untyped_data(), d[0], d[1], row_bytes, cp, reverse ? 1 : 0,
                                           as_stream(stream)),
                  "kvax_b200_permute_tokens");
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------
ffi::Error fill_shape(kvax_b200_attn_shape* s, const ffi::AnyBuffer& q, const ffi::AnyBuffer& k, const ffi::AnyBuffer& v,
                      ffi::Span<const int64_t> o_dims, const ffi::Buffer<ffi::S32>& q_pos, const ffi::Buffer<ffi::S32>& q_seg,
                      const ffi::Buffer<ffi::S32>& kv_pos, const ffi::Buffer<ffi::S32>& kv_seg, float scale, bool sequential,
                      int32_t off_first, int32_t off_second) {
  const auto qd = q.dimensions(), kd = k.dimensions(), vd = v.dimensions();
  if (qd.size() != 4 || kd.size() != 4 || vd.size() != 4) return ffi::Error::InvalidArgument("q, k, v must have rank 4");
  const bool f16 = q.element_type() == ffi::F16;
  if ((q.element_type() != ffi::BF16 && !f16) || k.element_type() != q.element_type() || v.element_type() != q.element_type())
    return ffi::Error::InvalidArgument("q, k, v must all be bf16 or all be fp16 (the Python side casts other dtypes)");
  s->batch = int32_t(qd[0]);
  s->q_len = int32_t(qd[1]);
  s->kv_len = int32_t(kd[1]);
  s->q_heads = int32_t(qd[2]);
  s->kv_heads = int32_t(kd[2]);
  s->head_dim = int32_t(qd[3]);
  s->dtype = f16 ? KVAX_B200_F16 : KVAX_B200_BF16;
  s->assume_sequential_positions = sequential ? 1 : 0;
  s->scale = scale;
  dense_strides(qd, s->q_strides);
  dense_strides(kd, s->k_strides);
  dense_strides(vd, s->v_strides);
  dense_strides(o_dims, s->o_strides);
  s->q_positions = q_pos.typed_data();
  s->q_segment_ids = q_seg.typed_data();
  s->kv_positions = kv_pos.typed_data();
  s->kv_segment_ids = kv_seg.typed_data();
  s->q_global_offset_first = off_first;
  s->q_global_offset_second = off_second;
  return ffi::Error::Success();
}

kvax_b200_block_mask block_mask(const ffi::Buffer<ffi::S32>& bounds, int32_t q_block, int32_t kv_block) {
  const int64_t per = int64_t(bounds.element_count()) / 4;
  const int32_t* base = bounds.typed_data();
  kvax_b200_block_mask m;
  m.lower = base;
  m.upper = base + per;
  m.lower_full = base + 2 * per;
  m.upper_full = base + 3 * per;
  m.q_block = q_block;
  m.kv_block = kv_block;
  return m;
}

ffi::Error AttnFwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::Buffer<ffi::S32> q_pos,
                   ffi::Buffer<ffi::S32> q_seg, ffi::Buffer<ffi::S32> kv_pos, ffi::Buffer<ffi::S32> kv_seg,
                   ffi::Buffer<ffi::S32> fwd_bounds,             // (4, B, 1, n_q_blocks) stacked forward mask
                   ffi::Result<ffi::AnyBuffer> out, ffi::ResultBuffer<ffi::F32> lse, ffi::ResultBuffer<ffi::U8> workspace,
                   ffi::ResultBuffer<ffi::S32> status, float scale, int32_t q_block, int32_t kv_block, bool sequential,
                   int32_t off_first, int32_t off_second) {
  kvax_b200_attn_fwd_params p = {};
  ffi::Error e = fill_shape(&p.shape, q, k, v, out->dimensions(), q_pos, q_seg, kv_pos, kv_seg, scale, sequential, off_first, off_second);
  if (e.failure()) return e;
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.mask = block_mask(fwd_bounds, q_block, kv_block);
  p.out = out->untyped_data();
  p.lse = lse->typed_data();
  p.status = status->typed_data();
  if (workspace->size_bytes() < kvax_b200_attn_fwd_workspace_bytes(&p)) return ffi::Error::InvalidArgument("forward workspace too small");
  cudaMemsetAsync(p.status, 0, sizeof(int32_t), stream);          // the status word must be 0 on entry
  return to_error(kvax_b200_attn_fwd(&p, workspace->untyped_data(), workspace->size_bytes(), as_stream(stream)), "kvax_b200_attn_fwd");
}

ffi::Error AttnBwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer out,
                   ffi::AnyBuffer dout, ffi::Buffer<ffi::F32> lse, ffi::Buffer<ffi::S32> q_pos, ffi::Buffer<ffi::S32> q_seg,
                   ffi::Buffer<ffi::S32> kv_pos, ffi::Buffer<ffi::S32> kv_seg, ffi::Buffer<ffi::S32> dq_bounds,
                   ffi::Buffer<ffi::S32> dkdv_bounds, ffi::Result<ffi::AnyBuffer> dq, ffi::ResultBuffer<ffi::F32> dk,
                   ffi::ResultBuffer<ffi::F32> dv, ffi::ResultBuffer<ffi::U8> workspace, ffi::ResultBuffer<ffi::S32> status,
                   float scale, int32_t q_block, int32_t kv_block, bool sequential, int32_t off_first, int32_t off_second,
                   bool two_kernel) {
  kvax_b200_attn_bwd_params p = {};
  ffi::Error e = fill_shape(&p.shape, q, k, v, out.dimensions(), q_pos, q_seg, kv_pos, kv_seg, scale, sequential, off_first, off_second);
  if (e.failure()) return e;
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.out = out.untyped_data();
  p.dout = dout.untyped_data();
  p.lse = lse.typed_data();
  p.mask_dq = block_mask(dq_bounds, kv_block, q_block);           // dq mask: block sizes swapped
  p.mask_dkdv = block_mask(dkdv_bounds, q_block, kv_block);
  p.dq = dq->untyped_data();
  p.dk = dk->typed_data();
  p.dv = dv->typed_data();
  p.status = status->typed_data();
  p.flags = two_kernel ? KVAX_B200_BWD_TWO_KERNEL : 0;
  dense_strides(dq->dimensions(), p.dq_strides);
  if (workspace->size_bytes() < kvax_b200_attn_bwd_workspace_bytes(&p)) return ffi::Error::InvalidArgument("backward workspace too small");
  cudaMemsetAsync(p.status, 0, sizeof(int32_t), stream);
  return to_error(kvax_b200_attn_bwd(&p, workspace->untyped_data(), workspace->size_bytes(), as_stream(stream)), "kvax_b200_attn_bwd");
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(kvax_b200_ffi_mask_build, MaskBuild,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::S32>>()      // query_positions
                                  .Arg<ffi::Buffer<ffi::S32>>()      // query_segment_ids
                                  .Arg<ffi::Buffer<ffi::S32>>()      // kv_positions
                                  .Arg<ffi::Buffer<ffi::S32>>()      // kv_segment_ids
                                  .Ret<ffi::Buffer<ffi::S32>>()      // forward mask, stacked
                                  .Ret<ffi::Buffer<ffi::S32>>()      // dq mask, stacked
                                  .Ret<ffi::Buffer<ffi::S32>>()      // dkdv mask, stacked
                                  .Ret<ffi::Buffer<ffi::U8>>()       // workspace
                                  .Attr<int32_t>("fwd_q_block")
                                  .Attr<int32_t>("fwd_kv_block")
                                  .Attr<int32_t>("bwd_q_block")
                                  .Attr<int32_t>("bwd_kv_block")
                                  .Attr<bool>("calc_bwd_mask")
                                  .Attr<bool>("skip_pad_tokens"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(kvax_b200_ffi_permute_tokens, PermuteTokens,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("cp")
                                  .Attr<bool>("reverse"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(kvax_b200_ffi_attn_fwd, AttnFwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()             // q (B, Sq, Hq, D) bf16
                                  .Arg<ffi::AnyBuffer>()             // k (B, Skv, Hkv, D)
                                  .Arg<ffi::AnyBuffer>()             // v
                                  .Arg<ffi::Buffer<ffi::S32>>()      // query_positions
                                  .Arg<ffi::Buffer<ffi::S32>>()      // query_segment_ids
                                  .Arg<ffi::Buffer<ffi::S32>>()      // kv_positions
                                  .Arg<ffi::Buffer<ffi::S32>>()      // kv_segment_ids
                                  .Arg<ffi::Buffer<ffi::S32>>()      // forward mask, stacked
                                  .Ret<ffi::AnyBuffer>()             // out
                                  .Ret<ffi::Buffer<ffi::F32>>()      // lse2 (B, Hq, Sq)
                                  .Ret<ffi::Buffer<ffi::U8>>()       // workspace
                                  .Ret<ffi::Buffer<ffi::S32>>()      // status (1,)
                                  .Attr<float>("scale")
                                  .Attr<int32_t>("q_block")
                                  .Attr<int32_t>("kv_block")
                                  .Attr<bool>("assume_sequential_positions")
                                  .Attr<int32_t>("q_global_offset_first")
                                  .Attr<int32_t>("q_global_offset_second"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(kvax_b200_ffi_attn_bwd, AttnBwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()             // q
                                  .Arg<ffi::AnyBuffer>()             // k
                                  .Arg<ffi::AnyBuffer>()             // v
                                  .Arg<ffi::AnyBuffer>()             // out
                                  .Arg<ffi::AnyBuffer>()             // dout
                                  .Arg<ffi::Buffer<ffi::F32>>()      // lse2
                                  .Arg<ffi::Buffer<ffi::S32>>()      // query_positions
                                  .Arg<ffi::Buffer<ffi::S32>>()      // query_segment_ids
                                  .Arg<ffi::Buffer<ffi::S32>>()      // kv_positions
                                  .Arg<ffi::Buffer<ffi::S32>>()      // kv_segment_ids
                                  .Arg<ffi::Buffer<ffi::S32>>()      // dq mask, stacked
                                  .Arg<ffi::Buffer<ffi::S32>>()      // dkdv mask, stacked
                                  .Ret<ffi::AnyBuffer>()             // dq
                                  .Ret<ffi::Buffer<ffi::F32>>()      // dk fp32
                                  .Ret<ffi::Buffer<ffi::F32>>()      // dv fp32
                                  .Ret<ffi::Buffer<ffi::U8>>()       // workspace
                                  .Ret<ffi::Buffer<ffi::S32>>()      // status (1,)
                                  .Attr<float>("scale")
                                  .Attr<int32_t>("q_block")
                                  .Attr<int32_t>("kv_block")
                                  .Attr<bool>("assume_sequential_positions")
                                  .Attr<int32_t>("q_global_offset_first")
                                  .Attr<int32_t>("q_global_offset_second")
                                  .Attr<bool>("two_kernel"));
