// XLA FFI handlers that forward jax.Array buffers to the C ABI of libtops_b200.so
// (include/tops_b200.h).  One handler per entry point; each only fills the params struct from the
// buffers' shapes and pointers, takes its scratch from XLA's allocator and enqueues on XLA's stream.
//
// Built only where JAX is installed (pallas-kernel_b200/build.py --jax: compiled against
// jax.ffi.include_dir() and linked to libtops_b200.so); registered and wrapped in jax.custom_vjp by
// tops_b200/jax_ops.py.  Reference-side form this mirrors: the custom_vjp ops of
// tops/ops/simple_gla/chunk.py:778-827 and tops/ops/kda/chunk.py:193-255.
#include <cuda_runtime.h>

#include <cstdint>

#include "tops_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int dtype_code(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F32: return TOPS_F32;
    case ffi::DataType::BF16: return TOPS_BF16;
    case ffi::DataType::F16: return TOPS_F16;
    default: return -1;
  }
}

ffi::Error fail(int rc) { return ffi::Error::Internal(tops_b200_strerror(rc)); }

tops_chunk_problem problem(const ffi::AnyBuffer& q, const ffi::AnyBuffer& v, const ffi::AnyBuffer& g, int32_t chunk,
                           float scale) {
  const auto d = q.dimensions();   // [B,T,H,K]
  tops_chunk_problem pb = {};
  pb.B = (int32_t)d[0]; pb.T = (int32_t)d[1]; pb.H = (int32_t)d[2]; pb.K = (int32_t)d[3];
  pb.V = (int32_t)v.dimensions()[3];
  pb.chunk = chunk;
  pb.dtype = dtype_code(q.element_type());
  pb.gate_dtype = dtype_code(g.element_type());
  pb.gate_kind = g.dimensions().size() == 4 ? TOPS_GATE_PER_CHANNEL : TOPS_GATE_SCALAR;
  pb.impl = TOPS_IMPL_AUTO;
  pb.scale = scale;
  return pb;
}

// chunk_gla / chunk_simple_gla forward: (q, k, v, g, h0) -> (o, ht, saved)
// `saved` is the residual the backward takes back ([B,NT,H,K,V] in q's dtype).
ffi::Error ChunkFwd(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::AnyBuffer q, ffi::AnyBuffer k,
                    ffi::AnyBuffer v, ffi::AnyBuffer g, ffi::AnyBuffer h0, ffi::Result<ffi::AnyBuffer> o,
                    ffi::Result<ffi::AnyBuffer> ht, ffi::Result<ffi::AnyBuffer> saved, float scale, int32_t chunk) {
  tops_chunk_fwd_params p = {};
  p.pb = problem(q, v, g, chunk, scale);
  p.q = q.untyped_data(); p.k = k.untyped_data(); p.v = v.untyped_data(); p.g = g.untyped_data();
  p.h0 = reinterpret_cast<const float*>(h0.untyped_data());
  p.o = o->untyped_data();
  p.ht = reinterpret_cast<float*>(ht->untyped_data());
  if (tops_b200_chunk_selected_impl(&p.pb) == TOPS_IMPL_SM100) p.saved_out = saved->untyped_data();
  const size_t n = tops_b200_chunk_fwd_workspace_bytes(&p);
  auto ws = scratch.Allocate(n);
  if (!ws.has_value()) return ffi::Error::Internal("tops_b200: no scratch memory");
  const int rc = tops_b200_chunk_gla_fwd(&p, *ws, n, stream);
  return rc ? fail(rc) : ffi::Error::Success();
}

// backward: (q, k, v, g, h0, do, dht, saved) -> (dq, dk, dv, dg, dh0); cotangents in the primal dtypes
ffi::Error ChunkBwd(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::AnyBuffer q, ffi::AnyBuffer k,
                    ffi::AnyBuffer v, ffi::AnyBuffer g, ffi::AnyBuffer h0, ffi::AnyBuffer d_o, ffi::AnyBuffer dht,
                    ffi::AnyBuffer saved, ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> dk,
                    ffi::Result<ffi::AnyBuffer> dv, ffi::Result<ffi::AnyBuffer> dg, ffi::Result<ffi::AnyBuffer> dh0,
                    float scale, int32_t chunk) {
  tops_chunk_bwd_params p = {};
  p.pb = problem(q, v, g, chunk, scale);
  p.q = q.untyped_data(); p.k = k.untyped_data(); p.v = v.untyped_data(); p.g = g.untyped_data();
  p.h0 = reinterpret_cast<const float*>(h0.untyped_data());
  p.do_ = d_o.untyped_data();
  p.dht = reinterpret_cast<const float*>(dht.untyped_data());
  p.dq = dq->untyped_data(); p.dk = dk->untyped_data(); p.dv = dv->untyped_data(); p.dg = dg->untyped_data();
  p.dh0 = reinterpret_cast<float*>(dh0->untyped_data());
  p.grad_dtype = dtype_code(dq->element_type());
  p.dg_dtype = dtype_code(dg->element_type());
  if (tops_b200_chunk_selected_impl(&p.pb) == TOPS_IMPL_SM100) p.h_saved = saved.untyped_data();
  const size_t n = tops_b200_chunk_bwd_workspace_bytes(&p);
  auto ws = scratch.Allocate(n);
  if (!ws.has_value()) return ffi::Error::Internal("tops_b200: no scratch memory");
  const int rc = tops_b200_chunk_gla_bwd(&p, *ws, n, stream);
  return rc ? fail(rc) : ffi::Error::Success();
}

// one decode step (or a short token-serial pass): (q, k, v, gk, state) -> (o, state'); with the state
// operand aliased to the state result (input_output_aliases) the update is in place
ffi::Error RecurrentStep(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer gk,
                         ffi::AnyBuffer state, ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::AnyBuffer> state_out,
                         float scale) {
  tops_recurrent_fwd_params p = {};
  const auto d = q.dimensions();
  p.B = (int32_t)d[0]; p.T = (int32_t)d[1]; p.H = (int32_t)d[2]; p.K = (int32_t)d[3];
  p.V = (int32_t)v.dimensions()[3];
  p.dtype = dtype_code(q.element_type());
  p.gate_dtype = dtype_code(gk.element_type());
  p.o_dtype = dtype_code(o->element_type());
  p.scale = scale;
  p.q = q.untyped_data(); p.k = k.untyped_data(); p.v = v.untyped_data(); p.gk = gk.untyped_data();
  p.state_in = reinterpret_cast<const float*>(state.untyped_data());
  p.state_out = reinterpret_cast<float*>(state_out->untyped_data());
  p.o = o->untyped_data();
  p.N = p.B;
  const int rc = tops_b200_fused_recurrent_gla_fwd(&p, stream);
  return rc ? fail(rc) : ffi::Error::Success();
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    tops_b200_ffi_chunk_fwd, ChunkFwd,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Ctx<ffi::ScratchAllocator>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Attr<float>("scale").Attr<int32_t>("chunk"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    tops_b200_ffi_chunk_bwd, ChunkBwd,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Ctx<ffi::ScratchAllocator>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Attr<float>("scale").Attr<int32_t>("chunk"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    tops_b200_ffi_recurrent_step, RecurrentStep,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Attr<float>("scale"));
