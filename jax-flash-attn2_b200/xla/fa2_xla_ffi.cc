// XLA FFI handlers over the C ABI of libfa2_b200.so.
//
// They stand where the reference hands its Triton kernels to XLA through
// eformer.callib.triton_call (jax_flash_attn2/flash_attention_triton/_forward_triton.py:547-588 and
// _backward_triton.py:1049-1154): XLA owns every buffer, the handlers only unpack them into
// fa2_fwd_params / fa2_bwd_params and call fa2_fwd / fa2_bwd on XLA's stream.
//
// NOT COMPILED OR RUN WHERE THIS LIBRARY IS BUILT AND TESTED: the XLA FFI headers ship with jaxlib
// (jax.ffi.include_dir()), which is not installed there. Build, next to libfa2_b200.so:
//   g++ -std=c++17 -O2 -fPIC -shared fa2_xla_ffi.cc -o libfa2_b200_xla.so \
//       -I"$(python -c 'import jax.ffi; print(jax.ffi.include_dir())')" -I../../include \
//       -I/usr/local/cuda/include -L.. -lfa2_b200 -Wl,-rpath,'$ORIGIN/..'
//
// Operands an attention call does not have (bias, mask, seqlens) are passed as one-element dummies,
// as the reference does (_forward_triton.py:551-554); a dummy is recognised by element_count() <= 1.
// Operand layout: q, o, d_o, dq [B, Sq, Hq, D]; k, v, dk, dv [B, Sk, Hkv, D]; bias / mask
// [1|B, 1|Hq, 1|Sq, Sk]; lse [B, Hq, ceil(Sq/128)*128] float32; seqlens [B] int32.
#include <cstdint>
#include <string>

#include <cuda_runtime_api.h>

#include "fa2_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

fa2_strides ContiguousBSHD(const ffi::AnyBuffer& x) {
  const auto d = x.dimensions();
  return {static_cast<int64_t>(d[1] * d[2] * d[3]), static_cast<int64_t>(d[2] * d[3]),
          static_cast<int64_t>(d[3])};
}

bool DtypeOf(const ffi::AnyBuffer& x, int32_t* out) {
  switch (x.element_type()) {
    case ffi::DataType::F16: *out = FA2_FP16; return true;
    case ffi::DataType::BF16: *out = FA2_BF16; return true;
    case ffi::DataType::F32: *out = FA2_FP32; return true;
    default: return false;
  }
}

// Additive score term [1|B, 1|Hq, 1|Sq, Sk] (row-major): stride 0 on broadcast dimensions, the
// rules of calc_bias_strides (flash_attention_triton/_utils.py:151-193).
bool ScoreTerm(const ffi::AnyBuffer& x, fa2_score_term* t) {
  *t = fa2_score_term{};
  if (x.element_count() <= 1) return true;   // dummy: absent
  const auto d = x.dimensions();
  if (d.size() != 4 || !DtypeOf(x, &t->dtype)) return false;
  t->ptr = x.untyped_data();
  t->stride_q = d[2] == 1 ? 0 : d[3];
  t->stride_h = d[1] == 1 ? 0 : d[2] * d[3];
  t->stride_b = d[0] == 1 ? 0 : d[1] * d[2] * d[3];
  return true;
}

bool Problem(const ffi::AnyBuffer& q, const ffi::AnyBuffer& k, bool causal, float softmax_scale,
             float dropout_p, int64_t dropout_seed, int32_t batch_offset, int32_t head_offset,
             int32_t heads_q_global, fa2_problem* p) {
  const auto qd = q.dimensions();
  const auto kd = k.dimensions();
  if (qd.size() != 4 || kd.size() != 4) return false;
  *p = fa2_problem{};
  p->batch = static_cast<int32_t>(qd[0]);
  p->seqlen_q = static_cast<int32_t>(qd[1]);
  p->seqlen_k = static_cast<int32_t>(kd[1]);
  p->heads_q = static_cast<int32_t>(qd[2]);
  p->heads_kv = static_cast<int32_t>(kd[2]);
  p->head_dim = static_cast<int32_t>(qd[3]);
  if (!DtypeOf(q, &p->dtype)) return false;
  p->causal = causal ? 1 : 0;
  p->softmax_scale = softmax_scale;
  p->dropout_p = dropout_p;
  p->dropout_seed = static_cast<uint64_t>(dropout_seed);
  p->batch_offset = batch_offset;
  p->head_offset = head_offset;
  p->heads_q_global = heads_q_global > 0 ? heads_q_global : p->heads_q;
  return true;
}

// Per-batch lengths: an int32 [B] array; anything else (the caller's dummy is a one-element array
// of the q dtype) means "absent".
const int32_t* SeqlensOrNull(const ffi::AnyBuffer& x, int32_t batch) {
  if (x.element_type() != ffi::DataType::S32 || x.dimensions().size() != 1 ||
      x.dimensions()[0] != batch)
    return nullptr;
  return static_cast<const int32_t*>(x.untyped_data());
}

// Dropout seed as an operand: two uint32 words (low, high) or one 64-bit integer, read by the
// kernels on the device, so that a traced seed never re-specialises the call. Anything else (the
// caller's one-element dummy of the q dtype) means "absent": the dropout_seed attribute is used.
const uint64_t* SeedOrNull(const ffi::AnyBuffer& x) {
  const bool two_words = x.element_type() == ffi::DataType::U32 && x.element_count() == 2;
  const bool one_word = (x.element_type() == ffi::DataType::U64 || x.element_type() == ffi::DataType::S64) &&
                        x.element_count() == 1;
  return (two_words || one_word) ? static_cast<const uint64_t*>(x.untyped_data()) : nullptr;
}

ffi::Error Failed(const char* what) {
  return ffi::Error::InvalidArgument(std::string(what) + ": " + fa2_last_error());
}

ffi::Error FwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                   ffi::AnyBuffer bias, ffi::AnyBuffer mask, ffi::AnyBuffer seqlens, ffi::AnyBuffer seed,
                   float softmax_scale, float dropout_p, bool causal, int64_t dropout_seed,
                   int32_t batch_offset, int32_t head_offset, int32_t heads_q_global,
                   ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::AnyBuffer> lse,
                   ffi::Result<ffi::AnyBuffer> workspace) {
  fa2_fwd_params a = {};
  if (!Problem(q, k, causal, softmax_scale, dropout_p, dropout_seed, batch_offset, head_offset,
               heads_q_global, &a.p))
    return ffi::Error::InvalidArgument("fa2_b200_fwd: q and k must be 4-D fp16 / bf16 arrays");
  a.q = q.untyped_data(); a.q_strides = ContiguousBSHD(q);
  a.k = k.untyped_data(); a.k_strides = ContiguousBSHD(k);
  a.v = v.untyped_data(); a.v_strides = ContiguousBSHD(v);
  a.o = o->untyped_data(); a.o_strides = ContiguousBSHD(q);
  a.lse = static_cast<float*>(lse->untyped_data());
  a.lse_stride_h = lse->dimensions()[2];
  a.lse_stride_b = a.lse_stride_h * lse->dimensions()[1];
  if (!ScoreTerm(bias, &a.bias) || !ScoreTerm(mask, &a.mask))
    return ffi::Error::InvalidArgument("fa2_b200_fwd: bias / mask must be 4-D fp16, bf16 or fp32");
  a.seqlens = SeqlensOrNull(seqlens, a.p.batch);
  a.dropout_seed_dev = SeedOrNull(seed);
  // scratch for split-KV: a uint8 result of fa2_fwd_workspace_bytes(problem) bytes (one byte when
  // the problem is not split); fa2_fwd ignores scratch that is too small
  a.workspace = workspace->untyped_data();
  a.workspace_bytes = static_cast<size_t>(workspace->element_count());
  if (fa2_fwd(&a, stream) != FA2_OK) return Failed("fa2_b200_fwd");
  return ffi::Error::Success();
}

ffi::Error BwdImpl(cudaStream_t stream, ffi::AnyBuffer d_o, ffi::AnyBuffer q, ffi::AnyBuffer k,
                   ffi::AnyBuffer v, ffi::AnyBuffer bias, ffi::AnyBuffer mask, ffi::AnyBuffer o,
                   ffi::AnyBuffer lse, ffi::AnyBuffer seqlens, ffi::AnyBuffer seed, float softmax_scale,
                   float dropout_p,
                   bool causal, int64_t dropout_seed, int32_t batch_offset, int32_t head_offset,
                   int32_t heads_q_global, ffi::Result<ffi::AnyBuffer> dq,
                   ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv,
                   ffi::Result<ffi::AnyBuffer> workspace) {
  fa2_bwd_params a = {};
  if (!Problem(q, k, causal, softmax_scale, dropout_p, dropout_seed, batch_offset, head_offset,
               heads_q_global, &a.p))
    return ffi::Error::InvalidArgument("fa2_b200_bwd: q and k must be 4-D fp16 / bf16 arrays");
  a.q = q.untyped_data(); a.q_strides = ContiguousBSHD(q);
  a.k = k.untyped_data(); a.k_strides = ContiguousBSHD(k);
  a.v = v.untyped_data(); a.v_strides = ContiguousBSHD(v);
  a.o = o.untyped_data(); a.o_strides = ContiguousBSHD(q);
  a.d_o = d_o.untyped_data(); a.do_strides = ContiguousBSHD(q);
  a.lse = static_cast<const float*>(lse.untyped_data());
  a.lse_stride_h = lse.dimensions()[2];
  a.lse_stride_b = a.lse_stride_h * lse.dimensions()[1];
  if (!ScoreTerm(bias, &a.bias) || !ScoreTerm(mask, &a.mask))
    return ffi::Error::InvalidArgument("fa2_b200_bwd: bias / mask must be 4-D fp16, bf16 or fp32");
  a.dq = dq->untyped_data(); a.dq_strides = ContiguousBSHD(q);
  a.dk = dk->untyped_data(); a.dk_strides = ContiguousBSHD(k);
  a.dv = dv->untyped_data(); a.dv_strides = ContiguousBSHD(k);
  // the workspace is a uint8 result of fa2_bwd_workspace_bytes(problem) bytes, so XLA allocates it
  a.workspace = workspace->untyped_data();
  a.workspace_bytes = static_cast<size_t>(workspace->element_count());
  a.seqlens = SeqlensOrNull(seqlens, a.p.batch);
  a.dropout_seed_dev = SeedOrNull(seed);
  if (fa2_bwd(&a, stream) != FA2_OK) return Failed("fa2_b200_bwd");
  return ffi::Error::Success();
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fa2_b200_fwd, FwdImpl,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>()   // q
        .Arg<ffi::AnyBuffer>()   // k
        .Arg<ffi::AnyBuffer>()   // v
        .Arg<ffi::AnyBuffer>()   // bias   (or a one-element dummy)
        .Arg<ffi::AnyBuffer>()   // mask   (or a one-element dummy)
        .Arg<ffi::AnyBuffer>()   // seqlens int32 [B] (or a one-element dummy of another dtype)
        .Arg<ffi::AnyBuffer>()   // seed: uint32 [2] (low, high) or one 64-bit integer (or a dummy)
        .Attr<float>("softmax_scale")
        .Attr<float>("dropout_p")
        .Attr<bool>("causal")
        .Attr<int64_t>("dropout_seed")
        .Attr<int32_t>("batch_offset")
        .Attr<int32_t>("head_offset")
        .Attr<int32_t>("heads_q_global")
        .Ret<ffi::AnyBuffer>()    // o
        .Ret<ffi::AnyBuffer>()    // lse
        .Ret<ffi::AnyBuffer>());  // workspace (uint8)

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fa2_b200_bwd, BwdImpl,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>()   // d_o
        .Arg<ffi::AnyBuffer>()   // q
        .Arg<ffi::AnyBuffer>()   // k
        .Arg<ffi::AnyBuffer>()   // v
        .Arg<ffi::AnyBuffer>()   // bias
        .Arg<ffi::AnyBuffer>()   // mask
        .Arg<ffi::AnyBuffer>()   // o
        .Arg<ffi::AnyBuffer>()   // lse
        .Arg<ffi::AnyBuffer>()   // seqlens
        .Arg<ffi::AnyBuffer>()   // seed
        .Attr<float>("softmax_scale")
        .Attr<float>("dropout_p")
        .Attr<bool>("causal")
        .Attr<int64_t>("dropout_seed")
        .Attr<int32_t>("batch_offset")
        .Attr<int32_t>("head_offset")
        .Attr<int32_t>("heads_q_global")
        .Ret<ffi::AnyBuffer>()    // dq
        .Ret<ffi::AnyBuffer>()    // dk
        .Ret<ffi::AnyBuffer>()    // dv
        .Ret<ffi::AnyBuffer>());  // workspace (uint8)
