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
// Operands an attention call does not have (bias, mask, seqlens, seed, offsets) are passed as
// one-element dummies, as the reference does (_forward_triton.py:551-554); a dummy is recognised by
// its element count or element type.
// Operand layout: q, o, d_o, dq [B, Sq, Hq, D]; k, v, dk, dv [B, Sk, Hkv, D]; bias
// [1|B, 1|Hkv|Hq, 1|Sq, Sk]; mask [1|B, 1|Hq, 1|Sq, Sk]; lse [B, Hq, ceil(Sq/128)*128] float32;
// seqlens [B] int32; seed uint32 [2] or one 64-bit integer; offsets int32 [2] = (batch offset, head
// offset) of this shard, a traced value under shard_map.
// Scratch results are declared kScratchSlack bytes larger than the library asks for and aligned up
// here, so the handlers do not depend on the alignment XLA gives a sub-allocated result.
#include <cstdint>
#include <string>

#include <cuda_runtime_api.h>

#include "fa2_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

constexpr size_t kScratchAlign = 128;   // what fa2_fwd / fa2_bwd require of a workspace pointer
constexpr size_t kScratchSlack = 128;   // extra bytes the JAX side declares for the alignment

// The first call refuses a core library whose structures have another layout than this file's.
bool AbiMatches() {
  static const bool ok = (fa2_version() / 1000 == FA2_ABI_VERSION / 1000) && fa2_version() >= FA2_ABI_VERSION;
  return ok;
}

struct Scratch {
  void* ptr;
  size_t bytes;
};
Scratch AlignedScratch(void* data, size_t total) {
  const uintptr_t raw = reinterpret_cast<uintptr_t>(data);
  const uintptr_t up = (raw + kScratchAlign - 1) / kScratchAlign * kScratchAlign;
  const size_t lost = static_cast<size_t>(up - raw);
  return {reinterpret_cast<void*>(up), total > lost ? total - lost : 0};
}

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
// rules of calc_bias_strides (flash_attention_triton/_utils.py:151-193). A term with heads_kv heads
// (1 < heads_kv < heads_q) is read by query head / group size instead of being repeated.
bool ScoreTerm(const ffi::AnyBuffer& x, int32_t heads_q, int32_t heads_kv, fa2_score_term* t) {
  *t = fa2_score_term{};
  if (x.element_count() <= 1) return true;   // dummy: absent
  const auto d = x.dimensions();
  if (d.size() != 4 || !DtypeOf(x, &t->dtype)) return false;
  t->ptr = x.untyped_data();
  t->head_div = (d[1] == heads_kv && d[1] != heads_q && d[1] != 1) ? heads_q / heads_kv : 1;
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

// Shard offsets as an operand: int32 [2]; anything else means "absent" (the attributes are used).
const int32_t* OffsetsOrNull(const ffi::AnyBuffer& x) {
  return (x.element_type() == ffi::DataType::S32 && x.element_count() == 2)
             ? static_cast<const int32_t*>(x.untyped_data())
             : nullptr;
}

ffi::Error Failed(const char* what) {
  return ffi::Error::InvalidArgument(std::string(what) + ": " + fa2_last_error());
}

ffi::Error FwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                   ffi::AnyBuffer bias, ffi::AnyBuffer mask, ffi::AnyBuffer seqlens, ffi::AnyBuffer seed,
                   ffi::AnyBuffer offsets, float softmax_scale, float dropout_p, bool causal,
                   int64_t dropout_seed, int32_t batch_offset, int32_t head_offset, int32_t heads_q_global,
                   ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::AnyBuffer> lse,
                   ffi::Result<ffi::AnyBuffer> dropout_bits, ffi::Result<ffi::AnyBuffer> workspace) {
  if (!AbiMatches()) return ffi::Error::InvalidArgument("fa2_b200_fwd: libfa2_b200.so has another ABI version");
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
  if (!ScoreTerm(bias, a.p.heads_q, a.p.heads_kv, &a.bias) || !ScoreTerm(mask, a.p.heads_q, a.p.heads_q, &a.mask))
    return ffi::Error::InvalidArgument("fa2_b200_fwd: bias / mask must be 4-D fp16, bf16 or fp32");
  a.seqlens = SeqlensOrNull(seqlens, a.p.batch);
  a.dropout_seed_dev = SeedOrNull(seed);
  a.offsets_dev = OffsetsOrNull(offsets);
  // record of the dropout keep bits for the backward: a uint32 result of
  // fa2_dropout_bits_bytes(problem) / 4 elements, or a one-element dummy when it is not wanted
  if (dropout_bits->element_type() == ffi::DataType::U32 && dropout_bits->element_count() > 1) {
    a.dropout_bits = static_cast<uint32_t*>(dropout_bits->untyped_data());
    a.dropout_bits_bytes = static_cast<size_t>(dropout_bits->element_count()) * 4;
  }
  // scratch for split-KV: a uint8 result of fa2_fwd_workspace_bytes(problem) + kScratchSlack bytes
  // (just the slack when the problem is not split); fa2_fwd ignores scratch that is too small
  const Scratch ws = AlignedScratch(workspace->untyped_data(), static_cast<size_t>(workspace->element_count()));
  a.workspace = ws.ptr;
  a.workspace_bytes = ws.bytes;
  if (fa2_fwd(&a, stream) != FA2_OK) return Failed("fa2_b200_fwd");
  return ffi::Error::Success();
}

ffi::Error BwdImpl(cudaStream_t stream, ffi::AnyBuffer d_o, ffi::AnyBuffer q, ffi::AnyBuffer k,
                   ffi::AnyBuffer v, ffi::AnyBuffer bias, ffi::AnyBuffer mask, ffi::AnyBuffer o,
                   ffi::AnyBuffer lse, ffi::AnyBuffer seqlens, ffi::AnyBuffer seed, ffi::AnyBuffer offsets,
                   ffi::AnyBuffer dropout_bits, float softmax_scale, float dropout_p, bool causal, int64_t dropout_seed,
                   int32_t batch_offset, int32_t head_offset, int32_t heads_q_global, bool deterministic,
                   ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> dk,
                   ffi::Result<ffi::AnyBuffer> dv, ffi::Result<ffi::AnyBuffer> dbias,
                   ffi::Result<ffi::AnyBuffer> workspace) {
  if (!AbiMatches()) return ffi::Error::InvalidArgument("fa2_b200_bwd: libfa2_b200.so has another ABI version");
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
  if (!ScoreTerm(bias, a.p.heads_q, a.p.heads_kv, &a.bias) || !ScoreTerm(mask, a.p.heads_q, a.p.heads_q, &a.mask))
    return ffi::Error::InvalidArgument("fa2_b200_bwd: bias / mask must be 4-D fp16, bf16 or fp32");
  // gradient of the bias: a float32 result of the bias's shape when it is wanted, a one-element
  // dummy otherwise
  if (dbias->element_count() > 1) {
    const auto bd = dbias->dimensions();
    if (bd.size() != 4 || dbias->element_type() != ffi::DataType::F32)
      return ffi::Error::InvalidArgument("fa2_b200_bwd: dbias must be a 4-D float32 result");
    a.dbias.ptr = static_cast<float*>(dbias->untyped_data());
    a.dbias.batch = static_cast<int32_t>(bd[0]);
    a.dbias.heads = static_cast<int32_t>(bd[1]);
  }
  a.dq = dq->untyped_data(); a.dq_strides = ContiguousBSHD(q);
  a.dk = dk->untyped_data(); a.dk_strides = ContiguousBSHD(k);
  a.dv = dv->untyped_data(); a.dv_strides = ContiguousBSHD(k);
  // the workspace is a uint8 result of fa2_bwd_workspace_bytes(problem) + kScratchSlack bytes, so
  // XLA allocates it
  const Scratch ws = AlignedScratch(workspace->untyped_data(), static_cast<size_t>(workspace->element_count()));
  a.workspace = ws.ptr;
  a.workspace_bytes = ws.bytes;
  a.seqlens = SeqlensOrNull(seqlens, a.p.batch);
  a.dropout_seed_dev = SeedOrNull(seed);
  a.offsets_dev = OffsetsOrNull(offsets);
  if (dropout_bits.element_type() == ffi::DataType::U32 && dropout_bits.element_count() > 1) {
    a.dropout_bits = static_cast<const uint32_t*>(dropout_bits.untyped_data());
    a.dropout_bits_bytes = static_cast<size_t>(dropout_bits.element_count()) * 4;
  }
  a.deterministic = deterministic ? 1 : 0;
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
        .Arg<ffi::AnyBuffer>()   // offsets: int32 [2] (batch offset, head offset) (or a dummy)
        .Attr<float>("softmax_scale")
        .Attr<float>("dropout_p")
        .Attr<bool>("causal")
        .Attr<int64_t>("dropout_seed")
        .Attr<int32_t>("batch_offset")
        .Attr<int32_t>("head_offset")
        .Attr<int32_t>("heads_q_global")
        .Ret<ffi::AnyBuffer>()    // o
        .Ret<ffi::AnyBuffer>()    // lse
        .Ret<ffi::AnyBuffer>()    // dropout bits: uint32 record for the backward (or a one-element dummy)
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
        .Arg<ffi::AnyBuffer>()   // offsets
        .Arg<ffi::AnyBuffer>()   // dropout bits written by the forward (or a one-element dummy)
        .Attr<float>("softmax_scale")
        .Attr<float>("dropout_p")
        .Attr<bool>("causal")
        .Attr<int64_t>("dropout_seed")
        .Attr<int32_t>("batch_offset")
        .Attr<int32_t>("head_offset")
        .Attr<int32_t>("heads_q_global")
        .Attr<bool>("deterministic")
        .Ret<ffi::AnyBuffer>()    // dq
        .Ret<ffi::AnyBuffer>()    // dk
        .Ret<ffi::AnyBuffer>()    // dv
        .Ret<ffi::AnyBuffer>()    // dbias: float32, the bias's shape (or a one-element dummy)
        .Ret<ffi::AnyBuffer>());  // workspace (uint8)
