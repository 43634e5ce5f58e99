// C ABI of the library: argument validation, tensor-map construction, kernel dispatch.
// Host half of the reference's launchers _fwd_attention_kernel_call
// (jax_flash_attn2/flash_attention_triton/_forward_triton.py:462-592) and
// _bwd_attention_kernel_call (_backward_triton.py:948-1173); the shape and broadcast rules
// follow calc_bias_strides (flash_attention_triton/_utils.py:151-193).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/fa2_b200.h"
#include "../../include/fa2_b200_debug.h"
#include "bwd_launch.cuh"
#include "fwd_launch.cuh"
#include "launch_util.cuh"

namespace fa2 {
namespace {

thread_local char g_err[512] = "";
thread_local cudaEvent_t g_bwd_events[4] = {nullptr, nullptr, nullptr, nullptr};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

__device__ int g_status_word;   // set by kernels whose bounded wait ran out

int* status_ptr() {
  // Looked up per call: the address differs per device and the caller chooses the device.
  int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word) != cudaSuccess) return nullptr;
  return p;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// The kernels exist for head dims 64, 128 and 256 (1, 2 and 4 blocks of 64 columns). Any other
// head dim is cut into the same number of equal blocks of D / nblk columns, each padded with zeros
// to 64: the tensor maps below give the first dimension the extent D / nblk while the box stays 64
// wide, so the TMA unit zero-fills the padding on loads and clips it on stores. Every operand is
// cut the same way, so the dot products over the head dim are unchanged, and outputs leave through
// the same kind of map, which puts their columns back in place. The block stride must be a multiple
// of 16 bytes, hence D % 8 == 0 up to 64, D % 16 == 0 up to 128, D % 32 == 0 up to 256.
struct HeadDim {
  int padded;   // 64, 128 or 256: selects the kernel
  int nblk;     // padded / 64
  int blk;      // real columns per block (64 when the head dim is one the kernels are built for)
};
bool split_head_dim(int D, HeadDim* hd) {
  if (D <= 0 || D > 256) return false;
  hd->padded = D <= 64 ? 64 : D <= 128 ? 128 : 256;
  hd->nblk = hd->padded / 64;
  if (D % (8 * hd->nblk) != 0) return false;
  hd->blk = D / hd->nblk;
  return true;
}

// Tensor map of a [B, S, H, D] operand (any strides, unit head-dim stride) viewed as the 5-D
// tensor (D/nblk, S, nblk, H, B); one box is (64, rows, nblk, 1, 1) and lands in shared memory as
// nblk consecutive [rows][64] blocks with the 128-byte swizzle the MMA descriptors expect.
int make_tmap(CUtensorMap* tm, const void* ptr, bool bf16, int B, int S, int H, const HeadDim& hd,
              const fa2_strides& st, int box_rows, const char* what, int box_dblocks = 0) {
  if (box_dblocks == 0) box_dblocks = hd.nblk;   // default: the full head dim
  const int D = hd.blk * hd.nblk;
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(FA2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0)
    return fail(FA2_ERR_UNSUPPORTED, "%s: pointer must be 16-byte aligned", what);
  if ((st.b % 8) || (st.s % 8) || (st.h % 8))
    return fail(FA2_ERR_UNSUPPORTED, "%s: strides must be multiples of 8 elements", what);
  if (st.s <= 0 || (H > 1 && st.h <= 0) || (B > 1 && st.b <= 0))
    return fail(FA2_ERR_INVALID_ARG, "%s: strides must be positive", what);
  const cuuint64_t dims[5] = {static_cast<cuuint64_t>(hd.blk), static_cast<cuuint64_t>(S),
                              static_cast<cuuint64_t>(hd.nblk), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  // A dimension of extent 1 still needs a legal (multiple of 16 bytes) stride.
  const cuuint64_t sh = static_cast<cuuint64_t>(st.h > 0 ? st.h : D) * 2;
  const cuuint64_t sb = static_cast<cuuint64_t>(st.b > 0 ? st.b : static_cast<int64_t>(D)) * 2;
  const cuuint64_t strides[4] = {static_cast<cuuint64_t>(st.s) * 2,
                                 static_cast<cuuint64_t>(hd.blk) * 2, sh, sb};
  const cuuint32_t box[5] = {64, static_cast<cuuint32_t>(box_rows),
                             static_cast<cuuint32_t>(box_dblocks), 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r =
      enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
          const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FA2_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what,
                static_cast<int>(r));
  return FA2_OK;
}

int check_problem(const fa2_problem& p) {
  if (p.batch <= 0 || p.seqlen_q <= 0 || p.seqlen_k <= 0 || p.heads_q <= 0 || p.heads_kv <= 0)
    return fail(FA2_ERR_INVALID_ARG, "batch, sequence lengths and head counts must be positive");
  if (p.heads_q % p.heads_kv != 0)
    return fail(FA2_ERR_INVALID_ARG, "query heads (%d) must be divisible by key/value heads (%d)",
                p.heads_q, p.heads_kv);
  if (p.dtype != FA2_FP16 && p.dtype != FA2_BF16)
    return fail(FA2_ERR_UNSUPPORTED, "only fp16 and bf16 inputs are supported");
  HeadDim hd;
  if (!split_head_dim(p.head_dim, &hd))
    return fail(FA2_ERR_UNSUPPORTED,
                "head_dim %d is not supported (multiples of 8 up to 64, of 16 up to 128, of 32 up to 256 are)",
                p.head_dim);
  if (!(p.dropout_p >= 0.f) || !(p.dropout_p < 1.f))
    return fail(FA2_ERR_INVALID_ARG, "dropout_p must be in [0, 1)");
  if (!std::isfinite(p.softmax_scale))
    return fail(FA2_ERR_INVALID_ARG, "softmax_scale must be finite");
  if (p.dropout_p > 0.f && (p.heads_q_global < p.head_offset + p.heads_q || p.batch_offset < 0 ||
                            p.head_offset < 0))
    return fail(FA2_ERR_INVALID_ARG, "dropout offsets: head_offset + heads_q exceeds heads_q_global");
  // The kernels count work items and blocks in 32-bit integers (one item per 128 query rows and
  // query head at most, times up to 32 key splits): refuse what would not fit instead of wrapping.
  const long long q_tiles = (static_cast<long long>(p.seqlen_q) + 127) / 128;
  const long long k_tiles = (static_cast<long long>(p.seqlen_k) + 127) / 128;
  const long long bh = static_cast<long long>(p.batch) * p.heads_q;
  if (bh > INT_MAX || bh * q_tiles * 32 > INT_MAX || bh * k_tiles * 2 > INT_MAX ||
      bh * p.seqlen_q > INT_MAX)
    return fail(FA2_ERR_UNSUPPORTED,
                "problem too large: batch * heads_q * max(seqlen_q, 64 * ceil(seqlen / 128)) must stay below 2^31");
  return FA2_OK;
}

int make_score_term(ScoreTermDev* out, const fa2_score_term& t, const fa2_problem& p,
                    const char* what) {
  std::memset(out, 0, sizeof(*out));
  out->head_div = 1;
  if (!t.ptr) return FA2_OK;
  if (t.head_div < 0 || (t.head_div > 1 && p.heads_q % t.head_div != 0))
    return fail(FA2_ERR_INVALID_ARG, "%s: head_div must divide heads_q", what);
  out->head_div = t.head_div > 1 ? t.head_div : 1;
  if (t.dtype != p.dtype && t.dtype != FA2_FP32)
    return fail(FA2_ERR_UNSUPPORTED, "%s: dtype must be the q dtype or fp32", what);
  if (t.stride_b < 0 || t.stride_h < 0 || t.stride_q < 0)
    return fail(FA2_ERR_INVALID_ARG, "%s: strides must be non-negative", what);
  out->ptr = t.ptr;
  out->sb = t.stride_b;
  out->sh = t.stride_h;
  out->sq = t.stride_q;
  out->is_f32 = (t.dtype == FA2_FP32);
  const int vec = out->is_f32 ? 4 : 8;
  out->vec_ok = ((reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0) && (t.stride_b % vec == 0) &&
                (t.stride_h % vec == 0) && (t.stride_q % vec == 0);
  return FA2_OK;
}

// Tensor map of an additive score term for the kernels that stage it in shared memory: the 4-D
// tensor (Sk, Sq, heads, batch) of 16-bit elements, broadcast dimensions with extent 1, box
// (64 keys, box_rows query rows). Sets t->staged when the term qualifies: the q dtype, a real query
// dimension, 16-byte aligned base and strides (the TMA unit's rules). Otherwise the term stays on
// the direct-load path and the map is left untouched.
void try_stage_term(CUtensorMap* tm, ScoreTermDev* t, const fa2_problem& p, int box_rows) {
  t->staged = 0;
  if (!t->ptr || t->is_f32 || t->sq <= 0) return;
  if ((reinterpret_cast<uintptr_t>(t->ptr) & 15) || (t->sq % 8) || (t->sh % 8) || (t->sb % 8)) return;
  if (p.seqlen_k < 8) return;
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return;
  const cuuint64_t nh = t->sh ? static_cast<cuuint64_t>(p.heads_q / t->head_div) : 1;
  const cuuint64_t nb = t->sb ? static_cast<cuuint64_t>(p.batch) : 1;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(p.seqlen_k), static_cast<cuuint64_t>(p.seqlen_q), nh, nb};
  // a dimension of extent 1 still needs a legal stride: the natural one
  const cuuint64_t s_q = static_cast<cuuint64_t>(t->sq) * 2;
  const cuuint64_t s_h = t->sh ? static_cast<cuuint64_t>(t->sh) * 2 : s_q * dims[1];
  const cuuint64_t s_b = t->sb ? static_cast<cuuint64_t>(t->sb) * 2 : s_h * nh;
  const cuuint64_t strides[3] = {s_q, s_h, s_b};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r =
      enc(tm, p.dtype == FA2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
          const_cast<void*>(t->ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) t->staged = 1;
}

void make_dropout(DropoutDev* d, const fa2_problem& p) {
  std::memset(d, 0, sizeof(*d));
  d->enabled = p.dropout_p > 0.f;
  d->inv_keep = 1.f;
  if (!d->enabled) return;
  // 16-bit draws: the drop probability is realised in steps of 2^-16
  const double thr = std::floor(static_cast<double>(p.dropout_p) * 65536.0 + 0.5);
  d->threshold = thr >= 65535.0 ? 65535u : static_cast<uint32_t>(thr);
  d->inv_keep = static_cast<float>(1.0 / (1.0 - static_cast<double>(p.dropout_p)));
  d->seed_lo = static_cast<uint32_t>(p.dropout_seed & 0xffffffffu);
  d->seed_hi = static_cast<uint32_t>(p.dropout_seed >> 32);
  d->b_off = p.batch_offset;
  d->h_off = p.head_offset;
  d->hq_global = p.heads_q_global;
}

size_t dropout_bits_bytes(const fa2_problem& p) {
  if (!(p.dropout_p > 0.f)) return 0;
  const size_t nqt = (static_cast<size_t>(p.seqlen_q) + 127) / 128, nkt = (static_cast<size_t>(p.seqlen_k) + 127) / 128;
  return static_cast<size_t>(p.batch) * p.heads_q * nqt * nkt * 2048;
}

// The optional record of the keep bits (written by the forward, read by the backward).
int set_dropout_bits(DropoutDev* d, const fa2_problem& p, const uint32_t* bits, size_t bytes) {
  d->bits = nullptr;
  if (!bits || !d->enabled) return FA2_OK;
  if (reinterpret_cast<uintptr_t>(bits) & 15)
    return fail(FA2_ERR_INVALID_ARG, "dropout_bits must be 16-byte aligned");
  if (bytes < dropout_bits_bytes(p))
    return fail(FA2_ERR_INVALID_ARG, "dropout_bits must hold %zu bytes", dropout_bits_bytes(p));
  d->bits = const_cast<uint32_t*>(bits);
  d->bits_nqt = (p.seqlen_q + 127) / 128;
  d->bits_nkt = (p.seqlen_k + 127) / 128;
  return FA2_OK;
}

// The optional device-resident operands of the dropout stream (seed, shard offsets).
int set_dropout_operands(DropoutDev* d, const uint64_t* seed_dev, const int32_t* offsets_dev) {
  if (seed_dev && (reinterpret_cast<uintptr_t>(seed_dev) & 7))
    return fail(FA2_ERR_INVALID_ARG, "dropout_seed_dev must be 8-byte aligned");
  if (offsets_dev && (reinterpret_cast<uintptr_t>(offsets_dev) & 3))
    return fail(FA2_ERR_INVALID_ARG, "offsets_dev must be 4-byte aligned");
  d->seed_dev = reinterpret_cast<const unsigned long long*>(seed_dev);
  d->offsets_dev = offsets_dev;
  return FA2_OK;
}

// What the kernels need of a scratch pointer: 16-byte bulk copies and float4 accesses; 128 bytes is
// what allocators of every framework (XLA's sub-allocated temporaries included) guarantee.
constexpr uintptr_t kWorkspaceAlign = 128;

// Bytes of Q, dO and dq-accumulator tiles that one chunk of the backward's launch order may span.
// Measured on B=8, S=4096, Hq=32, Hkv=8, D=128 causal (16 MiB per group): main kernel 2.76 ms with
// chunks of 1 or 2 groups, 2.58-2.63 ms with 4, 8 or 16; only a few of a chunk's key tiles run at
// any time, so the live set stays well below this figure.
constexpr size_t kSchedL2Bytes = 128u << 20;

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct BwdWorkspace {
  size_t delta_off, dq_off, absmax_off, xstats_off, order_off, total;
  int sq_pad;
};
BwdWorkspace bwd_workspace(const fa2_problem& p) {
  BwdWorkspace w;
  w.sq_pad = (p.seqlen_q + 127) / 128 * 128;
  const size_t rows = static_cast<size_t>(p.batch) * p.heads_q * w.sq_pad;
  w.delta_off = 0;
  w.dq_off = align_up(2 * rows * sizeof(float), 256);   // (lse2, delta) per row
  HeadDim hd;
  split_head_dim(p.head_dim, &hd);   // checked by the callers
  w.absmax_off = w.dq_off + align_up(rows * hd.padded * sizeof(float), 256);
  w.xstats_off = w.absmax_off + 256;   // one word: max|dO| of the call (fp16 range guard)
  // the row statistics once more as MMA operand tiles, 4 KiB per 128 rows (head dim 128)
  const bool fold = hd.padded == 128;
  w.order_off = w.xstats_off + (fold ? rows / 128 * 4096 : 0);
  // counters for the bit-reproducible mode: one per 128-row dQ tile, at head dim 256 one per
  // 64 rows and half of the head dim
  w.total = w.order_off + align_up(rows / 128 * (hd.padded <= 128 ? 1 : 4) * sizeof(int), 256);
  return w;
}

// Split-KV plan of the forward: how many parts the key sequence is
// cut into and how many K/V tiles each part gets. A problem is split when its (query block,
// batch, head) items would leave more than half of the SMs idle and the key sequence is long
// enough to share out.
struct SplitPlan {
  int n_splits, split_tiles;
  int sq_k, hq_k;          // the problem as the kernel sees it (after packing grouped heads)
  size_t part_o_bytes, part_lse_off, total;
};
SplitPlan plan_splits(const fa2_problem& p, const HeadDim& hd, bool pack_heads) {
  SplitPlan s{};
  s.n_splits = 1;
  s.sq_k = pack_heads ? p.heads_q / p.heads_kv : p.seqlen_q;
  s.hq_k = pack_heads ? p.heads_kv : p.heads_q;
  const int n_tiles = (p.seqlen_k + 127) / 128;
  // work items: 256 query rows per item in the head dim <= 128 kernel, 128 in the head dim 256 one
  const int item_rows = hd.padded > 128 ? 128 : 256;
  const long long items = static_cast<long long>((s.sq_k + item_rows - 1) / item_rows) * p.batch * s.hq_k;
  const int sms = sm_count();
  if (n_tiles < 8 || items * 2 > sms) return s;
  int want = static_cast<int>(std::min<long long>(std::min<long long>(sms / items, n_tiles / 4), 32));
  if (want < 2) return s;
  s.split_tiles = (n_tiles + want - 1) / want;
  s.n_splits = (n_tiles + s.split_tiles - 1) / s.split_tiles;
  if (s.n_splits < 2) {
    s.n_splits = 1;
    return s;
  }
  const size_t rows = static_cast<size_t>(s.n_splits) * p.batch * s.sq_k * s.hq_k;
  s.part_o_bytes = align_up(rows * hd.padded * sizeof(float), 256);
  s.part_lse_off = s.part_o_bytes;
  const size_t sq_pad = static_cast<size_t>((s.sq_k + 127) / 128) * 128;
  s.total = s.part_lse_off + align_up(static_cast<size_t>(s.n_splits) * p.batch * s.hq_k * sq_pad * 4, 256);
  return s;
}

bool can_pack_heads(const fa2_problem& p) {
  const int group = p.heads_kv > 0 ? p.heads_q / p.heads_kv : 0;
  return p.seqlen_q == 1 && group > 1 && group <= 128 && !(p.dropout_p > 0.f);
}

}  // namespace
}  // namespace fa2

using namespace fa2;

extern "C" {

int fa2_version(void) { return FA2_ABI_VERSION; }

const char* fa2_last_error(void) { return g_err; }

int fa2_debug_device_status(void* cuda_stream) {
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int* dptr = status_ptr();
  if (!dptr) return fail(FA2_ERR_CUDA, "status word is not addressable");
  int v = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess ||
      cudaMemcpy(&v, dptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fail(FA2_ERR_CUDA, "reading the status word failed: %s",
                cudaGetErrorString(cudaGetLastError()));
  if (v != 0) cudaMemset(dptr, 0, sizeof(int));
  return v;
}

int fa2_debug_bwd_stage_events(void* const* events) {
  for (int i = 0; i < 4; ++i) g_bwd_events[i] = events ? static_cast<cudaEvent_t>(events[i]) : nullptr;
  return FA2_OK;
}

int fa2_fwd(const fa2_fwd_params* a, void* cuda_stream) {
  if (!a) return fail(FA2_ERR_INVALID_ARG, "params is null");
  const fa2_problem& p = a->p;
  int rc = check_problem(p);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->o || !a->lse)
    return fail(FA2_ERR_INVALID_ARG, "q, k, v, o and lse must be non-null");
  if (a->lse_stride_h < p.seqlen_q || a->lse_stride_b < 0)
    return fail(FA2_ERR_INVALID_ARG, "lse_stride_h must be at least seqlen_q");
  // First CUDA call of the entry point, on purpose a runtime call: it makes the device's primary
  // context current on a host thread that has not touched the runtime yet (a framework's worker
  // thread served from a memory cache), which the driver-level tensor-map encoder below needs.
  int* const status_word = status_ptr();
  if (!status_word) return fail(FA2_ERR_CUDA, "status word is not addressable");

  FwdLaunch L;
  std::memset(&L, 0, sizeof(L));
  const bool bf16 = p.dtype == FA2_BF16;
  HeadDim hd;
  split_head_dim(p.head_dim, &hd);
  const int D = hd.padded;
  // The problem as the kernel sees it. Decode shape (one query row per head, grouped heads,
  // nothing that depends on the (query, head) position): the G query heads of a key/value head
  // become G query rows of one head through the strides alone, so K and V are streamed once per
  // group instead of once per query head, by one CTA instead of G. A single row sees every key
  // whether the call is causal or not (bottom-right alignment).
  const int group = p.heads_q / p.heads_kv;
  const bool pack_heads = can_pack_heads(p) && !a->bias.ptr && !a->mask.ptr && !a->seqlens &&
                          a->q_strides.h > 0 && a->o_strides.h > 0;
  int sq_k = p.seqlen_q, hq_k = p.heads_q;
  fa2_strides q_st = a->q_strides, o_st = a->o_strides;
  long long lse_sh = a->lse_stride_h, lse_sq = 1;
  bool causal = p.causal != 0;
  if (pack_heads) {
    sq_k = group;
    hq_k = p.heads_kv;
    q_st.s = a->q_strides.h;  q_st.h = a->q_strides.h * group;
    o_st.s = a->o_strides.h;  o_st.h = a->o_strides.h * group;
    lse_sq = a->lse_stride_h; lse_sh = a->lse_stride_h * group;
    causal = false;
  }
  // Split-KV: the kernel writes per-split partial results into the workspace (as batch elements
  // split * B + b of a contiguous fp32 [n_splits * B, Sq, Hq, kernel head dim] output and its lse),
  // merged afterwards; o itself is written by the merge alone.
  SplitPlan sp = plan_splits(p, hd, pack_heads);
  if (sp.n_splits > 1 && (!a->workspace || a->workspace_bytes < sp.total ||
                          (reinterpret_cast<uintptr_t>(a->workspace) & (kWorkspaceAlign - 1))))
    sp.n_splits = 1;   // not enough scratch: run unsplit
  const bool split = sp.n_splits > 1;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  // head dim 256: K arrives in halves of the head dim, V in halves of the 128 key rows
  if ((rc = make_tmap(&L.tmQ, a->q, bf16, p.batch, sq_k, hq_k, hd, q_st, 128, "q")) ||
      (rc = make_tmap(&L.tmK, a->k, bf16, p.batch, p.seqlen_k, p.heads_kv, hd, a->k_strides, 128, "k",
                      D == 256 ? 4 / kKV256Parts : 0)) ||
      (rc = make_tmap(&L.tmV, a->v, bf16, p.batch, p.seqlen_k, p.heads_kv, hd, a->v_strides,
                      D == 256 ? 128 / kKV256Parts : 128, "v")) ||
      (rc = make_tmap(&L.tmO, a->o, bf16, p.batch, sq_k, hq_k, hd, o_st, 128, "o")) ||
      (rc = make_tmap(&L.tmO1, a->o, bf16, p.batch, sq_k, hq_k, hd, o_st, 128, "o", 1)))
    return rc;

  FwdKernelParams& kp = L.kp;
  kp.B = p.batch; kp.Sq = sq_k; kp.Sk = p.seqlen_k;
  kp.Hq = hq_k; kp.Hkv = p.heads_kv; kp.G = hq_k / p.heads_kv;
  kp.causal_off = p.seqlen_k - sq_k;
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.lse = a->lse; kp.lse_sb = a->lse_stride_b; kp.lse_sh = lse_sh; kp.lse_sq = lse_sq;
  kp.n_splits = 1;
  kp.split_tiles = 0;
  kp.part_o = nullptr;
  const int sq_pad = (sq_k + 127) / 128 * 128;
  if (split) {
    kp.n_splits = sp.n_splits;
    kp.split_tiles = sp.split_tiles;
    kp.part_o = reinterpret_cast<float*>(ws);
    kp.lse = reinterpret_cast<float*>(ws + sp.part_lse_off);
    kp.lse_sq = 1;
    kp.lse_sh = sq_pad;
    kp.lse_sb = static_cast<long long>(hq_k) * sq_pad;
  }
  if ((rc = make_score_term(&kp.bias, a->bias, p, "bias")) ||
      (rc = make_score_term(&kp.mask, a->mask, p, "mask")))
    return rc;
  make_dropout(&kp.drop, p);
  if (a->seqlens && p.seqlen_q != p.seqlen_k)
    return fail(FA2_ERR_INVALID_ARG, "seqlens requires seqlen_q == seqlen_k");
  if (a->seqlens && (reinterpret_cast<uintptr_t>(a->seqlens) & 3))
    return fail(FA2_ERR_INVALID_ARG, "seqlens must be 4-byte aligned");
  kp.seqlens = a->seqlens;
  if ((rc = set_dropout_operands(&kp.drop, a->dropout_seed_dev, a->offsets_dev))) return rc;
  // (grouped decode rows are only packed without dropout, so the record's row / head indices are
  // always those of the caller's problem)
  if ((rc = set_dropout_bits(&kp.drop, p, a->dropout_bits, a->dropout_bits_bytes))) return rc;
  kp.n_qblk = (sq_k + 255) / 256;
  kp.status = status_word;

  L.head_dim = D;
  L.bf16 = bf16;
  L.causal = causal;
  // The plain path assumes a positive scale (it takes the row maximum before scaling).
  L.feat = kp.bias.ptr || kp.mask.ptr || kp.drop.enabled || !(p.softmax_scale > 0.f);
  if (L.feat && D == 64) {
    // the head-dim-64 kernel streams 16-bit bias / mask tiles through shared memory
    try_stage_term(&L.tmBias, &kp.bias, p, 32);
    try_stage_term(&L.tmMask, &kp.mask, p, 32);
  }

  cudaError_t e = launch_fwd(L, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess)
    return fail(FA2_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(e));
  if (split) {
    FwdCombine c{};
    c.part_o = reinterpret_cast<const float*>(ws);
    c.part_lse = reinterpret_cast<const float*>(ws + sp.part_lse_off);
    c.o = a->o;
    c.o_strides[0] = o_st.b; c.o_strides[1] = o_st.s; c.o_strides[2] = o_st.h;
    c.lse = a->lse;
    c.lse_sb = a->lse_stride_b; c.lse_sh = lse_sh; c.lse_sq = lse_sq;
    c.n_splits = sp.n_splits; c.B = p.batch; c.Sq = sq_k; c.Hq = hq_k; c.D = p.head_dim;
    c.D_part = D;
    c.d_blk = hd.blk;
    c.sq_pad = sq_pad;
    c.bf16 = bf16;
    e = launch_fwd_combine(c, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess)
      return fail(FA2_ERR_CUDA, "split-KV merge launch failed: %s", cudaGetErrorString(e));
  }
  return FA2_OK;
}

size_t fa2_fwd_workspace_bytes(const fa2_problem* problem) {
  if (!problem || check_problem(*problem)) return 0;
  HeadDim hd;
  split_head_dim(problem->head_dim, &hd);
  // whether grouped heads get packed also depends on operands this function does not see
  // (bias, mask, lengths): report what the larger of the two plans needs
  size_t need = plan_splits(*problem, hd, false).total;
  if (can_pack_heads(*problem)) need = std::max(need, plan_splits(*problem, hd, true).total);
  return need;
}

size_t fa2_dropout_bits_bytes(const fa2_problem* problem) {
  if (!problem || check_problem(*problem)) return 0;
  return dropout_bits_bytes(*problem);
}

size_t fa2_bwd_workspace_bytes(const fa2_problem* problem) {
  if (!problem || check_problem(*problem)) return 0;
  return bwd_workspace(*problem).total;
}

int fa2_bwd(const fa2_bwd_params* a, void* cuda_stream) {
  if (!a) return fail(FA2_ERR_INVALID_ARG, "params is null");
  const fa2_problem& p = a->p;
  int rc = check_problem(p);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->o || !a->d_o || !a->lse || !a->dq || !a->dk || !a->dv)
    return fail(FA2_ERR_INVALID_ARG, "q, k, v, o, d_o, lse, dq, dk and dv must be non-null");
  if (a->lse_stride_h < p.seqlen_q || a->lse_stride_b < 0)
    return fail(FA2_ERR_INVALID_ARG, "lse_stride_h must be at least seqlen_q");
  const BwdWorkspace w = bwd_workspace(p);
  if (!a->workspace || a->workspace_bytes < w.total)
    return fail(FA2_ERR_WORKSPACE, "workspace must hold %zu bytes", w.total);
  if (reinterpret_cast<uintptr_t>(a->workspace) & (kWorkspaceAlign - 1))
    return fail(FA2_ERR_WORKSPACE, "workspace must be 128-byte aligned");
  if (a->dbias.ptr) {
    if (!a->bias.ptr) return fail(FA2_ERR_INVALID_ARG, "dbias is given but bias is not");
    if ((a->dbias.batch != 1 && a->dbias.batch != p.batch) ||
        (a->dbias.heads != 1 && a->dbias.heads != p.heads_kv && a->dbias.heads != p.heads_q))
      return fail(FA2_ERR_INVALID_ARG, "dbias: batch must be 1 or %d and heads 1, %d or %d", p.batch,
                  p.heads_kv, p.heads_q);
    if (reinterpret_cast<uintptr_t>(a->dbias.ptr) & 3)
      return fail(FA2_ERR_INVALID_ARG, "dbias must be 4-byte aligned");
  }

  // a runtime call before the driver-level tensor-map encoder: see fa2_fwd
  int* const status_word = status_ptr();
  if (!status_word) return fail(FA2_ERR_CUDA, "status word is not addressable");

  BwdLaunch L;
  std::memset(&L, 0, sizeof(L));
  const bool bf16 = p.dtype == FA2_BF16;
  HeadDim hd;
  split_head_dim(p.head_dim, &hd);
  const int D = hd.padded;
  // head dim 256: 64-row query tiles, and dk / dv leave in halves of the head dim
  const int q_rows = (D == 256) ? 64 : 128;
  const int dkv_blocks = (D == 256) ? 2 : D / 64;
  if ((rc = make_tmap(&L.tmQ, a->q, bf16, p.batch, p.seqlen_q, p.heads_q, hd, a->q_strides, q_rows, "q")) ||
      // head dim 256: K is loaded in halves of the head dim (two 64-column blocks per copy)
      (rc = make_tmap(&L.tmK, a->k, bf16, p.batch, p.seqlen_k, p.heads_kv, hd, a->k_strides, 128, "k",
                      D == 256 ? 2 : 0)) ||
      (rc = make_tmap(&L.tmV, a->v, bf16, p.batch, p.seqlen_k, p.heads_kv, hd, a->v_strides, 128, "v")) ||
      (rc = make_tmap(&L.tmdO, a->d_o, bf16, p.batch, p.seqlen_q, p.heads_q, hd, a->do_strides, q_rows, "d_o")) ||
      (rc = make_tmap(&L.tmdK, a->dk, bf16, p.batch, p.seqlen_k, p.heads_kv, hd, a->dk_strides, 128, "dk", dkv_blocks)) ||
      (rc = make_tmap(&L.tmdV, a->dv, bf16, p.batch, p.seqlen_k, p.heads_kv, hd, a->dv_strides, 128, "dv", dkv_blocks)))
    return rc;
  if ((a->o_strides.b % 8) || (a->o_strides.s % 8) || (a->o_strides.h % 8) ||
      (a->dq_strides.b % 8) || (a->dq_strides.s % 8) || (a->dq_strides.h % 8) ||
      (reinterpret_cast<uintptr_t>(a->o) & 15) || (reinterpret_cast<uintptr_t>(a->dq) & 15))
    return fail(FA2_ERR_UNSUPPORTED, "o / dq: 16-byte aligned pointers and strides in multiples of 8 are required");

  BwdKernelParams& kp = L.kp;
  kp.B = p.batch; kp.Sq = p.seqlen_q; kp.Sk = p.seqlen_k;
  kp.Hq = p.heads_q; kp.Hkv = p.heads_kv; kp.G = p.heads_q / p.heads_kv;
  kp.causal_off = p.seqlen_k - p.seqlen_q;
  kp.scale = p.softmax_scale;
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.lse = a->lse; kp.lse_sb = a->lse_stride_b; kp.lse_sh = a->lse_stride_h;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  kp.delta = reinterpret_cast<float*>(ws + w.delta_off);
  kp.dq_acc = reinterpret_cast<float*>(ws + w.dq_off);
  kp.Sq_pad = w.sq_pad;
  kp.do_absmax_bits = reinterpret_cast<const unsigned*>(ws + w.absmax_off);
  if ((rc = make_score_term(&kp.bias, a->bias, p, "bias")) ||
      (rc = make_score_term(&kp.mask, a->mask, p, "mask")))
    return rc;
  make_dropout(&kp.drop, p);
  if (a->seqlens && p.seqlen_q != p.seqlen_k)
    return fail(FA2_ERR_INVALID_ARG, "seqlens requires seqlen_q == seqlen_k");
  if (a->seqlens && (reinterpret_cast<uintptr_t>(a->seqlens) & 3))
    return fail(FA2_ERR_INVALID_ARG, "seqlens must be 4-byte aligned");
  kp.seqlens = a->seqlens;
  if ((rc = set_dropout_operands(&kp.drop, a->dropout_seed_dev, a->offsets_dev))) return rc;
  if ((rc = set_dropout_bits(&kp.drop, p, a->dropout_bits, a->dropout_bits_bytes))) return rc;
  kp.n_kvblk = (p.seqlen_k + 127) / 128;
  // Launch order (bwd_work_item): causal problems take as many (batch, kv head) groups per chunk as
  // keep a chunk's Q, dO and fp32 dq accumulator tiles within a share of L2; uniform problems keep
  // the group-after-group order.
  kp.sched_groups = 1;
  if (p.causal) {
    const size_t per_group = static_cast<size_t>(kp.G) * p.seqlen_q * D * (2 + 2 + 4);
    const size_t budget = kSchedL2Bytes;
    const long long groups = static_cast<long long>(p.batch) * p.heads_kv;
    kp.sched_groups = static_cast<int>(std::max<long long>(1, std::min<long long>(groups, budget / std::max<size_t>(per_group, 1))));
  }
  kp.status = status_word;

  L.head_dim = D;
  L.bf16 = bf16;
  L.causal = p.causal != 0;
  // (the plain head-dim-128 kernel divides the log-sum-exp by the scale once, in the pre-pass)
  L.feat = kp.bias.ptr || kp.mask.ptr || kp.drop.enabled || !(std::fabs(p.softmax_scale) >= 1e-30f);
  kp.xstats = (!L.feat && D == 128) ? reinterpret_cast<const uint4*>(ws + w.xstats_off) : nullptr;
  kp.dq_order = a->deterministic ? reinterpret_cast<int*>(ws + w.order_off) : nullptr;
  if (L.feat && D == 64) {
    // the head-dim-64 kernel brings 16-bit bias / mask tiles in through the TMA unit
    try_stage_term(&L.tmBias, &kp.bias, p, 128);
    try_stage_term(&L.tmMask, &kp.mask, p, 128);
  }
  if (a->dbias.ptr) {
    const long long plane = static_cast<long long>(p.seqlen_q) * p.seqlen_k;
    kp.dbias.ptr = a->dbias.ptr;
    kp.dbias.sh = a->dbias.heads == 1 ? 0 : plane;
    kp.dbias.sb = a->dbias.batch == 1 ? 0 : plane * a->dbias.heads;
    kp.dbias.head_div = a->dbias.heads == p.heads_q ? 1 : p.heads_q / p.heads_kv;
    // entries no step touches (above the causal diagonal, behind a batch element's length) stay 0
    const cudaError_t ez = cudaMemsetAsync(a->dbias.ptr, 0, sizeof(float) * plane * a->dbias.heads * a->dbias.batch,
                                           static_cast<cudaStream_t>(cuda_stream));
    if (ez != cudaSuccess)
      return fail(FA2_ERR_CUDA, "clearing dbias failed: %s", cudaGetErrorString(ez));
  }
  L.o = a->o; L.o_strides[0] = a->o_strides.b; L.o_strides[1] = a->o_strides.s; L.o_strides[2] = a->o_strides.h;
  L.d_o = a->d_o; L.do_strides[0] = a->do_strides.b; L.do_strides[1] = a->do_strides.s; L.do_strides[2] = a->do_strides.h;
  L.dq = a->dq; L.dq_strides[0] = a->dq_strides.b; L.dq_strides[1] = a->dq_strides.s; L.dq_strides[2] = a->dq_strides.h;
  L.delta = reinterpret_cast<float*>(ws + w.delta_off);
  L.dq_acc_bytes = w.absmax_off - w.dq_off;
  L.head_dim_real = p.head_dim;
  L.head_blk = hd.blk;

  for (int i = 0; i < 4; ++i) {
    L.stage_events[i] = g_bwd_events[i];
    g_bwd_events[i] = nullptr;   // armed for one call only
  }
  const cudaError_t e = launch_bwd(L, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess)
    return fail(FA2_ERR_CUDA, "backward launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward without a caller-provided workspace
// ---------------------------------------------------------------------------------------------
namespace {
// Scratch of the backward (row statistics + fp32 dq accumulator) for callers that cannot hand
// in device memory of their own. One array per GPU that loads the library, held until exit.
static __device__ __align__(256) unsigned char g_bwd_static_scratch[FA2_BWD_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of the array on the current device. In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so the address is looked up once per
// device (with that device current) and cached.
int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(FA2_ERR_CUDA, "cannot identify the current CUDA device");
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_bwd_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(FA2_ERR_CUDA, "cudaGetSymbolAddress failed for the static scratch: %s",
                  cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return FA2_OK;
}
}  // namespace

int fa2_bwd_static_scratch(const fa2_bwd_params* a, void* cuda_stream) {
  if (!a) return fail(FA2_ERR_INVALID_ARG, "params is null");
  const int rc = check_problem(a->p);
  if (rc) return rc;
  const size_t need = bwd_workspace(a->p).total;
  if (need > static_cast<size_t>(FA2_BWD_STATIC_SCRATCH_BYTES))
    return fail(FA2_ERR_WORKSPACE,
                "this problem needs %zu bytes of scratch; the built-in scratch holds %zu bytes "
                "(batch * heads_q * ceil(seqlen_q/128)*128 * (head_dim + 2) * 4 must not exceed it); "
                "use fa2_bwd with a workspace instead",
                need, static_cast<size_t>(FA2_BWD_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  const int rs = static_scratch_address(&scratch);
  if (rs) return rs;
  fa2_bwd_params b = *a;
  b.workspace = scratch;
  b.workspace_bytes = FA2_BWD_STATIC_SCRATCH_BYTES;
  return fa2_bwd(&b, cuda_stream);
}

}  // extern "C"
