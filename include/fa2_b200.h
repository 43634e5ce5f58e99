/*
 * fa2_b200 — C ABI of the B200 (sm_100a) FlashAttention-2 kernels.
 *
 * This is the boundary an XLA FFI custom call (or any other host runtime) binds. It replaces
 * the two Triton launch sites of erfanzar/jax-flash-attn2:
 *   - forward : jax_flash_attn2/flash_attention_triton/_forward_triton.py:462-592
 *               (_fwd_attention_kernel_call -> triton_call(_attn_fwd))
 *   - backward: jax_flash_attn2/flash_attention_triton/_backward_triton.py:948-1173
 *               (_bwd_attention_kernel_call -> triton_call(_attn_bwd_preprocess), triton_call(_attn_bwd))
 *
 * Conventions
 *   - Every pointer is a device pointer owned by the caller. The library allocates nothing,
 *     frees nothing and keeps no pointer after a call returns. Its only device memory of its own
 *     is part of the library image: one status word and the fixed scratch array of
 *     fa2_bwd_static_scratch (see there).
 *   - Work is launched on the CUDA stream passed in (a cudaStream_t cast to void*); no call
 *     synchronises the host with the device.
 *   - Tensors are addressed by element strides, so [B,S,H,D] and [B,H,S,D] storage (and
 *     broadcast bias / mask dimensions, stride 0) need no copy. The head-dim stride must be 1.
 *   - Return value: 0 on success, a negative fa2_status otherwise. fa2_last_error() returns a
 *     thread-local message for the last failing call. Validation happens before any launch.
 *   - Two hooks for tests and measurements (device status word, per-kernel events of the backward)
 *     are declared apart, in fa2_b200_debug.h: no caller of the attention path needs them.
 */
#ifndef FA2_B200_H_
#define FA2_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FA2_OK = 0,
  FA2_ERR_INVALID_ARG = -1,   /* null pointer, bad shape, bad stride, bad dropout ...        */
  FA2_ERR_UNSUPPORTED = -2,   /* head dim / dtype / alignment outside what the kernels take  */
  FA2_ERR_CUDA = -3,          /* a CUDA runtime or driver call failed                        */
  FA2_ERR_WORKSPACE = -4      /* workspace pointer missing or too small                      */
} fa2_status;

typedef enum {
  FA2_FP16 = 0,               /* same numbering as dtype_index(), _utils.py:75-82            */
  FA2_BF16 = 1,
  FA2_FP32 = 2                /* accepted for bias / mask only                               */
} fa2_dtype;

/* Element strides of a 4-D operand, indexed as (batch, sequence, head, 1). */
typedef struct {
  int64_t b, s, h;
} fa2_strides;

/* Additive score term (bias or mask): x[b, h, i, j]; stride 0 broadcasts a dimension, the j
 * stride is 1. Same broadcasting rules as calc_bias_strides(), _utils.py:151-193. */
typedef struct {
  const void* ptr;            /* NULL = absent                                               */
  int32_t dtype;              /* fa2_dtype: the q/k/v dtype or FA2_FP32                      */
  /* Query head h reads head h / head_div of the term (0 and 1 both mean one term head per query
   * head). A bias with one head per key/value head passes heads_q / heads_kv here and is never
   * repeated in memory (the reference repeats it: flash_attention.py:161-164). */
  int32_t head_div;
  int64_t stride_b, stride_h, stride_q;
} fa2_score_term;

/* Optional gradient of the bias (no counterpart in the reference, which returns no bias cotangent:
 * flash_attention_triton/_flash_attention.py:88). Dense float32 [batch, heads, seqlen_q, seqlen_k]
 * with batch in {1, B} and heads in {1, heads_kv, heads_q}: the gradient of the scores, summed over
 * the batch elements / query heads that share a bias entry. The library zeroes it and then adds
 * into it, so its previous contents do not matter. */
typedef struct {
  float* ptr;                 /* NULL = not wanted                                           */
  int32_t batch, heads;
} fa2_score_grad;

typedef struct {
  /* head_dim: any multiple of 8 up to 64, of 16 up to 128, of 32 up to 256. Head dims other than
   * 64 / 128 / 256 run on the next larger kernel with zero-padded columns (the reference pads
   * them too: PADDED_HEADS, _forward_triton.py:337-346); nothing is copied. */
  int32_t batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim;
  int32_t dtype;              /* fa2_dtype of q, k, v, o, do, dq, dk, dv                     */
  int32_t causal;             /* bottom-right aligned when seqlen_q != seqlen_k              */
  float softmax_scale;        /* multiplies q.k ; callers default it to 1/sqrt(head_dim)     */
  float dropout_p;            /* probability of dropping an attention weight, [0, 1),
                                 realised in steps of 2^-16                                   */
  /* Philox-4x32-10 key. Counter (key_index / 8, query_index, batch * heads_q_global + head, 0);
   * output word (key_index % 8) / 2 carries the 16-bit draw of an even key in its low half and of
   * the following key in its high half; a weight is kept iff draw >= round(dropout_p * 65536). */
  uint64_t dropout_seed;
  /* A sharded caller passes the global position of its slice so that every shard draws the
   * dropout bits the unsharded call would draw. */
  int32_t batch_offset, head_offset, heads_q_global;
} fa2_problem;

/* Both parameter blocks end with `offsets_dev`: optional (NULL = absent) int32 [2] on the device,
 * (batch_offset, head_offset). When given it replaces the two fields of fa2_problem, so that a
 * caller whose position in the mesh is a traced value (jax.lax.axis_index under shard_map) passes
 * it as an operand instead of compiling one call per mesh position. */

typedef struct {
  fa2_problem p;
  const void* q; fa2_strides q_strides;       /* [B, Sq, Hq,  D] */
  const void* k; fa2_strides k_strides;       /* [B, Sk, Hkv, D] */
  const void* v; fa2_strides v_strides;       /* [B, Sk, Hkv, D] */
  void* o;       fa2_strides o_strides;       /* [B, Sq, Hq,  D] */
  float* lse;                                  /* [B, Hq, lse_stride_h >= Sq], natural log    */
  int64_t lse_stride_b, lse_stride_h;
  fa2_score_term bias;                         /* added to scale * q.k                        */
  fa2_score_term mask;                         /* added as well; 0 keeps, -inf / finfo.min drops */
  /* Optional (NULL = absent): int32 [batch] on the device. Batch element b is attended as if
   * seqlen_q = seqlen_k = seqlens[b] (its first seqlens[b] rows are the real tokens, the rest is
   * padding): keys past that length are not seen, key tiles past it are not visited, and output
   * rows past it are written as zeros (their lse as -inf). Requires seqlen_q == seqlen_k. This is
   * the reference's varlen mode for a [batch, seqlen] padding mask (_forward_triton.py:267-279,
   * 500-510) without its pack / unpack copies (_utils.py:196-294); values are clamped to
   * [0, seqlen_q]. */
  const int32_t* seqlens;
  /* Optional (NULL = absent): the 64-bit dropout seed at a device address (8-byte aligned). When
   * given, the kernels read the seed from there and p.dropout_seed is ignored, so a seed that only
   * exists on the device (the reference passes it as a traced operand,
   * flash_attention_triton/_flash_attention.py:91-92; _forward_triton.py:554) needs no host copy and
   * a new seed never changes the launch. */
  const uint64_t* dropout_seed_dev;
  /* Optional scratch for split-KV (NULL / 0 = none). A problem with too few (batch, head, query
   * tile) items to fill the GPU, typically a decode step, is cut along the key sequence into
   * several items whose partial results are merged by a second small kernel; that needs
   * fa2_fwd_workspace_bytes(&p) bytes of scratch (128-byte aligned; contents undefined before and
   * after the call). Without enough scratch the call runs unsplit: same result, fewer SMs busy. */
  void* workspace;
  size_t workspace_bytes;
  const int32_t* offsets_dev;
  /* Optional (NULL = absent) record of the dropout keep bits, written by the forward and read by
   * the backward so that the backward need not draw them again (fa2_dropout_bits_bytes(&p) bytes,
   * 16-byte aligned): uint32 [batch, heads_q, ceil(Sq/128), ceil(Sk/128), 4, 128]. For query tile
   * i, key tile n, word w and row r, bit p (p < 16) says "keep key 128 n + 32 w + 2 p", bit 16 + p
   * the same for key 128 n + 32 w + 2 p + 1, both for query row 128 i + r. Tiles no query row can
   * see (causal, per-batch lengths) are not written. The bits are those of the Philox stream
   * described above: the record is a cache, never a different mask. */
  uint32_t* dropout_bits;
  size_t dropout_bits_bytes;
} fa2_fwd_params;

typedef struct {
  fa2_problem p;
  const void* q;  fa2_strides q_strides;
  const void* k;  fa2_strides k_strides;
  const void* v;  fa2_strides v_strides;
  const void* o;  fa2_strides o_strides;
  const void* d_o; fa2_strides do_strides;    /* cotangent of o, [B, Sq, Hq, D]               */
  const float* lse; int64_t lse_stride_b, lse_stride_h;
  fa2_score_term bias;
  fa2_score_term mask;
  void* dq; fa2_strides dq_strides;           /* [B, Sq, Hq,  D] in the q dtype               */
  void* dk; fa2_strides dk_strides;           /* [B, Sk, Hkv, D], already summed over a group */
  void* dv; fa2_strides dv_strides;
  void* workspace;                             /* fa2_bwd_workspace_bytes() bytes, 128-aligned */
  size_t workspace_bytes;
  /* Optional per-batch lengths: the array that was given to the forward call.
   * Rows of dq, dk and dv past a batch element's length are written as zeros and its d_o rows
   * past it are never read (_backward_triton.py:973-1025, 1163-1171). */
  const int32_t* seqlens;
  const uint64_t* dropout_seed_dev;            /* optional device-resident seed, see above        */
  const int32_t* offsets_dev;
  fa2_score_grad dbias;                        /* optional gradient of `bias`                     */
  /* Optional: the record the forward call wrote (same problem, seed and offsets). Kernels that
   * have shared memory to stage it (head dim up to 64) read the keep bits from it; the others
   * ignore it and draw the bits again. */
  const uint32_t* dropout_bits;
  size_t dropout_bits_bytes;
  /* Non-zero: dq is bit-reproducible from call to call, as the reference's is (its dq program owns
   * a query tile and adds the key tiles in a loop, _backward_triton.py:438-516; here every key tile
   * adds its part to a float32 accumulator, by default in whatever order the tiles get there). The
   * key tiles then add their parts in descending order of their index, each waiting for the one
   * above it, and are launched in that order; the backward takes longer. dk, dv and the forward are
   * bit-reproducible either way. */
  int32_t deterministic;
} fa2_bwd_params;

/* Forward: o = softmax(scale q k^T + bias + mask [causal]) v with dropout on the weights, and
 * lse = log sum exp of the (pre-dropout) scores. Replaces _fwd_attention_kernel_call
 * (_forward_triton.py:462-592) and the kernel _attn_fwd (_forward_triton.py:213-459). */
int fa2_fwd(const fa2_fwd_params* params, void* cuda_stream);

/* Backward: dq, dk, dv from d_o, the saved o and lse. Replaces _bwd_attention_kernel_call
 * (_backward_triton.py:948-1173): the rowsum(o * d_o) pre-pass (_attn_bwd_preprocess, :79-147),
 * the main kernel (_attn_bwd, :712-945) and the per-group reduction of dk / dv (:1156-1161). */
int fa2_bwd(const fa2_bwd_params* params, void* cuda_stream);

/* Bytes of scratch with which fa2_fwd would split this problem along the key sequence; 0 when it
 * would not split it (most problems). Depends on the GPU the calling thread has current. No
 * counterpart in the reference, whose forward is one program per query tile
 * (_forward_triton.py:213-459). */
size_t fa2_fwd_workspace_bytes(const fa2_problem* problem);

/* Bytes of scratch the backward needs for this problem (fp32 dq accumulator and the row sums). */
size_t fa2_bwd_workspace_bytes(const fa2_problem* problem);

/* Bytes of the optional dropout-bit record of this problem (0 without dropout). No counterpart in
 * the reference, whose backward does not regenerate the mask at all (_backward_triton.py:187-188). */
size_t fa2_dropout_bits_bytes(const fa2_problem* problem);

/* Message of the last failing call on this thread ("" if none). */
const char* fa2_last_error(void);

/* ABI version of this header: major * 1000 + minor. A change to the layout or meaning of a
 * structure is a new major version; bindings compare fa2_version() with the FA2_ABI_VERSION they
 * were written against and refuse a library whose major version differs. */
#define FA2_ABI_VERSION 3000
int fa2_version(void);

/* Size of the scratch array built into the library for fa2_bwd_static_scratch (32 MiB). */
#define FA2_BWD_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

/* Backward for callers that cannot give the library a workspace. This entry point has no
 * counterpart in the reference (there XLA allocates every temporary of the Triton launches).
 *
 * Who needs it: code that runs where device memory must not be allocated or where no allocator
 * is reachable - a host function called from inside a running inference server whose memory
 * pool is owned by another component, a plugin interface that only forwards input and output
 * buffers, a real-time loop in which an allocation could stall. Such callers pass the same
 * inputs and outputs as for fa2_bwd and leave `workspace` / `workspace_bytes` unset (they are
 * ignored). The scratch (row statistics and the float32 dq accumulator) lives in an array that
 * is part of the library image: FA2_BWD_STATIC_SCRATCH_BYTES on every GPU that loads the
 * library, for as long as the process lives.
 *
 *  - Limit: fa2_bwd_workspace_bytes(problem) must not exceed FA2_BWD_STATIC_SCRATCH_BYTES,
 *    i.e. batch * heads_q * ceil(seqlen_q / 128) * 128 * (head_dim + 2) * 4 bytes <= 32 MiB
 *    with head_dim rounded up to 64, 128 or 256
 *    (for head_dim 128: 64512 query rows over all batches and heads). Larger problems are
 *    refused with FA2_ERR_WORKSPACE and a message; nothing is launched.
 *  - The call allocates and frees nothing (no cudaMalloc / cudaFree, no allocating library
 *    routine). The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and caches it; make that first call before
 *    starting any stream capture.
 *  - Every call on a device uses the same array. Its contents from the previous call are
 *    overwritten: the pre-pass rewrites the statistics and zeroes the accumulator before the main
 *    kernel adds to it. Two calls that overlap on the GPU (different streams, or the same call
 *    from two threads) race on the array and give wrong gradients: keep calls on one device in
 *    stream order. fa2_bwd with caller-owned workspaces has no such restriction. */
int fa2_bwd_static_scratch(const fa2_bwd_params* params, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* FA2_B200_H_ */
