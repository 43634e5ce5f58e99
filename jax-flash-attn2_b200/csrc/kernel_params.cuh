// Device-side parameter blocks shared by the host launcher and the kernels.
#pragma once
#include <cstdint>

namespace fa2 {

// Additive score term (bias or mask) as the kernels see it: element strides, j stride 1.
struct ScoreTermDev {
  const void* ptr;      // nullptr = absent
  long long sb, sh, sq;
  int is_f32;           // 1: float32 elements, 0: the 16-bit dtype of q
  int vec_ok;           // 1: rows can be read with 16-byte loads (pointer and strides aligned)
  int head_div;         // >= 1: query head h reads head h / head_div of the term
  int staged;           // 1: the kernel reads this term through its tensor map (TMA-staged tiles in
                        // shared memory) instead of with loads from ptr
};

// Gradient of the bias: float32 [batch, heads, Sq, Sk], added into with atomics (several batch
// elements / query heads may share an entry). sb / sh are 0 on broadcast dimensions.
struct ScoreGradDev {
  float* ptr;           // nullptr = not wanted
  long long sb, sh;
  int head_div;         // >= 1: query head h adds into head h / head_div
};

struct DropoutDev {
  uint32_t threshold;   // keep an element iff its 16-bit draw >= threshold (0 .. 65535)
  float inv_keep;       // 1 / (1 - p)
  uint32_t seed_lo, seed_hi;
  // optional: the 64-bit seed is read from this device address instead (a seed that only exists
  // on the device, e.g. a traced value of the calling framework)
  const unsigned long long* seed_dev;
  int b_off, h_off, hq_global;
  // optional: (batch offset, head offset) read from this device address instead of b_off / h_off
  const int* offsets_dev;
  // optional record of the keep bits: uint32 [B, Hq, bits_nqt, bits_nkt, 4, 128]; written by the
  // forward, read by the backward kernels that stage it
  uint32_t* bits;
  int bits_nqt, bits_nkt;
  int enabled;
};

// First word of the record's block for (batch b, head h, query tile qt, key tile kt).
__device__ __forceinline__ uint32_t* dropout_bits_block(const DropoutDev& d, int b, int h, int Hq, int qt, int kt) {
  return d.bits + (((static_cast<long long>(b) * Hq + h) * d.bits_nqt + qt) * d.bits_nkt + kt) * 512;
}

// The Philox key of a call: (low, high) half of the seed.
__device__ __forceinline__ void dropout_key(const DropoutDev& d, uint32_t& lo, uint32_t& hi) {
  lo = d.seed_lo;
  hi = d.seed_hi;
  if (d.seed_dev != nullptr) {
    const unsigned long long s = __ldg(d.seed_dev);
    lo = static_cast<uint32_t>(s);
    hi = static_cast<uint32_t>(s >> 32);
  }
}

// Index of (batch b, head h) of this call in the Philox counter: its position in the unsharded
// problem, so that every partitioning draws the same bits.
__device__ __forceinline__ uint32_t dropout_bh_index(const DropoutDev& d, int b, int h) {
  int b_off = d.b_off, h_off = d.h_off;
  if (d.offsets_dev != nullptr) {
    b_off = __ldg(d.offsets_dev);
    h_off = __ldg(d.offsets_dev + 1);
  }
  return static_cast<uint32_t>((b_off + b) * d.hq_global + h_off + h);
}

struct FwdKernelParams {
  int B, Sq, Sk, Hq, Hkv, G;
  int causal_off;       // Sk - Sq: query row i may see key j iff j <= i + causal_off
  float scale_log2;     // softmax_scale * log2(e)
  float* lse;
  long long lse_sb, lse_sh;
  long long lse_sq;     // stride between the lse entries of consecutive query rows (1, except when
                        // the rows of the problem the kernel sees are really query heads)
  ScoreTermDev bias, mask;
  DropoutDev drop;
  int n_qblk;           // number of 256-row query blocks
  // Optional per-batch lengths (Sq == Sk): batch element b is attended as if both sequences had
  // seqlens[b] rows; output rows at or beyond it are written as zeros.
  const int* seqlens;
  // Split-KV (low-occupancy problems): every work item is cut into n_splits items of
  // split_tiles K/V tiles each; split s writes its normalised partial output and its lse as
  // "batch element" s * B + b of the partial buffers that o / lse then point to.
  int n_splits;         // >= 1
  int split_tiles;
  // Split-KV only, else null: the partial outputs in fp32, contiguous
  // [n_splits * B][Sq][Hq][kernel head dim]; the 16-bit output is then written by the merge alone.
  float* part_o;
  int* status;          // device status word (bounded-wait time-outs)
};

struct BwdKernelParams;
// Which (batch * kv head) group and key tile block index `idx` works on. With causal masking a key
// tile's work shrinks with its index (tile 0 is seen by every query tile, the last one by a single
// one). Blocks are dispatched in index order as SMs become free, so the order decides how ragged the
// end of the launch is: group after group (every group's heavy tiles arrive late in its turn)
// leaves SMs idle at the end for about one heavy tile's duration (8 % of the headline launch), all
// tiles of all groups heaviest first balances best but makes every group's Q / dO tiles live in L2
// for the whole launch. Chunks of `sched_groups` groups, key-tile-major inside a chunk, keep the
// working set of a chunk in L2 and leave only the last chunk's tail.
// `descending`: the key tiles of a chunk come last tile first instead (the order in which the
// bit-reproducible mode adds them to dQ: a block then only ever waits for blocks launched before it).
__device__ __forceinline__ void bwd_work_item(int idx, int groups, int n_kvblk, int sched_groups, bool descending,
                                              int& bhk, int& n) {
  const int per_chunk = sched_groups * n_kvblk;
  const int chunk = idx / per_chunk;
  const int rem = idx - chunk * per_chunk;
  const int in_chunk = min(sched_groups, groups - chunk * sched_groups);   // the last chunk may be short
  n = rem / in_chunk;
  bhk = chunk * sched_groups + (rem - n * in_chunk);
  if (descending) n = n_kvblk - 1 - n;
}

struct BwdKernelParams {
  int B, Sq, Sk, Hq, Hkv, G;
  int causal_off;
  float scale;          // softmax_scale
  float scale_log2;     // softmax_scale * log2(e)
  const float* lse;     // natural log, [B, Hq, >= Sq]
  long long lse_sb, lse_sh;
  const float* delta;   // rowsum(o * do), [B, Hq, Sq_pad]
  // Row statistics as MMA operand tiles, or null: one [128 query rows][16] bf16 tile per (batch,
  // head, query tile) that a rank-3 MMA adds to S^T and dP^T (see bwd_pre_kernel)
  const uint4* xstats;
  float* dq_acc;        // fp32 [B, Hq, Sq_pad, D]
  int Sq_pad;           // Sq rounded up to 128
  ScoreTermDev bias, mask;
  DropoutDev drop;
  int n_kvblk;          // number of 128-row key blocks
  // Launch order of the (batch, kv head, key tile) work items: the (batch, kv head) groups are taken
  // `sched_groups` at a time, and inside such a chunk the key tiles of all its groups come
  // heaviest first (see bwd_work_item).
  int sched_groups;     // >= 1
  const int* seqlens;   // optional per-batch lengths (Sq == Sk), as in the forward
  // fp16 only: bit pattern of max|dO| over the whole call (written by the pre-pass); dS is
  // scaled by a power of two derived from it so that small cotangents do not underflow in fp16.
  const unsigned* do_absmax_bits;
  ScoreGradDev dbias;
  // Bit-reproducible dq, or null: dq_order[(b * Hq + h) * nQ + i] counts the key tiles that have
  // added their part of dQ tile i (zeroed by the pre-pass). Key tile n adds its part when the
  // tiles above it that contribute have, i.e. in descending order, and the launch order is
  // descending too, so that a block only waits for blocks with a lower index.
  int* dq_order;
  int* status;
};

}  // namespace fa2
