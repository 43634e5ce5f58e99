// Pieces shared by the backward kernels of all head dims: bulk-copy wrappers, the fp16 cotangent
// scale, score-term loads and the pre-pass kernel.
#pragma once
#include <cuda_bf16.h>
#include "kernel_params.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

constexpr int kBM = 128;   // query rows per tile of the row statistics / dq accumulator
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxDynSmem = 232448;

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

// dst[0 .. bytes) += src[0 .. bytes) as float32, done by the TMA unit (asynchronous).
__device__ __forceinline__ void bulk_reduce_add_f32(float* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}

// Power of two that brings max|dO| to [1, 2): fp16 inputs only. With a loss like mean(out) the
// cotangent is ~1e-6 and dS = P (dP - delta) would sit in fp16's subnormal range; scaling dS by
// this factor (and dK, dQ back by its inverse) keeps the 16-bit operand of the dK / dQ MMAs in
// the normal range. Exact: powers of two do not round.
__device__ __forceinline__ float do_scale_from_bits(const unsigned* bits) {
  if (bits == nullptr) return 1.f;
  const float mx = __uint_as_float(__ldg(bits));
  if (!(mx > 0.f) || !(mx < INFINITY)) return 1.f;
  const int e = static_cast<int>(floorf(log2f(mx)));
  return exp2f(static_cast<float>(-max(-60, min(60, e))));
}

// Dropout keep bits of one key row (this thread) for kCols consecutive query columns, in the
// backward's transposed layout. One Philox call covers eight adjacent keys of one query
// (counter = (key/8, query, batch*Hq+head, 0); output word (key%8)/2 holds the 16-bit draws of an
// even key in its low half and of the next key in its high half), which suits the forward (one
// thread owns a query row) but would make every backward thread throw away seven of its eight
// draws. Instead the eight lanes that share key/8 each draw for a different query of a group of
// eight and exchange the resulting bits with warp votes. All 32 lanes must call this together;
// the key index of lane l must be a multiple of 8 plus (l % 8).
template <int kCols>
__device__ __forceinline__ void dropout_keep_bits_transposed(const DropoutDev& d, uint32_t bh_glob,
                                                             int kv, int q_first, int lane,
                                                             uint32_t (&bits)[kCols / 32]) {
  const int member = lane & 7;
  uint32_t key_lo, key_hi;
  dropout_key(d, key_lo, key_hi);
#pragma unroll
  for (int w = 0; w < kCols / 32; ++w) bits[w] = 0u;
#pragma unroll
  for (int m = 0; m < kCols / 8; ++m) {
    uint32_t rnd[4];
    philox4x32_10(static_cast<uint32_t>(kv >> 3), static_cast<uint32_t>(q_first + 8 * m + member),
                  bh_glob, 0u, key_lo, key_hi, rnd);
    // vote k: bit l says whether key (8*(l/8) + k) keeps query 8m + (l%8); this lane keeps the
    // vote about its own key
    uint32_t mine = 0u;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t draw = (k & 1) ? (rnd[k >> 1] >> 16) : (rnd[k >> 1] & 0xffffu);
      const uint32_t vote = __ballot_sync(0xffffffffu, draw >= d.threshold);
      if (member == k) mine = vote;
    }
    const uint32_t eight = (mine >> (lane & ~7)) & 0xffu;    // queries 8m .. 8m+7 for this key
    bits[(8 * m) >> 5] |= eight << ((8 * m) & 31);
  }
}

// x[c] += log2(e) * term[b, h, q_first + c, kv] for kCols consecutive queries of this thread's key
// row (x holds float bits). The loads of 16 columns are issued back to back, without branches in
// between, so that their latencies overlap; indices are clamped instead of predicated (entries
// outside the problem are masked or clipped later anyway).
template <bool kBf16, int kCols>
__device__ __forceinline__ void add_term_column(const ScoreTermDev& t, int b, int h, int q_first,
                                                int kv, int Sq, int Sk, uint32_t (&x)[kCols]) {
  if (t.ptr == nullptr) return;
  const long long base = static_cast<long long>(b) * t.sb + static_cast<long long>(h / t.head_div) * t.sh +
                         min(kv, Sk - 1);
  if (t.is_f32) {
    const float* ptr = static_cast<const float*>(t.ptr) + base;
#pragma unroll
    for (int c0 = 0; c0 < kCols; c0 += 16) {
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k)
        v[k] = __ldg(ptr + static_cast<long long>(min(q_first + c0 + k, Sq - 1)) * t.sq);
#pragma unroll
      for (int k = 0; k < 16; ++k)
        x[c0 + k] = __float_as_uint(fmaf(v[k], kLog2e, __uint_as_float(x[c0 + k])));
    }
  } else {
    const uint16_t* ptr = static_cast<const uint16_t*>(t.ptr) + base;
#pragma unroll
    for (int c0 = 0; c0 < kCols; c0 += 16) {
      uint16_t v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k)
        v[k] = __ldg(ptr + static_cast<long long>(min(q_first + c0 + k, Sq - 1)) * t.sq);
#pragma unroll
      for (int k = 0; k < 16; ++k)
        x[c0 + k] = __float_as_uint(fmaf(to_float16bit<kBf16>(v[k]), kLog2e, __uint_as_float(x[c0 + k])));
    }
  }
}

// Gradient of the bias: g[b, h / head_div, q_first + c, kv] += ds[c] / ds_scale for kCols
// consecutive queries of this thread's key row. `ds` holds the 16-bit pairs the thread has just
// stored as dS^T (queries c, c + 1 in the low and high half of word c / 2); ds_scale is the power
// of two fp16 problems multiply dS with. The threads of a warp own consecutive keys, so every
// atomic of the warp covers 128 contiguous bytes. Entries that are masked hold exact zeros and are
// skipped, which also keeps the causal upper triangle free of traffic.
template <bool kBf16, int kCols>
__device__ __forceinline__ void add_bias_grad(const ScoreGradDev& g, int b, int h, int q_first, int kv,
                                              int Sq, int Sk, const uint32_t* ds, float ds_scale) {
  if (kv >= Sk) return;
  float* row = g.ptr + static_cast<long long>(b) * g.sb + static_cast<long long>(h / g.head_div) * g.sh +
               static_cast<long long>(q_first) * Sk + kv;
  const float inv = 1.f / ds_scale;
#pragma unroll
  for (int c = 0; c < kCols; c += 2) {
    const float d0 = unpack_lo<kBf16>(ds[c >> 1]) * inv, d1 = unpack_hi<kBf16>(ds[c >> 1]) * inv;
    if (q_first + c < Sq && d0 != 0.f) atomicAdd(row + static_cast<long long>(c) * Sk, d0);
    if (q_first + c + 1 < Sq && d1 != 0.f) atomicAdd(row + static_cast<long long>(c + 1) * Sk, d1);
  }
}


// ---------------------------------------------------------------------------------------------
// 1. pre-pass
// ---------------------------------------------------------------------------------------------
// stats layout: [B, Hq, nQ, 2, 128] float: (-lse * log2e | -inf for rows that take no gradient,
// delta). dq_acc layout: [B, Hq, nQ, D/4, 128, 4] float.
//
// xstats (optional, bf16 kernels without score terms): the same two statistics as operand tiles
// for the tensor cores, so that the main kernel adds them to its accumulators with one MMA k-step
// each instead of every thread loading all 128 of them from shared memory in every step (a
// broadcast load moves 4 bytes per shared-memory cycle: 4 KiB per step over the 8 warps, a fifth
// of the shared-memory cycles of a kernel that is bound by them). Per (batch, head, query tile)
// one [128 rows][16] bf16 tile in the unswizzled K-major core-matrix layout (row r: 16 bytes at
// (r / 8) * 256 + (r % 8) * 16 for columns 0-7, the same + 128 for columns 8-15). Row r holds
//   columns 0-2:  -lse / softmax_scale as a sum of three bf16 terms (24 mantissa bits),
//   columns 8-10: -delta, likewise,    all other columns: zero.
// Multiplied by a tile of ones in columns 0-2 (or 8-10) this adds -lse / scale to every S^T entry
// of the row's query (so P = exp2(scale * log2e * S')), or -delta to every dP^T entry.
__device__ __forceinline__ void split3_bf16(float x, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(h);
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
  hi = __bfloat16_as_ushort(h);
  mid = __bfloat16_as_ushort(m);
  lo = __bfloat16_as_ushort(l);
}

// Number of key tiles whose CTA has a step for the query tile of `tile_rows` rows with index i, in
// a batch element with sq_b query and sk_b key rows: the step rule of the main kernels (a CTA works
// iff its first key is below sk_b, from the first query tile that sees its first key under the
// causal limit). The contributing key tiles are 0 .. count - 1.
__device__ __forceinline__ int bwd_tile_contributors(bool causal, int i, int tile_rows, int sq_b, int sk_b,
                                                     int n_kvblk, int causal_off) {
  if (i >= (sq_b + tile_rows - 1) / tile_rows) return 0;
  const int n_live = min(n_kvblk, (sk_b + 127) / 128);
  if (!causal) return n_live;
  // key tile n takes part iff n * 128 - causal_off < (i + 1) * tile_rows
  const long long lim = static_cast<long long>(i + 1) * tile_rows + causal_off;
  if (lim <= 0) return 0;
  return static_cast<int>(min(static_cast<long long>(n_live), (lim + 127) / 128));
}

// Bit-reproducible dq: waits (bounded, like the mbarrier waits) until `*counter == want`, i.e. until
// the key tiles that add before this one have added their part of the dQ tile.
__device__ __forceinline__ bool wait_for_turn(const int* counter, int want, volatile int* abort_flag) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    int seen;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (seen == want) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
    __nanosleep(100);
  }
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(128)
bwd_pre_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ d_o,
               long long o_sb, long long o_ss, long long o_sh, long long do_sb, long long do_ss,
               long long do_sh, const float* __restrict__ lse, long long lse_sb, long long lse_sh,
               float* __restrict__ stats, float* __restrict__ dq_acc, int Sq, int Hq, int nQ,
               unsigned* __restrict__ do_absmax_bits, int d_real,
               const int* __restrict__ seqlens, uint4* __restrict__ xstats, float inv_scale_log2,
               int* __restrict__ dq_order, int order_per_tile) {
  // one-dimensional grid (the y and z extents of a grid stop at 65535): tile index fastest
  const int i = blockIdx.x % nQ;
  const int bh = blockIdx.x / nQ;
  const int b = bh / Hq, h = bh - b * Hq;
  // rows past a batch element's own length take no gradient (and their dO is never read)
  const int sq_b = seqlens ? max(0, min(__ldg(seqlens + b), Sq)) : Sq;
  const int tid = threadIdx.x;
  constexpr int kLanesPerRow = D / 8;            // 16-byte loads
  constexpr int kRowsPerPass = 128 / kLanesPerRow;
  const int sub = tid % kLanesPerRow;
  const long long tile = (static_cast<long long>(bh) * nQ + i);
  float* st = stats + tile * 256;
  float amax = 0.f;
  for (int r0 = 0; r0 < kBM; r0 += kRowsPerPass) {
    const int r = r0 + tid / kLanesPerRow;
    const int row = i * kBM + r;
    float acc = 0.f;
    if (row < sq_b && 8 * sub < d_real) {   // d_real < D: the head dim is padded, rows are d_real wide
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + b * o_sb + row * o_ss + h * o_sh) + sub);
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(d_o + b * do_sb + row * do_ss + h * do_sh) + sub);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc = fmaf(to_float16bit<kBf16>(static_cast<uint16_t>(aw[k] & 0xffff)),
                   to_float16bit<kBf16>(static_cast<uint16_t>(gw[k] & 0xffff)), acc);
        acc = fmaf(to_float16bit<kBf16>(static_cast<uint16_t>(aw[k] >> 16)),
                   to_float16bit<kBf16>(static_cast<uint16_t>(gw[k] >> 16)), acc);
        if constexpr (!kBf16) {
          const float g0 = fabsf(to_float16bit<kBf16>(static_cast<uint16_t>(gw[k] & 0xffff)));
          const float g1 = fabsf(to_float16bit<kBf16>(static_cast<uint16_t>(gw[k] >> 16)));
          if (g0 < INFINITY) amax = fmaxf(amax, g0);
          if (g1 < INFINITY) amax = fmaxf(amax, g1);
        }
      }
    }
#pragma unroll
    for (int off = kLanesPerRow / 2; off > 0; off >>= 1)
      acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sub == 0) {
      float l2 = -INFINITY;      // -lse*log2(e); -inf makes every weight of the row exp2(-inf) = 0
      if (row < sq_b) {
        const float l = lse[b * lse_sb + h * lse_sh + row];
        if (l > -INFINITY && l < INFINITY) l2 = -l * kLog2e;
      }
      st[r] = l2;
      st[128 + r] = (row < sq_b) ? acc : 0.f;
      if (xstats != nullptr) {
        // a row without gradient gets a finite, huge negative shift: exp2 of it is 0, and the
        // zero columns of the ones tile still multiply it to 0 rather than to NaN
        uint32_t lh, lm, ll, dh, dm, dl;
        split3_bf16(l2 > -INFINITY ? l2 * inv_scale_log2 : -1e30f, lh, lm, ll);
        split3_bf16((row < sq_b) ? -acc : 0.f, dh, dm, dl);
        uint4* xr = xstats + tile * 256 + (r >> 3) * 16 + (r & 7);
        xr[0] = make_uint4(lh | (lm << 16), ll, 0u, 0u);
        xr[8] = make_uint4(dh | (dm << 16), dl, 0u, 0u);
      }
    }
  }
  float4* acc4 = reinterpret_cast<float4*>(dq_acc + tile * (kBM * D));
  for (int k = tid; k < kBM * D / 4; k += 128) acc4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (dq_order != nullptr && tid < order_per_tile) dq_order[tile * order_per_tile + tid] = 0;
  if constexpr (!kBf16) {
    // block maximum of |dO| -> one atomic per block (non-negative floats order like their bits)
    __shared__ float warp_max[4];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31) == 0) warp_max[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0 && do_absmax_bits != nullptr)
      atomicMax(do_absmax_bits, __float_as_uint(fmaxf(fmaxf(warp_max[0], warp_max[1]),
                                                      fmaxf(warp_max[2], warp_max[3]))));
  }
}


}  // namespace fa2
