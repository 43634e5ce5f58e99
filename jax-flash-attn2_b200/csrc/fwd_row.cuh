// Per-row pieces of the forward kernels: one thread owns one query row (one tensor-memory lane).
// Shared by the two-tile kernel (head dim 64 / 128) and the one-tile kernel (head dim 256).
#pragma once
#include "kernel_params.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

constexpr int kBM = 128;            // rows of one query tile
constexpr int kBN = 128;            // keys per K/V tile
constexpr int kBlockBytes = kBM * 128;   // one [128 rows][64 elements] block of a swizzled tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // in log2 units: P stays below 2^8

// P of one K/V tile is handed to the MMA warp in two pieces of 64 keys (measured: four pieces
// are slower, and neither an FMA-pipe polynomial for part of the exponentials nor a strictly
// ordered hand-over between the pieces gains anything: the XU pipe is not what limits the kernel).
constexpr int kPSplit = 2;
constexpr int kPCols = kBN / kPSplit;   // keys per piece

template <bool kBf16>
__device__ __forceinline__ void add_score_term(float (&x)[kBN], const ScoreTermDev& t, int b,
                                               int h, int qi, int kv0, int Sk, float coef) {
  const long long base = static_cast<long long>(b) * t.sb + static_cast<long long>(h / t.head_div) * t.sh +
                         static_cast<long long>(qi) * t.sq + kv0;
  const bool full = (kv0 + kBN <= Sk);
  if (t.is_f32) {
    const float* p = static_cast<const float*>(t.ptr) + base;
    if (t.vec_ok && full) {
#pragma unroll
      for (int c4 = 0; c4 < kBN / 4; ++c4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p) + c4);
        x[4 * c4 + 0] = fmaf(v.x, coef, x[4 * c4 + 0]);
        x[4 * c4 + 1] = fmaf(v.y, coef, x[4 * c4 + 1]);
        x[4 * c4 + 2] = fmaf(v.z, coef, x[4 * c4 + 2]);
        x[4 * c4 + 3] = fmaf(v.w, coef, x[4 * c4 + 3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < kBN; ++c)
        if (kv0 + c < Sk) x[c] = fmaf(__ldg(p + c), coef, x[c]);
    }
  } else {
    const uint16_t* p = static_cast<const uint16_t*>(t.ptr) + base;
    if (t.vec_ok && full) {
#pragma unroll
      for (int c8 = 0; c8 < kBN / 8; ++c8) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + c8);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[8 * c8 + 2 * k + 0] =
              fmaf(to_float16bit<kBf16>(static_cast<uint16_t>(w[k] & 0xffff)), coef,
                   x[8 * c8 + 2 * k + 0]);
          x[8 * c8 + 2 * k + 1] = fmaf(to_float16bit<kBf16>(static_cast<uint16_t>(w[k] >> 16)),
                                       coef, x[8 * c8 + 2 * k + 1]);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < kBN; ++c)
        if (kv0 + c < Sk) x[c] = fmaf(to_float16bit<kBf16>(__ldg(p + c)), coef, x[c]);
    }
  }
}


// Where the score terms of a row come from. The default reads them straight from global memory; a
// kernel with shared memory to spare passes a provider that reads pieces staged by the TMA unit.
template <bool kBf16>
struct DirectTerms {
  const FwdKernelParams& p;
  int b, h, qi;
  float coef;   // what a term is multiplied with before it is added (see FeatScale)
  __device__ __forceinline__ void operator()(float (&x)[kBN], int kv0) const {
    if (qi < p.Sq) {
      if (p.bias.ptr) add_score_term<kBf16>(x, p.bias, b, h, qi, kv0, p.Sk, coef);
      if (p.mask.ptr) add_score_term<kBf16>(x, p.mask, b, h, qi, kv0, p.Sk, coef);
    }
  }
};

// Units of the score registers x[] in the kernels with score terms. The softmax computes
// exp2(x * sc - m * sc). With a positive softmax scale x holds the raw dot products, sc is
// scale * log2(e) as in the plain kernels, and a term enters as term / scale (coef = 1 / scale), so
// that no separate scaling pass over the 128 scores is needed. A zero or negative scale cannot be
// factored out of the row maximum: then x is first multiplied by scale * log2(e) (`prescale`),
// sc is 1 and a term enters as term * log2(e).
struct FeatScale {
  float sc, coef;
  bool prescale;
  __device__ __forceinline__ explicit FeatScale(float scale_log2) {
    prescale = !(scale_log2 > 0.f);
    sc = prescale ? 1.f : scale_log2;
    coef = prescale ? kLog2e : kLog2e / scale_log2;
  }
};
// Dropout keep bits of one query row for the 128 keys of one K/V tile. One Philox-4x32-10 call
// covers eight adjacent keys (counter = (key / 8, query row, batch * heads + head, 0); every 32-bit
// output word holds two 16-bit draws, the lower key in the low half; keep iff draw >= threshold).
// The sixteen calls are independent, so the softmax threads draw the bits of their NEXT tile right
// after handing P of the current one to the MMA warp: the scores' registers are free then, the
// calls interleave, and the work overlaps the tensor core instead of sitting between S and P.
// Layout of the result: word w covers keys [32 w, 32 w + 32) as sixteen pairs; bit p holds the flag
// of the even key 32 w + 2 p, bit 16 + p that of the odd key 32 w + 2 p + 1 (the two halves of the
// 16-bit pair P is packed into), which is what KeepBitsDropout needs to mask a pair in three
// integer instructions.
__device__ __forceinline__ uint4 draw_row_keep_bits(const DropoutDev& d, uint32_t key_lo, uint32_t key_hi,
                                                    uint32_t bh_glob, int qi, int kv0) {
  const uint32_t thr_hi = d.threshold << 16;    // draw in the high half >= threshold
  uint32_t w[4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t word = 0u;
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) {
      uint32_t rnd[4];
      philox4x32_10(static_cast<uint32_t>(kv0 >> 3) + 4 * wd + g4, static_cast<uint32_t>(qi), bh_glob, 0u,
                    key_lo, key_hi, rnd);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if ((rnd[k] & 0xffffu) >= d.threshold) word |= 1u << (4 * g4 + k);
        if (rnd[k] >= thr_hi) word |= 1u << (16 + 4 * g4 + k);
      }
    }
    w[wd] = word;
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Writes a row's keep bits of one (query tile, key tile) into the caller's record, from which the
// backward reads them instead of drawing them again: word w of row r at [w][r] of the tile's block.
__device__ __forceinline__ void store_row_keep_bits(const DropoutDev& d, const uint4& bits, int b, int h,
                                                    int Hq, int q_tile, int kv_tile, int r) {
  if (d.bits == nullptr) return;
  uint32_t* dst = dropout_bits_block(d, b, h, Hq, q_tile, kv_tile) + r;
  dst[0] = bits.x;
  dst[128] = bits.y;
  dst[256] = bits.z;
  dst[384] = bits.w;
}

// Zeroes the dropped weights of one piece (64 keys) of a row: `pk` holds the piece's P as 32 words
// of two 16-bit values (even key in the low half). Per pair: shift the pair's two flags to the
// sign bits of bytes 1 and 3, let a byte permute replicate them over the two halves, and mask.
struct KeepBitsDropout {
  bool enabled;
  uint4 bits;
  __device__ __forceinline__ void operator()(uint32_t (&pk)[kBN / 4], int half) const {
    if (!enabled) return;
    const uint32_t w0 = half == 0 ? bits.x : bits.z, w1 = half == 0 ? bits.y : bits.w;
#pragma unroll
    for (int pr = 0; pr < 16; ++pr) {
      uint32_t m0, m1;
      asm("prmt.b32 %0, %1, %1, 0xBB99;" : "=r"(m0) : "r"(w0 << (15 - pr)));
      asm("prmt.b32 %0, %1, %1, 0xBB99;" : "=r"(m1) : "r"(w1 << (15 - pr)));
      pk[pr] &= m0;
      pk[16 + pr] &= m1;
    }
  }
};

// One K/V tile of the online softmax for this thread's row:
//   S (tensor memory, 128 fp32 columns at tS) -> scores in the log2 domain (+ bias / mask),
//   causal / padding mask, running maximum with lazy rescaling of O (D columns at tO, only if
//   `have_o`), P = exp2(.) summed into l, dropout, P written back over S as 16-bit pairs.
// `before_o_rescale()` is called (by the whole warp) just before O is touched, so that a kernel
// whose P.V MMA may still be running can wait for it there.
// `after_half(h)` is called after piece h (keys [kPCols h, kPCols (h+1))) of P has been stored and
// fenced: the caller signals the MMA warp there.
// `terms(x, kv0)` adds coef * (bias + mask) to the scores (see FeatScale) and `dropout(pk, half)`
// zeroes the dropped weights of one packed piece (both only with kFeat; see DirectTerms /
// KeepBitsDropout).
template <int D, bool kBf16, bool kFeat, class BeforeRescale, class AfterHalf, class Terms, class Dropout>
__device__ __forceinline__ void softmax_tile_row(uint32_t tS, uint32_t tO, int j, bool have_o,
                                                 const FwdKernelParams& p, int row_lim, float sc,
                                                 bool prescale, float& m, float& l,
                                                 BeforeRescale before_o_rescale, AfterHalf after_half,
                                                 Terms terms, Dropout dropout) {
  tc_fence_after();
  float x[kBN];
  {
    uint32_t(&xr)[kBN] = reinterpret_cast<uint32_t(&)[kBN]>(x);
#pragma unroll
    for (int c = 0; c < kBN / 32; ++c)
      tmem_ld32(tS + c * 32, reinterpret_cast<uint32_t(&)[32]>(xr[c * 32]));
    tc_wait_ld();
  }
  const int kv0 = j * kBN;
  if constexpr (kFeat) {
    if (prescale) {
#pragma unroll
      for (int c = 0; c < kBN; ++c) x[c] *= p.scale_log2;
    }
    terms(x, kv0);
  }
  if (kv0 + kBN - 1 > row_lim) {   // boundary tile for this row: causal edge or key padding
#pragma unroll
    for (int c = 0; c < kBN; ++c)
      if (kv0 + c > row_lim) x[c] = -INFINITY;
  }
  float mx0 = fmaxf(x[0], x[1]), mx1 = fmaxf(x[2], x[3]), mx2 = fmaxf(x[4], x[5]),
        mx3 = fmaxf(x[6], x[7]);
#pragma unroll
  for (int c = 8; c < kBN; c += 8) {
    mx0 = max3(mx0, x[c], x[c + 1]);
    mx1 = max3(mx1, x[c + 2], x[c + 3]);
    mx2 = max3(mx2, x[c + 4], x[c + 5]);
    mx3 = max3(mx3, x[c + 6], x[c + 7]);
  }
  const float m_new = max3(m, fmaxf(mx0, mx1), fmaxf(mx2, mx3));
  // Lazy rescaling: keep the stale maximum while the true one is less than 2^8 above it.
  const bool resc = (m_new - m) * sc > kRescaleThreshold;
  if (__any_sync(0xffffffffu, resc)) {
    float alpha = 1.f;
    if (resc) {
      alpha = ex2_approx((m - m_new) * sc);
      m = m_new;
      l *= alpha;
    }
    if (have_o) {
      before_o_rescale();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tc_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
        tmem_st32(tO + c * 32, o);
      }
    }
  }
  const float m_use = (m == -INFINITY) ? 0.f : m;
  const float neg_ms = -m_use * sc;
  // P is produced and handed over in two halves of 64 keys: the P.V MMAs of the first half run
  // while the exponentials of the second half are still being computed.
  float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
  for (int half = 0; half < kPSplit; ++half) {
#pragma unroll
    for (int c = half * kPCols; c < (half + 1) * kPCols; c += 4) {
      fma2(x[c], x[c + 1], x[c], x[c + 1], sc, sc, neg_ms, neg_ms);
      fma2(x[c + 2], x[c + 3], x[c + 2], x[c + 3], sc, sc, neg_ms, neg_ms);
      x[c] = ex2_approx(x[c]);
      x[c + 1] = ex2_approx(x[c + 1]);
      x[c + 2] = ex2_approx(x[c + 2]);
      x[c + 3] = ex2_approx(x[c + 3]);
      add2(l0, l1, l0, l1, x[c], x[c + 1]);
      add2(l2, l3, l2, l3, x[c + 2], x[c + 3]);
    }
    uint32_t pk[kPCols / 2];
#pragma unroll
    for (int c = 0; c < kPCols / 2; ++c)
      pk[c] = pack2<kBf16>(x[half * kPCols + 2 * c], x[half * kPCols + 2 * c + 1]);
    if constexpr (kFeat) dropout(pk, half);
    static_assert(kPCols == 64, "one 32-column store per piece");
    tmem_st32(tS + 32 * half, reinterpret_cast<const uint32_t(&)[32]>(pk[0]));
    tc_wait_st();
    tc_fence_before();
    after_half(half);
  }
  l += (l0 + l1) + (l2 + l3);
}

// Split-KV: N scaled accumulator values of this thread's row go to the fp32 partial buffer.
template <int N>
__device__ __forceinline__ void store_partial_row(float* dst, const uint32_t (&o)[N], float inv) {
#pragma unroll
  for (int c = 0; c < N / 4; ++c)
    reinterpret_cast<float4*>(dst)[c] =
        make_float4(__uint_as_float(o[4 * c + 0]) * inv, __uint_as_float(o[4 * c + 1]) * inv,
                    __uint_as_float(o[4 * c + 2]) * inv, __uint_as_float(o[4 * c + 3]) * inv);
}
// Row `qi` of head `h`, "batch element" `b` (split * B + b) in the fp32 partial buffer.
template <int D>
__device__ __forceinline__ float* partial_row(const FwdKernelParams& p, int b, int h, int qi) {
  return p.part_o + ((static_cast<long long>(b) * p.Sq + qi) * p.Hq + h) * D;
}

// Final scaling of this thread's output row: O / l (and 1/(1-p)) -> 16 bit -> 128-byte-swizzled
// tile in shared memory at `so_gen` (D/64 blocks of [128][64]), or, for a split-KV part, in fp32
// straight to the partial buffer; stores the row's log-sum-exp.
template <int D, bool kBf16, bool kFeat>
__device__ __forceinline__ void epilogue_row(uint32_t tO, bool has_acc, uint8_t* so_gen, int r,
                                             const FwdKernelParams& p, int b, int h, int qi, float sc,
                                             float m, float l) {
  tc_fence_after();
  const float inv = (l > 0.f) ? (kFeat ? p.drop.inv_keep : 1.f) / l : 0.f;
  const float lse = (l > 0.f) ? (m * sc + lg2_approx(l)) * kLn2 : -INFINITY;
  if (qi < p.Sq)
    p.lse[static_cast<long long>(b) * p.lse_sb + static_cast<long long>(h) * p.lse_sh +
          static_cast<long long>(qi) * p.lse_sq] = lse;
  #pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t o[32];
    if (has_acc) {
      tmem_ld32(tO + c * 32, o);
      tc_wait_ld();
    } else {
#pragma unroll
      for (int k = 0; k < 32; ++k) o[k] = 0u;
    }
    if (p.part_o) {
      if (qi < p.Sq) store_partial_row(partial_row<D>(p, b, h, qi) + c * 32, o, inv);
      continue;
    }
    // 32 columns = 64 bytes = four 16-byte chunks of this row's 128-byte line
    uint8_t* line = so_gen + (c >> 1) * kBlockBytes + r * 128;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      uint4 v;
      v.x = pack2<kBf16>(__uint_as_float(o[8 * q4 + 0]) * inv, __uint_as_float(o[8 * q4 + 1]) * inv);
      v.y = pack2<kBf16>(__uint_as_float(o[8 * q4 + 2]) * inv, __uint_as_float(o[8 * q4 + 3]) * inv);
      v.z = pack2<kBf16>(__uint_as_float(o[8 * q4 + 4]) * inv, __uint_as_float(o[8 * q4 + 5]) * inv);
      v.w = pack2<kBf16>(__uint_as_float(o[8 * q4 + 6]) * inv, __uint_as_float(o[8 * q4 + 7]) * inv);
      const int chunk = (c & 1) * 4 + q4;
      *reinterpret_cast<uint4*>(line + ((chunk ^ (r & 7)) << 4)) = v;
    }
  }
  fence_proxy_async_smem();
}

// The same in pieces, for a kernel that stages one 64-column block at a time:
// epilogue_stats stores the log-sum-exp and returns the factor the O row is multiplied with;
// epilogue_block converts 64 accumulator values (two 32-column groups) and writes them as the
// row's 128-byte line of a swizzled [128][64] block.
template <bool kFeat>
__device__ __forceinline__ float epilogue_stats(const FwdKernelParams& p, int b, int h, int qi,
                                                float sc, float m, float l) {
  const float inv = (l > 0.f) ? (kFeat ? p.drop.inv_keep : 1.f) / l : 0.f;
  const float lse = (l > 0.f) ? (m * sc + lg2_approx(l)) * kLn2 : -INFINITY;
  if (qi < p.Sq)
    p.lse[static_cast<long long>(b) * p.lse_sb + static_cast<long long>(h) * p.lse_sh +
          static_cast<long long>(qi) * p.lse_sq] = lse;
  return inv;
}
template <bool kBf16>
__device__ __forceinline__ void epilogue_block(const uint32_t (&o64)[64], uint8_t* block_gen, int r,
                                               float inv) {
  uint8_t* line = block_gen + r * 128;
#pragma unroll
  for (int chunk = 0; chunk < 8; ++chunk) {
    uint4 v;
    v.x = pack2<kBf16>(__uint_as_float(o64[8 * chunk + 0]) * inv, __uint_as_float(o64[8 * chunk + 1]) * inv);
    v.y = pack2<kBf16>(__uint_as_float(o64[8 * chunk + 2]) * inv, __uint_as_float(o64[8 * chunk + 3]) * inv);
    v.z = pack2<kBf16>(__uint_as_float(o64[8 * chunk + 4]) * inv, __uint_as_float(o64[8 * chunk + 5]) * inv);
    v.w = pack2<kBf16>(__uint_as_float(o64[8 * chunk + 6]) * inv, __uint_as_float(o64[8 * chunk + 7]) * inv);
    *reinterpret_cast<uint4*>(line + ((chunk ^ (r & 7)) << 4)) = v;
  }
}

}  // namespace fa2
