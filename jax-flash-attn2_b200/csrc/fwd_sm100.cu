// Forward attention kernel for sm_100a.
//
// Replaces the Triton kernel _attn_fwd / _attn_fwd_inner of the reference
// (jax_flash_attn2/flash_attention_triton/_forward_triton.py:60-164, 213-459).
//
// One CTA owns 256 query rows of one (batch, query head): two 128-row tiles that share one
// stream of K/V tiles. Roles (12 warps; registers are moved from the last warpgroup to the
// softmax warpgroups with setmaxnreg):
//   warps 0-3  : softmax of query tile 0, one thread per row (TMEM lane == row)
//   warps 4-7  : softmax of query tile 1
//   warp  8    : tcgen05.mma issuer (one elected thread)
//   warp  9    : TMA producer (Q once, then K_j, V_j into a ring of shared-memory slots)
//   warps 10-11: idle (they complete the warpgroup that gives up its registers)
// Tensor memory (columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// P (16-bit, two values per column) overwrites the first 64 columns of its S tile and is the
// A operand of the P.V MMA, read straight from tensor memory.
// The two query tiles ping-pong: while the softmax warps of one tile work on S_j, the tensor
// core runs the MMAs of the other tile.
#include "fwd_launch.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

constexpr int kBM = 128;            // rows of one query tile
constexpr int kBN = 128;            // keys per K/V tile
constexpr int kTilesPerCta = 2;
constexpr int kThreads = 384;
constexpr int kRegsSoftmax = 208;   // per scheduler: 2 softmax warps + 1 other warp share the 3 * 168 registers of the launch
constexpr int kRegsOther = 88;
// Of every 8 column pairs, this many take their exponential from the FMA-pipe polynomial
// instead of the XU pipe. Measured on B200 (B=8, S=4096, Hq=32, D=128, causal): 0 -> 1.016 ms,
// 2 -> 1.019 ms, 3 -> 1.048 ms, 4 -> 1.039 ms, 5 -> 1.083 ms, so the default is 0: with packed
// f32x2 arithmetic the XU pipe is not what limits the kernel.
#ifndef FA2_FWD_POLY_PER8
#define FA2_FWD_POLY_PER8 0
#endif
constexpr int kPolyPer8 = FA2_FWD_POLY_PER8;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // in log2 units: P stays below 2^8

template <int D>
struct FwdSmem {
  static constexpr int kQTileBytes = kBM * D * 2;
  static constexpr int kKVTileBytes = kBN * D * 2;
  static constexpr int kStages = (D == 64) ? 8 : 4;
  static constexpr int kBlockBytes = kBM * 128;       // one [128 rows][64 elements] block
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = kQOff + kTilesPerCta * kQTileBytes;
  static constexpr int kBarOff = kKVOff + kStages * kKVTileBytes;
  // barriers: q_full[2], kv_full[S], kv_empty[S], s_full[2], p_full[2], o_full[2]
  static constexpr int kNumBars = 2 + 2 * kStages + 6;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;  // room to align the base to 1024 B
};

template <bool kBf16>
__device__ __forceinline__ void add_score_term(float (&x)[kBN], const ScoreTermDev& t, int b,
                                               int h, int qi, int kv0, int Sk) {
  const long long base = static_cast<long long>(b) * t.sb + static_cast<long long>(h) * t.sh +
                         static_cast<long long>(qi) * t.sq + kv0;
  const bool full = (kv0 + kBN <= Sk);
  if (t.is_f32) {
    const float* p = static_cast<const float*>(t.ptr) + base;
    if (t.vec_ok && full) {
#pragma unroll
      for (int c4 = 0; c4 < kBN / 4; ++c4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p) + c4);
        x[4 * c4 + 0] = fmaf(v.x, kLog2e, x[4 * c4 + 0]);
        x[4 * c4 + 1] = fmaf(v.y, kLog2e, x[4 * c4 + 1]);
        x[4 * c4 + 2] = fmaf(v.z, kLog2e, x[4 * c4 + 2]);
        x[4 * c4 + 3] = fmaf(v.w, kLog2e, x[4 * c4 + 3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < kBN; ++c)
        if (kv0 + c < Sk) x[c] = fmaf(__ldg(p + c), kLog2e, x[c]);
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
              fmaf(to_float16bit<kBf16>(static_cast<uint16_t>(w[k] & 0xffff)), kLog2e,
                   x[8 * c8 + 2 * k + 0]);
          x[8 * c8 + 2 * k + 1] = fmaf(to_float16bit<kBf16>(static_cast<uint16_t>(w[k] >> 16)),
                                       kLog2e, x[8 * c8 + 2 * k + 1]);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < kBN; ++c)
        if (kv0 + c < Sk) x[c] = fmaf(to_float16bit<kBf16>(__ldg(p + c)), kLog2e, x[c]);
    }
  }
}

}  // namespace

template <int D, bool kBf16, bool kCausal, bool kFeat>
__global__ void __launch_bounds__(kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
           const FwdKernelParams p) {
  using L = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sQ = smem_base + L::kQOff;
  const uint32_t sKV = smem_base + L::kKVOff;
  const uint32_t bars = smem_base + L::kBarOff;
  auto bar_q_full = [&](int t) { return bars + 8u * t; };
  auto bar_kv_full = [&](int s) { return bars + 8u * (2 + s); };
  auto bar_kv_empty = [&](int s) { return bars + 8u * (2 + L::kStages + s); };
  auto bar_s_full = [&](int t) { return bars + 8u * (2 + 2 * L::kStages + t); };
  auto bar_p_full = [&](int t) { return bars + 8u * (4 + 2 * L::kStages + t); };
  auto bar_o_full = [&](int t) { return bars + 8u * (6 + 2 * L::kStages + t); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- work item ----------------------------------------------------------------------------
  const int nbh = p.B * p.Hq;
  const int qb_rank = blockIdx.x / nbh;
  const int bh = blockIdx.x - qb_rank * nbh;
  // causal: the longest blocks are scheduled first
  const int qblk = kCausal ? (p.n_qblk - 1 - qb_rank) : qb_rank;
  const int b = bh / p.Hq;
  const int h = bh - b * p.Hq;
  const int hk = h / p.G;
  const int q0 = qblk * (kBM * kTilesPerCta);

  int n_tiles[kTilesPerCta];
#pragma unroll
  for (int t = 0; t < kTilesPerCta; ++t) {
    const int row_first = q0 + t * kBM;
    if (row_first >= p.Sq) {
      n_tiles[t] = 0;
    } else if (kCausal) {
      const int row_last = min(row_first + kBM - 1, p.Sq - 1);
      const int last_col = min(p.Sk - 1, row_last + p.causal_off);
      n_tiles[t] = last_col >= 0 ? last_col / kBN + 1 : 0;
    } else {
      n_tiles[t] = (p.Sk + kBN - 1) / kBN;
    }
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);

  // ---- set-up ---------------------------------------------------------------------------------
  if (tid == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_q_full(t), 1);
      mbar_init(bar_s_full(t), 1);
      mbar_init(bar_p_full(t), kBM);
      mbar_init(bar_o_full(t), 1);
    }
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColO = 256;


  if (warp >= 8) {
    // One warpgroup, one instruction: all four warps release their registers here.
    setmaxnreg_dec<kRegsOther>();
  }
  if (warp >= 10) {
    // idle
  } else if (warp == 9) {
    // =========================== TMA producer ================================================
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < kTilesPerCta; ++t) {
        mbar_arrive_expect_tx(bar_q_full(t), L::kQTileBytes);
        tma_load_5d(sQ + t * L::kQTileBytes, &tmQ, bar_q_full(t), 0, q0 + t * kBM, 0, h, b);
      }
      bool ok = true;
      for (int i = 0; i < 2 * n_max && ok; ++i) {
        const int slot = i % L::kStages;
        const uint32_t round = static_cast<uint32_t>(i / L::kStages);
        ok = mbar_wait(bar_kv_empty(slot), (round & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        const int j = i >> 1;
        mbar_arrive_expect_tx(bar_kv_full(slot), L::kKVTileBytes);
        tma_load_5d(sKV + slot * L::kKVTileBytes, (i & 1) ? &tmV : &tmK, bar_kv_full(slot), 0,
                    j * kBN, 0, hk, b);
      }
      if (!ok) atomicOr(p.status, 1);
    }
    __syncwarp();
  } else if (warp == 8) {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kBf16, kBM, kBN, false, false);
      constexpr uint32_t idesc_o = make_idesc(kBf16, kBM, D, false, true);
      bool ok = true;

      // Descriptors are built once; each MMA adds a constant to the start address.
      const uint64_t dQ0 = make_sdesc(sQ, 16, 1024);
      const uint64_t dKV_k0 = make_sdesc(sKV, 16, 1024);                 // K tile, K-major
      const uint64_t dKV_mn0 = make_sdesc(sKV, L::kBlockBytes, 1024);    // V tile, MN-major
      auto issue_s = [&](int t, int slot) {
        const uint64_t a0 = sdesc_advance(dQ0, t * L::kQTileBytes);
        const uint64_t b0 = sdesc_advance(dKV_k0, slot * L::kKVTileBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * L::kBlockBytes + (k & 3) * 32;
          mma_ss(tmem_base + kColS + t * kBN, sdesc_advance(a0, off), sdesc_advance(b0, off), idesc_s,
                 k > 0 ? 1u : 0u);
        }
        mma_commit(bar_s_full(t));
      };
      auto issue_o = [&](int t, int slot, bool first) {
        const uint64_t b0 = sdesc_advance(dKV_mn0, slot * L::kKVTileBytes);
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k) {
          mma_ts(tmem_base + kColO + t * D, tmem_base + kColS + t * kBN + k * 8,
                 sdesc_advance(b0, k * 2048), idesc_o, (first && k == 0) ? 0u : 1u);
        }
      };

      if (n_max > 0) {
        for (int t = 0; t < kTilesPerCta && ok; ++t)
          if (n_tiles[t] > 0) ok = mbar_wait(bar_q_full(t), 0, abort_flag);
        if (ok) ok = mbar_wait(bar_kv_full(0), 0, abort_flag);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < kTilesPerCta; ++t)
            if (n_tiles[t] > 0) issue_s(t, 0);
          mma_commit(bar_kv_empty(0));
        }
        for (int j = 0; j < n_max && ok; ++j) {
          const int iv = 2 * j + 1, ik = 2 * j + 2;
          const int slot_v = iv % L::kStages, slot_k = ik % L::kStages;
          ok = mbar_wait(bar_kv_full(slot_v), (iv / L::kStages) & 1, abort_flag);
          if (!ok) break;
          const bool has_next = (j + 1 < n_max);
          if (has_next) {
            ok = mbar_wait(bar_kv_full(slot_k), (ik / L::kStages) & 1, abort_flag);
            if (!ok) break;
          }
#pragma unroll
          for (int t = 0; t < kTilesPerCta; ++t) {
            if (j < n_tiles[t]) {
              ok = mbar_wait(bar_p_full(t), j & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
              issue_o(t, slot_v, j == 0);
              if (j + 1 < n_tiles[t]) {
                issue_s(t, slot_k);
              } else {
                mma_commit(bar_o_full(t));
              }
            }
          }
          if (!ok) break;
          mma_commit(bar_kv_empty(slot_v));
          if (has_next) mma_commit(bar_kv_empty(slot_k));
        }
      }
      if (!ok) atomicOr(p.status, 2);
    }
    __syncwarp();
  } else if (warp < 8) {
    // =========================== softmax + epilogue ==========================================
    setmaxnreg_inc<kRegsSoftmax>();
    const int t = warp >> 2;                   // query tile of this warpgroup
    const int r = tid & (kBM - 1);             // row inside the tile == TMEM lane
    const int qi = q0 + t * kBM + r;           // global query row
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + t * kBN;
    const uint32_t tO = tmem_base + lane_base + kColO + t * D;
    const int nt = n_tiles[t];
    const bool tile_valid = (q0 + t * kBM) < p.Sq;
    // last visible key of this row
    const int row_lim = kCausal ? min(p.Sk - 1, qi + p.causal_off) : p.Sk - 1;
    const float sc = kFeat ? 1.0f : p.scale_log2;   // multiplies the values held in x[]

    float m = -INFINITY;   // running (possibly stale) row maximum, in the units of x[]
    float l = 0.f;         // running row sum of exp2(x*sc - m*sc)
    bool ok = true;

    for (int j = 0; j < nt; ++j) {
      ok = mbar_wait(bar_s_full(t), j & 1, abort_flag);
      if (!ok) break;
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
#pragma unroll
        for (int c = 0; c < kBN; ++c) x[c] *= p.scale_log2;
        if (qi < p.Sq) {
          if (p.bias.ptr) add_score_term<kBf16>(x, p.bias, b, h, qi, kv0, p.Sk);
          if (p.mask.ptr) add_score_term<kBf16>(x, p.mask, b, h, qi, kv0, p.Sk);
        }
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
        if (j > 0) {
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
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int c = 0; c < kBN; c += 4) {
        fma2(x[c], x[c + 1], x[c], x[c + 1], sc, sc, neg_ms, neg_ms);
        fma2(x[c + 2], x[c + 3], x[c + 2], x[c + 3], sc, sc, neg_ms, neg_ms);
        if (((c >> 1) & 7) < kPolyPer8) {
          ex2_poly2(x[c], x[c + 1]);
        } else {
          x[c] = ex2_approx(x[c]);
          x[c + 1] = ex2_approx(x[c + 1]);
        }
        if ((((c >> 1) + 1) & 7) < kPolyPer8) {
          ex2_poly2(x[c + 2], x[c + 3]);
        } else {
          x[c + 2] = ex2_approx(x[c + 2]);
          x[c + 3] = ex2_approx(x[c + 3]);
        }
        add2(l0, l1, l0, l1, x[c], x[c + 1]);
        add2(l2, l3, l2, l3, x[c + 2], x[c + 3]);
      }
      l += (l0 + l1) + (l2 + l3);
      if constexpr (kFeat) {
        if (p.drop.enabled) {
          const uint32_t bh_glob = static_cast<uint32_t>(
              (p.drop.b_off + b) * p.drop.hq_global + p.drop.h_off + h);
#pragma unroll
          for (int c = 0; c < kBN; c += 4) {
            uint32_t rnd[4];
            philox4x32_10(static_cast<uint32_t>((kv0 + c) >> 2), static_cast<uint32_t>(qi),
                          bh_glob, 0u, p.drop.seed_lo, p.drop.seed_hi, rnd);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (rnd[k] < p.drop.threshold) x[c + k] = 0.f;
          }
        }
      }
      {
        uint32_t pk[kBN / 2];
#pragma unroll
        for (int c = 0; c < kBN / 2; ++c) pk[c] = pack2<kBf16>(x[2 * c], x[2 * c + 1]);
        tmem_st32(tS, reinterpret_cast<const uint32_t(&)[32]>(pk[0]));
        tmem_st32(tS + 32, reinterpret_cast<const uint32_t(&)[32]>(pk[32]));
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full(t));
    }

    // ---- epilogue: O / l -> 16 bit -> swizzled shared memory -> TMA store; LSE ---------------
    if (ok && tile_valid) {
      ok = mbar_wait(bar_q_full(t), 0, abort_flag);   // Q tile landed: its slot is reused below
      if (ok && nt > 0) ok = mbar_wait(bar_o_full(t), 0, abort_flag);
    }
    if (ok && tile_valid) {
      tc_fence_after();
      const float inv = (l > 0.f) ? (kFeat ? p.drop.inv_keep : 1.f) / l : 0.f;
      const float lse = (l > 0.f) ? (m * sc + lg2_approx(l)) * kLn2 : -INFINITY;
      if (qi < p.Sq)
        p.lse[static_cast<long long>(b) * p.lse_sb + static_cast<long long>(h) * p.lse_sh + qi] =
            lse;
      uint8_t* so_gen = smem_gen + L::kQOff + t * L::kQTileBytes;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (nt > 0) {
          tmem_ld32(tO + c * 32, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) o[k] = 0u;
        }
        // 32 columns = 64 bytes = four 16-byte chunks of this row's 128-byte line
        uint8_t* line = so_gen + (c >> 1) * L::kBlockBytes + r * 128;
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
    // All 128 threads of the warpgroup reach this barrier, whatever happened above.
    named_bar_sync(1 + t, kBM);
    if (ok && tile_valid && r == 0 && !*abort_flag) {
      tma_store_5d(&tmO, sQ + t * L::kQTileBytes, 0, q0 + t * kBM, 0, h, b);
      tma_store_commit();
      tma_store_wait_read0();
    }
    if (!ok && r == 0) atomicOr(p.status, 4);
  }

  // ---- teardown -------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// launcher
// ---------------------------------------------------------------------------------------------
template <int D, bool kBf16, bool kCausal, bool kFeat>
static cudaError_t launch_one(const FwdLaunch& a, cudaStream_t stream) {
  using L = FwdSmem<D>;
  auto kern = fwd_kernel<D, kBf16, kCausal, kFeat>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  if (e != cudaSuccess) return e;
  const long long nblocks =
      static_cast<long long>(a.kp.n_qblk) * a.kp.B * a.kp.Hq;
  if (nblocks <= 0) return cudaSuccess;
  kern<<<static_cast<unsigned>(nblocks), kThreads, L::kDynamicBytes, stream>>>(a.tmQ, a.tmK, a.tmV,
                                                                               a.tmO, a.kp);
  return cudaGetLastError();
}

template <int D>
static cudaError_t launch_d(const FwdLaunch& a, cudaStream_t stream) {
  const int key = (a.bf16 ? 4 : 0) | (a.causal ? 2 : 0) | (a.feat ? 1 : 0);
  switch (key) {
    case 0: return launch_one<D, false, false, false>(a, stream);
    case 1: return launch_one<D, false, false, true>(a, stream);
    case 2: return launch_one<D, false, true, false>(a, stream);
    case 3: return launch_one<D, false, true, true>(a, stream);
    case 4: return launch_one<D, true, false, false>(a, stream);
    case 5: return launch_one<D, true, false, true>(a, stream);
    case 6: return launch_one<D, true, true, false>(a, stream);
    default: return launch_one<D, true, true, true>(a, stream);
  }
}

cudaError_t launch_fwd(const FwdLaunch& a, cudaStream_t stream) {
  switch (a.head_dim) {
    case 64: return launch_d<64>(a, stream);
    case 128: return launch_d<128>(a, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fa2
