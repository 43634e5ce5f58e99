// Forward attention kernel for head dim 256 on sm_100a.
//
// Same job as fwd_kernel (fwd_sm100.cu) and the same reference counterpart
// (jax_flash_attn2/flash_attention_triton/_forward_triton.py:60-164, 213-459), with the tile
// plan the tensor-memory budget of D = 256 forces: the O accumulator alone takes 256 of the 512
// columns, so one CTA owns ONE 128-row query tile and the other 256 columns hold two S buffers.
// While the softmax warpgroup works on S_j, the tensor core already computes S_{j+1} into the
// other buffer, and P_j (16 bit, over S_j) then feeds O += P_j V_j.
//   warps 0-3 : softmax, one thread per query row
//   warp  4   : tcgen05.mma issuer
//   warp  5   : TMA producer: Q once; K tiles through one slot and V tiles through another
// Shared memory: Q 64 KiB + K slot 64 KiB + V slot 64 KiB. There is no room for second slots, so
// each slot is handed over in two halves with their own full / empty barriers: K by head-dim blocks
// (the first eight S MMAs contract over dims 0-127, the last eight over 128-255), V by key rows (the
// P.V MMAs of the first half of P read keys 0-63). The next tile's first half then loads while the
// MMAs still read the second half of the current one.
#include "fwd_launch.cuh"
#include "fwd_row.cuh"
#include "launch_util.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

constexpr int kD = 256;
constexpr int kThreads256 = 192;

struct Smem256 {
  static constexpr int kQTileBytes = kBM * kD * 2;    // 64 KiB = 4 blocks of [128][64]
  static constexpr int kKVTileBytes = kBN * kD * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQTileBytes;
  static constexpr int kVOff = kKOff + kKVTileBytes;
  static constexpr int kBarOff = kVOff + kKVTileBytes;
  // barriers: q_full, k_full, k_empty, v_full, v_empty, s_full[2], p_full[2 buffers][2 halves],
  // pv_done, o_full, then the second-half barriers k_full, k_empty, v_full, v_empty
  static constexpr int kParts = kKV256Parts;           // pieces a K / V slot is handed over in
  static constexpr int kNumBars = 9 + 2 * kPSplit + 4 * kParts;
  static constexpr int kHalfBytes = kKVTileBytes / kParts;
  static_assert(kPSplit == 2, "V halves follow the two halves of P");
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;
};

}  // namespace

template <bool kBf16, bool kCausal, bool kFeat>
__global__ void __launch_bounds__(kThreads256, 1)
fwd256_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
              const FwdKernelParams p) {
  using L = Smem256;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + L::kQOff, sK = smem_base + L::kKOff, sV = smem_base + L::kVOff;
  const uint32_t bars = smem_base + L::kBarOff;
  const uint32_t bar_q_full = bars;
  const uint32_t bars2 = bars + 8u * (9 + 2 * kPSplit);   // per-piece barriers
  auto bar_k_full = [&](int part) { return bars2 + 8u * (4 * part); };
  auto bar_k_empty = [&](int part) { return bars2 + 8u * (4 * part + 1); };
  auto bar_v_full = [&](int part) { return bars2 + 8u * (4 * part + 2); };
  auto bar_v_empty = [&](int part) { return bars2 + 8u * (4 * part + 3); };
  auto bar_s_full = [&](int s) { return bars + 8u * (5 + s); };
  auto bar_p_full = [&](int s, int half) { return bars + 8u * (7 + kPSplit * s + half); };
  const uint32_t bar_pv_done = bars + 8u * (7 + 2 * kPSplit), bar_o_full = bars + 8u * (8 + 2 * kPSplit);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- work item: one 128-row query tile of one (batch, head); longest tiles first if causal --
  // split-KV: the grid holds n_splits CTAs per item, each with its own range of K/V tiles
  const int split = p.n_splits > 1 ? static_cast<int>(blockIdx.x % p.n_splits) : 0;
  const int item = p.n_splits > 1 ? static_cast<int>(blockIdx.x / p.n_splits) : static_cast<int>(blockIdx.x);
  const int j0 = split * p.split_tiles;          // first K/V tile of this CTA
  const int nbh = p.B * p.Hq;
  const int n_qtiles = (p.Sq + kBM - 1) / kBM;
  const int rank = item / nbh;
  const int bh = item - rank * nbh;
  const int qt = kCausal ? (n_qtiles - 1 - rank) : rank;
  const int b = bh / p.Hq;
  const int h = bh - b * p.Hq;
  const int hk = h / p.G;
  const int q0 = qt * kBM;
  // rows of this batch element that take part: the problem's, or its seqlens entry
  int sq_b = p.Sq, sk_b = p.Sk;
  if (p.seqlens != nullptr) {
    sq_b = max(0, min(__ldg(p.seqlens + b), p.Sq));
    sk_b = min(sq_b, p.Sk);
  }
  int nt;
  if (q0 >= sq_b) {
    nt = 0;
  } else if (kCausal) {
    const int row_last = min(q0 + kBM - 1, sq_b - 1);
    const int last_col = min(sk_b - 1, row_last + p.causal_off);
    nt = last_col >= 0 ? last_col / kBN + 1 : 0;
  } else {
    nt = (sk_b + kBN - 1) / kBN;
  }
  if (p.n_splits > 1) nt = max(0, min(nt - j0, p.split_tiles));
  const int b_out = b + split * p.B;             // where this CTA's output and lse go

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    for (int half = 0; half < L::kParts; ++half) {
      mbar_init(bar_k_full(half), 1);
      mbar_init(bar_k_empty(half), 1);
      mbar_init(bar_v_full(half), 1);
      mbar_init(bar_v_empty(half), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_s_full(s), 1);
      for (int hh = 0; hh < kPSplit; ++hh) mbar_init(bar_p_full(s, hh), kBM);
    }
    mbar_init(bar_pv_done, 1);
    mbar_init(bar_o_full, 1);
    fence_mbar_init();
  }
  if (warp == 5 && lane == 0) {
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
  constexpr uint32_t kColO = 0, kColS = 256;   // S buffer s at kColS + 128 s

  if (warp == 5) {
    // =========================== TMA producer ================================================
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q_full, L::kQTileBytes);
      tma_load_5d(sQ, &tmQ, bar_q_full, 0, q0, 0, h, b);
      bool ok = true;
      for (int j = 0; j < nt && ok; ++j) {
        // K: two head-dim blocks per copy (the K map's box); V: 64 key rows per copy (the V map's
        // box), which land as four [64 rows][64 dims] blocks
        for (int half = 0; half < L::kParts && ok; ++half) {
          ok = mbar_wait(bar_k_empty(half), (j & 1) ^ 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_k_full(half), L::kHalfBytes);
          tma_load_5d(sK + half * L::kHalfBytes, &tmK, bar_k_full(half), 0, (j0 + j) * kBN, (4 / L::kParts) * half, hk, b);
        }
        for (int half = 0; half < L::kParts && ok; ++half) {
          ok = mbar_wait(bar_v_empty(half), (j & 1) ^ 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_v_full(half), L::kHalfBytes);
          tma_load_5d(sV + half * L::kHalfBytes, &tmV, bar_v_full(half), 0, (j0 + j) * kBN + (kBN / L::kParts) * half, 0, hk, b);
        }
      }
      if (!ok) atomicOr(p.status, 1);
    }
    __syncwarp();
  } else if (warp == 4) {
    // =========================== MMA issuer ==================================================
    if (nt > 0) {
      constexpr uint32_t idesc_s = make_idesc(kBf16, kBM, kBN, false, false);
      constexpr uint32_t idesc_o = make_idesc(kBf16, kBM, kD, false, true);
      const uint64_t dQ = make_sdesc(sQ, 16, 1024);
      const uint64_t dK = make_sdesc(sK, 16, 1024);
      // a V half is four [64 rows][64 dims] blocks, 8 KiB apart
      const uint64_t dVh = make_sdesc(sV, kBlockBytes / L::kParts, 1024);
      bool ok = true;
      // S = Q K^T into buffer `buf`, K tile number jk: each half of K is released as soon as the
      // MMAs that contract over its dims have been issued
      auto issue_s = [&](int buf, int jk) {
#pragma unroll
        for (int half = 0; half < L::kParts; ++half) {
          if (ok) ok = mbar_wait_warp(bar_k_full(half), jk & 1, abort_flag);
          if (!ok) return;
          tc_fence_after();
#pragma unroll
          for (int k = half * (kD / 16 / L::kParts); k < (half + 1) * (kD / 16 / L::kParts); ++k) {
            const uint32_t off = (k >> 2) * kBlockBytes + (k & 3) * 32;
            mma_ss_e(tmem_base + kColS + buf * kBN, sdesc_advance(dQ, off), sdesc_advance(dK, off),
                   idesc_s, k > 0 ? 1u : 0u);
          }
          mma_commit_e(bar_k_empty(half));
        }
        mma_commit_e(bar_s_full(buf));
      };
      ok = mbar_wait_warp(bar_q_full, 0, abort_flag);
      if (ok) issue_s(0, 0);
      for (int j = 0; j < nt && ok; ++j) {
        const int buf = j & 1;
        if (j + 1 < nt) {
          issue_s(buf ^ 1, j + 1);
          if (!ok) break;
        }
#pragma unroll
        for (int part = 0; part < L::kParts; ++part) {
          constexpr int kStepsPerPart = kBN / 16 / L::kParts;          // 16-key MMA steps per piece of V
          constexpr int kPartsPerHalf = L::kParts / kPSplit;           // pieces of V per half of P
          if (ok) ok = mbar_wait_warp(bar_v_full(part), j & 1, abort_flag);
          if (ok && part % kPartsPerHalf == 0)
            ok = mbar_wait_warp(bar_p_full(buf, part / kPartsPerHalf), (j >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kStepsPerPart; ++k) {
            mma_ts_e(tmem_base + kColO, tmem_base + kColS + buf * kBN + (part * kStepsPerPart + k) * 8,
                   sdesc_advance(dVh, part * L::kHalfBytes + k * 2048), idesc_o,
                   (j == 0 && part == 0 && k == 0) ? 0u : 1u);
          }
          mma_commit_e(bar_v_empty(part));
        }
        if (!ok) break;
        mma_commit_e(bar_pv_done);
        if (j + 1 == nt) mma_commit_e(bar_o_full);
      }
      if (!ok && lane == 0) atomicOr(p.status, 2);
    }
    __syncwarp();
  } else {
    // =========================== softmax + epilogue ==========================================
    const int r = tid;                         // row inside the tile == TMEM lane
    const int qi = q0 + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + kColO;
    const int row_lim = qi < sq_b ? (kCausal ? min(sk_b - 1, qi + p.causal_off) : sk_b - 1) : -1;
    const FeatScale fs(p.scale_log2);
    const float sc = kFeat ? fs.sc : p.scale_log2;
    const bool prescale = kFeat && fs.prescale;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // dropout keep bits of this row: those of tile j + 1 are drawn after P of tile j has gone out
    const bool drop_on = kFeat && p.drop.enabled;
    uint32_t key_lo = 0u, key_hi = 0u;
    if (drop_on) dropout_key(p.drop, key_lo, key_hi);
    const uint32_t bh_glob = drop_on ? dropout_bh_index(p.drop, b, h) : 0u;
    KeepBitsDropout keep{drop_on, make_uint4(0u, 0u, 0u, 0u)};
    auto draw_keep = [&](int jt) {     // keep bits of K/V tile jt, also recorded for the backward
      keep.bits = draw_row_keep_bits(p.drop, key_lo, key_hi, bh_glob, qi, jt * kBN);
      store_row_keep_bits(p.drop, keep.bits, b, h, p.Hq, q0 >> 7, jt, r);
    };
    if (drop_on && nt > 0) draw_keep(j0);

    for (int j = 0; j < nt; ++j) {
      const int buf = j & 1;
      ok = mbar_wait(bar_s_full(buf), (j >> 1) & 1, abort_flag);
      if (!ok) break;
      const uint32_t tS = tmem_base + lane_base + kColS + buf * kBN;
      // O may only be rescaled once the previous P.V has finished accumulating into it
      auto wait_pv = [&] {
        if (!mbar_wait(bar_pv_done, (j - 1) & 1, abort_flag)) ok = false;
        tc_fence_after();
      };
      softmax_tile_row<kD, kBf16, kFeat>(tS, tO, j0 + j, j > 0, p, row_lim, sc, prescale, m, l, wait_pv,
                                         [&](int half) { mbar_arrive(bar_p_full(buf, half)); },
                                         DirectTerms<kBf16>{p, b, h, qi, fs.coef}, keep);
      if (!ok) break;
      if (drop_on && j + 1 < nt) draw_keep(j0 + j + 1);
    }

    if (ok) ok = mbar_wait(bar_q_full, 0, abort_flag);
    if (ok && nt > 0) ok = mbar_wait(bar_o_full, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      epilogue_row<kD, kBf16, kFeat>(tO, nt > 0, smem_gen + L::kQOff, r, p, b_out, h, qi, sc, m, l);
    }
    named_bar_sync(1, kBM);
    if (ok && r == 0 && !*abort_flag && !p.part_o) {
      tma_store_5d(&tmO, sQ, 0, q0, 0, h, b_out);
      tma_store_commit();
      tma_store_wait_read0();
    }
    if (!ok && r == 0) atomicOr(p.status, 4);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool kBf16, bool kCausal, bool kFeat>
static cudaError_t launch256_one(const FwdLaunch& a, cudaStream_t stream) {
  auto kern = fwd256_kernel<kBf16, kCausal, kFeat>;
  static bool smem_opted_in[64] = {};
  cudaError_t e = opt_in_dynamic_smem(kern, Smem256::kDynamicBytes, smem_opted_in);
  if (e != cudaSuccess) return e;
  const long long nblocks =
      static_cast<long long>((a.kp.Sq + kBM - 1) / kBM) * a.kp.B * a.kp.Hq * a.kp.n_splits;
  kern<<<static_cast<unsigned>(nblocks), kThreads256, Smem256::kDynamicBytes, stream>>>(
      a.tmQ, a.tmK, a.tmV, a.tmO, a.kp);
  return cudaGetLastError();
}

cudaError_t launch_fwd256(const FwdLaunch& a, cudaStream_t stream) {
  const int key = (a.bf16 ? 4 : 0) | (a.causal ? 2 : 0) | (a.feat ? 1 : 0);
  switch (key) {
    case 0: return launch256_one<false, false, false>(a, stream);
    case 1: return launch256_one<false, false, true>(a, stream);
    case 2: return launch256_one<false, true, false>(a, stream);
    case 3: return launch256_one<false, true, true>(a, stream);
    case 4: return launch256_one<true, false, false>(a, stream);
    case 5: return launch256_one<true, false, true>(a, stream);
    case 6: return launch256_one<true, true, false>(a, stream);
    default: return launch256_one<true, true, true>(a, stream);
  }
}

}  // namespace fa2
