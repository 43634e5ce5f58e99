// Forward attention kernel for sm_100a (head dim 64 and 128).
//
// Replaces the Triton kernel _attn_fwd / _attn_fwd_inner of the reference
// (jax_flash_attn2/flash_attention_triton/_forward_triton.py:60-164, 213-459).
//
// Persistent kernel: one CTA per SM walks over work items. A work item is 256 query rows of one
// (batch, query head): two 128-row tiles that share one stream of K/V tiles. Items are ordered
// longest first (causal) and dealt round-robin to the CTAs. Roles (12 warps; registers are moved
// from the last warpgroup to the softmax warpgroups with setmaxnreg):
//   warps 0-3  : softmax + epilogue of query tile 0, one thread per row (TMEM lane == row)
//   warps 4-7  : softmax + epilogue of query tile 1
//   warp  8    : tcgen05.mma issuer (one elected thread)
//   warp  9    : TMA producer (Q tiles per item, K_j / V_j through a ring of shared-memory slots)
//   warps 10-11: idle (they complete the warpgroup that gives up its registers)
// Tensor memory (columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// P (16-bit, two values per column) overwrites the first 64 columns of its S tile and is the
// A operand of the P.V MMA, read straight from tensor memory.
// The two query tiles ping-pong: while the softmax warps of one tile work on S_j, the tensor
// core runs the MMAs of the other tile. Across items the roles run ahead of each other: the
// producer refills a Q tile as soon as its last S MMA has completed and the K/V ring never drains,
// so the next item's first MMAs overlap the epilogue (O -> shared memory -> TMA store) of this one.
//
// Bias, mask and dropout (`kFeat`) are kept off the S -> softmax -> P.V chain of a tile:
//   * dropout: a softmax thread draws the Philox keep bits of its row for the NEXT K/V tile right
//     after it has handed P of the current tile to the MMA warp (128 bits in four registers);
//   * bias / mask at head dim 64, where shared memory has room: every softmax warp streams the
//     [32 rows x 64 keys] pieces of the tiles it needs through its own ring of three 4 KiB slots;
//     lane 0 issues the TMA copy of piece n + 3 as soon as the warp has read piece n, so a piece has
//     most of a tile period to arrive from L2. At head dim 128 the K/V ring leaves no room for
//     that and the terms are read straight from global memory.
#include "fwd_launch.cuh"
#include "fwd_row.cuh"
#include "launch_util.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

constexpr int kTilesPerCta = 2;
constexpr int kThreads = 384;
// per scheduler: 2 softmax warps + 1 other warp share the 3 * 168 registers of the launch
template <bool kStaged> constexpr int kRegsSoftmax = kStaged ? 216 : 208;   // staged score terms keep more state per softmax thread
template <bool kStaged> constexpr int kRegsOther = kStaged ? 72 : 88;

template <int D, bool kStaged>
struct FwdSmem {
  static constexpr int kQTileBytes = kBM * D * 2;
  static constexpr int kKVTileBytes = kBN * D * 2;
  static constexpr int kStages = kStaged ? 4 : (D == 64) ? 8 : 4;
  static constexpr int kBlockBytes = kBM * 128;       // one [128 rows][64 elements] block
  // staged score terms: per softmax warp a ring of [32 rows][64 keys] 16-bit pieces
  static constexpr int kTermSlots = 3;
  static constexpr int kTermPieceBytes = 32 * 128;
  static constexpr int kQOff = 0;
  static constexpr int kOOff = kQOff + kTilesPerCta * kQTileBytes;     // O staging: one 64-column block per tile
  static constexpr int kKVOff = kOOff + kTilesPerCta * kBlockBytes;
  static constexpr int kTermOff = kKVOff + kStages * kKVTileBytes;
  static constexpr int kBarOff = kTermOff + (kStaged ? 8 * kTermSlots * kTermPieceBytes : 0);
  // barriers: q_full[2], q_free[2], kv_full[S], kv_empty[S], s_full[2], p_full[2][kPSplit],
  // o_full[2], o_free[2]; staged: term_full[8 warps][kTermSlots]
  static constexpr int kNumBarsBase = 4 + 2 * kStages + 2 + 2 * kPSplit + 4;
  static constexpr int kNumBars = kNumBarsBase + (kStaged ? 8 * kTermSlots : 0);
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;  // room to align the base to 1024 B
  static_assert(kDynamicBytes <= 232448, "shared memory budget exceeded");
};

// One work item as every role sees it.
struct FwdItem {
  int b, h, hk, q0;
  int split, j0;   // split-KV: which part of the K/V sequence, and its first tile
  int sq, sk;   // rows of this batch element that take part (the problem's, or its seqlens entry)
  int n_tiles[kTilesPerCta];
  int n_max;
};

template <bool kCausal>
__device__ __forceinline__ void decode_item(const FwdKernelParams& p, int w, FwdItem& it) {
  it.split = 0;
  if (p.n_splits > 1) {
    it.split = w % p.n_splits;
    w /= p.n_splits;
  }
  it.j0 = it.split * p.split_tiles;
  const int nbh = p.B * p.Hq;
  const int qb_rank = w / nbh;
  const int bh = w - qb_rank * nbh;
  // causal: the longest blocks come first
  const int qblk = kCausal ? (p.n_qblk - 1 - qb_rank) : qb_rank;
  it.b = bh / p.Hq;
  it.h = bh - it.b * p.Hq;
  it.hk = it.h / p.G;
  it.q0 = qblk * (kBM * kTilesPerCta);
  it.sq = p.Sq;
  it.sk = p.Sk;
  if (p.seqlens != nullptr) {
    const int len = max(0, min(__ldg(p.seqlens + it.b), p.Sq));
    it.sq = len;
    it.sk = min(len, p.Sk);
  }
#pragma unroll
  for (int t = 0; t < kTilesPerCta; ++t) {
    const int row_first = it.q0 + t * kBM;
    if (row_first >= it.sq) {
      it.n_tiles[t] = 0;
    } else if (kCausal) {
      const int row_last = min(row_first + kBM - 1, it.sq - 1);
      const int last_col = min(it.sk - 1, row_last + p.causal_off);
      it.n_tiles[t] = last_col >= 0 ? last_col / kBN + 1 : 0;
    } else {
      it.n_tiles[t] = (it.sk + kBN - 1) / kBN;
    }
    if (p.n_splits > 1) it.n_tiles[t] = max(0, min(it.n_tiles[t] - it.j0, p.split_tiles));
  }
  it.n_max = max(it.n_tiles[0], it.n_tiles[1]);
}

}  // namespace

template <int D, bool kBf16, bool kCausal, bool kFeat>
__global__ void __launch_bounds__(kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO1,
           const __grid_constant__ CUtensorMap tmBias, const __grid_constant__ CUtensorMap tmMask,
           const FwdKernelParams p) {
  constexpr bool kStaged = kFeat && D == 64;
  using L = FwdSmem<D, kStaged>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sQ = smem_base + L::kQOff;
  const uint32_t sO = smem_base + L::kOOff;
  const uint32_t sKV = smem_base + L::kKVOff;
  const uint32_t bars = smem_base + L::kBarOff;
  auto bar_q_full = [&](int t) { return bars + 8u * t; };
  auto bar_q_free = [&](int t) { return bars + 8u * (2 + t); };
  auto bar_kv_full = [&](int s) { return bars + 8u * (4 + s); };
  auto bar_kv_empty = [&](int s) { return bars + 8u * (4 + L::kStages + s); };
  auto bar_s_full = [&](int t) { return bars + 8u * (4 + 2 * L::kStages + t); };
  auto bar_p_full = [&](int t, int hh) { return bars + 8u * (6 + 2 * L::kStages + kPSplit * t + hh); };
  auto bar_o_full = [&](int t) { return bars + 8u * (6 + 2 * L::kStages + 2 * kPSplit + t); };
  auto bar_o_free = [&](int t) { return bars + 8u * (8 + 2 * L::kStages + 2 * kPSplit + t); };
  auto bar_term_full = [&](int wi, int s) { return bars + 8u * (L::kNumBarsBase + wi * L::kTermSlots + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int total_items = p.n_qblk * p.B * p.Hq * p.n_splits;
  // Items are dealt to the CTAs in rounds of gridDim.x, forwards in even rounds and backwards in odd
  // ones: causal items come longest first, so the CTA that drew the longest item of one round draws
  // the shortest of the next, which evens out what a plain round-robin deal leaves unequal (3 % of
  // the launch at B=8, S=4096, 32 heads; 13 % at a quarter of that batch).
  auto first_item = [&]() { return static_cast<int>(blockIdx.x); };
  auto next_item = [&](int w) {
    const int grid = static_cast<int>(gridDim.x);
    const int round = w / grid + 1;
    const int pos = (round & 1) ? grid - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
    const int nw = round * grid + pos;
    // the last, partial round: a CTA whose mirrored slot lies beyond the end takes no further item
    return nw;
  };

  // ---- set-up ---------------------------------------------------------------------------------
  if (tid == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_q_full(t), 1);
      mbar_init(bar_q_free(t), 1);
      mbar_init(bar_s_full(t), 1);
      for (int hh = 0; hh < kPSplit; ++hh) mbar_init(bar_p_full(t, hh), kBM);
      mbar_init(bar_o_full(t), 1);
      mbar_init(bar_o_free(t), kBM);
    }
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    if constexpr (kStaged) {
      for (int wi = 0; wi < 8; ++wi)
        for (int s = 0; s < L::kTermSlots; ++s) mbar_init(bar_term_full(wi, s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO1);
    if constexpr (kStaged) {
      if (p.bias.staged) tma_prefetch_desc(&tmBias);
      if (p.mask.staged) tma_prefetch_desc(&tmMask);
    }
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
    setmaxnreg_dec<kRegsOther<kStaged>>();
  }
  if (warp >= 10) {
    // idle
  } else if (warp == 9) {
    // =========================== TMA producer ================================================
    if (lane == 0) {
      bool ok = true;
      uint32_t kv_count = 0;     // K/V tiles loaded so far (over all items)
      uint32_t item_idx = 0;
      for (int w = first_item(); w < total_items && ok; w = next_item(w), ++item_idx) {
        FwdItem it;
        decode_item<kCausal>(p, w, it);
#pragma unroll
        for (int t = 0; t < kTilesPerCta; ++t) {
          // the last S MMA of the previous item that read this Q tile has completed
          ok = ok && mbar_wait(bar_q_free(t), (item_idx & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_q_full(t), L::kQTileBytes);
          tma_load_5d(sQ + t * L::kQTileBytes, &tmQ, bar_q_full(t), 0, it.q0 + t * kBM, 0, it.h, it.b);
        }
        for (int i = 0; i < 2 * it.n_max && ok; ++i, ++kv_count) {
          const int slot = kv_count % L::kStages;
          const uint32_t round = kv_count / L::kStages;
          ok = mbar_wait(bar_kv_empty(slot), (round & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_kv_full(slot), L::kKVTileBytes);
          tma_load_5d(sKV + slot * L::kKVTileBytes, (i & 1) ? &tmV : &tmK, bar_kv_full(slot), 0,
                      (it.j0 + (i >> 1)) * kBN, 0, it.hk, it.b);
        }
      }
      if (!ok) atomicOr(p.status, 1);
    }
    __syncwarp();
  } else if (warp == 8) {
    // =========================== MMA issuer ==================================================
    {
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
          mma_ss_e(tmem_base + kColS + t * kBN, sdesc_advance(a0, off), sdesc_advance(b0, off), idesc_s,
                 k > 0 ? 1u : 0u);
        }
        mma_commit_e(bar_s_full(t));
      };
      auto issue_o = [&](int t, int slot, bool first, int hh) {
        const uint64_t b0 = sdesc_advance(dKV_mn0, slot * L::kKVTileBytes);
#pragma unroll
        for (int k = hh * (kPCols / 16); k < (hh + 1) * (kPCols / 16); ++k) {
          mma_ts_e(tmem_base + kColO + t * D, tmem_base + kColS + t * kBN + k * 8,
                 sdesc_advance(b0, k * 2048), idesc_o, (first && k == 0) ? 0u : 1u);
        }
      };

      uint32_t kv_count = 0;                 // K/V tiles consumed so far (over all items)
      uint32_t it_cnt[kTilesPerCta] = {0, 0};   // tile-iterations so far: phase of s_full / p_full
      uint32_t item_idx = 0;
      for (int w = first_item(); w < total_items && ok; w = next_item(w), ++item_idx) {
        FwdItem it;
        decode_item<kCausal>(p, w, it);
        // Q tiles of this item have landed (also for tiles without work: their buffer is handed
        // back at once so that the producer's next load into it is ordered after this one)
#pragma unroll
        for (int t = 0; t < kTilesPerCta; ++t) {
          ok = ok && mbar_wait_warp(bar_q_full(t), item_idx & 1u, abort_flag);
          if (ok && it.n_tiles[t] == 0) {
            mma_commit_e(bar_q_free(t));
            // Keep the o_free / o_full hand-shake in step for tiles without work, so that neither
            // side ever gets two phases ahead of the other.
            ok = mbar_wait_warp(bar_o_free(t), (item_idx & 1u) ^ 1u, abort_flag);
            if (ok) mma_commit_e(bar_o_full(t));
          }
        }
        if (!ok || it.n_max == 0) continue;
        {
          const int slot = kv_count % L::kStages;
          ok = mbar_wait_warp(bar_kv_full(slot), (kv_count / L::kStages) & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < kTilesPerCta; ++t) {
            if (it.n_tiles[t] > 0) {
              issue_s(t, slot);
              if (it.n_tiles[t] == 1) mma_commit_e(bar_q_free(t));   // that was the last S of tile t
            }
          }
          mma_commit_e(bar_kv_empty(slot));
          ++kv_count;
        }
        for (int j = 0; j < it.n_max && ok; ++j) {
          const bool has_next = (j + 1 < it.n_max);
          const int slot_v = kv_count % L::kStages;
          const int slot_k = (kv_count + 1) % L::kStages;
          ok = mbar_wait_warp(bar_kv_full(slot_v), (kv_count / L::kStages) & 1u, abort_flag);
          if (!ok) break;
          if (has_next) {
            ok = mbar_wait_warp(bar_kv_full(slot_k), ((kv_count + 1) / L::kStages) & 1u, abort_flag);
            if (!ok) break;
          }
#pragma unroll
          for (int t = 0; t < kTilesPerCta; ++t) {
            if (j < it.n_tiles[t]) {
              if (j == 0) {
                // the epilogue of the previous item has read O_t out of tensor memory
                ok = mbar_wait_warp(bar_o_free(t), (item_idx & 1u) ^ 1u, abort_flag);
                if (!ok) break;
              }
#pragma unroll
              for (int hh = 0; hh < kPSplit; ++hh) {
                ok = mbar_wait_warp(bar_p_full(t, hh), it_cnt[t] & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                issue_o(t, slot_v, j == 0, hh);
              }
              if (!ok) break;
              ++it_cnt[t];
              if (j + 1 < it.n_tiles[t]) {
                issue_s(t, slot_k);
                if (j + 2 == it.n_tiles[t]) mma_commit_e(bar_q_free(t));   // last S of tile t issued
              } else {
                mma_commit_e(bar_o_full(t));
              }
            }
          }
          if (!ok) break;
          mma_commit_e(bar_kv_empty(slot_v));
          if (has_next) mma_commit_e(bar_kv_empty(slot_k));
          kv_count += has_next ? 2 : 1;
        }
      }
      if (!ok && lane == 0) atomicOr(p.status, 2);
    }
    __syncwarp();
  } else if (warp < 8) {
    // =========================== softmax + epilogue ==========================================
    setmaxnreg_inc<kRegsSoftmax<kStaged>>();
    const int t = warp >> 2;                   // query tile of this warpgroup
    const int r = tid & (kBM - 1);             // row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + t * kBN;
    const uint32_t tO = tmem_base + lane_base + kColO + t * D;
    const FeatScale fs(p.scale_log2);
    const float sc = kFeat ? fs.sc : p.scale_log2;   // multiplies the values held in x[]
    const bool prescale = kFeat && fs.prescale;
    uint32_t it_cnt = 0;       // tile-iterations so far: phase of s_full / p_full
    uint32_t o_cnt = 0;        // items so far: phase of o_full
    bool ok = true;
    // staged terms: pieces this warp has loaded so far (slot and phase of its ring)
    uint32_t term_cnt = 0;
    const int n_staged = kStaged ? (p.bias.staged ? 1 : 0) + (p.mask.staged ? 1 : 0) : 0;
    const int per_tile = 2 * n_staged;   // pieces per K/V tile: two halves of 64 keys per term
    // dropout: Philox key of the call
    uint32_t key_lo = 0u, key_hi = 0u;
    const bool drop_on = kFeat && p.drop.enabled;
    if (drop_on) dropout_key(p.drop, key_lo, key_hi);

    for (int w = first_item(); w < total_items; w = next_item(w)) {
      FwdItem it;
      decode_item<kCausal>(p, w, it);
      const int b = it.b, h = it.h;
      const int b_out = it.b + it.split * p.B;   // where this item's output and lse go
      const int qi = it.q0 + t * kBM + r;      // global query row
      const int nt = it.n_tiles[t];
      const bool tile_valid = (it.q0 + t * kBM) < p.Sq;
      // last visible key of this row (none for rows past the end of the sequence)
      const int row_lim =
          qi < it.sq ? (kCausal ? min(it.sk - 1, qi + p.causal_off) : it.sk - 1) : -1;
      float m = -INFINITY;   // running (possibly stale) row maximum, in the units of x[]
      float l = 0.f;         // running row sum of exp2(x*sc - m*sc)

      // keep bits of this row for the tile about to be processed; those of tile j + 1 are drawn
      // after P of tile j has been handed over
      KeepBitsDropout keep{drop_on, make_uint4(0u, 0u, 0u, 0u)};
      const uint32_t bh_glob = drop_on ? dropout_bh_index(p.drop, b, h) : 0u;
      auto draw_keep = [&](int jt) {     // keep bits of K/V tile jt, also recorded for the backward
        keep.bits = draw_row_keep_bits(p.drop, key_lo, key_hi, bh_glob, qi, jt * kBN);
        store_row_keep_bits(p.drop, keep.bits, b, h, p.Hq, (it.q0 >> 7) + t, jt, r);
      };
      if (drop_on && nt > 0) draw_keep(it.j0);

      if constexpr (kStaged) {
        // ---- this warp's stream of term pieces for the item: piece n = (K/V tile n / per_tile,
        // term (n % per_tile) / 2, half n % 2); lane 0 keeps kTermSlots copies in flight
        const int wi = warp;                       // 0..7
        const int n_pieces = nt * per_tile;
        const uint32_t term_smem = smem_base + L::kTermOff + wi * (L::kTermSlots * L::kTermPieceBytes);
        const int row0 = it.q0 + t * kBM + 32 * (warp & 3);   // first query row of this warp
        auto issue_piece = [&](int n, uint32_t cnt) {          // lane 0 only
          const int jj = n / per_tile, rr = n - jj * per_tile;
          const bool second = (rr >> 1) == 1 || !p.bias.staged;   // which of the staged terms
          const ScoreTermDev& tt = second ? p.mask : p.bias;
          const int slot = cnt % L::kTermSlots;
          mbar_arrive_expect_tx(bar_term_full(wi, slot), L::kTermPieceBytes);
          tma_load_4d(term_smem + slot * L::kTermPieceBytes, second ? &tmMask : &tmBias,
                      bar_term_full(wi, slot), (it.j0 + jj) * kBN + 64 * (rr & 1), row0,
                      tt.sh ? h / tt.head_div : 0, tt.sb ? b : 0);
        };
        if (lane == 0 && ok)
          for (int n = 0; n < n_pieces && n < L::kTermSlots; ++n) issue_piece(n, term_cnt + n);
        int piece = 0;                             // next piece this warp reads

        auto terms = [&](float (&x)[kBN], int kv0) {
#pragma unroll 1
          for (int tt = 0; tt < n_staged; ++tt) {
#pragma unroll
            for (int half = 0; half < 2; ++half, ++piece, ++term_cnt) {
              const int slot = term_cnt % L::kTermSlots;
              if (ok) ok = mbar_wait(bar_term_full(wi, slot), (term_cnt / L::kTermSlots) & 1u, abort_flag);
              if (ok) {
                // this lane's row of the piece: 64 keys = 8 chunks of 16 bytes, 128-byte swizzle
                const uint32_t line = term_smem + slot * L::kTermPieceBytes + lane * 128;
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                  const uint4 v = lds128(line + ((c8 ^ (lane & 7)) << 4));
                  const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float& x0 = x[64 * half + 8 * c8 + 2 * e];
                    float& x1 = x[64 * half + 8 * c8 + 2 * e + 1];
                    fma2(x0, x1, unpack_lo<kBf16>(wv[e]), unpack_hi<kBf16>(wv[e]), fs.coef, fs.coef, x0, x1);
                  }
                }
              }
              __syncwarp();
              if (lane == 0 && ok && piece + L::kTermSlots < n_pieces) {
                fence_proxy_async_smem();          // the warp's reads of the slot precede the copy
                issue_piece(piece + L::kTermSlots, term_cnt + L::kTermSlots);
              }
            }
          }
          // terms that cannot be staged (fp32, a key-padding row, unaligned) are read directly
          if (qi < p.Sq) {
            if (p.bias.ptr && !p.bias.staged) add_score_term<kBf16>(x, p.bias, b, h, qi, kv0, p.Sk, fs.coef);
            if (p.mask.ptr && !p.mask.staged) add_score_term<kBf16>(x, p.mask, b, h, qi, kv0, p.Sk, fs.coef);
          }
        };
        for (int j = 0; j < nt && ok; ++j, ++it_cnt) {
          ok = mbar_wait(bar_s_full(t), it_cnt & 1u, abort_flag);
          if (!ok) break;
          softmax_tile_row<D, kBf16, kFeat>(tS, tO, it.j0 + j, j > 0, p, row_lim, sc, prescale, m, l, [] {},
                                            [&](int hh) { mbar_arrive(bar_p_full(t, hh)); }, terms, keep);
          if (drop_on && j + 1 < nt) draw_keep(it.j0 + j + 1);
        }
      } else {
        for (int j = 0; j < nt && ok; ++j, ++it_cnt) {
          ok = mbar_wait(bar_s_full(t), it_cnt & 1u, abort_flag);
          if (!ok) break;
          softmax_tile_row<D, kBf16, kFeat>(tS, tO, it.j0 + j, j > 0, p, row_lim, sc, prescale, m, l, [] {},
                                            [&](int hh) { mbar_arrive(bar_p_full(t, hh)); },
                                            DirectTerms<kBf16>{p, b, h, qi, fs.coef}, keep);
          if (drop_on && j + 1 < nt) draw_keep(it.j0 + j + 1);
        }
      }

      // ---- epilogue: O / l -> 16 bit -> swizzled shared memory -> TMA store; LSE -------------
      // (a split-KV part instead goes to the partial buffer in fp32, row by row)
      if (ok) ok = mbar_wait(bar_o_full(t), o_cnt & 1u, abort_flag);   // once per item, work or not
      ++o_cnt;
      // One 64-column block at a time through this tile's 16 KiB staging block. O_t is handed
      // back to the MMA warp as soon as its last columns have been read out of tensor memory.
      const float inv = (ok && tile_valid) ? epilogue_stats<kFeat>(p, b_out, h, qi, sc, m, l) : 0.f;
      uint8_t* stage_gen = smem_gen + L::kOOff + t * L::kBlockBytes;
      tc_fence_after();
#pragma unroll
      for (int blk = 0; blk < D / 64; ++blk) {
        // the previous TMA store out of the staging block has finished reading it
        if (r == 0) tma_store_wait_read0();
        named_bar_sync(1 + t, kBM);
        uint32_t o[64];
        if (nt > 0) {
          tmem_ld32(tO + blk * 64, reinterpret_cast<uint32_t(&)[32]>(o[0]));
          tmem_ld32(tO + blk * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(o[32]));
          tc_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 64; ++c) o[c] = 0u;
        }
        if (blk == D / 64 - 1) {
          tc_fence_before();
          mbar_arrive(bar_o_free(t));
        }
        if (ok && tile_valid) {
          if (p.part_o) {   // split-KV part: fp32, rounded to 16 bit once, by the merge
            if (qi < p.Sq) store_partial_row(partial_row<D>(p, b_out, h, qi) + blk * 64, o, inv);
          } else {
            epilogue_block<kBf16>(o, stage_gen, r, inv);
            fence_proxy_async_smem();
          }
        }
        named_bar_sync(1 + t, kBM);
        if (ok && tile_valid && r == 0 && !*abort_flag && !p.part_o) {
          tma_store_5d(&tmO1, sO + t * L::kBlockBytes, 0, it.q0 + t * kBM, blk, h, b_out);
          tma_store_commit();
        }
      }
      // No early exit when a wait has given up: a thread that left alone would strand the rest
      // of its tile at the (unbounded) named barriers of the next epilogue. With `ok` false the
      // remaining items cost only those barriers: the loops and waits above are skipped.
    }
    if (r == 0) tma_store_wait_read0();
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
  using L = FwdSmem<D, kFeat && D == 64>;
  auto kern = fwd_kernel<D, kBf16, kCausal, kFeat>;
  static bool smem_opted_in[64] = {};
  cudaError_t e = opt_in_dynamic_smem(kern, L::kDynamicBytes, smem_opted_in);
  if (e != cudaSuccess) return e;
  const long long items = static_cast<long long>(a.kp.n_qblk) * a.kp.B * a.kp.Hq * a.kp.n_splits;
  if (items <= 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>(items < sm_count() ? items : sm_count());
  kern<<<grid, kThreads, L::kDynamicBytes, stream>>>(a.tmQ, a.tmK, a.tmV, a.tmO1, a.tmBias, a.tmMask, a.kp);
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
    case 256: return launch_fwd256(a, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fa2
