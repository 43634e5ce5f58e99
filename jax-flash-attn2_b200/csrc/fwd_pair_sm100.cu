// Forward attention kernel for sm_100a, head dim 128, grouped query heads, on CTA pairs.
//
// Same job as fwd_kernel (fwd_sm100.cu; it replaces _attn_fwd / _attn_fwd_inner of the reference,
// jax_flash_attn2/flash_attention_triton/_forward_triton.py:60-164, 213-459) for the plain case
// (no bias, mask or dropout) when the number of query heads per key/value head is even.
//
// The single-CTA kernel is bound by shared-memory bandwidth: per K/V tile the MMAs read 96 KiB of
// operands and the TMA unit writes 32 KiB. Two query heads of one group read the same K and V, so
// two CTAs (a cluster of two) run them together with 2-CTA MMAs (tcgen05, cta_group::2):
//   * CTA r of the pair owns query head 2g + r: its own Q tiles, S / P / O in its own tensor
//     memory, its own softmax warps and epilogue, exactly as in the single-CTA kernel;
//   * every K tile is loaded half by each CTA (64 of its 128 keys), every V tile half by each CTA
//     (64 of its 128 head dims): the B operand of an M = 256 MMA is read half from each CTA's
//     shared memory, so a CTA's K/V traffic into and out of shared memory halves;
//   * one thread of the even CTA issues all MMAs of the pair. It learns that both CTAs' loads have
//     landed and that both CTAs' softmax warps have handed over P through mbarriers in the even
//     CTA's shared memory (the odd CTA arrives there remotely; its loads count their bytes there),
//     and it tells both CTAs that S / O are ready or that a K/V slot is free with commits that
//     arrive on the same barrier in both CTAs.
// Every CTA fetches its own pieces with ordinary (non-multicast) tensor copies.
// Roles, registers, tensor-memory columns and the per-row softmax are those of fwd_kernel.
#include "fwd_launch.cuh"
#include "fwd_row.cuh"
#include "launch_util.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

constexpr int kD = 128;
constexpr int kTiles = 2;           // query tiles per CTA (they share the K/V stream)
constexpr int kPairThreads = 384;
constexpr int kPairRegsSoftmax = 208;
constexpr int kPairRegsOther = 88;

struct PairSmem {
  static constexpr int kQTileBytes = kBM * kD * 2;        // 32 KiB: two [128][64] blocks
  static constexpr int kHalfBytes = kBN * kD;             // 16 KiB: half of a K or V tile
  static constexpr int kKBlockBytes = 64 * 128;           // K half: two [64 keys][64 dims] blocks
  static constexpr int kStages = 8;
  static constexpr int kQOff = 0;
  static constexpr int kOOff = kQOff + kTiles * kQTileBytes;      // O staging: one 64-column block per tile
  static constexpr int kKVOff = kOOff + kTiles * kBlockBytes;
  static constexpr int kBarOff = kKVOff + kStages * kHalfBytes;
  // barriers: q_full[2], q_free[2], kv_full[S], kv_empty[S], s_full[2], p_full[2][2], o_full[2], o_free[2]
  static constexpr int kNumBars = 4 + 2 * kStages + 2 + 2 * kPSplit + 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;
  static_assert(kDynamicBytes <= 232448, "shared memory budget exceeded");
};

// One work item of a pair: 256 query rows of two adjacent query heads of one key/value head.
struct PairItem {
  int b, h, hk, q0;
  int sq, sk;
  int n_tiles[kTiles];
  int n_max;
};

template <bool kCausal>
__device__ __forceinline__ void decode_pair_item(const FwdKernelParams& p, int w, int rank, PairItem& it) {
  const int hp = p.Hq >> 1;              // head pairs per batch element
  const int nbh = p.B * hp;
  const int qb_rank = w / nbh;
  const int bh = w - qb_rank * nbh;
  const int qblk = kCausal ? (p.n_qblk - 1 - qb_rank) : qb_rank;   // causal: longest blocks first
  it.b = bh / hp;
  it.h = 2 * (bh - it.b * hp) + rank;
  it.hk = it.h / p.G;
  it.q0 = qblk * (kBM * kTiles);
  it.sq = p.Sq;
  it.sk = p.Sk;
  if (p.seqlens != nullptr) {
    const int len = max(0, min(__ldg(p.seqlens + it.b), p.Sq));
    it.sq = len;
    it.sk = min(len, p.Sk);
  }
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
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
  }
  it.n_max = max(it.n_tiles[0], it.n_tiles[1]);
}

}  // namespace

template <bool kBf16, bool kCausal>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKh,
                const __grid_constant__ CUtensorMap tmVh, const __grid_constant__ CUtensorMap tmO1,
                const FwdKernelParams p) {
  using L = PairSmem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // the same offset in both CTAs
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
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs of the pair
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int total_items = p.n_qblk * p.B * (p.Hq >> 1);
  // barriers of the even CTA, as the odd CTA addresses them
  auto at_leader = [&](uint32_t bar) { return mapa_shared(bar, 0); };

  // ---- set-up ---------------------------------------------------------------------------------
  if (tid == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_q_full(t), 1);                  // even CTA: expect_tx for both CTAs' Q tiles
      mbar_init(bar_q_free(t), 1);
      mbar_init(bar_s_full(t), 1);
      for (int hh = 0; hh < kPSplit; ++hh) mbar_init(bar_p_full(t, hh), 2 * kBM);   // rows of both CTAs
      mbar_init(bar_o_full(t), 1);
      mbar_init(bar_o_free(t), 2 * kBM);
    }
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKh);
    tma_prefetch_desc(&tmVh);
    tma_prefetch_desc(&tmO1);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers exist before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColO = 256;

  if (warp >= 8) setmaxnreg_dec<kPairRegsOther>();
  if (warp >= 10) {
    // idle
  } else if (warp == 9) {
    // =========================== TMA producer (both CTAs) ====================================
    if (lane == 0) {
      bool ok = true;
      uint32_t kv_count = 0;
      uint32_t item_idx = 0;
      for (int w = pair_id; w < total_items && ok; w += n_pairs, ++item_idx) {
        PairItem it;
        decode_pair_item<kCausal>(p, w, rank, it);
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
          ok = ok && mbar_wait(bar_q_free(t), (item_idx & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          if (leader) mbar_arrive_expect_tx(bar_q_full(t), 2 * L::kQTileBytes);
          tma_load_5d_pair(sQ + t * L::kQTileBytes, &tmQ, at_leader(bar_q_full(t)), 0, it.q0 + t * kBM, 0,
                           it.h, it.b);
        }
        for (int i = 0; i < 2 * it.n_max && ok; ++i, ++kv_count) {
          const int slot = kv_count % L::kStages;
          const uint32_t round = kv_count / L::kStages;
          ok = mbar_wait(bar_kv_empty(slot), (round & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          if (leader) mbar_arrive_expect_tx(bar_kv_full(slot), 2 * L::kHalfBytes);
          const int key0 = (i >> 1) * kBN;
          if ((i & 1) == 0)      // K: this CTA's 64 keys of the tile, both 64-dim blocks
            tma_load_5d_pair(sKV + slot * L::kHalfBytes, &tmKh, at_leader(bar_kv_full(slot)), 0,
                             key0 + 64 * static_cast<int>(rank), 0, it.hk, it.b);
          else                   // V: all 128 keys, this CTA's 64-dim block
            tma_load_5d_pair(sKV + slot * L::kHalfBytes, &tmVh, at_leader(bar_kv_full(slot)), 0, key0,
                             static_cast<int>(rank), it.hk, it.b);
        }
      }
      if (!ok) atomicOr(p.status, 1);
    }
    __syncwarp();
  } else if (warp == 8) {
    // =========================== MMA issuer (even CTA only) ==================================
    if (leader) {
      constexpr uint32_t idesc_s = make_idesc(kBf16, 2 * kBM, kBN, false, false);
      constexpr uint32_t idesc_o = make_idesc(kBf16, 2 * kBM, kD, false, true);
      bool ok = true;
      const uint64_t dQ0 = make_sdesc(sQ, 16, 1024);
      const uint64_t dK0 = make_sdesc(sKV, 16, 1024);                  // K half, K-major: [64 keys][64] blocks
      const uint64_t dV0 = make_sdesc(sKV, kBlockBytes, 1024);         // V half, MN-major: one [128 keys][64] block
      auto issue_s = [&](int t, int slot) {
        const uint64_t a0 = sdesc_advance(dQ0, t * L::kQTileBytes);
        const uint64_t b0 = sdesc_advance(dK0, slot * L::kHalfBytes);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t offa = (k >> 2) * kBlockBytes + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * L::kKBlockBytes + (k & 3) * 32;
          mma_ss_pair_e(tmem_base + kColS + t * kBN, sdesc_advance(a0, offa), sdesc_advance(b0, offb),
                        idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit_pair_e(bar_s_full(t));
      };
      auto issue_o = [&](int t, int slot, bool first, int hh) {
        const uint64_t b0 = sdesc_advance(dV0, slot * L::kHalfBytes);
#pragma unroll
        for (int k = hh * (kPCols / 16); k < (hh + 1) * (kPCols / 16); ++k) {
          mma_ts_pair_e(tmem_base + kColO + t * kD, tmem_base + kColS + t * kBN + k * 8,
                        sdesc_advance(b0, k * 2048), idesc_o, (first && k == 0) ? 0u : 1u);
        }
      };

      uint32_t kv_count = 0;
      uint32_t it_cnt[kTiles] = {0, 0};
      uint32_t item_idx = 0;
      for (int w = pair_id; w < total_items && ok; w += n_pairs, ++item_idx) {
        PairItem it;
        decode_pair_item<kCausal>(p, w, 0, it);   // tile counts are the same for both CTAs
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
          ok = ok && mbar_wait_warp(bar_q_full(t), item_idx & 1u, abort_flag);
          if (ok && it.n_tiles[t] == 0) {
            mma_commit_pair_e(bar_q_free(t));
            ok = mbar_wait_warp(bar_o_free(t), (item_idx & 1u) ^ 1u, abort_flag);
            if (ok) mma_commit_pair_e(bar_o_full(t));
          }
        }
        if (!ok || it.n_max == 0) continue;
        {
          const int slot = kv_count % L::kStages;
          ok = mbar_wait_warp(bar_kv_full(slot), (kv_count / L::kStages) & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < kTiles; ++t) {
            if (it.n_tiles[t] > 0) {
              issue_s(t, slot);
              if (it.n_tiles[t] == 1) mma_commit_pair_e(bar_q_free(t));
            }
          }
          mma_commit_pair_e(bar_kv_empty(slot));
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
          for (int t = 0; t < kTiles; ++t) {
            if (j < it.n_tiles[t]) {
              if (j == 0) {
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
                if (j + 2 == it.n_tiles[t]) mma_commit_pair_e(bar_q_free(t));
              } else {
                mma_commit_pair_e(bar_o_full(t));
              }
            }
          }
          if (!ok) break;
          mma_commit_pair_e(bar_kv_empty(slot_v));
          if (has_next) mma_commit_pair_e(bar_kv_empty(slot_k));
          kv_count += has_next ? 2 : 1;
        }
      }
      if (!ok && lane == 0) atomicOr(p.status, 2);
    }
    __syncwarp();
  } else {
    // =========================== softmax + epilogue (both CTAs) ==============================
    setmaxnreg_inc<kPairRegsSoftmax>();
    const int t = warp >> 2;
    const int r = tid & (kBM - 1);
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + t * kBN;
    const uint32_t tO = tmem_base + lane_base + kColO + t * kD;
    const float sc = p.scale_log2;
    // hand-overs to the MMA warp go to the even CTA's barriers
    const uint32_t p_full0 = at_leader(bar_p_full(t, 0)), p_full1 = at_leader(bar_p_full(t, 1));
    const uint32_t o_free_l = at_leader(bar_o_free(t));
    uint32_t it_cnt = 0, o_cnt = 0;
    bool ok = true;

    for (int w = pair_id; w < total_items; w += n_pairs) {
      PairItem it;
      decode_pair_item<kCausal>(p, w, rank, it);
      const int b = it.b, h = it.h;
      const int qi = it.q0 + t * kBM + r;
      const int nt = it.n_tiles[t];
      const bool tile_valid = (it.q0 + t * kBM) < p.Sq;
      const int row_lim = qi < it.sq ? (kCausal ? min(it.sk - 1, qi + p.causal_off) : it.sk - 1) : -1;
      float m = -INFINITY, l = 0.f;

      for (int j = 0; j < nt && ok; ++j, ++it_cnt) {
        ok = mbar_wait(bar_s_full(t), it_cnt & 1u, abort_flag);
        if (!ok) break;
        softmax_tile_row<kD, kBf16, false>(tS, tO, j, j > 0, p, row_lim, sc, m, l, [] {},
                                           [&](int hh) { mbar_arrive_cluster(hh ? p_full1 : p_full0); },
                                           DirectTerms<kBf16>{p, b, h, qi}, KeepBitsDropout{false, make_uint4(0u, 0u, 0u, 0u)});
      }

      if (ok) ok = mbar_wait(bar_o_full(t), o_cnt & 1u, abort_flag);
      ++o_cnt;
      const float inv = (ok && tile_valid) ? epilogue_stats<false>(p, b, h, qi, sc, m, l) : 0.f;
      uint8_t* stage_gen = smem_gen + L::kOOff + t * kBlockBytes;
      tc_fence_after();
#pragma unroll
      for (int blk = 0; blk < kD / 64; ++blk) {
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
        if (blk == kD / 64 - 1) {
          tc_fence_before();
          mbar_arrive_cluster(o_free_l);
        }
        if (ok && tile_valid) {
          epilogue_block<kBf16>(o, stage_gen, r, inv);
          fence_proxy_async_smem();
        }
        named_bar_sync(1 + t, kBM);
        if (ok && tile_valid && r == 0 && !*abort_flag) {
          tma_store_5d(&tmO1, sO + t * kBlockBytes, 0, it.q0 + t * kBM, blk, h, b);
          tma_store_commit();
        }
      }
    }
    if (r == 0) tma_store_wait_read0();
    if (!ok && r == 0) atomicOr(p.status, 4);
  }

  // ---- teardown: neither CTA may leave while the other can still touch its shared or tensor
  // memory (remote arrivals, the pair MMAs) ------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// launcher
// ---------------------------------------------------------------------------------------------
template <bool kBf16, bool kCausal>
static cudaError_t launch_pair_one(const FwdLaunch& a, cudaStream_t stream) {
  using L = PairSmem;
  auto kern = fwd_pair_kernel<kBf16, kCausal>;
  static bool smem_opted_in[64] = {};
  cudaError_t e = opt_in_dynamic_smem(kern, L::kDynamicBytes, smem_opted_in);
  if (e != cudaSuccess) return e;
  const long long items = static_cast<long long>(a.kp.n_qblk) * a.kp.B * (a.kp.Hq / 2);
  if (items <= 0) return cudaSuccess;
  // persistent: one pair of CTAs per pair of SMs that can hold a cluster at the same time
  static int max_clusters[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (max_clusters[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count()), 1, 1);
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamicBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2;
    max_clusters[dev] = n;
  }
  const long long pairs = items < max_clusters[dev] ? items : max_clusters[dev];
  kern<<<static_cast<unsigned>(2 * pairs), kPairThreads, L::kDynamicBytes, stream>>>(a.tmQ, a.tmKh, a.tmVh,
                                                                                      a.tmO1, a.kp);
  return cudaGetLastError();
}

cudaError_t launch_fwd_pair(const FwdLaunch& a, cudaStream_t stream) {
  const int key = (a.bf16 ? 2 : 0) | (a.causal ? 1 : 0);
  switch (key) {
    case 0: return launch_pair_one<false, false>(a, stream);
    case 1: return launch_pair_one<false, true>(a, stream);
    case 2: return launch_pair_one<true, false>(a, stream);
    default: return launch_pair_one<true, true>(a, stream);
  }
}

}  // namespace fa2
