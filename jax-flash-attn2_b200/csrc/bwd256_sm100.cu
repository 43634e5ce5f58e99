// Backward attention kernels for head dim 256 on sm_100a.
//
// Same job and reference counterparts as bwd_sm100.cu (_attn_bwd_preprocess, _attn_bwd and the
// per-group dk / dv reduction of jax_flash_attn2/flash_attention_triton/_backward_triton.py:79-147,
// 150-945, 1156-1161). At D = 256 the dK and dV accumulators of one 128-key tile would fill
// tensor memory on their own (2 x 256 columns), and full-width K, V, Q and dO tiles do not fit
// shared memory next to each other, so the plan changes:
//   * one CTA owns (batch, kv head, 128-key tile, HALF of the head dim): it accumulates
//     dK[:, half] and dV[:, half] (128 columns each) and produces dQ[:, half]; the two halves are
//     two CTAs, each recomputing S and dP over the full head dim (14 instead of 10 GEMM units);
//   * a step covers 64 query rows: S^T = K Q^T and dP^T = V dO^T are [128 keys x 64 queries];
//   * dQ is produced transposed, dQ^T[:, half] = K[:, half]^T dS^T ([128 dims x 64 queries]), so
//     that every MMA keeps M = 128.
//   * only the CTA's own half of K stays in shared memory (it is the MN-major A operand of
//     dQ^T); the other half, which S^T alone contracts over, is copied once into tensor memory
//     and read from there (TS MMAs). That makes room for a second Q stage, so S^T of the next
//     step overlaps the dS phase of the current one.
// Tensor memory: S^T 64 | dP^T 64 | dQ^T 64 | other half of K 64 | dK_half 128 | dV_half 128.
// Shared memory: K half 32 KiB, V 64 KiB, Q 2 x 32 KiB, dO 32 KiB (single buffer), dS^T 16 KiB,
// dQ staging 2 x 8 KiB.
#include "bwd_common.cuh"
#include "bwd_launch.cuh"
#include "launch_util.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

constexpr int kD = 256;
constexpr int kBQ = 64;      // query rows per step
constexpr int kBK = 128;     // keys per CTA
constexpr int kThreads256 = 512;
constexpr int kRegsDrain256 = 152;   // 2 * 128 + 152 + 104 = 4 * 128 registers per scheduler lane
constexpr int kRegsOther256 = 104;

struct BSmem256 {
  static constexpr int kKVBytes = kBK * kD * 2;     // 64 KiB: 4 blocks of [128][64]
  static constexpr int kKhBytes = kKVBytes / 2;     // 32 KiB: this CTA's half of K (2 blocks)
  static constexpr int kQBytes = kBQ * kD * 2;      // 32 KiB: 4 blocks of [64][64]
  static constexpr int kKBlock = kBK * 128;         // 16 KiB
  static constexpr int kQBlock = kBQ * 128;         // 8 KiB
  static constexpr int kdSBytes = kBK * kBQ * 2;    // 16 KiB: one [128][64] block
  static constexpr int kChunkBytes = 16 * 128 * 4;  // 16 query columns x 128 dims, fp32
  // K: only the half of the head dim this CTA produces dQ for stays in shared memory; the other
  // half (needed for S^T alone) is copied once into tensor memory and read from there as the A
  // operand, which is what makes room for the second Q stage.
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kKhBytes;
  static constexpr int kQOff = kVOff + kKVBytes;            // 2 stages
  static constexpr int kdOOff = kQOff + 2 * kQBytes;        // 1 stage
  static constexpr int kdSOff = kdOOff + kQBytes;
  static constexpr int kStageOff = kdSOff + kdSBytes;
  static constexpr int kStatsOff = kStageOff + 2 * kChunkBytes;   // 2 stages x (-lse*log2e [64], delta [64])
  static constexpr int kBarOff = kStatsOff + 2 * 512;
  static constexpr int kNumBars = 16;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = (kTotal + 1024 <= kMaxDynSmem) ? kTotal + 1024 : kMaxDynSmem;
  static_assert(kTotal + 1024 <= kMaxDynSmem, "shared memory budget exceeded");
};

}  // namespace

// dq accumulator layout at D = 256: [B, Hq, ceil(Sq/64), 2 halves, 16 (query/4), 128 dims, 4 queries].
template <bool kBf16>
__global__ void __launch_bounds__(256)
bwd256_dq_convert(const float* __restrict__ dq_acc, uint16_t* __restrict__ dq, long long sb,
                  long long ss, long long sh, int Sq, int Hq, int nQ64, float scale_in,
                  const unsigned* __restrict__ do_absmax_bits, int blk_real) {
  const float scale = scale_in / (kBf16 ? 1.f : do_scale_from_bits(do_absmax_bits));
  const int i = blockIdx.x % nQ64;   // one-dimensional grid, tile index fastest
  const int bh = blockIdx.x / nQ64;
  const int b = bh / Hq, h = bh - b * Hq;
  const int tid = threadIdx.x;
  const int dpair = tid & 63;                 // dims 2*dpair, 2*dpair + 1 of a half
  const float4* src = reinterpret_cast<const float4*>(dq_acc) +
                      (static_cast<long long>(bh) * nQ64 + i) * (kBQ * kD / 4);
  // 32 (half, query/4) slabs of [128 dims][4 queries]; four slabs per pass
#pragma unroll 1
  for (int pass = 0; pass < 8; ++pass) {
    const int slab = pass * 4 + (tid >> 6);
    const int half = slab >> 4, c4 = slab & 15;
    const float4 x = src[slab * 128 + 2 * dpair];
    const float4 y = src[slab * 128 + 2 * dpair + 1];
    const float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
    // a padded head dim keeps blk_real real columns at the start of every 64-column block
    const int col = half * 128 + 2 * dpair;          // column in the padded head dim
    const int blk = col >> 6, x_in = col & 63;
    const int pair_real = (blk * blk_real + x_in) >> 1;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = i * kBQ + c4 * 4 + e;
      if (row < Sq && x_in < blk_real)
        reinterpret_cast<uint32_t*>(dq + b * sb + row * ss + h * sh)[pair_real] =
            pack2<kBf16>(xs[e] * scale, ys[e] * scale);
    }
  }
}

template <bool kBf16, bool kCausal, bool kFeat>
__global__ void __launch_bounds__(kThreads256, 1)
bwd256_main_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                   const float* __restrict__ stats, const BwdKernelParams p) {
  using L = BSmem256;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t pad = smem_base - smem_u32(smem_raw);
  if (pad + L::kTotal > static_cast<uint32_t>(L::kDynamicBytes)) {
    if (threadIdx.x == 0) atomicOr(p.status, 64);
    return;
  }
  uint8_t* smem_gen = smem_raw + pad;
  const uint32_t sK = smem_base + L::kKOff, sV = smem_base + L::kVOff;
  const uint32_t sQ = smem_base + L::kQOff, sdO = smem_base + L::kdOOff;
  const uint32_t sdS = smem_base + L::kdSOff, sStats = smem_base + L::kStatsOff;
  const uint32_t bars = smem_base + L::kBarOff;
  const uint32_t bar_kv_full = bars;
  auto bar_q_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_q_empty = [&](int s) { return bars + 8u * (12 + s); };
  const uint32_t bar_kx_full = bars + 8u * 14, bar_kx_done = bars + 8u * 15;
  const uint32_t bar_do_full = bars + 24, bar_do_empty = bars + 32;
  const uint32_t bar_s_full = bars + 40, bar_p_full = bars + 48;
  const uint32_t bar_dp_full = bars + 56, bar_ds_full = bars + 64;
  const uint32_t bar_dq_full = bars + 72, bar_dq_drained = bars + 80, bar_dkv_full = bars + 88;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- work item: (batch, kv head, key tile, half of the head dim) ---------------------------
  const int half = blockIdx.x & 1;
  const int rest = blockIdx.x >> 1;
  int n, bhk;
  bwd_work_item(rest, p.B * p.Hkv, p.n_kvblk, p.sched_groups, p.dq_order != nullptr, bhk, n);
  const int b = bhk / p.Hkv;
  const int hk = bhk - b * p.Hkv;
  const int nQ64 = (p.Sq + kBQ - 1) / kBQ;      // tiles in the accumulator layout
  const int nQ128 = (p.Sq + 127) / 128;
  // rows of this batch element that take part: the problem's, or its seqlens entry
  int sq_b = p.Sq, sk_b = p.Sk;
  if (p.seqlens != nullptr) {
    sq_b = max(0, min(__ldg(p.seqlens + b), p.Sq));
    sk_b = min(sq_b, p.Sk);
  }
  const int nQ64_b = (sq_b + kBQ - 1) / kBQ;
  int i_start = 0;
  if (kCausal) {
    const int first_row = n * kBK - p.causal_off;   // first query row that sees key n*128
    i_start = first_row > 0 ? first_row / kBQ : 0;
  }
  if (i_start > nQ64_b) i_start = nQ64_b;
  const int nI = nQ64_b - i_start;
  const int T = (n * kBK < sk_b) ? nI * p.G : 0;    // steps of this CTA (none: dK = dV = 0)
  const bool dead_keys = n * kBK + kBK > sk_b;      // some key rows lie past the end

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv_full, 1);
    for (int st = 0; st < 2; ++st) {
      mbar_init(bar_q_full(st), 1);
      mbar_init(bar_q_empty(st), 1);
    }
    mbar_init(bar_kx_full, 1);
    mbar_init(bar_kx_done, 128);
    mbar_init(bar_do_full, 1);
    mbar_init(bar_do_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, 256);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_ds_full, 256);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_drained, 128);
    mbar_init(bar_dkv_full, 1);
    fence_mbar_init();
  }
  if (warp == 13 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // tensor memory: S^T 64 | dP^T 64 | dQ^T 64 | other half of K (16 bit, 128 dims) 64 | dK 128 | dV 128
  constexpr uint32_t kColS = 0, kColdP = 64, kColdQ = 128, kColKx = 192, kColdK = 256, kColdV = 384;

  auto step_coords = [&](int it, int& h, int& i) {
    const int g = it / nI;
    i = i_start + (it - g * nI);
    h = hk * p.G + g;
  };

  if (warp >= 12) setmaxnreg_dec<kRegsOther256>();
  if (warp >= 14) {
    // idle
  } else if (warp == 13) {
    // =========================== TMA producer ================================================
    if (lane == 0 && T > 0) {
      // K arrives in halves of the head dim (the K map's box is two 64-column blocks): this
      // CTA's half stays in its own buffer, the other half lands in the second Q stage, from
      // where the P/dS warps move it into tensor memory before that stage is first used.
      mbar_arrive_expect_tx(bar_kv_full, L::kKhBytes + L::kKVBytes);
      tma_load_5d(sK, &tmK, bar_kv_full, 0, n * kBK, 2 * half, hk, b);
      tma_load_5d(sV, &tmV, bar_kv_full, 0, n * kBK, 0, hk, b);
      mbar_arrive_expect_tx(bar_kx_full, L::kKhBytes);
      tma_load_5d(sQ + L::kQBytes, &tmK, bar_kx_full, 0, n * kBK, 2 * (1 - half), hk, b);
      bool ok = true;
      for (int it = 0; it < T && ok; ++it) {
        const int stg = it & 1;
        int h, i;
        step_coords(it, h, i);
        if (it == 1) ok = mbar_wait(bar_kx_done, 0, abort_flag);   // stage 1 no longer holds K
        if (ok) ok = mbar_wait(bar_q_empty(stg), ((it >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_q_full(stg), L::kQBytes + 512);
        tma_load_5d(sQ + stg * L::kQBytes, &tmQ, bar_q_full(stg), 0, i * kBQ, 0, h, b);
        const float* st =
            stats + ((static_cast<long long>(b) * p.Hq + h) * nQ128 + (i >> 1)) * 256 + (i & 1) * 64;
        bulk_load_1d(sStats + stg * 512, st, 256, bar_q_full(stg));
        bulk_load_1d(sStats + stg * 512 + 256, st + 128, 256, bar_q_full(stg));
        ok = mbar_wait(bar_do_empty, (it & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_do_full, L::kQBytes);
        tma_load_5d(sdO, &tmdO, bar_do_full, 0, i * kBQ, 0, h, b);
      }
      if (!ok) atomicOr(p.status, 8);
    }
    __syncwarp();
  } else if (warp == 12) {
    // =========================== MMA issuer ==================================================
    if (T > 0) {
      constexpr uint32_t idesc_s = make_idesc(kBf16, 128, kBQ, false, false);
      constexpr uint32_t idesc_dkv = make_idesc(kBf16, 128, 128, false, true);
      constexpr uint32_t idesc_dq = make_idesc(kBf16, 128, kBQ, true, true);
      const uint64_t dKh_k = make_sdesc(sK, 16, 1024), dV_k = make_sdesc(sV, 16, 1024);
      const uint64_t dQ_k0 = make_sdesc(sQ, 16, 1024), ddO_k = make_sdesc(sdO, 16, 1024);
      // halves of Q / dO as MN-major B operands: two 64-dim blocks, L::kQBlock apart
      const uint64_t dQ_mn0 = make_sdesc(sQ + 2 * half * L::kQBlock, L::kQBlock, 1024);
      const uint64_t ddO_mn = make_sdesc(sdO + 2 * half * L::kQBlock, L::kQBlock, 1024);
      // this CTA's half of K as MN-major A operand (M = head dim): two 64-dim blocks
      const uint64_t dKh_mn = make_sdesc(sK, L::kKBlock, 1024);
      const uint64_t ddS_k = make_sdesc(sdS, 16, 1024), ddS_mn = make_sdesc(sdS, 16, 1024);
      bool ok = true;

      // D[key, query] = A[key, d] * B[query, d]^T over the full head dim
      auto issue_kd = [&](uint32_t d_col, uint64_t a_desc, uint64_t b_desc) {
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t offa = (k >> 2) * L::kKBlock + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * L::kQBlock + (k & 3) * 32;
          mma_ss_e(tmem_base + d_col, sdesc_advance(a_desc, offa), sdesc_advance(b_desc, offb),
                 idesc_s, k > 0 ? 1u : 0u);
        }
      };
      auto issue_dv = [&](bool first) {
#pragma unroll
        for (int k = 0; k < kBQ / 16; ++k) {
          // P^T for queries [16k, 16k+16): 8 packed columns; queries [0,32) were written by
          // warpgroup 0 at column 0, queries [32,64) by warpgroup 1 at column 32
          const uint32_t a_col = kColS + (k < 2 ? 8 * k : 32 + 8 * (k - 2));
          mma_ts_e(tmem_base + kColdV, tmem_base + a_col, sdesc_advance(ddO_mn, k * 2048), idesc_dkv,
                 (first && k == 0) ? 0u : 1u);
        }
      };
      // S^T[key, query] over the full head dim: this CTA's half of K from shared memory, the
      // other half from tensor memory (8 columns per 16 dims)
      auto issue_s = [&](int stg) {
        const uint64_t q_k = sdesc_advance(dQ_k0, stg * L::kQBytes);
#pragma unroll
        for (int k = 0; k < kD / 32; ++k) {
          const uint32_t offa = (k >> 2) * L::kKBlock + (k & 3) * 32;
          const uint32_t offb = (2 * half + (k >> 2)) * L::kQBlock + (k & 3) * 32;
          mma_ss_e(tmem_base + kColS, sdesc_advance(dKh_k, offa), sdesc_advance(q_k, offb), idesc_s,
                 k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kD / 32; ++k) {
          const uint32_t offb = (2 * (1 - half) + (k >> 2)) * L::kQBlock + (k & 3) * 32;
          mma_ts_e(tmem_base + kColS, tmem_base + kColKx + 8 * k, sdesc_advance(q_k, offb), idesc_s, 1u);
        }
      };
      auto issue_dk = [&](int stg, bool first) {
        const uint64_t q_mn = sdesc_advance(dQ_mn0, stg * L::kQBytes);
#pragma unroll
        for (int k = 0; k < kBQ / 16; ++k)
          mma_ss_e(tmem_base + kColdK, sdesc_advance(ddS_k, k * 32), sdesc_advance(q_mn, k * 2048),
                 idesc_dkv, (first && k == 0) ? 0u : 1u);
      };
      auto issue_dq = [&]() {
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          mma_ss_e(tmem_base + kColdQ, sdesc_advance(dKh_mn, k * 2048), sdesc_advance(ddS_mn, k * 2048),
                 idesc_dq, k > 0 ? 1u : 0u);
      };

      ok = mbar_wait_warp(bar_kv_full, 0, abort_flag);
      if (ok) ok = mbar_wait_warp(bar_kx_done, 0, abort_flag);   // the other half of K is in tensor memory
      if (ok) ok = mbar_wait_warp(bar_q_full(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        mma_commit_e(bar_s_full);
        ok = mbar_wait_warp(bar_do_full, 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        issue_kd(kColdP, dV_k, ddO_k);
        mma_commit_e(bar_dp_full);
      }
      for (int it = 0; it < T && ok; ++it) {
        const uint32_t par = it & 1;
        const int stg = it & 1, nxt = stg ^ 1;
        const bool has_next = it + 1 < T;
        ok = mbar_wait_warp(bar_p_full, par, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_dv(it == 0);
        mma_commit_e(bar_do_empty);
        if (has_next) {
          // S^T of the next step runs while the P/dS warps are still busy with dS of this one; it
          // is issued behind dV, which is the last reader of the P^T columns it overwrites
          ok = mbar_wait_warp(bar_q_full(nxt), ((it + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_s(nxt);
          mma_commit_e(bar_s_full);
        }
        ok = mbar_wait_warp(bar_ds_full, par, abort_flag);
        if (ok && it > 0) ok = mbar_wait_warp(bar_dq_drained, (it - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_dq();
        mma_commit_e(bar_dq_full);
        issue_dk(stg, it == 0);
        mma_commit_e(bar_q_empty(stg));
        if (has_next) {
          ok = mbar_wait_warp(bar_do_full, (it + 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_kd(kColdP, dV_k, ddO_k);
          mma_commit_e(bar_dp_full);
        }
      }
      if (ok) mma_commit_e(bar_dkv_full);
      if (!ok && lane == 0) atomicOr(p.status, 16);
    }
    __syncwarp();
  } else if (warp >= 8) {
    // =========================== dQ^T drain ==================================================
    setmaxnreg_inc<kRegsDrain256>();
    const int r = tid - 256;   // head-dim index inside the half == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tdQ = tmem_base + lane_base + kColdQ;
    bool ok = true;
    // Bit-reproducible dq (p.dq_order, as in bwd_sm100.cu): this key tile adds its part of a dQ
    // tile (64 query rows, this CTA's half of the head dim) when the contributing key tiles above
    // it have, and counts up once its reductions have been performed. Two more barriers per step.
    const bool ordered = p.dq_order != nullptr;
    for (int it = 0; it < T; ++it) {
      int h, i;
      step_coords(it, h, i);
      if (ok) ok = mbar_wait(bar_dq_full, it & 1, abort_flag);
      if (!ok) {
        // No early exit: a thread that left alone would strand the other 127 at the (unbounded)
        // named barriers of the staging loop. Keep in step with them: eight barriers per step.
#pragma unroll 1
        for (int k = 0; k < 8 + (ordered ? 2 : 0); ++k) named_bar_sync(3, 128);
        continue;
      }
      tc_fence_after();
      uint32_t v[kBQ];
      tmem_ld32(tdQ, reinterpret_cast<uint32_t(&)[32]>(v[0]));
      tmem_ld32(tdQ + 32, reinterpret_cast<uint32_t(&)[32]>(v[32]));
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_dq_drained);
      float* dst_tile = p.dq_acc +
                        (((static_cast<long long>(b) * p.Hq + h) * nQ64 + i) * 2 + half) * (kBQ * 128);
      // four counters per 128-row tile of the pre-pass: (64-row half, head-dim half)
      int* turn = ordered ? p.dq_order + ((static_cast<long long>(b) * p.Hq + h) * nQ128 + (i >> 1)) * 4 +
                                (i & 1) * 2 + half
                          : nullptr;
      if (ordered) {
        if (r == 0) {
          const int above = bwd_tile_contributors(kCausal, i, kBQ, sq_b, sk_b, p.n_kvblk, p.causal_off) - 1 - n;
          if (!wait_for_turn(turn, above, abort_flag)) atomicOr(p.status, 256);
        }
        named_bar_sync(3, 128);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int buf = c & 1;
        if (r == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        named_bar_sync(3, 128);
        uint8_t* stage = smem_gen + L::kStageOff + buf * L::kChunkBytes;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int cc = c * 4 + c4;
          *reinterpret_cast<uint4*>(stage + (c4 * 128 + r) * 16) =
              make_uint4(v[4 * cc], v[4 * cc + 1], v[4 * cc + 2], v[4 * cc + 3]);
        }
        fence_proxy_async_smem();
        named_bar_sync(3, 128);
        if (r == 0) {
          bulk_reduce_add_f32(dst_tile + c * (16 * 128), smem_base + L::kStageOff + buf * L::kChunkBytes,
                              L::kChunkBytes);
          tma_store_commit();
        }
      }
      if (ordered) {
        named_bar_sync(3, 128);
        if (r == 0) {
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // performed, not only read
          __threadfence();
          atomicAdd(turn, 1);
        }
      }
    }
    if (r == 0) tma_store_wait_read0();
    if (!ok && r == 0) atomicOr(p.status, 32);
  } else {
    // =========================== P / dS warps + dK, dV epilogue ==============================
    const int w = warp >> 2;            // 0: queries [0,32) of each step, dK; 1: [32,64), dV
    const int r = tid & 127;            // key row inside the tile == TMEM lane
    const int kv = n * kBK + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + 32 * w;
    const uint32_t tdP = tmem_base + lane_base + kColdP + 32 * w;
    uint8_t* ds_row = smem_gen + L::kdSOff + r * 128;
    const float do_scale = kBf16 ? 1.f : do_scale_from_bits(p.do_absmax_bits);
    bool ok = true;

    if (w == 0 && T > 0) {
      // One-time: the half of K that landed in the second Q stage goes into tensor memory, one key
      // row per thread (= lane), two 16-bit values per column in head-dim order: the layout of
      // a 16-bit A operand (the same one P^T is written in).
      ok = mbar_wait(bar_kx_full, 0, abort_flag);
      if (ok) {
        const uint8_t* src = smem_gen + L::kQOff + L::kQBytes;
        uint32_t kx[64];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 v4 = *reinterpret_cast<const uint4*>(src + blk * L::kKBlock + r * 128 +
                                                             ((j ^ (r & 7)) << 4));
            kx[blk * 32 + 4 * j + 0] = v4.x;
            kx[blk * 32 + 4 * j + 1] = v4.y;
            kx[blk * 32 + 4 * j + 2] = v4.z;
            kx[blk * 32 + 4 * j + 3] = v4.w;
          }
        }
        const uint32_t tKx = tmem_base + lane_base + kColKx;
        tmem_st32(tKx, reinterpret_cast<const uint32_t(&)[32]>(kx[0]));
        tmem_st32(tKx + 32, reinterpret_cast<const uint32_t(&)[32]>(kx[32]));
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_kx_done);
      }
    }

    // Dropout keep bits of this key row for the step's 32 query columns, drawn one step ahead (after
    // dS of the previous step has been handed over) so that the Philox rounds overlap the MMAs.
    uint32_t keep_bits[1] = {0xffffffffu};
    auto draw_keep = [&](int step) {
      if constexpr (kFeat) {
        if (p.drop.enabled && step < T) {
          int hh, ii;
          step_coords(step, hh, ii);
          dropout_keep_bits_transposed<32>(p.drop, dropout_bh_index(p.drop, b, hh), kv, ii * kBQ + 32 * w, lane,
                                           keep_bits);
        }
      }
    };
    draw_keep(0);

    for (int it = 0; it < T && ok; ++it) {
      const int stg = it & 1;
      int h, i;
      step_coords(it, h, i);
      const int q_first = i * kBQ + 32 * w;
      const float4* nlse4 = reinterpret_cast<const float4*>(smem_gen + L::kStatsOff + stg * 512) + 8 * w;
      const float4* delta4 = nlse4 + 16;
      ok = mbar_wait(bar_q_full(stg), (it >> 1) & 1, abort_flag);
      if (ok) ok = mbar_wait(bar_s_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (kCausal && (n * kBK + kBK - 1 > i * kBQ + p.causal_off)) || dead_keys;
      // masked iff query index < q_lim: every query for a key past the end
      const int q_lim = kv >= sk_b ? 0x7fffffff : (kCausal ? kv - p.causal_off : -0x7fffffff - 1);

      uint32_t pk[16];
      const uint32_t keep = keep_bits[0];
      {
        uint32_t s[32];
        tmem_ld32(tS, s);
        tc_wait_ld();
        if constexpr (kFeat) {
#pragma unroll
          for (int c = 0; c < 32; ++c) s[c] = __float_as_uint(__uint_as_float(s[c]) * p.scale_log2);
          add_term_column<kBf16, 32>(p.bias, b, h, q_first, kv, p.Sq, p.Sk, s);
          add_term_column<kBf16, 32>(p.mask, b, h, q_first, kv, p.Sq, p.Sk, s);
        }
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 nl = nlse4[c4];
          const float nlv[4] = {nl.x, nl.y, nl.z, nl.w};
#pragma unroll
          for (int k2 = 0; k2 < 2; ++k2) {
            const int c = 4 * c4 + 2 * k2;
            float x0 = __uint_as_float(s[c]), x1 = __uint_as_float(s[c + 1]);
            if constexpr (kFeat) {
              x0 += nlv[2 * k2];      // already scaled, bias and mask added (below the loads)
              x1 += nlv[2 * k2 + 1];
            } else {
              fma2(x0, x1, x0, x1, p.scale_log2, p.scale_log2, nlv[2 * k2], nlv[2 * k2 + 1]);
            }
            float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            if (diag) {
              if (q_first + c < q_lim) p0 = 0.f;
              if (q_first + c + 1 < q_lim) p1 = 0.f;
            }
            pk[c >> 1] = pack2<kBf16>(p0, p1);
          }
        }
      }
      if constexpr (kFeat) {
        if (p.drop.enabled) {
          uint32_t pd[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float a0 = ((keep >> (2 * c)) & 1u) ? unpack_lo<kBf16>(pk[c]) * p.drop.inv_keep : 0.f;
            float a1 = ((keep >> (2 * c + 1)) & 1u) ? unpack_hi<kBf16>(pk[c]) * p.drop.inv_keep : 0.f;
            pd[c] = pack2<kBf16>(a0, a1);
          }
          tmem_st16(tS, pd);
        } else {
          tmem_st16(tS, pk);
        }
      } else {
        tmem_st16(tS, pk);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full);

      ok = mbar_wait(bar_dp_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t dp[32];
        tmem_ld32(tdP, dp);
        tc_wait_ld();
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 dl = delta4[c4];
          const float dlv[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
          for (int k2 = 0; k2 < 2; ++k2) {
            const int c = 4 * c4 + 2 * k2;
            float d0 = __uint_as_float(dp[c]), d1 = __uint_as_float(dp[c + 1]);
            if constexpr (kFeat) {
              d0 = ((keep >> c) & 1u) ? d0 * p.drop.inv_keep : 0.f;
              d1 = ((keep >> (c + 1)) & 1u) ? d1 * p.drop.inv_keep : 0.f;
            }
            float t0, t1;
            add2(t0, t1, d0, d1, -dlv[2 * k2], -dlv[2 * k2 + 1]);
            if constexpr (!kBf16) fma2(t0, t1, t0, t1, do_scale, do_scale, 0.f, 0.f);
            const float p0 = unpack_lo<kBf16>(pk[c >> 1]), p1 = unpack_hi<kBf16>(pk[c >> 1]);
            dp[c >> 1] = pack2<kBf16>(p0 * t0, p1 * t1);
          }
        }
        // dS^T row r, queries [32w, 32w + 32): chunks 4w .. 4w+3 of the row's 128-byte line
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = 4 * w + q4;
          *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(dp[4 * q4], dp[4 * q4 + 1], dp[4 * q4 + 2], dp[4 * q4 + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_ds_full);
        if constexpr (kFeat) {
          // both halves of the head dim compute the same dS^T: the first one reports it
          if (p.dbias.ptr != nullptr && half == 0)
            add_bias_grad<kBf16, 32>(p.dbias, b, h, q_first, kv, p.Sq, p.Sk, dp, do_scale);
        }
      }
      draw_keep(it + 1);
    }

    // ---- epilogue: warpgroup 0 writes dK[:, half] (scaled), warpgroup 1 writes dV[:, half] ----
    if (ok && T > 0) ok = mbar_wait(bar_dkv_full, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      const uint32_t tAcc = tmem_base + lane_base + (w == 0 ? kColdK : kColdV);
      const float f = (w == 0) ? p.scale / do_scale : 1.f;
      uint8_t* stage = smem_gen + (w == 0 ? L::kQOff : L::kdOOff);   // 32 KiB each, free by now
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t a[32];
        if (T > 0) {
          tmem_ld32(tAcc + c * 32, a);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) a[k] = 0u;
        }
        uint8_t* line = stage + (c >> 1) * L::kKBlock + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack2<kBf16>(__uint_as_float(a[8 * q4 + 0]) * f, __uint_as_float(a[8 * q4 + 1]) * f);
          v.y = pack2<kBf16>(__uint_as_float(a[8 * q4 + 2]) * f, __uint_as_float(a[8 * q4 + 3]) * f);
          v.z = pack2<kBf16>(__uint_as_float(a[8 * q4 + 4]) * f, __uint_as_float(a[8 * q4 + 5]) * f);
          v.w = pack2<kBf16>(__uint_as_float(a[8 * q4 + 6]) * f, __uint_as_float(a[8 * q4 + 7]) * f);
          const int chunk = (c & 1) * 4 + q4;
          *reinterpret_cast<uint4*>(line + ((chunk ^ (r & 7)) << 4)) = v;
        }
      }
      fence_proxy_async_smem();
    }
    named_bar_sync(1 + w, 128);
    if (ok && r == 0 && !*abort_flag) {
      tma_store_5d(w == 0 ? &tmdK : &tmdV, w == 0 ? sQ : sdO, 0, n * kBK, 2 * half, hk, b);
      tma_store_commit();
      tma_store_wait_read0();
    }
    if (!ok && r == 0) atomicOr(p.status, 128);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool kBf16, bool kCausal, bool kFeat>
static cudaError_t launch256_main(const BwdLaunch& a, cudaStream_t stream) {
  using L = BSmem256;
  auto kern = bwd256_main_kernel<kBf16, kCausal, kFeat>;
  static bool smem_opted_in[64] = {};
  cudaError_t e = opt_in_dynamic_smem(kern, L::kDynamicBytes, smem_opted_in);
  if (e != cudaSuccess) return e;
  const long long nblocks = 2LL * a.kp.n_kvblk * a.kp.B * a.kp.Hkv;
  kern<<<static_cast<unsigned>(nblocks), kThreads256, L::kDynamicBytes, stream>>>(
      a.tmQ, a.tmK, a.tmV, a.tmdO, a.tmdK, a.tmdV, a.delta, a.kp);
  return cudaGetLastError();
}

template <bool kBf16>
static cudaError_t launch256_all(const BwdLaunch& a, cudaStream_t stream) {
  const BwdKernelParams& kp = a.kp;
  const int nQ128 = (kp.Sq + 127) / 128, nQ64 = (kp.Sq + kBQ - 1) / kBQ;
  auto mark = [&](int i) {
    if (a.stage_events[i]) cudaEventRecord(a.stage_events[i], stream);
  };
  unsigned* absmax = const_cast<unsigned*>(kp.do_absmax_bits);
  if (!kBf16) {
    const cudaError_t em = cudaMemsetAsync(absmax, 0, sizeof(unsigned), stream);
    if (em != cudaSuccess) return em;
  }
  mark(0);
  bwd_pre_kernel<kD, kBf16><<<static_cast<unsigned>(static_cast<long long>(nQ128) * kp.B * kp.Hq), 128, 0, stream>>>(
      static_cast<const uint16_t*>(a.o), static_cast<const uint16_t*>(a.d_o), a.o_strides[0],
      a.o_strides[1], a.o_strides[2], a.do_strides[0], a.do_strides[1], a.do_strides[2], kp.lse,
      kp.lse_sb, kp.lse_sh, a.delta, kp.dq_acc, kp.Sq, kp.Hq, nQ128, kBf16 ? nullptr : absmax,
      a.head_dim_real, kp.seqlens, nullptr, 0.f, kp.dq_order, 4);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  mark(1);
  const int key = (a.causal ? 2 : 0) | (a.feat ? 1 : 0);
  switch (key) {
    case 0: e = launch256_main<kBf16, false, false>(a, stream); break;
    case 1: e = launch256_main<kBf16, false, true>(a, stream); break;
    case 2: e = launch256_main<kBf16, true, false>(a, stream); break;
    default: e = launch256_main<kBf16, true, true>(a, stream); break;
  }
  if (e != cudaSuccess) return e;
  mark(2);
  bwd256_dq_convert<kBf16><<<static_cast<unsigned>(static_cast<long long>(nQ64) * kp.B * kp.Hq), 256, 0, stream>>>(
      kp.dq_acc, static_cast<uint16_t*>(a.dq), a.dq_strides[0], a.dq_strides[1], a.dq_strides[2],
      kp.Sq, kp.Hq, nQ64, kp.scale, kBf16 ? nullptr : kp.do_absmax_bits, a.head_blk);
  mark(3);
  return cudaGetLastError();
}

cudaError_t launch_bwd256(const BwdLaunch& a, cudaStream_t stream) {
  return a.bf16 ? launch256_all<true>(a, stream) : launch256_all<false>(a, stream);
}

}  // namespace fa2
