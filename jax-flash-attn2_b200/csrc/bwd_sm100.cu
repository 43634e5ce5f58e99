// Backward attention kernels for sm_100a.
//
// Replace the reference's _attn_bwd_preprocess (jax_flash_attn2/flash_attention_triton/
// _backward_triton.py:79-147), _attn_bwd with its dk/dv and dq halves (:150-945) and the
// per-group reduction of dk / dv done afterwards in XLA (:1156-1161).
//
// Three launches:
//   1. bwd_pre_kernel   : delta = rowsum(o * do), lse converted to base 2, both padded to 128
//                         rows per tile; zeroes the fp32 dq accumulator. HBM-bound.
//   2. bwd_main_kernel  : one CTA per (batch, kv head, 128-key tile). It keeps K and V in shared
//                         memory, walks over the query heads of the group and their query tiles,
//                         and runs five tcgen05 GEMMs per step, in the transposed form where the
//                         TMEM lane is the key row:
//                           S^T  = K Q^T          dP^T = V dO^T
//                           dV  += P^T dO         (P^T read from tensor memory)
//                           dK  += dS^T Q         (dS^T staged in shared memory)
//                           dQ_i = dS K           (fresh per step, reduced into fp32 global)
//                         dK / dV accumulate in tensor memory over the whole group, so there is
//                         no per-query-head temporary and no second reduction.
//   3. bwd_dq_convert   : fp32 dq accumulator (tiled layout) * scale -> dq in the input dtype.
#include "bwd_common.cuh"
#include "bwd_launch.cuh"
#include "launch_util.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

constexpr int kBN = 128;   // keys per CTA
// Warpgroups that compute P and dS: each owns 128 / kPW query columns of every step, and they come
// first in the block, followed by the dQ drain warpgroup and the MMA / TMA warpgroup. At D = 128
// two warpgroups measured a little faster than four (the step is bound by the dQ reductions and
// by broadcast shared-memory loads whose number does not shrink with more warps); at D = 64 the
// element-wise phases weigh more and four warpgroups hide more of their latencies.
// Registers per thread after setmaxnreg (the pool is the launch allocation):
//   kPW = 2: launch 128: 2 * 128 + 152 + 104 = 4 * 128
//   kPW = 4: launch  80, nobody trades: the MMA / TMA warps spill below 80 and the drain, which
//            then takes a D = 128 tile in two halves, fits in 80
template <int D>
struct BwdRoles {
  static constexpr int kPW = (D == 64) ? 4 : 2;
  static_assert(kPW == 2 || kPW == 4, "2 or 4 P/dS warpgroups");
  static constexpr int kCW = 128 / kPW;                 // query columns per P/dS warpgroup
  static constexpr int kThreads = (kPW + 2) * 128;
  static constexpr int kRegsDrain = kPW == 2 ? 152 : 80;
  static constexpr int kRegsOther = kPW == 2 ? 104 : 80;
  static_assert(kPW == 4 || 2 * 128 + kRegsDrain + kRegsOther == 4 * 128,
                "setmaxnreg must hand out exactly the launch allocation");
  static constexpr int kWarpDrain = 4 * kPW, kWarpMma = 4 * kPW + 4, kWarpTma = 4 * kPW + 5;
};

// kStaged (score terms / dropout at head dim 64): bias and mask tiles of a step, [128 queries][128
// keys] 16-bit each, are brought in by the TMA unit one step ahead (single-buffered: they are read
// at the very start of a step) instead of being gathered column by column from global memory, and
// when the caller hands over the forward's record of the dropout keep bits, the step's 2 KiB of it
// arrive with the Q tile, so that no Philox round runs in the backward.
//
// kFold (no score terms, head dim 128): the row statistics arrive as a [128 queries][16] bf16
// operand tile per step and are added to S^T and dP^T by one extra MMA k-step each against
// constant ones (see bwd_pre_kernel), so the P / dS threads load no statistics at all. The ones
// are three 128-byte core matrices (ones in columns 0-2 | zeros | ones in columns 0-2) that a
// descriptor with a zero row-group stride repeats down all 128 rows: started at the first one it
// selects columns 0-2 of the statistics tile, started at the second one columns 8-10. The 8 KiB of
// the two statistics stages come out of the dQ staging, which becomes a ring of three eighths of a
// tile instead of two quarters.
template <int D, bool kStaged = false, bool kFold = false>
struct BwdSmem {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kBlockBytes = 128 * 128;   // one [128 rows][64 elements] block
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kTileBytes;
  static constexpr int kQOff = kVOff + kTileBytes;         // 2 stages
  static constexpr int kdOOff = kQOff + 2 * kTileBytes;    // 1 stage
  // dQ leaves through kStageBufs staging chunks of [D/4/kChunks][128 rows][4 floats]
  static constexpr int kChunks = kFold ? 8 : 4;            // chunks per fp32 tile
  static constexpr int kStageBufs = kFold ? 3 : 2;
  // kFold: the drain is bound by the rate at which the TMA unit gets bulk reductions into L2
  // (the staging loop runs at 86 % of what a kernel doing nothing else reaches), so the last chunk
  // of every tile leaves as vector reductions from registers instead, through the load/store
  // path. Measured on B=8, S=4096, Hq=32, Hkv=8 causal: main kernel 2.59-2.62 ms with none,
  // 2.56 with one chunk of eight, 2.62-2.67 with two, 2.71 with three (all of them: 3.4 ms).
  static constexpr int kDirectChunks = kFold ? 1 : 0;
  static constexpr int kChunkBytes = 2 * kTileBytes / kChunks;
  static constexpr int kStageOff = kdOOff + kTileBytes;
  static constexpr int kdSOff = kStageOff + kStageBufs * kChunkBytes;   // [128 keys][128 queries] 16 bit
  // 2 stages x (lse2[128], delta[128]) floats; kFold: 2 stages x one statistics tile, then the
  // three core matrices of the ones operand
  static constexpr int kStatsOff = kdSOff + 128 * 128 * 2;
  static constexpr int kFoldTileBytes = 128 * 16 * 2;
  static constexpr int kStatsStage = kFold ? kFoldTileBytes : 1024;
  static constexpr int kOnesOff = kStatsOff + 2 * kStatsStage;
  static constexpr int kTermBytes = 128 * 128 * 2;          // one term tile: two [128 q][64 keys] blocks
  static constexpr int kTermOff = kOnesOff + (kFold ? 512 : 0);   // bias tile, mask tile
  // recorded dropout bits of a step's (query tile, key tile): [4 words][128 queries], 2 stages
  static constexpr int kBitsBytes = 4 * 128 * 4;
  static constexpr int kBitsOff = kTermOff + (kStaged ? 2 * kTermBytes : 0);
  static constexpr int kBarOff = kBitsOff + (kStaged ? 2 * kBitsBytes : 0);
  static constexpr int kNumBars = 17 + 4;                   // + term_full[2], term_empty[2]
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = (kTotal + 1024 <= kMaxDynSmem) ? kTotal + 1024 : kMaxDynSmem;
  static_assert(kTotal <= kMaxDynSmem, "shared memory budget exceeded");
};

__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&x)[32]) { tmem_st32(taddr, x); }
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&x)[16]) { tmem_st16(taddr, x); }


}  // namespace

// ---------------------------------------------------------------------------------------------
// 3. dq conversion
// ---------------------------------------------------------------------------------------------
// One block converts one 128-row tile. The accumulator is read in its own order (coalesced
// float4 runs), transposed through shared memory 64 columns at a time, and written so that eight
// consecutive threads cover the 128 contiguous bytes those columns take in a row of dq.
template <int D, bool kBf16>
__global__ void __launch_bounds__(256)
bwd_dq_convert(const float* __restrict__ dq_acc, uint16_t* __restrict__ dq, long long sb,
               long long ss, long long sh, int Sq, int Hq, int nQ, float scale_in,
               const unsigned* __restrict__ do_absmax_bits, int blk_real) {
  const float scale = scale_in / (kBf16 ? 1.f : do_scale_from_bits(do_absmax_bits));
  constexpr int kPitch = 129;                       // float4 per column chunk: 128 rows + 1 pad
  __shared__ float4 tile[16 * kPitch];              // 16 chunks of 4 columns = 64 columns
  const int i = blockIdx.x % nQ;     // one-dimensional grid, tile index fastest
  const int bh = blockIdx.x / nQ;
  const int b = bh / Hq, h = bh - b * Hq;
  const int tid = threadIdx.x;
  const float4* src = reinterpret_cast<const float4*>(dq_acc) +
                      (static_cast<long long>(bh) * nQ + i) * (kBM * D / 4);
  for (int part = 0; part < D / 64; ++part) {
    if (part) __syncthreads();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int idx = tid + k * 256;                // 0 .. 2047 = 16 chunks x 128 rows
      tile[(idx >> 7) * kPitch + (idx & 127)] = src[part * 2048 + idx];
    }
    __syncthreads();
    const int j = tid & 7;                          // 16-byte piece of the 128-byte row segment
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int r = pass * 32 + (tid >> 3);
      const int row = i * kBM + r;
      // a padded head dim keeps blk_real real columns at the start of every 64-column block
      if (row < Sq && 8 * j < blk_real) {
        const float4 x = tile[(2 * j) * kPitch + r];
        const float4 y = tile[(2 * j + 1) * kPitch + r];
        uint4 v;
        v.x = pack2<kBf16>(x.x * scale, x.y * scale);
        v.y = pack2<kBf16>(x.z * scale, x.w * scale);
        v.z = pack2<kBf16>(y.x * scale, y.y * scale);
        v.w = pack2<kBf16>(y.z * scale, y.w * scale);
        reinterpret_cast<uint4*>(dq + b * sb + row * ss + h * sh)[part * (blk_real >> 3) + j] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// 2. main kernel
// ---------------------------------------------------------------------------------------------
template <int D, bool kBf16, bool kCausal, bool kFeat>
__global__ void __launch_bounds__(BwdRoles<D>::kThreads, 1)
bwd_main_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                const __grid_constant__ CUtensorMap tmBias, const __grid_constant__ CUtensorMap tmMask,
                const float* __restrict__ stats, const BwdKernelParams p) {
  constexpr bool kStaged = kFeat && D == 64;
  constexpr bool kFold = !kFeat && D == 128;
  using L = BwdSmem<D, kStaged, kFold>;
  using R = BwdRoles<D>;
  constexpr int kPW = R::kPW, kCW = R::kCW;
  constexpr int kWarpDrain = R::kWarpDrain, kWarpMma = R::kWarpMma, kWarpTma = R::kWarpTma;
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
  const uint32_t bar_do_full = bars + 8u * 3, bar_do_empty = bars + 8u * 4;
  auto bar_q_empty = [&](int s) { return bars + 8u * (5 + s); };
  const uint32_t bar_s_full = bars + 8u * 9, bar_p_full = bars + 8u * 10;
  const uint32_t bar_dp_full = bars + 8u * 11, bar_ds_full = bars + 8u * 12;
  const uint32_t bar_dq_full = bars + 8u * 13, bar_dq_drained = bars + 8u * 14;
  const uint32_t bar_dkv_full = bars + 8u * 15;
  const uint32_t bar_kv_tmem = bars + 8u * 16;   // D = 64: K and V have been copied into tensor memory
  auto bar_term_full = [&](int x) { return bars + 8u * (17 + x); };    // x = 0: bias, 1: mask
  auto bar_term_empty = [&](int x) { return bars + 8u * (19 + x); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- work item: (batch, kv head, key tile); later key tiles (fewest steps when causal) last
  int n, bhk;
  bwd_work_item(blockIdx.x, p.B * p.Hkv, p.n_kvblk, p.sched_groups, p.dq_order != nullptr, bhk, n);
  const int b = bhk / p.Hkv;
  const int hk = bhk - b * p.Hkv;
  const int nQ = (p.Sq + kBM - 1) / kBM;   // query tiles in the statistics / accumulator layout
  // rows of this batch element that take part: the problem's, or its seqlens entry
  int sq_b = p.Sq, sk_b = p.Sk;
  if (p.seqlens != nullptr) {
    sq_b = max(0, min(__ldg(p.seqlens + b), p.Sq));
    sk_b = min(sq_b, p.Sk);
  }
  const int nQ_b = (sq_b + kBM - 1) / kBM;
  int i_start = 0;
  if (kCausal) {
    const int first_row = n * kBN - p.causal_off;   // first query row that sees key n*128
    i_start = first_row > 0 ? first_row / kBM : 0;
  }
  if (i_start > nQ_b) i_start = nQ_b;
  const int nI = nQ_b - i_start;                     // query tiles per head
  const int T = (n * kBN < sk_b) ? nI * p.G : 0;     // steps of this CTA (none: dK = dV = 0)
  const bool dead_keys = n * kBN + kBN > sk_b;       // some key rows lie past the end

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_q_full(s), 1);
      mbar_init(bar_q_empty(s), 1);
    }
    mbar_init(bar_do_full, 1);
    mbar_init(bar_do_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, 128 * kPW);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_ds_full, 128 * kPW);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_drained, 128);
    mbar_init(bar_dkv_full, 1);
    mbar_init(bar_kv_tmem, 256);
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar_term_full(x), 1);
      mbar_init(bar_term_empty(x), 128 * kPW);
    }
    fence_mbar_init();
  }
  if (warp == kWarpTma && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    if constexpr (kStaged) {
      if (p.bias.staged) tma_prefetch_desc(&tmBias);
      if (p.mask.staged) tma_prefetch_desc(&tmMask);
    }
  }
  if constexpr (kFold) {
    // three core matrices of 8 rows x 16 bytes: 1.0 (bf16) in columns 0-2 | zeros | like the first
    if (tid < 24)
      reinterpret_cast<uint4*>(smem_gen + L::kOnesOff)[tid] =
          (tid >> 3) == 1 ? make_uint4(0u, 0u, 0u, 0u) : make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
    fence_proxy_async_smem();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColdP = 128, kColdK = 256, kColdV = 256 + D;
  constexpr uint32_t kColdQ = (D == 128) ? 128 : 384;
  // D = 64 leaves 64 columns free: K and V (16 bit, 32 columns each) live there as well, so that
  // S^T = K Q^T and dP^T = V dO^T read their loop-invariant A operand from tensor memory instead of
  // shared memory, the resource this kernel is bound by.
  constexpr bool kKvInTmem = (D == 64);
  constexpr uint32_t kColKt = 448, kColVt = 480;

  auto step_coords = [&](int it, int& h, int& i) {
    const int g = it / nI;
    i = i_start + (it - g * nI);
    h = hk * p.G + g;
  };

  if constexpr (kPW == 2) {
    if (warp >= kWarpMma) setmaxnreg_dec<R::kRegsOther>();   // one site for the whole warpgroup
  }
  if (warp >= kWarpTma + 1) {
    // idle: these two warps only complete the warpgroup that gives up registers
  } else if (warp == kWarpTma) {
    // =========================== TMA producer ================================================
    if (lane == 0 && T > 0) {
      mbar_arrive_expect_tx(bar_kv_full, 2 * L::kTileBytes);
      tma_load_5d(sK, &tmK, bar_kv_full, 0, n * kBN, 0, hk, b);
      tma_load_5d(sV, &tmV, bar_kv_full, 0, n * kBN, 0, hk, b);
      bool ok = true;
      for (int it = 0; it < T && ok; ++it) {
        const int st = it & 1;
        const uint32_t par = ((it >> 1) & 1) ^ 1;
        int h, i;
        step_coords(it, h, i);
        ok = mbar_wait(bar_q_empty(st), par, abort_flag);
        if (!ok) break;
        const bool with_bits = kStaged && p.drop.bits != nullptr;
        mbar_arrive_expect_tx(bar_q_full(st), L::kTileBytes + L::kStatsStage + (with_bits ? L::kBitsBytes : 0));
        tma_load_5d(sQ + st * L::kTileBytes, &tmQ, bar_q_full(st), 0, i * kBM, 0, h, b);
        if constexpr (kStaged) {
          if (with_bits)
            bulk_load_1d(smem_base + L::kBitsOff + st * L::kBitsBytes, dropout_bits_block(p.drop, b, h, p.Hq, i, n),
                         L::kBitsBytes, bar_q_full(st));
        }
        if constexpr (kFold)
          bulk_load_1d(sStats + st * L::kStatsStage,
                       p.xstats + ((static_cast<long long>(b) * p.Hq + h) * nQ + i) * (L::kFoldTileBytes / 16),
                       L::kFoldTileBytes, bar_q_full(st));
        else
          bulk_load_1d(sStats + st * 1024,
                       stats + ((static_cast<long long>(b) * p.Hq + h) * nQ + i) * 256, 1024,
                       bar_q_full(st));
        if constexpr (kStaged) {
          // the step's bias / mask tiles: their buffers were read at the start of the previous step
#pragma unroll
          for (int x = 0; x < 2 && ok; ++x) {
            const ScoreTermDev& tt = x ? p.mask : p.bias;
            if (!tt.staged) continue;
            ok = mbar_wait(bar_term_empty(x), (it & 1) ^ 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(bar_term_full(x), L::kTermBytes);
            const uint32_t dst = smem_base + L::kTermOff + x * L::kTermBytes;
            const int hx = tt.sh ? h / tt.head_div : 0, bx = tt.sb ? b : 0;
            tma_load_4d(dst, x ? &tmMask : &tmBias, bar_term_full(x), n * kBN, i * kBM, hx, bx);
            tma_load_4d(dst + L::kBlockBytes, x ? &tmMask : &tmBias, bar_term_full(x), n * kBN + 64, i * kBM, hx, bx);
          }
          if (!ok) break;
        }
        ok = mbar_wait(bar_do_empty, (it & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_do_full, L::kTileBytes);
        tma_load_5d(sdO, &tmdO, bar_do_full, 0, i * kBM, 0, h, b);
      }
      if (!ok) atomicOr(p.status, 8);
    }
    __syncwarp();
  } else if (warp == kWarpMma) {
    // =========================== MMA issuer ==================================================
    if (T > 0) {
      constexpr uint32_t idesc_s = make_idesc(kBf16, 128, 128, false, false);
      constexpr uint32_t idesc_dv = make_idesc(kBf16, 128, D, false, true);
      constexpr uint32_t idesc_dk = make_idesc(kBf16, 128, D, false, true);
      constexpr uint32_t idesc_dq = make_idesc(kBf16, 128, D, true, true);
      bool ok = true;

      // Shared-memory descriptors are built once; every MMA only adds a constant to the start
      // address (the issuing thread is a serial instruction stream: what it executes per MMA
      // delays every barrier it has to look at).
      const uint64_t dK_k = make_sdesc(sK, 16, 1024), dK_mn = make_sdesc(sK, L::kBlockBytes, 1024);
      const uint64_t dV_k = make_sdesc(sV, 16, 1024);
      const uint64_t dQ_k0 = make_sdesc(sQ, 16, 1024), dQ_mn0 = make_sdesc(sQ, L::kBlockBytes, 1024);
      const uint64_t ddO_k = make_sdesc(sdO, 16, 1024), ddO_mn = make_sdesc(sdO, L::kBlockBytes, 1024);
      const uint64_t ddS_k = make_sdesc(sdS, 16, 1024), ddS_mn = make_sdesc(sdS, L::kBlockBytes, 1024);

      // kFold: the ones (A; every 8-row group reads the same core matrices) and the statistics
      // tiles of the two stages (B), unswizzled
      const uint64_t dOnes = make_sdesc_plain(smem_base + L::kOnesOff, 128, 0);
      const uint64_t dStat = make_sdesc_plain(sStats, 128, 256);
      constexpr uint32_t idesc_fold = make_idesc(true, 128, 128, false, false);   // bf16 whatever the dtype

      // D[kv, q] = A[kv, d] * B[q, d]^T, both operands K-major over the head dim; at D = 64 the A
      // operand (K for S^T, V for dP^T) comes from tensor memory: 8 columns per 16 dims.
      // kFold: the accumulator starts from the statistic of stage `st` (-lse / scale for S^T,
      // -delta for dP^T), one k-step of ones times the statistics tile.
      auto issue_kd = [&](uint32_t d_col, uint64_t a_desc, uint64_t b_desc, int st) {
        if constexpr (kFold)
          mma_ss_e(tmem_base + d_col, sdesc_advance(dOnes, d_col == kColS ? 0 : 128),
                   sdesc_advance(dStat, st * L::kStatsStage), idesc_fold, 0u);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * L::kBlockBytes + (k & 3) * 32;
          const uint32_t acc = (kFold || k > 0) ? 1u : 0u;
          if constexpr (kKvInTmem) {
            const uint32_t a_col = (d_col == kColS ? kColKt : kColVt) + 8 * k;
            mma_ts_e(tmem_base + d_col, tmem_base + a_col, sdesc_advance(b_desc, off), idesc_s, acc);
            continue;
          }
          mma_ss_e(tmem_base + d_col, sdesc_advance(a_desc, off), sdesc_advance(b_desc, off), idesc_s, acc);
        }
      };
      auto issue_dv = [&](bool first) {
#pragma unroll
        for (int k = 0; k < kBM / 16; ++k) {
          // P^T for queries [16k, 16k+16): 8 packed columns; every P/dS warpgroup wrote its kCW
          // queries at the start of the S columns it had read (column kCW * g).
          const uint32_t a_col = kColS + kCW * (k / (kCW / 16)) + 8 * (k % (kCW / 16));
          mma_ts_e(tmem_base + kColdV, tmem_base + a_col, sdesc_advance(ddO_mn, k * 2048), idesc_dv,
                 (first && k == 0) ? 0u : 1u);
        }
      };
      auto issue_dk = [&](uint64_t q_mn, bool first) {
#pragma unroll
        for (int k = 0; k < kBM / 16; ++k) {
          const uint32_t a_off = (k >> 2) * L::kBlockBytes + (k & 3) * 32;
          mma_ss_e(tmem_base + kColdK, sdesc_advance(ddS_k, a_off), sdesc_advance(q_mn, k * 2048),
                 idesc_dk, (first && k == 0) ? 0u : 1u);
        }
      };
      auto issue_dq = [&]() {
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k) {
          // A = dS (M = query, contiguous in the dS^T rows; K = key rows), B = K tile, both MN-major
          mma_ss_e(tmem_base + kColdQ, sdesc_advance(ddS_mn, k * 2048), sdesc_advance(dK_mn, k * 2048),
                 idesc_dq, k > 0 ? 1u : 0u);
        }
      };

      ok = mbar_wait_warp(bar_kv_full, 0, abort_flag);
      if (kKvInTmem && ok) ok = mbar_wait_warp(bar_kv_tmem, 0, abort_flag);
      if (ok) ok = mbar_wait_warp(bar_q_full(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_kd(kColS, dK_k, dQ_k0, 0);
        mma_commit_e(bar_s_full);
        ok = mbar_wait_warp(bar_do_full, 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        issue_kd(kColdP, dV_k, ddO_k, 0);
        mma_commit_e(bar_dp_full);
      }
      for (int it = 0; it < T && ok; ++it) {
        const int st = it & 1, nx = st ^ 1;
        const uint32_t par = it & 1;
        const uint32_t par_next = ((it + 1) >> 1) & 1;
        const bool has_next = it + 1 < T;
        ok = mbar_wait_warp(bar_p_full, par, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_dv(it == 0);
        mma_commit_e(bar_do_empty);          // the single dO buffer can be refilled
        if (has_next) {
          ok = mbar_wait_warp(bar_q_full(nx), par_next, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_kd(kColS, dK_k, sdesc_advance(dQ_k0, nx * L::kTileBytes), nx);
          mma_commit_e(bar_s_full);
        }
        ok = mbar_wait_warp(bar_ds_full, par, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_dq();
        mma_commit_e(bar_dq_full);
        issue_dk(sdesc_advance(dQ_mn0, st * L::kTileBytes), it == 0);
        mma_commit_e(bar_q_empty(st));
        if (has_next) {
          ok = mbar_wait_warp(bar_dq_drained, par, abort_flag);
          if (ok) ok = mbar_wait_warp(bar_do_full, (it + 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_kd(kColdP, dV_k, ddO_k, nx);
          mma_commit_e(bar_dp_full);
        }
      }
      if (ok) mma_commit_e(bar_dkv_full);
      if (!ok && lane == 0) atomicOr(p.status, 16);
    }
    __syncwarp();
  } else if (warp >= kWarpDrain) {
    // =========================== dQ drain ====================================================
    if constexpr (kPW == 2) setmaxnreg_inc<R::kRegsDrain>();
    const int r = tid - 128 * kPW;   // query row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tdQ = tmem_base + lane_base + kColdQ;
    bool ok = true;
    uint32_t ring = 0;   // staging buffer of the next chunk
    // Bit-reproducible dq (p.dq_order): this key tile adds its part of a dQ tile when the
    // contributing key tiles above it have added theirs, and says so once its own reductions have
    // been performed. Two more named barriers per step.
    const bool ordered = p.dq_order != nullptr;
    for (int it = 0; it < T; ++it) {
      int h, i;
      step_coords(it, h, i);
      if (ok) ok = mbar_wait(bar_dq_full, it & 1, abort_flag);
      if (!ok) {
        // No early exit: a thread that left alone would strand the other 127 at the (unbounded)
        // named barriers of the staging loop. Keep in step with them: two barriers per chunk.
#pragma unroll 1
        for (int k = 0; k < 2 * (L::kChunks - L::kDirectChunks) + (ordered ? 2 : 0); ++k) named_bar_sync(3, 128);
        continue;
      }
      tc_fence_after();
      // Pull the tile into registers first so that the tensor-memory columns are handed back
      // early; the reductions (slow: they queue in the memory pipe) then overlap with the MMAs of
      // the next step. With four P/dS warpgroups the register file only leaves room for half a
      // D = 128 tile here, so the tile is taken in two parts and handed back after the second load.
      // Each part leaves through the TMA unit in chunks of D/kChunks columns through the staging
      // buffers: cp.reduce.async.bulk adds a chunk to the global fp32 accumulator while the next
      // one is written. (All reductions issued from registers would queue in the memory pipe in
      // front of the tensor-memory traffic of the other warps; a small share of them does not, and
      // takes load off the TMA unit: kDirectChunks.)
      constexpr int kParts = (kPW == 4 && D == 128) ? 2 : 1;
      constexpr int kPartCols = D / kParts;
      const long long tile = (static_cast<long long>(b) * p.Hq + h) * nQ + i;
      float* dst_tile = p.dq_acc + tile * (kBM * D);

#pragma unroll
      for (int part = 0; part < kParts; ++part) {
        uint32_t v[kPartCols];
#pragma unroll
        for (int c = 0; c < kPartCols / 32; ++c)
          tmem_ld32(tdQ + part * kPartCols + c * 32, reinterpret_cast<uint32_t(&)[32]>(v[c * 32]));
        tc_wait_ld();
        if (part == kParts - 1) {
          tc_fence_before();
          mbar_arrive(bar_dq_drained);
        }
        if (ordered && part == 0) {
          // the tensor-memory columns have been handed back: only the reductions are held back
          // until it is this key tile's turn, not the MMAs of the next step
          if (r == 0) {
            const int above = bwd_tile_contributors(kCausal, i, kBM, sq_b, sk_b, p.n_kvblk, p.causal_off) - 1 - n;
            if (!wait_for_turn(p.dq_order + tile, above, abort_flag)) atomicOr(p.status, 256);
          }
          named_bar_sync(3, 128);
        }
        constexpr int kChunkVecs = D / 4 / L::kChunks;   // float4 columns per chunk
        // the last kDirect chunks of a tile go out as vector reductions from registers
        constexpr int kDirect = L::kDirectChunks;
#pragma unroll
        for (int cl = L::kChunks / kParts - kDirect; cl < L::kChunks / kParts; ++cl) {
          const int c = part * (L::kChunks / kParts) + cl;
#pragma unroll
          for (int c4 = 0; c4 < kChunkVecs; ++c4) {
            const int cc = cl * kChunkVecs + c4;
            float* dst = dst_tile + c * (kBM * D / L::kChunks) + (c4 * 128 + r) * 4;
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v[4 * cc])),
                         "f"(__uint_as_float(v[4 * cc + 1])), "f"(__uint_as_float(v[4 * cc + 2])),
                         "f"(__uint_as_float(v[4 * cc + 3]))
                         : "memory");
          }
        }
#pragma unroll
        for (int cl = 0; cl < L::kChunks / kParts - kDirect; ++cl) {
          const int c = part * (L::kChunks / kParts) + cl;
          const uint32_t buf = ring;
          ring = (ring + 1 == L::kStageBufs) ? 0u : ring + 1;
          // the reductions out of the other buffers may still be reading, not the one issued
          // kStageBufs chunks ago out of this buffer
          if (r == 0) {
            if constexpr (L::kStageBufs == 3) asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          }
          named_bar_sync(3, 128);
          uint8_t* stage = smem_gen + L::kStageOff + buf * L::kChunkBytes;
#pragma unroll
          for (int c4 = 0; c4 < kChunkVecs; ++c4) {
            const int cc = cl * kChunkVecs + c4;
            *reinterpret_cast<uint4*>(stage + (c4 * 128 + r) * 16) =
                make_uint4(v[4 * cc], v[4 * cc + 1], v[4 * cc + 2], v[4 * cc + 3]);
          }
          fence_proxy_async_smem();
          named_bar_sync(3, 128);
          if (r == 0) {
            bulk_reduce_add_f32(dst_tile + c * (kBM * D / L::kChunks),
                                smem_base + L::kStageOff + buf * L::kChunkBytes, L::kChunkBytes);
            tma_store_commit();
          }
        }
      }
      if (ordered) {
        if (L::kDirectChunks > 0) __threadfence();   // this thread's reductions from registers
        named_bar_sync(3, 128);
        if (r == 0) {
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // performed, not only read
          __threadfence();
          atomicAdd(p.dq_order + tile, 1);
        }
      }
    }
    if (r == 0) tma_store_wait_read0();   // staging buffers stay valid until the TMA unit has read them
    if (!ok && r == 0) atomicOr(p.status, 32);
  } else {
    // =========================== P / dS warps + dK, dV epilogue ==============================
    const int w = warp >> 2;            // warpgroup: queries [kCW*w, kCW*w + kCW) of each tile
    const int r = tid & 127;            // key row inside the tile == TMEM lane
    const int kv = n * kBN + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + kCW * w;
    const uint32_t tdP = tmem_base + lane_base + kColdP + kCW * w;
    const float* stats_s = reinterpret_cast<const float*>(smem_gen + L::kStatsOff);
    // dS^T row r: queries [kCW*w, +kCW) are chunks [chunk0, chunk0 + kCW/8) of one 128-byte line
    uint8_t* ds_row = smem_gen + L::kdSOff + ((kCW * w) >> 6) * L::kBlockBytes + r * 128;
    const int chunk0 = ((kCW * w) & 63) >> 3;
    const float do_scale = kBf16 ? 1.f : do_scale_from_bits(p.do_absmax_bits);
    bool ok = true;

    if constexpr (kKvInTmem) {
      // One-time: warpgroup 0 copies K, warpgroup 1 copies V into tensor memory, one key row per
      // thread (= lane), two 16-bit values per column in head-dim order (the layout of a 16-bit
      // A operand, the one P^T is written in). K also stays in shared memory for dQ.
      if (w < 2 && T > 0) {
        ok = mbar_wait(bar_kv_full, 0, abort_flag);
        if (ok) {
          const uint8_t* src = smem_gen + (w == 0 ? L::kKOff : L::kVOff) + r * 128;
          uint32_t kx[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 v4 = *reinterpret_cast<const uint4*>(src + ((j ^ (r & 7)) << 4));
            kx[4 * j + 0] = v4.x;
            kx[4 * j + 1] = v4.y;
            kx[4 * j + 2] = v4.z;
            kx[4 * j + 3] = v4.w;
          }
          tmem_st32(tmem_base + lane_base + (w == 0 ? kColKt : kColVt), kx);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar_kv_tmem);
        }
      }
    }

    // Dropout keep bits of this key row for the step's kCW query columns. They are drawn one step
    // ahead, after dS of the previous step has been handed over, so that the Philox rounds overlap
    // the MMAs instead of sitting between S^T and P^T.
    uint32_t keep[kCW / 32];
#pragma unroll
    for (int k = 0; k < kCW / 32; ++k) keep[k] = 0xffffffffu;
    const bool recorded_bits = kStaged && p.drop.bits != nullptr;   // read instead of drawn
    auto draw_keep = [&](int step) {
      if constexpr (kFeat) {
        if (p.drop.enabled && !recorded_bits && step < T) {
          int hh, ii;
          step_coords(step, hh, ii);
          dropout_keep_bits_transposed<kCW>(p.drop, dropout_bh_index(p.drop, b, hh), kv, ii * kBM + kCW * w,
                                            lane, keep);
        }
      }
    };
    draw_keep(0);

    for (int it = 0; it < T && ok; ++it) {
      const int st = it & 1;
      int h, i;
      step_coords(it, h, i);
      // per query column of this warpgroup: -lse*log2(e) (or -inf) and delta
      const float4* nlse4 = reinterpret_cast<const float4*>(stats_s + st * 256 + kCW * w);
      const float4* delta4 = nlse4 + 32;
      const int q_first = i * kBM + kCW * w;
      // (kFold: nothing of the Q stage is read by these threads, its statistics are in S^T already)
      if constexpr (!kFold) ok = mbar_wait(bar_q_full(st), (it >> 1) & 1, abort_flag);
      if (ok) ok = mbar_wait(bar_s_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      if constexpr (kStaged) {
        if (recorded_bits) {
          // word r / 32 of every query row holds the flags of this thread's 32-key group: the even
          // keys in the low half, the odd keys in the high half
          const uint32_t src = smem_base + L::kBitsOff + st * L::kBitsBytes + ((r >> 5) * 128 + kCW * w) * 4;
          const int pos = ((r & 31) >> 1) + 16 * (r & 1);
#pragma unroll
          for (int k = 0; k < kCW / 32; ++k) keep[k] = 0u;
#pragma unroll
          for (int c4 = 0; c4 < kCW / 4; ++c4) {
            const uint4 wv = lds128(src + 16 * c4);
            const uint32_t four = ((wv.x >> pos) & 1u) | (((wv.y >> pos) & 1u) << 1) | (((wv.z >> pos) & 1u) << 2) |
                                  (((wv.w >> pos) & 1u) << 3);
            keep[(4 * c4) >> 5] |= four << ((4 * c4) & 31);
          }
        }
      }
      // some (query, key) pairs of this step are above the causal diagonal
      const bool diag = (kCausal && (n * kBN + kBN - 1 > i * kBM + p.causal_off)) || dead_keys;
      // masked iff query index < q_lim: every query for a key past the end
      const int q_lim = kv >= sk_b ? 0x7fffffff : (kCausal ? kv - p.causal_off : -0x7fffffff - 1);

      // ---- P^T = exp2(S^T * scale*log2e - lse*log2e): kCW query columns of this key row ------
      uint32_t pk[kCW / 2];                     // P as 16-bit pairs; also the input of dS below
      {
        uint32_t s[kCW];
#pragma unroll
        for (int c = 0; c < kCW / 32; ++c)
          tmem_ld32(tS + 32 * c, reinterpret_cast<uint32_t(&)[32]>(s[32 * c]));
        tc_wait_ld();
        if constexpr (kFeat) {
#pragma unroll
          for (int c = 0; c < kCW; ++c) s[c] = __float_as_uint(__uint_as_float(s[c]) * p.scale_log2);
          if constexpr (kStaged) {
#pragma unroll
            for (int x = 0; x < 2; ++x) {
              const ScoreTermDev& tt = x ? p.mask : p.bias;
              if (!tt.staged) continue;
              if (ok) ok = mbar_wait(bar_term_full(x), it & 1, abort_flag);
              if (ok) {
                // column r of the staged [128 queries][128 keys] tile: element (query, key r) sits in
                // block r / 64, row `query`, 16-byte chunk (r % 64) / 8 (swizzled with the row)
                const uint32_t col = smem_base + L::kTermOff + x * L::kTermBytes + (r >> 6) * L::kBlockBytes +
                                     (r & 7) * 2;
                const uint32_t chunk = static_cast<uint32_t>((r & 63) >> 3);
#pragma unroll
                for (int c = 0; c < kCW; ++c) {
                  const int qrow = kCW * w + c;
                  const uint16_t v = lds16(col + qrow * 128 + ((chunk ^ (qrow & 7)) << 4));
                  s[c] = __float_as_uint(fmaf(to_float16bit<kBf16>(v), kLog2e, __uint_as_float(s[c])));
                }
              }
              mbar_arrive(bar_term_empty(x));
            }
            if (!p.bias.staged) add_term_column<kBf16, kCW>(p.bias, b, h, q_first, kv, p.Sq, p.Sk, s);
            if (!p.mask.staged) add_term_column<kBf16, kCW>(p.mask, b, h, q_first, kv, p.Sq, p.Sk, s);
          } else {
            add_term_column<kBf16, kCW>(p.bias, b, h, q_first, kv, p.Sq, p.Sk, s);
            add_term_column<kBf16, kCW>(p.mask, b, h, q_first, kv, p.Sq, p.Sk, s);
          }
        }
#pragma unroll
        for (int c4 = 0; c4 < kCW / 4; ++c4) {
          const float4 nl = kFold ? make_float4(0.f, 0.f, 0.f, 0.f) : nlse4[c4];
          const float nlv[4] = {nl.x, nl.y, nl.z, nl.w};
#pragma unroll
          for (int k2 = 0; k2 < 2; ++k2) {
            const int c = 4 * c4 + 2 * k2;     // columns c, c + 1
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
      auto store_p = [&](const uint32_t (&x)[kCW / 2]) { tmem_st_cols(tS, x); };
      if constexpr (kFeat) {
        if (p.drop.enabled) {
          // the weights that reach dV carry the dropout mask and its 1/(1-p)
          uint32_t pd[kCW / 2];
#pragma unroll
          for (int c = 0; c < kCW / 2; ++c) {
            const uint32_t bits = keep[(2 * c) >> 5];
            const int sh = (2 * c) & 31;
            float a0 = ((bits >> sh) & 1u) ? unpack_lo<kBf16>(pk[c]) * p.drop.inv_keep : 0.f;
            float a1 = ((bits >> (sh + 1)) & 1u) ? unpack_hi<kBf16>(pk[c]) * p.drop.inv_keep : 0.f;
            pd[c] = pack2<kBf16>(a0, a1);
          }
          store_p(pd);
        } else {
          store_p(pk);
        }
      } else {
        store_p(pk);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full);

      // ---- dS^T = P^T * (dP^T * keep/(1-p) - delta) -> shared memory, 16 bit ------------------
      ok = mbar_wait(bar_dp_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t dp[kCW];
#pragma unroll
        for (int c = 0; c < kCW / 32; ++c)
          tmem_ld32(tdP + 32 * c, reinterpret_cast<uint32_t(&)[32]>(dp[32 * c]));
        tc_wait_ld();
#pragma unroll
        for (int c4 = 0; c4 < kCW / 4; ++c4) {
          const float4 dl = kFold ? make_float4(0.f, 0.f, 0.f, 0.f) : delta4[c4];
          const float dlv[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
          for (int k2 = 0; k2 < 2; ++k2) {
            const int c = 4 * c4 + 2 * k2;
            float d0 = __uint_as_float(dp[c]), d1 = __uint_as_float(dp[c + 1]);
            if constexpr (kFeat) {
              const uint32_t bits = keep[c >> 5];
              d0 = ((bits >> (c & 31)) & 1u) ? d0 * p.drop.inv_keep : 0.f;
              d1 = ((bits >> ((c + 1) & 31)) & 1u) ? d1 * p.drop.inv_keep : 0.f;
            }
            float t0 = d0, t1 = d1;
            if constexpr (!kFold) add2(t0, t1, d0, d1, -dlv[2 * k2], -dlv[2 * k2 + 1]);
            if constexpr (!kBf16) fma2(t0, t1, t0, t1, do_scale, do_scale, 0.f, 0.f);
            const float p0 = unpack_lo<kBf16>(pk[c >> 1]), p1 = unpack_hi<kBf16>(pk[c >> 1]);
            dp[c >> 1] = pack2<kBf16>(p0 * t0, p1 * t1);     // reuse dp[0..kCW/2) for the packed dS
          }
        }
#pragma unroll
        for (int q4 = 0; q4 < kCW / 8; ++q4) {
          *reinterpret_cast<uint4*>(ds_row + (((chunk0 + q4) ^ (r & 7)) << 4)) =
              make_uint4(dp[4 * q4], dp[4 * q4 + 1], dp[4 * q4 + 2], dp[4 * q4 + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_ds_full);
        if constexpr (kFeat) {
          // off the critical path: the MMAs of dQ and dK are already free to start
          if (p.dbias.ptr != nullptr)
            add_bias_grad<kBf16, kCW>(p.dbias, b, h, q_first, kv, p.Sq, p.Sk, dp, do_scale);
        }
      }
      draw_keep(it + 1);
    }

    // ---- epilogue: the first half of the warpgroups writes dK (scaled), the second half dV ----
    constexpr int kWgPerAcc = kPW / 2;                 // warpgroups that share one accumulator
    constexpr int kUnits = D / 32 / kWgPerAcc;         // 32-column units per warpgroup
    const int acc = w / kWgPerAcc;                     // 0: dK, 1: dV
    const int part = w % kWgPerAcc;
    if (ok && T > 0) ok = mbar_wait(bar_dkv_full, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      const uint32_t tAcc = tmem_base + lane_base + (acc == 0 ? kColdK : kColdV);
      const float f = (acc == 0) ? p.scale / do_scale : 1.f;
      uint8_t* stage = smem_gen + L::kQOff + acc * L::kTileBytes;   // both Q stages are free now
#pragma unroll
      for (int cu = 0; cu < kUnits; ++cu) {
        const int c = part * kUnits + cu;
        uint32_t a[32];
        if (T > 0) {
          tmem_ld32(tAcc + c * 32, a);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) a[k] = 0u;
        }
        uint8_t* line = stage + (c >> 1) * L::kBlockBytes + r * 128;
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
    named_bar_sync(1 + acc, 128 * kWgPerAcc);
    if (ok && part == 0 && r == 0 && !*abort_flag) {
      tma_store_5d(acc == 0 ? &tmdK : &tmdV, sQ + acc * L::kTileBytes, 0, n * kBN, 0, hk, b);
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

// ---------------------------------------------------------------------------------------------
// launcher
// ---------------------------------------------------------------------------------------------
template <int D, bool kBf16, bool kCausal, bool kFeat>
static cudaError_t launch_main(const BwdLaunch& a, cudaStream_t stream) {
  using L = BwdSmem<D, kFeat && D == 64>;
  auto kern = bwd_main_kernel<D, kBf16, kCausal, kFeat>;
  static bool smem_opted_in[64] = {};
  cudaError_t e = opt_in_dynamic_smem(kern, L::kDynamicBytes, smem_opted_in);
  if (e != cudaSuccess) return e;
  const long long nblocks = static_cast<long long>(a.kp.n_kvblk) * a.kp.B * a.kp.Hkv;
  kern<<<static_cast<unsigned>(nblocks), BwdRoles<D>::kThreads, L::kDynamicBytes, stream>>>(
      a.tmQ, a.tmK, a.tmV, a.tmdO, a.tmdK, a.tmdV, a.tmBias, a.tmMask, a.delta, a.kp);
  return cudaGetLastError();
}

template <int D, bool kBf16>
static cudaError_t launch_all(const BwdLaunch& a, cudaStream_t stream) {
  const BwdKernelParams& kp = a.kp;
  const int nQ = (kp.Sq + kBM - 1) / kBM;
  const unsigned grid = static_cast<unsigned>(static_cast<long long>(nQ) * kp.B * kp.Hq);
  auto mark = [&](int i) {
    if (a.stage_events[i]) cudaEventRecord(a.stage_events[i], stream);
  };
  unsigned* absmax = const_cast<unsigned*>(kp.do_absmax_bits);
  if (!kBf16) {
    const cudaError_t em = cudaMemsetAsync(absmax, 0, sizeof(unsigned), stream);
    if (em != cudaSuccess) return em;
  }
  mark(0);
  bwd_pre_kernel<D, kBf16><<<grid, 128, 0, stream>>>(
      static_cast<const uint16_t*>(a.o), static_cast<const uint16_t*>(a.d_o), a.o_strides[0],
      a.o_strides[1], a.o_strides[2], a.do_strides[0], a.do_strides[1], a.do_strides[2], kp.lse,
      kp.lse_sb, kp.lse_sh, a.delta, kp.dq_acc, kp.Sq, kp.Hq, nQ, kBf16 ? nullptr : absmax,
      a.head_dim_real, kp.seqlens, const_cast<uint4*>(kp.xstats), 1.f / kp.scale_log2, kp.dq_order, 1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int key = (a.causal ? 2 : 0) | (a.feat ? 1 : 0);
  mark(1);
  switch (key) {
    case 0: e = launch_main<D, kBf16, false, false>(a, stream); break;
    case 1: e = launch_main<D, kBf16, false, true>(a, stream); break;
    case 2: e = launch_main<D, kBf16, true, false>(a, stream); break;
    default: e = launch_main<D, kBf16, true, true>(a, stream); break;
  }
  if (e != cudaSuccess) return e;
  mark(2);
  bwd_dq_convert<D, kBf16><<<grid, 256, 0, stream>>>(kp.dq_acc, static_cast<uint16_t*>(a.dq),
                                                     a.dq_strides[0], a.dq_strides[1],
                                                     a.dq_strides[2], kp.Sq, kp.Hq, nQ, kp.scale,
                                                     kBf16 ? nullptr : kp.do_absmax_bits, a.head_blk);
  mark(3);
  return cudaGetLastError();
}


cudaError_t launch_bwd(const BwdLaunch& a, cudaStream_t stream) {
  if (a.head_dim == 64) return a.bf16 ? launch_all<64, true>(a, stream) : launch_all<64, false>(a, stream);
  if (a.head_dim == 128) return a.bf16 ? launch_all<128, true>(a, stream) : launch_all<128, false>(a, stream);
  if (a.head_dim == 256) return launch_bwd256(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace fa2
