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
#include "fwd_row.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

namespace {

#ifdef FA2_TRACE
// Development aid (not compiled by default): per-role time stamps of one CTA.
__device__ long long g_trace_fwd[40 * 1024];
#define FA2_TF(role, idx) do { if (blockIdx.x == FA2_TRACE_CTA && (idx) < 1024) g_trace_fwd[(role) * 1024 + (idx)] = clock64(); } while (0)
#else
#define FA2_TF(role, idx) do { } while (0)
#endif

constexpr int kTilesPerCta = 2;
constexpr int kThreads = 384;
constexpr int kRegsSoftmax = 208;   // per scheduler: 2 softmax warps + 1 other warp share the 3 * 168 registers of the launch
constexpr int kRegsOther = 88;

template <int D>
struct FwdSmem {
  static constexpr int kQTileBytes = kBM * D * 2;
  static constexpr int kKVTileBytes = kBN * D * 2;
  static constexpr int kStages = (D == 64) ? 8 : 4;
  static constexpr int kBlockBytes = kBM * 128;       // one [128 rows][64 elements] block
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = kQOff + kTilesPerCta * kQTileBytes;
  static constexpr int kBarOff = kKVOff + kStages * kKVTileBytes;
  // barriers: q_full[2], kv_full[S], kv_empty[S], s_full[2], p_full[2 tiles][2 halves], o_full[2]
  static constexpr int kNumBars = 2 + 2 * kStages + 4 + 2 * kPSplit;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;  // room to align the base to 1024 B
};

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
  auto bar_p_full = [&](int t, int half) { return bars + 8u * (4 + 2 * L::kStages + kPSplit * t + half); };
  auto bar_o_full = [&](int t) { return bars + 8u * (4 + 2 * L::kStages + 2 * kPSplit + t); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  if (tid == 0) FA2_TF(32, 0);

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
      for (int hh = 0; hh < kPSplit; ++hh) mbar_init(bar_p_full(t, hh), kBM);
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
      auto issue_o = [&](int t, int slot, bool first, int half) {
        const uint64_t b0 = sdesc_advance(dKV_mn0, slot * L::kKVTileBytes);
#pragma unroll
        for (int k = half * (kPCols / 16); k < (half + 1) * (kPCols / 16); ++k) {
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
#pragma unroll
              for (int hh = 0; hh < kPSplit; ++hh) {
                ok = mbar_wait(bar_p_full(t, hh), j & 1, abort_flag);
                if (!ok) break;
                if (hh == 0) FA2_TF(t, j);
                tc_fence_after();
                issue_o(t, slot_v, j == 0, hh);
              }
              if (!ok) break;
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
      if (lane == 0) FA2_TF(8 + warp, j);
      softmax_tile_row<D, kBf16, kFeat>(tS, tO, j, j > 0, p, b, h, qi, row_lim, sc, m, l, [] {},
                                        [&](int half) { mbar_arrive(bar_p_full(t, half)); });
      if (lane == 0) FA2_TF(16 + warp, j);
    }
    if (lane == 0) FA2_TF(24 + warp, 0);

    // ---- epilogue: O / l -> 16 bit -> swizzled shared memory -> TMA store; LSE ---------------
    if (ok && tile_valid) {
      ok = mbar_wait(bar_q_full(t), 0, abort_flag);   // Q tile landed: its slot is reused below
      if (ok && nt > 0) ok = mbar_wait(bar_o_full(t), 0, abort_flag);
    }
    if (ok && tile_valid) {
      epilogue_row<D, kBf16, kFeat>(tO, nt > 0, smem_gen + L::kQOff + t * L::kQTileBytes, r, p, b, h, qi, sc, m, l);
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

  if (tid == 0) FA2_TF(33, 0);
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

#ifdef FA2_TRACE
extern "C" int fa2_trace_read_fwd(long long* host, int n) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_trace_fwd, sizeof(long long) * n));
}
#endif

cudaError_t launch_fwd(const FwdLaunch& a, cudaStream_t stream) {
  switch (a.head_dim) {
    case 64: return launch_d<64>(a, stream);
    case 128: return launch_d<128>(a, stream);
    case 256: return launch_fwd256(a, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fa2
