// Host-side launch records handed from the C-ABI layer to the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel_params.cuh"

namespace fa2 {

// Head dim 256: a K / V slot of the forward is handed over in this many pieces (K by head-dim
// blocks, V by key rows); the host builds the tensor maps of K and V with matching boxes.
// Measured on B=4, S=8192, H=8 causal fp16: one piece 1.20 ms, two 1.10-1.12 ms, four 1.11 ms.
constexpr int kKV256Parts = 2;

struct FwdLaunch {
  CUtensorMap tmQ, tmK, tmV, tmO;
  CUtensorMap tmO1;   // o with a box of one 64-column block (head dim 64 / 128 kernel)
  // bias / mask as 4-D tensors (Sk, Sq, heads, batch) with a box of 64 keys x 32 query rows: used
  // by the kernels that stage these terms in shared memory (kp.bias.staged / kp.mask.staged)
  CUtensorMap tmBias, tmMask;
  FwdKernelParams kp;
  int head_dim;
  bool bf16, causal, feat;
};

// Split-KV: merges the partial results of the splits into the caller's output and lse.
//   part_o   [n_splits, B, Sq, Hq, D]  normalised partial outputs (the q dtype, contiguous)
//   part_lse [n_splits, B, Hq, sq_pad] natural-log lse of every split (-inf: the split saw no key)
struct FwdCombine {
  const float* part_o;        // [n_splits * B][Sq][Hq][D_part], fp32
  const float* part_lse;
  void* o;
  long long o_strides[3];     // (batch, sequence, head) element strides of o
  float* lse;
  long long lse_sb, lse_sh, lse_sq;
  int n_splits, B, Sq, Hq, D, sq_pad;
  int D_part;                 // row length of part_o: the kernel's (padded) head dim
  int d_blk;                  // real columns in each 64-column block of a part_o row
  bool bf16;
};
cudaError_t launch_fwd_combine(const FwdCombine& c, cudaStream_t stream);

// Launches the forward kernel specialised for (head_dim, dtype, causal, score terms/dropout).
cudaError_t launch_fwd(const FwdLaunch& a, cudaStream_t stream);

// Head dim 256 variant (one query tile per CTA, two S buffers); called by launch_fwd.
cudaError_t launch_fwd256(const FwdLaunch& a, cudaStream_t stream);

}  // namespace fa2
