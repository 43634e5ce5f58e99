// Host-side launch record of the backward pass (pre-pass, main kernel, dq conversion).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel_params.cuh"

namespace fa2 {

struct BwdLaunch {
  CUtensorMap tmQ, tmK, tmV, tmdO, tmdK, tmdV;
  // bias / mask as 4-D tensors (Sk, Sq, heads, batch), box 64 keys x 128 query rows: used by the
  // head-dim-64 kernel when it stages these terms in shared memory (kp.bias.staged / kp.mask.staged)
  CUtensorMap tmBias, tmMask;
  BwdKernelParams kp;
  int head_dim;        // 64, 128 or 256: the kernel's (padded) head dim
  int head_dim_real;   // the operands' head dim
  int head_blk;        // real columns in each 64-column block of the padded head dim
  bool bf16, causal, feat;
  const void* o;   long long o_strides[3];    // (batch, sequence, head) element strides
  const void* d_o; long long do_strides[3];
  void* dq;        long long dq_strides[3];
  float* delta;    // start of the row-statistics area of the workspace
  size_t dq_acc_bytes;
  // Optional: recorded before the pre-pass, before the main kernel, after it, after the dq
  // conversion (profiling hook; null = not recorded).
  cudaEvent_t stage_events[4];
};

// Runs the three kernels of the backward pass on `stream`.
cudaError_t launch_bwd(const BwdLaunch& a, cudaStream_t stream);

// Head dim 256 variant (64-query steps, one half of the head dim per CTA); called by launch_bwd.
cudaError_t launch_bwd256(const BwdLaunch& a, cudaStream_t stream);

}  // namespace fa2
