// Host-side launch records handed from the C-ABI layer to the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel_params.cuh"

namespace fa2 {

struct FwdLaunch {
  CUtensorMap tmQ, tmK, tmV, tmO;
  CUtensorMap tmO1;   // o with a box of one 64-column block (head dim 64 / 128 kernel)
  FwdKernelParams kp;
  int head_dim;
  bool bf16, causal, feat;
};

// Launches the forward kernel specialised for (head_dim, dtype, causal, score terms/dropout).
cudaError_t launch_fwd(const FwdLaunch& a, cudaStream_t stream);

// Head dim 256 variant (one query tile per CTA, two S buffers); called by launch_fwd.
cudaError_t launch_fwd256(const FwdLaunch& a, cudaStream_t stream);

}  // namespace fa2
