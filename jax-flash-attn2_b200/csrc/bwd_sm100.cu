#include "bwd_launch.cuh"
namespace fa2 {
cudaError_t launch_bwd(const BwdLaunch&, cudaStream_t) { return cudaErrorNotSupported; }
}
