// Split-KV forward: merge of the per-split partial results.
//
// The reference has no counterpart (its forward always walks all keys of a query tile in one
// program, jax_flash_attn2/flash_attention_triton/_forward_triton.py:60-164); splitting exists here
// for problems with too few (batch, head, query tile) items to fill the GPU, e.g. decode steps.
// Every split s produced o_s = softmax over its own keys (already divided by its own row sum, kept
// in fp32 so that the 16-bit rounding happens once, here) and lse_s; the result over all keys is  o = sum_s exp(lse_s - lse) o_s,  lse = log sum_s exp(lse_s).
#include "fwd_launch.cuh"
#include "ptx_sm100.cuh"

namespace fa2 {

template <bool kBf16>
__global__ void __launch_bounds__(128)
fwd_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                   uint16_t* __restrict__ o, long long osb, long long oss, long long osh,
                   float* __restrict__ lse, long long lse_sb, long long lse_sh, long long lse_sq,
                   int n_splits, int B, int Sq, int Hq, int D, int D_part, int d_blk, int sq_pad) {
  // one-dimensional grid (the y and z extents of a grid stop at 65535): row fastest, then head
  const int s = blockIdx.x % Sq;
  const int h = (blockIdx.x / Sq) % Hq;
  const int b = blockIdx.x / (Sq * Hq);
  const long long lse_split = static_cast<long long>(B) * Hq * sq_pad;
  const float* pl = part_lse + (static_cast<long long>(b) * Hq + h) * sq_pad + s;
  float m = -INFINITY;
  for (int k = 0; k < n_splits; ++k) m = fmaxf(m, pl[k * lse_split]);
  float sum = 0.f;
  if (m > -INFINITY)
    for (int k = 0; k < n_splits; ++k) sum += __expf(pl[k * lse_split] - m);
  const float total = (m > -INFINITY) ? m + __logf(sum) : -INFINITY;
  if (threadIdx.x == 0)
    lse[static_cast<long long>(b) * lse_sb + static_cast<long long>(h) * lse_sh +
        static_cast<long long>(s) * lse_sq] = total;
  const long long o_split = static_cast<long long>(B) * Sq * Hq * D_part;
  const float* po = part_o + ((static_cast<long long>(b) * Sq + s) * Hq + h) * D_part;
  uint16_t* dst = o + b * osb + s * oss + h * osh;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    // a head dim the kernels are not built for sits in 64-column blocks of d_blk real columns
    const int col = (d / d_blk) * 64 + d % d_blk;
    float acc = 0.f;
    if (m > -INFINITY)
      for (int k = 0; k < n_splits; ++k)
        acc += __expf(pl[k * lse_split] - total) * po[k * o_split + col];
    dst[d] = static_cast<uint16_t>(pack2<kBf16>(acc, 0.f) & 0xffffu);
  }
}

cudaError_t launch_fwd_combine(const FwdCombine& c, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>(static_cast<long long>(c.Sq) * c.Hq * c.B);
  if (c.bf16)
    fwd_combine_kernel<true><<<grid, 128, 0, stream>>>(
        c.part_o, c.part_lse, static_cast<uint16_t*>(c.o), c.o_strides[0],
        c.o_strides[1], c.o_strides[2], c.lse, c.lse_sb, c.lse_sh, c.lse_sq, c.n_splits, c.B, c.Sq, c.Hq,
        c.D, c.D_part, c.d_blk, c.sq_pad);
  else
    fwd_combine_kernel<false><<<grid, 128, 0, stream>>>(
        c.part_o, c.part_lse, static_cast<uint16_t*>(c.o), c.o_strides[0],
        c.o_strides[1], c.o_strides[2], c.lse, c.lse_sb, c.lse_sh, c.lse_sq, c.n_splits, c.B, c.Sq, c.Hq,
        c.D, c.D_part, c.d_blk, c.sq_pad);
  return cudaGetLastError();
}

}  // namespace fa2
