// Second stage of the deterministic dgamma / dbeta reduction.
//
// Stage one (the backward kernels) leaves P partial rows of [2][F] floats in the
// workspace: row p holds the dgamma contributions of one CTA / cluster / batch
// item followed by its dbeta contributions.  This kernel sums the P rows per
// column.  Thread (tx, ty) of a 32 x 32 CTA adds rows ty, ty+32, ... of column
// blockIdx.x*32 + tx in increasing order; the 32 ty-partials are then added in
// increasing ty.  The order never depends on timing, so the result is
// bit-identical from run to run.
//
// Replaces LayerNormGradBetaGammaTempToOut (atex/nv_norms/cc/kernels/
// fused_layer_norm_op.cu:784-803) and ReduceNCtoC (fused_instance_norm_op.cu:442-457).
#include "nvn_host.h"

namespace nvn {

namespace {
constexpr int kTX = 32;
constexpr int kTY = 32;

__global__ void __launch_bounds__(kTX* kTY)
    colreduce_kernel(const float* __restrict__ partials, int64_t P, int64_t F,
                     float* __restrict__ dgamma, float* __restrict__ dbeta) {
  __shared__ float tile[kTY][kTX + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t F2 = 2 * F;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * kTX + tx;
  float s = 0.f;
  if (col < F2) {
    for (int64_t p = ty; p < P; p += kTY) s += partials[p * F2 + col];
  }
  tile[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < F2) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < kTY; ++k) t += tile[k][tx];
    if (col < F) {
      dgamma[col] = t;
    } else {
      dbeta[col - F] = t;
    }
  }
}
}  // namespace

cudaError_t colreduce_launch(const float* partials, int64_t P, int64_t F, float* dgamma,
                             float* dbeta, cudaStream_t s) {
  const int64_t blocks = (2 * F + kTX - 1) / kTX;
  count_launch();
  colreduce_kernel<<<static_cast<unsigned>(blocks), dim3(kTX, kTY), 0, s>>>(partials, P, F,
                                                                           dgamma, dbeta);
  return cudaGetLastError();
}

}  // namespace nvn
