// Second stage of the deterministic dgamma / dbeta reduction.
//
// Stage one (the backward kernels) leaves P partial rows of [2][F] floats in the
// workspace: row p holds the dgamma contributions of one CTA / cluster / batch
// item / row slice followed by its dbeta contributions.  This kernel sums the P
// rows per column.  Thread (tx, ty) of a 32 x TY CTA adds rows ty, ty+TY, ... of
// its columns in increasing order; the TY partial sums are then added in
// increasing ty.  The order never depends on timing, so the result is
// bit-identical from run to run.  TY follows P (few partial rows: small CTAs and
// many of them; many partial rows: 32 row lanes); when 2F is a multiple of 4 a
// thread covers four adjacent columns with 128-bit loads.
//
// Replaces LayerNormGradBetaGammaTempToOut (atex/nv_norms/cc/kernels/
// fused_layer_norm_op.cu:784-803) and ReduceNCtoC (fused_instance_norm_op.cu:442-457).
#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

namespace {
constexpr int kTX = 32;

template <int TY, int W>  // W columns per thread: 4 (float4) or 1
__global__ void __launch_bounds__(kTX* TY)
    colreduce_kernel(const float* __restrict__ partials, int64_t P, int64_t F,
                     float* __restrict__ dgamma, float* __restrict__ dbeta,
                     int64_t slab_rows, float* __restrict__ slab_out) {
  __shared__ float tile[TY][kTX * W + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t F2 = 2 * F;
  const int64_t col = (static_cast<int64_t>(blockIdx.x) * kTX + tx) * W;
  // blockIdx.y selects a slab of rows (a single slab covers all rows)
  const int64_t p_begin = static_cast<int64_t>(blockIdx.y) * slab_rows;
  const int64_t p_end = p_begin + slab_rows < P ? p_begin + slab_rows : P;
  griddep_launch_dependents();  // the next kernel in the stream may be scheduled early
  griddep_wait();  // the partial rows come from the kernel launched just before
  float s[W];
#pragma unroll
  for (int w = 0; w < W; ++w) s[w] = 0.f;
  if (col < F2) {
    for (int64_t p = p_begin + ty; p < p_end; p += TY) {
      if constexpr (W == 4) {
        const float4 v = *reinterpret_cast<const float4*>(partials + p * F2 + col);
        s[0] += v.x;
        s[1] += v.y;
        s[2] += v.z;
        s[3] += v.w;
      } else {
        s[0] += partials[p * F2 + col];
      }
    }
  }
#pragma unroll
  for (int w = 0; w < W; ++w) tile[ty][tx * W + w] = s[w];
  __syncthreads();
  if (ty == 0 && col < F2) {
#pragma unroll
    for (int w = 0; w < W; ++w) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < TY; ++k) t += tile[k][tx * W + w];
      const int64_t c = col + w;
      if (slab_out != nullptr) {
        slab_out[static_cast<int64_t>(blockIdx.y) * F2 + c] = t;
      } else if (c < F) {
        dgamma[c] = t;
      } else {
        dbeta[c - F] = t;
      }
    }
  }
}

template <int TY, int W>
cudaError_t launch(const float* partials, int64_t P, int64_t F, float* dgamma, float* dbeta,
                   cudaStream_t s, int64_t slabs = 1, float* slab_out = nullptr) {
  const int64_t blocks = (2 * F + kTX * W - 1) / (kTX * W);
  const int64_t slab_rows = (P + slabs - 1) / slabs;
  count_launch();
  cudaLaunchAttribute attr;
  const cudaLaunchConfig_t cfg = dependent_launch_config(
      dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(slabs)), dim3(kTX, TY), 0, s, &attr);
  return cudaLaunchKernelEx(&cfg, colreduce_kernel<TY, W>, partials, P, F, dgamma, dbeta,
                            slab_rows, slab_out);
}
}  // namespace

// With few columns and very many partial rows (InstanceNorm over a large batch: one partial
// row per item) the column tiles alone give a handful of CTAs.  Given scratch for
// `scratch_rows` rows of [2F], the rows are then cut into slabs that are reduced side by side
// and a second launch sums the slab results; the order of the additions stays fixed.
cudaError_t colreduce_launch(const float* partials, int64_t P, int64_t F, float* dgamma,
                             float* dbeta, cudaStream_t s, float* scratch, int64_t scratch_rows) {
  const bool vec = (2 * F) % 4 == 0 && (reinterpret_cast<uintptr_t>(partials) & 15) == 0;
  const int64_t col_blocks = (2 * F + kTX * (vec ? 4 : 1) - 1) / (kTX * (vec ? 4 : 1));
  if (scratch != nullptr && scratch_rows >= 2 && P >= 4096 && col_blocks < 64) {
    int64_t slabs = P / 1024;  // at least 1024 rows per slab
    if (slabs > scratch_rows) slabs = scratch_rows;
    if (slabs * col_blocks > 1024) slabs = 1024 / col_blocks;
    if (slabs >= 2) {
      const cudaError_t e = vec ? launch<32, 4>(partials, P, F, dgamma, dbeta, s, slabs, scratch)
                                : launch<32, 1>(partials, P, F, dgamma, dbeta, s, slabs, scratch);
      if (e != cudaSuccess) return e;
      return colreduce_launch(scratch, slabs, F, dgamma, dbeta, s, nullptr, 0);
    }
  }
  if (vec) {
    if (P <= 4) return launch<1, 4>(partials, P, F, dgamma, dbeta, s);
    if (P <= 32) return launch<4, 4>(partials, P, F, dgamma, dbeta, s);
    // Few columns and more than a handful of partial rows (LayerNorm backward at D = 1024: 444
    // rows of 2048 floats): four columns per thread would leave 16 CTAs to fetch 3.6 MB, a
    // chain of L2 latencies.  One column per thread gives four times as many CTAs; the row
    // lanes (TY), hence the order of every column's additions, stay the same.
    const bool narrow = col_blocks < 64;
    if (P <= 128 || 2 * F >= 32768)
      return narrow ? launch<8, 1>(partials, P, F, dgamma, dbeta, s)
                    : launch<8, 4>(partials, P, F, dgamma, dbeta, s);
    return narrow ? launch<32, 1>(partials, P, F, dgamma, dbeta, s)
                  : launch<32, 4>(partials, P, F, dgamma, dbeta, s);
  }
  if (P <= 32) return launch<4, 1>(partials, P, F, dgamma, dbeta, s);
  return launch<32, 1>(partials, P, F, dgamma, dbeta, s);
}

}  // namespace nvn
