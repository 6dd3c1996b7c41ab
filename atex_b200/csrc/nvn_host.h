// Host-side declarations shared by the kernel translation units and the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace nvn {

// Arguments of the row-cached kernels (rows_kernels.cuh).  `out` is y (forward)
// or dx (backward); `mean` / `ivar` are forward outputs, `mean_in` / `ivar_in`
// backward inputs.  C is the channel count when gamma / beta are indexed by
// row % C (InstanceNorm "NC..."), unused otherwise.
struct RowsArgs {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  const float* mean_in;
  const float* ivar_in;
  void* out;
  float* mean;
  float* ivar;
  float* ws;
  int64_t N;
  int64_t D;
  int64_t C;
  float eps;
};

struct RowsPlan {
  int grid;
  int block;
  int cluster;
  int tpr;
  int vpt;
  int epv;
  int partial_rows;  // rows of [2][D] dgamma/dbeta partials the backward kernel writes
};

int device_sm_count();
void count_launch();

// Row-group shapes (TPR threads per row, VPT vectors per thread, CS CTAs per
// cluster), ordered by capacity TPR*VPT*CS vectors.  X(index, TPR, VPT, CS).
// Forward keeps VPT*EPV values (+ gamma/beta) per thread, backward about twice
// that plus the dgamma/dbeta accumulators, so backward uses more threads per row.
#define NVN_ROW_SHAPES_FWD(X)                                                                \
  X(0, 4, 1, 1)    X(1, 8, 1, 1)    X(2, 16, 1, 1)   X(3, 32, 1, 1)   X(4, 32, 2, 1)         \
  X(5, 32, 4, 1)   X(6, 64, 2, 1)   X(7, 64, 4, 1)   X(8, 128, 2, 1)  X(9, 128, 4, 1)        \
  X(10, 256, 2, 1) X(11, 256, 4, 1) X(12, 512, 2, 1) X(13, 512, 4, 1) X(14, 1024, 2, 1)      \
  X(15, 512, 4, 2) X(16, 512, 4, 4) X(17, 256, 4, 8) X(18, 512, 4, 8) X(19, 512, 4, 16)      \
  X(20, 512, 8, 16)

#define NVN_ROW_SHAPES_BWD(X)                                                                \
  X(0, 4, 1, 1)    X(1, 8, 1, 1)    X(2, 16, 1, 1)   X(3, 32, 1, 1)   X(4, 32, 2, 1)         \
  X(5, 64, 2, 1)   X(6, 128, 2, 1)  X(7, 256, 2, 1)  X(8, 512, 2, 1)  X(9, 256, 2, 4)        \
  X(10, 512, 2, 2) X(11, 512, 2, 4) X(12, 256, 2, 8) X(13, 512, 2, 8) X(14, 512, 2, 16)      \
  X(15, 512, 4, 16)

// Scalar (EPV == 1) rows only get a coarse subset: they exist for odd D and
// misaligned buffers, where correctness matters more than the last GB/s.
#define NVN_ROW_SHAPES_SCALAR(X)                                                             \
  X(0, 8, 4, 1) X(1, 32, 8, 1) X(2, 256, 8, 1) X(3, 512, 8, 2) X(4, 512, 8, 8)               \
  X(5, 512, 8, 16)

// One entry point per (dtype, direction) translation unit.  `scalar` selects
// the EPV == 1 family, `row_affine` the InstanceNorm "NC..." parameter indexing.
// With dry_run the plan is filled in and nothing is launched.
#define NVN_DECLARE_ROWS(NAME)                                                              \
  cudaError_t NAME(bool row_affine, bool scalar, int shape, const RowsArgs& a, cudaStream_t s, \
                   bool dry_run, RowsPlan* plan);
NVN_DECLARE_ROWS(rows_f32_fwd)
NVN_DECLARE_ROWS(rows_f32_bwd)
NVN_DECLARE_ROWS(rows_f16_fwd)
NVN_DECLARE_ROWS(rows_f16_bwd)
NVN_DECLARE_ROWS(rows_bf16_fwd)
NVN_DECLARE_ROWS(rows_bf16_bwd)

// Deterministic second stage of the dgamma / dbeta reduction: sums P partial
// rows of [2][F] floats (dgamma then dbeta) in a fixed order.
cudaError_t colreduce_launch(const float* partials, int64_t P, int64_t F, float* dgamma,
                             float* dbeta, cudaStream_t s);

}  // namespace nvn
