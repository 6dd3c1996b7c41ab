// Host interface of the two-phase kernels (twophase.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace nvn {

// Family R2: [rows, D] with D contiguous.
struct R2Plan {
  int64_t chunk;  // elements of D per phase-1 CTA
  int nchunks;
  int grid_y;
  int64_t rows_per_slice;  // LayerNorm backward: rows per dgamma/dbeta partial row
  int slices;
};

struct R2Args {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  float* mean;  // forward: output; backward: the saved statistics (read only)
  float* ivar;
  void* out;
  float* ws_part;     // fwd: [rows][nchunks][3]   bwd: [rows][nchunks][2]
  float* ws_coef;     // bwd: [rows][2]
  float* ws_colpart;  // bwd: LayerNorm [slices][2][D]; row-affine [N][2][C]
  int64_t rows;
  int64_t D;
  int64_t C;
  float eps;
  bool row_affine;
};

R2Plan r2_plan(int64_t rows, int64_t D, int epv, bool ln_bwd);
cudaError_t r2_launch(int dtype, bool bwd, bool scalar, const R2Args& a, const R2Plan& p,
                      cudaStream_t s);

// Family S2: x[n, d, c] with C contiguous, reduced over d.
struct S2Plan {
  int64_t chunk;  // voxels per phase-1 CTA
  int nchunks;
  int cvt;     // channel vectors per CTA tile
  int lanes;   // voxel lanes per CTA
  int ctiles;  // channel tiles
  int group;   // batch items per launch group
  size_t smem_fwd;
  size_t smem_bwd;
};

struct S2Args {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  float* mean;
  float* ivar;
  void* out;
  float* ws_part;     // fwd: [N][nchunks][3][C]   bwd: [N][nchunks][2][C]
  float* ws_coef;     // bwd: [N][3][C]
  float* ws_colpart;  // bwd: [N][2][C]
  int64_t N;
  int64_t C;
  int64_t D;
  float eps;
};

S2Plan s2_plan(int dtype, bool bwd, int64_t N, int64_t C, int64_t D, int epv);
cudaError_t s2_launch(int dtype, bool bwd, bool scalar, const S2Args& a, const S2Plan& p,
                      cudaStream_t s);

}  // namespace nvn
