// Row-cached normalisation kernels: the reduced axis is the contiguous one
// (LayerNorm [N, D]; InstanceNorm "NC..." with one row per (n, c)).
//
// One row is owned by a *row group*: TPR threads of a CTA (4 ... 1024), or a
// whole thread-block cluster of CS CTAs for very wide rows.  Every thread keeps
// VPT vectors of EPV elements of its row in registers, so x (and dy) are read
// from HBM exactly once; the statistics are exact two-pass sums over the cached
// values (mean first, then centred squares), combined with nvn::group_allreduce.
// CTAs are persistent: the grid is sized to the number of resident CTAs and each
// row group strides over the rows.
//
// Backward additionally accumulates, per thread, the dgamma / dbeta contributions
// of its fixed columns over all rows it visits and writes one partial row per
// CTA (cluster) to the workspace; nvn::colreduce sums the partial rows in a
// fixed order (deterministic two-stage reduction).
//
// These kernels replace, for every D they can cache,
//   LayerNormWarpImplWelford / LayerNormBlockSMemImpl / LayerNormRowReduce*Welford
//     (atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:374-433, 143-193, 445-481, 572-684)
//   LayerNormGradWarpImpl / LayerNormGradBlockSMemImpl / LayerNormGradBetaGamma*
//     (fused_layer_norm_op.cu:21-98, 195-255, 741-803)
//   InstanceNormBlockSMemChnlFirstImpl / GeneralNormRowReduceInToOutWelford /
//   InstanceNormGradBlockSMemImpl / InstanceNormRowReduceInToOutFused
//     (atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:959-1003, 1167-1194, 169-250, 315-366)
#pragma once

#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

template <int TPR>
struct RowBlock {
  static constexpr int kBlock = TPR >= 256 ? TPR : 256;
  static constexpr int kRowsPerCta = kBlock / TPR;
};

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T, int EPV, int VPT, int TPR, int CS, bool ROW_AFFINE>
__global__ void __launch_bounds__(RowBlock<TPR>::kBlock)
    rows_fwd_kernel(const RowsArgs a) {
  constexpr int BLOCK = RowBlock<TPR>::kBlock;
  constexpr int RPC = RowBlock<TPR>::kRowsPerCta;
  static_assert(CS == 1 || RPC == 1, "cluster kernels own one row per cluster");
  constexpr bool PARAMS_IN_REGS = !ROW_AFFINE && (VPT * EPV <= 32);

  __shared__ ReduceSmem<1, BLOCK> sm;
  int phase = 0;

  // y may alias x (in-place forward), so neither pointer is __restrict__.
  const T* x = static_cast<const T*>(a.x);
  T* y = static_cast<T*>(a.out);
  const int tid = threadIdx.x;
  const int group = tid / TPR;
  const int lir = tid % TPR;
  unsigned crank = 0;
  if constexpr (CS > 1) crank = cg::this_cluster().block_rank();
  const int64_t unit = blockIdx.x / CS;
  const int64_t nunits = gridDim.x / CS;
  const int64_t D = a.D;
  const int nvec = static_cast<int>(D / EPV);
  const float fD = static_cast<float>(D);

  int col[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int vi = v * (TPR * CS) + static_cast<int>(crank) * TPR + lir;
    col[v] = vi < nvec ? vi * EPV : -1;
  }

  float g[PARAMS_IN_REGS ? VPT : 1][EPV], b[PARAMS_IN_REGS ? VPT : 1][EPV];
  if constexpr (PARAMS_IN_REGS) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (col[v] >= 0) {
        load_params<EPV>(a.gamma, col[v], g[v]);
        load_params<EPV>(a.beta, col[v], b[v]);
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) g[v][e] = b[v][e] = 0.f;
      }
    }
  }

  for (int64_t row0 = unit * RPC; row0 < a.N; row0 += nunits * RPC) {
    const int64_t row = row0 + group;
    const bool rv = row < a.N;
    const int64_t base = row * D;

    float xf[VPT][EPV];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && col[v] >= 0) {
        const Pack<T, EPV> p = load_stream<T, EPV>(x, base + col[v]);
#pragma unroll
        for (int e = 0; e < EPV; ++e) xf[v][e] = Cvt<T>::to_f32(p.v[e]);
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) xf[v][e] = 0.f;
      }
    }

    float s[1] = {0.f};
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
      for (int e = 0; e < EPV; ++e) s[0] += xf[v][e];
    group_allreduce<1, TPR, BLOCK, CS>(s, sm, phase);
    const float mean = s[0] / fD;

    float q[1] = {0.f};
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (col[v] >= 0) {
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
          const float d = xf[v][e] - mean;
          q[0] = fmaf(d, d, q[0]);
        }
      }
    }
    group_allreduce<1, TPR, BLOCK, CS>(q, sm, phase);
    const float ivar = 1.0f / sqrtf(q[0] / fD + a.eps);

    float gr = 1.f, br = 0.f;
    if constexpr (ROW_AFFINE) {
      if (rv) {
        const int64_t c = row % a.C;
        gr = __ldg(a.gamma + c);
        br = __ldg(a.beta + c);
      }
    }

#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && col[v] >= 0) {
        Pack<T, EPV> o;
        if constexpr (ROW_AFFINE) {
          const float sc = ivar * gr;
#pragma unroll
          for (int e = 0; e < EPV; ++e)
            o.v[e] = Cvt<T>::from_f32(fmaf(xf[v][e] - mean, sc, br));
        } else if constexpr (PARAMS_IN_REGS) {
#pragma unroll
          for (int e = 0; e < EPV; ++e)
            o.v[e] = Cvt<T>::from_f32(fmaf((xf[v][e] - mean) * ivar, g[v][e], b[v][e]));
        } else {
          float gg[EPV], bb[EPV];
          load_params<EPV>(a.gamma, col[v], gg);
          load_params<EPV>(a.beta, col[v], bb);
#pragma unroll
          for (int e = 0; e < EPV; ++e)
            o.v[e] = Cvt<T>::from_f32(fmaf((xf[v][e] - mean) * ivar, gg[e], bb[e]));
        }
        store_stream<T, EPV>(y, base + col[v], o);
      }
    }
    if (rv && lir == 0 && crank == 0) {
      a.mean[row] = mean;
      a.ivar[row] = ivar;
    }
  }
  // A CTA's shared memory must stay mapped until its cluster peers have read it.
  if constexpr (CS > 1) cg::this_cluster().sync();
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
template <typename T, int EPV, int VPT, int TPR, int CS, bool ROW_AFFINE>
__global__ void __launch_bounds__(RowBlock<TPR>::kBlock)
    rows_bwd_kernel(const RowsArgs a) {
  constexpr int BLOCK = RowBlock<TPR>::kBlock;
  constexpr int RPC = RowBlock<TPR>::kRowsPerCta;
  static_assert(CS == 1 || RPC == 1, "cluster kernels own one row per cluster");
  constexpr bool PARAMS_IN_REGS = !ROW_AFFINE && (VPT * EPV <= 16);
  constexpr int CAP = TPR * VPT * EPV;  // columns one row group covers (CS == 1)

  __shared__ ReduceSmem<2, BLOCK> sm;
  __shared__ float comb[(!ROW_AFFINE && RPC > 1) ? 2 * CAP : 1];
  int phase = 0;

  const T* __restrict__ x = static_cast<const T*>(a.x);
  const T* __restrict__ dy = static_cast<const T*>(a.dy);
  T* __restrict__ dx = static_cast<T*>(a.out);
  const int tid = threadIdx.x;
  const int group = tid / TPR;
  const int lir = tid % TPR;
  unsigned crank = 0;
  if constexpr (CS > 1) crank = cg::this_cluster().block_rank();
  const int64_t unit = blockIdx.x / CS;
  const int64_t nunits = gridDim.x / CS;
  const int64_t D = a.D;
  const int nvec = static_cast<int>(D / EPV);
  const float inv_D = 1.0f / static_cast<float>(D);

  int col[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int vi = v * (TPR * CS) + static_cast<int>(crank) * TPR + lir;
    col[v] = vi < nvec ? vi * EPV : -1;
  }

  float g[PARAMS_IN_REGS ? VPT : 1][EPV];
  float dg[ROW_AFFINE ? 1 : VPT][EPV], db[ROW_AFFINE ? 1 : VPT][EPV];
  if constexpr (PARAMS_IN_REGS) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (col[v] >= 0) {
        load_params<EPV>(a.gamma, col[v], g[v]);
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) g[v][e] = 0.f;
      }
    }
  }
  if constexpr (!ROW_AFFINE) {
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
      for (int e = 0; e < EPV; ++e) dg[v][e] = db[v][e] = 0.f;
  }

  for (int64_t row0 = unit * RPC; row0 < a.N; row0 += nunits * RPC) {
    const int64_t row = row0 + group;
    const bool rv = row < a.N;
    const int64_t base = row * D;

    Pack<T, EPV> px[VPT], pdy[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && col[v] >= 0) {
        px[v] = load_stream<T, EPV>(x, base + col[v]);
        pdy[v] = load_stream<T, EPV>(dy, base + col[v]);
      }
    }
    float mean = 0.f, ivar = 0.f;
    if (rv) {
      mean = __ldg(a.mean_in + row);
      ivar = __ldg(a.ivar_in + row);
    }

    // xh = (x - mean) * ivar ; gy = dy * gamma (LayerNorm) or dy (row-affine)
    float xh[VPT][EPV], gy[VPT][EPV];
    float r[2] = {0.f, 0.f};
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && col[v] >= 0) {
        float gg[EPV];
        if constexpr (!ROW_AFFINE && !PARAMS_IN_REGS) load_params<EPV>(a.gamma, col[v], gg);
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
          const float xv = (Cvt<T>::to_f32(px[v].v[e]) - mean) * ivar;
          const float dv = Cvt<T>::to_f32(pdy[v].v[e]);
          xh[v][e] = xv;
          if constexpr (ROW_AFFINE) {
            gy[v][e] = dv;
          } else {
            dg[v][e] = fmaf(dv, xv, dg[v][e]);
            db[v][e] += dv;
            if constexpr (PARAMS_IN_REGS) {
              gy[v][e] = dv * g[v][e];
            } else {
              gy[v][e] = dv * gg[e];
            }
          }
          r[0] += gy[v][e];
          r[1] = fmaf(gy[v][e], xv, r[1]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) xh[v][e] = gy[v][e] = 0.f;
      }
    }
    group_allreduce<2, TPR, BLOCK, CS>(r, sm, phase);

    float scale = ivar;
    if constexpr (ROW_AFFINE) {
      if (rv) {
        const int64_t n = row / a.C;
        const int64_t c = row - n * a.C;
        scale = ivar * __ldg(a.gamma + c);
        if (lir == 0 && crank == 0) {
          // per-(n, c) partials laid out [n][2][C]: dgamma then dbeta
          a.ws[(n * 2 + 0) * a.C + c] = r[1];
          a.ws[(n * 2 + 1) * a.C + c] = r[0];
        }
      }
    }
    const float m0 = r[0] * inv_D, m1 = r[1] * inv_D;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && col[v] >= 0) {
        Pack<T, EPV> o;
#pragma unroll
        for (int e = 0; e < EPV; ++e)
          o.v[e] = Cvt<T>::from_f32(scale * (gy[v][e] - fmaf(xh[v][e], m1, m0)));
        store_stream<T, EPV>(dx, base + col[v], o);
      }
    }
  }

  if constexpr (!ROW_AFFINE) {
    float* __restrict__ wg = a.ws + (unit * 2 + 0) * D;
    float* __restrict__ wb = a.ws + (unit * 2 + 1) * D;
    if constexpr (RPC > 1) {
      // Fold the row groups of this CTA in group order, then group 0 writes.
      for (int rgrp = 0; rgrp < RPC; ++rgrp) {
        if (group == rgrp) {
#pragma unroll
          for (int v = 0; v < VPT; ++v)
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
              const int idx = (v * EPV + e) * TPR + lir;
              if (rgrp == 0) {
                comb[idx] = dg[v][e];
                comb[CAP + idx] = db[v][e];
              } else {
                comb[idx] += dg[v][e];
                comb[CAP + idx] += db[v][e];
              }
            }
        }
        __syncthreads();
      }
      if (group == 0) {
#pragma unroll
        for (int v = 0; v < VPT; ++v)
#pragma unroll
          for (int e = 0; e < EPV; ++e) {
            const int idx = (v * EPV + e) * TPR + lir;
            dg[v][e] = comb[idx];
            db[v][e] = comb[CAP + idx];
          }
      }
    }
    if (group == 0) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        if (col[v] >= 0) {
          store_params<EPV>(wg, col[v], dg[v]);
          store_params<EPV>(wb, col[v], db[v]);
        }
      }
    }
  }
  if constexpr (CS > 1) cg::this_cluster().sync();
}

// ---------------------------------------------------------------------------
// host-side launcher for one (T, EPV, affine, direction) family
// ---------------------------------------------------------------------------
template <typename Kernel>
inline int resident_units(Kernel kernel, int block, int cs) {
  // Number of CTAs (CS == 1) or clusters that fit on the current device at once.
  int sms = device_sm_count();
  if (cs == 1) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, 0) != cudaSuccess ||
        per_sm < 1)
      per_sm = 1;
    return sms * per_sm;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sms * cs), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(block), 1, 1);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cs);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
    (void)cudaGetLastError();
    clusters = sms / cs > 0 ? sms / cs : 1;
  }
  return clusters;
}

template <typename T, int EPV, int VPT, int TPR, int CS, bool ROW_AFFINE, bool BWD>
inline cudaError_t launch_rows_one(const RowsArgs& a, cudaStream_t stream, bool dry_run,
                                   RowsPlan* plan) {
  constexpr int BLOCK = RowBlock<TPR>::kBlock;
  constexpr int RPC = RowBlock<TPR>::kRowsPerCta;
  void (*kernel)(const RowsArgs);
  if constexpr (BWD) {
    kernel = rows_bwd_kernel<T, EPV, VPT, TPR, CS, ROW_AFFINE>;
  } else {
    kernel = rows_fwd_kernel<T, EPV, VPT, TPR, CS, ROW_AFFINE>;
  }
  // Cached per process: every device this library runs on is the same part.
  static std::atomic<int> cached_units{0};
  int units = cached_units.load(std::memory_order_relaxed);
  if (units == 0) {
    if (CS > 8) {
      cudaError_t e =
          cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) return e;
    }
    units = resident_units(kernel, BLOCK, CS);
    cached_units.store(units, std::memory_order_relaxed);
  }
  const int64_t need = (a.N + RPC - 1) / RPC;
  const int64_t use = need < units ? need : units;
  plan->grid = static_cast<int>(use) * CS;
  plan->block = BLOCK;
  plan->cluster = CS;
  plan->tpr = TPR;
  plan->vpt = VPT;
  plan->epv = EPV;
  plan->partial_rows = static_cast<int>(use);
  if (dry_run) return cudaSuccess;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan->grid), 1, 1);
  cfg.blockDim = dim3(BLOCK, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (CS > 1) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <typename T, bool ROW_AFFINE, bool BWD>
cudaError_t launch_rows_vec(int shape, const RowsArgs& a, cudaStream_t s, bool dry, RowsPlan* p) {
  constexpr int EPV = VecTraits<T>::kFull;
#define X(I, TPR, VPT, CS) \
  case I:                  \
    return launch_rows_one<T, EPV, VPT, TPR, CS, ROW_AFFINE, BWD>(a, s, dry, p);
  if constexpr (BWD) {
    switch (shape) {
      NVN_ROW_SHAPES_BWD(X)
      default:
        return cudaErrorInvalidValue;
    }
  } else {
    switch (shape) {
      NVN_ROW_SHAPES_FWD(X)
      default:
        return cudaErrorInvalidValue;
    }
  }
#undef X
}

template <typename T, bool ROW_AFFINE, bool BWD>
cudaError_t launch_rows_scalar(int shape, const RowsArgs& a, cudaStream_t s, bool dry,
                               RowsPlan* p) {
  switch (shape) {
#define X(I, TPR, VPT, CS) \
  case I:                  \
    return launch_rows_one<T, 1, VPT, TPR, CS, ROW_AFFINE, BWD>(a, s, dry, p);
    NVN_ROW_SHAPES_SCALAR(X)
#undef X
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace nvn
