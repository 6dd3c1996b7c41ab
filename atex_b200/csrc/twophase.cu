// Two-phase normalisation kernels for reductions that cannot be cached on chip.
//
// Family R2 - the reduced axis is contiguous ([rows, D]; LayerNorm rows too wide
//   for a 16-CTA cluster, InstanceNorm "NC..." with huge spatial extents).
// Family S2 - channels-last InstanceNorm, x[n, d, c] reduced over d with the
//   C channels contiguous.  One thread owns EPV adjacent channels and walks the
//   voxels of its D-chunk, so every access is a full vector and (n, c) comes from
//   the tile coordinates instead of a per-element division.
//
// Phase 1 reduces each (row | n, channel) over chunks of D into workspace
// partials: Welford (mean, M2, count) triples forward, plain sums backward.  A
// small finalize kernel merges the chunk partials in chunk order; phase 2 is the
// element-wise pass.  All merges happen in a fixed order (shuffle butterfly,
// shared-memory tree, then chunk index), so results are bit-identical run to run.
//
// Replaces the reference's temp-buffer paths:
//   LayerNormRowReduceInToTemp(Welford) / TempToOut(Welford) / Forward|BackwardUpdate
//     (atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:523-719)
//   InstanceNormToTempWelford / TempToOutWelford / InstanceNormUpdate(Vectorized)
//     (atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:23-101, 774-818)
//   InstanceNormRowReduceInToTempFused(Vectorized) / TempToOutFused / UpdateFused(Vectorized)
//     (fused_instance_norm_op.cu:594-763, 103-146)
#include "nvn_common.cuh"
#include "nvn_host.h"
#include "twophase.h"

namespace nvn {
namespace {

constexpr int kBlock = 256;
constexpr int kUnroll = 4;

// ---------------------------------------------------------------------------
// Welford / Chan merge (norm_util.h:182-211 semantics: biased variance = m2 / n)
// ---------------------------------------------------------------------------
struct WF {
  float mean, m2, n;
};

__device__ __forceinline__ WF wf_merge(const WF& a, const WF& b) {
  WF r;
  r.n = a.n + b.n;
  if (r.n == 0.f) {
    r.mean = 0.f;
    r.m2 = 0.f;
    return r;
  }
  const float delta = b.mean - a.mean;
  const float f = b.n / r.n;
  r.mean = fmaf(delta, f, a.mean);
  r.m2 = a.m2 + b.m2 + delta * delta * a.n * f;
  return r;
}

// Merge a batch of K values given as (sum, centred M2 about the batch mean).
template <int K>
__device__ __forceinline__ void wf_add_batch(WF& acc, const float (&v)[K]) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < K; ++i) s += v[i];
  WF b;
  b.mean = s * (1.0f / K);
  b.m2 = 0.f;
#pragma unroll
  for (int i = 0; i < K; ++i) {
    const float d = v[i] - b.mean;
    b.m2 = fmaf(d, d, b.m2);
  }
  b.n = static_cast<float>(K);
  acc = wf_merge(acc, b);
}

__device__ __forceinline__ WF wf_block_reduce(WF w, WF* smem /*[kBlock/32]*/) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    WF o;
    o.mean = __shfl_xor_sync(0xffffffffu, w.mean, off);
    o.m2 = __shfl_xor_sync(0xffffffffu, w.m2, off);
    o.n = __shfl_xor_sync(0xffffffffu, w.n, off);
    // keep the merge order independent of the lane: lower lane is always "a"
    const bool low = (threadIdx.x & off) == 0;
    w = low ? wf_merge(w, o) : wf_merge(o, w);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = w;
  __syncthreads();
  WF t = smem[0];
#pragma unroll
  for (int k = 1; k < kBlock / 32; ++k) t = wf_merge(t, smem[k]);
  __syncthreads();
  return t;  // identical in all threads
}

template <int NV>
__device__ __forceinline__ void sum_block_reduce(float (&v)[NV], float* smem /*[NV][kBlock/32]*/) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
#pragma unroll
    for (int k = 0; k < NV; ++k) v[k] += __shfl_xor_sync(0xffffffffu, v[k], off);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k) smem[k * (kBlock / 32) + warp] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kBlock / 32; ++w) s += smem[k * (kBlock / 32) + w];
    v[k] = s;
  }
  __syncthreads();
}

// a - b on math lanes
template <typename M>
__device__ __forceinline__ typename M::E lane_sub(typename M::E a, typename M::E b) {
  return M::fma(b, M::bcast(-1.f), a);
}

// ===========================================================================
// Family R2: [rows, D], D contiguous
//
// grid = (rows, chunks of D).  Phase 1 reads with ordinary cached loads so that,
// when the whole problem is smaller than L2, phase 2 re-reads it from there.
// ===========================================================================

// ws_wf: [rows][nchunks][3] = (mean, m2, n) of each chunk.  A thread reduces
// batches of kUnroll vectors exactly (two passes over registers, fp32x2 lanes)
// and folds each batch into its running triple with one Chan merge.
template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    r2_stats_fwd_kernel(const T* __restrict__ x, int64_t D, int64_t chunk, int nchunks,
                        float* __restrict__ ws_wf) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  __shared__ WF sm[kBlock / 32];
  const int64_t row = blockIdx.x;
  const int64_t step = static_cast<int64_t>(kBlock) * EPV;
  for (int c = blockIdx.y; c < nchunks; c += gridDim.y) {
    const int64_t d0 = static_cast<int64_t>(c) * chunk;
    const int64_t d1 = d0 + chunk < D ? d0 + chunk : D;
    WF acc = {0.f, 0.f, 0.f};
    const T* p = x + row * D + d0 + static_cast<int64_t>(threadIdx.x) * EPV;
    int64_t d = d0 + static_cast<int64_t>(threadIdx.x) * EPV;
    for (; d + (kUnroll - 1) * step < d1; d += kUnroll * step, p += kUnroll * step) {
      Pack<T, EPV> pk[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) pk[u] = load_keep<T, EPV>(p + u * step);
      E v[kUnroll][NE];
      E sum = M::bcast(0.f);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        unpack<T, EPV>(pk[u], v[u]);
#pragma unroll
        for (int e = 0; e < NE; ++e) sum = M::add(sum, v[u][e]);
      }
      WF b;
      b.n = static_cast<float>(kUnroll * EPV);
      b.mean = M::hsum(sum) * (1.0f / (kUnroll * EPV));
      const E bm = M::bcast(b.mean);
      E q = M::bcast(0.f);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          const E dl = lane_sub<M>(v[u][e], bm);
          q = M::fma(dl, dl, q);
        }
      b.m2 = M::hsum(q);
      acc = wf_merge(acc, b);
    }
    for (; d < d1; d += step, p += step) {
      const Pack<T, EPV> pk = load_keep<T, EPV>(p);
      float v[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) v[e] = Cvt<T>::to_f32(pk.v[e]);
      wf_add_batch<EPV>(acc, v);
    }
    const WF t = wf_block_reduce(acc, sm);
    if (threadIdx.x == 0) {
      float* o = ws_wf + (row * nchunks + c) * 3;
      o[0] = t.mean;
      o[1] = t.m2;
      o[2] = t.n;
    }
  }
}

// One warp per row: lane l merges chunks l, l+32, ... in increasing order, then a
// fixed-pairing butterfly merges the 32 lanes.
__global__ void r2_finalize_fwd_kernel(const float* __restrict__ ws_wf, int64_t rows, int nchunks,
                                       float eps, float* __restrict__ mean,
                                       float* __restrict__ ivar) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  WF t = {0.f, 0.f, 0.f};
  for (int c = lane; c < nchunks; c += 32) {
    const float* p = ws_wf + (row * nchunks + c) * 3;
    WF b = {p[0], p[1], p[2]};
    t = wf_merge(t, b);
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    WF o;
    o.mean = __shfl_xor_sync(0xffffffffu, t.mean, off);
    o.m2 = __shfl_xor_sync(0xffffffffu, t.m2, off);
    o.n = __shfl_xor_sync(0xffffffffu, t.n, off);
    const bool low = (lane & off) == 0;
    t = low ? wf_merge(t, o) : wf_merge(o, t);
  }
  if (lane == 0) {
    mean[row] = t.mean;
    ivar[row] = 1.0f / sqrtf(t.m2 / t.n + eps);
  }
}

template <typename T, int EPV, bool ROW_AFFINE>
__global__ void __launch_bounds__(kBlock)
    r2_apply_fwd_kernel(const T* x, const float* __restrict__ gamma,
                        const float* __restrict__ beta, const float* __restrict__ mean,
                        const float* __restrict__ ivar, int64_t D, int64_t C, int64_t chunk,
                        int nchunks, T* y) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  const int64_t row = blockIdx.x;
  const float mu = mean[row], iv = ivar[row];
  float gr = 1.f, br = 0.f;
  if constexpr (ROW_AFFINE) {
    gr = gamma[row % C];
    br = beta[row % C];
  }
  const E nmu = M::bcast(-mu), iv2 = M::bcast(iv), sc2 = M::bcast(iv * gr), br2 = M::bcast(br);
  const int64_t step = static_cast<int64_t>(kBlock) * EPV;
  for (int c = blockIdx.y; c < nchunks; c += gridDim.y) {
    const int64_t d0 = static_cast<int64_t>(c) * chunk;
    const int64_t d1 = d0 + chunk < D ? d0 + chunk : D;
    for (int64_t d = d0 + static_cast<int64_t>(threadIdx.x) * EPV; d < d1; d += kUnroll * step) {
      const T* p = x + row * D + d;
      T* q = y + row * D + d;
      Pack<T, EPV> pk[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (d + u * step < d1) pk[u] = load_stream<T, EPV>(p + u * step, 0);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (d + u * step < d1) {
          E v[NE], o[NE];
          unpack<T, EPV>(pk[u], v);
          if constexpr (ROW_AFFINE) {
#pragma unroll
            for (int e = 0; e < NE; ++e) o[e] = M::fma(M::add(v[e], nmu), sc2, br2);
          } else {
            E g[NE], b[NE];
            load_param_lanes<EPV>(gamma, d + u * step, g);
            load_param_lanes<EPV>(beta, d + u * step, b);
#pragma unroll
            for (int e = 0; e < NE; ++e) o[e] = M::fma(M::mul(M::add(v[e], nmu), iv2), g[e], b[e]);
          }
          store_stream<T, EPV>(q + u * step, 0, repack<T, EPV>(o));
        }
      }
    }
  }
}

// ws_sums: [rows][nchunks][2] = (sum gy, sum gy*xhat) of each chunk
template <typename T, int EPV, bool ROW_AFFINE>
__global__ void __launch_bounds__(kBlock)
    r2_stats_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                        const float* __restrict__ gamma, const float* __restrict__ mean,
                        const float* __restrict__ ivar, int64_t D, int64_t chunk, int nchunks,
                        float* __restrict__ ws_sums) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  __shared__ float sm[2 * (kBlock / 32)];
  const int64_t row = blockIdx.x;
  const E nmu = M::bcast(-mean[row]), iv2 = M::bcast(ivar[row]);
  const int64_t step = static_cast<int64_t>(kBlock) * EPV;
  for (int c = blockIdx.y; c < nchunks; c += gridDim.y) {
    const int64_t d0 = static_cast<int64_t>(c) * chunk;
    const int64_t d1 = d0 + chunk < D ? d0 + chunk : D;
    E a0 = M::bcast(0.f), a1 = M::bcast(0.f);
    for (int64_t d = d0 + static_cast<int64_t>(threadIdx.x) * EPV; d < d1; d += kUnroll * step) {
      const T* px = x + row * D + d;
      const T* pd = dy + row * D + d;
      Pack<T, EPV> kx[kUnroll], kd[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (d + u * step < d1) {
          kx[u] = load_keep<T, EPV>(px + u * step);
          kd[u] = load_keep<T, EPV>(pd + u * step);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (d + u * step < d1) {
          E vx[NE], vd[NE], g[NE];
          unpack<T, EPV>(kx[u], vx);
          unpack<T, EPV>(kd[u], vd);
          if constexpr (!ROW_AFFINE) load_param_lanes<EPV>(gamma, d + u * step, g);
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            const E xh = M::mul(M::add(vx[e], nmu), iv2);
            E gy = vd[e];
            if constexpr (!ROW_AFFINE) gy = M::mul(gy, g[e]);
            a0 = M::add(a0, gy);
            a1 = M::fma(gy, xh, a1);
          }
        }
      }
    }
    float r[2] = {M::hsum(a0), M::hsum(a1)};
    sum_block_reduce<2>(r, sm);
    if (threadIdx.x == 0) {
      float* o = ws_sums + (row * nchunks + c) * 2;
      o[0] = r[0];
      o[1] = r[1];
    }
  }
}

// coef: [rows][2] = (sum gy / D, sum gy*xhat / D).  With ROW_AFFINE the raw sums
// are also written as the per-(n, c) dgamma / dbeta partials, laid out [n][2][C].
// One warp per row, chunks summed lane-strided then by a butterfly (fixed order).
template <bool ROW_AFFINE>
__global__ void r2_finalize_bwd_kernel(const float* __restrict__ ws_sums, int64_t rows,
                                       int nchunks, int64_t D, int64_t C,
                                       float* __restrict__ coef, float* __restrict__ part) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  float r0 = 0.f, r1 = 0.f;
  for (int c = lane; c < nchunks; c += 32) {
    r0 += ws_sums[(row * nchunks + c) * 2 + 0];
    r1 += ws_sums[(row * nchunks + c) * 2 + 1];
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    r0 += __shfl_xor_sync(0xffffffffu, r0, off);
    r1 += __shfl_xor_sync(0xffffffffu, r1, off);
  }
  if (lane == 0) {
    const float inv_D = 1.0f / static_cast<float>(D);
    coef[row * 2 + 0] = r0 * inv_D;
    coef[row * 2 + 1] = r1 * inv_D;
    if constexpr (ROW_AFFINE) {
      const int64_t n = row / C, ch = row - n * C;
      part[(n * 2 + 0) * C + ch] = r1;
      part[(n * 2 + 1) * C + ch] = r0;
    }
  }
}

// InstanceNorm "NC...": dx element-wise, one (row, chunk) per CTA.
template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    r2_apply_bwd_affine_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                               const float* __restrict__ gamma, const float* __restrict__ mean,
                               const float* __restrict__ ivar, const float* __restrict__ coef,
                               int64_t D, int64_t C, int64_t chunk, int nchunks,
                               T* __restrict__ dx) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  const int64_t row = blockIdx.x;
  const float iv = ivar[row];
  const E nmu = M::bcast(-mean[row]), iv2 = M::bcast(iv), sc2 = M::bcast(iv * gamma[row % C]);
  const E nm0 = M::bcast(-coef[row * 2 + 0]), nm1 = M::bcast(-coef[row * 2 + 1]);
  const int64_t step = static_cast<int64_t>(kBlock) * EPV;
  for (int c = blockIdx.y; c < nchunks; c += gridDim.y) {
    const int64_t d0 = static_cast<int64_t>(c) * chunk;
    const int64_t d1 = d0 + chunk < D ? d0 + chunk : D;
    for (int64_t d = d0 + static_cast<int64_t>(threadIdx.x) * EPV; d < d1; d += kUnroll * step) {
      const T* px = x + row * D + d;
      const T* pd = dy + row * D + d;
      T* po = dx + row * D + d;
      Pack<T, EPV> kx[kUnroll], kd[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (d + u * step < d1) {
          kx[u] = load_stream<T, EPV>(px + u * step, 0);
          kd[u] = load_stream<T, EPV>(pd + u * step, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (d + u * step < d1) {
          E vx[NE], vd[NE], o[NE];
          unpack<T, EPV>(kx[u], vx);
          unpack<T, EPV>(kd[u], vd);
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            const E xh = M::mul(M::add(vx[e], nmu), iv2);
            o[e] = M::mul(M::add(vd[e], M::fma(xh, nm1, nm0)), sc2);
          }
          store_stream<T, EPV>(po + u * step, 0, repack<T, EPV>(o));
        }
      }
    }
  }
}

// LayerNorm: a thread owns EPV columns and walks the rows of its slice, so the
// dgamma / dbeta contributions accumulate in registers.  grid = (column blocks,
// row slices); one partial row [2][D] per slice.  The four per-row scalars are
// staged through shared memory, kRowTile rows at a time.
constexpr int kRowTile = 128;

template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    r2_apply_bwd_ln_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                           const float* __restrict__ gamma, const float* __restrict__ mean,
                           const float* __restrict__ ivar, const float* __restrict__ coef,
                           int64_t N, int64_t D, int64_t rows_per_slice, T* __restrict__ dx,
                           float* __restrict__ part) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  __shared__ float4 rowc[kRowTile];  // (-mean, ivar, -m0, -m1)
  const int64_t col = (static_cast<int64_t>(blockIdx.x) * kBlock + threadIdx.x) * EPV;
  const bool live = col < D;
  const int64_t slice = blockIdx.y;
  const int64_t r0 = slice * rows_per_slice;
  const int64_t r1 = r0 + rows_per_slice < N ? r0 + rows_per_slice : N;
  E g[NE], dg[NE], db[NE];
  if (live) load_param_lanes<EPV>(gamma, col, g);
#pragma unroll
  for (int e = 0; e < NE; ++e) dg[e] = db[e] = M::bcast(0.f);
  for (int64_t base = r0; base < r1; base += kRowTile) {
    const int tile = static_cast<int>(r1 - base < kRowTile ? r1 - base : kRowTile);
    __syncthreads();
    if (threadIdx.x < tile) {
      const int64_t row = base + threadIdx.x;
      rowc[threadIdx.x] = make_float4(-mean[row], ivar[row], -coef[row * 2], -coef[row * 2 + 1]);
    }
    __syncthreads();
    if (live) {
      const T* px = x + base * D + col;
      const T* pd = dy + base * D + col;
      T* po = dx + base * D + col;
      for (int i = 0; i < tile; i += 2) {
        Pack<T, EPV> kx[2], kd[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (i + u < tile) {
            kx[u] = load_stream<T, EPV>(px + (i + u) * D, 0);
            kd[u] = load_stream<T, EPV>(pd + (i + u) * D, 0);
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (i + u < tile) {
            const float4 rc = rowc[i + u];
            const E nmu = M::bcast(rc.x), iv2 = M::bcast(rc.y);
            const E nm0 = M::bcast(rc.z), nm1 = M::bcast(rc.w);
            E vx[NE], vd[NE], o[NE];
            unpack<T, EPV>(kx[u], vx);
            unpack<T, EPV>(kd[u], vd);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              const E xh = M::mul(M::add(vx[e], nmu), iv2);
              dg[e] = M::fma(vd[e], xh, dg[e]);
              db[e] = M::add(db[e], vd[e]);
              o[e] = M::mul(M::add(M::mul(vd[e], g[e]), M::fma(xh, nm1, nm0)), iv2);
            }
            store_stream<T, EPV>(po + (i + u) * D, 0, repack<T, EPV>(o));
          }
        }
      }
    }
  }
  if (live) {
    store_param_lanes<EPV>(part + (slice * 2 + 0) * D, col, dg);
    store_param_lanes<EPV>(part + (slice * 2 + 1) * D, col, db);
  }
}

// ===========================================================================
// Family S2: x[n, d, c], C contiguous, reduce over d
//
// CTA = 256 threads arranged as (cvt channel-vectors) x (ty voxel lanes).
// grid = (d-chunks, channel tiles, N).
// ===========================================================================
struct S2Geom {
  int64_t N, D, C;
  int64_t chunk;  // voxels per d-chunk
  int nchunks;
  int cvt;    // channel vectors per tile (<= 256)
  int lanes;  // voxel lanes per CTA = 256 / cvt
  int64_t n0;   // first batch item of this launch (grid.z counts items from here)
  int reverse;  // phase 2: visit items and chunks last-to-first, so that what phase 1
                // read most recently (and is most likely still in L2) is re-read first
};

__device__ __forceinline__ int64_t s2_item(const S2Geom& gm) {
  return gm.n0 + (gm.reverse ? (gridDim.z - 1 - blockIdx.z) : blockIdx.z);
}
__device__ __forceinline__ int s2_chunk(const S2Geom& gm) {
  return gm.reverse ? (gm.nchunks - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
}

// Per-thread geometry of the S2 kernels: which channel vector and which voxels
// (d0 + ty, d0 + ty + lanes, ...) of the chunk this thread owns.
struct S2Thread {
  int tx, ty;
  int64_t cv;      // channel-vector index
  bool active;
  int64_t count;   // voxels of this thread inside the chunk
  int64_t first;   // element offset of its first vector
  int64_t step;    // element distance between its consecutive voxels
};

template <int EPV>
__device__ __forceinline__ S2Thread s2_thread(const S2Geom& gm) {
  S2Thread t;
  t.tx = threadIdx.x % gm.cvt;
  t.ty = threadIdx.x / gm.cvt;
  t.cv = static_cast<int64_t>(blockIdx.y) * gm.cvt + t.tx;
  const int64_t n = s2_item(gm);
  const int64_t d0 = static_cast<int64_t>(s2_chunk(gm)) * gm.chunk;
  const int64_t d1 = d0 + gm.chunk < gm.D ? d0 + gm.chunk : gm.D;
  t.active = t.ty < gm.lanes && t.cv * EPV < gm.C && d0 + t.ty < d1;
  t.count = t.active ? (d1 - d0 - t.ty + gm.lanes - 1) / gm.lanes : 0;
  t.first = ((n * gm.D) + d0 + t.ty) * gm.C + t.cv * EPV;
  t.step = static_cast<int64_t>(gm.lanes) * gm.C;
  return t;
}

// ws layout for phase-1 partials: [n][chunk][k][C], k = 0..K-1
//
// Forward statistics.  Every thread walks its voxels in batches of kUnroll: the
// batch is reduced exactly (mean, then centred squares, on fp32x2 lanes) and
// folded into the running (mean, M2, n) with Chan's update, whose two weights are
// shared by all channels of the thread.  Leftover voxels use the per-element
// Welford update.
template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    s2_stats_fwd_kernel(const T* __restrict__ x, const S2Geom gm, float* __restrict__ ws) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  extern __shared__ float dyn[];  // [lanes][cvt*EPV] x (mean, m2) ; counts [lanes][cvt]
  const S2Thread th = s2_thread<EPV>(gm);
  const int tx = th.tx, ty = th.ty;
  const int64_t n = s2_item(gm);
  const int chunk_id = s2_chunk(gm);

  E mean[NE], m2[NE];
#pragma unroll
  for (int e = 0; e < NE; ++e) mean[e] = m2[e] = M::bcast(0.f);
  float cnt = 0.f;
  if (th.active) {
    const T* p = x + th.first;
    int64_t i = 0;
    for (; i + kUnroll <= th.count; i += kUnroll) {
      Pack<T, EPV> pk[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) pk[u] = load_keep<T, EPV>(p + u * th.step);
      p += kUnroll * th.step;
      E v[kUnroll][NE];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) unpack<T, EPV>(pk[u], v[u]);
      const float nn = cnt + static_cast<float>(kUnroll);
      const float w1 = __fdividef(static_cast<float>(kUnroll), nn);
      const E w1v = M::bcast(w1), w2v = M::bcast(cnt * w1);
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        E sum = v[0][e];
#pragma unroll
        for (int u = 1; u < kUnroll; ++u) sum = M::add(sum, v[u][e]);
        const E bm = M::mul(sum, M::bcast(1.0f / kUnroll));
        E bq = M::bcast(0.f);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const E d = lane_sub<M>(v[u][e], bm);
          bq = M::fma(d, d, bq);
        }
        const E delta = lane_sub<M>(bm, mean[e]);
        mean[e] = M::fma(delta, w1v, mean[e]);
        m2[e] = M::fma(M::mul(delta, delta), w2v, M::add(m2[e], bq));
      }
      cnt = nn;
    }
    for (; i < th.count; ++i) {
      const Pack<T, EPV> pk = load_keep<T, EPV>(p);
      p += th.step;
      E v[NE];
      unpack<T, EPV>(pk, v);
      cnt += 1.f;
      const E inv = M::bcast(1.0f / cnt);
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const E dl = lane_sub<M>(v[e], mean[e]);
        mean[e] = M::fma(dl, inv, mean[e]);
        m2[e] = M::fma(dl, lane_sub<M>(v[e], mean[e]), m2[e]);
      }
    }
  }
  // tree merge over the voxel lanes (fixed pairing => deterministic)
  const int width = gm.cvt * EPV;
  float* s_mean = dyn;
  float* s_m2 = dyn + gm.lanes * width;
  float* s_cnt = dyn + 2 * gm.lanes * width;  // [lanes][cvt]
  if (ty < gm.lanes) {
    float fm[EPV], fq[EPV];
    if constexpr (EPV == 1) {
      fm[0] = mean[0];
      fq[0] = m2[0];
    } else {
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        fm[2 * e] = mean[e].x;
        fm[2 * e + 1] = mean[e].y;
        fq[2 * e] = m2[e].x;
        fq[2 * e + 1] = m2[e].y;
      }
    }
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
      s_mean[ty * width + tx * EPV + e] = fm[e];
      s_m2[ty * width + tx * EPV + e] = fq[e];
    }
    s_cnt[ty * gm.cvt + tx] = cnt;
  }
  __syncthreads();
  int span = 1;
  while (span < gm.lanes) span <<= 1;
  for (int sft = span >> 1; sft > 0; sft >>= 1) {
    if (ty < sft && ty + sft < gm.lanes) {
      const float na = s_cnt[ty * gm.cvt + tx], nb = s_cnt[(ty + sft) * gm.cvt + tx];
#pragma unroll
      for (int e = 0; e < EPV; ++e) {
        const int ia = ty * width + tx * EPV + e, ib = (ty + sft) * width + tx * EPV + e;
        WF a = {s_mean[ia], s_m2[ia], na};
        WF b = {s_mean[ib], s_m2[ib], nb};
        const WF r = wf_merge(a, b);
        s_mean[ia] = r.mean;
        s_m2[ia] = r.m2;
      }
      s_cnt[ty * gm.cvt + tx] = na + nb;
    }
    __syncthreads();
  }
  if (ty == 0 && th.cv * EPV < gm.C) {
    float* o = ws + ((n * gm.nchunks + chunk_id) * 3) * gm.C + th.cv * EPV;
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
      o[e] = s_mean[tx * EPV + e];
      o[gm.C + e] = s_m2[tx * EPV + e];
      o[2 * gm.C + e] = s_cnt[tx];
    }
  }
}

// One warp per (n, c): lane l merges chunks l, l+32, ... in increasing order, then
// the 32 lane results are merged by a butterfly whose pairing is fixed.
__global__ void s2_finalize_fwd_kernel(const float* __restrict__ ws, int64_t n0, int64_t items,
                                       int64_t C, int nchunks, float eps,
                                       float* __restrict__ mean, float* __restrict__ ivar) {
  const int lane = threadIdx.x & 31;
  const int64_t local = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (local >= items * C) return;  // whole warps leave together
  const int64_t i = n0 * C + local;
  const int64_t n = i / C, c = i - n * C;
  WF t = {0.f, 0.f, 0.f};
  for (int k = lane; k < nchunks; k += 32) {
    const float* p = ws + ((n * nchunks + k) * 3) * C + c;
    WF b = {p[0], p[C], p[2 * C]};
    t = wf_merge(t, b);
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    WF o;
    o.mean = __shfl_xor_sync(0xffffffffu, t.mean, off);
    o.m2 = __shfl_xor_sync(0xffffffffu, t.m2, off);
    o.n = __shfl_xor_sync(0xffffffffu, t.n, off);
    const bool low = (lane & off) == 0;
    t = low ? wf_merge(t, o) : wf_merge(o, t);
  }
  if (lane == 0) {
    mean[i] = t.mean;
    ivar[i] = 1.0f / sqrtf(t.m2 / t.n + eps);
  }
}

template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    s2_apply_fwd_kernel(const T* x, const float* __restrict__ gamma,
                        const float* __restrict__ beta, const float* __restrict__ mean,
                        const float* __restrict__ ivar, const S2Geom gm, T* y) {
  const int tx = threadIdx.x % gm.cvt;
  const int ty = threadIdx.x / gm.cvt;
  const int64_t n = s2_item(gm);
  const int64_t cv = static_cast<int64_t>(blockIdx.y) * gm.cvt + tx;
  if (!(ty < gm.lanes && cv * EPV < gm.C)) return;
  const int64_t d0 = static_cast<int64_t>(s2_chunk(gm)) * gm.chunk;
  const int64_t d1 = d0 + gm.chunk < gm.D ? d0 + gm.chunk : gm.D;
  float mu[EPV], sc[EPV], sh[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) {
    const int64_t c = cv * EPV + e;
    mu[e] = mean[n * gm.C + c];
    sc[e] = ivar[n * gm.C + c] * gamma[c];
    sh[e] = beta[c];
  }
  const T* xb = x + (n * gm.D) * gm.C + cv * EPV;
  T* yb = y + (n * gm.D) * gm.C + cv * EPV;
  for (int64_t d = d0 + ty; d < d1; d += static_cast<int64_t>(kUnroll) * gm.lanes) {
    Pack<T, EPV> p[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (d + static_cast<int64_t>(u) * gm.lanes < d1)
        p[u] = load_stream<T, EPV>(xb, (d + static_cast<int64_t>(u) * gm.lanes) * gm.C);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t dd = d + static_cast<int64_t>(u) * gm.lanes;
      if (dd < d1) {
        Pack<T, EPV> o;
#pragma unroll
        for (int e = 0; e < EPV; ++e)
          o.v[e] = Cvt<T>::from_f32(fmaf(Cvt<T>::to_f32(p[u].v[e]) - mu[e], sc[e], sh[e]));
        store_stream<T, EPV>(yb, dd * gm.C, o);
      }
    }
  }
}

// phase-1 partials backward: [n][chunk][2][C] = (sum dy, sum dy*(x-mean))
template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    s2_stats_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                        const float* __restrict__ mean, const S2Geom gm,
                        float* __restrict__ ws) {
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  extern __shared__ float dyn[];  // [2][lanes][cvt*EPV]
  const S2Thread th = s2_thread<EPV>(gm);
  const int tx = th.tx, ty = th.ty;
  const int64_t n = s2_item(gm);
  const int chunk_id = s2_chunk(gm);
  E s0[NE], s1[NE];
#pragma unroll
  for (int e = 0; e < NE; ++e) s0[e] = s1[e] = M::bcast(0.f);
  if (th.active) {
    E nmu[NE];
    {
      float t[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) t[e] = -mean[n * gm.C + th.cv * EPV + e];
      if constexpr (EPV == 1) {
        nmu[0] = t[0];
      } else {
#pragma unroll
        for (int e = 0; e < NE; ++e) nmu[e] = make_float2(t[2 * e], t[2 * e + 1]);
      }
    }
    const T* px = x + th.first;
    const T* pd = dy + th.first;
    for (int64_t i = 0; i < th.count; i += kUnroll) {
      Pack<T, EPV> kx[kUnroll], kd[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (i + u < th.count) {
          kx[u] = load_keep<T, EPV>(px + u * th.step);
          kd[u] = load_keep<T, EPV>(pd + u * th.step);
        }
      }
      px += kUnroll * th.step;
      pd += kUnroll * th.step;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (i + u < th.count) {
          E vx[NE], vd[NE];
          unpack<T, EPV>(kx[u], vx);
          unpack<T, EPV>(kd[u], vd);
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            s0[e] = M::add(s0[e], vd[e]);
            s1[e] = M::fma(vd[e], M::add(vx[e], nmu[e]), s1[e]);
          }
        }
      }
    }
  }
  const int width = gm.cvt * EPV;
  float* a0 = dyn;
  float* a1 = dyn + gm.lanes * width;
  if (ty < gm.lanes) {
    float f0[EPV], f1[EPV];
    if constexpr (EPV == 1) {
      f0[0] = s0[0];
      f1[0] = s1[0];
    } else {
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        f0[2 * e] = s0[e].x;
        f0[2 * e + 1] = s0[e].y;
        f1[2 * e] = s1[e].x;
        f1[2 * e + 1] = s1[e].y;
      }
    }
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
      a0[ty * width + tx * EPV + e] = f0[e];
      a1[ty * width + tx * EPV + e] = f1[e];
    }
  }
  __syncthreads();
  int span = 1;
  while (span < gm.lanes) span <<= 1;
  for (int sft = span >> 1; sft > 0; sft >>= 1) {
    if (ty < sft && ty + sft < gm.lanes) {
#pragma unroll
      for (int e = 0; e < EPV; ++e) {
        const int ia = ty * width + tx * EPV + e, ib = (ty + sft) * width + tx * EPV + e;
        a0[ia] += a0[ib];
        a1[ia] += a1[ib];
      }
    }
    __syncthreads();
  }
  if (ty == 0 && th.cv * EPV < gm.C) {
    float* o = ws + ((n * gm.nchunks + chunk_id) * 2) * gm.C + th.cv * EPV;
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
      o[e] = a0[tx * EPV + e];
      o[gm.C + e] = a1[tx * EPV + e];
    }
  }
}

// coef: [n][3][C] = (gamma*ivar, sum dy / D, ivar * sum dy*xhat / D);
// part: [n][2][C] = (dgamma_nc, dbeta_nc)
__global__ void s2_finalize_bwd_kernel(const float* __restrict__ ws,
                                       const float* __restrict__ gamma,
                                       const float* __restrict__ ivar, int64_t n0,
                                       int64_t items, int64_t C, int64_t D, int nchunks,
                                       float* __restrict__ coef, float* __restrict__ part) {
  const int lane = threadIdx.x & 31;
  const int64_t local = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (local >= items * C) return;  // whole warps leave together
  const int64_t i = n0 * C + local;
  const int64_t n = i / C, c = i - n * C;
  float r0 = 0.f, r1 = 0.f;
  for (int k = lane; k < nchunks; k += 32) {
    const float* p = ws + ((n * nchunks + k) * 2) * C + c;
    r0 += p[0];
    r1 += p[C];
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    r0 += __shfl_xor_sync(0xffffffffu, r0, off);
    r1 += __shfl_xor_sync(0xffffffffu, r1, off);
  }
  if (lane == 0) {
    const float iv = ivar[i];
    const float inv_D = 1.0f / static_cast<float>(D);
    const float dgam = r1 * iv;  // sum dy * xhat
    coef[(n * 3 + 0) * C + c] = gamma[c] * iv;
    coef[(n * 3 + 1) * C + c] = r0 * inv_D;
    coef[(n * 3 + 2) * C + c] = dgam * inv_D * iv;  // multiplies (x - mean)
    part[(n * 2 + 0) * C + c] = dgam;
    part[(n * 2 + 1) * C + c] = r0;
  }
}

template <typename T, int EPV>
__global__ void __launch_bounds__(kBlock)
    s2_apply_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                        const float* __restrict__ mean, const float* __restrict__ coef,
                        const S2Geom gm, T* __restrict__ dx) {
  const int tx = threadIdx.x % gm.cvt;
  const int ty = threadIdx.x / gm.cvt;
  const int64_t n = s2_item(gm);
  const int64_t cv = static_cast<int64_t>(blockIdx.y) * gm.cvt + tx;
  if (!(ty < gm.lanes && cv * EPV < gm.C)) return;
  const int64_t d0 = static_cast<int64_t>(s2_chunk(gm)) * gm.chunk;
  const int64_t d1 = d0 + gm.chunk < gm.D ? d0 + gm.chunk : gm.D;
  float mu[EPV], sc[EPV], m0[EPV], m1[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) {
    const int64_t c = cv * EPV + e;
    mu[e] = mean[n * gm.C + c];
    sc[e] = coef[(n * 3 + 0) * gm.C + c];
    m0[e] = coef[(n * 3 + 1) * gm.C + c];
    m1[e] = coef[(n * 3 + 2) * gm.C + c];
  }
  const T* xb = x + (n * gm.D) * gm.C + cv * EPV;
  const T* db = dy + (n * gm.D) * gm.C + cv * EPV;
  T* ob = dx + (n * gm.D) * gm.C + cv * EPV;
  for (int64_t d = d0 + ty; d < d1; d += static_cast<int64_t>(kUnroll) * gm.lanes) {
    Pack<T, EPV> px[kUnroll], pd[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t dd = d + static_cast<int64_t>(u) * gm.lanes;
      if (dd < d1) {
        px[u] = load_stream<T, EPV>(xb, dd * gm.C);
        pd[u] = load_stream<T, EPV>(db, dd * gm.C);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t dd = d + static_cast<int64_t>(u) * gm.lanes;
      if (dd < d1) {
        Pack<T, EPV> o;
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
          const float xc = Cvt<T>::to_f32(px[u].v[e]) - mu[e];
          const float dv = Cvt<T>::to_f32(pd[u].v[e]);
          // dx = gamma*ivar * (dy - mean(dy) - xhat * mean(dy*xhat))
          o.v[e] = Cvt<T>::from_f32(sc[e] * (dv - fmaf(xc, m1[e], m0[e])));
        }
        store_stream<T, EPV>(ob, dd * gm.C, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

#define NVN_CHECK(expr)                 \
  do {                                  \
    cudaError_t e_ = (expr);            \
    if (e_ != cudaSuccess) return e_;   \
  } while (0)

#define NVN_LAUNCHED()                       \
  do {                                       \
    count_launch();                          \
    cudaError_t e_ = cudaGetLastError();     \
    if (e_ != cudaSuccess) return e_;        \
  } while (0)

}  // namespace

// ---- R2 planning -----------------------------------------------------------
R2Plan r2_plan(int64_t rows, int64_t D, int epv, bool ln_bwd) {
  R2Plan p = {};
  const int sms = device_sm_count();
  // One chunk is a whole number of CTA sweeps (kBlock*epv*kUnroll elements) and
  // there are enough (row, chunk) CTAs for ~8 per SM.
  const int64_t sweep = static_cast<int64_t>(kBlock) * epv * kUnroll;
  int64_t want = ceil_div(static_cast<int64_t>(sms) * 8, rows);
  if (want < 1) want = 1;
  int64_t chunk = round_up(ceil_div(D, want), sweep);
  if (chunk < sweep) chunk = sweep;
  p.chunk = chunk;
  p.nchunks = static_cast<int>(ceil_div(D, chunk));
  p.grid_y = p.nchunks < 65535 ? p.nchunks : 65535;
  if (ln_bwd) {
    const int64_t colblocks = ceil_div(D, static_cast<int64_t>(kBlock) * epv);
    int64_t slices = ceil_div(static_cast<int64_t>(sms) * 2, colblocks);
    if (slices > rows) slices = rows;
    if (slices > 65535) slices = 65535;
    if (slices < 1) slices = 1;
    p.rows_per_slice = ceil_div(rows, slices);
    p.slices = static_cast<int>(ceil_div(rows, p.rows_per_slice));
  }
  return p;
}

template <typename T, int EPV>
static cudaError_t r2_fwd_t(const R2Args& a, const R2Plan& p, cudaStream_t s) {
  const dim3 grid(static_cast<unsigned>(a.rows), static_cast<unsigned>(p.grid_y));
  r2_stats_fwd_kernel<T, EPV><<<grid, kBlock, 0, s>>>(static_cast<const T*>(a.x), a.D, p.chunk,
                                                      p.nchunks, a.ws_part);
  NVN_LAUNCHED();
  r2_finalize_fwd_kernel<<<static_cast<unsigned>(ceil_div(a.rows, 4)), 128, 0, s>>>(
      a.ws_part, a.rows, p.nchunks, a.eps, a.mean, a.ivar);
  NVN_LAUNCHED();
  if (a.row_affine) {
    r2_apply_fwd_kernel<T, EPV, true><<<grid, kBlock, 0, s>>>(
        static_cast<const T*>(a.x), a.gamma, a.beta, a.mean, a.ivar, a.D, a.C, p.chunk,
        p.nchunks, static_cast<T*>(a.out));
  } else {
    r2_apply_fwd_kernel<T, EPV, false><<<grid, kBlock, 0, s>>>(
        static_cast<const T*>(a.x), a.gamma, a.beta, a.mean, a.ivar, a.D, a.C, p.chunk,
        p.nchunks, static_cast<T*>(a.out));
  }
  NVN_LAUNCHED();
  return cudaSuccess;
}

template <typename T, int EPV>
static cudaError_t r2_bwd_t(const R2Args& a, const R2Plan& p, cudaStream_t s) {
  const dim3 grid(static_cast<unsigned>(a.rows), static_cast<unsigned>(p.grid_y));
  const T* x = static_cast<const T*>(a.x);
  const T* dy = static_cast<const T*>(a.dy);
  T* dx = static_cast<T*>(a.out);
  if (a.row_affine) {
    r2_stats_bwd_kernel<T, EPV, true><<<grid, kBlock, 0, s>>>(dy, x, a.gamma, a.mean, a.ivar,
                                                              a.D, p.chunk, p.nchunks, a.ws_part);
    NVN_LAUNCHED();
    r2_finalize_bwd_kernel<true><<<static_cast<unsigned>(ceil_div(a.rows, 4)), 128, 0, s>>>(
        a.ws_part, a.rows, p.nchunks, a.D, a.C, a.ws_coef, a.ws_colpart);
    NVN_LAUNCHED();
    r2_apply_bwd_affine_kernel<T, EPV><<<grid, kBlock, 0, s>>>(
        dy, x, a.gamma, a.mean, a.ivar, a.ws_coef, a.D, a.C, p.chunk, p.nchunks, dx);
    NVN_LAUNCHED();
  } else {
    r2_stats_bwd_kernel<T, EPV, false><<<grid, kBlock, 0, s>>>(
        dy, x, a.gamma, a.mean, a.ivar, a.D, p.chunk, p.nchunks, a.ws_part);
    NVN_LAUNCHED();
    r2_finalize_bwd_kernel<false><<<static_cast<unsigned>(ceil_div(a.rows, 4)), 128, 0, s>>>(
        a.ws_part, a.rows, p.nchunks, a.D, a.C, a.ws_coef, nullptr);
    NVN_LAUNCHED();
    const dim3 g2(static_cast<unsigned>(ceil_div(a.D, static_cast<int64_t>(kBlock) * EPV)),
                  static_cast<unsigned>(p.slices));
    r2_apply_bwd_ln_kernel<T, EPV><<<g2, kBlock, 0, s>>>(dy, x, a.gamma, a.mean, a.ivar,
                                                         a.ws_coef, a.rows, a.D,
                                                         p.rows_per_slice, dx, a.ws_colpart);
    NVN_LAUNCHED();
  }
  return cudaSuccess;
}

template <typename T>
static cudaError_t r2_dispatch(bool bwd, bool scalar, const R2Args& a, const R2Plan& p,
                               cudaStream_t s) {
  constexpr int V = VecTraits<T>::kFull;
  if (bwd) return scalar ? r2_bwd_t<T, 1>(a, p, s) : r2_bwd_t<T, V>(a, p, s);
  return scalar ? r2_fwd_t<T, 1>(a, p, s) : r2_fwd_t<T, V>(a, p, s);
}

cudaError_t r2_launch(int dtype, bool bwd, bool scalar, const R2Args& a, const R2Plan& p,
                      cudaStream_t s) {
  switch (dtype) {
    case 0:
      return r2_dispatch<float>(bwd, scalar, a, p, s);
    case 1:
      return r2_dispatch<__half>(bwd, scalar, a, p, s);
    default:
      return r2_dispatch<__nv_bfloat16>(bwd, scalar, a, p, s);
  }
}

// ---- S2 planning -----------------------------------------------------------
S2Plan s2_plan(int dtype, bool bwd, int64_t N, int64_t C, int64_t D, int epv) {
  S2Plan p = {};
  const int sms = device_sm_count();
  const int64_t CV = C / epv;
  p.cvt = static_cast<int>(CV < kBlock ? CV : kBlock);
  p.lanes = kBlock / p.cvt;
  p.ctiles = static_cast<int>(ceil_div(CV, p.cvt));
  // All items go into one launch group.  (Splitting the batch into L2-sized groups so that
  // phase 2 re-reads a group straight from L2 was measured on B200 with 134 MB items and lost
  // more to small launches than it gained; the launch code still supports groups.)  Phase 2
  // walks items and chunks in reverse, which keeps the tail of phase 1 an L2 hit.
  (void)dtype;
  (void)bwd;
  const int64_t group = N < 65535 ? N : 65535;  // grid.z counts the items of a group
  p.group = static_cast<int>(group);
  // voxels one CTA sweep covers
  const int64_t sweep = static_cast<int64_t>(p.lanes) * kUnroll;
  int64_t want = ceil_div(static_cast<int64_t>(sms) * 8, group * p.ctiles);
  if (want < 1) want = 1;
  int64_t chunk = round_up(ceil_div(D, want), sweep);
  // keep at least 8 sweeps per chunk so the per-chunk merge stays negligible
  if (chunk < 8 * sweep) chunk = 8 * sweep;
  p.chunk = chunk;
  p.nchunks = static_cast<int>(ceil_div(D, chunk));
  p.smem_fwd = static_cast<size_t>(p.lanes) * p.cvt * (2 * epv + 1) * sizeof(float);
  p.smem_bwd = static_cast<size_t>(p.lanes) * p.cvt * (2 * epv) * sizeof(float);
  return p;
}

template <typename T, int EPV>
static cudaError_t s2_t(bool bwd, const S2Args& a, const S2Plan& p, cudaStream_t s) {
  S2Geom gm;
  gm.N = a.N;
  gm.D = a.D;
  gm.C = a.C;
  gm.chunk = p.chunk;
  gm.nchunks = p.nchunks;
  gm.cvt = p.cvt;
  gm.lanes = p.lanes;
  const T* x = static_cast<const T*>(a.x);
  const T* dy = static_cast<const T*>(a.dy);
  for (int64_t n0 = 0; n0 < a.N; n0 += p.group) {
    const int64_t items = n0 + p.group <= a.N ? p.group : a.N - n0;
    const dim3 grid(static_cast<unsigned>(p.nchunks), static_cast<unsigned>(p.ctiles),
                    static_cast<unsigned>(items));
    // finalize kernels use one warp per (n, c): 4 per 128-thread block
    const unsigned fin_blocks = static_cast<unsigned>(ceil_div(items * a.C, 4));
    gm.n0 = n0;
    gm.reverse = 0;
    S2Geom back = gm;
    back.reverse = 1;
    if (!bwd) {
      s2_stats_fwd_kernel<T, EPV><<<grid, kBlock, p.smem_fwd, s>>>(x, gm, a.ws_part);
      NVN_LAUNCHED();
      s2_finalize_fwd_kernel<<<fin_blocks, 128, 0, s>>>(a.ws_part, n0, items, a.C, p.nchunks,
                                                        a.eps, a.mean, a.ivar);
      NVN_LAUNCHED();
      s2_apply_fwd_kernel<T, EPV><<<grid, kBlock, 0, s>>>(x, a.gamma, a.beta, a.mean, a.ivar,
                                                          back, static_cast<T*>(a.out));
      NVN_LAUNCHED();
    } else {
      s2_stats_bwd_kernel<T, EPV><<<grid, kBlock, p.smem_bwd, s>>>(dy, x, a.mean, gm, a.ws_part);
      NVN_LAUNCHED();
      s2_finalize_bwd_kernel<<<fin_blocks, 128, 0, s>>>(a.ws_part, a.gamma, a.ivar, n0, items,
                                                        a.C, a.D, p.nchunks, a.ws_coef,
                                                        a.ws_colpart);
      NVN_LAUNCHED();
      s2_apply_bwd_kernel<T, EPV><<<grid, kBlock, 0, s>>>(dy, x, a.mean, a.ws_coef, back,
                                                          static_cast<T*>(a.out));
      NVN_LAUNCHED();
    }
  }
  return cudaSuccess;
}

cudaError_t s2_launch(int dtype, bool bwd, bool scalar, const S2Args& a, const S2Plan& p,
                      cudaStream_t s) {
  switch (dtype) {
    case 0:
      return scalar ? s2_t<float, 1>(bwd, a, p, s) : s2_t<float, 4>(bwd, a, p, s);
    case 1:
      return scalar ? s2_t<__half, 1>(bwd, a, p, s) : s2_t<__half, 8>(bwd, a, p, s);
    default:
      return scalar ? s2_t<__nv_bfloat16, 1>(bwd, a, p, s)
                    : s2_t<__nv_bfloat16, 8>(bwd, a, p, s);
  }
}

}  // namespace nvn
