// Column-sliced LayerNorm kernels for wide rows.
//
// The row kernels give a row to one CTA or one thread-block cluster.  For rows of tens of
// thousands of elements that leaves few rows in flight and one cluster barrier per row, and
// gamma / beta no longer fit the registers of the threads that own a row.  Here the work is
// cut the other way: CTA b owns the columns [b*S, (b+1)*S) of EVERY row (S = LPR lanes x 4
// 128-bit vectors), so
//   * gamma / beta (and the dgamma / dbeta accumulators) of a lane's columns stay in
//     registers for the whole kernel, and the backward kernel writes the final dgamma /
//     dbeta itself - there is no second reduction stage;
//   * LPR = 8, 16 or 32 lanes share a row slice, a warp works on 32 / LPR rows at once, and
//     all reductions are shuffle butterflies inside the lane group;
//   * row groups are staged in a two-stage shared-memory ring by cp.async (16 bytes per
//     lane, every lane reads back only what it copied itself, so the ring needs no
//     barrier); both passes over a group read it from there, which keeps the register
//     budget for gamma / beta and the accumulators;
//   * the per-row statistics meet in global memory: every warp writes the partial sums of
//     its (row, slice), all CTAs pass a grid barrier, every warp adds the G partials of its
//     rows in a fixed order.  Rows are processed in groups (W warps x RPW x 32 / LPR rows)
//     with one grid barrier per group, and the copies of the next group are issued before
//     waiting.
//
// The grid barrier is a monotonic arrival counter in the workspace (zeroed by a memset node
// ahead of the launch).  The kernel is launched cooperatively, which guarantees that all
// CTAs are resident; the wait is bounded all the same and raises the device status word
// instead of hanging.  x (and dy) are read from HBM exactly once; the partials are 8 bytes
// per (row, slice) and stay in L2.
//
// Replaces, for wide rows, LayerNormRowReduceInToTemp* / TempToOut* / *Update
// (atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:523-719) and LayerNormGradBetaGamma*
// (:741-803).
#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

namespace {

constexpr unsigned kGridSpinLimit = 1u << 21;
constexpr int kMaxGrid = 160;  // most column slices (CTAs); a multiple of 32

// 16-byte asynchronous copy global -> shared; `bytes` = 16, or 0 to write zeros instead.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, unsigned bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Grid barrier, arrival half: one arrival per CTA.  The CTA barrier makes every warp's
// partial stores visible to thread 0, whose fence then orders them before the arrival.
__device__ __forceinline__ void grid_arrive(unsigned* counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
  }
}

// Waiting half: thread 0 polls (one poller per CTA keeps the counter's cache line free for
// the arrivals) until `target` CTAs have arrived, bounded; false when it gave up.
__device__ __forceinline__ bool grid_wait(const unsigned* counter, unsigned target, int* flag) {
  if (threadIdx.x == 0) {
    int ok = 0;
    for (unsigned i = 0; i < kGridSpinLimit; ++i) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) {
        ok = 1;
        break;
      }
      __nanosleep(64);
    }
    *flag = ok;
  }
  __syncthreads();
  return *flag != 0;
}

struct ColsliceArgs {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  const float* mean_in;
  const float* ivar_in;
  void* out;        // y or dx
  float* mean;      // forward outputs
  float* ivar;
  float* dgamma;    // backward outputs (final values)
  float* dbeta;
  float2* partials;  // [N][G]
  unsigned* counter;
  int64_t N, D;
  float eps;
  int* status;
};

// Shape of the work inside a CTA
//   LPR  lanes that share one row slice (8, 16 or 32): a warp works on 32 / LPR rows at once,
//        so the shuffle butterflies (log2 LPR levels) and the merge of the partials are
//        paid once per 32 / LPR rows;
//   kVPL vectors per lane and row: the slice is LPR * kVPL vectors wide;
//   W    warps per CTA;  RPW  row sets (of 32 / LPR rows) per warp and group.
constexpr int kVPL = 4;

template <int LPR>
__device__ __forceinline__ float lane_group_sum(float v) {
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// Elements of a row inside slice j (slices are `slice_elems` wide; the last one may be short).
__device__ __forceinline__ float slice_count(int j, int last_slice, float slice_elems,
                                             float tail_elems) {
  return j < last_slice ? slice_elems : (j == last_slice ? tail_elems : 0.f);
}

template <typename T, int LPR, int W, int RPW>
__global__ void __launch_bounds__(W * 32, 1) colslice_fwd_kernel(const ColsliceArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;
  constexpr int VPL = kVPL;
  constexpr int RW = 32 / LPR;        // rows a warp works on at once
  constexpr int GR = W * RPW * RW;    // rows per group
  constexpr int SLICE = LPR * VPL;    // vectors per slice
  constexpr int KMAX = kMaxGrid / LPR;  // partials of one row per lane

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / LPR;  // which of the warp's RW rows
  const int l = lane % LPR;
  const int G = gridDim.x;
  const int b = blockIdx.x;
  const int64_t N = a.N;
  const int64_t D = a.D;
  const int64_t rowvecs = D / EPV;
  const int64_t vec0 = static_cast<int64_t>(b) * SLICE + l;
  int nvalid = 0;
#pragma unroll
  for (int v = 0; v < VPL; ++v) nvalid += (vec0 + v * LPR < rowvecs) ? 1 : 0;
  const int last_slice = static_cast<int>((rowvecs - 1) / SLICE);
  const float slice_elems = static_cast<float>(SLICE * EPV);
  const float tail_elems = static_cast<float>(D - static_cast<int64_t>(last_slice) * SLICE * EPV);
  const float my_count = slice_count(b, last_slice, slice_elems, tail_elems);
  const float inv_count = my_count > 0.f ? 1.0f / my_count : 0.f;
  const float inv_D = 1.0f / static_cast<float>(D);

  E g[VPL][NE], be[VPL][NE];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    if (v < nvalid) {
      load_param_lanes<EPV>(a.gamma, (vec0 + v * LPR) * EPV, g[v]);
      load_param_lanes<EPV>(a.beta, (vec0 + v * LPR) * EPV, be[v]);
    } else {
#pragma unroll
      for (int e = 0; e < NE; ++e) g[v][e] = be[v][e] = M::bcast(0.f);
    }
  }

  const P* xp = reinterpret_cast<const P*>(a.x) + vec0;
  P* yp = reinterpret_cast<P*>(a.out) + vec0;
  const int64_t ngroups = (N + GR - 1) / GR;
  bool alive = true;  // false once a grid wait gave up: stop waiting, keep going
  __shared__ int wait_flag;

  // ring: [stage][r][v][warp][lane] 16-byte slots; a lane only ever reads its own slots
  extern __shared__ __align__(16) unsigned char ring_mem[];
  P* ring = reinterpret_cast<P*>(ring_mem);
  auto slot = [&](int stage, int r, int v) -> P* {
    return ring + ((((stage * RPW + r) * VPL + v) * W + warp) * 32 + lane);
  };
  auto row_of = [&](int64_t grp, int r) -> int64_t {
    return grp * GR + (static_cast<int64_t>(r) * W + warp) * RW + sub;
  };
  auto issue_group = [&](int64_t grp, int stage) {
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row_of(grp, r);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const bool ok = row < N && v < nvalid;
        cp_async16(slot(stage, r, v),
                   ok ? static_cast<const void*>(xp + row * rowvecs + v * LPR) : a.x, ok ? 16u : 0u);
      }
    }
    cp_async_commit();
  };
  if (ngroups > 0) issue_group(0, 0);

  for (int64_t grp = 0; grp < ngroups; ++grp) {
    const int stage = static_cast<int>(grp & 1);
    cp_async_wait_all();
    // slice statistics of this lane group's rows: exact two-pass over the staged values
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row_of(grp, r);
      E xe[VPL][NE];
      E acc = M::bcast(0.f);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        unpack<T, EPV>(*slot(stage, r, v), xe[v]);
#pragma unroll
        for (int e = 0; e < NE; ++e) acc = M::add(acc, xe[v][e]);
      }
      const float smean = lane_group_sum<LPR>(M::hsum(acc)) * inv_count;
      const E nm = M::bcast(-smean);
      acc = M::bcast(0.f);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        if (v < nvalid) {
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            const E c = M::add(xe[v][e], nm);
            acc = M::fma(c, c, acc);
          }
        }
      }
      const float m2 = lane_group_sum<LPR>(M::hsum(acc));
      if (l == 0 && row < N) a.partials[row * G + b] = make_float2(smean, m2);
    }
    grid_arrive(a.counter);
    if (grp + 1 < ngroups) issue_group(grp + 1, stage ^ 1);
    if (alive) {
      const unsigned target = static_cast<unsigned>(grp + 1) * static_cast<unsigned>(G);
      if (!grid_wait(a.counter, target, &wait_flag)) {
        alive = false;
        if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, 1);
      }
    }
    // row statistics out of the G partials, in a fixed order
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row_of(grp, r);
      const bool rv = row < N;
      const float2* pr = a.partials + (rv ? row : 0) * G;
      float2 pp[KMAX];
      float s1 = 0.f;
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        const int j = l + LPR * k;
        pp[k] = (rv && j < G) ? __ldcg(&pr[j]) : make_float2(0.f, 0.f);
        s1 = fmaf(slice_count(j, last_slice, slice_elems, tail_elems), pp[k].x, s1);
      }
      const float mean = lane_group_sum<LPR>(s1) * inv_D;
      float s2 = 0.f;
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        const int j = l + LPR * k;
        const float d = pp[k].x - mean;
        s2 += fmaf(slice_count(j, last_slice, slice_elems, tail_elems) * d, d, pp[k].y);
      }
      const float ivar = rsqrtf(fmaf(lane_group_sum<LPR>(s2), inv_D, a.eps));
      if (rv) {
        if (b == 0 && l == 0) {
          a.mean[row] = mean;
          a.ivar[row] = ivar;
        }
        const E nm = M::bcast(-mean), iv2 = M::bcast(ivar);
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          if (v < nvalid) {
            E xe[NE], o[NE];
            unpack<T, EPV>(*slot(stage, r, v), xe);
#pragma unroll
            for (int e = 0; e < NE; ++e)
              o[e] = M::fma(M::mul(M::add(xe[e], nm), iv2), g[v][e], be[v][e]);
            store_stream<T, EPV>(reinterpret_cast<T*>(yp + row * rowvecs + v * LPR), 0,
                                 repack<T, EPV>(o));
          }
        }
      }
    }
  }
}

template <typename T, int LPR, int W, int RPW>
__global__ void __launch_bounds__(W * 32, 1) colslice_bwd_kernel(const ColsliceArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;
  constexpr int VPL = kVPL;
  constexpr int RW = 32 / LPR;
  constexpr int GR = W * RPW * RW;
  constexpr int SLICE = LPR * VPL;
  constexpr int KMAX = kMaxGrid / LPR;

  // dgamma / dbeta of all lanes that own the same columns meet here at the end:
  // [warp][dgamma | dbeta][e][lane]
  __shared__ float2 fold[W][2][NE][32];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / LPR;
  const int l = lane % LPR;
  const int G = gridDim.x;
  const int b = blockIdx.x;
  const int64_t N = a.N;
  const int64_t D = a.D;
  const int64_t rowvecs = D / EPV;
  const int64_t vec0 = static_cast<int64_t>(b) * SLICE + l;
  int nvalid = 0;
#pragma unroll
  for (int v = 0; v < VPL; ++v) nvalid += (vec0 + v * LPR < rowvecs) ? 1 : 0;
  const float inv_D = 1.0f / static_cast<float>(D);

  E g[VPL][NE], dg[VPL][NE], db[VPL][NE];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    if (v < nvalid) {
      load_param_lanes<EPV>(a.gamma, (vec0 + v * LPR) * EPV, g[v]);
    } else {
#pragma unroll
      for (int e = 0; e < NE; ++e) g[v][e] = M::bcast(0.f);
    }
#pragma unroll
    for (int e = 0; e < NE; ++e) dg[v][e] = db[v][e] = M::bcast(0.f);
  }

  const P* xp = reinterpret_cast<const P*>(a.x) + vec0;
  const P* dyp = reinterpret_cast<const P*>(a.dy) + vec0;
  P* dxp = reinterpret_cast<P*>(a.out) + vec0;
  const int64_t ngroups = (N + GR - 1) / GR;
  bool alive = true;
  __shared__ int wait_flag;

  // ring: [stage][x | dy][r][v][warp][lane] 16-byte slots
  extern __shared__ __align__(16) unsigned char ring_mem[];
  P* ring = reinterpret_cast<P*>(ring_mem);
  auto slot = [&](int stage, int t, int r, int v) -> P* {
    return ring + (((((stage * 2 + t) * RPW + r) * VPL + v) * W + warp) * 32 + lane);
  };
  auto row_of = [&](int64_t grp, int r) -> int64_t {
    return grp * GR + (static_cast<int64_t>(r) * W + warp) * RW + sub;
  };
  float cmean[RPW], civar[RPW], nmean[RPW], nivar[RPW];
  auto issue_group = [&](int64_t grp, int stage, float (&bm)[RPW], float (&bi)[RPW]) {
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row_of(grp, r);
      const bool rv = row < N;
      bm[r] = rv ? __ldg(a.mean_in + row) : 0.f;
      bi[r] = rv ? __ldg(a.ivar_in + row) : 0.f;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const bool ok = rv && v < nvalid;
        cp_async16(slot(stage, 0, r, v),
                   ok ? static_cast<const void*>(xp + row * rowvecs + v * LPR) : a.x, ok ? 16u : 0u);
        cp_async16(slot(stage, 1, r, v),
                   ok ? static_cast<const void*>(dyp + row * rowvecs + v * LPR) : a.dy,
                   ok ? 16u : 0u);
      }
    }
    cp_async_commit();
  };
  if (ngroups > 0) issue_group(0, 0, cmean, civar);

  for (int64_t grp = 0; grp < ngroups; ++grp) {
    const int stage = static_cast<int>(grp & 1);
    cp_async_wait_all();
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row_of(grp, r);
      const E nm = M::bcast(-cmean[r]), iv2 = M::bcast(civar[r]);
      E r0 = M::bcast(0.f), r1 = M::bcast(0.f);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        E xe[NE], ge[NE];
        unpack<T, EPV>(*slot(stage, 0, r, v), xe);
        unpack<T, EPV>(*slot(stage, 1, r, v), ge);
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          xe[e] = M::mul(M::add(xe[e], nm), iv2);  // zero-filled lanes: dy and gamma are zero
          dg[v][e] = M::fma(ge[e], xe[e], dg[v][e]);
          db[v][e] = M::add(db[v][e], ge[e]);
          ge[e] = M::mul(ge[e], g[v][e]);
          r0 = M::add(r0, ge[e]);
          r1 = M::fma(ge[e], xe[e], r1);
        }
      }
      const float s0 = lane_group_sum<LPR>(M::hsum(r0));
      const float s1 = lane_group_sum<LPR>(M::hsum(r1));
      if (l == 0 && row < N) a.partials[row * G + b] = make_float2(s0, s1);
    }
    grid_arrive(a.counter);
    if (grp + 1 < ngroups) issue_group(grp + 1, stage ^ 1, nmean, nivar);
    if (alive) {
      const unsigned target = static_cast<unsigned>(grp + 1) * static_cast<unsigned>(G);
      if (!grid_wait(a.counter, target, &wait_flag)) {
        alive = false;
        if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, 1);
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row_of(grp, r);
      const bool rv = row < N;
      const float2* pr = a.partials + (rv ? row : 0) * G;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        const int j = l + LPR * k;
        const float2 p = (rv && j < G) ? __ldcg(&pr[j]) : make_float2(0.f, 0.f);
        s0 += p.x;
        s1 += p.y;
      }
      s0 = lane_group_sum<LPR>(s0);
      s1 = lane_group_sum<LPR>(s1);
      if (rv) {
        // dx = ivar * (gy - (m0 + xh * m1)): subtraction before scaling (exact cancellation)
        const E nm = M::bcast(-cmean[r]), iv2 = M::bcast(civar[r]);
        const E nm0 = M::bcast(-(s0 * inv_D)), nm1 = M::bcast(-(s1 * inv_D));
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          if (v < nvalid) {
            E xe[NE], ge[NE], o[NE];
            unpack<T, EPV>(*slot(stage, 0, r, v), xe);
            unpack<T, EPV>(*slot(stage, 1, r, v), ge);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              xe[e] = M::mul(M::add(xe[e], nm), iv2);
              ge[e] = M::mul(ge[e], g[v][e]);
              o[e] = M::mul(M::add(ge[e], M::fma(xe[e], nm1, nm0)), iv2);
            }
            store_stream<T, EPV>(reinterpret_cast<T*>(dxp + row * rowvecs + v * LPR), 0,
                                 repack<T, EPV>(o));
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      cmean[r] = nmean[r];
      civar[r] = nivar[r];
    }
  }

  // Fold dgamma / dbeta over the warps and the RW lane groups of a warp, in a fixed order,
  // one vector slot at a time; the first lane group of warp 0 writes the final values.
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      fold[warp][0][e][lane] = dg[v][e];
      fold[warp][1][e][lane] = db[v][e];
    }
    __syncthreads();
    if (warp == 0 && sub == 0 && v < nvalid) {
      E tg[NE], tb[NE];
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        float2 sg = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
        for (int w = 0; w < W; ++w) {
#pragma unroll
          for (int q = 0; q < RW; ++q) {
            const float2 pg = fold[w][0][e][q * LPR + l], pb = fold[w][1][e][q * LPR + l];
            sg = make_float2(sg.x + pg.x, sg.y + pg.y);
            sb = make_float2(sb.x + pb.x, sb.y + pb.y);
          }
        }
        tg[e] = sg;
        tb[e] = sb;
      }
      store_param_lanes<EPV>(a.dgamma, (vec0 + v * LPR) * EPV, tg);
      store_param_lanes<EPV>(a.dbeta, (vec0 + v * LPR) * EPV, tb);
    }
    __syncthreads();
  }
}

template <typename Kernel>
cudaError_t launch_cooperative(Kernel kernel, int grid, int block, size_t ring_bytes,
                               ColsliceArgs& a, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(ring_bytes));
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(a.counter, 0, sizeof(unsigned), s);
  if (e != cudaSuccess) return e;
  void* params[] = {&a};
  count_launch();
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(grid), dim3(block),
                                     params, ring_bytes, s);
}

// two stages x tensors x RPW row sets x kVPL vectors x W warps x 32 lanes x 16 bytes
constexpr size_t ring_bytes(int tensors, int rpw, int warps) {
  return static_cast<size_t>(2) * tensors * rpw * kVPL * warps * 32 * 16;
}

constexpr int kFwdWarps = 8, kFwdRpw = 6;   // 192 KB ring
constexpr int kBwdWarps = 8, kBwdRpw = 3;   // 192 KB ring

template <typename T>
cudaError_t fwd_t(int lpr, int grid, ColsliceArgs& a, cudaStream_t s) {
  constexpr size_t ring = ring_bytes(1, kFwdRpw, kFwdWarps);
  switch (lpr) {
    case 8: return launch_cooperative(colslice_fwd_kernel<T, 8, kFwdWarps, kFwdRpw>, grid, kFwdWarps * 32, ring, a, s);
    case 16: return launch_cooperative(colslice_fwd_kernel<T, 16, kFwdWarps, kFwdRpw>, grid, kFwdWarps * 32, ring, a, s);
    case 32: return launch_cooperative(colslice_fwd_kernel<T, 32, kFwdWarps, kFwdRpw>, grid, kFwdWarps * 32, ring, a, s);
  }
  return cudaErrorInvalidValue;
}
template <typename T>
cudaError_t bwd_t(int lpr, int grid, ColsliceArgs& a, cudaStream_t s) {
  constexpr size_t ring = ring_bytes(2, kBwdRpw, kBwdWarps);
  switch (lpr) {
    case 8: return launch_cooperative(colslice_bwd_kernel<T, 8, kBwdWarps, kBwdRpw>, grid, kBwdWarps * 32, ring, a, s);
    case 16: return launch_cooperative(colslice_bwd_kernel<T, 16, kBwdWarps, kBwdRpw>, grid, kBwdWarps * 32, ring, a, s);
    case 32: return launch_cooperative(colslice_bwd_kernel<T, 32, kBwdWarps, kBwdRpw>, grid, kBwdWarps * 32, ring, a, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

// Geometry for rows of `nvec` 128-bit vectors: the fewest lanes per row slice (slices of
// 4 * lanes vectors) that keep the grid within one CTA per SM.  Returns false when the rows
// are too narrow to be worth it or too wide.
bool colslice_plan(int64_t nvec, int64_t rows, ColslicePlan* p) {
  const int sms = device_sm_count();
  if (sms <= 0 || rows <= 0) return false;
  for (int lpr = 8; lpr <= 32; lpr *= 2) {
    const int64_t grid = (nvec + kVPL * lpr - 1) / (kVPL * lpr);
    if (grid <= sms && grid <= kMaxGrid) {
      // at least 5/8 of the SMs busy, and the arrival counter must not wrap
      if (grid * 8 < static_cast<int64_t>(sms) * 5) return false;
      if (rows * grid >= (1ll << 31)) return false;
      p->vpl = lpr;
      p->grid = static_cast<int>(grid);
      p->partial_bytes = static_cast<size_t>(rows) * static_cast<size_t>(grid) * sizeof(float2);
      return true;
    }
  }
  return false;
}

cudaError_t colslice_launch(int dtype, bool bwd, const ColslicePlan& p, const RowsArgs& r,
                            float* dgamma, float* dbeta, void* partials, void* counter,
                            cudaStream_t s) {
  ColsliceArgs a = {};
  a.x = r.x;
  a.dy = r.dy;
  a.gamma = r.gamma;
  a.beta = r.beta;
  a.mean_in = r.mean_in;
  a.ivar_in = r.ivar_in;
  a.out = r.out;
  a.mean = r.mean;
  a.ivar = r.ivar;
  a.dgamma = dgamma;
  a.dbeta = dbeta;
  a.partials = static_cast<float2*>(partials);
  a.counter = static_cast<unsigned*>(counter);
  a.N = r.N;
  a.D = r.D;
  a.eps = r.eps;
  a.status = r.status;
  if (dtype == 0) return bwd ? bwd_t<float>(p.vpl, p.grid, a, s) : fwd_t<float>(p.vpl, p.grid, a, s);
  if (dtype == 1) return bwd ? bwd_t<__half>(p.vpl, p.grid, a, s) : fwd_t<__half>(p.vpl, p.grid, a, s);
  return bwd ? bwd_t<__nv_bfloat16>(p.vpl, p.grid, a, s) : fwd_t<__nv_bfloat16>(p.vpl, p.grid, a, s);
}

}  // namespace nvn
