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

#include <stdlib.h>

#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

// Threads per CTA: a row group when it is at least BLK threads, otherwise as many row
// groups as fill BLK threads (BLK == 0 selects the default of 256).
template <int TPR, int BLK>
struct RowBlock {
  static constexpr int kMin = BLK == 0 ? 256 : BLK;
  static constexpr int kBlock = TPR >= kMin ? TPR : kMin;
  static constexpr int kRowsPerCta = kBlock / TPR;
};

// Template parameters shared by the forward and backward kernels
//   EPV   elements per vector access (16 bytes / sizeof(T), or 1 for the scalar family)
//   TPR   threads per row inside one CTA
//   VPT   vectors per thread and row
//   CS    CTAs per cluster (all working on the same row)
//   RB    rows a row group works on at once: their loads are issued back to back and
//         their reductions share one barrier
//   PR    keep gamma (and beta) for the thread's columns in registers for the whole
//         kernel instead of re-reading them (L1 / L2 hits) for every row
//   MINB  CTA size when a row group is smaller than that: 0 = 256 threads, else the value
//         (128 gives finer-grained CTAs: fewer row groups share a barrier)
//   PF    load mode.  0: plain loads at the top of each iteration.  1: register prefetch -
//         the loads of the next row batch are issued as soon as the current batch has been
//         converted to fp32, so they are in flight during the reductions and the stores.
//         >= 2: a shared-memory ring of PF stages filled by cp.async.bulk (TMA); one thread
//         issues whole row batches, mbarriers signal arrival, and the bytes in flight no
//         longer depend on registers or occupancy.
//         >= 10 (backward only): a ring of PF - 10 stages whose row batch stays in shared
//         memory until its dx has been written; both passes over the batch read it from
//         there, so no fp32 copy of the batch lives in registers across the reduction and
//         two CTAs of 256 threads fit on an SM.
//
// All element-wise math runs on fp32x2 lanes (nvn::P2) when EPV is even.

//   EXACT the row is exactly TPR*VPT*CS vectors wide: no per-vector bounds checks
//
// Instruction count matters as much as bytes here: at ~23 bytes per clock per SM a
// 16-bit row leaves ~20-30 issue slots per element.  Hence fp32x2 math, pointer
// arithmetic that leaves only immediate offsets inside the vector loops, 1/D and
// rsqrt instead of divisions, and the EXACT specialisation.

template <typename T, int EPV, int VPT, int RB>
struct RowTile {
  Pack<T, EPV> p[RB][VPT];
};

// Loads the RB x VPT vectors of one row batch.  `src` already points at this
// thread's first vector of row 0; rows are `rowvecs` vectors apart and a thread's
// vectors VSTRIDE apart (a compile-time constant, so they become immediate offsets).
template <typename T, int EPV, int VPT, int RB, int RPC, int VSTRIDE, bool EXACT>
__device__ __forceinline__ void load_tile(const Pack<T, EPV>* __restrict__ src, int64_t row_first,
                                          int64_t N, int64_t rowvecs, int nvalid,
                                          RowTile<T, EPV, VPT, RB>& t) {
#pragma unroll
  for (int r = 0; r < RB; ++r) {
    const int64_t row = row_first + r * RPC;
    const Pack<T, EPV>* rp = src + row * rowvecs;
    const bool rv = row < N;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && (EXACT || v < nvalid)) {
        t.p[r][v] = load_stream<T, EPV>(reinterpret_cast<const T*>(rp + v * VSTRIDE), 0);
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) t.p[r][v].v[e] = Cvt<T>::from_f32(0.f);
      }
    }
  }
}

// Shared-memory ring of the TMA load mode.  A stage holds one row batch of this CTA:
// RPC*RB consecutive rows when a CTA owns whole rows (CS == 1), or RB row slices of
// D/CS elements when a cluster shares the rows.  NT tensors (x, or x and dy) sit one after
// the other inside a stage.
template <typename T, int EPV, int VPT, int RB, int RPC, int CS, int STAGES, int NT>
struct RowRing {
  unsigned char* base;
  uint64_t* full;       // [STAGES]
  unsigned stage_bytes;
  unsigned tensor_bytes;  // bytes of one tensor inside a stage
  unsigned row_bytes;     // bytes of one row (CS == 1) or one row slice (CS > 1)
  bool dead;              // a wait gave up: stop issuing and stop waiting

  __device__ __forceinline__ void init(unsigned char* smem, uint64_t* bars, int64_t D) {
    base = smem;
    full = bars;
    row_bytes = static_cast<unsigned>((D / CS) * sizeof(T));
    tensor_bytes = row_bytes * (CS == 1 ? RPC * RB : RB);
    stage_bytes = tensor_bytes * NT;
    dead = false;
    if (threadIdx.x == 0) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
      mbar_init_fence();
    }
    __syncthreads();
  }

  // Called by one thread: start the copies of the batch whose first row is `row_first`
  // (the CTA's batch base, without the row-group offset) into stage `s`.
  __device__ __forceinline__ void issue(int s, const T* const (&src)[NT], int64_t row_first,
                                        int64_t N, int64_t D, unsigned crank) {
    unsigned char* dst = base + static_cast<size_t>(s) * stage_bytes;
    if constexpr (CS == 1) {
      const int64_t left = N - row_first;
      const unsigned rows = static_cast<unsigned>(left < RPC * RB ? left : RPC * RB);
      const unsigned bytes = rows * row_bytes;
      mbar_expect_tx(&full[s], bytes * NT);
#pragma unroll
      for (int t = 0; t < NT; ++t)
        bulk_load(dst + t * tensor_bytes, src[t] + row_first * D, bytes, &full[s]);
    } else {
      const int64_t left = N - row_first;
      const unsigned rows = static_cast<unsigned>(left < RB ? left : RB);
      mbar_expect_tx(&full[s], rows * row_bytes * NT);
      const int64_t slice = (D / CS) * static_cast<int64_t>(crank);
#pragma unroll
      for (int t = 0; t < NT; ++t)
        for (unsigned r = 0; r < rows; ++r)
          bulk_load(dst + t * tensor_bytes + r * row_bytes, src[t] + (row_first + r) * D + slice,
                    row_bytes, &full[s]);
    }
  }

  __device__ __forceinline__ bool wait(int s, unsigned use) {
    if (dead) return true;
    return mbar_wait_bounded(&full[s], use & 1u);
  }

  // Byte offset, inside a stage, of this thread's first vector of row-slot `rowslot` of
  // tensor t.  Computed once per thread; the per-vector offsets are compile-time constants.
  __device__ __forceinline__ unsigned thread_offset(int t, int rowslot, int slot_vec) const {
    return t * tensor_bytes + rowslot * row_bytes +
           static_cast<unsigned>(slot_vec) * static_cast<unsigned>(sizeof(Pack<T, EPV>));
  }
  __device__ __forceinline__ const unsigned char* stage_ptr(int s) const {
    return base + static_cast<size_t>(s) * stage_bytes;
  }
};

// Per-thread view of a row: which vectors it owns.
//   plain / register-prefetch modes: vector v of a thread is  v*TPR*CS + crank*TPR + lir
//     (the CTAs of a cluster interleave, every access is a full coalesced segment);
//   TMA mode in a cluster: every CTA owns one contiguous slice of D/CS elements (a single
//     bulk copy per row), vector v is  crank*TPR*VPT + v*TPR + lir.
template <int TPR, int VPT, int CS, bool TMA>
struct VecMap {
  static constexpr int kStride = (TMA && CS > 1) ? TPR : TPR * CS;
  static __device__ __forceinline__ int first(unsigned crank, int lir) {
    return (TMA && CS > 1) ? static_cast<int>(crank) * TPR * VPT + lir
                           : static_cast<int>(crank) * TPR + lir;
  }
};

// Tile of the current row batch out of a ring stage (TMA mode).  `off[r]` are the thread's
// precomputed byte offsets (RowRing::thread_offset) of its RB row slots.
template <typename T, int EPV, int VPT, int RB, int RPC, int TPR, bool EXACT>
__device__ __forceinline__ void ring_tile(const unsigned char* stage, const unsigned (&off)[RB],
                                          int64_t row_first, int64_t N, int nvalid,
                                          RowTile<T, EPV, VPT, RB>& tile) {
#pragma unroll
  for (int r = 0; r < RB; ++r) {
    const bool rv = row_first + r * RPC < N;
    const Pack<T, EPV>* p = reinterpret_cast<const Pack<T, EPV>*>(stage + off[r]);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (rv && (EXACT || v < nvalid)) {
        tile.p[r][v] = p[v * TPR];
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) tile.p[r][v].v[e] = Cvt<T>::from_f32(0.f);
      }
    }
  }
}

// After a bounded wait gave up: raise the status word and wait (bounded again) for the
// copies that are still in flight, so none of them lands after the CTA has gone.
// `ahead` = how many batches, counting batch j, have been issued and not yet waited for.
template <typename Ring, int STAGES>
__device__ __forceinline__ void ring_give_up(Ring& ring, int* status, int64_t j, int64_t nb,
                                             int ahead = STAGES) {
  ring.dead = true;
  if (threadIdx.x == 0) {
    if (status != nullptr) atomicExch(status, 1);
    const int64_t last = j + ahead < nb ? j + ahead : nb;
    for (int64_t k = j; k < last; ++k)
      (void)mbar_wait_bounded(&ring.full[k % STAGES], static_cast<unsigned>(k / STAGES) & 1u);
  }
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
//   RES   (forward only) the row that is normalised is s = T(x + res); s is written to
//         a.sum_out.  Plain or register-prefetch loads only.
template <typename T, int EPV, int TPR, int VPT, int CS, int RB, bool PR, int MINB, int PF,
          bool EXACT, bool ROW_AFFINE, bool RES = false>
__global__ void __launch_bounds__(RowBlock<TPR, MINB>::kBlock)
    rows_fwd_kernel(const typename std::conditional<RES, RowsResArgs, RowsArgs>::type a) {
  constexpr int BLOCK = RowBlock<TPR, MINB>::kBlock;
  constexpr int RPC = RowBlock<TPR, MINB>::kRowsPerCta;
  constexpr bool TMA = PF >= 2;
  constexpr int STAGES = TMA ? PF : 1;
  using Map = VecMap<TPR, VPT, CS, TMA>;
  constexpr int VSTRIDE = Map::kStride;
  static_assert(CS == 1 || RPC == 1, "cluster kernels own one row per cluster");
  static_assert(!(TMA && CS > 1) || EXACT, "cluster slices need rows that fill the shape");
  static_assert(!RES || (!TMA && CS == 1 && !ROW_AFFINE), "residual add: LayerNorm, one CTA per row, no ring");
  constexpr bool PARAMS_IN_REGS = !ROW_AFFINE && PR;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;

  // Programmatic dependent launch: the kernel that follows in the stream may be scheduled
  // as CTAs of this one retire, and this one may have been scheduled while its predecessor
  // was still running - nothing that the predecessor may have written (activations,
  // parameters) is read before griddep_wait().
  // (cluster kernels neither launch early nor let their successor: see the launcher)
  if constexpr (CS == 1) griddep_launch_dependents();
  griddep_wait();
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(8) uint64_t ring_bars[STAGES];
  __shared__ ReduceSmem<RB, BLOCK> sm;
  int phase = 0;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int group = tid / TPR;
  const int lir = tid % TPR;
  unsigned crank = 0;
  if constexpr (CS > 1) {
    crank = cg::this_cluster().block_rank();
    // the reductions write into the peers' shared memory: every CTA of the cluster must
    // have started before the first such write
    cg::this_cluster().sync();
  }
  const int64_t unit = blockIdx.x / CS;
  const int64_t nunits = gridDim.x / CS;
  const int64_t N = a.N;
  const int64_t D = a.D;
  const int64_t rowvecs = D / EPV;
  const float inv_D = 1.0f / static_cast<float>(D);
  const float eps = a.eps;
  const int vec0 = Map::first(crank, lir);
  // number of this thread's vectors that fall inside the row (all VPT when EXACT)
  int nvalid = VPT;
  if constexpr (!EXACT) {
    const int left = static_cast<int>(rowvecs) - vec0;
    nvalid = left <= 0 ? 0 : (left + VSTRIDE - 1) / VSTRIDE;
    nvalid = nvalid > VPT ? VPT : nvalid;
  }
  // y may alias x (in-place forward), so these are not __restrict__.
  const P* xp = reinterpret_cast<const P*>(a.x) + vec0;
  P* yp = reinterpret_cast<P*>(a.out) + vec0;
  const P* rsp = nullptr;
  P* sop = nullptr;
  if constexpr (RES) {
    rsp = reinterpret_cast<const P*>(a.res) + vec0;
    sop = reinterpret_cast<P*>(a.sum_out) + vec0;
  }

  E g[PARAMS_IN_REGS ? VPT : 1][NE], b[PARAMS_IN_REGS ? VPT : 1][NE];
  if constexpr (PARAMS_IN_REGS) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (EXACT || v < nvalid) {
        load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, g[v]);
        load_param_lanes<EPV>(a.beta, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, b[v]);
      } else {
#pragma unroll
        for (int e = 0; e < NE; ++e) g[v][e] = b[v][e] = M::bcast(0.f);
      }
    }
  }

  const int64_t stride = nunits * (RPC * RB);
  const int64_t batch0 = unit * (RPC * RB);  // first row of this CTA's first batch
  const int64_t nb = batch0 < N ? (N - batch0 + stride - 1) / stride : 0;
  RowTile<T, EPV, VPT, RB> tile;
  RowTile<T, EPV, VPT, RES ? RB : 1> rtile;   // the residual's row batch
  RowRing<T, EPV, VPT, RB, RPC, CS, STAGES, 1> ring;
  const T* const srcs[1] = {static_cast<const T*>(a.x)};
  unsigned roff[RB];
  if constexpr (TMA) {
    ring.init(ring_mem, ring_bars, D);
#pragma unroll
    for (int r = 0; r < RB; ++r)
      roff[r] = ring.thread_offset(0, CS == 1 ? r * RPC + group : r, lir);
    if (tid == 0) {
      for (int64_t k = 0; k < STAGES && k < nb; ++k)
        ring.issue(static_cast<int>(k), srcs, batch0 + k * stride, N, D, crank);
    }
  } else if constexpr (PF == 1) {
    load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(xp, batch0 + group, N, rowvecs, nvalid, tile);
    if constexpr (RES)
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(rsp, batch0 + group, N, rowvecs, nvalid, rtile);
  }
  for (int64_t j = 0; j < nb; ++j) {
    const int64_t row0 = batch0 + j * stride + group;
    if constexpr (TMA) {
      const int s = static_cast<int>(j % STAGES);
      const bool ok = ring.wait(s, static_cast<unsigned>(j / STAGES));
      ring_tile<T, EPV, VPT, RB, RPC, TPR, EXACT>(ring.stage_ptr(s), roff, row0, N, nvalid, tile);
      // every thread has its copy of the stage: it can be refilled
      if (__syncthreads_or(!ok) && !ring.dead) ring_give_up<decltype(ring), STAGES>(ring, a.status, j, nb);
      if (tid == 0 && !ring.dead && j + STAGES < nb)
        ring.issue(s, srcs, batch0 + (j + STAGES) * stride, N, D, crank);
    } else if constexpr (PF == 0) {
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(xp, row0, N, rowvecs, nvalid, tile);
      if constexpr (RES)
        load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(rsp, row0, N, rowvecs, nvalid, rtile);
    }

    E xv[RB][VPT][NE];
    float s_[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      E acc = M::bcast(0.f);
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        unpack<T, EPV>(tile.p[r][v], xv[r][v]);
        if constexpr (RES) {
          // s = T(x + res): the sum is rounded to the activation type before anything else
          // uses it, because the backward pass will read the stored s
          E rv[NE];
          unpack<T, EPV>(rtile.p[r][v], rv);
#pragma unroll
          for (int e = 0; e < NE; ++e) rv[e] = M::add(xv[r][v][e], rv[e]);
          const P sp = repack<T, EPV>(rv);
          if (row0 + r * RPC < N && (EXACT || v < nvalid))
            store_stream<T, EPV>(reinterpret_cast<T*>(sop + (row0 + r * RPC) * rowvecs + v * VSTRIDE), 0, sp);
          unpack<T, EPV>(sp, xv[r][v]);
        }
#pragma unroll
        for (int e = 0; e < NE; ++e) acc = M::add(acc, xv[r][v][e]);
      }
      s_[r] = M::hsum(acc);
    }
    if constexpr (PF == 1) {
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(xp, row0 + stride, N, rowvecs, nvalid, tile);
      if constexpr (RES)
        load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(rsp, row0 + stride, N, rowvecs, nvalid, rtile);
    }
    group_allreduce<RB, TPR, BLOCK, CS>(s_, sm, phase, warp, lane);

    float mean[RB], q[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      mean[r] = s_[r] * inv_D;
      const E nm = M::bcast(-mean[r]);
      E acc = M::bcast(0.f);
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        if (EXACT || v < nvalid) {
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            xv[r][v][e] = M::add(xv[r][v][e], nm);  // centred value, reused below
            acc = M::fma(xv[r][v][e], xv[r][v][e], acc);
          }
        }
      }
      q[r] = M::hsum(acc);
    }
    group_allreduce<RB, TPR, BLOCK, CS>(q, sm, phase, warp, lane);

#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int64_t row = row0 + r * RPC;
      const float ivar = rsqrtf(fmaf(q[r], inv_D, eps));
      if (row < N) {
        float gr = 1.f, br = 0.f;
        if constexpr (ROW_AFFINE) {
          const int64_t c = row % a.C;
          gr = __ldg(a.gamma + c);
          br = __ldg(a.beta + c);
        }
        const E iv2 = M::bcast(ivar);
        const E sc2 = M::bcast(ivar * gr);
        const E br2 = M::bcast(br);
        P* rp = yp + row * rowvecs;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
          if (EXACT || v < nvalid) {
            E o[NE];
            if constexpr (ROW_AFFINE) {
#pragma unroll
              for (int e = 0; e < NE; ++e) o[e] = M::fma(xv[r][v][e], sc2, br2);
            } else if constexpr (PARAMS_IN_REGS) {
#pragma unroll
              for (int e = 0; e < NE; ++e)
                o[e] = M::fma(M::mul(xv[r][v][e], iv2), g[v][e], b[v][e]);
            } else {
              E gg[NE], bb[NE];
              load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, gg);
              load_param_lanes<EPV>(a.beta, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, bb);
#pragma unroll
              for (int e = 0; e < NE; ++e) o[e] = M::fma(M::mul(xv[r][v][e], iv2), gg[e], bb[e]);
            }
            store_stream<T, EPV>(reinterpret_cast<T*>(rp + v * VSTRIDE), 0, repack<T, EPV>(o));
          }
        }
        if (lir == 0 && crank == 0) {
          a.mean[row] = mean[r];
          a.ivar[row] = ivar;
        }
      }
    }
  }
  // A CTA's shared memory must stay mapped until its cluster peers have read it.
  if constexpr (CS > 1) cg::this_cluster().sync();
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
template <typename T, int EPV, int TPR, int VPT, int CS, int RB, bool PR, int MINB, int PF,
          bool EXACT, bool ROW_AFFINE>
__global__ void __launch_bounds__(RowBlock<TPR, MINB>::kBlock)
    rows_bwd_kernel(const RowsArgs a) {
  constexpr int BLOCK = RowBlock<TPR, MINB>::kBlock;
  constexpr int RPC = RowBlock<TPR, MINB>::kRowsPerCta;
  constexpr bool TMA = PF >= 2;
  constexpr bool HOLD = PF >= 10;
  constexpr int STAGES = HOLD ? PF - 10 : (TMA ? PF : 1);
  static_assert(!HOLD || STAGES >= 2, "a held ring needs a stage to refill while one is read");
  using Map = VecMap<TPR, VPT, CS, TMA>;
  constexpr int VSTRIDE = Map::kStride;
  static_assert(CS == 1 || RPC == 1, "cluster kernels own one row per cluster");
  static_assert(!(TMA && CS > 1) || EXACT, "cluster slices need rows that fill the shape");
  constexpr bool PARAMS_IN_REGS = !ROW_AFFINE && PR;
  constexpr int CAP = TPR * VPT * EPV;  // columns one row group covers (CS == 1)
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;

  // The column reduction that follows may be scheduled as CTAs of this kernel retire; this
  // kernel itself reads nothing its predecessor may have written before griddep_wait().
  // (cluster kernels neither launch early nor let their successor: see the launcher)
  if constexpr (CS == 1) griddep_launch_dependents();
  griddep_wait();
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(8) uint64_t ring_bars[STAGES];
  __shared__ ReduceSmem<2 * RB, BLOCK> sm;
  __shared__ float comb[(!ROW_AFFINE && RPC > 1) ? 2 * CAP : 1];
  int phase = 0;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int group = tid / TPR;
  const int lir = tid % TPR;
  unsigned crank = 0;
  if constexpr (CS > 1) {
    crank = cg::this_cluster().block_rank();
    // the reductions write into the peers' shared memory: every CTA of the cluster must
    // have started before the first such write
    cg::this_cluster().sync();
  }
  const int64_t unit = blockIdx.x / CS;
  const int64_t nunits = gridDim.x / CS;
  const int64_t N = a.N;
  const int64_t D = a.D;
  const int64_t rowvecs = D / EPV;
  const float inv_D = 1.0f / static_cast<float>(D);
  const int vec0 = Map::first(crank, lir);
  int nvalid = VPT;
  if constexpr (!EXACT) {
    const int left = static_cast<int>(rowvecs) - vec0;
    nvalid = left <= 0 ? 0 : (left + VSTRIDE - 1) / VSTRIDE;
    nvalid = nvalid > VPT ? VPT : nvalid;
  }
  const P* __restrict__ xp = reinterpret_cast<const P*>(a.x) + vec0;
  const P* __restrict__ dyp = reinterpret_cast<const P*>(a.dy) + vec0;
  P* __restrict__ dxp = reinterpret_cast<P*>(a.out) + vec0;

  E g[PARAMS_IN_REGS ? VPT : 1][NE];
  E dg[ROW_AFFINE ? 1 : VPT][NE], db[ROW_AFFINE ? 1 : VPT][NE];
  if constexpr (PARAMS_IN_REGS) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (EXACT || v < nvalid) {
        load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, g[v]);
      } else {
#pragma unroll
        for (int e = 0; e < NE; ++e) g[v][e] = M::bcast(0.f);
      }
    }
  }
  if constexpr (!ROW_AFFINE) {
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
      for (int e = 0; e < NE; ++e) dg[v][e] = db[v][e] = M::bcast(0.f);
  }

  const int64_t stride = nunits * (RPC * RB);
  const int64_t batch0 = unit * (RPC * RB);
  const int64_t nb = batch0 < N ? (N - batch0 + stride - 1) / stride : 0;
  RowTile<T, EPV, VPT, RB> tx, tdy;
  RowRing<T, EPV, VPT, RB, RPC, CS, STAGES, 2> ring;
  const T* const srcs[2] = {static_cast<const T*>(a.x), static_cast<const T*>(a.dy)};
  unsigned xoff[RB], dyoff[RB];
  if constexpr (TMA) {
    ring.init(ring_mem, ring_bars, D);
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      xoff[r] = ring.thread_offset(0, CS == 1 ? r * RPC + group : r, lir);
      dyoff[r] = ring.thread_offset(1, CS == 1 ? r * RPC + group : r, lir);
    }
    if (tid == 0) {
      for (int64_t k = 0; k < STAGES && k < nb; ++k)
        ring.issue(static_cast<int>(k), srcs, batch0 + k * stride, N, D, crank);
    }
  } else if constexpr (PF == 1) {
    load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(xp, batch0 + group, N, rowvecs, nvalid, tx);
    load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(dyp, batch0 + group, N, rowvecs, nvalid, tdy);
  }
  // The saved statistics of a row are needed the moment its data arrives; fetched on demand
  // they would expose a full memory latency per row batch, so they run two batches ahead.
  float st_mean[3][RB], st_ivar[3][RB];
  auto load_stats = [&](int slot, int64_t first_row) {
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int64_t row = first_row + r * RPC;
      const bool rv = row < N;
      st_mean[slot][r] = rv ? __ldg(a.mean_in + row) : 0.f;
      st_ivar[slot][r] = rv ? __ldg(a.ivar_in + row) : 0.f;
    }
  };
  load_stats(0, batch0 + group);
  load_stats(1, batch0 + stride + group);
  for (int64_t j = 0; j < nb; ++j) {
    const int64_t row0 = batch0 + j * stride + group;
    const unsigned char* stage = nullptr;
    if constexpr (TMA) {
      const int s = static_cast<int>(j % STAGES);
      const bool ok = ring.wait(s, static_cast<unsigned>(j / STAGES));
      stage = ring.stage_ptr(s);
      if constexpr (!HOLD) {
        ring_tile<T, EPV, VPT, RB, RPC, TPR, EXACT>(stage, xoff, row0, N, nvalid, tx);
        ring_tile<T, EPV, VPT, RB, RPC, TPR, EXACT>(stage, dyoff, row0, N, nvalid, tdy);
      }
      if (__syncthreads_or(!ok) && !ring.dead)
        ring_give_up<decltype(ring), STAGES>(ring, a.status, j, nb,
                                             HOLD && j >= 1 ? STAGES - 1 : STAGES);
      if constexpr (!HOLD) {
        if (tid == 0 && !ring.dead && j + STAGES < nb)
          ring.issue(s, srcs, batch0 + (j + STAGES) * stride, N, D, crank);
      } else {
        // Every thread is past the barrier above, hence past its last read of the previous
        // batch: that batch's stage is free to be refilled.
        if (tid == 0 && !ring.dead && j >= 1 && j - 1 + STAGES < nb)
          ring.issue(static_cast<int>((j - 1) % STAGES), srcs, batch0 + (j - 1 + STAGES) * stride,
                     N, D, crank);
      }
    } else if constexpr (PF == 0) {
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(xp, row0, N, rowvecs, nvalid, tx);
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(dyp, row0, N, rowvecs, nvalid, tdy);
    }
    // Held ring: the batch's packed values come out of the stage, in both passes.
    auto held = [&](int r, int v, P& px, P& pdy) {
      if (row0 + r * RPC < N && (EXACT || v < nvalid)) {
        px = reinterpret_cast<const P*>(stage + xoff[r])[v * TPR];
        pdy = reinterpret_cast<const P*>(stage + dyoff[r])[v * TPR];
      } else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) px.v[e] = pdy.v[e] = Cvt<T>::from_f32(0.f);
      }
    };
    float ivar[RB];
    load_stats(2, row0 + 2 * stride);
    // xh = (x - mean) * ivar ; gy = dy * gamma (LayerNorm) or dy (row-affine, where
    // gamma is a per-row scalar applied at the end).  red = (sum gy, sum gy * xh).
    E xh[HOLD ? 1 : RB][HOLD ? 1 : VPT][NE], gy[HOLD ? 1 : RB][HOLD ? 1 : VPT][NE];
    float red[2 * RB];
    float mean_of[HOLD ? RB : 1];
    if constexpr (!HOLD) {
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const float mean = st_mean[0][r];
        ivar[r] = st_ivar[0][r];
        const E nm = M::bcast(-mean), iv2 = M::bcast(ivar[r]);
        E r0 = M::bcast(0.f), r1 = M::bcast(0.f);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
          unpack<T, EPV>(tx.p[r][v], xh[r][v]);
          unpack<T, EPV>(tdy.p[r][v], gy[r][v]);
          if (EXACT || v < nvalid) {
            E gg[NE];
            if constexpr (!ROW_AFFINE && !PARAMS_IN_REGS)
              load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, gg);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              xh[r][v][e] = M::mul(M::add(xh[r][v][e], nm), iv2);
              if constexpr (!ROW_AFFINE) {
                dg[v][e] = M::fma(gy[r][v][e], xh[r][v][e], dg[v][e]);
                db[v][e] = M::add(db[v][e], gy[r][v][e]);
                if constexpr (PARAMS_IN_REGS) {
                  gy[r][v][e] = M::mul(gy[r][v][e], g[v][e]);
                } else {
                  gy[r][v][e] = M::mul(gy[r][v][e], gg[e]);
                }
              }
              r0 = M::add(r0, gy[r][v][e]);
              r1 = M::fma(gy[r][v][e], xh[r][v][e], r1);
            }
          }
        }
        red[2 * r] = M::hsum(r0);
        red[2 * r + 1] = M::hsum(r1);
      }
    } else {
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const float mean = mean_of[r] = st_mean[0][r];
        ivar[r] = st_ivar[0][r];
        const E nm = M::bcast(-mean), iv2 = M::bcast(ivar[r]);
        E r0 = M::bcast(0.f), r1 = M::bcast(0.f);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
          E xv[NE], gv[NE];
          P px, pdy;
          held(r, v, px, pdy);
          unpack<T, EPV>(px, xv);
          unpack<T, EPV>(pdy, gv);
          if (EXACT || v < nvalid) {
            E gg[NE];
            if constexpr (!ROW_AFFINE && !PARAMS_IN_REGS)
              load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, gg);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              xv[e] = M::mul(M::add(xv[e], nm), iv2);
              if constexpr (!ROW_AFFINE) {
                dg[v][e] = M::fma(gv[e], xv[e], dg[v][e]);
                db[v][e] = M::add(db[v][e], gv[e]);
                if constexpr (PARAMS_IN_REGS) {
                  gv[e] = M::mul(gv[e], g[v][e]);
                } else {
                  gv[e] = M::mul(gv[e], gg[e]);
                }
              }
              r0 = M::add(r0, gv[e]);
              r1 = M::fma(gv[e], xv[e], r1);
            }
          }
        }
        red[2 * r] = M::hsum(r0);
        red[2 * r + 1] = M::hsum(r1);
      }
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      st_mean[0][r] = st_mean[1][r];
      st_ivar[0][r] = st_ivar[1][r];
      st_mean[1][r] = st_mean[2][r];
      st_ivar[1][r] = st_ivar[2][r];
    }
    if constexpr (PF == 1) {
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(xp, row0 + stride, N, rowvecs, nvalid, tx);
      load_tile<T, EPV, VPT, RB, RPC, VSTRIDE, EXACT>(dyp, row0 + stride, N, rowvecs, nvalid, tdy);
    }
    group_allreduce<2 * RB, TPR, BLOCK, CS>(red, sm, phase, warp, lane);

#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int64_t row = row0 + r * RPC;
      if (row < N) {
        float scale = ivar[r];
        if constexpr (ROW_AFFINE) {
          const int64_t n = row / a.C;
          const int64_t c = row - n * a.C;
          scale = ivar[r] * __ldg(a.gamma + c);
          if (lir == 0 && crank == 0) {
            // per-(n, c) partials laid out [n][2][C]: dgamma then dbeta
            a.ws[(n * 2 + 0) * a.C + c] = red[2 * r + 1];
            a.ws[(n * 2 + 1) * a.C + c] = red[2 * r];
          }
        }
        // dx = scale * (gy - (m0 + xh * m1)), m0 = red0 / D, m1 = red1 / D.  The
        // subtraction happens before the scaling so that rows whose terms cancel
        // exactly (D == 1, constant rows) give exactly zero.
        const E sc2 = M::bcast(scale);
        const E nm0 = M::bcast(-(red[2 * r] * inv_D));
        const E nm1 = M::bcast(-(red[2 * r + 1] * inv_D));
        P* rp = dxp + row * rowvecs;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
          if (EXACT || v < nvalid) {
            E o[NE];
            if constexpr (HOLD) {
              // second pass over the batch, again out of the ring stage
              E xv[NE], gv[NE], gg[NE];
              P px, pdy;
              held(r, v, px, pdy);
              unpack<T, EPV>(px, xv);
              unpack<T, EPV>(pdy, gv);
              if constexpr (!ROW_AFFINE && !PARAMS_IN_REGS)
                load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, gg);
              const E nm = M::bcast(-mean_of[r]), iv2 = M::bcast(ivar[r]);
#pragma unroll
              for (int e = 0; e < NE; ++e) {
                xv[e] = M::mul(M::add(xv[e], nm), iv2);
                if constexpr (!ROW_AFFINE) {
                  if constexpr (PARAMS_IN_REGS) {
                    gv[e] = M::mul(gv[e], g[v][e]);
                  } else {
                    gv[e] = M::mul(gv[e], gg[e]);
                  }
                }
                o[e] = M::mul(M::add(gv[e], M::fma(xv[e], nm1, nm0)), sc2);
              }
            } else {
#pragma unroll
              for (int e = 0; e < NE; ++e)
                o[e] = M::mul(M::add(gy[r][v][e], M::fma(xh[r][v][e], nm1, nm0)), sc2);
            }
            store_stream<T, EPV>(reinterpret_cast<T*>(rp + v * VSTRIDE), 0, repack<T, EPV>(o));
          }
        }
      }
    }
  }

  if constexpr (!ROW_AFFINE) {
    float* __restrict__ wg = a.ws + (unit * 2 + 0) * D;
    float* __restrict__ wb = a.ws + (unit * 2 + 1) * D;
    if constexpr (RPC > 1) {
      // Fold the row groups of this CTA in group order, then group 0 writes.
      float* cg_ = comb;
      float* cb_ = comb + CAP;
      for (int rgrp = 0; rgrp < RPC; ++rgrp) {
        if (group == rgrp) {
#pragma unroll
          for (int v = 0; v < VPT; ++v)
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              // lane-major layout keeps the shared-memory accesses conflict-free
              if constexpr (EPV == 1) {
                const int idx = v * TPR + lir;
                cg_[idx] = (rgrp == 0 ? 0.f : cg_[idx]) + dg[v][e];
                cb_[idx] = (rgrp == 0 ? 0.f : cb_[idx]) + db[v][e];
              } else {
                float2* cg2 = reinterpret_cast<float2*>(cg_);
                float2* cb2 = reinterpret_cast<float2*>(cb_);
                const int idx = (v * NE + e) * TPR + lir;
                float2 pg = rgrp == 0 ? make_float2(0.f, 0.f) : cg2[idx];
                float2 pb = rgrp == 0 ? make_float2(0.f, 0.f) : cb2[idx];
                cg2[idx] = make_float2(pg.x + dg[v][e].x, pg.y + dg[v][e].y);
                cb2[idx] = make_float2(pb.x + db[v][e].x, pb.y + db[v][e].y);
              }
            }
        }
        __syncthreads();
      }
      if (group == 0) {
#pragma unroll
        for (int v = 0; v < VPT; ++v)
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            if constexpr (EPV == 1) {
              dg[v][e] = cg_[v * TPR + lir];
              db[v][e] = cb_[v * TPR + lir];
            } else {
              dg[v][e] = reinterpret_cast<float2*>(cg_)[(v * NE + e) * TPR + lir];
              db[v][e] = reinterpret_cast<float2*>(cb_)[(v * NE + e) * TPR + lir];
            }
          }
      }
    }
    if (group == 0) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        if (EXACT || v < nvalid) {
          store_param_lanes<EPV>(wg, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, dg[v]);
          store_param_lanes<EPV>(wb, static_cast<int64_t>(vec0 + v * VSTRIDE) * EPV, db[v]);
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
inline int resident_units(Kernel kernel, int block, int cs, size_t dyn_smem) {
  // Number of CTAs (CS == 1) or clusters that fit on the current device at once.
  int sms = device_sm_count();
  if (cs == 1) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, dyn_smem) !=
            cudaSuccess ||
        per_sm < 1)
      per_sm = 1;
    return sms * per_sm;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sms * cs), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(block), 1, 1);
  cfg.dynamicSmemBytes = dyn_smem;
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

// Largest ring a TMA-mode kernel may ask for; wider problems use register prefetch.  Held
// rings belong to shapes chosen so that the ring, not the register file, sets the number of
// CTAs per SM, so they may take most of the SM's shared memory.
constexpr size_t kMaxRingBytes = 96 * 1024;
constexpr size_t kMaxHeldRingBytes = 200 * 1024;

template <typename T, int EPV, int TPR, int VPT, int CS, int RB, bool PR, int MINB, int PF,
          bool EXACT, bool ROW_AFFINE, bool BWD>
inline cudaError_t launch_rows_exact(const RowsArgs& a, cudaStream_t stream, bool dry_run,
                                     RowsPlan* plan) {
  constexpr int BLOCK = RowBlock<TPR, MINB>::kBlock;
  constexpr int RPC = RowBlock<TPR, MINB>::kRowsPerCta;
  constexpr bool TMA = PF >= 2;
  size_t ring = 0;
  if constexpr (TMA) {
    const size_t row_bytes = static_cast<size_t>(a.D / CS) * sizeof(T);
    ring = row_bytes * (CS == 1 ? RPC * RB : RB) * (BWD ? 2 : 1) * (PF >= 10 ? PF - 10 : PF);
    // rows that would need too large a ring, or clusters on rows that do not fill the
    // shape, fall back to the register-prefetch twin of this shape
    if (ring > (PF >= 10 ? kMaxHeldRingBytes : kMaxRingBytes) || (CS > 1 && !EXACT) ||
        sizeof(Pack<T, EPV>) < 16)
      // (a held ring affords row batches that the register file does not)
      return launch_rows_exact<T, EPV, TPR, VPT, CS, (PF >= 10 ? 1 : RB), PR, MINB, 1, EXACT,
                               ROW_AFFINE, BWD>(a, stream, dry_run, plan);
  }
  void (*kernel)(const RowsArgs);
  if constexpr (BWD) {
    kernel = rows_bwd_kernel<T, EPV, TPR, VPT, CS, RB, PR, MINB, PF, (EXACT || (TMA && CS > 1)),
                             ROW_AFFINE>;
  } else {
    kernel = rows_fwd_kernel<T, EPV, TPR, VPT, CS, RB, PR, MINB, PF, (EXACT || (TMA && CS > 1)),
                             ROW_AFFINE>;
  }
  // The attributes are set once per device; the occupancy is cached per process (every
  // device this library runs on is the same part) and depends on the ring size, hence on D.
  static std::atomic<int64_t> cached{0};  // (ring bytes << 20) | units
  static std::atomic<uint64_t> prepared{0};
  {
    const cudaError_t e = once_per_device(prepared, [&]() -> cudaError_t {
      if (CS > 8) {
        cudaError_t e1 =
            cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e1 != cudaSuccess) return e1;
      }
      if (TMA) {
        // the ring shares the SM's 227 KB with the kernel's static shared memory
        cudaFuncAttributes fa;
        cudaError_t e1 = cudaFuncGetAttributes(&fa, kernel);
        if (e1 != cudaSuccess) return e1;
        const size_t room = 227 * 1024 - fa.sharedSizeBytes - 1024;
        const size_t most = PF >= 10 ? kMaxHeldRingBytes : kMaxRingBytes;
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(most < room ? most : room));
      }
      return cudaSuccess;
    });
    if (e != cudaSuccess) return e;
  }
  int units = 0;
  const int64_t c = cached.load(std::memory_order_relaxed);
  if (c != 0 && static_cast<size_t>(c >> 20) == ring) {
    units = static_cast<int>(c & 0xfffff);
  } else {
    units = resident_units(kernel, BLOCK, CS, ring);
    cached.store((static_cast<int64_t>(ring) << 20) | units, std::memory_order_relaxed);
  }
  const int64_t need = (a.N + RPC * RB - 1) / (RPC * RB);
  int64_t use = need < units ? need : units;
  plan->grid = static_cast<int>(use) * CS;
  plan->block = BLOCK;
  plan->cluster = CS;
  plan->tpr = TPR;
  plan->vpt = VPT;
  plan->epv = EPV;
  plan->rb = RB;
  plan->load_mode = PF;
  plan->partial_rows = static_cast<int>(use);
  if (dry_run) return cudaSuccess;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan->grid), 1, 1);
  cfg.blockDim = dim3(BLOCK, 1, 1);
  cfg.dynamicSmemBytes = ring;
  cfg.stream = stream;
  // programmatic stream serialization: see griddep_wait() in the kernels
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  // Worth it for short kernels only: it hides a microsecond or two of launch latency
  // (LayerNorm [4096, 4096] bf16: 36.6 -> 35.4 us per step), but CTAs of the next kernel that
  // become resident early and wait take room from a long kernel's successors - InstanceNorm
  // bf16 NC... [64, 256, 128, 128] ran 3 % slower with it, fp16 [64, 256, 32, 32, 32] with
  // its cluster backward 44 % slower.  Cluster kernels of any size stay out of it: [2, 256,
  // 32, 32, 32] (33 MB) took 49 us per step with dependent launches and 39 us without.
  const bool short_kernel =
      static_cast<int64_t>(a.N) * a.D * static_cast<int64_t>(sizeof(T)) <= (int64_t(128) << 20);
  attr[0].val.programmaticStreamSerializationAllowed =
      use_dependent_launch() && short_kernel && CS == 1 ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (CS > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CS;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <typename T, int EPV, int TPR, int VPT, int CS, int RB, bool PR, int MINB, int PF,
          bool ROW_AFFINE, bool BWD>
inline cudaError_t launch_rows_one(const RowsArgs& a, cudaStream_t stream, bool dry_run,
                                   RowsPlan* plan) {
  // Rows that fill the shape exactly skip every per-vector bounds check.
  if (a.D == static_cast<int64_t>(TPR) * VPT * CS * EPV)
    return launch_rows_exact<T, EPV, TPR, VPT, CS, RB, PR, MINB, PF, true, ROW_AFFINE, BWD>(
        a, stream, dry_run, plan);
  return launch_rows_exact<T, EPV, TPR, VPT, CS, RB, PR, MINB, PF, false, ROW_AFFINE, BWD>(
      a, stream, dry_run, plan);
}

// The LayerNorm backward kernels carry the dgamma / dbeta accumulators and use
// their own shape table; everything else (LayerNorm forward, InstanceNorm
// forward and backward) shares the light table.
template <typename T, bool ROW_AFFINE, bool BWD>
cudaError_t launch_rows_vec(int shape, const RowsArgs& a, cudaStream_t s, bool dry, RowsPlan* p) {
  constexpr int EPV = VecTraits<T>::kFull;
#define X(I, TPR, VPT, CS, RB, PR, MINB, PF) \
  case I:                                    \
    return launch_rows_one<T, EPV, TPR, VPT, CS, RB, PR != 0, MINB, PF, ROW_AFFINE, BWD>( \
        a, s, dry, p);
  if constexpr (BWD && !ROW_AFFINE) {
    switch (shape) {
      NVN_ROW_SHAPES_HEAVY(X)
      default:
        return cudaErrorInvalidValue;
    }
  } else if constexpr (BWD && ROW_AFFINE) {
    switch (shape) {
      NVN_ROW_SHAPES_LIGHT(X)
      NVN_ROW_SHAPES_AFFINE_WIDE(X)
      default:
        return cudaErrorInvalidValue;
    }
  } else {
    switch (shape) {
      NVN_ROW_SHAPES_LIGHT(X)
      default:
        return cudaErrorInvalidValue;
    }
  }
#undef X
}

// Narrower accesses (EPV below a full 128-bit vector, down to single elements) exist for
// rows whose width or alignment rules out 128-bit accesses.  They share one coarse table.
template <typename T, int EPV, bool ROW_AFFINE, bool BWD>
cudaError_t launch_rows_coarse(int shape, const RowsArgs& a, cudaStream_t s, bool dry,
                               RowsPlan* p) {
  switch (shape) {
#define X(I, TPR, VPT, CS, RB, PR, MINB, PF) \
  case I:                                    \
    return launch_rows_one<T, EPV, TPR, VPT, CS, RB, PR != 0, MINB, PF, ROW_AFFINE, BWD>( \
        a, s, dry, p);
    NVN_ROW_SHAPES_SCALAR(X)
#undef X
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace nvn
