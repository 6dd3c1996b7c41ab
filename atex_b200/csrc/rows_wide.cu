// LayerNorm for rows that one CTA cannot hold (thousands of 128-bit vectors per row, few
// rows): a thread-block cluster of CS CTAs owns a row, CTA k its k-th contiguous slice.
//
// What bounds such problems is latency, not bytes: [256, 65536] fp16 is 32 MB per tensor,
// a handful of rows per cluster, and every row needs a reduction across the cluster.  So
//   * each CTA streams its slices through a shared-memory ring filled by cp.async.bulk
//     (one copy per row slice, bounded mbarrier waits): the loads of the next rows are in
//     flight whatever the threads are doing, and the slice stays in its stage until the
//     output is written (read twice from shared memory, once from HBM);
//   * the cluster reduction is ONE exchange per row - forward sends (mean, M2) of the slice
//     and merges with Chan's formula, backward sends the two sums;
//   * the exchange uses no cluster barrier.  barrier.cluster.arrive has release semantics:
//     it waits until the CTA's earlier global stores (the row just written) have been
//     acknowledged, a full L2 round trip per row for every warp.  Instead each CTA sends
//     its 8 bytes into every peer's shared memory with st.async, which also completes
//     8 bytes on an mbarrier in the RECEIVER's shared memory; a CTA waits (bounded) on its
//     own mbarrier until CS * 8 bytes have arrived.  The output stores are never waited for;
//   * a CTA sends the partial of row j+1 before it waits for the totals of row j, so the
//     DSMEM latency hides under the normalisation of row j.
// gamma / beta and the dgamma / dbeta accumulators of the thread's fixed columns live in
// registers for the whole kernel; backward leaves one partial row per cluster for the
// column reduction (colreduce.cu), like the row-cached kernels.
//
// Every addition has a fixed order, so results are bit-identical run to run.  No multicast
// copy is used: each CTA copies only its own slice of this GPU's memory.
//
// Replaces, for rows that fill one of the shapes below, the reference's temp-buffer path
// LayerNormRowReduceInToTempWelford / TempToOutWelford / LayerNormForwardUpdate
// (atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:572-684) and LayerNormRowReduceInToTemp /
// TempToOut / LayerNormBackwardUpdate (fused_layer_norm_op.cu:523-561, 635-658, 694-719).
#include <atomic>

#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {
namespace {

// Full cluster barrier (release / acquire); used once at the start and once at the end.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (an address in this CTA's shared window) in CTA `rank`
__device__ __forceinline__ unsigned map_to_rank(unsigned local, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// 8 bytes into a peer's shared memory; completes 8 bytes on the peer's mbarrier
__device__ __forceinline__ void st_async_pair(unsigned remote_addr, float a, float b,
                                              unsigned remote_bar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::
          "r"(remote_addr),
      "f"(a), "f"(b), "r"(remote_bar)
      : "memory");
}

// Receive slots of the per-row exchange.  Row k uses slot k % kSlots; a CTA sends row k+1
// before it waits for row k, and four slots keep a slot's previous reader (row k-3) done.
constexpr int kSlots = 4;

// (mean, M2) of two sets with the same number of elements n each
__device__ __forceinline__ void chan_equal(float& mean, float& m2, float om, float oq, float n) {
  const float delta = om - mean;
  mean = 0.5f * (mean + om);
  m2 = m2 + oq + delta * delta * (0.5f * n);
}

template <int BLOCK, int CS, int STAGES, int NV>
struct WideSmem {
  static_assert((BLOCK & (BLOCK - 1)) == 0 && (CS & (CS - 1)) == 0 && BLOCK <= 1024,
                "the merge trees pair warps (at most 32) and cluster ranks by powers of two");
  alignas(8) uint64_t full[STAGES];
  alignas(8) uint64_t recv[kSlots];   // one per receive slot: CS * 8 bytes complete a phase
  alignas(8) float peer[kSlots][CS][NV];  // [slot][cluster rank][value], written by the peers
  float warp_part[2][NV][BLOCK / 32];

  // Called by one thread: expect the CS pairs of the next row that uses `slot`.
  __device__ __forceinline__ void arm(int slot) { mbar_expect_tx(&recv[slot], CS * 8u); }
  // Sends this CTA's pair of row k to every CTA of the cluster (itself included).
  __device__ __forceinline__ void send(int64_t k, unsigned crank, int warp, int lane, float v0,
                                       float v1) {
    if (warp == 0 && lane < CS) {
      const int slot = static_cast<int>(k % kSlots);
      st_async_pair(map_to_rank(smem_u32(&peer[slot][crank][0]), lane), v0, v1,
                    map_to_rank(smem_u32(&recv[slot]), lane));
    }
  }
  // Waits (bounded) until every CTA's pair of row k has arrived; `dead` is set when a wait
  // gave up (the status word is raised and later waits are skipped).
  __device__ __forceinline__ void receive(int64_t k, bool& dead, int* status) {
    const int slot = static_cast<int>(k % kSlots);
    if (!dead && !mbar_wait_bounded(&recv[slot], static_cast<unsigned>(k / kSlots) & 1u)) {
      dead = true;
      if (status != nullptr) atomicExch(status, 1);
    }
  }
};

// The ring of row slices of one CTA.  NT tensors (x, or x and dy) sit one after the other
// inside a stage.
template <typename T, int SLICE_VECS, int STAGES, int NT>
struct SliceRing {
  static constexpr unsigned kTensorBytes = SLICE_VECS * 16u;
  static constexpr unsigned kStageBytes = kTensorBytes * NT;
  unsigned char* base;
  uint64_t* full;
  bool dead;  // a wait gave up: stop waiting (and, in the issuing thread, stop issuing)

  __device__ __forceinline__ void issue(int64_t k, const T* const (&src)[NT], int64_t elem_off) {
    const int s = static_cast<int>(k % STAGES);
    mbar_expect_tx(&full[s], kStageBytes);
#pragma unroll
    for (int t = 0; t < NT; ++t)
      bulk_load(base + s * kStageBytes + t * kTensorBytes, src[t] + elem_off, kTensorBytes,
                &full[s]);
  }
  __device__ __forceinline__ const unsigned char* wait(int64_t k, int* status) {
    const int s = static_cast<int>(k % STAGES);
    if (!dead && !mbar_wait_bounded(&full[s], static_cast<unsigned>(k / STAGES) & 1u)) {
      dead = true;
      if (status != nullptr) atomicExch(status, 1);
    }
    return base + s * kStageBytes;
  }
};

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T, int BLOCK, int VPT, int CS, int STAGES>
__global__ void __launch_bounds__(BLOCK) wide_fwd_kernel(const RowsArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  constexpr int SLICE_VECS = BLOCK * VPT;
  constexpr int NW = BLOCK / 32;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;

  // Programmatic dependent launch: see griddep_wait() below.
  griddep_launch_dependents();
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ WideSmem<BLOCK, CS, STAGES, 2> sm;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned crank = cluster.block_rank();
  const int64_t unit = blockIdx.x / CS, nunits = gridDim.x / CS;
  const int64_t N = a.N, D = a.D;
  const int64_t nb = unit < N ? (N - unit + nunits - 1) / nunits : 0;
  const int64_t slice_off = static_cast<int64_t>(crank) * SLICE_VECS * EPV;
  const float inv_D = 1.0f / static_cast<float>(D);
  const float n_thread = static_cast<float>(VPT * EPV);

  SliceRing<T, SLICE_VECS, STAGES, 1> ring;
  ring.base = ring_mem;
  ring.full = sm.full;
  ring.dead = false;
  const T* const srcs[1] = {static_cast<const T*>(a.x)};
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&sm.full[s], 1);
#pragma unroll
    for (int s = 0; s < kSlots; ++s) mbar_init(&sm.recv[s], 1);
    mbar_init_fence();
    for (int s = 0; s < kSlots && s < nb; ++s) sm.arm(s);
  }
  // every CTA of the cluster has initialised its barriers before anyone sends to them
  cluster_sync_all();
  // this kernel may have been scheduled while its predecessor in the stream was still
  // running: nothing the predecessor may have written is read before this point
  griddep_wait();
  if (tid == 0)
    for (int64_t k = 0; k < STAGES && k < nb; ++k)
      ring.issue(k, srcs, (unit + k * nunits) * D + slice_off);

  // gamma / beta of this thread's columns
  E g[VPT][NE], b[VPT][NE];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int64_t col = slice_off + static_cast<int64_t>(v * BLOCK + tid) * EPV;
    load_param_lanes<EPV>(a.gamma, col, g[v]);
    load_param_lanes<EPV>(a.beta, col, b[v]);
  }

  int phase = 0;
  // (mean, M2) of this CTA's slice of batch k: exact two-pass sums per thread, then Chan
  // merges in a fixed order (lanes by butterfly, warps by index).
  auto local_stats = [&](int64_t k, float& cmean, float& cm2) {
    const P* p = reinterpret_cast<const P*>(ring.wait(k, a.status)) + tid;
    E xv[VPT][NE];
    E acc = M::bcast(0.f);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      unpack<T, EPV>(p[v * BLOCK], xv[v]);
#pragma unroll
      for (int e = 0; e < NE; ++e) acc = M::add(acc, xv[v][e]);
    }
    float mean = M::hsum(acc) * (1.0f / (VPT * EPV));
    const E nm = M::bcast(-mean);
    E q = M::bcast(0.f);
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const E d = M::add(xv[v][e], nm);
        q = M::fma(d, d, q);
      }
    float m2 = M::hsum(q);
    float n = n_thread;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mean, off);
      const float oq = __shfl_xor_sync(0xffffffffu, m2, off);
      chan_equal(mean, m2, om, oq, n);
      n *= 2.f;
    }
    if (lane == 0) {
      sm.warp_part[phase][0][warp] = mean;
      sm.warp_part[phase][1][warp] = m2;
    }
    __syncthreads();
    // the NW warps hold equally many elements: lane l takes warp l's pair and a butterfly
    // of equal-count merges (no division, log2(NW) steps) leaves the CTA's pair in every lane
    cmean = sm.warp_part[phase][0][lane % NW];
    cm2 = sm.warp_part[phase][1][lane % NW];
#pragma unroll
    for (int off = 1; off < NW; off <<= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, cmean, off);
      const float oq = __shfl_xor_sync(0xffffffffu, cm2, off);
      chan_equal(cmean, cm2, om, oq, n);
      n *= 2.f;
    }
    phase ^= 1;
  };
  bool xdead = false;
  float lm = 0.f, lq = 0.f;
  if (nb > 0) {
    local_stats(0, lm, lq);
    sm.send(0, crank, warp, lane, lm, lq);
  }
  for (int64_t j = 0; j < nb; ++j) {
    // the next row's partial is on its way before this row's totals are waited for
    if (j + 1 < nb) {
      local_stats(j + 1, lm, lq);
      sm.send(j + 1, crank, warp, lane, lm, lq);
    }
    sm.receive(j, xdead, a.status);
    const int slot = static_cast<int>(j % kSlots);
    float pm[CS], pq[CS];
#pragma unroll
    for (int r = 0; r < CS; ++r) {
      pm[r] = sm.peer[slot][r][0];
      pq[r] = sm.peer[slot][r][1];
    }
    float n_merge = static_cast<float>(SLICE_VECS * EPV);
#pragma unroll
    for (int span = 1; span < CS; span <<= 1) {
#pragma unroll
      for (int r = 0; r + span < CS; r += 2 * span) chan_equal(pm[r], pq[r], pm[r + span], pq[r + span], n_merge);
      n_merge *= 2.f;
    }
    const float mean = pm[0], m2 = pq[0];
    const float ivar = rsqrtf(fmaf(m2, inv_D, a.eps));
    const int64_t row = unit + j * nunits;
    const P* p = reinterpret_cast<const P*>(ring.base + (j % STAGES) * ring.kStageBytes) + tid;
    P* yp = reinterpret_cast<P*>(static_cast<T*>(a.out) + row * D + slice_off) + tid;
    const E nm = M::bcast(-mean), iv2 = M::bcast(ivar);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      E xv[NE], o[NE];
      unpack<T, EPV>(p[v * BLOCK], xv);
#pragma unroll
      for (int e = 0; e < NE; ++e) o[e] = M::fma(M::mul(M::add(xv[e], nm), iv2), g[v][e], b[v][e]);
      store_stream<T, EPV>(reinterpret_cast<T*>(yp + v * BLOCK), 0, repack<T, EPV>(o));
    }
    if (crank == 0 && tid == 0) {
      a.mean[row] = mean;
      a.ivar[row] = ivar;
    }
    // every thread is done with the stage and the receive slot of row j: refill / re-arm
    __syncthreads();
    if (tid == 0) {
      if (!ring.dead && j + STAGES < nb)
        ring.issue(j + STAGES, srcs, (unit + (j + STAGES) * nunits) * D + slice_off);
      if (j + kSlots < nb) sm.arm(slot);
    }
  }
  // no CTA leaves (and unmaps its shared memory) while a peer may still send to it
  cluster_sync_all();
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
template <typename T, int BLOCK, int VPT, int CS, int STAGES>
__global__ void __launch_bounds__(BLOCK) wide_bwd_kernel(const RowsArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  constexpr int SLICE_VECS = BLOCK * VPT;
  constexpr int NW = BLOCK / 32;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;

  // The column reduction that follows may be scheduled as CTAs of this kernel retire.
  // Programmatic dependent launch: see griddep_wait() below.
  griddep_launch_dependents();
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ WideSmem<BLOCK, CS, STAGES, 2> sm;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned crank = cluster.block_rank();
  const int64_t unit = blockIdx.x / CS, nunits = gridDim.x / CS;
  const int64_t N = a.N, D = a.D;
  const int64_t nb = unit < N ? (N - unit + nunits - 1) / nunits : 0;
  const int64_t slice_off = static_cast<int64_t>(crank) * SLICE_VECS * EPV;
  const float inv_D = 1.0f / static_cast<float>(D);

  SliceRing<T, SLICE_VECS, STAGES, 2> ring;
  ring.base = ring_mem;
  ring.full = sm.full;
  ring.dead = false;
  const T* const srcs[2] = {static_cast<const T*>(a.x), static_cast<const T*>(a.dy)};
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&sm.full[s], 1);
#pragma unroll
    for (int s = 0; s < kSlots; ++s) mbar_init(&sm.recv[s], 1);
    mbar_init_fence();
    for (int s = 0; s < kSlots && s < nb; ++s) sm.arm(s);
  }
  // every CTA of the cluster has initialised its barriers before anyone sends to them
  cluster_sync_all();
  griddep_wait();
  if (tid == 0)
    for (int64_t k = 0; k < STAGES && k < nb; ++k)
      ring.issue(k, srcs, (unit + k * nunits) * D + slice_off);

  E g[VPT][NE], dg[VPT][NE], db[VPT][NE];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int64_t col = slice_off + static_cast<int64_t>(v * BLOCK + tid) * EPV;
    load_param_lanes<EPV>(a.gamma, col, g[v]);
#pragma unroll
    for (int e = 0; e < NE; ++e) dg[v][e] = db[v][e] = M::bcast(0.f);
  }

  // saved statistics: row k's are needed when its slice arrives; they run two rows ahead
  auto stat = [&](const float* p, int64_t k) {
    return k < nb ? __ldg(p + unit + k * nunits) : 0.f;
  };
  float mean_c = 0.f, ivar_c = 0.f;              // row j (dx pass)
  float mean_n = stat(a.mean_in, 0), ivar_n = stat(a.ivar_in, 0);  // row of the next local pass
  float mean_p = stat(a.mean_in, 1), ivar_p = stat(a.ivar_in, 1);  // one further

  int phase = 0;
  // local sums of batch k over this CTA's slice: (sum gy, sum gy * xhat), gy = dy * gamma;
  // also the dgamma / dbeta contributions of the row
  auto local_sums = [&](int64_t k, float mean, float ivar, float& c0, float& c1) {
    const unsigned char* st = ring.wait(k, a.status);
    const P* px = reinterpret_cast<const P*>(st) + tid;
    const P* pd = reinterpret_cast<const P*>(st + ring.kTensorBytes) + tid;
    const E nm = M::bcast(-mean), iv2 = M::bcast(ivar);
    E r0 = M::bcast(0.f), r1 = M::bcast(0.f);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      E xv[NE], gv[NE];
      unpack<T, EPV>(px[v * BLOCK], xv);
      unpack<T, EPV>(pd[v * BLOCK], gv);
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        xv[e] = M::mul(M::add(xv[e], nm), iv2);
        dg[v][e] = M::fma(gv[e], xv[e], dg[v][e]);
        db[v][e] = M::add(db[v][e], gv[e]);
        gv[e] = M::mul(gv[e], g[v][e]);
        r0 = M::add(r0, gv[e]);
        r1 = M::fma(gv[e], xv[e], r1);
      }
    }
    float s0 = M::hsum(r0), s1 = M::hsum(r1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      s0 += __shfl_xor_sync(0xffffffffu, s0, off);
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
    }
    if (lane == 0) {
      sm.warp_part[phase][0][warp] = s0;
      sm.warp_part[phase][1][warp] = s1;
    }
    __syncthreads();
    c0 = sm.warp_part[phase][0][lane % NW];
    c1 = sm.warp_part[phase][1][lane % NW];
#pragma unroll
    for (int off = 1; off < NW; off <<= 1) {
      c0 += __shfl_xor_sync(0xffffffffu, c0, off);
      c1 += __shfl_xor_sync(0xffffffffu, c1, off);
    }
    phase ^= 1;
  };
  bool xdead = false;
  float l0 = 0.f, l1 = 0.f;
  if (nb > 0) {
    local_sums(0, mean_n, ivar_n, l0, l1);
    sm.send(0, crank, warp, lane, l0, l1);
  }
  for (int64_t j = 0; j < nb; ++j) {
    mean_c = mean_n;
    ivar_c = ivar_n;
    mean_n = mean_p;
    ivar_n = ivar_p;
    mean_p = stat(a.mean_in, j + 2);
    ivar_p = stat(a.ivar_in, j + 2);
    if (j + 1 < nb) {
      local_sums(j + 1, mean_n, ivar_n, l0, l1);
      sm.send(j + 1, crank, warp, lane, l0, l1);
    }
    sm.receive(j, xdead, a.status);
    const int slot = static_cast<int>(j % kSlots);
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int r = 0; r < CS; ++r) {
      t0 += sm.peer[slot][r][0];
      t1 += sm.peer[slot][r][1];
    }
    // dx = ivar * (gy - (m0 + xhat * m1)), m0 = t0 / D, m1 = t1 / D; the subtraction comes
    // before the scaling so that rows whose terms cancel exactly give exactly zero
    const int64_t row = unit + j * nunits;
    const unsigned char* st = ring.base + (j % STAGES) * ring.kStageBytes;
    const P* px = reinterpret_cast<const P*>(st) + tid;
    const P* pd = reinterpret_cast<const P*>(st + ring.kTensorBytes) + tid;
    P* op = reinterpret_cast<P*>(static_cast<T*>(a.out) + row * D + slice_off) + tid;
    const E nm = M::bcast(-mean_c), iv2 = M::bcast(ivar_c);
    const E nm0 = M::bcast(-(t0 * inv_D)), nm1 = M::bcast(-(t1 * inv_D));
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      E xv[NE], gv[NE], o[NE];
      unpack<T, EPV>(px[v * BLOCK], xv);
      unpack<T, EPV>(pd[v * BLOCK], gv);
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        xv[e] = M::mul(M::add(xv[e], nm), iv2);
        gv[e] = M::mul(gv[e], g[v][e]);
        o[e] = M::mul(M::add(gv[e], M::fma(xv[e], nm1, nm0)), iv2);
      }
      store_stream<T, EPV>(reinterpret_cast<T*>(op + v * BLOCK), 0, repack<T, EPV>(o));
    }
    __syncthreads();
    if (tid == 0) {
      if (!ring.dead && j + STAGES < nb)
        ring.issue(j + STAGES, srcs, (unit + (j + STAGES) * nunits) * D + slice_off);
      if (j + kSlots < nb) sm.arm(slot);
    }
  }
  cluster_sync_all();

  // one partial row [2][D] per cluster: dgamma then dbeta, this thread's columns
  float* wg = a.ws + (unit * 2 + 0) * D;
  float* wb = a.ws + (unit * 2 + 1) * D;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int64_t col = slice_off + static_cast<int64_t>(v * BLOCK + tid) * EPV;
    store_param_lanes<EPV>(wg, col, dg[v]);
    store_param_lanes<EPV>(wb, col, db[v]);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename T, int BLOCK, int VPT, int CS, int STAGES, bool BWD>
cudaError_t launch_wide(const RowsArgs& a, cudaStream_t stream, bool dry_run, WidePlan* plan) {
  void (*kernel)(const RowsArgs);
  if constexpr (BWD) {
    kernel = wide_bwd_kernel<T, BLOCK, VPT, CS, STAGES>;
  } else {
    kernel = wide_fwd_kernel<T, BLOCK, VPT, CS, STAGES>;
  }
  const size_t ring = static_cast<size_t>(BLOCK) * VPT * 16 * (BWD ? 2 : 1) * STAGES;
  static std::atomic<uint64_t> prepared{0};
  static std::atomic<int> cached_clusters{0};  // per process: every device is the same part
  cudaError_t e = once_per_device(prepared, [&]() -> cudaError_t {
    if (CS > 8) {
      cudaError_t e1 = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e1 != cudaSuccess) return e1;
    }
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(ring));
  });
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(BLOCK, 1, 1);
  cfg.dynamicSmemBytes = ring;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int clusters = cached_clusters.load(std::memory_order_relaxed);
  if (clusters == 0) {
    cfg.gridDim = dim3(static_cast<unsigned>(device_sm_count() * CS), 1, 1);
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      clusters = device_sm_count() / CS > 0 ? device_sm_count() / CS : 1;
    }
    cached_clusters.store(clusters, std::memory_order_relaxed);
  }
  const int64_t use = a.N < clusters ? a.N : clusters;
  plan->grid = static_cast<int>(use) * CS;
  plan->block = BLOCK;
  plan->cluster = CS;
  plan->vpt = VPT;
  plan->stages = STAGES;
  plan->partial_rows = static_cast<int>(use);
  if (dry_run) return cudaSuccess;
  cfg.gridDim = dim3(static_cast<unsigned>(plan->grid), 1, 1);
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

// Shapes: X(index, vectors per row, BLOCK, VPT, CS, STAGES).  A row must fill its shape
// exactly; the first entry for a width is the default, the others can be forced for tuning
// runs (`forced` index).  Chosen so that gamma (and beta, or the two gradient accumulators)
// of a thread's columns fit in registers and the ring holds several rows per SM.
#define NVN_WIDE_FWD(X)                                                              \
  X(0, 4096, 256, 4, 4, 4) X(1, 8192, 512, 4, 4, 4) X(2, 16384, 512, 4, 8, 4)        \
  X(3, 8192, 256, 4, 8, 3)
#define NVN_WIDE_BWD(X)                                                              \
  X(0, 4096, 256, 2, 8, 4) X(1, 8192, 256, 4, 8, 4) X(2, 8192, 512, 2, 8, 4)         \
  X(3, 8192, 512, 4, 4, 3)

template <typename T, bool BWD>
cudaError_t wide_dispatch(int64_t nvec, int forced, const RowsArgs& a, cudaStream_t s, bool dry,
                          WidePlan* plan) {
#define X(I, NVEC, BLOCK, VPT, CS, STAGES) \
  if (forced == I && nvec == NVEC) return launch_wide<T, BLOCK, VPT, CS, STAGES, BWD>(a, s, dry, plan);
  if constexpr (BWD) {
    NVN_WIDE_BWD(X)
  } else {
    NVN_WIDE_FWD(X)
  }
#undef X
#define X(I, NVEC, BLOCK, VPT, CS, STAGES) \
  if (nvec == NVEC) return launch_wide<T, BLOCK, VPT, CS, STAGES, BWD>(a, s, dry, plan);
  if constexpr (BWD) {
    NVN_WIDE_BWD(X)
  } else {
    NVN_WIDE_FWD(X)
  }
#undef X
  return cudaErrorInvalidValue;
}

}  // namespace

bool wide_ok(int64_t nvec, bool bwd) {
#define X(I, NVEC, BLOCK, VPT, CS, STAGES) \
  if (nvec == NVEC) return true;
  if (bwd) {
    NVN_WIDE_BWD(X)
  } else {
    NVN_WIDE_FWD(X)
  }
#undef X
  return false;
}

cudaError_t wide_launch(int dtype, bool bwd, int forced, const RowsArgs& a, cudaStream_t s,
                        bool dry_run, WidePlan* plan) {
  const int64_t nvec = a.D / (dtype == 0 ? 4 : 8);
  switch (dtype) {
    case 0:
      return bwd ? wide_dispatch<float, true>(nvec, forced, a, s, dry_run, plan)
                 : wide_dispatch<float, false>(nvec, forced, a, s, dry_run, plan);
    case 1:
      return bwd ? wide_dispatch<__half, true>(nvec, forced, a, s, dry_run, plan)
                 : wide_dispatch<__half, false>(nvec, forced, a, s, dry_run, plan);
    default:
      return bwd ? wide_dispatch<__nv_bfloat16, true>(nvec, forced, a, s, dry_run, plan)
                 : wide_dispatch<__nv_bfloat16, false>(nvec, forced, a, s, dry_run, plan);
  }
}

}  // namespace nvn
