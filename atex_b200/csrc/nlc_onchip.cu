// On-chip InstanceNorm kernels for the channels-last layout (x[n, d, c]) when one batch item
// fits in shared memory.
//
// In this layout an item is one contiguous block of D*C elements.  A CTA copies the whole item
// into shared memory with one bulk asynchronous copy (TMA, cp.async.bulk + mbarrier), walks it
// two (backward) or three (forward) times and writes the result: x (and dy) are read from HBM
// exactly once, in one launch.  Thread t owns the 128-bit vectors t, t + 256, ... of the item;
// because the channel vectors per voxel (C / EPV) divide the CTA size, all of a thread's
// vectors belong to the same EPV channels, so gamma / beta and the statistics of those
// channels live in registers.  Per-channel sums: xor shuffles over the lanes of a warp that
// share a channel vector, one deposit per warp and channel in shared memory, then a sum over
// the warps in a fixed order (=> bit-identical from run to run).
// Forward statistics are exact two-pass (mean, then centred squares).
//
// Replaces InstanceNormBlockSMemChnlLastImpl (atex/nv_norms/cc/kernels/
// fused_instance_norm_op.cu:1065-1165) for the forward pass and, for items that fit, the
// three-kernel channels-last backward (:666-730, :103-146, :744-763).  Larger items take the
// two-phase kernels of twophase.cu.
#include "nvn_common.cuh"
#include "nvn_host.h"

#include <atomic>

namespace nvn {

namespace {

constexpr int kBlock = 256;
constexpr size_t kSlabBudget = 88 * 1024;  // dynamic shared memory per CTA for two CTAs per SM
constexpr size_t kSlabMax = 192 * 1024;    // largest slab: one CTA per SM
constexpr int kMaxChannels = 512;  // bounds the per-channel arrays in shared memory

// EPV consecutive floats of a shared-memory array as math lanes
template <int EPV>
__device__ __forceinline__ void lanes_from_smem(const float* p,
                                                typename MathSel<EPV>::M::E (&out)[MathSel<EPV>::NE]) {
  if constexpr (EPV == 1) {
    out[0] = p[0];
  } else {
#pragma unroll
    for (int i = 0; i < EPV / 2; ++i) out[i] = make_float2(p[2 * i], p[2 * i + 1]);
  }
}

struct NlcOnchipArgs {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  const float* mean_in;  // backward: saved statistics [N][C]
  const float* ivar_in;
  void* out;
  float* mean;  // forward outputs [N][C]
  float* ivar;
  float* colpart;  // backward: [N][2][C] per-item (dgamma, dbeta) contributions
  int64_t N, C, D;
  float eps;
  int* status;
};

// Per-channel sum over the CTA of every thread's EPV partial sums `acc`; the total of channel
// c lands in tot[c] (valid after the trailing barrier).  `scratch` holds kBlock * EPV floats.
// The cv threads-per-voxel pattern repeats inside a warp when cv <= 16, so the lanes that
// share a channel vector are first summed with xor shuffles; each warp then deposits one
// value per channel and channel c is summed over the warps (or, for cv >= 32, over the
// kBlock / cv threads that hold it), always in the same order.
template <int EPV>
__device__ __forceinline__ void channel_totals(
    typename MathSel<EPV>::M::E (&acc)[MathSel<EPV>::NE], float* scratch, float* tot, int C,
    int cv) {
  using M = typename MathSel<EPV>::M;
  constexpr int NE = MathSel<EPV>::NE;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  if (cv <= 32) {
    for (int off = 16; off >= cv; off >>= 1) {
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        if constexpr (EPV == 1) {
          acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
        } else {
          acc[e].x += __shfl_xor_sync(0xffffffffu, acc[e].x, off);
          acc[e].y += __shfl_xor_sync(0xffffffffu, acc[e].y, off);
        }
      }
    }
    if (lane < cv) store_param_lanes<EPV>(scratch + warp * C + lane * EPV, 0, acc);
    __syncthreads();
    for (int c = t; c < C; c += kBlock) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kBlock / 32; ++w) s += scratch[w * C + c];
      tot[c] = s;
    }
  } else {
    store_param_lanes<EPV>(scratch + t * EPV, 0, acc);
    __syncthreads();
    const int holders = kBlock / cv;
    for (int c = t; c < C; c += kBlock) {
      const int v = c / EPV, e = c % EPV;
      float s = 0.f;
      for (int k = 0; k < holders; ++k) s += scratch[(v + cv * k) * EPV + e];
      tot[c] = s;
    }
  }
  __syncthreads();
}

// STAGES = 2: the next item is copied into the other half of the slab while this one is
// processed (items of at most half the slab budget); STAGES = 1: one item at a time.
template <typename T, bool BWD, int STAGES>
__global__ void __launch_bounds__(kBlock, BWD ? 2 : 3) nlc_onchip_kernel(const NlcOnchipArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;
  constexpr int NT = BWD ? 2 : 1;

  extern __shared__ __align__(128) unsigned char slab_mem[];  // [STAGES][NT][item bytes]
  __shared__ __align__(8) uint64_t bars[STAGES];
  __shared__ __align__(16) float red[NT][kBlock][EPV];
  __shared__ __align__(16) float tot[2][kMaxChannels];

  const int t = threadIdx.x;
  const int C = static_cast<int>(a.C);
  const int cv = C / EPV;  // channel vectors per voxel; divides kBlock
  const int my_cv = t % cv;
  const int64_t item_elems = a.D * a.C;
  const int nvec = static_cast<int>(item_elems / EPV);
  const unsigned item_bytes = static_cast<unsigned>(item_elems * sizeof(T));
  const float inv_D = 1.0f / static_cast<float>(a.D);
  const unsigned stage_bytes = item_bytes * NT;

  // parameters of this thread's EPV channels
  E g[NE], be[NE];
  load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(my_cv) * EPV, g);
  if constexpr (!BWD) load_param_lanes<EPV>(a.beta, static_cast<int64_t>(my_cv) * EPV, be);

  if (t == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  bool dead = false;  // a bounded wait gave up: stop copying and waiting, finish the loop
  auto issue = [&](int64_t n, int stage) {
    unsigned char* dst = slab_mem + static_cast<size_t>(stage) * stage_bytes;
    mbar_expect_tx(&bars[stage], stage_bytes);
    bulk_load(dst, static_cast<const T*>(a.x) + n * item_elems, item_bytes, &bars[stage]);
    if constexpr (BWD)
      bulk_load(dst + item_bytes, static_cast<const T*>(a.dy) + n * item_elems, item_bytes,
                &bars[stage]);
  };
  if (STAGES == 2 && t == 0 && blockIdx.x < a.N) issue(blockIdx.x, 0);

  unsigned use = 0;
  for (int64_t n = blockIdx.x; n < a.N; n += gridDim.x, ++use) {
    const int stage = STAGES == 2 ? static_cast<int>(use & 1u) : 0;
    if (t == 0 && !dead) {
      if constexpr (STAGES == 2) {
        // the other stage was released by the barrier that ended the previous iteration
        if (n + gridDim.x < a.N) issue(n + gridDim.x, stage ^ 1);
      } else {
        issue(n, 0);
      }
    }
    const unsigned parity = STAGES == 2 ? ((use >> 1) & 1u) : (use & 1u);
    const bool ok = dead ? true : mbar_wait_bounded(&bars[stage], parity);
    if (__syncthreads_or(!ok) && !dead) {
      dead = true;
      if (t == 0 && a.status != nullptr) atomicExch(a.status, 1);
    }
    const P* sx = reinterpret_cast<const P*>(slab_mem + static_cast<size_t>(stage) * stage_bytes);
    const P* sdy = reinterpret_cast<const P*>(slab_mem + static_cast<size_t>(stage) * stage_bytes +
                                              item_bytes);

    if constexpr (!BWD) {
      // pass 1: per-channel sums
      E acc[NE];
#pragma unroll
      for (int e = 0; e < NE; ++e) acc[e] = M::bcast(0.f);
      for (int i = t; i < nvec; i += kBlock) {
        E xe[NE];
        unpack<T, EPV>(sx[i], xe);
#pragma unroll
        for (int e = 0; e < NE; ++e) acc[e] = M::add(acc[e], xe[e]);
      }
      channel_totals<EPV>(acc, &red[0][0][0], tot[0], C, cv);
      E mean[NE];
      lanes_from_smem<EPV>(&tot[0][my_cv * EPV], mean);
#pragma unroll
      for (int e = 0; e < NE; ++e) mean[e] = M::mul(mean[e], M::bcast(-inv_D));  // -mean
      // pass 2: centred squares
#pragma unroll
      for (int e = 0; e < NE; ++e) acc[e] = M::bcast(0.f);
      for (int i = t; i < nvec; i += kBlock) {
        E xe[NE];
        unpack<T, EPV>(sx[i], xe);
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          const E d = M::add(xe[e], mean[e]);
          acc[e] = M::fma(d, d, acc[e]);
        }
      }
      channel_totals<EPV>(acc, &red[0][0][0], tot[1], C, cv);
      // per-channel results: inverse std in tot[1], outputs to global
      for (int c = t; c < C; c += kBlock) {
        const float m = tot[0][c] * inv_D;
        const float iv = rsqrtf(fmaf(tot[1][c], inv_D, a.eps));
        a.mean[n * C + c] = m;
        a.ivar[n * C + c] = iv;
        tot[1][c] = iv;
      }
      __syncthreads();
      E sc[NE];
      lanes_from_smem<EPV>(&tot[1][my_cv * EPV], sc);
#pragma unroll
      for (int e = 0; e < NE; ++e) sc[e] = M::mul(sc[e], g[e]);  // ivar * gamma
      // pass 3: y = (x - mean) * ivar * gamma + beta
      P* yp = reinterpret_cast<P*>(static_cast<T*>(a.out) + n * item_elems);
      for (int i = t; i < nvec; i += kBlock) {
        E xe[NE], o[NE];
        unpack<T, EPV>(sx[i], xe);
#pragma unroll
        for (int e = 0; e < NE; ++e) o[e] = M::fma(M::add(xe[e], mean[e]), sc[e], be[e]);
        store_stream<T, EPV>(reinterpret_cast<T*>(yp + i), 0, repack<T, EPV>(o));
      }
    } else {
      // saved statistics of this thread's channels
      E nm[NE], iv[NE];
      load_param_lanes<EPV>(a.mean_in + n * C, static_cast<int64_t>(my_cv) * EPV, nm);
      load_param_lanes<EPV>(a.ivar_in + n * C, static_cast<int64_t>(my_cv) * EPV, iv);
#pragma unroll
      for (int e = 0; e < NE; ++e) nm[e] = M::mul(nm[e], M::bcast(-1.f));
      // pass 1: s1 = sum dy, s2 = sum dy * xhat per channel
      E s1[NE], s2[NE];
#pragma unroll
      for (int e = 0; e < NE; ++e) s1[e] = s2[e] = M::bcast(0.f);
      for (int i = t; i < nvec; i += kBlock) {
        E xe[NE], de[NE];
        unpack<T, EPV>(sx[i], xe);
        unpack<T, EPV>(sdy[i], de);
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          const E xh = M::mul(M::add(xe[e], nm[e]), iv[e]);
          s1[e] = M::add(s1[e], de[e]);
          s2[e] = M::fma(de[e], xh, s2[e]);
        }
      }
      channel_totals<EPV>(s1, &red[0][0][0], tot[0], C, cv);
      channel_totals<EPV>(s2, &red[1][0][0], tot[1], C, cv);
      // per-item contributions to dgamma (sum dy * xhat) and dbeta (sum dy): [n][2][C]
      for (int c = t; c < C; c += kBlock) {
        a.colpart[(n * 2 + 0) * C + c] = tot[1][c];
        a.colpart[(n * 2 + 1) * C + c] = tot[0][c];
      }
      E m0[NE], m1[NE], sc[NE];
      lanes_from_smem<EPV>(&tot[0][my_cv * EPV], m0);
      lanes_from_smem<EPV>(&tot[1][my_cv * EPV], m1);
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        m0[e] = M::mul(m0[e], M::bcast(-inv_D));
        m1[e] = M::mul(m1[e], M::bcast(-inv_D));
        sc[e] = M::mul(iv[e], g[e]);
      }
      // pass 2: dx = gamma * ivar * (dy - (s1 + xhat * s2) / D)
      P* op = reinterpret_cast<P*>(static_cast<T*>(a.out) + n * item_elems);
      for (int i = t; i < nvec; i += kBlock) {
        E xe[NE], de[NE], o[NE];
        unpack<T, EPV>(sx[i], xe);
        unpack<T, EPV>(sdy[i], de);
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          const E xh = M::mul(M::add(xe[e], nm[e]), iv[e]);
          o[e] = M::mul(M::add(de[e], M::fma(xh, m1[e], m0[e])), sc[e]);
        }
        store_stream<T, EPV>(reinterpret_cast<T*>(op + i), 0, repack<T, EPV>(o));
      }
    }
    // every thread is done with the slab and the reduction arrays before the next item
    __syncthreads();
  }
}

template <typename T, bool BWD, int STAGES>
cudaError_t launch_s(NlcOnchipArgs& a, size_t slab_bytes, cudaStream_t s) {
  auto kernel = nlc_onchip_kernel<T, BWD, STAGES>;
  const size_t smem = slab_bytes * STAGES;
  // The opt-in to large dynamic shared memory is set once per device; the occupancy for the
  // last slab size seen is cached per process (every device this library runs on is the
  // same part).
  static std::atomic<uint64_t> prepared{0};
  static std::atomic<int64_t> cached{0};  // (smem << 8) | CTAs per SM
  {
    const cudaError_t e = once_per_device(prepared, [&]() -> cudaError_t {
      return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(kSlabMax));
    });
    if (e != cudaSuccess) return e;
  }
  int per_sm = 0;
  const int64_t c = cached.load(std::memory_order_relaxed);
  if (c != 0 && static_cast<size_t>(c >> 8) == smem) {
    per_sm = static_cast<int>(c & 0xff);
  } else {
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) per_sm = 1;
    cached.store((static_cast<int64_t>(smem) << 8) | per_sm, std::memory_order_relaxed);
  }
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * per_sm;
  const unsigned grid = static_cast<unsigned>(a.N < resident ? a.N : resident);
  count_launch();
  kernel<<<grid, kBlock, smem, s>>>(a);
  return cudaGetLastError();
}

template <typename T, bool BWD>
cudaError_t launch_t(NlcOnchipArgs& a, size_t slab_bytes, cudaStream_t s) {
  // two stages when both fit the budget and there is a next item to prefetch
  if (2 * slab_bytes <= kSlabBudget && a.N > device_sm_count())
    return launch_s<T, BWD, 2>(a, slab_bytes, s);
  return launch_s<T, BWD, 1>(a, slab_bytes, s);
}

}  // namespace

// Items of at most this many bytes (x, plus dy in the backward pass) are handled on chip.
constexpr size_t kNlcOnchipMaxSlab = kSlabMax;

bool nlc_onchip_ok(int dtype, bool bwd, int64_t C, int64_t D) {
  const int epv = dtype == 0 ? 4 : 8;
  const size_t es = dtype == 0 ? 4 : 2;
  if (C % epv != 0) return false;
  const int64_t cv = C / epv;
  if (C > kMaxChannels || cv > kBlock || kBlock % cv != 0) return false;
  const size_t slab = static_cast<size_t>(D) * C * es * (bwd ? 2 : 1);
  return slab <= kNlcOnchipMaxSlab;
}

cudaError_t nlc_onchip_launch(int dtype, bool bwd, const void* dy, const void* x,
                              const float* gamma, const float* beta, const float* mean_in,
                              const float* ivar_in, int64_t N, int64_t C, int64_t D, float eps,
                              void* out, float* mean, float* ivar, float* colpart, int* status,
                              cudaStream_t s) {
  NlcOnchipArgs a = {};
  a.x = x;
  a.dy = dy;
  a.gamma = gamma;
  a.beta = beta;
  a.mean_in = mean_in;
  a.ivar_in = ivar_in;
  a.out = out;
  a.mean = mean;
  a.ivar = ivar;
  a.colpart = colpart;
  a.N = N;
  a.C = C;
  a.D = D;
  a.eps = eps;
  a.status = status;
  const size_t es = dtype == 0 ? 4 : 2;
  const size_t slab = static_cast<size_t>(D) * C * es * (bwd ? 2 : 1);
  if (dtype == 0) return bwd ? launch_t<float, true>(a, slab, s) : launch_t<float, false>(a, slab, s);
  if (dtype == 1) return bwd ? launch_t<__half, true>(a, slab, s) : launch_t<__half, false>(a, slab, s);
  return bwd ? launch_t<__nv_bfloat16, true>(a, slab, s) : launch_t<__nv_bfloat16, false>(a, slab, s);
}

}  // namespace nvn
