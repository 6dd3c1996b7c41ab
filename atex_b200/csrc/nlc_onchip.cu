// On-chip InstanceNorm kernels for the channels-last layout (x[n, d, c]) when one batch item
// fits in shared memory.
//
// In this layout an item is one contiguous block of D*C elements.  A CTA copies the whole item
// into shared memory with one bulk asynchronous copy (TMA, cp.async.bulk + mbarrier), walks it
// two (backward) or three (forward) times and writes the result: x (and dy) are read from HBM
// exactly once, in one launch.  Thread t owns the 128-bit vectors t, t + 256, ... of the item;
// because the channel vectors per voxel (C / EPV) divide the CTA size, all of a thread's
// vectors belong to the same EPV channels, so gamma / beta and the statistics of those
// channels live in registers.  Per-channel sums go through a [256][EPV] shared-memory array:
// every thread deposits its partial sums, then channel c is summed over the 256 * EPV / C
// threads that hold it, in thread order (fixed order => bit-identical from run to run).
// Forward statistics are exact two-pass (mean, then centred squares).
//
// Replaces InstanceNormBlockSMemChnlLastImpl (atex/nv_norms/cc/kernels/
// fused_instance_norm_op.cu:1065-1165) for the forward pass and, for items that fit, the
// three-kernel channels-last backward (:666-730, :103-146, :744-763).  Larger items take the
// two-phase kernels of twophase.cu.
#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

namespace {

constexpr int kBlock = 256;
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

// Sum, per channel, of the per-thread partials in red[256][EPV]; the result for channel c
// lands in tot[c].  Threads cooperate: thread t handles channels t, t + 256, ...
template <int EPV>
__device__ __forceinline__ void channel_totals(const float (*red)[EPV], float* tot, int C, int cv) {
  const int holders = kBlock / cv;  // threads that hold a given channel vector
  for (int c = threadIdx.x; c < C; c += kBlock) {
    const int v = c / EPV, e = c % EPV;
    float s = 0.f;
    for (int k = 0; k < holders; ++k) s += red[v + cv * k][e];
    tot[c] = s;
  }
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(kBlock) nlc_onchip_kernel(const NlcOnchipArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;
  constexpr int NT = BWD ? 2 : 1;

  extern __shared__ __align__(128) unsigned char slab[];  // [NT][item bytes]
  __shared__ __align__(8) uint64_t bar;
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
  const P* sx = reinterpret_cast<const P*>(slab);
  const P* sdy = reinterpret_cast<const P*>(slab + item_bytes);

  // parameters of this thread's EPV channels
  E g[NE], be[NE];
  load_param_lanes<EPV>(a.gamma, static_cast<int64_t>(my_cv) * EPV, g);
  if constexpr (!BWD) load_param_lanes<EPV>(a.beta, static_cast<int64_t>(my_cv) * EPV, be);

  if (t == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  __syncthreads();
  bool dead = false;  // a bounded wait gave up: stop copying and waiting, finish the loop

  unsigned use = 0;
  for (int64_t n = blockIdx.x; n < a.N; n += gridDim.x, ++use) {
    if (t == 0 && !dead) {
      mbar_expect_tx(&bar, item_bytes * NT);
      bulk_load(slab, static_cast<const T*>(a.x) + n * item_elems, item_bytes, &bar);
      if constexpr (BWD)
        bulk_load(slab + item_bytes, static_cast<const T*>(a.dy) + n * item_elems, item_bytes, &bar);
    }
    const bool ok = dead ? true : mbar_wait_bounded(&bar, use & 1u);
    if (__syncthreads_or(!ok) && !dead) {
      dead = true;
      if (t == 0 && a.status != nullptr) atomicExch(a.status, 1);
    }

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
      store_param_lanes<EPV>(&red[0][t][0], 0, acc);
      __syncthreads();
      channel_totals<EPV>(red[0], tot[0], C, cv);
      __syncthreads();
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
      store_param_lanes<EPV>(&red[0][t][0], 0, acc);
      __syncthreads();
      channel_totals<EPV>(red[0], tot[1], C, cv);
      __syncthreads();
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
      store_param_lanes<EPV>(&red[0][t][0], 0, s1);
      store_param_lanes<EPV>(&red[1][t][0], 0, s2);
      __syncthreads();
      channel_totals<EPV>(red[0], tot[0], C, cv);
      channel_totals<EPV>(red[1], tot[1], C, cv);
      __syncthreads();
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

template <typename T, bool BWD>
cudaError_t launch_t(NlcOnchipArgs& a, size_t slab_bytes, cudaStream_t s) {
  auto kernel = nlc_onchip_kernel<T, BWD>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(slab_bytes));
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, slab_bytes);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) per_sm = 1;
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * per_sm;
  const unsigned grid = static_cast<unsigned>(a.N < resident ? a.N : resident);
  count_launch();
  kernel<<<grid, kBlock, slab_bytes, s>>>(a);
  return cudaGetLastError();
}

}  // namespace

// Items of at most this many bytes (x, plus dy in the backward pass) are handled on chip.
constexpr size_t kNlcOnchipMaxSlab = 88 * 1024;  // two CTAs per SM

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
