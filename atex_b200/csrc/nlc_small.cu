// Warp-per-item InstanceNorm kernels for small channels-last items (x[n, d, c], C <= 32,
// D * C <= 4096 elements), any dtype, any alignment, any C.
//
// An item is one contiguous block of D*C elements.  A warp owns an item: in every step its
// first VL*C lanes (VL = 32 / C voxels) read VL consecutive voxels, so lane l always sees
// channel l % C and the loads are contiguous.  Per-lane sums are combined over the VL lanes
// of a channel with shuffles in a fixed order.  The item is read from HBM once; the second
// and third pass hit L1.  Eight items per CTA, one launch.
//
// Covers the small end of InstanceNormBlockSMemChnlLastImpl and of the thread-per-channel
// kernels (atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:1065-1165, :52-69, :666-730),
// where a CTA per item (or three launches over tiny CTAs) leaves most threads idle.
#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

namespace {

constexpr int kWarpsPerCta = 8;

struct NlcSmallArgs {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  const float* mean_in;
  const float* ivar_in;
  void* out;
  float* mean;
  float* ivar;
  float* colpart;  // backward: [N][2][C]
  int64_t N;
  int C, D;
  float eps;
};

// Sum of v over the lanes that hold channel c (lanes c, c + C, ...), same value and same order
// of additions in every lane.
__device__ __forceinline__ float channel_sum(float v, int c, int C, int VL) {
  float s = 0.f;
  for (int k = 0; k < VL; ++k) s += __shfl_sync(0xffffffffu, v, c + k * C);
  return s;
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(kWarpsPerCta * 32) nlc_small_kernel(const NlcSmallArgs a) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int C = a.C, D = a.D;
  const int VL = 32 / C;          // voxels per step
  const int span = VL * C;        // active lanes = elements per step
  const bool active = lane < span;
  const int c = lane % C;
  const int L = D * C;
  const float inv_D = 1.0f / static_cast<float>(D);
  const float g = __ldg(a.gamma + c);
  const float be = BWD ? 0.f : __ldg(a.beta + c);
  const int64_t item0 = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + warp;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarpsPerCta;
  for (int64_t n = item0; n < a.N; n += stride) {
    const T* x = static_cast<const T*>(a.x) + n * L;
    T* out = static_cast<T*>(a.out) + n * L;
    if constexpr (!BWD) {
      float s = 0.f;
      if (active)
        for (int e = lane; e < L; e += span) s += Cvt<T>::to_f32(x[e]);
      const float mean = channel_sum(s, c, C, VL) * inv_D;
      float q = 0.f;
      if (active)
        for (int e = lane; e < L; e += span) {
          const float d = Cvt<T>::to_f32(x[e]) - mean;
          q = fmaf(d, d, q);
        }
      const float ivar = rsqrtf(fmaf(channel_sum(q, c, C, VL), inv_D, a.eps));
      if (lane < C) {
        a.mean[n * C + c] = mean;
        a.ivar[n * C + c] = ivar;
      }
      const float sc = ivar * g;
      if (active)
        for (int e = lane; e < L; e += span)
          out[e] = Cvt<T>::from_f32(fmaf(Cvt<T>::to_f32(x[e]) - mean, sc, be));
    } else {
      const T* dy = static_cast<const T*>(a.dy) + n * L;
      const float mean = __ldg(a.mean_in + n * C + c);
      const float ivar = __ldg(a.ivar_in + n * C + c);
      float s1 = 0.f, s2 = 0.f;
      if (active)
        for (int e = lane; e < L; e += span) {
          const float d = Cvt<T>::to_f32(dy[e]);
          const float xh = (Cvt<T>::to_f32(x[e]) - mean) * ivar;
          s1 += d;
          s2 = fmaf(d, xh, s2);
        }
      s1 = channel_sum(s1, c, C, VL);
      s2 = channel_sum(s2, c, C, VL);
      if (lane < C) {
        a.colpart[(n * 2 + 0) * C + c] = s2;  // dgamma contribution
        a.colpart[(n * 2 + 1) * C + c] = s1;  // dbeta contribution
      }
      // dx = gamma * ivar * (dy - (s1 + xhat * s2) / D)
      const float m0 = -s1 * inv_D, m1 = -s2 * inv_D, sc = ivar * g;
      if (active)
        for (int e = lane; e < L; e += span) {
          const float d = Cvt<T>::to_f32(dy[e]);
          const float xh = (Cvt<T>::to_f32(x[e]) - mean) * ivar;
          out[e] = Cvt<T>::from_f32((d + fmaf(xh, m1, m0)) * sc);
        }
    }
  }
}

template <typename T, bool BWD>
cudaError_t launch_t(const NlcSmallArgs& a, cudaStream_t s) {
  const int64_t ctas = (a.N + kWarpsPerCta - 1) / kWarpsPerCta;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;  // 2048 threads per SM
  count_launch();
  nlc_small_kernel<T, BWD><<<static_cast<unsigned>(ctas < cap ? ctas : cap), kWarpsPerCta * 32, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace

bool nlc_small_ok(int64_t C, int64_t D) { return C >= 1 && C <= 32 && D * C <= 4096; }

cudaError_t nlc_small_launch(int dtype, bool bwd, const void* dy, const void* x,
                             const float* gamma, const float* beta, const float* mean_in,
                             const float* ivar_in, int64_t N, int64_t C, int64_t D, float eps,
                             void* out, float* mean, float* ivar, float* colpart, cudaStream_t s) {
  NlcSmallArgs a = {};
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
  a.C = static_cast<int>(C);
  a.D = static_cast<int>(D);
  a.eps = eps;
  if (dtype == 0) return bwd ? launch_t<float, true>(a, s) : launch_t<float, false>(a, s);
  if (dtype == 1) return bwd ? launch_t<__half, true>(a, s) : launch_t<__half, false>(a, s);
  return bwd ? launch_t<__nv_bfloat16, true>(a, s) : launch_t<__nv_bfloat16, false>(a, s);
}

}  // namespace nvn
