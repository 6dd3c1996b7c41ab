// LayerNorm forward fused with the residual add in front of it: s = T(x + res) is written
// out and normalised in the same pass, so the sum is never re-read (4 tensor passes of
// traffic instead of 5 for an add kernel followed by the norm).  Instantiates
// rows_fwd_kernel<..., RES = true> for one dtype; compiled three times with -DNVN_T={0,1,2}.
//
// The reference has no such op: its Keras wrapper calls the bare norm
// (atex/nv_norms/python/ops/nv_norm_ops.py:85-99) and the add runs as a separate TensorFlow
// kernel.  Widths beyond the table, or buffers that rule out 128-bit accesses, are served by
// residual_add_kernel + the plain forward (nvnorms_api.cu).
#include "rows_kernels.cuh"

#if NVN_T == 0
using T = float;
#define NVN_RES_NAME rows_res_f32
#define NVN_ADD_NAME residual_add_f32
#elif NVN_T == 1
using T = __half;
#define NVN_RES_NAME rows_res_f16
#define NVN_ADD_NAME residual_add_f16
#else
using T = __nv_bfloat16;
#define NVN_RES_NAME rows_res_bf16
#define NVN_ADD_NAME residual_add_bf16
#endif

namespace nvn {

// X(TPR, VPT, RB, PR, MINB): rows of up to TPR * VPT vectors; the first sufficient entry
// is used.  All with register prefetch of the next row batch (x and res).
#define NVN_RES_SHAPES(X)                                                                  \
  X(4, 1, 4, 1, 0) X(8, 1, 4, 1, 0) X(8, 2, 4, 1, 0) X(32, 1, 4, 1, 0) X(32, 2, 2, 1, 0)  \
  X(32, 4, 2, 1, 0) X(128, 2, 1, 1, 128) X(128, 4, 1, 1, 0) X(256, 4, 1, 1, 0)            \
  X(512, 4, 1, 1, 0) X(512, 8, 1, 0, 0)

template <int TPR, int VPT, int RB, bool PR, int MINB, bool EXACT>
static cudaError_t launch_res(const RowsResArgs& a, cudaStream_t stream) {
  constexpr int EPV = VecTraits<T>::kFull;
  constexpr int BLOCK = RowBlock<TPR, MINB>::kBlock;
  constexpr int RPC = RowBlock<TPR, MINB>::kRowsPerCta;
  auto kernel = rows_fwd_kernel<T, EPV, TPR, VPT, 1, RB, PR, MINB, 1, EXACT, false, true>;
  static std::atomic<int> cached_units{0};   // per process: every device is the same part
  int units = cached_units.load(std::memory_order_relaxed);
  if (units == 0) {
    units = resident_units(kernel, BLOCK, 1, 0);
    cached_units.store(units, std::memory_order_relaxed);
  }
  const int64_t need = (a.N + RPC * RB - 1) / (RPC * RB);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(need < units ? need : units), 1, 1);
  cfg.blockDim = dim3(BLOCK, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

cudaError_t NVN_RES_NAME(const RowsResArgs& a, cudaStream_t s) {
  constexpr int EPV = VecTraits<T>::kFull;
  const int64_t nvec = a.D / EPV;
#define X(TPR, VPT, RB, PR, MINB)                                                        \
  if (nvec <= static_cast<int64_t>(TPR) * VPT)                                            \
    return nvec == static_cast<int64_t>(TPR) * VPT                                        \
               ? launch_res<TPR, VPT, RB, PR != 0, MINB, true>(a, s)                      \
               : launch_res<TPR, VPT, RB, PR != 0, MINB, false>(a, s);
  NVN_RES_SHAPES(X)
#undef X
  return cudaErrorInvalidValue;
}

// s = T(x + res), element-wise, any count and alignment (the fallback's first step)
__global__ void __launch_bounds__(256) residual_add_kernel(const T* __restrict__ x,
                                                           const T* __restrict__ res,
                                                           T* __restrict__ out, int64_t count) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += step)
    out[i] = Cvt<T>::from_f32(Cvt<T>::to_f32(x[i]) + Cvt<T>::to_f32(res[i]));
}

cudaError_t NVN_ADD_NAME(const void* x, const void* res, void* out, int64_t count, cudaStream_t s) {
  int64_t blocks = (count + 255) / 256;
  const int64_t most = static_cast<int64_t>(device_sm_count()) * 16;
  if (blocks > most) blocks = most;
  count_launch();
  residual_add_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      static_cast<const T*>(x), static_cast<const T*>(res), static_cast<T*>(out), count);
  return cudaGetLastError();
}

}  // namespace nvn
