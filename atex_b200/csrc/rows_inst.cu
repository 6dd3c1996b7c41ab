// Instantiates the row-cached kernels for one (dtype, direction) pair.  Compiled
// six times with -DNVN_T={0,1,2} (f32, f16, bf16) and -DNVN_BWD={0,1} so the
// instantiations build in parallel.
#include "rows_kernels.cuh"

#if NVN_T == 0
using T = float;
#define NVN_TNAME f32
#elif NVN_T == 1
using T = __half;
#define NVN_TNAME f16
#else
using T = __nv_bfloat16;
#define NVN_TNAME bf16
#endif

#if NVN_BWD
#define NVN_DIR bwd
#else
#define NVN_DIR fwd
#endif

#define NVN_CAT3_(a, b, c) a##_##b##_##c
#define NVN_CAT3(a, b, c) NVN_CAT3_(a, b, c)

namespace nvn {

template <int EPV>
static cudaError_t coarse(bool row_affine, int shape, const RowsArgs& a, cudaStream_t s,
                          bool dry_run, RowsPlan* plan) {
  constexpr bool BWD = NVN_BWD != 0;
  return row_affine ? launch_rows_coarse<T, EPV, true, BWD>(shape, a, s, dry_run, plan)
                    : launch_rows_coarse<T, EPV, false, BWD>(shape, a, s, dry_run, plan);
}

cudaError_t NVN_CAT3(rows, NVN_TNAME, NVN_DIR)(bool row_affine, int epv, int shape,
                                                const RowsArgs& a, cudaStream_t s, bool dry_run,
                                                RowsPlan* plan) {
  constexpr bool BWD = NVN_BWD != 0;
  constexpr int V = VecTraits<T>::kFull;
  if (epv == V) {
    return row_affine ? launch_rows_vec<T, true, BWD>(shape, a, s, dry_run, plan)
                      : launch_rows_vec<T, false, BWD>(shape, a, s, dry_run, plan);
  }
  if (epv == 1) return coarse<1>(row_affine, shape, a, s, dry_run, plan);
  if (epv == 2) return coarse<2>(row_affine, shape, a, s, dry_run, plan);
  if constexpr (V == 8) {
    if (epv == 4) return coarse<4>(row_affine, shape, a, s, dry_run, plan);
  }
  return cudaErrorInvalidValue;
}

}  // namespace nvn
