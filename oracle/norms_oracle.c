/* CPU oracle for the fused LayerNorm / InstanceNorm forward and gradient ops.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product path (atex_b200/) may call
 * this; it exists so tests, the smoke check and the benchmark's cpu_baseline leg
 * have an independent answer to compare against or to time.
 *
 * It is a plain-C restatement of the reference's formulas (the citations are in
 * norms_core.inc).  Parity status: the backward formulas are pinned against the
 * reference's own NumPy gradient functions (layer_norm_grad_np,
 * instance_norm_grad_np) run in the build container, see tests/golden/.  The
 * forward formulas are restated from the reference's CPU functors, which need
 * TensorFlow and Eigen to compile and so could not be executed: forward is
 * "parity unpinned" with respect to the compiled reference.
 *
 * dtype: 0 = float, 1 = IEEE half, 2 = bfloat16 (16-bit types passed as raw
 * uint16_t bit patterns).  gamma, beta and the saved statistics are fp32.
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bits_to_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

static inline float half_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  const uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_f32(sign);
    /* subnormal: man * 2^-24 */
    const float v = (float)man * (1.0f / 16777216.0f);
    return sign ? -v : v;
  }
  if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
  return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

static inline float bf16_to_f32(uint16_t b) { return bits_to_f32((uint32_t)b << 16); }

/* round-to-nearest-even conversions (only used by the fp32 baseline port) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f32_to_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline uint16_t f32_to_half(float f) {
  const uint32_t u = f32_to_bits(f);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536 -> inf (65520 rounds up) */
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
  if (a < 0x33000001u) return (uint16_t)sign; /* below half of the smallest subnormal */
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t hexp;
  if (e < -14) {
    shift = 13 + (-14 - e);
    hexp = 0;
  } else {
    shift = 13;
    hexp = (uint32_t)(e + 15);
  }
  uint32_t r = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (r & 1u))) r += 1;
  uint32_t out;
  if (hexp == 0) {
    out = r; /* may carry into exponent 1, which is the correct encoding */
  } else {
    out = ((hexp - 1) << 10) + r; /* r includes the hidden bit (0x400) */
  }
  return (uint16_t)(sign | out);
}

static inline float load_elem(int dtype, const void* p, int64_t i) {
  switch (dtype) {
    case 0:
      return ((const float*)p)[i];
    case 1:
      return half_to_f32(((const uint16_t*)p)[i]);
    default:
      return bf16_to_f32(((const uint16_t*)p)[i]);
  }
}

static inline void store_elem_t(int dtype, void* p, int64_t i, float v) {
  switch (dtype) {
    case 0:
      ((float*)p)[i] = v;
      break;
    case 1:
      ((uint16_t*)p)[i] = f32_to_half(v);
      break;
    default:
      ((uint16_t*)p)[i] = f32_to_bf16(v);
      break;
  }
}

/* checker: float64 accumulation, float64 outputs */
#define ACC double
#define SUFFIX 64
#define SQRT sqrt
#define STORE_OUT(dtype, p, i, v) (((double*)(p))[i] = (v))
#include "norms_core.inc"
#undef ACC
#undef SUFFIX
#undef SQRT
#undef STORE_OUT

/* baseline port: fp32 arithmetic and outputs of type T, like the reference's CPU functors */
#define ACC float
#define SUFFIX 32
#define SQRT sqrtf
#define STORE_OUT(dtype, p, i, v) store_elem_t(dtype, p, i, v)
#include "norms_core.inc"
#undef ACC
#undef SUFFIX
#undef SQRT
#undef STORE_OUT

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timed baseline that is meant to use
 * every host core sets the team size explicitly.  Returns the team size now in effect. */
int oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* exposed for the oracle's own unit tests */
float oracle_half_to_f32(uint16_t h) { return half_to_f32(h); }
uint16_t oracle_f32_to_half(float f) { return f32_to_half(f); }
uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16(f); }
