// Device-side building blocks shared by all nvnorms kernels: typed packs for
// vector loads/stores, dtype conversion, and the deterministic reductions
// (warp shuffle butterfly -> shared-memory combine -> cluster DSMEM combine).
//
// Replaces the helper layer of the reference (atex/nv_norms/cc/kernels/norm_util.h:
// Pack/Load/Store :29-180, WelfordWarpReduce/BlockAllReduce :423-464) with
// sm_100a-only code: 128-bit accesses, explicit shuffles, thread-block clusters.
#pragma once

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace nvn {

namespace cg = cooperative_groups;

// ---------------------------------------------------------------------------
// dtype conversion (compute type is always fp32)
// ---------------------------------------------------------------------------
template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) {
    return __float2bfloat16_rn(v);
  }
};

// Elements of T in one 128-bit access.
template <typename T>
struct VecTraits {
  static constexpr int kFull = 16 / sizeof(T);
};

// EPV elements of T moved as one access of EPV*sizeof(T) bytes (16, 8, 4 or 2).
template <typename T, int EPV>
struct alignas(sizeof(T) * EPV) Pack {
  T v[EPV];
};

// Streaming (read-once / write-once) global accesses.  Activations are touched
// exactly once per kernel, so they are marked evict-first; parameters and
// statistics use ordinary cached loads.
template <typename T, int EPV>
__device__ __forceinline__ Pack<T, EPV> load_stream(const T* base, int64_t elem_off) {
  using P = Pack<T, EPV>;
  const P* p = reinterpret_cast<const P*>(base + elem_off);
  if constexpr (sizeof(P) == 16) {
    union {
      uint4 u;
      P p;
    } c;
    c.u = __ldcs(reinterpret_cast<const uint4*>(p));
    return c.p;
  } else if constexpr (sizeof(P) == 8) {
    union {
      uint2 u;
      P p;
    } c;
    c.u = __ldcs(reinterpret_cast<const uint2*>(p));
    return c.p;
  } else if constexpr (sizeof(P) == 4) {
    union {
      unsigned u;
      P p;
    } c;
    c.u = __ldcs(reinterpret_cast<const unsigned*>(p));
    return c.p;
  } else {
    return *p;
  }
}

// Ordinary cached load for data that a following kernel reads again and should
// find in L2 (phase 1 of the two-phase paths).
template <typename T, int EPV>
__device__ __forceinline__ Pack<T, EPV> load_keep(const T* p) {
  return *reinterpret_cast<const Pack<T, EPV>*>(p);
}

template <typename T, int EPV>
__device__ __forceinline__ void store_stream(T* base, int64_t elem_off, const Pack<T, EPV>& v) {
  using P = Pack<T, EPV>;
  P* p = reinterpret_cast<P*>(base + elem_off);
  if constexpr (sizeof(P) == 16) {
    union {
      uint4 u;
      P p;
    } c;
    c.p = v;
    __stcs(reinterpret_cast<uint4*>(p), c.u);
  } else if constexpr (sizeof(P) == 8) {
    union {
      uint2 u;
      P p;
    } c;
    c.p = v;
    __stcs(reinterpret_cast<uint2*>(p), c.u);
  } else if constexpr (sizeof(P) == 4) {
    union {
      unsigned u;
      P p;
    } c;
    c.p = v;
    __stcs(reinterpret_cast<unsigned*>(p), c.u);
  } else {
    *p = v;
  }
}

// EPV consecutive fp32 parameters (gamma / beta / dgamma ...).  When EPV > 1
// the dispatcher guarantees 16-byte alignment of the base pointer.
template <int EPV>
__device__ __forceinline__ void load_params(const float* __restrict__ p, int64_t off,
                                            float (&out)[EPV]) {
  if constexpr (EPV % 4 == 0) {
#pragma unroll
    for (int i = 0; i < EPV / 4; ++i) {
      float4 t = __ldg(reinterpret_cast<const float4*>(p + off) + i);
      out[4 * i + 0] = t.x;
      out[4 * i + 1] = t.y;
      out[4 * i + 2] = t.z;
      out[4 * i + 3] = t.w;
    }
  } else if constexpr (EPV == 2) {
    float2 t = __ldg(reinterpret_cast<const float2*>(p + off));
    out[0] = t.x;
    out[1] = t.y;
  } else {
#pragma unroll
    for (int i = 0; i < EPV; ++i) out[i] = __ldg(p + off + i);
  }
}

template <int EPV>
__device__ __forceinline__ void store_params(float* __restrict__ p, int64_t off,
                                             const float (&v)[EPV]) {
  if constexpr (EPV % 4 == 0) {
#pragma unroll
    for (int i = 0; i < EPV / 4; ++i) {
      reinterpret_cast<float4*>(p + off)[i] =
          make_float4(v[4 * i + 0], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
  } else if constexpr (EPV == 2) {
    *reinterpret_cast<float2*>(p + off) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int i = 0; i < EPV; ++i) p[off + i] = v[i];
  }
}

// ---------------------------------------------------------------------------
// Packed fp32 arithmetic.
//
// sm_100 executes add / mul / fma on two fp32 values per lane in one instruction
// (fma.rn.f32x2 and friends, exposed as __ffma2_rn / __fadd2_rn / __fmul2_rn).
// At B200's HBM bandwidth a 16-bit norm kernel only has ~20-30 issue slots per
// element, so the element-wise math is written on float2 lanes (P2); the
// scalar family (EPV == 1) uses the same code with plain floats (P1).
// ---------------------------------------------------------------------------
struct P2 {
  using E = float2;
  static __device__ __forceinline__ E bcast(float s) { return make_float2(s, s); }
  static __device__ __forceinline__ E add(E a, E b) { return __fadd2_rn(a, b); }
  static __device__ __forceinline__ E mul(E a, E b) { return __fmul2_rn(a, b); }
  static __device__ __forceinline__ E fma(E a, E b, E c) { return __ffma2_rn(a, b, c); }
  static __device__ __forceinline__ float hsum(E a) { return a.x + a.y; }
};
struct P1 {
  using E = float;
  static __device__ __forceinline__ E bcast(float s) { return s; }
  static __device__ __forceinline__ E add(E a, E b) { return a + b; }
  static __device__ __forceinline__ E mul(E a, E b) { return a * b; }
  static __device__ __forceinline__ E fma(E a, E b, E c) { return fmaf(a, b, c); }
  static __device__ __forceinline__ float hsum(E a) { return a; }
};
template <int EPV>
struct MathSel {
  using M = P2;
  static constexpr int NE = EPV / 2;  // float2 lanes per vector
};
template <>
struct MathSel<1> {
  using M = P1;
  static constexpr int NE = 1;
};

// Pack<T, EPV>  <->  fp32 lanes
template <typename T, int EPV>
__device__ __forceinline__ void unpack(const Pack<T, EPV>& p,
                                       typename MathSel<EPV>::M::E (&out)[MathSel<EPV>::NE]) {
  if constexpr (EPV == 1) {
    out[0] = Cvt<T>::to_f32(p.v[0]);
  } else {
#pragma unroll
    for (int i = 0; i < EPV / 2; ++i) {
      if constexpr (sizeof(T) == 4) {
        out[i] = make_float2(p.v[2 * i], p.v[2 * i + 1]);
      } else if constexpr (std::is_same<T, __half>::value) {
        out[i] = __half22float2(*reinterpret_cast<const __half2*>(&p.v[2 * i]));
      } else {
        out[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&p.v[2 * i]));
      }
    }
  }
}

template <typename T, int EPV>
__device__ __forceinline__ Pack<T, EPV> repack(
    const typename MathSel<EPV>::M::E (&in)[MathSel<EPV>::NE]) {
  Pack<T, EPV> p;
  if constexpr (EPV == 1) {
    p.v[0] = Cvt<T>::from_f32(in[0]);
  } else {
#pragma unroll
    for (int i = 0; i < EPV / 2; ++i) {
      if constexpr (sizeof(T) == 4) {
        p.v[2 * i] = in[i].x;
        p.v[2 * i + 1] = in[i].y;
      } else if constexpr (std::is_same<T, __half>::value) {
        *reinterpret_cast<__half2*>(&p.v[2 * i]) = __float22half2_rn(in[i]);
      } else {
        *reinterpret_cast<__nv_bfloat162*>(&p.v[2 * i]) = __float22bfloat162_rn(in[i]);
      }
    }
  }
  return p;
}

// EPV consecutive fp32 parameters as math lanes
template <int EPV>
__device__ __forceinline__ void load_param_lanes(const float* __restrict__ p, int64_t off,
                                                 typename MathSel<EPV>::M::E (&out)[MathSel<EPV>::NE]) {
  float t[EPV];
  load_params<EPV>(p, off, t);
  if constexpr (EPV == 1) {
    out[0] = t[0];
  } else {
#pragma unroll
    for (int i = 0; i < EPV / 2; ++i) out[i] = make_float2(t[2 * i], t[2 * i + 1]);
  }
}

template <int EPV>
__device__ __forceinline__ void store_param_lanes(
    float* __restrict__ p, int64_t off, const typename MathSel<EPV>::M::E (&in)[MathSel<EPV>::NE]) {
  float t[EPV];
  if constexpr (EPV == 1) {
    t[0] = in[0];
  } else {
#pragma unroll
    for (int i = 0; i < EPV / 2; ++i) {
      t[2 * i] = in[i].x;
      t[2 * i + 1] = in[i].y;
    }
  }
  store_params<EPV>(p, off, t);
}

// ---------------------------------------------------------------------------
// Bulk asynchronous copies (TMA, non-tensor form) into a shared-memory ring.
//
// cp.async.bulk moves a contiguous, 16-byte aligned block global -> shared without
// touching registers and signals an mbarrier with the number of bytes written.  The
// row kernels use it to keep several row batches in flight per CTA independently of
// the register budget.  No multicast form is used anywhere.
//
// Waits are bounded: a wait that does not complete within kMbarPollLimit polls gives
// up and reports it; the caller then stops issuing copies, finishes its loop on
// whatever is in shared memory and raises the device status word, so a mistake in
// the byte accounting shows up as an error status and never as a hung GPU.
// ---------------------------------------------------------------------------
constexpr unsigned kMbarPollLimit = 1u << 22;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, unsigned bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// true when the phase with the given parity has completed
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
  const unsigned addr = smem_u32(bar);
  for (unsigned i = 0; i < kMbarPollLimit; ++i) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the programmatic-stream-
// serialization attribute may start while its predecessor in the stream still runs; it
// must call griddep_wait() before touching anything the predecessor writes (the wait
// returns once the predecessor has completed and its writes are visible).  The
// predecessor calls griddep_launch_dependents() so that the dependent's CTAs are
// scheduled as soon as SM resources free up.  Both are no-ops in launches without the
// attribute.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;");
}

// ---------------------------------------------------------------------------
// Row-group all-reduce (sum) of NV values.
//
// A "row group" is TPR consecutive threads of a CTA (TPR a power of two).  For
// TPR <= 32 the sum is a shuffle butterfly.  For TPR > 32 each warp's butterfly
// result goes to shared memory and every thread adds the TPR/32 warp values in
// index order.  With CS > 1 every CTA writes its total into all CTAs of the
// thread-block cluster through distributed shared memory and every thread adds the
// CS totals in rank order.  The order of every addition is fixed, so the
// result is identical in all threads and from run to run.
//
// Shared-memory slots are double-buffered on `phase` (toggled by the caller
// after each call) so one barrier per reduction is enough.
// ---------------------------------------------------------------------------
template <int NV, int BLOCK>
struct ReduceSmem {
  float warp_part[2][NV][BLOCK / 32];
  float cta_total[2][NV][16];  // [phase][value][cluster rank]; 16 = largest cluster
};

template <int NV, int TPR, int BLOCK, int CS>
__device__ __forceinline__ void group_allreduce(float (&v)[NV], ReduceSmem<NV, BLOCK>& sm,
                                                int& phase, int warp, int lane) {
  constexpr int kShuffleSpan = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int off = kShuffleSpan / 2; off > 0; off >>= 1) {
#pragma unroll
    for (int k = 0; k < NV; ++k) v[k] += __shfl_xor_sync(0xffffffffu, v[k], off);
  }
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;  // warps per row group
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < NV; ++k) sm.warp_part[phase][k][warp] = v[k];
    }
    __syncthreads();
    const int first = (warp / WPR) * WPR;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) s += sm.warp_part[phase][k][first + w];
      v[k] = s;
    }
  }
  if constexpr (CS > 1) {
    static_assert(TPR == BLOCK, "a cluster shares one row, so the CTA is one row group");
    static_assert(CS <= 16, "cta_total holds 16 ranks");
    // Every CTA pushes its total into the slot of its rank in every CTA of the cluster
    // (CS remote stores by CS lanes), then all threads read the CS totals from their own
    // shared memory: far less distributed-shared-memory traffic than every thread
    // fetching CS remote values.
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned me = cluster.block_rank();
    if (warp == 0 && lane < CS) {
#pragma unroll
      for (int k = 0; k < NV; ++k)
        *cluster.map_shared_rank(&sm.cta_total[phase][k][me], lane) = v[k];
    }
    cluster.sync();
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < CS; ++r) s += sm.cta_total[phase][k][r];
      v[k] = s;
    }
  }
  phase ^= 1;
}

}  // namespace nvn
