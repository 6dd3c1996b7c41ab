// Column reduction fused with the data-parallel all-reduce of [dgamma | dbeta].
//
// In a data-parallel job every rank (one process, one GPU) ends its backward pass with
// P partial rows of [2][F] floats.  nvn::colreduce sums them locally; the ranks then
// still have to add their vectors up.  That exchange is a few KB, so it is pure
// latency.  This kernel does both steps in one launch over NVLink peer memory:
//
//   1. every CTA sums its 128 columns over the P local partial rows (same fixed order
//      as colreduce_kernel);
//   2. it stores that slice into the receive buffer of EVERY rank with plain 8-byte peer
//      stores, each carrying one value and the epoch number (slot = epoch mod 4, row = own
//      rank).  An aligned 8-byte store arrives as a whole, so the epoch next to a value
//      says the value is there: no fence and no separate flag, one NVLink traversal;
//   3. it polls - BOUNDED - the `world` rows of its own receive buffer until every element
//      carries this epoch and adds the values in rank order.
//
// Every rank adds the same numbers in the same order, so dgamma / dbeta are
// bit-identical on all ranks and from run to run.  Each CTA pushes before it polls and
// only waits for CTAs of other GPUs, so no CTA waits for one that cannot be scheduled.
// Four receive slots (epoch mod 4): with a single fused launch a rank can only get one
// epoch ahead of the slowest rank (finishing epoch e needs every rank's push of e).  In
// the deferred form (push now, finish later on another stream) the caller keeps the push
// of epoch e behind its own finish of epoch e-2.  That is enough across ranks: rank A's
// finish of e-2 needed rank B's push of e-2, which B issued after its own finish of e-4,
// the last reader of the slot that A's push of e overwrites at B.  (Lagging the finish by
// L epochs needs 2L slots; the four slots here give L = 2.)  Every slot's readers are done
// before it is overwritten.  A poll that exceeds its limit raises the device status word
// and the kernel finishes with whatever arrived; it never hangs.  No multimem and no
// multicast instruction is used: plain st / ld.
//
// The reference has no communication at all (its ops are single-device); this stands
// where a data-parallel TensorFlow job would run an all-reduce after the op.
#include "../../include/nvnorms.h"
#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {

namespace {
constexpr int kTX = 32;
constexpr int kW = 4;            // columns per thread
constexpr unsigned kPollLimit = 1u << 22;

struct DpPtrs {
  uint2* recv[NVN_DP_MAX_RANKS];  // (value bits, epoch) pairs
  int rank, world;
  unsigned epoch;
  int* status;
  unsigned* ctr;  // device-side epochs (nvn_dp_comm::device_epochs) or nullptr
};

// Device-side epochs: with nvn_dp_comm::device_epochs set, a kernel takes its epoch from
// device memory instead of from its arguments, so that a CUDA graph that holds these
// launches can be replayed (a replay repeats the arguments, and a repeated epoch would match
// the stale pairs of the previous replay).  Four words: [0] epoch of the last completed
// push (or fused) kernel, [1] its CTA ticket, [2] epoch of the last completed finish
// kernel, [3] its ticket.  Every CTA reads the epoch at its start; the last CTA to leave
// (ticket == grid size - 1) publishes epoch + 1 for the next launch of the same kind, which
// stream order keeps behind this one.
__device__ __forceinline__ unsigned epoch_of(const DpPtrs& c, int word) {
  if (c.ctr == nullptr) return c.epoch;
  unsigned v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(c.ctr + word) : "memory");
  return v + 1;
}
__device__ __forceinline__ void publish_epoch(const DpPtrs& c, int word, unsigned epoch) {
  // called by one thread per CTA after the CTA's last use of the epoch
  if (c.ctr == nullptr) return;
  __threadfence();
  const unsigned t = atomicAdd(c.ctr + word + 1, 1u);
  if (t == gridDim.x - 1) {
    atomicExch(c.ctr + word + 1, 0u);
    __threadfence();
    atomicExch(c.ctr + word, epoch);
  }
}

__device__ __forceinline__ void st_pair(uint2* p, float v, unsigned epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)),
               "r"(epoch)
               : "memory");
}
// two neighbouring pairs with one 16-byte load: {value, epoch, value, epoch}
__device__ __forceinline__ uint4 ld_two_pairs(const uint2* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// PUSH: steps 1 and 2.  FINISH: step 3.  <true, true> is the single fused launch;
// <true, false> followed later (possibly on another stream) by <false, true> lets the
// caller overlap the wait with other work.
template <int TY, bool PUSH, bool FINISH>
__global__ void __launch_bounds__(kTX* TY)
    colreduce_allreduce_kernel(const float* __restrict__ partials, int64_t P, int64_t F,
                               const DpPtrs c, float* __restrict__ dgamma,
                               float* __restrict__ dbeta) {
  __shared__ float tile[TY][kTX * kW + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t F2 = 2 * F;
  const int64_t col = (static_cast<int64_t>(blockIdx.x) * kTX + tx) * kW;
  if constexpr (PUSH) griddep_wait();  // the partial rows come from the kernel launched just before
  constexpr int kWord = PUSH ? 0 : 2;
  const unsigned epoch = epoch_of(c, kWord);
  const int64_t slot = static_cast<int64_t>(epoch & 3u) * c.world;
  if constexpr (PUSH) {
  float s[kW] = {0.f, 0.f, 0.f, 0.f};
  if (col < F2) {
    for (int64_t p = ty; p < P; p += TY) {
      const float4 v = *reinterpret_cast<const float4*>(partials + p * F2 + col);
      s[0] += v.x;
      s[1] += v.y;
      s[2] += v.z;
      s[3] += v.w;
    }
  }
#pragma unroll
  for (int w = 0; w < kW; ++w) tile[ty][tx * kW + w] = s[w];
  __syncthreads();
  if (ty == 0 && col < F2) {
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < TY; ++k) {
      t.x += tile[k][tx * kW + 0];
      t.y += tile[k][tx * kW + 1];
      t.z += tile[k][tx * kW + 2];
      t.w += tile[k][tx * kW + 3];
    }
    const float o[kW] = {t.x, t.y, t.z, t.w};
    for (int p = 0; p < c.world; ++p) {
      uint2* dst = c.recv[p] + (slot + c.rank) * F2 + col;
#pragma unroll
      for (int w = 0; w < kW; ++w) st_pair(dst + w, o[w], epoch);
    }
  }
  }  // PUSH
  if constexpr (!FINISH) {
    __syncthreads();
    if (tx == 0 && ty == 0) publish_epoch(c, kWord, epoch);
    return;
  }
  // Bounded poll of this rank's own receive rows, then the sum in rank order.  The pairs of
  // four ranks are fetched together (eight independent 16-byte loads): in the steady state
  // everything has arrived, and reading world * kW pairs one after the other would cost as
  // many L2 round trips (20 us at eight ranks).  Only pairs whose epoch is still old are
  // read again.
  int ok = 1;
  unsigned polls = 0;
  float acc[kW] = {0.f, 0.f, 0.f, 0.f};
  static_assert(kW == 4, "two 16-byte loads per rank and thread");
  if (ty == 0 && col < F2) {
    const uint2* base = c.recv[c.rank] + slot * F2 + col;
    for (int r0 = 0; r0 < c.world; r0 += 4) {
      uint4 got[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (r0 + i < c.world) {
          got[i][0] = ld_two_pairs(base + (r0 + i) * F2);
          got[i][1] = ld_two_pairs(base + (r0 + i) * F2 + 2);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (r0 + i < c.world) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4 v = got[i][h];
            // one budget for the whole thread: after the first element that never arrives the
            // rest are read once and not waited for, so a missing peer costs one time-out
            while ((v.y != epoch || v.w != epoch) && ok) {
              if (++polls > kPollLimit) ok = 0;
              v = ld_two_pairs(base + (r0 + i) * F2 + 2 * h);
            }
            acc[2 * h] += __uint_as_float(v.x);
            acc[2 * h + 1] += __uint_as_float(v.z);
          }
        }
      }
    }
#pragma unroll
    for (int w = 0; w < kW; ++w) {
      const int64_t cc = col + w;
      if (cc < F) {
        dgamma[cc] = acc[w];
      } else {
        dbeta[cc - F] = acc[w];
      }
    }
  }
  if (!__syncthreads_and(ok)) {
    if (tx == 0 && ty == 0 && c.status != nullptr) atomicExch(c.status, 1);
  }
  if (tx == 0 && ty == 0) publish_epoch(c, kWord, epoch);
}

template <int TY, bool PUSH, bool FINISH>
cudaError_t launch(const float* partials, int64_t P, int64_t F, const DpPtrs& c, float* dgamma,
                   float* dbeta, cudaStream_t s) {
  const int64_t blocks = (2 * F + kTX * kW - 1) / (kTX * kW);
  count_launch();
  if constexpr (PUSH) {
    cudaLaunchAttribute attr;
    const cudaLaunchConfig_t cfg =
        dependent_launch_config(dim3(static_cast<unsigned>(blocks)), dim3(kTX, TY), 0, s, &attr);
    return cudaLaunchKernelEx(&cfg, colreduce_allreduce_kernel<TY, PUSH, FINISH>, partials, P, F,
                              c, dgamma, dbeta);
  }
  colreduce_allreduce_kernel<TY, PUSH, FINISH><<<static_cast<unsigned>(blocks), dim3(kTX, TY), 0, s>>>(
      partials, P, F, c, dgamma, dbeta);
  return cudaGetLastError();
}

DpPtrs make_ptrs(const nvn_dp_comm* comm) {
  DpPtrs c;
  c.rank = comm->rank;
  c.world = comm->world;
  c.epoch = comm->epoch;
  c.status = device_status_word();
  c.ctr = static_cast<unsigned*>(comm->device_epochs);
  for (int i = 0; i < NVN_DP_MAX_RANKS; ++i) {
    c.recv[i] = i < comm->world ? static_cast<uint2*>(comm->recv[i]) : nullptr;
  }
  return c;
}

template <bool FINISH>
cudaError_t launch_push(const float* partials, int64_t P, int64_t F, const DpPtrs& c,
                        float* dgamma, float* dbeta, cudaStream_t s) {
  if (P <= 4) return launch<1, true, FINISH>(partials, P, F, c, dgamma, dbeta, s);
  if (P <= 32) return launch<4, true, FINISH>(partials, P, F, c, dgamma, dbeta, s);
  if (P <= 128 || 2 * F >= 32768) return launch<8, true, FINISH>(partials, P, F, c, dgamma, dbeta, s);
  return launch<32, true, FINISH>(partials, P, F, c, dgamma, dbeta, s);
}
}  // namespace

cudaError_t colreduce_allreduce_launch(const float* partials, int64_t P, int64_t F,
                                       const nvn_dp_comm* comm, float* dgamma, float* dbeta,
                                       cudaStream_t s) {
  const DpPtrs c = make_ptrs(comm);
  // comm->defer: only reduce and push here; nvn_dp_finish completes the exchange later
  return comm->defer ? launch_push<false>(partials, P, F, c, dgamma, dbeta, s)
                     : launch_push<true>(partials, P, F, c, dgamma, dbeta, s);
}

cudaError_t dp_finish_launch(int64_t F, const nvn_dp_comm* comm, float* dgamma, float* dbeta,
                             cudaStream_t s) {
  return launch<1, false, true>(nullptr, 0, F, make_ptrs(comm), dgamma, dbeta, s);
}

}  // namespace nvn
