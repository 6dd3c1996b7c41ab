// Channels-last InstanceNorm (x[n, d, c]) for batch items far larger than shared memory,
// as ONE persistent kernel per direction.
//
// The statistics of an item need the whole item before any of it can be normalised, so
// such items were moved 3 times forward (read, read, write) and 5 times backward
// (x and dy twice, dx once) by separate launches: the second read of an item of 134 MB
// finds nothing of it in the 126 MB L2.  This kernel makes the second read cheap:
//
//   * one cooperative launch, one or two CTAs per SM, all SMs work on the same item.  The
//     item is cut into chunks of one ring stage, dealt round-robin to the CTAs (a thread's
//     128-bit vectors t, t + BLOCK, ... of a chunk always hold the same channels, so
//     per-channel state lives in registers);
//   * a CTA's chunks stream through shared memory with cp.async (16 bytes per thread and
//     copy): every thread owns its slots of every ring stage - it copies
//     into them, waits for its own copy groups and is the only reader - so the streaming
//     phases need no barrier of any kind, and the warps drift apart freely.  (A ring filled
//     by cp.async.bulk topped out near 16 bytes per clock and SM, 3.5 TB/s for the whole
//     chip, whatever the copy size: too slow for a phase that only reads.)
//     Phase 1 reduces the chunks (Welford / Chan forward, two sums backward) and
//     leaves the CTA's LAST chunks in the ring: ~190 KB per SM, 28 MB per GPU, never
//     fetched again;
//   * the per-CTA partials meet in global memory behind one grid barrier per item (one
//     arrival per CTA on a monotonic counter, one poller per CTA, bounded: a poll that runs
//     out raises the device status word and the kernel carries on);
//   * phase 2 walks the chunks BACKWARDS: first the chunks still in shared memory, then
//     the ones read most recently, which L2 still holds in part; outputs are written
//     with streaming stores so that they displace as little of that as possible;
//   * while phase 2 drains, the freed slots already load the next item;
//   * for items of a few MB the barrier and the merge behind it (~7 us in which a CTA
//     moves nothing) would cost more than the streaming: the grid then splits into GROUPS
//     of CTAs (CTA i belongs to group i % groups), each with its own barrier and its own
//     items (n = group, group + groups, ...), so that one group streams while another
//     one waits; such items stay in shared memory as a whole or nearly so;
//   * ROW MODE serves channel-first ("NC...") tensors whose rows are too long for the
//     row-cached kernels: a row is an item of one channel vector per voxel, and the lanes
//     of the vector are merged into the row's totals at the end (see the ROWS flag).
//
// All merges have a fixed order (lanes by butterfly, warps and CTAs by index), so results
// are bit-identical run to run.  No multicast copy; every copy reads this GPU's memory.
//
// Replaces, for large items, the reference's thread-per-channel kernels
// InstanceNormToTempWelford / TempToOutWelford / InstanceNormUpdate
// (atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:52-69, 80-101, 809-818) and
// InstanceNormRowReduceInToTempFused / TempToOutFused / UpdateFusedVectorized
// (fused_instance_norm_op.cu:666-730, 103-146, 744-763), and the host functions that
// launch them (:1314-1407); in row mode, for rows beyond the shared-memory kernels, the
// channel-first chain GeneralNormRowReduceInToOutWelford + InstanceNormUpdate
// (fused_instance_norm_op.cu:1167-1194, 809-818), InstanceNormToTempWelford (NC... branch,
// :23-70) and InstanceNormRowReduceInToOutFused / UpdateFusedVectorized (:315-366, 744-763).
#include <atomic>

#include "nvn_common.cuh"
#include "nvn_host.h"

namespace nvn {
namespace {

constexpr int kVPC = 4;      // 128-bit vectors per consumer thread and chunk (all tensors together)
constexpr int kStages = 6;   // ring stages of BLOCK * kVPC * 16 bytes
constexpr int kMaxC = 256;   // bounds the per-channel arrays in shared memory
constexpr int kSlotC = 128;  // channels per warp slot of the partial buffer; wider items share slots
constexpr unsigned kGridPollLimit = 1u << 24;
constexpr int kMaxGroups = 160;   // up to one group per CTA
constexpr int kCounterStride = 32;   // unsigneds between two groups' barrier counters (128 bytes)
constexpr size_t kHeaderBytes = kMaxGroups * kCounterStride * sizeof(unsigned);
constexpr int kMergeBatch = 8;  // per-CTA partials fetched together when the item's totals are formed

struct StreamArgs {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  const float* mean_in;  // backward: saved statistics [N][C]
  const float* ivar_in;
  void* out;
  float* mean;  // forward outputs [N][C]
  float* ivar;
  float* part;      // [2][grid][3][C] per-CTA partials, double-buffered by item parity
  float* colpart;   // backward: [N][2][C] per-item (dgamma, dbeta) contributions
  unsigned* counter;  // one barrier counter per group, kCounterStride apart, zero at launch
  int groups;         // CTA groups; gridDim.x is a multiple
  int64_t row_channels;  // row mode (ROWS): channels of the "NC..." tensor whose rows are the items
  int64_t N, C, D;
  float eps;
  int* status;
};

// 16 bytes global -> shared, asynchronous, bypassing L1.  (The form with an L2 cache-hint
// operand raised "illegal instruction" on B200 with driver 580 and is not used.)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// EPV consecutive floats of a shared-memory array as math lanes
template <int EPV>
__device__ __forceinline__ void lanes_from(const float* p,
                                           typename MathSel<EPV>::M::E (&out)[MathSel<EPV>::NE]) {
#pragma unroll
  for (int i = 0; i < EPV / 2; ++i) out[i] = make_float2(p[2 * i], p[2 * i + 1]);
}

// Welford triple merge (biased variance = m2 / n), safe for empty sides.
__device__ __forceinline__ void wf_merge(float& mean, float& m2, float& n, float om, float oq,
                                         float on) {
  const float t = n + on;
  if (t == 0.f) return;
  const float delta = om - mean;
  const float f = on / t;
  mean = fmaf(delta, f, mean);
  m2 = m2 + oq + delta * delta * n * f;
  n = t;
}

// ROWS: the items are contiguous rows of a channel-first tensor ("NC...": item n is row
// (n / row_channels, n % row_channels), one scale and one offset per row).  A row is read as
// D voxels of one channel vector (C = EPV), so everything up to the per-channel totals is
// the channels-last code; one thread then merges the EPV "channels" into the row's totals.
template <typename T, bool BWD, int BLOCK, bool ROWS>
__global__ void __launch_bounds__(BLOCK, BLOCK <= 256 ? 2 : 1)
    nlc_stream_kernel(const StreamArgs a) {
  constexpr int EPV = VecTraits<T>::kFull;
  using M = typename MathSel<EPV>::M;
  using E = typename M::E;
  constexpr int NE = MathSel<EPV>::NE;
  using P = Pack<T, EPV>;
  constexpr int NT = BWD ? 2 : 1;
  constexpr int VPT = kVPC / NT;                    // vectors per thread, tensor and chunk
  constexpr int NW = BLOCK / 32;
  constexpr unsigned kStageBytes = BLOCK * kVPC * 16u;
  constexpr unsigned kTensorBytes = kStageBytes / NT;

  extern __shared__ __align__(128) unsigned char ring[];  // [kStages][NT][VPT][BLOCK] vectors
  __shared__ float wpart[3][NW * kSlotC];  // per-warp partials [slot][C], then per-slice partials
  __shared__ float fin[3][kMaxC];         // per-channel coefficients of the current item

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t C = a.C, D = a.D, N = a.N;
  const int CV = static_cast<int>(C / EPV);   // channel vectors per voxel; a power of two <= 32
  const int cv = tid % CV;
  // this CTA's group: G CTAs, of which it is number b, working on items grp, grp + groups, ...
  const int groups = a.groups, grp = blockIdx.x % groups;
  const int G = gridDim.x / groups, b = blockIdx.x / groups;
  unsigned* const counter = a.counter + grp * kCounterStride;
  float* const part = a.part + static_cast<int64_t>(grp) * 2 * G * 3 * C;
  // The item in chunks of VPT * BLOCK vectors (one ring stage); CTA b takes chunks b, b + G,
  // b + 2G, ...: at any moment the CTAs read one contiguous window of the item.
  const int64_t item_vecs = D * CV;
  constexpr int64_t kChunkVecs = static_cast<int64_t>(VPT) * BLOCK;
  const int64_t item_chunks = (item_vecs + kChunkVecs - 1) / kChunkVecs;
  const int64_t NC = b < item_chunks ? (item_chunks - b + G - 1) / G : 0;   // chunks of this CTA
  const float inv_D = 1.0f / static_cast<float>(ROWS ? D * EPV : D);

  // Index arithmetic is kept out of the streaming loops (a chunk is only VPT vectors per
  // thread): chunk offsets advance by a fixed stride, ring stages by a wrapping counter.
  const P* const src[2] = {static_cast<const P*>(a.x), static_cast<const P*>(a.dy)};
  const int64_t stride = static_cast<int64_t>(G) * kChunkVecs;   // between a CTA's chunks
  const int NCi = static_cast<int>(NC);
  // number of this thread's vectors (tid, tid + BLOCK, ...) in the chunk that starts at v0
  auto count_at = [&](int64_t v0) {
    const int64_t left = item_vecs - v0 - tid;
    const int nv = left <= 0 ? 0 : static_cast<int>((left + BLOCK - 1) / BLOCK);
    return nv > VPT ? VPT : nv;
  };
  // Starts the copies of this thread's vectors of the chunk at vector offset v0 of item n
  // into its slots of `stage`.  Every call site commits exactly one copy group afterwards,
  // also when nothing was issued.
  auto issue = [&](int64_t n, int64_t v0, int stage) {
    const bool whole = v0 + kChunkVecs <= item_vecs;
    const int nv = whole ? VPT : count_at(v0);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      P* dst = reinterpret_cast<P*>(ring + stage * kStageBytes + t * kTensorBytes) + tid;
      const P* from = src[t] + n * item_vecs + v0 + tid;
#pragma unroll
      for (int u = 0; u < VPT; ++u)
        if (whole || u < nv) cp_async16(dst + u * BLOCK, from + u * BLOCK);
    }
  };
  const int64_t first_v0 = static_cast<int64_t>(b) * kChunkVecs;             // chunk 0
  const int last_stage = NCi > 0 ? (NCi - 1) % kStages : 0;                  // of chunk NC - 1
  // Only the item's last chunk can be short, and it is the last chunk of the CTA that has
  // it.  Every other chunk takes a path without a single per-vector test or address
  // computation: this thread's view of a stage is one pointer (its slot of vector 0; the
  // other slots, tensors and the global vectors lie at compile-time offsets from it).
  const bool tail_short = NCi > 0 && first_v0 + (NC - 1) * stride + kChunkVecs > item_vecs;
  const int n_whole = NCi - (tail_short ? 1 : 0);
  unsigned char* const my_ring = ring + tid * 16;
  auto issue_whole = [&](const P* const (&from)[NT], unsigned char* tp) {
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int u = 0; u < VPT; ++u)
        cp_async16(tp + t * kTensorBytes + u * (BLOCK * 16), from[t] + u * BLOCK);
  };

  // Copy groups: one per step, committed right after the step's data has been consumed,
  // for the chunk that will occupy the same stage kStages steps later; a step first waits
  // until at most kStages - 1 groups are pending, i.e. until its own chunk has landed.
  for (int c = 0; c < kStages; ++c) {
    if (c < NCi && grp < N) issue(grp, first_v0 + c * stride, c);
    cp_async_commit();
  }

  unsigned barriers = 0;   // also the number of this group's items so far
  for (int64_t n = grp; n < N; n += groups) {
    // ------------------------------------------------------------------ phase 1
    E acc0[NE], acc1[NE];   // forward: running mean, M2; backward: sum dy, sum dy * (x - mean)
    float cnt = 0.f;
    E nmu[NE];              // backward: -mean of this thread's channels
#pragma unroll
    for (int e = 0; e < NE; ++e) acc0[e] = acc1[e] = nmu[e] = M::bcast(0.f);
    if constexpr (BWD) {
      float t[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) t[e] = -__ldg(a.mean_in + (ROWS ? n : n * C + cv * EPV + e));
#pragma unroll
      for (int e = 0; e < NE; ++e) nmu[e] = make_float2(t[2 * e], t[2 * e + 1]);
    }
    // the first chunks of this item were started during the last steps of the previous
    // phase 2, in an order that the group count does not cover: wait for all of them once
    if (barriers > 0) cp_async_wait<0>();
    {
      // this thread's vector 0 of the chunk being read, and of the chunk kStages further on
      const P* ahead[NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) ahead[t] = src[t] + n * item_vecs + first_v0 + kStages * stride + tid;
      unsigned char* tp = my_ring;
      int c = 0;
      for (; c < n_whole; ++c) {
        cp_async_wait<kStages - 1>();
        const P* px = reinterpret_cast<const P*>(tp);
        if constexpr (!BWD) {
          // exact batch (mean, centred squares) folded into the running triple (Chan)
          E v[VPT][NE];
#pragma unroll
          for (int u = 0; u < VPT; ++u) unpack<T, EPV>(px[u * BLOCK], v[u]);
          const float nn = cnt + static_cast<float>(VPT);
          const float w1 = __fdividef(static_cast<float>(VPT), nn);
          const E w1v = M::bcast(w1), w2v = M::bcast(cnt * w1);
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            E sum = v[0][e];
#pragma unroll
            for (int u = 1; u < VPT; ++u) sum = M::add(sum, v[u][e]);
            const E bm = M::mul(sum, M::bcast(1.0f / VPT));
            const E nbm = M::mul(bm, M::bcast(-1.f));
            E bq = M::bcast(0.f);
#pragma unroll
            for (int u = 0; u < VPT; ++u) {
              const E d = M::add(v[u][e], nbm);
              bq = M::fma(d, d, bq);
            }
            const E delta = M::fma(acc0[e], M::bcast(-1.f), bm);
            acc0[e] = M::fma(delta, w1v, acc0[e]);
            acc1[e] = M::fma(M::mul(delta, delta), w2v, M::add(acc1[e], bq));
          }
          cnt = nn;
        } else {
          const P* pd = reinterpret_cast<const P*>(tp + kTensorBytes);
#pragma unroll
          for (int u = 0; u < VPT; ++u) {
            E vx[NE], vd[NE];
            unpack<T, EPV>(px[u * BLOCK], vx);
            unpack<T, EPV>(pd[u * BLOCK], vd);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              acc0[e] = M::add(acc0[e], vd[e]);
              acc1[e] = M::fma(vd[e], M::add(vx[e], nmu[e]), acc1[e]);
            }
          }
        }
        // the last kStages chunks stay where they are for phase 2
        if (c + kStages < n_whole) {
          issue_whole(ahead, tp);
        } else if (c + kStages < NCi) {
          issue(n, first_v0 + (c + kStages) * stride, c % kStages);   // the short tail
        }
        cp_async_commit();
#pragma unroll
        for (int t = 0; t < NT; ++t) ahead[t] += stride;
        tp = tp + kStageBytes == my_ring + kStages * kStageBytes ? my_ring : tp + kStageBytes;
      }
      if (tail_short) {   // vector by vector, with per-element Welford updates
        cp_async_wait<kStages - 1>();
        const int nv = count_at(first_v0 + (NC - 1) * stride);
        const P* px = reinterpret_cast<const P*>(tp);
        for (int u = 0; u < nv; ++u) {
          E v[NE];
          unpack<T, EPV>(px[u * BLOCK], v);
          if constexpr (!BWD) {
            cnt += 1.f;
            const E inv = M::bcast(1.0f / cnt);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              const E dl = M::fma(acc0[e], M::bcast(-1.f), v[e]);
              acc0[e] = M::fma(dl, inv, acc0[e]);
              acc1[e] = M::fma(dl, M::fma(acc0[e], M::bcast(-1.f), v[e]), acc1[e]);
            }
          } else {
            E vd[NE];
            unpack<T, EPV>(reinterpret_cast<const P*>(tp + kTensorBytes)[u * BLOCK], vd);
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              acc0[e] = M::add(acc0[e], vd[e]);
              acc1[e] = M::fma(vd[e], M::add(v[e], nmu[e]), acc1[e]);
            }
          }
        }
        cp_async_commit();
      }
    }

    // ------------------------------------------- CTA partial of every channel
    {
      float f0[EPV], f1[EPV];
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        f0[2 * e] = acc0[e].x;
        f0[2 * e + 1] = acc0[e].y;
        f1[2 * e] = acc1[e].x;
        f1[2 * e + 1] = acc1[e].y;
      }
      // Lanes of a warp that share a channel vector (lane % CV) are summed by a butterfly
      // of plain additions.  Forward: every lane first restates its (mean, M2, n) as sums
      // about the mean K of the first such lane - S1 = n (mean - K), S2 = M2 + n (mean - K)^2
      // - which add up exactly like the sums backward uses; K is within a few standard
      // errors of the true mean, so turning the totals back into (mean, M2) loses nothing.
      // (A butterfly of Chan merges, with a division each, cost 10 us per item.)
      float K[EPV];
      if constexpr (!BWD) {
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
          K[e] = __shfl_sync(0xffffffffu, f0[e], lane % CV);
          const float d = f0[e] - K[e];
          f0[e] = cnt * d;
          f1[e] = fmaf(cnt * d, d, f1[e]);
        }
      }
      for (int off = CV; off < 32; off <<= 1) {
        cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
          f0[e] += __shfl_xor_sync(0xffffffffu, f0[e], off);
          f1[e] += __shfl_xor_sync(0xffffffffu, f1[e], off);
        }
      }
      if constexpr (!BWD) {
        const float inv = cnt > 0.f ? 1.0f / cnt : 0.f;
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
          const float d = f0[e] * inv;          // warp mean - K
          f1[e] = fmaf(-f0[e], d, f1[e]);       // M2 about the warp mean
          f0[e] = K[e] + d;
        }
      }
      // One slot of C floats per warp; with more than kSlotC channels there are half as many
      // slots as warps: the upper half of the warps writes first, then each warp of the lower
      // half folds its own partial on top of its partner's.
      const int nslots = C > kSlotC ? NW / 2 : NW;
      auto put = [&](int slot) {
        if (lane < CV) {
#pragma unroll
          for (int e = 0; e < EPV; ++e) {
            wpart[0][slot * C + lane * EPV + e] = f0[e];
            wpart[1][slot * C + lane * EPV + e] = f1[e];
            wpart[2][slot * C + lane * EPV + e] = cnt;
          }
        }
      };
      if (C > kSlotC) {
        if (warp >= nslots) put(warp - nslots);
        __syncthreads();
        if (warp < nslots && lane < CV) {
          const float on = wpart[2][warp * C + lane * EPV];
          float nn = cnt;
#pragma unroll
          for (int e = 0; e < EPV; ++e) {
            const float om = wpart[0][warp * C + lane * EPV + e];
            const float oq = wpart[1][warp * C + lane * EPV + e];
            if constexpr (BWD) {
              f0[e] += om;
              f1[e] += oq;
            } else {
              nn = cnt;
              wf_merge(f0[e], f1[e], nn, om, oq, on);
            }
          }
          if constexpr (!BWD) cnt = nn;
        }
        if (warp < nslots) put(warp);
      } else {
        put(warp);
      }
      __syncthreads();
      float* mine = part + ((barriers & 1) * G + b) * 3 * C;
      if (tid < C) {
        float m = wpart[0][tid], s = wpart[1][tid], k = wpart[2][tid];
        if constexpr (BWD) {
          for (int w = 1; w < nslots; ++w) {
            m += wpart[0][w * C + tid];
            s += wpart[1][w * C + tid];
          }
        } else {
          // sums about warp 0's mean (see above), added in warp order
          const float K0 = m;
          float s1 = 0.f;
          for (int w = 1; w < nslots; ++w) {
            const float kw = wpart[2][w * C + tid], d = wpart[0][w * C + tid] - K0;
            k += kw;
            s1 = fmaf(kw, d, s1);
            s += fmaf(kw * d, d, wpart[1][w * C + tid]);
          }
          const float d = k > 0.f ? s1 / k : 0.f;
          m = K0 + d;
          s = fmaf(-s1, d, s);
        }
        mine[tid] = m;
        mine[C + tid] = s;
        mine[2 * C + tid] = k;
        __threadfence();
      }
    }
    // ------------------------------------------------------------ grid barrier
    __syncthreads();
    const unsigned parity = barriers & 1u;   // of this item's partials
    ++barriers;
    if (tid == 0) {
      atomicAdd(counter, 1u);
      const unsigned target = barriers * static_cast<unsigned>(G);
      unsigned polls = 0;
      bool gave_up = false;
      while (!gave_up && ld_acquire(counter) < target) {
        if (++polls > kGridPollLimit) {
          gave_up = true;
          if (a.status != nullptr) atomicExch(a.status, 2);
        }
      }
    }
    __syncthreads();

    // ------------------------------- totals of the item: every CTA merges all partials
    {
      const int SL = BLOCK / static_cast<int>(C);   // threads per channel (C <= 256 <= BLOCK)
      const int c = tid % static_cast<int>(C), slice = tid / static_cast<int>(C);
      const float* all = part + parity * G * 3 * C;
      // Forward: the (mean, M2, n) partials are restated as sums about CTA 0's mean K of
      // the channel, so that slices and CTAs combine by plain additions in a fixed order.
      float m = 0.f, s = 0.f, k = 0.f;
      const float K0 = BWD ? 0.f : __ldcg(all + c);
      // the partials of kMergeBatch CTAs are fetched together (independent L2 reads), then
      // added in CTA order
      for (int g0 = slice; g0 < G; g0 += SL * kMergeBatch) {
        float pm[kMergeBatch], ps[kMergeBatch], pk[kMergeBatch];
#pragma unroll
        for (int i = 0; i < kMergeBatch; ++i) {
          const int g = g0 + i * SL;
          const bool in = g < G;
          pm[i] = in ? __ldcg(all + (g * 3 + 0) * C + c) : 0.f;
          ps[i] = in ? __ldcg(all + (g * 3 + 1) * C + c) : 0.f;
          pk[i] = in ? __ldcg(all + (g * 3 + 2) * C + c) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < kMergeBatch; ++i) {
          if constexpr (BWD) {
            m += pm[i];
            s += ps[i];
          } else {
            const float d = pm[i] - K0;
            k += pk[i];
            m = fmaf(pk[i], d, m);                 // S1
            s += fmaf(pk[i] * d, d, ps[i]);        // S2
          }
        }
      }
      float* flat0 = &wpart[0][0];
      float* flat1 = &wpart[1][0];
      float* flat2 = &wpart[2][0];
      // (every thread passed the grid barrier after its last read of wpart)
      flat0[slice * C + c] = m;
      flat1[slice * C + c] = s;
      flat2[slice * C + c] = k;
      __syncthreads();
      if (tid < C) {
        m = flat0[tid];
        s = flat1[tid];
        k = flat2[tid];
        for (int j = 1; j < SL; ++j) {
          m += flat0[j * C + tid];
          s += flat1[j * C + tid];
          k += flat2[j * C + tid];
        }
        if constexpr (!BWD) {
          const float d = m / k;          // mean - K
          s = fmaf(-m, d, s);             // M2 about the mean
          m = K0 + d;
        }
        if constexpr (ROWS) {
          // per-"channel" totals, merged below
          fin[0][tid] = m;
          fin[1][tid] = s;
          fin[2][tid] = k;
        } else if constexpr (!BWD) {
          const float iv = 1.0f / sqrtf(s / k + a.eps);
          fin[0][tid] = -m;                               // -mean
          fin[1][tid] = iv * __ldg(a.gamma + tid);        // scale
          fin[2][tid] = __ldg(a.beta + tid);              // shift
          if (b == 0) {
            a.mean[n * C + tid] = m;
            a.ivar[n * C + tid] = iv;
          }
        } else {
          // m = sum dy, s = sum dy * (x - mean)
          const float iv = __ldg(a.ivar_in + n * C + tid);
          const float dgam = s * iv;                      // sum dy * xhat
          fin[0][tid] = __ldg(a.gamma + tid) * iv;        // gamma * ivar
          fin[1][tid] = m * inv_D;                        // mean(dy)
          fin[2][tid] = dgam * inv_D * iv;                // multiplies (x - mean)
          if (b == 0) {
            a.colpart[(n * 2 + 0) * C + tid] = dgam;
            a.colpart[(n * 2 + 1) * C + tid] = m;
          }
        }
      }
      __syncthreads();
      if constexpr (ROWS) {
        float c0 = 0.f, c1 = 0.f, c2 = 0.f;   // the row's three coefficients
        if (tid == 0) {
          const int64_t ch = n % a.row_channels, nb = n / a.row_channels;
          if constexpr (!BWD) {
            // (mean, M2, n) of the EPV lanes as sums about lane 0's mean, added in lane order
            const float K = fin[0][0];
            float s1 = 0.f, s2 = fin[1][0], kk = fin[2][0];
            for (int e = 1; e < EPV; ++e) {
              const float d = fin[0][e] - K, ke = fin[2][e];
              kk += ke;
              s1 = fmaf(ke, d, s1);
              s2 += fmaf(ke * d, d, fin[1][e]);
            }
            const float d = s1 / kk;
            const float mean = K + d, m2 = fmaf(-s1, d, s2);
            const float iv = 1.0f / sqrtf(m2 / kk + a.eps);
            c0 = -mean;
            c1 = iv * __ldg(a.gamma + ch);
            c2 = __ldg(a.beta + ch);
            if (b == 0) {
              a.mean[n] = mean;
              a.ivar[n] = iv;
            }
          } else {
            float sdy = fin[0][0], sdx = fin[1][0];
            for (int e = 1; e < EPV; ++e) {
              sdy += fin[0][e];
              sdx += fin[1][e];
            }
            const float iv = __ldg(a.ivar_in + n);
            const float dgam = sdx * iv;
            c0 = __ldg(a.gamma + ch) * iv;
            c1 = sdy * inv_D;
            c2 = dgam * inv_D * iv;
            if (b == 0) {
              a.colpart[(nb * 2 + 0) * a.row_channels + ch] = dgam;
              a.colpart[(nb * 2 + 1) * a.row_channels + ch] = sdy;
            }
          }
          for (int e = 0; e < EPV; ++e) {
            fin[0][e] = c0;
            fin[1][e] = c1;
            fin[2][e] = c2;
          }
        }
        __syncthreads();
      }
    }

    // ------------------------------------------------------------------ phase 2
    E k0[NE], k1[NE], k2[NE];
    lanes_from<EPV>(&fin[0][cv * EPV], k0);
    lanes_from<EPV>(&fin[1][cv * EPV], k1);
    lanes_from<EPV>(&fin[2][cv * EPV], k2);
    {
      // normalises vector u of the stage at tp into po[u * BLOCK]
      auto emit = [&](const unsigned char* tp, P* po, int u) {
        E vx[NE], o[NE];
        unpack<T, EPV>(reinterpret_cast<const P*>(tp)[u * BLOCK], vx);
        if constexpr (!BWD) {
#pragma unroll
          for (int e = 0; e < NE; ++e) o[e] = M::fma(M::add(vx[e], k0[e]), k1[e], k2[e]);
        } else {
          E vd[NE];
          unpack<T, EPV>(reinterpret_cast<const P*>(tp + kTensorBytes)[u * BLOCK], vd);
          // dx = gamma * ivar * (dy - mean(dy) - (x - mean) * ivar * mean(dy * xhat))
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            const E t = M::fma(M::add(vx[e], nmu[e]), k2[e], k1[e]);
            o[e] = M::mul(k0[e], M::fma(t, M::bcast(-1.f), vd[e]));
          }
        }
        store_stream<T, EPV>(reinterpret_cast<T*>(po + u * BLOCK), 0, repack<T, EPV>(o));
      };
      // The first kStages steps find their chunk where phase 1 left it; later steps reuse
      // the stage freed kStages steps earlier: the stage simply keeps counting down.  The
      // freed slots take the chunk kStages steps further down the backward walk or, once
      // there is none, this CTA's chunk `stage` of the group's next item.
      int stage = last_stage;
      unsigned char* tp = my_ring + last_stage * kStageBytes;
      const int64_t top = n * item_vecs + first_v0 + (NC - 1) * stride + tid;   // vector 0 of the last chunk
      P* po = static_cast<P*>(a.out) + top;
      const P* behind[NT];   // this thread's vector 0 of the chunk kStages steps further down
#pragma unroll
      for (int t = 0; t < NT; ++t) behind[t] = src[t] + top - kStages * stride;
      for (int r = 0; r < NCi; ++r) {
        cp_async_wait<kStages - 1>();
        if (r == 0 && tail_short) {
          const int nv = count_at(first_v0 + (NC - 1) * stride);
          for (int u = 0; u < nv; ++u) emit(tp, po, u);
        } else {
#pragma unroll
          for (int u = 0; u < VPT; ++u) emit(tp, po, u);
        }
        if (r + kStages < NCi) {
          issue_whole(behind, tp);
        } else if (n + groups < N && stage < NCi) {
          issue(n + groups, first_v0 + stage * stride, stage);
        }
        cp_async_commit();
        po -= stride;
#pragma unroll
        for (int t = 0; t < NT; ++t) behind[t] -= stride;
        tp = stage == 0 ? tp + (kStages - 1) * kStageBytes : tp - kStageBytes;
        stage = stage == 0 ? kStages - 1 : stage - 1;
      }
    }
    // the coefficients in `fin` and the partials in `wpart` are rewritten by the next item
    __syncthreads();
  }
  cp_async_wait<0>();
}

}  // namespace

bool nlc_stream_ok(int dtype, int64_t N, int64_t C, int64_t D) {
  const int epv = dtype == 0 ? 4 : 8;
  if (N < 1 || C % epv != 0 || C > kMaxC) return false;
  const int64_t cv = C / epv;
  return cv <= 32 && (cv & (cv - 1)) == 0;
}

constexpr int kMaxCtasPerSm = 2;

size_t nlc_stream_workspace_bytes(bool bwd, int64_t N, int64_t C) {
  const size_t ctas = static_cast<size_t>(device_sm_count()) * kMaxCtasPerSm;
  size_t b = kHeaderBytes;                          // the barrier counters
  b += (2 * ctas * 3 * C * 4 + 255) / 256 * 256;    // per-CTA partials, two item parities
  if (bwd) b += (static_cast<size_t>(N) * 2 * C * 4 + 255) / 256 * 256;
  return b;
}

template <typename T, bool BWD, int BLOCK, bool ROWS>
static cudaError_t stream_launch_b(StreamArgs& a, cudaStream_t s) {
  auto kernel = nlc_stream_kernel<T, BWD, BLOCK, ROWS>;
  const size_t smem = static_cast<size_t>(kStages) * BLOCK * kVPC * 16;
  static std::atomic<uint64_t> prepared{0};
  static std::atomic<int> cached_per_sm{0};  // per process: every device is the same part
  cudaError_t e = once_per_device(prepared, [&]() -> cudaError_t {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem));
  });
  if (e != cudaSuccess) return e;
  int per_sm = cached_per_sm.load(std::memory_order_relaxed);
  if (per_sm == 0) {
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, BLOCK, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
    cached_per_sm.store(per_sm, std::memory_order_relaxed);
  }
  e = cudaMemsetAsync(a.counter, 0, kHeaderBytes, s);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  if (a.groups > device_sm_count() * per_sm) a.groups = device_sm_count() * per_sm;
  const int ctas = device_sm_count() * per_sm / a.groups * a.groups;
  cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  cfg.blockDim = dim3(BLOCK, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  // cooperative: every CTA is resident, so the grid barrier cannot wait for a CTA that has
  // not been scheduled
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

// block: consumer threads per CTA, 512 (one CTA per SM, 32 KB stages) or 256 (two CTAs per
// SM, 16 KB stages)
template <typename T, bool BWD>
static cudaError_t stream_launch_t(StreamArgs& a, int block, cudaStream_t s) {
  if (a.row_channels > 0) return stream_launch_b<T, BWD, 512, true>(a, s);
  return block == 256 ? stream_launch_b<T, BWD, 256, false>(a, s)
                      : stream_launch_b<T, BWD, 512, false>(a, s);
}

cudaError_t nlc_stream_launch(int dtype, bool bwd, const void* dy, const void* x,
                              const float* gamma, const float* beta, const float* mean_in,
                              const float* ivar_in, int64_t N, int64_t C, int64_t D, float eps,
                              void* out, float* mean, float* ivar, void* ws, float* colpart,
                              int* status, int block, int groups, int64_t row_channels,
                              cudaStream_t s) {
  StreamArgs a = {};
  a.row_channels = row_channels;
  a.groups = groups < 1 ? 1 : (groups > kMaxGroups ? kMaxGroups : groups);
  if (a.groups > N) a.groups = static_cast<int>(N > 0 ? N : 1);
  a.x = x;
  a.dy = dy;
  a.gamma = gamma;
  a.beta = beta;
  a.mean_in = mean_in;
  a.ivar_in = ivar_in;
  a.out = out;
  a.mean = mean;
  a.ivar = ivar;
  a.counter = static_cast<unsigned*>(ws);
  a.part = reinterpret_cast<float*>(static_cast<char*>(ws) + kHeaderBytes);
  a.colpart = colpart;
  a.N = N;
  a.C = C;
  a.D = D;
  a.eps = eps;
  a.status = status;
  if (dtype == 0)
    return bwd ? stream_launch_t<float, true>(a, block, s) : stream_launch_t<float, false>(a, block, s);
  if (dtype == 1)
    return bwd ? stream_launch_t<__half, true>(a, block, s)
               : stream_launch_t<__half, false>(a, block, s);
  return bwd ? stream_launch_t<__nv_bfloat16, true>(a, block, s)
             : stream_launch_t<__nv_bfloat16, false>(a, block, s);
}

}  // namespace nvn
