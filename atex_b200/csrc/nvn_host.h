// Host-side declarations shared by the kernel translation units and the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

struct nvn_dp_comm;

namespace nvn {

// Arguments of the row-cached kernels (rows_kernels.cuh).  `out` is y (forward)
// or dx (backward); `mean` / `ivar` are forward outputs, `mean_in` / `ivar_in`
// backward inputs.  C is the channel count when gamma / beta are indexed by
// row % C (InstanceNorm "NC..."), unused otherwise.
struct RowsArgs {
  const void* x;
  const void* dy;
  const float* gamma;
  const float* beta;
  const float* mean_in;
  const float* ivar_in;
  void* out;
  float* mean;
  float* ivar;
  float* ws;
  int64_t N;
  int64_t D;
  int64_t C;
  float eps;
  int* status;  // device status word: set non-zero when a bounded wait gave up
};

// Arguments of the residual-add forward (rows_fwd_kernel<..., RES = true>): the row that is
// normalised is s = T(x + res), which is also written to sum_out.  A type of its own, so
// that the parameter block - and with it the generated code - of every other instantiation
// of the row kernels stays what their shapes were tuned with.
struct RowsResArgs : RowsArgs {
  const void* res;
  void* sum_out;
};

struct RowsPlan {
  int grid;
  int block;
  int cluster;
  int tpr;
  int vpt;
  int epv;
  int rb;
  int load_mode;  // 0 plain, 1 register prefetch, 2..9 TMA ring with that many stages,
                  // >= 10 held TMA ring with (load_mode - 10) stages
  int partial_rows;  // rows of [2][D] dgamma/dbeta partials the backward kernel writes
};

// Cluster kernels for LayerNorm rows of thousands of vectors (rows_wide.cu): a row must
// fill one of the compiled shapes exactly (wide_ok).  Backward leaves `partial_rows` rows of
// [2][D] dgamma / dbeta partials in RowsArgs::ws.
struct WidePlan {
  int grid;
  int block;
  int cluster;
  int vpt;
  int stages;
  int partial_rows;
};
bool wide_ok(int64_t nvec, bool bwd);
// `forced`: index of a shape of rows_wide.cu to use instead of the default for the row's
// width (tuning runs), or -1.
cudaError_t wide_launch(int dtype, bool bwd, int forced, const RowsArgs& a, cudaStream_t s,
                        bool dry_run, WidePlan* plan);

// On-chip channels-last InstanceNorm (nlc_onchip.cu): one CTA holds a whole batch item in
// shared memory.  nlc_onchip_ok: the item fits and C / vector divides the CTA size.  The
// backward launch leaves per-item (dgamma, dbeta) contributions in colpart[N][2][C].
bool nlc_onchip_ok(int dtype, bool bwd, int64_t C, int64_t D);
cudaError_t nlc_onchip_launch(int dtype, bool bwd, const void* dy, const void* x,
                              const float* gamma, const float* beta, const float* mean_in,
                              const float* ivar_in, int64_t N, int64_t C, int64_t D, float eps,
                              void* out, float* mean, float* ivar, float* colpart, int* status,
                              cudaStream_t s);

// Persistent channels-last InstanceNorm for items far larger than shared memory
// (nlc_stream.cu): one cooperative launch per direction, the tail of every item stays on
// chip between the statistics and the normalisation.  nlc_stream_ok: 128-bit accesses, a
// power-of-two number (<= 32) of channel vectors, C <= 256 (whether the items are large
// enough to be worth it is the dispatcher's decision).  `ws` holds
// nlc_stream_workspace_bytes; the backward launch leaves colpart[N][2][C].  `block`: 512
// threads (one CTA per SM) or 256 (two per SM).  `groups`: CTA groups that work on
// different items at the same time (clamped to N and to the grid).  `row_channels` > 0: row
// mode for channel-first tensors - the N items are contiguous rows of D * C elements (pass
// C = the vector width and D = row length / C), item n being row (n / row_channels,
// n % row_channels) with gamma[n % row_channels]; mean / ivar are [N], colpart is
// [N / row_channels][2][row_channels].
bool nlc_stream_ok(int dtype, int64_t N, int64_t C, int64_t D);
size_t nlc_stream_workspace_bytes(bool bwd, int64_t N, int64_t C);
cudaError_t nlc_stream_launch(int dtype, bool bwd, const void* dy, const void* x,
                              const float* gamma, const float* beta, const float* mean_in,
                              const float* ivar_in, int64_t N, int64_t C, int64_t D, float eps,
                              void* out, float* mean, float* ivar, void* ws, float* colpart,
                              int* status, int block, int groups, int64_t row_channels,
                              cudaStream_t s);

// Warp-per-item channels-last InstanceNorm for small items (nlc_small.cu): any dtype, C and
// alignment, C <= 32 and D * C <= 4096 elements.  Backward leaves colpart[N][2][C].
bool nlc_small_ok(int64_t C, int64_t D);
cudaError_t nlc_small_launch(int dtype, bool bwd, const void* dy, const void* x,
                             const float* gamma, const float* beta, const float* mean_in,
                             const float* ivar_in, int64_t N, int64_t C, int64_t D, float eps,
                             void* out, float* mean, float* ivar, float* colpart, cudaStream_t s);

// Launch configuration for a kernel that follows the kernel it depends on in the same
// stream and calls griddep_wait() (nvn_common.cuh) before reading that kernel's output:
// its launch overlaps the predecessor's tail.  `attr` must outlive the launch call.
inline cudaLaunchConfig_t dependent_launch_config(dim3 grid, dim3 block, size_t smem,
                                                  cudaStream_t s, cudaLaunchAttribute* attr) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cfg;
}

int device_sm_count();
void count_launch();
// Whether the row kernels are launched with the programmatic-stream-serialization
// attribute (their launch then overlaps the predecessor's tail); see variant key `pdl`.
bool use_dependent_launch();

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory, non-portable
// cluster sizes) belong to one device's context, and one process may drive several devices
// (a TensorFlow process owns every GPU of the node).  `mask` is a kernel's own set of device
// ordinals whose context already has the attributes; `set` runs with the calling thread's
// current device when that device is not in the set yet.  Two threads may both run `set`
// the first time: the calls are idempotent.
template <typename F>
inline cudaError_t once_per_device(std::atomic<uint64_t>& mask, F&& set) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  // ordinals beyond 63 are not remembered: every call sets the attributes again
  const uint64_t bit = (dev >= 0 && dev < 64) ? (1ull << dev) : 0;
  if (bit != 0 && (mask.load(std::memory_order_acquire) & bit) != 0) return cudaSuccess;
  e = set();
  if (e != cudaSuccess) return e;
  if (bit != 0) mask.fetch_or(bit, std::memory_order_release);
  return cudaSuccess;
}
// Device address of the library's status word on the current device (nullptr on failure).
int* device_status_word();

// Row-group shapes: X(index, TPR, VPT, CS, RB, PR, MINB, PF)
//   TPR threads per row, VPT vectors per thread, CS CTAs per cluster, RB rows in
//   flight per row group, PR gamma/beta cached in registers, MINB the CTA size for
//   row groups smaller than a CTA (0 = 256 threads), PF load mode: 0 = plain loads,
//   1 = register prefetch of the next row batch, 2..9 = TMA (cp.async.bulk) ring in
//   shared memory with that many stages, 10 + s = (backward) held ring of s stages: the
//   row batch stays in its stage until dx is written and is read from there twice.
// "Light" kernels keep only the row itself in registers (LayerNorm forward,
// InstanceNorm forward/backward); "heavy" is LayerNorm backward, which adds the
// per-column dgamma/dbeta accumulators and therefore spreads a row over more
// threads.  Capacity of a shape is TPR*VPT*CS vectors; the dispatcher takes the
// first entry (in listing order) among those of the smallest sufficient capacity.
#ifndef NVN_ROW_SHAPES_LIGHT
#define NVN_ROW_SHAPES_LIGHT(X)                                                              \
  X(0, 4, 1, 1, 4, 1, 0, 1)     X(1, 8, 1, 1, 4, 1, 0, 1)     X(2, 8, 2, 1, 4, 1, 0, 3)      \
  X(3, 32, 1, 1, 4, 1, 0, 3)    X(4, 32, 2, 1, 2, 1, 0, 3)    X(5, 32, 4, 1, 2, 1, 0, 3)     \
  X(6, 128, 2, 1, 1, 1, 128, 1)  X(7, 128, 4, 1, 1, 1, 0, 2)   X(8, 256, 4, 1, 1, 1, 0, 2)    \
  X(9, 512, 4, 1, 1, 1, 0, 2)   X(10, 512, 8, 1, 1, 0, 0, 1)  X(11, 512, 4, 4, 1, 1, 0, 1)   \
  X(12, 512, 8, 4, 1, 0, 0, 1)  X(13, 512, 8, 8, 1, 0, 0, 1)  X(14, 512, 8, 16, 1, 0, 0, 1)  \
  /* three or five vectors per thread: widths of 3 * 2^k and 5 * 2^k elements */            \
  X(15, 32, 3, 1, 2, 1, 0, 3)   X(16, 64, 3, 1, 2, 1, 0, 3)   X(17, 128, 3, 1, 1, 1, 0, 2)   \
  X(18, 128, 5, 1, 1, 1, 0, 2)  X(19, 256, 3, 1, 1, 1, 0, 2)  X(20, 256, 5, 1, 1, 1, 0, 2)   \
  X(21, 512, 3, 1, 1, 1, 0, 2)
#endif

// In the heavy table a held-ring entry (PF >= 10) is followed by the register-prefetch
// entry of the same capacity: the held ring wins once the problem is large enough to be
// bandwidth-bound, the other on small problems, where the ring's start-up shows.
#ifndef NVN_ROW_SHAPES_HEAVY
#define NVN_ROW_SHAPES_HEAVY(X)                                                              \
  X(0, 4, 1, 1, 4, 1, 128, 3)      X(1, 8, 1, 1, 4, 1, 128, 3)     X(2, 16, 1, 1, 4, 1, 128, 3) \
  X(3, 32, 1, 1, 4, 1, 128, 3)     X(4, 32, 2, 1, 2, 1, 128, 3)    X(5, 64, 2, 1, 2, 1, 128, 3) \
  X(6, 128, 2, 1, 2, 1, 128, 12)   X(7, 64, 4, 1, 1, 1, 128, 1)                                \
  X(8, 128, 4, 1, 1, 1, 128, 13)   X(9, 256, 2, 1, 2, 1, 0, 1)                                 \
  X(10, 256, 4, 1, 1, 1, 0, 12)    X(11, 512, 2, 1, 1, 1, 0, 1)                                \
  X(12, 512, 4, 1, 1, 1, 0, 12)    X(13, 512, 2, 2, 1, 1, 0, 1)                                \
  X(14, 128, 4, 8, 2, 1, 128, 12)  X(15, 512, 2, 4, 1, 1, 0, 1)                                \
  X(16, 128, 4, 16, 2, 1, 128, 12) X(17, 512, 2, 8, 1, 1, 0, 1)                                \
  X(18, 512, 2, 16, 1, 1, 0, 1)    X(19, 512, 4, 16, 1, 0, 0, 1)                               \
  /* three or five vectors per thread: widths of 3 * 2^k and 5 * 2^k elements */            \
  X(20, 32, 3, 1, 2, 1, 128, 3)    X(21, 64, 3, 1, 2, 1, 128, 12)  X(22, 128, 3, 1, 1, 1, 128, 13) \
  X(23, 128, 5, 1, 1, 1, 128, 12)  X(24, 256, 3, 1, 1, 1, 0, 12)   X(25, 512, 3, 1, 1, 1, 0, 12)
#endif

// InstanceNorm "NC..." backward for rows of more than 2048 vectors.  The light table's wide
// shapes hold 8 vectors per thread, which the backward kernel (x-hat and dy of the batch in
// registers across the reduction) cannot afford at 512 threads; these shapes keep at most 4
// vectors per thread or hold the batch in the ring.  Indices start at 256; wider rows take
// the two-phase kernels.
#ifndef NVN_ROW_SHAPES_AFFINE_WIDE
#define NVN_ROW_SHAPES_AFFINE_WIDE(X)                                                        \
  X(256, 256, 4, 4, 1, 0, 0, 1)    X(257, 512, 4, 4, 1, 0, 0, 1)
#endif
constexpr int kAffineWideBase = 256;

// Rows accessed with less than 128 bits per access (64-, 32-bit or single elements: widths
// that are not a multiple of the vector, misaligned buffers) share this coarser table.
#define NVN_ROW_SHAPES_SCALAR(X)                                                             \
  X(0, 8, 4, 1, 2, 0, 0, 1) X(1, 32, 8, 1, 1, 0, 0, 1) X(2, 256, 8, 1, 1, 0, 0, 1)           \
  X(3, 512, 8, 2, 1, 0, 0, 1) X(4, 512, 8, 8, 1, 0, 0, 1) X(5, 512, 8, 16, 1, 0, 0, 1)

// One entry point per (dtype, direction) translation unit.  `epv` (elements per access: the
// full 128-bit width, or 4 / 2 / 1) selects the family, `row_affine` the InstanceNorm
// "NC..." parameter indexing.
// With dry_run the plan is filled in and nothing is launched.
#define NVN_DECLARE_ROWS(NAME)                                                              \
  cudaError_t NAME(bool row_affine, int epv, int shape, const RowsArgs& a, cudaStream_t s, \
                   bool dry_run, RowsPlan* plan);
NVN_DECLARE_ROWS(rows_f32_fwd)
NVN_DECLARE_ROWS(rows_f32_bwd)
NVN_DECLARE_ROWS(rows_f16_fwd)
NVN_DECLARE_ROWS(rows_f16_bwd)
NVN_DECLARE_ROWS(rows_bf16_fwd)
NVN_DECLARE_ROWS(rows_bf16_bwd)

// LayerNorm forward fused with the residual add that precedes it in a pre-norm transformer
// block (rows_res_inst.cu): s = T(x + res) is written to a.sum_out and normalised in the same
// pass.  Covers rows of up to 4096 128-bit vectors with 128-bit accesses; rows_res_ok says
// whether a problem qualifies (the C ABI falls back to an add kernel plus the plain forward).
bool rows_res_ok(int dtype, int64_t D, size_t align, size_t par_align);
cudaError_t rows_res_launch(int dtype, const RowsResArgs& a, cudaStream_t s);
cudaError_t rows_res_f32(const RowsResArgs& a, cudaStream_t s);
cudaError_t rows_res_f16(const RowsResArgs& a, cudaStream_t s);
cudaError_t rows_res_bf16(const RowsResArgs& a, cudaStream_t s);
cudaError_t residual_add_f32(const void* x, const void* res, void* out, int64_t count, cudaStream_t s);
cudaError_t residual_add_f16(const void* x, const void* res, void* out, int64_t count, cudaStream_t s);
cudaError_t residual_add_bf16(const void* x, const void* res, void* out, int64_t count, cudaStream_t s);
// The fallback's element-wise s = T(x + res) for any size and alignment.
cudaError_t residual_add_launch(int dtype, const void* x, const void* res, void* sum_out,
                                int64_t count, cudaStream_t s);

// Deterministic second stage of the dgamma / dbeta reduction: sums P partial
// rows of [2][F] floats (dgamma then dbeta) in a fixed order.
// `scratch` (optional, `scratch_rows` rows of [2F] floats, 16-byte aligned) lets the kernel
// split very many partial rows into slabs when there are few columns.
constexpr int64_t kColreduceScratchRows = 256;
cudaError_t colreduce_launch(const float* partials, int64_t P, int64_t F, float* dgamma,
                             float* dbeta, cudaStream_t s, float* scratch = nullptr,
                             int64_t scratch_rows = 0);

// Column reduction fused with the all-reduce over peer memory (colreduce_dp.cu).  Needs
// 2F % 4 == 0.
cudaError_t colreduce_allreduce_launch(const float* partials, int64_t P, int64_t F,
                                       const struct ::nvn_dp_comm* comm, float* dgamma,
                                       float* dbeta, cudaStream_t s);
cudaError_t dp_finish_launch(int64_t F, const struct ::nvn_dp_comm* comm, float* dgamma,
                             float* dbeta, cudaStream_t s);

}  // namespace nvn
