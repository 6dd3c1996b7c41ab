/*
 * nvnorms.h - C ABI of libnvnorms: fused LayerNorm / InstanceNorm forward and
 * gradient kernels for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a TensorFlow OpKernel (or any other host runtime) binds
 * to.  It replaces the GPU functors of NVIDIA/atex's nv_norms package:
 *
 *   functor::FusedLayerNorm<GPUDevice,T,U>         atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:805-893
 *   functor::FusedLayerNormGrad<GPUDevice,T,U>     atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:895-1030
 *   functor::FusedInstanceNorm<GPUDevice,T,U>      atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:1457-1517
 *   functor::FusedInstanceNormGrad<GPUDevice,T,U>  atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:1519-1561
 *
 * and the shape bookkeeping the OpKernels do before calling them
 * (GetBatchAndFeatureSizes, atex/nv_norms/cc/kernels/fused_layer_norm_op.cc:252-282;
 * FormatFromSuccinctString, atex/nv_norms/cc/kernels/fused_instance_norm_op.cc:25-34).
 *
 * Conventions
 *   - Every function returns NVN_OK (0) or a negative nvn_status; nothing throws,
 *     aborts, allocates device memory or synchronises the device or the stream.
 *   - All device buffers (inputs, outputs, workspace) are owned by the caller and
 *     must belong to the device that is current on the calling thread.
 *   - Work is enqueued asynchronously on `stream` (a cudaStream_t passed as void*).
 *   - T is the activation type named by `dtype`; gamma, beta, the saved statistics
 *     and the parameter gradients are always fp32 (the reference's `U`).
 *   - Pointers only need the natural alignment of their element type; the library
 *     selects 128-bit vector kernels when the actual alignment allows it.
 *   - `y` may alias `x` in the forward calls (the reference forwards its input
 *     buffer to the output, fused_layer_norm_op.cc:337, fused_instance_norm_op.cc:390).
 *   - The second saved statistic is 1/sqrt(var + epsilon) (the reference calls it
 *     "inv_var", norm_util.h:255-258).
 *   - Backward uses the mean / inverse-std passed in; it never recomputes them.
 *   - Empty inputs (N*D == 0 or N*C*D == 0) launch nothing, except that backward
 *     zero-fills dgamma / dbeta (the reference's CPU kernels do,
 *     fused_layer_norm_op.cc:96-103; its GPU kernels leave them unwritten).
 *   - Calls are re-entrant and thread-safe.
 */
#ifndef NVNORMS_H_
#define NVNORMS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define NVN_API
#else
#define NVN_API __attribute__((visibility("default")))
#endif

typedef enum nvn_dtype {
  NVN_F32 = 0,  /* float            (reference T = float)       */
  NVN_F16 = 1,  /* IEEE half        (reference T = Eigen::half) */
  NVN_BF16 = 2  /* bfloat16         (extension: not in the reference's T list, norm_ops.cc:155) */
} nvn_dtype;

typedef enum nvn_status {
  NVN_OK = 0,
  NVN_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, unknown dtype        */
  NVN_ERR_AXIS_RANGE = -2,       /* "axis contains invalid value"                      */
  NVN_ERR_AXIS_NOT_PACKED = -3,  /* "axis is not packed from last dim."                */
  NVN_ERR_DATA_FORMAT = -4,      /* "We only accept 'NC...' or 'N...C' data format"    */
  NVN_ERR_RANK = -5,             /* rank below 1 (LayerNorm) or below 4 (InstanceNorm) */
  NVN_ERR_WORKSPACE = -6,        /* workspace missing, misaligned or too small         */
  NVN_ERR_CUDA = -7,             /* a CUDA runtime call failed (see nvn_last_cuda_error) */
  NVN_ERR_UNSUPPORTED = -8,      /* size beyond what the kernels index                 */
  NVN_ERR_LIMIT = -9,            /* size beyond a fixed built-in capacity              */
  NVN_ERR_TIMEOUT = -10          /* a kernel gave up a bounded wait (see nvn_device_status) */
} nvn_status;

/* Library version: major*10000 + minor*100 + patch. */
NVN_API int nvn_version(void);

/* Human-readable text for a status.  For the shape errors the text is the
 * InvalidArgument message of the reference op. */
NVN_API const char* nvn_status_string(int status);

/* cudaError_t value of the most recent failing CUDA call on this thread (0 if none). */
NVN_API int nvn_last_cuda_error(void);

/* Diagnostic: synchronises with the current device and reports whether any kernel of this
 * library has given up a bounded wait on an asynchronous copy since the process started
 * (NVN_OK, NVN_ERR_TIMEOUT, or NVN_ERR_CUDA).  Every wait inside the kernels has an
 * iteration limit, so a logic error surfaces here instead of as a hung GPU.  The reference
 * has no counterpart (its kernels do not wait on anything). */
NVN_API int nvn_device_status(void);

/* Number of kernel launches this library has issued in this process so far. */
NVN_API uint64_t nvn_launch_count(void);

/* ---- shape bookkeeping (host only, no CUDA) ------------------------------- */

/* LayerNorm: normalise `axis` entries (negative allowed), require them to be the
 * trailing dimensions, return N = product of the leading dims, D = product of
 * the normalised dims.  Replaces GetBatchAndFeatureSizes
 * (fused_layer_norm_op.cc:252-282, norm_ops.cc:18-52). */
NVN_API int nvn_ln_dims(int rank, const int64_t* dims, int n_axis, const int* axis,
                        int64_t* N, int64_t* D);

/* InstanceNorm: parse `data_format` (accepted iff longer than 2 characters,
 * starting with 'N', with 'C' second or last: "NC...", "N...C", "NCHW", "NDHWC"
 * ...), require rank >= 4, return N, C, D = product of the spatial dims and
 * whether channels come first.  Replaces FormatFromSuccinctString and the
 * reshaping in FusedInstanceNormOp::Compute (fused_instance_norm_op.cc:25-34, 333-376). */
NVN_API int nvn_in_dims(int rank, const int64_t* dims, const char* data_format,
                        int64_t* N, int64_t* C, int64_t* D, int* channel_first);

/* ---- workspace sizes -------------------------------------------------------
 * Bytes of device scratch each call needs for the given problem on the current
 * device (0 is possible).  The workspace must be 256-byte aligned.  Replaces
 * the context->allocate_temp calls inside the reference functors
 * (fused_layer_norm_op.cu:852-868, 925-935; fused_instance_norm_op.cu:1238-1250,
 * 1326-1340, 1534-1545).  Contents on entry are ignored; nothing needs zeroing. */
NVN_API size_t nvn_ln_fwd_workspace_bytes(int dtype, int64_t N, int64_t D);
NVN_API size_t nvn_ln_bwd_workspace_bytes(int dtype, int64_t N, int64_t D);
NVN_API size_t nvn_in_fwd_workspace_bytes(int dtype, int64_t N, int64_t C, int64_t D,
                                          int channel_first);
NVN_API size_t nvn_in_bwd_workspace_bytes(int dtype, int64_t N, int64_t C, int64_t D,
                                          int channel_first);

/* ---- LayerNorm --------------------------------------------------------------
 * x, y: [N, D] of T, row-major.  gamma, beta: [D] fp32.  mean, inv_std: [N] fp32.
 *   mean_i    = sum_j x_ij / D
 *   inv_std_i = 1 / sqrt(sum_j (x_ij - mean_i)^2 / D + epsilon)
 *   y_ij      = (x_ij - mean_i) * inv_std_i * gamma_j + beta_j
 * Replaces FusedLayerNorm<GPUDevice> (fused_layer_norm_op.cu:805-893). */
NVN_API int nvn_ln_fwd(int dtype, const void* x, const float* gamma, const float* beta,
                       int64_t N, int64_t D, float epsilon, void* y, float* mean,
                       float* inv_std, void* workspace, size_t workspace_bytes,
                       void* stream);

/* LayerNorm forward fused with the residual add that precedes it in a pre-norm block:
 *   s_ij = T(x_ij + residual_ij)      (the sum in fp32, rounded once to T, written to sum_out)
 *   y, mean, inv_std = LayerNorm(s)   as in nvn_ln_fwd
 * The backward pass is nvn_ln_bwd on s: its dx is the gradient of both x and residual.
 * sum_out may alias x or residual; y may alias any of them.  Workspace: as for nvn_ln_fwd
 * (nvn_ln_fwd_workspace_bytes).  Rows of up to 4096 128-bit vectors in 16-byte aligned
 * buffers run as one kernel that reads x and residual once (4 tensor passes); anything else
 * runs an add kernel followed by nvn_ln_fwd (5 passes), with identical results.
 * No counterpart in the reference: nv_norms.LayerNormalization calls the bare op
 * (nv_norm_ops.py:85-99) and the add is a separate TensorFlow kernel. */
NVN_API int nvn_ln_fwd_residual(int dtype, const void* x, const void* residual,
                                const float* gamma, const float* beta, int64_t N, int64_t D,
                                float epsilon, void* sum_out, void* y, float* mean,
                                float* inv_std, void* workspace, size_t workspace_bytes,
                                void* stream);

/* dy, x, dx: [N, D] of T.  dgamma, dbeta: [D] fp32.
 *   dgamma_j = sum_i dy_ij (x_ij - mean_i) inv_std_i      dbeta_j = sum_i dy_ij
 *   dx_ij    = dy_ij gamma_j inv_std_i
 *              + (2 (x_ij - mean_i) dL/dvar_i + dL/dmean_i) / D
 *   dL/dvar_i  = sum_j dy_ij gamma_j (x_ij - mean_i) (-1/2) inv_std_i^3
 *   dL/dmean_i = sum_j -dy_ij gamma_j inv_std_i
 * (LnNorm::DxOp, DvarOp, DmeanOp: norm_util.h:343-421, 486-513.)  The column
 * sums are formed in a fixed order: results are bit-identical run to run.
 * Replaces FusedLayerNormGrad<GPUDevice> (fused_layer_norm_op.cu:895-1030). */
NVN_API int nvn_ln_bwd(int dtype, const void* dy, const void* x, const float* gamma,
                       const float* mean, const float* inv_std, int64_t N, int64_t D,
                       void* dx, float* dgamma, float* dbeta, void* workspace,
                       size_t workspace_bytes, void* stream);

/* ---- InstanceNorm -----------------------------------------------------------
 * x, y: [N, C, D] (channel_first != 0, "NC...") or [N, D, C] ("N...C") of T.
 * gamma, beta: [C] fp32.  mean, inv_std: [N, C] fp32.  Statistics are taken
 * over D for every (n, c).
 * Replaces FusedInstanceNorm<GPUDevice> (fused_instance_norm_op.cu:1457-1517). */
NVN_API int nvn_in_fwd(int dtype, const void* x, const float* gamma, const float* beta,
                       int64_t N, int64_t C, int64_t D, int channel_first, float epsilon,
                       void* y, float* mean, float* inv_std, void* workspace,
                       size_t workspace_bytes, void* stream);

/* dgamma_c = sum_{n,d} dy (x - mean_nc) inv_std_nc,  dbeta_c = sum_{n,d} dy,
 * dx = (S2_nc (x - mean_nc) + S1_nc) / D + dy gamma_c inv_std_nc  with
 * S1_nc = sum_d -dy inv_std gamma,  S2_nc = sum_d -dy inv_std^3 gamma (x - mean)
 * (InNorm::DwStatFusedOp, DxFusedOp: norm_util.h:518-557, 590-617).
 * Replaces FusedInstanceNormGrad<GPUDevice> (fused_instance_norm_op.cu:1519-1561). */
NVN_API int nvn_in_bwd(int dtype, const void* dy, const void* x, const float* gamma,
                       const float* mean, const float* inv_std, int64_t N, int64_t C,
                       int64_t D, int channel_first, void* dx, float* dgamma,
                       float* dbeta, void* workspace, size_t workspace_bytes,
                       void* stream);

/* ---- data-parallel backward: column reduction fused with the all-reduce -------
 * One process per GPU, every rank calling with the same N-shard shapes.  Instead of
 * finishing with a local dgamma / dbeta that the caller must all-reduce, the last
 * kernel of the backward pass exchanges the per-rank vectors over NVLink peer memory
 * and every rank ends up with the global sums (bit-identical on all ranks).
 *
 * The caller provides, for every rank r, a receive buffer that all ranks can address
 * (peer-mapped / symmetric memory, e.g. from cudaIpc*, cuMem* or torch's symmetric memory):
 *   recv[r] : nvn_dp_recv_bytes(F, world) bytes, 16-byte aligned, zero-filled once before
 *             the first call
 * in rank order (recv[rank] is this rank's own).  `epoch` must be 1 on the first call and
 * grow by one per call, the same on all ranks; calls of one communicator must not overlap
 * on a GPU.  F must be even.  A set of receive buffers is bound to ONE feature count F: the
 * slot offsets depend on F, so layers with different F need their own buffers and their
 * own epoch sequence.  Device-side waits are bounded: if a peer never shows up the kernel
 * gives up (after one time-out per thread, not one per element), nvn_device_status()
 * reports NVN_ERR_TIMEOUT and the gradients of that call are undefined.  world == 1 is
 * allowed (pure self-exchange).
 * No counterpart in the reference (its ops are single-device, norm_ops.cc has no
 * collective); this replaces the separate all-reduce of a data-parallel job. */
#define NVN_DP_MAX_RANKS 16
typedef struct nvn_dp_comm {
  int rank;
  int world;
  void* recv[NVN_DP_MAX_RANKS];
  uint32_t epoch;
  int defer; /* 0: the backward call completes the exchange.  1: it only reduces and pushes;
                nvn_dp_finish (same comm contents) waits and writes dgamma / dbeta later. */
  void* device_epochs; /* NULL, or four zero-initialised uint32 in device memory of this rank:
                the kernels then count the epochs themselves and ignore `epoch`, which makes
                the calls replayable from a CUDA graph (a replay repeats its arguments; the
                epochs must not repeat).  Every rank must use the same mode. */
} nvn_dp_comm;

/* Second half of a deferred exchange (comm->defer was 1 in the backward call of this
 * epoch): waits - bounded - for every rank's push of `comm->epoch` and writes the summed
 * dgamma / dbeta (F floats each).  May run on another stream than the backward call, after
 * it in stream / event order.  The caller must not start the backward call of epoch e on a
 * rank before that rank's nvn_dp_finish of epoch e - 2 has completed: there are four receive
 * slots (epoch mod 4), and a finish that lags its push by L epochs needs 2L of them. */
NVN_API int nvn_dp_finish(int64_t F, const nvn_dp_comm* comm, float* dgamma, float* dbeta,
                          void* stream);

NVN_API size_t nvn_dp_recv_bytes(int64_t F, int world);

NVN_API int nvn_ln_bwd_dp(int dtype, const void* dy, const void* x, const float* gamma,
                          const float* mean, const float* inv_std, int64_t N, int64_t D,
                          void* dx, float* dgamma, float* dbeta, void* workspace,
                          size_t workspace_bytes, const nvn_dp_comm* comm, void* stream);

NVN_API int nvn_in_bwd_dp(int dtype, const void* dy, const void* x, const float* gamma,
                          const float* mean, const float* inv_std, int64_t N, int64_t C,
                          int64_t D, int channel_first, void* dx, float* dgamma, float* dbeta,
                          void* workspace, size_t workspace_bytes, const nvn_dp_comm* comm,
                          void* stream);

/* ---- LayerNorm backward without a caller-provided workspace ------------------
 * Same computation and results as nvn_ln_bwd, for callers that cannot supply
 * scratch memory: a plugin callback that receives only input and output
 * pointers, a process whose device memory is entirely owned by another pool, or
 * a loop in which cudaMalloc / cudaFree are not allowed.  The dgamma / dbeta
 * partial rows go to a fixed array of NVN_NOALLOC_SCRATCH_BYTES that is part of
 * the library image (every GPU that loads the library holds it until exit).
 *   - Returns NVN_ERR_LIMIT when nvn_ln_bwd_workspace_bytes(dtype, N, D) exceeds
 *     NVN_NOALLOC_SCRATCH_BYTES; nothing is launched in that case.
 *   - Allocates nothing, on the host or the device.
 *   - All calls on a device share the array: calls that may overlap on the GPU
 *     race on it and must be ordered by the caller (one stream, or events).
 *     No part of the array needs zeroing between calls.
 *   - The first call on each device looks up the array's address; make it before
 *     any stream capture on that device.
 * This entry point has no counterpart in the reference. */
#define NVN_NOALLOC_SCRATCH_BYTES (16u << 20)
NVN_API int nvn_ln_bwd_noalloc(int dtype, const void* dy, const void* x, const float* gamma,
                               const float* mean, const float* inv_std, int64_t N, int64_t D,
                               void* dx, float* dgamma, float* dbeta, void* stream);

/* ---- introspection (for tests, benchmarks and profiles) ---------------------
 * Writes a short description of the kernel variant the dispatcher would pick,
 * e.g. "rows tpr=256 vpt=2 cluster=1 epv=8 grid=592".  op: 0 = ln_fwd,
 * 1 = ln_bwd, 2 = in_fwd, 3 = in_bwd.  C and channel_first are ignored for
 * LayerNorm.  No reference counterpart. */
NVN_API int nvn_describe_plan(int op, int dtype, int64_t N, int64_t C, int64_t D,
                              int channel_first, char* out, size_t out_bytes);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* NVNORMS_H_ */
