// nvn_ln_bwd_noalloc: LayerNorm backward for callers that have no way to hand
// the library a scratch buffer.
//
// nvn_ln_bwd needs device scratch for the per-CTA dgamma / dbeta partial rows
// and expects the caller to provide it.  Some callers cannot: an enqueue-style
// plugin callback that is given input and output pointers and nothing else (no
// temp allocator such as TensorFlow's allocate_temp), a host runtime that has
// already handed every byte of device memory to its own pool so that a raw
// cudaMalloc would fail, or a latency-critical loop in which cudaMalloc /
// cudaFree are off limits because they synchronise the device.  For them the
// scratch lives in a fixed array that is part of the library image.
//
// Consequences the caller has to know about:
//   - The array has a fixed size, NVN_NOALLOC_SCRATCH_BYTES.  Problems whose
//     partial rows do not fit are rejected with NVN_ERR_LIMIT; use nvn_ln_bwd
//     with your own workspace for those.
//   - Every GPU that loads the library carries the array until the process
//     exits, whether or not this entry point is ever called.
//   - All calls on a device share the one array.  Calls that can overlap on the
//     GPU (different streams without an ordering between them) race on it and
//     produce wrong parameter gradients; keep such calls on one stream or order
//     them with events.
//   - Nothing in the array has to start at zero: every partial row that the
//     reduction stage reads is fully overwritten by the main kernel first, so the
//     previous call's contents are harmless.
//   - The first call on each device looks up the array's device address (one
//     cudaGetSymbolAddress).  Make that first call before starting any stream
//     capture on that device.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/nvnorms.h"

namespace {

// The scratch itself.  In host code the name `g_noalloc_scratch` is only a
// handle for the runtime, not a device address; the address the kernels get
// comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NVN_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch on the current device, looked up once per device
// with that device current.  Returns a CUDA error code.
cudaError_t scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    if (p == nullptr) return cudaErrorInvalidSymbol;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int nvn_ln_bwd_noalloc(int dtype, const void* dy, const void* x, const float* gamma,
                                  const float* mean, const float* inv_std, int64_t N, int64_t D,
                                  void* dx, float* dgamma, float* dbeta, void* stream) {
  if (N < 0 || D < 0) return NVN_ERR_INVALID_ARGUMENT;
  // Empty problems need no scratch: the regular entry point only zero-fills.
  if (N == 0 || D == 0)
    return nvn_ln_bwd(dtype, dy, x, gamma, mean, inv_std, N, D, dx, dgamma, dbeta, nullptr, 0,
                      stream);
  const size_t need = nvn_ln_bwd_workspace_bytes(dtype, N, D);
  if (need > static_cast<size_t>(NVN_NOALLOC_SCRATCH_BYTES)) return NVN_ERR_LIMIT;
  void* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != cudaSuccess) {
    (void)cudaGetLastError();
    return NVN_ERR_CUDA;
  }
  return nvn_ln_bwd(dtype, dy, x, gamma, mean, inv_std, N, D, dx, dgamma, dbeta, scratch,
                    static_cast<size_t>(NVN_NOALLOC_SCRATCH_BYTES), stream);
}
