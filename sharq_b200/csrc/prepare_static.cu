// RMSNorm-fused activation prepare for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to obtain scratch memory at call time: a
// serving process that has already handed every free byte of HBM to its own pool, or a
// latency-critical thread on which cudaMalloc (which synchronises the whole device) is
// forbidden, may hold input and output buffers but no spare workspace.  For them this file
// provides a variant of sharq_fused_rmsnorm_sparse_residual_quantize_x whose scratch (the
// tensor absmax word and the per-row inv_rms values) lives in a fixed array inside the
// library image instead of a caller-provided workspace.
//
// Facts a caller must know:
//   * Capacity: kNoAllocMaxRows rows (65536); larger M is rejected with an error.  The
//     array costs 256 KiB + 256 B of device memory on every GPU that loads the library,
//     for the life of the process.
//   * The first call on each device resolves the array's device address
//     (cudaGetSymbolAddress) and caches it; that first call should be made before any
//     stream capture begins.  No call allocates or frees anything.
//   * All calls on a device share the one array.  The kernels re-initialise the word that
//     must start at zero on every call, so stale contents are harmless, but two calls that
//     overlap on the GPU (different streams without an ordering between them) race on it
//     and produce undefined results.  Serialise them, or use the workspace variant.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/sharq_b200.h"
#include "prepare.cuh"

namespace {

constexpr int kNoAllocMaxRows = 65536;
constexpr size_t kNoAllocScratchBytes = 256 + sizeof(float) * (size_t)kNoAllocMaxRows;
constexpr int kMaxDevices = 64;

// Scratch of the no-allocation entry point.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_setup_mutex;
void *g_scratch_ptr[kMaxDevices] = {};
thread_local char g_noalloc_error[256] = "";

// Device address of the scratch array on the current device (resolved once per device).
cudaError_t scratch_for_current_device(void **out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (err != cudaSuccess) return err;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" {

const char *sharq_noalloc_last_error(void) { return g_noalloc_error; }

int sharq_noalloc_max_rows(void) { return kNoAllocMaxRows; }

int sharq_fused_rmsnorm_sparse_residual_quantize_x_noalloc(const void *x, const void *gamma, float eps, int m, int n,
                                                           int k, void *a_comp, void *e, void *sfa_sparse, void *q_res,
                                                           void *sf_res, float *scale_out, void *stream) {
  (void)n;
  g_noalloc_error[0] = 0;
  if (m <= 0 || k <= 0) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "X must be shaped [M, K]");
    return 1;
  }
  if (m > kNoAllocMaxRows) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "M = %d exceeds the built-in scratch capacity of %d rows; use "
             "sharq_fused_rmsnorm_sparse_residual_quantize_x with a caller-provided workspace",
             m, kNoAllocMaxRows);
    return 1;
  }
  if (k % 128 != 0 || k / 32 > 1024) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "K must be a multiple of 128 with K/32 <= 1024, got %d", k);
    return 1;
  }
  if (!x || !gamma || !a_comp || !e || !sfa_sparse || !q_res || !sf_res) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "null buffer");
    return 1;
  }
  void *scratch = nullptr;
  cudaError_t err = scratch_for_current_device(&scratch);
  if (err == cudaSuccess)
    err = sharq::run_scaled_prepare(x, gamma, eps, m, k, scratch, nullptr, a_comp, e, sfa_sparse, q_res, sf_res,
                                    scale_out, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "fused_rmsnorm_sparse_residual_quantize_x_noalloc: %s",
             cudaGetErrorString(err));
    return 1;
  }
  return 0;
}

}  // extern "C"
