// Small device helpers of the engine.
#include "common.cuh"

namespace spconvb {

__global__ void set_count_kernel(uint32_t* dst, uint32_t value) { *dst = value; }

// Publishes a host-known row count to the device word the kernels read.  The
// value travels as a kernel argument, so no host buffer has to outlive the call.
int launch_set_count(uint32_t* dst, uint32_t value, cudaStream_t st) {
  set_count_kernel<<<1, 1, 0, st>>>(dst, value);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

__global__ void clamp_count_kernel(uint32_t* dst, const uint32_t* src, uint32_t cap,
                                   uint32_t* status) {
  const uint32_t n = *src;
  if (n > cap) set_status(status, SPCONVB_ST_OVERFLOW, n);
  *dst = min(n, cap);
}

// The caller's device-side row count, clamped to the rows its buffers hold, in the word the
// engine's kernels read; a larger count sets SPCONVB_ST_OVERFLOW.
int launch_clamp_count(uint32_t* dst, const uint32_t* src, uint32_t cap, uint32_t* status,
                       cudaStream_t st) {
  clamp_count_kernel<<<1, 1, 0, st>>>(dst, src, cap, status);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

}  // namespace spconvb
