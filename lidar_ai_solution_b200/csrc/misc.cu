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

}  // namespace spconvb
