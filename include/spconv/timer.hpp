// spconv::EventTimer: elapsed device time between start(stream) and stop()
// (interface of libraries/3DSparseConvolution/libspconv/include/spconv/timer.hpp:22-51).
#ifndef __SPCONV_TIMER_HPP__
#define __SPCONV_TIMER_HPP__

#include <cuda_runtime.h>
#include <stdio.h>

#include <spconv/check.hpp>

namespace spconv {

class EventTimer {
 public:
  EventTimer() {
    check_cuda_api(cudaEventCreate(&t0_));
    check_cuda_api(cudaEventCreate(&t1_));
  }
  virtual ~EventTimer() {
    check_cuda_api(cudaEventDestroy(t0_));
    check_cuda_api(cudaEventDestroy(t1_));
  }
  EventTimer(const EventTimer&) = delete;
  EventTimer& operator=(const EventTimer&) = delete;

  void start(void* stream) {
    stream_ = (cudaStream_t)stream;
    check_cuda_api(cudaEventRecord(t0_, stream_));
  }

  // Milliseconds since start(); synchronises on the stop event.
  float stop(const char* prefix, bool print = true) {
    float ms = 0.f;
    check_cuda_api(cudaEventRecord(t1_, stream_));
    check_cuda_api(cudaEventSynchronize(t1_));
    check_cuda_api(cudaEventElapsedTime(&ms, t0_, t1_));
    if (print) printf("[Times %s]: %.3f ms\n", prefix, ms);
    return ms;
  }

 private:
  cudaStream_t stream_ = nullptr;
  cudaEvent_t t0_ = nullptr, t1_ = nullptr;
};

}  // namespace spconv

#endif  // __SPCONV_TIMER_HPP__
