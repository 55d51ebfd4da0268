// Error-reporting helpers of the v1.3 interface
// (libraries/3DSparseConvolution/libspconv/include/spconv/check.hpp:23-57): CUDA errors and
// failed assertions are reported through the logger, nothing aborts.
#ifndef __SPCONV_CHECK_HPP__
#define __SPCONV_CHECK_HPP__

#include <cuda_runtime.h>

#include <string>

#include <spconv/engine.hpp>

namespace spconv {

Exported std::string format(const char* fmt, ...);
Exported bool check_cuda_api_(cudaError_t e, const char* call, int line, const char* file);

#define check_cuda_api(call) spconv::check_cuda_api_(call, #call, __LINE__, __FILE__)

#define check_cuda_kernel(...)                                                          \
  do {                                                                                  \
    __VA_ARGS__;                                                                        \
    spconv::check_cuda_api_(cudaPeekAtLastError(), #__VA_ARGS__, __LINE__, __FILE__);   \
  } while (0)

#define spconv_logf(level, fmt, ...) spconv::logger_output(__FILE__, __LINE__, level, fmt, __VA_ARGS__);
#define spconv_log(level, msg) spconv::logger_output(__FILE__, __LINE__, level, "%s", msg);

#define spconv_assert(cond)                                                                     \
  do {                                                                                          \
    if (!(cond))                                                                                \
      spconv::logger_output(__FILE__, __LINE__, spconv::LoggerLevel::Error,                     \
                            "Assert failed: %s in file %s:%d", #cond, __FILE__, __LINE__);      \
  } while (false)

#define spconv_asserts(cond, s)                                                                 \
  do {                                                                                          \
    if (!(cond))                                                                                \
      spconv::logger_output(__FILE__, __LINE__, spconv::LoggerLevel::Error,                     \
                            "Assert failed: %s in file %s:%d, message: " s, #cond, __FILE__,    \
                            __LINE__);                                                          \
  } while (false)

#define spconv_assertf(cond, fmt, ...)                                                          \
  do {                                                                                          \
    if (!(cond))                                                                                \
      spconv::logger_output(__FILE__, __LINE__, spconv::LoggerLevel::Error,                     \
                            "Assert failed: %s in file %s:%d, message: " fmt, #cond, __FILE__,  \
                            __LINE__, __VA_ARGS__);                                             \
  } while (false)

}  // namespace spconv

#endif  // __SPCONV_CHECK_HPP__
