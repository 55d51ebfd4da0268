// The libspconv v1.3 C++ interface (EngineBuilder / Engine / SparseDTensor / logging) for the
// B200 library.  Every class here is a thin layer over the C ABI in spconvb.h.
//
// Interface parity: libraries/3DSparseConvolution/libspconv/include/spconv/engine.hpp:25-176 of
// NVIDIA-AI-IOT/Lidar_AI_Solution.  Virtual function order, argument order and defaults are
// the reference's, so code written against it compiles and links unchanged.
#ifndef __SPCONV_ENGINE_HPP__
#define __SPCONV_ENGINE_HPP__

#include <memory>
#include <string>
#include <vector>

#include <spconv/tensor.hpp>

namespace spconv {

#ifndef Exported
#define Exported __attribute__((visibility("default")))
#endif

enum class Precision : int { None = 0, Float16 = 1, Int8 = 2 };
enum class TensorLayout : int { None = 0, NCHW = 1, NCHW32 = 2, NHWzC = 3 };
enum class LoggerLevel : int { Verb = 0, Warn = 1, Error = 2, Quiet = 99 };

// ---------------------------------------------------------------- logging
class ILogger {
 public:
  virtual ~ILogger() = default;
  virtual void log(const char* message, LoggerLevel level, const char* file, int line) const = 0;
};

Exported void set_logger(ILogger* logger);
Exported ILogger* get_logger();
Exported void set_logger_level(LoggerLevel level);
Exported LoggerLevel get_logger_level();
Exported const char* logger_level_string(LoggerLevel level);
Exported void logger_output(const char* file, int line, LoggerLevel level, const char* fmt, ...);
Exported const char* get_precision_string(Precision precision);
Exported const char* get_tensor_layout_string(TensorLayout layout);

// ---------------------------------------------------------------- run time
// One sparse (or, for a ScatterDense result, dense) tensor of an engine.
// features(): [rows, channels] (dense: e.g. [1, 256, 180, 180]);
// indices():  int32 [rows, 4] = (batch, c0, c1, c2).
class SparseDTensor {
 public:
  virtual ~SparseDTensor() {}
  virtual Tensor& features() = 0;
  virtual Tensor& indices() = 0;
  virtual void set_grid_size(const std::vector<int>& grid_size) = 0;
  virtual std::vector<int> grid_size() const = 0;
  virtual int device() const = 0;
  virtual const char* name() const = 0;
  // DDS: a device word holding the number of valid rows, read by the kernels, so that the
  // bound buffers (and a captured CUDA graph) can stay fixed while the row count changes.
  virtual void set_dds_num_of_points_pointer(uint32_t* pointer) = 0;
  virtual uint32_t* get_dds_num_of_points_pointer() = 0;
};

class Engine {
 public:
  Exported virtual ~Engine() {}
  // Enqueue one inference on `stream`.  Bind the input first:
  //   input(0)->features().reference(ptr, {n, C}, DataType::Float16);
  //   input(0)->indices().reference(ptr, {n, 4}, DataType::Int32);
  //   input(0)->set_grid_size({41, 1440, 1440});
  // Outputs are valid once the stream has run; batch size is 1.
  Exported virtual void forward(void* stream = nullptr) = 0;
  Exported virtual size_t num_input() const = 0;
  Exported virtual SparseDTensor* input(unsigned int index) = 0;
  Exported virtual size_t num_output() const = 0;
  Exported virtual SparseDTensor* output(unsigned int index) = 0;
};

// ---------------------------------------------------------------- build time
class ITensor {
 public:
  virtual ~ITensor() {}
  virtual const char* name() = 0;
};

class INode {
 public:
  virtual ~INode() {}
  virtual const char* name() = 0;
  virtual const char* optype() = 0;
  virtual ITensor* input(unsigned int index) = 0;
  virtual ITensor* output(unsigned int index) = 0;
  virtual unsigned int num_output() = 0;
  virtual unsigned int num_input() = 0;
};

class EngineBuilder {
 public:
  Exported virtual ~EngineBuilder() {}
  Exported virtual ITensor* push_input(const char* name) = 0;

  Exported virtual INode* push_add(const char* name, ITensor* a, ITensor* b, float a_dynamic_range,
                                   float b_dynamic_range, const char* output_name,
                                   Precision precision, Precision output_precision,
                                   uint32_t fixed_launch_points) = 0;

  Exported virtual INode* push_relu(const char* name, ITensor* x, const char* output_name) = 0;

  // input_dynamic_range is used when the dense output is int8
  Exported virtual INode* push_dense(const char* name, ITensor* x, const char* format,
                                     const char* output_name,
                                     const std::vector<int>& input_spatial_shape,
                                     const std::vector<int>& output_shape,
                                     TensorLayout output_layout = TensorLayout::NCHW,
                                     float input_dynamic_range = 0.0f,
                                     uint32_t input_bound = 0) = 0;

  Exported virtual INode* push_reshape(const char* name, ITensor* x,
                                       const std::vector<int64_t>& shape,
                                       const char* output_name) = 0;

  Exported virtual INode* push_transpose(const char* name, ITensor* x,
                                         const std::vector<int64_t>& dims,
                                         const char* output_name) = 0;

  // weight: fp16 bits [Cout, k0, k1, k2, Cin]; bias: fp16 bits [Cout]
  Exported virtual INode* push_sparse_conv(
      const char* name, ITensor* x, const std::vector<unsigned short>& weight,
      const std::vector<int>& weight_shape, const std::vector<float>& weight_dynamic_ranges,
      const std::vector<unsigned short>& bias, const std::vector<int>& bias_shape,
      const char* activation, const std::vector<int>& kernel_size, const std::vector<int>& stride,
      const std::vector<int>& padding, const std::vector<int>& dilation,
      float input_dynamic_range, bool submanifold, uint32_t max_output_points,
      uint32_t fixed_launch_points, const char* rulebook, Precision precision,
      Precision output_precision, const char* output_name, bool inverse) = 0;

  Exported virtual void push_output(ITensor* value) = 0;

  // sortmask, enable_blackwell and with_auxiliary_stream are accepted for source
  // compatibility; this library has a single (Blackwell) kernel path.
  Exported virtual std::shared_ptr<Engine> build(Precision precision, bool sortmask = false,
                                                 bool enable_blackwell = false,
                                                 bool with_auxiliary_stream = false,
                                                 void* stream = nullptr) = 0;
};

Exported std::shared_ptr<EngineBuilder> create_engine_builder();

}  // namespace spconv

#endif  // __SPCONV_ENGINE_HPP__
