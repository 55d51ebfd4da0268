// The libspconv v1.0 C++ interface, as CUDA-CenterPoint uses it, for the B200 library
// (libspconv_v10.so; a thin layer over the C ABI of spconvb.h).
//
// Interface parity: CUDA-CenterPoint/3rdparty/libspconv/include/spconv/engine.hpp:34-115 of
// NVIDIA-AI-IOT/Lidar_AI_Solution: same names, virtual order, argument order and defaults.
#ifndef __SPCONV_ENGINE_HPP__
#define __SPCONV_ENGINE_HPP__

#include <memory>
#include <string>
#include <vector>

namespace spconv {

#ifndef Exported
#define Exported __attribute__((visibility("default")))
#endif

enum class DType : int { None = 0, Int32 = 1, Float16 = 2 };
enum class Precision : int { None = 0, Float16 = 1, Int8 = 2 };

// The result of Engine::forward.  It belongs to the engine and is valid, once the stream has
// run, until the next forward.  For a model ending in ScatterDense, features_data() is the
// dense fp16 tensor (e.g. [1, 256, 180, 180]).
class DTensor {
 public:
  virtual std::vector<int64_t> features_shape() const = 0;
  virtual DType features_dtype() const = 0;
  virtual void* features_data() = 0;

  virtual std::vector<int64_t> indices_shape() const = 0;
  virtual DType indices_dtype() const = 0;
  virtual void* indices_data() = 0;

  virtual std::vector<int> grid_size() const = 0;
  virtual int device() const = 0;
};

class Engine {
 public:
  // features_data: device pointer, Float16 [n, C]; indices_data: device pointer, Int32 [n, 4]
  // = (batch, c0, c1, c2); batch must be 1; grid_size e.g. {41, 1440, 1440}.  The work is
  // enqueued on `stream`.
  Exported virtual DTensor* forward(const std::vector<int64_t>& features_shape, DType features_dtype,
                                    void* features_data, const std::vector<int64_t>& indices_shape,
                                    DType indices_dtype, void* indices_data, int batch,
                                    std::vector<int> grid_size, void* stream = nullptr) = 0;

  // The four calls below belong to the reference's implicit-calibration workflow.  This
  // library takes precisions and dynamic ranges from the model file only: they log a warning
  // and change nothing.
  Exported virtual void reconfigure() = 0;
  Exported virtual void set_int8_calibration(bool enable) = 0;
  Exported virtual void set_node_precision_byname(const char* name, Precision compute_precision,
                                                  Precision output_precision) = 0;
  Exported virtual void set_node_precision_byoptype(const char* optype, Precision compute_precision,
                                                    Precision output_precision) = 0;
};

// precision == Float16 ignores the per-layer precision attributes of the file.
// Returns a null pointer when the file cannot be loaded.
Exported std::shared_ptr<Engine> load_engine_from_onnx(const std::string& onnx_file,
                                                       Precision precision = Precision::Float16);

Exported void set_verbose(bool enable);
Exported const char* get_precision_string(Precision precision);

}  // namespace spconv

#endif  // __SPCONV_ENGINE_HPP__
