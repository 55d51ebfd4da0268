// spconv::Tensor - the tensor container of the libspconv v1.3 interface,
// re-implemented on the CUDA runtime for the B200 library.
//
// Interface parity: libraries/3DSparseConvolution/libspconv/include/spconv/tensor.hpp:28-124
// of NVIDIA-AI-IOT/Lidar_AI_Solution (names, argument order and meaning are kept so that
// callers compile unchanged).  File format of save()/load(): int32 header
// {0x33ff1101, ndim, dtype code}, int32 dims, raw data (tool/tensor.py:24-69).
#ifndef __SPCONV_TENSOR_HPP__
#define __SPCONV_TENSOR_HPP__

#include <stdint.h>
#include <stdlib.h>

#include <memory>
#include <string>
#include <vector>

namespace spconv {

#ifndef Exported
#define Exported __attribute__((visibility("default")))
#endif

// Element types; the integer values are the codes stored in tensor files.
enum class DataType : int {
  None = 0, Int32 = 1, Float16 = 2, Float32 = 3, Int64 = 4, UInt64 = 5, UInt32 = 6, Int8 = 7, UInt8 = 8
};

Exported const char* dtype_string(DataType dtype);
Exported size_t dtype_bytes(DataType dtype);
Exported float native_half2float(const unsigned short h);
Exported std::vector<int64_t> toshape(const std::vector<int>& ishape);
Exported std::vector<int> toshape(const std::vector<int64_t>& ishape);

// "2 x 3 x 4" style text of a shape.  Returns a pointer into a static buffer:
// not thread safe, valid until the next call.
template <typename _T>
Exported const char* format_shape(const std::vector<_T>& shape, bool space = true);

// A block of host or device memory.  `owner` tells whether free() releases it;
// reference() only borrows the caller's pointer.
struct TensorData {
  void* data = nullptr;
  DataType dtype = DataType::None;
  size_t bytes = 0;     // bytes in use
  size_t capacity = 0;  // bytes allocated
  bool device = true;
  bool owner = false;

  virtual ~TensorData();
  bool empty() const { return data == nullptr; }
  void free();
  void reference(void* data, size_t bytes, DataType dtype, bool device);
  void rearrange_and_realloc(size_t bytes, DataType dtype, bool device);

  static TensorData* create(size_t bytes, DataType dtype, bool device);
  static TensorData* reference_new(void* data, size_t bytes, DataType dtype, bool device);
};

struct Tensor {
  std::vector<int64_t> shape;
  std::shared_ptr<TensorData> data;
  size_t numel = 0;
  size_t ndim = 0;

  Exported Tensor() = default;
  Exported Tensor(std::vector<int64_t> shape, DataType dtype, bool device = true);

  // ---- raw access
  void* ptr() const { return data ? data->data : nullptr; }
  template <typename T> T* ptr() const { return data ? (T*)data->data : nullptr; }
  template <typename T> T* begin() const { return ptr<T>(); }
  template <typename T> T* end() const { return data ? (T*)data->data + numel : nullptr; }

  // ---- description
  Exported int64_t size(int index) const { return shape[index]; }
  Exported size_t bytes() const { return data ? data->bytes : 0; }
  Exported bool empty() const { return data == nullptr || data->empty(); }
  Exported DataType dtype() const { return data ? data->dtype : DataType::None; }
  Exported bool device() const { return data ? data->device : false; }

  // ---- storage
  Exported void create_(const std::vector<int64_t>& shape, DataType dtype, bool device = true);
  Exported void reference(void* data, std::vector<int64_t> shape, DataType dtype, bool device = true);
  Exported void memset(unsigned char value = 0, void* stream = nullptr);
  Exported void arange(size_t num, void* stream = nullptr);

  // ---- movement and conversion (the *_ forms work in place)
  Exported void to_device_(void* stream = nullptr);
  Exported void to_host_(void* stream = nullptr);
  Exported Tensor to_device(void* stream = nullptr) const;
  Exported Tensor to_host(void* stream = nullptr) const;
  Exported Tensor clone(void* stream = nullptr) const;
  Exported Tensor to_half(void* stream = nullptr) const;
  Exported float absmax(void* stream = nullptr) const;

  // ---- output
  Exported void print(const char* prefix = "Tensor", size_t offset = 0, size_t num_per_line = 10,
                      size_t lines = 1, void* stream = nullptr) const;
  Exported bool save(const char* file, void* stream = nullptr) const;

  // ---- factories
  Exported static Tensor create(std::vector<int64_t> shape, DataType dtype, bool device = true);
  Exported static Tensor create(std::vector<int32_t> shape, DataType dtype, bool device = true);
  Exported static Tensor from_data(void* data, std::vector<int64_t> shape, DataType dtype,
                                   bool device = true, void* stream = nullptr);
  Exported static Tensor from_data(void* data, std::vector<int32_t> shape, DataType dtype,
                                   bool device = true, void* stream = nullptr);
  Exported static Tensor from_data_reference(void* data, std::vector<int64_t> shape,
                                             DataType dtype, bool device = true);
  Exported static Tensor load(const char* file, bool device = true, void* stream = nullptr);
  Exported static Tensor load_from_raw(const char* file, std::vector<int64_t> shape,
                                       DataType dtype, bool device = true, void* stream = nullptr);
  Exported static bool save(const Tensor& tensor, const char* file, void* stream = nullptr);
};

}  // namespace spconv

#endif  // __SPCONV_TENSOR_HPP__
