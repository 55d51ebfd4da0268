// Growable host-pinned and device buffers, and a name-keyed pool of device buffers, with the
// class and method names of the v1.3 interface
// (libraries/3DSparseConvolution/libspconv/include/spconv/memory.hpp:24-183).  Header only.
#ifndef __SPCONV_MEMORY_HPP__
#define __SPCONV_MEMORY_HPP__

#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <unordered_map>

#include <spconv/check.hpp>

namespace spconv {

namespace detail {
// Shared behaviour of the two buffer kinds: grow-only capacity, logical size <= capacity.
template <bool kDevice>
class GrowBuffer {
 public:
  GrowBuffer() = default;
  explicit GrowBuffer(const std::string& name) : name_(name) {}
  GrowBuffer(const GrowBuffer&) = delete;
  GrowBuffer& operator=(const GrowBuffer&) = delete;
  virtual ~GrowBuffer() { free_memory(nullptr); }

  void* ptr() const { return ptr_; }
  size_t bytes() const { return bytes_; }
  bool empty() const { return ptr_ == nullptr; }

  void alloc_or_resize_to(size_t nbytes, cudaStream_t stream) {
    if (nbytes > capacity_) {
      free_memory(stream);
      if (kDevice) check_cuda_api(cudaMalloc(&ptr_, nbytes));
      else check_cuda_api(cudaMallocHost(&ptr_, nbytes));
      capacity_ = nbytes;
    }
    bytes_ = nbytes;
  }
  void alloc(size_t nbytes, cudaStream_t stream) { alloc_or_resize_to(nbytes, stream); }

  // Shrink or re-grow inside the existing allocation; never allocates.
  void resize(size_t nbytes) {
    spconv_assertf(nbytes <= capacity_, "%s Failed to resize memory to %ld bytes. capacity = %ld",
                   name_.c_str(), (long)nbytes, (long)capacity_);
    if (nbytes <= capacity_) bytes_ = nbytes;
  }

  void free_memory(cudaStream_t) {
    if (!ptr_) return;
    if (kDevice) check_cuda_api(cudaFree(ptr_));
    else check_cuda_api(cudaFreeHost(ptr_));
    ptr_ = nullptr;
    bytes_ = capacity_ = 0;
  }

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0, capacity_ = 0;
  std::string name_;
};
}  // namespace detail

class PinnedMemoryData : public detail::GrowBuffer<false> {
 public:
  using detail::GrowBuffer<false>::GrowBuffer;
};

class GPUData : public detail::GrowBuffer<true> {
 public:
  using detail::GrowBuffer<true>::GrowBuffer;
};

// Typed view over a shared GPUData.
template <typename T>
class GPUMemory {
 public:
  virtual ~GPUMemory() { data_.reset(); }
  void set_gpudata(std::shared_ptr<GPUData> data) { data_ = data; }
  T* ptr() const { return data_ ? (T*)data_->ptr() : nullptr; }
  size_t size() const { return size_; }
  size_t bytes() const { return data_ ? data_->bytes() : 0; }
  bool empty() const { return !data_ || data_->empty(); }
  bool unset() const { return data_ == nullptr; }

  void alloc_or_resize_to(size_t size, cudaStream_t stream) {
    spconv_asserts(data_ != nullptr, "Failed to alloc or resize memory that because data is nullptr.");
    if (!data_) return;
    size_ = size;
    data_->alloc_or_resize_to(size * sizeof(T), stream);
  }
  void alloc(size_t size, cudaStream_t stream) { alloc_or_resize_to(size, stream); }
  void resize(size_t size) {
    spconv_asserts(data_ != nullptr, "Failed to resize memory that because data is nullptr.");
    if (!data_) return;
    size_ = size;
    data_->resize(size * sizeof(T));
  }

 private:
  std::shared_ptr<GPUData> data_;
  size_t size_ = 0;
};

// Buffers looked up by tensor id, so that tensors with the same id share memory.  The id
// "__no_reuse_policy_here__" always yields a fresh, unshared buffer.
class GPUDataManager {
 public:
  explicit GPUDataManager(size_t max_bytes_for_io_tensor = 0)
      : max_bytes_for_io_tensor_(max_bytes_for_io_tensor) {}

  std::shared_ptr<GPUData> query_or_alloc(const std::string& tensor_id, bool is_iotensor = false,
                                          cudaStream_t stream = nullptr) {
    if (tensor_id == "__no_reuse_policy_here__") return std::make_shared<GPUData>(tensor_id);
    std::shared_ptr<GPUData>& slot = pool_[tensor_id];
    if (!slot) {
      slot = std::make_shared<GPUData>(tensor_id);
      if (is_iotensor && max_bytes_for_io_tensor_ > 0) slot->alloc(max_bytes_for_io_tensor_, stream);
    }
    return slot;
  }

 private:
  size_t max_bytes_for_io_tensor_ = 0;
  std::unordered_map<std::string, std::shared_ptr<GPUData>> pool_;
};

}  // namespace spconv

#endif  // __SPCONV_MEMORY_HPP__
