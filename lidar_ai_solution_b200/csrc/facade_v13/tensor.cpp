// spconv::Tensor / TensorData for the v1.3 interface (see include/spconv/tensor.hpp).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <spconv/check.hpp>
#include <spconv/tensor.hpp>

namespace spconv {

namespace {
constexpr int32_t kTensorMagic = 0x33ff1101;
size_t count_of(const std::vector<int64_t>& shape) {
  size_t n = shape.empty() ? 0 : 1;
  for (auto v : shape) n *= (size_t)(v < 0 ? 0 : v);
  return n;
}
cudaStream_t S(void* stream) { return (cudaStream_t)stream; }
}  // namespace

const char* dtype_string(DataType dtype) {
  switch (dtype) {
    case DataType::Int32: return "Int32";
    case DataType::Float16: return "Float16";
    case DataType::Float32: return "Float32";
    case DataType::Int64: return "Int64";
    case DataType::UInt64: return "UInt64";
    case DataType::UInt32: return "UInt32";
    case DataType::Int8: return "Int8";
    case DataType::UInt8: return "UInt8";
    default: return "None";
  }
}

size_t dtype_bytes(DataType dtype) {
  switch (dtype) {
    case DataType::Int32: case DataType::Float32: case DataType::UInt32: return 4;
    case DataType::Float16: return 2;
    case DataType::Int64: case DataType::UInt64: return 8;
    case DataType::Int8: case DataType::UInt8: return 1;
    default: return 0;
  }
}

float native_half2float(const unsigned short h) {
  __half_raw r;
  r.x = h;
  return __half2float(__half(r));
}

std::vector<int64_t> toshape(const std::vector<int>& ishape) {
  return std::vector<int64_t>(ishape.begin(), ishape.end());
}
std::vector<int> toshape(const std::vector<int64_t>& ishape) {
  std::vector<int> out;
  for (auto v : ishape) out.push_back((int)v);
  return out;
}

template <typename _T>
const char* format_shape(const std::vector<_T>& shape, bool space) {
  static char buf[256];
  size_t pos = 0;
  buf[0] = 0;
  for (size_t i = 0; i < shape.size() && pos + 32 < sizeof(buf); ++i) {
    pos += snprintf(buf + pos, sizeof(buf) - pos, "%lld", (long long)shape[i]);
    if (i + 1 < shape.size()) pos += snprintf(buf + pos, sizeof(buf) - pos, space ? " x " : "x");
  }
  return buf;
}
template Exported const char* format_shape<int>(const std::vector<int>&, bool);
template Exported const char* format_shape<int64_t>(const std::vector<int64_t>&, bool);
template Exported const char* format_shape<unsigned int>(const std::vector<unsigned int>&, bool);
template Exported const char* format_shape<size_t>(const std::vector<size_t>&, bool);

// ------------------------------------------------------------- TensorData
TensorData::~TensorData() { free(); }

void TensorData::free() {
  if (data && owner) {
    if (device) check_cuda_api(cudaFree(data));
    else check_cuda_api(cudaFreeHost(data));
  }
  data = nullptr;
  bytes = capacity = 0;
  owner = false;
}

void TensorData::reference(void* p, size_t nbytes, DataType dt, bool dev) {
  free();
  data = p;
  bytes = capacity = nbytes;
  dtype = dt;
  device = dev;
  owner = false;
}

void TensorData::rearrange_and_realloc(size_t nbytes, DataType dt, bool dev) {
  if (!owner || dev != device || nbytes > capacity) {
    free();
    if (nbytes) {
      if (dev) check_cuda_api(cudaMalloc(&data, nbytes));
      else check_cuda_api(cudaMallocHost(&data, nbytes));
    }
    capacity = nbytes;
    owner = true;
  }
  bytes = nbytes;
  dtype = dt;
  device = dev;
}

TensorData* TensorData::create(size_t nbytes, DataType dt, bool dev) {
  TensorData* t = new TensorData();
  t->rearrange_and_realloc(nbytes, dt, dev);
  return t;
}

TensorData* TensorData::reference_new(void* p, size_t nbytes, DataType dt, bool dev) {
  TensorData* t = new TensorData();
  t->reference(p, nbytes, dt, dev);
  return t;
}

// ----------------------------------------------------------------- Tensor
Tensor::Tensor(std::vector<int64_t> shape_, DataType dtype, bool device) { create_(shape_, dtype, device); }

void Tensor::create_(const std::vector<int64_t>& shape_, DataType dtype, bool device) {
  shape = shape_;
  ndim = shape.size();
  numel = count_of(shape);
  if (!data) data.reset(new TensorData());
  data->rearrange_and_realloc(numel * dtype_bytes(dtype), dtype, device);
}

void Tensor::reference(void* p, std::vector<int64_t> shape_, DataType dtype, bool device) {
  shape = shape_;
  ndim = shape.size();
  numel = count_of(shape);
  if (!data) data.reset(new TensorData());
  data->reference(p, numel * dtype_bytes(dtype), dtype, device);
}

Tensor Tensor::create(std::vector<int64_t> shape_, DataType dtype, bool device) {
  return Tensor(shape_, dtype, device);
}
Tensor Tensor::create(std::vector<int32_t> shape_, DataType dtype, bool device) {
  return Tensor(toshape(shape_), dtype, device);
}

Tensor Tensor::from_data_reference(void* p, std::vector<int64_t> shape_, DataType dtype, bool device) {
  Tensor t;
  t.reference(p, shape_, dtype, device);
  return t;
}

Tensor Tensor::from_data(void* p, std::vector<int64_t> shape_, DataType dtype, bool device, void* stream) {
  Tensor t(shape_, dtype, device);
  if (t.bytes()) {
    check_cuda_api(cudaMemcpyAsync(t.ptr(), p, t.bytes(), cudaMemcpyDefault, S(stream)));
    check_cuda_api(cudaStreamSynchronize(S(stream)));
  }
  return t;
}
Tensor Tensor::from_data(void* p, std::vector<int32_t> shape_, DataType dtype, bool device, void* stream) {
  return from_data(p, toshape(shape_), dtype, device, stream);
}

void Tensor::memset(unsigned char value, void* stream) {
  if (empty()) return;
  if (device()) check_cuda_api(cudaMemsetAsync(ptr(), value, bytes(), S(stream)));
  else ::memset(ptr(), value, bytes());
}

Tensor Tensor::clone(void* stream) const {
  if (empty()) return Tensor();
  Tensor t(shape, dtype(), device());
  check_cuda_api(cudaMemcpyAsync(t.ptr(), ptr(), bytes(), cudaMemcpyDefault, S(stream)));
  check_cuda_api(cudaStreamSynchronize(S(stream)));
  return t;
}

static Tensor moved_copy(const Tensor& src, bool device, void* stream) {
  if (src.empty()) return Tensor();
  Tensor t(src.shape, src.dtype(), device);
  check_cuda_api(cudaMemcpyAsync(t.ptr(), src.ptr(), src.bytes(), cudaMemcpyDefault, S(stream)));
  check_cuda_api(cudaStreamSynchronize(S(stream)));
  return t;
}

Tensor Tensor::to_device(void* stream) const { return device() ? *this : moved_copy(*this, true, stream); }
Tensor Tensor::to_host(void* stream) const { return !device() ? *this : moved_copy(*this, false, stream); }
void Tensor::to_device_(void* stream) {
  if (!empty() && !device()) *this = moved_copy(*this, true, stream);
}
void Tensor::to_host_(void* stream) {
  if (!empty() && device()) *this = moved_copy(*this, false, stream);
}

void Tensor::arange(size_t num, void* stream) {
  Tensor host({(int64_t)num}, DataType::Int32, false);
  for (size_t i = 0; i < num; ++i) host.ptr<int32_t>()[i] = (int32_t)i;
  *this = device() || empty() ? host.to_device(stream) : host;
}

// element i of a host tensor as double
static double host_value(const Tensor& t, size_t i) {
  switch (t.dtype()) {
    case DataType::Int32: return t.ptr<int32_t>()[i];
    case DataType::Float16: return native_half2float(t.ptr<unsigned short>()[i]);
    case DataType::Float32: return t.ptr<float>()[i];
    case DataType::Int64: return (double)t.ptr<int64_t>()[i];
    case DataType::UInt64: return (double)t.ptr<uint64_t>()[i];
    case DataType::UInt32: return t.ptr<uint32_t>()[i];
    case DataType::Int8: return t.ptr<int8_t>()[i];
    case DataType::UInt8: return t.ptr<uint8_t>()[i];
    default: return 0.0;
  }
}

Tensor Tensor::to_half(void* stream) const {
  if (empty() || dtype() == DataType::Float16) return *this;
  Tensor h = to_host(stream);
  Tensor out(shape, DataType::Float16, false);
  for (size_t i = 0; i < numel; ++i) {
    __half_raw r = __half_raw(__float2half_rn((float)host_value(h, i)));
    out.ptr<unsigned short>()[i] = r.x;
  }
  return device() ? out.to_device(stream) : out;
}

float Tensor::absmax(void* stream) const {
  if (empty()) return 0.f;
  Tensor h = to_host(stream);
  double m = 0.0;
  for (size_t i = 0; i < numel; ++i) m = fmax(m, fabs(host_value(h, i)));
  return (float)m;
}

void Tensor::print(const char* prefix, size_t offset, size_t num_per_line, size_t lines, void* stream) const {
  printf("%s[%s, %s, %s]", prefix, dtype_string(dtype()), format_shape(shape), device() ? "device" : "host");
  if (empty()) {
    printf(": empty\n");
    return;
  }
  Tensor h = to_host(stream);
  size_t i = offset;
  for (size_t l = 0; l < lines && i < numel; ++l) {
    printf("\n  ");
    for (size_t c = 0; c < num_per_line && i < numel; ++c, ++i) printf("%g ", host_value(h, i));
  }
  printf("\n");
}

bool Tensor::save(const char* file, void* stream) const { return save(*this, file, stream); }

bool Tensor::save(const Tensor& tensor, const char* file, void* stream) {
  FILE* f = fopen(file, "wb");
  if (!f) {
    spconv_logf(LoggerLevel::Error, "Failed to open %s for writing", file);
    return false;
  }
  Tensor h = tensor.to_host(stream);
  int32_t head[3] = {kTensorMagic, (int32_t)tensor.ndim, (int32_t)tensor.dtype()};
  bool ok = fwrite(head, sizeof(head), 1, f) == 1;
  for (auto d : tensor.shape) {
    int32_t v = (int32_t)d;
    ok = ok && fwrite(&v, 4, 1, f) == 1;
  }
  if (h.bytes()) ok = ok && fwrite(h.ptr(), 1, h.bytes(), f) == h.bytes();
  fclose(f);
  return ok;
}

Tensor Tensor::load(const char* file, bool device, void* stream) {
  FILE* f = fopen(file, "rb");
  if (!f) {
    spconv_logf(LoggerLevel::Error, "Failed to open %s", file);
    return Tensor();
  }
  int32_t head[3] = {0, 0, 0};
  Tensor out;
  if (fread(head, sizeof(head), 1, f) == 1 && head[0] == kTensorMagic && head[1] >= 0 && head[1] <= 16 &&
      dtype_bytes((DataType)head[2]) > 0) {
    std::vector<int64_t> shape;
    bool ok = true;
    for (int i = 0; i < head[1]; ++i) {
      int32_t d = 0;
      ok = ok && fread(&d, 4, 1, f) == 1 && d >= 0;
      shape.push_back(d);
    }
    if (ok) {
      Tensor host(shape, (DataType)head[2], false);
      ok = host.bytes() == 0 || fread(host.ptr(), 1, host.bytes(), f) == host.bytes();
      if (ok) out = device ? host.to_device(stream) : host;
    }
    if (!ok) spconv_logf(LoggerLevel::Error, "Tensor file %s is truncated", file);
  } else {
    spconv_logf(LoggerLevel::Error, "%s is not a tensor file", file);
  }
  fclose(f);
  return out;
}

Tensor Tensor::load_from_raw(const char* file, std::vector<int64_t> shape_, DataType dtype, bool device,
                             void* stream) {
  FILE* f = fopen(file, "rb");
  if (!f) {
    spconv_logf(LoggerLevel::Error, "Failed to open %s", file);
    return Tensor();
  }
  Tensor host(shape_, dtype, false);
  const bool ok = host.bytes() == 0 || fread(host.ptr(), 1, host.bytes(), f) == host.bytes();
  fclose(f);
  if (!ok) {
    spconv_logf(LoggerLevel::Error, "%s holds fewer than %zu bytes", file, host.bytes());
    return Tensor();
  }
  return device ? host.to_device(stream) : host;
}

}  // namespace spconv
