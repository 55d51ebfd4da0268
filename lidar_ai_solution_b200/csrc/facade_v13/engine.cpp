// EngineBuilder / Engine / logging of the v1.3 interface on top of the C ABI
// (include/spconv/engine.hpp; spconvb.h).
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <memory>
#include <string>
#include <vector>

#include <spconv/check.hpp>
#include <spconv/engine.hpp>
#include <spconv/onnx-parser.hpp>

#include "spconvb.h"

namespace spconv {

// ------------------------------------------------------------------ logging
namespace {
ILogger* g_logger = nullptr;
LoggerLevel g_level = LoggerLevel::Warn;

void core_log_bridge(int32_t level, const char* message) {
  const LoggerLevel l = level <= 0 ? LoggerLevel::Verb : (level == 1 ? LoggerLevel::Warn : LoggerLevel::Error);
  logger_output("libspconvb", 0, l, "%s", message);
}
struct BridgeInstaller {
  BridgeInstaller() {
    spconvb_set_log_callback(core_log_bridge);
    spconvb_set_log_level(0);  // filtering happens in logger_output
  }
} g_bridge_installer;
}  // namespace

void set_logger(ILogger* logger) { g_logger = logger; }
ILogger* get_logger() { return g_logger; }
void set_logger_level(LoggerLevel level) { g_level = level; }
LoggerLevel get_logger_level() { return g_level; }

const char* logger_level_string(LoggerLevel level) {
  switch (level) {
    case LoggerLevel::Verb: return "verb";
    case LoggerLevel::Warn: return "warn";
    case LoggerLevel::Error: return "error";
    case LoggerLevel::Quiet: return "quiet";
  }
  return "unknown";
}

void logger_output(const char* file, int line, LoggerLevel level, const char* fmt, ...) {
  if ((int)level < (int)g_level) return;
  char msg[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  if (g_logger) {
    g_logger->log(msg, level, file, line);
    return;
  }
  fprintf(level == LoggerLevel::Error ? stderr : stdout, "[%s][%s:%d]: %s\n", logger_level_string(level),
          file ? file : "", line, msg);
}

const char* get_precision_string(Precision precision) {
  switch (precision) {
    case Precision::Float16: return "Float16";
    case Precision::Int8: return "Int8";
    default: return "None";
  }
}

const char* get_tensor_layout_string(TensorLayout layout) {
  switch (layout) {
    case TensorLayout::NCHW: return "NCHW";
    case TensorLayout::NCHW32: return "NCHW32";
    case TensorLayout::NHWzC: return "NHWzC";
    default: return "None";
  }
}

std::string format(const char* fmt, ...) {
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return buf;
}

bool check_cuda_api_(cudaError_t e, const char* call, int line, const char* file) {
  if (e == cudaSuccess) return true;
  logger_output(file, line, LoggerLevel::Error, "CUDA Runtime error %s # %s, code = %s [ %d ]", call,
                cudaGetErrorString(e), cudaGetErrorName(e), (int)e);
  return false;
}

// --------------------------------------------------------------- run time
namespace {

class SparseTensorImpl : public SparseDTensor {
 public:
  explicit SparseTensorImpl(const std::string& name) : name_(name) {}
  Tensor& features() override { return features_; }
  Tensor& indices() override { return indices_; }
  void set_grid_size(const std::vector<int>& grid_size) override { grid_ = grid_size; }
  std::vector<int> grid_size() const override { return grid_; }
  int device() const override { return device_; }
  const char* name() const override { return name_.c_str(); }
  void set_dds_num_of_points_pointer(uint32_t* pointer) override { dds_ = pointer; }
  uint32_t* get_dds_num_of_points_pointer() override { return dds_; }

  Tensor features_, indices_;
  std::vector<int> grid_;
  std::string name_;
  uint32_t* dds_ = nullptr;
  int device_ = 0;
};

class EngineImpl : public Engine {
 public:
  EngineImpl(spconvb_engine* e, const std::string& input_name) : e_(e) {
    cudaGetDevice(&device_);
    inputs_.emplace_back(new SparseTensorImpl(input_name));
    inputs_[0]->device_ = device_;
    const int n = spconvb_engine_num_outputs(e_);
    for (int i = 0; i < n; ++i) {
      outputs_.emplace_back(new SparseTensorImpl("output" + std::to_string(i)));
      outputs_[i]->device_ = device_;
    }
    refresh_outputs();
  }
  ~EngineImpl() override { spconvb_engine_destroy(e_); }

  void forward(void* stream) override {
    SparseTensorImpl& in = *inputs_[0];
    if (in.features_.empty() || in.indices_.empty() || in.grid_.size() != 3) {
      logger_output(__FILE__, __LINE__, LoggerLevel::Error,
                    "forward: bind input(0)->features(), indices() and set_grid_size() first");
      return;
    }
    if (in.features_.dtype() != DataType::Float16 || in.indices_.dtype() != DataType::Int32 ||
        in.features_.ndim != 2 || in.indices_.ndim != 2 || in.indices_.size(1) != 4) {
      logger_output(__FILE__, __LINE__, LoggerLevel::Error,
                    "forward: features must be Float16 [n, C] and indices Int32 [n, 4]");
      return;
    }
    const int32_t grid[3] = {in.grid_[0], in.grid_[1], in.grid_[2]};
    const uint32_t rows = (uint32_t)in.features_.size(0);
    int rc;
    if (in.dds_)
      rc = spconvb_engine_forward_dds(e_, in.features_.ptr(), in.indices_.ptr<int32_t>(), rows, in.dds_,
                                      grid, 1, stream);
    else
      rc = spconvb_engine_forward(e_, in.features_.ptr(), rows, in.indices_.ptr<int32_t>(), grid, 1,
                                  stream);
    if (rc != SPCONVB_OK)
      logger_output(__FILE__, __LINE__, LoggerLevel::Error, "forward failed: %s", spconvb_error_string(rc));
    refresh_outputs();
  }

  size_t num_input() const override { return inputs_.size(); }
  SparseDTensor* input(unsigned int index) override {
    return index < inputs_.size() ? inputs_[index].get() : nullptr;
  }
  size_t num_output() const override { return outputs_.size(); }
  SparseDTensor* output(unsigned int index) override {
    return index < outputs_.size() ? outputs_[index].get() : nullptr;
  }

 private:
  // Point the output tensors at the engine's buffers (they exist after the first forward).
  // A sparse output also gets its indices and grid.  Its row count lives in device memory
  // (nothing here waits for the stream): get_dds_num_of_points_pointer() of the output gives
  // that word, rows beyond it are undefined, and the shapes report the capacity - except for
  // an output on the input's own rows with a host-known count, which reports that count.
  void refresh_outputs() {
    for (size_t i = 0; i < outputs_.size(); ++i) {
      void* data = nullptr;
      int64_t shape[8];
      int32_t ndim = 0, kind = 0, dense = 0;
      if (spconvb_engine_output(e_, (int)i, &data, shape, &ndim, &kind, &dense) != SPCONVB_OK) continue;
      std::vector<int64_t> s(shape, shape + ndim);
      SparseTensorImpl& out = *outputs_[i];
      if (!dense) {
        int32_t* coords = nullptr;
        uint32_t* n_ptr = nullptr;
        uint32_t cap = 0;
        int32_t grid[3] = {0, 0, 0}, on_input = 0;
        if (spconvb_engine_output_rows(e_, (int)i, &coords, &n_ptr, &cap, grid, &on_input) == SPCONVB_OK) {
          const SparseTensorImpl& in = *inputs_[0];
          int64_t rows = cap;
          if (on_input && !in.indices_.empty()) {
            coords = const_cast<int32_t*>(in.indices_.ptr<int32_t>());
            if (!in.dds_) rows = in.features_.size(0);
          }
          if (!s.empty()) s[0] = rows;
          if (coords) out.indices_.reference(coords, std::vector<int64_t>{rows, 4}, DataType::Int32);
          out.grid_ = {grid[0], grid[1], grid[2]};
          out.dds_ = n_ptr;
        }
      }
      out.features_.reference(data, s, kind == SPCONVB_I8 ? DataType::Int8 : DataType::Float16);
    }
  }

  spconvb_engine* e_;
  int device_ = 0;
  std::vector<std::unique_ptr<SparseTensorImpl>> inputs_, outputs_;
};

// --------------------------------------------------------------- build time
class TensorHandle : public ITensor {
 public:
  TensorHandle(int id, const std::string& name) : id(id), name_(name) {}
  const char* name() override { return name_.c_str(); }
  int id;
  std::string name_;
};

class NodeHandle : public INode {
 public:
  NodeHandle(const std::string& name, const char* op, std::vector<ITensor*> in, ITensor* out)
      : name_(name), op_(op), in_(std::move(in)), out_(out) {}
  const char* name() override { return name_.c_str(); }
  const char* optype() override { return op_; }
  ITensor* input(unsigned int i) override { return i < in_.size() ? in_[i] : nullptr; }
  ITensor* output(unsigned int i) override { return i == 0 ? out_ : nullptr; }
  unsigned int num_output() override { return 1; }
  unsigned int num_input() override { return (unsigned int)in_.size(); }

 private:
  std::string name_;
  const char* op_;
  std::vector<ITensor*> in_;
  ITensor* out_;
};

int prec(Precision p) { return p == Precision::Int8 ? SPCONVB_PRECISION_INT8 : SPCONVB_PRECISION_FP16; }

class BuilderImpl : public EngineBuilder {
 public:
  BuilderImpl() : b_(spconvb_builder_create()) {}
  ~BuilderImpl() override { spconvb_builder_destroy(b_); }

  ITensor* push_input(const char* name) override {
    if (input_name_.empty()) input_name_ = name ? name : "";
    return tensor(spconvb_builder_input(b_, name), name);
  }

  INode* push_add(const char* name, ITensor* a, ITensor* b, float a_dynamic_range, float b_dynamic_range,
                  const char* output_name, Precision precision, Precision output_precision,
                  uint32_t fixed_launch_points) override {
    if (!a || !b) return fail(name, "Add");
    int id = spconvb_builder_add(b_, name, id_of(a), id_of(b), a_dynamic_range, b_dynamic_range,
                                 output_name, prec(precision), prec(output_precision), fixed_launch_points);
    return node(name, "Add", {a, b}, id, output_name);
  }

  INode* push_relu(const char* name, ITensor* x, const char* output_name) override {
    if (!x) return fail(name, "Relu");
    return node(name, "Relu", {x}, spconvb_builder_relu(b_, name, id_of(x), output_name), output_name);
  }

  INode* push_dense(const char* name, ITensor* x, const char* format, const char* output_name,
                    const std::vector<int>& input_spatial_shape, const std::vector<int>& output_shape,
                    TensorLayout output_layout, float input_dynamic_range, uint32_t input_bound) override {
    if (!x) return fail(name, "ScatterDense");
    int id = spconvb_builder_dense(b_, name, id_of(x), format, output_name, input_spatial_shape.data(),
                                   (int)input_spatial_shape.size(), output_shape.data(),
                                   (int)output_shape.size(), (int)output_layout, input_dynamic_range,
                                   input_bound);
    return node(name, "ScatterDense", {x}, id, output_name);
  }

  INode* push_reshape(const char* name, ITensor* x, const std::vector<int64_t>& shape,
                      const char* output_name) override {
    if (!x) return fail(name, "Reshape");
    int id = spconvb_builder_reshape(b_, name, id_of(x), shape.data(), (int)shape.size(), output_name);
    return node(name, "Reshape", {x}, id, output_name);
  }

  INode* push_transpose(const char* name, ITensor* x, const std::vector<int64_t>& dims,
                        const char* output_name) override {
    if (!x) return fail(name, "Transpose");
    int id = spconvb_builder_transpose(b_, name, id_of(x), dims.data(), (int)dims.size(), output_name);
    return node(name, "Transpose", {x}, id, output_name);
  }

  INode* push_sparse_conv(const char* name, ITensor* x, const std::vector<unsigned short>& weight,
                          const std::vector<int>& weight_shape,
                          const std::vector<float>& weight_dynamic_ranges,
                          const std::vector<unsigned short>& bias, const std::vector<int>& bias_shape,
                          const char* activation, const std::vector<int>& kernel_size,
                          const std::vector<int>& stride, const std::vector<int>& padding,
                          const std::vector<int>& dilation, float input_dynamic_range, bool submanifold,
                          uint32_t max_output_points, uint32_t fixed_launch_points, const char* rulebook,
                          Precision precision, Precision output_precision, const char* output_name,
                          bool inverse) override {
    (void)bias_shape;
    if (!x || weight_shape.size() != 5 || kernel_size.size() != 3 || stride.size() != 3 ||
        padding.size() != 3 || dilation.size() != 3) {
      logger_output(__FILE__, __LINE__, LoggerLevel::Error,
                    "conv '%s': weight must be [Cout,k0,k1,k2,Cin] and the geometry lists 3 long",
                    name ? name : "");
      return fail(name, "SparseConvolution");
    }
    size_t vol = 1;
    for (int v : weight_shape) vol *= (size_t)(v > 0 ? v : 0);
    if (vol != weight.size()) {
      logger_output(__FILE__, __LINE__, LoggerLevel::Error, "conv '%s': weight data does not match its shape",
                    name ? name : "");
      return fail(name, "SparseConvolution");
    }
    int id = spconvb_builder_sparse_conv(
        b_, name, id_of(x), weight.data(), weight_shape.data(), weight_dynamic_ranges.data(),
        (int)weight_dynamic_ranges.size(), bias.data(), (int)bias.size(), activation, kernel_size.data(),
        stride.data(), padding.data(), dilation.data(), input_dynamic_range, submanifold ? 1 : 0,
        max_output_points, fixed_launch_points, rulebook, prec(precision), prec(output_precision),
        output_name, inverse ? 1 : 0);
    return node(name, "SparseConvolution", {x}, id, output_name);
  }

  void push_output(ITensor* value) override {
    if (value) spconvb_builder_output(b_, id_of(value));
  }

  // sortmask and enable_blackwell select kernels of the reference's engine and mean nothing
  // here; with_auxiliary_stream = false keeps the rulebook kernels on the caller's stream.
  std::shared_ptr<Engine> build(Precision precision, bool, bool, bool with_auxiliary_stream,
                                void* stream) override {
    int err = 0;
    spconvb_engine* e = spconvb_builder_build(
        b_, prec(precision), with_auxiliary_stream ? 0u : SPCONVB_BUILD_SINGLE_STREAM, stream, &err);
    if (!e) {
      logger_output(__FILE__, __LINE__, LoggerLevel::Error, "build failed: %s", spconvb_error_string(err));
      return nullptr;
    }
    return std::make_shared<EngineImpl>(e, input_name_);
  }

 private:
  static int id_of(ITensor* t) { return static_cast<TensorHandle*>(t)->id; }
  ITensor* tensor(int id, const char* name) {
    if (id < 0) {
      logger_output(__FILE__, __LINE__, LoggerLevel::Error, "builder: %s", spconvb_error_string(id));
      return nullptr;
    }
    tensors_.emplace_back(new TensorHandle(id, name ? name : ""));
    return tensors_.back().get();
  }
  INode* node(const char* name, const char* op, std::vector<ITensor*> in, int out_id, const char* out_name) {
    ITensor* out = tensor(out_id, out_name);
    if (!out) return fail(name, op);
    nodes_.emplace_back(new NodeHandle(name ? name : "", op, std::move(in), out));
    return nodes_.back().get();
  }
  // A node whose output is null: callers that go on with n->output(0) get a null tensor,
  // which the next push rejects, and build() fails.
  INode* fail(const char* name, const char* op) {
    nodes_.emplace_back(new NodeHandle(name ? name : "", op, {}, nullptr));
    return nodes_.back().get();
  }

  spconvb_builder* b_;
  std::string input_name_;
  std::vector<std::unique_ptr<TensorHandle>> tensors_;
  std::vector<std::unique_ptr<NodeHandle>> nodes_;
};

}  // namespace

std::shared_ptr<EngineBuilder> create_engine_builder() { return std::make_shared<BuilderImpl>(); }

std::shared_ptr<Engine> load_engine_from_onnx(const std::string& onnx_file, Precision inference_precision,
                                              bool, bool, bool with_auxiliary_stream,
                                              unsigned int fixed_launch_points, void* stream) {
  int err = 0;
  spconvb_engine* e = spconvb_engine_load_onnx(
      onnx_file.c_str(), prec(inference_precision),
      with_auxiliary_stream ? 0u : SPCONVB_BUILD_SINGLE_STREAM, fixed_launch_points, stream, &err);
  if (!e) {
    logger_output(__FILE__, __LINE__, LoggerLevel::Error, "load_engine_from_onnx(%s) failed: %s",
                  onnx_file.c_str(), spconvb_error_string(err));
    return nullptr;
  }
  return std::make_shared<EngineImpl>(e, "0");
}

}  // namespace spconv
