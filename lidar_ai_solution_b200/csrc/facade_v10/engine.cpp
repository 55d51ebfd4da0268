// The v1.0 interface (include/spconv_v10/spconv/engine.hpp) on top of the C ABI.
#include <cuda_runtime.h>
#include <stdio.h>

#include <spconv/engine.hpp>

#include "spconvb.h"

namespace spconv {

namespace {

class ResultTensor : public DTensor {
 public:
  std::vector<int64_t> features_shape() const override { return fshape; }
  DType features_dtype() const override { return DType::Float16; }
  void* features_data() override { return fdata; }
  std::vector<int64_t> indices_shape() const override { return ishape; }
  DType indices_dtype() const override { return DType::Int32; }
  void* indices_data() override { return idata; }
  std::vector<int> grid_size() const override { return grid; }
  int device() const override { return dev; }

  std::vector<int64_t> fshape, ishape;
  void* fdata = nullptr;
  void* idata = nullptr;
  std::vector<int> grid;
  int dev = 0;
};

int to_c(spconv::Precision p) {
  return p == spconv::Precision::Int8 ? SPCONVB_PRECISION_INT8 : SPCONVB_PRECISION_FP16;
}

class EngineImpl : public Engine {
 public:
  explicit EngineImpl(spconvb_engine* e) : e_(e) { cudaGetDevice(&result_.dev); }
  virtual ~EngineImpl() { spconvb_engine_destroy(e_); }

  DTensor* forward(const std::vector<int64_t>& features_shape, DType features_dtype, void* features_data,
                   const std::vector<int64_t>& indices_shape, DType indices_dtype, void* indices_data,
                   int batch, std::vector<int> grid_size, void* stream) override {
    if (features_shape.size() != 2 || indices_shape.size() != 2 || indices_shape[1] != 4 ||
        features_dtype != DType::Float16 || indices_dtype != DType::Int32 || batch != 1 ||
        grid_size.size() != 3 || features_shape[0] != indices_shape[0]) {
      fprintf(stderr, "[spconv error] forward: expects Float16 [n,C] features, Int32 [n,4] indices, "
                      "batch 1 and a 3-element grid size\n");
      return nullptr;
    }
    const int32_t grid[3] = {grid_size[0], grid_size[1], grid_size[2]};
    const int rc = spconvb_engine_forward(e_, features_data, (uint32_t)features_shape[0],
                                          (const int32_t*)indices_data, grid, 1, stream);
    if (rc != SPCONVB_OK) {
      fprintf(stderr, "[spconv error] forward failed: %s\n", spconvb_error_string(rc));
      return nullptr;
    }
    int64_t shape[8];
    int32_t ndim = 0, kind = 0, dense = 0;
    if (spconvb_engine_output(e_, 0, &result_.fdata, shape, &ndim, &kind, &dense) != SPCONVB_OK)
      return nullptr;
    result_.fshape.assign(shape, shape + ndim);
    result_.grid = grid_size;
    return &result_;
  }

  void reconfigure() override {
    const int rc = spconvb_engine_reconfigure(e_, nullptr);
    if (rc != SPCONVB_OK) fprintf(stderr, "[spconv] reconfigure failed: %s\n", spconvb_error_string(rc));
  }
  void set_int8_calibration(bool enable) override {
    const int rc = spconvb_engine_set_int8_calibration(e_, enable ? 1 : 0);
    if (rc != SPCONVB_OK)
      fprintf(stderr, "[spconv] set_int8_calibration failed: %s\n", spconvb_error_string(rc));
  }
  void set_node_precision_byname(const char* name, Precision compute_precision,
                                 Precision output_precision) override {
    if (spconvb_engine_set_node_precision(e_, name, 0, to_c(compute_precision),
                                          to_c(output_precision)) <= 0)
      fprintf(stderr, "[spconv] set_node_precision_byname: no node named '%s'\n", name ? name : "");
  }
  void set_node_precision_byoptype(const char* optype, Precision compute_precision,
                                   Precision output_precision) override {
    if (spconvb_engine_set_node_precision(e_, optype, 1, to_c(compute_precision),
                                          to_c(output_precision)) <= 0)
      fprintf(stderr, "[spconv] set_node_precision_byoptype: no node of type '%s'\n",
              optype ? optype : "");
  }

 private:
  spconvb_engine* e_;
  ResultTensor result_;
};

}  // namespace

std::shared_ptr<Engine> load_engine_from_onnx(const std::string& onnx_file, Precision precision) {
  int err = 0;
  spconvb_engine* e = spconvb_engine_load_onnx(
      onnx_file.c_str(), precision == Precision::Int8 ? SPCONVB_PRECISION_INT8 : SPCONVB_PRECISION_FP16, 0,
      0, nullptr, &err);
  if (!e) {
    fprintf(stderr, "[spconv error] load_engine_from_onnx(%s) failed: %s\n", onnx_file.c_str(),
            spconvb_error_string(err));
    return nullptr;
  }
  return std::shared_ptr<Engine>(new EngineImpl(e));
}

void set_verbose(bool enable) { spconvb_set_log_level(enable ? 0 : 1); }

const char* get_precision_string(Precision precision) {
  switch (precision) {
    case Precision::Float16: return "Float16";
    case Precision::Int8: return "Int8";
    default: return "None";
  }
}

}  // namespace spconv
