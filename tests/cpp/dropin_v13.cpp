// Drives the v1.3 C++ interface the way the reference's applications do
// (CUDA-BEVFusion/src/bevfusion/lidar-scn.cpp:39-49 and
// libraries/3DSparseConvolution/src/infer.cpp:264-345): load an engine from an ONNX file, bind
// the inputs by reference, forward on a stream, save output 0 as a tensor file.
//   dropin_v13 model.onnx fp16|int8 features.tensor indices.tensor Z Y X out.tensor [dds]
// With "dds" the row count is read on the device and the engine's auxiliary stream is on;
// without it the host knows the count and with_auxiliary_stream is false.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <spconv/engine.hpp>
#include <spconv/onnx-parser.hpp>
#include <spconv/tensor.hpp>
#include <spconv/timer.hpp>
#include <spconv/version.hpp>

int main(int argc, char** argv) {
  if (argc < 9) return 2;
  spconv::set_logger_level(spconv::LoggerLevel::Warn);
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  auto precision = strcmp(argv[2], "int8") == 0 ? spconv::Precision::Int8 : spconv::Precision::Float16;
  const bool use_dds = argc > 9 && strcmp(argv[9], "dds") == 0;
  auto engine = spconv::load_engine_from_onnx(argv[1], precision, false, false, use_dds, 10000, stream);
  if (engine == nullptr) {
    printf("load failed\n");
    return 1;
  }
  auto features = spconv::Tensor::load(argv[3], true, stream);
  auto indices = spconv::Tensor::load(argv[4], true, stream);
  if (features.empty() || indices.empty()) return 1;
  std::vector<int> grid = {atoi(argv[5]), atoi(argv[6]), atoi(argv[7])};

  engine->input(0)->features().reference(features.ptr(), features.shape, spconv::DataType::Float16);
  engine->input(0)->indices().reference(indices.ptr(), indices.shape, spconv::DataType::Int32);
  engine->input(0)->set_grid_size(grid);

  uint32_t* dds = nullptr;
  if (use_dds) {
    uint32_t n = (uint32_t)features.size(0);
    cudaMalloc(&dds, sizeof(uint32_t));
    cudaMemcpyAsync(dds, &n, sizeof(n), cudaMemcpyHostToDevice, stream);
    engine->input(0)->set_dds_num_of_points_pointer(dds);
  }

  spconv::EventTimer timer;
  engine->forward(stream);  // allocates on the first call
  timer.start(stream);
  engine->forward(stream);
  float ms = timer.stop("forward", false);
  cudaStreamSynchronize(stream);

  auto& out = engine->output(0)->features();
  printf("libspconv interface %s, output %s %s, %.3f ms\n", NVSPCONV_VERSION,
         spconv::dtype_string(out.dtype()), spconv::format_shape(out.shape), ms);
  // a sparse output also carries its coordinates, its grid and the device word with its rows
  auto& oidx = engine->output(0)->indices();
  if (!oidx.empty()) {
    uint32_t rows = 0;
    uint32_t* rows_dev = engine->output(0)->get_dds_num_of_points_pointer();
    if (rows_dev) cudaMemcpy(&rows, rows_dev, sizeof(rows), cudaMemcpyDeviceToHost);
    auto g = engine->output(0)->grid_size();
    printf("sparse output: indices %s, rows on device %u, grid %d %d %d\n",
           spconv::format_shape(oidx.shape), rows, g.size() > 0 ? g[0] : -1, g.size() > 1 ? g[1] : -1,
           g.size() > 2 ? g[2] : -1);
  }
  bool ok = out.save(argv[8], stream);
  if (dds) cudaFree(dds);
  cudaStreamDestroy(stream);
  return ok ? 0 : 1;
}
