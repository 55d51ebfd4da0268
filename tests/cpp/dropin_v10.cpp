// Drives the v1.0 C++ interface exactly as CUDA-CenterPoint does
// (CUDA-CenterPoint/src/centerpoint.cpp:55 and :145-149): load_engine_from_onnx(file),
// forward(features shape/type/pointer, indices shape/type/pointer, batch, grid, stream),
// then read result->features_data().
//   dropin_v10 model.onnx fp16|int8 features.f16 indices.i32 N C Z Y X out.f16
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include <spconv/engine.hpp>

static std::vector<char> read_file(const char* path) {
  std::vector<char> buf;
  FILE* f = fopen(path, "rb");
  if (!f) return buf;
  fseek(f, 0, SEEK_END);
  long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  buf.resize(n);
  if (fread(buf.data(), 1, n, f) != (size_t)n) buf.clear();
  fclose(f);
  return buf;
}

int main(int argc, char** argv) {
  if (argc < 11) return 2;
  auto precision = strcmp(argv[2], "int8") == 0 ? spconv::Precision::Int8 : spconv::Precision::Float16;
  std::shared_ptr<spconv::Engine> scn_engine_ = spconv::load_engine_from_onnx(argv[1], precision);
  if (!scn_engine_) return 1;
  const unsigned int valid_num = (unsigned int)atoi(argv[5]);
  const int channels = atoi(argv[6]);
  std::vector<int> sparse_shape = {atoi(argv[7]), atoi(argv[8]), atoi(argv[9])};
  auto f = read_file(argv[3]);
  auto i = read_file(argv[4]);
  if (f.size() != (size_t)valid_num * channels * 2 || i.size() != (size_t)valid_num * 16) return 1;
  void *d_voxel_features, *d_voxel_indices;
  cudaMalloc(&d_voxel_features, f.size());
  cudaMalloc(&d_voxel_indices, i.size());
  cudaMemcpy(d_voxel_features, f.data(), f.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(d_voxel_indices, i.data(), i.size(), cudaMemcpyHostToDevice);
  cudaStream_t stream;
  cudaStreamCreate(&stream);

  auto result = scn_engine_->forward(
      {valid_num, channels}, spconv::DType::Float16, d_voxel_features,
      {valid_num, 4}, spconv::DType::Int32, d_voxel_indices,
      1, sparse_shape, stream);
  if (!result) return 1;
  cudaStreamSynchronize(stream);

  size_t numel = 1;
  for (auto d : result->features_shape()) numel *= (size_t)d;
  std::vector<char> host(numel * 2);
  cudaMemcpy(host.data(), result->features_data(), host.size(), cudaMemcpyDeviceToHost);
  printf("precision %s, output dims %zu, %zu elements\n", spconv::get_precision_string(precision),
         result->features_shape().size(), numel);
  FILE* out = fopen(argv[10], "wb");
  bool ok = out && fwrite(host.data(), 1, host.size(), out) == host.size();
  if (out) fclose(out);
  scn_engine_->reconfigure();  // logs that it does nothing
  return ok ? 0 : 1;
}
