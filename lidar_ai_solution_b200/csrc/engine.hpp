// Graph builder and executor of the sparse-convolution engine (host side).
// The classes here sit behind the C ABI (spconvb_builder_* / spconvb_engine_*);
// they only enqueue work through the kernel-level entry points of spconvb.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "spconvb.h"

namespace spconvb {

void log_msg(int level, const char* fmt, ...);
enum { LOG_VERB = 0, LOG_WARN = 1, LOG_ERROR = 2 };

int launch_set_count(uint32_t* dst, uint32_t value, cudaStream_t st);
int launch_clamp_count(uint32_t* dst, const uint32_t* src, uint32_t cap, uint32_t* status,
                       cudaStream_t st);
// spconvb_scatter_dense / spconvb_scatter_dense_layout with the zero fill of `out` optional
// (clear = false: the caller has already zeroed it, e.g. on another stream)
int scatter_dense_launch(const void* feat, int32_t in_kind, float in_scale, const int32_t* coords,
                         const uint32_t* n_ptr, uint32_t launch_rows, int32_t channels,
                         int32_t batch, const int32_t grid[3], const int32_t perm[3], void* out,
                         bool clear, void* stream);
int scatter_dense_layout_launch(const void* feat, int32_t in_kind, float in_scale,
                                const int32_t* coords, const uint32_t* n_ptr, uint32_t launch_rows,
                                int32_t channels, int32_t batch, const int32_t grid[3],
                                const int32_t perm[3], int32_t layout, int32_t out_kind,
                                float inv_out_scale, void* out, bool clear, void* stream);

enum OpKind { OP_INPUT, OP_CONV, OP_ADD, OP_RELU, OP_DENSE, OP_RESHAPE, OP_TRANSPOSE };

struct GNode {
  OpKind op = OP_INPUT;
  std::string name;
  int in0 = -1, in1 = -1, out = -1;
  // conv
  std::vector<uint16_t> weight;  // fp16 bits [cout][kvol][cin]
  std::vector<float> wdr;
  std::vector<uint16_t> bias;
  int cin = 0, cout = 0;
  bool relu_act = false;
  int ksize[3] = {1, 1, 1}, stride[3] = {1, 1, 1}, pad[3] = {0, 0, 0}, dil[3] = {1, 1, 1};
  float in_dr = 0.f;
  bool subm = false;
  bool inverse = false;  // runs over the pairs of the strided rulebook named `rulebook`, swapped
  uint32_t out_bound = 0, fixed_launch = 0;
  std::string rulebook;
  int prec = SPCONVB_PRECISION_FP16, out_prec = SPCONVB_PRECISION_FP16;
  // add
  float a_dr = 0.f, b_dr = 0.f;
  // dense
  std::string format;
  std::vector<int> in_spatial, out_shape;
  int layout = 1;
  float dense_dr = 0.f;
  // reshape / transpose
  std::vector<int64_t> dims;
};

struct GTensor {
  std::string name;
  int producer = -1;
  std::vector<int> consumers;
};

class Builder {
 public:
  std::vector<GNode> nodes;
  std::vector<GTensor> tensors;
  std::vector<int> outputs;
  int new_tensor(const std::string& name, int producer);
  bool valid_tensor(int t) const { return t >= 0 && t < (int)tensors.size(); }
  int push(GNode&& n, const std::string& out_name);
};

struct CoordSet {
  bool external = false;     // the engine input: coordinates owned by the caller
  uint32_t bound = 0;        // rows the model says it may hold (output_bound)
  bool need_table = false;
  int made_by_rule = -1;     // the strided rulebook whose outputs these rows are
  // filled by prepare()
  uint32_t cap = 0;
  int32_t grid[3] = {0, 0, 0};
  int32_t* coords = nullptr;
  uint32_t* n_ptr = nullptr;
  uint64_t* table = nullptr;
  uint32_t slots = 0;
};

struct Rule {
  bool subm = true;
  int ksize[3], stride[3], pad[3], dil[3];
  int kvol = 1;
  int in_cs = -1, out_cs = -1;
  int inverse_of = -1;       // >= 0: the strided rule whose pairs this rule swaps
  int32_t* map = nullptr;
  void* ws = nullptr;
  size_t ws_bytes = 0;
};

struct RTensor {
  std::string name;
  int cs = -1;
  int channels = 0;          // as stored (after padding)
  int kind = SPCONVB_F16;
  float dr = 0.f;            // dynamic range when int8 (scale = dr/127)
  bool dense = false;
  bool external = false;
  bool is_output = false;
  int alias_of = -1;         // shares the buffer of another tensor (Reshape)
  std::vector<int64_t> shape;  // dense shape (logical, NCHW order)
  int layout = 1;              // dense: physical TensorLayout
  std::vector<int64_t> phys_shape;  // dense: dimensions as laid out in memory
  int first_step = 1 << 30, last_step = -1;
  void* data = nullptr;
  size_t bytes = 0;
};

struct LayerWeights {
  void* plain = nullptr;
  void* packed = nullptr;
  float* scale = nullptr;
  float* bias = nullptr;
};

struct Step {
  enum Kind { HASH, SUBM_MAP, DOWN_MAP, CONVERT, CONV, ADD, RELU, DENSE, INV_MAP } kind;
  std::string name;
  int cs = -1, rule = -1;
  int in0 = -1, in1 = -1, out = -1;  // runtime tensors
  spconvb_conv_params cp{};
  int weights = -1;
  int relu = 0;
  int cin = 0, cout = 0;
  float s = 1.f;              // convert: scale or inverse scale
  float a_scale = 1.f, b_scale = 1.f, inv_out = 1.f;
  int perm[3] = {0, 1, 2};
  bool has_perm = false;
  int layout = 1;             // dense: TensorLayout of the output
};

struct Profile {
  float* step_ms = nullptr;
  int max_steps = 0;
  int reps = 1;
  void* flush = nullptr;
  size_t flush_bytes = 0;
};

class Engine {
 public:
  ~Engine();
  int compile(const Builder& b, int precision, uint32_t flags, cudaStream_t st);
  int prepare(const int32_t grid[3], int batch);
  int forward(const void* features, const int32_t* indices, uint32_t cap_rows, uint32_t n_host,
              const uint32_t* n_dev, const int32_t grid[3], int batch, cudaStream_t st,
              const Profile* prof = nullptr);

  // Folds max |x| of every sparse runtime tensor of the last forward into out[r] (device
  // floats, one per runtime tensor), on the stream of that forward.
  int collect_absmax(float* out, cudaStream_t st);

  std::vector<CoordSet> coordsets;
  std::vector<Rule> rules;
  std::vector<RTensor> rt;
  std::vector<Step> steps;
  std::vector<LayerWeights> weights;
  std::vector<int> outputs;  // runtime tensor ids
  std::unordered_map<std::string, int> by_name;
  std::string names_text, describe_text;
  uint32_t* status = nullptr;
  int last_launches = 0;
  uint32_t flags = 0;

 private:
  int input_rt_ = -1;
  int input_channels_ = 0;
  const uint32_t* last_in_n_ = nullptr;  // row count of the caller's rows in the last forward
  uint32_t last_in_cap_ = 0;
  bool prepared_ = false;
  int32_t grid_[3] = {0, 0, 0};
  int batch_ = 0;
  std::vector<void*> allocations_;
  // Rulebook steps depend on coordinates only: they run ahead on this stream while the
  // caller's stream does the convolutions, joined by one event per rulebook step.
  cudaStream_t aux_ = nullptr;
  cudaEvent_t fork_ev_ = nullptr;
  std::vector<cudaEvent_t> rule_ev_;
  void* zero_arena_ = nullptr;
  size_t zero_bytes_ = 0;
  uint32_t* counts_ = nullptr;
  void free_prepared();
  int dev_alloc(void** p, size_t bytes);
};

// ONNX reader: fills a Builder from a model file (protobuf wire format).
int load_onnx(const char* path, uint32_t fixed_launch_points, Builder* out);

}  // namespace spconvb
