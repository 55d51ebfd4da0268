// extern "C" surface of the builder and the engine (see include/spconvb.h).
#include <stdio.h>
#include <string.h>

#include <cuda_fp16.h>
#include <math.h>

#include <memory>
#include <string>
#include <vector>

#include "engine.hpp"

using namespace spconvb;

struct spconvb_builder {
  Builder b;
};
struct spconvb_engine {
  std::unique_ptr<Engine> e;   // the executable engine, rebuilt by reconfigure
  Builder graph;               // what it was built from, edited by the precision setters
  int32_t precision = SPCONVB_PRECISION_FP16;
  uint32_t flags = 0;
  std::vector<char> user_prec;   // per node: precision set explicitly by the caller
  bool want_calibration = false; // state asked for; applied by the next reconfigure
  bool collecting = false;       // the live engine is the fp16 calibration engine
  float* absmax = nullptr;       // device, one per runtime tensor of the calibration engine
  ~spconvb_engine() {
    if (absmax) cudaFree(absmax);
  }
};

namespace {
const char* nz(const char* s) { return s ? s : ""; }
bool bad(const spconvb_builder* b, int t) { return !b || !b->b.valid_tensor(t); }
}  // namespace

extern "C" {

spconvb_builder* spconvb_builder_create(void) { return new (std::nothrow) spconvb_builder(); }
void spconvb_builder_destroy(spconvb_builder* b) { delete b; }

int spconvb_builder_input(spconvb_builder* b, const char* name) {
  if (!b) return SPCONVB_E_ARG;
  GNode n;
  n.op = OP_INPUT;
  n.name = nz(name);
  return b->b.push(std::move(n), nz(name));
}

int spconvb_builder_sparse_conv(spconvb_builder* b, const char* name, int x,
                                const uint16_t* weight, const int32_t weight_shape[5],
                                const float* weight_dynamic_ranges, int32_t n_ranges,
                                const uint16_t* bias, int32_t n_bias, const char* activation,
                                const int32_t kernel_size[3], const int32_t stride[3],
                                const int32_t padding[3], const int32_t dilation[3],
                                float input_dynamic_range, int32_t submanifold,
                                uint32_t max_output_points, uint32_t fixed_launch_points,
                                const char* rulebook, int32_t precision, int32_t output_precision,
                                const char* output_name, int32_t inverse) {
  if (bad(b, x) || !weight || !weight_shape || !kernel_size || !stride || !padding || !dilation)
    return SPCONVB_E_ARG;
  const std::string act = nz(activation);
  if (!act.empty() && act != "ReLU" && act != "None") {
    log_msg(LOG_ERROR, "conv '%s': activation '%s' is not supported", nz(name), act.c_str());
    return SPCONVB_E_UNSUPPORTED;
  }
  GNode n;
  n.op = OP_CONV;
  n.name = nz(name);
  n.in0 = x;
  n.cout = weight_shape[0];
  n.cin = weight_shape[4];
  size_t vol = 1;
  for (int i = 0; i < 5; ++i) {
    if (weight_shape[i] < 1) return SPCONVB_E_ARG;
    vol *= (size_t)weight_shape[i];
  }
  for (int a = 0; a < 3; ++a) {
    n.ksize[a] = kernel_size[a];
    n.stride[a] = stride[a];
    n.pad[a] = padding[a];
    n.dil[a] = dilation[a];
    if (kernel_size[a] != weight_shape[1 + a] || stride[a] < 1 || dilation[a] < 1 || padding[a] < 0)
      return SPCONVB_E_ARG;
  }
  n.weight.assign(weight, weight + vol);
  if (weight_dynamic_ranges && n_ranges > 0)
    n.wdr.assign(weight_dynamic_ranges, weight_dynamic_ranges + n_ranges);
  if (bias && n_bias > 0) n.bias.assign(bias, bias + n_bias);
  n.relu_act = act == "ReLU";
  n.in_dr = input_dynamic_range;
  n.subm = submanifold != 0;
  n.inverse = inverse != 0;
  n.out_bound = max_output_points ? max_output_points : 150000u;
  n.fixed_launch = fixed_launch_points;
  n.rulebook = nz(rulebook);
  n.prec = precision;
  n.out_prec = output_precision;
  return b->b.push(std::move(n), nz(output_name));
}

int spconvb_builder_add(spconvb_builder* b, const char* name, int a, int bb, float a_dynamic_range,
                        float b_dynamic_range, const char* output_name, int32_t precision,
                        int32_t output_precision, uint32_t fixed_launch_points) {
  if (bad(b, a) || bad(b, bb)) return SPCONVB_E_ARG;
  GNode n;
  n.op = OP_ADD;
  n.name = nz(name);
  n.in0 = a;
  n.in1 = bb;
  n.a_dr = a_dynamic_range;
  n.b_dr = b_dynamic_range;
  n.prec = precision;
  n.out_prec = output_precision;
  n.fixed_launch = fixed_launch_points;
  return b->b.push(std::move(n), nz(output_name));
}

int spconvb_builder_relu(spconvb_builder* b, const char* name, int x, const char* output_name) {
  if (bad(b, x)) return SPCONVB_E_ARG;
  GNode n;
  n.op = OP_RELU;
  n.name = nz(name);
  n.in0 = x;
  return b->b.push(std::move(n), nz(output_name));
}

int spconvb_builder_dense(spconvb_builder* b, const char* name, int x, const char* format,
                          const char* output_name, const int32_t* input_spatial_shape,
                          int32_t n_spatial, const int32_t* output_shape, int32_t n_output_shape,
                          int32_t output_layout, float input_dynamic_range, uint32_t input_bound) {
  (void)input_bound;
  if (bad(b, x) || !output_shape || n_output_shape < 1) return SPCONVB_E_ARG;
  GNode n;
  n.op = OP_DENSE;
  n.name = nz(name);
  n.in0 = x;
  n.format = nz(format);
  if (input_spatial_shape) n.in_spatial.assign(input_spatial_shape, input_spatial_shape + n_spatial);
  n.out_shape.assign(output_shape, output_shape + n_output_shape);
  n.layout = output_layout ? output_layout : 1;
  n.dense_dr = input_dynamic_range;
  return b->b.push(std::move(n), nz(output_name));
}

int spconvb_builder_reshape(spconvb_builder* b, const char* name, int x, const int64_t* shape,
                            int32_t n, const char* output_name) {
  if (bad(b, x) || !shape || n < 1) return SPCONVB_E_ARG;
  GNode g;
  g.op = OP_RESHAPE;
  g.name = nz(name);
  g.in0 = x;
  g.dims.assign(shape, shape + n);
  return b->b.push(std::move(g), nz(output_name));
}

int spconvb_builder_transpose(spconvb_builder* b, const char* name, int x, const int64_t* dims,
                              int32_t n, const char* output_name) {
  if (bad(b, x) || !dims || n < 1) return SPCONVB_E_ARG;
  GNode g;
  g.op = OP_TRANSPOSE;
  g.name = nz(name);
  g.in0 = x;
  g.dims.assign(dims, dims + n);
  return b->b.push(std::move(g), nz(output_name));
}

int spconvb_builder_output(spconvb_builder* b, int x) {
  if (bad(b, x)) return SPCONVB_E_ARG;
  b->b.outputs.push_back(x);
  return SPCONVB_OK;
}

spconvb_engine* spconvb_builder_build(spconvb_builder* b, int32_t precision, uint32_t flags,
                                      void* stream, int* err) {
  int rc = SPCONVB_E_ARG;
  spconvb_engine* e = nullptr;
  if (b) {
    e = new (std::nothrow) spconvb_engine();
    if (e) {
      e->e.reset(new (std::nothrow) Engine());
      e->graph = b->b;
      e->precision = precision;
      e->flags = flags;
      e->user_prec.assign(b->b.nodes.size(), 0);
    }
    rc = e && e->e ? e->e->compile(e->graph, precision, flags, (cudaStream_t)stream)
                   : SPCONVB_E_NOMEM;
    if (rc != SPCONVB_OK) {
      delete e;
      e = nullptr;
    }
  }
  if (err) *err = rc;
  return e;
}

spconvb_engine* spconvb_engine_load_onnx(const char* path, int32_t precision, uint32_t flags,
                                         uint32_t fixed_launch_points, void* stream, int* err) {
  int rc = SPCONVB_E_ARG;
  spconvb_engine* e = nullptr;
  if (path) {
    spconvb_builder b;
    rc = load_onnx(path, fixed_launch_points, &b.b);
    if (rc == SPCONVB_OK) e = spconvb_builder_build(&b, precision, flags, stream, &rc);
  }
  if (err) *err = rc;
  return e;
}

int spconvb_onnx_inspect(const char* path, char* buf, size_t buf_bytes) {
  if (!path || !buf || buf_bytes < 2) return SPCONVB_E_ARG;
  Builder b;
  buf[0] = 0;
  const int rc = load_onnx(path, 0, &b);
  if (rc != SPCONVB_OK) return rc;
  std::string out;
  char line[1024];
  static const char* ops[] = {"Input", "SparseConvolution", "Add", "Relu", "ScatterDense",
                              "Reshape", "Transpose"};
  for (const GNode& n : b.nodes) {
    const char* in0 = n.in0 >= 0 ? b.tensors[n.in0].name.c_str() : "-";
    const char* in1 = n.in1 >= 0 ? b.tensors[n.in1].name.c_str() : "-";
    snprintf(line, sizeof(line), "%s %s in=%s,%s out=%s", ops[n.op], n.name.c_str(), in0, in1,
             b.tensors[n.out].name.c_str());
    out += line;
    if (n.op == OP_CONV) {
      snprintf(line, sizeof(line),
               " cin=%d cout=%d k=%d,%d,%d s=%d,%d,%d p=%d,%d,%d d=%d,%d,%d subm=%d relu=%d "
               "bound=%u rulebook=%s prec=%d out_prec=%d in_dr=%.9g n_wdr=%zu bias=%zu",
               n.cin, n.cout, n.ksize[0], n.ksize[1], n.ksize[2], n.stride[0], n.stride[1],
               n.stride[2], n.pad[0], n.pad[1], n.pad[2], n.dil[0], n.dil[1], n.dil[2],
               (int)n.subm, (int)n.relu_act, n.out_bound, n.rulebook.c_str(), n.prec, n.out_prec,
               (double)n.in_dr, n.wdr.size(), n.bias.size());
      out += line;
    } else if (n.op == OP_ADD) {
      snprintf(line, sizeof(line), " a_dr=%.9g b_dr=%.9g prec=%d out_prec=%d", (double)n.a_dr,
               (double)n.b_dr, n.prec, n.out_prec);
      out += line;
    } else if (n.op == OP_DENSE) {
      out += " format=" + n.format + " out_shape=";
      for (int v : n.out_shape) out += std::to_string(v) + ",";
      snprintf(line, sizeof(line), " layout=%d in_dr=%.9g", n.layout, (double)n.dense_dr);
      out += line;
    } else if (n.op == OP_RESHAPE || n.op == OP_TRANSPOSE) {
      out += " dims=";
      for (auto v : n.dims) out += std::to_string(v) + ",";
    }
    out += "\n";
  }
  for (int t : b.outputs) out += "Output " + b.tensors[t].name + "\n";
  if (out.size() + 1 > buf_bytes) return SPCONVB_E_NOMEM;
  memcpy(buf, out.c_str(), out.size() + 1);
  return SPCONVB_OK;
}

int spconvb_engine_set_node_precision(spconvb_engine* e, const char* key, int32_t by_optype,
                                      int32_t compute_precision, int32_t output_precision) {
  if (!e || !key) return SPCONVB_E_ARG;
  auto ok = [](int32_t p) { return p == SPCONVB_PRECISION_FP16 || p == SPCONVB_PRECISION_INT8; };
  if (!ok(compute_precision) || !ok(output_precision)) return SPCONVB_E_ARG;
  static const struct { const char* name; OpKind op; } kinds[] = {
      {"SparseConvolution", OP_CONV}, {"Add", OP_ADD}, {"QuantAdd", OP_ADD}, {"Relu", OP_RELU},
      {"ScatterDense", OP_DENSE}};
  int changed = 0;
  for (size_t i = 0; i < e->graph.nodes.size(); ++i) {
    GNode& n = e->graph.nodes[i];
    bool hit = false;
    if (by_optype) {
      for (const auto& k : kinds) hit = hit || (n.op == k.op && strcmp(key, k.name) == 0);
    } else {
      hit = n.name == key;
    }
    if (!hit) continue;
    n.prec = compute_precision;
    n.out_prec = output_precision;
    e->user_prec[i] = 1;
    ++changed;
  }
  return changed;
}

int spconvb_engine_set_int8_calibration(spconvb_engine* e, int32_t enable) {
  if (!e) return SPCONVB_E_ARG;
  if (enable) {
    e->want_calibration = true;
    return SPCONVB_OK;
  }
  e->want_calibration = false;
  if (!e->collecting) return SPCONVB_OK;
  // the running maxima become the dynamic ranges of the graph
  if (cudaDeviceSynchronize() != cudaSuccess) return SPCONVB_E_DEVICE;
  std::vector<float> host(e->e->rt.size(), 0.f);
  if (cudaMemcpy(host.data(), e->absmax, sizeof(float) * host.size(), cudaMemcpyDeviceToHost) !=
      cudaSuccess)
    return SPCONVB_E_DEVICE;
  auto range_of = [&](int graph_tensor) -> float {
    if (!e->graph.valid_tensor(graph_tensor)) return 1e-6f;
    auto it = e->e->by_name.find(e->graph.tensors[graph_tensor].name);
    const float v = it == e->e->by_name.end() ? 0.f : host[it->second];
    return v > 1e-6f ? v : 1e-6f;
  };
  for (size_t i = 0; i < e->graph.nodes.size(); ++i) {
    GNode& n = e->graph.nodes[i];
    if (n.op == OP_CONV) {
      n.in_dr = range_of(n.in0);
      const size_t per_out = n.cout > 0 ? n.weight.size() / (size_t)n.cout : 0;
      n.wdr.assign(n.cout, 0.f);
      for (int c = 0; c < n.cout; ++c) {
        float m = 0.f;
        for (size_t j = 0; j < per_out; ++j) {
          __half_raw r;
          r.x = n.weight[(size_t)c * per_out + j];
          m = fmaxf(m, fabsf(__half2float(__half(r))));
        }
        n.wdr[c] = m;
      }
    } else if (n.op == OP_ADD) {
      n.a_dr = n.b_dr = fmaxf(range_of(n.in0), range_of(n.in1));
    } else {
      continue;
    }
    if (!e->user_prec[i]) n.prec = n.out_prec = SPCONVB_PRECISION_INT8;
  }
  e->precision = SPCONVB_PRECISION_INT8;
  e->collecting = false;  // the fp16 engine keeps running until the next reconfigure
  return SPCONVB_OK;
}

int spconvb_engine_reconfigure(spconvb_engine* e, void* stream) {
  if (!e) return SPCONVB_E_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) return SPCONVB_E_DEVICE;
  const bool calib = e->want_calibration;
  std::unique_ptr<Engine> fresh(new (std::nothrow) Engine());
  if (!fresh) return SPCONVB_E_NOMEM;
  const int rc = fresh->compile(
      e->graph, calib ? SPCONVB_PRECISION_FP16 : e->precision,
      calib ? (SPCONVB_BUILD_KEEP_TENSORS | SPCONVB_BUILD_NO_FUSION) : e->flags,
      (cudaStream_t)stream);
  if (rc != SPCONVB_OK) return rc;
  if (e->absmax) {
    cudaFree(e->absmax);
    e->absmax = nullptr;
  }
  if (calib) {
    const size_t bytes = sizeof(float) * (fresh->rt.size() + 1);
    if (cudaMalloc((void**)&e->absmax, bytes) != cudaSuccess) return SPCONVB_E_NOMEM;
    cudaMemset(e->absmax, 0, bytes);
  }
  e->e = std::move(fresh);
  e->collecting = calib;
  return SPCONVB_OK;
}

void spconvb_engine_destroy(spconvb_engine* e) { delete e; }

int spconvb_engine_forward(spconvb_engine* e, const void* features, uint32_t n,
                           const int32_t* indices, const int32_t grid[3], int32_t batch,
                           void* stream) {
  if (!e) return SPCONVB_E_ARG;
  int rc = e->e->forward(features, indices, n, n, nullptr, grid, batch, (cudaStream_t)stream);
  if (rc == SPCONVB_OK && e->collecting)
    rc = e->e->collect_absmax(e->absmax, (cudaStream_t)stream);
  return rc;
}

int spconvb_engine_forward_dds(spconvb_engine* e, const void* features, const int32_t* indices,
                               uint32_t cap_rows, const uint32_t* n_dev, const int32_t grid[3],
                               int32_t batch, void* stream) {
  if (!e || !n_dev) return SPCONVB_E_ARG;
  int rc = e->e->forward(features, indices, cap_rows, 0, n_dev, grid, batch,
                         (cudaStream_t)stream);
  if (rc == SPCONVB_OK && e->collecting)
    rc = e->e->collect_absmax(e->absmax, (cudaStream_t)stream);
  return rc;
}

int spconvb_engine_prepare(spconvb_engine* e, const int32_t grid[3], int32_t batch) {
  if (!e || !grid) return SPCONVB_E_ARG;
  return e->e->prepare(grid, batch);
}

int spconvb_engine_num_outputs(const spconvb_engine* e) {
  return e ? (int)e->e->outputs.size() : SPCONVB_E_ARG;
}

int spconvb_engine_output(const spconvb_engine* e, int i, void** data, int64_t shape[8],
                          int32_t* ndim, int32_t* kind, int32_t* dense) {
  if (!e || i < 0 || i >= (int)e->e->outputs.size()) return SPCONVB_E_ARG;
  const RTensor& t = e->e->rt[e->e->outputs[i]];
  if (data) *data = t.data;
  if (kind) *kind = t.kind;
  if (dense) *dense = t.dense ? 1 : 0;
  int nd = 0;
  if (t.dense) {
    for (auto v : t.shape)
      if (nd < 8 && shape) shape[nd++] = v;
  } else if (shape) {
    shape[0] = t.cs >= 0 ? e->e->coordsets[t.cs].cap : 0;
    shape[1] = t.channels;
    nd = 2;
  }
  if (ndim) *ndim = nd;
  return SPCONVB_OK;
}

int spconvb_engine_output_layout(const spconvb_engine* e, int i, int32_t* layout,
                                 int64_t physical_shape[8], int32_t* ndim, size_t* bytes) {
  if (!e || i < 0 || i >= (int)e->e->outputs.size()) return SPCONVB_E_ARG;
  const RTensor& t = e->e->rt[e->e->outputs[i]];
  if (layout) *layout = t.dense ? t.layout : 0;
  int nd = 0;
  if (t.dense) {
    for (auto v : t.phys_shape)
      if (nd < 8 && physical_shape) physical_shape[nd++] = v;
  }
  if (ndim) *ndim = nd;
  if (bytes) *bytes = t.bytes;
  return SPCONVB_OK;
}

int spconvb_engine_output_rows(const spconvb_engine* e, int i, int32_t** coords,
                               uint32_t** n_ptr, uint32_t* cap, int32_t grid[3],
                               int32_t* on_input_rows) {
  if (!e || i < 0 || i >= (int)e->e->outputs.size()) return SPCONVB_E_ARG;
  const RTensor& t = e->e->rt[e->e->outputs[i]];
  if (t.dense || t.cs < 0) return SPCONVB_E_ARG;
  const CoordSet& cs = e->e->coordsets[t.cs];
  if (coords) *coords = cs.external ? nullptr : cs.coords;
  if (n_ptr) *n_ptr = cs.n_ptr;
  if (cap) *cap = cs.cap;
  if (grid)
    for (int a = 0; a < 3; ++a) grid[a] = cs.grid[a];
  if (on_input_rows) *on_input_rows = cs.external ? 1 : 0;
  return SPCONVB_OK;
}

int spconvb_engine_tensor(const spconvb_engine* e, const char* name, spconvb_tensor_view* v) {
  if (!e || !name || !v) return SPCONVB_E_ARG;
  auto it = e->e->by_name.find(name);
  if (it == e->e->by_name.end()) return SPCONVB_E_ARG;
  const RTensor& t = e->e->rt[it->second];
  memset(v, 0, sizeof(*v));
  v->features = t.data;
  v->kind = t.kind;
  v->channels = t.channels;
  v->scale = t.kind == SPCONVB_I8 ? t.dr / 127.0f : 1.f;
  v->dense = t.dense ? 1 : 0;
  if (t.cs >= 0) {
    const CoordSet& cs = e->e->coordsets[t.cs];
    v->coords = cs.coords;
    v->n_ptr = cs.n_ptr;
    v->cap = cs.cap;
    for (int a = 0; a < 3; ++a) v->grid[a] = cs.grid[a];
  }
  return SPCONVB_OK;
}

const char* spconvb_engine_tensor_names(const spconvb_engine* e) {
  return e ? e->e->names_text.c_str() : "";
}

const char* spconvb_engine_describe(const spconvb_engine* e) {
  return e ? e->e->describe_text.c_str() : "";
}

int spconvb_engine_num_steps(const spconvb_engine* e) { return e ? (int)e->e->steps.size() : 0; }

int spconvb_engine_profile(spconvb_engine* e, const void* features, uint32_t n,
                           const int32_t* indices, const int32_t grid[3], int32_t batch,
                           void* stream, float* step_ms, int32_t max_steps, int32_t reps,
                           void* flush, size_t flush_bytes) {
  if (!e || !step_ms || max_steps < 1) return SPCONVB_E_ARG;
  Profile p;
  p.step_ms = step_ms;
  p.max_steps = max_steps;
  p.reps = reps < 1 ? 1 : reps;
  p.flush = flush;
  p.flush_bytes = flush_bytes;
  return e->e->forward(features, indices, n, n, nullptr, grid, batch, (cudaStream_t)stream, &p);
}

int spconvb_engine_coordset(const spconvb_engine* e, int i, uint32_t** n_ptr, uint32_t* cap,
                            int32_t grid[3]) {
  if (!e || i < 0 || i >= (int)e->e->coordsets.size()) return SPCONVB_E_ARG;
  const CoordSet& cs = e->e->coordsets[i];
  if (n_ptr) *n_ptr = cs.n_ptr;
  if (cap) *cap = cs.cap;
  if (grid)
    for (int a = 0; a < 3; ++a) grid[a] = cs.grid[a];
  return SPCONVB_OK;
}

int spconvb_engine_num_rules(const spconvb_engine* e) { return e ? (int)e->e->rules.size() : 0; }

int spconvb_engine_rule(const spconvb_engine* e, int i, int32_t** map, uint32_t* cap,
                        int32_t* kvol, uint32_t** n_out_ptr, uint32_t** n_in_ptr) {
  if (!e || i < 0 || i >= (int)e->e->rules.size()) return SPCONVB_E_ARG;
  const Rule& r = e->e->rules[i];
  if (map) *map = r.map;
  if (cap) *cap = e->e->coordsets[r.out_cs].cap;
  if (kvol) *kvol = r.kvol;
  if (n_out_ptr) *n_out_ptr = e->e->coordsets[r.out_cs].n_ptr;
  if (n_in_ptr) *n_in_ptr = e->e->coordsets[r.in_cs].n_ptr;
  return SPCONVB_OK;
}

int spconvb_read_device(const void* device_src, void* host_dst, size_t bytes, void* stream) {
  if (!device_src || !host_dst) return SPCONVB_E_ARG;
  cudaError_t ce = cudaStreamSynchronize((cudaStream_t)stream);
  if (ce != cudaSuccess) return (int)ce;
  ce = cudaMemcpy(host_dst, device_src, bytes, cudaMemcpyDeviceToHost);
  return ce == cudaSuccess ? SPCONVB_OK : (int)ce;
}

int spconvb_copy_async(void* dst, const void* src, size_t bytes, int32_t direction, void* stream) {
  if (!dst || !src || direction < 0 || direction > 2) return SPCONVB_E_ARG;
  const cudaMemcpyKind kind = direction == 0 ? cudaMemcpyHostToDevice
                              : direction == 1 ? cudaMemcpyDeviceToHost
                                               : cudaMemcpyDeviceToDevice;
  cudaError_t ce = cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream);
  return ce == cudaSuccess ? SPCONVB_OK : (int)ce;
}

int spconvb_engine_status(const spconvb_engine* e, uint32_t out[4], void* stream) {
  if (!e || !out) return SPCONVB_E_ARG;
  if (!e->e->status) {
    memset(out, 0, 4 * sizeof(uint32_t));
    return SPCONVB_OK;
  }
  return spconvb_read_device(e->e->status, out, 4 * sizeof(uint32_t), stream);
}

int spconvb_engine_last_launches(const spconvb_engine* e) { return e ? e->e->last_launches : 0; }

}  // extern "C"
