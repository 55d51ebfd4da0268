// Reads the custom sparse-convolution ONNX files the reference's exporters write
// and replays them into a Builder, following the operator schema of
// libraries/3DSparseConvolution/src/onnx-parser.cpp:101-231 (op types
// SparseConvolution, Add / QuantAdd, Relu, ScatterDense, Reshape, Transpose;
// missing attributes read as 0 / "" / empty; output_bound defaults to 150000).
//
// The file is decoded straight from the protobuf wire format, so no protobuf
// library or generated code is needed.  Field numbers used (onnx.proto):
//   ModelProto.graph = 7
//   GraphProto.node = 1, initializer = 5, input = 11, output = 12
//   NodeProto.input = 1, output = 2, name = 3, op_type = 4, attribute = 5
//   AttributeProto.name = 1, f = 2, i = 3, s = 4, floats = 7, ints = 8
//   TensorProto.dims = 1, data_type = 2, name = 8, raw_data = 9  (FLOAT16 = 10)
//   ValueInfoProto.name = 1
#include <stdio.h>
#include <string.h>

#include <map>

#include "engine.hpp"

namespace spconvb {
namespace {

struct Span {
  const uint8_t* p = nullptr;
  const uint8_t* e = nullptr;
  bool ok = true;
  bool done() const { return !ok || p >= e; }
};

uint64_t read_varint(Span& s) {
  uint64_t v = 0;
  for (int shift = 0; shift < 64; shift += 7) {
    if (s.p >= s.e) { s.ok = false; return 0; }
    const uint8_t b = *s.p++;
    v |= (uint64_t)(b & 0x7f) << shift;
    if (!(b & 0x80)) return v;
  }
  s.ok = false;
  return 0;
}

struct Field {
  uint32_t number = 0;
  uint32_t wire = 0;
  uint64_t value = 0;   // varint / fixed
  Span bytes;           // length-delimited payload
};

bool next_field(Span& s, Field& f) {
  if (s.done()) return false;
  const uint64_t key = read_varint(s);
  if (!s.ok) return false;
  f.number = (uint32_t)(key >> 3);
  f.wire = (uint32_t)(key & 7);
  switch (f.wire) {
    case 0: f.value = read_varint(s); break;
    case 1:
      if (s.e - s.p < 8) { s.ok = false; return false; }
      memcpy(&f.value, s.p, 8); s.p += 8; break;
    case 2: {
      const uint64_t len = read_varint(s);
      if (!s.ok || (uint64_t)(s.e - s.p) < len) { s.ok = false; return false; }
      f.bytes.p = s.p; f.bytes.e = s.p + len; f.bytes.ok = true;
      s.p += len;
      break;
    }
    case 5: {
      if (s.e - s.p < 4) { s.ok = false; return false; }
      uint32_t v; memcpy(&v, s.p, 4); f.value = v; s.p += 4; break;
    }
    default: s.ok = false; return false;
  }
  return s.ok;
}

std::string to_string(const Span& b) { return std::string((const char*)b.p, (size_t)(b.e - b.p)); }

struct Attr {
  float f = 0.f;
  int64_t i = 0;
  std::string s;
  std::vector<float> floats;
  std::vector<int64_t> ints;
};

struct Init {
  std::vector<int64_t> dims;
  int data_type = 0;
  Span raw;
};

struct Node {
  std::string name, op;
  std::vector<std::string> in, out;
  std::map<std::string, Attr> attrs;
};

bool parse_attr(Span s, std::string& name, Attr& a) {
  Field f;
  while (next_field(s, f)) {
    switch (f.number) {
      case 1: name = to_string(f.bytes); break;
      case 2: { uint32_t v = (uint32_t)f.value; memcpy(&a.f, &v, 4); break; }
      case 3: a.i = (int64_t)f.value; break;
      case 4: a.s = to_string(f.bytes); break;
      case 7:
        if (f.wire == 2) {
          for (const uint8_t* p = f.bytes.p; p + 4 <= f.bytes.e; p += 4) {
            float v; memcpy(&v, p, 4); a.floats.push_back(v);
          }
        } else { uint32_t v = (uint32_t)f.value; float x; memcpy(&x, &v, 4); a.floats.push_back(x); }
        break;
      case 8:
        if (f.wire == 2) {
          Span in = f.bytes;
          while (!in.done()) { int64_t v = (int64_t)read_varint(in); if (in.ok) a.ints.push_back(v); }
          if (!in.ok) return false;
        } else a.ints.push_back((int64_t)f.value);
        break;
      default: break;
    }
  }
  return s.ok;
}

bool parse_tensor(Span s, std::string& name, Init& t) {
  Field f;
  while (next_field(s, f)) {
    switch (f.number) {
      case 1:
        if (f.wire == 2) {
          Span in = f.bytes;
          while (!in.done()) { int64_t v = (int64_t)read_varint(in); if (in.ok) t.dims.push_back(v); }
          if (!in.ok) return false;
        } else t.dims.push_back((int64_t)f.value);
        break;
      case 2: t.data_type = (int)f.value; break;
      case 8: name = to_string(f.bytes); break;
      case 9: t.raw = f.bytes; break;
      default: break;
    }
  }
  return s.ok;
}

bool parse_node(Span s, Node& n) {
  Field f;
  while (next_field(s, f)) {
    switch (f.number) {
      case 1: n.in.push_back(to_string(f.bytes)); break;
      case 2: n.out.push_back(to_string(f.bytes)); break;
      case 3: n.name = to_string(f.bytes); break;
      case 4: n.op = to_string(f.bytes); break;
      case 5: {
        std::string an;
        Attr a;
        if (f.wire != 2 || !parse_attr(f.bytes, an, a)) return false;
        n.attrs[an] = a;
        break;
      }
      default: break;
    }
  }
  return s.ok;
}

std::string value_info_name(Span s) {
  Field f;
  while (next_field(s, f))
    if (f.number == 1 && f.wire == 2) return to_string(f.bytes);
  return std::string();
}

const Attr& attr(const Node& n, const char* name) {
  static const Attr empty;
  auto it = n.attrs.find(name);
  if (it == n.attrs.end()) {
    log_msg(LOG_VERB, "node '%s' has no attribute '%s', the default is used", n.name.c_str(), name);
    return empty;
  }
  return it->second;
}

void ints3(const Attr& a, int out[3], int fill) {
  for (int i = 0; i < 3; ++i) out[i] = i < (int)a.ints.size() ? (int)a.ints[i] : fill;
}

bool fp16_initializer(const std::map<std::string, Init>& inits, const std::string& name,
                      std::vector<uint16_t>& data, std::vector<int>& shape) {
  auto it = inits.find(name);
  if (it == inits.end()) {
    log_msg(LOG_ERROR, "initializer '%s' not found", name.c_str());
    return false;
  }
  const Init& t = it->second;
  if (t.data_type != 10) {
    log_msg(LOG_ERROR, "initializer '%s' has data type %d, only FLOAT16 raw data is supported",
            name.c_str(), t.data_type);
    return false;
  }
  size_t vol = 1;
  for (auto d : t.dims) { shape.push_back((int)d); vol *= (size_t)d; }
  if (vol * 2 != (size_t)(t.raw.e - t.raw.p)) {
    log_msg(LOG_ERROR, "initializer '%s': %zu bytes of raw data for %zu elements", name.c_str(),
            (size_t)(t.raw.e - t.raw.p), vol);
    return false;
  }
  data.resize(vol);
  memcpy(data.data(), t.raw.p, vol * 2);
  return true;
}

int prec_of(const std::string& s) {
  return s == "int8" ? SPCONVB_PRECISION_INT8 : SPCONVB_PRECISION_FP16;
}

}  // namespace

int load_onnx(const char* path, uint32_t fixed_launch_points, Builder* out) {
  FILE* fp = fopen(path, "rb");
  if (!fp) {
    log_msg(LOG_ERROR, "cannot open '%s'", path);
    return SPCONVB_E_PARSE;
  }
  std::vector<uint8_t> buf;
  fseek(fp, 0, SEEK_END);
  const long size = ftell(fp);
  fseek(fp, 0, SEEK_SET);
  if (size <= 0) { fclose(fp); return SPCONVB_E_PARSE; }
  buf.resize((size_t)size);
  const size_t got = fread(buf.data(), 1, buf.size(), fp);
  fclose(fp);
  if (got != buf.size()) return SPCONVB_E_PARSE;

  Span model;
  model.p = buf.data();
  model.e = buf.data() + buf.size();
  Span graph;
  bool have_graph = false;
  Field f;
  while (next_field(model, f))
    if (f.number == 7 && f.wire == 2) { graph = f.bytes; have_graph = true; }
  if (!model.ok || !have_graph) {
    log_msg(LOG_ERROR, "'%s' is not an ONNX model (no graph)", path);
    return SPCONVB_E_PARSE;
  }

  std::vector<Node> nodes;
  std::map<std::string, Init> inits;
  std::vector<std::string> inputs, outputs;
  while (next_field(graph, f)) {
    if (f.wire != 2) continue;
    if (f.number == 1) {
      Node n;
      if (!parse_node(f.bytes, n)) return SPCONVB_E_PARSE;
      nodes.push_back(std::move(n));
    } else if (f.number == 5) {
      std::string name;
      Init t;
      if (!parse_tensor(f.bytes, name, t)) return SPCONVB_E_PARSE;
      inits[name] = t;
    } else if (f.number == 11) {
      inputs.push_back(value_info_name(f.bytes));
    } else if (f.number == 12) {
      outputs.push_back(value_info_name(f.bytes));
    }
  }
  if (!graph.ok) {
    log_msg(LOG_ERROR, "'%s' is truncated or corrupt", path);
    return SPCONVB_E_PARSE;
  }

  std::map<std::string, int> tensor_of;
  for (const auto& name : inputs) {
    if (inits.count(name)) continue;  // some exporters list initializers as inputs
    GNode n;
    n.op = OP_INPUT;
    n.name = name;
    tensor_of[name] = out->push(std::move(n), name);
  }
  auto find = [&](const std::string& name) -> int {
    auto it = tensor_of.find(name);
    if (it == tensor_of.end()) {
      log_msg(LOG_ERROR, "tensor '%s' is used before it is produced", name.c_str());
      return -1;
    }
    return it->second;
  };

  for (const Node& n : nodes) {
    if (n.out.empty() || n.in.empty()) return SPCONVB_E_PARSE;
    GNode g;
    g.name = n.name;
    uint32_t flp = fixed_launch_points;
    if (n.attrs.count("fixed_launch_points")) flp = (uint32_t)attr(n, "fixed_launch_points").i;
    if (n.op == "SparseConvolution") {
      if (n.in.size() < 2) return SPCONVB_E_PARSE;
      g.op = OP_CONV;
      if ((g.in0 = find(n.in[0])) < 0) return SPCONVB_E_PARSE;
      std::vector<int> wshape, bshape;
      if (!fp16_initializer(inits, n.in[1], g.weight, wshape)) return SPCONVB_E_PARSE;
      if (n.in.size() > 2 && !fp16_initializer(inits, n.in[2], g.bias, bshape)) return SPCONVB_E_PARSE;
      if (wshape.size() != 5) {
        log_msg(LOG_ERROR, "conv '%s': weight must be [Cout,K0,K1,K2,Cin]", n.name.c_str());
        return SPCONVB_E_PARSE;
      }
      g.cout = wshape[0];
      g.cin = wshape[4];
      ints3(attr(n, "kernel_size"), g.ksize, 1);
      ints3(attr(n, "stride"), g.stride, 1);
      ints3(attr(n, "padding"), g.pad, 0);
      ints3(attr(n, "dilation"), g.dil, 1);
      if (g.ksize[0] != wshape[1] || g.ksize[1] != wshape[2] || g.ksize[2] != wshape[3]) {
        log_msg(LOG_ERROR, "conv '%s': kernel_size does not match the weight shape", n.name.c_str());
        return SPCONVB_E_PARSE;
      }
      g.wdr = attr(n, "weight_dynamic_ranges").floats;
      g.relu_act = attr(n, "activation").s == "ReLU";
      const std::string& act = attr(n, "activation").s;
      if (!act.empty() && act != "ReLU" && act != "None") {
        log_msg(LOG_ERROR, "conv '%s': activation '%s' is not supported", n.name.c_str(), act.c_str());
        return SPCONVB_E_UNSUPPORTED;
      }
      g.in_dr = attr(n, "input_dynamic_range").f;
      g.subm = attr(n, "subm").i != 0;
      g.out_bound = n.attrs.count("output_bound") ? (uint32_t)attr(n, "output_bound").i : 150000u;
      g.fixed_launch = flp;
      if (n.attrs.count("rulebook")) g.rulebook = attr(n, "rulebook").s;
      g.prec = prec_of(attr(n, "precision").s);
      g.out_prec = prec_of(attr(n, "output_precision").s);
      g.inverse = attr(n, "inverse").i != 0;
    } else if (n.op == "Add" || n.op == "QuantAdd") {
      if (n.in.size() < 2) return SPCONVB_E_PARSE;
      g.op = OP_ADD;
      if ((g.in0 = find(n.in[0])) < 0 || (g.in1 = find(n.in[1])) < 0) return SPCONVB_E_PARSE;
      g.a_dr = attr(n, "input0_dynamic_range").f;
      g.b_dr = attr(n, "input1_dynamic_range").f;
      g.prec = prec_of(attr(n, "precision").s);
      g.out_prec = prec_of(attr(n, "output_precision").s);
      g.fixed_launch = flp;
    } else if (n.op == "Relu") {
      g.op = OP_RELU;
      if ((g.in0 = find(n.in[0])) < 0) return SPCONVB_E_PARSE;
    } else if (n.op == "ScatterDense") {
      g.op = OP_DENSE;
      if ((g.in0 = find(n.in[0])) < 0) return SPCONVB_E_PARSE;
      for (auto v : attr(n, "input_spatial_shape").ints) g.in_spatial.push_back((int)v);
      for (auto v : attr(n, "output_shape").ints) g.out_shape.push_back((int)v);
      g.format = attr(n, "format").s;
      g.dense_dr = attr(n, "input_dynamic_range").f;
      const std::string& lay = attr(n, "output_layout").s;
      g.layout = lay == "NCHW32" ? 2 : (lay == "NHWzC" ? 3 : 1);
    } else if (n.op == "Reshape" || n.op == "Transpose") {
      g.op = n.op == "Reshape" ? OP_RESHAPE : OP_TRANSPOSE;
      if ((g.in0 = find(n.in[0])) < 0) return SPCONVB_E_PARSE;
      g.dims = attr(n, "dims").ints;
    } else {
      log_msg(LOG_ERROR, "Unsupport operator [%s]", n.op.c_str());
      return SPCONVB_E_UNSUPPORTED;
    }
    tensor_of[n.out[0]] = out->push(std::move(g), n.out[0]);
  }
  for (const auto& name : outputs) {
    const int t = find(name);
    if (t < 0) return SPCONVB_E_PARSE;
    out->outputs.push_back(t);
  }
  return SPCONVB_OK;
}

}  // namespace spconvb
