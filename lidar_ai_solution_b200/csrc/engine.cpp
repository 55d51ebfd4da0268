// Engine: turns the builder's graph into a list of kernel launches and runs it.
//
// compile()  resolves precisions and int8 scales, fuses Add/ReLU into the
//            producing convolution, shares rulebooks between layers of one
//            resolution, quantises + packs + uploads the weights;
// prepare()  sizes every buffer for a grid and allocates them once;
// forward()  zeroes the hash tables / bitmaps with one memset and enqueues the
//            steps.  No host synchronisation and no allocation happens in
//            forward(), so a caller may capture it in a CUDA graph.
#include "engine.hpp"

#include <cuda_fp16.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>

namespace spconvb {

// ------------------------------------------------------------------ logging
static int g_log_level = LOG_WARN;
static spconvb_log_fn g_log_fn = nullptr;

void log_msg(int level, const char* fmt, ...) {
  if (level < g_log_level) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (g_log_fn) {
    g_log_fn(level, buf);
    return;
  }
  const char* tag = level == LOG_VERB ? "verb" : (level == LOG_WARN ? "warn" : "error");
  fprintf(stderr, "[spconvb %s] %s\n", tag, buf);
}

static float half_bits_to_float(uint16_t h) {
  __half_raw r;
  r.x = h;
  return __half2float(__half(r));
}
// ------------------------------------------------------------------ builder
int Builder::new_tensor(const std::string& name, int producer) {
  GTensor t;
  t.name = name;
  t.producer = producer;
  tensors.push_back(t);
  return (int)tensors.size() - 1;
}

int Builder::push(GNode&& n, const std::string& out_name) {
  const int idx = (int)nodes.size();
  if (n.in0 >= 0) tensors[n.in0].consumers.push_back(idx);
  if (n.in1 >= 0) tensors[n.in1].consumers.push_back(idx);
  n.out = new_tensor(out_name, idx);
  nodes.push_back(std::move(n));
  return nodes.back().out;
}

// ------------------------------------------------------------------- engine
Engine::~Engine() {
  free_prepared();
  for (cudaEvent_t e : rule_ev_)
    if (e) cudaEventDestroy(e);
  if (fork_ev_) cudaEventDestroy(fork_ev_);
  if (aux_) cudaStreamDestroy(aux_);
  for (auto& w : weights) {
    cudaFree(w.plain);
    cudaFree(w.packed);
    cudaFree(w.scale);
    cudaFree(w.bias);
  }
}

void Engine::free_prepared() {
  for (void* p : allocations_) cudaFree(p);
  allocations_.clear();
  prepared_ = false;
}

int Engine::dev_alloc(void** p, size_t bytes) {
  if (bytes == 0) bytes = 256;
  cudaError_t e = cudaMalloc(p, bytes);
  if (e != cudaSuccess) {
    log_msg(LOG_ERROR, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return SPCONVB_E_NOMEM;
  }
  allocations_.push_back(*p);
  return SPCONVB_OK;
}

static int eff_precision(int global, int layer) {
  if (global == SPCONVB_PRECISION_FP16) return SPCONVB_PRECISION_FP16;
  return layer == SPCONVB_PRECISION_INT8 ? SPCONVB_PRECISION_INT8 : SPCONVB_PRECISION_FP16;
}
static int kind_of_precision(int p) {
  return p == SPCONVB_PRECISION_INT8 ? SPCONVB_I8 : SPCONVB_F16;
}

// Channels as stored for the tensor-core kernel: rows of 16, 32, 64, 128 or
// 256 bytes.  Returns 0 when the shape has to take the CUDA-core kernel.
static int padded_cin(int compute, int cin) {
  const int es = compute == SPCONVB_I8 ? 1 : 2;
  int rb = 16;
  while (rb < cin * es) rb <<= 1;
  if (rb > 256) return 0;
  return rb / es;
}

static bool same3(const int* a, const int* b) { return a[0] == b[0] && a[1] == b[1] && a[2] == b[2]; }

int Engine::compile(const Builder& b, int precision, uint32_t build_flags, cudaStream_t st) {
  flags = build_flags;
  const int nn = (int)b.nodes.size();
  const int nt = (int)b.tensors.size();
  if (b.outputs.empty()) {
    log_msg(LOG_ERROR, "graph has no output");
    return SPCONVB_E_ARG;
  }
  const bool fuse = !(flags & SPCONVB_BUILD_NO_FUSION);
  std::vector<char> is_output(nt, 0);
  for (int t : b.outputs) is_output[t] = 1;

  // ---- effective precisions and storage kinds
  std::vector<int> prec(nn), out_prec(nn);
  for (int i = 0; i < nn; ++i) {
    prec[i] = eff_precision(precision, b.nodes[i].prec);
    out_prec[i] = eff_precision(precision, b.nodes[i].out_prec);
  }
  std::vector<int> kind(nt, SPCONVB_F16);
  for (int i = 0; i < nn; ++i) {
    const GNode& n = b.nodes[i];
    switch (n.op) {
      case OP_CONV:
      case OP_ADD: kind[n.out] = kind_of_precision(out_prec[i]); break;
      case OP_RELU: kind[n.out] = kind[n.in0]; break;
      default: kind[n.out] = SPCONVB_F16; break;
    }
    if (n.op == OP_INPUT) kind[n.out] = SPCONVB_F16;
  }

  // ---- fusion decisions
  std::vector<char> dead(nn, 0);
  std::vector<int> add_relu(nn, 0), final_out(nn, -1), fused_add(nn, -1);
  for (int i = 0; i < nn; ++i) final_out[i] = b.nodes[i].out;
  if (fuse) {
    for (int i = 0; i < nn; ++i) {
      const GNode& n = b.nodes[i];
      if (n.op != OP_ADD) continue;
      const GTensor& o = b.tensors[n.out];
      if (is_output[n.out] || o.consumers.size() != 1) continue;
      const int r = o.consumers[0];
      if (b.nodes[r].op != OP_RELU) continue;
      add_relu[i] = 1;
      final_out[i] = b.nodes[r].out;
      dead[r] = 1;
    }
    for (int i = 0; i < nn; ++i) {
      const GNode& n = b.nodes[i];
      if (n.op != OP_CONV) continue;
      const GTensor& o = b.tensors[n.out];
      if (is_output[n.out] || o.consumers.size() != 1) continue;
      const int a = o.consumers[0];
      const GNode& an = b.nodes[a];
      if (an.op != OP_ADD || dead[a] || an.in0 == an.in1) continue;
      const int other = an.in0 == n.out ? an.in1 : an.in0;
      if (b.tensors[other].producer >= i) continue;  // not yet computed when the conv runs
      fused_add[i] = a;
      dead[a] = 1;
    }
  }

  // ---- int8 scales: a tensor is stored with the dynamic range its consumer expects
  std::vector<float> dr(nt, 0.f);
  for (int t = nt - 1; t >= 0; --t) {
    if (kind[t] != SPCONVB_I8) continue;
    float v = 0.f;
    for (int c : b.tensors[t].consumers) {
      const GNode& cn = b.nodes[c];
      if (cn.op == OP_CONV && prec[c] == SPCONVB_PRECISION_INT8 && cn.in_dr > 0.f) v = cn.in_dr;
      else if (cn.op == OP_ADD) v = (cn.in0 == t) ? cn.a_dr : cn.b_dr;
      else if (cn.op == OP_DENSE) v = cn.dense_dr;
      else if (cn.op == OP_RELU) v = dr[cn.out];
      if (v > 0.f) break;
    }
    if (v > 0.f) {
      dr[t] = v;
    } else {
      log_msg(LOG_WARN, "tensor '%s' is int8 but no consumer gives it a dynamic range; stored as fp16",
              b.tensors[t].name.c_str());
      kind[t] = SPCONVB_F16;
    }
  }
  // ReLU keeps the representation of its input
  for (int i = 0; i < nn; ++i)
    if (b.nodes[i].op == OP_RELU && kind[b.nodes[i].in0] != kind[b.nodes[i].out]) {
      kind[b.nodes[i].out] = kind[b.nodes[i].in0];
      dr[b.nodes[i].out] = dr[b.nodes[i].in0];
    }

  // ---- walk the graph, emit steps
  std::vector<int> g2r(nt, -1);  // graph tensor -> runtime tensor
  std::vector<char> hash_emitted;
  std::unordered_map<std::string, int> rule_by_name;  // strided rulebooks, for inverse convs
  struct ConvKey { int src, kind, ch; float s; int rt; };
  std::vector<ConvKey> converted;

  auto new_rt = [&](const std::string& name, int cs, int ch, int k, float d) {
    RTensor t;
    t.name = name;
    t.cs = cs;
    t.channels = ch;
    t.kind = k;
    t.dr = d;
    rt.push_back(t);
    return (int)rt.size() - 1;
  };
  auto touch = [&](int r, int step) {
    while (r >= 0) {
      rt[r].first_step = std::min(rt[r].first_step, step);
      rt[r].last_step = std::max(rt[r].last_step, step);
      r = rt[r].alias_of;
    }
  };
  // Only the caller's rows need a hash table; rows made by a strided rulebook are
  // looked up by rank in the bitmap that rulebook leaves behind.
  auto ensure_hash = [&](int cs) {
    if (!coordsets[cs].external) return;
    coordsets[cs].need_table = true;
    if ((int)hash_emitted.size() <= cs) hash_emitted.resize(cs + 1, 0);
    if (coordsets[cs].external && !hash_emitted[cs]) {
      Step s;
      s.kind = Step::HASH;
      s.name = "hash";
      s.cs = cs;
      steps.push_back(s);
      hash_emitted[cs] = 1;
    }
  };

  for (int i = 0; i < nn; ++i) {
    if (dead[i]) continue;
    const GNode& n = b.nodes[i];
    switch (n.op) {
      case OP_INPUT: {
        if (input_rt_ >= 0) {
          log_msg(LOG_ERROR, "only one sparse input is supported");
          return SPCONVB_E_UNSUPPORTED;
        }
        CoordSet cs;
        cs.external = true;
        coordsets.push_back(cs);
        input_rt_ = new_rt(b.tensors[n.out].name, (int)coordsets.size() - 1, 0, SPCONVB_F16, 0.f);
        rt[input_rt_].external = true;
        g2r[n.out] = input_rt_;
        break;
      }
      case OP_CONV: {
        int src = g2r[n.in0];
        if (src < 0 || rt[src].dense) return SPCONVB_E_ARG;
        const int compute = kind_of_precision(prec[i]);
        if (src == input_rt_ && rt[src].channels == 0) {
          rt[src].channels = n.cin;  // the first conv tells the input width
          input_channels_ = n.cin;
        }
        const int in_cs = rt[src].cs;
        coordsets[in_cs].bound = std::max(coordsets[in_cs].bound, n.subm ? n.out_bound : 0u);
        if (coordsets[in_cs].external && coordsets[in_cs].bound == 0)
          coordsets[in_cs].bound = n.out_bound;
        // --- input representation
        const bool cout_ok = n.cout == 16 || n.cout == 32 || n.cout == 64 || n.cout == 128;
        const bool taps_ok = n.ksize[0] * n.ksize[1] * n.ksize[2] <= 27;
        int cpad = (flags & SPCONVB_BUILD_FORCE_SIMT) || !cout_ok || !taps_ok ? 0 : padded_cin(compute, n.cin);
        const bool umma = cpad != 0;
        if (!umma) cpad = n.cin;
        float in_scale = 1.f;  // scale of the int8 input actually fed to the MMA
        int feed = src;
        if (rt[src].channels != n.cin) {
          log_msg(LOG_ERROR, "conv '%s': input has %d channels, weights expect %d", n.name.c_str(),
                  rt[src].channels, n.cin);
          return SPCONVB_E_ARG;
        }
        float conv_s = 1.f;
        bool need_convert = rt[src].kind != compute || rt[src].channels != cpad;
        if (compute == SPCONVB_I8) {
          if (rt[src].kind == SPCONVB_I8) in_scale = rt[src].dr / 127.0f;
          else {
            if (!(n.in_dr > 0.f)) {
              log_msg(LOG_ERROR, "conv '%s' is int8 but has no input_dynamic_range", n.name.c_str());
              return SPCONVB_E_ARG;
            }
            in_scale = n.in_dr / 127.0f;
            conv_s = 127.0f / n.in_dr;
          }
        } else if (rt[src].kind == SPCONVB_I8) {
          conv_s = rt[src].dr / 127.0f;
        }
        if (need_convert) {
          int found = -1;
          for (auto& c : converted)
            if (c.src == src && c.kind == compute && c.ch == cpad && c.s == conv_s) found = c.rt;
          if (found < 0) {
            found = new_rt(rt[src].name + ":as_" + (compute == SPCONVB_I8 ? "i8" : "f16") +
                               std::to_string(cpad),
                           in_cs, cpad, compute, compute == SPCONVB_I8 ? in_scale * 127.0f : 0.f);
            Step s;
            s.kind = Step::CONVERT;
            s.cs = in_cs;
            s.name = "convert:" + n.name;
            s.in0 = src;
            s.out = found;
            s.cin = rt[src].channels;
            s.cout = cpad;
            s.s = conv_s;
            steps.push_back(s);
            touch(src, (int)steps.size() - 1);
            touch(found, (int)steps.size() - 1);
            converted.push_back({src, compute, cpad, conv_s, found});
          }
          feed = found;
        }
        // --- rulebook (shared by structure)
        const int kvol = n.ksize[0] * n.ksize[1] * n.ksize[2];
        int rule = -1;
        if (n.inverse) {
          // the pairs of an earlier strided conv, found by its rulebook name, with input and
          // output swapped; the geometry is that conv's (an inverse conv module carries only
          // the kernel size)
          auto it = rule_by_name.find(n.rulebook);
          if (n.rulebook.empty() || it == rule_by_name.end()) {
            log_msg(LOG_ERROR, "conv '%s': inverse needs the rulebook of an earlier strided conv",
                    n.name.c_str());
            return SPCONVB_E_ARG;
          }
          const int fwd = it->second;
          if (rules[fwd].out_cs != in_cs || rules[fwd].kvol != kvol) {
            log_msg(LOG_ERROR, "conv '%s': input rows or kernel do not match rulebook '%s'",
                    n.name.c_str(), n.rulebook.c_str());
            return SPCONVB_E_ARG;
          }
          for (int r = 0; r < (int)rules.size(); ++r)
            if (rules[r].inverse_of == fwd) rule = r;
          if (rule < 0) {
            Rule R = rules[fwd];
            R.inverse_of = fwd;
            R.in_cs = rules[fwd].out_cs;
            R.out_cs = rules[fwd].in_cs;
            R.map = nullptr;
            R.ws = nullptr;
            R.ws_bytes = 0;
            rules.push_back(R);
            rule = (int)rules.size() - 1;
            Step s;
            s.kind = Step::INV_MAP;
            s.name = "inverse_map:" + n.rulebook;
            s.rule = rule;
            s.cs = R.out_cs;
            steps.push_back(s);
          }
        }
        for (int r = 0; r < (int)rules.size() && !n.inverse; ++r) {
          const Rule& R = rules[r];
          if (R.inverse_of < 0 && R.subm == n.subm && R.in_cs == in_cs && same3(R.ksize, n.ksize) &&
              same3(R.dil, n.dil) && (n.subm || (same3(R.stride, n.stride) && same3(R.pad, n.pad))))
            rule = r;
        }
        if (rule < 0) {
          Rule R;
          R.subm = n.subm;
          R.kvol = kvol;
          R.in_cs = in_cs;
          for (int a = 0; a < 3; ++a) {
            R.ksize[a] = n.ksize[a]; R.stride[a] = n.subm ? 1 : n.stride[a];
            R.pad[a] = n.pad[a]; R.dil[a] = n.dil[a];
          }
          if (n.subm) ensure_hash(in_cs);
          Step s;
          if (n.subm) {
            R.out_cs = in_cs;
            s.kind = Step::SUBM_MAP;
            s.name = "subm_map:" + (n.rulebook.empty() ? n.name : n.rulebook);
          } else {
            CoordSet cs;
            cs.bound = n.out_bound;
            cs.made_by_rule = (int)rules.size();
            coordsets.push_back(cs);
            R.out_cs = (int)coordsets.size() - 1;
            s.kind = Step::DOWN_MAP;
            s.name = "down_map:" + (n.rulebook.empty() ? n.name : n.rulebook);
          }
          rules.push_back(R);
          rule = (int)rules.size() - 1;
          s.rule = rule;
          s.cs = in_cs;
          steps.push_back(s);
        }
        if (!n.subm && !n.inverse && !n.rulebook.empty()) rule_by_name[n.rulebook] = rule;
        // --- weights
        LayerWeights lw;
        {
          const size_t per_out = (size_t)kvol * n.cin;
          if (n.weight.size() != per_out * n.cout) return SPCONVB_E_ARG;
          std::vector<float> bias_f(n.cout, 0.f);
          for (size_t c = 0; c < n.bias.size() && c < (size_t)n.cout; ++c)
            bias_f[c] = half_bits_to_float(n.bias[c]);
          std::vector<float> scale_f(n.cout, 1.f);
          std::vector<uint8_t> plain;  // [cout][kvol][cpad]
          const int es = compute == SPCONVB_I8 ? 1 : 2;
          plain.assign((size_t)n.cout * kvol * cpad * es, 0);
          if (compute == SPCONVB_I8) {
            if ((int)n.wdr.size() != n.cout && n.wdr.size() != 1) {
              log_msg(LOG_ERROR, "conv '%s': %zu weight_dynamic_ranges for %d output channels",
                      n.name.c_str(), n.wdr.size(), n.cout);
              return SPCONVB_E_ARG;
            }
            for (int c = 0; c < n.cout; ++c) {
              const float amax = n.wdr.size() == 1 ? n.wdr[0] : n.wdr[c];
              const float inv = amax > 0.f ? 127.0f / amax : 0.f;
              scale_f[c] = in_scale * (amax / 127.0f);
              for (int k = 0; k < kvol; ++k)
                for (int ci = 0; ci < n.cin; ++ci) {
                  float r = rintf(half_bits_to_float(n.weight[c * per_out + (size_t)k * n.cin + ci]) * inv);
                  r = fminf(fmaxf(r, -127.f), 127.f);
                  ((int8_t*)plain.data())[((size_t)c * kvol + k) * cpad + ci] = (int8_t)r;
                }
            }
          } else {
            for (int c = 0; c < n.cout; ++c)
              for (int k = 0; k < kvol; ++k)
                for (int ci = 0; ci < n.cin; ++ci)
                  ((uint16_t*)plain.data())[((size_t)c * kvol + k) * cpad + ci] =
                      n.weight[c * per_out + (size_t)k * n.cin + ci];
          }
          auto upload = [&](void** dst, const void* src_h, size_t bytes) -> int {
            if (cudaMalloc(dst, bytes) != cudaSuccess) return SPCONVB_E_NOMEM;
            if (cudaMemcpyAsync(*dst, src_h, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess)
              return SPCONVB_E_NOMEM;
            return cudaStreamSynchronize(st) == cudaSuccess ? SPCONVB_OK : SPCONVB_E_NOMEM;
          };
          int rc = SPCONVB_OK;
          if (umma) {
            std::vector<uint8_t> packed(spconvb_conv_packed_bytes(compute, cpad, n.cout, kvol));
            rc = spconvb_conv_pack_weights(compute, cpad, n.cout, kvol, plain.data(), packed.data());
            if (rc == SPCONVB_OK) rc = upload(&lw.packed, packed.data(), packed.size());
          } else {
            rc = upload(&lw.plain, plain.data(), plain.size());
          }
          if (rc == SPCONVB_OK) rc = upload((void**)&lw.bias, bias_f.data(), sizeof(float) * n.cout);
          if (rc == SPCONVB_OK && compute == SPCONVB_I8)
            rc = upload((void**)&lw.scale, scale_f.data(), sizeof(float) * n.cout);
          weights.push_back(lw);
          if (rc != SPCONVB_OK) return rc;
        }
        // --- the conv step
        Step s;
        s.kind = Step::CONV;
        s.name = n.name;
        s.rule = rule;
        s.cs = rules[rule].out_cs;
        s.in0 = feed;
        s.weights = (int)weights.size() - 1;
        s.cin = n.cin;
        s.cout = n.cout;
        s.cp.compute = compute;
        s.cp.cin = cpad;
        s.cp.cout = n.cout;
        s.cp.kvol = kvol;
        s.cp.act = n.relu_act ? SPCONVB_ACT_RELU : SPCONVB_ACT_NONE;
        s.cp.force_simt = umma ? 0 : 1;
        int out_t = n.out;
        if (fused_add[i] >= 0) {
          const int a = fused_add[i];
          const GNode& an = b.nodes[a];
          const int other = an.in0 == n.out ? an.in1 : an.in0;
          const int res = g2r[other];
          if (res < 0 || rt[res].cs != s.cs || rt[res].channels != n.cout) {
            log_msg(LOG_ERROR, "add '%s': operands do not share rows/channels", an.name.c_str());
            return SPCONVB_E_ARG;
          }
          s.in1 = res;
          s.cp.res_kind = rt[res].kind;
          s.cp.res_scale = rt[res].kind == SPCONVB_I8 ? rt[res].dr / 127.0f : 1.f;
          s.cp.mid_kind = kind[n.out];
          s.cp.mid_inv_scale = kind[n.out] == SPCONVB_I8 ? 127.0f / dr[n.out] : 1.f;
          s.cp.mid_scale = kind[n.out] == SPCONVB_I8 ? dr[n.out] / 127.0f : 1.f;
          s.cp.res_relu = add_relu[a];
          s.name += "+" + an.name;
          out_t = final_out[a];
        }
        s.cp.out_kind = kind[out_t];
        s.cp.inv_out_scale = kind[out_t] == SPCONVB_I8 ? 127.0f / dr[out_t] : 1.f;
        s.out = new_rt(b.tensors[out_t].name, s.cs, n.cout, kind[out_t], dr[out_t]);
        g2r[out_t] = s.out;
        steps.push_back(s);
        const int si = (int)steps.size() - 1;
        touch(feed, si);
        touch(s.in1, si);
        touch(s.out, si);
        break;
      }
      case OP_ADD: {
        const int a = g2r[n.in0], c = g2r[n.in1];
        if (a < 0 || c < 0 || rt[a].cs != rt[c].cs || rt[a].channels != rt[c].channels) {
          log_msg(LOG_ERROR, "add '%s': operands do not share rows/channels", n.name.c_str());
          return SPCONVB_E_ARG;
        }
        const int out_t = final_out[i];
        Step s;
        s.kind = Step::ADD;
        s.name = n.name;
        s.cs = rt[a].cs;
        s.in0 = a;
        s.in1 = c;
        s.relu = add_relu[i];
        s.cout = rt[a].channels;
        s.a_scale = rt[a].kind == SPCONVB_I8 ? rt[a].dr / 127.0f : 1.f;
        s.b_scale = rt[c].kind == SPCONVB_I8 ? rt[c].dr / 127.0f : 1.f;
        s.inv_out = kind[out_t] == SPCONVB_I8 ? 127.0f / dr[out_t] : 1.f;
        s.out = new_rt(b.tensors[out_t].name, s.cs, s.cout, kind[out_t], dr[out_t]);
        g2r[out_t] = s.out;
        steps.push_back(s);
        const int si = (int)steps.size() - 1;
        touch(a, si);
        touch(c, si);
        touch(s.out, si);
        break;
      }
      case OP_RELU: {
        const int a = g2r[n.in0];
        if (a < 0) return SPCONVB_E_ARG;
        Step s;
        s.kind = Step::RELU;
        s.name = n.name;
        s.cs = rt[a].cs;
        s.in0 = a;
        s.cout = rt[a].channels;
        s.out = new_rt(b.tensors[n.out].name, s.cs, s.cout, rt[a].kind, rt[a].dr);
        g2r[n.out] = s.out;
        steps.push_back(s);
        const int si = (int)steps.size() - 1;
        touch(a, si);
        touch(s.out, si);
        break;
      }
      case OP_DENSE: {
        const int a = g2r[n.in0];
        if (a < 0 || rt[a].dense) return SPCONVB_E_ARG;
        if (n.layout < 1 || n.layout > 3) {
          log_msg(LOG_ERROR, "dense '%s': unknown output layout %d", n.name.c_str(), n.layout);
          return SPCONVB_E_ARG;
        }
        Step s;
        s.kind = Step::DENSE;
        s.name = n.name;
        s.cs = rt[a].cs;
        s.in0 = a;
        s.cout = rt[a].channels;
        s.a_scale = rt[a].kind == SPCONVB_I8 ? rt[a].dr / 127.0f : 1.f;
        // Transpose of the spatial axes right after the scatter is folded into it;
        // a Reshape only renames the shape.
        std::vector<int64_t> shape;
        for (int v : n.out_shape) shape.push_back(v);
        std::vector<int64_t> shape5 = shape;  // the scatter's own (permuted) shape
        int cur = n.out;
        while (true) {
          const GTensor& t = b.tensors[cur];
          if (is_output[cur] || t.consumers.size() != 1) break;
          const int c = t.consumers[0];
          const GNode& cn = b.nodes[c];
          if (cn.op == OP_TRANSPOSE && !s.has_perm && shape.size() == 5 && cn.dims.size() == 5 &&
              cn.dims[0] == 0 && cn.dims[1] == 1) {
            int p[3] = {(int)cn.dims[2] - 2, (int)cn.dims[3] - 2, (int)cn.dims[4] - 2};
            if ((1 << p[0] | 1 << p[1] | 1 << p[2]) != 7) break;
            std::vector<int64_t> ns = shape;
            for (int a2 = 0; a2 < 3; ++a2) { s.perm[a2] = p[a2]; ns[2 + a2] = shape[2 + p[a2]]; }
            shape = ns;
            shape5 = ns;
            s.has_perm = true;
          } else if (cn.op == OP_RESHAPE) {
            int64_t total = 1, known = 1;
            int infer = -1;
            for (auto v : shape) total *= v;
            std::vector<int64_t> ns = cn.dims;
            for (size_t d = 0; d < ns.size(); ++d) {
              if (ns[d] == -1) infer = (int)d; else known *= ns[d];
            }
            if (infer >= 0 && known > 0) ns[infer] = total / known;
            int64_t chk = 1;
            for (auto v : ns) chk *= v;
            if (chk != total) {
              log_msg(LOG_ERROR, "reshape '%s' changes the element count", cn.name.c_str());
              return SPCONVB_E_ARG;
            }
            shape = ns;
          } else {
            break;
          }
          dead[c] = 1;
          cur = cn.out;
        }
        // input_dynamic_range switches the dense tensor to int8 with that range
        const bool i8_out = n.dense_dr > 0.f;
        s.layout = n.layout;
        s.inv_out = i8_out ? 127.0f / n.dense_dr : 1.f;
        if (s.layout != 1) {
          // the vectorised layouts are defined on the [N, C*D, H, W] view of the scatter
          const bool ok5 = shape.size() == 5;
          const bool ok4 = shape.size() == 4 && shape5.size() == 5 && shape[0] == shape5[0] &&
                           shape[1] == shape5[1] * shape5[2] && shape[2] == shape5[3] &&
                           shape[3] == shape5[4];
          if (!ok5 && !ok4) {
            log_msg(LOG_ERROR, "dense '%s': layout %d needs the [N,C,D,H,W] tensor or its [N,C*D,H,W] view",
                    n.name.c_str(), s.layout);
            return SPCONVB_E_UNSUPPORTED;
          }
        }
        s.out = new_rt(b.tensors[cur].name, s.cs, s.cout, i8_out ? SPCONVB_I8 : SPCONVB_F16,
                       i8_out ? n.dense_dr : 0.f);
        rt[s.out].dense = true;
        rt[s.out].shape = shape;
        rt[s.out].layout = s.layout;
        rt[s.out].phys_shape = shape;
        if (s.layout == 2)
          rt[s.out].phys_shape = {shape5[0], (shape5[1] * shape5[2] + 31) / 32, shape5[3], shape5[4], 32};
        else if (s.layout == 3)
          rt[s.out].phys_shape = {shape5[0], shape5[3], shape5[4], shape5[2], shape5[1]};
        g2r[cur] = s.out;
        steps.push_back(s);
        const int si = (int)steps.size() - 1;
        touch(a, si);
        touch(s.out, si);
        break;
      }
      case OP_RESHAPE:
      case OP_TRANSPOSE:
        log_msg(LOG_ERROR, "%s '%s' is only supported directly after ScatterDense",
                n.op == OP_RESHAPE ? "Reshape" : "Transpose", n.name.c_str());
        return SPCONVB_E_UNSUPPORTED;
    }
  }

  for (int t : b.outputs) {
    if (g2r[t] < 0) {
      log_msg(LOG_ERROR, "output '%s' was fused away or never produced", b.tensors[t].name.c_str());
      return SPCONVB_E_ARG;
    }
    rt[g2r[t]].is_output = true;
    outputs.push_back(g2r[t]);
  }
  for (int r = 0; r < (int)rt.size(); ++r) {
    by_name[rt[r].name] = r;
    names_text += rt[r].name + "\n";
  }
  for (const Step& s : steps) {
    static const char* kn[] = {"hash", "subm_map", "down_map", "convert", "conv", "add", "relu",
                               "dense", "inverse_map"};
    char line[512];
    snprintf(line, sizeof(line),
             "%s %s rule=%d in_cs=%d out_cs=%d cin=%d cout=%d kvol=%d in=%s out=%s res=%d\n",
             kn[s.kind], s.name.c_str(), s.rule, s.rule >= 0 ? rules[s.rule].in_cs : s.cs,
             s.rule >= 0 ? rules[s.rule].out_cs : s.cs, s.cin, s.cout,
             s.rule >= 0 ? rules[s.rule].kvol : 0,
             s.in0 >= 0 ? (rt[s.in0].kind == SPCONVB_I8 ? "i8" : "f16") : "-",
             s.out >= 0 ? (rt[s.out].kind == SPCONVB_I8 ? "i8" : "f16") : "-", s.in1 >= 0 ? 1 : 0);
    describe_text += line;
  }
  if (cudaStreamSynchronize(st) != cudaSuccess) return SPCONVB_E_NOMEM;
  return SPCONVB_OK;
}

int Engine::collect_absmax(float* out, cudaStream_t st) {
  if (!prepared_ || !out || !last_in_n_) return SPCONVB_E_ARG;
  for (int r = 0; r < (int)rt.size(); ++r) {
    const RTensor& t = rt[r];
    if (t.dense || t.alias_of >= 0 || !t.data || t.cs < 0) continue;
    const CoordSet& cs = coordsets[t.cs];
    const bool ext = cs.external;
    const int ch = r == input_rt_ ? input_channels_ : t.channels;
    if (ch < 1) continue;
    const int rc = spconvb_absmax(t.data, t.kind, ch, ext ? last_in_n_ : cs.n_ptr,
                                  ext ? last_in_cap_ : cs.cap, out + r, st);
    if (rc != SPCONVB_OK) return rc;
  }
  return SPCONVB_OK;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static bool is_rulebook_step(const Step& s) {
  return s.kind == Step::HASH || s.kind == Step::SUBM_MAP || s.kind == Step::DOWN_MAP ||
         s.kind == Step::INV_MAP;
}

int Engine::prepare(const int32_t grid[3], int batch) {
  if (prepared_ && same3(grid_, grid) && batch_ == batch) return SPCONVB_OK;
  cudaDeviceSynchronize();
  free_prepared();
  if (batch < 1 || grid[0] < 1 || grid[1] < 1 || grid[2] < 1) return SPCONVB_E_ARG;
  for (int a = 0; a < 3; ++a) grid_[a] = grid[a];
  batch_ = batch;

  // capacities and grids, in creation order (inputs of a rule come before its outputs)
  // output_bound is what one frame may hold (the reference runs one frame per call): a
  // batch of frames gets that much room per frame
  auto batch_cap = [&](uint32_t per_frame) {
    const unsigned long long v = (unsigned long long)(per_frame ? per_frame : 200000u) * batch;
    return (uint32_t)std::min(v, 0x7fffffffull);
  };
  for (auto& cs : coordsets)
    if (cs.external) {
      for (int a = 0; a < 3; ++a) cs.grid[a] = grid[a];
      cs.cap = batch_cap(cs.bound);
    }
  for (auto& R : rules) {
    if (R.subm || R.inverse_of >= 0) continue;
    CoordSet& in = coordsets[R.in_cs];
    CoordSet& out = coordsets[R.out_cs];
    unsigned long long cells = batch;
    for (int a = 0; a < 3; ++a) {
      out.grid[a] = spconvb_out_extent(in.grid[a], R.ksize[a], R.stride[a], R.pad[a], R.dil[a]);
      if (out.grid[a] < 1) {
        log_msg(LOG_ERROR, "strided conv produces an empty grid");
        return SPCONVB_E_ARG;
      }
      cells *= out.grid[a];
    }
    unsigned long long cap = batch_cap(out.bound);
    unsigned long long reach = (unsigned long long)in.cap * R.kvol;
    out.cap = (uint32_t)std::min(std::min(cap, cells), reach);
    R.ws_bytes = spconvb_down_workspace_bytes(out.grid, batch);
    if (R.ws_bytes == 0) return SPCONVB_E_RANGE;
  }

  // ---- the zeroed arena: status, counts, hash tables, bitmaps
  size_t zoff = 0;
  const size_t status_off = zoff; zoff += 256;
  const size_t counts_off = zoff; zoff += align256(sizeof(uint32_t) * 64 * coordsets.size());
  std::vector<size_t> table_off(coordsets.size(), 0), ws_off(rules.size(), 0);
  for (size_t c = 0; c < coordsets.size(); ++c) {
    CoordSet& cs = coordsets[c];
    if (!cs.need_table) continue;
    cs.slots = spconvb_hash_slots(cs.cap);
    table_off[c] = zoff;
    zoff += align256(sizeof(uint64_t) * (size_t)cs.slots);
  }
  for (size_t r = 0; r < rules.size(); ++r) {
    if (rules[r].subm || rules[r].inverse_of >= 0) continue;
    ws_off[r] = zoff;
    // only the bitmap (first third of the workspace) must be zero, but the
    // rest is small next to it and one memset is cheaper than two
    zoff += align256(rules[r].ws_bytes);
  }
  zero_bytes_ = zoff;
  int rc = dev_alloc(&zero_arena_, zero_bytes_);
  if (rc != SPCONVB_OK) return rc;
  cudaMemset(zero_arena_, 0, zero_bytes_);
  uint8_t* zb = (uint8_t*)zero_arena_;
  status = (uint32_t*)(zb + status_off);
  counts_ = (uint32_t*)(zb + counts_off);
  for (size_t c = 0; c < coordsets.size(); ++c) {
    CoordSet& cs = coordsets[c];
    cs.n_ptr = counts_ + 64 * c;
    cs.table = cs.need_table ? (uint64_t*)(zb + table_off[c]) : nullptr;
    if (!cs.external) {
      void* p = nullptr;
      if ((rc = dev_alloc(&p, sizeof(int32_t) * 4 * (size_t)cs.cap)) != SPCONVB_OK) return rc;
      cs.coords = (int32_t*)p;
    }
  }
  for (size_t r = 0; r < rules.size(); ++r) {
    Rule& R = rules[r];
    void* p = nullptr;
    if ((rc = dev_alloc(&p, sizeof(int32_t) * (size_t)R.kvol * coordsets[R.out_cs].cap)) != SPCONVB_OK)
      return rc;
    R.map = (int32_t*)p;
    R.ws = (R.subm || R.inverse_of >= 0) ? nullptr : (void*)(zb + ws_off[r]);
  }

  // ---- feature buffers, reused by liveness unless every tensor must stay readable
  struct Slot { size_t bytes; int free_after; void* ptr; };
  std::vector<Slot> slots;
  const bool keep = flags & SPCONVB_BUILD_KEEP_TENSORS;
  for (int r = 0; r < (int)rt.size(); ++r) {
    RTensor& t = rt[r];
    if (t.external || t.alias_of >= 0) continue;
    if (t.dense) {
      // the model writes the dense shape for one frame: the leading dimension is the batch
      if (!t.shape.empty()) t.shape[0] = batch;
      if (!t.phys_shape.empty()) t.phys_shape[0] = batch;
      size_t numel = 1;
      for (auto v : t.phys_shape) numel *= (size_t)v;
      t.bytes = numel * (t.kind == SPCONVB_I8 ? 1 : sizeof(uint16_t));
    } else {
      t.bytes = (size_t)coordsets[t.cs].cap * t.channels * (t.kind == SPCONVB_I8 ? 1 : 2);
    }
    int pick = -1;
    if (!keep && !t.is_output && !t.dense) {
      for (int s = 0; s < (int)slots.size(); ++s)
        if (slots[s].free_after < t.first_step && slots[s].bytes >= t.bytes &&
            (pick < 0 || slots[s].bytes < slots[pick].bytes))
          pick = s;
    }
    if (pick < 0) {
      Slot s;
      s.bytes = t.bytes;
      s.ptr = nullptr;
      if ((rc = dev_alloc(&s.ptr, s.bytes)) != SPCONVB_OK) return rc;
      slots.push_back(s);
      pick = (int)slots.size() - 1;
    }
    slots[pick].free_after = (keep || t.is_output || t.dense) ? (1 << 30) : t.last_step;
    t.data = slots[pick].ptr;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return SPCONVB_E_NOMEM;
  if (!(flags & SPCONVB_BUILD_SINGLE_STREAM) && !aux_) {
    bool ok = cudaStreamCreateWithFlags(&aux_, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&fork_ev_, cudaEventDisableTiming) == cudaSuccess;
    rule_ev_.assign(steps.size(), nullptr);
    for (size_t i = 0; ok && i < steps.size(); ++i)
      if (is_rulebook_step(steps[i]))
        ok = cudaEventCreateWithFlags(&rule_ev_[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) return SPCONVB_E_NOMEM;
  }
  prepared_ = true;
  return SPCONVB_OK;
}

int Engine::forward(const void* features, const int32_t* indices, uint32_t cap_rows,
                    uint32_t n_host, const uint32_t* n_dev, const int32_t grid[3], int batch,
                    cudaStream_t caller_stream, const Profile* prof) {
  if (input_rt_ < 0 || !features || !indices || !grid) return SPCONVB_E_ARG;
  cudaStream_t st = caller_stream;  // the stream run_step launches on; switched for rulebook steps
  int rc = prepare(grid, batch);
  if (rc != SPCONVB_OK) return rc;
  CoordSet& in = coordsets[rt[input_rt_].cs];
  if (n_dev == nullptr && n_host > in.cap) {
    log_msg(LOG_ERROR, "%u input rows exceed the model's bound of %u", n_host, in.cap);
    return SPCONVB_E_ARG;
  }
  last_launches = 0;
  cudaError_t ce = cudaMemsetAsync(zero_arena_, 0, zero_bytes_, st);
  if (ce != cudaSuccess) return (int)ce;
  const uint32_t in_cap = n_dev ? std::min(cap_rows, in.cap) : in.cap;
  // Every step reads the input's row count from the engine's own word: the host's value, or
  // the caller's device-side value clamped to the rows the caller's buffers (and the model's
  // bound) hold, so that no kernel can be led past them.
  uint32_t* in_n = counts_ + 64 * (size_t)rt[input_rt_].cs;
  if (n_dev) rc = launch_clamp_count(in_n, n_dev, in_cap, status, st);
  else rc = launch_set_count(in_n, n_host, st);
  if (rc != SPCONVB_OK) return rc;
  ++last_launches;
  rt[input_rt_].data = const_cast<void*>(features);
  last_in_n_ = in_n;
  last_in_cap_ = in_cap;

  auto cs_coords = [&](int c) { return coordsets[c].external ? indices : coordsets[c].coords; };
  auto cs_n = [&](int c) { return coordsets[c].external ? in_n : coordsets[c].n_ptr; };
  auto cs_cap = [&](int c) { return coordsets[c].external ? in_cap : coordsets[c].cap; };
  // rows a launch should cover: known exactly for the input when the host knows n
  auto cs_launch = [&](int c) {
    if (coordsets[c].external && !n_dev) return std::max(n_host, 1u);
    return cs_cap(c);
  };

  bool clear_dense = true;  // false while a dense step's output was zeroed ahead of time
  auto run_step = [&](const Step& s) -> int {
    int rc = SPCONVB_OK;
    switch (s.kind) {
      case Step::HASH: {
        const CoordSet& cs = coordsets[s.cs];
        rc = spconvb_hash_build(cs_coords(s.cs), cs_n(s.cs), cs_cap(s.cs), cs_launch(s.cs),
                                cs.grid, batch, cs.table, cs.slots, SPCONVB_FLAG_PREZEROED, status,
                                st);
        last_launches += 1;
        break;
      }
      case Step::SUBM_MAP: {
        const Rule& R = rules[s.rule];
        const CoordSet& cs = coordsets[R.in_cs];
        if (cs.external)
          rc = spconvb_subm_map(cs_coords(R.in_cs), cs_n(R.in_cs), coordsets[R.in_cs].cap,
                                cs_launch(R.in_cs), cs.grid, batch, R.ksize, R.dil, cs.table,
                                cs.slots, R.map, status, st);
        else
          rc = spconvb_subm_map_ranked(cs.coords, cs.n_ptr, cs.cap, cs.cap, cs.grid, batch, R.ksize,
                                       R.dil, rules[cs.made_by_rule].ws, R.map, status, st);
        last_launches += 1;
        break;
      }
      case Step::DOWN_MAP: {
        const Rule& R = rules[s.rule];
        const CoordSet& ci = coordsets[R.in_cs];
        CoordSet& co = coordsets[R.out_cs];
        if (ci.made_by_rule >= 0) {
          // rows made by a strided rulebook: the map is looked up by rank from the output side
          rc = spconvb_down_map_ranked(ci.coords, ci.n_ptr, ci.cap, ci.cap, ci.grid, batch, R.ksize,
                                       R.stride, R.pad, R.dil, rules[ci.made_by_rule].ws, R.ws,
                                       co.coords, co.n_ptr, co.cap, R.map, co.table, co.slots,
                                       SPCONVB_FLAG_PREZEROED, status, st);
          last_launches += 4 + (co.table ? 1 : 0);  // mark, scan, emit, gather (+ hash)
        } else {
          rc = spconvb_down_map(cs_coords(R.in_cs), cs_n(R.in_cs), cs_cap(R.in_cs),
                                cs_launch(R.in_cs), ci.grid, batch, R.ksize, R.stride, R.pad,
                                R.dil, ci.table, ci.slots, R.ws, co.coords, co.n_ptr, co.cap,
                                R.map, co.table, co.slots, SPCONVB_FLAG_PREZEROED, status, st);
          last_launches += 5 + (co.table ? 1 : 0);  // mark, scan, emit, map fill, scatter (+ hash)
        }
        break;
      }
      case Step::INV_MAP: {
        const Rule& R = rules[s.rule];
        const Rule& F = rules[R.inverse_of];
        rc = spconvb_inverse_map(cs_coords(R.out_cs), cs_n(R.out_cs), coordsets[R.out_cs].cap,
                                 cs_launch(R.out_cs), coordsets[R.out_cs].grid, batch, F.ksize,
                                 F.stride, F.pad, F.dil, F.ws, coordsets[F.out_cs].cap, R.map,
                                 status, st);
        last_launches += 1;
        break;
      }
      case Step::CONVERT:
        rc = spconvb_convert(rt[s.in0].data, rt[s.in0].kind, s.cin, rt[s.out].kind, s.cout, s.s,
                             cs_n(rt[s.in0].cs), cs_launch(rt[s.in0].cs), rt[s.out].data, st);
        last_launches += 1;
        break;
      case Step::CONV: {
        const Rule& R = rules[s.rule];
        const LayerWeights& w = weights[s.weights];
        spconvb_conv_params p = s.cp;
        p.res = s.in1 >= 0 ? rt[s.in1].data : nullptr;
        p.n_in_ptr = cs_n(R.in_cs);
        p.cap_in = cs_cap(R.in_cs);
        rc = spconvb_conv_forward(&p, rt[s.in0].data, R.map, coordsets[R.out_cs].cap,
                                  cs_n(R.out_cs), cs_launch(R.out_cs), w.plain, w.packed, w.scale,
                                  w.bias, rt[s.out].data, status, st);
        last_launches += 1;
        break;
      }
      case Step::ADD:
        rc = spconvb_add(rt[s.in0].data, rt[s.in0].kind, s.a_scale, rt[s.in1].data, rt[s.in1].kind,
                         s.b_scale, s.cout, cs_n(s.cs), cs_launch(s.cs), s.relu, rt[s.out].kind,
                         s.inv_out, rt[s.out].data, st);
        last_launches += 1;
        break;
      case Step::RELU:
        rc = spconvb_relu(rt[s.in0].data, rt[s.in0].kind, s.cout, cs_n(s.cs), cs_launch(s.cs),
                          rt[s.out].data, st);
        last_launches += 1;
        break;
      case Step::DENSE: {
        const CoordSet& cs = coordsets[s.cs];
        rc = scatter_dense_layout_launch(rt[s.in0].data, rt[s.in0].kind, s.a_scale,
                                         cs_coords(s.cs), cs_n(s.cs), cs_launch(s.cs), s.cout,
                                         batch, cs.grid, s.has_perm ? s.perm : nullptr, s.layout,
                                         rt[s.out].kind, s.inv_out, rt[s.out].data, clear_dense,
                                         st);
        last_launches += 2;  // the zero fill and the scatter
        break;
      }
    }
    return rc;
  };

  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  if (prof) {
    if (cudaEventCreate(&ev0) != cudaSuccess || cudaEventCreate(&ev1) != cudaSuccess)
      return SPCONVB_E_NOMEM;
  }
  // Fork: the rulebook steps go to the auxiliary stream in their original order; a feature
  // step waits for the last rulebook step that precedes it in the program, which covers its
  // rulebook, its coordinate set and its row count.  Nothing a rulebook step reads is written
  // by a feature step.  The caller's stream joins the auxiliary one before returning, so the
  // whole call remains one unit of work on that stream (and one capturable region).
  const bool fork = !prof && aux_ != nullptr;
  int last_rule = -1, waited = -1;
  if (fork) {
    if (cudaEventRecord(fork_ev_, caller_stream) != cudaSuccess ||
        cudaStreamWaitEvent(aux_, fork_ev_, 0) != cudaSuccess)
      return SPCONVB_E_DEVICE;
  }
  // Dense outputs are zeroed on the auxiliary stream right away (bandwidth the convolutions
  // leave unused) when a rulebook step precedes the dense step: its event, which the dense step
  // waits for, then also covers the zero fill.
  std::vector<char> precleared(steps.size(), 0);
  if (fork) {
    bool rule_seen = false;
    for (size_t si = 0; si < steps.size() && rc == SPCONVB_OK; ++si) {
      const Step& s = steps[si];
      if (is_rulebook_step(s)) rule_seen = true;
      if (s.kind != Step::DENSE || !rule_seen) continue;
      const CoordSet& cs = coordsets[s.cs];
      const size_t bytes = spconvb_dense_bytes(s.cout, batch, cs.grid, s.has_perm ? s.perm : nullptr,
                                               s.layout, rt[s.out].kind);
      if (bytes == 0) continue;
      if (cudaMemsetAsync(rt[s.out].data, 0, bytes, aux_) != cudaSuccess) rc = SPCONVB_E_DEVICE;
      else precleared[si] = 1;
    }
  }
  for (size_t si = 0; si < steps.size() && rc == SPCONVB_OK; ++si) {
    const Step& s = steps[si];
    clear_dense = !precleared[si];
    if (fork) {
      if (is_rulebook_step(s)) {
        st = aux_;
        rc = run_step(s);
        st = caller_stream;
        if (rc == SPCONVB_OK && cudaEventRecord(rule_ev_[si], aux_) != cudaSuccess)
          rc = SPCONVB_E_DEVICE;
        last_rule = (int)si;
      } else {
        if (last_rule > waited) {
          if (cudaStreamWaitEvent(caller_stream, rule_ev_[last_rule], 0) != cudaSuccess)
            rc = SPCONVB_E_DEVICE;
          waited = last_rule;
        }
        if (rc == SPCONVB_OK) rc = run_step(s);
      }
    } else if (!prof) {
      rc = run_step(s);
    } else {
      // Per-step device time: rulebook steps change state and run once; the
      // others overwrite their output and are repeated, each time behind an L2
      // flush, and averaged.
      const bool repeatable = s.kind == Step::CONV || s.kind == Step::ADD || s.kind == Step::RELU ||
                              s.kind == Step::DENSE || s.kind == Step::CONVERT;
      const int reps = repeatable && prof->reps > 0 ? prof->reps : 1;
      float total = 0.f;
      const int launches_before = last_launches;
      for (int r = 0; r < reps && rc == SPCONVB_OK; ++r) {
        if (prof->flush && prof->flush_bytes)
          cudaMemsetAsync(prof->flush, r & 0xff, prof->flush_bytes, st);
        cudaEventRecord(ev0, st);
        rc = run_step(s);
        cudaEventRecord(ev1, st);
        if (cudaEventSynchronize(ev1) != cudaSuccess) rc = SPCONVB_E_DEVICE;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev0, ev1);
        total += ms;
      }
      last_launches = launches_before + (last_launches - launches_before) / reps;
      if (prof->step_ms && (int)si < prof->max_steps) prof->step_ms[si] = total / reps;
    }
    if (rc != SPCONVB_OK) {
      log_msg(LOG_ERROR, "step '%s' failed: %s", s.name.c_str(), spconvb_error_string(rc));
      break;
    }
  }
  if (fork) {  // join, also after a failed step, so that the auxiliary stream never outlives the call
    if (cudaEventRecord(fork_ev_, aux_) != cudaSuccess ||
        cudaStreamWaitEvent(caller_stream, fork_ev_, 0) != cudaSuccess)
      rc = rc == SPCONVB_OK ? SPCONVB_E_DEVICE : rc;
  }
  if (prof) {
    cudaEventDestroy(ev0);
    cudaEventDestroy(ev1);
  }
  return rc;
}

}  // namespace spconvb

extern "C" {
void spconvb_set_log_level(int32_t level) { spconvb::g_log_level = level; }
void spconvb_set_log_callback(spconvb_log_fn fn) { spconvb::g_log_fn = fn; }
}
