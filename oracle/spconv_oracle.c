/*
 * CPU oracle for the sparse-convolution hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm that the closed libspconv
 * engine of NVIDIA-AI-IOT/Lidar_AI_Solution executes for a lidar backbone.
 * It exists to check the CUDA kernels; nothing in the shipped library links
 * or calls it.  Only the test-suite, the smoke check and the cpu_baseline leg
 * of the benchmark may load it.
 *
 * PARITY UNPINNED: the reference engine is a closed binary with no golden
 * output tensors available, so this restatement is pinned only by
 *   - a dense cross-correlation (torch conv3d) on small grids, and
 *   - per-stage voxel / pair counts of the reference's own input fixtures.
 *
 * What each function follows in the reference tree:
 *   rulebooks      operator attributes of EngineBuilder::push_sparse_conv
 *                  (libraries/3DSparseConvolution/libspconv/include/spconv/engine.hpp:135-156)
 *                  and the output-size rule the exporters use
 *                  (libraries/3DSparseConvolution/tool/centerpoint-export/exptool.py:79-81)
 *   conv numerics  int8 attributes written by
 *                  CUDA-CenterPoint/qat/onnx_export/exptool.py:141-231
 *                  (input_dynamic_range, weight_dynamic_ranges, precision,
 *                  output_precision); weight layout [Cout][K][Cin]
 *                  (libraries/3DSparseConvolution/tool/centerpoint-export/funcs.py:43-60)
 *   add / relu     EngineBuilder::push_add, push_relu (engine.hpp:100-112)
 *   scatter dense  EngineBuilder::push_dense (engine.hpp:114-123)
 *   voxelizer      CUDA-CenterPoint/src/preprocess_kernels.cu:26-173, executed
 *                  sequentially in point order
 *   canonical row order  libraries/3DSparseConvolution/tool/compare.py:62-69
 *
 * Conventions shared with the CUDA side
 *   coords   int32 [N][4] = (batch, c0, c1, c2); c0..c2 follow the grid order
 *            the caller passes (z,y,x for CenterPoint).
 *   map      int32 [KVOL][cap]  map[k*cap + o] = input row feeding output row o
 *            through kernel tap k, or -1.  Tap k = (k0*K1 + k1)*K2 + k2 and
 *            in = out*stride - pad + k*dilation   (cross-correlation).
 *   strided outputs are unique and sorted ascending by ((b*G0+c0)*G1+c1)*G2+c2.
 *   weights  [Cout][KVOL][Cin]
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 half_t;

static inline float h2f(uint16_t h) {
  half_t v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) {
  half_t v = (half_t)f; /* round-to-nearest-even */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
static inline int8_t sat8(float v) {
  float r = rintf(v); /* round-half-even in the default rounding mode */
  if (r > 127.f) r = 127.f;
  if (r < -128.f) r = -128.f;
  return (int8_t)r;
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the OpenMP team size of the calls that follow (launchers such as
 * torch.distributed.run export OMP_NUM_THREADS=1, which would otherwise make
 * the CPU baseline single-threaded).  Returns the size now in effect. */
int orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* sorted key table: the oracle's coordinate lookup (no hashing on purpose). */

typedef struct {
  int64_t key;
  int32_t row;
} keyrow_t;

static int cmp_keyrow(const void* a, const void* b) {
  const keyrow_t* x = (const keyrow_t*)a;
  const keyrow_t* y = (const keyrow_t*)b;
  if (x->key < y->key) return -1;
  if (x->key > y->key) return 1;
  return (x->row > y->row) - (x->row < y->row);
}

static inline int64_t lin_key(int b, int c0, int c1, int c2, const int* g) {
  return (((int64_t)b * g[0] + c0) * g[1] + c1) * g[2] + c2;
}

static int32_t find_row(const keyrow_t* t, int n, int64_t key) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    int mid = (lo + hi) >> 1;
    if (t[mid].key == key) return t[mid].row;
    if (t[mid].key < key)
      lo = mid + 1;
    else
      hi = mid - 1;
  }
  return -1;
}

static keyrow_t* build_table(const int32_t* coords, int n, const int* grid) {
  keyrow_t* t = (keyrow_t*)malloc(sizeof(keyrow_t) * (size_t)(n > 0 ? n : 1));
  for (int i = 0; i < n; ++i) {
    const int32_t* c = coords + 4 * (size_t)i;
    t[i].key = lin_key(c[0], c[1], c[2], c[3], grid);
    t[i].row = i;
  }
  qsort(t, (size_t)n, sizeof(keyrow_t), cmp_keyrow);
  return t;
}

/* Returns the number of duplicated coordinates (0 for a valid sparse tensor). */
int orc_count_duplicates(const int32_t* coords, int n, const int* grid) {
  keyrow_t* t = build_table(coords, n, grid);
  int dup = 0;
  for (int i = 1; i < n; ++i) dup += (t[i].key == t[i - 1].key);
  free(t);
  return dup;
}

/* Output extent of one axis: floor((in + 2p - d(k-1) - 1)/s) + 1. */
int orc_out_extent(int in, int k, int s, int p, int d) {
  int v = in + 2 * p - d * (k - 1) - 1;
  if (v < 0) return 0;
  return v / s + 1;
}

/* Submanifold rulebook: outputs are the inputs; pad = dil*(k/2). */
int64_t orc_subm_map(const int32_t* coords, int n, const int* grid, const int* ksize,
                     const int* dil, int32_t* map, int cap) {
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  keyrow_t* t = build_table(coords, n, grid);
  int64_t pairs = 0;
#pragma omp parallel for reduction(+ : pairs) schedule(static)
  for (int o = 0; o < n; ++o) {
    const int32_t* c = coords + 4 * (size_t)o;
    for (int k = 0; k < kvol; ++k) {
      int k2 = k % ksize[2], k1 = (k / ksize[2]) % ksize[1], k0 = k / (ksize[2] * ksize[1]);
      int p0 = c[1] + (k0 - ksize[0] / 2) * dil[0];
      int p1 = c[2] + (k1 - ksize[1] / 2) * dil[1];
      int p2 = c[3] + (k2 - ksize[2] / 2) * dil[2];
      int32_t r = -1;
      if (p0 >= 0 && p0 < grid[0] && p1 >= 0 && p1 < grid[1] && p2 >= 0 && p2 < grid[2])
        r = find_row(t, n, lin_key(c[0], p0, p1, p2, grid));
      map[(size_t)k * cap + o] = r;
      pairs += (r >= 0);
    }
  }
  free(t);
  return pairs;
}

static int cmp_i64(const void* a, const void* b) {
  int64_t x = *(const int64_t*)a, y = *(const int64_t*)b;
  return (x > y) - (x < y);
}

/* Strided (regular) sparse conv rulebook.  Writes sorted unique output
 * coordinates and the output-stationary map.  Returns the pair count; the
 * number of outputs is stored in *n_out (not clipped; rows beyond cap are not
 * written). */
int64_t orc_down_map(const int32_t* coords, int n, const int* grid, const int* ksize,
                     const int* stride, const int* pad, const int* dil, int32_t* out_coords,
                     int32_t* map, int cap, int* n_out, int* out_grid) {
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  int og[3];
  for (int a = 0; a < 3; ++a) og[a] = orc_out_extent(grid[a], ksize[a], stride[a], pad[a], dil[a]);
  if (out_grid) memcpy(out_grid, og, sizeof(og));

  int64_t* cand = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1) * kvol);
  size_t nc = 0;
  for (int i = 0; i < n; ++i) {
    const int32_t* c = coords + 4 * (size_t)i;
    for (int k = 0; k < kvol; ++k) {
      int kk[3] = {k / (ksize[2] * ksize[1]), (k / ksize[2]) % ksize[1], k % ksize[2]};
      int o[3];
      int ok = 1;
      for (int a = 0; a < 3; ++a) {
        int v = c[1 + a] + pad[a] - kk[a] * dil[a];
        if (v < 0 || v % stride[a] != 0) { ok = 0; break; }
        o[a] = v / stride[a];
        if (o[a] >= og[a]) { ok = 0; break; }
      }
      if (ok) cand[nc++] = lin_key(c[0], o[0], o[1], o[2], og);
    }
  }
  qsort(cand, nc, sizeof(int64_t), cmp_i64);
  size_t nu = 0;
  for (size_t i = 0; i < nc; ++i)
    if (i == 0 || cand[i] != cand[i - 1]) cand[nu++] = cand[i];
  *n_out = (int)nu;
  int m = (int)nu < cap ? (int)nu : cap;

  keyrow_t* t = build_table(coords, n, grid);
  int64_t pairs = 0;
#pragma omp parallel for reduction(+ : pairs) schedule(static)
  for (int o = 0; o < m; ++o) {
    int64_t key = cand[o];
    int c2 = (int)(key % og[2]); key /= og[2];
    int c1 = (int)(key % og[1]); key /= og[1];
    int c0 = (int)(key % og[0]); key /= og[0];
    int b = (int)key;
    int32_t* oc = out_coords + 4 * (size_t)o;
    oc[0] = b; oc[1] = c0; oc[2] = c1; oc[3] = c2;
    for (int k = 0; k < kvol; ++k) {
      int k2 = k % ksize[2], k1 = (k / ksize[2]) % ksize[1], k0 = k / (ksize[2] * ksize[1]);
      int p0 = c0 * stride[0] - pad[0] + k0 * dil[0];
      int p1 = c1 * stride[1] - pad[1] + k1 * dil[1];
      int p2 = c2 * stride[2] - pad[2] + k2 * dil[2];
      int32_t r = -1;
      if (p0 >= 0 && p0 < grid[0] && p1 >= 0 && p1 < grid[1] && p2 >= 0 && p2 < grid[2])
        r = find_row(t, n, lin_key(b, p0, p1, p2, grid));
      map[(size_t)k * cap + o] = r;
      pairs += (r >= 0);
    }
  }
  free(t);
  free(cand);
  return pairs;
}

/* ------------------------------------------------------------------------ */
/* convolutions                                                             */

enum { ORC_ACT_NONE = 0, ORC_ACT_RELU = 1 };
enum { ORC_OUT_F16 = 0, ORC_OUT_I8 = 1, ORC_OUT_F32 = 2 };

/* fp32 reference conv (BASELINE config 0). */
void orc_conv_f32(const float* in, const int32_t* map, int cap, int n_out, int kvol, int cin,
                  int cout, const float* w, const float* bias, int act, float* out) {
#pragma omp parallel for schedule(static)
  for (int o = 0; o < n_out; ++o) {
    float* y = out + (size_t)o * cout;
    for (int c = 0; c < cout; ++c) y[c] = bias ? bias[c] : 0.f;
    for (int k = 0; k < kvol; ++k) {
      int32_t r = map[(size_t)k * cap + o];
      if (r < 0) continue;
      const float* x = in + (size_t)r * cin;
      for (int c = 0; c < cout; ++c) {
        const float* wk = w + ((size_t)c * kvol + k) * cin;
        float a = 0.f;
        for (int i = 0; i < cin; ++i) a += wk[i] * x[i];
        y[c] += a;
      }
    }
    if (act == ORC_ACT_RELU)
      for (int c = 0; c < cout; ++c) y[c] = y[c] > 0.f ? y[c] : 0.f;
  }
}

/* Symmetric per-output-channel int8 weight quantisation:
 * q = clamp(rint(w * (127/amax_c)), -127, 127). */
void orc_quantize_weights(const float* w, int cout, int per_channel, const float* amax,
                          int8_t* q) {
  for (int c = 0; c < cout; ++c) {
    float inv = amax[c] > 0.f ? 127.0f / amax[c] : 0.f;
    for (int i = 0; i < per_channel; ++i) {
      float r = rintf(w[(size_t)c * per_channel + i] * inv);
      if (r > 127.f) r = 127.f;
      if (r < -127.f) r = -127.f;
      q[(size_t)c * per_channel + i] = (int8_t)r;
    }
  }
}

/* fp16 -> int8 activation quantisation with inv_scale = 127/dynamic_range. */
void orc_quantize_f16(const uint16_t* x, size_t n, float inv_scale, int8_t* q) {
  for (size_t i = 0; i < n; ++i) q[i] = sat8(h2f(x[i]) * inv_scale);
}

static inline void epilogue_store(float y, int act, int out_kind, float inv_out_scale, void* out,
                                  size_t idx) {
  if (act == ORC_ACT_RELU) y = y > 0.f ? y : 0.f;
  if (out_kind == ORC_OUT_I8)
    ((int8_t*)out)[idx] = sat8(y * inv_out_scale);
  else if (out_kind == ORC_OUT_F16)
    ((uint16_t*)out)[idx] = f2h(y);
  else
    ((float*)out)[idx] = y;
}

/* Int8 conv: acc = sum q_x*q_w (int32, exact); y = fma(acc, scale[c], bias[c]);
 * activation; store int8 (y*inv_out_scale, round-half-even, clamp) or fp16.
 * Optional fused residual (engine's Add&ReLU fused after a conv):
 *   the conv result is first stored at its own output precision
 *   (mid_kind / mid_inv_scale / mid_scale), then
 *   z = deq(mid) + deq(residual); z = relu(z) if res_relu; store as out_kind. */
void orc_conv_i8(const int8_t* in, const int32_t* map, int cap, int n_out, int kvol, int cin,
                 int cout, const int8_t* wq, const float* scale, const float* bias, int act,
                 int out_kind, float inv_out_scale, void* out) {
#pragma omp parallel for schedule(static)
  for (int o = 0; o < n_out; ++o) {
    int32_t acc[512];
    for (int c = 0; c < cout; ++c) acc[c] = 0;
    for (int k = 0; k < kvol; ++k) {
      int32_t r = map[(size_t)k * cap + o];
      if (r < 0) continue;
      const int8_t* x = in + (size_t)r * cin;
      for (int c = 0; c < cout; ++c) {
        const int8_t* wk = wq + ((size_t)c * kvol + k) * cin;
        int32_t a = 0;
        for (int i = 0; i < cin; ++i) a += (int32_t)wk[i] * (int32_t)x[i];
        acc[c] += a;
      }
    }
    for (int c = 0; c < cout; ++c) {
      float y = fmaf((float)acc[c], scale[c], bias ? bias[c] : 0.f);
      epilogue_store(y, act, out_kind, inv_out_scale, out, (size_t)o * cout + c);
    }
  }
}

/* fp16 conv: fp16 inputs and weights, fp32 accumulation, y = acc + bias. */
void orc_conv_f16(const uint16_t* in, const int32_t* map, int cap, int n_out, int kvol, int cin,
                  int cout, const uint16_t* w, const float* bias, int act, int out_kind,
                  float inv_out_scale, void* out) {
  float* wf = (float*)malloc(sizeof(float) * (size_t)cout * kvol * cin);
  for (size_t i = 0; i < (size_t)cout * kvol * cin; ++i) wf[i] = h2f(w[i]);
#pragma omp parallel for schedule(static)
  for (int o = 0; o < n_out; ++o) {
    float acc[512];
    float x[512];
    for (int c = 0; c < cout; ++c) acc[c] = 0.f;
    for (int k = 0; k < kvol; ++k) {
      int32_t r = map[(size_t)k * cap + o];
      if (r < 0) continue;
      for (int i = 0; i < cin; ++i) x[i] = h2f(in[(size_t)r * cin + i]);
      for (int c = 0; c < cout; ++c) {
        const float* wk = wf + ((size_t)c * kvol + k) * cin;
        float a = 0.f;
        for (int i = 0; i < cin; ++i) a += wk[i] * x[i];
        acc[c] += a;
      }
    }
    for (int c = 0; c < cout; ++c) {
      float y = acc[c] + (bias ? bias[c] : 0.f);
      epilogue_store(y, act, out_kind, inv_out_scale, out, (size_t)o * cout + c);
    }
  }
  free(wf);
}

/* Add (+ReLU).  kind: 0 fp16, 1 int8 (dequantised with the scale given). */
void orc_add(const void* a, int a_kind, float a_scale, const void* b, int b_kind, float b_scale,
             size_t numel, int relu, int out_kind, float inv_out_scale, void* out) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < numel; ++i) {
    float x = a_kind == ORC_OUT_I8 ? (float)((const int8_t*)a)[i] * a_scale
                                   : h2f(((const uint16_t*)a)[i]);
    float y = b_kind == ORC_OUT_I8 ? (float)((const int8_t*)b)[i] * b_scale
                                   : h2f(((const uint16_t*)b)[i]);
    epilogue_store(x + y, relu ? ORC_ACT_RELU : ORC_ACT_NONE, out_kind, inv_out_scale, out, i);
  }
}

/* ReLU on a stored tensor (scale unchanged). */
void orc_relu(const void* x, int kind, size_t numel, void* out) {
  for (size_t i = 0; i < numel; ++i) {
    if (kind == ORC_OUT_I8) {
      int8_t v = ((const int8_t*)x)[i];
      ((int8_t*)out)[i] = v > 0 ? v : 0;
    } else {
      uint16_t v = ((const uint16_t*)x)[i];
      ((uint16_t*)out)[i] = (v & 0x8000u) && ((v & 0x7fffu) <= 0x7c00u) ? 0 : v;
    }
  }
}

/* Sparse -> dense.  out is [B][C][G0][G1][G2] (layout 0, "NCHW" with the
 * spatial axes in the order of the coordinates), fp16.  in_kind int8 inputs
 * are dequantised with in_scale.  `perm` != NULL scatters to
 * [B][C][g(perm0)][g(perm1)][g(perm2)] instead (ScatterDense fused with a
 * Transpose of the three spatial axes). */
void orc_scatter_dense(const void* feat, int in_kind, float in_scale, const int32_t* coords,
                       int n, int channels, int batch, const int* grid, const int* perm,
                       uint16_t* out) {
  int p[3] = {0, 1, 2};
  if (perm) memcpy(p, perm, sizeof(p));
  int g[3] = {grid[p[0]], grid[p[1]], grid[p[2]]};
  size_t vol = (size_t)g[0] * g[1] * g[2];
  memset(out, 0, sizeof(uint16_t) * vol * channels * batch);
  for (int i = 0; i < n; ++i) {
    const int32_t* c = coords + 4 * (size_t)i;
    int s[3] = {c[1 + p[0]], c[1 + p[1]], c[1 + p[2]]};
    size_t cell = ((size_t)s[0] * g[1] + s[1]) * g[2] + s[2];
    for (int ch = 0; ch < channels; ++ch) {
      uint16_t v;
      if (in_kind == ORC_OUT_I8)
        v = f2h((float)((const int8_t*)feat)[(size_t)i * channels + ch] * in_scale);
      else
        v = ((const uint16_t*)feat)[(size_t)i * channels + ch];
      out[((size_t)c[0] * channels + ch) * vol + cell] = v;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* voxelizer: the reference kernels run one point at a time in point order.  */
/* A voxel's id is the order of first appearance; the first max_pts points of */
/* a voxel are kept and averaged in fp32 (sum in arrival order, then divide). */

/* points: fp32 [n][nfeat] (points_kind 0) or fp16 (points_kind 1).
 * range = {min_x,min_y,min_z,max_x,max_y,max_z}; vsize = {vx,vy,vz};
 * gridxyz = {gx,gy,gz}.  order 0 writes (0,z,y,x), order 1 writes (0,x,y,z).
 * Returns the voxel count (not clipped); at most max_voxels rows are written. */
int orc_voxelize(const void* points, int points_kind, int n, int nfeat, const float* range,
                 const float* vsize, const int* gridxyz, int max_voxels, int max_pts, int order,
                 uint16_t* feat_out, int32_t* coords_out) {
  typedef struct { uint32_t key; int id; } slot_t;
  size_t hs = 1;
  while (hs < (size_t)n * 2 + 16) hs <<= 1;
  slot_t* tab = (slot_t*)malloc(sizeof(slot_t) * hs);
  for (size_t i = 0; i < hs; ++i) tab[i].id = -1;
  float* sum = (float*)calloc((size_t)max_voxels * nfeat, sizeof(float));
  int* cnt = (int*)calloc((size_t)max_voxels, sizeof(int));
  int nv = 0;
  float p[16];
  for (int i = 0; i < n; ++i) {
    for (int f = 0; f < nfeat; ++f)
      p[f] = points_kind ? h2f(((const uint16_t*)points)[(size_t)i * nfeat + f])
                         : ((const float*)points)[(size_t)i * nfeat + f];
    if (p[0] < range[0] || p[0] >= range[3] || p[1] < range[1] || p[1] >= range[4] ||
        p[2] < range[2] || p[2] >= range[5])
      continue;
    int ivx = (int)floorf((p[0] - range[0]) / vsize[0]);
    int ivy = (int)floorf((p[1] - range[1]) / vsize[1]);
    int ivz = (int)floorf((p[2] - range[2]) / vsize[2]);
    /* a quotient that rounds up to the grid size is outside (the BEVFusion copy
     * of the kernel checks this, lidar-voxelization.cu:86-93) */
    if (ivx < 0 || ivx >= gridxyz[0] || ivy < 0 || ivy >= gridxyz[1] || ivz < 0 ||
        ivz >= gridxyz[2])
      continue;
    unsigned vx = (unsigned)ivx, vy = (unsigned)ivy, vz = (unsigned)ivz;
    uint32_t key = (vz * (uint32_t)gridxyz[1] + vy) * (uint32_t)gridxyz[0] + vx;
    uint64_t h = key;
    h ^= h >> 16; h *= 0x85ebca6bull; h ^= h >> 13; h *= 0xc2b2ae35ull; h ^= h >> 16;
    size_t s = (size_t)(h & (hs - 1));
    while (tab[s].id >= 0 && tab[s].key != key) s = (s + 1) & (hs - 1);
    if (tab[s].id < 0) {
      tab[s].key = key;
      tab[s].id = nv++;
      if (tab[s].id < max_voxels) {
        int32_t* c = coords_out + 4 * (size_t)tab[s].id;
        c[0] = 0;
        if (order == 0) { c[1] = (int)vz; c[2] = (int)vy; c[3] = (int)vx; }
        else            { c[1] = (int)vx; c[2] = (int)vy; c[3] = (int)vz; }
      }
    }
    int id = tab[s].id;
    if (id >= max_voxels) continue;
    if (cnt[id] < max_pts) {
      for (int f = 0; f < nfeat; ++f) sum[(size_t)id * nfeat + f] += p[f];
      cnt[id]++;
    }
  }
  int m = nv < max_voxels ? nv : max_voxels;
  for (int v = 0; v < m; ++v)
    for (int f = 0; f < nfeat; ++f)
      feat_out[(size_t)v * nfeat + f] = f2h(sum[(size_t)v * nfeat + f] / (float)cnt[v]);
  free(tab); free(sum); free(cnt);
  return nv;
}
