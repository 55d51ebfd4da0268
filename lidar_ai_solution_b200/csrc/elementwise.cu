// HBM-bound helpers around the convolutions: Add / Add&ReLU / ReLU, precision
// and channel-padding conversion, and the sparse -> dense BEV scatter.
#include "common.cuh"

namespace spconvb {

__device__ __forceinline__ float load_deq(const void* p, int kind, float scale, size_t i) {
  if (kind == SPCONVB_I8) return __fmul_rn((float)((const int8_t*)p)[i], scale);
  return __half2float(((const __half*)p)[i]);
}

__device__ __forceinline__ void store_q(void* p, int kind, float inv_scale, size_t i, float y) {
  if (kind == SPCONVB_I8)
    ((int8_t*)p)[i] = (int8_t)sat8(__fmul_rn(y, inv_scale));
  else
    ((__half*)p)[i] = __float2half_rn(y);
}

// 16 consecutive elements per thread, 16-byte loads and stores.
template <int AK, int BK, int OK>
__global__ void add_vec_kernel(const void* __restrict__ a, float a_scale,
                               const void* __restrict__ b, float b_scale, int channels,
                               const uint32_t* n_ptr, uint32_t cap, int relu,
                               float inv_out_scale, void* __restrict__ out) {
  const size_t groups = (size_t)min(*n_ptr, cap) * channels / 16;
  for (size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < groups;
       gidx += (size_t)gridDim.x * blockDim.x) {
    float x[16], y[16];
    if (AK == SPCONVB_I8) {
      uint4 q = ((const uint4*)a)[gidx];
      const int8_t* s = (const int8_t*)&q;
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] = __fmul_rn((float)s[i], a_scale);
    } else {
      uint4 q0 = ((const uint4*)a)[2 * gidx], q1 = ((const uint4*)a)[2 * gidx + 1];
      const __half* h0 = (const __half*)&q0;
      const __half* h1 = (const __half*)&q1;
#pragma unroll
      for (int i = 0; i < 8; ++i) { x[i] = __half2float(h0[i]); x[8 + i] = __half2float(h1[i]); }
    }
    if (BK == SPCONVB_I8) {
      uint4 q = ((const uint4*)b)[gidx];
      const int8_t* s = (const int8_t*)&q;
#pragma unroll
      for (int i = 0; i < 16; ++i) y[i] = __fmul_rn((float)s[i], b_scale);
    } else {
      uint4 q0 = ((const uint4*)b)[2 * gidx], q1 = ((const uint4*)b)[2 * gidx + 1];
      const __half* h0 = (const __half*)&q0;
      const __half* h1 = (const __half*)&q1;
#pragma unroll
      for (int i = 0; i < 8; ++i) { y[i] = __half2float(h0[i]); y[8 + i] = __half2float(h1[i]); }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      x[i] = __fadd_rn(x[i], y[i]);
      if (relu) x[i] = fmaxf(x[i], 0.f);
    }
    if (OK == SPCONVB_I8) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w[i] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          w[i] |= (uint32_t)(uint8_t)(int8_t)sat8(__fmul_rn(x[4 * i + j], inv_out_scale))
                  << (8 * j);
      }
      ((uint4*)out)[gidx] = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
        w[i] = *(uint32_t*)&h;
      }
      ((uint4*)out)[2 * gidx] = make_uint4(w[0], w[1], w[2], w[3]);
      ((uint4*)out)[2 * gidx + 1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

__global__ void add_scalar_kernel(const void* a, int a_kind, float a_scale, const void* b,
                                  int b_kind, float b_scale, int channels, const uint32_t* n_ptr,
                                  uint32_t cap, int relu, int out_kind, float inv_out_scale,
                                  void* out) {
  const size_t total = (size_t)min(*n_ptr, cap) * channels;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    float y = __fadd_rn(load_deq(a, a_kind, a_scale, i), load_deq(b, b_kind, b_scale, i));
    if (relu) y = fmaxf(y, 0.f);
    store_q(out, out_kind, inv_out_scale, i, y);
  }
}

__global__ void relu_kernel(const void* x, int kind, int channels, const uint32_t* n_ptr,
                            uint32_t cap, void* out) {
  const size_t total = (size_t)min(*n_ptr, cap) * channels;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    if (kind == SPCONVB_I8) {
      int8_t v = ((const int8_t*)x)[i];
      ((int8_t*)out)[i] = v > 0 ? v : (int8_t)0;
    } else {
      uint16_t v = ((const uint16_t*)x)[i];
      // negative non-NaN values (including -0) become +0
      ((uint16_t*)out)[i] = ((v & 0x8000u) && ((v & 0x7fffu) <= 0x7c00u)) ? (uint16_t)0 : v;
    }
  }
}

// max |x| over the first *n_ptr rows, folded into *out with an integer atomicMax (the bit
// patterns of non-negative floats order like the values).  NaN elements are skipped.
__global__ void absmax_kernel(const void* x, int kind, int channels, const uint32_t* n_ptr,
                              uint32_t cap, float* out) {
  const size_t total = (size_t)min(*n_ptr, cap) * channels;
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const float v = kind == SPCONVB_I8 ? fabsf((float)((const int8_t*)x)[i])
                                       : fabsf(__half2float(((const __half*)x)[i]));
    if (v == v) m = fmaxf(m, v);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax((int*)out, __float_as_int(m));
}

__global__ void convert_kernel(const void* x, int in_kind, int cin, int out_kind, int cout,
                               float s, const uint32_t* n_ptr, uint32_t cap, void* out) {
  const size_t total = (size_t)min(*n_ptr, cap) * cout;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / cout;
    const int c = (int)(i % cout);
    if (c >= cin) {
      if (out_kind == SPCONVB_I8) ((int8_t*)out)[i] = 0;
      else ((uint16_t*)out)[i] = 0;
      continue;
    }
    const size_t j = row * cin + c;
    if (in_kind == out_kind) {
      if (out_kind == SPCONVB_I8) ((int8_t*)out)[i] = ((const int8_t*)x)[j];
      else ((uint16_t*)out)[i] = ((const uint16_t*)x)[j];
    } else if (out_kind == SPCONVB_I8) {
      ((int8_t*)out)[i] = (int8_t)sat8(__fmul_rn(__half2float(((const __half*)x)[j]), s));
    } else {
      ((__half*)out)[i] = __float2half_rn(__fmul_rn((float)((const int8_t*)x)[j], s));
    }
  }
}

// fp16 rows padded to 8 channels (the first layer of a lidar backbone: 4 or 5 point features in
// 16-byte rows): one thread per row, one 16-byte store.
__global__ void pad8_f16_kernel(const __half* __restrict__ x, int cin, const uint32_t* n_ptr,
                                uint32_t cap, uint4* __restrict__ out) {
  const uint32_t n = min(*n_ptr, cap);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x) {
    const __half* src = x + (size_t)row * cin;
    uint16_t h[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) h[c] = c < cin ? __half_as_ushort(__ldg(src + c)) : (uint16_t)0;
    out[row] = make_uint4(h[0] | (uint32_t)h[1] << 16, h[2] | (uint32_t)h[3] << 16,
                          h[4] | (uint32_t)h[5] << 16, h[6] | (uint32_t)h[7] << 16);
  }
}

// 32 rows per block: rows are read coalesced into shared memory, then written
// channel by channel so that neighbouring rows (neighbouring cells when the
// rows are in canonical order) share write sectors.
__global__ void scatter_dense_kernel(const void* __restrict__ feat, int in_kind, float in_scale,
                                     const int4* __restrict__ coords, const uint32_t* n_ptr,
                                     uint32_t cap, int channels, Grid3 g, int p0, int p1, int p2,
                                     __half* __restrict__ out) {
  extern __shared__ __half tile[];  // [channels][33]
  __shared__ long long s_cell[32];
  const uint32_t n = min(*n_ptr, cap);
  const int gp[3] = {g.g[p0], g.g[p1], g.g[p2]};
  const size_t vol = (size_t)gp[0] * gp[1] * gp[2];
  for (uint32_t row0 = blockIdx.x * 32; row0 < n; row0 += gridDim.x * 32) {
    __syncthreads();
    if (threadIdx.x < 32) {
      long long cell = -1;
      uint32_t row = row0 + threadIdx.x;
      if (row < n) {
        int4 c = coords[row];
        const int sp[3] = {c.y, c.z, c.w};
        const int s0 = sp[p0], s1 = sp[p1], s2 = sp[p2];
        if ((unsigned)c.x < (unsigned)g.batch && (unsigned)s0 < (unsigned)gp[0] &&
            (unsigned)s1 < (unsigned)gp[1] && (unsigned)s2 < (unsigned)gp[2])
          cell = (long long)c.x * channels * (long long)vol + ((long long)s0 * gp[1] + s1) * gp[2] + s2;
      }
      s_cell[threadIdx.x] = cell;
    }
    for (int i = threadIdx.x; i < 32 * channels; i += blockDim.x) {
      const int r = i / channels, ch = i % channels;
      const uint32_t row = row0 + r;
      __half v = __float2half(0.f);
      if (row < n) {
        const size_t j = (size_t)row * channels + ch;
        v = in_kind == SPCONVB_I8
                ? __float2half_rn(__fmul_rn((float)((const int8_t*)feat)[j], in_scale))
                : ((const __half*)feat)[j];
      }
      tile[ch * 33 + r] = v;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * channels; i += blockDim.x) {
      const int ch = i >> 5, r = i & 31;
      const long long cell = s_cell[r];
      if (cell >= 0) out[cell + (long long)ch * (long long)vol] = tile[ch * 33 + r];
    }
  }
}

// ScatterDense into the vectorised layouts and/or int8.  One thread per (row, channel): reads
// are coalesced along the row, writes land in the 32-channel (NCHW32) or C-channel (NHWzC)
// group of the voxel's cell.  With m = channel * g(p0) + s0 the channel of the [N, C*D, H, W]
// view:  NCHW   out[b][m][s1][s2]
//        NCHW32 out[b][m / 32][s1][s2][m % 32]      (channel count padded up to 32)
//        NHWzC  out[b][s1][s2][s0][channel]
template <typename OutT>
__global__ void scatter_dense_layout_kernel(const void* __restrict__ feat, int in_kind,
                                            float in_scale, const int4* __restrict__ coords,
                                            const uint32_t* n_ptr, uint32_t cap, int channels,
                                            Grid3 g, int p0, int p1, int p2, int layout,
                                            float inv_out, int copy_bytes,
                                            OutT* __restrict__ out) {
  const size_t total = (size_t)min(*n_ptr, cap) * channels;
  const int g0 = g.g[p0], g1 = g.g[p1], g2 = g.g[p2];
  const long long plane = (long long)g1 * g2;
  const long long merged = (long long)channels * g0;
  const long long blocks32 = (merged + 31) / 32;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / channels;
    const int ch = (int)(i % channels);
    const int4 c = coords[row];
    const int sp[3] = {c.y, c.z, c.w};
    const int s0 = sp[p0], s1 = sp[p1], s2 = sp[p2];
    if ((unsigned)c.x >= (unsigned)g.batch || (unsigned)s0 >= (unsigned)g0 ||
        (unsigned)s1 >= (unsigned)g1 || (unsigned)s2 >= (unsigned)g2)
      continue;
    const long long m = (long long)ch * g0 + s0;
    long long dst;
    if (layout == 2)
      dst = (((long long)c.x * blocks32 + m / 32) * plane + (long long)s1 * g2 + s2) * 32 + m % 32;
    else if (layout == 3)
      dst = ((((long long)c.x * g1 + s1) * g2 + s2) * g0 + s0) * channels + ch;
    else
      dst = ((long long)c.x * merged + m) * plane + (long long)s1 * g2 + s2;
    if (sizeof(OutT) == 1) {
      int8_t q;
      if (in_kind == SPCONVB_I8) {
        const int8_t v = ((const int8_t*)feat)[i];
        q = copy_bytes ? v : (int8_t)sat8(__fmul_rn(__fmul_rn((float)v, in_scale), inv_out));
      } else {
        q = (int8_t)sat8(__fmul_rn(__half2float(((const __half*)feat)[i]), inv_out));
      }
      ((int8_t*)out)[dst] = q;
    } else {
      ((__half*)out)[dst] =
          in_kind == SPCONVB_I8
              ? __float2half_rn(__fmul_rn((float)((const int8_t*)feat)[i], in_scale))
              : ((const __half*)feat)[i];
    }
  }
}

static inline uint32_t clamp_u32(size_t v) { return v > 0xffffffffull ? 0xffffffffu : (uint32_t)v; }

// the two dense launchers with the zero fill optional (declared for the engine in engine.hpp)
int scatter_dense_launch(const void* feat, int32_t in_kind, float in_scale, const int32_t* coords,
                         const uint32_t* n_ptr, uint32_t launch_rows, int32_t channels,
                         int32_t batch, const int32_t grid[3], const int32_t perm[3], void* out,
                         bool clear, void* stream);
int scatter_dense_layout_launch(const void* feat, int32_t in_kind, float in_scale,
                                const int32_t* coords, const uint32_t* n_ptr, uint32_t launch_rows,
                                int32_t channels, int32_t batch, const int32_t grid[3],
                                const int32_t perm[3], int32_t layout, int32_t out_kind,
                                float inv_out_scale, void* out, bool clear, void* stream);

}  // namespace spconvb

using namespace spconvb;

extern "C" {

int spconvb_add(const void* a, int32_t a_kind, float a_scale, const void* b, int32_t b_kind,
                float b_scale, int32_t channels, const uint32_t* n_ptr, uint32_t launch_rows,
                int32_t relu, int32_t out_kind, float inv_out_scale, void* out, void* stream) {
  if (!a || !b || !out || !n_ptr || channels < 1 || launch_rows < 1) return SPCONVB_E_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const bool aligned = !(((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15u);
  if (channels % 16 == 0 && aligned) {
    const uint32_t groups = (uint32_t)((size_t)launch_rows * channels / 16);
    const int blocks = blocks_for(groups, 256);
#define SPCONVB_ADD_CASE(AK, BK, OK)                                                        \
  if (a_kind == AK && b_kind == BK && out_kind == OK) {                                     \
    add_vec_kernel<AK, BK, OK><<<blocks, 256, 0, st>>>(                                     \
        a, a_scale, b, b_scale, channels, n_ptr, launch_rows, relu, inv_out_scale, out);    \
    SPCONVB_LAUNCH_CHECK();                                                                 \
    return SPCONVB_OK;                                                                      \
  }
    SPCONVB_ADD_CASE(0, 0, 0) SPCONVB_ADD_CASE(0, 0, 1) SPCONVB_ADD_CASE(0, 1, 0)
    SPCONVB_ADD_CASE(0, 1, 1) SPCONVB_ADD_CASE(1, 0, 0) SPCONVB_ADD_CASE(1, 0, 1)
    SPCONVB_ADD_CASE(1, 1, 0) SPCONVB_ADD_CASE(1, 1, 1)
#undef SPCONVB_ADD_CASE
    return SPCONVB_E_ARG;
  }
  const uint32_t work = clamp_u32((size_t)launch_rows * channels);
  add_scalar_kernel<<<blocks_for(work, 256), 256, 0, st>>>(a, a_kind, a_scale, b, b_kind, b_scale,
                                                           channels, n_ptr, launch_rows, relu,
                                                           out_kind, inv_out_scale, out);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_relu(const void* x, int32_t kind, int32_t channels, const uint32_t* n_ptr,
                 uint32_t launch_rows, void* out, void* stream) {
  if (!x || !out || !n_ptr || channels < 1 || launch_rows < 1) return SPCONVB_E_ARG;
  const uint32_t work = clamp_u32((size_t)launch_rows * channels);
  relu_kernel<<<blocks_for(work, 256), 256, 0, (cudaStream_t)stream>>>(x, kind, channels, n_ptr,
                                                                       launch_rows, out);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_absmax(const void* x, int32_t kind, int32_t channels, const uint32_t* n_ptr,
                   uint32_t launch_rows, float* out, void* stream) {
  if (!x || !out || !n_ptr || channels < 1 || launch_rows < 1) return SPCONVB_E_ARG;
  const uint32_t work = clamp_u32((size_t)launch_rows * channels);
  absmax_kernel<<<blocks_for(work, 256), 256, 0, (cudaStream_t)stream>>>(x, kind, channels, n_ptr,
                                                                         launch_rows, out);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_convert(const void* x, int32_t in_kind, int32_t cin, int32_t out_kind,
                    int32_t cout_pad, float scale_or_inv, const uint32_t* n_ptr,
                    uint32_t launch_rows, void* out, void* stream) {
  if (!x || !out || !n_ptr || cin < 1 || cout_pad < cin || launch_rows < 1) return SPCONVB_E_ARG;
  if (in_kind == SPCONVB_F16 && out_kind == SPCONVB_F16 && cout_pad == 8 &&
      !((uintptr_t)out & 15u)) {
    pad8_f16_kernel<<<blocks_for(launch_rows, 128), 128, 0, (cudaStream_t)stream>>>(
        (const __half*)x, cin, n_ptr, launch_rows, (uint4*)out);
    SPCONVB_LAUNCH_CHECK();
    return SPCONVB_OK;
  }
  const uint32_t work = clamp_u32((size_t)launch_rows * cout_pad);
  convert_kernel<<<blocks_for(work, 256), 256, 0, (cudaStream_t)stream>>>(
      x, in_kind, cin, out_kind, cout_pad, scale_or_inv, n_ptr, launch_rows, out);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_scatter_dense(const void* feat, int32_t in_kind, float in_scale,
                          const int32_t* coords, const uint32_t* n_ptr, uint32_t launch_rows,
                          int32_t channels, int32_t batch, const int32_t grid[3],
                          const int32_t perm[3], void* out, void* stream) {
  return spconvb::scatter_dense_launch(feat, in_kind, in_scale, coords, n_ptr, launch_rows,
                                       channels, batch, grid, perm, out, true, stream);
}

extern "C++" int spconvb::scatter_dense_launch(const void* feat, int32_t in_kind, float in_scale,
                                  const int32_t* coords, const uint32_t* n_ptr,
                                  uint32_t launch_rows, int32_t channels, int32_t batch,
                                  const int32_t grid[3], const int32_t perm[3], void* out,
                                  bool clear, void* stream) {
  if (!feat || !coords || !n_ptr || !grid || !out || channels < 1 || channels > 1024 ||
      batch < 1 || launch_rows < 1)
    return SPCONVB_E_ARG;
  int p[3] = {0, 1, 2};
  if (perm) {
    p[0] = perm[0]; p[1] = perm[1]; p[2] = perm[2];
    if ((1 << p[0] | 1 << p[1] | 1 << p[2]) != 7) return SPCONVB_E_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t tile_bytes = sizeof(__half) * 33 * (size_t)channels;
  if (tile_bytes > 48 * 1024) {
    // wider rows than the default shared-memory window: raise the kernel's limit (once per
    // device; channels <= 1024 needs 66 KB)
    static bool raised[64] = {};
    int dev = 0;
    SPCONVB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !raised[dev]) {
      SPCONVB_CUDA_TRY(cudaFuncSetAttribute(scatter_dense_kernel,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)(sizeof(__half) * 33 * 1024)));
      if (dev >= 0 && dev < 64) raised[dev] = true;
    }
  }
  Grid3 g;
  g.g[0] = grid[0]; g.g[1] = grid[1]; g.g[2] = grid[2];
  g.batch = batch;
  const size_t bytes = sizeof(__half) * (size_t)batch * channels * grid[0] * grid[1] * grid[2];
  if (clear) SPCONVB_CUDA_TRY(cudaMemsetAsync(out, 0, bytes, st));
  size_t want_blocks = ((size_t)launch_rows + 31) / 32;
  if (want_blocks > (size_t)kSmCount * 16) want_blocks = (size_t)kSmCount * 16;
  const int blocks = (int)want_blocks;
  scatter_dense_kernel<<<blocks, 256, sizeof(__half) * 33 * channels, st>>>(
      feat, in_kind, in_scale, (const int4*)coords, n_ptr, launch_rows, channels, g, p[0], p[1],
      p[2], (__half*)out);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_scatter_dense_layout(const void* feat, int32_t in_kind, float in_scale,
                                 const int32_t* coords, const uint32_t* n_ptr,
                                 uint32_t launch_rows, int32_t channels, int32_t batch,
                                 const int32_t grid[3], const int32_t perm[3], int32_t layout,
                                 int32_t out_kind, float inv_out_scale, void* out, void* stream) {
  return spconvb::scatter_dense_layout_launch(feat, in_kind, in_scale, coords, n_ptr, launch_rows,
                                              channels, batch, grid, perm, layout, out_kind,
                                              inv_out_scale, out, true, stream);
}

extern "C++" int spconvb::scatter_dense_layout_launch(const void* feat, int32_t in_kind, float in_scale,
                                         const int32_t* coords, const uint32_t* n_ptr,
                                         uint32_t launch_rows, int32_t channels, int32_t batch,
                                         const int32_t grid[3], const int32_t perm[3],
                                         int32_t layout, int32_t out_kind, float inv_out_scale,
                                         void* out, bool clear, void* stream) {
  if (layout == 0) layout = 1;
  if (layout == 1 && out_kind == SPCONVB_F16)
    return scatter_dense_launch(feat, in_kind, in_scale, coords, n_ptr, launch_rows, channels,
                                batch, grid, perm, out, clear, stream);
  if (!feat || !coords || !n_ptr || !grid || !out || channels < 1 || channels > 1024 ||
      batch < 1 || launch_rows < 1 || layout < 1 || layout > 3 ||
      (out_kind != SPCONVB_F16 && out_kind != SPCONVB_I8) ||
      (in_kind != SPCONVB_F16 && in_kind != SPCONVB_I8))
    return SPCONVB_E_ARG;
  if (out_kind == SPCONVB_I8 && !(inv_out_scale > 0.f)) return SPCONVB_E_ARG;
  int p[3] = {0, 1, 2};
  if (perm) {
    p[0] = perm[0]; p[1] = perm[1]; p[2] = perm[2];
    if ((1 << p[0] | 1 << p[1] | 1 << p[2]) != 7) return SPCONVB_E_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  Grid3 g;
  g.g[0] = grid[0]; g.g[1] = grid[1]; g.g[2] = grid[2];
  g.batch = batch;
  const size_t bytes = spconvb_dense_bytes(channels, batch, grid, perm, layout, out_kind);
  if (clear) SPCONVB_CUDA_TRY(cudaMemsetAsync(out, 0, bytes, st));
  // int8 rows stored with the scale the dense tensor is asked in are copied byte for byte
  const int copy_bytes = in_kind == SPCONVB_I8 && out_kind == SPCONVB_I8 &&
                         fabsf(in_scale * inv_out_scale - 1.f) < 1e-6f;
  const uint32_t work = clamp_u32((size_t)launch_rows * channels);
  const int blocks = blocks_for(work, 256);
  if (out_kind == SPCONVB_I8)
    scatter_dense_layout_kernel<int8_t><<<blocks, 256, 0, st>>>(
        feat, in_kind, in_scale, (const int4*)coords, n_ptr, launch_rows, channels, g, p[0], p[1],
        p[2], layout, inv_out_scale, copy_bytes, (int8_t*)out);
  else
    scatter_dense_layout_kernel<__half><<<blocks, 256, 0, st>>>(
        feat, in_kind, in_scale, (const int4*)coords, n_ptr, launch_rows, channels, g, p[0], p[1],
        p[2], layout, inv_out_scale, 0, (__half*)out);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

size_t spconvb_dense_bytes(int32_t channels, int32_t batch, const int32_t grid[3],
                           const int32_t perm[3], int32_t layout, int32_t out_kind) {
  if (!grid || channels < 1 || batch < 1) return 0;
  const int p0 = perm ? perm[0] : 0;
  if (p0 < 0 || p0 > 2) return 0;
  size_t merged = (size_t)channels * grid[p0];
  if (layout == 2) merged = (merged + 31) / 32 * 32;
  const size_t cells = (size_t)grid[0] * grid[1] * grid[2] / grid[p0];
  return (size_t)batch * merged * cells * (out_kind == SPCONVB_I8 ? 1 : 2);
}

}  // extern "C"
