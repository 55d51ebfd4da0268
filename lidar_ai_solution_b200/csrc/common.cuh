// Shared device helpers: voxel keys, the coordinate hash table, status bits,
// and the epilogue arithmetic that every convolution kernel applies.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "spconvb.h"

namespace spconvb {

#define SPCONVB_CUDA_TRY(expr)                 \
  do {                                         \
    cudaError_t e__ = (expr);                  \
    if (e__ != cudaSuccess) return (int)e__;   \
  } while (0)

#define SPCONVB_LAUNCH_CHECK()                 \
  do {                                         \
    cudaError_t e__ = cudaPeekAtLastError();   \
    if (e__ != cudaSuccess) return (int)e__;   \
  } while (0)

constexpr int kSmCount = 148;  // B200: grids are sized in multiples of this

inline int blocks_for(uint32_t rows, int threads, int max_waves = 8) {
  // enough blocks to cover `rows` once, capped at a few waves (kernels stride)
  long long b = ((long long)rows + threads - 1) / threads;
  long long cap = (long long)kSmCount * max_waves * (2048 / threads);
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

struct Grid3 {
  int32_t g[3];
  int32_t batch;
};

__host__ __device__ inline uint32_t voxel_key(int b, int c0, int c1, int c2, const Grid3& g) {
  return (((uint32_t)b * g.g[0] + c0) * g.g[1] + c1) * g.g[2] + c2;
}

__device__ __forceinline__ uint32_t hash32(uint32_t k) {  // murmur3 finaliser
  k ^= k >> 16;
  k *= 0x85ebca6bu;
  k ^= k >> 13;
  k *= 0xc2b2ae35u;
  k ^= k >> 16;
  return k;
}

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t bit, uint32_t detail) {
  if (status) {
    uint32_t old = atomicOr(status, bit);
    if (!(old & bit)) status[1] = detail;
  }
}

// slot = (key+1) << 32 | row ; 0 = empty.  The table is a sequence of blocks of 8 slots (one
// 64-byte line each): the 8 cells of an aligned run along the innermost axis hash to the same
// block and take the slot of their position in the run, so the three x-neighbours a 3-wide
// kernel asks for lie in one line (two when the run ends between them) instead of three
// random ones.  A collision moves on block by block, same position.  Probe count is bounded
// by the number of blocks.  `mask` = slots - 1, slots a power of two >= 8.
__device__ __forceinline__ uint32_t hash_first_slot(uint32_t key, uint32_t mask) {
  return ((hash32(key >> 3) & (mask >> 3)) << 3) | (key & 7u);
}

__device__ __forceinline__ int hash_insert(uint64_t* table, uint32_t mask, uint32_t key,
                                           uint32_t row, uint32_t* status) {
  const uint64_t packed = ((uint64_t)(key + 1u) << 32) | row;
  uint32_t s = hash_first_slot(key, mask);
  for (uint32_t probe = 0; probe <= (mask >> 3); ++probe) {
    unsigned long long old =
        atomicCAS((unsigned long long*)(table + s), 0ull, (unsigned long long)packed);
    if (old == 0ull) return 0;
    if ((uint32_t)(old >> 32) == key + 1u) {
      set_status(status, SPCONVB_ST_DUPLICATE, row);
      return 1;
    }
    s = (s + 8u) & mask;
  }
  set_status(status, SPCONVB_ST_HASH_FULL, row);
  return 2;
}

__device__ __forceinline__ int32_t hash_lookup(const uint64_t* __restrict__ table, uint32_t mask,
                                               uint32_t key) {
  uint32_t s = hash_first_slot(key, mask);
  for (uint32_t probe = 0; probe <= (mask >> 3); ++probe) {
    uint64_t v = __ldg((const unsigned long long*)(table + s));
    if (v == 0ull) return -1;
    if ((uint32_t)(v >> 32) == key + 1u) return (int32_t)(uint32_t)v;
    s = (s + 8u) & mask;
  }
  return -1;
}

// ---------------------------------------------------------------- epilogue
// One definition of the output arithmetic, used by the CUDA-core and the
// tensor-core kernels alike, so that both round exactly like the CPU oracle.

__device__ __forceinline__ int sat8(float v) {
  float r = rintf(v);  // round-half-even
  r = fminf(fmaxf(r, -128.f), 127.f);
  return (int)r;
}

struct Epilogue {
  int act;
  int out_kind;
  float inv_out_scale;
  int has_res;
  int res_kind;
  float res_scale;
  int mid_kind;
  float mid_inv_scale;
  float mid_scale;
  int res_relu;
};

__host__ inline Epilogue make_epilogue(const spconvb_conv_params& p) {
  Epilogue e;
  e.act = p.act;
  e.out_kind = p.out_kind;
  e.inv_out_scale = p.inv_out_scale;
  e.has_res = p.res != nullptr;
  e.res_kind = p.res_kind;
  e.res_scale = p.res_scale;
  e.mid_kind = p.mid_kind;
  e.mid_inv_scale = p.mid_inv_scale;
  e.mid_scale = p.mid_scale;
  e.res_relu = p.res_relu;
  return e;
}

// y = conv result after dequant + bias.  r = raw residual element (int8 value or
// fp16 bits widened), ignored without residual.  Returns the value to store:
// an int in [-128,127] for int8 outputs (as float), or the fp32 to round to fp16.
__device__ __forceinline__ float epilogue_value(float y, const Epilogue& e, float r_deq) {
  if (e.act == SPCONVB_ACT_RELU) y = fmaxf(y, 0.f);
  if (e.has_res) {
    float m;
    if (e.mid_kind == SPCONVB_I8)
      m = __fmul_rn((float)sat8(__fmul_rn(y, e.mid_inv_scale)), e.mid_scale);
    else
      m = __half2float(__float2half_rn(y));
    y = __fadd_rn(m, r_deq);
    if (e.res_relu) y = fmaxf(y, 0.f);
  }
  if (e.out_kind == SPCONVB_I8) return (float)sat8(__fmul_rn(y, e.inv_out_scale));
  return y;
}

}  // namespace spconvb
