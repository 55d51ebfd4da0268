// Rulebook construction: coordinate hash table, submanifold neighbour map and
// strided-convolution map.  All HBM/L2-bound integer work; every kernel reads
// its row count from device memory and strides, so launches never depend on
// host knowledge of the counts.
//
// Strided outputs are made unique and ordered without sorting: each candidate
// output cell sets one bit in a bitmap over the output grid, an exclusive scan
// of the per-word popcounts ranks the set bits, and the rank is the output row.
#include <mutex>

#include "common.cuh"

namespace spconvb {

constexpr int kThreads = 256;
constexpr int kScanThreads = 1024;
constexpr int kScanWordsPerBlock = kScanThreads;  // one bitmap word per thread

// ------------------------------------------------------------------ hash build
__global__ void hash_build_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                  uint32_t cap, Grid3 g, uint64_t* table, uint32_t mask,
                                  uint32_t* status) {
  const uint32_t n = min(*n_ptr, cap);
  if (blockIdx.x == 0 && threadIdx.x == 0 && *n_ptr > cap)
    set_status(status, SPCONVB_ST_OVERFLOW, *n_ptr);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x) {
    int4 c = __ldg(coords + row);
    if ((unsigned)c.x >= (unsigned)g.batch || (unsigned)c.y >= (unsigned)g.g[0] ||
        (unsigned)c.z >= (unsigned)g.g[1] || (unsigned)c.w >= (unsigned)g.g[2]) {
      set_status(status, SPCONVB_ST_COORD_RANGE, row);
      continue;
    }
    hash_insert(table, mask, voxel_key(c.x, c.y, c.z, c.w, g), row, status);
  }
}

// ------------------------------------------------------------------- SubM map
struct Kernel3 {
  int32_t k[3];
  int32_t s[3];
  int32_t p[3];
  int32_t d[3];
  int32_t sh[3];  // log2 of the stride when it is a power of two (1, 2, 4, ...), else -1
};

// v % s == 0 and v / s for v >= 0, without the integer division when the stride is a power
// of two (every strided layer of the lidar backbones has stride 1 or 2).
__device__ __forceinline__ bool stride_divides(int v, int s, int sh) {
  return sh >= 0 ? (v & (s - 1)) == 0 : v % s == 0;
}
__device__ __forceinline__ int stride_quotient(int v, int s, int sh) {
  return sh >= 0 ? v >> sh : v / s;
}

// One thread per row: the row's coordinate is read once, its taps are walked in tap order
// (so a warp's stores of one tap land in one or two lines of map[k][.]), and the lookups of
// the 27 taps are independent loads the compiler overlaps when the kernel size is known at
// compile time (K333: the 3x3x3, dilation-1 case of every backbone layer).
template <bool K333, typename Lookup>
__device__ __forceinline__ void subm_row_taps(const int4 c, uint32_t row, const Grid3& g,
                                              const Kernel3& kr, uint32_t cap,
                                              int32_t* __restrict__ map, Lookup lookup) {
  const int K0 = K333 ? 3 : kr.k[0], K1 = K333 ? 3 : kr.k[1], K2 = K333 ? 3 : kr.k[2];
  const int D0 = K333 ? 1 : kr.d[0], D1 = K333 ? 1 : kr.d[1], D2 = K333 ? 1 : kr.d[2];
  const bool bok = (unsigned)c.x < (unsigned)g.batch;
  int32_t* dst = map + row;
#pragma unroll
  for (int k0 = 0; k0 < K0; ++k0) {
    const int p0 = c.y + (k0 - K0 / 2) * D0;
    const bool ok0 = bok && (unsigned)p0 < (unsigned)g.g[0];
#pragma unroll
    for (int k1 = 0; k1 < K1; ++k1) {
      const int p1 = c.z + (k1 - K1 / 2) * D1;
      const bool ok1 = ok0 && (unsigned)p1 < (unsigned)g.g[1];
#pragma unroll
      for (int k2 = 0; k2 < K2; ++k2) {
        const int p2 = c.w + (k2 - K2 / 2) * D2;
        int32_t r = -1;
        if (k0 == K0 / 2 && k1 == K1 / 2 && k2 == K2 / 2) r = (int32_t)row;
        else if (ok1 && (unsigned)p2 < (unsigned)g.g[2]) r = lookup(voxel_key(c.x, p0, p1, p2, g));
        *dst = r;
        dst += cap;
      }
    }
  }
}

template <bool K333>
__global__ void subm_map_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                uint32_t cap, Grid3 g, Kernel3 kr,
                                const uint64_t* __restrict__ table, uint32_t mask,
                                int32_t* __restrict__ map) {
  const uint32_t n = min(*n_ptr, cap);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x)
    subm_row_taps<K333>(__ldg(coords + row), row, g, kr, cap, map,
                        [&](uint32_t key) { return hash_lookup(table, mask, key); });
}

// ---------------------------------------------------------------- strided map
// workspace layout (32-bit words):
//   [0, W)        bitmap over the output grid
//   [W, 2W)       exclusive popcount prefix per word (global after emit)
//   [2W, 2W+B)    per-scan-block popcount sums
struct DownWs {
  uint32_t* bitmap;
  uint32_t* prefix;
  uint32_t* block_sums;
  uint32_t words;
  uint32_t blocks;
};

__host__ __device__ inline uint32_t down_words(const int32_t og[3], int batch) {
  unsigned long long cells = (unsigned long long)batch * og[0] * og[1] * og[2];
  return (uint32_t)((cells + 31) / 32);
}

// The output cell that input coordinate c reaches through tap k of a strided conv, if any.
__device__ __forceinline__ bool tap_output_cell(const int4 c, int k, const Grid3& gout,
                                                const Kernel3& kr, uint32_t* cell) {
  const int k2 = k % kr.k[2], k1 = (k / kr.k[2]) % kr.k[1], k0 = k / (kr.k[2] * kr.k[1]);
  const int v0 = c.y + kr.p[0] - k0 * kr.d[0];
  const int v1 = c.z + kr.p[1] - k1 * kr.d[1];
  const int v2 = c.w + kr.p[2] - k2 * kr.d[2];
  if (v0 < 0 || v1 < 0 || v2 < 0 || !stride_divides(v0, kr.s[0], kr.sh[0]) ||
      !stride_divides(v1, kr.s[1], kr.sh[1]) || !stride_divides(v2, kr.s[2], kr.sh[2]))
    return false;
  const int o0 = stride_quotient(v0, kr.s[0], kr.sh[0]), o1 = stride_quotient(v1, kr.s[1], kr.sh[1]),
            o2 = stride_quotient(v2, kr.s[2], kr.sh[2]);
  if (o0 >= gout.g[0] || o1 >= gout.g[1] || o2 >= gout.g[2]) return false;
  *cell = voxel_key(c.x, o0, o1, o2, gout);
  return true;
}

// Visits the output cells one input row reaches: for every axis only the taps with
// (c + pad - k*dil) divisible by the stride and inside the output grid survive, so
// the nest below does ~14 divisions per row instead of 81, and `visit` runs once
// per (input row, tap) pair of the rulebook.
template <typename F>
__device__ __forceinline__ void for_each_output(const int4 c, const Grid3& gout, const Kernel3& kr,
                                                F visit) {
  for (int k0 = 0; k0 < kr.k[0]; ++k0) {
    const int v0 = c.y + kr.p[0] - k0 * kr.d[0];
    if (v0 < 0 || !stride_divides(v0, kr.s[0], kr.sh[0])) continue;
    const int o0 = stride_quotient(v0, kr.s[0], kr.sh[0]);
    if (o0 >= gout.g[0]) continue;
    for (int k1 = 0; k1 < kr.k[1]; ++k1) {
      const int v1 = c.z + kr.p[1] - k1 * kr.d[1];
      if (v1 < 0 || !stride_divides(v1, kr.s[1], kr.sh[1])) continue;
      const int o1 = stride_quotient(v1, kr.s[1], kr.sh[1]);
      if (o1 >= gout.g[1]) continue;
      for (int k2 = 0; k2 < kr.k[2]; ++k2) {
        const int v2 = c.w + kr.p[2] - k2 * kr.d[2];
        if (v2 < 0 || !stride_divides(v2, kr.s[2], kr.sh[2])) continue;
        const int o2 = stride_quotient(v2, kr.s[2], kr.sh[2]);
        if (o2 >= gout.g[2]) continue;
        visit((k0 * kr.k[1] + k1) * kr.k[2] + k2, voxel_key(c.x, o0, o1, o2, gout));
      }
    }
  }
}

// With dilation 1 the outputs an input coordinate c reaches along one axis are a range:
// tap k = c + pad - o * stride lies in [0, K) exactly for
// ceil((c + pad - K + 1) / stride) <= o <= floor((c + pad) / stride), clipped to the grid.
// No divisibility tests, no tap loop.
struct AxisRange { int lo, hi; };
__device__ __forceinline__ AxisRange output_range(int c, int a, const Grid3& gout,
                                                  const Kernel3& kr) {
  const int top = c + kr.p[a], t = top - kr.k[a] + 1;
  AxisRange r;
  r.hi = min(stride_quotient(top, kr.s[a], kr.sh[a]), gout.g[a] - 1);
  r.lo = t <= 0 ? 0 : stride_quotient(t + kr.s[a] - 1, kr.s[a], kr.sh[a]);
  return r;
}
__host__ __device__ inline bool unit_dilation(const Kernel3& kr) {
  return kr.d[0] == 1 && kr.d[1] == 1 && kr.d[2] == 1;
}

__global__ void down_mark_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                 uint32_t cap, Grid3 gin, Grid3 gout, Kernel3 kr,
                                 uint32_t* bitmap) {
  const uint32_t n = min(*n_ptr, cap);
  const bool unit = unit_dilation(kr) && kr.k[2] <= 32 * kr.s[2];
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x) {
    const int4 c = __ldg(coords + row);
    if ((unsigned)c.x >= (unsigned)gin.batch) continue;
    if (unit) {
      // the reached cells are a box; its cells along the innermost axis are adjacent bits,
      // set with one atomic (two when the run crosses a word)
      const AxisRange r0 = output_range(c.y, 0, gout, kr), r1 = output_range(c.z, 1, gout, kr),
                      r2 = output_range(c.w, 2, gout, kr);
      if (r2.lo > r2.hi) continue;
      const uint32_t nbits = (uint32_t)(r2.hi - r2.lo + 1);
      for (int o0 = r0.lo; o0 <= r0.hi; ++o0)
        for (int o1 = r1.lo; o1 <= r1.hi; ++o1) {
          const uint32_t cell = voxel_key(c.x, o0, o1, r2.lo, gout);
          const unsigned long long run =
              (nbits >= 64u ? ~0ull : (1ull << nbits) - 1ull) << (cell & 31u);
          uint32_t* word = bitmap + (cell >> 5);
          const uint32_t m0 = (uint32_t)run, m1 = (uint32_t)(run >> 32);
          // up to kvol inputs reach the same cells: look before the atomic, most find them set
          if ((*(volatile uint32_t*)word & m0) != m0) atomicOr(word, m0);
          if (m1 && (*(volatile uint32_t*)(word + 1) & m1) != m1) atomicOr(word + 1, m1);
        }
      continue;
    }
    for_each_output(c, gout, kr, [&](int, uint32_t cell) {
      const uint32_t bit = 1u << (cell & 31);
      uint32_t* word = bitmap + (cell >> 5);
      if (!(*(volatile uint32_t*)word & bit)) atomicOr(word, bit);
    });
  }
}

// Up to 64 bits of a bitmap starting at cell `line + x0` of a line of `gx` cells that starts
// at linear cell `line`: bit i of the result is cell x0 + i, zero outside the line.
__device__ __forceinline__ unsigned long long line_bits64(const uint32_t* __restrict__ bitmap,
                                                          uint32_t words, uint32_t line, int x0,
                                                          int count, int gx) {
  const int lo = max(x0, 0), hi = min(x0 + count - 1, gx - 1);
  if (lo > hi) return 0ull;
  const uint32_t start = line + (uint32_t)lo, w = start >> 5, off = start & 31u;
  unsigned long long v = (unsigned long long)__ldg(bitmap + w) >> off;
  if (w + 1 < words) v |= (unsigned long long)__ldg(bitmap + w + 1) << (32u - off);
  if (off && w + 2 < words) v |= (unsigned long long)__ldg(bitmap + w + 2) << (64u - off);
  const int nb = hi - lo + 1;
  if (nb < 64) v &= (1ull << nb) - 1ull;
  return v << (lo - x0);
}

// The mark step when the input rows were made by a strided rulebook themselves: the output
// bitmap is computed from the input's bitmap, 16 output cells of one line per thread.  Output
// cell o is set when any input cell of its window (o * stride - pad + [0, K) per axis, dilation
// 1) is set: the K0 x K1 input lines that matter are OR-ed as bit strings, then each output
// bit tests its K2-wide piece.  No rows are read, no two threads fight for a word (the two
// atomics per thread only merge neighbouring segments of a word).  Input cells whose rank is
// beyond the capacity of the input rows (an overflow the rulebook that made them has already
// reported) count as set.
constexpr int kMarkCells = 16;
__global__ void down_mark_ranked_kernel(const uint32_t* __restrict__ in_bitmap, uint32_t in_words,
                                        Grid3 gin, Grid3 gout, Kernel3 kr,
                                        uint32_t* __restrict__ out_bitmap) {
  const int segs = (gout.g[2] + kMarkCells - 1) / kMarkCells;
  const unsigned long long lines = (unsigned long long)gout.batch * gout.g[0] * gout.g[1];
  const unsigned long long kmask = (1ull << kr.k[2]) - 1ull;
  for (unsigned long long item = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       item < lines * segs; item += (unsigned long long)gridDim.x * blockDim.x) {
    const unsigned long long line = item / segs;
    const int ox0 = (int)(item - line * segs) * kMarkCells;
    const int ncell = min(kMarkCells, gout.g[2] - ox0);
    const int o1 = (int)(line % gout.g[1]);
    const int o0 = (int)((line / gout.g[1]) % gout.g[0]);
    const int b = (int)(line / ((unsigned long long)gout.g[1] * gout.g[0]));
    const int x0 = ox0 * kr.s[2] - kr.p[2];
    const int count = (ncell - 1) * kr.s[2] + kr.k[2];  // <= 64 (checked by the launcher)
    unsigned long long win = 0ull;
    for (int k0 = 0; k0 < kr.k[0]; ++k0) {
      const int i0 = o0 * kr.s[0] - kr.p[0] + k0;
      if ((unsigned)i0 >= (unsigned)gin.g[0]) continue;
      for (int k1 = 0; k1 < kr.k[1]; ++k1) {
        const int i1 = o1 * kr.s[1] - kr.p[1] + k1;
        if ((unsigned)i1 >= (unsigned)gin.g[1]) continue;
        win |= line_bits64(in_bitmap, in_words, voxel_key(b, i0, i1, 0, gin), x0, count, gin.g[2]);
      }
    }
    if (!win) continue;
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < kMarkCells; ++i)
      if (i < ncell && ((win >> (i * kr.s[2])) & kmask)) r |= 1u << i;
    if (!r) continue;
    const uint32_t cell = (uint32_t)(line * gout.g[2]) + (uint32_t)ox0;
    const unsigned long long run = (unsigned long long)r << (cell & 31u);
    atomicOr(out_bitmap + (cell >> 5), (uint32_t)run);
    if (run >> 32) atomicOr(out_bitmap + (cell >> 5) + 1, (uint32_t)(run >> 32));
  }
}

// Row of an output cell from the bitmap and its (global) popcount prefix, -1 if
// the cell is not an output or lies beyond the capacity.
__device__ __forceinline__ int32_t rank_lookup(const uint32_t* __restrict__ bitmap,
                                               const uint32_t* __restrict__ prefix,
                                               uint32_t cell, uint32_t cap) {
  const uint32_t bits = __ldg(bitmap + (cell >> 5));
  const uint32_t b = cell & 31u;
  if (!((bits >> b) & 1u)) return -1;
  const uint32_t row = __ldg(prefix + (cell >> 5)) + __popc(bits & ((1u << b) - 1u));
  return row < cap ? (int32_t)row : -1;
}

// Per block of kScanWordsPerBlock words: exclusive scan of popcounts.
__global__ void __launch_bounds__(kScanThreads) down_scan_kernel(DownWs ws) {
  __shared__ uint32_t warp_sums[kScanThreads / 32];
  const uint32_t w = blockIdx.x * kScanWordsPerBlock + threadIdx.x;
  const uint32_t local = w < ws.words ? __popc(ws.bitmap[w]) : 0u;
  uint32_t incl = local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t v = warp_sums[lane];
    uint32_t s = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += t;
    }
    warp_sums[lane] = s - v;  // exclusive
    if (lane == 31) ws.block_sums[blockIdx.x] = s;
  }
  __syncthreads();
  if (w < ws.words) ws.prefix[w] = warp_sums[warp] + incl - local;
}

// Ranks every set bit: writes the output coordinate, makes the prefix global, and the
// last block publishes the count.  No atomics.
__global__ void __launch_bounds__(kScanThreads)
down_emit_kernel(DownWs ws, Grid3 gout, int4* __restrict__ out_coords, uint32_t* n_out_ptr,
                 uint32_t cap_out, uint32_t* status) {
  __shared__ uint32_t red[32];
  __shared__ uint32_t s_base;
  uint32_t part = 0;
  for (uint32_t i = threadIdx.x; i < blockIdx.x; i += blockDim.x) part += ws.block_sums[i];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  if (threadIdx.x < 32) {
    uint32_t v = red[threadIdx.x];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    if (threadIdx.x == 0) {
      s_base = v;
      if (blockIdx.x == gridDim.x - 1) {
        uint32_t total = v + ws.block_sums[blockIdx.x];
        if (total > cap_out) set_status(status, SPCONVB_ST_OVERFLOW, total);
        *n_out_ptr = min(total, cap_out);
      }
    }
  }
  __syncthreads();
  // Every thread reads one word and makes its prefix global; then the warp goes through its
  // non-empty words together, one lane per bit: the rows of a word are consecutive, so the
  // coordinate stores of a word coalesce, and no lane loops over the bits of a dense word
  // while the others wait.
  const uint32_t w = blockIdx.x * kScanWordsPerBlock + threadIdx.x;
  const uint32_t lane = threadIdx.x & 31u;
  uint32_t bits = 0, row0 = 0;
  int c2 = 0, c1 = 0, c0 = 0, bq = 0;
  if (w < ws.words) {
    bits = ws.bitmap[w];
    row0 = s_base + ws.prefix[w];
    ws.prefix[w] = row0;
    if (bits) {  // the word's first cell
      uint32_t t = w << 5;
      c2 = t % gout.g[2]; t /= gout.g[2];
      c1 = t % gout.g[1]; t /= gout.g[1];
      c0 = t % gout.g[0]; t /= gout.g[0];
      bq = (int)t;
    }
  }
  uint32_t nonempty = __ballot_sync(0xffffffffu, bits != 0u);
  while (nonempty) {
    const int src = __ffs(nonempty) - 1;
    nonempty &= nonempty - 1;
    const uint32_t wb = __shfl_sync(0xffffffffu, bits, src);
    const uint32_t r0 = __shfl_sync(0xffffffffu, row0, src);
    int x = __shfl_sync(0xffffffffu, c2, src) + (int)lane;
    int y = __shfl_sync(0xffffffffu, c1, src);
    int z = __shfl_sync(0xffffffffu, c0, src);
    int b = __shfl_sync(0xffffffffu, bq, src);
    if ((wb >> lane) & 1u) {
      const uint32_t row = r0 + __popc(wb & ((1u << lane) - 1u));
      while (x >= gout.g[2]) {
        x -= gout.g[2];
        if (++y >= gout.g[1]) {
          y = 0;
          if (++z >= gout.g[0]) { z = 0; ++b; }
        }
      }
      if (row < cap_out) out_coords[row] = make_int4(b, z, y, x);
    }
  }
}

// The map rows of the outputs start as "no input" (-1); the scatter kernel then
// writes the pairs that exist.  16-byte stores where the row range allows.
__global__ void map_fill_kernel(const uint32_t* n_out_ptr, uint32_t cap_out, int kvol,
                                int32_t* __restrict__ map) {
  const uint32_t n = min(*n_out_ptr, cap_out);
  const uint32_t n4 = (n + 3) / 4;  // int4 groups per tap (cap_out rows are 16-byte aligned
                                    // only when cap_out % 4 == 0; else fall back to scalars)
  const bool vec = (cap_out & 3u) == 0 && (((uintptr_t)map) & 15u) == 0;
  const unsigned long long work = (unsigned long long)kvol * (vec ? n4 : n);
  for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       idx < work; idx += (unsigned long long)gridDim.x * blockDim.x) {
    if (vec) {
      const uint32_t k = (uint32_t)(idx / n4), g4 = (uint32_t)(idx - (unsigned long long)k * n4);
      ((int4*)(map + (size_t)k * cap_out))[g4] = make_int4(-1, -1, -1, -1);
    } else {
      const uint32_t k = (uint32_t)(idx / n), r = (uint32_t)(idx - (unsigned long long)k * n);
      map[(size_t)k * cap_out + r] = -1;
    }
  }
}

// Input-stationary fill of the output-stationary map: every (input row, tap) pair
// finds its output row by rank and writes itself there.  One rank query (two
// cached loads) per existing pair, instead of kvol hash probes per output row.
__global__ void down_scatter_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                    uint32_t cap, Grid3 gin, Grid3 gout, Kernel3 kr, DownWs ws,
                                    uint32_t cap_out, int32_t* __restrict__ map) {
  const uint32_t n = min(*n_ptr, cap);
  const bool unit = unit_dilation(kr);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x) {
    const int4 c = __ldg(coords + row);
    if ((unsigned)c.x >= (unsigned)gin.batch) continue;
    if (unit) {
      const AxisRange r0 = output_range(c.y, 0, gout, kr), r1 = output_range(c.z, 1, gout, kr),
                      r2 = output_range(c.w, 2, gout, kr);
      for (int o0 = r0.lo; o0 <= r0.hi; ++o0) {
        const int k0 = c.y + kr.p[0] - o0 * kr.s[0];
        for (int o1 = r1.lo; o1 <= r1.hi; ++o1) {
          const int k01 = k0 * kr.k[1] + (c.z + kr.p[1] - o1 * kr.s[1]);
          for (int o2 = r2.lo; o2 <= r2.hi; ++o2) {
            const int k = k01 * kr.k[2] + (c.w + kr.p[2] - o2 * kr.s[2]);
            const int32_t o =
                rank_lookup(ws.bitmap, ws.prefix, voxel_key(c.x, o0, o1, o2, gout), cap_out);
            if (o >= 0) map[(size_t)k * cap_out + o] = (int32_t)row;
          }
        }
      }
      continue;
    }
    for_each_output(c, gout, kr, [&](int k, uint32_t cell) {
      const int32_t o = rank_lookup(ws.bitmap, ws.prefix, cell, cap_out);
      if (o >= 0) map[(size_t)k * cap_out + o] = (int32_t)row;
    });
  }
}

// Optional: the outputs' hash table, for callers that want one.
__global__ void hash_rows_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                 uint32_t cap, Grid3 g, uint64_t* table, uint32_t mask,
                                 uint32_t* status) {
  const uint32_t n = min(*n_ptr, cap);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x) {
    const int4 c = __ldg(coords + row);
    hash_insert(table, mask, voxel_key(c.x, c.y, c.z, c.w, g), row, status);
  }
}

// Submanifold map of a coordinate set that came out of down_map: neighbours are
// found by rank in that set's bitmap, no hash table involved.  One thread per row;
// rows are in cell order, so a warp's lookups of one tap fall into the same or
// adjacent bitmap words and its map stores coalesce.
template <bool K333>
__global__ void subm_ranked_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                   uint32_t cap, Grid3 g, Kernel3 kr, DownWs ws,
                                   int32_t* __restrict__ map) {
  const uint32_t n = min(*n_ptr, cap);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x)
    subm_row_taps<K333>(__ldg(coords + row), row, g, kr, cap, map, [&](uint32_t key) {
      return rank_lookup(ws.bitmap, ws.prefix, key, cap);
    });
}

// Blocks for one thread per row: small blocks, so that a few thousand rows still spread
// over the SMs, capped at a few waves (the kernels stride).
static int row_blocks(uint32_t rows, int threads) {
  unsigned long long b = ((unsigned long long)rows + threads - 1) / threads;
  const unsigned long long most = (unsigned long long)kSmCount * 16;
  if (b > most) b = most;
  if (b < 1) b = 1;
  return (int)b;
}

static bool is_k333(const Kernel3& kr) {
  return kr.k[0] == 3 && kr.k[1] == 3 && kr.k[2] == 3 && kr.d[0] == 1 && kr.d[1] == 1 &&
         kr.d[2] == 1;
}

static void set_stride_shifts(Kernel3& kr) {
  for (int a = 0; a < 3; ++a) {
    kr.sh[a] = -1;
    for (int b = 0; b < 16; ++b)
      if (kr.s[a] == (1 << b)) kr.sh[a] = b;
  }
}

// Output-stationary form of the strided map, for inputs that were themselves made by a
// strided rulebook (their bitmap and rank prefix exist): one thread per output row walks the
// taps in tap order, finds the input cell of each (out * stride - pad + tap * dilation) and
// ranks it in the input's bitmap.  Every map entry is written exactly once, so there is no
// fill pass, and a warp's stores of one tap land in one or two lines of map[k][.].
template <bool K333>
__global__ void down_gather_ranked_kernel(const int4* __restrict__ out_coords,
                                          const uint32_t* n_out_ptr, uint32_t cap_out, Grid3 gin,
                                          Kernel3 kr, DownWs in_ws, uint32_t cap_in,
                                          int32_t* __restrict__ map) {
  const uint32_t n = min(*n_out_ptr, cap_out);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n;
       row += gridDim.x * blockDim.x) {
    const int4 c = __ldg(out_coords + row);
    int32_t* dst = map + row;
    if (K333) {
      // 3x3x3, dilation 1: the taps unrolled, 27 independent rank lookups
      const bool bok = (unsigned)c.x < (unsigned)gin.batch;
#pragma unroll
      for (int k0 = 0; k0 < 3; ++k0) {
        const int p0 = c.y * kr.s[0] - kr.p[0] + k0;
        const bool ok0 = bok && (unsigned)p0 < (unsigned)gin.g[0];
#pragma unroll
        for (int k1 = 0; k1 < 3; ++k1) {
          const int p1 = c.z * kr.s[1] - kr.p[1] + k1;
          const bool ok1 = ok0 && (unsigned)p1 < (unsigned)gin.g[1];
#pragma unroll
          for (int k2 = 0; k2 < 3; ++k2) {
            const int p2 = c.w * kr.s[2] - kr.p[2] + k2;
            int32_t r = -1;
            if (ok1 && (unsigned)p2 < (unsigned)gin.g[2])
              r = rank_lookup(in_ws.bitmap, in_ws.prefix, voxel_key(c.x, p0, p1, p2, gin), cap_in);
            *dst = r;
            dst += cap_out;
          }
        }
      }
      continue;
    }
    for (int k0 = 0; k0 < kr.k[0]; ++k0) {
      const int p0 = c.y * kr.s[0] - kr.p[0] + k0 * kr.d[0];
      const bool ok0 = (unsigned)p0 < (unsigned)gin.g[0];
      for (int k1 = 0; k1 < kr.k[1]; ++k1) {
        const int p1 = c.z * kr.s[1] - kr.p[1] + k1 * kr.d[1];
        const bool ok1 = ok0 && (unsigned)p1 < (unsigned)gin.g[1];
#pragma unroll 3
        for (int k2 = 0; k2 < kr.k[2]; ++k2) {
          const int p2 = c.w * kr.s[2] - kr.p[2] + k2 * kr.d[2];
          int32_t r = -1;
          if (ok1 && (unsigned)p2 < (unsigned)gin.g[2])
            r = rank_lookup(in_ws.bitmap, in_ws.prefix, voxel_key(c.x, p0, p1, p2, gin), cap_in);
          *dst = r;
          dst += cap_out;
        }
      }
    }
  }
}

// Fixed-size grids: a multiple of the SM count, independent of the row count.
static int flat_blocks(unsigned long long work_cap) {
  unsigned long long b = (work_cap + kThreads - 1) / kThreads;
  const unsigned long long most = (unsigned long long)kSmCount * 8;
  if (b > most) b = most;
  if (b < 1) b = 1;
  return (int)b;
}

static bool grid_fits(const int32_t g[3], int batch) {
  if (batch < 1 || g[0] < 1 || g[1] < 1 || g[2] < 1) return false;
  unsigned long long cells = (unsigned long long)batch * g[0] * g[1] * g[2];
  return cells < 0xffffffffull;
}

static Grid3 make_grid(const int32_t g[3], int batch) {
  Grid3 r;
  r.g[0] = g[0]; r.g[1] = g[1]; r.g[2] = g[2];
  r.batch = batch;
  return r;
}

// ------------------------------------------------- allocation-free variant
// Scratch for spconvb_down_map_static: part of the library image, so every GPU
// that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = SPCONVB_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_down_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_down_scratch_ptr[kMaxDevices] = {};
static std::mutex g_down_scratch_mutex;

// The array's name is only a host-side handle; the address kernels can use
// comes from cudaGetSymbolAddress, asked once per device with that device current.
static int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return (int)ce;
  if (dev < 0 || dev >= kMaxDevices) return SPCONVB_E_ARG;
  std::lock_guard<std::mutex> lock(g_down_scratch_mutex);
  if (!g_down_scratch_ptr[dev]) {
    void* p = nullptr;
    ce = cudaGetSymbolAddress(&p, g_down_scratch);
    if (ce != cudaSuccess) return (int)ce;
    if (!p) return SPCONVB_E_STATE;
    g_down_scratch_ptr[dev] = p;
  }
  *out = g_down_scratch_ptr[dev];
  return SPCONVB_OK;
}

}  // namespace spconvb

using namespace spconvb;

extern "C" {

uint32_t spconvb_hash_slots(uint32_t cap_rows) {
  uint32_t s = 1024;
  while (s < 2u * cap_rows && s < 0x80000000u) s <<= 1;
  return s;
}

int32_t spconvb_out_extent(int32_t in, int32_t k, int32_t stride, int32_t pad, int32_t dilation) {
  int v = in + 2 * pad - dilation * (k - 1) - 1;
  if (v < 0 || stride < 1) return 0;
  return v / stride + 1;
}

int spconvb_hash_build(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                       uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                       uint64_t* table, uint32_t slots, uint32_t flags, uint32_t* status,
                       void* stream) {
  if (!coords || !n_ptr || !table || !grid) return SPCONVB_E_ARG;
  if (slots < 8 || (slots & (slots - 1)) || slots < 2ull * cap) return SPCONVB_E_ARG;
  if (!grid_fits(grid, batch)) return SPCONVB_E_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (!(flags & SPCONVB_FLAG_PREZEROED))
    SPCONVB_CUDA_TRY(cudaMemsetAsync(table, 0, sizeof(uint64_t) * (size_t)slots, st));
  if (launch_rows == 0 || launch_rows > cap) launch_rows = cap;
  hash_build_kernel<<<flat_blocks(launch_rows), kThreads, 0, st>>>(
      (const int4*)coords, n_ptr, cap, make_grid(grid, batch), table, slots - 1, status);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_subm_map(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                     uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                     const int32_t ksize[3], const int32_t dilation[3], const uint64_t* table,
                     uint32_t slots, int32_t* map, uint32_t* status, void* stream) {
  (void)status;
  if (!coords || !n_ptr || !table || !map || !grid || !ksize || !dilation) return SPCONVB_E_ARG;
  if (slots < 8 || (slots & (slots - 1))) return SPCONVB_E_ARG;
  if (!grid_fits(grid, batch)) return SPCONVB_E_RANGE;
  Kernel3 kr;
  for (int a = 0; a < 3; ++a) {
    if (ksize[a] < 1 || !(ksize[a] & 1) || dilation[a] < 1) return SPCONVB_E_ARG;
    kr.k[a] = ksize[a]; kr.d[a] = dilation[a]; kr.s[a] = 1; kr.p[a] = 0;
  }
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  if (kvol > 65535) return SPCONVB_E_ARG;
  if (launch_rows == 0 || launch_rows > cap) launch_rows = cap;
  constexpr int kRowThreads = 128;
  const int blocks = row_blocks(launch_rows, kRowThreads);
  if (is_k333(kr))
    subm_map_kernel<true><<<blocks, kRowThreads, 0, (cudaStream_t)stream>>>(
        (const int4*)coords, n_ptr, cap, make_grid(grid, batch), kr, table, slots - 1, map);
  else
    subm_map_kernel<false><<<blocks, kRowThreads, 0, (cudaStream_t)stream>>>(
        (const int4*)coords, n_ptr, cap, make_grid(grid, batch), kr, table, slots - 1, map);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_subm_map_ranked(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                            uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                            const int32_t ksize[3], const int32_t dilation[3],
                            const void* down_workspace, int32_t* map, uint32_t* status,
                            void* stream) {
  (void)status;
  if (!coords || !n_ptr || !down_workspace || !map || !grid || !ksize || !dilation)
    return SPCONVB_E_ARG;
  if (!grid_fits(grid, batch)) return SPCONVB_E_RANGE;
  Kernel3 kr;
  for (int a2 = 0; a2 < 3; ++a2) {
    if (ksize[a2] < 1 || !(ksize[a2] & 1) || dilation[a2] < 1) return SPCONVB_E_ARG;
    kr.k[a2] = ksize[a2]; kr.d[a2] = dilation[a2]; kr.s[a2] = 1; kr.p[a2] = 0;
  }
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  if (kvol > 65535) return SPCONVB_E_ARG;
  DownWs ws;
  ws.words = down_words(grid, batch);
  ws.blocks = (ws.words + kScanWordsPerBlock - 1) / kScanWordsPerBlock;
  ws.bitmap = (uint32_t*)down_workspace;
  ws.prefix = ws.bitmap + ws.words;
  ws.block_sums = ws.prefix + ws.words;
  if (launch_rows == 0 || launch_rows > cap) launch_rows = cap;
  constexpr int kRowThreads = 128;
  const int blocks = row_blocks(launch_rows, kRowThreads);
  if (is_k333(kr))
    subm_ranked_kernel<true><<<blocks, kRowThreads, 0, (cudaStream_t)stream>>>(
        (const int4*)coords, n_ptr, cap, make_grid(grid, batch), kr, ws, map);
  else
    subm_ranked_kernel<false><<<blocks, kRowThreads, 0, (cudaStream_t)stream>>>(
        (const int4*)coords, n_ptr, cap, make_grid(grid, batch), kr, ws, map);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

// Map of an inverse (transposed) convolution: it runs over the pairs of a strided
// rulebook with input and output swapped, so its outputs are that rulebook's input rows
// and map[k][i] is the strided output row that input row i reaches through tap k.  One
// thread per (row, tap): the strided conv's cell arithmetic for that tap, then a rank
// lookup in the bitmap the strided rulebook left behind.
__global__ void inverse_map_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                   uint32_t cap, Grid3 gin, Grid3 gout, Kernel3 kr, int kvol,
                                   DownWs ws, uint32_t cap_coarse, int32_t* __restrict__ map) {
  const uint32_t n = min(*n_ptr, cap);
  const unsigned long long work = (unsigned long long)n * kvol;
  for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       idx < work; idx += (unsigned long long)gridDim.x * blockDim.x) {
    const int k = (int)(idx / n);  // rows fastest: coalesced stores of map[k][row]
    const uint32_t row = (uint32_t)(idx - (unsigned long long)k * n);
    const int4 c = __ldg(coords + row);
    int32_t o = -1;
    uint32_t cell;
    if ((unsigned)c.x < (unsigned)gin.batch && tap_output_cell(c, k, gout, kr, &cell))
      o = rank_lookup(ws.bitmap, ws.prefix, cell, cap_coarse);
    map[(size_t)k * cap + row] = o;
  }
}

int spconvb_inverse_map(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                        uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                        const int32_t ksize[3], const int32_t stride[3], const int32_t pad[3],
                        const int32_t dilation[3], const void* down_workspace,
                        uint32_t cap_coarse, int32_t* map, uint32_t* status, void* stream) {
  (void)status;
  if (!coords || !n_ptr || !grid || !ksize || !stride || !pad || !dilation || !down_workspace ||
      !map)
    return SPCONVB_E_ARG;
  if (!grid_fits(grid, batch)) return SPCONVB_E_RANGE;
  Kernel3 kr;
  int32_t og[3];
  for (int a2 = 0; a2 < 3; ++a2) {
    if (ksize[a2] < 1 || stride[a2] < 1 || pad[a2] < 0 || dilation[a2] < 1) return SPCONVB_E_ARG;
    kr.k[a2] = ksize[a2]; kr.s[a2] = stride[a2]; kr.p[a2] = pad[a2]; kr.d[a2] = dilation[a2];
    og[a2] = spconvb_out_extent(grid[a2], ksize[a2], stride[a2], pad[a2], dilation[a2]);
    if (og[a2] < 1) return SPCONVB_E_ARG;
  }
  set_stride_shifts(kr);
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  if (kvol > 65535) return SPCONVB_E_ARG;
  if (!grid_fits(og, batch)) return SPCONVB_E_RANGE;
  DownWs ws;
  ws.words = down_words(og, batch);
  ws.blocks = (ws.words + kScanWordsPerBlock - 1) / kScanWordsPerBlock;
  ws.bitmap = (uint32_t*)down_workspace;
  ws.prefix = ws.bitmap + ws.words;
  ws.block_sums = ws.prefix + ws.words;
  if (launch_rows == 0 || launch_rows > cap) launch_rows = cap;
  inverse_map_kernel<<<flat_blocks((unsigned long long)launch_rows * kvol), kThreads, 0,
                       (cudaStream_t)stream>>>((const int4*)coords, n_ptr, cap,
                                               make_grid(grid, batch), make_grid(og, batch), kr,
                                               kvol, ws, cap_coarse, map);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

size_t spconvb_down_workspace_bytes(const int32_t out_grid[3], int32_t batch) {
  if (!out_grid || !grid_fits(out_grid, batch)) return 0;
  size_t words = down_words(out_grid, batch);
  size_t blocks = (words + kScanWordsPerBlock - 1) / kScanWordsPerBlock;
  return sizeof(uint32_t) * (2 * words + blocks + 16);
}

// Shared body of spconvb_down_map and spconvb_down_map_ranked.
static int down_map_impl(const int32_t* in_coords, const uint32_t* n_in_ptr, uint32_t cap_in,
                         uint32_t launch_rows, const int32_t in_grid[3], int32_t batch,
                         const int32_t ksize[3], const int32_t stride[3], const int32_t pad[3],
                         const int32_t dilation[3], const void* in_workspace, void* workspace,
                         int32_t* out_coords, uint32_t* n_out_ptr, uint32_t cap_out, int32_t* map,
                         uint64_t* out_table, uint32_t out_slots, uint32_t flags,
                         uint32_t* status, void* stream) {
  if (!in_coords || !n_in_ptr || !in_grid || !ksize || !stride || !pad || !dilation ||
      !workspace || !out_coords || !n_out_ptr || !map)
    return SPCONVB_E_ARG;
  if (out_table && (out_slots < 8 || (out_slots & (out_slots - 1)) || out_slots < 2ull * cap_out))
    return SPCONVB_E_ARG;
  if (!grid_fits(in_grid, batch)) return SPCONVB_E_RANGE;
  Kernel3 kr;
  int32_t og[3];
  for (int a = 0; a < 3; ++a) {
    if (ksize[a] < 1 || stride[a] < 1 || dilation[a] < 1 || pad[a] < 0) return SPCONVB_E_ARG;
    kr.k[a] = ksize[a]; kr.s[a] = stride[a]; kr.p[a] = pad[a]; kr.d[a] = dilation[a];
    og[a] = spconvb_out_extent(in_grid[a], ksize[a], stride[a], pad[a], dilation[a]);
    if (og[a] < 1) return SPCONVB_E_ARG;
  }
  set_stride_shifts(kr);
  if (!grid_fits(og, batch)) return SPCONVB_E_RANGE;
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  if (kvol > 65535) return SPCONVB_E_ARG;
  cudaStream_t st = (cudaStream_t)stream;

  DownWs ws;
  ws.words = down_words(og, batch);
  ws.blocks = (ws.words + kScanWordsPerBlock - 1) / kScanWordsPerBlock;
  ws.bitmap = (uint32_t*)workspace;
  ws.prefix = ws.bitmap + ws.words;
  ws.block_sums = ws.prefix + ws.words;
  if (!(flags & SPCONVB_FLAG_PREZEROED)) {
    SPCONVB_CUDA_TRY(cudaMemsetAsync(ws.bitmap, 0, sizeof(uint32_t) * (size_t)ws.words, st));
    if (out_table)
      SPCONVB_CUDA_TRY(cudaMemsetAsync(out_table, 0, sizeof(uint64_t) * (size_t)out_slots, st));
  }
  Grid3 gin = make_grid(in_grid, batch), gout = make_grid(og, batch);
  if (launch_rows == 0 || launch_rows > cap_in) launch_rows = cap_in;
  // rows made by a rulebook: their bitmap gives the outputs' bitmap directly (when a
  // thread's window of input cells fits 64 bits)
  const bool from_bitmap = in_workspace && unit_dilation(kr) && kr.k[2] <= 32 &&
                           (kMarkCells - 1) * kr.s[2] + kr.k[2] <= 64;
  if (from_bitmap) {
    const unsigned long long items = (unsigned long long)batch * og[0] * og[1] *
                                     (unsigned long long)((og[2] + kMarkCells - 1) / kMarkCells);
    down_mark_ranked_kernel<<<flat_blocks(items), kThreads, 0, st>>>(
        (const uint32_t*)in_workspace, down_words(in_grid, batch), gin, gout, kr, ws.bitmap);
  } else {
    down_mark_kernel<<<flat_blocks(launch_rows), kThreads, 0, st>>>(
        (const int4*)in_coords, n_in_ptr, cap_in, gin, gout, kr, ws.bitmap);
  }
  SPCONVB_LAUNCH_CHECK();
  down_scan_kernel<<<ws.blocks, kScanThreads, 0, st>>>(ws);
  SPCONVB_LAUNCH_CHECK();
  down_emit_kernel<<<ws.blocks, kScanThreads, 0, st>>>(ws, gout, (int4*)out_coords, n_out_ptr,
                                                       cap_out, status);
  SPCONVB_LAUNCH_CHECK();
  if (in_workspace) {
    // the inputs can be ranked: every map entry is looked up from the output side
    DownWs in_ws;
    in_ws.words = down_words(in_grid, batch);
    in_ws.blocks = 0;
    in_ws.bitmap = (uint32_t*)in_workspace;
    in_ws.prefix = in_ws.bitmap + in_ws.words;
    in_ws.block_sums = nullptr;
    constexpr int kRowThreads = 128;
    if (is_k333(kr))
      down_gather_ranked_kernel<true><<<row_blocks(cap_out, kRowThreads), kRowThreads, 0, st>>>(
          (const int4*)out_coords, n_out_ptr, cap_out, gin, kr, in_ws, cap_in, map);
    else
      down_gather_ranked_kernel<false><<<row_blocks(cap_out, kRowThreads), kRowThreads, 0, st>>>(
          (const int4*)out_coords, n_out_ptr, cap_out, gin, kr, in_ws, cap_in, map);
  } else {
    map_fill_kernel<<<flat_blocks((unsigned long long)cap_out * kvol / 4 + 1), kThreads, 0, st>>>(
        n_out_ptr, cap_out, kvol, map);
    SPCONVB_LAUNCH_CHECK();
    down_scatter_kernel<<<flat_blocks(launch_rows), kThreads, 0, st>>>(
        (const int4*)in_coords, n_in_ptr, cap_in, gin, gout, kr, ws, cap_out, map);
  }
  if (out_table) {
    SPCONVB_LAUNCH_CHECK();
    hash_rows_kernel<<<flat_blocks(cap_out), kThreads, 0, st>>>(
        (const int4*)out_coords, n_out_ptr, cap_out, gout, out_table, out_slots - 1, status);
  }
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_down_map(const int32_t* in_coords, const uint32_t* n_in_ptr, uint32_t cap_in,
                     uint32_t launch_rows, const int32_t in_grid[3], int32_t batch,
                     const int32_t ksize[3], const int32_t stride[3], const int32_t pad[3],
                     const int32_t dilation[3], const uint64_t* in_table, uint32_t in_slots,
                     void* workspace, int32_t* out_coords, uint32_t* n_out_ptr, uint32_t cap_out,
                     int32_t* map, uint64_t* out_table, uint32_t out_slots, uint32_t flags,
                     uint32_t* status, void* stream) {
  (void)in_table;
  (void)in_slots;
  return down_map_impl(in_coords, n_in_ptr, cap_in, launch_rows, in_grid, batch, ksize, stride,
                       pad, dilation, nullptr, workspace, out_coords, n_out_ptr, cap_out, map,
                       out_table, out_slots, flags, status, stream);
}

int spconvb_down_map_ranked(const int32_t* in_coords, const uint32_t* n_in_ptr, uint32_t cap_in,
                            uint32_t launch_rows, const int32_t in_grid[3], int32_t batch,
                            const int32_t ksize[3], const int32_t stride[3],
                            const int32_t pad[3], const int32_t dilation[3],
                            const void* in_workspace, void* workspace, int32_t* out_coords,
                            uint32_t* n_out_ptr, uint32_t cap_out, int32_t* map,
                            uint64_t* out_table, uint32_t out_slots, uint32_t flags,
                            uint32_t* status, void* stream) {
  if (!in_workspace) return SPCONVB_E_ARG;
  return down_map_impl(in_coords, n_in_ptr, cap_in, launch_rows, in_grid, batch, ksize, stride,
                       pad, dilation, in_workspace, workspace, out_coords, n_out_ptr, cap_out, map,
                       out_table, out_slots, flags, status, stream);
}

int spconvb_down_map_static(const int32_t* in_coords, const uint32_t* n_in_ptr, uint32_t cap_in,
                            uint32_t launch_rows, const int32_t in_grid[3], int32_t batch,
                            const int32_t ksize[3], const int32_t stride[3],
                            const int32_t pad[3], const int32_t dilation[3],
                            const uint64_t* in_table, uint32_t in_slots, int32_t* out_coords,
                            uint32_t* n_out_ptr, uint32_t cap_out, int32_t* map,
                            uint64_t* out_table, uint32_t out_slots, uint32_t flags,
                            uint32_t* status, void* stream) {
  // every argument check of spconvb_down_map that can fail comes first: nothing of the
  // caller's memory (the optional output table) is cleared for a call that is then refused
  if (!in_coords || !n_in_ptr || !in_grid || !ksize || !stride || !pad || !dilation ||
      !out_coords || !n_out_ptr || !map)
    return SPCONVB_E_ARG;
  if (out_table && (out_slots < 8 || (out_slots & (out_slots - 1)) || out_slots < 2ull * cap_out))
    return SPCONVB_E_ARG;
  if (!grid_fits(in_grid, batch)) return SPCONVB_E_RANGE;
  int32_t og[3];
  for (int a = 0; a < 3; ++a) {
    if (ksize[a] < 1 || stride[a] < 1 || dilation[a] < 1 || pad[a] < 0) return SPCONVB_E_ARG;
    og[a] = spconvb_out_extent(in_grid[a], ksize[a], stride[a], pad[a], dilation[a]);
    if (og[a] < 1) return SPCONVB_E_ARG;
  }
  if (ksize[0] * ksize[1] * ksize[2] > 65535) return SPCONVB_E_ARG;
  const size_t need = spconvb_down_workspace_bytes(og, batch);
  if (need == 0) return SPCONVB_E_RANGE;
  if (need > kStaticScratchBytes) return SPCONVB_E_SCRATCH_LIMIT;
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != SPCONVB_OK) return rc;
  // The array still holds the previous call's bitmap: it is cleared on every
  // call, whatever the caller says about its own buffers.
  cudaStream_t st = (cudaStream_t)stream;
  const size_t bitmap_bytes = sizeof(uint32_t) * (size_t)down_words(og, batch);
  SPCONVB_CUDA_TRY(cudaMemsetAsync(scratch, 0, bitmap_bytes, st));
  if (out_table && !(flags & SPCONVB_FLAG_PREZEROED))
    SPCONVB_CUDA_TRY(cudaMemsetAsync(out_table, 0, sizeof(uint64_t) * (size_t)out_slots, st));
  return spconvb_down_map(in_coords, n_in_ptr, cap_in, launch_rows, in_grid, batch, ksize, stride,
                          pad, dilation, in_table, in_slots, scratch, out_coords, n_out_ptr,
                          cap_out, map, out_table, out_slots, flags | SPCONVB_FLAG_PREZEROED,
                          status, stream);
}


}  // extern "C"
