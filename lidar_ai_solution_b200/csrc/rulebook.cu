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
};

__global__ void subm_map_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                uint32_t cap, Grid3 g, Kernel3 kr, int kvol,
                                const uint64_t* __restrict__ table, uint32_t mask,
                                int32_t* __restrict__ map) {
  const uint32_t n = min(*n_ptr, cap);
  const unsigned long long work = (unsigned long long)n * kvol;
  for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       idx < work; idx += (unsigned long long)gridDim.x * blockDim.x) {
    const int k = (int)(idx / n);
    const uint32_t row = (uint32_t)(idx - (unsigned long long)k * n);
    const int k2 = k % kr.k[2], k1 = (k / kr.k[2]) % kr.k[1], k0 = k / (kr.k[2] * kr.k[1]);
    const int d0 = (k0 - kr.k[0] / 2) * kr.d[0];
    const int d1 = (k1 - kr.k[1] / 2) * kr.d[1];
    const int d2 = (k2 - kr.k[2] / 2) * kr.d[2];
    int32_t r = -1;
    if ((d0 | d1 | d2) == 0) {
      r = (int32_t)row;
    } else {
      int4 c = __ldg(coords + row);
      int p0 = c.y + d0, p1 = c.z + d1, p2 = c.w + d2;
      if ((unsigned)p0 < (unsigned)g.g[0] && (unsigned)p1 < (unsigned)g.g[1] &&
          (unsigned)p2 < (unsigned)g.g[2] && (unsigned)c.x < (unsigned)g.batch)
        r = hash_lookup(table, mask, voxel_key(c.x, p0, p1, p2, g));
    }
    map[(size_t)k * cap + row] = r;
  }
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

__global__ void down_mark_kernel(const int4* __restrict__ coords, const uint32_t* n_ptr,
                                 uint32_t cap, Grid3 gin, Grid3 gout, Kernel3 kr, int kvol,
                                 uint32_t* bitmap) {
  const uint32_t n = min(*n_ptr, cap);
  const unsigned long long work = (unsigned long long)n * kvol;
  for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       idx < work; idx += (unsigned long long)gridDim.x * blockDim.x) {
    const int k = (int)(idx / n);
    const uint32_t row = (uint32_t)(idx - (unsigned long long)k * n);
    const int kk[3] = {k / (kr.k[2] * kr.k[1]), (k / kr.k[2]) % kr.k[1], k % kr.k[2]};
    int4 c = __ldg(coords + row);
    if ((unsigned)c.x >= (unsigned)gin.batch) continue;
    const int ci[3] = {c.y, c.z, c.w};
    int o[3];
    bool ok = true;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      int v = ci[a] + kr.p[a] - kk[a] * kr.d[a];
      ok = ok && v >= 0 && (v % kr.s[a]) == 0;
      o[a] = v / kr.s[a];
      ok = ok && o[a] < gout.g[a];
    }
    if (!ok) continue;
    uint32_t cell = voxel_key(c.x, o[0], o[1], o[2], gout);
    atomicOr(bitmap + (cell >> 5), 1u << (cell & 31));
  }
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

// Ranks every set bit (one word per thread, so at most 32 rows each): writes
// the output coordinate, makes the prefix global, and the last block publishes
// the count.  No atomics: rows are inserted in the hash table by the map kernel.
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
  const uint32_t w = blockIdx.x * kScanWordsPerBlock + threadIdx.x;
  if (w >= ws.words) return;
  uint32_t bits = ws.bitmap[w];
  uint32_t row = s_base + ws.prefix[w];
  ws.prefix[w] = row;
  if (!bits) return;
  // decode the word's first cell once, then walk the set bits
  uint32_t t = w << 5;
  int c2 = t % gout.g[2]; t /= gout.g[2];
  int c1 = t % gout.g[1]; t /= gout.g[1];
  int c0 = t % gout.g[0]; t /= gout.g[0];
  int bq = (int)t;
  int prev = 0;
  while (bits) {
    const int b = __ffs(bits) - 1;
    bits &= bits - 1;
    c2 += b - prev;
    prev = b;
    while (c2 >= gout.g[2]) {
      c2 -= gout.g[2];
      if (++c1 >= gout.g[1]) {
        c1 = 0;
        if (++c0 >= gout.g[0]) { c0 = 0; ++bq; }
      }
    }
    if (row < cap_out) out_coords[row] = make_int4(bq, c0, c1, c2);
    ++row;
  }
}

__global__ void down_map_kernel(const int4* __restrict__ out_coords, const uint32_t* n_out_ptr,
                                uint32_t cap_out, Grid3 gin, Grid3 gout, Kernel3 kr, int kvol,
                                const uint64_t* __restrict__ in_table, uint32_t in_mask,
                                int32_t* __restrict__ map, uint64_t* out_table,
                                uint32_t out_mask, uint32_t* status) {
  const uint32_t n = min(*n_out_ptr, cap_out);
  const unsigned long long work = (unsigned long long)n * kvol;
  for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       idx < work; idx += (unsigned long long)gridDim.x * blockDim.x) {
    const int k = (int)(idx / n);
    const uint32_t row = (uint32_t)(idx - (unsigned long long)k * n);
    const int k2 = k % kr.k[2], k1 = (k / kr.k[2]) % kr.k[1], k0 = k / (kr.k[2] * kr.k[1]);
    int4 c = __ldg(out_coords + row);
    // the thread of tap 0 also enters the row in the output hash table
    if (k == 0 && out_table)
      hash_insert(out_table, out_mask, voxel_key(c.x, c.y, c.z, c.w, gout), row, status);
    int p0 = c.y * kr.s[0] - kr.p[0] + k0 * kr.d[0];
    int p1 = c.z * kr.s[1] - kr.p[1] + k1 * kr.d[1];
    int p2 = c.w * kr.s[2] - kr.p[2] + k2 * kr.d[2];
    int32_t r = -1;
    if ((unsigned)p0 < (unsigned)gin.g[0] && (unsigned)p1 < (unsigned)gin.g[1] &&
        (unsigned)p2 < (unsigned)gin.g[2])
      r = hash_lookup(in_table, in_mask, voxel_key(c.x, p0, p1, p2, gin));
    map[(size_t)k * cap_out + row] = r;
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
  if (slots < 2 || (slots & (slots - 1)) || slots < 2ull * cap) return SPCONVB_E_ARG;
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
  if (slots < 2 || (slots & (slots - 1))) return SPCONVB_E_ARG;
  if (!grid_fits(grid, batch)) return SPCONVB_E_RANGE;
  Kernel3 kr;
  for (int a = 0; a < 3; ++a) {
    if (ksize[a] < 1 || !(ksize[a] & 1) || dilation[a] < 1) return SPCONVB_E_ARG;
    kr.k[a] = ksize[a]; kr.d[a] = dilation[a]; kr.s[a] = 1; kr.p[a] = 0;
  }
  const int kvol = ksize[0] * ksize[1] * ksize[2];
  if (kvol > 65535) return SPCONVB_E_ARG;
  if (launch_rows == 0 || launch_rows > cap) launch_rows = cap;
  subm_map_kernel<<<flat_blocks((unsigned long long)launch_rows * kvol), kThreads, 0,
                    (cudaStream_t)stream>>>((const int4*)coords, n_ptr, cap,
                                            make_grid(grid, batch), kr, kvol, table, slots - 1,
                                            map);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

size_t spconvb_down_workspace_bytes(const int32_t out_grid[3], int32_t batch) {
  if (!out_grid || !grid_fits(out_grid, batch)) return 0;
  size_t words = down_words(out_grid, batch);
  size_t blocks = (words + kScanWordsPerBlock - 1) / kScanWordsPerBlock;
  return sizeof(uint32_t) * (2 * words + blocks + 16);
}

int spconvb_down_map(const int32_t* in_coords, const uint32_t* n_in_ptr, uint32_t cap_in,
                     uint32_t launch_rows, const int32_t in_grid[3], int32_t batch,
                     const int32_t ksize[3], const int32_t stride[3], const int32_t pad[3],
                     const int32_t dilation[3], const uint64_t* in_table, uint32_t in_slots,
                     void* workspace, int32_t* out_coords, uint32_t* n_out_ptr, uint32_t cap_out,
                     int32_t* map, uint64_t* out_table, uint32_t out_slots, uint32_t flags,
                     uint32_t* status, void* stream) {
  if (!in_coords || !n_in_ptr || !in_grid || !ksize || !stride || !pad || !dilation ||
      !in_table || !workspace || !out_coords || !n_out_ptr || !map)
    return SPCONVB_E_ARG;
  if (in_slots < 2 || (in_slots & (in_slots - 1))) return SPCONVB_E_ARG;
  if (out_table && (out_slots < 2 || (out_slots & (out_slots - 1)) || out_slots < 2ull * cap_out))
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
  down_mark_kernel<<<flat_blocks((unsigned long long)launch_rows * kvol), kThreads, 0, st>>>(
      (const int4*)in_coords, n_in_ptr, cap_in, gin, gout, kr, kvol, ws.bitmap);
  SPCONVB_LAUNCH_CHECK();
  down_scan_kernel<<<ws.blocks, kScanThreads, 0, st>>>(ws);
  SPCONVB_LAUNCH_CHECK();
  down_emit_kernel<<<ws.blocks, kScanThreads, 0, st>>>(ws, gout, (int4*)out_coords, n_out_ptr,
                                                       cap_out, status);
  SPCONVB_LAUNCH_CHECK();
  down_map_kernel<<<flat_blocks((unsigned long long)cap_out * kvol), kThreads, 0, st>>>(
      (const int4*)out_coords, n_out_ptr, cap_out, gin, gout, kr, kvol, in_table, in_slots - 1, map,
      out_table, out_slots - 1, status);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_down_map_static(const int32_t* in_coords, const uint32_t* n_in_ptr, uint32_t cap_in,
                            uint32_t launch_rows, const int32_t in_grid[3], int32_t batch,
                            const int32_t ksize[3], const int32_t stride[3],
                            const int32_t pad[3], const int32_t dilation[3],
                            const uint64_t* in_table, uint32_t in_slots, int32_t* out_coords,
                            uint32_t* n_out_ptr, uint32_t cap_out, int32_t* map,
                            uint64_t* out_table, uint32_t out_slots, uint32_t flags,
                            uint32_t* status, void* stream) {
  if (!in_grid || !ksize || !stride || !pad || !dilation) return SPCONVB_E_ARG;
  int32_t og[3];
  for (int a = 0; a < 3; ++a) {
    if (ksize[a] < 1 || stride[a] < 1 || dilation[a] < 1 || pad[a] < 0) return SPCONVB_E_ARG;
    og[a] = spconvb_out_extent(in_grid[a], ksize[a], stride[a], pad[a], dilation[a]);
    if (og[a] < 1) return SPCONVB_E_ARG;
  }
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
