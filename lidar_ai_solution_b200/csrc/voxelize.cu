// Point cloud -> voxels (mean of the first P points of every voxel), with a
// result that does not depend on thread scheduling:
//   * the P kept points of a voxel are its P smallest point indices, found with
//     a cascade of atomicMin over P slots (slot s ends up holding the (s+1)-th
//     smallest index), and they are summed in ascending order;
//   * voxel ids are the ranks of the voxels' first points, from a two-level
//     exclusive scan over the points.
// This is what the reference's three kernels compute when points are processed
// one after another; run in parallel they return an arbitrary voxel order and,
// for crowded voxels, an arbitrary subset of points.
#include "common.cuh"

namespace spconvb {

constexpr int kVoxThreads = 256;
constexpr int kVoxScanThreads = 1024;
constexpr uint32_t kNoPoint = 0xffffffffu;

struct VoxWs {
  uint32_t* keys;        // [slots]   key+1, 0 = empty           (zeroed per call)
  uint32_t* counter;     // [4]       number of distinct voxels  (zeroed per call)
  uint32_t* block_sums;  // [blocks]
  uint32_t* vals;        // [slots]   temporary voxel id of a slot
  uint32_t* pslot;       // [points]  slot of a point, kNoPoint if outside
  uint32_t* pprefix;     // [points]  exclusive rank of first points inside a scan block
  uint32_t* kept;        // [max_points][P] smallest point indices (0xFF-filled per call)
  uint32_t slots;
  uint32_t blocks;
};

__host__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

__host__ inline uint32_t vox_slots(uint32_t max_points) {
  uint32_t s = 1024;
  while (s < 2u * max_points && s < 0x80000000u) s <<= 1;
  return s;
}

__host__ inline VoxWs vox_layout(void* base, const spconvb_voxel_params& p, uint32_t max_points,
                                 size_t* zero_bytes, size_t* total_bytes) {
  VoxWs w;
  w.slots = vox_slots(max_points);
  w.blocks = (max_points + kVoxScanThreads - 1) / kVoxScanThreads;
  if (w.blocks < 1) w.blocks = 1;
  uint8_t* b = (uint8_t*)base;
  size_t off = 0;
  w.keys = (uint32_t*)(b + off); off += align_up(sizeof(uint32_t) * (size_t)w.slots, 256);
  w.counter = (uint32_t*)(b + off); off += 256;
  if (zero_bytes) *zero_bytes = off;
  w.block_sums = (uint32_t*)(b + off); off += align_up(sizeof(uint32_t) * (size_t)w.blocks, 256);
  w.vals = (uint32_t*)(b + off); off += align_up(sizeof(uint32_t) * (size_t)w.slots, 256);
  w.pslot = (uint32_t*)(b + off); off += align_up(sizeof(uint32_t) * (size_t)max_points, 256);
  w.pprefix = (uint32_t*)(b + off); off += align_up(sizeof(uint32_t) * (size_t)max_points, 256);
  w.kept = (uint32_t*)(b + off);
  off += align_up(sizeof(uint32_t) * (size_t)max_points * p.max_points_per_voxel, 256);
  if (total_bytes) *total_bytes = off;
  return w;
}

__device__ __forceinline__ float point_feat(const void* points, int kind, size_t i) {
  return kind ? __half2float(((const __half*)points)[i]) : ((const float*)points)[i];
}

// Pass 1: insert the voxel key of every in-range point; the inserting thread
// draws a temporary id for the voxel.
__global__ void vox_hash_kernel(const void* __restrict__ points, uint32_t n,
                                spconvb_voxel_params p, VoxWs w, uint32_t* status) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float px = point_feat(points, p.points_kind, (size_t)i * p.num_features);
  const float py = point_feat(points, p.points_kind, (size_t)i * p.num_features + 1);
  const float pz = point_feat(points, p.points_kind, (size_t)i * p.num_features + 2);
  uint32_t slot = kNoPoint;
  if (px >= p.range_min[0] && px < p.range_max[0] && py >= p.range_min[1] &&
      py < p.range_max[1] && pz >= p.range_min[2] && pz < p.range_max[2]) {
    const int vx = (int)floorf(__fdiv_rn(__fsub_rn(px, p.range_min[0]), p.voxel_size[0]));
    const int vy = (int)floorf(__fdiv_rn(__fsub_rn(py, p.range_min[1]), p.voxel_size[1]));
    const int vz = (int)floorf(__fdiv_rn(__fsub_rn(pz, p.range_min[2]), p.voxel_size[2]));
    if (vx >= 0 && vx < p.grid[0] && vy >= 0 && vy < p.grid[1] && vz >= 0 && vz < p.grid[2]) {
      const uint32_t key = ((uint32_t)vz * p.grid[1] + vy) * p.grid[0] + vx;
      const uint32_t mask = w.slots - 1;
      uint32_t s = hash32(key) & mask;
      for (uint32_t probe = 0; probe <= mask; ++probe) {
        const uint32_t old = atomicCAS(w.keys + s, 0u, key + 1u);
        if (old == 0u) {
          w.vals[s] = atomicAdd(w.counter, 1u);
          slot = s;
          break;
        }
        if (old == key + 1u) {
          slot = s;
          break;
        }
        s = (s + 1) & mask;
      }
      if (slot == kNoPoint) set_status(status, SPCONVB_ST_HASH_FULL, i);
    }
  }
  w.pslot[i] = slot;
}

// Pass 2: keep the P smallest point indices of every voxel.
__global__ void vox_collect_kernel(uint32_t n, int P, VoxWs w) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t slot = w.pslot[i];
  if (slot == kNoPoint) return;
  uint32_t* k = w.kept + (size_t)w.vals[slot] * P;
  uint32_t v = i;
  for (int s = 0; s < P; ++s) {
    const uint32_t old = atomicMin(k + s, v);
    v = max(old, v);
    if (v == kNoPoint) break;
  }
}

// Pass 3: rank the first points (exclusive scan inside a block of 1024 points).
__global__ void __launch_bounds__(kVoxScanThreads)
vox_scan_kernel(uint32_t n, int P, VoxWs w) {
  __shared__ uint32_t warp_sums[32];
  const uint32_t i = blockIdx.x * kVoxScanThreads + threadIdx.x;
  uint32_t flag = 0;
  if (i < n) {
    const uint32_t slot = w.pslot[i];
    if (slot != kNoPoint) flag = (w.kept[(size_t)w.vals[slot] * P] == i) ? 1u : 0u;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t ballot = __ballot_sync(0xffffffffu, flag);
  const uint32_t in_warp = __popc(ballot & ((1u << lane) - 1u));
  if (lane == 0) warp_sums[warp] = __popc(ballot);
  __syncthreads();
  if (warp == 0) {
    const uint32_t v = warp_sums[lane];
    uint32_t s = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += t;
    }
    warp_sums[lane] = s - v;
    if (lane == 31) w.block_sums[blockIdx.x] = s;
  }
  __syncthreads();
  if (i < n) w.pprefix[i] = flag ? warp_sums[warp] + in_warp : kNoPoint;
}

// Pass 4: the first point of a voxel writes the voxel: its index and the mean
// of the kept points, summed in ascending point order in fp32.
__global__ void __launch_bounds__(kVoxScanThreads)
vox_emit_kernel(const void* __restrict__ points, uint32_t n, spconvb_voxel_params p, VoxWs w,
                __half* __restrict__ features, int4* __restrict__ indices,
                uint32_t* n_voxels_ptr, uint32_t* status) {
  __shared__ uint32_t red[32];
  __shared__ uint32_t s_base;
  uint32_t part = 0;
  for (uint32_t b = threadIdx.x; b < blockIdx.x; b += blockDim.x) part += w.block_sums[b];
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
        const uint32_t total = v + w.block_sums[blockIdx.x];
        if (total > (uint32_t)p.max_voxels) set_status(status, SPCONVB_ST_OVERFLOW, total);
        *n_voxels_ptr = min(total, (uint32_t)p.max_voxels);
      }
    }
  }
  __syncthreads();
  const uint32_t i = blockIdx.x * kVoxScanThreads + threadIdx.x;
  if (i >= n) return;
  const uint32_t pre = w.pprefix[i];
  if (pre == kNoPoint) return;
  const uint32_t id = s_base + pre;
  if (id >= (uint32_t)p.max_voxels) return;
  const int P = p.max_points_per_voxel, F = p.num_features;
  const uint32_t* k = w.kept + (size_t)w.vals[w.pslot[i]] * P;
  float sum[8];
#pragma unroll
  for (int f = 0; f < 8; ++f) sum[f] = 0.f;
  int cnt = 0;
  for (int s = 0; s < P; ++s) {
    const uint32_t q = k[s];
    if (q == kNoPoint) break;
    ++cnt;
    for (int f = 0; f < F; ++f)
      sum[f] = __fadd_rn(sum[f], point_feat(points, p.points_kind, (size_t)q * F + f));
  }
  for (int f = 0; f < F; ++f)
    features[(size_t)id * F + f] = __float2half_rn(__fdiv_rn(sum[f], (float)cnt));
  const float px = point_feat(points, p.points_kind, (size_t)i * F);
  const float py = point_feat(points, p.points_kind, (size_t)i * F + 1);
  const float pz = point_feat(points, p.points_kind, (size_t)i * F + 2);
  const int vx = (int)floorf(__fdiv_rn(__fsub_rn(px, p.range_min[0]), p.voxel_size[0]));
  const int vy = (int)floorf(__fdiv_rn(__fsub_rn(py, p.range_min[1]), p.voxel_size[1]));
  const int vz = (int)floorf(__fdiv_rn(__fsub_rn(pz, p.range_min[2]), p.voxel_size[2]));
  indices[id] = p.order == 0 ? make_int4(0, vz, vy, vx) : make_int4(0, vx, vy, vz);
}

}  // namespace spconvb

using namespace spconvb;

extern "C" {

size_t spconvb_voxelize_workspace_bytes(const spconvb_voxel_params* p, uint32_t max_points) {
  if (!p || max_points < 1 || p->max_points_per_voxel < 1) return 0;
  size_t total = 0;
  vox_layout(nullptr, *p, max_points, nullptr, &total);
  return total;
}

int spconvb_voxelize(const spconvb_voxel_params* p, const void* points, uint32_t num_points,
                     void* workspace, void* features, int32_t* indices, uint32_t* n_voxels_ptr,
                     uint32_t* status, void* stream) {
  if (!p || !points || !workspace || !features || !indices || !n_voxels_ptr)
    return SPCONVB_E_ARG;
  if (p->num_features < 3 || p->num_features > 8 || p->max_points_per_voxel < 1 ||
      p->max_points_per_voxel > 16 || p->max_voxels < 1)
    return SPCONVB_E_ARG;
  unsigned long long cells = (unsigned long long)p->grid[0] * p->grid[1] * p->grid[2];
  if (p->grid[0] < 1 || p->grid[1] < 1 || p->grid[2] < 1 || cells >= 0xffffffffull)
    return SPCONVB_E_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (num_points == 0) {
    SPCONVB_CUDA_TRY(cudaMemsetAsync(n_voxels_ptr, 0, sizeof(uint32_t), st));
    return SPCONVB_OK;
  }
  size_t zero_bytes = 0, total = 0;
  VoxWs w = vox_layout(workspace, *p, num_points, &zero_bytes, &total);
  SPCONVB_CUDA_TRY(cudaMemsetAsync(workspace, 0, zero_bytes, st));
  SPCONVB_CUDA_TRY(cudaMemsetAsync(
      w.kept, 0xFF, sizeof(uint32_t) * (size_t)num_points * p->max_points_per_voxel, st));
  const int blocks = (num_points + kVoxThreads - 1) / kVoxThreads;
  vox_hash_kernel<<<blocks, kVoxThreads, 0, st>>>(points, num_points, *p, w, status);
  SPCONVB_LAUNCH_CHECK();
  vox_collect_kernel<<<blocks, kVoxThreads, 0, st>>>(num_points, p->max_points_per_voxel, w);
  SPCONVB_LAUNCH_CHECK();
  vox_scan_kernel<<<w.blocks, kVoxScanThreads, 0, st>>>(num_points, p->max_points_per_voxel, w);
  SPCONVB_LAUNCH_CHECK();
  vox_emit_kernel<<<w.blocks, kVoxScanThreads, 0, st>>>(points, num_points, *p, w,
                                                        (__half*)features, (int4*)indices,
                                                        n_voxels_ptr, status);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

}  // extern "C"
