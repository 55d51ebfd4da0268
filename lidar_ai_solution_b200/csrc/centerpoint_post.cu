// CenterPoint head decode + rotated-box NMS, entirely on the device.
//
// Stage replaced: PostProcessCuda and the per-task host loop of CUDA-CenterPoint
// (src/postprocess_kernels.cu:28-403, src/centerpoint.cpp:163-216), which per task copies the
// candidate list to the host, sorts it there, copies it back, copies the suppression mask to
// the host and scans it there: three stream synchronisations per task, six tasks per frame.
//
// Here one call enqueues four kernels for all tasks together (blockIdx selects the task):
//   candidates  one thread per heat-map cell: class arg-max of the sigmoid, score and centre
//               range filters; survivors append a 64-bit key (score bits | cell | label)
//   rank        one CTA per task: if more than 1024 candidates, an 8-pass radix select finds
//               the max_det largest keys; a bitonic sort in shared memory orders them; the
//               box parameters (exp, atan2) are evaluated for the ranked cells only
//   mask        pairwise rotated IoU >= threshold above the diagonal, in tiles of 16 x 64
//               pairs: a reach test queues the pairs that can overlap, then the queue is
//               spread over full warps; corners and the trigonometry of every box are
//               prepared once by the rank kernel
//   scan        one warp per task walks the ranking with the mask in shared memory and keeps
//               the first nms_post_max survivors; the last CTA to finish packs all tasks'
//               boxes into the caller's list
//
// This file is compiled without multiply-add contraction so that every product and sum rounds
// as in the reference's expression order on a CPU; only the library functions (expf, sinf,
// cosf, atan2f) may differ from a host libm by a few ulp.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"
#include "spconvb.h"
#include "spconvb_centerpoint.h"

namespace spconvb {
namespace {

constexpr int kDet = 11;         // floats per detection
constexpr int kBoxStride = 16;   // floats per prepared NMS box (struct BoxRec)
constexpr int kRankThreads = 1024;
constexpr int kMaskWords = 16;   // 64-bit words per mask row: 1024 / 64
constexpr int kScanStagedRows = 320;  // mask rows the scan keeps in shared memory (40 KB)

struct TaskBuffers {
  uint32_t* n_cand;
  uint32_t* n_det;
  uint32_t* n_kept;
  unsigned long long* cand;  // [H*W]
  float* det;                // [max_det][11]
  float* box;                // [max_det][16], BoxRec
  unsigned long long* mask;  // [max_det][16]
  float* kept;               // [post_max][11]
};

struct PostArgs {
  spconvb_cp_head head[SPCONVB_CP_MAX_TASKS];
  TaskBuffers buf[SPCONVB_CP_MAX_TASKS];
  spconvb_cp_params p;
  int num_tasks;
  uint32_t* ticket;
  float* out_boxes;
  uint32_t* out_count;
};

struct Layout {
  size_t counters_bytes;  // zeroed before every call
  size_t per_task;
  size_t cand, det, box, mask, kept;
  size_t total;
};

__host__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

__host__ Layout layout_of(const spconvb_cp_params& p, int tasks) {
  Layout l{};
  l.counters_bytes = align_up(sizeof(uint32_t) * (1 + 3 * (size_t)SPCONVB_CP_MAX_TASKS), 256);
  size_t off = 0;
  l.cand = off; off += align_up(sizeof(unsigned long long) * (size_t)p.H * p.W, 256);
  l.det = off;  off += align_up(sizeof(float) * kDet * (size_t)p.max_det, 256);
  l.box = off;  off += align_up(sizeof(float) * kBoxStride * (size_t)p.max_det, 256);
  l.mask = off; off += align_up(sizeof(unsigned long long) * kMaskWords * (size_t)p.max_det, 256);
  l.kept = off; off += align_up(sizeof(float) * kDet * (size_t)p.nms_post_max, 256);
  l.per_task = off;
  l.total = l.counters_bytes + l.per_task * (size_t)tasks;
  return l;
}

__host__ void bind_buffers(const Layout& l, void* workspace, int tasks, PostArgs& a) {
  char* base = (char*)workspace;
  uint32_t* counters = (uint32_t*)base;
  a.ticket = counters;
  for (int t = 0; t < tasks; ++t) {
    char* tb = base + l.counters_bytes + l.per_task * (size_t)t;
    a.buf[t].n_cand = counters + 1 + 3 * t;
    a.buf[t].n_det = counters + 2 + 3 * t;
    a.buf[t].n_kept = counters + 3 + 3 * t;
    a.buf[t].cand = (unsigned long long*)(tb + l.cand);
    a.buf[t].det = (float*)(tb + l.det);
    a.buf[t].box = (float*)(tb + l.box);
    a.buf[t].mask = (unsigned long long*)(tb + l.mask);
    a.buf[t].kept = (float*)(tb + l.kept);
  }
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float ldh(const void* p, int i) {
  return __half2float(((const __half*)p)[i]);
}

// ------------------------------------------------------------------ candidates
__global__ void cp_candidates_kernel(const PostArgs a) {
  const int task = blockIdx.y;
  const spconvb_cp_head& hd = a.head[task];
  const int HW = a.p.H * a.p.W;
  const int cell = blockIdx.x * blockDim.x + threadIdx.x;
  if (cell >= HW) return;
  const int h = cell / a.p.W, w = cell % a.p.W;
  int label = 0;
  float score = sigmoid_f(ldh(hd.hm, cell));
  for (int c = 1; c < hd.num_classes; ++c) {
    const float s = sigmoid_f(ldh(hd.hm, c * HW + cell));
    if (s > score) {
      score = s;
      label = c;
    }
  }
  if (score < a.p.score_threshold) return;
  float xs = ldh(hd.reg, cell) + (float)w;
  float ys = ldh(hd.reg, HW + cell) + (float)h;
  xs = xs * a.p.out_size_factor * a.p.voxel_size[0] + a.p.pc_range[0];
  ys = ys * a.p.out_size_factor * a.p.voxel_size[1] + a.p.pc_range[1];
  const float zs = ldh(hd.height, cell);
  const float* r = a.p.post_center_range;
  if (xs < r[0] || xs > r[3] || ys < r[1] || ys > r[4] || zs < r[2] || zs > r[5]) return;
  // positive floats order like their bit patterns; a smaller cell index ranks first on ties
  const unsigned long long key = ((unsigned long long)__float_as_uint(score) << 32) |
                                 ((unsigned long long)(0xFFFFFFu - (uint32_t)cell) << 8) |
                                 (unsigned long long)label;
  const uint32_t slot = atomicAdd(a.buf[task].n_cand, 1u);
  a.buf[task].cand[slot] = key;  // at most one key per cell, so slot < H*W
}

// ------------------------------------------------------------------ rotated overlap
struct Pt { float x, y; };

// A box as the overlap test wants it: centre, extents, the rotation by -angle used by the
// corner-inside-box test, and the four corners turned by +angle about the centre.
struct BoxRec {
  float x, y, dx, dy;
  float cos_neg, sin_neg;
  Pt corner[4];
  float angle, reach;  // reach: half the diagonal, the farthest any point of the box is from its centre
};
static_assert(sizeof(BoxRec) == sizeof(float) * kBoxStride, "BoxRec layout");

__device__ __forceinline__ void prepare_box(const float* box, BoxRec& r) {
  r.x = box[0]; r.y = box[1]; r.dx = box[3]; r.dy = box[4];
  r.angle = box[6];
  r.reach = 0.5f * sqrtf(box[3] * box[3] + box[4] * box[4]);
  r.cos_neg = cosf(-box[6]);
  r.sin_neg = sinf(-box[6]);
  const float hx = box[3] / 2, hy = box[4] / 2;
  const float x1 = box[0] - hx, y1 = box[1] - hy, x2 = box[0] + hx, y2 = box[1] + hy;
  const float co = cosf(box[6]), si = sinf(box[6]);
  const float rx[4] = {x1, x2, x2, x1}, ry[4] = {y1, y1, y2, y2};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    r.corner[k].x = (rx[k] - box[0]) * co + (ry[k] - box[1]) * (-si) + box[0];
    r.corner[k].y = (rx[k] - box[0]) * si + (ry[k] - box[1]) * co + box[1];
  }
}

__device__ __forceinline__ float cross3(Pt p1, Pt p2, Pt p0) {
  return (p1.x - p0.x) * (p2.y - p0.y) - (p2.x - p0.x) * (p1.y - p0.y);
}

__device__ __forceinline__ bool inside_with_margin(const BoxRec& box, Pt p) {
  const float margin = 1e-2f;
  const float rx = (p.x - box.x) * box.cos_neg + (p.y - box.y) * (-box.sin_neg);
  const float ry = (p.x - box.x) * box.sin_neg + (p.y - box.y) * box.cos_neg;
  return fabsf(rx) < box.dx / 2 + margin && fabsf(ry) < box.dy / 2 + margin;
}

__device__ __forceinline__ bool segments_cross(Pt p1, Pt p0, Pt q1, Pt q0, Pt& ans) {
  if (!(fminf(p0.x, p1.x) <= fmaxf(q0.x, q1.x) && fminf(q0.x, q1.x) <= fmaxf(p0.x, p1.x) &&
        fminf(p0.y, p1.y) <= fmaxf(q0.y, q1.y) && fminf(q0.y, q1.y) <= fmaxf(p0.y, p1.y)))
    return false;
  const float s1 = cross3(q0, p1, p0);
  const float s2 = cross3(p1, q1, p0);
  const float s3 = cross3(p0, q1, q0);
  const float s4 = cross3(q1, p1, q0);
  if (!(s1 * s2 > 0 && s3 * s4 > 0)) return false;
  const float s5 = cross3(q1, p1, p0);
  if ((double)fabsf(s5 - s1) > 1e-8) {
    ans.x = (s5 * q0.x - s1 * q1.x) / (s5 - s1);
    ans.y = (s5 * q0.y - s1 * q1.y) / (s5 - s1);
  } else {
    const float a0 = p0.y - p1.y, b0 = p1.x - p0.x, c0 = p0.x * p1.y - p1.x * p0.y;
    const float a1 = q0.y - q1.y, b1 = q1.x - q0.x, c1 = q0.x * q1.y - q1.x * q0.y;
    const float D = a0 * b1 - a1 * b0;
    ans.x = (b0 * c1 - b1 * c0) / D;
    ans.y = (a1 * c0 - a0 * c1) / D;
  }
  return true;
}

__device__ float rotated_iou(const BoxRec& A, const BoxRec& B) {
  // Boxes farther apart than their reaches (plus far more than the 1e-2 margin of the corner
  // test and any rounding) share no edge crossing and no corner: the full computation below
  // would find no point and return 0 as well.
  {
    const float ddx = A.x - B.x, ddy = A.y - B.y, far = A.reach + B.reach + 0.1f;
    if (ddx * ddx + ddy * ddy > far * far) return 0.f;
  }
  Pt pts[16];
  float ang[16];
  int cnt = 0;
  Pt centre = {0.f, 0.f};
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      Pt x;
      if (segments_cross(A.corner[(i + 1) & 3], A.corner[i], B.corner[(j + 1) & 3], B.corner[j], x)) {
        centre.x = centre.x + x.x;
        centre.y = centre.y + x.y;
        pts[cnt++] = x;
      }
    }
  for (int k = 0; k < 4; ++k) {
    if (inside_with_margin(A, B.corner[k])) {
      centre.x = centre.x + B.corner[k].x;
      centre.y = centre.y + B.corner[k].y;
      pts[cnt++] = B.corner[k];
    }
    if (inside_with_margin(B, A.corner[k])) {
      centre.x = centre.x + A.corner[k].x;
      centre.y = centre.y + A.corner[k].y;
      pts[cnt++] = A.corner[k];
    }
  }
  if (cnt == 0) return 0.f;
  centre.x /= (float)cnt;
  centre.y /= (float)cnt;
  // stable ascending order of the polar angle about the centre
  for (int k = 0; k < cnt; ++k) ang[k] = atan2f(pts[k].y - centre.y, pts[k].x - centre.x);
  for (int k = 1; k < cnt; ++k) {
    const Pt p = pts[k];
    const float ak = ang[k];
    int j = k - 1;
    while (j >= 0 && ang[j] > ak) {
      pts[j + 1] = pts[j];
      ang[j + 1] = ang[j];
      --j;
    }
    pts[j + 1] = p;
    ang[j + 1] = ak;
  }
  float area = 0.f;
  for (int k = 0; k + 1 < cnt; ++k) {
    const float ax = pts[k].x - pts[0].x, ay = pts[k].y - pts[0].y;
    const float bx = pts[k + 1].x - pts[0].x, by = pts[k + 1].y - pts[0].y;
    area += ax * by - ay * bx;
  }
  const float overlap = fabsf(area) / 2.0f;
  const float sa = A.dx * A.dy, sb = B.dx * B.dy;
  return overlap / fmaxf(sa + sb - overlap, 1e-8f);
}

__global__ void rotated_iou_pairs_kernel(const float* a, const float* b, int n, float* iou) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  BoxRec A, B;
  prepare_box(a + (size_t)i * 7, A);
  prepare_box(b + (size_t)i * 7, B);
  iou[i] = rotated_iou(A, B);
}

__device__ __forceinline__ void load_box(const float* p, BoxRec& r) {
  float4* d = (float4*)&r;
  const float4* s4 = (const float4*)p;
#pragma unroll
  for (int k = 0; k < 4; ++k) d[k] = s4[k];
}

// ------------------------------------------------------------------ rank
__global__ void __launch_bounds__(kRankThreads) cp_rank_kernel(const PostArgs a) {
  const int task = blockIdx.x;
  const TaskBuffers& b = a.buf[task];
  const spconvb_cp_head& hd = a.head[task];
  const int HW = a.p.H * a.p.W;
  const int tid = threadIdx.x;
  __shared__ unsigned long long keys[kRankThreads];
  __shared__ uint32_t hist[256];
  __shared__ unsigned long long s_prefix;
  __shared__ uint32_t s_need, s_fill;

  const uint32_t n = min(*b.n_cand, (uint32_t)HW);
  const uint32_t K = min(n, (uint32_t)a.p.max_det);
  keys[tid] = 0ull;
  if (n <= (uint32_t)kRankThreads) {
    if ((uint32_t)tid < n) keys[tid] = b.cand[tid];
    __syncthreads();
  } else {
    // the K-th largest key, most significant byte first (keys are distinct)
    if (tid == 0) { s_prefix = 0ull; s_need = K; s_fill = 0u; }
    for (int shift = 56; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0u;
      __syncthreads();
      const unsigned long long prefix = s_prefix;
      const unsigned long long hi = shift == 56 ? 0ull : (~0ull << (shift + 8));
      for (uint32_t base = 0; base < n; base += kRankThreads) {
        // keys of one score share their upper bytes: lanes with the same digit add once
        const uint32_t i = base + tid;
        const unsigned long long k = i < n ? b.cand[i] : 0ull;
        const bool live = i < n && ((k ^ prefix) & hi) == 0ull;
        const uint32_t digit = live ? ((uint32_t)(k >> shift) & 255u) : 256u;
        const uint32_t peers = __match_any_sync(0xffffffffu, digit);
        if (live && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
      }
      __syncthreads();
      if (tid < 32) {
        // lane l owns bins 8l..8l+7; the digit is the highest bin whose count, together with
        // everything above it, reaches what is still needed
        uint32_t mine[8], sum = 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k) { mine[k] = hist[tid * 8 + k]; sum += mine[k]; }
        uint32_t incl = sum;  // becomes the count in this lane's bins and in all higher lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const uint32_t v = __shfl_down_sync(0xffffffffu, incl, d);
          if (tid + d < 32) incl += v;
        }
        const uint32_t above = incl - sum;
        const uint32_t need = s_need;
        const bool here = above < need && incl >= need;  // exactly one lane
        if (here) {
          uint32_t acc = above;
          int k = 7;
          for (; k > 0; --k) {
            if (acc + mine[k] >= need) break;
            acc += mine[k];
          }
          s_need = need - acc;
          s_prefix = prefix | ((unsigned long long)(tid * 8 + k) << shift);
        }
      }
      __syncthreads();
    }
    const unsigned long long kth = s_prefix;
    for (uint32_t i = tid; i < n; i += kRankThreads) {
      const unsigned long long k = b.cand[i];
      if (k >= kth) {
        const uint32_t pos = atomicAdd(&s_fill, 1u);
        if (pos < (uint32_t)kRankThreads) keys[pos] = k;
      }
    }
    __syncthreads();
  }

  // bitonic sort, descending (padding keys are 0 and end up last)
  const int filled = n <= (uint32_t)kRankThreads ? (int)n : (int)K;  // keys beyond are zero padding
  int sort_n = 32;
  while (sort_n < filled) sort_n <<= 1;
  for (int size = 2; size <= sort_n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int partner = tid ^ stride;
      if (partner > tid && partner < sort_n) {
        const unsigned long long x = keys[tid], y = keys[partner];
        const bool descending = (tid & size) == 0;
        if ((x < y) == descending) { keys[tid] = y; keys[partner] = x; }
      }
      __syncthreads();
    }
  }

  if (tid == 0) *b.n_det = K;
  if ((uint32_t)tid >= K) return;
  const unsigned long long key = keys[tid];
  const int cell = (int)(0xFFFFFFu - (uint32_t)((key >> 8) & 0xFFFFFFull));
  const int label = (int)(key & 0xFFull);
  const float score = __uint_as_float((uint32_t)(key >> 32));
  const int h = cell / a.p.W, w = cell % a.p.W;
  float xs = ldh(hd.reg, cell) + (float)w;
  float ys = ldh(hd.reg, HW + cell) + (float)h;
  xs = xs * a.p.out_size_factor * a.p.voxel_size[0] + a.p.pc_range[0];
  ys = ys * a.p.out_size_factor * a.p.voxel_size[1] + a.p.pc_range[1];
  const float zs = ldh(hd.height, cell);
  const float dx = expf(ldh(hd.dim, cell));
  const float dy = expf(ldh(hd.dim, HW + cell));
  const float dz = expf(ldh(hd.dim, 2 * HW + cell));
  const float vx = ldh(hd.vel, cell), vy = ldh(hd.vel, HW + cell);
  const float rs = atan2f(ldh(hd.rot, cell), ldh(hd.rot, HW + cell));
  float* d = b.det + (size_t)tid * kDet;
  d[0] = xs; d[1] = ys; d[2] = zs; d[3] = dx; d[4] = dy; d[5] = dz;
  d[6] = vx; d[7] = vy; d[8] = rs; d[9] = (float)label; d[10] = score;
  // the box NMS sees: length and width swapped, yaw turned into the lidar frame
  const float nms_box[7] = {xs, ys, zs, dy, dx, dz, (float)(-(double)rs - 3.141592653 * 0.5)};
  prepare_box(nms_box, *(BoxRec*)(b.box + (size_t)tid * kBoxStride));
}

// ------------------------------------------------------------------ mask
constexpr int kMaskRows = 16;          // ranked boxes per tile; divides 64, so a tile's rows share a word
constexpr int kMaskCtasPerTask = 148;
constexpr int kMaskThreads = 128;

// One tile = 16 rows x 64 partners.  Pass 1: every thread tests 8 pairs for reach (three floats
// per box, staged in shared memory) and queues the few that can overlap.  Pass 2: the queued
// pairs are spread over the threads one by one, so the long overlap computation runs with full
// warps instead of one lane in 32.
__global__ void __launch_bounds__(kMaskThreads) cp_mask_kernel(const PostArgs a) {
  const int task = blockIdx.y;
  const TaskBuffers& b = a.buf[task];
  const int m = (int)*b.n_det;
  const int tid = threadIdx.x;
  __shared__ float col_x[64], col_y[64], col_r[64], row_x[kMaskRows], row_y[kMaskRows], row_r[kMaskRows];
  __shared__ unsigned long long words[kMaskRows];
  __shared__ uint16_t queue[kMaskRows * 64];
  __shared__ uint32_t queued;
  const int col_blocks = (m + 63) / 64, row_groups = (m + kMaskRows - 1) / kMaskRows;
  for (int tile = blockIdx.x; tile < col_blocks * row_groups; tile += gridDim.x) {
    const int row0 = (tile / col_blocks) * kMaskRows, col0 = (tile % col_blocks) * 64;
    if (col0 / 64 < row0 / 64) continue;  // left of the diagonal: never read
    __syncthreads();                      // the previous tile's shared state is no longer needed
    if (tid < 64) {
      const BoxRec* r = (const BoxRec*)(b.box + (size_t)min(col0 + tid, m - 1) * kBoxStride);
      col_x[tid] = r->x; col_y[tid] = r->y; col_r[tid] = r->reach;
    } else if (tid < 64 + kMaskRows) {
      const int k = tid - 64;
      const BoxRec* r = (const BoxRec*)(b.box + (size_t)min(row0 + k, m - 1) * kBoxStride);
      row_x[k] = r->x; row_y[k] = r->y; row_r[k] = r->reach;
      words[k] = 0ull;
    } else if (tid == 64 + kMaskRows) {
      queued = 0u;
    }
    __syncthreads();
    for (int pair = tid; pair < kMaskRows * 64; pair += kMaskThreads) {
      const int r = pair >> 6, c = pair & 63;
      const int i = row0 + r, j = col0 + c;
      if (i >= m || j >= m || j <= i) continue;
      const float ddx = row_x[r] - col_x[c], ddy = row_y[r] - col_y[c];
      const float far = row_r[r] + col_r[c] + 0.1f;
      if (ddx * ddx + ddy * ddy > far * far) continue;  // the same test rotated_iou starts with
      queue[atomicAdd(&queued, 1u)] = (uint16_t)pair;
    }
    __syncthreads();
    const uint32_t n_pairs = queued;
    for (uint32_t q = tid; q < n_pairs; q += kMaskThreads) {
      const int pair = queue[q], r = pair >> 6, c = pair & 63;
      BoxRec A, B;
      load_box(b.box + (size_t)(row0 + r) * kBoxStride, A);
      load_box(b.box + (size_t)(col0 + c) * kBoxStride, B);
      if (rotated_iou(A, B) >= a.p.nms_iou_threshold) atomicOr(&words[r], 1ull << c);
    }
    __syncthreads();
    if (tid < kMaskRows && row0 + tid < m)
      b.mask[(size_t)(row0 + tid) * kMaskWords + col0 / 64] = words[tid];
  }
}

// ------------------------------------------------------------------ scan
__global__ void __launch_bounds__(512) cp_scan_kernel(const PostArgs a) {
  __shared__ __align__(16) unsigned long long s_mask[kScanStagedRows * kMaskWords];
  __shared__ bool s_last;
  __shared__ int s_kept[kRankThreads];
  __shared__ uint32_t s_nkept;
  const int task = blockIdx.x;
  const TaskBuffers& b = a.buf[task];
  const int m = (int)*b.n_det;
  const int words = (m + 63) / 64;
  // The walk usually ends (nms_post_max survivors) within the first few hundred boxes: those
  // rows are staged in shared memory, later ones are read from global memory when needed.
  const int staged = min(m, kScanStagedRows);
  {
    // 16-byte loads issued back to back; words left of the diagonal tile and right of the last
    // box were never written and are zeroed here
    const ulonglong2* src = (const ulonglong2*)b.mask;
    ulonglong2* dst = (ulonglong2*)s_mask;
    const int vecs = staged * (kMaskWords / 2);
#pragma unroll 5
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      ulonglong2 x = src[v];
      const int row = v / (kMaskWords / 2), wd = (v % (kMaskWords / 2)) * 2;
      if (wd < row / 64 || wd >= words) x.x = 0ull;
      if (wd + 1 < row / 64 || wd + 1 >= words) x.y = 0ull;
      dst[v] = x;
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    unsigned long long removed = 0ull;  // lane w holds word w of the removed set
    uint32_t kept = 0;
    // Word by word: the lowest ranked box of the word that nobody has removed survives, its
    // mask row joins the removed set, and so on; removed boxes cost nothing.  Boxes after the
    // first nms_post_max survivors cannot reach the output.
    for (int w = 0; w < words && kept < (uint32_t)a.p.nms_post_max; ++w) {
      const unsigned long long valid =
          (w == words - 1 && (m & 63)) ? ((1ull << (m & 63)) - 1ull) : ~0ull;
      while (kept < (uint32_t)a.p.nms_post_max) {
        const unsigned long long alive = ~__shfl_sync(0xffffffffu, removed, w) & valid;
        if (alive == 0ull) break;
        const int bit = __ffsll((long long)alive) - 1;
        const int i = w * 64 + bit;
        if (lane == 0) s_kept[kept] = i;
        ++kept;
        if (lane == w) removed |= 1ull << bit;  // done with this box
        if (lane < kMaskWords) {
          if (i < staged) removed |= s_mask[i * kMaskWords + lane];
          else if (lane >= w && lane < words) removed |= b.mask[(size_t)i * kMaskWords + lane];
        }
      }
    }
    if (lane == 0) {
      s_nkept = kept;
      *b.n_kept = kept;
    }
  }
  __syncthreads();
  for (uint32_t e = threadIdx.x; e < s_nkept * kDet; e += blockDim.x) {
    const uint32_t k = e / kDet, f = e % kDet;
    float v = b.det[(size_t)s_kept[k] * kDet + f];
    if (f == 9) v = (float)(a.head[task].label_offset + (int)v);
    b.kept[e] = v;
  }
  __threadfence();  // every thread's rows are visible device-wide before the ticket is taken
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(a.ticket, 1u) == (uint32_t)(a.num_tasks - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the last task to finish packs every task's boxes into the caller's list, in task order
  uint32_t count[SPCONVB_CP_MAX_TASKS], base = 0;
#pragma unroll
  for (int t = 0; t < SPCONVB_CP_MAX_TASKS; ++t)
    count[t] = t < a.num_tasks ? __ldcg(a.buf[t].n_kept) : 0u;
#pragma unroll
  for (int t = 0; t < SPCONVB_CP_MAX_TASKS; ++t) {
    for (uint32_t i = threadIdx.x; i < count[t] * kDet; i += blockDim.x)
      a.out_boxes[(size_t)base * kDet + i] = __ldcg(a.buf[t].kept + i);
    base += count[t];
  }
  if (threadIdx.x == 0) *a.out_count = base;
}

bool params_ok(const spconvb_cp_params* p) {
  return p && p->H >= 1 && p->W >= 1 && (size_t)p->H * p->W <= 0xFFFFFFu && p->max_det >= 1 &&
         p->max_det <= kRankThreads && p->nms_post_max >= 1 && p->nms_post_max <= p->max_det;
}

}  // namespace
}  // namespace spconvb

using namespace spconvb;

extern "C" {

void spconvb_cp_default_params(spconvb_cp_params* p) {
  if (!p) return;
  p->H = 180; p->W = 180;
  p->out_size_factor = 8.f;
  p->voxel_size[0] = p->voxel_size[1] = 0.075f;
  p->pc_range[0] = p->pc_range[1] = -54.f;
  p->score_threshold = 0.1f;
  const float r[6] = {-61.2f, -61.2f, -10.0f, 61.2f, 61.2f, 10.0f};
  for (int i = 0; i < 6; ++i) p->post_center_range[i] = r[i];
  p->nms_iou_threshold = 0.2f;
  p->max_det = 1000;
  p->nms_post_max = 83;
}

size_t spconvb_cp_workspace_bytes(const spconvb_cp_params* p, int32_t num_tasks) {
  if (!params_ok(p) || num_tasks < 1 || num_tasks > SPCONVB_CP_MAX_TASKS) return 0;
  return layout_of(*p, num_tasks).total;
}

int spconvb_cp_postprocess(const spconvb_cp_head* heads, int32_t num_tasks,
                           const spconvb_cp_params* p, void* workspace, size_t workspace_bytes,
                           float* out_boxes, uint32_t* out_count, void* stream) {
  if (!heads || !params_ok(p) || !workspace || !out_boxes || !out_count || num_tasks < 1 ||
      num_tasks > SPCONVB_CP_MAX_TASKS || ((uintptr_t)workspace & 255u))
    return SPCONVB_E_ARG;
  const Layout l = layout_of(*p, num_tasks);
  if (workspace_bytes < l.total) return SPCONVB_E_NOMEM;
  PostArgs a{};
  for (int t = 0; t < num_tasks; ++t) {
    const spconvb_cp_head& h = heads[t];
    if (!h.reg || !h.height || !h.dim || !h.rot || !h.vel || !h.hm || h.num_classes < 1 ||
        h.num_classes > 256)
      return SPCONVB_E_ARG;
    a.head[t] = h;
  }
  a.p = *p;
  a.num_tasks = num_tasks;
  a.out_boxes = out_boxes;
  a.out_count = out_count;
  bind_buffers(l, workspace, num_tasks, a);
  cudaStream_t st = (cudaStream_t)stream;
  SPCONVB_CUDA_TRY(cudaMemsetAsync(workspace, 0, l.counters_bytes, st));
  const int HW = p->H * p->W;
  cp_candidates_kernel<<<dim3((HW + 255) / 256, num_tasks), 256, 0, st>>>(a);
  SPCONVB_LAUNCH_CHECK();
  cp_rank_kernel<<<num_tasks, kRankThreads, 0, st>>>(a);
  SPCONVB_LAUNCH_CHECK();
  cp_mask_kernel<<<dim3(kMaskCtasPerTask, num_tasks), kMaskThreads, 0, st>>>(a);
  SPCONVB_LAUNCH_CHECK();
  cp_scan_kernel<<<num_tasks, 512, 0, st>>>(a);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

int spconvb_cp_task_detections(const spconvb_cp_params* p, int32_t num_tasks,
                               const void* workspace, int32_t task, const float** detections,
                               const uint32_t** n_det) {
  if (!params_ok(p) || !workspace || num_tasks < 1 || num_tasks > SPCONVB_CP_MAX_TASKS ||
      task < 0 || task >= num_tasks)
    return SPCONVB_E_ARG;
  PostArgs a{};
  bind_buffers(layout_of(*p, num_tasks), (void*)workspace, num_tasks, a);
  if (detections) *detections = a.buf[task].det;
  if (n_det) *n_det = a.buf[task].n_det;
  return SPCONVB_OK;
}

int spconvb_cp_rotated_iou(const float* boxes_a, const float* boxes_b, int32_t n, float* iou,
                           void* stream) {
  if (!boxes_a || !boxes_b || !iou || n < 0) return SPCONVB_E_ARG;
  if (n == 0) return SPCONVB_OK;
  rotated_iou_pairs_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(boxes_a, boxes_b, n,
                                                                              iou);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

}  // extern "C"
