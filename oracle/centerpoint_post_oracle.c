/*
 * CPU oracle for the CenterPoint head decode and rotated-box NMS.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links or calls it.
 *
 * PARITY UNPINNED: the reference has no test vectors for this stage; the restatement follows
 * its CUDA source and host loop operation by operation (single precision, no contraction):
 *   decode   predictKernel, CUDA-CenterPoint/src/postprocess_kernels.cu:28-117
 *   overlap  devIoU and its helpers, same file :119-264
 *   mask     nms_cuda, same file :266-306
 *   boxes    permute_cuda, same file :372-386
 *   host     sort by score, greedy scan of the mask, nms_post_max_size cut,
 *            CUDA-CenterPoint/src/centerpoint.cpp:163-216
 *
 * Two places where the reference's result depends on thread timing are made deterministic
 * (the CUDA side does the same): detections are ordered by (score descending, cell index
 * ascending) instead of by arrival order followed by an unstable sort, and when more than
 * max_det cells pass the filters the max_det best in that order are kept instead of the
 * first max_det to arrive.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 half_t;

static inline float h2f(uint16_t h) {
  half_t v;
  memcpy(&v, &h, 2);
  return (float)v;
}

#define DET_FLOATS 11

typedef struct {
  float score;
  int32_t cell;
  int32_t label;
} cand_t;

static int cand_before(const void* pa, const void* pb) {
  const cand_t* a = (const cand_t*)pa;
  const cand_t* b = (const cand_t*)pb;
  if (a->score != b->score) return a->score > b->score ? -1 : 1;
  return a->cell < b->cell ? -1 : (a->cell > b->cell ? 1 : 0);
}

static inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

/* Heads are fp16 [C][H][W] (batch 1).  det: [max_det][11] = x y z dx dy dz vx vy rot label
 * score, sorted; cells: the cell index h*W+w of each.  Returns the number written. */
int orc_centerpoint_decode(int H, int W, int C_hm, const uint16_t* reg, const uint16_t* height,
                           const uint16_t* dim, const uint16_t* rot, const uint16_t* vel,
                           const uint16_t* hm, const float* post_center_range,
                           float out_size_factor, const float* voxel_size, const float* pc_range,
                           float score_threshold, int max_det, float* det, int32_t* cells) {
  const int HW = H * W;
  cand_t* cand = (cand_t*)malloc(sizeof(cand_t) * (size_t)(HW > 0 ? HW : 1));
  int n = 0;
  for (int cell = 0; cell < HW; ++cell) {
    const int h = cell / W, w = cell % W;
    int label = 0;
    float score = sigmoidf_(h2f(hm[cell]));
    for (int c = 1; c < C_hm; ++c) {
      const float s = sigmoidf_(h2f(hm[c * HW + cell]));
      if (s > score) {
        score = s;
        label = c;
      }
    }
    if (score < score_threshold) continue;
    float xs = h2f(reg[cell]) + (float)w;
    float ys = h2f(reg[HW + cell]) + (float)h;
    xs = xs * out_size_factor * voxel_size[0] + pc_range[0];
    ys = ys * out_size_factor * voxel_size[1] + pc_range[1];
    const float zs = h2f(height[cell]);
    if (xs < post_center_range[0] || xs > post_center_range[3]) continue;
    if (ys < post_center_range[1] || ys > post_center_range[4]) continue;
    if (zs < post_center_range[2] || zs > post_center_range[5]) continue;
    cand[n].score = score;
    cand[n].cell = cell;
    cand[n].label = label;
    ++n;
  }
  qsort(cand, (size_t)n, sizeof(cand_t), cand_before);
  if (n > max_det) n = max_det;
  for (int i = 0; i < n; ++i) {
    const int cell = cand[i].cell;
    const int h = cell / W, w = cell % W;
    float* d = det + (size_t)i * DET_FLOATS;
    float xs = h2f(reg[cell]) + (float)w;
    float ys = h2f(reg[HW + cell]) + (float)h;
    d[0] = xs * out_size_factor * voxel_size[0] + pc_range[0];
    d[1] = ys * out_size_factor * voxel_size[1] + pc_range[1];
    d[2] = h2f(height[cell]);
    d[3] = expf(h2f(dim[cell]));
    d[4] = expf(h2f(dim[HW + cell]));
    d[5] = expf(h2f(dim[2 * HW + cell]));
    d[6] = h2f(vel[cell]);
    d[7] = h2f(vel[HW + cell]);
    d[8] = atan2f(h2f(rot[cell]), h2f(rot[HW + cell]));
    d[9] = (float)cand[i].label;
    d[10] = cand[i].score;
    if (cells) cells[i] = cell;
  }
  free(cand);
  return n;
}

/* ---- rotated overlap ------------------------------------------------------------------- */
typedef struct { float x, y; } pt_t;

static inline float cross3(pt_t p1, pt_t p2, pt_t p0) {
  return (p1.x - p0.x) * (p2.y - p0.y) - (p2.x - p0.x) * (p1.y - p0.y);
}

static inline int inside_with_margin(const float* box, pt_t p) {
  const float margin = 1e-2f;
  const float c = cosf(-box[6]), s = sinf(-box[6]);
  const float rx = (p.x - box[0]) * c + (p.y - box[1]) * (-s);
  const float ry = (p.x - box[0]) * s + (p.y - box[1]) * c;
  return fabsf(rx) < box[3] / 2 + margin && fabsf(ry) < box[4] / 2 + margin;
}

static inline int segments_cross(pt_t p1, pt_t p0, pt_t q1, pt_t q0, pt_t* ans) {
  if (!(fminf(p0.x, p1.x) <= fmaxf(q0.x, q1.x) && fminf(q0.x, q1.x) <= fmaxf(p0.x, p1.x) &&
        fminf(p0.y, p1.y) <= fmaxf(q0.y, q1.y) && fminf(q0.y, q1.y) <= fmaxf(p0.y, p1.y)))
    return 0;
  const float s1 = cross3(q0, p1, p0);
  const float s2 = cross3(p1, q1, p0);
  const float s3 = cross3(p0, q1, q0);
  const float s4 = cross3(q1, p1, q0);
  if (!(s1 * s2 > 0 && s3 * s4 > 0)) return 0;
  const float s5 = cross3(q1, p1, p0);
  if ((double)fabsf(s5 - s1) > 1e-8) {
    ans->x = (s5 * q0.x - s1 * q1.x) / (s5 - s1);
    ans->y = (s5 * q0.y - s1 * q1.y) / (s5 - s1);
  } else {
    const float a0 = p0.y - p1.y, b0 = p1.x - p0.x, c0 = p0.x * p1.y - p1.x * p0.y;
    const float a1 = q0.y - q1.y, b1 = q1.x - q0.x, c1 = q0.x * q1.y - q1.x * q0.y;
    const float D = a0 * b1 - a1 * b0;
    ans->x = (b0 * c1 - b1 * c0) / D;
    ans->y = (a1 * c0 - a0 * c1) / D;
  }
  return 1;
}

static void box_corners(const float* box, pt_t* c5) {
  const float hx = box[3] / 2, hy = box[4] / 2;
  const float x1 = box[0] - hx, y1 = box[1] - hy, x2 = box[0] + hx, y2 = box[1] + hy;
  const float co = cosf(box[6]), si = sinf(box[6]);
  const pt_t raw[4] = {{x1, y1}, {x2, y1}, {x2, y2}, {x1, y2}};
  for (int k = 0; k < 4; ++k) {
    c5[k].x = (raw[k].x - box[0]) * co + (raw[k].y - box[1]) * (-si) + box[0];
    c5[k].y = (raw[k].x - box[0]) * si + (raw[k].y - box[1]) * co + box[1];
  }
  c5[4] = c5[0];
}

/* Bird's-eye IoU of two boxes [x y z dx dy dz angle]. */
float orc_rotated_iou(const float* box_a, const float* box_b) {
  pt_t ca[5], cb[5], pts[16];
  float ang[16];
  box_corners(box_a, ca);
  box_corners(box_b, cb);
  int cnt = 0;
  pt_t centre = {0.f, 0.f};
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j)
      if (segments_cross(ca[i + 1], ca[i], cb[j + 1], cb[j], &pts[cnt])) {
        centre.x = centre.x + pts[cnt].x;
        centre.y = centre.y + pts[cnt].y;
        ++cnt;
      }
  for (int k = 0; k < 4; ++k) {
    if (inside_with_margin(box_a, cb[k])) {
      centre.x = centre.x + cb[k].x;
      centre.y = centre.y + cb[k].y;
      pts[cnt++] = cb[k];
    }
    if (inside_with_margin(box_b, ca[k])) {
      centre.x = centre.x + ca[k].x;
      centre.y = centre.y + ca[k].y;
      pts[cnt++] = ca[k];
    }
  }
  centre.x /= (float)cnt;
  centre.y /= (float)cnt;
  /* stable ascending order of the polar angle about the centre */
  for (int k = 0; k < cnt; ++k) ang[k] = atan2f(pts[k].y - centre.y, pts[k].x - centre.x);
  for (int k = 1; k < cnt; ++k) {
    const pt_t p = pts[k];
    const float a = ang[k];
    int j = k - 1;
    while (j >= 0 && ang[j] > a) {
      pts[j + 1] = pts[j];
      ang[j + 1] = ang[j];
      --j;
    }
    pts[j + 1] = p;
    ang[j + 1] = a;
  }
  float area = 0.f;
  for (int k = 0; k + 1 < cnt; ++k) {
    const float ax = pts[k].x - pts[0].x, ay = pts[k].y - pts[0].y;
    const float bx = pts[k + 1].x - pts[0].x, by = pts[k + 1].y - pts[0].y;
    area += ax * by - ay * bx;
  }
  const float overlap = fabsf(area) / 2.0f;
  const float sa = box_a[3] * box_a[4], sb = box_b[3] * box_b[4];
  return overlap / fmaxf(sa + sb - overlap, 1e-8f);
}

/* det: n sorted detections [n][11].  Writes the kept ones as [x y z w l h vx vy rot id score]
 * with id = label + label_offset, at most post_max of them; kept_index (optional) receives
 * their positions in det; margin (optional) receives the smallest |iou - threshold| met among
 * the pairs the greedy scan evaluated, so that a test can tell a decision that rounding could
 * flip.  Returns the number written. */
int orc_centerpoint_nms(const float* det, int n, float iou_threshold, int post_max,
                        int label_offset, float* out, int32_t* kept_index, float* margin) {
  float* boxes = (float*)malloc(sizeof(float) * 7 * (size_t)(n > 0 ? n : 1));
  uint8_t* removed = (uint8_t*)calloc((size_t)(n > 0 ? n : 1), 1);
  for (int i = 0; i < n; ++i) {
    const float* d = det + (size_t)i * DET_FLOATS;
    float* b = boxes + (size_t)i * 7;
    b[0] = d[0]; b[1] = d[1]; b[2] = d[2];
    b[3] = d[4]; b[4] = d[3]; b[5] = d[5];
    b[6] = (float)(-(double)d[8] - 3.141592653 * 0.5);
  }
  int kept = 0, written = 0;
  float closest = 1e30f;
  for (int i = 0; i < n; ++i) {
    if (removed[i]) continue;
    if (kept++ < post_max) {
      const float* d = det + (size_t)i * DET_FLOATS;
      float* o = out + (size_t)written * DET_FLOATS;
      memcpy(o, d, sizeof(float) * 9);
      o[9] = (float)(label_offset + (int)d[9]);
      o[10] = d[10];
      if (kept_index) kept_index[written] = i;
      ++written;
    }
    for (int j = i + 1; j < n; ++j) {
      const float iou = orc_rotated_iou(boxes + (size_t)i * 7, boxes + (size_t)j * 7);
      if (!removed[j]) {
        const float m = fabsf(iou - iou_threshold);
        if (m < closest) closest = m;
      }
      if (iou >= iou_threshold) removed[j] = 1;
    }
  }
  if (margin) *margin = closest;
  free(boxes);
  free(removed);
  return written;
}
