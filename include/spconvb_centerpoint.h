/*
 * C ABI of the CenterPoint detection-head post-processing: decode of the six task heads
 * and rotated-box NMS, the stage that follows the lidar backbone and the RPN.
 *
 * Replaces, in CUDA-CenterPoint:
 *   PostProcessCuda::doPostDecodeCuda / doPermuteCuda / doPostNMSCuda
 *       include/postprocess.h:55-88, src/postprocess.cpp:47-122
 *   predictKernel, nms_cuda, permute_cuda and their launchers
 *       src/postprocess_kernels.cu:28-117, 266-306, 372-403
 *   the per-task host loop (copy to host, std::sort by score, copy back, mask to host,
 *   greedy scan, nms_post_max_size cut)
 *       src/centerpoint.cpp:163-216
 *
 * The whole stage runs on the device in stream order: no host synchronisation, no host
 * sort, CUDA-graph capturable.  Results are deterministic: detections are ranked by
 * (score descending, cell index ascending), and when more than max_det cells pass the
 * filters the max_det best of that ranking go to NMS (the reference takes whichever
 * max_det threads arrive first and sorts them with an unstable sort).
 */
#ifndef SPCONVB_CENTERPOINT_H_
#define SPCONVB_CENTERPOINT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef SPCONVB_API
#define SPCONVB_API __attribute__((visibility("default")))
#endif

#define SPCONVB_CP_MAX_TASKS 8
#define SPCONVB_CP_BOX_FLOATS 11 /* x y z w l h vx vy rt id score, as struct Bndbox */

/* One task head: device pointers to fp16 [C][H][W] tensors (batch 1), as bound to the
 * RPN engine's outputs (src/centerpoint.cpp:145-158). */
typedef struct spconvb_cp_head {
  const void* reg;    /* 2 channels */
  const void* height; /* 1 */
  const void* dim;    /* 3 */
  const void* rot;    /* 2: sin, cos */
  const void* vel;    /* 2 */
  const void* hm;     /* num_classes channels */
  int32_t num_classes;
  int32_t label_offset; /* Params::task_num_stride[task] (include/common.h:58) */
} spconvb_cp_head;

/* Params of include/common.h:55-70. */
typedef struct spconvb_cp_params {
  int32_t H, W;
  float out_size_factor;
  float voxel_size[2];
  float pc_range[2];
  float score_threshold;
  float post_center_range[6];
  float nms_iou_threshold;
  int32_t max_det;      /* nms_pre_max_size, at most 1024 */
  int32_t nms_post_max; /* nms_post_max_size, per task */
} spconvb_cp_params;

/* Fills p with the reference's constants (180 x 180 heads, factor 8, voxel 0.075, range -54,
 * score 0.1, centre range +-61.2 / +-10, IoU 0.2, 1000 before NMS, 83 after). */
SPCONVB_API void spconvb_cp_default_params(spconvb_cp_params* p);

/* Device bytes spconvb_cp_postprocess needs for num_tasks heads. */
SPCONVB_API size_t spconvb_cp_workspace_bytes(const spconvb_cp_params* p, int32_t num_tasks);

/* Decode + NMS of num_tasks heads.  out_boxes: device float [num_tasks * nms_post_max][11],
 * the kept boxes of task 0 first, each task in score order; out_count: device uint32, the
 * number of boxes written.  Returns SPCONVB_OK or a negative SPCONVB_E_* code; work is only
 * enqueued on the stream. */
SPCONVB_API int spconvb_cp_postprocess(const spconvb_cp_head* heads, int32_t num_tasks,
                                       const spconvb_cp_params* p, void* workspace,
                                       size_t workspace_bytes, float* out_boxes,
                                       uint32_t* out_count, void* stream);

/* Per-task intermediate results left in the workspace by the last call, for tests:
 * n_det detections ranked by score as [n_det][11] = x y z dx dy dz vx vy rot label score
 * (the reference's d_detections_ after its host sort). */
SPCONVB_API int spconvb_cp_task_detections(const spconvb_cp_params* p, int32_t num_tasks,
                                           const void* workspace, int32_t task,
                                           const float** detections, const uint32_t** n_det);

/* Bird's-eye IoU of rotated boxes [x y z dx dy dz angle]: iou[i] for pairs (a[i], b[i]). */
SPCONVB_API int spconvb_cp_rotated_iou(const float* boxes_a, const float* boxes_b, int32_t n,
                                       float* iou, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPCONVB_CENTERPOINT_H_ */
