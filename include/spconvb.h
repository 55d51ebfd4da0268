/*
 * spconvb.h - C ABI of the B200 sparse-convolution library (libspconvb.so).
 *
 * Every entry point takes plain pointers and sizes, enqueues work on the CUDA
 * stream it is given (a cudaStream_t passed as void*) and returns 0 on success
 * or a negative SPCONVB_E_* / positive cudaError_t value.  Nothing here
 * synchronises the stream unless its comment says so.
 *
 * Row counts live in device memory (`const uint32_t* n_ptr`): kernels read
 * them on the device, so a whole frame runs without a host round trip and can
 * be captured in a CUDA graph.  This is what the reference calls DDS
 * (SparseDTensor::set_dds_num_of_points_pointer,
 * libraries/3DSparseConvolution/libspconv/include/spconv/engine.hpp:48-49);
 * `launch_rows` plays the role of its `fixed_launch_points`
 * (libraries/3DSparseConvolution/src/onnx-parser.hpp:38): it only sizes the
 * grid, every kernel strides over the rows that are really there.
 *
 * Device-side problems (full hash table, duplicated coordinates, more outputs
 * than capacity, a wait that ran out) never fault: they set bits in a 4-word
 * status block in device memory (SPCONVB_ST_*), which the host reads when it
 * wants to.
 *
 * Data conventions
 *   coords   int32 [rows][4] = (batch, c0, c1, c2)
 *   map      int32 [kvol][cap]; map[k*cap + o] = input row of output row o
 *            under kernel tap k, or -1.  k = (k0*K1 + k1)*K2 + k2,
 *            in = out*stride - pad + k*dilation.
 *   features row-major [rows][channels], int8 or fp16
 *   weights  [Cout][kvol][Cin] (the ONNX initialiser layout written by
 *            libraries/3DSparseConvolution/tool/centerpoint-export/funcs.py:43-60)
 */
#ifndef SPCONVB_H_
#define SPCONVB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPCONVB_API __attribute__((visibility("default")))

/* host-side error codes (returned) */
#define SPCONVB_OK 0
#define SPCONVB_E_ARG (-1)        /* bad argument / unsupported shape */
#define SPCONVB_E_RANGE (-2)      /* grid too large for 32-bit voxel keys */
#define SPCONVB_E_NOMEM (-3)
#define SPCONVB_E_PARSE (-4)      /* model file could not be read */
#define SPCONVB_E_UNSUPPORTED (-5)
#define SPCONVB_E_STATE (-6)      /* call made in the wrong state */
#define SPCONVB_E_DEVICE (-7)     /* status block reported a device-side error */
#define SPCONVB_E_SCRATCH_LIMIT (-8) /* problem needs more than the built-in scratch area */

/* device status bits (status[0]); status[1] = first offending row / count */
#define SPCONVB_ST_HASH_FULL 1u
#define SPCONVB_ST_DUPLICATE 2u
#define SPCONVB_ST_OVERFLOW 4u    /* more rows than capacity; extra rows dropped */
#define SPCONVB_ST_TIMEOUT 8u     /* a bounded wait inside a kernel ran out */
#define SPCONVB_ST_COORD_RANGE 16u

/* element kinds */
#define SPCONVB_F16 0
#define SPCONVB_I8 1

/* activations */
#define SPCONVB_ACT_NONE 0
#define SPCONVB_ACT_RELU 1

/* flags */
#define SPCONVB_FLAG_PREZEROED 1u /* caller already zeroed table / workspace */

SPCONVB_API const char* spconvb_version(void);
SPCONVB_API const char* spconvb_error_string(int code);

/* ---------------------------------------------------------------- rulebooks
 * Replaces the closed rulebook / index-pair construction that
 * EngineBuilder::push_sparse_conv implies through its `submanifold`,
 * `kernel_size`, `stride`, `padding`, `dilation` and `rulebook` arguments
 * (libraries/3DSparseConvolution/libspconv/include/spconv/engine.hpp:135-156). */

/* Number of 8-byte slots of the coordinate hash table for `cap_rows` rows
 * (power of two >= 1024, load factor <= 0.5).  A table passed to the functions below must
 * have a power-of-two number of slots >= 8; its contents are opaque (the 8 cells of an
 * aligned run along the innermost axis share one 64-byte block of slots). */
SPCONVB_API uint32_t spconvb_hash_slots(uint32_t cap_rows);

/* Insert rows 0..*n_ptr-1 of `coords` into `table` (slot = (key+1)<<32 | row,
 * 0 = empty).  Zeroes the table first unless SPCONVB_FLAG_PREZEROED. */
SPCONVB_API int spconvb_hash_build(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                                   uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                                   uint64_t* table, uint32_t slots, uint32_t flags,
                                   uint32_t* status, void* stream);

/* Submanifold map: outputs are the inputs.  map is [kvol][cap]. */
SPCONVB_API int spconvb_subm_map(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                                 uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                                 const int32_t ksize[3], const int32_t dilation[3],
                                 const uint64_t* table, uint32_t slots, int32_t* map,
                                 uint32_t* status, void* stream);

/* Submanifold map of a coordinate set produced by spconvb_down_map: neighbours
 * are ranked in that call's workspace (its bitmap and popcount prefix, which
 * must still be intact), so no hash table is needed for these rows. */
SPCONVB_API int spconvb_subm_map_ranked(const int32_t* coords, const uint32_t* n_ptr,
                                        uint32_t cap, uint32_t launch_rows,
                                        const int32_t grid[3], int32_t batch,
                                        const int32_t ksize[3], const int32_t dilation[3],
                                        const void* down_workspace, int32_t* map,
                                        uint32_t* status, void* stream);

/* Map of an inverse (transposed) sparse convolution: the pairs of the strided
 * rulebook built by spconvb_down_map with the same geometry, input and output
 * swapped (the `inverse` argument of EngineBuilder::push_sparse_conv, engine.hpp:156;
 * "SparseInverseConvolution", libraries/3DSparseConvolution/README.md:151).
 * `coords` are the rows that were the INPUT of that spconvb_down_map call (they are the
 * outputs here), `grid` their grid, `down_workspace` that call's workspace (still
 * intact) and `cap_coarse` its cap_out.  map is [kvol][cap]: map[k][i] = row of the
 * strided output that row i contributed to through tap k, or -1. */
SPCONVB_API int spconvb_inverse_map(const int32_t* coords, const uint32_t* n_ptr, uint32_t cap,
                                    uint32_t launch_rows, const int32_t grid[3], int32_t batch,
                                    const int32_t ksize[3], const int32_t stride[3],
                                    const int32_t pad[3], const int32_t dilation[3],
                                    const void* down_workspace, uint32_t cap_coarse,
                                    int32_t* map, uint32_t* status, void* stream);

/* Output grid of a strided conv along one axis. */
SPCONVB_API int32_t spconvb_out_extent(int32_t in, int32_t k, int32_t stride, int32_t pad,
                                       int32_t dilation);

/* Bytes of scratch spconvb_down_map needs for an output grid. */
SPCONVB_API size_t spconvb_down_workspace_bytes(const int32_t out_grid[3], int32_t batch);

/* Strided sparse conv rulebook.  Produces the unique output coordinates in
 * ascending ((b*G0+c0)*G1+c1)*G2+c2 order, their count (*n_out_ptr, clipped to
 * cap_out, SPCONVB_ST_OVERFLOW on clipping), the map [kvol][cap_out] and, when
 * out_table != NULL, the hash table of the outputs.  `workspace` keeps the
 * outputs' bitmap and rank prefix afterwards (see spconvb_subm_map_ranked).
 * `in_table` / `in_slots` are not used (kept in the signature; may be NULL / 0). */
SPCONVB_API int spconvb_down_map(const int32_t* in_coords, const uint32_t* n_in_ptr,
                                 uint32_t cap_in, uint32_t launch_rows, const int32_t in_grid[3],
                                 int32_t batch, const int32_t ksize[3], const int32_t stride[3],
                                 const int32_t pad[3], const int32_t dilation[3],
                                 const uint64_t* in_table, uint32_t in_slots, void* workspace,
                                 int32_t* out_coords, uint32_t* n_out_ptr, uint32_t cap_out,
                                 int32_t* map, uint64_t* out_table, uint32_t out_slots,
                                 uint32_t flags, uint32_t* status, void* stream);

/* The same rulebook for input rows that were themselves produced by spconvb_down_map (or by
 * this call): `in_workspace` is that call's workspace, still intact.  The map is then looked
 * up from the output side by rank in the input's bitmap (one pass that writes every entry
 * once) instead of being filled with -1 and scattered from the input side.  Results are
 * identical to spconvb_down_map's. */
SPCONVB_API int spconvb_down_map_ranked(const int32_t* in_coords, const uint32_t* n_in_ptr,
                                        uint32_t cap_in, uint32_t launch_rows,
                                        const int32_t in_grid[3], int32_t batch,
                                        const int32_t ksize[3], const int32_t stride[3],
                                        const int32_t pad[3], const int32_t dilation[3],
                                        const void* in_workspace, void* workspace,
                                        int32_t* out_coords, uint32_t* n_out_ptr,
                                        uint32_t cap_out, int32_t* map, uint64_t* out_table,
                                        uint32_t out_slots, uint32_t flags, uint32_t* status,
                                        void* stream);

/* Allocation-free variant of spconvb_down_map.  It has no counterpart in the
 * reference library; it exists for callers that are not allowed to allocate
 * device memory at all: a perception stack that freezes its memory map after
 * start-up (the usual rule on the automotive targets this code serves), or a
 * host that runs the rulebook step from a callback in which cudaMalloc is
 * forbidden or would stall every stream of the device.  Such a caller cannot
 * provide the `workspace` of spconvb_down_map, so this entry point brings its
 * own: SPCONVB_STATIC_SCRATCH_BYTES of device memory that are part of the
 * library image (each GPU that loads the library holds them until exit).
 *
 * Arguments and results are those of spconvb_down_map without `workspace`;
 * inputs, outputs and the optional output hash table are still the caller's.
 *  - The output grid must fit: spconvb_down_workspace_bytes(out_grid, batch)
 *    <= SPCONVB_STATIC_SCRATCH_BYTES (about 16 million output cells), else
 *    SPCONVB_E_SCRATCH_LIMIT is returned and nothing is launched.
 *  - Nothing is allocated or freed, here or in anything this calls.
 *  - The first call on a device looks the scratch address up (once per device,
 *    with that device current).  Make that first call outside stream capture.
 *  - All calls on a device share the one scratch area.  It is cleared at the
 *    start of every call, so back-to-back calls on one stream are fine; calls
 *    that can overlap on the GPU (different streams, no dependency) race.
 *  - The looked-up address is kept for the life of the process: do not call
 *    cudaDeviceReset (or otherwise destroy the device's primary context) between
 *    calls. */
#define SPCONVB_STATIC_SCRATCH_BYTES (4u << 20)
SPCONVB_API int spconvb_down_map_static(const int32_t* in_coords, const uint32_t* n_in_ptr,
                                        uint32_t cap_in, uint32_t launch_rows,
                                        const int32_t in_grid[3], int32_t batch,
                                        const int32_t ksize[3], const int32_t stride[3],
                                        const int32_t pad[3], const int32_t dilation[3],
                                        const uint64_t* in_table, uint32_t in_slots,
                                        int32_t* out_coords, uint32_t* n_out_ptr,
                                        uint32_t cap_out, int32_t* map, uint64_t* out_table,
                                        uint32_t out_slots, uint32_t flags, uint32_t* status,
                                        void* stream);

/* ------------------------------------------------------------- convolution
 * Replaces the closed gather-GEMM-scatter kernel behind
 * EngineBuilder::push_sparse_conv (engine.hpp:135-156) with its fused
 * dequant + bias + activation + requant epilogue, and optionally the
 * following Add(+ReLU) node (engine.hpp:100-112). */

typedef struct spconvb_conv_params {
  int32_t compute;        /* SPCONVB_I8 or SPCONVB_F16: operand type of the MMA */
  int32_t cin;            /* input channels as stored (a power of two >= 16 bytes per row) */
  int32_t cout;           /* 16, 32, 64 or 128 for the tensor-core path */
  int32_t kvol;           /* kernel taps */
  int32_t act;            /* SPCONVB_ACT_* applied to the conv result */
  int32_t out_kind;       /* SPCONVB_I8 / SPCONVB_F16 of `out` */
  float inv_out_scale;    /* 127 / dynamic range of the consumer (int8 out) */
  /* fused residual add (res == NULL: none).  The conv result is first rounded
   * to mid_kind exactly as if it had been stored, then
   * out = store(relu?(deq(mid) + deq(res))). */
  const void* res;
  int32_t res_kind;
  float res_scale;
  int32_t mid_kind;
  float mid_inv_scale;
  float mid_scale;
  int32_t res_relu;
  int32_t force_simt;     /* use the CUDA-core kernel (any channel count) */
  int32_t wait_test;      /* 0 in normal use.  Self-test of the bounded waits of the tensor-core
                           * kernel: w > 0 makes its producers withhold the "stage full" signal
                           * from the w-th K chunk of every CTA on, so the consumer's wait must
                           * run out; the launch then ends with SPCONVB_ST_TIMEOUT in the status
                           * block, its output undefined, the context and TMEM usable */
  /* Optional hint for the tensor-core kernel's L2 prefetch of input rows: the device-side
   * row count of `in` and the rows its buffer holds.  NULL / 0: input rows are not
   * prefetched (results are the same either way).  The prefetch is off unless the environment
   * variable SPCONVB_CONV_PREFETCH gives a depth in tiles: it measured slower than no prefetch. */
  const uint32_t* n_in_ptr;
  uint32_t cap_in;
} spconvb_conv_params;

/* Bytes of the packed device image of a weight tensor for the tensor-core path. */
SPCONVB_API size_t spconvb_conv_packed_bytes(int32_t compute, int32_t cin, int32_t cout,
                                             int32_t kvol);

/* Host-side packing: `w` is [cout][kvol][cin] int8 (compute I8) or fp16
 * (compute F16) in host memory; `dst` is a host buffer of
 * spconvb_conv_packed_bytes() to be copied to the device by the caller. */
SPCONVB_API int spconvb_conv_pack_weights(int32_t compute, int32_t cin, int32_t cout,
                                          int32_t kvol, const void* w, void* dst);

/* 1 when the tensor-core kernel covers this shape (and kvol <= 27). */
SPCONVB_API int spconvb_conv_supported(int32_t compute, int32_t cin, int32_t cout);

/* out[o,:] = epilogue(sum_k W[:,k,:] . in[map[k][o],:]).
 * `w_plain` ([cout][kvol][cin], device) is read by the CUDA-core kernel,
 * `w_packed` by the tensor-core kernel; either may be NULL if unused.
 * `scale` (int8: s_in*s_w[c]) and `bias` are fp32 [cout] on the device. */
SPCONVB_API int spconvb_conv_forward(const spconvb_conv_params* p, const void* in,
                                     const int32_t* map, uint32_t cap,
                                     const uint32_t* n_out_ptr, uint32_t launch_rows,
                                     const void* w_plain, const void* w_packed,
                                     const float* scale, const float* bias, void* out,
                                     uint32_t* status, void* stream);

/* ------------------------------------------------------------ elementwise
 * Add / Add&ReLU / ReLU (EngineBuilder::push_add, push_relu, engine.hpp:100-112),
 * precision changes between layers, and channel padding of the input.
 * In this group and in the two ScatterDense calls `launch_rows` is also the row capacity of
 * the buffers: rows [0, min(*n_ptr, launch_rows)) are processed, so a device-side count
 * larger than the buffers never makes a kernel read or write past them. */

SPCONVB_API int spconvb_add(const void* a, int32_t a_kind, float a_scale, const void* b,
                            int32_t b_kind, float b_scale, int32_t channels,
                            const uint32_t* n_ptr, uint32_t launch_rows, int32_t relu,
                            int32_t out_kind, float inv_out_scale, void* out, void* stream);

SPCONVB_API int spconvb_relu(const void* x, int32_t kind, int32_t channels, const uint32_t* n_ptr,
                             uint32_t launch_rows, void* out, void* stream);

/* Folds max |x| over rows [0, min(*n_ptr, launch_rows)) x channels into *out (a float in
 * device memory that the caller zeroed before the first call; calls accumulate).  int8
 * tensors count in quantised units.  This is the statistic of plain absmax calibration. */
SPCONVB_API int spconvb_absmax(const void* x, int32_t kind, int32_t channels,
                               const uint32_t* n_ptr, uint32_t launch_rows, float* out,
                               void* stream);

/* Copy rows [*n_ptr][cin] to [*n_ptr][cout_pad] with zero padding and an
 * optional precision change (fp16 -> int8 with inv_scale, int8 -> fp16 with scale). */
SPCONVB_API int spconvb_convert(const void* x, int32_t in_kind, int32_t cin, int32_t out_kind,
                                int32_t cout_pad, float scale_or_inv, const uint32_t* n_ptr,
                                uint32_t launch_rows, void* out, void* stream);

/* ScatterDense (+ Transpose of the spatial axes), EngineBuilder::push_dense
 * (engine.hpp:114-123).  out is fp16 [batch][channels][g(perm0)][g(perm1)][g(perm2)]
 * and is fully written (zeros where no voxel). */
SPCONVB_API int spconvb_scatter_dense(const void* feat, int32_t in_kind, float in_scale,
                                      const int32_t* coords, const uint32_t* n_ptr,
                                      uint32_t launch_rows, int32_t channels, int32_t batch,
                                      const int32_t grid[3], const int32_t perm[3], void* out,
                                      void* stream);

/* ScatterDense into one of the engine's output layouts, optionally quantised to int8
 * (EngineBuilder::push_dense with output_layout and input_dynamic_range, engine.hpp:114-123;
 * enum TensorLayout, engine.hpp:26).  With (s0, s1, s2) the cell after perm, C = channels,
 * D = grid[perm0] and m = c * D + s0 the channel of the [N, C*D, H, W] view the backbones
 * reshape to:
 *   layout 1 NCHW    out[b][m][s1][s2]
 *   layout 2 NCHW32  out[b][m / 32][s1][s2][m % 32], C*D padded up to a multiple of 32
 *   layout 3 NHWzC   out[b][s1][s2][s0][c]
 * out_kind SPCONVB_F16 or SPCONVB_I8; int8 values are clamp(rint(x * inv_out_scale)) with
 * inv_out_scale = 127 / input_dynamic_range.  out holds spconvb_dense_bytes() bytes and is
 * fully written.  The engine is closed, so the two vectorised layouts follow the usual
 * meaning of their names (TensorRT's CHW32; height, width, z, channel). */
SPCONVB_API int spconvb_scatter_dense_layout(const void* feat, int32_t in_kind, float in_scale,
                                             const int32_t* coords, const uint32_t* n_ptr,
                                             uint32_t launch_rows, int32_t channels,
                                             int32_t batch, const int32_t grid[3],
                                             const int32_t perm[3], int32_t layout,
                                             int32_t out_kind, float inv_out_scale, void* out,
                                             void* stream);
SPCONVB_API size_t spconvb_dense_bytes(int32_t channels, int32_t batch, const int32_t grid[3],
                                       const int32_t perm[3], int32_t layout, int32_t out_kind);

/* -------------------------------------------------------------- voxelizer
 * Replaces buildHashKernel / voxelizationKernel / featureExtractionKernel
 * (CUDA-CenterPoint/src/preprocess_kernels.cu:70-173 and the two copies in
 * libraries/3DSparseConvolution/src/voxelization.cu and
 * CUDA-BEVFusion/src/bevfusion/lidar-voxelization.cu).  Deterministic: voxel
 * ids follow the first point of each voxel in point order and the first
 * `max_points_per_voxel` points (by index) are averaged, which is what the
 * reference kernels compute when they run one point at a time. */

typedef struct spconvb_voxel_params {
  float range_min[3];     /* x, y, z */
  float range_max[3];
  float voxel_size[3];
  int32_t grid[3];        /* gx, gy, gz */
  int32_t num_features;   /* <= 8 */
  int32_t points_kind;    /* 0 = fp32 points, 1 = fp16 points */
  int32_t max_points_per_voxel; /* <= 16 */
  int32_t max_voxels;
  int32_t order;          /* 0: indices (0,z,y,x); 1: indices (0,x,y,z) */
} spconvb_voxel_params;

SPCONVB_API size_t spconvb_voxelize_workspace_bytes(const spconvb_voxel_params* p,
                                                    uint32_t max_points);

/* features fp16 [max_voxels][num_features], indices int32 [max_voxels][4];
 * *n_voxels_ptr (device) receives min(count, max_voxels). */
SPCONVB_API int spconvb_voxelize(const spconvb_voxel_params* p, const void* points,
                                 uint32_t num_points, void* workspace, void* features,
                                 int32_t* indices, uint32_t* n_voxels_ptr, uint32_t* status,
                                 void* stream);

/* ------------------------------------------------------------------ engine
 * A whole backbone behind the C ABI.  These are the entry points the C++
 * `spconv::` classes (include/spconv/engine.hpp) are written on; they mirror
 * EngineBuilder / Engine of the reference one to one
 * (libraries/3DSparseConvolution/libspconv/include/spconv/engine.hpp:55-167).
 * Tensors are referred to by the integer ids the push functions return
 * (negative = SPCONVB_E_*).  Precision: 1 = fp16, 2 = int8 (the reference's
 * Precision enum); layout 1 = NCHW. */

typedef struct spconvb_builder spconvb_builder;
typedef struct spconvb_engine spconvb_engine;

#define SPCONVB_PRECISION_FP16 1
#define SPCONVB_PRECISION_INT8 2

/* build flags */
#define SPCONVB_BUILD_KEEP_TENSORS 1u   /* no buffer reuse: every tensor stays readable */
#define SPCONVB_BUILD_NO_FUSION 2u      /* run Add / ReLU as their own kernels */
#define SPCONVB_BUILD_FORCE_SIMT 4u     /* CUDA-core convolution everywhere */
#define SPCONVB_BUILD_SINGLE_STREAM 8u  /* no auxiliary stream: rulebooks and convolutions in program order */

SPCONVB_API spconvb_builder* spconvb_builder_create(void);
SPCONVB_API void spconvb_builder_destroy(spconvb_builder* b);

/* EngineBuilder::push_input (engine.hpp:99) */
SPCONVB_API int spconvb_builder_input(spconvb_builder* b, const char* name);

/* EngineBuilder::push_sparse_conv (engine.hpp:135-156).  weight: fp16 bits
 * [cout][k0][k1][k2][cin]; bias fp16 bits [cout] or NULL. */
SPCONVB_API int spconvb_builder_sparse_conv(
    spconvb_builder* b, const char* name, int x, const uint16_t* weight,
    const int32_t weight_shape[5], const float* weight_dynamic_ranges, int32_t n_ranges,
    const uint16_t* bias, int32_t n_bias, const char* activation, const int32_t kernel_size[3],
    const int32_t stride[3], const int32_t padding[3], const int32_t dilation[3],
    float input_dynamic_range, int32_t submanifold, uint32_t max_output_points,
    uint32_t fixed_launch_points, const char* rulebook, int32_t precision,
    int32_t output_precision, const char* output_name, int32_t inverse);

/* EngineBuilder::push_add (engine.hpp:100-107) */
SPCONVB_API int spconvb_builder_add(spconvb_builder* b, const char* name, int a, int bb,
                                    float a_dynamic_range, float b_dynamic_range,
                                    const char* output_name, int32_t precision,
                                    int32_t output_precision, uint32_t fixed_launch_points);

/* EngineBuilder::push_relu (engine.hpp:109-112) */
SPCONVB_API int spconvb_builder_relu(spconvb_builder* b, const char* name, int x,
                                     const char* output_name);

/* EngineBuilder::push_dense (engine.hpp:114-123) */
SPCONVB_API int spconvb_builder_dense(spconvb_builder* b, const char* name, int x,
                                      const char* format, const char* output_name,
                                      const int32_t* input_spatial_shape, int32_t n_spatial,
                                      const int32_t* output_shape, int32_t n_output_shape,
                                      int32_t output_layout, float input_dynamic_range,
                                      uint32_t input_bound);

/* EngineBuilder::push_reshape / push_transpose (engine.hpp:125-133) */
SPCONVB_API int spconvb_builder_reshape(spconvb_builder* b, const char* name, int x,
                                        const int64_t* shape, int32_t n, const char* output_name);
SPCONVB_API int spconvb_builder_transpose(spconvb_builder* b, const char* name, int x,
                                          const int64_t* dims, int32_t n, const char* output_name);

/* EngineBuilder::push_output (engine.hpp:158) */
SPCONVB_API int spconvb_builder_output(spconvb_builder* b, int x);

/* EngineBuilder::build (engine.hpp:161).  Uploads packed weights on `stream`
 * and synchronises it.  Returns NULL and sets *err on failure. */
SPCONVB_API spconvb_engine* spconvb_builder_build(spconvb_builder* b, int32_t precision,
                                                  uint32_t flags, void* stream, int* err);

/* spconv::load_engine_from_onnx
 * (libraries/3DSparseConvolution/src/onnx-parser.cpp:101-231; exported by the
 * v1.0 library, CUDA-CenterPoint/3rdparty/libspconv/include/spconv/engine.hpp:103-104).
 * Reads the ONNX protobuf wire format directly; no protobuf library needed. */
SPCONVB_API spconvb_engine* spconvb_engine_load_onnx(const char* path, int32_t precision,
                                                     uint32_t flags,
                                                     uint32_t fixed_launch_points, void* stream,
                                                     int* err);

/* Parses a model file and writes a text summary into `buf` (one line per
 * node: op, name, inputs, output, the attributes the loader uses).  Needs no
 * GPU.  Returns SPCONVB_OK or the loader's error code. */
SPCONVB_API int spconvb_onnx_inspect(const char* path, char* buf, size_t buf_bytes);

SPCONVB_API void spconvb_engine_destroy(spconvb_engine* e);

/* Engine::forward of the v1.0 interface
 * (CUDA-CenterPoint/3rdparty/libspconv/include/spconv/engine.hpp:73-77):
 * features fp16 [n][C] and indices int32 [n][4] in device memory, used in
 * place; n known on the host.  Asynchronous on `stream`; outputs are valid once
 * the stream has run.  The first call for a given grid allocates buffers (and
 * synchronises): make it before any stream capture. */
SPCONVB_API int spconvb_engine_forward(spconvb_engine* e, const void* features, uint32_t n,
                                       const int32_t* indices, const int32_t grid[3],
                                       int32_t batch, void* stream);

/* Engine::forward(stream) of the v1.3 interface with a DDS row count
 * (engine.hpp:48-49,71): buffers hold up to `cap_rows` rows, the device word
 * *n_dev says how many are valid.  Capturable in a CUDA graph once the grid
 * has been seen by spconvb_engine_prepare or an earlier forward. */
SPCONVB_API int spconvb_engine_forward_dds(spconvb_engine* e, const void* features,
                                           const int32_t* indices, uint32_t cap_rows,
                                           const uint32_t* n_dev, const int32_t grid[3],
                                           int32_t batch, void* stream);

/* Allocate everything for a grid ahead of time (synchronises). */
SPCONVB_API int spconvb_engine_prepare(spconvb_engine* e, const int32_t grid[3], int32_t batch);

SPCONVB_API int spconvb_engine_num_outputs(const spconvb_engine* e);

/* Output i: device pointer, shape (up to 8 dims), element kind (SPCONVB_F16 /
 * SPCONVB_I8), and whether it is dense.  For a sparse output shape = {cap, C}
 * and spconvb_engine_tensor gives the rows. */
SPCONVB_API int spconvb_engine_output(const spconvb_engine* e, int i, void** data,
                                      int64_t shape[8], int32_t* ndim, int32_t* kind,
                                      int32_t* dense);

/* Memory layout of dense output i: the TensorLayout value (1 NCHW, 2 NCHW32, 3 NHWzC; 0 for
 * a sparse output), the dimensions as they lie in memory (NCHW32: {N, ceil(C*D/32), H, W, 32};
 * NHWzC: {N, H, W, D, C}; NCHW: the shape spconvb_engine_output reports) and the byte size.
 * spconvb_engine_output keeps reporting the logical NCHW shape, as
 * SparseDTensor::features().shape does (engine.hpp:38-50). */
SPCONVB_API int spconvb_engine_output_layout(const spconvb_engine* e, int i, int32_t* layout,
                                             int64_t physical_shape[8], int32_t* ndim,
                                             size_t* bytes);

/* Rows of sparse output i (SparseDTensor::indices() / grid_size() of an engine output,
 * engine.hpp:38-50): its coordinates [cap][4] (the caller's own index buffer when the output
 * lives on the input's rows: then *coords is NULL and *on_input_rows is 1), the device word
 * holding the row count (rows beyond it are undefined), the capacity and the grid.  Any
 * out-pointer may be NULL.  Dense outputs: SPCONVB_E_ARG. */
SPCONVB_API int spconvb_engine_output_rows(const spconvb_engine* e, int i, int32_t** coords,
                                           uint32_t** n_ptr, uint32_t* cap, int32_t grid[3],
                                           int32_t* on_input_rows);

/* Any tensor by name (needs SPCONVB_BUILD_KEEP_TENSORS for intermediates):
 * features pointer, element kind, channels as stored, int8 scale, coordinates
 * pointer, device row-count pointer, capacity, grid. */
typedef struct spconvb_tensor_view {
  void* features;
  int32_t kind;
  int32_t channels;
  float scale;
  int32_t* coords;
  uint32_t* n_ptr;
  uint32_t cap;
  int32_t grid[3];
  int32_t dense;
} spconvb_tensor_view;
SPCONVB_API int spconvb_engine_tensor(const spconvb_engine* e, const char* name,
                                      spconvb_tensor_view* view);

/* Names of all tensors in execution order, '\n' separated (owned by the engine). */
SPCONVB_API const char* spconvb_engine_tensor_names(const spconvb_engine* e);

/* Per-step device times of one forward call, like the reference's verbose
 * per-layer timing (spconv::EventTimer, libspconv/include/spconv/timer.hpp:22-51).
 * Steps are the lines of spconvb_engine_describe.  Convolution, Add, ReLU,
 * conversion and dense steps are run `reps` times, each behind a write of
 * `flush_bytes` to `flush` (NULL: none) that evicts L2, and averaged; rulebook
 * steps run once.  Synchronises after every step: a measurement aid, not a
 * way to run inference. */
SPCONVB_API int spconvb_engine_num_steps(const spconvb_engine* e);
SPCONVB_API int spconvb_engine_profile(spconvb_engine* e, const void* features, uint32_t n,
                                       const int32_t* indices, const int32_t grid[3],
                                       int32_t batch, void* stream, float* step_ms,
                                       int32_t max_steps, int32_t reps, void* flush,
                                       size_t flush_bytes);

/* Coordinate set i (the `cs=` column of spconvb_engine_describe): device row
 * count, capacity and grid. */
SPCONVB_API int spconvb_engine_coordset(const spconvb_engine* e, int i, uint32_t** n_ptr,
                                        uint32_t* cap, int32_t grid[3]);

/* Rulebook i of the engine (measurement helper): the map [kvol][cap], and the
 * device row counts of its output and input coordinate sets. */
SPCONVB_API int spconvb_engine_num_rules(const spconvb_engine* e);
SPCONVB_API int spconvb_engine_rule(const spconvb_engine* e, int i, int32_t** map, uint32_t* cap,
                                    int32_t* kvol, uint32_t** n_out_ptr, uint32_t** n_in_ptr);

/* Copies device memory to the host after synchronising `stream` (test helper). */
SPCONVB_API int spconvb_read_device(const void* device_src, void* host_dst, size_t bytes,
                                    void* stream);

/* cudaMemcpyAsync on `stream`; direction 0 = host to device, 1 = device to
 * host, 2 = device to device.  For callers (ctypes, FFI) that hold raw pointers
 * and no CUDA runtime binding of their own. */
SPCONVB_API int spconvb_copy_async(void* dst, const void* src, size_t bytes, int32_t direction,
                                   void* stream);

/* Synchronises `stream` and copies the 4-word status block (SPCONVB_ST_*). */
SPCONVB_API int spconvb_engine_status(const spconvb_engine* e, uint32_t out[4], void* stream);

/* Kernels launched by the last forward call (host-side count of launches). */
SPCONVB_API int spconvb_engine_last_launches(const spconvb_engine* e);

/* Algorithmic work of the engine's graph for given per-coordinate-set counts is
 * reported by spconvb_engine_describe: a '\n' separated text table, one line
 * per executed step: "kind name rows_ptr_index cin cout kvol in_bytes out_bytes". */
SPCONVB_API const char* spconvb_engine_describe(const spconvb_engine* e);

/* Run-time precision control of the v1.0 interface
 * (CUDA-CenterPoint/3rdparty/libspconv/include/spconv/engine.hpp:81-91).  The engine keeps
 * the graph it was built from; these calls edit it and spconvb_engine_reconfigure rebuilds
 * the executable engine from it (weights are re-quantised and re-packed, buffers are
 * re-planned at the next forward; outputs of earlier forwards become invalid).
 *
 * set_node_precision: `key` is a node name (by_optype = 0) or an operator type
 * ("SparseConvolution", "Add", "Relu", "ScatterDense"; by_optype = 1); returns the number of
 * nodes changed or a negative error.  Takes effect at the next reconfigure.
 *
 * set_int8_calibration(1) + reconfigure: the engine runs in fp16 and every forward folds
 * the absmax of every tensor into a running maximum.  set_int8_calibration(0): the maxima
 * become the dynamic ranges of the graph (conv: its input's range and per-output-channel
 * weight ranges; Add: the larger of its operands' for both), every node not touched by
 * set_node_precision is set to int8, and the engine's main precision becomes int8; the next
 * reconfigure builds that engine. */
SPCONVB_API int spconvb_engine_set_node_precision(spconvb_engine* e, const char* key,
                                                  int32_t by_optype, int32_t compute_precision,
                                                  int32_t output_precision);
SPCONVB_API int spconvb_engine_set_int8_calibration(spconvb_engine* e, int32_t enable);
SPCONVB_API int spconvb_engine_reconfigure(spconvb_engine* e, void* stream);

/* Logging (spconv::set_logger_level, engine.hpp:171): 0 verbose, 1 warn, 2 error, 99 quiet. */
SPCONVB_API void spconvb_set_log_level(int32_t level);
typedef void (*spconvb_log_fn)(int32_t level, const char* message);
SPCONVB_API void spconvb_set_log_callback(spconvb_log_fn fn);

#ifdef __cplusplus
}
#endif
#endif /* SPCONVB_H_ */
