// C entry points of the convolution: argument checks and the choice between
// the tensor-core kernel and the CUDA-core kernel.
#include "common.cuh"

namespace spconvb {
bool conv_umma_supported(int compute, int cin, int cout);
size_t conv_umma_packed_bytes(int compute, int cin, int cout, int kvol);
int conv_umma_pack(int compute, int cin, int cout, int kvol, const void* w, void* dst);
int conv_umma_launch(const spconvb_conv_params& p, const void* in, const int32_t* map,
                     uint32_t cap, const uint32_t* n_out_ptr, uint32_t launch_rows,
                     const void* w_packed, const float* scale, const float* bias, void* out,
                     uint32_t* status, cudaStream_t st);
int conv_simt_launch(const spconvb_conv_params& p, const void* in, const int32_t* map,
                     uint32_t cap, const uint32_t* n_out_ptr, uint32_t launch_rows,
                     const void* w_plain, const float* scale, const float* bias, void* out,
                     cudaStream_t st);
}  // namespace spconvb

using namespace spconvb;

extern "C" {

int spconvb_conv_supported(int32_t compute, int32_t cin, int32_t cout) {
  return conv_umma_supported(compute, cin, cout) ? 1 : 0;
}

size_t spconvb_conv_packed_bytes(int32_t compute, int32_t cin, int32_t cout, int32_t kvol) {
  if (!conv_umma_supported(compute, cin, cout) || kvol < 1) return 0;
  return conv_umma_packed_bytes(compute, cin, cout, kvol);
}

int spconvb_conv_pack_weights(int32_t compute, int32_t cin, int32_t cout, int32_t kvol,
                              const void* w, void* dst) {
  return conv_umma_pack(compute, cin, cout, kvol, w, dst);
}

int spconvb_conv_forward(const spconvb_conv_params* p, const void* in, const int32_t* map,
                         uint32_t cap, const uint32_t* n_out_ptr, uint32_t launch_rows,
                         const void* w_plain, const void* w_packed, const float* scale,
                         const float* bias, void* out, uint32_t* status, void* stream) {
  if (!p || !in || !map || !n_out_ptr || !out) return SPCONVB_E_ARG;
  if (p->compute != SPCONVB_I8 && p->compute != SPCONVB_F16) return SPCONVB_E_ARG;
  if (p->out_kind != SPCONVB_I8 && p->out_kind != SPCONVB_F16) return SPCONVB_E_ARG;
  if (p->cin < 1 || p->cout < 1 || p->kvol < 1 || p->cin > 512 || p->cout > 512)
    return SPCONVB_E_ARG;
  if (launch_rows == 0 || launch_rows > cap) launch_rows = cap;
  cudaStream_t st = (cudaStream_t)stream;
  if (!p->force_simt && w_packed && p->kvol <= 27 &&
      conv_umma_supported(p->compute, p->cin, p->cout))
    return conv_umma_launch(*p, in, map, cap, n_out_ptr, launch_rows, w_packed, scale, bias, out,
                            status, st);
  return conv_simt_launch(*p, in, map, cap, n_out_ptr, launch_rows, w_plain, scale, bias, out,
                          st);
}

const char* spconvb_version(void) { return "spconvb 0.1 (sm_100a)"; }

const char* spconvb_error_string(int code) {
  switch (code) {
    case SPCONVB_OK: return "ok";
    case SPCONVB_E_ARG: return "bad argument or unsupported shape";
    case SPCONVB_E_RANGE: return "grid too large for 32-bit voxel keys";
    case SPCONVB_E_NOMEM: return "out of memory";
    case SPCONVB_E_PARSE: return "model file could not be parsed";
    case SPCONVB_E_UNSUPPORTED: return "unsupported operator or shape";
    case SPCONVB_E_STATE: return "call made in the wrong state";
    case SPCONVB_E_DEVICE: return "device-side status reported an error";
    case SPCONVB_E_SCRATCH_LIMIT: return "output grid needs more than the built-in scratch area";
  }
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  return "unknown error";
}

}  // extern "C"
