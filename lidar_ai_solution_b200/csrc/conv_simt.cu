// CUDA-core sparse convolution for channel counts the tensor-core kernel does
// not cover.  One thread per (output row, output channel); accumulation runs
// in the same order as the CPU oracle (taps ascending, channels ascending,
// products and sums rounded separately), so fp16 results match it bit for bit.
#include "common.cuh"

namespace spconvb {

template <bool INT8>
__global__ void conv_simt_kernel(const void* __restrict__ in_, const int32_t* __restrict__ map,
                                 uint32_t cap, const uint32_t* n_out_ptr, int kvol, int cin,
                                 int cout, const void* __restrict__ w_, const float* scale,
                                 const float* bias, Epilogue ep, const void* res_, void* out_) {
  const uint32_t n = min(*n_out_ptr, cap);
  const unsigned long long total = (unsigned long long)n * cout;
  for (unsigned long long t = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       t < total; t += (unsigned long long)gridDim.x * blockDim.x) {
    const uint32_t row = (uint32_t)(t / cout);
    const int c = (int)(t % cout);
    float y;
    if (INT8) {
      const int8_t* in = (const int8_t*)in_;
      const int8_t* w = (const int8_t*)w_;
      int acc = 0;
      for (int k = 0; k < kvol; ++k) {
        int r = __ldg(map + (size_t)k * cap + row);
        if (r < 0) continue;
        const int8_t* x = in + (size_t)r * cin;
        const int8_t* wk = w + ((size_t)c * kvol + k) * cin;
        int a = 0;
        for (int i = 0; i < cin; ++i) a += (int)wk[i] * (int)x[i];
        acc += a;
      }
      y = fmaf((float)acc, scale[c], bias ? bias[c] : 0.f);
    } else {
      const __half* in = (const __half*)in_;
      const __half* w = (const __half*)w_;
      float acc = 0.f;
      for (int k = 0; k < kvol; ++k) {
        int r = __ldg(map + (size_t)k * cap + row);
        if (r < 0) continue;
        const __half* x = in + (size_t)r * cin;
        const __half* wk = w + ((size_t)c * kvol + k) * cin;
        float a = 0.f;
        for (int i = 0; i < cin; ++i)
          a = __fadd_rn(a, __fmul_rn(__half2float(wk[i]), __half2float(x[i])));
        acc = __fadd_rn(acc, a);
      }
      y = __fadd_rn(acc, bias ? bias[c] : 0.f);
    }
    float r_deq = 0.f;
    if (ep.has_res) {
      if (ep.res_kind == SPCONVB_I8)
        r_deq = __fmul_rn((float)((const int8_t*)res_)[t], ep.res_scale);
      else
        r_deq = __half2float(((const __half*)res_)[t]);
    }
    float v = epilogue_value(y, ep, r_deq);
    if (ep.out_kind == SPCONVB_I8)
      ((int8_t*)out_)[t] = (int8_t)(int)v;
    else
      ((__half*)out_)[t] = __float2half_rn(v);
  }
}

int conv_simt_launch(const spconvb_conv_params& p, const void* in, const int32_t* map,
                     uint32_t cap, const uint32_t* n_out_ptr, uint32_t launch_rows,
                     const void* w_plain, const float* scale, const float* bias, void* out,
                     cudaStream_t st) {
  if (!w_plain) return SPCONVB_E_ARG;
  Epilogue ep = make_epilogue(p);
  unsigned long long work = (unsigned long long)launch_rows * p.cout;
  unsigned long long want = (work + 255) / 256;
  const unsigned long long most = (unsigned long long)kSmCount * 64;
  int blocks = (int)(want < most ? want : most);
  if (blocks < 1) blocks = 1;
  if (p.compute == SPCONVB_I8) {
    if (!scale) return SPCONVB_E_ARG;
    conv_simt_kernel<true><<<blocks, 256, 0, st>>>(in, map, cap, n_out_ptr, p.kvol, p.cin, p.cout,
                                                   w_plain, scale, bias, ep, p.res, out);
  } else {
    conv_simt_kernel<false><<<blocks, 256, 0, st>>>(in, map, cap, n_out_ptr, p.kvol, p.cin,
                                                    p.cout, w_plain, scale, bias, ep, p.res, out);
  }
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

}  // namespace spconvb
