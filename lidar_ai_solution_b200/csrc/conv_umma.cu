// Tensor-core convolution, host side: the supported shapes, the pre-swizzled weight
// image the kernel streams, argument checks and the launch.
#include "umma_common.cuh"

namespace spconvb {

using namespace umma_detail;

int conv_umma_kernel_launch(const UmmaArgs& a, bool int8, int rb, int cout, uint32_t launch_rows,
                       cudaStream_t st);

bool conv_umma_supported(int compute, int cin, int cout) {
  const int rb = row_bytes(compute, cin);
  const bool rb_ok = rb == 16 || rb == 32 || rb == 64 || rb == 128 || (rb == 256);
  const bool co_ok = cout == 16 || cout == 32 || cout == 64 || cout == 128;
  return (compute == SPCONVB_I8 || compute == SPCONVB_F16) && rb_ok && co_ok;
}

size_t conv_umma_packed_bytes(int compute, int cin, int cout, int kvol) {
  const size_t kbytes = (size_t)kvol * row_bytes(compute, cin);
  const size_t nchunk = (kbytes + kChunk - 1) / kChunk;
  return nchunk * (size_t)cout * kChunk;
}

// Host: lay the weights out as the shared-memory image of each 128-byte K chunk
// (row n of a chunk = bytes [j*128, j*128+128) of W[n] flattened over (tap, cin),
// zero padded; 16-byte segment c of row n stored at segment c ^ (n % 8)).
int conv_umma_pack(int compute, int cin, int cout, int kvol, const void* w, void* dst) {
  if (!conv_umma_supported(compute, cin, cout) || !w || !dst || kvol < 1) return SPCONVB_E_ARG;
  const size_t rowlen = (size_t)kvol * row_bytes(compute, cin);
  const size_t nchunk = (rowlen + kChunk - 1) / kChunk;
  const uint8_t* src = (const uint8_t*)w;
  uint8_t* out = (uint8_t*)dst;
  for (size_t j = 0; j < nchunk; ++j)
    for (int n = 0; n < cout; ++n)
      for (int c = 0; c < 8; ++c) {
        uint8_t* d = out + j * (size_t)cout * kChunk + (size_t)(n / 8) * 1024 + (n % 8) * 128 +
                     ((c ^ (n % 8)) << 4);
        const size_t kb = j * kChunk + (size_t)c * 16;
        for (int b = 0; b < 16; ++b)
          d[b] = (kb + b < rowlen) ? src[(size_t)n * rowlen + kb + b] : (uint8_t)0;
      }
  return SPCONVB_OK;
}

int conv_umma_launch(const spconvb_conv_params& p, const void* in, const int32_t* map,
                     uint32_t cap, const uint32_t* n_out_ptr, uint32_t launch_rows,
                     const void* w_packed, const float* scale, const float* bias, void* out,
                     uint32_t* status, cudaStream_t st) {
  if (!w_packed) return SPCONVB_E_ARG;
  if (p.kvol > kMaxTaps) return SPCONVB_E_UNSUPPORTED;
  if (p.compute == SPCONVB_I8 && !scale) return SPCONVB_E_ARG;
  if (((uintptr_t)in | (uintptr_t)out | (uintptr_t)w_packed | (uintptr_t)p.res) & 15u)
    return SPCONVB_E_ARG;
  UmmaArgs a;
  a.in = (const uint8_t*)in;
  a.map = map;
  a.cap = cap;
  a.n_out_ptr = n_out_ptr;
  a.wpk = (const uint8_t*)w_packed;
  a.scale = p.compute == SPCONVB_I8 ? scale : nullptr;
  a.bias = bias;
  a.res = (const uint8_t*)p.res;
  a.out = (uint8_t*)out;
  a.status = status;
  a.kvol = p.kvol;
  a.wait_test = p.wait_test;
  // Copies of the weights along the accumulator lanes, and residency.  Every copy lets
  // more epilogue warps share a tile, but a streamed stage always moves 128 weight rows,
  // as much L2 traffic as the gathered rows cost.  So: the most copies with which all
  // chunks of the layer still fit in the 64 KB the weight stages occupy, loaded once;
  // if not even one copy fits, stream with full replication.
  {
    const int rbytes = row_bytes(p.compute, p.cin);
    const size_t nchunk = ((size_t)p.kvol * rbytes + kChunk - 1) / kChunk;
    const int full = 128 / p.cout;
    int rep = full;
    while (rep >= 1 && nchunk * (size_t)rep * p.cout * kChunk > 65536) rep /= 2;
    a.w_resident = rep >= 1;
    a.w_rep = rep >= 1 ? rep : full;
  }
  a.ep = make_epilogue(p);
  const int rb = row_bytes(p.compute, p.cin);
  return conv_umma_kernel_launch(a, p.compute == SPCONVB_I8, rb, p.cout, launch_rows, st);
}

}  // namespace spconvb
