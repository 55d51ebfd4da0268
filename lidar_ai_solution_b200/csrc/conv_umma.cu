// Tensor-core convolution, host side: the supported shapes, the pre-swizzled weight
// image the kernel streams, argument checks and the launch.
#include <stdlib.h>

#include "umma_common.cuh"

namespace spconvb {

using namespace umma_detail;

int conv_umma_kernel_launch(const UmmaArgs& a, bool int8, int rb, int cout, uint32_t launch_rows,
                            size_t smem, cudaStream_t st);

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

// Launch configuration: copies of the weights along the accumulator rows, residency of the
// weights, depth of the row-stage ring, and how far the L2 prefetch runs ahead.
struct UmmaConfig {
  int w_rep;
  int w_resident;
  int nstages;
  int prefetch;
  size_t smem;
};

// Tuning overrides, read once: SPCONVB_CONV_M (64 or 128 accumulator rows), SPCONVB_CONV_RESIDENT
// (0 / 1), SPCONVB_CONV_STAGES (2..6), SPCONVB_CONV_PREFETCH (tiles ahead, 0 = off).  Unset or
// out of range: the built-in choice.  Results do not depend on any of them.
static int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  if (!v || !*v) return fallback;
  return atoi(v);
}

static bool config_fits(int cout, int nchunk, int rep, int resident, int stages, size_t* smem) {
  *smem = umma_smem_bytes(cout, nchunk, rep, resident, stages);
  return *smem <= 232448;
}

// Measured on the B200 (layer sweep, 200 k - 1 M rows, every channel width): streaming the
// weight chunk with every stage, copied to all 128 accumulator rows, is as fast as or faster
// than keeping the weights resident, because it leaves the deepest ring of row stages and
// lets all lanes of the 8 epilogue warps work (with 64 accumulator rows half of them carry
// nothing, and the epilogue of a tile then outlasts the next tile's main loop).  The weight
// chunk comes from L2 by one bulk copy per stage and costs no producer instructions.  So:
// stream with the most copies; resident configurations remain for the overrides.
static UmmaConfig choose_config(int rb, int cout, int kvol) {
  static const int force_m = env_int("SPCONVB_CONV_M", 0);
  static const int force_res = env_int("SPCONVB_CONV_RESIDENT", -1);
  static const int force_stages = env_int("SPCONVB_CONV_STAGES", 0);
  // Off by default: with the current producers the bulk L2 prefetch of a tile's map lines,
  // input rows and residual rows costs 1-4 % at every batch size (it was worth 3-5 % before the
  // indices moved into registers and the producers were split into two groups).
  static const int prefetch = env_int("SPCONVB_CONV_PREFETCH", 0);
  const int nchunk = (kvol * rb + kChunk - 1) / kChunk;
  const int full = 128 / cout, half = cout <= 64 ? 64 / cout : 0;
  auto best_stages = [&](int rep, int resident) {
    size_t smem;
    int st = 0;
    for (int n = 2; n <= kMaxStages; ++n)
      if (config_fits(cout, nchunk, rep, resident, n, &smem)) st = n;
    if (force_stages >= 2 && force_stages <= st) st = force_stages;
    return st;
  };
  struct Cand { int rep, resident, need; };
  Cand order[4] = {{full, 0, 2}, {half, 0, 2}, {full, 1, 2}, {half, 1, 2}};
  UmmaConfig c{};
  for (const Cand& o : order) {
    if (o.rep < 1) continue;
    if (force_m == 64 && o.rep != half) continue;
    if (force_m == 128 && o.rep != full) continue;
    if (force_res >= 0 && o.resident != force_res) continue;
    const int st = best_stages(o.rep, o.resident);
    if (st < o.need) continue;
    c.w_rep = o.rep;
    c.w_resident = o.resident;
    c.nstages = st;
    break;
  }
  if (c.nstages == 0) {  // the overrides excluded everything: fall back to streaming, full rows
    c.w_rep = full;
    c.w_resident = 0;
    c.nstages = best_stages(full, 0);
  }
  c.prefetch = prefetch < 0 ? 0 : (prefetch > 8 ? 8 : prefetch);
  c.smem = umma_smem_bytes(cout, nchunk, c.w_rep, c.w_resident, c.nstages);
  return c;
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
  a.n_in_ptr = p.cap_in ? p.n_in_ptr : nullptr;
  a.cap_in = p.cap_in;
  a.kvol = p.kvol;
  a.wait_test = p.wait_test;
  const int rb = row_bytes(p.compute, p.cin);
  const UmmaConfig c = choose_config(rb, p.cout, p.kvol);
  if (c.nstages < 2) return SPCONVB_E_UNSUPPORTED;
  a.w_rep = c.w_rep;
  a.w_resident = c.w_resident;
  a.nstages = c.nstages;
  a.prefetch = c.prefetch;
  a.ep = make_epilogue(p);
  return conv_umma_kernel_launch(a, p.compute == SPCONVB_I8, rb, p.cout, launch_rows, c.smem, st);
}

}  // namespace spconvb
