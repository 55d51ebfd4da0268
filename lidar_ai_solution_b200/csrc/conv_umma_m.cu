// Sparse convolution as an implicit GEMM on the sm_100a tensor cores, voxel rows on
// the M side of the MMA (the variant used for narrow outputs, Cout <= 32).
//
//   out[o, :] = epilogue( sum_k  W[:, k, :] . in[map[k][o], :] )
//
// is a GEMM with M = output rows, N = Cout and K = kvol * Cin whose A operand
// does not exist in memory: row o of A is the concatenation of the feature
// rows of o's neighbours (zeros where a neighbour is absent).  The kernel is
// persistent (one CTA per SM, tiles of 128 output rows) and warp-specialised:
//
//   warps 0-3  epilogue: tcgen05.ld the accumulator tile out of TMEM, apply
//              dequant + bias + activation (+ residual add) + requant, store
//              one output row per thread with 16-byte stores
//   warp  4    allocates TMEM; one lane issues tcgen05.mma (kind::i8 with int32
//              accumulators or kind::f16 with fp32 accumulators)
//   warps 5-12 producers: prefetch the tile's neighbour indices one tile ahead,
//              gather the neighbour rows with 16-byte cp.async (8 lanes per
//              row, so a row is one contiguous request; zero-fill for missing
//              neighbours) straight into the 128-byte-swizzled K-major layout
//              the MMA reads, fence the generic-proxy writes for the async
//              proxy and arrive once per warp; thread 0 also streams the
//              pre-swizzled weight chunk with one bulk async copy
//
// K is walked in chunks of 128 bytes (one swizzle atom per row): a chunk is 8
// taps of a 16-byte row, ..., 1 tap of a 128-byte row, or half a 256-byte row.
// Stages cycle through a 6- to 8-deep ring guarded by mbarriers; the accumulator
// is double-buffered in TMEM so the epilogue of tile t overlaps the MMAs of t+1.
//
// Every wait is bounded: a wait that runs out sets SPCONVB_ST_TIMEOUT in the
// status block, raises a CTA-wide abort flag and all roles leave their loops,
// drain their copies and free TMEM.
#include "umma_common.cuh"

namespace spconvb {

using namespace umma_detail;

namespace {

constexpr int kTileM = 128;
// Depth of the stage ring: as deep as shared memory allows next to the index
// staging area, so that enough gather bytes are in flight to cover L2 latency.
template <int COUT>
struct Ring {
  static constexpr int kStages = COUT <= 32 ? 8 : (COUT == 64 ? 7 : 6);
  // A producer signals a stage "full" kLag chunks after issuing its copies; the
  // other kStages - kLag stages are slack for the round trip through the MMA.
  static constexpr int kLag = 2;
};
constexpr int kABytes = kTileM * kChunk;
constexpr int kEpiWarps = 4;
constexpr int kMmaWarp = 4;
constexpr int kProdWarp0 = 5;
constexpr int kProdThreads = 256;
constexpr int kCtaThreads = 32 * 5 + kProdThreads;

// 32-bit instruction descriptor: [4,6) D format (1 = f32, 2 = s32), [7,10) A
// format, [10,13) B format (f16 kind: 0 = f16; i8 kind: 1 = signed), bits 15/16
// A/B major (0 = K), [17,23) N>>3, [24,29) M>>4.
template <bool INT8, int COUT>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (INT8 ? ((2u << 4) | (1u << 7) | (1u << 10)) : (1u << 4)) |
         ((uint32_t)(COUT >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

template <int COUT>
constexpr size_t umma_smem_bytes() {
  return 1024 + (size_t)Ring<COUT>::kStages * (kABytes + COUT * kChunk) +
         2 * (kMaxTaps + 1) * kTileM * sizeof(int32_t) + 256 + 2 * COUT * sizeof(float);
}

// ------------------------------------------------------------------- kernel
template <bool INT8, int RB, int COUT>
__global__ void __launch_bounds__(kCtaThreads, 1) conv_umma_m_kernel(const UmmaArgs a) {
  constexpr int kBBytes = COUT * kChunk;
  constexpr int kStages = Ring<COUT>::kStages;
  constexpr int kLag = Ring<COUT>::kLag;
  constexpr uint32_t kTmemCols = (2 * COUT < 32) ? 32 : 2 * COUT;
  constexpr int OPC = RB <= kChunk ? kChunk / RB : 1;   // taps per chunk
  constexpr int SPO = RB <= kChunk ? RB / 16 : 8;       // 16-byte segments per tap per chunk
  constexpr int CPT = RB <= kChunk ? 1 : RB / kChunk;   // chunks per tap
  constexpr int OUT_MAX_B = 2;                          // bytes per output element (max)
  (void)OUT_MAX_B;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sA = smem;
  uint8_t* sB = sA + kStages * kABytes;
  int32_t* sIdx = (int32_t*)(sB + kStages * kBBytes);  // [2][kMaxTaps + 1][kTileM]
  uint64_t* bars = (uint64_t*)(sIdx + 2 * (kMaxTaps + 1) * kTileM);
  uint32_t* tmem_holder = (uint32_t*)(bars + 2 * kStages + 6);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  float* s_scale = (float*)(tmem_holder + 4);
  float* s_bias = s_scale + COUT;

  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_idx = bar_tempty + 16;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, kProdThreads / 32 + 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, kEpiWarps);
    }
    mbar_init(bar_idx, kProdThreads / 32);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 2 * kTileM; i += blockDim.x)
    sIdx[((i >> 7) * (kMaxTaps + 1) + kMaxTaps) * kTileM + (i & 127)] = -1;
  for (int i = threadIdx.x; i < COUT; i += blockDim.x) {
    s_scale[i] = a.scale ? a.scale[i] : 1.f;
    s_bias[i] = a.bias ? a.bias[i] : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const uint32_t n_out = min(*a.n_out_ptr, a.cap);
  const uint32_t ntiles = (n_out + kTileM - 1) / kTileM;
  const int kbytes = a.kvol * RB;
  const int nchunk = (kbytes + kChunk - 1) / kChunk;
  const int last_ksteps = ((kbytes - (nchunk - 1) * kChunk) + 31) / 32;

  if (warp >= kProdWarp0) {
    // ------------------------------------------------------------ producers
    // A chunk of the A tile is 128 rows x 8 segments of 16 bytes = 1024 copies,
    // 4 per producer thread.  Lanes run over the segments first (8 lanes per
    // row), so the lanes that read the same neighbour row ask for one contiguous
    // piece of it and a warp instruction touches 4..32 cache lines, not always 32.
    // The code is branch-free (missing neighbours are zero-filled copies) so the
    // index loads, address arithmetic and copies of the 4 items overlap.
    const uint32_t r = threadIdx.x - kProdWarp0 * 32;
    const uint32_t seg = r & 7u;           // 16-byte segment of the chunk this thread copies
    const uint32_t rb = r >> 3;            // rows rb, rb+32, rb+64, rb+96
    const uint32_t rsw = rb & 7u;
    const uint32_t dst_off = (rb >> 3) * 1024u + rsw * 128u + ((seg ^ rsw) << 4);
    // tap (within the chunk) and byte offset (within the neighbour row) of `seg`
    const uint32_t seg_tap = RB <= kChunk ? seg / SPO : 0u;
    const uint32_t seg_byte = RB <= kChunk ? (seg % SPO) * 16u : seg * 16u;
    // Neighbour indices: thread t fetches taps of parity t/128 of row t%128 into
    // registers one tile ahead, publishes them in shared memory (double
    // buffered); the producers meet on an mbarrier before gathering.
    constexpr int kFetch = (kMaxTaps + 1) / 2;
    const uint32_t frow = r & 127u, fpar = r >> 7;
    auto fetch_indices = [&](uint32_t tile, int32_t (&v)[kFetch]) {
      const uint32_t row = tile * kTileM + frow;
      const bool valid = tile < ntiles && row < n_out;
      const int32_t* src = a.map + row;
#pragma unroll
      for (int i = 0; i < kFetch; ++i) {
        const int k = 2 * i + (int)fpar;
        v[i] = (valid && k < a.kvol) ? __ldg(src + (size_t)k * a.cap) : -1;
      }
    };
    // mbarrier traffic is kept per warp: one lane polls and broadcasts, one lane
    // arrives after __syncwarp.
    auto warp_wait = [&](uint32_t bar, uint32_t parity, uint32_t where) -> bool {
      uint32_t ok = 1u;
      if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, a.status, where) ? 1u : 0u;
      return __shfl_sync(0xffffffffu, ok, 0) != 0u;
    };
    uint32_t it = 0, lt = 0;
    bool alive = true;
    int32_t nxt[kFetch];
    fetch_indices(blockIdx.x, nxt);
    for (uint32_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++lt) {
      int32_t* idx = sIdx + (size_t)(lt & 1u) * (kMaxTaps + 1) * kTileM;
#pragma unroll
      for (int i = 0; i < kFetch; ++i) idx[(2 * i + fpar) * kTileM + frow] = nxt[i];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_idx);
      fetch_indices(tile + gridDim.x, nxt);
      if (!warp_wait(bar_idx, lt & 1u, 5u)) {
        alive = false;
        break;
      }
      for (int j = 0; j < nchunk; ++j, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (!warp_wait(bar_empty + 8 * s, ph ^ 1u, 1u)) {
          alive = false;
          break;
        }
        if (r == 0) {
          mbar_expect_tx(bar_full + 8 * s, kBBytes);
          bulk_g2s(smem_u32(sB + s * kBBytes), a.wpk + (size_t)j * kBBytes, kBBytes,
                   bar_full + 8 * s);
        }
        const int k = (RB <= kChunk) ? j * OPC + (int)seg_tap : j / CPT;
        const uint32_t byte = seg_byte + (RB > kChunk ? (uint32_t)(j % CPT) * kChunk : 0u);
        // taps beyond kvol read the all -1 row kMaxTaps of the index buffer
        const int32_t* idx_k = idx + (k < a.kvol ? k : kMaxTaps) * kTileM + rb;
        const uint32_t dst0 = smem_u32(sA + s * kABytes) + dst_off;
        int32_t src_row[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) src_row[i] = idx_k[i * 32];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int32_t sr = src_row[i];
          cp_async16(dst0 + (uint32_t)i * 4096u, a.in + (size_t)(sr < 0 ? 0 : sr) * RB + byte,
                     sr < 0 ? 0u : 16u);
        }
        cp_async_commit();
        if (it >= (uint32_t)kLag) {
          cp_async_wait<kLag>();
          fence_proxy_async();  // generic-proxy writes -> async-proxy reads of the MMA
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full + 8 * ((it - kLag) % kStages));
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async();
    __syncwarp();
    if (alive && lane == 0) {
      const uint32_t first = it > (uint32_t)kLag ? it - kLag : 0u;
      for (uint32_t i = first; i < it; ++i) mbar_arrive(bar_full + 8 * (i % kStages));
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // The tensor pipe takes one MMA at a time (about M cycles each), and issuing the
      // next one blocks until it is free.  Everything that is not an MMA therefore sits
      // between the second-to-last and the last MMA of a chunk, or is short: the next
      // stage's barrier is probed while the pipe is busy, so that the first MMA of the
      // next chunk can follow the last one of this chunk without a bubble.
      constexpr uint32_t idesc = make_idesc<INT8, COUT>();
      const uint64_t adesc0 = make_smem_desc(smem_u32(sA));
      const uint64_t bdesc0 = make_smem_desc(smem_u32(sB));
      uint32_t s = 0, ph = 0, tl = 0;
      bool ready = false;  // full[s] already seen complete by a probe
      bool alive = true;
      for (uint32_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tl) {
        const uint32_t buf = tl & 1u;
        if (!mbar_wait(bar_tempty + 8 * buf, ((tl >> 1) & 1u) ^ 1u, abort_flag, a.status, 2u))
          break;
        const uint32_t d_tmem = tmem_base + buf * COUT;
        for (int j = 0; j < nchunk; ++j) {
          if (!ready && !mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, 3u)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint64_t ad = adesc0 + (uint64_t)(s * (uint32_t)(kABytes >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (uint32_t)(kBBytes >> 4));
          const int nk = (j == nchunk - 1) ? last_ksteps : kChunk / 32;
          for (int ks = 0; ks + 1 < nk; ++ks)
            umma<INT8>(d_tmem, ad + 2u * ks, bd + 2u * ks, idesc, (uint32_t)((j | ks) != 0));
          const uint32_t s1 = s + 1 == (uint32_t)kStages ? 0u : s + 1;
          const uint32_t ph1 = s1 == 0u ? ph ^ 1u : ph;
          ready = mbar_try_wait(bar_full + 8 * s1, ph1);
          umma<INT8>(d_tmem, ad + 2u * (nk - 1), bd + 2u * (nk - 1), idesc,
                     (uint32_t)((j | (nk - 1)) != 0));
          tc_commit(bar_empty + 8 * s);
          s = s1;
          ph = ph1;
        }
        if (alive) tc_commit(bar_tfull + 8 * buf);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue
    const Epilogue ep = a.ep;
    const int out_b = ep.out_kind == SPCONVB_I8 ? 1 : 2;
    const int res_b = ep.res_kind == SPCONVB_I8 ? 1 : 2;
    uint32_t tl = 0;
    for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tl) {
      const uint32_t buf = tl & 1u;
      const uint32_t row = tile * kTileM + warp * 32 + lane;
      // the residual row is fetched before the accumulator is waited for, so its
      // latency hides behind the tile's MMAs
      constexpr int kResVecs = COUT / 8;  // 16-byte vectors of an fp16 row (int8: half of them)
      uint4 rres[kResVecs];
      if (ep.has_res && row < n_out) {
        const uint4* rp = (const uint4*)(a.res + (size_t)row * COUT * res_b);
        const int nv = ep.res_kind == SPCONVB_I8 ? COUT / 16 : COUT / 8;
#pragma unroll
        for (int i = 0; i < kResVecs; ++i)
          if (i < nv) rres[i] = __ldg(rp + i);
      }
      uint32_t ok = 1u;
      if (lane == 0)
        ok = mbar_wait(bar_tfull + 8 * buf, (tl >> 1) & 1u, abort_flag, a.status, 4u) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * COUT;
#pragma unroll
      for (int c0 = 0; c0 < COUT; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(taddr + c0, v);
        tmem_ld_wait();
        if (c0 + 16 == COUT) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        }
        if (row < n_out) {
          // Same arithmetic as common.cuh:epilogue_value, written so that the per-element
          // work is a handful of instructions: vector loads of scale and bias, ReLU as a
          // max with 0 or -inf, float -> int8 as one saturating round-to-nearest-even
          // convert, and the layer-wide switches hoisted out of the element loops.
          float y[16];
          const float lo = ep.act == SPCONVB_ACT_RELU ? 0.f : -INFINITY;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const float4 bi = ((const float4*)(s_bias + c0))[g];
            if (INT8) {
              const float4 sc = ((const float4*)(s_scale + c0))[g];
              y[4 * g + 0] = fmaxf(fmaf((float)(int)v[4 * g + 0], sc.x, bi.x), lo);
              y[4 * g + 1] = fmaxf(fmaf((float)(int)v[4 * g + 1], sc.y, bi.y), lo);
              y[4 * g + 2] = fmaxf(fmaf((float)(int)v[4 * g + 2], sc.z, bi.z), lo);
              y[4 * g + 3] = fmaxf(fmaf((float)(int)v[4 * g + 3], sc.w, bi.w), lo);
            } else {
              y[4 * g + 0] = fmaxf(__fadd_rn(__uint_as_float(v[4 * g + 0]), bi.x), lo);
              y[4 * g + 1] = fmaxf(__fadd_rn(__uint_as_float(v[4 * g + 1]), bi.y), lo);
              y[4 * g + 2] = fmaxf(__fadd_rn(__uint_as_float(v[4 * g + 2]), bi.z), lo);
              y[4 * g + 3] = fmaxf(__fadd_rn(__uint_as_float(v[4 * g + 3]), bi.w), lo);
            }
          }
          if (ep.has_res) {
            // the conv result as it would have been stored (mid), plus the residual
            float r[16];
            if (ep.res_kind == SPCONVB_I8) {
              const uint4 q = rres[c0 / 16];
              const int8_t* qb = (const int8_t*)&q;
#pragma unroll
              for (int i = 0; i < 16; ++i) r[i] = __fmul_rn((float)qb[i], ep.res_scale);
            } else {
              const uint4 q0 = rres[(c0 / 8) % kResVecs];
              const uint4 q1 = rres[(c0 / 8 + 1) % kResVecs];
              const __half* h0 = (const __half*)&q0;
              const __half* h1 = (const __half*)&q1;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                r[i] = __half2float(h0[i]);
                r[8 + i] = __half2float(h1[i]);
              }
            }
            const float lo2 = ep.res_relu ? 0.f : -INFINITY;
            if (ep.mid_kind == SPCONVB_I8) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float m = __fmul_rn((float)cvt_sat_s8(__fmul_rn(y[i], ep.mid_inv_scale)),
                                          ep.mid_scale);
                y[i] = fmaxf(__fadd_rn(m, r[i]), lo2);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                y[i] = fmaxf(__fadd_rn(__half2float(__float2half_rn(y[i])), r[i]), lo2);
            }
          }
          uint8_t* op = a.out + ((size_t)row * COUT + c0) * out_b;
          if (ep.out_kind == SPCONVB_I8) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              w[i] = pack_s8x4(cvt_sat_s8(__fmul_rn(y[4 * i + 0], ep.inv_out_scale)),
                               cvt_sat_s8(__fmul_rn(y[4 * i + 1], ep.inv_out_scale)),
                               cvt_sat_s8(__fmul_rn(y[4 * i + 2], ep.inv_out_scale)),
                               cvt_sat_s8(__fmul_rn(y[4 * i + 3], ep.inv_out_scale)));
            *(uint4*)op = make_uint4(w[0], w[1], w[2], w[3]);
          } else {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              __half2 h = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
              w[i] = *(uint32_t*)&h;
            }
            *(uint4*)op = make_uint4(w[0], w[1], w[2], w[3]);
            *(uint4*)(op + 16) = make_uint4(w[4], w[5], w[6], w[7]);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies already issued a bounded time to land before the CTA exits
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 50000ull) {
    }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

template <bool INT8, int RB, int COUT>
int launch_one(const UmmaArgs& args, uint32_t launch_rows, cudaStream_t st) {
  static bool attr_done[64] = {};
  int dev = 0;
  SPCONVB_CUDA_TRY(cudaGetDevice(&dev));
  constexpr size_t smem = umma_smem_bytes<COUT>();
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    SPCONVB_CUDA_TRY(cudaFuncSetAttribute(conv_umma_m_kernel<INT8, RB, COUT>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  uint32_t tiles = (launch_rows + kTileM - 1) / kTileM;
  int grid = (int)(tiles < (uint32_t)kSmCount ? (tiles ? tiles : 1u) : (uint32_t)kSmCount);
  conv_umma_m_kernel<INT8, RB, COUT><<<grid, kCtaThreads, smem, st>>>(args);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

template <bool INT8, int RB>
int launch_cout(int cout, const UmmaArgs& args, uint32_t launch_rows, cudaStream_t st) {
  switch (cout) {
    case 16: return launch_one<INT8, RB, 16>(args, launch_rows, st);
    case 32: return launch_one<INT8, RB, 32>(args, launch_rows, st);
    case 64: return launch_one<INT8, RB, 64>(args, launch_rows, st);
    case 128: return launch_one<INT8, RB, 128>(args, launch_rows, st);
  }
  return SPCONVB_E_UNSUPPORTED;
}

template <bool INT8>
int launch_rb(int rb, int cout, const UmmaArgs& args, uint32_t launch_rows, cudaStream_t st) {
  switch (rb) {
    case 16: return launch_cout<INT8, 16>(cout, args, launch_rows, st);
    case 32: return launch_cout<INT8, 32>(cout, args, launch_rows, st);
    case 64: return launch_cout<INT8, 64>(cout, args, launch_rows, st);
    case 128: return launch_cout<INT8, 128>(cout, args, launch_rows, st);
    case 256: return launch_cout<INT8, 256>(cout, args, launch_rows, st);
  }
  return SPCONVB_E_UNSUPPORTED;
}

}  // namespace

int conv_umma_m_launch(const UmmaArgs& a, bool int8, int rb, int cout, uint32_t launch_rows,
                       cudaStream_t st) {
  return int8 ? launch_rb<true>(rb, cout, a, launch_rows, st)
              : launch_rb<false>(rb, cout, a, launch_rows, st);
}

}  // namespace spconvb
