// Sparse convolution as an implicit GEMM on the sm_100a tensor cores, voxel rows on
// the N side of the MMA.
//
//   out[o, :] = epilogue( sum_k  W[:, k, :] . in[map[k][o], :] )
//
// is a GEMM between the weights [Cout x K] and a matrix [rows x K], K = kvol *
// Cin, that does not exist in memory: its row o is the concatenation of the
// feature rows of o's neighbours (zeros where a neighbour is absent).  A
// tcgen05.mma with 128 accumulator lanes takes the same time whether it is 16
// or 256 columns wide, so the voxel rows are put on the wide side: the weights
// are the M operand (128 accumulator lanes = output channels), a tile of 256
// voxel rows is the N operand, and the accumulator in TMEM is the transposed
// output tile  D[channel][row].  With fewer than 128 output channels the weight
// chunk is copied several times into the M operand, so that more lane quadrants
// hold all channels and the epilogue warps of different quadrants can share the
// rows of the tile between them instead of idling.  When all chunks of the layer
// (times the copies) fit in 64 KB they are loaded once and stay in shared memory;
// otherwise a chunk is streamed with every stage.  Streaming costs as much L2
// traffic as the gathers themselves (128 weight rows per 256 gathered rows), so
// the host side trades copies for residency.  The kernel is persistent (one CTA
// per SM) and warp-specialised:
//
//   warps 0-7   epilogue: warp w reads lanes 32*(w%4).. (its channels) and
//               Cout columns (its share of the tile's rows) of the accumulator with
//               tcgen05.ld, applies dequant + bias + activation (+ residual
//               add) + requant with per-lane scale and bias, transposes 4x4
//               blocks inside lane quads with two shuffles, and stores 4 (int8)
//               or 8 (fp16) contiguous bytes of one output row per lane
//   warp  8     allocates TMEM; one lane issues tcgen05.mma (kind::i8 with int32
//               accumulators or kind::f16 with fp32 accumulators)
//   warps 9-16  producers: each warp owns 32 rows of the tile.  It prefetches
//               their neighbour indices one tile ahead into registers and
//               stages them in its own piece of shared memory (no CTA-wide
//               synchronisation), gathers the neighbour rows with 16-byte
//               cp.async (8 lanes per row, so a row is one contiguous request;
//               zero-fill for missing neighbours) straight into the
//               128-byte-swizzled K-major layout the MMA reads, fences the
//               generic-proxy writes for the async proxy and arrives once per
//               warp; one thread also streams the pre-swizzled weight chunk
//               with one bulk async copy
//
// K is walked in chunks of 128 bytes (one swizzle atom per row): a chunk is 8
// taps of a 16-byte row, ..., 1 tap of a 128-byte row, or half a 256-byte row.
// Stages cycle through a 4-deep ring guarded by mbarriers; the accumulator
// is double-buffered in TMEM (2 x 256 columns) so the epilogue of tile t
// overlaps the MMAs of tile t+1.
//
// Every wait is bounded: a wait that runs out sets SPCONVB_ST_TIMEOUT in the
// status block, raises a CTA-wide abort flag and all roles leave their loops,
// drain their copies and free TMEM.
#include "umma_common.cuh"

namespace spconvb {

using namespace umma_detail;

namespace {

constexpr int kTileRows = 256;  // most voxel rows per tile: the largest N of the MMA
constexpr int kMmaM = 128;      // accumulator lanes: output channels, padded
// Stage ring: as deep as shared memory allows next to the index staging area (a stage is
// 32 KB of rows + 16 KB of weights).  A producer signals a stage "full" kLag chunks after
// issuing its copies; the other kStages - kLag stages are slack for the round trip
// through the MMA.
constexpr int kStages = 4;
constexpr int kLag = 1;
constexpr int kRowsBytes = kTileRows * kChunk;  // gathered rows of one stage
constexpr int kEpiWarps = 8;
constexpr int kMmaWarp = 8;
constexpr int kProdWarp0 = 9;
constexpr int kProdThreads = 256;
constexpr int kCtaThreads = 32 * kProdWarp0 + kProdThreads;
constexpr uint32_t kTmemCols = 2 * kTileRows;

// 32-bit instruction descriptor: [4,6) D format (1 = f32, 2 = s32), [7,10) A
// format, [10,13) B format (f16 kind: 0 = f16; i8 kind: 1 = signed), bits 15/16
// A/B major (0 = K), [17,23) N>>3, [24,29) M>>4.
template <bool INT8>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (INT8 ? ((2u << 4) | (1u << 7) | (1u << 10)) : (1u << 4)) |
         ((uint32_t)(kMmaM >> 4) << 24);  // N is added per launch: (tile rows >> 3) << 17
}

// Transposes inside a quad of lanes (lane = 4g + j): they turn "my channel for a
// few rows" into "4 adjacent channels of one row", and back.
// A 16 x 4 byte block spread over a quad: lane j holds 4 words, word t = bytes of 4
// consecutive rows 4t..4t+3 of channel j.  quad_words_transpose gives lane j word j
// of every lane (2 x 2 shuffles); bytes_transpose4 then turns "word c = 4 rows of
// channel c" into "word r = 4 channels of row r" inside the lane.  Together: lane j
// holds rows 4j..4j+3 of the 4 channels, one word per row.  The inverse applies the
// two steps in the opposite order (each is its own inverse).
__device__ __forceinline__ void quad_words_transpose(uint32_t (&w)[4], uint32_t lane) {
  const bool odd = lane & 1u, hi = lane & 2u;
  uint32_t s0 = odd ? w[0] : w[1], s1 = odd ? w[2] : w[3];
  s0 = __shfl_xor_sync(0xffffffffu, s0, 1);
  s1 = __shfl_xor_sync(0xffffffffu, s1, 1);
  const uint32_t a0 = odd ? s0 : w[0], a1 = odd ? w[1] : s0;
  const uint32_t a2 = odd ? s1 : w[2], a3 = odd ? w[3] : s1;
  uint32_t u0 = hi ? a0 : a2, u1 = hi ? a1 : a3;
  u0 = __shfl_xor_sync(0xffffffffu, u0, 2);
  u1 = __shfl_xor_sync(0xffffffffu, u1, 2);
  w[0] = hi ? u0 : a0;
  w[1] = hi ? u1 : a1;
  w[2] = hi ? a2 : u0;
  w[3] = hi ? a3 : u1;
}
__device__ __forceinline__ void bytes_transpose4(uint32_t (&w)[4]) {
  const uint32_t l01 = __byte_perm(w[0], w[1], 0x5140), h01 = __byte_perm(w[0], w[1], 0x7362);
  const uint32_t l23 = __byte_perm(w[2], w[3], 0x5140), h23 = __byte_perm(w[2], w[3], 0x7362);
  w[0] = __byte_perm(l01, l23, 0x5410);
  w[1] = __byte_perm(l01, l23, 0x7632);
  w[2] = __byte_perm(h01, h23, 0x5410);
  w[3] = __byte_perm(h01, h23, 0x7632);
}
// 16-bit elements: lane j holds 4 halves e[0..3] in two words; afterwards it holds
// element j of lanes 0..3 of its quad, in lane order (the call is its own inverse).
__device__ __forceinline__ void quad_transpose_h16(uint32_t& w0, uint32_t& w1, uint32_t lane) {
  const bool odd = lane & 1u;
  const uint32_t send = __byte_perm(w0, w1, odd ? 0x5410 : 0x7632);
  const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
  w0 = __byte_perm(w0, recv, odd ? 0x3254 : 0x5410);
  w1 = __byte_perm(w1, recv, odd ? 0x3276 : 0x7610);
  const bool hi = lane & 2u;
  const uint32_t other = __shfl_xor_sync(0xffffffffu, hi ? w0 : w1, 2);
  if (hi) w0 = other; else w1 = other;
}

constexpr size_t umma_smem_bytes() {
  return 1024 + (size_t)kStages * (kRowsBytes + kMmaM * kChunk) +
         (size_t)kMaxTaps * kTileRows * sizeof(int32_t) + 256;
}

// ------------------------------------------------------------------- kernel
template <bool INT8, int RB, int COUT>
__global__ void __launch_bounds__(kCtaThreads, 1) conv_umma_kernel(const UmmaArgs a) {
  constexpr int kWBytes = kMmaM * kChunk;      // weight stage when streaming: 128 rows
  constexpr int kWChunk = COUT * kChunk;       // one copy of a chunk, as packed in global memory
  constexpr int OPC = RB <= kChunk ? kChunk / RB : 1;   // taps per chunk
  constexpr int SPO = RB <= kChunk ? RB / 16 : 8;       // 16-byte segments per tap per chunk
  constexpr int CPT = RB <= kChunk ? 1 : RB / kChunk;   // chunks per tap

  // Shared memory: the weight stages (128 rows each: the replicated chunk), the
  // gathered-row stages, the producers' neighbour indices of the current tile, the
  // barriers.
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sW = smem;
  uint8_t* sR = sW + kStages * kWBytes;
  int32_t* sIdx = (int32_t*)(sR + kStages * kRowsBytes);  // [kMaxTaps][kTileRows]
  uint64_t* bars = (uint64_t*)(sIdx + kMaxTaps * kTileRows);
  uint32_t* tmem_holder = (uint32_t*)(bars + 2 * kStages + 5);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_w = bar_tempty + 16;  // resident weights have landed

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, kProdThreads / 32 + 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, kEpiWarps);
    }
    mbar_init(bar_w, 1);
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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const uint32_t n_out = min(*a.n_out_ptr, a.cap);
  // Tile height: the rows are dealt out in rounds over the CTAs, so a fixed 256-row tile
  // can leave most CTAs idle in the last round (227 tiles on 148 CTAs run as long as 296).
  // The height is instead the smallest multiple of 32 with which every CTA gets the same
  // number of tiles: per-CTA rows / rounds, rounded up.
  const uint32_t per_cta = (n_out + gridDim.x - 1) / gridDim.x;
  const uint32_t rounds = max(1u, (per_cta + kTileRows - 1) / kTileRows);
  const uint32_t tile_rows =
      min((uint32_t)kTileRows, max(32u, ((per_cta + rounds - 1) / rounds + 31u) & ~31u));
  const uint32_t ntiles = (n_out + tile_rows - 1) / tile_rows;
  const int kbytes = a.kvol * RB;
  const int nchunk = (kbytes + kChunk - 1) / kChunk;
  const int last_ksteps = ((kbytes - (nchunk - 1) * kChunk) + 31) / 32;
  const uint32_t w_rep = (uint32_t)a.w_rep;
  const bool w_resident = a.w_resident != 0;
  const uint32_t w_chunk_smem = w_rep * kWChunk;  // bytes of one chunk with its copies

  if (warp >= kProdWarp0) {
    // ------------------------------------------------------------ producers
    // A chunk of the row tile is 256 rows x 8 segments of 16 bytes = 2048 copies,
    // 8 per producer thread.  Producer warp w owns rows 32w..32w+31; lanes run over
    // the segments first (8 lanes per row), so the lanes that read the same
    // neighbour row ask for one contiguous piece of it and a warp instruction
    // touches 4..32 cache lines, not always 32.  The code is branch-free (missing
    // neighbours are zero-filled copies) so the index loads, address arithmetic and
    // copies of the 8 items overlap.
    const uint32_t pw = (uint32_t)warp - kProdWarp0;
    const uint32_t r = threadIdx.x - kProdWarp0 * 32;  // thread 0 also copies the weights
    const uint32_t seg = lane & 7u;        // 16-byte segment of the chunk this thread copies
    const uint32_t slot = lane >> 3;       // rows 32w + slot + 4i, i = 0..7
    // row R of the tile lives at (R / 8) * 1024 + (R % 8) * 128, its segments XOR-ed
    // with R % 8; R % 8 is slot for even i and slot + 4 for odd i
    const uint32_t dst_even = pw * 4096u + slot * 128u + ((seg ^ slot) << 4);
    const uint32_t dst_odd = pw * 4096u + (slot + 4u) * 128u + ((seg ^ (slot + 4u)) << 4);
    // tap (within the chunk) and byte offset (within the neighbour row) of `seg`
    const uint32_t seg_tap = RB <= kChunk ? seg / SPO : 0u;
    const uint32_t seg_byte = RB <= kChunk ? (seg % SPO) * 16u : seg * 16u;
    // Neighbour indices: lane l fetches the taps of row 32w + l of the next tile
    // into registers while the current tile is gathered, and stores them in the
    // warp's own staging area when the warp is done with the current tile.  The area
    // is [tap][slot][i] for row slot + 4i, so that the 8 indices a gathering thread
    // needs for a tap are two 16-byte loads.
    int32_t* widx = sIdx + pw * (kMaxTaps * 32);
    auto fetch_indices = [&](uint32_t tile, int32_t (&v)[kMaxTaps]) {
      const uint32_t row = tile * tile_rows + pw * 32u + lane;
      const bool valid = tile < ntiles && row < n_out && pw * 32u < tile_rows;
      const int32_t* src = a.map + row;
#pragma unroll
      for (int k = 0; k < kMaxTaps; ++k)
        v[k] = (valid && k < a.kvol) ? __ldg(src + (size_t)k * a.cap) : -1;
    };
    // mbarrier traffic is kept per warp: one lane polls and broadcasts, one lane
    // arrives after __syncwarp.
    auto warp_wait = [&](uint32_t bar, uint32_t parity, uint32_t where) -> bool {
      uint32_t ok = 1u;
      if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, a.status, where) ? 1u : 0u;
      return __shfl_sync(0xffffffffu, ok, 0) != 0u;
    };
    uint32_t it = 0;
    bool alive = true;
    const bool has_rows = pw * 32u < tile_rows;  // else this warp only keeps the barriers going
    int32_t nxt[kMaxTaps];
    fetch_indices(blockIdx.x, nxt);
    if (r == 0 && w_resident && blockIdx.x < ntiles) {
      mbar_expect_tx(bar_w, (uint32_t)nchunk * w_chunk_smem);
      for (int j = 0; j < nchunk; ++j)
        for (uint32_t c = 0; c < w_rep; ++c)
          bulk_g2s(smem_u32(sW + j * w_chunk_smem + c * kWChunk), a.wpk + (size_t)j * kWChunk,
                   kWChunk, bar_w);
    }
    for (uint32_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
      __syncwarp();  // the warp's reads of the previous tile's indices are done
#pragma unroll
      for (int k = 0; k < kMaxTaps; ++k) widx[k * 32 + (lane & 3u) * 8u + (lane >> 2)] = nxt[k];
      __syncwarp();
      fetch_indices(tile + gridDim.x, nxt);
      for (int j = 0; j < nchunk; ++j, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (!warp_wait(bar_empty + 8 * s, ph ^ 1u, 1u)) {
          alive = false;
          break;
        }
        if (r == 0) {
          if (w_resident) {
            mbar_arrive(bar_full + 8 * s);
          } else {
            mbar_expect_tx(bar_full + 8 * s, w_chunk_smem);
            for (uint32_t c = 0; c < w_rep; ++c)
              bulk_g2s(smem_u32(sW + s * kWBytes + c * kWChunk), a.wpk + (size_t)j * kWChunk,
                       kWChunk, bar_full + 8 * s);
          }
        }
        const int k = (RB <= kChunk) ? j * OPC + (int)seg_tap : j / CPT;
        const uint32_t byte = seg_byte + (RB > kChunk ? (uint32_t)(j % CPT) * kChunk : 0u);
        // taps beyond the staged ones (K padding of the last chunk) gather nothing;
        // staged taps beyond kvol hold -1
        const bool staged = k < kMaxTaps;
        if (has_rows) {
          const int4* idx_k = (const int4*)(widx + (staged ? k : 0) * 32 + slot * 8u);
          const uint32_t stage_addr = smem_u32(sR + s * kRowsBytes);
          const int4 ia = idx_k[0], ib = idx_k[1];
          int32_t src_row[8] = {ia.x, ia.y, ia.z, ia.w, ib.x, ib.y, ib.z, ib.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) src_row[i] = staged ? src_row[i] : -1;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int32_t sr = src_row[i];
            cp_async16(stage_addr + ((i & 1) ? dst_odd : dst_even) + (uint32_t)(i >> 1) * 1024u,
                       a.in + (size_t)(sr < 0 ? 0 : sr) * RB + byte, sr < 0 ? 0u : 16u);
          }
        }
        cp_async_commit();
        if (it >= (uint32_t)kLag) {
          cp_async_wait<kLag>();
          fence_proxy_async();  // generic-proxy writes -> async-proxy reads of the MMA
          __syncwarp();
          if (lane == 0 && !(a.wait_test > 0 && it - kLag + 1u >= (uint32_t)a.wait_test))
            mbar_arrive(bar_full + 8 * ((it - kLag) % kStages));
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async();
    __syncwarp();
    if (alive && lane == 0) {
      const uint32_t first = it > (uint32_t)kLag ? it - kLag : 0u;
      for (uint32_t i = first; i < it; ++i)
        if (!(a.wait_test > 0 && i + 1u >= (uint32_t)a.wait_test))
          mbar_arrive(bar_full + 8 * (i % kStages));
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // The tensor pipe takes one MMA at a time, and issuing the next one blocks until
      // it is free.  Everything that is not an MMA therefore sits between the
      // second-to-last and the last MMA of a chunk, or is short: the next stage's
      // barrier is probed while the pipe is busy, so that the first MMA of the next
      // chunk can follow the last one of this chunk without a bubble.
      const uint32_t idesc = make_idesc<INT8>() | ((tile_rows >> 3) << 17);
      const uint64_t wdesc0 = make_smem_desc(smem_u32(sW));  // M operand: weights
      const uint64_t rdesc0 = make_smem_desc(smem_u32(sR));  // N operand: gathered rows
      uint32_t s = 0, ph = 0, tl = 0;
      bool ready = false;  // full[s] already seen complete by a probe
      bool alive = true;
      if (w_resident && blockIdx.x < ntiles)
        alive = mbar_wait(bar_w, 0u, abort_flag, a.status, 6u);
      for (uint32_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tl) {
        const uint32_t buf = tl & 1u;
        if (!mbar_wait(bar_tempty + 8 * buf, ((tl >> 1) & 1u) ^ 1u, abort_flag, a.status, 2u))
          break;
        const uint32_t d_tmem = tmem_base + buf * kTileRows;
        for (int j = 0; j < nchunk; ++j) {
          if (!ready && !mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, 3u)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint64_t wd = wdesc0 + (uint64_t)(w_resident ? (uint32_t)j * (w_chunk_smem >> 4)
                                                             : s * (uint32_t)(kWBytes >> 4));
          const uint64_t rd = rdesc0 + (uint64_t)(s * (uint32_t)(kRowsBytes >> 4));
          const int nk = (j == nchunk - 1) ? last_ksteps : kChunk / 32;
          for (int ks = 0; ks + 1 < nk; ++ks)
            umma<INT8>(d_tmem, wd + 2u * ks, rd + 2u * ks, idesc, (uint32_t)((j | ks) != 0));
          const uint32_t s1 = s + 1 == (uint32_t)kStages ? 0u : s + 1;
          const uint32_t ph1 = s1 == 0u ? ph ^ 1u : ph;
          ready = mbar_try_wait(bar_full + 8 * s1, ph1);
          umma<INT8>(d_tmem, wd + 2u * (nk - 1), rd + 2u * (nk - 1), idesc,
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
    // Same arithmetic as common.cuh:epilogue_value, written so that the per-element
    // work is a handful of instructions: ReLU as a max with 0 or -inf, float -> int8
    // as one saturating round-to-nearest-even convert, and the layer-wide switches
    // hoisted out of the element loops.
    const Epilogue ep = a.ep;
    // The weights are copied w_rep times along the accumulator lanes: lanes below
    // w_rep * COUT hold a valid channel.  Copy r owns the tile's rows [r, r + 1) * 256 /
    // w_rep, and the two warps of a lane quadrant split those rows again, so a warp works
    // on 128 / w_rep rows of the tile: 8 / w_rep groups of 16.
    const uint32_t q = (uint32_t)warp & 3u;        // TMEM lane quadrant of this warp
    const uint32_t half = (uint32_t)warp >> 2;
    const uint32_t acc_lane = 32u * q + lane;
    const uint32_t ch = acc_lane % COUT;           // this lane's channel
    const uint32_t chq = ch & ~3u;                 // first of the 4 channels this lane stores
    const uint32_t j4 = lane & 3u;                 // row within a group of 4 this lane stores
    const uint32_t cols_rep = (uint32_t)kTileRows / w_rep, cols_warp = cols_rep / 2u;
    const bool lane_active = acc_lane / COUT < w_rep;
    const bool warp_active = (32u * q) / COUT < w_rep;
    // first row (of the tile) of this lane, and of lane 0 of the warp: they differ only for
    // COUT = 16, where the two halves of a warp belong to different copies
    const uint32_t col_lane = (acc_lane / COUT) * cols_rep + half * cols_warp;
    const uint32_t col_warp = ((32u * q) / COUT) * cols_rep + half * cols_warp;
    const float sc = (INT8 && a.scale) ? __ldg(a.scale + ch) : 1.f;
    const float bi = a.bias ? __ldg(a.bias + ch) : 0.f;
    const float lo = ep.act == SPCONVB_ACT_RELU ? 0.f : -INFINITY;
    const float lo2 = ep.res_relu ? 0.f : -INFINITY;
    const bool res_i8 = ep.res_kind == SPCONVB_I8;
    const uint32_t out_b = ep.out_kind == SPCONVB_I8 ? 1u : 2u;
    const uint32_t res_b = res_i8 ? 1u : 2u;
    // residual words of 16 rows: lane (g, j) loads channels 4g..4g+3 of rows 4j + t
    // (int8, a word each) or of rows 4t + j (fp16, two words each), t = 0..3
    auto load_res = [&](uint32_t row0, bool in_tile, uint2 (&rq)[4]) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t row = res_i8 ? row0 + 4u * j4 + t : row0 + 4u * t + j4;
        rq[t] = make_uint2(0u, 0u);
        if (in_tile && row < n_out) {
          const uint8_t* p = a.res + ((size_t)row * COUT + chq) * res_b;
          if (res_i8) rq[t].x = __ldg((const uint32_t*)p);
          else rq[t] = __ldg((const uint2*)p);
        }
      }
    };
    uint32_t tl = 0;
    for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tl) {
      const uint32_t buf = tl & 1u;
      const uint32_t trow0 = tile * tile_rows + col_lane;
      // the first residual rows are fetched before the accumulator is waited for;
      // after that the loads run one group of 16 rows ahead of the arithmetic.  A group
      // lies inside the tile or not as a whole (the tile height is a multiple of 32);
      // rows past it belong to the next tile.
      uint2 rq[4];
      if (ep.has_res) load_res(trow0, lane_active && col_lane < tile_rows, rq);
      uint32_t ok = 1u;
      if (lane == 0)
        ok = mbar_wait(bar_tfull + 8 * buf, (tl >> 1) & 1u, abort_flag, a.status, 4u) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      // groups of this warp that lie inside the tile (by its lower-numbered rows)
      const uint32_t ng = (!warp_active || col_warp >= tile_rows)
                              ? 0u
                              : min(cols_warp / 16u, (tile_rows - col_warp + 15u) / 16u);
      const uint32_t taddr = tmem_base + ((32u * q) << 16) + buf * kTileRows + col_warp;
      if (ng == 0u) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
      }
#pragma unroll 1
      for (uint32_t g = 0; g < ng; ++g) {
        const uint32_t row0 = trow0 + 16u * g;
        const bool in_tile = lane_active && col_lane + 16u * g < tile_rows;
        uint32_t v[16];
        tmem_ld16(taddr + 16u * g, v);
        if (COUT == 16 && w_rep > 1u) {
          // the upper half of the warp belongs to the next copy: its rows are one copy's
          // worth of columns further on
          uint32_t vm[16];
          tmem_ld16(taddr + cols_rep + 16u * g, vm);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = lane >= 16u ? vm[i] : v[i];
        } else {
          tmem_ld_wait();
        }
        if (g + 1u == ng) {
          // every accumulator element of this warp is in registers: release the buffer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        }
        uint2 rcur[4];
        if (ep.has_res) {
#pragma unroll
          for (int t = 0; t < 4; ++t) rcur[t] = rq[t];
          if (g + 1u < ng)
            load_res(row0 + 16, lane_active && col_lane + 16u * (g + 1u) < tile_rows, rq);
        }
        float y[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (INT8) y[i] = fmaxf(fmaf((float)(int)v[i], sc, bi), lo);
          else y[i] = fmaxf(__fadd_rn(__uint_as_float(v[i]), bi), lo);
        }
        if (ep.has_res) {
          // the conv result as it would have been stored (mid), plus the residual
          float rr[16];
          if (res_i8) {
            uint32_t w[4] = {rcur[0].x, rcur[1].x, rcur[2].x, rcur[3].x};
            bytes_transpose4(w);
            quad_words_transpose(w, lane);
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
              for (int i = 0; i < 4; ++i)
                rr[4 * t + i] = __fmul_rn((float)(int8_t)(w[t] >> (8 * i)), ep.res_scale);
          } else {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              uint32_t w0 = rcur[t].x, w1 = rcur[t].y;
              quad_transpose_h16(w0, w1, lane);
              const __half2 h0 = *(const __half2*)&w0, h1 = *(const __half2*)&w1;
              rr[4 * t + 0] = __low2float(h0);
              rr[4 * t + 1] = __high2float(h0);
              rr[4 * t + 2] = __low2float(h1);
              rr[4 * t + 3] = __high2float(h1);
            }
          }
          if (ep.mid_kind == SPCONVB_I8) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float m = __fmul_rn((float)cvt_sat_s8(__fmul_rn(y[i], ep.mid_inv_scale)),
                                        ep.mid_scale);
              y[i] = fmaxf(__fadd_rn(m, rr[i]), lo2);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              y[i] = fmaxf(__fadd_rn(__half2float(__float2half_rn(y[i])), rr[i]), lo2);
          }
        }
        if (ep.out_kind == SPCONVB_I8) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t)
            w[t] = pack_s8x4(cvt_sat_s8(__fmul_rn(y[4 * t + 0], ep.inv_out_scale)),
                             cvt_sat_s8(__fmul_rn(y[4 * t + 1], ep.inv_out_scale)),
                             cvt_sat_s8(__fmul_rn(y[4 * t + 2], ep.inv_out_scale)),
                             cvt_sat_s8(__fmul_rn(y[4 * t + 3], ep.inv_out_scale)));
          quad_words_transpose(w, lane);
          bytes_transpose4(w);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint32_t row = row0 + 4u * j4 + t;
            if (in_tile && row < n_out) *(uint32_t*)(a.out + (size_t)row * COUT + chq) = w[t];
          }
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __half2 h0 = __floats2half2_rn(y[4 * t + 0], y[4 * t + 1]);
            __half2 h1 = __floats2half2_rn(y[4 * t + 2], y[4 * t + 3]);
            uint32_t w0 = *(uint32_t*)&h0, w1 = *(uint32_t*)&h1;
            quad_transpose_h16(w0, w1, lane);
            const uint32_t row = row0 + 4u * t + j4;
            if (in_tile && row < n_out)
              *(uint2*)(a.out + ((size_t)row * COUT + chq) * out_b) = make_uint2(w0, w1);
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
  constexpr size_t smem = umma_smem_bytes();
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    SPCONVB_CUDA_TRY(cudaFuncSetAttribute(conv_umma_kernel<INT8, RB, COUT>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  uint32_t tiles = (launch_rows + 31) / 32;  // the kernel picks the tile height per launch
  int grid = (int)(tiles < (uint32_t)kSmCount ? (tiles ? tiles : 1u) : (uint32_t)kSmCount);
  conv_umma_kernel<INT8, RB, COUT><<<grid, kCtaThreads, smem, st>>>(args);
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

int conv_umma_kernel_launch(const UmmaArgs& a, bool int8, int rb, int cout, uint32_t launch_rows,
                       cudaStream_t st) {
  return int8 ? launch_rb<true>(rb, cout, a, launch_rows, st)
              : launch_rb<false>(rb, cout, a, launch_rows, st);
}

}  // namespace spconvb
