// Sparse convolution as an implicit GEMM on the sm_100a tensor cores, voxel rows on
// the N side of the MMA.
//
//   out[o, :] = epilogue( sum_k  W[:, k, :] . in[map[k][o], :] )
//
// is a GEMM between the weights [Cout x K] and a matrix [rows x K], K = kvol *
// Cin, that does not exist in memory: its row o is the concatenation of the
// feature rows of o's neighbours (zeros where a neighbour is absent).  A
// tcgen05.mma takes the same time whether its accumulator has 64 or 128 rows, and
// its time grows with its columns, so the voxel rows are put on the wide side: the
// weights are the M operand (64 or 128 accumulator rows = output channels, copied
// w_rep times when Cout is smaller), a tile of up to 256 voxel rows is the N
// operand, and the accumulator in TMEM is the transposed output tile
// D[channel][row].  Copies of the weights let more epilogue warps share a tile.
// When all chunks of the layer (times the copies) fit beside the row stages they
// are loaded once and stay in shared memory; otherwise a chunk is streamed with
// every stage.  The host side (conv_umma.cu) picks copies, residency and the depth
// of the stage ring from the shared-memory budget.  The kernel is persistent (one
// CTA per SM) and warp-specialised:
//
//   warps 0-7   epilogue: warp w reads its lane quadrant (its channels) and its
//               share of the tile's rows from the accumulator with tcgen05.ld,
//               applies dequant + bias + activation (+ residual add) + requant
//               with per-lane scale and bias, transposes 4x4 blocks inside lane
//               quads with two shuffles, and stores 4 (int8) or 8 (fp16)
//               contiguous bytes of one output row per lane
//   warp  8     allocates TMEM; one lane issues tcgen05.mma (kind::i8 with int32
//               accumulators or kind::f16 with fp32 accumulators)
//   warps 9-24  producers, two groups of 8 warps that take the chunks in turn (the
//               work of a warp per chunk is a chain of dependent steps - wait for
//               the stage, neighbour indices, addresses, copies, arrival - that
//               takes longer than the tensor pipe needs for the chunk; two groups
//               give each warp two chunk periods for it).  Within a group each warp
//               owns 32 rows of the tile.  A thread loads the 8 neighbour indices
//               it needs for its next chunk straight into registers (two 16-byte
//               loads, a round ahead) and gathers with 16-byte cp.async (8 lanes
//               per row, so a row is one contiguous request; zero-fill for missing
//               neighbours) straight into the 128-byte-swizzled K-major layout the
//               MMA reads.
//               A producer never waits for its copies: every thread lets them
//               arrive on the stage's mbarrier when they land, so all free stages
//               of the ring are in flight.  One thread also streams the
//               pre-swizzled weight chunk with one bulk async copy.  Optionally
//               (UmmaArgs.prefetch > 0; off by default, it measured slower) a few
//               lanes ask L2 (bulk prefetch) for the map lines, input rows and
//               residual rows of the tile the CTA will reach some rounds later.
//
// K is walked in chunks of 128 bytes (one swizzle atom per row): a chunk is 8
// taps of a 16-byte row, ..., 1 tap of a 128-byte row, or half a 256-byte row.
// The accumulator is double-buffered in TMEM (2 x 256 columns) so the epilogue of
// tile t overlaps the MMAs of tile t+1.
//
// Every wait is bounded: a wait that runs out sets SPCONVB_ST_TIMEOUT in the
// status block, raises a CTA-wide abort flag and all roles leave their loops,
// drain their copies and free TMEM.
#include "umma_common.cuh"

// Per-role cycle accounting, compiled in only with -DSPCONVB_CONV_PROFILE (a measurement
// build, never the shipped one): one lane of a producer warp, the MMA thread and one
// epilogue lane add up the clock cycles they spend in each part of their loops, per CTA;
// spconvb_debug_conv_profile() copies the table out.  In that build a negative
// spconvb_conv_params.wait_test -f switches work off: f & 1 no gather copies, f & 2 no MMAs.
#ifdef SPCONVB_CONV_PROFILE
#define PROF(...) __VA_ARGS__
#else
#define PROF(...)
#endif
// The work switches alone (-DSPCONVB_CONV_SWITCHES, implied by the profile build): the same
// experiments timed from outside, without the clock reads in the loops.
#if defined(SPCONVB_CONV_PROFILE) || defined(SPCONVB_CONV_SWITCHES)
#define DBG(...) __VA_ARGS__
#else
#define DBG(...)
#endif

namespace spconvb {

using namespace umma_detail;

PROF(__device__ unsigned long long g_conv_profile[148][16];)

namespace {

constexpr int kTileRows = 256;  // most voxel rows per tile: the largest N of the MMA
constexpr int kRowsBytes = kTileRows * kChunk;  // gathered rows of one stage
constexpr int kEpiWarps = 8;
constexpr int kMmaWarp = 8;
constexpr int kProdWarp0 = 9;
constexpr int kProdThreads = 512;   // two groups of 8 producer warps
constexpr int kCtaThreads = 32 * kProdWarp0 + kProdThreads;
constexpr uint32_t kTmemCols = 2 * kTileRows;
constexpr size_t kMaxSmem = 232448;  // 227 KB: the most dynamic shared memory of a CTA

// 32-bit instruction descriptor: [4,6) D format (1 = f32, 2 = s32), [7,10) A
// format, [10,13) B format (f16 kind: 0 = f16; i8 kind: 1 = signed), bits 15/16
// A/B major (0 = K), [17,23) N>>3, [24,29) M>>4.  M and N are added per launch.
template <bool INT8>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return INT8 ? ((2u << 4) | (1u << 7) | (1u << 10)) : (1u << 4);
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

// ------------------------------------------------------------------- kernel
template <bool INT8, int RB, int COUT>
__global__ void __launch_bounds__(kCtaThreads, 1) conv_umma_kernel(const UmmaArgs a) {
  constexpr int OPC = RB <= kChunk ? kChunk / RB : 1;   // taps per chunk
  constexpr int SPO = RB <= kChunk ? RB / 16 : 8;       // 16-byte segments per tap per chunk
  constexpr int CPT = RB <= kChunk ? 1 : RB / kChunk;   // chunks per tap

  const int kbytes = a.kvol * RB;
  const int nchunk = (kbytes + kChunk - 1) / kChunk;
  const int last_ksteps = ((kbytes - (nchunk - 1) * kChunk) + 31) / 32;
  const uint32_t w_rep = (uint32_t)a.w_rep;
  const uint32_t m_rows = w_rep * COUT;            // accumulator rows of the MMA: 64 or 128
  const bool w_resident = a.w_resident != 0;
  const uint32_t w_chunk_smem = m_rows * kChunk;   // bytes of one chunk with its copies
  const uint32_t nst = (uint32_t)a.nstages;

  // Shared memory: the weights (all chunks, or one per stage), the gathered-row stages,
  // the barriers.
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sW = smem;
  uint8_t* sR = sW + (w_resident ? (uint32_t)nchunk : nst) * w_chunk_smem;
  uint64_t* bars = (uint64_t*)(sR + nst * kRowsBytes);
  uint32_t* tmem_holder = (uint32_t*)(bars + 2 * kMaxStages + 5);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kMaxStages;
  const uint32_t bar_tfull = bar_empty + 8 * kMaxStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_w = bar_tempty + 16;  // resident weights have landed

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  PROF(const long long k_c0 = clock64(); const unsigned long long k_t0 = global_ns();)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(bar_full + 8 * s, kProdThreads / 2 + 1);  // a group's threads + the weights
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

  if (warp >= kProdWarp0) {
    // ------------------------------------------------------------ producers
    // Two groups of 8 warps take the chunks in turn (group g the chunks g, g + 2, ...), so a
    // warp has two chunk periods for the round trip of one chunk: wait for the stage, look
    // up the neighbours, issue the copies.  Within a group, warp w owns rows 32w..32w+31 of
    // the tile.  A chunk of the row tile is 256 rows x 8 segments of 16 bytes = 2048 copies,
    // 8 per thread: a thread copies segment `seg` of rows 32w + 8 slot + i, i = 0..7 (8
    // lanes per row, so the lanes that read the same neighbour row ask for one contiguous
    // piece of it).  Missing neighbours are zero-filled copies, so the 8 items are
    // branch-free and their address arithmetic and copies overlap.
    const uint32_t pw_all = (uint32_t)warp - kProdWarp0;
    const uint32_t grp = pw_all >> 3, pw = pw_all & 7u;
    const bool w_thread = pw == 0u && lane == 0u;  // also streams the weights of its chunks
    const uint32_t seg = lane & 7u;        // 16-byte segment of the chunk this thread copies
    const uint32_t slot = lane >> 3;       // its 8 rows of the warp's 32
    // row R of the tile lives at (R / 8) * 1024 + (R % 8) * 128, its segments XOR-ed
    // with R % 8; here R / 8 = 4 pw + slot and R % 8 = i
    const uint32_t dst_base = (pw * 4u + slot) * 1024u;
    // tap (within the chunk) and byte offset (within the neighbour row) of `seg`
    const uint32_t seg_tap = RB <= kChunk ? seg / SPO : 0u;
    const uint32_t seg_byte = RB <= kChunk ? (seg % SPO) * 16u : seg * 16u;
    const bool has_rows = pw * 32u < tile_rows;  // else this warp only keeps the barriers going
    const uint32_t row_in_tile = pw * 32u + slot * 8u;
    // 16-byte index loads need the map rows 16-byte aligned and whole groups of 8 inside them
    const bool vec_ok = (a.cap & 7u) == 0u && ((uintptr_t)a.map & 15u) == 0u;

    // The 8 neighbour indices this thread needs for chunk j of a tile: its tap's map entries
    // of its 8 rows, straight from global memory into registers (two 16-byte loads; the 8
    // lanes of a row group that share a tap read the same 32 bytes).  Rows past the end,
    // taps past the kernel and tiles past the last give -1.
    auto load_idx = [&](uint32_t tile, int j, int32_t (&v)[8]) {
      const int k = RB <= kChunk ? j * OPC + (int)seg_tap : j / CPT;
      const uint32_t row = tile * tile_rows + row_in_tile;
      const bool live = has_rows && tile < ntiles && k < a.kvol && row < n_out;
      const int32_t* src = a.map + (size_t)k * a.cap + row;
      if (live && vec_ok && row + 8u <= n_out) {
        const int4 lo = __ldg((const int4*)src), hi = __ldg((const int4*)src + 1);
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
        v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      } else {
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) v[i] = (live && row + i < n_out) ? __ldg(src + i) : -1;
      }
    };
    // L2 prefetch of what tile `pt` will read: its map lines (lanes 0-3 of every warp take
    // the taps w, w+8, ...), its share of the input rows and its residual rows.  Bulk
    // prefetches: one instruction per contiguous piece, nothing returns to the SM.
    const uint32_t n_in = a.n_in_ptr ? min(*a.n_in_ptr, a.cap_in) : 0u;
    const bool map_pf = (a.cap & 3u) == 0u && ((uintptr_t)a.map & 15u) == 0u;
    auto prefetch_tile = [&](uint32_t pt) {
      if (pt >= ntiles || lane > 4u) return;
      const uint32_t prow0 = pt * tile_rows;
      const uint32_t prows = min(tile_rows, n_out - prow0);
      if (lane < 4u) {
        const uint32_t k = pw + 8u * lane;
        if (map_pf && k < (uint32_t)a.kvol)
          bulk_prefetch_l2(a.map + (size_t)k * a.cap + prow0, ((prows + 3u) & ~3u) * 4u);
      } else if (pw == 0u) {
        if (n_in) {
          const uint32_t in0 = (uint32_t)((unsigned long long)prow0 * n_in / n_out);
          uint32_t cnt = (uint32_t)((unsigned long long)prows * n_in / n_out) + 1u;
          if (in0 < n_in) {
            cnt = min(cnt, n_in - in0);
            bulk_prefetch_l2(a.in + (size_t)in0 * RB, cnt * (uint32_t)RB);
          }
        }
      } else if (pw == 1u) {
        if (a.ep.has_res) {
          const uint32_t rb = (uint32_t)COUT * (a.ep.res_kind == SPCONVB_I8 ? 1u : 2u);
          bulk_prefetch_l2(a.res + (size_t)prow0 * rb, prows * rb);
        }
      }
    };
    if (grp == 0u)
      for (int p = 0; p < a.prefetch; ++p) prefetch_tile(blockIdx.x + (uint32_t)p * gridDim.x);

    if (grp == 0u && w_thread && w_resident && blockIdx.x < ntiles) {
      mbar_expect_tx(bar_w, (uint32_t)nchunk * w_chunk_smem);
      for (int j = 0; j < nchunk; ++j)
        for (uint32_t c = 0; c < w_rep; ++c)
          bulk_g2s(smem_u32(sW + j * w_chunk_smem + c * (COUT * kChunk)),
                   a.wpk + (size_t)j * (COUT * kChunk), COUT * kChunk, bar_w);
    }

    // This group's chunks: numbers it = grp, grp + 2, ... of the CTA's chunk sequence (tile
    // after tile, nchunk chunks each); chunk `it` uses stage it % nst.
    auto advance2 = [&](uint32_t& tile, int& j) {  // two chunks on
      j += 2;
      while (j >= nchunk) {
        j -= nchunk;
        tile += gridDim.x;
      }
    };
    uint32_t tile = blockIdx.x;
    int j = 0;
    if (grp == 1u) {
      j = 1;
      while (j >= nchunk) {
        j -= nchunk;
        tile += gridDim.x;
      }
    }
    uint32_t it = grp, s = grp % nst, ph = (grp / nst) & 1u;
    int32_t cur[8], nxt[8];
    load_idx(tile, j, cur);
    PROF(long long p_idx = 0, p_wait = 0, p_issue = 0, p_t0 = clock64(), t_a, t_b; uint32_t p_n = 0;)
    DBG(const bool no_copies = a.wait_test < 0 && ((-a.wait_test) & 1);)
    while (tile < ntiles) {
      PROF(t_a = clock64();)
      uint32_t ntile = tile;
      int nj = j;
      advance2(ntile, nj);
      load_idx(ntile, nj, nxt);  // used a round from now
      if (j == 0 && a.prefetch > 0) prefetch_tile(tile + (uint32_t)a.prefetch * gridDim.x);
      PROF(t_b = clock64(); p_idx += t_b - t_a;)
      // every lane polls: one shared-memory word, no divergence, no broadcast afterwards
      if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, a.status, 1u)) break;
      PROF(t_a = clock64(); p_wait += t_a - t_b;)
      if (w_thread) {
        if (w_resident) {
          mbar_arrive(bar_full + 8 * s);
        } else {
          mbar_expect_tx(bar_full + 8 * s, w_chunk_smem);
          for (uint32_t c = 0; c < w_rep; ++c)
            bulk_g2s(smem_u32(sW + s * w_chunk_smem + c * (COUT * kChunk)),
                     a.wpk + (size_t)j * (COUT * kChunk), COUT * kChunk, bar_full + 8 * s);
        }
      }
      // segments of the last chunk that lie in K steps past the kernel's last tap are never
      // read by an MMA: nothing to copy, nothing to zero
      const bool dead_seg = j == nchunk - 1 && (int)(seg >> 1) >= last_ksteps;
      if (has_rows && !dead_seg DBG(&& !no_copies)) {
        const uint32_t byte = seg_byte + (RB > kChunk ? (uint32_t)(j % CPT) * kChunk : 0u);
        const uint32_t stage_addr = smem_u32(sR + s * kRowsBytes) + dst_base;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
          const int32_t sr = cur[i];
          cp_async16(stage_addr + i * 128u + ((seg ^ i) << 4),
                     a.in + (size_t)(sr < 0 ? 0 : sr) * RB + byte, sr < 0 ? 0u : 16u);
        }
      }
      if (!(a.wait_test > 0 && it + 1u >= (uint32_t)a.wait_test))
        cp_async_arrive_noinc(bar_full + 8 * s);
#pragma unroll
      for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
      tile = ntile;
      j = nj;
      it += 2;
      s += 2;
      if (s >= nst) {
        s -= nst;
        ph ^= 1u;
      }
      PROF(p_issue += clock64() - t_a; ++p_n;)
    }
    PROF(if (pw_all == 7 && lane == 0 && blockIdx.x < 148) {
      unsigned long long* o = g_conv_profile[blockIdx.x];
      o[0] = clock64() - p_t0; o[1] = p_idx; o[2] = p_wait; o[3] = p_issue; o[4] = 2 * p_n;
    })
    cp_async_wait_all();  // nothing of this thread may still be writing when the CTA exits
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // The tensor pipe takes one MMA at a time, and issuing the next one blocks until
      // it is free.  Everything that is not an MMA therefore sits between the
      // second-to-last and the last MMA of a chunk, or is short: the next stage's
      // barrier is probed while the pipe is busy, so that the first MMA of the next
      // chunk can follow the last one of this chunk without a bubble.
      const uint32_t idesc =
          make_idesc<INT8>() | ((tile_rows >> 3) << 17) | ((m_rows >> 4) << 24);
      const uint64_t wdesc0 = make_smem_desc(smem_u32(sW));  // M operand: weights
      const uint64_t rdesc0 = make_smem_desc(smem_u32(sR));  // N operand: gathered rows
      uint32_t ph = 0, tl = 0;
      bool alive = true;
      if (w_resident && blockIdx.x < ntiles)
        alive = mbar_wait_spin(bar_w, 0u, abort_flag, a.status, 6u);
      // The loop is entered with the current chunk's stage known to be full.
      if (blockIdx.x < ntiles && alive)
        alive = mbar_wait_spin(bar_full, 0u, abort_flag, a.status, 3u);
      // The thread that issues the MMAs runs one lane of one warp: every instruction
      // between two MMAs that the tensor pipe cannot hide (it queues about one MMA ahead)
      // is a bubble.  So the loop carries its descriptors and barrier addresses along
      // instead of recomputing them, asks about the next stage once, early (right after
      // the first MMA, so the answer is there when the last one has been issued), and
      // issues the K steps of a full chunk without a loop.
      // 32-bit arithmetic only: the descriptors differ in their low word (the address)
      const uint32_t w_step = w_chunk_smem >> 4, r_step = (uint32_t)(kRowsBytes >> 4);
      const uint32_t desc_hi = (uint32_t)(wdesc0 >> 32);
      const uint32_t w_lo0 = (uint32_t)wdesc0, r_lo0 = (uint32_t)rdesc0;
      uint32_t s = 0;  // stage of the current chunk
      PROF(long long m_full = 0, m_issue = 0, m_tempty = 0, m_t0 = clock64(), t_a, t_b;)
      DBG(const bool no_mma = a.wait_test < 0 && ((-a.wait_test) & 2);)
      for (uint32_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tl) {
        const uint32_t buf = tl & 1u;
        PROF(t_a = clock64();)
        if (!mbar_wait_spin(bar_tempty + 8 * buf, ((tl >> 1) & 1u) ^ 1u, abort_flag, a.status, 2u))
          break;
        PROF(m_tempty += clock64() - t_a;)
        tc_fence_after();  // the epilogue's reads of this accumulator come before these MMAs
        const uint32_t d_tmem = tmem_base + buf * kTileRows;
        const bool last_tile = tile + gridDim.x >= ntiles;
        for (int j = 0; j < nchunk; ++j) {
          // No fence here: the rows arrive by cp.async completions on the stage's mbarrier,
          // which is what the MMA's shared-memory reads are ordered behind.
          const uint32_t rd = r_lo0 + s * r_step;
          const uint32_t wd = w_lo0 + (w_resident ? (uint32_t)j : s) * w_step;
          // the next stage (of this tile's next chunk or of the next tile's first)
          const uint32_t s1 = s + 1 == nst ? 0u : s + 1;
          const uint32_t ph1 = s1 == 0u ? ph ^ 1u : ph;
          const uint32_t full_n = bar_full + 8 * s1;
          const bool more = j + 1 < nchunk || !last_tile;
          bool ready;
          PROF(t_a = clock64();)
          DBG(if (no_mma) ready = !more || mbar_test_wait(full_n, ph1); else)
          if (j + 1 < nchunk) {
            umma_lohi<INT8>(d_tmem, wd, rd, desc_hi, idesc, (uint32_t)(j != 0));
            ready = mbar_test_wait(full_n, ph1);
            umma_lohi<INT8>(d_tmem, wd + 2u, rd + 2u, desc_hi, idesc, 1u);
            umma_lohi<INT8>(d_tmem, wd + 4u, rd + 4u, desc_hi, idesc, 1u);
            umma_lohi<INT8>(d_tmem, wd + 6u, rd + 6u, desc_hi, idesc, 1u);
          } else {
            ready = !more || mbar_test_wait(full_n, ph1);
            for (int ks = 0; ks < last_ksteps; ++ks)
              umma_lohi<INT8>(d_tmem, wd + 2u * ks, rd + 2u * ks, desc_hi, idesc,
                              (uint32_t)((j | ks) != 0));
          }
          tc_commit(bar_empty + 8 * s);
          PROF(t_b = clock64(); m_issue += t_b - t_a;)
          if (!ready && more && !mbar_wait_spin(full_n, ph1, abort_flag, a.status, 3u)) {
            alive = false;
            break;
          }
          PROF(m_full += clock64() - t_b;)
          s = s1;
          ph = ph1;
        }
        if (alive) tc_commit(bar_tfull + 8 * buf);
      }
      PROF(if (blockIdx.x < 148) {
        unsigned long long* o = g_conv_profile[blockIdx.x];
        o[5] = clock64() - m_t0; o[6] = m_full; o[7] = m_issue; o[8] = m_tempty;
      })
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue
    // Same arithmetic as common.cuh:epilogue_value, written so that the per-element
    // work is a handful of instructions: ReLU as a max with 0 or -inf, float -> int8
    // as one saturating round-to-nearest-even convert, and the layer-wide switches
    // hoisted out of the element loops.
    const Epilogue ep = a.ep;
    // Accumulator row m holds channel m % COUT of weight copy m / COUT.  With 128 rows
    // TMEM lane = m; with 64 rows the accumulator sits in lanes 0-15 of every 32-lane
    // quadrant (m = 16 * quadrant + lane) and lanes 16-31 carry nothing.  Copy c owns the
    // tile's rows [c, c + 1) * 256 / w_rep, and the two warps of a lane quadrant split
    // those rows again, so a warp works on 128 / w_rep rows of the tile.
    const uint32_t q = (uint32_t)warp & 3u;        // TMEM lane quadrant of this warp
    const uint32_t half = (uint32_t)warp >> 2;
    const bool wide = m_rows == 128u;
    const bool lane_valid = wide || lane < 16u;
    const uint32_t acc_row = wide ? 32u * q + lane : 16u * q + (lane & 15u);
    const uint32_t acc_row0 = wide ? 32u * q : 16u * q;   // of lane 0 of the warp
    const uint32_t ch = acc_row % COUT;            // this lane's channel
    const uint32_t chq = ch & ~3u;                 // first of the 4 channels this lane stores
    const uint32_t j4 = lane & 3u;                 // row within a group of 4 this lane stores
    const uint32_t cols_rep = (uint32_t)kTileRows / w_rep, cols_warp = cols_rep / 2u;
    const bool lane_active = lane_valid && acc_row / COUT < w_rep;
    const bool warp_active = acc_row0 / COUT < w_rep;
    // first row (of the tile) of this lane, and of lane 0 of the warp: they differ only for
    // COUT = 16 with 128 accumulator rows, where the two halves of a warp belong to
    // different copies
    const bool split_warp = COUT == 16 && wide && w_rep > 1u;
    const uint32_t col_lane = (acc_row / COUT) * cols_rep + half * cols_warp;
    const uint32_t col_warp = (acc_row0 / COUT) * cols_rep + half * cols_warp;
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
    PROF(long long e_wait = 0, e_body = 0, e_t0 = clock64(), t_a, t_b;)
    for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tl) {
      const uint32_t buf = tl & 1u;
      const uint32_t trow0 = tile * tile_rows + col_lane;
      PROF(t_a = clock64();)
      // the first residual rows are fetched before the accumulator is waited for;
      // after that the loads run one group of 16 rows ahead of the arithmetic.  A group
      // lies inside the tile or not as a whole (the tile height is a multiple of 32);
      // rows past it belong to the next tile.
      uint2 rq[4];
      if (ep.has_res) load_res(trow0, lane_active && col_lane < tile_rows, rq);
      uint32_t ok = 1u;
      if (lane == 0) {
        PROF(if (a.wait_test < 0 && ((-a.wait_test) & 16)) {
          for (int i = 0; i < 4000 && !mbar_test_wait(bar_tfull + 8 * buf, (tl >> 1) & 1u); ++i)
            __nanosleep(500);
        })
        ok = mbar_wait(bar_tfull + 8 * buf, (tl >> 1) & 1u, abort_flag, a.status, 4u) ? 1u : 0u;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      PROF(t_b = clock64(); e_wait += t_b - t_a;)
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
        if (split_warp) {
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
      PROF(e_body += clock64() - t_b;)
    }
    PROF(if (threadIdx.x == 0 && blockIdx.x < 148) {
      unsigned long long* o = g_conv_profile[blockIdx.x];
      o[9] = clock64() - e_t0; o[10] = e_wait; o[11] = e_body; o[12] = tl;
    })
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  PROF(if (threadIdx.x == 0 && blockIdx.x < 148) {
    g_conv_profile[blockIdx.x][13] = clock64() - k_c0;   // SM cycles of the CTA ...
    g_conv_profile[blockIdx.x][14] = global_ns() - k_t0;  // ... and the nanoseconds they took
  })
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
int launch_one(const UmmaArgs& args, uint32_t launch_rows, size_t smem, cudaStream_t st) {
  static bool attr_done[64] = {};
  int dev = 0;
  SPCONVB_CUDA_TRY(cudaGetDevice(&dev));
  if (smem > kMaxSmem) return SPCONVB_E_UNSUPPORTED;
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    SPCONVB_CUDA_TRY(cudaFuncSetAttribute(conv_umma_kernel<INT8, RB, COUT>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kMaxSmem));
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  uint32_t tiles = (launch_rows + 31) / 32;  // the kernel picks the tile height per launch
  int grid = (int)(tiles < (uint32_t)kSmCount ? (tiles ? tiles : 1u) : (uint32_t)kSmCount);
  conv_umma_kernel<INT8, RB, COUT><<<grid, kCtaThreads, smem, st>>>(args);
  SPCONVB_LAUNCH_CHECK();
  return SPCONVB_OK;
}

template <bool INT8, int RB>
int launch_cout(int cout, const UmmaArgs& args, uint32_t launch_rows, size_t smem,
                cudaStream_t st) {
  switch (cout) {
    case 16: return launch_one<INT8, RB, 16>(args, launch_rows, smem, st);
    case 32: return launch_one<INT8, RB, 32>(args, launch_rows, smem, st);
    case 64: return launch_one<INT8, RB, 64>(args, launch_rows, smem, st);
    case 128: return launch_one<INT8, RB, 128>(args, launch_rows, smem, st);
  }
  return SPCONVB_E_UNSUPPORTED;
}

template <bool INT8>
int launch_rb(int rb, int cout, const UmmaArgs& args, uint32_t launch_rows, size_t smem,
              cudaStream_t st) {
  switch (rb) {
    case 16: return launch_cout<INT8, 16>(cout, args, launch_rows, smem, st);
    case 32: return launch_cout<INT8, 32>(cout, args, launch_rows, smem, st);
    case 64: return launch_cout<INT8, 64>(cout, args, launch_rows, smem, st);
    case 128: return launch_cout<INT8, 128>(cout, args, launch_rows, smem, st);
    case 256: return launch_cout<INT8, 256>(cout, args, launch_rows, smem, st);
  }
  return SPCONVB_E_UNSUPPORTED;
}

}  // namespace

int conv_umma_kernel_launch(const UmmaArgs& a, bool int8, int rb, int cout, uint32_t launch_rows,
                            size_t smem, cudaStream_t st) {
  return int8 ? launch_rb<true>(rb, cout, a, launch_rows, smem, st)
              : launch_rb<false>(rb, cout, a, launch_rows, smem, st);
}

}  // namespace spconvb

#ifdef SPCONVB_CONV_PROFILE
extern "C" __attribute__((visibility("default"))) int spconvb_debug_conv_profile(
    unsigned long long* host) {
  return (int)cudaMemcpyFromSymbol(host, spconvb::g_conv_profile, sizeof(spconvb::g_conv_profile));
}
#endif
