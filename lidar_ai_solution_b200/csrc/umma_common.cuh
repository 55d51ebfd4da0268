// What the tensor-core convolution kernel (conv_umma_kernel.cu) and its host side
// (conv_umma.cu) share: the kernel arguments, thin wrappers over the PTX the kernel
// uses (mbarrier, cp.async, bulk copy, tcgen05 alloc/mma/commit/ld), the
// shared-memory operand descriptor and the bounded wait.
#pragma once
#include "common.cuh"

namespace spconvb {
namespace umma_detail {

constexpr int kChunk = 128;   // bytes of K per pipeline stage: one 128-byte swizzle atom per row
constexpr int kMaxTaps = 27;  // most taps of a layer the tensor-core kernel takes
constexpr int kMaxStages = 6; // deepest ring of gathered-row stages
constexpr unsigned long long kWaitLimitNs = 250ull * 1000 * 1000;

struct UmmaArgs {
  const uint8_t* in;
  const int32_t* map;
  uint32_t cap;
  const uint32_t* n_out_ptr;
  const uint8_t* wpk;
  const float* scale;
  const float* bias;
  const uint8_t* res;
  uint8_t* out;
  uint32_t* status;
  const uint32_t* n_in_ptr;  // rows of `in` (for the L2 prefetch of input rows); may be null
  uint32_t cap_in;           // rows the buffer of `in` holds
  int kvol;
  int w_rep;       // copies of each weight chunk along the accumulator rows: w_rep * Cout = 64 or 128
  int w_resident;  // 1: all chunks stay in shared memory for the whole launch; 0: streamed
  int nstages;     // depth of the ring of gathered-row stages (2..kMaxStages)
  int prefetch;    // tiles (per CTA) the L2 prefetch runs ahead of the gather; 0 = off
  int wait_test;   // > 0: producers withhold "stage full" from this chunk on (self-test)
  Epilogue ep;
};

// Shared-memory footprint of one launch configuration (the kernel carves it the same way).
__host__ __device__ inline size_t umma_smem_bytes(int cout, int nchunk, int w_rep, int w_resident,
                                                  int nstages) {
  const size_t wchunk = (size_t)w_rep * cout * kChunk;
  const size_t w = w_resident ? (size_t)nchunk * wchunk : (size_t)nstages * wchunk;
  return 1024 + w + (size_t)nstages * 256 * kChunk + 256;
}

// ------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking form: try_wait may hold the thread for a hardware-defined time before it
// answers "not yet"; test_wait answers at once.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same test, but the hardware may park the thread for up to `ns` nanoseconds while the
// phase is incomplete (it resumes when the phase completes): a waiting role then stops
// taking issue slots from the working ones.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded waits.  They return false when the CTA is aborting.
//
// Two flavours.  A role whose wait is on the critical path of every chunk (the thread that
// issues the MMAs) spins on the non-blocking test: a thread parked in try_wait wakes up late.
// Roles that wait often and long (producers for a free stage, epilogue warps for a finished
// tile) park in try_wait instead: a hot spin of 16 + 8 warps takes issue slots from the
// warps that have work.  Both read the clock only after a first batch of polls has failed.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity,
                                            volatile uint32_t* abort_flag, uint32_t* status,
                                            uint32_t where) {
  const unsigned long long t0 = global_ns();
  while (true) {
    for (int i = 0; i < 16; ++i)
      if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1u;
      set_status(status, SPCONVB_ST_TIMEOUT, where);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity,
                                               volatile uint32_t* abort_flag, uint32_t* status,
                                               uint32_t where) {
#pragma unroll 1
  for (int i = 0; i < 256; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, where);
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, uint32_t* status,
                                          uint32_t where) {
  if (mbar_test_wait(bar, parity)) return true;
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait_parked(bar, parity, 2000u)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, where);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void st_shared_s32(uint32_t dst, int32_t v) {
  asm volatile("st.shared.s32 [%0], %1;" ::"r"(dst), "r"(v) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// The calling thread's earlier cp.async copies arrive on the barrier when they have landed
// (the barrier's expected count includes this arrival: "noinc").
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Asks L2 to fetch a contiguous piece of global memory: address 16-byte aligned, size a
// multiple of 16 bytes.  No data reaches the SM.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                   "r"(bar)
               : "memory");
}
template <bool INT8>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                     uint32_t idesc, uint32_t accumulate) {
  if (INT8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// The same with the shared-memory descriptors given as halves: only the low word (the
// address field) changes from chunk to chunk, so the issuing thread does 32-bit arithmetic.
template <bool INT8>
__device__ __forceinline__ void umma_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                          uint32_t desc_hi, uint32_t idesc, uint32_t accumulate) {
  if (INT8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// float -> int8 value: round to nearest even, saturate to [-128, 127] (one convert).
__device__ __forceinline__ int cvt_sat_s8(float x) {
  int q;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(x));
  return q;
}
__device__ __forceinline__ uint32_t pack_s8x4(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile, 128-byte swizzle: rows are 128 bytes, groups of 8 rows
// are 1024 bytes apart.  Field layout of the 64-bit shared-memory descriptor:
// [0,14) address>>4, [16,30) leading offset>>4 (unused for swizzled K-major),
// [32,46) stride offset>>4, [46,48) version = 1, [61,64) swizzle mode (2 = 128 B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

inline int row_bytes(int compute, int cin) { return cin * (compute == SPCONVB_I8 ? 1 : 2); }

}  // namespace umma_detail
}  // namespace spconvb
