// What the tensor-core convolution kernel (conv_umma_kernel.cu) and its host side
// (conv_umma.cu) share: the kernel arguments, thin wrappers over the PTX the kernel
// uses (mbarrier, cp.async, bulk copy, tcgen05 alloc/mma/commit/ld), the
// shared-memory operand descriptor and the bounded wait.
#pragma once
#include "common.cuh"

namespace spconvb {
namespace umma_detail {

constexpr int kChunk = 128;   // bytes of K per pipeline stage: one 128-byte swizzle atom per row
constexpr int kMaxTaps = 27;  // taps whose neighbour indices are staged in shared memory
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
  int kvol;
  int w_rep;       // copies of each weight chunk along the 128 accumulator lanes (1..128/Cout)
  int w_resident;  // 1: all chunks stay in shared memory for the whole launch; 0: streamed
  int wait_test;   // > 0: producers withhold "stage full" from this chunk on (self-test)
  Epilogue ep;
};

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
// Bounded wait.  Returns false when the CTA is aborting.
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, uint32_t* status,
                                          uint32_t where) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, where);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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
