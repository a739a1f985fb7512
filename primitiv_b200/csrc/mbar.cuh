// mbarrier and bulk-copy helpers for kernels that stream a large operand through a shared-memory
// ring (a producer thread issues bulk copies, consumer warps work from shared memory).  Every wait
// is bounded: after `limit` SM clock cycles it gives up and returns false, and the caller raises
// its abort flag, lets its own copies land, and reports through the context's status word.
#ifndef PRIMITIV_B200_CSRC_MBAR_CUH_
#define PRIMITIV_B200_CSRC_MBAR_CUH_

#include <cstdint>

namespace b200 {
namespace ring {

constexpr long long kWaitLimitCycles = 2000000000ll;  // about a second at boost clock

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint32_t try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait.  false = the CTA is aborting, or the limit ran out (the flag is then raised here).
__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                     long long limit = kWaitLimitCycles) {
  if (try_wait(bar, parity)) return true;
  uint32_t spins = 0;
  long long t0 = 0;
  for (;;) {
    if (try_wait(bar, parity)) return true;
    if (++spins == 64u) t0 = clock64();
    if (spins > 64u && (spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Used on the way out only: waits a bounded time, raises nothing.
__device__ __forceinline__ void wait_quiet(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitLimitCycles / 4) return;
  }
}

// Contiguous global -> shared copy of `bytes` (a multiple of 16, both addresses 16-byte aligned),
// completion counted in bytes on `bar`.  This GPU's own memory only.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

}  // namespace ring
}  // namespace b200

#endif  // PRIMITIV_B200_CSRC_MBAR_CUH_
