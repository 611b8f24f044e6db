// Thin wrappers over the sm_100a PTX this library uses: mbarrier (with bounded waits), TMA
// tiled loads (each into one CTA), proxy fences and the packed fp32 FMA.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace ocb {

// Device status word values (read back by opencnn_last_device_status()).
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Non-blocking test of a phase (never suspends the thread).
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
__device__ __forceinline__ void nano_sleep(uint32_t ns) { asm volatile("nanosleep.u32 %0;" ::"r"(ns)); }
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for a phase of an mbarrier, but never for ever: after `limit_ns` of wall time (or as
// soon as another thread of the CTA has given up) it sets the CTA's `dead` word and the global
// status word and returns false.  What a caller does then depends on its role: a thread that
// issues asynchronous work (TMA loads, tensor-core MMAs) stops issuing and waits, again with a
// limit, for what it has in flight (mbar_wait_drain); every other thread carries on with
// whatever is in shared memory - all its later waits return at once - so that block-wide and
// group-wide barriers are still reached by everyone and the kernel terminates.  The host sees
// the failure in the status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *dead, int *status,
                                          uint64_t limit_ns = 2000000000ull) {
  // (Polling with the non-suspending test_wait first was measured and is slower: the spinning
  // lanes take issue slots from the warps that do the work.)
  if (mbar_try_wait(bar, parity)) return true;
  if (*dead) return false;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0u) {
      if (*dead) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *dead = 1;
        atomicExch(status, kStatusWaitTimeout);
        return false;
      }
    }
  }
}

// Bounded wait that ignores the CTA's `dead` word: used once a thread has given up, to let the
// asynchronous operations it issued earlier (whose completion this barrier phase signals) finish
// before the CTA exits or frees what they use.  Returns false if the limit ran out.
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0u && global_timer_ns() - t0 > limit_ns) return false;
  }
}

// True in exactly one lane of a fully converged warp.  Single-thread instructions that take their
// operands from uniform registers (tcgen05.mma, TMA) are issued under this predicate by a warp
// that executes the surrounding code convergently; issuing them from an `if (lane == 0)` branch
// instead costs on the order of a hundred cycles per instruction.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Orders this thread's earlier generic-proxy shared-memory accesses before later async-proxy
// (TMA) accesses to the same locations.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// TMA tiled loads global -> this CTA's shared memory, completion on an mbarrier.  The innermost
// coordinate times the element size must be a multiple of 16 bytes; other coordinates may be
// negative or past the end, where the box is filled with zeros.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Packed fp32 FMA: d.lo = a.lo*b.lo + d.lo, d.hi = a.hi*b.hi + d.hi, each rounded once exactly
// like a scalar fma.rn.f32.  One issue slot for two FMAs.
__device__ __forceinline__ void ffma2(uint64_t &d, uint64_t a, uint64_t b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

}  // namespace ocb
