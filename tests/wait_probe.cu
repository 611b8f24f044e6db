// Test-only kernel for the bounded waits of opencnn_b200/csrc/ptx.cuh (mbar_wait, mbar_wait_drain).
// The library's kernels never wait for ever: a wait that runs out sets the CTA's `dead` word and a
// device status word, the thread that issues asynchronous work stops and drains, everybody else
// falls through their later waits, and the kernel returns.  None of that can be seen in a
// healthy run, so this kernel makes a wait run out on purpose, in the only harmless way: an
// mbarrier on which, by a host-chosen flag, nobody arrives.  Nothing faults and nothing spins
// without a limit; the kernel returns after `limit_ns` and the context stays usable.
//
// One CTA of 96 threads, the roles of the library's rings in miniature:
//   warp 0  "issuer": lane 0 waits for `empty` (arrived on by warp 2 unless `skip_arrive`), then
//           stops and drains like a TMA issuer does;
//   warp 1  a second waiter on the same barrier: it must come back through the `dead` word (or
//           its own limit), and its following wait must return at once;
//   warp 2  the consumer that normally arrives.
#include <cuda_runtime.h>
#include <cstdint>

#include "../opencnn_b200/csrc/ptx.cuh"

namespace {

__device__ int g_status = 0;

struct ProbeOut {
  int issuer_ok;          // 1 if the issuer's wait succeeded
  int waiter_ok;          // 1 if the second waiter's wait succeeded
  int waiter_second_ok;   // after a give-up: result of the second waiter's next wait (on a barrier nobody ever arrives on)
  int drain_ok;           // 1 if mbar_wait_drain on a completed phase returned true
  int drain_timeout_ok;   // 1 if mbar_wait_drain on a phase that never completes returned false
  long long issuer_wait_ns, waiter_second_ns, drain_timeout_ns;
};

__global__ void __launch_bounds__(96, 1) wait_probe_kernel(ProbeOut *out, int skip_arrive, unsigned long long limit_ns, int *status) {
  __shared__ __align__(8) uint64_t bars[3];          // empty, never, done
  __shared__ int dead_word;
  volatile int *dead = &dead_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    dead_word = 0;
    ocb::mbar_init(ocb::smem_u32(bars + 0), 1);
    ocb::mbar_init(ocb::smem_u32(bars + 1), 1);
    ocb::mbar_init(ocb::smem_u32(bars + 2), 1);
    ocb::mbar_fence_init();
  }
  __syncthreads();
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t t0 = ocb::global_timer_ns();
      const bool ok = ocb::mbar_wait(ocb::smem_u32(bars + 0), 0, dead, status, limit_ns);
      out->issuer_wait_ns = (long long)(ocb::global_timer_ns() - t0);
      out->issuer_ok = ok ? 1 : 0;
      // the drain of an issuer: a phase that has completed, and one that never will
      ocb::mbar_arrive(ocb::smem_u32(bars + 2));
      out->drain_ok = ocb::mbar_wait_drain(ocb::smem_u32(bars + 2), 0, limit_ns) ? 1 : 0;
      const uint64_t t1 = ocb::global_timer_ns();
      out->drain_timeout_ok = ocb::mbar_wait_drain(ocb::smem_u32(bars + 1), 0, limit_ns) ? 0 : 1;
      out->drain_timeout_ns = (long long)(ocb::global_timer_ns() - t1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const bool ok = ocb::mbar_wait(ocb::smem_u32(bars + 0), 0, dead, status, 4 * limit_ns);
      out->waiter_ok = ok ? 1 : 0;
      if (!ok) {
        // after a give-up every later wait of the CTA returns at once, also on a barrier nobody
        // will ever arrive on
        const uint64_t t0 = ocb::global_timer_ns();
        out->waiter_second_ok = ocb::mbar_wait(ocb::smem_u32(bars + 1), 0, dead, status, limit_ns) ? 1 : 0;
        out->waiter_second_ns = (long long)(ocb::global_timer_ns() - t0);
      }
    }
  } else {
    if (lane == 0 && !skip_arrive) ocb::mbar_arrive(ocb::smem_u32(bars + 0));
  }
  __syncthreads();       // every thread gets here whatever the waits did
}

}  // namespace

// Runs the probe once, synchronously.  out[8]: issuer_ok, waiter_ok, waiter_second_ok, drain_ok,
// drain_timeout_ok, issuer_wait_ns, waiter_second_ns, drain_timeout_ns.  Returns a cudaError_t code.
extern "C" int wait_probe_run(int skip_arrive, unsigned long long limit_ns, long long *out8) {
  if (!out8 || limit_ns == 0 || limit_ns > 100000000ull) return (int)cudaErrorInvalidValue;   // at most 0.1 s per wait
  ProbeOut *d = nullptr;
  int *status = nullptr;
  cudaError_t e = cudaMalloc(&d, sizeof(ProbeOut));
  if (e == cudaSuccess) e = cudaMemset(d, 0xff, sizeof(ProbeOut));
  if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_status);
  if (e == cudaSuccess) {
    wait_probe_kernel<<<1, 96>>>(d, skip_arrive, limit_ns, status);
    e = cudaGetLastError();
  }
  ProbeOut h;
  if (e == cudaSuccess) e = cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) {
    out8[0] = h.issuer_ok; out8[1] = h.waiter_ok; out8[2] = h.waiter_second_ok; out8[3] = h.drain_ok;
    out8[4] = h.drain_timeout_ok; out8[5] = h.issuer_wait_ns; out8[6] = h.waiter_second_ns; out8[7] = h.drain_timeout_ns;
  }
  if (d) cudaFree(d);
  return (int)e;
}

// Same contract as the library's opencnn_last_device_status(): synchronise, read the status word,
// reset it to 0.
extern "C" int wait_probe_last_status(void) {
  int v = -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
  int zero = 0;
  cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  return v;
}
