// Measurement aid, not part of the operator: the FP32 FMA rate this GPU sustains, used as the
// roofline denominator of the FFMA path (no driver-supplied figure exists for the FP32 pipe).
// One persistent CTA per SM, 8 warps, 32 independent packed accumulators per lane issuing
// fma.rn.f32x2 back to back.  Two operand patterns: see the kernel.
#include <cuda_runtime.h>
#include <cstdint>

namespace {

// BUSY = false: multiplier and addend pairs with equal halves, accumulators that converge - the
// operands barely change, and the pipe issues one packed FMA every other clock: the issue-rate
// peak.  BUSY = true: the same instruction stream on operands whose mantissas keep changing
// (unequal halves, accumulators that grow), as in a real contraction: the same code then runs
// about 8 % slower per SM clock on this part (measured 0.458 instead of 0.500 instructions per
// clock and scheduler), i.e. the sustained rate depends on the data, not only on the code.
template <bool BUSY>
__global__ void __launch_bounds__(256, 1) ffma2_peak_kernel(float *out, int iters, float a, float b) {
  uint64_t acc[32], av, bv;
  if (BUSY) {
    asm("mov.b64 %0, {%1, %2};" : "=l"(av) : "f"(0.5f * a), "f"(1.5f * a));
    asm("mov.b64 %0, {%1, %2};" : "=l"(bv) : "f"(2.f * b), "f"(3.f * b));
  } else {
    asm("mov.b64 %0, {%1, %1};" : "=l"(av) : "f"(a));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bv) : "f"(b));
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float x = (float)(i + threadIdx.x), x2 = BUSY ? (float)i : x;
    asm("mov.b64 %0, {%1, %2};" : "=l"(acc[i]) : "f"(x2), "f"(x));
  }
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (BUSY) asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[i]) : "l"(av), "l"(bv));   // acc += a * b
      else      asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(av), "l"(bv));   // acc = acc * a + b
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[i]));
    s += lo + hi;
  }
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace

// Runs the kernel `reps` times and writes the best TFLOP/s (2 flops per FMA).  Returns a
// cudaError_t code.  Synchronous.
static int run_probe(bool busy, int iters, int reps, double *tflops) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  float *out = nullptr;
  e = cudaMalloc(&out, (size_t)sms * 256 * sizeof(float));
  if (e != cudaSuccess) return (int)e;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  double best = 0.0;
  for (int r = 0; r < reps + 1; ++r) {
    cudaEventRecord(t0, 0);
    if (busy) ffma2_peak_kernel<true><<<sms, 256>>>(out, iters, 1.0001f, 0.5f);
    else      ffma2_peak_kernel<false><<<sms, 256>>>(out, iters, 1.0001f, 0.5f);
    cudaEventRecord(t1, 0);
    e = cudaEventSynchronize(t1);
    if (e != cudaSuccess) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, t0, t1);
    const double tf = 2.0 * 64.0 * iters * 256.0 * sms / (ms * 1e-3) * 1e-12;
    if (r > 0 && tf > best) best = tf;
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(out);
  if (tflops) *tflops = best;
  return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

extern "C" int opencnn_peaks_fp32_tflops(int iters, int reps, double *tflops) { return run_probe(false, iters, reps, tflops); }
// The same loop on operands that keep changing (see the kernel's comment).
extern "C" int opencnn_peaks_fp32_tflops_busy(int iters, int reps, double *tflops) { return run_probe(true, iters, reps, tflops); }
