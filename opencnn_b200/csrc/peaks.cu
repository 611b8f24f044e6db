// Measurement aid, not part of the operator: the FP32 FMA rate this GPU sustains, used as the
// roofline denominator of the FFMA path (no driver-supplied figure exists for the FP32 pipe).
// One persistent CTA per SM, 8 warps, 64 independent packed accumulators per lane issuing
// fma.rn.f32x2 back to back.
#include <cuda_runtime.h>
#include <cstdint>

namespace {

__global__ void __launch_bounds__(256, 1) ffma2_peak_kernel(float *out, int iters, float a, float b) {
  uint64_t acc[32], av, bv;
  asm("mov.b64 %0, {%1, %1};" : "=l"(av) : "f"(a));
  asm("mov.b64 %0, {%1, %1};" : "=l"(bv) : "f"(b));
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float x = (float)(i + threadIdx.x);
    asm("mov.b64 %0, {%1, %1};" : "=l"(acc[i]) : "f"(x));
  }
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 32; ++i) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(av), "l"(bv));
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
extern "C" int opencnn_peaks_fp32_tflops(int iters, int reps, double *tflops) {
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
    ffma2_peak_kernel<<<sms, 256>>>(out, iters, 1.0001f, 0.5f);
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
