// Filter transform U = G g G^T for Winograd F(2x2,3x3): filter CRSK -> workspace [C][4][4][K].
//
// Replaces the reference kernel FX (src/FX_m2.cu:51-91, launched from
// src/convolutionForward_32x64x8.cu:274).  The reference dispatches the row and column
// combinations through device function-pointer tables and stages them in local memory; here
// one thread owns four consecutive k of one channel and does everything in registers with
// 128-bit coalesced loads (9 per thread) and stores (16 per thread).  The arithmetic keeps the
// reference's grouping, ((a + c) +/- b) * 0.5 with every operation rounded on its own, so the
// workspace is bit-identical to the reference's.
#pragma once
#include <cuda_runtime.h>

namespace ocb {

__device__ __forceinline__ float fx_half_sum(float a, float c, float b) {
  return __fmul_rn(0.5f, __fadd_rn(__fadd_rn(a, c), b));
}
__device__ __forceinline__ float fx_half_dif(float a, float c, float b) {
  return __fmul_rn(0.5f, __fsub_rn(__fadd_rn(a, c), b));
}

// One lane of the transform: w[9] (r-major 3x3) -> u[16] (i-major 4x4).
__device__ __forceinline__ void fx_one(const float (&w)[9], float (&u)[16]) {
  float t[12];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    t[j] = w[j];
    t[3 + j] = fx_half_sum(w[j], w[6 + j], w[3 + j]);
    t[6 + j] = fx_half_dif(w[j], w[6 + j], w[3 + j]);
    t[9 + j] = w[6 + j];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    u[4 * i + 0] = t[3 * i];
    u[4 * i + 1] = fx_half_sum(t[3 * i], t[3 * i + 2], t[3 * i + 1]);
    u[4 * i + 2] = fx_half_dif(t[3 * i], t[3 * i + 2], t[3 * i + 1]);
    u[4 * i + 3] = t[3 * i + 2];
  }
}

// grid: ceil(C*K/4 / 128) blocks of 128 threads.  k4 = K/4.
__global__ void __launch_bounds__(128) fx_kernel(const float4 *__restrict__ g, float4 *__restrict__ U, int C, int k4) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= C * k4) return;
  const int c = idx / k4, kq = idx - c * k4;
  const float4 *src = g + (size_t)c * 9 * k4 + kq;
  float4 in[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) in[i] = __ldg(src + (size_t)i * k4);
  float wx[9], wy[9], wz[9], ww[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) {
    wx[i] = in[i].x; wy[i] = in[i].y; wz[i] = in[i].z; ww[i] = in[i].w;
  }
  float ux[16], uy[16], uz[16], uw[16];
  fx_one(wx, ux);
  fx_one(wy, uy);
  fx_one(wz, uz);
  fx_one(ww, uw);
  float4 *dst = U + (size_t)c * 16 * k4 + kq;
#pragma unroll
  for (int i = 0; i < 16; ++i) dst[(size_t)i * k4] = make_float4(ux[i], uy[i], uz[i], uw[i]);
}

}  // namespace ocb
