// Layout adapters either side of the operator: the reference keeps its tensors in CHWN / CRSK /
// KHWN and converts from the cuDNN-style NCHW / KCRS with a scatter kernel, data_cpy
// (src/openCNN_winograd.cu:147-153, launched :229-235), one thread per element with the channel
// as threadIdx.x (so C <= 1024 and every access strided); it compares its KHWN output with an
// NCHW result by index arithmetic on the host (:185-186).  All three conversions are the
// transpose of a dense row-major matrix:
//   NCHW -> CHWN :  [N][C*H*W]   -> [C*H*W][N]
//   KCRS -> CRSK :  [K][C*9]     -> [C*9][K]
//   KHWN -> NKHW :  [K*H*W][N]   -> [N][K*H*W]
// HBM-bound: 8 bytes of traffic per element.  Two kernels: when both extents are multiples of 4
// and both pointers 16-byte aligned, a 64x64 tile moved with 128-bit loads and stores (16 KB in
// flight per CTA, eight CTAs per SM); otherwise a 32x32 tile moved element by element.  Both go
// through a padded shared-memory tile so that reads and writes are whole 128-byte (256-byte) rows.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace ocb {

// dst[c][r] = src[r][c] for a rows x cols matrix.  1-D grid of 32x32 tiles (column tiles fastest), block (32, 8).
__global__ void __launch_bounds__(256) transpose_kernel(const float *__restrict__ src, float *__restrict__ dst,
                                                       long long rows, long long cols, long long tiles_x) {
  __shared__ float tile[32][33];
  const long long t = blockIdx.x;
  const long long c0 = (t % tiles_x) * 32, r0 = (t / tiles_x) * 32;
#pragma unroll
  for (int i = threadIdx.y; i < 32; i += 8) {
    const long long r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = __ldg(src + r * cols + c);
  }
  __syncthreads();
#pragma unroll
  for (int i = threadIdx.y; i < 32; i += 8) {
    const long long c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[c * rows + r] = tile[threadIdx.x][i];
  }
}

// The same for rows % 4 == 0 and cols % 4 == 0: 64x64 tile, 256 threads, four 128-bit loads and four
// 128-bit stores per thread.  Tile pitch 65 floats: the element-wise shared-memory accesses of a
// warp (16 lanes along one axis with stride 4, the other 16 one step along the other axis) fall
// into 32 different banks on the way in and on the way out.
__global__ void __launch_bounds__(256) transpose4_kernel(const float *__restrict__ src, float *__restrict__ dst,
                                                        long long rows, long long cols, long long tiles_x) {
  __shared__ float tile[64][65];
  const long long t = blockIdx.x;
  const long long c0 = (t % tiles_x) * 64, r0 = (t / tiles_x) * 64;
  const int a = threadIdx.x >> 4, b4 = (threadIdx.x & 15) * 4;
  float4 v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long r = r0 + a + 16 * i, c = c0 + b4;
    v[i] = (r < rows && c < cols) ? __ldg(reinterpret_cast<const float4 *>(src + r * cols + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float *row = tile[a + 16 * i] + b4;
    row[0] = v[i].x; row[1] = v[i].y; row[2] = v[i].z; row[3] = v[i].w;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int cl = a + 16 * i;
    const long long c = c0 + cl, r = r0 + b4;
    if (r < rows && c < cols)
      *reinterpret_cast<float4 *>(dst + c * rows + r) = make_float4(tile[b4][cl], tile[b4 + 1][cl], tile[b4 + 2][cl], tile[b4 + 3][cl]);
  }
}

inline cudaError_t launch_transpose(const float *src, float *dst, long long rows, long long cols, cudaStream_t stream) {
  if (!src || !dst || rows <= 0 || cols <= 0) return cudaErrorInvalidValue;
  const bool vec = rows % 4 == 0 && cols % 4 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  const long long edge = vec ? 64 : 32;
  const long long gx = (cols + edge - 1) / edge, gy = (rows + edge - 1) / edge;
  if (gx * gy > 2147483647ll) return cudaErrorInvalidValue;
  if (vec) transpose4_kernel<<<(unsigned)(gx * gy), 256, 0, stream>>>(src, dst, rows, cols, gx);
  else     transpose_kernel<<<(unsigned)(gx * gy), dim3(32, 8), 0, stream>>>(src, dst, rows, cols, gx);
  return cudaGetLastError();
}

}  // namespace ocb
