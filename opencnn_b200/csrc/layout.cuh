// Layout adapters either side of the operator: the reference keeps its tensors in CHWN / CRSK /
// KHWN and converts from the cuDNN-style NCHW / KCRS with a scatter kernel, data_cpy
// (src/openCNN_winograd.cu:147-153, launched :229-235), one thread per element with the channel
// as threadIdx.x (so C <= 1024 and every access strided); it compares its KHWN output with an
// NCHW result by index arithmetic on the host (:185-186).  All three conversions are the
// transpose of a dense row-major matrix:
//   NCHW -> CHWN :  [N][C*H*W]   -> [C*H*W][N]
//   KCRS -> CRSK :  [K][C*9]     -> [C*9][K]
//   KHWN -> NKHW :  [K*H*W][N]   -> [N][K*H*W]
// done here through a 32x33 shared-memory tile so that both the reads and the writes are
// 128-byte rows.  HBM-bound: 8 bytes of traffic per element.
#pragma once
#include <cuda_runtime.h>

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

inline cudaError_t launch_transpose(const float *src, float *dst, long long rows, long long cols, cudaStream_t stream) {
  if (!src || !dst || rows <= 0 || cols <= 0) return cudaErrorInvalidValue;
  const long long gx = (cols + 31) / 32, gy = (rows + 31) / 32;
  if (gx * gy > 2147483647ll) return cudaErrorInvalidValue;
  transpose_kernel<<<(unsigned)(gx * gy), dim3(32, 8), 0, stream>>>(src, dst, rows, cols, gx);
  return cudaGetLastError();
}

}  // namespace ocb
