// Shared-memory LDS / STS issue-rate probes for sm_100a: the counterpart of the reference's
// Turing-only SASS microbenchmarks (bench/smem/LDS/main.cu:14-41, bench/smem/STS/main.cu:41-82,
// kernels bench/smem/{LDS,STS}/*.sass).  Same protocol - one CTA of one warp, 128 x 128
// back-to-back instructions between two clock reads, clocks per instruction and bytes per clock
// - but written as CUDA C++ with inline PTX so that it runs on the GPU the library targets.
// Measurement aid only; not part of the operator.
#include <cuda_runtime.h>
#include <cstdint>

namespace {

enum Op : int { kLds32 = 0, kLds64, kLds128, kSts32, kSts64, kSts128 };

// Byte offset of a lane for a pattern.
//  0 contiguous (conflict-free)        1 every lane the same address (broadcast)
//  2 two-way bank conflict (stride 2 accesses)
//  3 this library's STS.64 staging deposit (row pitch 34 floats, quarter-warp per position)
//  4 the reference's optSTS64 deposit pattern (src/store_and_transform_output_optSTS64.cuh:73-75, pitch 138 float2)
//  5 this library's main-loop image-pair LDS.128 (4 distinct quads per half-warp, swapped in odd quarters)
//  6 this library's main-loop filter LDS.128 (8 distinct quads per half-warp)
//  7 the reference's "opt3" 64-bit pattern, used for both its optLDS64 read-back and its STS.64 probe: the 32
//    lanes cover 256 contiguous bytes, but lanes 8-15 and 16-23 are swapped, so that lanes {0-7, 16-23} hold
//    the first 128 bytes and {8-15, 24-31} the second (bench/smem/LDS/lds64_opt3.sass:13-27,
//    bench/smem/STS/sts64_opt3.sass:14-29)
//  8 the reference's two-way-conflict STS.64: 64-bit words 0, 2, .. 30 in lanes 0-15 and 32, 34, .. 62 in
//    lanes 16-31 (bench/smem/STS/sts64_2bank_conflict.sass:13-22)
//  9 the reference's same-address STS.64: word (lane % 8), i.e. every address four times
//    (bench/smem/STS/sts64_broadcast.sass:13-27)
// 10 the reference's half-active STS.128: lane * 16 bytes, only lanes with lane % 16 <= 8 take part
//    (bench/smem/STS/sts128.sass:13-22, run at bench/smem/STS/main.cu:99-100)
__device__ __forceinline__ uint32_t lane_offset(int pattern, int lane, int width) {
  switch (pattern) {
    case 0: return lane * width;
    case 1: return 0;
    case 2: return lane * width * 2;
    case 3: {
      const int q = lane >> 3, qp = q & 1, nh = lane & 1, kg = (lane & 7) >> 1;
      return (uint32_t)(((q * 8 + 2 * kg + qp) * 34 + 4 * (4 * nh + qp)) * 4);
    }
    case 4: {
      const int a = ((lane % 8) / 2) * 34 + lane % 2 + (lane / 16) * 2 + ((lane / 8) % 2) * 8;
      return (uint32_t)(a * 8);
    }
    case 5: {
      const int q = lane >> 3, qp = q & 1, nh = lane & 1;
      return (uint32_t)((q * 32 + 16 * nh + 4 * qp) * 4);
    }
    case 6: {
      const int q = lane >> 3, qp = q & 1, kg = (lane & 7) >> 1;
      return (uint32_t)((q * 64 + 8 * kg + 4 * qp) * 4);
    }
    case 7: {
      const int a = lane % 16;
      return (uint32_t)((((lane / 16) * 8 + a) + (a >= 8 ? 8 : 0)) * 8);
    }
    case 8: return (uint32_t)((((lane * 2) % 32) + (lane / 16) * 32) * 8);
    case 9: return (uint32_t)((lane % 8) * 8);
    case 10: return lane * 16;
    default: return 0;
  }
}
// Pattern 10 runs with part of the warp switched off, like the reference's kernel (its inactive lanes exit).
__device__ __forceinline__ bool lane_active(int pattern, int lane) { return pattern != 10 || (lane % 16) <= 8; }

// clock read that the compiler may not move across the volatile loads and stores
__device__ __forceinline__ long long clock_now() {
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
  return t;
}

template <int OP>
__global__ void __launch_bounds__(32, 1) smem_probe_kernel(long long *clocks, int pattern, float *sink) {
  __shared__ __align__(16) float buf[12288];
  for (int i = threadIdx.x; i < 12288; i += 32) buf[i] = (float)i;
  __syncwarp();
  constexpr int width = (OP == kLds32 || OP == kSts32) ? 4 : (OP == kLds64 || OP == kSts64) ? 8 : 16;
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(buf) + lane_offset(pattern, threadIdx.x, width);
  float a = 1.f, b = 2.f, c = 3.f, d = 4.f;
  if (!lane_active(pattern, threadIdx.x)) return;
  const long long t0 = clock_now();
  for (int outer = 0; outer < 128; ++outer) {
#pragma unroll
    for (int i = 0; i < 128; ++i) {
      if (OP == kLds32) asm volatile("ld.volatile.shared.f32 %0, [%1];" : "=f"(a) : "r"(addr) : "memory");
      if (OP == kLds64) asm volatile("ld.volatile.shared.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "r"(addr) : "memory");
      if (OP == kLds128) asm volatile("ld.volatile.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "r"(addr) : "memory");
      if (OP == kSts32) asm volatile("st.volatile.shared.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
      if (OP == kSts64) asm volatile("st.volatile.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
      if (OP == kSts128) asm volatile("st.volatile.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
    }
  }
  const long long t1 = clock_now();
  if (threadIdx.x == 0) clocks[0] = t1 - t0;
  sink[threadIdx.x] = a + b + c + d + buf[threadIdx.x];
}

}  // namespace

// op: 0 LDS.32, 1 LDS.64, 2 LDS.128, 3 STS.32, 4 STS.64, 5 STS.128; pattern: see lane_offset.
// Writes clocks per warp instruction.  Synchronous.  Returns a cudaError_t code.
extern "C" int opencnn_smem_probe(int op, int pattern, double *clocks_per_instruction) {
  if (op < 0 || op > 5 || pattern < 0 || pattern > 10 || !clocks_per_instruction) return (int)cudaErrorInvalidValue;
  long long *d_clk = nullptr;
  float *d_sink = nullptr;
  cudaError_t e = cudaMalloc(&d_clk, sizeof(long long));
  if (e == cudaSuccess) e = cudaMalloc(&d_sink, 32 * sizeof(float));
  if (e == cudaSuccess) {
    for (int rep = 0; rep < 2; ++rep) {     // first run warms the instruction cache
      switch (op) {
        case 0: smem_probe_kernel<kLds32><<<1, 32>>>(d_clk, pattern, d_sink); break;
        case 1: smem_probe_kernel<kLds64><<<1, 32>>>(d_clk, pattern, d_sink); break;
        case 2: smem_probe_kernel<kLds128><<<1, 32>>>(d_clk, pattern, d_sink); break;
        case 3: smem_probe_kernel<kSts32><<<1, 32>>>(d_clk, pattern, d_sink); break;
        case 4: smem_probe_kernel<kSts64><<<1, 32>>>(d_clk, pattern, d_sink); break;
        default: smem_probe_kernel<kSts128><<<1, 32>>>(d_clk, pattern, d_sink); break;
      }
    }
    long long h = 0;
    e = cudaMemcpy(&h, d_clk, sizeof(h), cudaMemcpyDeviceToHost);
    *clocks_per_instruction = (double)h / (128.0 * 128.0);
  }
  if (d_clk) cudaFree(d_clk);
  if (d_sink) cudaFree(d_sink);
  return (int)(e != cudaSuccess ? e : cudaGetLastError());
}
