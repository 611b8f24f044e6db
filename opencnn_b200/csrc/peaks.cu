// Measurement aids, not part of the operator.
//  * The FP32 FMA rate this GPU sustains, used as the roofline denominator of the FFMA path (no
//    driver-supplied figure exists for the FP32 pipe): one persistent CTA per SM, 8 warps, 32
//    independent packed accumulators per lane issuing fma.rn.f32x2 back to back.  Two operand
//    patterns: see the kernel.
//  * The same loop with other instructions mixed in: does a packed FMA leave issue slots free?
//  * How long one SM waits for a TMA load of a filter slice out of L2 (tiled box or linear bulk
//    copy), with one to three loads in flight: the latency that a two-stage ring cannot hide.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <vector>

#include "ptx.cuh"

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

// ---- issue-port probe ---------------------------------------------------------------------------
namespace {
// 64 packed FMAs per loop body plus EXTRA independent instructions of one KIND spread between them:
// KIND 0 integer xor, 1 register move, 2 scalar add.f32 (which shares the FMA pipe).
template <int EXTRA, int KIND>
__global__ void __launch_bounds__(256, 1) issue_probe_kernel(float *out, int iters, float a, float b) {
  uint64_t acc[32], av, bv;
  asm("mov.b64 %0, {%1, %2};" : "=l"(av) : "f"(0.5f * a), "f"(1.5f * a));
  asm("mov.b64 %0, {%1, %2};" : "=l"(bv) : "f"(2.f * b), "f"(3.f * b));
#pragma unroll
  for (int i = 0; i < 32; ++i) asm("mov.b64 %0, {%1, %2};" : "=l"(acc[i]) : "f"((float)i), "f"((float)(i + threadIdx.x)));
  unsigned x[8];
  float fx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { x[i] = threadIdx.x + i; fx[i] = (float)i; }
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[i]) : "l"(av), "l"(bv));
        if ((i + 32 * r) * EXTRA / 64 != (i + 32 * r + 1) * EXTRA / 64) {
          if (KIND == 0) asm volatile("xor.b32 %0, %0, %1;" : "+r"(x[i & 7]) : "r"(x[(i + 1) & 7]));
          else if (KIND == 1) asm volatile("mov.b32 %0, %1;" : "=r"(x[i & 7]) : "r"(x[(i + 3) & 7]));
          else asm volatile("add.rn.f32 %0, %0, %1;" : "+f"(fx[i & 7]) : "f"(a));
        }
      }
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) { float lo, hi; asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[i])); s += lo + hi; }
#pragma unroll
  for (int i = 0; i < 8; ++i) s += (float)x[i] + fx[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

template <int EXTRA, int KIND> float time_issue_probe(float *out, int sms, int iters) {
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  float best = 1e30f;
  for (int r = 0; r < 4; ++r) {
    cudaEventRecord(t0, 0);
    issue_probe_kernel<EXTRA, KIND><<<sms, 256>>>(out, iters, 1.0001f, 0.5f);
    cudaEventRecord(t1, 0);
    if (cudaEventSynchronize(t1) != cudaSuccess) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, t0, t1);
    if (r > 0 && ms < best) best = ms;
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  return best;
}
}  // namespace

// Milliseconds for `iters` loop bodies of 64 packed FMAs + `extra` (0, 8, 16, 32 or 64) instructions of `kind`
// (0 xor, 1 mov, 2 add.f32) on every SM, 8 warps each.  Returns a cudaError_t code (1 for unsupported arguments).
extern "C" int opencnn_peaks_issue_probe(int extra, int kind, int iters, double *ms) {
  int dev = 0, sms = 0;
  if (!ms || cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return (int)cudaErrorInvalidValue;
  float *out = nullptr;
  if (cudaMalloc(&out, (size_t)sms * 256 * sizeof(float)) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
  float t = -1.f;
#define OCB_CASE(E, K) if (extra == E && kind == K) t = time_issue_probe<E, K>(out, sms, iters);
  OCB_CASE(0, 0) OCB_CASE(8, 0) OCB_CASE(16, 0) OCB_CASE(32, 0) OCB_CASE(64, 0)
  OCB_CASE(16, 1) OCB_CASE(32, 1) OCB_CASE(16, 2) OCB_CASE(32, 2)
#undef OCB_CASE
  cudaFree(out);
  if (t < 0.f) return (int)cudaErrorInvalidValue;
  *ms = t;
  return (int)cudaGetLastError();
}

// ---- TMA latency probe --------------------------------------------------------------------------
namespace {
__device__ __forceinline__ void bulk_load_linear(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// One thread per CTA issues loads of `bytes` into a ring of three 64 KB slots and waits for the load issued
// `depth - 1` iterations earlier.  Tiled: the 4-D box {64 bf16, 16 channels, 2 row blocks, bytes / 4096 positions}
// of a transformed-filter workspace [C][16][K]; linear: the same number of contiguous bytes.
__global__ void __launch_bounds__(128, 1) tma_latency_kernel(const __grid_constant__ CUtensorMap map, const uint8_t *lin, size_t lin_bytes,
                                                             uint32_t bytes, int tiled, int depth, int iters, int n_ci, long long *out,
                                                             int *status) {
  extern __shared__ __align__(1024) uint8_t sm[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 3 * 65536);
  __shared__ int dead;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < 3; ++s) ocb::mbar_init(ocb::smem_u32(bars + s), 1);
    ocb::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    for (int it = 0; it < iters + depth; ++it) {
      if (it < iters) {
        const int s = it % 3;
        const uint32_t bar = ocb::smem_u32(bars + s), dst = ocb::smem_u32(sm + s * 65536);
        ocb::mbar_arrive_expect_tx(bar, bytes);
        const int ci = (it * 7 + (int)blockIdx.x) % n_ci;
        if (tiled) ocb::tma_load_4d(dst, &map, bar, 0, ci * 16, 0, 0);
        else bulk_load_linear(dst, lin + ((size_t)ci * bytes) % (lin_bytes - bytes), bytes, bar);
      }
      const int w = it - depth + 1;
      if (w >= 0 && w < iters && !ocb::mbar_wait(ocb::smem_u32(bars + w % 3), (w / 3) & 1, &dead, status)) break;
    }
    out[blockIdx.x] = clock64() - t0;
  }
}
__device__ int g_probe_status = 0;
}  // namespace

// Tensor map of a BF16 transformed-filter workspace [C][16][K] with boxes {64 filters, 16 channels, 2 row blocks,
// bytes / 4096 positions} and 128-byte swizzle.
static cudaError_t make_workspace_map(CUtensorMap *map, void *ws, int C, int K, int bytes) {
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  using Enc = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                           const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                           CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return cudaErrorNotSupported;
  cuuint64_t dims[4] = {64, (cuuint64_t)C, (cuuint64_t)K / 64, 16};
  cuuint64_t strides[3] = {(cuuint64_t)16 * K * 2, 128, (cuuint64_t)K * 2};
  cuuint32_t box[4] = {64, 16, 2, (cuuint32_t)(bytes / 4096)};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (reinterpret_cast<Enc>(fn)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ws, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  return cudaSuccess;
}

// Average cycles per load (issue to completion, `depth` loads in flight) over `grid` CTAs, one per SM.
// bytes: 32768 or 65536; tiled: 1 = 4-D TMA box, 0 = linear bulk copy.  Returns a cudaError_t code.
extern "C" int opencnn_peaks_tma_latency(int bytes, int tiled, int depth, int iters, int grid, double *cycles_per_load) {
  if (!cycles_per_load || (bytes != 32768 && bytes != 65536) || depth < 1 || depth > 3 || iters < 1 || grid < 1)
    return (int)cudaErrorInvalidValue;
  const int C = 1024, K = 128;                                  // bf16 workspace of 4 MB: stays in L2
  const size_t ws_bytes = (size_t)C * 16 * K * 2;
  uint8_t *ws = nullptr;
  long long *out = nullptr;
  int *status = nullptr;
  cudaError_t e = cudaMalloc(&ws, ws_bytes);
  if (e == cudaSuccess) e = cudaMemset(ws, 0, ws_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&out, (size_t)grid * sizeof(long long));
  if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_probe_status);
  CUtensorMap map;
  if (e == cudaSuccess) e = make_workspace_map(&map, ws, C, K, bytes);
  const size_t smem = 3 * 65536 + 64;
  if (e == cudaSuccess) e = cudaFuncSetAttribute(tma_latency_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    for (int rep = 0; rep < 2; ++rep)                          // the first run warms L2 and the instruction cache
      tma_latency_kernel<<<grid, 128, smem>>>(map, ws, ws_bytes, (uint32_t)bytes, tiled, depth, iters, C / 16, out, status);
    e = cudaDeviceSynchronize();
  }
  if (e == cudaSuccess) {
    std::vector<long long> h(grid);
    e = cudaMemcpy(h.data(), out, (size_t)grid * sizeof(long long), cudaMemcpyDeviceToHost);
    double s = 0.0;
    for (long long v : h) s += (double)v;
    *cycles_per_load = s / grid / iters;
  }
  if (ws) cudaFree(ws);
  if (out) cudaFree(out);
  return (int)e;
}

// ---- tcgen05.mma issue-rate probe ---------------------------------------------------------------
#include "wino_tc.cuh"   // tcgen05 helpers: tmem_alloc_512, tc_commit, smem_desc, fences

namespace {
struct MmaRateCfg {
  uint32_t idesc;
  uint32_t a_lbo, a_sbo, a_mode, b_lbo, b_sbo, b_mode;
  uint32_t a_off[16], b_off[16];   // byte offsets of the 16 operand tiles inside the A and B regions
  uint32_t n;                      // MMA N: accumulator j sits at TMEM column (j * n) % 512
  uint32_t sync;                   // 1: commit and wait after every group (the round trip of a one-stage pipeline)
};
constexpr uint32_t kRateABytes = 64 * 1024, kRateBBytes = 128 * 1024;

// `issuers` threads of a CTA (lane 0 of warps 0 .. issuers-1) each issue `iters` groups of 16 / issuers MMAs
// (M = 128, accumulators in disjoint TMEM columns) on zero-filled shared memory, commit once and wait; the other
// threads only clear shared memory.  Results are never read: only the issue-to-completion time of the chains
// counts (the slowest issuer's).  KIND 0 = kind::f16 (BF16, K = 16), 1 = kind::tf32 (K = 8).
template <int KIND, int ISSUERS>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(const MmaRateCfg cfg, int iters, long long *out, int *status) {
  extern __shared__ __align__(1024) uint8_t sm[];
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar[4];
  __shared__ long long took[4];
  __shared__ int dead;
  for (uint32_t i = threadIdx.x; i < (kRateABytes + kRateBBytes) / 16; i += blockDim.x)
    reinterpret_cast<uint4 *>(sm)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    dead = 0;
    for (int i = 0; i < 4; ++i) ocb::mbar_init(ocb::smem_u32(bar + i), 1);
    ocb::mbar_fence_init();
  }
  if (threadIdx.x < 32) ocb::tmem_alloc_512(ocb::smem_u32(&tmem_slot));
  ocb::fence_proxy_async_smem();
  ocb::tc_fence_before();
  __syncthreads();
  ocb::tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0 && warp < ISSUERS) {
    constexpr int kPer = 16 / ISSUERS;
    const uint32_t a0 = ocb::smem_u32(sm), b0 = a0 + kRateABytes;
    uint64_t ad[kPer], bd[kPer];
    uint32_t col[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int x = warp * kPer + j;
      ad[j] = ocb::smem_desc(a0 + cfg.a_off[x], cfg.a_lbo, cfg.a_sbo, cfg.a_mode);
      bd[j] = ocb::smem_desc(b0 + cfg.b_off[x], cfg.b_lbo, cfg.b_sbo, cfg.b_mode);
      col[j] = tmem + ((uint32_t)x * cfg.n) % 512u;
    }
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int j = 0; j < kPer; ++j) ocb::tc_mma<KIND>(col[j], ad[j], bd[j], cfg.idesc, 1u);
      if (cfg.sync) {
        ocb::tc_commit(ocb::smem_u32(bar + warp));
        if (!ocb::mbar_wait(ocb::smem_u32(bar + warp), (uint32_t)it & 1u, &dead, status)) break;
        ocb::tc_fence_after();
      }
    }
    if (!cfg.sync) {
      ocb::tc_commit(ocb::smem_u32(bar + warp));
      ocb::mbar_wait(ocb::smem_u32(bar + warp), 0, &dead, status);
    }
    took[warp] = clock64() - t0;
  }
  ocb::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    long long m = 0;
    for (int i = 0; i < ISSUERS; ++i) m = took[i] > m ? took[i] : m;
    out[blockIdx.x] = m;
  }
  if (threadIdx.x < 32) ocb::tmem_dealloc_512(tmem);
}
}  // namespace

// Average SM cycles per tcgen05.mma (cta_group::1, M = 128, fp32 accumulate) when 16 * iters MMAs are issued by
// `issuers` (1, 2 or 4) threads of a CTA, over `grid` CTAs, one per SM.
//   kind    0 = BF16 (K = 16 per MMA), 1 = TF32 (K = 8)
//   n       MMA N: 32, 64, 128 or 256
//   layout  0 = both operands MN-major as the fused kernels hold them (A 128-byte swizzle, B 64-byte swizzle for
//               BF16; 128-byte swizzle with 32-byte atoms for TF32), 16 operand tiles at separate addresses;
//           1 = both K-major, no swizzle (8 x 16-byte core matrices), rows of one K-step (32 bytes);
//           2 = both K-major, 32-byte swizzle, rows of one K-step;
//           3 = both K-major, 128-byte swizzle, rows of four K-steps (the usual GEMM operand layout).
//   sync    0 = one commit at the end (the rate of the tensor pipe); 1 = every thread commits and waits after each
//           of its groups of 16 / issuers MMAs: cycles per MMA then include the commit -> mbarrier -> wake-up
//           round trip that a pipeline stage pays before it can be refilled.
// Returns a cudaError_t code; -1 if a wait ran out.
static int mma_rate(int kind, int n, int layout, int issuers, int sync, int iters, int grid, double *cycles_per_mma) {
  if (!cycles_per_mma || kind < 0 || kind > 1 || (n != 32 && n != 64 && n != 128 && n != 256) || layout < 0 || layout > 3 ||
      (issuers != 1 && issuers != 2 && issuers != 4) || iters < 1 || grid < 1)
    return (int)cudaErrorInvalidValue;
  MmaRateCfg c{};
  const uint32_t fmt = kind == 0 ? 1u : 2u, mn_major = layout == 0 ? 1u : 0u;
  c.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (mn_major << 15) | (mn_major << 16) | ((uint32_t)(n >> 3) << 17) | (8u << 24);
  c.n = (uint32_t)n;
  c.sync = sync ? 1u : 0u;
  uint32_t a_tile, b_tile, kdiv = 1, kstep = 0;
  switch (layout) {
    case 0:
      if (kind == 0) { c.a_lbo = 2048; c.a_sbo = 1024; c.a_mode = 2; c.b_lbo = 1024; c.b_sbo = 512; c.b_mode = 4; }
      else           { c.a_lbo = 1024; c.a_sbo = 512;  c.a_mode = 1; c.b_lbo = 1024; c.b_sbo = 512; c.b_mode = 1; }
      a_tile = 4096; b_tile = 32u * n;
      break;
    case 1:
      c.a_lbo = c.b_lbo = 128; c.a_sbo = c.b_sbo = 256; c.a_mode = c.b_mode = 0;
      a_tile = 4096; b_tile = 32u * n;
      break;
    case 2:
      c.a_lbo = c.b_lbo = 16; c.a_sbo = c.b_sbo = 256; c.a_mode = c.b_mode = 6;
      a_tile = 4096; b_tile = 32u * n;
      break;
    default:
      c.a_lbo = c.b_lbo = 16; c.a_sbo = c.b_sbo = 1024; c.a_mode = c.b_mode = 2;
      a_tile = 16384; b_tile = 128u * n; kdiv = 4; kstep = 32;
      break;
  }
  for (uint32_t j = 0; j < 16; ++j) {
    c.a_off[j] = (j / kdiv) * a_tile + (j % kdiv) * kstep;
    c.b_off[j] = (j / kdiv) * b_tile + (j % kdiv) * kstep;
    // (a K-step offset stays inside its tile: the rows of a 128-byte-swizzle tile hold four K-steps)
    if ((j / kdiv + 1) * a_tile > kRateABytes || (j / kdiv + 1) * b_tile > kRateBBytes) return (int)cudaErrorInvalidValue;
  }
  long long *out = nullptr;
  int *status = nullptr;
  cudaError_t e = cudaMalloc(&out, (size_t)grid * sizeof(long long));
  if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_probe_status);
  if (e == cudaSuccess) e = cudaMemset(status, 0, sizeof(int));
  const size_t smem = kRateABytes + kRateBBytes;
  using Kern = void (*)(const MmaRateCfg, int, long long *, int *);
  const Kern kerns[2][3] = {{mma_rate_kernel<0, 1>, mma_rate_kernel<0, 2>, mma_rate_kernel<0, 4>},
                            {mma_rate_kernel<1, 1>, mma_rate_kernel<1, 2>, mma_rate_kernel<1, 4>}};
  const Kern kern = kerns[kind][issuers == 1 ? 0 : issuers == 2 ? 1 : 2];
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    for (int rep = 0; rep < 2; ++rep) kern<<<grid, 128, smem>>>(c, iters, out, status);
    e = cudaDeviceSynchronize();
  }
  int st = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) {
    std::vector<long long> h(grid);
    e = cudaMemcpy(h.data(), out, (size_t)grid * sizeof(long long), cudaMemcpyDeviceToHost);
    double s = 0.0;
    for (long long v : h) s += (double)v;
    *cycles_per_mma = s / grid / iters / 16.0;
  }
  if (out) cudaFree(out);
  if (e == cudaSuccess && st != 0) return -1;
  return (int)e;
}

extern "C" int opencnn_peaks_mma_rate(int kind, int n, int layout, int issuers, int iters, int grid, double *cycles_per_mma) {
  return mma_rate(kind, n, layout, issuers, 0, iters, grid, cycles_per_mma);
}
// Cycles per group of 16 / issuers MMAs (layout 0) when each issuing thread commits and waits after every group.
extern "C" int opencnn_peaks_mma_round_trip(int kind, int n, int issuers, int iters, int grid, double *cycles_per_group) {
  const int e = mma_rate(kind, n, 0, issuers, 1, iters, grid, cycles_per_group);
  if (e == 0) *cycles_per_group *= 16.0;   // mma_rate divides by the 16 MMAs of a group
  return e;
}

// ---- do TMA writes and MMA operand reads share the shared-memory bandwidth of an SM? -------------------------
namespace {
constexpr uint32_t kShareOperandBytes = 80 * 1024;   // 16 A tiles of 4 KB + 16 B tiles of 1 KB
// Two threads issue `groups` groups of 8 MMAs each (BF16, 128 x 32 x 16, the operand layout of the fused kernels),
// a third issues `loads` TMA loads of 64 KB with two in flight into a ring beside the operands.  Each role records
// how long it took; a role with a count of 0 sits the run out.
__global__ void __launch_bounds__(128, 1) smem_share_kernel(const __grid_constant__ CUtensorMap map, const MmaRateCfg cfg, int groups,
                                                            int loads, int n_ci, long long *out, int *status) {
  extern __shared__ __align__(1024) uint8_t sm[];
  uint8_t *ring = sm + kShareOperandBytes;           // 80 KB is a multiple of 1024: the ring keeps the swizzle alignment
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar[4];
  __shared__ long long took[3];
  __shared__ int dead;
  for (uint32_t i = threadIdx.x; i < kShareOperandBytes / 16; i += blockDim.x) reinterpret_cast<uint4 *>(sm)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    dead = 0;
    took[0] = took[1] = took[2] = 0;
    for (int i = 0; i < 4; ++i) ocb::mbar_init(ocb::smem_u32(bar + i), 1);
    ocb::mbar_fence_init();
  }
  if (threadIdx.x < 32) ocb::tmem_alloc_512(ocb::smem_u32(&tmem_slot));
  ocb::fence_proxy_async_smem();
  ocb::tc_fence_before();
  __syncthreads();
  ocb::tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    if (warp < 2 && groups > 0) {
      const uint32_t a0 = ocb::smem_u32(sm), b0 = a0 + 64 * 1024;
      uint64_t ad[8], bd[8];
      uint32_t col[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int x = warp * 8 + j;
        ad[j] = ocb::smem_desc(a0 + x * 4096, cfg.a_lbo, cfg.a_sbo, cfg.a_mode);
        bd[j] = ocb::smem_desc(b0 + x * 1024, cfg.b_lbo, cfg.b_sbo, cfg.b_mode);
        col[j] = tmem + (uint32_t)x * 32u;
      }
      const long long t0 = clock64();
      for (int it = 0; it < groups; ++it) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ocb::tc_mma<0>(col[j], ad[j], bd[j], cfg.idesc, 1u);
      }
      ocb::tc_commit(ocb::smem_u32(bar + warp));
      ocb::mbar_wait(ocb::smem_u32(bar + warp), 0, &dead, status);
      took[warp] = clock64() - t0;
    } else if (warp == 2 && loads > 0) {
      const long long t0 = clock64();
      int issued = 0, waited = 0;
      for (int it = 0; it < loads + 1; ++it) {
        if (it < loads) {
          const int s = it & 1;
          const uint32_t b = ocb::smem_u32(bar + 2 + s);
          ocb::mbar_arrive_expect_tx(b, 65536u);
          ocb::tma_load_4d(ocb::smem_u32(ring + s * 65536), &map, b, 0, ((it * 7 + (int)blockIdx.x) % n_ci) * 16, 0, 0);
          issued = it + 1;
        }
        const int w = it - 1;                        // two in flight: wait for the load before the one just issued
        if (w >= 0) {
          if (!ocb::mbar_wait(ocb::smem_u32(bar + 2 + (w & 1)), (uint32_t)(w >> 1) & 1u, &dead, status)) break;
          waited = w + 1;
        }
      }
      took[2] = clock64() - t0;
      // after a wait that gave up: let what is still in flight land before the CTA exits
      for (int w = waited; w < issued; ++w) ocb::mbar_wait_drain(ocb::smem_u32(bar + 2 + (w & 1)), (uint32_t)(w >> 1) & 1u);
    }
  }
  ocb::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    out[3 * blockIdx.x + 0] = took[0] > took[1] ? took[0] : took[1];
    out[3 * blockIdx.x + 1] = took[2];
  }
  if (threadIdx.x < 32) ocb::tmem_dealloc_512(tmem);
}
}  // namespace

// Runs `groups` groups of 16 MMAs (two issuing threads) and `loads` 64 KB TMA loads (two in flight) at the same time
// on each of `grid` SMs and returns the average cycles each side took.  Either count may be 0.
extern "C" int opencnn_peaks_smem_share(int groups, int loads, int grid, double *mma_cycles, double *tma_cycles) {
  if (!mma_cycles || !tma_cycles || groups < 0 || loads < 0 || grid < 1) return (int)cudaErrorInvalidValue;
  const int C = 1024, K = 128;                                  // bf16 workspace of 4 MB: stays in L2
  const size_t ws_bytes = (size_t)C * 16 * K * 2;
  uint8_t *ws = nullptr;
  long long *out = nullptr;
  int *status = nullptr;
  cudaError_t e = cudaMalloc(&ws, ws_bytes);
  if (e == cudaSuccess) e = cudaMemset(ws, 0, ws_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&out, (size_t)grid * 3 * sizeof(long long));
  if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_probe_status);
  if (e == cudaSuccess) e = cudaMemset(status, 0, sizeof(int));
  CUtensorMap map;
  if (e == cudaSuccess) e = make_workspace_map(&map, ws, C, K, 65536);
  MmaRateCfg c{};
  c.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(32 >> 3) << 17) | (8u << 24);
  c.a_lbo = 2048; c.a_sbo = 1024; c.a_mode = 2; c.b_lbo = 1024; c.b_sbo = 512; c.b_mode = 4;
  const size_t smem = kShareOperandBytes + 2 * 65536;
  if (e == cudaSuccess) e = cudaFuncSetAttribute(smem_share_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    for (int rep = 0; rep < 2; ++rep) smem_share_kernel<<<grid, 128, smem>>>(map, c, groups, loads, C / 16, out, status);
    e = cudaDeviceSynchronize();
  }
  int st = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) {
    std::vector<long long> h((size_t)grid * 3);
    e = cudaMemcpy(h.data(), out, h.size() * sizeof(long long), cudaMemcpyDeviceToHost);
    double a = 0.0, b = 0.0;
    for (int i = 0; i < grid; ++i) { a += (double)h[3 * i]; b += (double)h[3 * i + 1]; }
    *mma_cycles = a / grid;
    *tma_cycles = b / grid;
  }
  if (ws) cudaFree(ws);
  if (out) cudaFree(out);
  if (e == cudaSuccess && st != 0) return -1;
  return (int)e;
}
