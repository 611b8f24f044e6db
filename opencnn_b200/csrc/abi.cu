// C ABI of the library (declared in include/opencnn_b200.h): argument validation, TMA
// descriptors, launches.  Host side of the operator that replaces the reference's
// convolutionForward (src/openCNN_winograd.cu:204-219) and convolutionForward_32x64x8
// (src/convolutionForward_32x64x8.cu:264-284).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <new>

#include "../../include/opencnn_b200.h"
#include "fx.cuh"
#include "layout.cuh"
#include "wino_fp32.cuh"
#include "wino_tc.cuh"
#include "wino_tc2.cuh"
#include "wino_tc64.cuh"

#if defined(BASE)
#define OCB_VARIANT ocb::kBase
#define OCB_VARIANT_NAME "BASE"
#elif defined(OPTSTS64_CMP)
#define OCB_VARIANT ocb::kOptSts64Cmp
#define OCB_VARIANT_NAME "OPTSTS64_CMP"
#elif defined(OPTLDS64)
#define OCB_VARIANT ocb::kOptLds64
#define OCB_VARIANT_NAME "OPTLDS64"
#else
#define OCB_VARIANT ocb::kOptSts64
#define OCB_VARIANT_NAME "OPTSTS64"
#endif

namespace {

__device__ int g_status = 0;

constexpr int kMaxDevices = 64;

struct DeviceState {
  std::once_flag once;
  cudaError_t init_error = cudaSuccess;
  int sm_count = 0;
  int max_clusters[2] = {0, 0};   // co-resident CTA pairs of wino_tc2_kernel<BF16 / TF32>
  int *status_ptr = nullptr;
};
DeviceState g_dev[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
  std::call_once(g_encode_once, [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  return g_encode;
}

// Per-device set-up: SM count, the opt-in to large dynamic shared memory, the address of the
// status word.  Runs once per device, with that device current.
cudaError_t device_state(DeviceState **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  DeviceState &st = g_dev[dev];
  std::call_once(st.once, [&] {
    cudaError_t err = cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_fp32_kernel<OCB_VARIANT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::SmemLayout<OCB_VARIANT>::kBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_fp32_kernel<OCB_VARIANT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::SmemLayout<OCB_VARIANT>::kBytes);
    if (err == cudaSuccess) {
      // The kernel redistributes registers with setmaxnreg; that only works if the compiler gave
      // the CTA at least the pool the budgets add up to.  Refuse to run a build where it did not
      // (its consumer warps would wait for registers for ever).
      constexpr int kBudget = ocb::kConsumerThreads * ocb::kConsumerRegs + ocb::kProducerThreads * ocb::kProducerRegs;
      cudaFuncAttributes fa;
      err = cudaFuncGetAttributes(&fa, ocb::wino_fp32_kernel<OCB_VARIANT, false>);
      if (err == cudaSuccess && fa.numRegs * ocb::kThreads < kBudget) err = cudaErrorLaunchOutOfResources;
      if (err == cudaSuccess) err = cudaFuncGetAttributes(&fa, ocb::wino_fp32_kernel<OCB_VARIANT, true>);
      if (err == cudaSuccess && fa.numRegs * ocb::kThreads < kBudget) err = cudaErrorLaunchOutOfResources;
    }
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc_kernel<ocb::kTcBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::TcCfg<ocb::kTcBf16>::kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc_kernel<ocb::kTcBf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::TcCfg<ocb::kTcBf16, true>::kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc_kernel<ocb::kTcTf32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::TcCfg<ocb::kTcTf32>::kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc2_kernel<ocb::kTcBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::P2Cfg<ocb::kTcBf16>::kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc2_kernel<ocb::kTcTf32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::P2Cfg<ocb::kTcTf32>::kSmemBytes);
    if (err == cudaSuccess) {
      // how many CTA pairs fit on the device at once (pairs must sit in one GPC)
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * (unsigned)st.sm_count);
      cfg.blockDim = dim3(ocb::kP2Threads);
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      cfg.dynamicSmemBytes = ocb::P2Cfg<ocb::kTcBf16>::kSmemBytes;
      err = cudaOccupancyMaxActiveClusters(&st.max_clusters[0], ocb::wino_tc2_kernel<ocb::kTcBf16>, &cfg);
      if (err == cudaSuccess) {
        cfg.dynamicSmemBytes = ocb::P2Cfg<ocb::kTcTf32>::kSmemBytes;
        err = cudaOccupancyMaxActiveClusters(&st.max_clusters[1], ocb::wino_tc2_kernel<ocb::kTcTf32>, &cfg);
      }
    }
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc64_kernel<ocb::kTcBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::T64Cfg<ocb::kTcBf16>::kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(ocb::wino_tc64_kernel<ocb::kTcTf32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ocb::T64Cfg<ocb::kTcTf32>::kSmemBytes);
    if (err == cudaSuccess) err = cudaGetSymbolAddress(reinterpret_cast<void **>(&st.status_ptr), g_status);
    st.init_error = err;
  });
  *out = &st;
  return st.init_error;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// What the output pointer must be aligned to: the tensor-core kernels store 32 bytes per lane
// (st.global.v8.f32), the fp32 kernel at most 8.
bool output_aligned(const void *p, int precision) {
  return (reinterpret_cast<uintptr_t>(p) & (precision == OPENCNN_FP32 ? 15u : 31u)) == 0;
}

// What the batch and the channel count must be multiples of.  The two legacy entry points keep
// the reference's rules (N % 32, C % 8).  The other entries accept a ragged last block of images
// - N % 4 on the fp32 path (rows of the tensors must stay 16-byte aligned for TMA), N % 8 on the
// tensor-core path (its epilogue stores eight images per lane) - and any channel count; on the
// fp32 path also a ragged last block of filters (K % 4; the tensor-core path views the
// transformed filter in rows of 64 filters and keeps K % 64).  Images, channels and filters
// beyond the end are zero-filled by TMA, which leaves every fma chain unchanged
// (fma(0, 0, acc) == acc for the accumulators that occur, which are never -0), and outputs of
// missing images and filters are not stored.
struct ShapeRule { int n_multiple, c_multiple, k_multiple; };
constexpr ShapeRule kLegacyRule = {32, 8, 64};
ShapeRule shape_rule(int precision) {
  return precision == OPENCNN_FP32 ? ShapeRule{4, 1, 4} : ShapeRule{8, 1, 64};
}

cudaError_t check_shape(int N, int C, int H, int W, int K, ShapeRule rule) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || K <= 0) return cudaErrorInvalidValue;
  if (N % rule.n_multiple || K % rule.k_multiple || C % rule.c_multiple) return cudaErrorInvalidValue;
  // 32-bit tile arithmetic and TMA extents
  if ((long long)N * C * H * W >= (1ll << 40) || (long long)N * K * H * W >= (1ll << 40)) return cudaErrorInvalidValue;
  return cudaSuccess;
}

cudaError_t launch_fx(const float *filter, float *workspace, int C, int K, cudaStream_t stream) {
  const int k4 = K / 4;
  const int total = C * k4;
  ocb::fx_kernel<<<(total + 127) / 128, 128, 0, stream>>>(reinterpret_cast<const float4 *>(filter),
                                                        reinterpret_cast<float4 *>(workspace), C, k4);
  return cudaGetLastError();
}

cudaError_t launch_wino_fp32(const float *input, const float *workspace, float *output, int N, int C, int H,
                             int W, int K, cudaStream_t stream) {
  DeviceState *st = nullptr;
  cudaError_t e = device_state(&st);
  if (e != cudaSuccess) return e;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;

  CUtensorMap tm_in, tm_u;
  {
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C};
    cuuint64_t strides[3] = {(cuuint64_t)N * 4, (cuuint64_t)W * N * 4, (cuuint64_t)H * W * N * 4};
    cuuint32_t box[4] = {(cuuint32_t)ocb::kBN, 4, 4, (cuuint32_t)ocb::kBC};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(input), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)K, 16, (cuuint64_t)C};
    cuuint64_t strides[2] = {(cuuint64_t)K * 4, (cuuint64_t)K * 16 * 4};
    cuuint32_t box[3] = {(cuuint32_t)ocb::kBK, 16, (cuuint32_t)ocb::kBC};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&tm_u, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(workspace), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }

  ocb::WinoParams p;
  p.y = output;
  p.N = N; p.C = C; p.K = K; p.H = H; p.W = W;
  p.tiles_h = (H + 1) / 2;
  p.tiles_w = (W + 1) / 2;
  p.n_blocks = (N + ocb::kBN - 1) / ocb::kBN;
  p.k_blocks = (K + ocb::kBK - 1) / ocb::kBK;
  const long long tiles = (long long)p.tiles_h * p.tiles_w * p.n_blocks * p.k_blocks;
  if (tiles > 0x7fffffffll / 8) return cudaErrorInvalidValue;
  p.total_tiles = (int)tiles;
  p.chunks_per_tile = (C + ocb::kBC - 1) / ocb::kBC;
  p.status = st->status_ptr;
  const int grid = p.total_tiles < st->sm_count ? p.total_tiles : st->sm_count;
  // The last round of the persistent schedule is usually only partly filled.  If its tiles, cut in
  // two (one item per consumer group), still fit on the SMs, cut them: that round then takes about
  // half as long (see item_tile in wino_fp32.cuh).
  const int full_rounds = p.total_tiles / grid, rest = p.total_tiles % grid;
  p.split_from = p.total_tiles;
  p.total_items = p.total_tiles;
  if (rest > 0 && 2 * rest <= grid) {
    p.split_from = full_rounds * grid;
    p.total_items = p.split_from + 2 * rest;
  }
  if (N % ocb::kBN == 0 && K % ocb::kBK == 0)
    ocb::wino_fp32_kernel<OCB_VARIANT, false><<<grid, ocb::kThreads, ocb::SmemLayout<OCB_VARIANT>::kBytes, stream>>>(tm_in, tm_u, p);
  else   // ragged last block of images or filters: stores masked
    ocb::wino_fp32_kernel<OCB_VARIANT, true><<<grid, ocb::kThreads, ocb::SmemLayout<OCB_VARIANT>::kBytes, stream>>>(tm_in, tm_u, p);
  return cudaGetLastError();
}

// Tensor-core path: filter transform rounded to the operand type, then the tcgen05 kernel.
template <int DT>
cudaError_t launch_fx_tc(const float *filter, float *workspace, int C, int K, cudaStream_t stream) {
  const int k4 = K / 4;
  const int total = C * k4;
  ocb::fx_tc_kernel<DT><<<(total + 127) / 128, 128, 0, stream>>>(reinterpret_cast<const float4 *>(filter), workspace, C, k4);
  return cudaGetLastError();
}

template <int DT>
cudaError_t launch_wino_tc(const float *input, const float *workspace, float *output, int N, int C, int H, int W,
                           int K, cudaStream_t stream) {
  DeviceState *st = nullptr;
  cudaError_t e = device_state(&st);
  if (e != cudaSuccess) return e;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  constexpr int KC = ocb::TcCfg<DT>::kKC;
  constexpr bool bf16 = DT == ocb::kTcBf16;
  constexpr cuuint64_t esz = bf16 ? 2 : 4;
  constexpr cuuint32_t row_elems = bf16 ? 64 : 32;            // filters in one 128-byte row

  CUtensorMap tm_in, tm_u;
  {
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C};
    cuuint64_t strides[3] = {(cuuint64_t)N * 4, (cuuint64_t)W * N * 4, (cuuint64_t)H * W * N * 4};
    cuuint32_t box[4] = {(cuuint32_t)ocb::kTcN, 4, 4, (cuuint32_t)KC};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(input), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  {
    // workspace [C][16][K] viewed as {filter within a 128-byte row, channel, 128-byte row, position}
    cuuint64_t dims[4] = {row_elems, (cuuint64_t)C, (cuuint64_t)K / row_elems, 16};
    cuuint64_t strides[3] = {(cuuint64_t)16 * K * esz, 128, (cuuint64_t)K * esz};
    // BF16 with at most 64 filters: only the first 64-filter row block is loaded (wino_tc.cuh, "half U")
    const bool half_u = bf16 && K <= 64;
    cuuint32_t box[4] = {row_elems, (cuuint32_t)KC, half_u ? 1u : (cuuint32_t)(ocb::kTcM / row_elems), 16};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_u, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
            const_cast<float *>(workspace), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            bf16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  ocb::WinoParams p;
  p.y = output;
  p.N = N; p.C = C; p.K = K; p.H = H; p.W = W;
  p.tiles_h = (H + 1) / 2;
  p.tiles_w = (W + 1) / 2;
  p.n_blocks = (N + ocb::kTcN - 1) / ocb::kTcN;
  p.k_blocks = (K + ocb::kTcM - 1) / ocb::kTcM;
  const long long tiles = (long long)p.tiles_h * p.tiles_w * p.n_blocks * p.k_blocks;
  if (tiles > 0x7fffffffll / 8) return cudaErrorInvalidValue;
  p.total_tiles = (int)tiles;
  p.split_from = p.total_items = p.total_tiles;
  p.chunks_per_tile = (C + KC - 1) / KC;
  p.status = st->status_ptr;
  const int grid = p.total_tiles < st->sm_count ? p.total_tiles : st->sm_count;
  if (bf16 && K <= 64)
    ocb::wino_tc_kernel<ocb::kTcBf16, true><<<grid, ocb::TcCfg<ocb::kTcBf16, true>::kThreads,
                                              ocb::TcCfg<ocb::kTcBf16, true>::kSmemBytes, stream>>>(tm_in, tm_u, p);
  else
    ocb::wino_tc_kernel<DT><<<grid, ocb::TcCfg<DT>::kThreads, ocb::TcCfg<DT>::kSmemBytes, stream>>>(tm_in, tm_u, p);
  return cudaGetLastError();
}

// Pair kernel: clusters of two CTAs share a tile of 128 filters x 64 images (wino_tc2.cuh).
template <int DT>
cudaError_t launch_wino_tc2(const float *input, const float *workspace, float *output, int N, int C, int H, int W,
                            int K, cudaStream_t stream) {
  DeviceState *st = nullptr;
  cudaError_t e = device_state(&st);
  if (e != cudaSuccess) return e;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  constexpr int KC = ocb::P2Cfg<DT>::kKC;
  constexpr bool bf16 = DT == ocb::kTcBf16;
  constexpr cuuint64_t esz = bf16 ? 2 : 4;
  constexpr cuuint32_t row_elems = bf16 ? 64 : 32;
  const int max_clusters = st->max_clusters[bf16 ? 0 : 1];
  if (max_clusters <= 0) return cudaErrorNotSupported;

  CUtensorMap tm_in, tm_u;
  {
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C};
    cuuint64_t strides[3] = {(cuuint64_t)N * 4, (cuuint64_t)W * N * 4, (cuuint64_t)H * W * N * 4};
    cuuint32_t box[4] = {(cuuint32_t)ocb::kP2N, 4, 3, (cuuint32_t)KC};   // three patch rows per CTA
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(input), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  {
    cuuint64_t dims[4] = {row_elems, (cuuint64_t)C, (cuuint64_t)K / row_elems, 16};
    cuuint64_t strides[3] = {(cuuint64_t)16 * K * esz, 128, (cuuint64_t)K * esz};
    cuuint32_t box[4] = {row_elems, (cuuint32_t)KC, (cuuint32_t)(ocb::kTcM / row_elems), 8};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_u, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
            const_cast<float *>(workspace), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            bf16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  ocb::WinoParams p;
  p.y = output;
  p.N = N; p.C = C; p.K = K; p.H = H; p.W = W;
  p.tiles_h = (H + 1) / 2;
  p.tiles_w = (W + 1) / 2;
  p.n_blocks = (N + ocb::kTcN - 1) / ocb::kTcN;
  p.k_blocks = (K + ocb::kTcM - 1) / ocb::kTcM;
  const long long tiles = (long long)p.tiles_h * p.tiles_w * ((p.n_blocks + 1) / 2) * p.k_blocks;
  if (tiles > 0x7fffffffll / 8) return cudaErrorInvalidValue;
  p.total_tiles = (int)tiles;
  p.split_from = p.total_items = p.total_tiles;
  p.chunks_per_tile = (C + KC - 1) / KC;
  p.status = st->status_ptr;
  const int clusters = p.total_tiles < max_clusters ? p.total_tiles : max_clusters;
  ocb::wino_tc2_kernel<DT><<<2 * clusters, ocb::kP2Threads, ocb::P2Cfg<DT>::kSmemBytes, stream>>>(tm_in, tm_u, p);
  return cudaGetLastError();
}

// Layers with at most 64 filters: two 32-image blocks share the 128 accumulator rows (wino_tc64.cuh).
template <int DT>
cudaError_t launch_wino_tc64(const float *input, const float *workspace, float *output, int N, int C, int H, int W,
                             int K, cudaStream_t stream) {
  if (K > 64) return cudaErrorInvalidValue;
  DeviceState *st = nullptr;
  cudaError_t e = device_state(&st);
  if (e != cudaSuccess) return e;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  constexpr int KC = ocb::T64Cfg<DT>::kKC;
  constexpr bool bf16 = DT == ocb::kTcBf16;
  CUtensorMap tm_in, tm_u;
  {
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C};
    cuuint64_t strides[3] = {(cuuint64_t)N * 4, (cuuint64_t)W * N * 4, (cuuint64_t)H * W * N * 4};
    cuuint32_t box[4] = {(cuuint32_t)ocb::kTcN, 4, 4, (cuuint32_t)KC};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(input), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  {
    // workspace [C][16][K] viewed as {filter within a 128-byte row, channel, 128-byte row, position}.
    // BF16: one row block of 64 filters.  TF32: a box of four row blocks of 32 filters, of which two exist -
    // the hardware fills the other two with zeros, which the kernel uses as the empty half of its A operand.
    constexpr cuuint64_t esz = bf16 ? 2 : 4;
    constexpr cuuint32_t row_elems = bf16 ? 64 : 32;
    cuuint64_t dims[4] = {row_elems, (cuuint64_t)C, (cuuint64_t)K / row_elems, 16};
    cuuint64_t strides[3] = {(cuuint64_t)16 * K * esz, 128, (cuuint64_t)K * esz};
    cuuint32_t box[4] = {row_elems, (cuuint32_t)KC, bf16 ? 1u : 4u, 16};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_u, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
            const_cast<float *>(workspace), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            bf16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  ocb::WinoParams p;
  p.y = output;
  p.N = N; p.C = C; p.K = K; p.H = H; p.W = W;
  p.tiles_h = (H + 1) / 2;
  p.tiles_w = (W + 1) / 2;
  p.n_blocks = (N + ocb::kTcN - 1) / ocb::kTcN;
  p.k_blocks = 1;
  const long long tiles = (long long)p.tiles_h * p.tiles_w * ((p.n_blocks + 1) / 2);
  if (tiles > 0x7fffffffll / 8) return cudaErrorInvalidValue;
  p.total_tiles = (int)tiles;
  p.split_from = p.total_items = p.total_tiles;
  p.chunks_per_tile = (C + KC - 1) / KC;
  p.status = st->status_ptr;
  const int grid = p.total_tiles < st->sm_count ? p.total_tiles : st->sm_count;
  ocb::wino_tc64_kernel<DT><<<grid, ocb::kT64Threads, ocb::T64Cfg<DT>::kSmemBytes, stream>>>(tm_in, tm_u, p);
  return cudaGetLastError();
}

// Which tensor-core kernel a problem gets.  Both compute the same thing.  The CTA-pair kernel
// (wino_tc2.cuh) has the cheaper main loop (half as many, twice as wide MMAs) but a dearer
// epilogue (two CTAs meet through L2), so it wins where a tile has many K-steps and the MMAs are
// many: in TF32 from 64 K-steps per tile (C >= 512: 6-20 % ahead).  In BF16 the single-CTA kernel
// is level or ahead everywhere since it issues its MMAs from two threads (C = 1024: within 1 %),
// so BF16 never takes the pair.
template <int DT>
cudaError_t launch_tc(const float *input, const float *workspace, float *output, int N, int C, int H, int W, int K,
                      cudaStream_t stream, int kernel = OPENCNN_TC_AUTO) {
  if (kernel == OPENCNN_TC_SINGLE_CTA) return launch_wino_tc<DT>(input, workspace, output, N, C, H, W, K, stream);
  if (kernel == OPENCNN_TC_PAIR_LOCAL) return launch_wino_tc2<DT>(input, workspace, output, N, C, H, W, K, stream);
  if (kernel == OPENCNN_TC_STACKED_BLOCKS) return launch_wino_tc64<DT>(input, workspace, output, N, C, H, W, K, stream);
  if (kernel != OPENCNN_TC_AUTO) return cudaErrorInvalidValue;
  // at most 64 filters and more than one 32-image block: two blocks share the accumulator rows
  if (K <= 64 && N > ocb::kTcN) return launch_wino_tc64<DT>(input, workspace, output, N, C, H, W, K, stream);
  const int k_steps = (C + ocb::TcCfg<DT>::kKC - 1) / ocb::TcCfg<DT>::kKC;
  const bool pair = DT == ocb::kTcTf32 && k_steps >= 64 && N >= 64;
  return pair ? launch_wino_tc2<DT>(input, workspace, output, N, C, H, W, K, stream)
              : launch_wino_tc<DT>(input, workspace, output, N, C, H, W, K, stream);
}

cudaError_t forward(const float *input, const float *filter, float *output, float *workspace, int N, int C, int H,
                    int W, int K, int precision, cudaStream_t stream, ShapeRule rule) {
  if (!input || !filter || !output || !workspace) return cudaErrorInvalidValue;
  if (!aligned16(input) || !aligned16(filter) || !aligned16(output) || !aligned16(workspace)) return cudaErrorInvalidValue;
  if (precision != OPENCNN_FP32 && precision != OPENCNN_TF32 && precision != OPENCNN_BF16) return cudaErrorInvalidValue;
  if (!output_aligned(output, precision)) return cudaErrorInvalidValue;
  cudaError_t e = check_shape(N, C, H, W, K, rule);
  if (e != cudaSuccess) return e;
  if (precision == OPENCNN_BF16) {
    e = launch_fx_tc<ocb::kTcBf16>(filter, workspace, C, K, stream);
    if (e != cudaSuccess) return e;
    return launch_tc<ocb::kTcBf16>(input, workspace, output, N, C, H, W, K, stream);
  }
  if (precision == OPENCNN_TF32) {
    e = launch_fx_tc<ocb::kTcTf32>(filter, workspace, C, K, stream);
    if (e != cudaSuccess) return e;
    return launch_tc<ocb::kTcTf32>(input, workspace, output, N, C, H, W, K, stream);
  }
  if (precision != OPENCNN_FP32) return cudaErrorInvalidValue;
  e = launch_fx(filter, workspace, C, K, stream);
  if (e != cudaSuccess) return e;
  return launch_wino_fp32(input, workspace, output, N, C, H, W, K, stream);
}

// Scratch for opencnn_convolutionForward_noalloc: the transformed filter, [C][16][K] floats, for
// problems up to OPENCNN_NOALLOC_MAX_CK channel-filter pairs.  In host code this name is only a
// handle for the runtime, not a device address; the address is looked up once per device below.
static __device__ __align__(256) float g_noalloc_workspace[(size_t)OPENCNN_NOALLOC_MAX_CK * 16];

struct NoAllocState {
  std::once_flag once;
  cudaError_t error = cudaSuccess;
  float *workspace = nullptr;     // device address of g_noalloc_workspace on this device
};
NoAllocState g_noalloc[kMaxDevices];

// Device address of the static workspace on the current device (looked up on first use).
cudaError_t noalloc_workspace(float **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  NoAllocState &st = g_noalloc[dev];
  std::call_once(st.once, [&] {
    void *p = nullptr;
    st.error = cudaGetSymbolAddress(&p, g_noalloc_workspace);
    if (st.error == cudaSuccess) st.workspace = static_cast<float *>(p);
  });
  *out = st.workspace;
  return st.error;
}

struct HostPlan {
  int N, C, H, W, K, precision;
  float *d_in = nullptr, *d_filt = nullptr, *d_out = nullptr, *d_ws = nullptr;
  cudaStream_t stream = nullptr;
};

}  // namespace

extern "C" {

int convolutionForward_32x64x8(float *k, int in_h, int in_w, float *w, int out_h, int out_w, int out_n,
                               int out_c, float *C, float *Ww, const unsigned int n, int tiles_dim, int in_n,
                               int tile_size, int in_c, int filt_k, int filt_c, int filt_h, int filt_w,
                               int alpha, int m) {
  (void)n;
  if (filt_h != 3 || filt_w != 3 || m != 2 || tile_size != 4 || alpha != 4) return (int)cudaErrorInvalidValue;
  if (filt_c != in_c || out_c != filt_k || out_n != in_n || out_h != in_h || out_w != in_w)
    return (int)cudaErrorInvalidValue;
  if (tiles_dim != (in_w + 1) / 2) return (int)cudaErrorInvalidValue;
  return (int)forward(k, w, C, Ww, in_n, in_c, in_h, in_w, filt_k, OPENCNN_FP32, (cudaStream_t)0, kLegacyRule);
}

int convolutionForward(float *k, int in_h, int in_w, float *w, int out_h, int out_w, int out_n, int out_c,
                       float *C, float *Ww, const unsigned int n, int tiles_dim, int in_n, int tile_size,
                       int elems_dim, int in_c, int filt_k, int filt_c, int filt_h, int filt_w, int alpha,
                       int m) {
  (void)elems_dim;
  return convolutionForward_32x64x8(k, in_h, in_w, w, out_h, out_w, out_n, out_c, C, Ww, n, tiles_dim, in_n,
                                    tile_size, in_c, filt_k, filt_c, filt_h, filt_w, alpha, m);
}

int opencnn_convolutionForward_stream(const float *input, const float *filter, float *output, float *workspace,
                                      int in_n, int in_c, int in_h, int in_w, int filt_k, int precision,
                                      opencnn_stream_t stream) {
  return (int)forward(input, filter, output, workspace, in_n, in_c, in_h, in_w, filt_k, precision,
                      (cudaStream_t)stream, shape_rule(precision));
}

int opencnn_filter_transform(const float *filter, float *workspace, int in_c, int filt_k, opencnn_stream_t stream) {
  return opencnn_filter_transform_p(filter, workspace, in_c, filt_k, OPENCNN_FP32, stream);
}

int opencnn_filter_transform_p(const float *filter, float *workspace, int in_c, int filt_k, int precision,
                               opencnn_stream_t stream) {
  if (!filter || !workspace || !aligned16(filter) || !aligned16(workspace)) return (int)cudaErrorInvalidValue;
  if (in_c <= 0 || filt_k <= 0 || filt_k % 4) return (int)cudaErrorInvalidValue;
  if (precision == OPENCNN_BF16) return (int)launch_fx_tc<ocb::kTcBf16>(filter, workspace, in_c, filt_k, (cudaStream_t)stream);
  if (precision == OPENCNN_TF32) return (int)launch_fx_tc<ocb::kTcTf32>(filter, workspace, in_c, filt_k, (cudaStream_t)stream);
  if (precision != OPENCNN_FP32) return (int)cudaErrorInvalidValue;
  return (int)launch_fx(filter, workspace, in_c, filt_k, (cudaStream_t)stream);
}

int opencnn_winograd_forward(const float *input, const float *workspace, float *output, int in_n, int in_c,
                             int in_h, int in_w, int filt_k, int precision, opencnn_stream_t stream) {
  if (!input || !workspace || !output) return (int)cudaErrorInvalidValue;
  if (!aligned16(input) || !aligned16(workspace) || !aligned16(output)) return (int)cudaErrorInvalidValue;
  if (precision != OPENCNN_FP32 && precision != OPENCNN_TF32 && precision != OPENCNN_BF16) return (int)cudaErrorInvalidValue;
  if (!output_aligned(output, precision)) return (int)cudaErrorInvalidValue;
  cudaError_t e = check_shape(in_n, in_c, in_h, in_w, filt_k, shape_rule(precision));
  if (e != cudaSuccess) return (int)e;
  if (precision == OPENCNN_BF16)
    return (int)launch_tc<ocb::kTcBf16>(input, workspace, output, in_n, in_c, in_h, in_w, filt_k, (cudaStream_t)stream);
  if (precision == OPENCNN_TF32)
    return (int)launch_tc<ocb::kTcTf32>(input, workspace, output, in_n, in_c, in_h, in_w, filt_k, (cudaStream_t)stream);
  if (precision != OPENCNN_FP32) return (int)cudaErrorInvalidValue;
  return (int)launch_wino_fp32(input, workspace, output, in_n, in_c, in_h, in_w, filt_k, (cudaStream_t)stream);
}

int opencnn_winograd_forward_kernel(const float *input, const float *workspace, float *output, int in_n, int in_c,
                                    int in_h, int in_w, int filt_k, int precision, int kernel, opencnn_stream_t stream) {
  if (!input || !workspace || !output) return (int)cudaErrorInvalidValue;
  if (!aligned16(input) || !aligned16(workspace) || !aligned16(output)) return (int)cudaErrorInvalidValue;
  if (precision != OPENCNN_TF32 && precision != OPENCNN_BF16) return (int)cudaErrorInvalidValue;
  if (!output_aligned(output, precision)) return (int)cudaErrorInvalidValue;
  cudaError_t e = check_shape(in_n, in_c, in_h, in_w, filt_k, shape_rule(precision));
  if (e != cudaSuccess) return (int)e;
  if (precision == OPENCNN_BF16)
    return (int)launch_tc<ocb::kTcBf16>(input, workspace, output, in_n, in_c, in_h, in_w, filt_k, (cudaStream_t)stream, kernel);
  return (int)launch_tc<ocb::kTcTf32>(input, workspace, output, in_n, in_c, in_h, in_w, filt_k, (cudaStream_t)stream, kernel);
}

int opencnn_convolutionForward_noalloc(const float *input, const float *filter, float *output, int in_n,
                                       int in_c, int in_h, int in_w, int filt_k, opencnn_stream_t stream) {
  if (!input || !filter || !output) return (int)cudaErrorInvalidValue;
  if (!aligned16(input) || !aligned16(filter) || !aligned16(output)) return (int)cudaErrorInvalidValue;
  cudaError_t e = check_shape(in_n, in_c, in_h, in_w, filt_k, shape_rule(OPENCNN_FP32));
  if (e != cudaSuccess) return (int)e;
  if ((long long)in_c * filt_k > (long long)OPENCNN_NOALLOC_MAX_CK) {
    std::fprintf(stderr,
                 "opencnn_convolutionForward_noalloc: in_c*filt_k = %lld exceeds the built-in workspace "
                 "(OPENCNN_NOALLOC_MAX_CK = %d); use opencnn_convolutionForward_stream with your own workspace\n",
                 (long long)in_c * filt_k, OPENCNN_NOALLOC_MAX_CK);
    return (int)cudaErrorInvalidValue;
  }
  float *ws = nullptr;
  e = noalloc_workspace(&ws);
  if (e != cudaSuccess) return (int)e;
  e = launch_fx(filter, ws, in_c, filt_k, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)launch_wino_fp32(input, ws, output, in_n, in_c, in_h, in_w, filt_k, (cudaStream_t)stream);
}

int opencnn_nchw_to_chwn(const float *src, float *dst, int n, int c, int h, int w, opencnn_stream_t stream) {
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0) return (int)cudaErrorInvalidValue;
  return (int)ocb::launch_transpose(src, dst, n, (long long)c * h * w, (cudaStream_t)stream);
}

int opencnn_kcrs_to_crsk(const float *src, float *dst, int k, int c, opencnn_stream_t stream) {
  if (k <= 0 || c <= 0) return (int)cudaErrorInvalidValue;
  return (int)ocb::launch_transpose(src, dst, k, (long long)c * 9, (cudaStream_t)stream);
}

int opencnn_khwn_to_nkhw(const float *src, float *dst, int n, int k, int h, int w, opencnn_stream_t stream) {
  if (n <= 0 || k <= 0 || h <= 0 || w <= 0) return (int)cudaErrorInvalidValue;
  return (int)ocb::launch_transpose(src, dst, (long long)k * h * w, n, (cudaStream_t)stream);
}

size_t opencnn_workspace_bytes(int in_c, int filt_k) {
  if (in_c <= 0 || filt_k <= 0) return 0;
  return (size_t)in_c * 16 * (size_t)filt_k * sizeof(float);
}

const char *opencnn_variant_name(void) { return OCB_VARIANT_NAME; }

int opencnn_last_device_status(void) {
  int v = -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
  int zero = 0;
  cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  return v;
}

int opencnn_host_plan_create(void **plan, int in_n, int in_c, int in_h, int in_w, int filt_k, int precision) {
  if (!plan) return (int)cudaErrorInvalidValue;
  *plan = nullptr;
  if (precision != OPENCNN_FP32 && precision != OPENCNN_TF32 && precision != OPENCNN_BF16) return (int)cudaErrorInvalidValue;
  cudaError_t e = check_shape(in_n, in_c, in_h, in_w, filt_k, shape_rule(precision));
  if (e != cudaSuccess) return (int)e;
  HostPlan *hp = new (std::nothrow) HostPlan;
  if (!hp) return (int)cudaErrorMemoryAllocation;
  hp->N = in_n; hp->C = in_c; hp->H = in_h; hp->W = in_w; hp->K = filt_k; hp->precision = precision;
  const size_t in_b = (size_t)in_n * in_c * in_h * in_w * 4, f_b = (size_t)in_c * 9 * filt_k * 4;
  const size_t out_b = (size_t)in_n * filt_k * in_h * in_w * 4;
  e = cudaMalloc(&hp->d_in, in_b);
  if (e == cudaSuccess) e = cudaMalloc(&hp->d_filt, f_b);
  if (e == cudaSuccess) e = cudaMalloc(&hp->d_out, out_b);
  if (e == cudaSuccess) e = cudaMalloc(&hp->d_ws, opencnn_workspace_bytes(in_c, filt_k));
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&hp->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    opencnn_host_plan_destroy(hp);
    return (int)e;
  }
  *plan = hp;
  return 0;
}

int opencnn_host_plan_run_async(void *plan, const float *input_host, const float *filter_host,
                                float *output_host) {
  HostPlan *hp = static_cast<HostPlan *>(plan);
  if (!hp || !input_host || !filter_host || !output_host) return (int)cudaErrorInvalidValue;
  const size_t in_b = (size_t)hp->N * hp->C * hp->H * hp->W * 4, f_b = (size_t)hp->C * 9 * hp->K * 4;
  const size_t out_b = (size_t)hp->N * hp->K * hp->H * hp->W * 4;
  cudaError_t e = cudaMemcpyAsync(hp->d_filt, filter_host, f_b, cudaMemcpyHostToDevice, hp->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(hp->d_in, input_host, in_b, cudaMemcpyHostToDevice, hp->stream);
  if (e == cudaSuccess)
    e = forward(hp->d_in, hp->d_filt, hp->d_out, hp->d_ws, hp->N, hp->C, hp->H, hp->W, hp->K, hp->precision, hp->stream,
                shape_rule(hp->precision));
  if (e == cudaSuccess) e = cudaMemcpyAsync(output_host, hp->d_out, out_b, cudaMemcpyDeviceToHost, hp->stream);
  return (int)e;
}

int opencnn_host_plan_copy_async(void *plan, const float *input_host, const float *filter_host, float *output_host) {
  HostPlan *hp = static_cast<HostPlan *>(plan);
  if (!hp || !input_host || !filter_host || !output_host) return (int)cudaErrorInvalidValue;
  const size_t in_b = (size_t)hp->N * hp->C * hp->H * hp->W * 4, f_b = (size_t)hp->C * 9 * hp->K * 4;
  const size_t out_b = (size_t)hp->N * hp->K * hp->H * hp->W * 4;
  cudaError_t e = cudaMemcpyAsync(hp->d_filt, filter_host, f_b, cudaMemcpyHostToDevice, hp->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(hp->d_in, input_host, in_b, cudaMemcpyHostToDevice, hp->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(output_host, hp->d_out, out_b, cudaMemcpyDeviceToHost, hp->stream);
  return (int)e;
}

int opencnn_host_plan_wait(void *plan) {
  HostPlan *hp = static_cast<HostPlan *>(plan);
  if (!hp) return (int)cudaErrorInvalidValue;
  return (int)cudaStreamSynchronize(hp->stream);
}

int opencnn_host_plan_run(void *plan, const float *input_host, const float *filter_host, float *output_host) {
  int e = opencnn_host_plan_run_async(plan, input_host, filter_host, output_host);
  return e != 0 ? e : opencnn_host_plan_wait(plan);
}

int opencnn_host_plan_destroy(void *plan) {
  HostPlan *hp = static_cast<HostPlan *>(plan);
  if (!hp) return 0;
  if (hp->d_in) cudaFree(hp->d_in);
  if (hp->d_filt) cudaFree(hp->d_filt);
  if (hp->d_out) cudaFree(hp->d_out);
  if (hp->d_ws) cudaFree(hp->d_ws);
  if (hp->stream) cudaStreamDestroy(hp->stream);
  delete hp;
  return 0;
}

}  // extern "C"
