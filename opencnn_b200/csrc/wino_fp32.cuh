// Fused Winograd F(2x2,3x3) forward kernel, fp32 FFMA path, for sm_100a.
//
// Replaces the reference's Winograd_kernel (src/convolutionForward_32x64x8.cu:169-262 and its
// ampere/ and _baseline copies) together with its device building blocks: prefetch_input_tile /
// prefetch_filter_tile (:102-147), load_and_transform_input_tile / load_filter_tile (:53-100),
// the fragment loads (:149-167), outer_product (src/outer_product*.cuh) and the four
// store_output_tile / transform_output_tile variants (src/store_and_transform_output_*.cuh).
//
// What one CTA computes is what one reference CTA computes - 32 images x one 2x2-output tile x
// 64 filters, all 16 Winograd positions, reduced over C in chunks of 8 - because that is what
// fills the register file (32768 accumulators).  Everything around it is different:
//   * persistent CTAs (one per SM) walk a list of tiles; loads run ahead across tile boundaries;
//   * the 4x4 input patch (with its halo) and the 64-filter slice of the transformed filter
//     arrive by TMA into a 3-stage shared-memory ring; out-of-range coordinates are zero-filled
//     by the hardware, which replaces the reference's halo masks and predicated loads;
//   * the input transform runs in place in shared memory, one thread per (image, channel);
//   * a warp owns two Winograd positions, one per half-warp; a lane owns 16 images x 8 filters
//     of one position as 64 packed register pairs and issues fma.rn.f32x2 (two FMAs per issue
//     slot); per channel it needs 4+2 128-bit shared loads, all bank-conflict free;
//   * the output is transposed through a dedicated staging buffer in four rounds of 16 filters
//     (variant-specific layout, see Staging below), transformed and stored with 128-byte rows.
//
// Every output is one fma chain over c = 0..C-1 starting from zero, and the transforms use
// the reference's operation order, so results are bit-identical to the reference kernels.
#pragma once
#include "ptx.cuh"

namespace ocb {

enum Variant : int { kBase = 0, kOptSts64 = 1, kOptSts64Cmp = 2, kOptLds64 = 3 };

constexpr int kBN = 32;                     // images per CTA tile
constexpr int kBK = 64;                     // filters per CTA tile
constexpr int kBC = 8;                      // channels per pipeline stage
constexpr int kStages = 3;
constexpr int kThreads = 256;
constexpr int kVStageFloats = 16 * kBC * kBN;   // [c][xi][n]   16 KiB
constexpr int kUStageFloats = 16 * kBC * kBK;   // [c][xi][k]   32 KiB
constexpr int kStageFloats = kVStageFloats + kUStageFloats;
constexpr uint32_t kStageBytes = kStageFloats * 4u;

// Staging buffer: rows are (xi, kl) with kl one of the 16 filters of a round, 32 images per row.
template <int V> struct Staging;
template <> struct Staging<kBase>       { static constexpr int kRowFloats = 36; static constexpr int kBuffers = 1; };
template <> struct Staging<kOptSts64>   { static constexpr int kRowFloats = 34; static constexpr int kBuffers = 1; };
template <> struct Staging<kOptSts64Cmp>{ static constexpr int kRowFloats = 32; static constexpr int kBuffers = 2; };
template <> struct Staging<kOptLds64>   { static constexpr int kRowFloats = 34; static constexpr int kBuffers = 1; };

template <int V> struct SmemLayout {
  static constexpr int kStagingFloats = 256 * Staging<V>::kRowFloats * Staging<V>::kBuffers;
  static constexpr size_t kBytes = (size_t)kStages * kStageBytes + (size_t)kStagingFloats * 4 + 64 /* mbarriers + dead flag */;
};

struct WinoParams {
  float *y;            // output, KHWN
  int N, C, K, H, W;
  int tiles_h, tiles_w, n_blocks, k_blocks, total_tiles, chunks_per_tile;
  int *status;         // device status word
};

struct TileCoord { int nb, tx, ty, kb; };

__device__ __forceinline__ TileCoord decode_tile(const WinoParams &p, int t) {
  TileCoord tc;
  tc.nb = t % p.n_blocks; t /= p.n_blocks;
  tc.tx = t % p.tiles_w;  t /= p.tiles_w;
  tc.ty = t % p.tiles_h;
  tc.kb = t / p.tiles_h;
  return tc;
}

// ---------------------------------------------------------------------------------------------
// Output transform Y = A^T M A for one (image, filter): rows first, then columns
// (operation order of src/store_and_transform_output_optSTS64.cuh:29-50).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void output_transform(const float (&m)[16], float (&y)[4]) {
  float a[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    a[j] = __fadd_rn(__fadd_rn(m[j], m[4 + j]), m[8 + j]);
    a[4 + j] = __fsub_rn(__fsub_rn(m[4 + j], m[8 + j]), m[12 + j]);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    y[2 * i + 0] = __fadd_rn(__fadd_rn(a[4 * i], a[4 * i + 1]), a[4 * i + 2]);
    y[2 * i + 1] = __fsub_rn(__fsub_rn(a[4 * i + 1], a[4 * i + 2]), a[4 * i + 3]);
  }
}

// Filter (within the CTA's 64) that staging row kl holds in round r.
__device__ __forceinline__ int round_filter(int kl, int r) {
  return 4 * (kl & 7) + 32 * (r >> 1) + 2 * (r & 1) + (kl >> 3);
}

// ---------------------------------------------------------------------------------------------
// Epilogue: transpose the accumulators through shared memory so that one thread holds all 16
// Winograd positions of an (image, filter), transform, store.  acc[kk][q]: kk = 4*j + e is the
// lane's filter 4*(kg + 8*j) + e, q = 2*i + ep is the image pair starting at
// 4*(4*ng + (i ^ h)) + 2*ep.
//
// Round r moves the lane's filters kk = 2r and 2r+1 (staging rows kl = kg and kg + 8).
//   BASE          deposit 8 x STS.128 (row pitch 36 floats), read back 32 x LDS.32, scalar stores
//   OPTSTS64      deposit 16 x STS.64 (row pitch 34 floats), read back 32 x LDS.32, scalar stores
//   OPTSTS64_CMP  as OPTSTS64 but unpadded rows rotated by (kl & 7) pairs, two buffers used
//                 alternately so that one barrier per round is enough
//   OPTLDS64      deposit as OPTSTS64, read back 16 x LDS.64, float2 stores
// ---------------------------------------------------------------------------------------------
template <int V>
__device__ __forceinline__ void epilogue(uint64_t (&acc)[8][8], float *stg, const WinoParams &p,
                                         const TileCoord &tc) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = lane >> 4, l = lane & 15, ng = l & 1, kg = l >> 1;
  const int xi = 2 * warp + h;
  constexpr int RF = Staging<V>::kRowFloats;

  const int oh0 = 2 * tc.ty, ow0 = 2 * tc.tx;
  const bool row1 = (oh0 + 1) < p.H, col1 = (ow0 + 1) < p.W;
  const size_t plane = (size_t)p.H * p.W * p.N;                       // one filter's output
  float *ybase = p.y + ((size_t)oh0 * p.W + ow0) * p.N + (size_t)tc.nb * kBN + (size_t)tc.kb * kBK * plane;
  const size_t dW = (size_t)p.N, dH = (size_t)p.W * p.N;

#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float *buf = stg + ((V == kOptSts64Cmp) ? (r & 1) * 256 * RF : 0);
    // ---- deposit ----
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int kl = kg + 8 * e;
      float *row = buf + (xi * 16 + kl) * RF;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int nq = 4 * ng + (i ^ h);                              // image quad of the row
        if (V == kBase) {
          *reinterpret_cast<ulonglong2 *>(row + 4 * nq) = make_ulonglong2(acc[2 * r + e][2 * i], acc[2 * r + e][2 * i + 1]);
        } else if (V == kOptSts64Cmp) {
          const int rot = kl & 7;
          *reinterpret_cast<uint64_t *>(row + 2 * ((2 * nq + 0 + rot) & 15)) = acc[2 * r + e][2 * i];
          *reinterpret_cast<uint64_t *>(row + 2 * ((2 * nq + 1 + rot) & 15)) = acc[2 * r + e][2 * i + 1];
        } else {
          *reinterpret_cast<uint64_t *>(row + 4 * nq) = acc[2 * r + e][2 * i];
          *reinterpret_cast<uint64_t *>(row + 4 * nq + 2) = acc[2 * r + e][2 * i + 1];
        }
      }
    }
    __syncthreads();
    // ---- read back, transform, store ----
    if (V == kOptLds64) {
      const int np = lane & 15, kl = 2 * warp + (lane >> 4);
      float m0[16], m1[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        const float2 v = *reinterpret_cast<const float2 *>(buf + (x * 16 + kl) * RF + 2 * np);
        m0[x] = v.x; m1[x] = v.y;
      }
      float y0[4], y1[4];
      output_transform(m0, y0);
      output_transform(m1, y1);
      float *dst = ybase + (size_t)round_filter(kl, r) * plane + 2 * np;
      *reinterpret_cast<float2 *>(dst) = make_float2(y0[0], y1[0]);
      if (col1) *reinterpret_cast<float2 *>(dst + dW) = make_float2(y0[1], y1[1]);
      if (row1) {
        *reinterpret_cast<float2 *>(dst + dH) = make_float2(y0[2], y1[2]);
        if (col1) *reinterpret_cast<float2 *>(dst + dH + dW) = make_float2(y0[3], y1[3]);
      }
    } else {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int kl = warp + 8 * half;
        float m[16];
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const float *row = buf + (x * 16 + kl) * RF;
          if (V == kOptSts64Cmp) m[x] = row[(lane + 2 * (kl & 7)) & 31];
          else                   m[x] = row[lane];
        }
        float yy[4];
        output_transform(m, yy);
        float *dst = ybase + (size_t)round_filter(kl, r) * plane + lane;
        dst[0] = yy[0];
        if (col1) dst[dW] = yy[1];
        if (row1) {
          dst[dH] = yy[2];
          if (col1) dst[dH + dW] = yy[3];
        }
      }
    }
    if (V != kOptSts64Cmp) __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// In-place input transform V = B^T d B of one (image, channel) patch inside a pipeline stage:
// columns first, then rows (operation order of src/convolutionForward_32x64x8.cu:59-80).
// The stage holds the raw patch as [c][h][w][n]; afterwards the same 16 slots hold [c][xi][n].
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void transform_patch(float *vstage) {
  float *R = vstage + ((threadIdx.x >> 5) * 16) * kBN + (threadIdx.x & 31);
  float d[16], b[16];
#pragma unroll
  for (int q = 0; q < 16; ++q) d[q] = R[q * kBN];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b[j] = __fsub_rn(d[j], d[8 + j]);
    b[4 + j] = __fadd_rn(d[4 + j], d[8 + j]);
    b[8 + j] = __fsub_rn(d[8 + j], d[4 + j]);
    b[12 + j] = __fsub_rn(d[4 + j], d[12 + j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    R[(4 * i + 0) * kBN] = __fsub_rn(b[4 * i + 0], b[4 * i + 2]);
    R[(4 * i + 1) * kBN] = __fadd_rn(b[4 * i + 1], b[4 * i + 2]);
    R[(4 * i + 2) * kBN] = __fsub_rn(b[4 * i + 2], b[4 * i + 1]);
    R[(4 * i + 3) * kBN] = __fsub_rn(b[4 * i + 1], b[4 * i + 3]);
  }
}

// One pipeline stage (8 channels) of the 16 batched GEMMs.
__device__ __forceinline__ void compute_stage(uint64_t (&acc)[8][8], const float *stage) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = lane >> 4, l = lane & 15, ng = l & 1, kg = l >> 1;
  const int xi = 2 * warp + h;
  const float *vrow = stage + xi * kBN + 16 * ng;
  const float *urow = stage + kVStageFloats + xi * kBK + 4 * kg;
#pragma unroll
  for (int c = 0; c < kBC; ++c) {
    ulonglong2 v[4];
    float4 u[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const ulonglong2 *>(vrow + c * 16 * kBN + 4 * (i ^ h));
#pragma unroll
    for (int j = 0; j < 2; ++j) u[j] = *reinterpret_cast<const float4 *>(urow + c * 16 * kBK + 32 * j);
    const float uu[8] = {u[0].x, u[0].y, u[0].z, u[0].w, u[1].x, u[1].y, u[1].z, u[1].w};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t dup = pack2(uu[kk], uu[kk]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ffma2(acc[kk][2 * i], v[i].x, dup);
        ffma2(acc[kk][2 * i + 1], v[i].y, dup);
      }
    }
  }
}

template <int V>
__global__ void __launch_bounds__(kThreads, 1)
wino_fp32_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_u,
                 const WinoParams p) {
  extern __shared__ __align__(1024) float smem[];
  float *stages = smem;
  float *stg = smem + kStages * kStageFloats;
  uint64_t *bars = reinterpret_cast<uint64_t *>(stg + SmemLayout<V>::kStagingFloats);
  volatile int *dead = reinterpret_cast<volatile int *>(bars + kStages);

  const int tid = threadIdx.x;
  const int my_tiles = (p.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int cpt = p.chunks_per_tile;
  const int total_chunks = my_tiles * cpt;

  if (tid == 0) {
    *dead = 0;
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(bars + s), 1);
    mbar_fence_init();
    tma_prefetch_descriptor(&tm_in);
    tma_prefetch_descriptor(&tm_u);
  }
  __syncthreads();

  // Issues the two TMA loads of chunk g (tile g / cpt of this CTA's list) into stage g % kStages.
  auto issue = [&](int g) {
    const int seq = g / cpt, ci = g - seq * cpt;
    const TileCoord tc = decode_tile(p, (int)blockIdx.x + seq * (int)gridDim.x);
    const int s = g % kStages;
    const uint32_t bar = smem_u32(bars + s);
    const uint32_t dst = smem_u32(stages + s * kStageFloats);
    mbar_arrive_expect_tx(bar, kStageBytes);
    tma_load_4d(dst, &tm_in, bar, tc.nb * kBN, 2 * tc.tx - 1, 2 * tc.ty - 1, ci * kBC);
    tma_load_3d(dst + kVStageFloats * 4u, &tm_u, bar, tc.kb * kBK, 0, ci * kBC);
  };

  if (tid == 0) {
    const int pre = total_chunks < kStages ? total_chunks : kStages;
    for (int g = 0; g < pre; ++g) issue(g);
  }

  uint64_t acc[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0ull;

  if (total_chunks > 0) {
    mbar_wait(smem_u32(bars + 0), 0, dead, p.status);
    transform_patch(stages);
    fence_proxy_async_smem();
    __syncthreads();
  }

  int ci = 0, seq = 0;
  for (int g = 0; g < total_chunks; ++g) {
    const int s = g % kStages;
    if (g + 1 < total_chunks) {
      const int s1 = (g + 1) % kStages;
      mbar_wait(smem_u32(bars + s1), ((g + 1) / kStages) & 1, dead, p.status);
      transform_patch(stages + s1 * kStageFloats);
      fence_proxy_async_smem();
    }
    compute_stage(acc, stages + s * kStageFloats);
    __syncthreads();   // chunk g+1 is transformed and visible; stage s may be refilled
    if (tid == 0 && g + kStages < total_chunks) issue(g + kStages);
    if (++ci == cpt) {
      const TileCoord tc = decode_tile(p, (int)blockIdx.x + seq * (int)gridDim.x);
      epilogue<V>(acc, stg, p, tc);
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0ull;
      ci = 0;
      ++seq;
    }
  }
}

}  // namespace ocb
