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
//   * warp-specialised, no block-wide barrier anywhere after set-up: four producer warps feed
//     eight consumer warps through a shared-memory ring guarded by mbarriers (full -> ready ->
//     empty per stage); register budgets are rebalanced with setmaxnreg;
//   * the 4x4 input patch (with its halo) and the 64-filter slice of the transformed filter
//     arrive by TMA; out-of-range coordinates are zero-filled by the hardware, which replaces
//     the reference's halo masks and predicated loads;
//   * the input transform runs in place in shared memory on three producer warps (a fourth
//     only issues TMA), one thread per (image, channel);
//   * the consumers form two groups of four warps, each owning 32 of the 64 filters and all 16
//     positions, so a group transposes, transforms and stores its outputs on its own (named
//     barrier of 128 threads) without stopping the other group;
//   * a lane owns 16 images x 8 filters of one position as 64 packed register pairs and issues
//     fma.rn.f32x2 (two FMAs per issue slot); per channel it needs 4+2 128-bit shared loads,
//     fetched one channel ahead, each served in the minimum two wavefronts.
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
constexpr int kGroupThreads = 128;          // one consumer group: 4 warps, 32 filters, 16 positions
constexpr int kConsumerThreads = 256;       // warps 0-3 group 0, warps 4-7 group 1
constexpr int kProducerThreads = 128;       // warp 8 issues TMA, warps 9-11 transform
constexpr int kTransformThreads = 96;
constexpr int kThreads = kConsumerThreads + kProducerThreads;
// setmaxnreg budgets.  The CTA owns what it was launched with, 384 threads x 168 registers =
// 64512, and can only redistribute that: 256*216 + 128*72 = 64512.  Asking for more than the
// producers give back would leave consumer warps waiting for registers for ever.
constexpr int kLaunchRegs = 168;
constexpr int kConsumerRegs = 216;
constexpr int kProducerRegs = 72;
static_assert(kConsumerThreads * kConsumerRegs + kProducerThreads * kProducerRegs <= kThreads * kLaunchRegs,
              "setmaxnreg budgets exceed the registers the CTA was launched with");
constexpr int kVStageFloats = 16 * kBC * kBN;   // [c][xi][n]   16 KiB
constexpr int kUStageFloats = 16 * kBC * kBK;   // [c][xi][k]   32 KiB
constexpr int kStageFloats = kVStageFloats + kUStageFloats;
constexpr uint32_t kStageBytes = kStageFloats * 4u;

// Staging buffer of a group: rows are (xi, kl), kl one of the 8 filters of a round, 32 images.
template <int V> struct Staging;
template <> struct Staging<kBase>       { static constexpr int kRowFloats = 36; static constexpr int kBuffers = 1; };
template <> struct Staging<kOptSts64>   { static constexpr int kRowFloats = 34; static constexpr int kBuffers = 1; };
template <> struct Staging<kOptSts64Cmp>{ static constexpr int kRowFloats = 32; static constexpr int kBuffers = 2; };
template <> struct Staging<kOptLds64>   { static constexpr int kRowFloats = 34; static constexpr int kBuffers = 1; };

// Shared memory: ring of kStages stages, two staging buffers, 3 mbarriers per stage, give-up flag.
template <int V> struct SmemLayout {
  static constexpr int kGroupStagingFloats = 128 * Staging<V>::kRowFloats * Staging<V>::kBuffers;
  static constexpr int kStagingFloats = 2 * kGroupStagingFloats;
  // four stages where the staging buffers leave room for them in 227 KB, else three
  static constexpr int kStages = ((size_t)4 * kStageBytes + (size_t)kStagingFloats * 4 + 128 <= 232448) ? 4 : 3;
  static constexpr size_t kBytes = (size_t)kStages * kStageBytes + (size_t)kStagingFloats * 4 + 128;
};

struct WinoParams {
  float *y;            // output, KHWN
  int N, C, K, H, W;
  int tiles_h, tiles_w, n_blocks, k_blocks, total_tiles, chunks_per_tile;
  // fp32 kernel only: work items.  Items below split_from are whole tiles; from there on each
  // tile is two items, one per consumer group (see item_tile).  split_from == total_tiles and
  // total_items == total_tiles mean "no split".
  int split_from, total_items;
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

// Work item -> tile and the consumer groups that compute it (bit 0 = group 0, bit 1 = group 1).
// The tiles of the last, partly filled round of the persistent schedule are cut in two items of 32
// filters each and given to two SMs: a group that has the FMA pipe to itself runs almost twice as
// fast, so that round takes about half as long.  The group that sits an item out only keeps the
// ring moving (it hands every stage straight back).
__device__ __forceinline__ int item_tile(const WinoParams &p, int item, int &groups) {
  if (item < p.split_from) {
    groups = 3;
    return item;
  }
  const int j = item - p.split_from;
  groups = 1 << (j & 1);
  return p.split_from + (j >> 1);
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

// Consumer lane roles.  Group gi owns filters 32*gi .. 32*gi+31 of the CTA tile and all 16
// Winograd positions: warp wq of a group owns positions 4*wq .. 4*wq+3, one per quarter-warp; a
// lane owns 16 images (half nh) x 8 filters (group of 8 kg) of its position.  Quarter-warps with
// an odd position read their image quads and filter quads in swapped order (qp), so that the
// two quarters of a half-warp never touch the same banks.
struct LaneRole {
  int gi, wq, qp, nh, kg, xi;
};
__device__ __forceinline__ LaneRole lane_role() {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  LaneRole r;
  r.gi = warp >> 2; r.wq = warp & 3; r.qp = (lane >> 3) & 1;
  r.nh = lane & 1; r.kg = (lane & 7) >> 1; r.xi = 4 * r.wq + (lane >> 3);
  return r;
}

// Staging row (one of 8 per position and round) for the lane's filter quad jj (0/1), and the
// filter (within the group's 32) which row kl holds in round r.  BASE spreads the rows of a
// quarter-warp differently because its 128-bit deposit is served per quarter-warp.
template <int V> __device__ __forceinline__ int staging_row(int kg, int jj) {
  return V == kBase ? kg + 4 * jj : 2 * kg + jj;
}
template <int V> __device__ __forceinline__ int round_filter(int kl, int r) {
  return V == kBase ? 8 * (kl & 3) + 4 * (kl >> 2) + r : 4 * kl + r;
}

__device__ __forceinline__ void group_barrier(int gi) {
  asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "n"(kGroupThreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Epilogue of one consumer group (128 threads): transpose the group's accumulators through its
// own staging buffer so that one thread holds all 16 Winograd positions of an (image, filter),
// transform, store.  acc[kk][qq]: kk = 4*j + e is filter 8*kg + 4*(j ^ qp) + e of the group,
// qq = 2*i + ep is the image pair starting at 4*(4*nh + (i ^ qp)) + 2*ep.
//
// Round r (0..3) moves e = r of both filter quads: 8 filters x 32 images x 16 positions.
//   BASE          deposit 8 x STS.128 (row pitch 36 floats), read back 32 x LDS.32, scalar stores
//   OPTSTS64      deposit 16 x STS.64 (row pitch 34 floats), read back 32 x LDS.32, scalar stores
//   OPTSTS64_CMP  as OPTSTS64 but unpadded rows rotated by (kl & 7) pairs, two buffers used
//                 alternately so that one barrier per round is enough
//   OPTLDS64      deposit as OPTSTS64, read back 16 x LDS.64, float2 stores
// Only the group's own named barrier is used, so the other group keeps computing meanwhile.
// ---------------------------------------------------------------------------------------------
template <int V, bool RAGGED>
__device__ __forceinline__ void epilogue(uint64_t (&acc)[8][8], float *stg, const WinoParams &p,
                                         const TileCoord &tc, const LaneRole &role) {
  const int lane = threadIdx.x & 31;
  constexpr int RF = Staging<V>::kRowFloats;

  const int oh0 = 2 * tc.ty, ow0 = 2 * tc.tx;
  const bool row1 = (oh0 + 1) < p.H, col1 = (ow0 + 1) < p.W;
  const size_t plane = (size_t)p.H * p.W * p.N;                       // one filter's output
  float *ybase = p.y + ((size_t)oh0 * p.W + ow0) * p.N + (size_t)tc.nb * kBN +
                 ((size_t)tc.kb * kBK + 32 * role.gi) * plane;
  const size_t dW = (size_t)p.N, dH = (size_t)p.W * p.N;
  // Ragged last block of images or filters (N not a multiple of 32, K not of 64; its own kernel
  // instantiation, so that the usual case pays nothing): what is missing was loaded as zeros and
  // is not stored.  N is a multiple of 4, so an image pair is either inside or outside.
  const bool n_ok = !RAGGED || (V == kOptLds64 ? 2 * (lane & 15) : lane) < p.N - tc.nb * kBN;
  const int k_left = p.K - (tc.kb * kBK + 32 * role.gi);              // filters of this group's 32 that exist

#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float *buf = stg + ((V == kOptSts64Cmp) ? (r & 1) * kGroupThreads * RF : 0);
    // ---- deposit ----
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int kl = staging_row<V>(role.kg, j ^ role.qp);
      float *row = buf + (role.xi * 8 + kl) * RF;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int nq = 4 * role.nh + (i ^ role.qp);                  // image quad of the row
        if (V == kBase) {
          *reinterpret_cast<ulonglong2 *>(row + 4 * nq) =
              make_ulonglong2(acc[4 * j + r][2 * i], acc[4 * j + r][2 * i + 1]);
        } else if (V == kOptSts64Cmp) {
          const int rot = kl & 7;
          *reinterpret_cast<uint64_t *>(row + 2 * ((2 * nq + 0 + rot) & 15)) = acc[4 * j + r][2 * i];
          *reinterpret_cast<uint64_t *>(row + 2 * ((2 * nq + 1 + rot) & 15)) = acc[4 * j + r][2 * i + 1];
        } else {
          *reinterpret_cast<uint64_t *>(row + 4 * nq) = acc[4 * j + r][2 * i];
          *reinterpret_cast<uint64_t *>(row + 4 * nq + 2) = acc[4 * j + r][2 * i + 1];
        }
      }
    }
    group_barrier(role.gi);
    // ---- read back, transform, store ----
    if (V == kOptLds64) {
      const int np = lane & 15, kl = 2 * role.wq + (lane >> 4);
      float m0[16], m1[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        const float2 v = *reinterpret_cast<const float2 *>(buf + (x * 8 + kl) * RF + 2 * np);
        m0[x] = v.x; m1[x] = v.y;
      }
      float y0[4], y1[4];
      output_transform(m0, y0);
      output_transform(m1, y1);
      float *dst = ybase + (size_t)round_filter<V>(kl, r) * plane + 2 * np;
      if (n_ok && (!RAGGED || round_filter<V>(kl, r) < k_left)) {
        *reinterpret_cast<float2 *>(dst) = make_float2(y0[0], y1[0]);
        if (col1) *reinterpret_cast<float2 *>(dst + dW) = make_float2(y0[1], y1[1]);
        if (row1) {
          *reinterpret_cast<float2 *>(dst + dH) = make_float2(y0[2], y1[2]);
          if (col1) *reinterpret_cast<float2 *>(dst + dH + dW) = make_float2(y0[3], y1[3]);
        }
      }
    } else {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int kl = role.wq + 4 * half;
        float m[16];
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const float *row = buf + (x * 8 + kl) * RF;
          if (V == kOptSts64Cmp) m[x] = row[(lane + 2 * (kl & 7)) & 31];
          else                   m[x] = row[lane];
        }
        float yy[4];
        output_transform(m, yy);
        float *dst = ybase + (size_t)round_filter<V>(kl, r) * plane + lane;
        if (n_ok && (!RAGGED || round_filter<V>(kl, r) < k_left)) {
          dst[0] = yy[0];
          if (col1) dst[dW] = yy[1];
          if (row1) {
            dst[dH] = yy[2];
            if (col1) dst[dH + dW] = yy[3];
          }
        }
      }
    }
    if (V != kOptSts64Cmp) group_barrier(role.gi);
  }
}

// ---------------------------------------------------------------------------------------------
// In-place input transform V = B^T d B of two adjacent images of one channel inside a pipeline
// stage: columns first, then rows (operation order of src/convolutionForward_32x64x8.cu:59-80),
// with packed add/sub (each half rounded exactly like the scalar operation).  The stage holds
// the raw patches as [c][h][w][n]; afterwards the same slots hold [c][xi][n].
// `t` in 0..127: channel t >> 4, image pair t & 15.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// Scalar form: one (image, channel) patch, `patch` = c * 32 + n.
__device__ __forceinline__ void transform_patch(float *vstage, int patch) {
  float *R = vstage + ((patch >> 5) * 16) * kBN + (patch & 31);
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
// Operands of one channel for one lane: 16 images as 8 pairs, 8 filters.
struct Frag {
  ulonglong2 v[4];
  float4 u[2];
};

// vp / up point at the lane's first image quad / filter quad of channel 0 in the stage; the
// swapped order of odd quarter-warps is folded into the two offsets o1 (0 or 4 floats).
__device__ __forceinline__ void load_frag(Frag &f, const float *vp, const float *up, int o1, int c) {
  const float *v = vp + c * 16 * kBN, *u = up + c * 16 * kBK;
  f.v[0] = *reinterpret_cast<const ulonglong2 *>(v + o1);
  f.v[1] = *reinterpret_cast<const ulonglong2 *>(v + (4 - o1));
  f.v[2] = *reinterpret_cast<const ulonglong2 *>(v + 8 + o1);
  f.v[3] = *reinterpret_cast<const ulonglong2 *>(v + 8 + (4 - o1));
  f.u[0] = *reinterpret_cast<const float4 *>(u + o1);
  f.u[1] = *reinterpret_cast<const float4 *>(u + (4 - o1));
}

// 64 packed FMAs of one channel.  Both nestings of the two loops measured the same inside the
// kernel (the image-pair-outermost one is ~4 % faster in isolation).
__device__ __forceinline__ void fma_frag(uint64_t (&acc)[8][8], const Frag &f) {
  const float uu[8] = {f.u[0].x, f.u[0].y, f.u[0].z, f.u[0].w, f.u[1].x, f.u[1].y, f.u[1].z, f.u[1].w};
  const uint64_t vv[8] = {f.v[0].x, f.v[0].y, f.v[1].x, f.v[1].y, f.v[2].x, f.v[2].y, f.v[3].x, f.v[3].y};
  uint64_t dup[8];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) dup[kk] = pack2(uu[kk], uu[kk]);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
#pragma unroll
    for (int qq = 0; qq < 8; ++qq) ffma2(acc[kk][qq], vv[qq], dup[kk]);
}

template <int V, bool RAGGED>
__global__ void __launch_bounds__(kThreads, 1)
wino_fp32_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_u,
                 const WinoParams p) {
  constexpr int S = SmemLayout<V>::kStages;
  extern __shared__ __align__(1024) float smem[];
  float *stages = smem;
  float *stg = smem + S * kStageFloats;
  uint64_t *bars = reinterpret_cast<uint64_t *>(stg + SmemLayout<V>::kStagingFloats);
  uint64_t *bar_full = bars, *bar_ready = bars + S, *bar_empty = bars + 2 * S;   // per stage
  volatile int *dead = reinterpret_cast<volatile int *>(bars + 3 * S);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int my_tiles = (p.total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // work items
  const int cpt = p.chunks_per_tile;
  const int total_chunks = my_tiles * cpt;

  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(bar_full + s), 1);                       // the TMA issuer + its bytes
      mbar_init(smem_u32(bar_ready + s), kTransformThreads / 32);  // one arrive per transform warp
      mbar_init(smem_u32(bar_empty + s), kConsumerThreads / 32);   // one arrive per consumer warp
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp >= kConsumerThreads / 32) {
    // =============================== producers ===============================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
    if (warp == kConsumerThreads / 32) {
      // ---- TMA issuer: one lane keeps the ring full ----
      if (lane == 0) {
        tma_prefetch_descriptor(&tm_in);
        tma_prefetch_descriptor(&tm_u);
        int seq = 0, ci = 0, groups_unused, issued = 0;
        TileCoord tc = decode_tile(p, item_tile(p, (int)blockIdx.x, groups_unused));
        for (int g = 0; g < total_chunks; ++g) {
          const int s = g % S;
          // A wait that gave up: stop issuing - the stage may still be in use.
          if (g >= S && !mbar_wait(smem_u32(bar_empty + s), ((g / S) - 1) & 1, dead, p.status)) break;
          const uint32_t bar = smem_u32(bar_full + s);
          const uint32_t dst = smem_u32(stages + s * kStageFloats);
          mbar_arrive_expect_tx(bar, kStageBytes);
          tma_load_4d(dst, &tm_in, bar, tc.nb * kBN, 2 * tc.tx - 1, 2 * tc.ty - 1, ci * kBC);
          tma_load_3d(dst + kVStageFloats * 4u, &tm_u, bar, tc.kb * kBK, 0, ci * kBC);
          issued = g + 1;
          if (++ci == cpt) {
            ci = 0;
            ++seq;
            if (seq < my_tiles) tc = decode_tile(p, item_tile(p, (int)blockIdx.x + seq * (int)gridDim.x, groups_unused));
          }
        }
        // The CTA must not exit with bulk copies in flight.  After a complete run the last loads
        // were consumed long ago and these waits return at once; after a give-up they let what
        // was issued land (with a limit of their own).
        for (int g = issued > S ? issued - S : 0; g < issued; ++g)
          mbar_wait_drain(smem_u32(bar_full + g % S), (g / S) & 1);
      }
    } else {
      // ---- transform warps: raw patch -> V, in place, as soon as a stage has landed ----
      const int t = tid - kConsumerThreads - 32;                  // 0..95
      for (int g = 0; g < total_chunks; ++g) {
        const int s = g % S;
        mbar_wait(smem_u32(bar_full + s), (g / S) & 1, dead, p.status);
        float *vst = stages + s * kStageFloats;
        for (int patch = t; patch < kBC * kBN; patch += kTransformThreads) transform_patch(vst, patch);
        fence_proxy_async_smem();     // these generic writes precede the TMA that refills the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bar_ready + s));
      }
    }
    return;
  }

  // ================================= consumers =================================================
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));
  const LaneRole role = lane_role();
  // lane's operand origins inside a stage and the 0/4-float swap of odd quarter-warps
  const int o1 = 4 * role.qp;
  const int voff = role.xi * kBN + 16 * role.nh;
  const int uoff = kVStageFloats + role.xi * kBK + 32 * role.gi + 8 * role.kg;
  float *my_stg = stg + role.gi * SmemLayout<V>::kGroupStagingFloats;

  uint64_t acc[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0ull;

  // Two operand buffers used alternately: channel c computes from frag[c & 1] while frag[(c + 1) & 1]
  // is being loaded.  With the channel loop unrolled the indices are constants, so no register
  // copies are needed (a "cur = nxt" hand-over cost 24 moves per channel).
  Frag frag[2];
  if (total_chunks > 0) {
    mbar_wait(smem_u32(bar_ready + 0), 0, dead, p.status);
    load_frag(frag[0], stages + voff, stages + uoff, o1, 0);   // harmless if this group sits the first item out
  }
  int g = 0;                                                       // chunk counter over all items of this CTA
  for (int seq = 0; seq < my_tiles; ++seq) {
    int groups;
    const int tile = item_tile(p, (int)blockIdx.x + seq * (int)gridDim.x, groups);
    if ((groups >> role.gi) & 1) {
      // ---- this group computes the item ----
      for (int ci = 0; ci < cpt; ++ci, ++g) {
        const int s = g % S;
        const float *st = stages + s * kStageFloats;
#pragma unroll
        for (int c = 0; c < kBC; ++c) {
          if (c + 1 < kBC) {
            load_frag(frag[(c + 1) & 1], st + voff, st + uoff, o1, c + 1);
          } else {
            // All reads of this stage have been issued.  With a ring of three stages it is handed
            // back right away (the look-ahead is short); with four, after the last FMAs (below).
            if (S < 4) {
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(bar_empty + s));
            }
            if (g + 1 < total_chunks) {
              const int s1 = (g + 1) % S;
              mbar_wait(smem_u32(bar_ready + s1), ((g + 1) / S) & 1, dead, p.status);
              const float *st1 = stages + s1 * kStageFloats;
              load_frag(frag[0], st1 + voff, st1 + uoff, o1, 0);
            }
          }
          fma_frag(acc, frag[c & 1]);
        }
        // Four stages: hand the stage back after the last FMAs rather than before them, so that the
        // warp-wide synchronisation does not sit in front of an FMA batch (0.5-0.8 % on the sweep;
        // with three stages the later release costs 2-4 % instead).
        if (S >= 4) {
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(bar_empty + s));
        }
      }
      const TileCoord tc = decode_tile(p, tile);
      epilogue<V, RAGGED>(acc, my_stg, p, tc, role);
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0ull;
    } else {
      // ---- the other group computes it: only keep the ring moving, stage by stage ----
      for (int ci = 0; ci < cpt; ++ci, ++g) {
        const int s = g % S;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bar_empty + s));
        if (g + 1 < total_chunks) {
          const int s1 = (g + 1) % S;
          mbar_wait(smem_u32(bar_ready + s1), ((g + 1) / S) & 1, dead, p.status);
          const float *st1 = stages + s1 * kStageFloats;
          load_frag(frag[0], st1 + voff, st1 + uoff, o1, 0);       // in case the next item is ours
        }
      }
    }
  }
}

}  // namespace ocb
