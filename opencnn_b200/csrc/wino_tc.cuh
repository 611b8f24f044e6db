// Fused Winograd F(2x2,3x3) forward kernel with the 16 batched GEMMs on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in TMEM), operands in BF16 or TF32, fp32 accumulate.
//
// Same operator as wino_fp32.cuh - it replaces the reference's Winograd_kernel
// (src/convolutionForward_32x64x8.cu:169-262) - but only the contraction of its main loop
// (outer_product, src/outer_product.cuh) moves to the tensor cores; the input and output
// transforms stay in fp32 on the CUDA cores.  The reference has no tensor-core path.
//
// One CTA tile = 128 filters x 32 images x one 2x2-output tile, all 16 Winograd positions: the
// 16 accumulators D[xi] (128 x 32 fp32 each) fill the SM's tensor memory exactly (512 columns).
// Filters are the M dimension of the MMA, images the N dimension, channels the K dimension:
//   D[xi][k][n] += sum_c U[xi][k][c] * V[xi][n][c]
// Both operands are "MN-major" in shared memory (M resp. N contiguous), which is how they exist
// anyway: U rows of consecutive filters come straight from the transformed-filter workspace by
// TMA (128-byte swizzle), V rows of consecutive images are written by the transform threads.
// Per K-step (16 channels in BF16, 8 in TF32) 16 MMAs are issued, by two threads.
//
// Warp roles (512 threads):
//   warp 0      TMA: raw input patches (4-D box, hardware zero-fill = halo), a ring of their own
//   warp 14     TMA: U slices (a loader of its own, so patches never queue behind filter slices)
//   warps 1-4   input transform B^T d B in fp32, rounding, V written in the UMMA layout
//   warps 5,15  MMA issue (one thread each, 8 positions per thread), tcgen05.commit to free stages
//               and to publish a finished tile; warp 5 also owns the TMEM allocation
//   warps 6-13  epilogue, two warps per TMEM lane quarter (each takes half of the 32 images):
//               tcgen05.ld one column of the 4x4 positions of (filter = TMEM lane, 8 images) at a
//               time, A^T M A accumulated in registers - no shared-memory transpose - neighbouring
//               lanes swap image halves, 32-byte stores in 64-byte runs
// All hand-offs are mbarriers with bounded waits.
#pragma once
#include "fx.cuh"
#include "ptx.cuh"
#include "wino_fp32.cuh"   // WinoParams, TileCoord, output_transform, add2/sub2

namespace ocb {

enum TcType : int { kTcBf16 = 0, kTcTf32 = 1 };

constexpr int kTcEpilogueWarps = 8;
// Four transform warps, two items per thread and K-step.  Eight warps with one item each were
// measured too: the CTA then has 640 threads, the register cap drops to 96 and the epilogue
// spills - 3-5 % slower; eight transform warps with four epilogue warps (two passes each), which
// keeps 512 threads, were 2-5 % slower too.  Two groups of two warps taking K-steps alternately were 8 % slower
// (the transform's latency per K-step matters, not only its throughput).
constexpr int kTcTransformWarps = 4;                          // warps 1 .. kTcTransformWarps
constexpr int kTcMmaWarp = 1 + kTcTransformWarps;             // first MMA-issuing thread (also owns the TMEM allocation)
constexpr int kTcFirstEpilogueWarp = kTcMmaWarp + 1;
constexpr int kTcULoaderWarp = kTcFirstEpilogueWarp + kTcEpilogueWarps;
constexpr int kTcMmaWarpB = kTcULoaderWarp + 1;               // first of the additional MMA-issuing warps
constexpr int kTcM = 128;                   // filters per CTA tile
constexpr int kTcN = 32;                    // images per CTA tile
constexpr int kTcStages = 2;
constexpr uint32_t kTcVBytes = 16 * 1024;   // 16 positions x (32 images x one K-step)

// HU ("half U"): BF16 problems with at most 64 filters.  Their A operand repeats its first
// 64-filter block (see tile_repeats_filters), so only that block is loaded: U stages are 32 KB
// instead of 64 KB, and the room goes to the raw-patch ring (four stages instead of two), which
// is what the large-image layers with few filters lack (their patches come from HBM, not L2).
template <int DT, bool HU = false> struct TcCfg {
  static constexpr int kKC = DT == kTcBf16 ? 16 : 8;                 // channels per K-step / stage
  static constexpr uint32_t kRawBytes = kKC * 16 * kTcN * 4;         // [c][h][w][n] fp32
  // The raw patches have their own ring, as deep as shared memory allows next to two stages of U
  // and V: TF32 stages are 16 KB (four fit), BF16 stages 32 KB (two).
  static constexpr int kRawStages = (DT == kTcBf16 && !HU) ? 2 : 4;
  static constexpr uint32_t kUPosBytes = HU ? 2048 : 4096;           // one position of a U stage
  static constexpr uint32_t kUBytes = 16 * kUPosBytes;
  // MMA-issuing threads (warp kTcMmaWarp and warps kTcMmaWarpB ..).  Two: one thread cannot issue
  // these small MMAs faster than one per ~52 cycles, two keep the tensor pipe fed (40 cycles per
  // MMA).  Four measured the same as two in BF16; in TF32 they cost more than they bring, because
  // 18 warps leave the epilogue 96 registers per thread instead of 128 (3-7 % slower).
  static constexpr int kIssuers = 2;
  static constexpr int kThreads = (kTcMmaWarpB + kIssuers - 1) * 32;
  static constexpr size_t kSmemBytes = (size_t)kRawStages * kRawBytes + (size_t)kTcStages * (kUBytes + kTcVBytes) + 1024;
};

// ---- tcgen05 wrappers ------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc_512(uint32_t smem_dst) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_dst) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_512(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int DT>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (DT == kTcBf16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
__device__ __forceinline__ void tmem_ld_x4(uint32_t taddr, float (&v)[4]) {
  uint32_t r0, r1, r2, r3;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(taddr) : "memory");
  v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
}
// 256-bit global store (one full 32-byte sector per lane); `p` must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(float *p, const float (&a)[4], const float (&b)[4]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(a[0]), "f"(a[1]), "f"(a[2]),
               "f"(a[3]), "f"(b[0]), "f"(b[1]), "f"(b[2]), "f"(b[3]) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets
// (all in 16-byte units), version 1, swizzle mode (2 = 128 B, 4 = 64 B, 6 = 32 B, 0 = none,
// 1 = 128 B with 32-byte atoms).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
// Instruction descriptor: fp32 accumulate, A and B of the same format, both MN-major, M x N.
template <int DT> __device__ __forceinline__ uint32_t instr_desc() {
  const uint32_t fmt = DT == kTcBf16 ? 1u : 2u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(kTcN >> 3) << 17) |
         ((uint32_t)(kTcM >> 4) << 24);
}

__device__ __forceinline__ float round_tf32_rne(float v) {
  uint32_t u = __float_as_uint(v);
  u += 0xFFFu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xFFFFE000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---- filter transform for the tensor-core path ------------------------------------------------
// Same arithmetic as fx_kernel, then one rounding to the operand type.  Output [C][16][K]:
// BF16 packed, or fp32 words holding TF32 values (low 13 mantissa bits zero).
template <int DT>
__global__ void __launch_bounds__(128) fx_tc_kernel(const float4 *__restrict__ g, void *__restrict__ U, int C, int k4) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= C * k4) return;
  const int c = idx / k4, kq = idx - c * k4;
  const float4 *src = g + (size_t)c * 9 * k4 + kq;
  float4 in[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) in[i] = __ldg(src + (size_t)i * k4);
  float wx[9], wy[9], wz[9], ww[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) { wx[i] = in[i].x; wy[i] = in[i].y; wz[i] = in[i].z; ww[i] = in[i].w; }
  float ux[16], uy[16], uz[16], uw[16];
  fx_one(wx, ux); fx_one(wy, uy); fx_one(wz, uz); fx_one(ww, uw);
  if (DT == kTcBf16) {
    uint2 *dst = reinterpret_cast<uint2 *>(U) + (size_t)c * 16 * k4 + kq;
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[(size_t)i * k4] = make_uint2(pack_bf16x2(ux[i], uy[i]), pack_bf16x2(uz[i], uw[i]));
  } else {
    float4 *dst = reinterpret_cast<float4 *>(U) + (size_t)c * 16 * k4 + kq;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      dst[(size_t)i * k4] = make_float4(round_tf32_rne(ux[i]), round_tf32_rne(uy[i]), round_tf32_rne(uz[i]), round_tf32_rne(uw[i]));
  }
}

// ---- input transform into the V operand --------------------------------------------------------
// BF16: item = (channel c of the stage, image pair np); V tile of a position is [16 c][32 n] bf16,
// rows of 64 bytes, 64-byte swizzle (16-byte chunk index ^= (c >> 1) & 3).
__device__ __forceinline__ void finish_v_bf16(const uint64_t (&d)[16], uint8_t *__restrict__ vst, int c, int np) {
  uint64_t b[16];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b[j] = sub2(d[j], d[8 + j]);
    b[4 + j] = add2(d[4 + j], d[8 + j]);
    b[8 + j] = sub2(d[8 + j], d[4 + j]);
    b[12 + j] = sub2(d[4 + j], d[12 + j]);
  }
  uint8_t *dst = vst + c * 64 + ((((np >> 2) ^ (c >> 1)) & 3) << 4) + ((np & 3) << 2);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint64_t o[4];
    o[0] = sub2(b[4 * i + 0], b[4 * i + 2]);
    o[1] = add2(b[4 * i + 1], b[4 * i + 2]);
    o[2] = sub2(b[4 * i + 2], b[4 * i + 1]);
    o[3] = sub2(b[4 * i + 1], b[4 * i + 3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float lo, hi;
      unpack2(o[j], lo, hi);
      *reinterpret_cast<uint32_t *>(dst + (4 * i + j) * 1024) = pack_bf16x2(lo, hi);
    }
  }
}
// The two items of a thread (channels c and c + 8 of image pair np): all loads first, so that
// the two shared-memory round trips overlap.
__device__ __forceinline__ void transform_to_v_bf16_x2(const float *__restrict__ raw, uint8_t *__restrict__ vst, int c, int np) {
  constexpr int P = kTcN / 2;
  const uint64_t *R0 = reinterpret_cast<const uint64_t *>(raw + (c * 16) * kTcN + 2 * np), *R1 = R0 + 8 * 16 * P;
  uint64_t d0[16], d1[16];
#pragma unroll
  for (int q = 0; q < 16; ++q) { d0[q] = R0[q * P]; d1[q] = R1[q * P]; }
  finish_v_bf16(d0, vst, c, np);
  finish_v_bf16(d1, vst, c + 8, np);
}
// TF32: item = (channel c of the stage, image n); V tile of a position is [8 c][32 n] fp32, rows
// of 128 bytes, in the "128-byte swizzle with 32-byte atoms" pattern that MN-major 32-bit operands
// need (32-byte chunk index ^= c & 3; the pattern repeats every 4 rows).
// Packed form: one item = (channel c, image pair np); the two images of a pair are adjacent in a
// V row, so each result is one 8-byte store.  Same operations per image as the scalar form.
__device__ __forceinline__ void transform_to_v_tf32_pair(const float *__restrict__ raw, uint8_t *__restrict__ vst, int c, int np) {
  constexpr int P = kTcN / 2;
  const uint64_t *R = reinterpret_cast<const uint64_t *>(raw + (c * 16) * kTcN + 2 * np);
  uint64_t d[16], b[16];
#pragma unroll
  for (int q = 0; q < 16; ++q) d[q] = R[q * P];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b[j] = sub2(d[j], d[8 + j]);
    b[4 + j] = add2(d[4 + j], d[8 + j]);
    b[8 + j] = sub2(d[8 + j], d[4 + j]);
    b[12 + j] = sub2(d[4 + j], d[12 + j]);
  }
  const int n = 2 * np;
  uint8_t *dst = vst + c * 128 + ((((n >> 3) ^ c) & 3) << 5) + ((n & 7) << 2);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint64_t o[4];
    o[0] = sub2(b[4 * i + 0], b[4 * i + 2]);
    o[1] = add2(b[4 * i + 1], b[4 * i + 2]);
    o[2] = sub2(b[4 * i + 2], b[4 * i + 1]);
    o[3] = sub2(b[4 * i + 1], b[4 * i + 3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float lo, hi;
      unpack2(o[j], lo, hi);
      *reinterpret_cast<float2 *>(dst + (4 * i + j) * 1024) = make_float2(round_tf32_rne(lo), round_tf32_rne(hi));
    }
  }
}
// True when the tile's accumulator rows 64-127 repeat rows 0-63 (see the MMA issuer).
template <int DT> __device__ __forceinline__ bool tile_repeats_filters(const WinoParams &p, const TileCoord &tc) {
  return DT == kTcBf16 && p.K - tc.kb * kTcM <= 64;
}

// p.k_blocks counts 128-filter blocks here.
template <int DT, bool HU = false>
__global__ void __launch_bounds__(TcCfg<DT, HU>::kThreads, 1)
wino_tc_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_u, const WinoParams p) {
  using Cfg = TcCfg<DT, HU>;
  static_assert(!HU || DT == kTcBf16, "the half-U variant relies on the BF16 block aliasing");
  constexpr int KC = Cfg::kKC;
  extern __shared__ __align__(1024) uint8_t tsmem[];
  uint8_t *raw_s = tsmem;                                              // [stage][KC][16][32] fp32
  constexpr int SR = Cfg::kRawStages;
  uint8_t *u_s = raw_s + SR * Cfg::kRawBytes;                          // [stage][16 xi][...]  4 KB per position
  uint8_t *v_s = u_s + kTcStages * Cfg::kUBytes;                       // [stage][16 xi][...]  1 KB per position
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_s + kTcStages * kTcVBytes);
  uint64_t *raw_full = bars, *raw_empty = bars + SR, *u_full = bars + 2 * SR, *uv_empty = u_full + 4;   // u_full: U landed and V written
  uint64_t *acc_full = u_full + 6;
  uint64_t *acc_empty = u_full + 14;                   // [4]: one per column of the 4x4 positions (see the epilogue)
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(u_full + 8);
  volatile int *dead = reinterpret_cast<volatile int *>(u_full + 9);
  uint64_t *mma_done = u_full + 10;                    // one per MMA-issuing thread: "all my MMAs have completed"

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int my_tiles = (p.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int cpt = p.chunks_per_tile;
  const int total_chunks = my_tiles * cpt;

  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < SR; ++s) {
      mbar_init(smem_u32(raw_full + s), 1);
      mbar_init(smem_u32(raw_empty + s), kTcTransformWarps);
    }
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(smem_u32(u_full + s), kTcTransformWarps + 1);   // U loader (with its bytes) + one arrive per transform warp
      mbar_init(smem_u32(uv_empty + s), Cfg::kIssuers);      // one tcgen05.commit per MMA-issuing thread
    }
    mbar_init(smem_u32(acc_full), Cfg::kIssuers);
    for (int j = 0; j < 4; ++j) mbar_init(smem_u32(acc_empty + j), kTcEpilogueWarps);
    for (int i = 0; i < Cfg::kIssuers; ++i) mbar_init(smem_u32(mma_done + i), 1);
    mbar_fence_init();
  }
  if (warp == kTcMmaWarp) tmem_alloc_512(smem_u32(tmem_slot));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == kTcULoaderWarp) {
    // ===================================== TMA producers =======================================
    // Two independent loaders, so that the input patches (needed early, by the transform) never
    // wait behind the filter slices (whose stage is released late, by the MMAs): warp 0 loads the
    // raw patches, the last warp loads U.
    const bool loads_u = warp != 0;
    if (lane == 0) {
      tma_prefetch_descriptor(loads_u ? &tm_u : &tm_in);
      int seq = 0, ci = 0, issued = 0;
      TileCoord tc = decode_tile(p, (int)blockIdx.x);
      for (int g = 0; g < total_chunks; ++g) {
        const int s = g % kTcStages;
        const uint32_t use = g / kTcStages;
        // A wait that gave up: stop issuing - the stage may still be in use.
        if (!loads_u) {
          const int sr = g % SR;
          const uint32_t use_r = g / SR;
          if (use_r > 0 && !mbar_wait(smem_u32(raw_empty + sr), (use_r - 1) & 1, dead, p.status)) break;
          mbar_arrive_expect_tx(smem_u32(raw_full + sr), Cfg::kRawBytes);
          tma_load_4d(smem_u32(raw_s + sr * Cfg::kRawBytes), &tm_in, smem_u32(raw_full + sr), tc.nb * kTcN,
                      2 * tc.tx - 1, 2 * tc.ty - 1, ci * KC);
        } else {
          if (use > 0 && !mbar_wait(smem_u32(uv_empty + s), (use - 1) & 1, dead, p.status)) break;
          mbar_arrive_expect_tx(smem_u32(u_full + s), Cfg::kUBytes);
          // U viewed as {filters within a 128-byte row, channel, 128-byte row of the filter axis, position}
          tma_load_4d(smem_u32(u_s + s * Cfg::kUBytes), &tm_u, smem_u32(u_full + s), 0, ci * KC,
                      tc.kb * (DT == kTcBf16 ? 2 : 4), 0);
        }
        issued = g + 1;
        if (++ci == cpt) {
          ci = 0;
          ++seq;
          if (seq < my_tiles) tc = decode_tile(p, (int)blockIdx.x + seq * (int)gridDim.x);
        }
      }
      // No exit with bulk copies in flight: wait (with a limit of its own) for the last loads of
      // every stage.  After a complete run these phases are long over.  u_full also counts the
      // transform warps' arrivals; after a give-up those may be missing, and then the limit ends
      // the wait.
      const int ring = loads_u ? kTcStages : SR;
      for (int g = issued > ring ? issued - ring : 0; g < issued; ++g)
        mbar_wait_drain(smem_u32((loads_u ? u_full : raw_full) + g % ring), (g / ring) & 1);
    }
  } else if (warp <= kTcTransformWarps) {
    // ===================================== input transform =====================================
    const int t = tid - 32;                                            // 0 .. 32 * kTcTransformWarps - 1
    for (int g = 0; g < total_chunks; ++g) {
      const int s = g % kTcStages, sr = g % SR;
      const uint32_t use = g / kTcStages;
      mbar_wait(smem_u32(raw_full + sr), (g / SR) & 1, dead, p.status);
      if (use > 0) mbar_wait(smem_u32(uv_empty + s), (use - 1) & 1, dead, p.status);   // V stage free again
      const float *raw = reinterpret_cast<const float *>(raw_s + sr * Cfg::kRawBytes);
      uint8_t *vst = v_s + s * kTcVBytes;
      if (DT == kTcBf16) {
        transform_to_v_bf16_x2(raw, vst, t >> 4, t & 15);          // 16 channels x 16 image pairs, two items per thread
      } else {
        transform_to_v_tf32_pair(raw, vst, t >> 4, t & 15);        // 8 channels x 16 image pairs = 128 threads
      }
      fence_proxy_async_smem();          // V is read by the tensor core through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(raw_empty + sr));
        mbar_arrive(smem_u32(u_full + s));
      }
    }
  } else if (warp == kTcMmaWarp || warp >= kTcMmaWarpB) {
    // ===================================== MMA issuers =========================================
    // Two threads, each issuing the MMAs of eight positions (disjoint accumulator columns, so no
    // ordering is needed between them).  One thread's waits and fences then overlap the other's
    // issuing; with a single issuer its instruction stream (16 MMAs plus ~500 cycles of waits,
    // fence and commit per K-step) was what bounded the main loop.
    // The descriptors are built once and only advanced by constants inside the fully unrolled
    // loop: building them per instruction made each of these small MMAs (N = 32 occupies the
    // tensor pipe ~50 cycles) cost ~180 cycles.
    if (lane == 0) {
      // A thread issues whole columns of the 4x4 positions (two columns each), column by column:
      // the epilogue hands the accumulators back per column, so the next tile's first MMAs start while the
      // other columns are still being read.
      constexpr int kPer = 16 / Cfg::kIssuers;                              // positions per issuing thread
      const int me = warp == kTcMmaWarp ? 0 : warp - kTcMmaWarpB + 1;
      const int col0 = me * (kPer / 4);                                     // first column of this thread
      const uint32_t idesc = instr_desc<DT>();
      // A: 128 filters x KC channels, filter-contiguous rows of 128 B (64 bf16 / 32 tf32 filters), 8-channel
      //    groups 1 KB apart, 128-byte-row blocks of the filter axis KC*128 B apart.
      // B: 32 images x KC channels, image-contiguous rows (64 B bf16 / 128 B tf32), 8-channel groups 512 B apart.
      // TF32 (32-bit, MN-major) uses the 128B-swizzle-with-32B-atom mode: 4-channel groups 512 B apart.
      const uint64_t a_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(u_s), KC * 128, 1024, 2) : smem_desc(smem_u32(u_s), KC * 128, 512, 1);
      // When at most 64 of the tile's 128 filters exist (K = 64 layers) the second 64-filter block of the BF16
      // A operand is made to alias the first (block stride 0): accumulator rows 64-127 then repeat rows 0-63,
      // and the epilogue warps that own those TMEM lanes take half of the images instead of idling.
      const uint64_t a_desc0_dup = smem_desc(smem_u32(u_s), 0, 1024, 2);
      bool dup = tile_repeats_filters<DT>(p, decode_tile(p, (int)blockIdx.x));
      const uint64_t b_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(v_s), 512, 512, 4) : smem_desc(smem_u32(v_s), 1024, 512, 1);
      int ci = 0, seq = 0;
      for (int g = 0; g < total_chunks; ++g) {
        const int s = g % kTcStages;
        const uint32_t use = g / kTcStages;
        // A wait that gave up: stop issuing (the operands or the accumulators are not ready).
        if (!mbar_wait(smem_u32(u_full + s), use & 1, dead, p.status)) break;      // U landed and V written
        tc_fence_after();
        const uint64_t ad = ((dup || HU) ? a_desc0_dup : a_desc0) + (uint64_t)(s * (Cfg::kUBytes >> 4)) + (uint64_t)(col0 * (Cfg::kUPosBytes >> 4)),
                       bd = b_desc0 + (uint64_t)(s * (kTcVBytes >> 4)) + (uint64_t)(col0 * (1024 >> 4));
        const uint32_t accumulate = ci > 0 ? 1u : 0u, d0 = tmem_base + col0 * kTcN;
        bool ok = true;
#pragma unroll
        for (int xo = 0; xo < kPer; ++xo) {
          const int xr = 4 * (xo & 3) + (xo >> 2);                          // position relative to col0: row xo & 3, column xo >> 2
          if ((xo & 3) == 0 && ci == 0 && seq > 0) {                         // first write to a column of a new tile: drained?
            if (!mbar_wait(smem_u32(acc_empty + col0 + (xo >> 2)), (seq - 1) & 1, dead, p.status)) { ok = false; break; }
            tc_fence_after();
          }
          tc_mma<DT>(d0 + xr * kTcN, ad + (uint64_t)(xr * (Cfg::kUPosBytes >> 4)), bd + (uint64_t)(xr * (1024 >> 4)), idesc, accumulate);
        }
        if (!ok) break;
        tc_commit(smem_u32(uv_empty + s));                 // stage reusable when these MMAs are done
        if (++ci == cpt) {
          tc_commit(smem_u32(acc_full));                   // tile finished
          ci = 0;
          ++seq;
          if (seq < my_tiles) dup = tile_repeats_filters<DT>(p, decode_tile(p, (int)blockIdx.x + seq * (int)gridDim.x));
        }
      }
      // Tensor memory is freed at the end of the kernel: every MMA this thread issued must have
      // completed by then, also after a give-up (then nobody waited for acc_full).
      tc_commit(smem_u32(mma_done + me));
      mbar_wait_drain(smem_u32(mma_done + me), 0);
    }
  } else {
    // ===================================== epilogue ============================================
    const int quarter = warp & 3;                                        // TMEM lanes this warp may read
    const int sub = (warp - kTcFirstEpilogueWarp) >> 2;                  // 0 / 1: the two warps of a lane quarter
    const size_t plane = (size_t)p.H * p.W * p.N;
    const size_t dW = (size_t)p.N, dH = (size_t)p.W * p.N;
    for (int seq = 0; seq < my_tiles; ++seq) {
      const TileCoord tc = decode_tile(p, (int)blockIdx.x + seq * (int)gridDim.x);
      mbar_wait(smem_u32(acc_full), seq & 1, dead, p.status);
      tc_fence_after();
      // Usually the quarter's lanes are filters 32*quarter .. +31 and the two warps of a quarter split the 32
      // images 16 / 16 (two steps of 8).  With repeated filters, quarters 2 and 3 hold filters 0-63 again, so
      // the eight warps split the images 8 each (one step).
      const bool dup = tile_repeats_filters<DT>(p, tc);
      const int fq = dup ? (quarter & 1) : quarter;                      // filter block of 32 this warp stores
      const int m = fq * 32 + lane;                                      // filter within the tile
      const int k = tc.kb * kTcM + m;
      const bool valid = k < p.K;
      const int oh0 = 2 * tc.ty, ow0 = 2 * tc.tx;
      const bool row1 = (oh0 + 1) < p.H, col1 = (ow0 + 1) < p.W;
      float *ybase = p.y + (size_t)k * plane + ((size_t)oh0 * p.W + ow0) * p.N + (size_t)tc.nb * kTcN;
      const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
      // Warps whose 32 filters all lie beyond K (K = 64 layers) have nothing to read or store.
      const bool warp_valid = (tc.kb * kTcM + fq * 32) < p.K;
      // this warp's share of the 32 images: image quads jbase .. jbase + nq - 1
      const int nq = dup ? 2 : 4;
      const int jbase = dup ? 2 * (2 * (quarter >> 1) + sub) : 4 * sub;
      // Y = A^T M A column by column of the 4x4 positions: column j (positions j, 4+j, 8+j, 12+j) gives the two
      // row sums a[j], a[4+j] of output_transform, which are folded into the four outputs at once - the same
      // operations in the same order.  After a column has been read it is handed back (acc_empty[j]), so the
      // MMAs of the next tile into those four accumulators overlap the rest of this epilogue.
      float y[4][4][4];                         // [image quad][output position][image]
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (warp_valid && 2 * h < nq) {
            float mm[2][4][4];                  // [quad of this half][row][image]
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
              for (int r = 0; r < 4; ++r) tmem_ld_x4(tlane + (4 * r + j) * kTcN + 4 * (jbase + 2 * h + q2), mm[q2][r]);
            tmem_ld_wait();
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = __fadd_rn(__fadd_rn(mm[q2][0][e], mm[q2][1][e]), mm[q2][2][e]);
                const float hi = __fsub_rn(__fsub_rn(mm[q2][1][e], mm[q2][2][e]), mm[q2][3][e]);
                float(&yy)[4][4] = y[2 * h + q2];
                if (j == 0) { yy[0][e] = lo; yy[2][e] = hi; }
                if (j == 1) { yy[0][e] = __fadd_rn(yy[0][e], lo); yy[1][e] = lo; yy[2][e] = __fadd_rn(yy[2][e], hi); yy[3][e] = hi; }
                if (j == 2) { yy[0][e] = __fadd_rn(yy[0][e], lo); yy[1][e] = __fsub_rn(yy[1][e], lo);
                              yy[2][e] = __fadd_rn(yy[2][e], hi); yy[3][e] = __fsub_rn(yy[3][e], hi); }
                if (j == 3) { yy[1][e] = __fsub_rn(yy[1][e], lo); yy[3][e] = __fsub_rn(yy[3][e], hi); }
              }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(acc_empty + j));
      }
      // Stores.  Lanes are filters, i.e. different output rows, so a warp-wide store touches 32 lines however it
      // is arranged; what can be halved is the number of lines per byte.  A lane holds 16 consecutive images
      // (64 bytes) of its filter per output position: neighbouring lanes swap halves, so that one instruction
      // writes the 64 bytes of the pair's even filter (32 bytes per lane) and the next those of the odd filter -
      // 16 lines of two full sectors per instruction instead of 32 lines of one.  (Measured on the 56x56 layer:
      // 7 % of the kernel; the memory pipe is shared with the transform warps' shared-memory traffic.)
      if (warp_valid) {
        if (nq == 4) {
          const bool odd = (lane & 1) != 0;
          float *pair_base = ybase - (odd ? plane : 0) + 16 * sub + (odd ? 8 : 0);   // even filter of the pair, this lane's half
          const bool n_ok = tc.nb * kTcN + 16 * sub + (odd ? 8 : 0) < p.N;         // N is a multiple of 8
          const bool ok_even = n_ok && (k - (odd ? 1 : 0)) < p.K, ok_odd = n_ok && (k + (odd ? 0 : 1)) < p.K;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float ev[2][4], od[2][4];           // this lane's half of the even / odd filter's 64 bytes
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = y[q2][q][e], hi = y[2 + q2][q][e];              // images 0-7 / 8-15 of this lane's filter
                const float got = __shfl_xor_sync(0xFFFFFFFFu, odd ? lo : hi, 1);
                ev[q2][e] = odd ? got : lo;
                od[q2][e] = odd ? hi : got;
              }
            const bool here = (q == 0) || (q == 1 && col1) || (q == 2 && row1) || (q == 3 && row1 && col1);
            float *dst = pair_base + ((q & 1) ? dW : 0) + ((q & 2) ? dH : 0);
            if (here && ok_even) st_global_v8(dst, ev[0], ev[1]);
            if (here && ok_odd) st_global_v8(dst + plane, od[0], od[1]);
          }
        } else if (valid && tc.nb * kTcN + 4 * jbase < p.N) {
          // eight images per lane (repeated-filter tiles): one full 32-byte sector per lane and store
          float *dst = ybase + 4 * jbase;
          st_global_v8(dst, y[0][0], y[1][0]);
          if (col1) st_global_v8(dst + dW, y[0][1], y[1][1]);
          if (row1) {
            st_global_v8(dst + dH, y[0][2], y[1][2]);
            if (col1) st_global_v8(dst + dH + dW, y[0][3], y[1][3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTcMmaWarp) {
    tc_fence_after();
    tmem_dealloc_512(tmem_base);
  }
}

}  // namespace ocb
