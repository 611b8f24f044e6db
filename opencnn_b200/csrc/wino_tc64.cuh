// Tensor-core Winograd kernel for layers with at most 64 filters (BF16 or TF32 operands): two
// 32-image blocks share the 128 accumulator rows of one CTA.
//
// Same operator as wino_tc.cuh (it replaces the reference's Winograd_kernel,
// src/convolutionForward_32x64x8.cu:169-262, with the contraction on the tensor cores; the reference
// has no tensor-core path).  There, a tile is 128 filters x 32 images because the 16 accumulators
// of 128 rows x 32 columns fill tensor memory; with 64 filters half of the rows would idle (the
// single-CTA kernel lets them repeat the other half).  Here rows 0-63 hold the 64 filters for
// image block 0 and rows 64-127 the same 64 filters for image block 1 of a 64-image tile:
//     D[xi] (128 x 32)  +=  [U ; 0] (128 x 16c) * V_block0 (16c x 32)      first MMA of a K-step
//     D[xi] (128 x 32)  +=  [0 ; U] (128 x 16c) * V_block1 (16c x 32)      second MMA
// The zero halves are not stored per position: the A operand of an MMA is two blocks of 64 filter
// rows whose distance is a free field of the shared-memory descriptor (the leading-dimension byte
// offset), so [U ; 0] is "first block at U, second block at a 2 KB region of zeros above all U
// stages" and [0 ; U] is "first block at a region of zeros below them, second block at U".
// What it buys: one filter slice (32 KB per K-step) now serves 64 images instead of 32, and the
// per-tile costs - the accumulator hand-over, the epilogue, the pipeline restart, which dominate
// layers with few channels - are paid once per 64 images, with all 128 TMEM lanes doing useful
// work in the epilogue.  The tensor pipe does twice the MMAs per image, which it has room for.
//
// TF32: the A operand of an MMA is four blocks of 32 filter rows at one fixed distance, which is the
// distance of U's own two blocks (1 KB), so the zero half has to lie right behind (resp. before)
// them.  It does: the filter slice is loaded as a box of 128 filters of which only 64 exist, and TMA
// fills the other half of every position (2 KB) with zeros.  [U ; 0] starts at a position's U,
// [0 ; U] 2 KB earlier, in the zero half of the position before (position 0 of the first stage
// has a region of zeros of its own below it; position 0 of the second stage finds the zero half of
// the first stage's last position there, which every reload rewrites with the same zeros).
//
// The pipeline runs in sub-steps: (K-step, image block).  Raw patches and V have rings of three
// sub-steps, U a ring of two K-steps.  Warp roles as in wino_tc.cuh (512 threads): warp 0 loads
// raw patches, warp 14 loads U, warps 1-4 transform, warps 5 and 15 issue the MMAs of eight
// positions each, warps 6-13 are the epilogue (quarters 0,1 store image block 0, quarters 2,3
// image block 1).  All hand-offs are mbarriers with bounded waits.
#pragma once
#include "wino_tc2.cuh"   // P2Tile / p2_decode (tiles over pairs of image blocks), wino_tc.cuh

namespace ocb {

constexpr int kT64RawStages = 3, kT64UStages = 2, kT64VStages = 3;
constexpr uint32_t kT64ZeroBytes = 2048;                   // one empty half of an A operand (64 filter rows x one K-step)
constexpr int kT64Threads = 512;
template <int DT> struct T64Cfg {
  static constexpr int kKC = DT == kTcBf16 ? 16 : 8;                       // channels per K-step
  static constexpr uint32_t kRawBytes = kKC * 16 * kTcN * 4;               // [c][4 h][4 w][32 n] fp32: one image block, one K-step
  static constexpr uint32_t kUPosBytes = DT == kTcBf16 ? 2048 : 4096;      // one position of a U stage (TF32: half of it zeros)
  static constexpr uint32_t kUBytes = 16 * kUPosBytes;
  // BF16 keeps a second region of zeros above the rings ([U ; 0]); TF32 needs only the one below the U ring.
  static constexpr size_t kSmemBytes = (DT == kTcBf16 ? 2 : 1) * kT64ZeroBytes + (size_t)kT64RawStages * kRawBytes +
                                       (size_t)kT64UStages * kUBytes + (size_t)kT64VStages * kTcVBytes + 512;
  static_assert(kSmemBytes <= 232448, "shared memory");
};

// p.n_blocks counts 32-image blocks; p.total_tiles counts 64-image tiles; p.k_blocks is 1.
template <int DT>
__global__ void __launch_bounds__(kT64Threads, 1)
wino_tc64_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_u, const WinoParams p) {
  using Cfg = T64Cfg<DT>;
  constexpr int SR = kT64RawStages, SU = kT64UStages, SV = kT64VStages;
  constexpr int KC = Cfg::kKC;
  constexpr uint32_t kT64RawBytes = Cfg::kRawBytes, kT64UBytes = Cfg::kUBytes;
  extern __shared__ __align__(1024) uint8_t tsmem64[];
  uint8_t *raw_s = tsmem64;
  uint8_t *zero_lo = raw_s + SR * kT64RawBytes;                        // directly below the U ring
  uint8_t *u_s = zero_lo + kT64ZeroBytes;
  uint8_t *v_s = u_s + SU * kT64UBytes;
  uint8_t *zero_hi = v_s + SV * kTcVBytes;                             // above every U stage (BF16 only)
  uint64_t *bars = reinterpret_cast<uint64_t *>(zero_hi + (DT == kTcBf16 ? kT64ZeroBytes : 0));
  uint64_t *raw_full = bars, *raw_empty = raw_full + SR, *u_full = raw_empty + SR, *u_empty = u_full + SU,
           *v_ready = u_empty + SU, *v_empty = v_ready + SV;
  uint64_t *acc_full = v_empty + SV, *mma_done = acc_full + 2;   // mma_done[2]
  uint64_t *acc_empty = acc_full + 6;                  // [4]: one per column of the 4x4 positions
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 4);
  volatile int *dead = reinterpret_cast<volatile int *>(acc_full + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_pairs = (p.n_blocks + 1) / 2;
  const int my_tiles = (p.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int cpt = p.chunks_per_tile;                                   // K-steps per tile
  const int total_steps = my_tiles * cpt;                              // K-steps of this CTA
  const int total_sub = 2 * total_steps;                               // sub-steps: (K-step, image block)

  // the two regions of zeros that stand in for the empty half of the A operand
  for (int i = tid; i < (int)(kT64ZeroBytes / 4); i += kT64Threads) {
    reinterpret_cast<uint32_t *>(zero_lo)[i] = 0u;
    if (DT == kTcBf16) reinterpret_cast<uint32_t *>(zero_hi)[i] = 0u;
  }
  fence_proxy_async_smem();                                            // read by the tensor core through the async proxy
  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < SR; ++s) {
      mbar_init(smem_u32(raw_full + s), 1);
      mbar_init(smem_u32(raw_empty + s), kTcTransformWarps);
    }
    for (int s = 0; s < SU; ++s) {
      mbar_init(smem_u32(u_full + s), 1);
      mbar_init(smem_u32(u_empty + s), 2);                             // one tcgen05.commit per MMA-issuing thread
    }
    for (int s = 0; s < SV; ++s) {
      mbar_init(smem_u32(v_ready + s), kTcTransformWarps);
      mbar_init(smem_u32(v_empty + s), 2);
    }
    mbar_init(smem_u32(acc_full), 2);
    for (int j = 0; j < 4; ++j) mbar_init(smem_u32(acc_empty + j), kTcEpilogueWarps);
    mbar_init(smem_u32(mma_done + 0), 1);
    mbar_init(smem_u32(mma_done + 1), 1);
    mbar_fence_init();
  }
  if (warp == kTcMmaWarp) tmem_alloc_512(smem_u32(tmem_slot));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == kTcULoaderWarp) {
    // ===================================== TMA loaders =========================================
    const bool loads_u = warp != 0;
    if (lane == 0) {
      tma_prefetch_descriptor(loads_u ? &tm_u : &tm_in);
      int seq = 0, ci = 0, issued = 0;
      P2Tile tc = p2_decode(p, (int)blockIdx.x, n_pairs);
      const int ring = loads_u ? SU : SR;
      const int count = loads_u ? total_steps : total_sub;             // U once per K-step, patches once per sub-step
      for (int g = 0; g < count; ++g) {
        const int s = g % ring;
        const uint32_t use = g / ring;
        // A wait that gave up: stop issuing - the stage may still be in use.
        if (use > 0 && !mbar_wait(smem_u32((loads_u ? u_empty : raw_empty) + s), (use - 1) & 1, dead, p.status)) break;
        if (loads_u) {
          mbar_arrive_expect_tx(smem_u32(u_full + s), kT64UBytes);
          tma_load_4d(smem_u32(u_s + s * kT64UBytes), &tm_u, smem_u32(u_full + s), 0, ci * KC, 0, 0);
        } else {
          const int b = g & 1;
          mbar_arrive_expect_tx(smem_u32(raw_full + s), kT64RawBytes);
          tma_load_4d(smem_u32(raw_s + s * kT64RawBytes), &tm_in, smem_u32(raw_full + s), (2 * tc.np + b) * kTcN,
                      2 * tc.tx - 1, 2 * tc.ty - 1, ci * KC);
        }
        issued = g + 1;
        if (loads_u || (g & 1)) {                                      // next K-step
          if (++ci == cpt) {
            ci = 0;
            ++seq;
            if (seq < my_tiles) tc = p2_decode(p, (int)blockIdx.x + seq * (int)gridDim.x, n_pairs);
          }
        }
      }
      // No exit with bulk copies in flight (after a complete run these phases are long over).
      for (int g = issued > ring ? issued - ring : 0; g < issued; ++g)
        mbar_wait_drain(smem_u32((loads_u ? u_full : raw_full) + g % ring), (g / ring) & 1);
    }
  } else if (warp <= kTcTransformWarps) {
    // ===================================== input transform =====================================
    const int t = tid - 32;                                            // 0..127: channel t >> 4 (BF16: and + 8), image pair t & 15
    for (int g = 0; g < total_sub; ++g) {
      const int sv = g % SV, sr = g % SR;
      const uint32_t use = g / SV;
      mbar_wait(smem_u32(raw_full + sr), (g / SR) & 1, dead, p.status);
      if (use > 0) mbar_wait(smem_u32(v_empty + sv), (use - 1) & 1, dead, p.status);   // V stage free again
      if (DT == kTcBf16)
        transform_to_v_bf16_x2(reinterpret_cast<const float *>(raw_s + sr * kT64RawBytes), v_s + sv * kTcVBytes, t >> 4, t & 15);
      else
        transform_to_v_tf32_pair(reinterpret_cast<const float *>(raw_s + sr * kT64RawBytes), v_s + sv * kTcVBytes, t >> 4, t & 15);
      fence_proxy_async_smem();          // V is read by the tensor core through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(raw_empty + sr));
        mbar_arrive(smem_u32(v_ready + sv));
      }
    }
  } else if (warp == kTcMmaWarp || warp == kTcMmaWarpB) {
    // ===================================== MMA issuers (two threads, two position columns each) ==
    if (lane == 0) {
      const int me = warp == kTcMmaWarp ? 0 : 1;
      const int col0 = 2 * me;                         // columns col0, col0 + 1 of the 4x4 positions, column by column
      const uint32_t idesc = instr_desc<DT>();
      // BF16.  A blocks: 64 filters x 16 channels, filter-contiguous rows of 128 B (128-byte swizzle), 8-channel
      // groups 1 KB apart; the second block lies `lbo` bytes after the first.  Per position the U block moves by
      // 2 KB, so
      //   [U ; 0]: start at U, second block at zero_hi  -> start + 2 KB, lbo - 2 KB per position
      //   [0 ; U]: start at zero_lo, second block at U  -> lbo + 2 KB per position
      // B: 32 images x 16 channels per position, rows of 64 B (64-byte swizzle), 8-channel groups 512 B apart.
      // TF32.  A blocks: 32 filters x 8 channels, rows of 128 B (128-byte swizzle with 32-byte atoms), 4-channel
      // groups 512 B apart, four blocks 1 KB apart: U, U, zeros, zeros from a position's start, and the other way
      // round from 2 KB earlier; 4 KB per position either way.  B: rows of 128 B, blocks 1 KB apart.
      const uint32_t u0 = smem_u32(u_s);
      const uint64_t a_top0 = DT == kTcBf16 ? smem_desc(u0, smem_u32(zero_hi) - u0, 1024, 2) : smem_desc(u0, 1024, 512, 1);
      const uint64_t a_bot0 = DT == kTcBf16 ? smem_desc(smem_u32(zero_lo), u0 - smem_u32(zero_lo), 1024, 2)
                                            : smem_desc(u0 - kT64ZeroBytes, 1024, 512, 1);
      constexpr uint64_t kPosStart = Cfg::kUPosBytes >> 4, kPosLbo = (uint64_t)(2048 >> 4) << 16;
      constexpr uint64_t kStageStart = kT64UBytes >> 4, kStageLbo = (uint64_t)(kT64UBytes >> 4) << 16;
      // what a position / a stage adds to the descriptor of [U ; 0] and of [0 ; U]
      constexpr uint64_t kTopPos = DT == kTcBf16 ? kPosStart - kPosLbo : kPosStart, kBotPos = DT == kTcBf16 ? kPosLbo : kPosStart;
      constexpr uint64_t kTopStage = DT == kTcBf16 ? kStageStart - kStageLbo : kStageStart, kBotStage = DT == kTcBf16 ? kStageLbo : kStageStart;
      const uint64_t b_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(v_s), 512, 512, 4) : smem_desc(smem_u32(v_s), 1024, 512, 1);
      int ci = 0, seq = 0;
      for (int g = 0; g < total_sub; ++g) {
        const int b = g & 1, su = (g >> 1) % SU, sv = g % SV;
        // A wait that gave up: stop issuing (the operands or the accumulators are not ready).
        if (b == 0 && !mbar_wait(smem_u32(u_full + su), ((g >> 1) / SU) & 1, dead, p.status)) break;
        if (!mbar_wait(smem_u32(v_ready + sv), (g / SV) & 1, dead, p.status)) break;
        tc_fence_after();
        const uint64_t astep = b == 0 ? kTopPos : kBotPos;
        const uint64_t ad = (b == 0 ? a_top0 + (uint64_t)su * kTopStage : a_bot0 + (uint64_t)su * kBotStage) + (uint64_t)col0 * astep;
        const uint64_t bd = b_desc0 + (uint64_t)(sv * (kTcVBytes >> 4)) + (uint64_t)(col0 * (1024 >> 4));
        const uint32_t accumulate = (ci > 0 || b > 0) ? 1u : 0u, d0 = tmem_base + col0 * kTcN;
        bool ok = true;
#pragma unroll
        for (int xo = 0; xo < 8; ++xo) {
          const int xr = 4 * (xo & 3) + (xo >> 2);     // position relative to col0: row xo & 3, column xo >> 2
          if ((xo & 3) == 0 && b == 0 && ci == 0 && seq > 0) {   // first write to a column of a new tile: drained?
            if (!mbar_wait(smem_u32(acc_empty + col0 + (xo >> 2)), (seq - 1) & 1, dead, p.status)) { ok = false; break; }
            tc_fence_after();
          }
          tc_mma<DT>(d0 + xr * kTcN, ad + (uint64_t)xr * astep, bd + (uint64_t)(xr * (1024 >> 4)), idesc, accumulate);
        }
        if (!ok) break;
        tc_commit(smem_u32(v_empty + sv));                 // V stage reusable when these MMAs are done
        if (b == 1) {
          tc_commit(smem_u32(u_empty + su));               // and the filter slice after the second image block
          if (++ci == cpt) {
            tc_commit(smem_u32(acc_full));                 // tile finished
            ci = 0;
            ++seq;
          }
        }
      }
      // Tensor memory is freed at the end of the kernel: every MMA this thread issued must have completed by then.
      tc_commit(smem_u32(mma_done + me));
      mbar_wait_drain(smem_u32(mma_done + me), 0);
    }
  } else {
    // ===================================== epilogue ============================================
    const int quarter = warp & 3;                                        // TMEM lanes this warp may read
    const int sub = (warp - kTcFirstEpilogueWarp) >> 2;                  // 0 / 1: which 16 of the block's 32 images
    const int fq = quarter & 1, ib = quarter >> 1;                       // filters 32*fq .. +31 of image block ib
    const int k = fq * 32 + lane;
    const bool warp_valid = fq * 32 < p.K;
    const size_t plane = (size_t)p.H * p.W * p.N;
    const size_t dW = (size_t)p.N, dH = (size_t)p.W * p.N;
    const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    for (int seq = 0; seq < my_tiles; ++seq) {
      const P2Tile tc = p2_decode(p, (int)blockIdx.x + seq * (int)gridDim.x, n_pairs);
      mbar_wait(smem_u32(acc_full), seq & 1, dead, p.status);
      tc_fence_after();
      const int nb = 2 * tc.np + ib;                                     // 32-image block this warp stores
      const int oh0 = 2 * tc.ty, ow0 = 2 * tc.tx;
      const bool row1 = (oh0 + 1) < p.H, col1 = (ow0 + 1) < p.W;
      float *ybase = p.y + (size_t)k * plane + ((size_t)oh0 * p.W + ow0) * p.N + (size_t)nb * kTcN + 16 * sub;
      const bool active = warp_valid && nb < p.n_blocks;
      // Y = A^T M A column by column of the 4x4 positions: column j (positions j, 4+j, 8+j, 12+j) gives the two
      // row sums a[j], a[4+j] of output_transform, which are folded into the four outputs at once - the same
      // operations in the same order.  After a column has been read it is handed back (acc_empty[j]), so the
      // MMAs of the next tile into those four accumulators overlap the rest of this epilogue.
      float y[4][4][4];                                                  // [image quad][output position][image]
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (active) {
            float mm[2][4][4];                                           // [quad of this half][row][image]
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
              for (int r = 0; r < 4; ++r) tmem_ld_x4(tlane + (4 * r + j) * kTcN + 16 * sub + 8 * h + 4 * q2, mm[q2][r]);
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
      // Stores: neighbouring lanes (filters) swap halves of their 16 images, so that one instruction writes the
      // 64 bytes of the pair's even filter (32 bytes per lane) and the next those of the odd filter - 16 lines of
      // two full sectors per instruction instead of 32 lines of one (see wino_tc_kernel).
      if (active) {
        const bool odd = (lane & 1) != 0;
        float *pair_base = ybase - (odd ? plane : 0) + (odd ? 8 : 0);           // even filter of the pair, this lane's half
        const bool n_ok = nb * kTcN + 16 * sub + (odd ? 8 : 0) < p.N;            // N is a multiple of 8
        const bool ok_even = n_ok && (k - (odd ? 1 : 0)) < p.K, ok_odd = n_ok && (k + (odd ? 0 : 1)) < p.K;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float ev[2][4], od[2][4];             // this lane's half of the even / odd filter's 64 bytes
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = y[q2][q][e], hi = y[2 + q2][q][e];                // images 0-7 / 8-15 of this lane's filter
              const float got = __shfl_xor_sync(0xFFFFFFFFu, odd ? lo : hi, 1);
              ev[q2][e] = odd ? got : lo;
              od[q2][e] = odd ? hi : got;
            }
          const bool here = (q == 0) || (q == 1 && col1) || (q == 2 && row1) || (q == 3 && row1 && col1);
          float *dst = pair_base + ((q & 1) ? dW : 0) + ((q & 2) ? dH : 0);
          if (here && ok_even) st_global_v8(dst, ev[0], ev[1]);
          if (here && ok_odd) st_global_v8(dst + plane, od[0], od[1]);
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
