// Tensor-core Winograd kernel, second generation: a pair of CTAs (thread-block cluster of 2) shares
// one tile of 128 filters x 64 images and splits the 16 Winograd positions, 8 each.
//
// Why: tensor memory holds 512 accumulator columns per SM.  With all 16 positions in one CTA that
// is 32 images per MMA (wino_tc.cuh), and an MMA with N <= 64 occupies the tensor pipe ~54 cycles
// whatever N is, while every K-step re-reads a 64 KB filter slice from L2 for just 32 images.
// With 8 positions per CTA the same 512 columns hold 64 images: half as many MMAs per image,
// each twice as wide, and a 32 KB filter slice serves twice the images - the L2 traffic per
// multiply-accumulate halves.  The reference has no counterpart (no tensor-core path at all).
//
// The two CTAs of a pair run their main loops independently - each loads and transforms the raw
// patches of all 64 images itself and keeps only its 8 positions (rows 2*rank, 2*rank+1 of the
// 4x4 transform), so there is no cross-CTA traffic per K-step.  Rows 0,1 of B^T d B need only
// patch rows 0..2 and rows 2,3 only patch rows 1..3, so each CTA loads three of the four rows.  They meet only in the epilogue:
// the output transform is linear in the 16 positions, so each CTA forms the partial result of its
// 8 positions; CTA r stores its partial for image block r, signals the peer through an mbarrier in
// the peer's shared memory, and for the other image block adds its partial onto what the peer
// stored with a vector reduction at L2 (red.global.add.v4.f32; two addends, so deterministic).  Both CTAs leave through a cluster
// barrier so that neither exits while the other may still signal it.
#pragma once
#include "wino_tc.cuh"

namespace ocb {

constexpr int kP2N = 64;                         // images per pair tile
constexpr int kP2TransformWarps = 8;
constexpr int kP2EpilogueWarps = 8;
constexpr int kP2MmaWarp = 1 + kP2TransformWarps;
constexpr int kP2FirstEpilogueWarp = kP2MmaWarp + 1;
constexpr int kP2ULoaderWarp = kP2FirstEpilogueWarp + kP2EpilogueWarps;
constexpr int kP2MmaWarpB = kP2ULoaderWarp + 1;   // second MMA-issuing thread (positions 4-7 of the CTA's eight)
constexpr int kP2Threads = (kP2MmaWarpB + 1) * 32;
constexpr uint32_t kP2UBytes = 8 * 4096;         // 8 positions x (128 filters x one K-step)
constexpr uint32_t kP2VBytes = 8 * 2048;         // 8 positions x (64 images x one K-step)

template <int DT> struct P2Cfg {
  static constexpr int kKC = DT == kTcBf16 ? 16 : 8;
  static constexpr uint32_t kRawBytes = kKC * 12 * kP2N * 4;          // [c][3 h][4 w][64 n] fp32
  // ring depth: what fits in 227 KB (BF16 stages are 96 KB, TF32 stages 72 KB)
  static constexpr int kStages = DT == kTcBf16 ? 2 : 3;
  static constexpr size_t kSmemBytes = (size_t)kStages * (kRawBytes + kP2UBytes + kP2VBytes) + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// Arrive (release, cluster scope) on the mbarrier at the same shared-memory offset in CTA `rank`.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(local_bar), "r"(rank) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
__device__ __forceinline__ void red_global_add_v4(float *p, const float (&a)[4]) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a[0]), "f"(a[1]), "f"(a[2]), "f"(a[3]) : "memory");
}

// ---- input transform, only the 8 positions of transform rows 2*RANK and 2*RANK+1 ---------------
// BF16: item = (channel c, image pair np of 32); V tile of a position is [16 c][64 n] bf16, rows of
// 128 bytes, 128-byte swizzle.
template <int RANK>
__device__ __forceinline__ void p2_finish_bf16(const uint64_t (&d)[12], uint8_t *__restrict__ vst, int c, int np) {
  uint64_t b[8];                             // transform rows 2*RANK, 2*RANK+1 (d: patch rows RANK..RANK+2)
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (RANK == 0) {
      b[j] = sub2(d[j], d[8 + j]);           // row 0 = d0 - d2
      b[4 + j] = add2(d[4 + j], d[8 + j]);   // row 1 = d1 + d2
    } else {
      b[j] = sub2(d[4 + j], d[j]);           // row 2 = d2 - d1
      b[4 + j] = sub2(d[j], d[8 + j]);       // row 3 = d1 - d3
    }
  }
  uint8_t *dst = vst + c * 128 + ((((np >> 2) ^ c) & 7) << 4) + ((np & 3) << 2);
#pragma unroll
  for (int ii = 0; ii < 2; ++ii) {
    uint64_t o[4];
    o[0] = sub2(b[4 * ii + 0], b[4 * ii + 2]);
    o[1] = add2(b[4 * ii + 1], b[4 * ii + 2]);
    o[2] = sub2(b[4 * ii + 2], b[4 * ii + 1]);
    o[3] = sub2(b[4 * ii + 1], b[4 * ii + 3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float lo, hi;
      unpack2(o[j], lo, hi);
      *reinterpret_cast<uint32_t *>(dst + (4 * ii + j) * 2048) = pack_bf16x2(lo, hi);
    }
  }
}
// Two items (channels c and c + 8 of image pair np) at once: all loads are issued before any
// arithmetic, so the two shared-memory round trips overlap.
template <int RANK>
__device__ __forceinline__ void p2_transform_bf16_x2(const float *__restrict__ raw, uint8_t *__restrict__ vst, int c, int np) {
  const uint64_t *R0 = reinterpret_cast<const uint64_t *>(raw + (c * 12) * kP2N + 2 * np), *R1 = R0 + 8 * 12 * (kP2N / 2);
  constexpr int P = kP2N / 2;
  uint64_t d0[12], d1[12];
#pragma unroll
  for (int q = 0; q < 12; ++q) { d0[q] = R0[q * P]; d1[q] = R1[q * P]; }
  p2_finish_bf16<RANK>(d0, vst, c, np);
  p2_finish_bf16<RANK>(d1, vst, c + 8, np);
}
// TF32: one item = (channel c, image pair np of 32); V tile of a position is [2 image blocks][8 c][32 n]
// fp32, rows of 128 bytes, 128-byte swizzle with 32-byte atoms; the two images of a pair are adjacent
// in a V row, so each result is one 8-byte store.
template <int RANK>
__device__ __forceinline__ void p2_transform_tf32_pair(const float *__restrict__ raw, uint8_t *__restrict__ vst, int c, int np) {
  const uint64_t *R = reinterpret_cast<const uint64_t *>(raw + (c * 12) * kP2N + 2 * np);
  constexpr int P = kP2N / 2;
  uint64_t d[12], b[8];
#pragma unroll
  for (int q = 0; q < 12; ++q) d[q] = R[q * P];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (RANK == 0) {
      b[j] = sub2(d[j], d[8 + j]);
      b[4 + j] = add2(d[4 + j], d[8 + j]);
    } else {
      b[j] = sub2(d[4 + j], d[j]);
      b[4 + j] = sub2(d[j], d[8 + j]);
    }
  }
  const int n = 2 * np, nl = n & 31;
  uint8_t *dst = vst + (n >> 5) * 1024 + c * 128 + ((((nl >> 3) ^ c) & 3) << 5) + ((nl & 7) << 2);
#pragma unroll
  for (int ii = 0; ii < 2; ++ii) {
    uint64_t o[4];
    o[0] = sub2(b[4 * ii + 0], b[4 * ii + 2]);
    o[1] = add2(b[4 * ii + 1], b[4 * ii + 2]);
    o[2] = sub2(b[4 * ii + 2], b[4 * ii + 1]);
    o[3] = sub2(b[4 * ii + 1], b[4 * ii + 3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float lo, hi;
      unpack2(o[j], lo, hi);
      *reinterpret_cast<float2 *>(dst + (4 * ii + j) * 2048) = make_float2(round_tf32_rne(lo), round_tf32_rne(hi));
    }
  }
}
// Partial output transform of one (filter, image) from the 8 positions of rows 2*RANK, 2*RANK+1:
// m[0..3] = row 2*RANK, m[4..7] = row 2*RANK+1.  The sum of the two ranks' results is A^T M A.
template <int RANK>
__device__ __forceinline__ void p2_partial_output(const float (&m)[8], float (&y)[4]) {
  float a0[4], a1[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (RANK == 0) { a0[j] = m[j] + m[4 + j]; a1[j] = m[4 + j]; }           // rows 0,1:  m0+m1 | m1
    else           { a0[j] = m[j];            a1[j] = -m[j] - m[4 + j]; }    // rows 2,3:  m2    | -m2-m3
  }
  y[0] = a0[0] + a0[1] + a0[2];
  y[1] = a0[1] - a0[2] - a0[3];
  y[2] = a1[0] + a1[1] + a1[2];
  y[3] = a1[1] - a1[2] - a1[3];
}

struct P2Tile { int np, tx, ty, kb; };
__device__ __forceinline__ P2Tile p2_decode(const WinoParams &p, int t, int n_pairs) {
  P2Tile tc;
  tc.np = t % n_pairs; t /= n_pairs;
  tc.tx = t % p.tiles_w; t /= p.tiles_w;
  tc.ty = t % p.tiles_h;
  tc.kb = t / p.tiles_h;
  return tc;
}

// p.n_blocks counts 32-image blocks, p.k_blocks 128-filter blocks; p.total_tiles counts pair tiles.
template <int DT, int RANK>
__device__ __forceinline__ void p2_body(const CUtensorMap &tm_in, const CUtensorMap &tm_u, const WinoParams &p,
                                        uint8_t *tsmem) {
  using Cfg = P2Cfg<DT>;
  constexpr int KC = Cfg::kKC;
  constexpr int S = Cfg::kStages;
  uint8_t *raw_s = tsmem;
  uint8_t *u_s = raw_s + S * Cfg::kRawBytes;
  uint8_t *v_s = u_s + S * kP2UBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_s + S * kP2VBytes);
  uint64_t *raw_full = bars, *raw_empty = bars + S, *u_full = bars + 2 * S, *v_ready = bars + 3 * S, *uv_empty = bars + 4 * S;
  uint64_t *acc_full = bars + 5 * S, *acc_empty = acc_full + 1, *peer_ready = acc_full + 2;   // peer_ready[2], used alternately
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 4);
  volatile int *dead = reinterpret_cast<volatile int *>(acc_full + 5);
  uint64_t *mma_done = acc_full + 6;                   // one per MMA-issuing thread: "all my MMAs have completed"

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_clusters = (int)gridDim.x / 2, cid = (int)blockIdx.x / 2;
  const int n_pairs = (p.n_blocks + 1) / 2;
  const int my_tiles = (p.total_tiles - cid + n_clusters - 1) / n_clusters;
  const int cpt = p.chunks_per_tile;
  const int total_chunks = my_tiles * cpt;

  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(raw_full + s), 1);
      mbar_init(smem_u32(raw_empty + s), kP2TransformWarps);
      mbar_init(smem_u32(u_full + s), 1);
      mbar_init(smem_u32(v_ready + s), kP2TransformWarps);
      mbar_init(smem_u32(uv_empty + s), 2);      // one tcgen05.commit per MMA-issuing thread
    }
    mbar_init(smem_u32(peer_ready + 0), kP2EpilogueWarps);
    mbar_init(smem_u32(peer_ready + 1), kP2EpilogueWarps);
    mbar_init(smem_u32(acc_full), 2);
    mbar_init(smem_u32(acc_empty), kP2EpilogueWarps);
    mbar_init(smem_u32(mma_done + 0), 1);
    mbar_init(smem_u32(mma_done + 1), 1);
    mbar_fence_init();
  }
  if (warp == kP2MmaWarp) tmem_alloc_512(smem_u32(tmem_slot));
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == kP2ULoaderWarp) {
    // ===================================== TMA loaders =========================================
    const bool loads_u = warp != 0;
    if (lane == 0) {
      tma_prefetch_descriptor(loads_u ? &tm_u : &tm_in);
      int seq = 0, ci = 0, issued = 0;
      P2Tile tc = p2_decode(p, cid, n_pairs);
      for (int g = 0; g < total_chunks; ++g) {
        const int s = g % S;
        const uint32_t use = g / S;
        // A wait that gave up: stop issuing - the stage may still be in use.
        if (!loads_u) {
          if (use > 0 && !mbar_wait(smem_u32(raw_empty + s), (use - 1) & 1, dead, p.status)) break;
          mbar_arrive_expect_tx(smem_u32(raw_full + s), Cfg::kRawBytes);
          tma_load_4d(smem_u32(raw_s + s * Cfg::kRawBytes), &tm_in, smem_u32(raw_full + s), tc.np * kP2N, 2 * tc.tx - 1,
                      2 * tc.ty - 1 + RANK, ci * KC);           // patch rows RANK .. RANK+2
        } else {
          if (use > 0 && !mbar_wait(smem_u32(uv_empty + s), (use - 1) & 1, dead, p.status)) break;
          mbar_arrive_expect_tx(smem_u32(u_full + s), kP2UBytes);
          tma_load_4d(smem_u32(u_s + s * kP2UBytes), &tm_u, smem_u32(u_full + s), 0, ci * KC,
                      tc.kb * (DT == kTcBf16 ? 2 : 4), 8 * RANK);
        }
        issued = g + 1;
        if (++ci == cpt) {
          ci = 0;
          ++seq;
          if (seq < my_tiles) tc = p2_decode(p, cid + seq * n_clusters, n_pairs);
        }
      }
      // No exit with bulk copies in flight (see wino_tc.cuh).
      for (int g = issued > S ? issued - S : 0; g < issued; ++g)
        mbar_wait_drain(smem_u32((loads_u ? u_full : raw_full) + g % S), (g / S) & 1);
    }
  } else if (warp >= 1 && warp <= kP2TransformWarps) {
    // ===================================== input transform =====================================
    const int t = tid - 32;                                            // 0..255
    for (int g = 0; g < total_chunks; ++g) {
      const int s = g % S;
      const uint32_t use = g / S;
      mbar_wait(smem_u32(raw_full + s), use & 1, dead, p.status);
      if (use > 0) mbar_wait(smem_u32(uv_empty + s), (use - 1) & 1, dead, p.status);   // V stage free again
      const float *__restrict__ raw = reinterpret_cast<const float *>(raw_s + s * Cfg::kRawBytes);
      uint8_t *__restrict__ vst = v_s + s * kP2VBytes;
      if (DT == kTcBf16) {
        p2_transform_bf16_x2<RANK>(raw, vst, t >> 5, t & 31);
      } else {
        p2_transform_tf32_pair<RANK>(raw, vst, t >> 5, t & 31);   // 8 channels x 32 image pairs = 256 threads
      }
      fence_proxy_async_smem();          // V is read by the tensor core through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(raw_empty + s));
        mbar_arrive(smem_u32(v_ready + s));
      }
    }
  } else if (warp == kP2MmaWarp || warp == kP2MmaWarpB) {
    // ===================================== MMA issuers (two threads, four positions each; see wino_tc.cuh) ====
    if (lane == 0) {
      const int x0 = warp == kP2MmaWarp ? 0 : 4;
      const uint32_t fmt = DT == kTcBf16 ? 1u : 2u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) |
                             ((uint32_t)(kP2N >> 3) << 17) | ((uint32_t)(kTcM >> 4) << 24);
      // A as in wino_tc.cuh.  B: 64 images x KC channels; BF16 rows of 128 B (128-byte swizzle, 8-channel groups
      // 1 KB apart); TF32 two 32-image blocks 1 KB apart, rows of 128 B, 4-channel groups 512 B apart.
      const uint64_t a_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(u_s), KC * 128, 1024, 2) : smem_desc(smem_u32(u_s), KC * 128, 512, 1);
      const uint64_t b_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(v_s), 1024, 1024, 2) : smem_desc(smem_u32(v_s), 1024, 512, 1);
      int ci = 0, seq = 0;
      for (int g = 0; g < total_chunks; ++g) {
        const int s = g % S;
        const uint32_t use = g / S;
        // A wait that gave up: stop issuing.
        if (!mbar_wait(smem_u32(u_full + s), use & 1, dead, p.status)) break;
        if (!mbar_wait(smem_u32(v_ready + s), use & 1, dead, p.status)) break;
        if (ci == 0 && seq > 0 && !mbar_wait(smem_u32(acc_empty), (seq - 1) & 1, dead, p.status)) break;   // TMEM drained
        tc_fence_after();
        const uint64_t ad = a_desc0 + (uint64_t)(s * (kP2UBytes >> 4)), bd = b_desc0 + (uint64_t)(s * (kP2VBytes >> 4));
        const uint32_t accumulate = ci > 0 ? 1u : 0u;
#pragma unroll
        for (int xo = 0; xo < 4; ++xo) {
          const int xl = x0 + xo;
          tc_mma<DT>(tmem_base + xl * kP2N, ad + (uint64_t)(xl * (4096 >> 4)), bd + (uint64_t)(xl * (2048 >> 4)), idesc, accumulate);
        }
        tc_commit(smem_u32(uv_empty + s));
        if (++ci == cpt) {
          tc_commit(smem_u32(acc_full));
          ci = 0;
          ++seq;
        }
      }
      // every MMA this thread issued must have completed before tensor memory is freed
      const int me = warp == kP2MmaWarp ? 0 : 1;
      tc_commit(smem_u32(mma_done + me));
      mbar_wait_drain(smem_u32(mma_done + me), 0);
    }
  } else {
    // ===================================== epilogue ============================================
    const int ew = warp - kP2FirstEpilogueWarp;                          // 0..7
    const int quarter = warp & 3;                                        // TMEM lanes this warp may read
    const int sub = ew >> 2;                                             // which 16 of a block's 32 images
    const int m = quarter * 32 + lane;
    const size_t plane = (size_t)p.H * p.W * p.N;
    const size_t dW = (size_t)p.N, dH = (size_t)p.W * p.N;
    const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    for (int seq = 0; seq < my_tiles; ++seq) {
      const P2Tile tc = p2_decode(p, cid + seq * n_clusters, n_pairs);
      mbar_wait(smem_u32(acc_full), seq & 1, dead, p.status);
      tc_fence_after();
      const int k = tc.kb * kTcM + m;
      const bool kvalid = k < p.K;
      const bool warp_valid = (tc.kb * kTcM + quarter * 32) < p.K;
      const int oh0 = 2 * tc.ty, ow0 = 2 * tc.tx;
      const bool row1 = (oh0 + 1) < p.H, col1 = (ow0 + 1) < p.W;
#pragma unroll 1
      for (int phase = 0; phase < 2; ++phase) {
        const int ib = phase == 0 ? RANK : 1 - RANK;                     // image block of the pair handled now
        const bool block_valid = (2 * tc.np + ib) < p.n_blocks;
        if (phase == 1) {
          // the peer has stored its partial results for this block (its phase 0 of the same tile)
          mbar_wait(smem_u32(peer_ready + (seq & 1)), (seq >> 1) & 1, dead, p.status);
          fence_acq_rel_cluster();       // pairs with the peer's release at cluster scope: its stores are visible
        }
        if (warp_valid && block_valid) {
          float *ybase = p.y + (size_t)k * plane + ((size_t)oh0 * p.W + ow0) * p.N + (size_t)(2 * tc.np + ib) * 32 + 16 * sub;
#pragma unroll 1
          for (int step = 0; step < 2; ++step) {
            const int col = 32 * ib + 16 * sub + 8 * step;
            float mm[8][8];
#pragma unroll
            for (int xl = 0; xl < 8; ++xl) {
              float lo[4], hi[4];
              tmem_ld_x4(tlane + xl * kP2N + col, lo);
              tmem_ld_x4(tlane + xl * kP2N + col + 4, hi);
#pragma unroll
              for (int e = 0; e < 4; ++e) { mm[xl][e] = lo[e]; mm[xl][4 + e] = hi[e]; }
            }
            tmem_ld_wait();
            float yq[4][8];                                              // [output position][image]
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float colv[8], yy[4];
#pragma unroll
              for (int xl = 0; xl < 8; ++xl) colv[xl] = mm[xl][e];
              p2_partial_output<RANK>(colv, yy);
#pragma unroll
              for (int q = 0; q < 4; ++q) yq[q][e] = yy[q];
            }
            // eight images per lane and step; N is a multiple of 8, so a step is inside N or outside
            if (kvalid && (2 * tc.np + ib) * 32 + 16 * sub + 8 * step < p.N) {
              float *dst = ybase + 8 * step;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if ((q & 1) && !col1) continue;
                if ((q & 2) && !row1) continue;
                float *d = dst + ((q & 1) ? dW : 0) + ((q & 2) ? dH : 0);
                float lo[4] = {yq[q][0], yq[q][1], yq[q][2], yq[q][3]}, hi[4] = {yq[q][4], yq[q][5], yq[q][6], yq[q][7]};
                if (phase == 0) {
                  st_global_v8(d, lo, hi);
                } else {
                  // add to the partial the peer stored: a reduction at L2, nothing to wait for.
                  // Two addends only, so the result does not depend on arrival order.
                  red_global_add_v4(d, lo);
                  red_global_add_v4(d + 4, hi);
                }
              }
            }
          }
        }
        if (phase == 0) {
          // publish this warp's partial results to the peer: stores -> fence -> remote arrive
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(smem_u32(peer_ready + (seq & 1)), 1 - RANK);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_empty));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither CTA leaves while the other may still signal its barriers
  if (warp == kP2MmaWarp) {
    tc_fence_after();
    tmem_dealloc_512(tmem_base);
  }
}

template <int DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kP2Threads, 1)
wino_tc2_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_u, const WinoParams p) {
  extern __shared__ __align__(1024) uint8_t tsmem2[];
  if (cluster_ctarank() == 0) p2_body<DT, 0>(tm_in, tm_u, p, tsmem2);
  else                        p2_body<DT, 1>(tm_in, tm_u, p, tsmem2);
}

}  // namespace ocb
