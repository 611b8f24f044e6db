// Tensor-core Winograd kernel for a pair of CTAs (thread-block cluster of 2) that share one tile
// of 128 filters x 64 images, split the 16 Winograd positions 8 / 8, and exchange the transformed
// input through distributed shared memory.
//
// Why a pair: tensor memory holds 512 accumulator columns per SM.  With all 16 positions in one
// CTA (wino_tc.cuh) that is 32 images per MMA, and such a small MMA is bound by the shared-memory
// read of its A operand: 4 KB of filters + 1 KB of images for 16 cycles of tensor-pipe work.  With
// 8 positions per CTA the same 512 columns hold 64 images: half as many MMAs per image, each
// twice as wide, and every filter byte read from shared memory (and from L2) serves twice the
// images.  The reference has no counterpart (no tensor-core path at all).
//
// Why the exchange: every CTA needs the transformed input V of all 64 images for its 8
// positions.  The kernels of this family are bound by what an SM can pull out of L2 (about 57
// bytes per clock): per K-step the single-CTA kernel pulls 32 KB of raw patches and 64 KB of
// filters for 32 images.  Here CTA r loads and transforms only ITS 32 images (image block r of
// the pair), for all 16 positions, keeps the 8 positions of transform rows 2r, 2r+1 and sends the
// other 8 to the peer: 32 KB of patches and 32 KB of filters per K-step for the same work per SM,
// and the transform work of a single-CTA kernel.
//
// How the exchange is done: with the asynchronous bulk copy between shared memories
// (cp.async.bulk.shared::cluster.shared::cta), one 8 KB copy per K-step and direction, issued by
// one thread after the transform warps have met at a named barrier, completing (complete_tx) on
// the mbarrier in the PEER's shared memory that its MMA threads wait on.  Element-wise remote
// stores were tried first and are several times slower: every transform warp then has to publish
// its stores with a release at cluster scope per K-step, which costs the issuing thread 1 000 to
// 2 500 cycles (it waits for the stores to be acknowledged).  A V stage is laid out as
// [image block][position][1 KB tile], so the half that a CTA contributes is 8 KB of contiguous
// bytes, and each tile is the single-CTA kernel's V tile; the MMA's B descriptor reaches the
// second image block through its leading-dimension offset.
//
// Hand-offs (all mbarriers, all waits bounded), rings of their own for raw patches, U and V:
//   raw_full / raw_empty   raw patches landed (TMA) / transformed
//   u_full / u_empty       this CTA's filter slice landed (TMA) / its MMAs have completed
//   v_ready                this CTA's V stage is complete: its own half written (one arrive after
//                          the transform warps' barrier) and the peer's 8 KB landed (tx bytes)
//   v_empty                this CTA's MMAs on the V stage have completed (tcgen05.commit)
//   peer_v_empty           the PEER's MMAs on ITS V stage have completed, so this CTA may copy
//                          there again: the peer's MMA threads commit to this barrier too (the
//                          address of a tcgen05.commit is a shared::cluster address)
// The CTAs meet again in the epilogue: the output transform is linear in the 16 positions, so
// each CTA forms the partial result of its 8 positions; CTA r stores its partial for image block
// r, signals the peer through an mbarrier in the peer's shared memory, and for the other block
// adds its partial onto what the peer stored (red.global.add.v4.f32 at L2; two addends, so the
// sum does not depend on the order).  Both CTAs leave through a cluster barrier, so neither
// exits while the other may still copy into its shared memory or signal its barriers.
//
// Warp roles, aligned to warpgroups of four warps because setmaxnreg is a warpgroup instruction:
//   warps 0-3    one thread each: raw-patch loader, filter loader, two MMA issuers (four positions
//                each; warp 2 also owns the TMEM allocation)                      -> 40 registers
//   warps 4-11   input transform (BF16: all eight per K-step, one (channel, image pair) per
//                thread; TF32: the two warpgroups take K-steps alternately)       -> 88 registers
//   warps 12-19  epilogue, two warps per TMEM lane quarter                        -> 128 registers
#pragma once
#include "wino_tc2.cuh"   // cluster helpers, partial output transform, P2Tile / p2_decode

namespace ocb {

constexpr int kP3TransformWarps = 8;
constexpr int kP3EpilogueWarps = 8;
constexpr int kP3RawLoaderWarp = 0, kP3ULoaderWarp = 1, kP3MmaWarp = 2, kP3MmaWarpB = 3;
constexpr int kP3FirstTransformWarp = 4;
constexpr int kP3FirstEpilogueWarp = kP3FirstTransformWarp + kP3TransformWarps;
constexpr int kP3Threads = (kP3FirstEpilogueWarp + kP3EpilogueWarps) * 32;       // 640
// setmaxnreg budgets: the CTA owns 640 x 96 registers and redistributes them.
constexpr int kP3LaunchRegs = 96, kP3ControlRegs = 40, kP3TransformRegs = 88, kP3EpilogueRegs = 128;
static_assert(128 * kP3ControlRegs + 256 * kP3TransformRegs + 256 * kP3EpilogueRegs <= kP3Threads * kP3LaunchRegs,
              "setmaxnreg budgets exceed the registers the CTA was launched with");
constexpr uint32_t kP3UBytes = 8 * 4096;         // 8 positions x (128 filters x one K-step)
constexpr uint32_t kP3VBytes = 2 * 8 * 1024;     // [2 image blocks][8 positions][1 KB tile: 32 images x one K-step]
constexpr uint32_t kP3HalfBytes = 8 * 1024;      // what one CTA contributes to a V stage; also one staging buffer

template <int DT> struct P3Cfg {
  static constexpr int kKC = DT == kTcBf16 ? 16 : 8;                  // channels per K-step
  static constexpr uint32_t kRawBytes = kKC * 16 * 32 * 4;            // [c][4 h][4 w][32 n] fp32, this CTA's image block
  // Rings: raw patches, filters (U), transformed input (V, with one outgoing staging buffer per
  // stage).  V is the deepest: a V stage is refilled across the cluster, so its turn-around
  // includes a copy between the two SMs.
  static constexpr int kRawStages = DT == kTcBf16 ? 2 : 4;
  static constexpr int kUStages = 2;
  static constexpr int kVStages = 4;
  // transform threads that work on one K-step: BF16 all 256, TF32 one warpgroup (K-steps alternate)
  static constexpr int kThreadsPerStep = DT == kTcBf16 ? 256 : 128;
  static constexpr size_t kSmemBytes = (size_t)kRawStages * kRawBytes + (size_t)kUStages * kP3UBytes +
                                       (size_t)kVStages * (kP3VBytes + kP3HalfBytes) + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory");
};

// Shared-memory address of the same offset in CTA `rank` of the cluster (a shared::cluster address).
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// Remote arrive that only tells the peer "you may overwrite": it publishes no data, so it needs
// no release (a release at cluster scope makes the thread wait for its earlier writes).
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Asynchronous copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) from this CTA's
// shared memory into the peer's, completing - with its byte count - on an mbarrier of the peer.
// Not a multicast: one source, one destination.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t remote_dst, uint32_t local_src, uint32_t bytes, uint32_t remote_bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(remote_dst), "r"(local_src), "r"(bytes), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ void st_cta_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cta_v2f32(uint32_t addr, float a, float b) {
  asm volatile("st.shared::cta.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}

// ---- input transform of one (channel, image pair) of this CTA's 32 images, all 16 positions ------
// d: the 4x4 patch of the two images (packed pairs), row-major.  The 8 positions of transform rows
// 2*RANK, 2*RANK+1 are this CTA's own (`own`: its image block inside its V stage), the other 8 go
// to the staging buffer that is then copied to the peer (`out`); both addresses are already offset
// for (channel, image pair) inside a 1 KB tile, tiles of consecutive positions are 1 KB apart.
// Tile formats are the single-CTA kernel's: BF16 [16 c][32 n], rows of 64 bytes, 64-byte swizzle;
// TF32 [8 c][32 n] fp32, rows of 128 bytes, 128-byte swizzle with 32-byte atoms.
template <int DT, int RANK>
__device__ __forceinline__ void p3_transform_store(const uint64_t (&d)[16], uint32_t own, uint32_t out) {
  uint64_t b[16];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b[j] = sub2(d[j], d[8 + j]);
    b[4 + j] = add2(d[4 + j], d[8 + j]);
    b[8 + j] = sub2(d[8 + j], d[4 + j]);
    b[12 + j] = sub2(d[4 + j], d[12 + j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint64_t o[4];
    o[0] = sub2(b[4 * i + 0], b[4 * i + 2]);
    o[1] = add2(b[4 * i + 1], b[4 * i + 2]);
    o[2] = sub2(b[4 * i + 2], b[4 * i + 1]);
    o[3] = sub2(b[4 * i + 1], b[4 * i + 3]);
    const uint32_t base = ((i >> 1) == RANK) ? own : out;          // compile-time after unrolling
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t addr = base + (uint32_t)((4 * (i & 1) + j) * 1024);     // position within the owner's eight
      float lo, hi;
      unpack2(o[j], lo, hi);
      if (DT == kTcBf16) st_cta_u32(addr, pack_bf16x2(lo, hi));
      else               st_cta_v2f32(addr, round_tf32_rne(lo), round_tf32_rne(hi));
    }
  }
}

// p.n_blocks counts 32-image blocks, p.k_blocks 128-filter blocks; p.total_tiles counts pair tiles.
template <int DT, int RANK>
__device__ __forceinline__ void p3_body(const CUtensorMap &tm_in, const CUtensorMap &tm_u, const WinoParams &p,
                                        uint8_t *tsmem) {
  using Cfg = P3Cfg<DT>;
  constexpr int KC = Cfg::kKC;
  constexpr int SR = Cfg::kRawStages, SU = Cfg::kUStages, SV = Cfg::kVStages;
  constexpr uint32_t PEER = 1 - RANK;
  uint8_t *raw_s = tsmem;
  uint8_t *u_s = raw_s + SR * Cfg::kRawBytes;
  uint8_t *v_s = u_s + SU * kP3UBytes;
  uint8_t *out_s = v_s + SV * kP3VBytes;                               // outgoing halves, one per V stage
  uint64_t *bars = reinterpret_cast<uint64_t *>(out_s + SV * kP3HalfBytes);
  uint64_t *raw_full = bars, *raw_empty = raw_full + SR, *u_full = raw_empty + SR, *u_empty = u_full + SU,
           *v_ready = u_empty + SU, *v_empty = v_ready + SV, *peer_v_empty = v_empty + SV;
  uint64_t *acc_full = peer_v_empty + SV, *acc_empty = acc_full + 1, *peer_ready = acc_full + 2;   // peer_ready[2], used alternately
  uint64_t *mma_done = acc_full + 4;                                                               // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 6);
  volatile int *dead = reinterpret_cast<volatile int *>(acc_full + 7);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_clusters = (int)gridDim.x / 2, cid = (int)blockIdx.x / 2;
  const int n_pairs = (p.n_blocks + 1) / 2;
  const int my_tiles = (p.total_tiles - cid + n_clusters - 1) / n_clusters;
  const int cpt = p.chunks_per_tile;
  const int total_chunks = my_tiles * cpt;

  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < SR; ++s) {
      mbar_init(smem_u32(raw_full + s), 1);
      mbar_init(smem_u32(raw_empty + s), 1);                       // one arrive after the transform warps' barrier
    }
    for (int s = 0; s < SU; ++s) {
      mbar_init(smem_u32(u_full + s), 1);
      mbar_init(smem_u32(u_empty + s), 2);                         // one tcgen05.commit per MMA-issuing thread
    }
    for (int s = 0; s < SV; ++s) {
      mbar_init(smem_u32(v_ready + s), 1);                         // own half (one arrive) + the peer's bytes
      mbar_init(smem_u32(v_empty + s), 2);
      mbar_init(smem_u32(peer_v_empty + s), 2);                    // the peer's two MMA threads commit here as well
    }
    mbar_init(smem_u32(peer_ready + 0), kP3EpilogueWarps);
    mbar_init(smem_u32(peer_ready + 1), kP3EpilogueWarps);
    mbar_init(smem_u32(acc_full), 2);
    mbar_init(smem_u32(acc_empty), kP3EpilogueWarps);
    mbar_init(smem_u32(mma_done + 0), 1);
    mbar_init(smem_u32(mma_done + 1), 1);
    mbar_fence_init();
  }
  if (warp == kP3MmaWarp) tmem_alloc_512(smem_u32(tmem_slot));
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < kP3FirstTransformWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kP3ControlRegs));
    if (warp == kP3RawLoaderWarp || warp == kP3ULoaderWarp) {
      // ===================================== TMA loaders =========================================
      const bool loads_u = warp == kP3ULoaderWarp;
      if (lane == 0) {
        tma_prefetch_descriptor(loads_u ? &tm_u : &tm_in);
        int seq = 0, ci = 0, issued = 0;
        P2Tile tc = p2_decode(p, cid, n_pairs);
        const int ring = loads_u ? SU : SR;
        for (int g = 0; g < total_chunks; ++g) {
          const int s = g % ring;
          const uint32_t use = g / ring;
          // A wait that gave up: stop issuing - the stage may still be in use.
          if (use > 0 && !mbar_wait(smem_u32((loads_u ? u_empty : raw_empty) + s), (use - 1) & 1, dead, p.status)) break;
          if (!loads_u) {
            mbar_arrive_expect_tx(smem_u32(raw_full + s), Cfg::kRawBytes);
            tma_load_4d(smem_u32(raw_s + s * Cfg::kRawBytes), &tm_in, smem_u32(raw_full + s), (2 * tc.np + RANK) * 32,
                        2 * tc.tx - 1, 2 * tc.ty - 1, ci * KC);          // this CTA's image block of the pair
          } else {
            mbar_arrive_expect_tx(smem_u32(u_full + s), kP3UBytes);
            tma_load_4d(smem_u32(u_s + s * kP3UBytes), &tm_u, smem_u32(u_full + s), 0, ci * KC,
                        tc.kb * (DT == kTcBf16 ? 2 : 4), 8 * RANK);      // this CTA's eight positions
          }
          issued = g + 1;
          if (++ci == cpt) {
            ci = 0;
            ++seq;
            if (seq < my_tiles) tc = p2_decode(p, cid + seq * n_clusters, n_pairs);
          }
        }
        // No exit with bulk copies in flight (after a complete run these phases are long over).
        for (int g = issued > ring ? issued - ring : 0; g < issued; ++g)
          mbar_wait_drain(smem_u32((loads_u ? u_full : raw_full) + g % ring), (g / ring) & 1);
      }
    } else {
      // ===================================== MMA issuers (two threads, four positions each) ======
      if (lane == 0) {
        const int me = warp == kP3MmaWarp ? 0 : 1;
        const int x0 = 4 * me;
        const uint32_t fmt = DT == kTcBf16 ? 1u : 2u;
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) |
                               ((uint32_t)(kP2N >> 3) << 17) | ((uint32_t)(kTcM >> 4) << 24);
        // A: 128 filters x KC channels per position, filter-contiguous rows of 128 B, 8-channel (TF32: 4-channel)
        //    groups 1 KB (512 B) apart, 128-byte-row blocks of the filter axis KC*128 B apart.
        // B: 64 images x KC channels per position as two 32-image tiles 8 KB apart (the two image blocks of the
        //    stage; leading-dimension offset); inside a tile 8-channel (TF32: 4-channel) groups 512 B apart.
        const uint64_t a_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(u_s), KC * 128, 1024, 2) : smem_desc(smem_u32(u_s), KC * 128, 512, 1);
        const uint64_t b_desc0 = DT == kTcBf16 ? smem_desc(smem_u32(v_s), kP3HalfBytes, 512, 4) : smem_desc(smem_u32(v_s), kP3HalfBytes, 512, 1);
        const uint32_t peer_v_empty0 = mapa_u32(smem_u32(peer_v_empty), PEER);
        int ci = 0, seq = 0;
        for (int g = 0; g < total_chunks; ++g) {
          const int su = g % SU, sv = g % SV;
          // A wait that gave up: stop issuing.
          if (!mbar_wait(smem_u32(u_full + su), (g / SU) & 1, dead, p.status)) break;
          if (!mbar_wait(smem_u32(v_ready + sv), (g / SV) & 1, dead, p.status)) break;     // both halves of V in place
          if (ci == 0 && seq > 0 && !mbar_wait(smem_u32(acc_empty), (seq - 1) & 1, dead, p.status)) break;   // TMEM drained
          tc_fence_after();
          const uint64_t ad = a_desc0 + (uint64_t)(su * (kP3UBytes >> 4)), bd = b_desc0 + (uint64_t)(sv * (kP3VBytes >> 4));
          const uint32_t accumulate = ci > 0 ? 1u : 0u;
#pragma unroll
          for (int xo = 0; xo < 4; ++xo) {
            const int xl = x0 + xo;
            tc_mma<DT>(tmem_base + xl * kP2N, ad + (uint64_t)(xl * (4096 >> 4)), bd + (uint64_t)(xl * (1024 >> 4)), idesc, accumulate);
          }
          tc_commit(smem_u32(u_empty + su));
          tc_commit(smem_u32(v_empty + sv));
          tc_commit(peer_v_empty0 + 8u * (uint32_t)sv);      // the same completion, signalled in the peer's shared memory
          if (++ci == cpt) {
            tc_commit(smem_u32(acc_full));
            ci = 0;
            ++seq;
          }
        }
        // every MMA this thread issued must have completed before tensor memory is freed
        tc_commit(smem_u32(mma_done + me));
        mbar_wait_drain(smem_u32(mma_done + me), 0);
      }
    }
  } else if (warp < kP3FirstEpilogueWarp) {
    // ===================================== input transform =====================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kP3TransformRegs));
    const int tt = tid - 32 * kP3FirstTransformWarp;                     // 0..255
    // BF16: 16 channels x 16 image pairs = 256 items per K-step, one per thread.
    // TF32:  8 channels x 16 image pairs = 128 items per K-step; warpgroup w takes the K-steps g = w mod 2.
    const int t = DT == kTcBf16 ? tt : (tt & 127);
    const int c = t >> 4, np = t & 15;
    const int group = DT == kTcBf16 ? 0 : (tt >> 7);
    const int g0 = group, gstep = DT == kTcBf16 ? 1 : 2;
    // byte offset of (channel, image pair) inside a 1 KB tile
    const uint32_t toff = DT == kTcBf16
        ? (uint32_t)(c * 64 + ((((np >> 2) ^ (c >> 1)) & 3) << 4) + ((np & 3) << 2))
        : (uint32_t)(c * 128 + (((((2 * np) >> 3) ^ c) & 3) << 5) + (((2 * np) & 7) << 2));
    const uint32_t own0 = smem_u32(v_s) + RANK * kP3HalfBytes + toff;   // this CTA's image block in its own V stage
    const uint32_t out0 = smem_u32(out_s) + toff;
    // the thread of a group that hands a finished K-step on
    const bool leader = t == 0;
    const uint32_t peer_v0 = mapa_u32(smem_u32(v_s) + RANK * kP3HalfBytes, PEER);   // this CTA's image block in the peer's V stage
    const uint32_t peer_ready0 = mapa_u32(smem_u32(v_ready), PEER);
    bool gave_up = false;
    for (int g = g0; g < total_chunks; g += gstep) {
      const int sv = g % SV, sr = g % SR;
      const uint32_t use = g / SV;
      bool ok = mbar_wait(smem_u32(raw_full + sr), (g / SR) & 1, dead, p.status);
      if (use > 0) {
        ok &= mbar_wait(smem_u32(v_empty + sv), (use - 1) & 1, dead, p.status);        // own V stage free again
        ok &= mbar_wait(smem_u32(peer_v_empty + sv), (use - 1) & 1, dead, p.status);   // the peer's too (so is the staging buffer)
      }
      const uint64_t *R = reinterpret_cast<const uint64_t *>(raw_s + sr * Cfg::kRawBytes) + (c * 16) * 16 + np;
      uint64_t d[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) d[q] = R[q * 16];
      p3_transform_store<DT, RANK>(d, own0 + sv * kP3VBytes, out0 + sv * kP3HalfBytes);
      fence_proxy_async_smem();          // both halves are read through the async proxy: tensor core, bulk copy
      asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(Cfg::kThreadsPerStep) : "memory");
      if (leader) {
        gave_up |= !ok;
        mbar_arrive(smem_u32(raw_empty + sr));
        // this CTA's V stage: its own half is written; the peer's 8 KB are still to land
        mbar_arrive_expect_tx(smem_u32(v_ready + sv), kP3HalfBytes);
        // A wait of this thread that gave up: no further copies (the peer's stage may be in use).
        if (!gave_up)
          bulk_copy_to_peer(peer_v0 + sv * kP3VBytes, smem_u32(out_s) + sv * kP3HalfBytes, kP3HalfBytes, peer_ready0 + 8u * (uint32_t)sv);
      }
    }
  } else {
    // ===================================== epilogue ============================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kP3EpilogueRegs));
    const int ew = warp - kP3FirstEpilogueWarp;                          // 0..7
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
          // publish this warp's partial results to the peer: stores -> fence -> remote arrive (release)
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(smem_u32(peer_ready + (seq & 1)), PEER);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_empty));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither CTA leaves while the other may still copy into its shared memory or signal it
  if (warp == kP3MmaWarp) {
    tc_fence_after();
    tmem_dealloc_512(tmem_base);
  }
}

template <int DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kP3Threads, 1)
wino_tc3_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_u, const WinoParams p) {
  extern __shared__ __align__(1024) uint8_t tsmem3[];
  if (cluster_ctarank() == 0) p3_body<DT, 0>(tm_in, tm_u, p, tsmem3);
  else                        p3_body<DT, 1>(tm_in, tm_u, p, tsmem3);
}

}  // namespace ocb
