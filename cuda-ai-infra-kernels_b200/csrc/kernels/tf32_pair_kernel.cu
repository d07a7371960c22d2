// TF32 tensor-core GEMM, CTA-pair kernel (tcgen05 cta_group::2, 256 x 256 tiles). Layouts, the
// parameter block and the epilogues are in tf32_umma.cuh.
#include "tf32_umma.cuh"

namespace b200 {

cudaError_t tf32_pair_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

// ---------------------------------------------------- TMA, CTA-pair kernel
// Two CTAs of a cluster share one 256 x 256 output tile through
// tcgen05.mma.cta_group::2: CTA r of the pair holds rows [128 r, 128 r + 128) of
// A, columns [128 r, 128 r + 128) of B and the accumulator rows [128 r, +128)
// (all 256 columns). Per CTA a stage is 16 KiB of A + 16 KiB of B for a
// 256 x 256 x 32 product, a third fewer operand bytes through L2 per flop than
// the single-CTA 128 x 256 tile. The even CTA issues the MMAs for both.
// Signals that both CTAs need (stage free, accumulator ready) are committed
// twice, once per CTA; no multicast form is used anywhere.
//
// The last, partial round of tiles runs as 256 x 128 half tiles on twice as many pairs, and
// differently in two ways (measured with one MMA thread and the whole tiles' ring: a half-tile
// stage took 1040 cycles where a whole tile's takes 1080, for half the product):
//  * a half-tile stage is 48 KiB per CTA, so the 192 KiB ring holds four of them instead of three
//    64 KiB ones, with barriers of their own: what a CTA has in flight, not the tensor pipe, sets
//    the pace of a half tile. A pair's whole tiles come before its halves; the two layouts
//    overlap, and the producer fills each half-tile slot as soon as the whole-tile slots under it
//    have been read.
//  * a half tile's instructions occupy the pipe for half as long, and one thread's 62 cycles per
//    instruction plus its barrier round trip per stage no longer fit beside them. A second thread
//    takes the second sub-block of every stage into an accumulator of its own, 128 columns beside
//    the first (the two partial sums fill the 256 columns of a whole tile's buffer; the epilogue
//    adds them). Its first wait is for the first half-tile stage, which nothing fills before the
//    whole tiles are done: a wait by phase parity is only right within one phase of its barrier,
//    and from there on the thread is.
constexpr int kPairN = 256;
constexpr uint32_t kPairSubBytes = kASlabBytes + (kPairN / 2 / 32) * kBBoxBytes;  // 32 floats of K: 32 KiB per CTA
constexpr uint32_t kHalfSubBytes = kASlabBytes + (kPairN / 4 / 32) * kBBoxBytes;  // the same of a half tile: 24 KiB

// A pipeline stage holds KSUB such 32-wide K sub-blocks behind one pair of barriers: the MMA
// thread's barrier wait, fence and commits are paid per stage, and they cost about as much as two
// of the eight instructions of a two-sub-block stage.
template <int STAGES, int KSUB>
__host__ __device__ constexpr size_t pair_smem_bytes() {
  return static_cast<size_t>(STAGES) * KSUB * kPairSubBytes + 1024 + 1024 + kStagingBytes;   // ring | barriers | staging
}
// Stages of two half-tile sub-blocks in the same ring.
template <int STAGES, int KSUB>
__host__ __device__ constexpr int pair_half_stages() {
  return static_cast<int>(STAGES * KSUB * kPairSubBytes / (2 * kHalfSubBytes));
}

// Work item of the CTA-pair kernel: a whole 256 x 256 tile, or (for the last, partial round of
// tiles) one 256 x 128 half of one, so that twice as many pairs share the tail.
struct PairItem {
  int tile;
  int half;   // -1: whole tile; 0 / 1: left / right 128 columns
};
__device__ __forceinline__ PairItem pair_item(int item, int full_tiles) {
  if (item < full_tiles) return PairItem{item, -1};
  const int h = item - full_tiles;
  return PairItem{full_tiles + (h >> 1), h & 1};
}

// One MMA thread's share of a 256 x 128 half tile: sub-block `sub` of every half-tile stage into
// its own 128 accumulator columns (free once `acc_empty` has completed the phase before
// `acc_parity`). Stage s lies in slot (s + rotation) % HSTAGES of the ring. Both threads commit
// every stage and the finished accumulator to both CTAs. Returns false when a wait ran out.
template <int HSTAGES>
__device__ __forceinline__ bool issue_half_tile(uint64_t* full, uint64_t* empty, uint64_t* acc_full, uint64_t* acc_empty,
                                                uint32_t acc_parity, const SubBlockDescs& ring, uint32_t idesc, uint32_t tmem_acc,
                                                int sub, int k_blocks, int rotation, int& stage, uint32_t& phase) {
  for (int kb = 0; kb < k_blocks; ++kb) {
    if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) return false;
    if (kb == 0 && !mbar_wait(acc_empty, acc_parity ^ 1u, kSiteUmmaAccEmpty)) return false;
    tcgen05_fence_after_sync();
    const uint32_t offset = static_cast<uint32_t>((stage + rotation) % HSTAGES) * (2 * kHalfSubBytes) + sub * kHalfSubBytes;
#pragma unroll
    for (int j = 0; j < kStageK / kInstK; ++j) {
      umma_tf32_pair(tmem_acc, umma_desc_advance(ring.a, offset + j * (kInstK * 4)),
                     umma_desc_advance(ring.b, offset + j * (kInstK * 128)), idesc, (kb > 0 || j > 0) ? 1u : 0u);
    }
    umma_commit_pair(smem_u32(&empty[stage]));
    umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 1));
    if (++stage == HSTAGES) stage = 0, phase ^= 1u;
  }
  umma_commit_pair(smem_u32(acc_full));
  umma_commit_pair(map_to_cta(smem_u32(acc_full), 1));
  return true;
}

template <int STAGES, int KSUB, int kAct>
__global__ void __launch_bounds__(kTileThreadsTwoIssuers, 1) umma_pair_kernel(const __grid_constant__ UmmaParams p) {
  static_assert(KSUB == 2, "a half tile's two MMA threads take one sub-block of a stage each");
  constexpr int kIssuers = 2;
  constexpr int kSecondIssuerWarp = 2 + 4 * kTileEpilogueShare;
  constexpr int HSTAGES = pair_half_stages<STAGES, KSUB>();
  extern __shared__ uint8_t smem_raw[];
  // Same carve-up in both CTAs: the MMA addresses the peer's shared memory by
  // the same offsets as its own.
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t kPairStageBytes = KSUB * kPairSubBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(STAGES) * kPairStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* half_full = empty + STAGES;       // the same two for the half tiles' stages
  uint64_t* half_empty = half_full + HSTAGES;
  uint64_t* acc_full = half_empty + HSTAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* peer_stage = reinterpret_cast<float*>(stages + static_cast<size_t>(STAGES) * kPairStageBytes + 1024);   // kStagingBytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0: issues the MMAs, 1: peer

  if (threadIdx.x == 0) {
    // The descriptors the copies will name, requested first of all (their fetch is part of the
    // latency of the first load and of the first store).
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(&p.map_b);
    if (p.b_strips == kPairN / 2 / 32) prefetch_tensormap(&p.map_b_strips);
    if (p.tma_store != 0) prefetch_tensormap(&p.map_d);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);   // used in CTA 0 only: one expect_tx arrival, bytes of both CTAs
      mbar_init(&empty[s], 1);  // one tcgen05.commit per use, sent to each CTA
    }
    for (int s = 0; s < HSTAGES; ++s) {
      mbar_init(&half_full[s], 1);
      mbar_init(&half_empty[s], kIssuers);   // one tcgen05.commit per MMA thread and use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], kIssuers);                 // both threads' commits (a whole tile: one commit, one plain arrival)
      mbar_init(&acc_empty[b], 8 * kTileEpilogueShare);  // used in CTA 0 only: the epilogue warps of both CTAs
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair<512>(tmem_ptr);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any remote arrival
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  grid_launch_dependents();   // the next kernel of the stream may set itself up beside this one (not before this
                              // kernel's TMEM is allocated: its CTAs could take the columns first)
  grid_dependency_wait();     // the kernel before this one has completed: global memory may be touched

  const int tiles_m = (p.m + 2 * kTileM - 1) / (2 * kTileM);
  const int tiles_n = (p.n + kPairN - 1) / kPairN;
  const int tiles = tiles_m * tiles_n;
  const int items = p.pair_full_tiles + 2 * (tiles - p.pair_full_tiles);   // whole tiles, then halves
  const int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages per tile; K past the end reads as zeros
  const int first_tile = blockIdx.x >> 1, tile_stride = gridDim.x >> 1;
  // This pair's whole tiles are its first `whole` items.
  const int whole = p.pair_full_tiles > first_tile ? (p.pair_full_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const int first_half = first_tile + whole * tile_stride;
  // The half tiles' four 48 KiB slots lie across the whole tiles' three 64 KiB ones (slot h across
  // {0}, {0, 1}, {1, 2}, {2}), which come free oldest first, starting with `oldest`. The half
  // tiles' stage 0 is put in the first slot that comes free entirely, so that the change of layout
  // does not let the ring run empty.
  static_assert(STAGES == 3 && HSTAGES == 4, "the overlap of the two layouts is spelled out for three and four stages");
  const int oldest = static_cast<int>((static_cast<long long>(whole) * k_blocks) % STAGES);
  const int rotation = oldest == 0 ? 0 : oldest + 1;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = first_tile; item < p.pair_full_tiles && ok; item += tile_stride) {
        int tm, tn;
        tile_coords(item, tiles_m, tiles_n, &tm, &tn);
        const int row0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
        const int col0 = tn * kPairN + static_cast<int>(rank) * (kPairN / 2);   // this CTA's 128 of the B columns
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, kSiteUmmaEmpty)) { ok = false; break; }
          // Completion bytes of both CTAs are counted on CTA 0's barrier.
          const uint32_t full_addr = map_to_cta(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * kPairStageBytes);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const int k0 = (kb * KSUB + sub) * kStageK;
            uint8_t* a_dst = stages + static_cast<size_t>(stage) * kPairStageBytes + sub * kPairSubBytes;
            uint8_t* b_dst = a_dst + kASlabBytes;
            tma_load_2d_pair(a_dst, &p.map_a, full_addr, k0, row0);
            if (p.b_strips == kPairN / 2 / 32) {
              tma_load_3d_pair(b_dst, &p.map_b_strips, full_addr, 0, k0, col0 / 32);
            } else {
#pragma unroll
              for (int j = 0; j < kPairN / 2 / 32; ++j) {
                tma_load_2d_pair(b_dst + j * kBBoxBytes, &p.map_b, full_addr, col0 + j * 32, k0);
              }
            }
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      // Before the first use of half-tile stage 0 .. 3: this many of the whole tiles' slots, in the
      // order they come free, have been read to the end (1 or 2, then 2, 3, 3: see `rotation`).
      int whole_stage = stage, released = 0, first_uses = 0;
      uint32_t whole_phase = phase;
      stage = 0;
      phase = 0;
      for (int item = first_half; item < items && ok; item += tile_stride) {
        const PairItem it = pair_item(item, p.pair_full_tiles);
        int tm, tn;
        tile_coords(it.tile, tiles_m, tiles_n, &tm, &tn);
        const int row0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
        const int col0 = tn * kPairN + it.half * (kPairN / 2) + static_cast<int>(rank) * (kPairN / 4);   // this CTA's 64 columns
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (first_uses < HSTAGES) {
            const int needed = first_uses == 0 ? (oldest == 1 ? 2 : 1) : (first_uses == 1 ? 2 : STAGES);
            for (; released < needed && ok; ++released) {
              ok = mbar_wait(&empty[whole_stage], whole_phase ^ 1u, kSiteUmmaEmpty);
              if (++whole_stage == STAGES) whole_stage = 0, whole_phase ^= 1u;
            }
            ++first_uses;
            if (!ok) break;
          }
          if (!mbar_wait(&half_empty[stage], phase ^ 1u, kSiteUmmaEmpty)) { ok = false; break; }
          const uint32_t full_addr = map_to_cta(smem_u32(&half_full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&half_full[stage], 2 * 2 * kHalfSubBytes);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int k0 = (kb * 2 + sub) * kStageK;
            uint8_t* a_dst = stages + static_cast<size_t>((stage + rotation) % HSTAGES) * (2 * kHalfSubBytes) + sub * kHalfSubBytes;
            uint8_t* b_dst = a_dst + kASlabBytes;
            tma_load_2d_pair(a_dst, &p.map_a, full_addr, k0, row0);
#pragma unroll
            for (int j = 0; j < kPairN / 4 / 32; ++j) {
              tma_load_2d_pair(b_dst + j * kBBoxBytes, &p.map_b, full_addr, col0 + j * 32, k0);
            }
          }
          if (++stage == HSTAGES) stage = 0, phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_whole = umma_idesc_tf32(2 * kTileM, kPairN, /*a_mn_major=*/false, /*b_mn_major=*/true);
      constexpr uint32_t idesc_half = umma_idesc_tf32(2 * kTileM, kPairN / 2, /*a_mn_major=*/false, /*b_mn_major=*/true);
      const SubBlockDescs ring = sub_block_descs(smem_u32(stages));   // of the ring's first sub-block
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      int item = first_tile;
      for (; item < p.pair_full_tiles && ok; item += tile_stride, ++local) {
        const int buf = local & 1;
        const uint32_t use_parity = (local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], use_parity ^ 1u, kSiteUmmaAccEmpty)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + buf * kPairN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) { ok = false; break; }
          tcgen05_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const uint32_t offset = static_cast<uint32_t>(stage) * kPairStageBytes + sub * kPairSubBytes;
#pragma unroll
            for (int j = 0; j < kStageK / kInstK; ++j) {
              umma_tf32_pair(tmem_acc, umma_desc_advance(ring.a, offset + j * (kInstK * 4)),
                             umma_desc_advance(ring.b, offset + j * (kInstK * 128)), idesc_whole,
                             (kb > 0 || sub > 0 || j > 0) ? 1u : 0u);
            }
          }
          // The stage is reusable in both CTAs once these MMAs have read it.
          umma_commit_pair(smem_u32(&empty[stage]));
          umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 1));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) {
          // The accumulator barriers count both threads; a whole tile has only this one's MMAs.
          umma_commit_pair(smem_u32(&acc_full[buf]));
          umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 1));
          mbar_arrive_relaxed(&acc_full[buf]);
          mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&acc_full[buf]), 1));
        }
      }
      stage = 0;
      phase = 0;
      for (; item < items && ok; item += tile_stride, ++local) {
        const int buf = local & 1;
        ok = issue_half_tile<HSTAGES>(half_full, half_empty, &acc_full[buf], &acc_empty[buf], (local >> 1) & 1u, ring, idesc_half,
                                      tmem_base + buf * kPairN, 0, k_blocks, rotation, stage, phase);
      }
    }
  } else if (warp == kSecondIssuerWarp) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_half = umma_idesc_tf32(2 * kTileM, kPairN / 2, /*a_mn_major=*/false, /*b_mn_major=*/true);
      const SubBlockDescs ring = sub_block_descs(smem_u32(stages));
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = whole;
      for (int item = first_half; item < items && ok; item += tile_stride, ++local) {
        const int buf = local & 1;
        ok = issue_half_tile<HSTAGES>(half_full, half_empty, &acc_full[buf], &acc_empty[buf], (local >> 1) & 1u, ring, idesc_half,
                                      tmem_base + buf * kPairN + kPairN / 2, 1, k_blocks, rotation, stage, phase);
      }
    }
  } else {
    const EpilogueArgs ep = epilogue_args(p);
    constexpr int kShare = kTileEpilogueShare;
    const int quarter = warp & 3, part = (warp - 2) >> 2;   // rows of the accumulator, place among the quarter's warps
    bool ok = true;
    int local = 0;
    const bool boxed = p.tma_store != 0 && ep.vector_io && ep.peers.count == 0;
    uint8_t* boxes = reinterpret_cast<uint8_t*>(peer_stage) + (part * 4 + quarter) * (kStagingBytes / (4 * kShare));
    uint32_t box_uses = 0;
    for (int item = first_tile; item < items && ok; item += tile_stride, ++local) {
      const PairItem it = pair_item(item, p.pair_full_tiles);
      const int buf = local & 1;
      const uint32_t use_parity = (local >> 1) & 1u;
      int tm, tn;
      tile_coords(it.tile, tiles_m, tiles_n, &tm, &tn);
      const int n0 = tn * kPairN + (it.half < 0 ? 0 : it.half * (kPairN / 2));
      const int m0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
      // Before the wait: the source of the warp's first chunk, fetched and turned in its box.
      SourceQuads first;
      uint8_t* first_box = nullptr;
      if (boxed) {
        fetch_source_coalesced(ep, first, m0 + quarter * 32, n0 + part * 32, lane);
        first_box = boxes + (box_uses++ % boxes_per_warp<kShare>()) * kOutBoxBytes;
        stage_source_boxed<boxes_per_warp<kShare>()>(ep, first, lane, first_box);
      }
      if (!mbar_wait(&acc_full[buf], use_parity, kSiteUmmaAccFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
      if (it.half < 0) {
        if (boxed) {
          epilogue_tile_boxed<kPairN, kAct, kShare>(p, ep, tmem_base + buf * kPairN, quarter, part, lane, m0, n0, first, boxes,
                                                    box_uses, first_box);
        } else {
          epilogue_tile<kPairN, kAct, kShare>(ep, tmem_base + buf * kPairN, quarter, part, lane, m0, n0, boxes);
        }
      } else if (boxed) {   // a half tile: the sum of the two threads' accumulators
        epilogue_tile_boxed<kPairN / 2, kAct, kShare, kIssuers>(p, ep, tmem_base + buf * kPairN, quarter, part, lane, m0, n0, first,
                                                                boxes, box_uses, first_box);
      } else {
        epilogue_tile<kPairN / 2, kAct, kShare, kIssuers>(ep, tmem_base + buf * kPairN, quarter, part, lane, m0, n0, boxes);
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      // The MMA issuer (CTA 0) waits for the epilogues of both CTAs.
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    if (boxed && lane == 0) tma_store_wait_read<0>();   // every store has read its box (the writes land before the grid completes)
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer may still be signalling this CTA's barriers or reading its operands
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair<512>(tmem_base);
  }
}
// ------------------------------------------- TMA, CTA-pair kernel, 256 x 128 tiles
// The same machinery on 256 x 128 tiles with TWO MMA issuers (mma_role in tf32_umma.cuh says why):
// CTA r of the pair holds rows [128 r, +128) of A and columns [64 r, +64) of B, 24 KiB per 32-wide
// K sub-block where the single-CTA 128 x 128 tile streams 32 KiB for the same share of the product.
// A stage holds two sub-blocks; issuer i (two threads of the even CTA) multiplies sub-block i of
// every stage into accumulator i (128 TMEM columns each, two buffers of two: all 512 columns, which
// is why the 256 x 256 kernel above cannot do the same) and both commit every stage to both CTAs.
// For mid-sized problems with a long K, where the 128 x 128 tile kernel is bound by what an SM takes
// in per K block.
constexpr int kMidN = 128;
constexpr uint32_t kMidSubBytes = kASlabBytes + (kMidN / 2 / 32) * kBBoxBytes;   // 24 KiB per 32 of K and CTA
constexpr int kMidStages = 4;                                                       // of two sub-blocks: 192 KiB
constexpr uint32_t kMidStageBytes = 2 * kMidSubBytes;
constexpr size_t kMidSmemBytes = static_cast<size_t>(kMidStages) * kMidStageBytes + 1024 + 1024 + kStagingBytes;

template <int kAct>
__global__ void __launch_bounds__(kTileThreadsTwoIssuers, 1) umma_pair_mid_kernel(const __grid_constant__ UmmaParams p) {
  constexpr int kIssuers = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(kMidStages) * kMidStageBytes);
  uint64_t* empty = full + kMidStages;
  uint64_t* acc_full = empty + kMidStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint8_t* staging = stages + static_cast<size_t>(kMidStages) * kMidStageBytes + 1024;   // kStagingBytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0: issues the MMAs, 1: peer

  if (threadIdx.x == 0) {
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(p.b_strips == kMidN / 2 / 32 ? &p.map_b_strips : &p.map_b);
    if (p.tma_store != 0) prefetch_tensormap(&p.map_d);
    for (int s = 0; s < kMidStages; ++s) {
      mbar_init(&full[s], 1);           // used in CTA 0 only: one expect_tx arrival, bytes of both CTAs
      mbar_init(&empty[s], kIssuers);   // one tcgen05.commit per issuer and use, sent to each CTA
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], kIssuers);
      mbar_init(&acc_empty[b], 8 * kTileEpilogueShare);  // used in CTA 0 only: the epilogue warps of both CTAs
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair<512>(tmem_ptr);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any remote arrival
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  grid_launch_dependents();   // the next kernel of the stream may set itself up beside this one (not before this
                              // kernel's TMEM is allocated: its CTAs could take the columns first)
  grid_dependency_wait();     // the kernel before this one has completed: global memory may be touched

  const int tiles_m = (p.m + 2 * kTileM - 1) / (2 * kTileM);
  const int tiles_n = (p.n + kMidN - 1) / kMidN;
  const int tiles = tiles_m * tiles_n;
  const int k_blocks = (p.k + 2 * kStageK - 1) / (2 * kStageK);   // stages per tile; K past the end reads as zeros
  const int first_tile = blockIdx.x >> 1, tile_stride = gridDim.x >> 1;
  constexpr int kSecondIssuerWarp = 2 + 4 * kTileEpilogueShare;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < tiles && ok; tile += tile_stride) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        const int row0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
        const int col0 = tn * kMidN + static_cast<int>(rank) * (kMidN / 2);   // this CTA's share of the B columns
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, kSiteUmmaEmpty)) { ok = false; break; }
          // Completion bytes of both CTAs are counted on CTA 0's barrier.
          const uint32_t full_addr = map_to_cta(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * kMidStageBytes);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int k0 = (kb * 2 + sub) * kStageK;
            uint8_t* a_dst = stages + static_cast<size_t>(stage) * kMidStageBytes + sub * kMidSubBytes;
            uint8_t* b_dst = a_dst + kASlabBytes;
            tma_load_2d_pair(a_dst, &p.map_a, full_addr, k0, row0);
            if (p.b_strips == kMidN / 2 / 32) {
              tma_load_3d_pair(b_dst, &p.map_b_strips, full_addr, 0, k0, col0 / 32);
            } else {
#pragma unroll
              for (int j = 0; j < kMidN / 2 / 32; ++j) {
                tma_load_2d_pair(b_dst + j * kBBoxBytes, &p.map_b, full_addr, col0 + j * 32, k0);
              }
            }
          }
          if (++stage == kMidStages) stage = 0, phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 || warp == kSecondIssuerWarp) {
    if (lane == 0 && rank == 0) {
      const uint32_t issuer = warp == 1 ? 0u : 1u;
      constexpr uint32_t idesc = umma_idesc_tf32(2 * kTileM, kMidN, /*a_mn_major=*/false, /*b_mn_major=*/true);
      const SubBlockDescs ring = sub_block_descs(smem_u32(stages));   // of the ring's first sub-block
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = first_tile; tile < tiles && ok; tile += tile_stride, ++local) {
        const int buf = local & 1;
        const uint32_t use_parity = (local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], use_parity ^ 1u, kSiteUmmaAccEmpty)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + (buf * kIssuers + issuer) * kMidN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) { ok = false; break; }
          tcgen05_fence_after_sync();
          const uint32_t offset = static_cast<uint32_t>(stage) * kMidStageBytes + issuer * kMidSubBytes;
#pragma unroll
          for (int j = 0; j < kStageK / kInstK; ++j) {
            umma_tf32_pair(tmem_acc, umma_desc_advance(ring.a, offset + j * (kInstK * 4)),
                           umma_desc_advance(ring.b, offset + j * (kInstK * 128)), idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          // The stage is reusable in both CTAs once both issuers' MMAs have read it.
          umma_commit_pair(smem_u32(&empty[stage]));
          umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 1));
          if (++stage == kMidStages) stage = 0, phase ^= 1u;
        }
        if (ok) {
          umma_commit_pair(smem_u32(&acc_full[buf]));
          umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 1));
        }
      }
    }
  } else {
    constexpr int kShare = kTileEpilogueShare;
    const EpilogueArgs ep = epilogue_args(p);
    const int quarter = warp & 3, part = (warp - 2) >> 2;
    bool ok = true;
    int local = 0;
    const bool boxed = p.tma_store != 0 && ep.vector_io && ep.peers.count == 0;
    uint8_t* boxes = staging + (part * 4 + quarter) * (kStagingBytes / (4 * kShare));
    uint32_t box_uses = 0;
    for (int tile = first_tile; tile < tiles && ok; tile += tile_stride, ++local) {
      const int buf = local & 1;
      const uint32_t use_parity = (local >> 1) & 1u;
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
      const int n0 = tn * kMidN;
      const int m0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
      SourceQuads first;
      uint8_t* first_box = nullptr;
      if (boxed) {   // before the wait
        fetch_source_coalesced(ep, first, m0 + quarter * 32, n0 + part * 32, lane);
        first_box = boxes + (box_uses++ % boxes_per_warp<kShare>()) * kOutBoxBytes;
        stage_source_boxed<boxes_per_warp<kShare>()>(ep, first, lane, first_box);
      }
      if (!mbar_wait(&acc_full[buf], use_parity, kSiteUmmaAccFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + buf * kIssuers * kMidN;
      if (boxed) {
        epilogue_tile_boxed<kMidN, kAct, kShare, kIssuers>(p, ep, tmem_acc, quarter, part, lane, m0, n0, first, boxes, box_uses,
                                                           first_box);
      } else {
        epilogue_tile<kMidN, kAct, kShare, kIssuers>(ep, tmem_acc, quarter, part, lane, m0, n0, boxes);
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      // The MMA issuers (CTA 0) wait for the epilogues of both CTAs.
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    if (boxed && lane == 0) tma_store_wait_read<0>();   // every store has read its box (the writes land before the grid completes)
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer may still be signalling this CTA's barriers or reading its operands
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair<512>(tmem_base);
  }
}

// ------------------------------------------------------------------- launcher

template <int STAGES, int kAct>
int launch_pair(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  constexpr int KSUB = 2;                       // 64 floats of K per stage
  static_assert(STAGES % KSUB == 0, "the registry states the ring depth in 32-wide K blocks");
  auto kernel = umma_pair_kernel<STAGES / KSUB, KSUB, kAct>;
  constexpr size_t smem = pair_smem_bytes<STAGES / KSUB, KSUB>();
  if (!ensure_dynamic_smem<umma_pair_kernel<STAGES / KSUB, KSUB, kAct>, smem>()) return B200_ERR_LAUNCH_FAILED;
  const size_t launch_smem = smem;
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.tma_store = (p.vector_io && make_tensor_map_2d(&p.map_d, q.d, q.m, q.n, q.ldd, 32, 32, Swizzle::k128B)) ? 1 : 0;
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK,
                                                        kPairN / 2 / 32, Swizzle::k128BAtom32B))
                   ? kPairN / 2 / 32
                   : 0;
  const int sms = sm_count();
  if (sms < 2) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + 2 * kTileM - 1) / (2 * kTileM)) * ((q.n + kPairN - 1) / kPairN);
  const int64_t all_pairs = sms / 2;
  // A last round that occupies at most half the pairs is run as 256 x 128 half tiles on twice as
  // many pairs: a half tile streams 24 instead of 32 KiB per K block and CTA and, with its MMAs
  // issued by two threads, takes about 0.6 of a whole tile's time (4096^3: 34 left-over tiles become
  // 68 halves on 74 pairs). A problem with no more tiles than half the pairs is such a last round
  // from the start.
  const int64_t remainder = tiles % all_pairs;
  p.pair_full_tiles = static_cast<int>((remainder != 0 && 2 * remainder <= all_pairs) ? tiles - remainder : tiles);
  const int64_t items = p.pair_full_tiles + 2 * (tiles - p.pair_full_tiles);
  const int64_t pairs = items < all_pairs ? items : all_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(kTileThreadsTwoIssuers);
  cfg.dynamicSmemBytes = launch_smem;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(2);
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}
template <int kAct>
int launch_pair_mid(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  auto kernel = umma_pair_mid_kernel<kAct>;
  if (!ensure_dynamic_smem<umma_pair_mid_kernel<kAct>, kMidSmemBytes>()) return B200_ERR_LAUNCH_FAILED;
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.tma_store = (p.vector_io && make_tensor_map_2d(&p.map_d, q.d, q.m, q.n, q.ldd, 32, 32, Swizzle::k128B)) ? 1 : 0;
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, kMidN / 2 / 32,
                                                        Swizzle::k128BAtom32B))
                   ? kMidN / 2 / 32
                   : 0;
  const int sms = sm_count();
  if (sms < 2) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + 2 * kTileM - 1) / (2 * kTileM)) * ((q.n + kMidN - 1) / kMidN);
  const int64_t all_pairs = sms / 2;
  const int64_t pairs = tiles < all_pairs ? tiles : all_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(kTileThreadsTwoIssuers);
  cfg.dynamicSmemBytes = kMidSmemBytes;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(2);
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}
}  // namespace

int launch_tf32_pair_mid(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  switch (act) {
    case B200_EPILOGUE_LINEAR: return launch_pair_mid<B200_EPILOGUE_LINEAR>(q, peers, stream);
    case B200_EPILOGUE_RELU: return launch_pair_mid<B200_EPILOGUE_RELU>(q, peers, stream);
    case B200_EPILOGUE_GELU: return launch_pair_mid<B200_EPILOGUE_GELU>(q, peers, stream);
    default: return B200_ERR_INVALID_ARGUMENT;
  }
}

int launch_tf32_pair(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  switch (act) {
    case B200_EPILOGUE_LINEAR: return launch_pair<6, B200_EPILOGUE_LINEAR>(q, peers, stream);
    case B200_EPILOGUE_RELU: return launch_pair<6, B200_EPILOGUE_RELU>(q, peers, stream);
    case B200_EPILOGUE_GELU: return launch_pair<6, B200_EPILOGUE_GELU>(q, peers, stream);
    default: return B200_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace b200
