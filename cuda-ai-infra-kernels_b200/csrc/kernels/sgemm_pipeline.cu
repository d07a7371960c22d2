// FP32 SIMT GEMM ladder, stages 6-8, rebuilt for sm_100a: persistent CTAs, a
// multi-stage shared-memory ring filled by TMA bulk-tensor loads, consumer
// warps running the FMA pipe off that ring, full/empty mbarrier pairs instead
// of block-wide barriers.
//
//   prefetch_smem : the ring alone (the reference's cp.async double buffer,
//                   csrc/gemm/gemm_prefetchSmem.cu:100-169, becomes N stages);
//                   fragments are loaded where they are used.
//   prefetch_reg  : ring + register double buffer of the shared-memory
//                   fragments carried across stage boundaries, and packed
//                   two-wide FMAs (csrc/gemm/gemm_prefetchRegister.cu:125-190).
//   split_k       : prefetch_reg with K split across CTAs and the partial sums
//                   reduced with 128-bit vector reductions into an output that
//                   the launcher clears on the same stream. The reference cuts
//                   every tile's K in two (csrc/gemm/gemm_splictK.cu:101-209) to
//                   balance waves; here the whole (tile, k block) iteration
//                   space is cut into one equal range per CTA (stream-K), which
//                   balances any shape.
//
// Few tiles, long K (fewer 128 x 128 tiles than SMs): prefetch_smem and prefetch_reg launch clusters
// of 2 or 4 CTAs per tile, each CTA runs an equal share of the K blocks, and the partial tiles of
// ranks 1.. travel through distributed shared memory into rank 0's idle operand ring, where they
// are added in rank order before the one store of the tile. No atomics, no cleared output, the
// same bits every run; 1024^3 runs on 128 SMs instead of 64.
//
// Layout in shared memory per stage: A slab [BK][128] (row kk = 128 consecutive
// m of storage row k) and B slab [BK][128]; both arrive exactly as one TMA box.
// K tails are handled by the tensor maps: rows past K read as zeros.
//
// What bounds the kernel: a 128-bit shared-memory load costs four cycles of the
// SM's single shared-memory pipe whatever its addresses, and with 8 x 8
// outputs per thread the loads of one k (4 per warp) take exactly as long as
// its FMAs. 8 x 16 outputs per thread cut that to three quarters; they need
// ~200 registers, which an SM sub-partition can give to two warps only, so
// that configuration runs four consumer warps per CTA, two CTAs per SM, and no
// separate producer warp (lane 0 of warp 0 issues the TMA loads a few stages
// ahead of the warps that consume them).
#include <atomic>

#include "sgemm.h"
#include "ptx_sm100.cuh"

namespace b200 {

cudaError_t sgemm_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

constexpr int kTile = 128;  // CTA tile is kTile x kTile

struct PipelineParams {
  CUtensorMap map_a;  // [K][M] view of A storage, boxes {128 m, BK k}
  CUtensorMap map_b;  // [K][N] view of B, boxes {128 n, BK k}
  float* c;
  PeerOutputs peers;  // further destinations of every output tile (fused all-gather), usually none
  int n;
  int tiles_m, tiles_n;
  int k_blocks;       // ceil(K / BK)
};

// Work decomposition of the consumer warps. Inside a warp the lanes form an
// 8 (rows) x 4 (columns) grid; a thread owns RM x RN register blocks of 4 x 4,
// row blocks 32 apart and column blocks 16 apart, so a warp covers
// (32 * RM) x (16 * RN) outputs and every 128-bit shared-memory load of a warp
// touches one contiguous 128-byte (A) or 64-byte (B) span.
//   RM = 2, RN = 2: 64 x 32 warp tiles, 2 x 4 = 8 consumer warps (8 x 8 per thread)
//   RM = 2, RN = 4: 64 x 64 warp tiles, 2 x 2 = 4 consumer warps (8 x 16 per thread);
//                   a quarter fewer shared-memory bytes per FMA.
template <int RM_, int RN_, bool kProducerWarp_ = true>
struct WarpGrid {
  static constexpr int RM = RM_, RN = RN_;
  static constexpr bool kProducerWarp = kProducerWarp_;
  static constexpr int kWarpsM = kTile / (32 * RM), kWarpsN = kTile / (16 * RN);
  static constexpr int kConsumerWarps = kWarpsM * kWarpsN;
  static constexpr int kConsumerThreads = kConsumerWarps * 32;
  static constexpr int kThreads = kConsumerThreads + (kProducerWarp ? 32 : 0);
};

template <int BK, int STAGES>
struct SmemLayout {
  static constexpr int kSlabFloats = BK * kTile;
  static constexpr uint32_t kStageBytes = 2u * kSlabFloats * sizeof(float);
  static constexpr size_t kBytes = static_cast<size_t>(STAGES) * kStageBytes + 2 * STAGES * sizeof(uint64_t) + 1024;
};

__device__ __forceinline__ float4 lds128(const float* p) { return *reinterpret_cast<const float4*>(p); }

__device__ __forceinline__ void red_add_v4(float* dst, float x, float y, float z, float w) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

// Grouped raster order: tiles are walked in bands of eight tile rows so that
// the CTAs running at any moment share a small set of A and B slabs in L2.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int* tm, int* tn) {
  constexpr int kBand = 8;
  const int per_band = kBand * tiles_n;
  const int band = tile / per_band;
  const int first_m = band * kBand;
  const int band_rows = min(kBand, tiles_m - first_m);
  const int in_band = tile - band * per_band;
  *tm = first_m + in_band % band_rows;
  *tn = in_band / band_rows;
}

// Fragment of one k: 4 * RM values of A and 4 * RN values of B.
template <int RM, int RN>
struct Fragment {
  float4 a[RM];
  float4 b[RN];
};

template <int RM, int RN>
__device__ __forceinline__ void load_fragment(Fragment<RM, RN>& f, const float* a_slab, const float* b_slab, int kk) {
#pragma unroll
  for (int r = 0; r < RM; ++r) f.a[r] = lds128(a_slab + kk * kTile + 32 * r);
#pragma unroll
  for (int c = 0; c < RN; ++c) f.b[c] = lds128(b_slab + kk * kTile + 16 * c);
}

// acc[i][j] += a[i] * b[j] over the (4 RM) x (4 RN) register tile.
template <bool kPacked, int RM, int RN>
__device__ __forceinline__ void outer_product(float (&acc)[4 * RM][4 * RN], const Fragment<RM, RN>& f) {
  float a[4 * RM];
#pragma unroll
  for (int r = 0; r < RM; ++r) a[4 * r] = f.a[r].x, a[4 * r + 1] = f.a[r].y, a[4 * r + 2] = f.a[r].z, a[4 * r + 3] = f.a[r].w;
  if constexpr (kPacked) {
    // fma.rn.f32x2: one instruction, two FMAs, half the issue slots. B supplies
    // natural pairs, A is broadcast into both halves.
    float2 b2[2 * RN];
#pragma unroll
    for (int c = 0; c < RN; ++c) b2[2 * c] = make_float2(f.b[c].x, f.b[c].y), b2[2 * c + 1] = make_float2(f.b[c].z, f.b[c].w);
#pragma unroll
    for (int i = 0; i < 4 * RM; ++i) {
      const float2 a2 = make_float2(a[i], a[i]);
#pragma unroll
      for (int j = 0; j < 2 * RN; ++j) {
        float2& d = *reinterpret_cast<float2*>(&acc[i][2 * j]);
        d = __ffma2_rn(a2, b2[j], d);
      }
    }
  } else {
    float b[4 * RN];
#pragma unroll
    for (int c = 0; c < RN; ++c) b[4 * c] = f.b[c].x, b[4 * c + 1] = f.b[c].y, b[4 * c + 2] = f.b[c].z, b[4 * c + 3] = f.b[c].w;
#pragma unroll
    for (int i = 0; i < 4 * RM; ++i)
#pragma unroll
      for (int j = 0; j < 4 * RN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// A run of consecutive k blocks of one output tile.
struct Segment {
  int tile;
  int kb_begin, kb_end;
};

// Hands a CTA its segments. Two schedules:
//   whole tiles - tile = blockIdx.x, + gridDim.x, ...; every segment is a full K
//                 range and its result is stored;
//   stream-K    - the (tile, k block) iteration space is cut into gridDim.x
//                 equal contiguous ranges, so every CTA does the same number of
//                 k blocks whatever the tile count; a range covers the tail of
//                 one tile, some whole tiles and the head of another, and every
//                 segment is reduced into the output.
// Producer and consumers walk identical copies.
//   cluster split - (kSplit > 1) one tile per cluster of kSplit CTAs; CTA rank r owns the r-th of
//                 kSplit equal shares of the K blocks; a single segment per CTA.
template <bool kStreamK, int kSplit = 1>
struct WorkIterator {
  int k_blocks;
  int tile, tile_end, tile_stride;  // whole tiles
  int64_t it, it_end;               // stream-K

  __device__ WorkIterator(int tiles, int k_blocks_) : k_blocks(k_blocks_) {
    if constexpr (kSplit > 1) {
      tile = blockIdx.x / kSplit, tile_end = tiles, tile_stride = 0;
      it = it_end = 0;
    } else if constexpr (kStreamK) {
      const int64_t total = static_cast<int64_t>(tiles) * k_blocks;
      it = total * blockIdx.x / gridDim.x;
      it_end = total * (blockIdx.x + 1) / gridDim.x;
      tile = tile_end = tile_stride = 0;
    } else {
      tile = blockIdx.x, tile_end = tiles, tile_stride = gridDim.x;
      it = it_end = 0;
    }
  }

  __device__ bool next(Segment* s) {
    if constexpr (kSplit > 1) {
      if (tile >= tile_end) return false;
      const int rank = static_cast<int>(cluster_cta_rank());
      s->tile = tile;
      s->kb_begin = k_blocks * rank / kSplit, s->kb_end = k_blocks * (rank + 1) / kSplit;
      tile = tile_end;   // one segment only
      return true;
    } else if constexpr (kStreamK) {
      if (it >= it_end) return false;
      s->tile = static_cast<int>(it / k_blocks);
      s->kb_begin = static_cast<int>(it - static_cast<int64_t>(s->tile) * k_blocks);
      const int64_t room = it_end - it;
      s->kb_end = room < k_blocks - s->kb_begin ? s->kb_begin + static_cast<int>(room) : k_blocks;
      it += s->kb_end - s->kb_begin;
      return true;
    } else {
      if (tile >= tile_end) return false;
      s->tile = tile, s->kb_begin = 0, s->kb_end = k_blocks;
      tile += tile_stride;
      return true;
    }
  }
};

// Position of the TMA producer: its own copy of the work iterator plus the
// ring slot it fills next.
template <bool kStreamK, int kSplit = 1>
struct ProducerCursor {
  WorkIterator<kStreamK, kSplit> work;
  Segment seg{0, 0, 0};
  int kb = 0;
  int tm = 0, tn = 0;
  bool active;
  int stage = 0;
  uint32_t phase = 0;

  __device__ ProducerCursor(const PipelineParams& p) : work(p.tiles_m * p.tiles_n, p.k_blocks) { advance_segment(p); }

  __device__ void advance_segment(const PipelineParams& p) {
    active = work.next(&seg);
    if (active) {
      kb = seg.kb_begin;
      tile_coords(seg.tile, p.tiles_m, p.tiles_n, &tm, &tn);
    }
  }
};

// Issues the loads of the cursor's stage and advances it. Returns false only
// when the bounded wait for a free stage expired.
template <int BK, int STAGES, bool kStreamK, int kSplit>
__device__ __forceinline__ bool produce_stage(const PipelineParams& p, ProducerCursor<kStreamK, kSplit>& c, float* slabs,
                                              uint64_t* full_bar, uint64_t* empty_bar) {
  using Layout = SmemLayout<BK, STAGES>;
  if (!c.active) return true;  // nothing left to fetch
  // A stage is free once every consumer warp released its previous use.
  if (!mbar_wait(&empty_bar[c.stage], c.phase ^ 1u, kSiteSgemmEmpty)) return false;
  mbar_expect_tx(&full_bar[c.stage], Layout::kStageBytes);
  float* a_slab = slabs + static_cast<size_t>(c.stage) * 2 * Layout::kSlabFloats;
  tma_load_2d(a_slab, &p.map_a, &full_bar[c.stage], c.tm * kTile, c.kb * BK);
  tma_load_2d(a_slab + Layout::kSlabFloats, &p.map_b, &full_bar[c.stage], c.tn * kTile, c.kb * BK);
  if (++c.stage == STAGES) c.stage = 0, c.phase ^= 1u;
  if (++c.kb == c.seg.kb_end) c.advance_segment(p);
  return true;
}


template <class Grid, int BK, int STAGES, bool kRegPrefetch, bool kPacked, bool kStreamK, int kCtasPerSm, bool kGather,
          int kSplit = 1>
__global__ void __launch_bounds__(Grid::kThreads, kCtasPerSm) sgemm_pipeline_kernel(const __grid_constant__ PipelineParams p) {
  using Layout = SmemLayout<BK, STAGES>;
  static_assert(kSplit == 1 || (!kStreamK && !kGather && Grid::kProducerWarp), "the cluster split stores each tile once, locally");
  static_assert(kSplit == 1 || static_cast<size_t>(kSplit - 1) * kTile * kTile * sizeof(float) <= STAGES * Layout::kStageBytes,
                "the partial tiles of ranks 1.. must fit rank 0's operand ring");
  constexpr int RM = Grid::RM, RN = Grid::RN;
  constexpr bool kInlineProducer = !Grid::kProducerWarp;
  // An inline producer runs this many stages ahead of warp 0. Two stages of
  // slack mean the stage it refills was released an iteration ago by the
  // slowest warp, so its wait is normally already satisfied.
  constexpr int kLookahead = STAGES - 2;
  static_assert(!kInlineProducer || STAGES >= 4, "inline producer needs a ring of at least four stages");
  extern __shared__ uint8_t smem_raw[];
  // TMA destinations want generous alignment; the dynamic window is only
  // guaranteed to 16 bytes.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* slabs = reinterpret_cast<float*>(smem);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(STAGES) * Layout::kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;

  const int tid = threadIdx.x;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);                      // one arrive.expect_tx from the producer
      mbar_init(&empty_bar[s], Grid::kConsumerWarps);  // one arrive per consumer warp
    }
    mbar_init_fence();
  }
  __syncthreads();
  // Launched under programmatic stream serialization (gemm_launch_attributes): the kernel after
  // this one in the stream may be scheduled from here on, and this one touches global memory only
  // once the kernel before it has completed.
  grid_launch_dependents();
  grid_dependency_wait();

  if (Grid::kProducerWarp && tid >= Grid::kConsumerThreads) {
    // ------------------------------------------------- dedicated producer warp
    if (tid != Grid::kConsumerThreads) return;
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(&p.map_b);
    ProducerCursor<kStreamK, kSplit> cursor(p);
    while (cursor.active) {
      if (!produce_stage<BK, STAGES>(p, cursor, slabs, full_bar, empty_bar)) return;
    }
    return;   // (an exited thread does not take part in the cluster barriers below)
  }

  // ---------------------------------------------------------------- consumers
  const int warp = tid >> 5, lane = tid & 31;
  const int row0 = (warp / Grid::kWarpsN) * (32 * RM) + (lane >> 2) * 4;
  const int col0 = (warp % Grid::kWarpsN) * (16 * RN) + (lane & 3) * 4;

  const bool produces = kInlineProducer && tid == 0;
  ProducerCursor<kStreamK, kSplit> cursor(p);
  if (produces) {
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(&p.map_b);
#pragma unroll 1
    for (int i = 0; i < kLookahead; ++i) {
      if (!produce_stage<BK, STAGES>(p, cursor, slabs, full_bar, empty_bar)) return;
    }
  }

  int stage = 0;
  uint32_t phase = 0;
  WorkIterator<kStreamK, kSplit> work(p.tiles_m * p.tiles_n, p.k_blocks);
  Segment seg;
  while (work.next(&seg)) {
    int tm, tn;
    tile_coords(seg.tile, p.tiles_m, p.tiles_n, &tm, &tn);
    const int seg_blocks = seg.kb_end - seg.kb_begin;

    float acc[4 * RM][4 * RN];
#pragma unroll
    for (int i = 0; i < 4 * RM; ++i)
#pragma unroll
      for (int j = 0; j < 4 * RN; ++j) acc[i][j] = 0.f;

    if constexpr (kRegPrefetch) {
      Fragment<RM, RN> frag[2];
      if (!mbar_wait(&full_bar[stage], phase, kSiteSgemmFull)) return;
      const float* a_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + row0;
      const float* b_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + Layout::kSlabFloats + col0;
      load_fragment(frag[0], a_slab, b_slab, 0);
      for (int kb = 0; kb < seg_blocks; ++kb) {
        if (produces) {
          if (!produce_stage<BK, STAGES>(p, cursor, slabs, full_bar, empty_bar)) return;
        }
        const int this_stage = stage;
        if (++stage == STAGES) stage = 0, phase ^= 1u;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
          if (kk + 1 < BK) {
            load_fragment(frag[(kk + 1) & 1], a_slab, b_slab, kk + 1);
          } else if (kb + 1 < seg_blocks) {
            // First fragment of the next stage is fetched before the last
            // k of this one is multiplied.
            if (!mbar_wait(&full_bar[stage], phase, kSiteSgemmFull)) return;
            a_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + row0;
            b_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + Layout::kSlabFloats + col0;
            load_fragment(frag[(kk + 1) & 1], a_slab, b_slab, 0);
          }
          outer_product<kPacked>(acc, frag[kk & 1]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[this_stage]);
      }
    } else {
      for (int kb = 0; kb < seg_blocks; ++kb) {
        if (produces) {
          if (!produce_stage<BK, STAGES>(p, cursor, slabs, full_bar, empty_bar)) return;
        }
        if (!mbar_wait(&full_bar[stage], phase, kSiteSgemmFull)) return;
        const float* a_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + row0;
        const float* b_slab = a_slab - row0 + Layout::kSlabFloats + col0;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
          Fragment<RM, RN> f;
          load_fragment(f, a_slab, b_slab, kk);
          outer_product<kPacked>(acc, f);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
    }

    if constexpr (kSplit > 1) {
      // Cluster split: every CTA holds a partial tile. After the first cluster barrier nobody reads
      // an operand ring any more (and every TMA write into one has been consumed), so ranks 1.. copy
      // their accumulators into rank 0's ring, laid out [rank - 1][value quad][thread] so that a warp
      // writes 512 contiguous bytes; after the second barrier rank 0 adds them in rank order.
      // (A wait that ran out above has returned early: the barriers below are reached by all
      // consumer threads or, after such a failure, the kernel ends on its bounded waits.)
      constexpr int kQuads = RM * RN * 4;   // float4 values per thread
      const uint32_t rank = cluster_cta_rank();
      cluster_sync_all();
      if (rank != 0) {
        const uint32_t remote = map_to_cta(smem_u32(slabs), 0) +
                                ((rank - 1) * kQuads * Grid::kConsumerThreads + tid) * static_cast<uint32_t>(sizeof(float4));
#pragma unroll
        for (int i = 0; i < 4 * RM; ++i)
#pragma unroll
          for (int cb = 0; cb < RN; ++cb) {
            st_shared_cluster_v4(remote + (i * RN + cb) * Grid::kConsumerThreads * static_cast<uint32_t>(sizeof(float4)),
                                 __float_as_uint(acc[i][4 * cb]), __float_as_uint(acc[i][4 * cb + 1]),
                                 __float_as_uint(acc[i][4 * cb + 2]), __float_as_uint(acc[i][4 * cb + 3]));
          }
      }
      cluster_sync_all();
      if (rank != 0) return;
      const float4* parts = reinterpret_cast<const float4*>(slabs) + tid;
#pragma unroll 1
      for (int r = 1; r < kSplit; ++r) {
#pragma unroll
        for (int i = 0; i < 4 * RM; ++i)
#pragma unroll
          for (int cb = 0; cb < RN; ++cb) {
            const float4 v = parts[((r - 1) * kQuads + i * RN + cb) * Grid::kConsumerThreads];
            acc[i][4 * cb] += v.x, acc[i][4 * cb + 1] += v.y, acc[i][4 * cb + 2] += v.z, acc[i][4 * cb + 3] += v.w;
          }
      }
    }

    // Epilogue straight from registers: every store instruction of a warp
    // covers eight rows x 64 contiguous bytes. Stream-K segments are partial
    // sums and are reduced into the cleared output instead.
    const int64_t tile_offset = static_cast<int64_t>(tm * kTile + row0) * p.n + tn * kTile + col0;
    // Destination 0 is this GPU's output; the others (fused all-gather) are the
    // same tile in peer GPUs' buffers, written with the same plain stores.
    // (kGather is a template flag so that the plain GEMM keeps a straight-line epilogue.)
    const int destinations = kGather ? 1 + p.peers.count : 1;
    for (int dest = 0; dest < destinations; ++dest) {
      float* c_tile = (dest == 0 ? p.c : p.peers.ptr[dest - 1]) + tile_offset;
#pragma unroll
      for (int rb = 0; rb < RM; ++rb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float* c_row = c_tile + static_cast<int64_t>(rb * 32 + i) * p.n;
          const float* v = acc[rb * 4 + i];
#pragma unroll
          for (int cb = 0; cb < RN; ++cb) {
            if (!B200_IN_BOUNDS(c_row + 16 * cb >= c_tile - tile_offset &&
                                c_row + 16 * cb + 4 <= c_tile - tile_offset + static_cast<int64_t>(p.tiles_m) * kTile * p.n)) {
              continue;
            }
            if constexpr (!kStreamK) {
              *reinterpret_cast<float4*>(c_row + 16 * cb) = make_float4(v[4 * cb], v[4 * cb + 1], v[4 * cb + 2], v[4 * cb + 3]);
            } else {
              red_add_v4(c_row + 16 * cb, v[4 * cb], v[4 * cb + 1], v[4 * cb + 2], v[4 * cb + 3]);
            }
          }
        }
    }
  }
}

// Clusters of `split` CTAs of the split kernel that the device keeps resident at once (cached per
// device; 0 when the query fails).
template <auto kKernel, size_t kSmem, int kThreads>
int max_resident_clusters(int split) {
  static std::atomic<int> cache[64][3];   // [device][log2 split], 0 = not asked yet
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  const int slot = split == 2 ? 1 : split == 4 ? 2 : 0;
  const int cached = cache[device][slot].load(std::memory_order_relaxed);
  if (cached != 0) return cached > 0 ? cached : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(split) * 64);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(split);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kKernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    clusters = 0;
  }
  cache[device][slot].store(clusters > 0 ? clusters : -1, std::memory_order_relaxed);
  return clusters;
}

// One tile per cluster of kSplit CTAs, K shared out over the ranks (see the kernel).
template <class Grid, int BK, int STAGES, bool kRegPrefetch, bool kPacked, int kSplit>
int launch_cluster_split(const PipelineParams& p, cudaStream_t stream) {
  using Layout = SmemLayout<BK, STAGES>;
  constexpr auto kernel = sgemm_pipeline_kernel<Grid, BK, STAGES, kRegPrefetch, kPacked, false, 1, false, kSplit>;
  if (!ensure_dynamic_smem<kernel, Layout::kBytes>()) return B200_ERR_LAUNCH_FAILED;
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * kSplit));
  cfg.blockDim = dim3(Grid::kThreads);
  cfg.dynamicSmemBytes = Layout::kBytes;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(kSplit);
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

// How many CTAs should share a tile's K range: the split with the fewest K blocks per CTA (plus the
// exchange, about 1.5 K blocks of 64) among those whose clusters are all resident at once. Splits
// that need more than one wave of clusters were measured and lose: 1024 x 4096 x 4096 (256 tiles)
// as 512 half-K CTAs took 655 us against 626 us for one persistent CTA per SM - every CTA of a
// split launch pays its own prologue and pipeline fill, and a wave of clusters only starts when
// whole clusters' worth of SMs are free. 1024^3 (64 tiles, 16 K blocks): two CTAs per tile on 128
// SMs, 80.7 -> 46.5 us; 512 x 512 x 4096: four per tile.
inline int choose_split(int64_t tiles, int k_blocks, int max_clusters2, int max_clusters4) {
  constexpr double kExchange = 1.5;
  double best = static_cast<double>(k_blocks);
  int split = 1;
  for (int s = 2; s <= 4; s *= 2) {
    if (k_blocks / s < 2) break;                                  // every rank keeps at least two K blocks
    if (tiles > (s == 2 ? max_clusters2 : max_clusters4)) break;  // all clusters resident at once
    const double cost = static_cast<double>(k_blocks) / s + kExchange;
    if (cost < best * 0.97) best = cost, split = s;               // a tie goes to the simpler launch
  }
  return split;
}

template <class Grid, int BK, int STAGES, bool kRegPrefetch, bool kPacked, bool kStreamK, int kCtasPerSm>
int launch_pipeline(const float* a, const float* b, float* c, const PeerOutputs& peers, int m, int n, int k,
                    cudaStream_t stream) {
  using Layout = SmemLayout<BK, STAGES>;
  if (kStreamK && peers.count > 0) return B200_ERR_NOT_SUPPORTED;   // partial sums need a cleared output
  constexpr auto kFanOut = sgemm_pipeline_kernel<Grid, BK, STAGES, kRegPrefetch, kPacked, kStreamK, kCtasPerSm, !kStreamK>;
  constexpr auto kLocal = sgemm_pipeline_kernel<Grid, BK, STAGES, kRegPrefetch, kPacked, kStreamK, kCtasPerSm, false>;
  const bool fan_out = !kStreamK && peers.count > 0;
  auto kernel = fan_out ? kFanOut : kLocal;
  if (!(fan_out ? ensure_dynamic_smem<kFanOut, Layout::kBytes>() : ensure_dynamic_smem<kLocal, Layout::kBytes>())) {
    return B200_ERR_LAUNCH_FAILED;
  }
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;

  PipelineParams p;
  // Rows past K read as zeros, which takes care of a K that is not a multiple
  // of the ring's stage depth.
  if (!make_tensor_map_2d(&p.map_a, a, k, m, m, BK, kTile, Swizzle::kNone) ||
      !make_tensor_map_2d(&p.map_b, b, k, n, n, BK, kTile, Swizzle::kNone)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.c = c;
  p.peers = peers;
  p.n = n;
  p.tiles_m = m / kTile;
  p.tiles_n = n / kTile;
  p.k_blocks = (k + BK - 1) / BK;

  if (kStreamK) {
    if (cudaMemsetAsync(c, 0, static_cast<size_t>(m) * n * sizeof(float), stream) != cudaSuccess) {
      return launch_failed();
    }
  }
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if constexpr (!kStreamK && kCtasPerSm == 1 && Grid::kProducerWarp) {
    // Tiles that fill the SMs badly: clusters of 2 or 4 CTAs share each tile's K range.
    if (!fan_out) {
      constexpr auto kSplit2 = sgemm_pipeline_kernel<Grid, BK, STAGES, kRegPrefetch, kPacked, false, 1, false, 2>;
      constexpr auto kSplit4 = sgemm_pipeline_kernel<Grid, BK, STAGES, kRegPrefetch, kPacked, false, 1, false, 4>;
      if (!ensure_dynamic_smem<kSplit2, Layout::kBytes>() || !ensure_dynamic_smem<kSplit4, Layout::kBytes>()) {
        return B200_ERR_LAUNCH_FAILED;
      }
      const int split = tiles >= sms ? 1
                                     : choose_split(tiles, p.k_blocks, max_resident_clusters<kSplit2, Layout::kBytes, Grid::kThreads>(2),
                                                    max_resident_clusters<kSplit4, Layout::kBytes, Grid::kThreads>(4));
      if (split == 4) return launch_cluster_split<Grid, BK, STAGES, kRegPrefetch, kPacked, 4>(p, stream);
      if (split == 2) return launch_cluster_split<Grid, BK, STAGES, kRegPrefetch, kPacked, 2>(p, stream);
    }
  }
  const int64_t units = kStreamK ? tiles * p.k_blocks : tiles;
  const int64_t slots = static_cast<int64_t>(sms) * kCtasPerSm;
  const int grid = static_cast<int>(units < slots ? units : slots);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(Grid::kThreads);
  cfg.dynamicSmemBytes = Layout::kBytes;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(1);
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

}  // namespace

int sgemm_pipeline_launch(int impl, const float* a, const float* b, float* c, const PeerOutputs& peers, int m, int n,
                          int k, cudaStream_t stream) {
  // Ring shapes come from a sweep on B200 at 4096^3: deeper stages amortise the
  // per-stage barrier traffic (58 -> 62 -> 63 TFLOP/s for 16 -> 32 -> 64 floats
  // of K per stage with 8 x 8 thread tiles). Larger thread tiles (a quarter
  // fewer shared-memory bytes per FMA) measured slower and are kept out of the
  // dispatch: 8 x 16 with an inline producer at two CTAs per SM 50 TFLOP/s;
  // 8 x 16 or 16 x 8 with four consumer warps + producer at 255 registers
  // 40-45 TFLOP/s (one warp per scheduler cannot keep the FMA pipe fed).
  switch (impl) {
    case B200_SGEMM_PREFETCH_SMEM:
      return launch_pipeline<WarpGrid<2, 2>, 64, 3, false, true, false, 1>(a, b, c, peers, m, n, k, stream);
    case B200_SGEMM_PREFETCH_REG:
      return launch_pipeline<WarpGrid<2, 2>, 64, 3, true, true, false, 1>(a, b, c, peers, m, n, k, stream);
    case B200_SGEMM_SPLIT_K:
      return launch_pipeline<WarpGrid<2, 2>, 64, 3, true, true, true, 1>(a, b, c, peers, m, n, k, stream);
    default:
      return B200_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace b200
