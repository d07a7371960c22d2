// TF32 tensor-core GEMM, kernels whose cluster splits K and meets in distributed shared memory:
// the 128 x 128 split-K tile kernel and the operand-swapped kernel for few rows, with their
// planners. Layouts, the parameter block and the epilogue pieces are in tf32_umma.cuh.
#include <atomic>

#include "tf32_umma.cuh"

namespace b200 {

cudaError_t tf32_cluster_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

// ------------------------------------------------ TMA, split-K cluster kernel
// For problems with too few 128 x 128 output tiles to occupy the SMs (few rows,
// or small M x N with a long K): the 1, 2, 4 or 8 CTAs of a cluster share one
// output tile and each reduces a contiguous range of K blocks into its own TMEM
// accumulator (same producer / MMA roles as above, one tile per CTA, up to
// two CTAs per SM). The partial tiles then meet in shared memory across the cluster:
//   1. cluster barrier: every main loop is finished, so every operand ring is
//      idle and becomes the exchange buffer;
//   2. each epilogue thread (one accumulator row) sends the columns
//      [r * W, (r + 1) * W), W = 128 / cluster, of its partial row to CTA r
//      (distributed-shared-memory stores), rows outside the matrix are skipped;
//   3. cluster barrier; CTA r adds the partials of its W columns in rank order
//      (a fixed order: results do not depend on timing) and applies the fused
//      epilogue. No scratch buffer, no atomics, no second launch.
namespace cg = cooperative_groups;

constexpr int kSplitN = 128;

// Scaling, source, bias and activation for four adjacent outputs of one row.
template <int kAct>
__device__ __forceinline__ void finish_quad(const EpilogueArgs& p, int row, int col, float4 acc) {
  float v[4] = {p.alpha * acc.x, p.alpha * acc.y, p.alpha * acc.z, p.alpha * acc.w};
  const float* c_row = p.c + static_cast<int64_t>(row) * p.ldc;
  float* d_row = p.d + static_cast<int64_t>(row) * p.ldd;
  if (p.vector_io) {  // n % 4 == 0: the quad is inside the matrix as a whole
    if (p.beta != 0.f) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(c_row + col));
      v[0] = fmaf(p.beta, s.x, v[0]), v[1] = fmaf(p.beta, s.y, v[1]);
      v[2] = fmaf(p.beta, s.z, v[2]), v[3] = fmaf(p.beta, s.w, v[3]);
    }
    if (p.bias != nullptr) {
      const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col));
      v[0] += bv.x, v[1] += bv.y, v[2] += bv.z, v[3] += bv.w;
    }
    const float4 out = make_float4(activate<kAct>(v[0]), activate<kAct>(v[1]), activate<kAct>(v[2]), activate<kAct>(v[3]));
    *reinterpret_cast<float4*>(d_row + col) = out;
    store_peers(p, static_cast<int64_t>(row) * p.ldd + col, out);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (col + e < p.n) {
        float out = v[e];
        if (p.beta != 0.f) out = fmaf(p.beta, __ldg(c_row + col + e), out);
        if (p.bias != nullptr) out += __ldg(p.bias + col + e);
        out = activate<kAct>(out);
        d_row[col + e] = out;
        store_peers(p, static_cast<int64_t>(row) * p.ldd + col + e, out);
      }
    }
  }
}

// Exchange buffer of a CTA: float4 elements [source][column quad of its share][row], kExchangePitch
// elements per (source, quad). Senders own a row each, so a warp writes 32 consecutive elements;
// the finishing pass reads row-wise (lanes = adjacent quads of one row) and the odd pitch spreads
// those reads over the banks.
constexpr int kExchangePitch = kTileM + 1;

// Step 2 of the split-K kernels for one epilogue thread (one accumulator row of kCols columns in
// TMEM at `tmem_row`): the columns of share s go to the CTA with cluster rank
// s * rank_stride + rank_offset, into that CTA's buffer for source `my_slice`. The next 32 columns
// are fetched from TMEM while the current ones are being sent; a share is at least 16 columns
// wide, so each half chunk (four quads) has a single destination. `send_chunk` sends one chunk;
// `exchange_addr` is the exchange buffer's shared-window address in this CTA (the same offset in
// every CTA), destinations are 32-bit shared::cluster addresses: a `mapa` and four stores with
// constant offsets per half chunk.
__device__ __forceinline__ void send_chunk(const uint32_t (&cur)[32], int chunk, uint32_t exchange_addr, int my_slice,
                                           int quads_log2, int rank_stride, int rank_offset, int row_in_tile) {
  const int quads = 1 << quads_log2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int quad0 = chunk * 8 + half * 4;
    const int dest_slice = quad0 >> quads_log2, local_quad0 = quad0 & (quads - 1);
    const uint32_t dst = map_to_cta(exchange_addr, static_cast<uint32_t>(dest_slice * rank_stride + rank_offset)) +
                         static_cast<uint32_t>((my_slice * quads + local_quad0) * kExchangePitch + row_in_tile) *
                             static_cast<uint32_t>(sizeof(float4));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = half * 16 + j * 4;
      st_shared_cluster_v4(dst + j * kExchangePitch * static_cast<uint32_t>(sizeof(float4)), cur[e + 0], cur[e + 1], cur[e + 2],
                           cur[e + 3]);
    }
  }
}

// With kAccumulators == 2 the partial row is the sum of two accumulators kCols columns apart (two
// MMA issuers, see mma_role in tf32_umma.cuh). kShare warps serve each quarter of the rows; warp
// `part` of them sends the 32-column chunks part, part + kShare, ...
template <int kCols, int kAccumulators = 1, int kShare = 1>
__device__ __forceinline__ void send_partial_row(uint32_t tmem_row, bool have_acc, uint32_t exchange_addr, int my_slice,
                                                 int quads_log2, int rank_stride, int rank_offset, int row_in_tile, int part = 0) {
  constexpr int kMine = kCols / 32 / kShare;   // chunks of this warp
  static_assert(kMine >= 2 && kMine % 2 == 0, "chunks are handled in pairs");
  // Two register sets, named rather than indexed so that both stay in registers.
  uint32_t even[32], odd[32];
  if (have_acc) {
    tmem_ld_32x32(tmem_row + part * 32, even);
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) even[e] = odd[e] = 0u;   // an empty K range contributes zeros
  }
#pragma unroll
  for (int i = 0; i < kMine; i += 2) {
    const int chunk = part + i * kShare;
    if (have_acc) {
      tmem_ld_wait();
      if constexpr (kAccumulators == 2) add_partial_accumulator(even, tmem_row + kCols + chunk * 32);
      tmem_ld_32x32(tmem_row + (chunk + kShare) * 32, odd);
    }
    send_chunk(even, chunk, exchange_addr, my_slice, quads_log2, rank_stride, rank_offset, row_in_tile);
    if (have_acc) {
      tmem_ld_wait();
      if constexpr (kAccumulators == 2) add_partial_accumulator(odd, tmem_row + kCols + (chunk + kShare) * 32);
      if (i + 2 < kMine) tmem_ld_32x32(tmem_row + (chunk + 2 * kShare) * 32, even);
    }
    send_chunk(odd, chunk + kShare, exchange_addr, my_slice, quads_log2, rank_stride, rank_offset, row_in_tile);
  }
}

// Step 3 of the split-K kernels for thread t of `threads`: adds the partials of this CTA's column
// share in source order and writes finished rows with lanes along the row, so that C is read and
// D is written in contiguous segments. Only a few warps run this, so four outputs per thread are
// kept in flight to cover the latencies.
template <int kAct>
__device__ __forceinline__ void exchange_finish(const EpilogueArgs& p, const float4* exchange, int sources, int quads_log2,
                                                int row0, int col_base, int t, int threads) {
  constexpr int kBatch = 4;
  const int quads = 1 << quads_log2;
  const int items = kTileM << quads_log2;
  for (int base = t; base < items; base += kBatch * threads) {
    float4 sum[kBatch];
    const float4* src_ptr[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int item = min(base + u * threads, items - 1);   // clamped: a duplicate read, no duplicate write below
      src_ptr[u] = exchange + (item & (quads - 1)) * kExchangePitch + (item >> quads_log2);
      sum[u] = *src_ptr[u];
    }
    for (int src = 1; src < sources; ++src) {
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const float4 v = src_ptr[u][src * quads * kExchangePitch];
        sum[u].x += v.x, sum[u].y += v.y, sum[u].z += v.z, sum[u].w += v.w;
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int item = base + u * threads;
      const int row = row0 + (item >> quads_log2), col = col_base + 4 * (item & (quads - 1));
      if (item < items && row < p.m && col < p.n) finish_quad<kAct>(p, row, col, sum[u]);
    }
  }
}

// The same pass for a share that lies inside the matrix as a whole, with 128-bit rows and neither
// bias nor peer outputs: the case of every large problem, and the one where the finishing pass is
// most of what the split costs. The few warps of this kernel issue a dependent instruction every
// five cycles or so, so the pass is bound by instructions per item: here a thread's items are one
// column quad of rows `first`, `first` + step, ... (threads is a multiple of the quads per row), every
// address advances by a constant, nothing is predicated but the end of the tile, and the source
// quads of the next four items are requested before the current four are finished. The first four
// are requested by `interior_sources` before the exchange. Sums run in source order and the
// arithmetic is finish_quad's: the bits are those of the general pass.
constexpr int kInteriorBatch = 4;

struct InteriorCursor {
  int row;                  // row of the tile of this thread's next item
  int step;                 // rows between consecutive items
  const float4* part;       // first source's partial of that item
  const float* c;           // null when beta == 0
  float* d;
  int64_t c_step, d_step;   // elements per item step
};

__device__ __forceinline__ InteriorCursor interior_cursor(const EpilogueArgs& p, const float4* exchange, int quads_log2,
                                                          int row0, int col_base, int t, int threads) {
  const int quads = 1 << quads_log2;
  const int quad = t & (quads - 1);
  InteriorCursor cur;
  cur.row = t >> quads_log2;
  cur.step = threads >> quads_log2;
  cur.part = exchange + quad * kExchangePitch + cur.row;
  const int col = col_base + 4 * quad;
  cur.c = p.beta != 0.f ? p.c + static_cast<int64_t>(row0 + cur.row) * p.ldc + col : nullptr;
  cur.d = p.d + static_cast<int64_t>(row0 + cur.row) * p.ldd + col;
  cur.c_step = static_cast<int64_t>(cur.step) * p.ldc;
  cur.d_step = static_cast<int64_t>(cur.step) * p.ldd;
  return cur;
}

__device__ __forceinline__ void interior_sources(const InteriorCursor& cur, int first_item, float4 (&out)[kInteriorBatch]) {
#pragma unroll
  for (int u = 0; u < kInteriorBatch; ++u) {
    const bool wanted = cur.c != nullptr && cur.row + (first_item + u) * cur.step < kTileM;
    out[u] = wanted ? __ldg(reinterpret_cast<const float4*>(cur.c + (first_item + u) * cur.c_step))
                    : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <int kAct>
__device__ __forceinline__ void exchange_finish_interior(const EpilogueArgs& p, InteriorCursor cur, float4 (&src)[kInteriorBatch],
                                                         int sources, int quads_log2) {
  const int source_stride = (1 << quads_log2) * kExchangePitch;
#pragma unroll 1
  while (cur.row < kTileM) {
    float4 next[kInteriorBatch];
    interior_sources(cur, kInteriorBatch, next);
    float4 sum[kInteriorBatch];
#pragma unroll
    for (int u = 0; u < kInteriorBatch; ++u) {
      sum[u] = cur.row + u * cur.step < kTileM ? cur.part[u * cur.step] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s = 1; s < sources; ++s) {
#pragma unroll
      for (int u = 0; u < kInteriorBatch; ++u) {
        if (cur.row + u * cur.step < kTileM) {
          const float4 v = cur.part[s * source_stride + u * cur.step];
          sum[u].x += v.x, sum[u].y += v.y, sum[u].z += v.z, sum[u].w += v.w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kInteriorBatch; ++u) {
      if (cur.row + u * cur.step < kTileM) {
        float4 v = make_float4(p.alpha * sum[u].x, p.alpha * sum[u].y, p.alpha * sum[u].z, p.alpha * sum[u].w);
        if (cur.c != nullptr) {
          v.x = fmaf(p.beta, src[u].x, v.x), v.y = fmaf(p.beta, src[u].y, v.y);
          v.z = fmaf(p.beta, src[u].z, v.z), v.w = fmaf(p.beta, src[u].w, v.w);
        }
        *reinterpret_cast<float4*>(cur.d + u * cur.d_step) =
            make_float4(activate<kAct>(v.x), activate<kAct>(v.y), activate<kAct>(v.z), activate<kAct>(v.w));
      }
    }
    cur.row += kInteriorBatch * cur.step;
    cur.part += kInteriorBatch * cur.step;
    if (cur.c != nullptr) cur.c += kInteriorBatch * cur.c_step;
    cur.d += kInteriorBatch * cur.d_step;
#pragma unroll
    for (int u = 0; u < kInteriorBatch; ++u) src[u] = next[u];
  }
}

// STAGES counts 32-wide K blocks of shared memory; KSUB of them form one pipeline stage (two when
// the CTA has its SM to itself and the ring can be twice as large: one barrier round trip per 64 of K).
// With two sub-blocks per stage (the CTA has its SM to itself) two threads issue the MMAs, one
// sub-block and one accumulator each (mma_role in tf32_umma.cuh says why), and eight warps instead
// of four send the partial rows, two per quarter of the rows: sending and finishing are bound by
// instructions per warp (send 2.7 k and finishing pass 2.4 k cycles with four and seven warps).
//   warp 0 producer, warp 1 first issuer, warps 2 .. 1 + 4 share: senders, then the second issuer.
template <int STAGES, int KSUB>
__host__ __device__ constexpr int splitk_issuers() { return KSUB == 2 ? 2 : 1; }
template <int STAGES, int KSUB>
__host__ __device__ constexpr int splitk_send_share() { return KSUB == 2 ? 2 : 1; }
template <int STAGES, int KSUB>
__host__ __device__ constexpr int splitk_threads() {
  return (2 + 4 * splitk_send_share<STAGES, KSUB>() + splitk_issuers<STAGES, KSUB>() - 1) * 32;
}

template <int STAGES, int kAct, int KSUB = 1>
__global__ void __launch_bounds__(splitk_threads<STAGES, KSUB>(), KSUB == 2 ? 1 : 2)
    umma_splitk_kernel(const __grid_constant__ UmmaParams p) {
  constexpr int BN = kSplitN;
  constexpr int kIssuers = splitk_issuers<STAGES, KSUB>();
  constexpr int kShare = splitk_send_share<STAGES, KSUB>();
  constexpr int kThreads = splitk_threads<STAGES, KSUB>();
  constexpr int kSecondIssuerWarp = 2 + 4 * kShare;   // exists only with two issuers
  static_assert(STAGES % KSUB == 0, "whole stages");
  constexpr int kRing = STAGES / KSUB;
  static_assert(static_cast<size_t>(STAGES) * stage_bytes<BN>() >= sizeof(float4) * kExchangePitch * (BN / 4),
                "the idle operand ring must hold one exchanged tile");
  cg::cluster_group cluster = cg::this_cluster();
  const int ranks = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  extern __shared__ uint8_t smem_raw[];
  const SmemCarve sm = carve<BN, STAGES>(smem_raw);
  B200_PROBE(p, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&p.map_a);   // first of all: the fetch is part of the first load's latency
    prefetch_tensormap(p.b_strips == BN / 32 ? &p.map_b_strips : &p.map_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], empty_barrier_arrivals<KSUB, kIssuers>());   // one commit per MMA issuer of the stage
    }
    mbar_init(&sm.acc_full[0], kIssuers);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc<kIssuers * BN>(sm.tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;
  grid_launch_dependents();   // the next kernel of the stream may set itself up beside this one (not before this
                              // kernel's TMEM is allocated: its CTAs could take the columns first)
  grid_dependency_wait();     // the kernel before this one has completed: global memory may be touched
  B200_PROBE(p, 1);

  const int tiles_m = (p.m + kTileM - 1) / kTileM;
  const int tiles_n = (p.n + BN - 1) / BN;
  int tm, tn;
  tile_coords(static_cast<int>(blockIdx.x) / ranks, tiles_m, tiles_n, &tm, &tn);
  const int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages; K past the end reads as zeros
  const int per_rank = (k_blocks + ranks - 1) / ranks;
  const int kb_begin = min(k_blocks, rank * per_rank);
  const int kb_end = min(k_blocks, kb_begin + per_rank);
  const bool has_work = kb_begin < kb_end;   // an empty range contributes zeros
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&sm.empty[stage], phase ^ 1u, kSiteUmmaEmpty)) break;
        mbar_expect_tx(&sm.full[stage], KSUB * stage_bytes<BN>());
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          const int k0 = (kb * KSUB + sub) * kStageK;
          uint8_t* a_dst = sm.stages + static_cast<size_t>(stage * KSUB + sub) * stage_bytes<BN>();
          uint8_t* b_dst = a_dst + kASlabBytes;
          tma_load_2d(a_dst, &p.map_a, &sm.full[stage], k0, tm * kTileM);
          if (p.b_strips == BN / 32) {
            tma_load_3d(b_dst, &p.map_b_strips, &sm.full[stage], 0, k0, tn * (BN / 32));
          } else {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) {
              tma_load_2d(b_dst + j * kBBoxBytes, &p.map_b, &sm.full[stage], tn * BN + j * 32, k0);
            }
          }
        }
        if (++stage == kRing) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1 || warp == kSecondIssuerWarp) {
    if (lane == 0 && has_work) {
      const int issuer = warp == 1 ? 0 : 1;
      const SubBlockDescs ring = sub_block_descs(smem_u32(sm.stages));   // of the ring's first sub-block
      int stage = 0;
      uint32_t phase = 0;
      bool fed = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&sm.full[stage], phase, kSiteUmmaFull)) { fed = false; break; }
        tcgen05_fence_after_sync();
#pragma unroll
        for (int sub = 0; sub < KSUB; sub += kIssuers) {
          const uint32_t offset = static_cast<uint32_t>(stage * KSUB + sub + issuer) * stage_bytes<BN>();
          const SubBlockDescs descs{umma_desc_advance(ring.a, offset), umma_desc_advance(ring.b, offset)};
          issue_stage_mmas<BN>(tmem_base + issuer * BN, descs, (kb > kb_begin || sub > 0) ? 1u : 0u);
        }
        umma_commit(&sm.empty[stage]);   // one arrival per issuer
        if (++stage == kRing) stage = 0, phase ^= 1u;
      }
      if (fed) umma_commit(&sm.acc_full[0]);
    }
  } else if (has_work) {
    ok = mbar_wait(&sm.acc_full[0], 0, kSiteUmmaAccFull);
    tcgen05_fence_after_sync();
  }

  B200_PROBE(p, 2);
  // 1. Every CTA of the cluster is past its main loop.
  tcgen05_fence_before_sync();
  cluster.sync();
  tcgen05_fence_after_sync();

  B200_PROBE(p, 3);
  // Exchange buffer of a CTA: float4 elements [source rank][column quad of its W columns][row]. Rows are
  // innermost so that the 32 lanes of a warp (32 rows) touch 512 contiguous bytes: no bank conflicts
  // on either side.
  float4* exchange = reinterpret_cast<float4*>(sm.stages);
  const int width = BN / ranks;                            // W: 128, 64, 32 or 16 columns per CTA
  const int quads = width / 4;
  const int quarter = warp & 3;
  const int row_in_tile = quarter * 32 + lane;
  const bool warp_rows = tm * kTileM + quarter * 32 < p.m;   // any row of this warp inside the matrix
  const int quads_log2 = 31 - __clz(quads);
  // The finishing pass of a share inside the matrix (see exchange_finish_interior): its first source
  // quads are requested now and arrive during the exchange.
  const EpilogueArgs args = epilogue_args(p);
  const int col_base = tn * BN + rank * width;
  const bool interior = args.vector_io && args.bias == nullptr && args.peers.count == 0 && (tm + 1) * kTileM <= p.m &&
                        col_base + width <= p.n;
  InteriorCursor cursor = interior_cursor(args, exchange, quads_log2, tm * kTileM, col_base, threadIdx.x, kThreads);
  float4 first_sources[kInteriorBatch];
  if (interior) interior_sources(cursor, 0, first_sources);
  if (warp >= 2 && warp < kSecondIssuerWarp && warp_rows) {
    // 2. Send this CTA's partial row, W columns to each CTA.
    send_partial_row<BN, kIssuers, kShare>(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16), has_work && ok,
                                           smem_u32(exchange), rank, quads_log2, 1, 0, row_in_tile, (warp - 2) >> 2);
  }
  B200_PROBE(p, 4);
  tcgen05_fence_before_sync();
  cluster.sync();
  B200_PROBE(p, 5);

  // 3. Add the partials of this CTA's columns in rank order and finish them.
  if (interior) {
    exchange_finish_interior<kAct>(args, cursor, first_sources, ranks, quads_log2);
  } else {
    exchange_finish<kAct>(args, exchange, ranks, quads_log2, tm * kTileM, col_base, threadIdx.x, kThreads);
  }

  B200_PROBE(p, 6);
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<kIssuers * BN>(tmem_base);
  }
}

// ------------------------------------------ TMA, CTA-pair split-K cluster kernel
// The split-K kernel above on CTA pairs (tcgen05 cta_group::2) with two MMA issuers: a cluster of
// 2 R CTAs shares one 256 x 128 output tile, pair r = cluster rank / 2 reduces the r-th range of K,
// and within a pair CTA h = rank % 2 holds rows [128 h, +128) of A, columns [64 h, +64) of B and the
// accumulator rows [128 h, +128). Per CTA a 32-wide K block is 16 KiB of A + 8 KiB of B for a
// 128 x 128 share of the product, against 32 KiB in the single-CTA kernel: a quarter fewer operand
// bytes per flop into the SM, which is what the main loop of these few-tile, long-K problems is bound
// by. A stage holds two sub-blocks; issuer i (two threads of the pair's even CTA) multiplies
// sub-block i into accumulator i and both commit every stage to both CTAs (with a single issuer
// this form was no faster than the single-CTA kernel: 897 cycles per stage, 300 of them the
// issuer's barrier round trip). The partial tiles then meet as above, among the R CTAs of the same
// h (cluster ranks h, h + 2, ...): CTA (r, h) finishes columns [r W, (r + 1) W), W = 128 / R, of its
// 128 rows. No multicast form is used anywhere.
//   warp 0 producer, warp 1 first issuer, warps 2-9 send (two per quarter of the rows), warp 10
//   second issuer; all eleven finish.
constexpr int kPairSplitN = 128;
constexpr uint32_t kPairSplitSubBytes = kASlabBytes + (kPairSplitN / 2 / 32) * kBBoxBytes;   // 24 KiB per 32 of K and CTA
constexpr int kPairSplitStages = 4;    // of two sub-blocks: 192 KiB of ring
constexpr uint32_t kPairSplitStageBytes = 2 * kPairSplitSubBytes;
constexpr size_t kPairSplitSmemBytes = static_cast<size_t>(kPairSplitStages) * kPairSplitStageBytes + 1024 + 1024;
constexpr int kPairSplitThreads = 11 * 32;
static_assert(static_cast<size_t>(kPairSplitStages) * kPairSplitStageBytes >= sizeof(float4) * kExchangePitch * (kPairSplitN / 4),
              "the idle operand ring must hold one exchanged tile");

template <int kAct>
__global__ void __launch_bounds__(kPairSplitThreads, 1) umma_pair_splitk_kernel(const __grid_constant__ UmmaParams p) {
  constexpr int BN = kPairSplitN;
  constexpr int kIssuers = 2;
  constexpr int kSecondIssuerWarp = 10;
  cg::cluster_group cluster = cg::this_cluster();
  const int ranks = static_cast<int>(cluster.num_blocks()) >> 1;   // K ranges = pairs in the cluster
  const uint32_t cta = cluster.block_rank();
  const int slice = static_cast<int>(cta >> 1);   // this pair's K range
  const uint32_t half = cta & 1u;                 // rows [128 half, +128) of the tile
  const uint32_t leader = cta & ~1u;              // cluster rank of the pair's even CTA, which issues the MMAs
  extern __shared__ uint8_t smem_raw[];
  // Same carve-up in every CTA: the MMA addresses the peer's shared memory by the same offsets as its own.
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(kPairSplitStages) * kPairSplitStageBytes);
  uint64_t* empty = full + kPairSplitStages;
  uint64_t* acc_full = empty + kPairSplitStages;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_full + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(p.b_strips == BN / 2 / 32 ? &p.map_b_strips : &p.map_b);
    for (int s = 0; s < kPairSplitStages; ++s) {
      mbar_init(&full[s], 1);           // used in the even CTA only: one expect_tx arrival, bytes of both CTAs
      mbar_init(&empty[s], kIssuers);   // one tcgen05.commit per issuer and use, sent to each CTA
    }
    mbar_init(&acc_full[0], kIssuers);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair<kIssuers * BN>(tmem_ptr);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster.sync();   // every CTA's barriers exist before any remote arrival
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  grid_launch_dependents();   // the next kernel of the stream may set itself up beside this one (not before this
                              // kernel's TMEM is allocated: its CTAs could take the columns first)
  grid_dependency_wait();     // the kernel before this one has completed: global memory may be touched

  const int tiles_m = (p.m + 2 * kTileM - 1) / (2 * kTileM);
  const int tiles_n = (p.n + BN - 1) / BN;
  int tm, tn;
  tile_coords(static_cast<int>(blockIdx.x) / (2 * ranks), tiles_m, tiles_n, &tm, &tn);
  const int row0 = tm * 2 * kTileM + static_cast<int>(half) * kTileM;   // this CTA's rows of A and of the output
  const int k_stages = (p.k + 2 * kStageK - 1) / (2 * kStageK);   // K past the end reads as zeros
  const int per_slice = (k_stages + ranks - 1) / ranks;
  const int kb_begin = min(k_stages, slice * per_slice);
  const int kb_end = min(k_stages, kb_begin + per_slice);
  const bool has_work = kb_begin < kb_end;   // an empty range contributes zeros
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      const int col0 = tn * BN + static_cast<int>(half) * (BN / 2);   // this CTA's share of the B columns
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, kSiteUmmaEmpty)) break;
        // Completion bytes of both CTAs are counted on the even CTA's barrier.
        const uint32_t full_addr = map_to_cta(smem_u32(&full[stage]), leader);
        if (half == 0) mbar_expect_tx(&full[stage], 2 * kPairSplitStageBytes);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const int k0 = (kb * 2 + sub) * kStageK;
          uint8_t* a_dst = stages + static_cast<size_t>(stage) * kPairSplitStageBytes + sub * kPairSplitSubBytes;
          uint8_t* b_dst = a_dst + kASlabBytes;
          tma_load_2d_pair(a_dst, &p.map_a, full_addr, k0, row0);
          if (p.b_strips == BN / 2 / 32) {
            tma_load_3d_pair(b_dst, &p.map_b_strips, full_addr, 0, k0, col0 / 32);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 2 / 32; ++j) {
              tma_load_2d_pair(b_dst + j * kBBoxBytes, &p.map_b, full_addr, col0 + j * 32, k0);
            }
          }
        }
        if (++stage == kPairSplitStages) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1 || warp == kSecondIssuerWarp) {
    if (lane == 0 && half == 0 && has_work) {
      const uint32_t issuer = warp == 1 ? 0u : 1u;
      constexpr uint32_t idesc = umma_idesc_tf32(2 * kTileM, BN, /*a_mn_major=*/false, /*b_mn_major=*/true);
      const SubBlockDescs ring = sub_block_descs(smem_u32(stages));   // of the ring's first sub-block
      int stage = 0;
      uint32_t phase = 0;
      bool fed = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) { fed = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t offset = static_cast<uint32_t>(stage) * kPairSplitStageBytes + issuer * kPairSplitSubBytes;
#pragma unroll
        for (int j = 0; j < kStageK / kInstK; ++j) {
          umma_tf32_pair(tmem_base + issuer * BN, umma_desc_advance(ring.a, offset + j * (kInstK * 4)),
                         umma_desc_advance(ring.b, offset + j * (kInstK * 128)), idesc, (kb > kb_begin || j > 0) ? 1u : 0u);
        }
        // The stage is reusable in both CTAs once both issuers' MMAs have read it.
        umma_commit_pair(smem_u32(&empty[stage]));
        umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), leader + 1));
        if (++stage == kPairSplitStages) stage = 0, phase ^= 1u;
      }
      if (fed) {
        umma_commit_pair(smem_u32(&acc_full[0]));
        umma_commit_pair(map_to_cta(smem_u32(&acc_full[0]), leader + 1));
      }
    }
  } else if (has_work) {
    ok = mbar_wait(&acc_full[0], 0, kSiteUmmaAccFull);
    tcgen05_fence_after_sync();
  }

  // 1. Every CTA of the cluster is past its main loop: the operand rings become exchange buffers.
  tcgen05_fence_before_sync();
  cluster.sync();
  tcgen05_fence_after_sync();

  float4* exchange = reinterpret_cast<float4*>(stages);
  const int width = BN / ranks;   // W: 128, 64 or 32 columns per CTA
  const int quarter = warp & 3;
  const int row_in_tile = quarter * 32 + lane;
  const bool warp_rows = row0 + quarter * 32 < p.m;   // any row of this warp inside the matrix
  const int quads_log2 = 31 - __clz(width / 4);
  const EpilogueArgs args = epilogue_args(p);
  const int col_base = tn * BN + slice * width;
  const bool interior = args.vector_io && args.bias == nullptr && args.peers.count == 0 && row0 + kTileM <= p.m &&
                        col_base + width <= p.n;
  InteriorCursor cursor = interior_cursor(args, exchange, quads_log2, row0, col_base, threadIdx.x, kPairSplitThreads);
  float4 first_sources[kInteriorBatch];
  if (interior) interior_sources(cursor, 0, first_sources);
  if (warp >= 2 && warp < kSecondIssuerWarp && warp_rows) {
    // 2. This CTA's partial rows, W columns to each CTA with the same rows: cluster ranks half, half + 2, ...
    send_partial_row<BN, kIssuers, 2>(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16), has_work && ok,
                                      smem_u32(exchange), slice, quads_log2, 2, static_cast<int>(half), row_in_tile,
                                      (warp - 2) >> 2);
  }
  tcgen05_fence_before_sync();
  cluster.sync();

  // 3. Add the partials of this CTA's columns in range order and finish them.
  if (interior) {
    exchange_finish_interior<kAct>(args, cursor, first_sources, ranks, quads_log2);
  } else {
    exchange_finish<kAct>(args, exchange, ranks, quads_log2, row0, col_base, threadIdx.x, kPairSplitThreads);
  }

  __syncthreads();
  cluster.sync();   // the pair's TMEM is given back by both CTAs together
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair<kIssuers * BN>(tmem_base);
  }
}

// ---------------------------------------- TMA, operand-swapped kernel for few rows
// Up to 64 rows (decode-like shapes): computing D^T = B^T * A^T puts the long
// dimension N on the 128 rows of the MMA and the few rows of A on its N side, so
// an instruction is 128 x NM x 8 with NM = 16 or 64 instead of 128 x 128 x 8 with
// most rows zero. What the tensor pipe reads from shared memory per K block drops
// from 32 KiB to 16 KiB + NM * 128 B, and that, not the arithmetic, is what the
// K-block time of the 128 x 128 form consists of.
//   MMA operand A = B^T: M-major, i.e. exactly the B slab of the other kernels
//     (32-column boxes of 32 K rows, 128-byte swizzle in 32-byte granules).
//   MMA operand B = A^T: K-major, i.e. the A slab of the other kernels with NM
//     rows (8-row groups 1024 bytes apart, 128-byte swizzle).
// The accumulator holds D^T: TMEM lane = column n of the tile, TMEM column = row
// m, so an epilogue thread owns one output column and a warp writes 32 adjacent
// floats of a row of D. A cluster of 1/2/4/8 CTAs splits K as in the split-K
// kernel; CTA r finishes the 128 / cluster columns it owns.
constexpr int kSwapTileN = 128;   // columns of D per CTA (the M side of the MMA)

// One 32-wide K sub-block: the B slab and NM rows of A.
template <int NM>
__host__ __device__ constexpr uint32_t swap_sub_bytes() {
  return (kSwapTileN / 32) * kBBoxBytes + NM * kStageK * 4;
}

// A pipeline stage holds KSUB sub-blocks: the small MMAs of this kernel (54 cycles each in
// isolation) are cheap next to the 380 cycles of a stage's barrier wait and commit.
template <int NM, int KSUB>
__host__ __device__ constexpr uint32_t swap_stage_bytes() {
  return KSUB * swap_sub_bytes<NM>();
}

template <int NM, int STAGES, int KSUB>
__host__ __device__ constexpr size_t swap_smem_bytes() {
  return static_cast<size_t>(STAGES) * swap_stage_bytes<NM, KSUB>() + 1024 + 256;
}

template <int NM, int STAGES, int KSUB, int kAct>
__global__ void __launch_bounds__(kTmaThreads, 1) umma_swap_kernel(const __grid_constant__ UmmaParams p) {
  static_assert(NM % 16 == 0 && NM >= 16 && NM <= 64, "rows of A per tile");
  static_assert(static_cast<size_t>(STAGES) * swap_stage_bytes<NM, KSUB>() >= sizeof(float) * NM * kSwapTileN,
                "the idle operand ring must hold one exchanged tile");
  constexpr uint32_t kTmemCols = NM < 32 ? 32 : NM;
  cg::cluster_group cluster = cg::this_cluster();
  const int ranks = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(STAGES) * swap_stage_bytes<NM, KSUB>());
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_full + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_PROBE(p, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  grid_launch_dependents();   // the next kernel of the stream may set itself up beside this one (not before this
                              // kernel's TMEM is allocated: its CTAs could take the columns first)
  grid_dependency_wait();     // the kernel before this one has completed: global memory may be touched
  B200_PROBE(p, 1);

  // Tiles: blocks of NM rows of A by 128 columns of B; row blocks innermost.
  const int tiles_m = (p.m + NM - 1) / NM;
  const int tile = static_cast<int>(blockIdx.x) / ranks;
  const int m0 = (tile % tiles_m) * NM, n0 = (tile / tiles_m) * kSwapTileN;
  const int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages; K past the end reads as zeros
  const int per_rank = (k_blocks + ranks - 1) / ranks;
  const int kb_begin = min(k_blocks, rank * per_rank);
  const int kb_end = min(k_blocks, kb_begin + per_rank);
  const bool has_work = kb_begin < kb_end;   // an empty K range contributes zeros
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&p.map_a);
      prefetch_tensormap(p.b_strips == kSwapTileN / 32 ? &p.map_b_strips : &p.map_b);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, kSiteUmmaEmpty)) break;
        mbar_expect_tx(&full[stage], swap_stage_bytes<NM, KSUB>());
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          const int k0 = (kb * KSUB + sub) * kStageK;
          uint8_t* b_dst = stages + static_cast<size_t>(stage) * swap_stage_bytes<NM, KSUB>() + sub * swap_sub_bytes<NM>();
          uint8_t* a_dst = b_dst + (kSwapTileN / 32) * kBBoxBytes;                // B slab first, then NM rows of A
          tma_load_2d(a_dst, &p.map_a, &full[stage], k0, m0);
          if (p.b_strips == kSwapTileN / 32) {
            tma_load_3d(b_dst, &p.map_b_strips, &full[stage], 0, k0, n0 / 32);
          } else {
#pragma unroll
            for (int j = 0; j < kSwapTileN / 32; ++j) {
              tma_load_2d(b_dst + j * kBBoxBytes, &p.map_b, &full[stage], n0 + j * 32, k0);
            }
          }
        }
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      // M = 128 (columns of D), N = NM (rows of D); operand A M-major, operand B K-major.
      constexpr uint32_t idesc = umma_idesc_tf32(kSwapTileN, NM, /*a_mn_major=*/true, /*b_mn_major=*/false);
      int stage = 0;
      uint32_t phase = 0;
      bool fed = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) { fed = false; break; }
        tcgen05_fence_after_sync();
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          const uint32_t b_addr =
              smem_u32(stages + static_cast<size_t>(stage) * swap_stage_bytes<NM, KSUB>() + sub * swap_sub_bytes<NM>());
          const uint32_t a_addr = b_addr + (kSwapTileN / 32) * kBBoxBytes;
#pragma unroll
          for (int j = 0; j < kStageK / kInstK; ++j) {
            const uint64_t desc_mma_a = umma_smem_desc(b_addr + j * (kInstK * 128), kBBoxBytes, 512, kUmmaSwizzle128B32BAtom);
            const uint64_t desc_mma_b = umma_smem_desc(a_addr + j * (kInstK * 4), 16, 1024, kUmmaSwizzle128B);
            umma_tf32(tmem_base, desc_mma_a, desc_mma_b, idesc, (kb > kb_begin || sub > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty[stage]);
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
      if (fed) umma_commit(&acc_full[0]);
    }
  } else if (has_work) {
    ok = mbar_wait(&acc_full[0], 0, kSiteUmmaAccFull);
    tcgen05_fence_after_sync();
  }

  B200_PROBE(p, 2);
  // 1. Every CTA of the cluster is past its main loop: the rings are idle.
  tcgen05_fence_before_sync();
  cluster.sync();
  tcgen05_fence_after_sync();

  B200_PROBE(p, 3);
  // Exchange buffer of a CTA: floats [source rank][row m][column of its share]; a thread owns one
  // column n of the tile, so all its values go to the one CTA that owns that column.
  float* exchange = reinterpret_cast<float*>(stages);
  const int width = kSwapTileN / ranks;                 // columns per CTA
  if (warp >= 2) {
    const int quarter = warp & 3;
    const int n_local = quarter * 32 + lane;
    float* remote = cluster.map_shared_rank(exchange, n_local / width) +
                    static_cast<size_t>(rank) * NM * width + (n_local % width);
#pragma unroll
    for (int chunk = 0; chunk < kTmemCols / 32; ++chunk) {
      uint32_t raw[32];
      if (has_work && ok) {
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 32, raw);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) raw[e] = 0u;
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int m = chunk * 32 + e;
        if (m < NM) remote[m * width] = __uint_as_float(raw[e]);   // columns past NM were never accumulated
      }
    }
  }
  B200_PROBE(p, 4);
  tcgen05_fence_before_sync();
  cluster.sync();
  B200_PROBE(p, 5);

  // 3. Add the partials of this CTA's columns in rank order, apply the epilogue, lanes along a row of D.
  {
    const EpilogueArgs ep = epilogue_args(p);
    const int col_base = n0 + rank * width;
    for (int item = threadIdx.x; item < NM * width; item += kTmaThreads) {
      const int m = item / width, nl = item % width;
      const int row = m0 + m, col = col_base + nl;
      if (row >= ep.m || col >= ep.n) continue;
      float sum = 0.f;
      for (int src = 0; src < ranks; ++src) sum += exchange[(src * NM + m) * width + nl];
      float v = ep.alpha * sum;
      if (ep.beta != 0.f) v = fmaf(ep.beta, __ldg(ep.c + static_cast<int64_t>(row) * ep.ldc + col), v);
      if (ep.bias != nullptr) v += __ldg(ep.bias + col);
      v = activate<kAct>(v);
      const int64_t offset = static_cast<int64_t>(row) * ep.ldd + col;
      ep.d[offset] = v;
      store_peers(ep, offset, v);
    }
  }

  B200_PROBE(p, 6);
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}
// ------------------------------------------------------------------ launchers

// Most clusters of `cluster_size` CTAs of the split-K kernel that the device keeps resident at once
// (cached per device; clusters of eight fit far fewer CTAs than the SM count suggests).
int splitk_max_clusters(int cluster_size) {
  static std::atomic<int> cache[64][4];   // [device][log2 cluster size], 0 = not asked yet
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  const int slot = cluster_size == 1 ? 0 : cluster_size == 2 ? 1 : cluster_size == 4 ? 2 : 3;
  const int cached = cache[device][slot].load(std::memory_order_relaxed);
  if (cached != 0) return cached;
  auto kernel = umma_splitk_kernel<3, B200_EPILOGUE_LINEAR>;   // the activation does not change the footprint
  constexpr size_t smem = smem_bytes<kSplitN, 3>() - kStagingBytes;   // no staging: two CTAs fit an SM
  if (!ensure_dynamic_smem<umma_splitk_kernel<3, B200_EPILOGUE_LINEAR>, smem>()) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(cluster_size) * 64);
  cfg.blockDim = dim3(kTmaThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(cluster_size);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) clusters = 0;
  const int result = clusters > 0 ? clusters : -1;   // concurrent first calls compute the same value
  cache[device][slot].store(result, std::memory_order_relaxed);
  return result;
}

// Cluster size of the split-K kernel, from a cost model fitted to timings of the kernel on a B200
// (microseconds, graph-timed, with a source and ReLU). With f the fraction of the tile's 128 rows
// that exist, a 32-wide K block costs 0.14 + 0.07 f when the CTA has its SM to itself and runs two
// sub-blocks per stage (one per MMA issuer), 0.26 + 0.04 f when the grid fits one CTA per SM but
// its clusters only fit the device at two (single-block stages), and 0.36 + 0.06 f per CTA when two
// share an SM. Launch, pipeline fill, barriers, exchange and the finishing pass cost 6.0 / 6.0 / 8.0 /
// 9.5 for clusters of 1 / 2 / 4 / 8 when few rows exist, 8.0 / 8.2 / 10.5 / 11.4 when all 128 do
// (interpolated by the row count; a cluster of one still runs the exchange through its own
// shared memory). Fitted to: 1024 x 1024 x K split in two 11.5 / 14.4 / 20.5 / 38.7 us at
// K = 1024 / 2048 / 4096 / 8192, in four 39.8 at 8192; 512 x 512 x 2048 in eight 10.8; 768 x 768 x 4096
// in four 20.8; 64 x 4096 x 4096 in four 15.1; 1280 x 1280 x 8192 in two 60.5. A candidate must keep two
// K blocks per range and fit the device in one wave (two CTAs per SM: twice the cluster count the
// occupancy query reports for one). `estimate_us` receives the modelled time of the choice.
int splitk_ranks(const b200_gemm_problem& q, int sms, float* estimate_us = nullptr) {
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + kSplitN - 1) / kSplitN);
  const int k_blocks = (q.k + kStageK - 1) / kStageK;
  constexpr float kExchangeFewRows[4] = {6.0f, 6.0f, 8.0f, 9.5f};
  constexpr float kExchangeAllRows[4] = {8.0f, 8.2f, 10.5f, 11.4f};
  const float row_fraction = static_cast<float>(q.m < kTileM ? q.m : kTileM) / kTileM;
  int best = 1;
  float best_us = 1e30f;
  for (int log2r = 0; log2r < 4; ++log2r) {
    const int ranks = 1 << log2r;
    const int64_t ctas = tiles * ranks;
    if (ctas > 2LL * sms) break;
    if (ranks > 1 && (k_blocks / ranks < 2 || tiles > 2LL * splitk_max_clusters(ranks))) break;
    const bool shared_sm = ctas > sms;
    const bool deep = !shared_sm && (ranks == 1 || tiles <= splitk_max_clusters(ranks));   // as launch_splitk_for decides
    const float exchange = kExchangeFewRows[log2r] + row_fraction * (kExchangeAllRows[log2r] - kExchangeFewRows[log2r]);
    const float per_block = shared_sm ? 0.36f + 0.06f * row_fraction
                                      : (deep ? 0.14f + 0.07f * row_fraction : 0.26f + 0.04f * row_fraction);
    const float us = static_cast<float>((k_blocks + ranks - 1) / ranks) * per_block + exchange;
    if (us < best_us) best_us = us, best = ranks;
  }
  if (estimate_us != nullptr) *estimate_us = best_us;
  return best;
}

template <int STAGES, int kAct, int KSUB = 1>
int launch_splitk(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  auto kernel = umma_splitk_kernel<STAGES, kAct, KSUB>;
  constexpr size_t smem = smem_bytes<kSplitN, STAGES>() - kStagingBytes;   // its finishing pass needs no staging
  if (!ensure_dynamic_smem<umma_splitk_kernel<STAGES, kAct, KSUB>, smem>()) return B200_ERR_LAUNCH_FAILED;
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, kSplitN / 32,
                                                        Swizzle::k128BAtom32B))
                   ? kSplitN / 32
                   : 0;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int ranks = splitk_ranks(q, sms);
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + kSplitN - 1) / kSplitN);
  if (tiles * ranks > 0x7fffffffLL) return B200_ERR_INVALID_PROBLEM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * ranks));
  cfg.blockDim = dim3(splitk_threads<STAGES, KSUB>());
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(static_cast<unsigned>(ranks));
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

// Most clusters of `cluster_ctas` (2, 4 or 8) CTAs of the CTA-pair split-K kernel that the device keeps
// resident at once (cached per device), or 0 when the query fails.
int pair_splitk_max_clusters(int cluster_ctas) {
  static std::atomic<int> cache[64][3];   // [device][log2 cluster size - 1], 0 = not asked yet
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  const int slot = cluster_ctas == 2 ? 0 : cluster_ctas == 4 ? 1 : 2;
  const int cached = cache[device][slot].load(std::memory_order_relaxed);
  if (cached != 0) return cached > 0 ? cached : 0;
  auto kernel = umma_pair_splitk_kernel<B200_EPILOGUE_LINEAR>;   // the activation does not change the footprint
  if (!ensure_dynamic_smem<umma_pair_splitk_kernel<B200_EPILOGUE_LINEAR>, kPairSplitSmemBytes>()) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(cluster_ctas) * 64);
  cfg.blockDim = dim3(kPairSplitThreads);
  cfg.dynamicSmemBytes = kPairSplitSmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(cluster_ctas);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) clusters = 0;
  cache[device][slot].store(clusters > 0 ? clusters : -1, std::memory_order_relaxed);   // concurrent first calls compute the same value
  return clusters > 0 ? clusters : 0;
}

// K ranges (pairs per cluster: 1, 2 or 4) of the CTA-pair split-K kernel for `q`, 0 when the occupancy
// query fails. A range keeps at least two 64-wide stages; clusters beyond what the device keeps
// resident at once run as further waves. The model (microseconds, fitted to graph timings on a B200
// with a source and ReLU: 1024 x 1024 x K in two ranges 19.8 / 33.3 / 62.9 at K = 4096 / 8192 / 16384,
// 256 x 4096 x 4096 in two 19.6, 768 x 768 x 4096 18.6, 512 x 512 x 2048 in four 10.8): a 64-wide stage
// of a CTA's range costs 0.42; launch, pipeline fill, exchange and finishing pass 6.5 / 6.5 / 9.0 for
// 1 / 2 / 4 ranges. `waves` receives the wave count of the choice.
int pair_splitk_ranks(const b200_gemm_problem& q, float* estimate_us = nullptr, int* waves = nullptr) {
  const int64_t tiles = static_cast<int64_t>((q.m + 2 * kTileM - 1) / (2 * kTileM)) * ((q.n + kPairSplitN - 1) / kPairSplitN);
  const int k_stages = (q.k + 2 * kStageK - 1) / (2 * kStageK);
  constexpr float kFixedUs[3] = {6.5f, 6.5f, 9.0f};
  int best = 0, best_waves = 0;
  float best_us = 1e30f;
  for (int log2r = 0; log2r < 3; ++log2r) {
    const int ranks = 1 << log2r;
    if (ranks > 1 && k_stages / ranks < 2) break;
    // Four fifths of what the occupancy query reports: on some GPUs of the same model the last few
    // clusters of four did not find room beside the others and ran as a second wave (1024 x 1024 x 4096,
    // 32 clusters: 20 us on most boxes, 35 on one).
    const int resident = pair_splitk_max_clusters(2 * ranks) * 4 / 5;
    if (resident <= 0) continue;
    const int64_t rounds = (tiles + resident - 1) / resident;
    const float us = static_cast<float>(rounds) * (static_cast<float>((k_stages + ranks - 1) / ranks) * 0.42f + kFixedUs[log2r]);
    if (us < best_us) best_us = us, best = ranks, best_waves = static_cast<int>(rounds < 0x7fffffff ? rounds : 0x7fffffff);
  }
  if (estimate_us != nullptr) *estimate_us = best_us;
  if (waves != nullptr) *waves = best_waves;
  return best;
}

template <int kAct>
int launch_pair_splitk(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  auto kernel = umma_pair_splitk_kernel<kAct>;
  if (!ensure_dynamic_smem<umma_pair_splitk_kernel<kAct>, kPairSplitSmemBytes>()) return B200_ERR_LAUNCH_FAILED;
  const int ranks = pair_splitk_ranks(q);
  if (ranks == 0) return B200_ERR_INTERNAL;   // the occupancy query failed
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK,
                                                        kPairSplitN / 2 / 32, Swizzle::k128BAtom32B))
                   ? kPairSplitN / 2 / 32
                   : 0;
  const int64_t tiles = static_cast<int64_t>((q.m + 2 * kTileM - 1) / (2 * kTileM)) * ((q.n + kPairSplitN - 1) / kPairSplitN);
  if (tiles * 2 * ranks > 0x7fffffffLL) return B200_ERR_INVALID_PROBLEM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * 2 * ranks));
  cfg.blockDim = dim3(kPairSplitThreads);
  cfg.dynamicSmemBytes = kPairSplitSmemBytes;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(static_cast<unsigned>(2 * ranks));
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

// Cluster size of the operand-swapped kernel: as many K ranges as keep every cluster resident at
// once (one CTA per SM) with at least two pipeline stages each.
int swap_ranks(int64_t tiles, int k_stages, int sms) {
  int ranks = 1;
  while (ranks < 8 && tiles * (ranks * 2) <= sms && k_stages / (ranks * 2) >= 2 &&
         tiles <= splitk_max_clusters(ranks * 2)) {
    ranks *= 2;
  }
  return ranks;
}

template <int NM, int kAct>
int run_swap(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  // About 144 KiB of ring either way: 2 stages x 4 sub-blocks of 18 KiB, or 3 x 2 of 24 KiB.
  constexpr int KSUB = NM <= 16 ? 4 : 2, STAGES = NM <= 16 ? 2 : 3;
  auto kernel = umma_swap_kernel<NM, STAGES, KSUB, kAct>;
  constexpr size_t smem = swap_smem_bytes<NM, STAGES, KSUB>();
  if (!ensure_dynamic_smem<umma_swap_kernel<NM, STAGES, KSUB, kAct>, smem>()) return B200_ERR_LAUNCH_FAILED;
  UmmaParams p;
  fill_common(&p, q, peers);
  // A: boxes of NM rows x 32 floats of K; B as in the other kernels.
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, NM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, kSwapTileN / 32,
                                                        Swizzle::k128BAtom32B))
                   ? kSwapTileN / 32
                   : 0;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + NM - 1) / NM) * ((q.n + kSwapTileN - 1) / kSwapTileN);
  const int ranks = swap_ranks(tiles, (q.k + KSUB * kStageK - 1) / (KSUB * kStageK), sms);
  if (tiles * ranks > 0x7fffffffLL) return B200_ERR_INVALID_PROBLEM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * ranks));
  cfg.blockDim = dim3(kTmaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(static_cast<unsigned>(ranks));
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

template <int kAct>
int launch_swap(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return q.m <= 16 ? run_swap<16, kAct>(q, peers, stream) : run_swap<64, kAct>(q, peers, stream);
}
}  // namespace

namespace {

// A CTA that has its SM to itself (and whose cluster count fits the device at one CTA per SM) runs
// a ring of six K blocks as three stages of two (against two stages of two: 512 x 1024 x 16384
// 57.5 -> 46.5 us, 256 x 4096 x 4096 30.5 -> 29.5, 1024 x 1024 x 8192 45.4 -> 44.4); otherwise three
// single-block stages leave room for a second CTA on the SM.
template <int kAct>
int launch_splitk_for(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int ranks = splitk_ranks(q, sms);
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + kSplitN - 1) / kSplitN);
  const bool alone = tiles * ranks <= sms && (ranks == 1 || tiles <= splitk_max_clusters(ranks));
  // (Single-block stages taken in turn by the two issuers, as in the 128 x 128 tile kernel for long
  // K, were tried here too: no faster, 39.7 against 38.7 us at 1024 x 1024 x 8192 in two ranges.)
  return alone ? launch_splitk<6, kAct, 2>(q, peers, stream) : launch_splitk<3, kAct, 1>(q, peers, stream);
}

}  // namespace

int launch_tf32_splitk(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  switch (act) {
    case B200_EPILOGUE_LINEAR: return launch_splitk_for<B200_EPILOGUE_LINEAR>(q, peers, stream);
    case B200_EPILOGUE_RELU: return launch_splitk_for<B200_EPILOGUE_RELU>(q, peers, stream);
    case B200_EPILOGUE_GELU: return launch_splitk_for<B200_EPILOGUE_GELU>(q, peers, stream);
    default: return B200_ERR_INVALID_ARGUMENT;
  }
}

int launch_tf32_swap(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  switch (act) {
    case B200_EPILOGUE_LINEAR: return launch_swap<B200_EPILOGUE_LINEAR>(q, peers, stream);
    case B200_EPILOGUE_RELU: return launch_swap<B200_EPILOGUE_RELU>(q, peers, stream);
    case B200_EPILOGUE_GELU: return launch_swap<B200_EPILOGUE_GELU>(q, peers, stream);
    default: return B200_ERR_INVALID_ARGUMENT;
  }
}

int launch_tf32_pair_splitk(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  switch (act) {
    case B200_EPILOGUE_LINEAR: return launch_pair_splitk<B200_EPILOGUE_LINEAR>(q, peers, stream);
    case B200_EPILOGUE_RELU: return launch_pair_splitk<B200_EPILOGUE_RELU>(q, peers, stream);
    case B200_EPILOGUE_GELU: return launch_pair_splitk<B200_EPILOGUE_GELU>(q, peers, stream);
    default: return B200_ERR_INVALID_ARGUMENT;
  }
}

int tf32_splitk_plan(const b200_gemm_problem& q, int sms, float* estimate_us) { return splitk_ranks(q, sms, estimate_us); }
int tf32_pair_splitk_plan(const b200_gemm_problem& q, float* estimate_us, int* waves) {
  return pair_splitk_ranks(q, estimate_us, waves);
}

}  // namespace b200
