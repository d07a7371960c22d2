// TF32 tensor-core GEMM, single-CTA persistent kernels: the TMA-fed tile kernel (128 x 64, 128 x 128,
// 128 x 256 tiles) and the kernel whose operand ring is filled by loader warps for operands TMA
// cannot describe. Layouts, roles and epilogues are in tf32_umma.cuh.
#include "tf32_umma.cuh"

namespace b200 {

cudaError_t tf32_tile_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

// ------------------------------------------------------- TMA, persistent kernel
// warp 0: TMA producer (one lane)      warp 1: TMEM owner + MMA issuer (one lane)
// warps 2-9: epilogue; warp w reads the TMEM lane quarter w % 4, two warps per quarter.
// warp 10 (kIssuers == 2): the second MMA issuer (one lane).

// STAGES counts 32-wide K blocks of shared memory; KSUB of them form one pipeline stage (an MMA
// thread's barrier wait and commit cost about as much as five MMAs at its issue rate); kIssuers
// threads issue the MMAs, each into its own accumulator (mma_role in tf32_umma.cuh).
template <int BN, int STAGES, int kAct, int KSUB = 1, int kIssuers = 1>
__global__ void __launch_bounds__(kIssuers == 2 ? kTileThreadsTwoIssuers : kTileThreads, 1)
    umma_tma_kernel(const __grid_constant__ UmmaParams p) {
  constexpr int kRing = STAGES / KSUB;
  extern __shared__ uint8_t smem_raw[];
  const SmemCarve sm = carve<BN, STAGES>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_PROBE(p, 0);

  if (threadIdx.x == 0) {
    // The descriptors the copies will name, requested first of all: their fetch is part of the
    // latency of the first load (and of the first store, which nothing hides).
    prefetch_tensormap(&p.map_a);
    prefetch_tensormap(p.b_strips == BN / 32 ? &p.map_b_strips : &p.map_b);
    if (p.tma_store != 0) prefetch_tensormap(&p.map_d);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], empty_barrier_arrivals<KSUB, kIssuers>());   // one commit per MMA issuer of the stage
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], kIssuers);
      mbar_init(&sm.acc_empty[b], 4 * kTileEpilogueShare);  // one arrive per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc<tmem_columns<BN, kIssuers>()>(sm.tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;
  // The next kernel of the stream may set itself up beside this one from here on: not earlier, or
  // its CTAs could take TMEM columns that a CTA of this kernel is still about to ask for.
  grid_launch_dependents();
  grid_dependency_wait();     // from here on global memory is read and written
  B200_PROBE(p, 1);

  const int tiles_m = (p.m + kTileM - 1) / kTileM;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages per tile; K past the end reads as zeros
  if constexpr (kIssuers == 2 && KSUB == 1) k_blocks = (k_blocks + 1) & ~1;   // issuers take alternate stages (mma_role)

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sm.empty[stage], phase ^ 1u, kSiteUmmaEmpty)) { ok = false; break; }
          mbar_expect_tx(&sm.full[stage], KSUB * stage_bytes<BN>());
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const int k0 = (kb * KSUB + sub) * kStageK;
            uint8_t* a_dst = sm.stages + static_cast<size_t>(stage * KSUB + sub) * stage_bytes<BN>();
            uint8_t* b_dst = a_dst + kASlabBytes;
            tma_load_2d(a_dst, &p.map_a, &sm.full[stage], k0, tm * kTileM);
            if (p.b_strips == BN / 32) {
              // The producer thread's issue rate matters: one copy instead of BN / 32.
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
    }
  } else if (warp == 1) {
    if (lane == 0) mma_role<BN, STAGES, KSUB, kIssuers>(sm, tmem_base, tiles, k_blocks, 0);
  } else if (warp < 2 + 4 * kTileEpilogueShare) {
    epilogue_role<BN, kAct, true, kTileEpilogueShare, kIssuers>(p, sm, tmem_base, warp & 3, (warp - 2) >> 2, lane, tiles, tiles_m,
                                                                tiles_n);
  } else {   // the second MMA issuer's warp
    if constexpr (kIssuers == 2) {
      if (lane == 0) mma_role<BN, STAGES, KSUB, kIssuers>(sm, tmem_base, tiles, k_blocks, 1);
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  B200_PROBE(p, 6);
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<tmem_columns<BN, kIssuers>()>(tmem_base);
  }
}

// ------------------------------------------------------- generic loader kernel
// For operands TMA cannot describe (base not 16-byte aligned, leading dimension
// not a multiple of four floats). Persistent like the TMA kernel, same MMA and
// epilogue roles, but the operand ring is filled by eight loader warps with
// predicated scalar loads (zeros outside the matrix):
//   warp 0: TMEM owner + MMA issuer     warps 1-4: epilogue     warps 5-12: loaders
// A loader warp moves one 128-byte row of a slab per instruction: coalesced in
// global memory, and conflict-free in shared memory because the swizzle only
// permutes the 16- or 32-byte granules inside that row. Each thread keeps the
// values of the next stage in registers while it stores the current one, so
// 32 loads per thread are in flight across the wait for a free slot.
constexpr int kLoaderWarps = 8;
constexpr int kGenericThreads = (1 + 4 + kLoaderWarps) * 32;
constexpr int kGenericARows = kTileM / kLoaderWarps;  // A rows per loader warp and stage

// Work split of one stage over the loader warps. Warp lw owns
//   A rows  m = lw + 8 i                      (m % 8 == lw for all of them),
//   B rows  k = lw % 4 + 4 (i % 8) of strips j = (lw / 4) * (BN / 64) + i / 8   (k % 4 == lw % 4),
// so the swizzle term of every store is a per-thread constant and the stores
// are a base address plus immediates.
template <int BN>
struct StageRegs {
  static constexpr int kBRows = kStageK * (BN / 32) / kLoaderWarps;  // 128-byte B rows per loader warp and stage
  float a[kGenericARows];
  float b[kBRows];
};

// Loads this thread's share of stage (m0, n0, k0) into registers.
template <int BN>
__device__ __forceinline__ void load_stage_regs(const UmmaParams& p, StageRegs<BN>& r, int lw, int lane, int m0, int n0,
                                                int k0) {
  constexpr int kStripsPerWarpHalf = BN / 64;
  const float* a_ptr = p.a + static_cast<int64_t>(m0 + lw) * p.lda + k0 + lane;
  const int kb0 = k0 + (lw & 3), nb0 = n0 + (lw >> 2) * kStripsPerWarpHalf * 32 + lane;
  const float* b_ptr = p.b + static_cast<int64_t>(kb0) * p.ldb + nb0;
  const int64_t a_step = static_cast<int64_t>(kLoaderWarps) * p.lda, b_step = 4 * p.ldb;
  if (m0 + kTileM <= p.m && n0 + BN <= p.n && k0 + kStageK <= p.k) {  // interior stage: no predicates
#pragma unroll
    for (int i = 0; i < kGenericARows; ++i) {
      r.a[i] = B200_IN_BOUNDS(a_ptr + i * a_step >= p.a && a_ptr + i * a_step < p.a + static_cast<int64_t>(p.m - 1) * p.lda + p.k)
                   ? __ldg(a_ptr + i * a_step) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < StageRegs<BN>::kBRows; ++i) {
      const float* src = b_ptr + (i & 7) * b_step + (i >> 3) * 32;
      r.b[i] = B200_IN_BOUNDS(src >= p.b && src < p.b + static_cast<int64_t>(p.k - 1) * p.ldb + p.n) ? __ldg(src) : 0.f;
    }
  } else {
    const bool k_ok = k0 + lane < p.k;
#pragma unroll
    for (int i = 0; i < kGenericARows; ++i) {
      r.a[i] = (k_ok && m0 + lw + kLoaderWarps * i < p.m) ? __ldg(a_ptr + i * a_step) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < StageRegs<BN>::kBRows; ++i) {
      const bool ok = kb0 + 4 * (i & 7) < p.k && nb0 + (i >> 3) * 32 < p.n;
      r.b[i] = ok ? __ldg(b_ptr + (i & 7) * b_step + (i >> 3) * 32) : 0.f;
    }
  }
}

// Stores them into the swizzled slabs.
//   A: element (m, k) at m * 128 + ((k / 4) ^ (m % 8)) * 16 + (k % 4) * 4.
//   B: box j = n / 32; element (k, n) at j * 4096 + k * 128 + (((n % 32) / 8) ^ (k % 4)) * 32 + (n % 8) * 4.
template <int BN>
__device__ __forceinline__ void store_stage_regs(const StageRegs<BN>& r, uint8_t* a_dst, uint8_t* b_dst, int lw, int lane) {
  constexpr int kStripsPerWarpHalf = BN / 64;
  float* a_base = reinterpret_cast<float*>(a_dst + lw * 128 + (((lane >> 2) ^ lw) << 4) + ((lane & 3) << 2));
#pragma unroll
  for (int i = 0; i < kGenericARows; ++i) a_base[i * (kLoaderWarps * 128 / 4)] = r.a[i];
  float* b_base = reinterpret_cast<float*>(b_dst + (lw >> 2) * kStripsPerWarpHalf * kBBoxBytes + (lw & 3) * 128 +
                                           (((lane >> 3) ^ (lw & 3)) << 5) + ((lane & 7) << 2));
#pragma unroll
  for (int i = 0; i < StageRegs<BN>::kBRows; ++i) b_base[(i >> 3) * (kBBoxBytes / 4) + (i & 7) * (4 * 128 / 4)] = r.b[i];
}

// Position of a loader in the (tile, k block) sequence of its CTA.
struct LoaderCursor {
  int tile, kb, tm, tn;
  __device__ __forceinline__ bool valid(int tiles) const { return tile < tiles; }
  __device__ __forceinline__ void advance(int tiles, int tiles_m, int tiles_n, int k_blocks) {
    if (++kb == k_blocks) {
      kb = 0;
      tile += gridDim.x;
      if (tile < tiles) tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
    }
  }
};

template <int BN, int STAGES, int kAct>
__global__ void __launch_bounds__(kGenericThreads, 1) umma_generic_kernel(const __grid_constant__ UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemCarve sm = carve<BN, STAGES>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], kLoaderWarps);  // one arrive per loader warp
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], 1);
      mbar_init(&sm.acc_empty[b], 4);
    }
    mbar_init_fence();
  }
  if (warp == 0) {
    tmem_alloc<tmem_columns<BN>()>(sm.tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;
  grid_launch_dependents();   // the next kernel of the stream may set itself up beside this one (not before this
                              // kernel's TMEM is allocated: its CTAs could take the columns first)
  grid_dependency_wait();     // the kernel before this one has completed: global memory may be touched

  const int tiles_m = (p.m + kTileM - 1) / kTileM;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  const int k_blocks = (p.k + kStageK - 1) / kStageK;

  if (warp == 0) {
    if (lane == 0) mma_role<BN, STAGES>(sm, tmem_base, tiles, k_blocks);
  } else if (warp <= 4) {
    epilogue_role<BN, kAct, false, 1>(p, sm, tmem_base, warp & 3, 0, lane, tiles, tiles_m, tiles_n);   // 416 threads: no room for two register sets
  } else {
    const int lw = warp - 5;
    LoaderCursor cursor{static_cast<int>(blockIdx.x), 0, 0, 0};  // the next stage to load
    if (cursor.valid(tiles)) tile_coords(cursor.tile, tiles_m, tiles_n, &cursor.tm, &cursor.tn);
    int stage = 0;
    uint32_t phase = 0;
    auto load = [&](StageRegs<BN>& r) {
      const bool have = cursor.valid(tiles);
      if (have) {
        load_stage_regs<BN>(p, r, lw, lane, cursor.tm * kTileM, cursor.tn * BN, cursor.kb * kStageK);
        cursor.advance(tiles, tiles_m, tiles_n, k_blocks);
      }
      return have;
    };
    auto commit = [&](const StageRegs<BN>& r) {
      if (!mbar_wait(&sm.empty[stage], phase ^ 1u, kSiteUmmaEmpty)) return false;
      uint8_t* a_dst = sm.stages + static_cast<size_t>(stage) * stage_bytes<BN>();
      store_stage_regs<BN>(r, a_dst, a_dst + kASlabBytes, lw, lane);
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the MMA unit
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.full[stage]);
      if (++stage == STAGES) stage = 0, phase ^= 1u;
      return true;
    };
    // Two register sets alternate, written out rather than copied, so that the
    // loads of one stage stay in flight while the other is being stored.
    StageRegs<BN> r0, r1;
    bool have0 = load(r0);
    while (have0) {
      const bool have1 = load(r1);
      if (!commit(r0)) break;
      if (!have1) break;
      have0 = load(r0);
      if (!commit(r1)) break;
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after_sync();
    tmem_dealloc<tmem_columns<BN>()>(tmem_base);
  }
}
// ------------------------------------------------------------------ launchers

template <int BN, int STAGES, int kAct, int KSUB>
int launch_tma_with(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  // Two MMA issuers (mma_role) wherever a stage has sub-blocks to share out and the tile leaves
  // TMEM for a second accumulator: the 128 x 64 and 128 x 128 tiles.
  constexpr int kIssuers = (BN <= 128 && (KSUB % 2 == 0 || STAGES % 2 == 0)) ? 2 : 1;
  auto kernel = umma_tma_kernel<BN, STAGES, kAct, KSUB, kIssuers>;
  constexpr size_t smem = smem_bytes<BN, STAGES>();
  if (!ensure_dynamic_smem<umma_tma_kernel<BN, STAGES, kAct, KSUB, kIssuers>, smem>()) return B200_ERR_LAUNCH_FAILED;
  const size_t launch_smem = smem;
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  // The output leaves through TMA stores of 32 x 32 boxes whenever its rows allow 128-bit accesses.
  p.tma_store = (p.vector_io && make_tensor_map_2d(&p.map_d, q.d, q.m, q.n, q.ldd, 32, 32, Swizzle::k128B)) ? 1 : 0;
  // One copy per B slab when the columns split into whole 32-wide strips.
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, BN / 32,
                                                        Swizzle::k128BAtom32B))
                   ? BN / 32
                   : 0;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kIssuers == 2 ? kTileThreadsTwoIssuers : kTileThreads);
  cfg.dynamicSmemBytes = launch_smem;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(1);
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

template <int BN, int STAGES, int kAct>
int launch_tma(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  // K sub-blocks per pipeline stage. An MMA thread pays about 300 cycles per stage (barrier wait,
  // fence, commit) next to 58 per instruction, so the 128 x 64 and 128 x 128 tiles put two sub-blocks
  // behind one pair of barriers and give each to its own issuing thread (kIssuers below); the ring
  // must still hold three or four such stages to cover the load latency. Measured on a B200 with one
  // issuer, unsplit, with a source: 128 x 128 at 1280 x 1280 x 8192 took 97 us with 2 stages of 2,
  // 72 us with 3 of 2, 81 us with 2 of 3, 84 us with 6 of 1; 128 x 64 at 1024 x 1024 x 4096 took 35.4 us
  // with 4 stages of 2 and 29.4 us with 2 of 4 - with two issuers 22.8 us with 4 of 2 against 26.2 with
  // 2 of 4 (graph-timed). The 128 x 256 tile (134 cycles of tensor pipe per instruction: the pipe, not
  // the thread, is its limit) is slower with two sub-blocks per stage (2048 x 2048 x 8192: 129-140
  // against 107-122 us): only two stages fit.
  // With two issuers the 128 x 128 tile has two forms: two sub-blocks per stage, one per issuer
  // (three stages), or single-block stages that the issuers take in turn (six stages: more bytes in
  // flight, 0.21 instead of 0.235 us per K block, but 0.6 us more to get going). Graph-timed with a
  // source and ReLU: 1536^3 15.8 against 16.4 us, 512 x 4096 x 4096 35.8 / 33.8, 1280 x 1280 x 8192
  // 65.9 / 60.8.
  if constexpr (BN == 128 && STAGES == 6) {
    if (q.k > 2560) return launch_tma_with<BN, STAGES, kAct, 1>(q, peers, stream);
  }
  constexpr int KSUB = (BN <= 128 && STAGES % 2 == 0 && STAGES >= 4) ? 2 : 1;
  return launch_tma_with<BN, STAGES, kAct, KSUB>(q, peers, stream);
}

template <int BN, int STAGES, int kAct>
int launch_generic(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  auto kernel = umma_generic_kernel<BN, STAGES, kAct>;
  constexpr size_t smem = smem_bytes<BN, STAGES>();
  if (!ensure_dynamic_smem<umma_generic_kernel<BN, STAGES, kAct>, smem>()) return B200_ERR_LAUNCH_FAILED;
  const size_t launch_smem = smem;
  UmmaParams p;
  fill_common(&p, q, peers);
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kGenericThreads);
  cfg.dynamicSmemBytes = launch_smem;
  cfg.stream = stream;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(1);
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}
}  // namespace

int launch_tf32_tile(int tile_n, int stages, int act, const b200_gemm_problem& q, const PeerOutputs& peers,
                     cudaStream_t stream) {
#define B200_TILE_CASE(BN, ST)                                                                     \
  if (tile_n == BN && stages == ST) {                                                              \
    switch (act) {                                                                                 \
      case B200_EPILOGUE_LINEAR: return launch_tma<BN, ST, B200_EPILOGUE_LINEAR>(q, peers, stream); \
      case B200_EPILOGUE_RELU: return launch_tma<BN, ST, B200_EPILOGUE_RELU>(q, peers, stream);     \
      case B200_EPILOGUE_GELU: return launch_tma<BN, ST, B200_EPILOGUE_GELU>(q, peers, stream);     \
      default: return B200_ERR_INVALID_ARGUMENT;                                                   \
    }                                                                                              \
  }
  B200_TILE_CASE(256, 4)
  B200_TILE_CASE(224, 4)
  B200_TILE_CASE(192, 4)
  B200_TILE_CASE(160, 5)
  B200_TILE_CASE(128, 6)
  B200_TILE_CASE(96, 6)
  B200_TILE_CASE(32, 8)
  B200_TILE_CASE(64, 8)
#undef B200_TILE_CASE
  // Configurations that exist with the linear epilogue only (the reference's stage and warp-shape variants).
  if (act != B200_EPILOGUE_LINEAR) return B200_ERR_INVALID_ARGUMENT;
  if (tile_n == 64 && stages == 4) return launch_tma<64, 4, B200_EPILOGUE_LINEAR>(q, peers, stream);
  if (tile_n == 128 && stages == 3) return launch_tma<128, 3, B200_EPILOGUE_LINEAR>(q, peers, stream);
  if (tile_n == 128 && stages == 2) return launch_tma<128, 2, B200_EPILOGUE_LINEAR>(q, peers, stream);
  return B200_ERR_INVALID_ARGUMENT;
}

int launch_tf32_generic(int tile_n, int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  if (tile_n == 128) {
    switch (act) {
      case B200_EPILOGUE_LINEAR: return launch_generic<128, 4, B200_EPILOGUE_LINEAR>(q, peers, stream);
      case B200_EPILOGUE_RELU: return launch_generic<128, 4, B200_EPILOGUE_RELU>(q, peers, stream);
      case B200_EPILOGUE_GELU: return launch_generic<128, 4, B200_EPILOGUE_GELU>(q, peers, stream);
      default: return B200_ERR_INVALID_ARGUMENT;
    }
  }
  if (tile_n == 64 && act == B200_EPILOGUE_LINEAR) return launch_generic<64, 4, B200_EPILOGUE_LINEAR>(q, peers, stream);
  return B200_ERR_INVALID_ARGUMENT;
}

}  // namespace b200
