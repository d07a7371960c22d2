// FP32 SIMT GEMM ladder, stages 6-8, rebuilt for sm_100a: persistent CTAs, one
// producer thread feeding a multi-stage shared-memory ring with TMA
// bulk-tensor loads, eight consumer warps running the FMA pipe off that ring,
// full/empty mbarrier pairs instead of block-wide barriers.
//
//   prefetch_smem : the ring alone (the reference's cp.async double buffer,
//                   csrc/gemm/gemm_prefetchSmem.cu:100-169, becomes N stages).
//   prefetch_reg  : ring + register double buffer of the shared-memory
//                   fragments carried across stage boundaries, and packed
//                   two-wide FMAs (csrc/gemm/gemm_prefetchRegister.cu:125-190).
//   split_k       : prefetch_reg on two K slices per output tile, reduced with
//                   128-bit vector reductions into an output that the launcher
//                   clears on the same stream (csrc/gemm/gemm_splictK.cu:101-209).
//
// Layout in shared memory per stage: A slab [BK][128] (row kk = 128 consecutive
// m of storage row k) and B slab [BK][128]; both arrive exactly as one TMA box.
// K tails and K slices are handled by the tensor maps: rows past a slice's
// extent read as zeros.
#include "sgemm.h"
#include "ptx_sm100.cuh"

namespace b200 {

cudaError_t sgemm_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

constexpr int kTile = 128;               // CTA tile is kTile x kTile
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one producer warp

struct PipelineParams {
  CUtensorMap map_a[2];  // per K slice: [k_slice][M] view of A storage
  CUtensorMap map_b[2];  // per K slice: [k_slice][N] view of B
  float* c;
  int n;
  int tiles_m, tiles_n;
  int k_blocks;          // ceil(k_slice / BK)
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

// Fragment of one k: eight A values (two groups of four rows, 32 apart) and
// eight B values (two groups of four columns, 16 apart).
struct Fragment {
  float4 a_lo, a_hi, b_lo, b_hi;
};

__device__ __forceinline__ void load_fragment(Fragment& f, const float* a_slab, const float* b_slab, int kk) {
  f.a_lo = lds128(a_slab + kk * kTile);
  f.a_hi = lds128(a_slab + kk * kTile + 32);
  f.b_lo = lds128(b_slab + kk * kTile);
  f.b_hi = lds128(b_slab + kk * kTile + 16);
}

// acc[i][j] += a[i] * b[j] for the 8 x 8 register tile.
template <bool kPacked>
__device__ __forceinline__ void outer_product(float (&acc)[8][8], const Fragment& f) {
  const float a[8] = {f.a_lo.x, f.a_lo.y, f.a_lo.z, f.a_lo.w, f.a_hi.x, f.a_hi.y, f.a_hi.z, f.a_hi.w};
  if constexpr (kPacked) {
    // fma.rn.f32x2: one instruction, two FMAs. B supplies natural pairs, A is
    // broadcast into both halves.
    const float2 b2[4] = {make_float2(f.b_lo.x, f.b_lo.y), make_float2(f.b_lo.z, f.b_lo.w),
                          make_float2(f.b_hi.x, f.b_hi.y), make_float2(f.b_hi.z, f.b_hi.w)};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 a2 = make_float2(a[i], a[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2& d = *reinterpret_cast<float2*>(&acc[i][2 * j]);
        d = __ffma2_rn(a2, b2[j], d);
      }
    }
  } else {
    const float b[8] = {f.b_lo.x, f.b_lo.y, f.b_lo.z, f.b_lo.w, f.b_hi.x, f.b_hi.y, f.b_hi.z, f.b_hi.w};
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

template <int BK, int STAGES, bool kRegPrefetch, bool kPacked, int SPLIT>
__global__ void __launch_bounds__(kThreads, 1) sgemm_pipeline_kernel(const __grid_constant__ PipelineParams p) {
  using Layout = SmemLayout<BK, STAGES>;
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
      mbar_init(&full_bar[s], 1);                // one arrive.expect_tx from the producer
      mbar_init(&empty_bar[s], kConsumerWarps);  // one arrive per consumer warp
    }
    mbar_init_fence();
  }
  __syncthreads();

  const int units = p.tiles_m * p.tiles_n * SPLIT;

  if (tid >= kConsumerThreads) {
    // ------------------------------------------------------------ producer
    if (tid != kConsumerThreads) return;
    prefetch_tensormap(&p.map_a[0]);
    prefetch_tensormap(&p.map_b[0]);
    int stage = 0;
    uint32_t phase = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const int slice = unit % SPLIT;
      int tm, tn;
      tile_coords(unit / SPLIT, p.tiles_m, p.tiles_n, &tm, &tn);
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        // A stage is free once every consumer warp released its previous use.
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, kSiteSgemmEmpty)) return;
        mbar_expect_tx(&full_bar[stage], Layout::kStageBytes);
        float* a_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats;
        tma_load_2d(a_slab, &p.map_a[slice], &full_bar[stage], tm * kTile, kb * BK);
        tma_load_2d(a_slab + Layout::kSlabFloats, &p.map_b[slice], &full_bar[stage], tn * kTile, kb * BK);
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
    }
    return;
  }

  // ---------------------------------------------------------------- consumers
  const int warp = tid >> 5, lane = tid & 31;
  // 2 x 4 warps of 64 x 32; 8 x 4 lanes; 2 x 2 blocks of 4 x 4 per thread.
  const int row0 = (warp >> 2) * 64 + (lane >> 2) * 4;
  const int col0 = (warp & 3) * 32 + (lane & 3) * 4;

  int stage = 0;
  uint32_t phase = 0;
  for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
    int tm, tn;
    tile_coords(unit / SPLIT, p.tiles_m, p.tiles_n, &tm, &tn);

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    if constexpr (kRegPrefetch) {
      Fragment frag[2];
      if (!mbar_wait(&full_bar[stage], phase, kSiteSgemmFull)) return;
      const float* a_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + row0;
      const float* b_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + Layout::kSlabFloats + col0;
      load_fragment(frag[0], a_slab, b_slab, 0);
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        const int this_stage = stage;
        if (++stage == STAGES) stage = 0, phase ^= 1u;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
          if (kk + 1 < BK) {
            load_fragment(frag[(kk + 1) & 1], a_slab, b_slab, kk + 1);
          } else if (kb + 1 < p.k_blocks) {
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
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, kSiteSgemmFull)) return;
        const float* a_slab = slabs + static_cast<size_t>(stage) * 2 * Layout::kSlabFloats + row0;
        const float* b_slab = a_slab - row0 + Layout::kSlabFloats + col0;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
          Fragment f;
          load_fragment(f, a_slab, b_slab, kk);
          outer_product<kPacked>(acc, f);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
    }

    // Epilogue straight from registers: every store instruction of a warp
    // covers eight rows x 64 contiguous bytes.
    float* c_tile = p.c + static_cast<int64_t>(tm * kTile + row0) * p.n + tn * kTile + col0;
#pragma unroll
    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float* c_row = c_tile + static_cast<int64_t>(rb * 32 + i) * p.n;
        const float* v = acc[rb * 4 + i];
        if constexpr (SPLIT == 1) {
          *reinterpret_cast<float4*>(c_row) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(c_row + 16) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          red_add_v4(c_row, v[0], v[1], v[2], v[3]);
          red_add_v4(c_row + 16, v[4], v[5], v[6], v[7]);
        }
      }
  }
}

template <int BK, int STAGES, bool kRegPrefetch, bool kPacked, int SPLIT>
int launch_pipeline(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream) {
  using Layout = SmemLayout<BK, STAGES>;
  auto kernel = sgemm_pipeline_kernel<BK, STAGES, kRegPrefetch, kPacked, SPLIT>;
  // Function attributes are per device; setting them again is cheap and keeps
  // the launcher free of per-device state.
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Layout::kBytes)) !=
      cudaSuccess) {
    return B200_ERR_LAUNCH_FAILED;
  }
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;

  PipelineParams p;
  const int k_slice = k / SPLIT;
  for (int s = 0; s < SPLIT; ++s) {
    const float* a_slice = a + static_cast<int64_t>(s) * k_slice * m;
    const float* b_slice = b + static_cast<int64_t>(s) * k_slice * n;
    if (!make_tensor_map_2d(&p.map_a[s], a_slice, k_slice, m, m, BK, kTile, Swizzle::kNone) ||
        !make_tensor_map_2d(&p.map_b[s], b_slice, k_slice, n, n, BK, kTile, Swizzle::kNone)) {
      return B200_ERR_MISALIGNED_OPERAND;
    }
  }
  for (int s = SPLIT; s < 2; ++s) p.map_a[s] = p.map_a[0], p.map_b[s] = p.map_b[0];
  p.c = c;
  p.n = n;
  p.tiles_m = m / kTile;
  p.tiles_n = n / kTile;
  p.k_blocks = (k_slice + BK - 1) / BK;

  if (SPLIT > 1) {
    if (cudaMemsetAsync(c, 0, static_cast<size_t>(m) * n * sizeof(float), stream) != cudaSuccess) {
      return B200_ERR_LAUNCH_FAILED;
    }
  }
  const int64_t units = static_cast<int64_t>(p.tiles_m) * p.tiles_n * SPLIT;
  const int grid = static_cast<int>(units < sms ? units : sms);
  kernel<<<grid, kThreads, Layout::kBytes, stream>>>(p);
  return launch_status();
}

}  // namespace

int sgemm_pipeline_launch(int impl, const float* a, const float* b, float* c, int m, int n, int k,
                          cudaStream_t stream) {
  switch (impl) {
    case B200_SGEMM_PREFETCH_SMEM:
      return launch_pipeline<16, 8, false, false, 1>(a, b, c, m, n, k, stream);
    case B200_SGEMM_PREFETCH_REG:
      return launch_pipeline<16, 8, true, true, 1>(a, b, c, m, n, k, stream);
    case B200_SGEMM_SPLIT_K:
      return launch_pipeline<16, 8, true, true, 2>(a, b, c, m, n, k, stream);
    default:
      return B200_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace b200
