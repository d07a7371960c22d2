// FP32 SIMT GEMM ladder, stages 1-5: one output per thread, shared-memory
// staging (scalar and 128-bit), register thread tiles and the warp-tiled
// mapping. C[M,N] = A[M,K] * B[K,N] with A stored column-major (a contiguous
// [K,M] array), B and C row-major. Full tiles only; sizes are validated on the
// host (b200_sgemm_check) and the kernels do no bounds checks.
//
// Stages 2-3 (one output per thread) have a small double-buffered kernel of
// their own; stages 4-5 share one kernel template: a CTA stages a [BK][BM] slab
// of A and a [BK][BN] slab of B in shared memory, and every thread accumulates
// RM x RN register blocks of 4 x 4 outputs whose origins inside the CTA tile
// come from a mapping policy. Tile sizes and work decomposition are those of
// each ladder step of the reference (csrc/gemm/gemm_block_tile.cu,
// gemm_block_tile_float4.cu, gemm_thread_tile.cu, gemm_warp_tile.cu).
#include "sgemm.h"

namespace b200 {
namespace {

// ---------------------------------------------------------------- stage 1

__global__ void __launch_bounds__(256) sgemm_naive_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          float* __restrict__ c, int m, int n, int k) {
  const int col = blockIdx.x * 16 + threadIdx.x;
  const int row = blockIdx.y * 16 + threadIdx.y;
  const float* a_col = a + row;  // walks k with stride m
  const float* b_col = b + col;  // walks k with stride n
  float acc = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    acc = fmaf(a_col[static_cast<int64_t>(kk) * m], b_col[static_cast<int64_t>(kk) * n], acc);
  }
  c[static_cast<int64_t>(row) * n + col] = acc;
}

// ------------------------------------------------- register-tiled stages

// One contiguous TM x TN rectangle per thread (stage 4). With kWarp4x8 the
// threads of a warp form 4 rows x 8 columns of rectangles instead of one row.
template <int BM, int BN, int TM, int TN, bool kWarp4x8>
struct MapThreadTile {
  static_assert(TM % 4 == 0 && TN % 4 == 0, "register blocks are 4 wide");
  static constexpr int kThreads = (BM / TM) * (BN / TN);
  static constexpr int kRowBlocks = TM / 4, kColBlocks = TN / 4, kBlockRows = 4, kBlockCols = 4;
  int ty, tx;
  __device__ explicit MapThreadTile(int tid) {
    if constexpr (kWarp4x8) {
      constexpr int kWarpsAcross = BN / (8 * TN);
      const int warp = tid >> 5, lane = tid & 31;
      ty = (warp / kWarpsAcross) * 4 + (lane >> 3);
      tx = (warp % kWarpsAcross) * 8 + (lane & 7);
    } else {
      ty = tid / (BN / TN);
      tx = tid % (BN / TN);
    }
  }
  __device__ int row_origin(int r) const { return ty * TM + 4 * r; }
  __device__ int col_origin(int c) const { return tx * TN + 4 * c; }
};

// Stage 5: 2 x 4 warps of 64 x 32; inside a warp 8 x 4 lanes; each thread owns
// 2 x 2 blocks of 4 x 4, the row blocks 32 apart and the column blocks 16
// apart, so that a warp-wide 128-bit shared load touches one 128-byte line.
struct MapWarpTile {
  static constexpr int kThreads = 256;
  static constexpr int kRowBlocks = 2, kColBlocks = 2, kBlockRows = 4, kBlockCols = 4;
  int row0, col0;
  __device__ explicit MapWarpTile(int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    row0 = (warp >> 2) * 64 + (lane >> 2) * 4;
    col0 = (warp & 3) * 32 + (lane & 3) * 4;
  }
  __device__ int row_origin(int r) const { return row0 + 32 * r; }
  __device__ int col_origin(int c) const { return col0 + 16 * c; }
};

// Register-tiled stages: BM x BN outputs per CTA, `[BK][BM]` / `[BK][BN]` slabs in shared memory,
// staged with 128-bit loads. The slabs are double-buffered and the next one travels from global
// memory in registers while the current one is multiplied: one barrier per slab, global-load
// latency off the critical path.
template <int BM, int BN, int BK, class Map>
__global__ void __launch_bounds__(Map::kThreads) sgemm_smem_kernel(const float* __restrict__ a,
                                                                     const float* __restrict__ b,
                                                                     float* __restrict__ c, int m, int n, int k) {
  constexpr int kThreads = Map::kThreads;
  constexpr int RM = Map::kRowBlocks, RN = Map::kColBlocks, CM = Map::kBlockRows, CN = Map::kBlockCols;
  constexpr int kItemsA = BK * BM / 4, kItemsB = BK * BN / 4;   // 128-bit items per slab
  constexpr int kPerThreadA = (kItemsA + kThreads - 1) / kThreads, kPerThreadB = (kItemsB + kThreads - 1) / kThreads;
  __shared__ __align__(16) float a_s2[2][BK][BM];
  __shared__ __align__(16) float b_s2[2][BK][BN];

  const int tid = threadIdx.x;
  const Map map(tid);
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;

  float acc[RM * CM][RN * CN];
#pragma unroll
  for (int i = 0; i < RM * CM; ++i)
#pragma unroll
    for (int j = 0; j < RN * CN; ++j) acc[i][j] = 0.f;

  // Row kk of either slab is contiguous in global memory.
  float4 ra[kPerThreadA], rb[kPerThreadB];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < kPerThreadA; ++i) {
      const int v = tid + i * kThreads, kk = v / (BM / 4), mm = (v % (BM / 4)) * 4;
      if (v < kItemsA) ra[i] = *reinterpret_cast<const float4*>(a + static_cast<int64_t>(k0 + kk) * m + m0 + mm);
    }
#pragma unroll
    for (int i = 0; i < kPerThreadB; ++i) {
      const int v = tid + i * kThreads, kk = v / (BN / 4), nn = (v % (BN / 4)) * 4;
      if (v < kItemsB) rb[i] = *reinterpret_cast<const float4*>(b + static_cast<int64_t>(k0 + kk) * n + n0 + nn);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < kPerThreadA; ++i) {
      const int v = tid + i * kThreads, kk = v / (BM / 4), mm = (v % (BM / 4)) * 4;
      if (v < kItemsA) *reinterpret_cast<float4*>(&a_s2[buf][kk][mm]) = ra[i];
    }
#pragma unroll
    for (int i = 0; i < kPerThreadB; ++i) {
      const int v = tid + i * kThreads, kk = v / (BN / 4), nn = (v % (BN / 4)) * 4;
      if (v < kItemsB) *reinterpret_cast<float4*>(&b_s2[buf][kk][nn]) = rb[i];
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < k; k0 += BK) {
    const bool more = k0 + BK < k;
    if (more) fetch(k0 + BK);
    const float (*a_s)[BM] = a_s2[buf];
    const float (*b_s)[BN] = b_s2[buf];

#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a_frag[RM * CM], b_frag[RN * CN];
#pragma unroll
      for (int r = 0; r < RM; ++r) {
        if constexpr (CM == 4) {
          const float4 v = *reinterpret_cast<const float4*>(&a_s[kk][map.row_origin(r)]);
          a_frag[4 * r + 0] = v.x, a_frag[4 * r + 1] = v.y, a_frag[4 * r + 2] = v.z, a_frag[4 * r + 3] = v.w;
        } else {
          a_frag[r] = a_s[kk][map.row_origin(r)];
        }
      }
#pragma unroll
      for (int cc = 0; cc < RN; ++cc) {
        if constexpr (CN == 4) {
          const float4 v = *reinterpret_cast<const float4*>(&b_s[kk][map.col_origin(cc)]);
          b_frag[4 * cc + 0] = v.x, b_frag[4 * cc + 1] = v.y, b_frag[4 * cc + 2] = v.z, b_frag[4 * cc + 3] = v.w;
        } else {
          b_frag[cc] = b_s[kk][map.col_origin(cc)];
        }
      }
#pragma unroll
      for (int i = 0; i < RM * CM; ++i)
#pragma unroll
        for (int j = 0; j < RN * CN; ++j) acc[i][j] = fmaf(a_frag[i], b_frag[j], acc[i][j]);
    }
    if (more) stash(buf ^ 1);
    // One barrier per slab: buffer buf ^ 1 was last read before the previous barrier.
    __syncthreads();
    buf ^= 1;
  }

#pragma unroll
  for (int r = 0; r < RM; ++r)
#pragma unroll
    for (int i = 0; i < CM; ++i) {
      const int64_t row = m0 + map.row_origin(r) + i;
#pragma unroll
      for (int cc = 0; cc < RN; ++cc) {
        const int col = n0 + map.col_origin(cc);
        if constexpr (CN == 4) {
          const float* v = acc[r * CM + i] + cc * 4;
          *reinterpret_cast<float4*>(c + row * n + col) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
          c[row * n + col] = acc[r * CM + i][cc];
        }
      }
    }
}

// Stages 2 to 5 (one output per thread, BM x BN outputs per CTA, operands staged in shared memory).
// With one output per thread every FMA needs one element of A and one of B from shared memory, so
// the kernel runs at the rate of the shared-memory pipe: the layout decides the speed. Slabs of
// kSlabK = 32 values of K are therefore stored K-innermost (a_s[row][k], b_s[column][k], row pitch
// 36 floats): a thread reads four consecutive K values of its row and of its column with two
// 128-bit loads, which cost 1 (A: the lanes of a warp share one or two rows) + 4 (B: 32 columns,
// conflict-free at this pitch) wavefronts for four FMAs where k-outermost slabs cost 8. The two
// slabs are double-buffered and the next slab travels from global memory in registers while the
// current one is multiplied (one barrier per slab). The accumulation order is k = 0, 1, 2, ... in
// one FMA chain, as in the reference's stages. Tile sizes, the staging width (scalar or 128-bit
// global loads) and therefore the shape rules (K a multiple of 8) are those of the reference's
// stages (csrc/gemm/gemm_block_tile.cu:4-35, gemm_block_tile_float4.cu); a last slab may hold 8,
// 16 or 24 values of K.
template <int BM, int BN, bool kVectorStaging>
__global__ void __launch_bounds__(BM* BN) sgemm_block_tile_kernel(const float* __restrict__ a,
                                                                   const float* __restrict__ b,
                                                                   float* __restrict__ c, int m, int n, int k) {
  constexpr int kSlabK = 32, kPitch = kSlabK + 4;
  constexpr int kThreads = BM * BN;
  constexpr int kWidth = kVectorStaging ? 4 : 1;                  // floats per staged item
  constexpr int kItemsA = kSlabK * BM / kWidth, kItemsB = kSlabK * BN / kWidth;
  constexpr int kPerThreadA = (kItemsA + kThreads - 1) / kThreads, kPerThreadB = (kItemsB + kThreads - 1) / kThreads;
  __shared__ __align__(16) float a_s[2][BM][kPitch];
  __shared__ __align__(16) float b_s[2][BN][kPitch];

  const int tid = threadIdx.x;
  const int ty = tid / BN, tx = tid % BN;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float4 ra[kPerThreadA], rb[kPerThreadB];
  // Item i of a slab: K row i / (B / kWidth), kWidth consecutive rows (A) or columns (B) of the tile.
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < kPerThreadA; ++i) {
      const int item = tid + i * kThreads, kk = item / (BM / kWidth), mm = (item % (BM / kWidth)) * kWidth;
      ra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (item < kItemsA && k0 + kk < k) {
        const float* src = a + static_cast<int64_t>(k0 + kk) * m + m0 + mm;
        if constexpr (kVectorStaging) ra[i] = *reinterpret_cast<const float4*>(src);
        else ra[i].x = *src;
      }
    }
#pragma unroll
    for (int i = 0; i < kPerThreadB; ++i) {
      const int item = tid + i * kThreads, kk = item / (BN / kWidth), nn = (item % (BN / kWidth)) * kWidth;
      rb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (item < kItemsB && k0 + kk < k) {
        const float* src = b + static_cast<int64_t>(k0 + kk) * n + n0 + nn;
        if constexpr (kVectorStaging) rb[i] = *reinterpret_cast<const float4*>(src);
        else rb[i].x = *src;
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < kPerThreadA; ++i) {
      const int item = tid + i * kThreads, kk = item / (BM / kWidth), mm = (item % (BM / kWidth)) * kWidth;
      if (item < kItemsA) {
        a_s[buf][mm][kk] = ra[i].x;
        if constexpr (kVectorStaging) a_s[buf][mm + 1][kk] = ra[i].y, a_s[buf][mm + 2][kk] = ra[i].z, a_s[buf][mm + 3][kk] = ra[i].w;
      }
    }
#pragma unroll
    for (int i = 0; i < kPerThreadB; ++i) {
      const int item = tid + i * kThreads, kk = item / (BN / kWidth), nn = (item % (BN / kWidth)) * kWidth;
      if (item < kItemsB) {
        b_s[buf][nn][kk] = rb[i].x;
        if constexpr (kVectorStaging) b_s[buf][nn + 1][kk] = rb[i].y, b_s[buf][nn + 2][kk] = rb[i].z, b_s[buf][nn + 3][kk] = rb[i].w;
      }
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  float acc = 0.f;
  int buf = 0;
  for (int k0 = 0; k0 < k; k0 += kSlabK) {
    const bool more = k0 + kSlabK < k;
    if (more) fetch(k0 + kSlabK);
    const float4* a_row = reinterpret_cast<const float4*>(&a_s[buf][ty][0]);
    const float4* b_row = reinterpret_cast<const float4*>(&b_s[buf][tx][0]);
    if (k - k0 >= kSlabK) {
#pragma unroll
      for (int q = 0; q < kSlabK / 4; ++q) {
        const float4 av = a_row[q], bv = b_row[q];
        acc = fmaf(av.x, bv.x, acc);
        acc = fmaf(av.y, bv.y, acc);
        acc = fmaf(av.z, bv.z, acc);
        acc = fmaf(av.w, bv.w, acc);
      }
    } else {
      const int quads = (k - k0) / 4;   // 2, 4 or 6
      for (int q = 0; q < quads; ++q) {
        const float4 av = a_row[q], bv = b_row[q];
        acc = fmaf(av.x, bv.x, acc);
        acc = fmaf(av.y, bv.y, acc);
        acc = fmaf(av.z, bv.z, acc);
        acc = fmaf(av.w, bv.w, acc);
      }
    }
    if (more) stash(buf ^ 1);
    // One barrier per iteration: buffer buf ^ 1 was last read before the previous barrier.
    __syncthreads();
    buf ^= 1;
  }
  c[static_cast<int64_t>(m0 + ty) * n + n0 + tx] = acc;
}

template <int BM, int BN, bool kVectorStaging>
int launch_block_tile(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream) {
  sgemm_block_tile_kernel<BM, BN, kVectorStaging><<<dim3(n / BN, m / BM), BM * BN, 0, stream>>>(a, b, c, m, n, k);
  return launch_status();
}

template <int BM, int BN, int BK, class Map>
int launch_smem(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream) {
  sgemm_smem_kernel<BM, BN, BK, Map>
      <<<dim3(n / BN, m / BM), Map::kThreads, 0, stream>>>(a, b, c, m, n, k);
  return launch_status();
}

}  // namespace

int sgemm_ladder_launch(int impl, const float* a, const float* b, float* c, int m, int n, int k,
                        cudaStream_t stream) {
  switch (impl) {
    case B200_SGEMM_NAIVE:
      sgemm_naive_kernel<<<dim3(n / 16, m / 16), dim3(16, 16), 0, stream>>>(a, b, c, m, n, k);
      return launch_status();
    case B200_SGEMM_BLOCK_TILE:
      return launch_block_tile<16, 16, false>(a, b, c, m, n, k, stream);
    case B200_SGEMM_BLOCK_TILE_F4_16x16:
      return launch_block_tile<16, 16, true>(a, b, c, m, n, k, stream);
    case B200_SGEMM_BLOCK_TILE_F4_16x32:
      return launch_block_tile<16, 32, true>(a, b, c, m, n, k, stream);
    case B200_SGEMM_BLOCK_TILE_F4_32x32:
      return launch_block_tile<32, 32, true>(a, b, c, m, n, k, stream);
    case B200_SGEMM_THREAD_TILE_4x4:
      return launch_smem<128, 128, 8, MapThreadTile<128, 128, 4, 4, false>>(a, b, c, m, n, k, stream);
    case B200_SGEMM_THREAD_TILE_4x8:
      return launch_smem<128, 128, 8, MapThreadTile<128, 128, 4, 8, false>>(a, b, c, m, n, k, stream);
    case B200_SGEMM_THREAD_TILE_8x8:
      return launch_smem<128, 128, 8, MapThreadTile<128, 128, 8, 8, false>>(a, b, c, m, n, k, stream);
    case B200_SGEMM_THREAD_TILE_8x8_WARP4x8:
      return launch_smem<128, 128, 8, MapThreadTile<128, 128, 8, 8, true>>(a, b, c, m, n, k, stream);
    case B200_SGEMM_WARP_TILE:
      return launch_smem<128, 128, 8, MapWarpTile>(a, b, c, m, n, k, stream);
    default:
      return B200_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace b200
