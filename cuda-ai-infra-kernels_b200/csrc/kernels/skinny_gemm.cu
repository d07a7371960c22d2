// Skinny GEMM for decode-like shapes: D[M,N] = act(alpha * A[M,K] @ B[K,N] + beta * C + bias)
// with M <= 16, all operands row-major FP32.
//
// With so few rows the product is a stream over B (K * N * 4 bytes, read once)
// and the bound is HBM bandwidth, not arithmetic: a 128-row tensor-core tile
// would leave most SMs idle (N / 128 tiles) and waste 7/8 of every MMA. Here
//   * a CTA owns 128 columns (one float4 per lane) and its eight warps take
//     eight different K ranges of those columns;
//   * 1, 2, 4 or 8 such CTAs form a thread-block cluster and split K further,
//     so that N / 128 * cluster CTAs cover the SMs about twice;
//   * each warp keeps its slice of A in shared memory (read back as broadcast
//     128-bit loads) and accumulates M x 4 outputs per lane in FP32 (plain FMA:
//     more exact than the TF32 kernels this entry stands in for);
//   * the K partials meet in shared memory: first across the warps of a CTA,
//     then across the cluster through distributed shared memory, where CTA r
//     finishes a 1/cluster share of the 16 x 128 outputs and applies the
//     epilogue. No scratch buffer, no atomics, no second launch.
// The shapes come from the reference's benchmark list (benchmarks/shapes/gemm.yaml:5-6,
// m = 1 and m = 16 with n = k = 4096), which its tile kernels cannot run.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "host_common.h"
#include "tf32_gemm.h"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kCols = 128;    // columns per CTA
constexpr int kChunk = 64;    // K rows of A staged per warp at a time
constexpr int kUnroll = 8;    // B rows in flight per thread

struct SkinnyParams {
  const float* a;
  const float* b;
  const float* c;     // null when beta == 0
  const float* bias;  // null when absent
  float* d;
  int64_t lda, ldb, ldc, ldd;
  int m, n, k;
  int k_per_split;    // K rows per (CTA, warp) range, a multiple of kUnroll
  float alpha, beta;
};

template <int kAct>
__device__ __forceinline__ float activate(float v) {
  if constexpr (kAct == B200_EPILOGUE_RELU) return fmaxf(v, 0.f);
  if constexpr (kAct == B200_EPILOGUE_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  return v;
}

template <int MR>
__host__ __device__ constexpr size_t skinny_smem_bytes() {
  // A slices [warps][MR][chunk] + warp partials [warps][MR][cols] + CTA sums [MR][cols]
  return sizeof(float) * (kWarps * MR * kChunk + kWarps * MR * kCols + MR * kCols);
}

template <int MR, int kAct>
__global__ void __launch_bounds__(kThreads, 2) skinny_gemm_kernel(const SkinnyParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  const int ranks = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = (blockIdx.x / ranks) * kCols;

  extern __shared__ __align__(16) float skinny_smem[];
  float* a_stage = skinny_smem + warp * MR * kChunk;              // this warp's slice of A
  float* partial = skinny_smem + kWarps * MR * kChunk;            // [warps][MR][cols]
  float* cta_sum = partial + kWarps * MR * kCols;                 // [MR][cols]

  const int split = rank * kWarps + warp;
  const int k_begin = static_cast<int>(min(static_cast<int64_t>(p.k), static_cast<int64_t>(split) * p.k_per_split));
  const int k_end = static_cast<int>(min(static_cast<int64_t>(p.k), static_cast<int64_t>(k_begin) + p.k_per_split));
  const int col = col0 + lane * 4;
  const bool col_ok = col < p.n;  // n % 4 == 0: a float4 is inside or outside as a whole

  float acc[MR][4];
#pragma unroll
  for (int m = 0; m < MR; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;

  for (int k0 = k_begin; k0 < k_end; k0 += kChunk) {
    __syncwarp();  // the previous chunk of A has been consumed
#pragma unroll
    for (int m = 0; m < MR; ++m) {
#pragma unroll
      for (int half = 0; half < kChunk / 32; ++half) {
        const int gk = k0 + half * 32 + lane;
        a_stage[m * kChunk + half * 32 + lane] =
            (m < p.m && gk < k_end) ? __ldg(p.a + static_cast<int64_t>(m) * p.lda + gk) : 0.f;
      }
    }
    __syncwarp();
    const int rows = min(kChunk, k_end - k0);
    for (int kk = 0; kk < rows; kk += kUnroll) {
      float4 bv[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int r = k0 + kk + u;
        bv[u] = (col_ok && r < k_end) ? __ldg(reinterpret_cast<const float4*>(p.b + static_cast<int64_t>(r) * p.ldb + col))
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float4 a_lo = *reinterpret_cast<const float4*>(a_stage + m * kChunk + kk);
        const float4 a_hi = *reinterpret_cast<const float4*>(a_stage + m * kChunk + kk + 4);
        const float av[kUnroll] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          acc[m][0] = fmaf(av[u], bv[u].x, acc[m][0]);
          acc[m][1] = fmaf(av[u], bv[u].y, acc[m][1]);
          acc[m][2] = fmaf(av[u], bv[u].z, acc[m][2]);
          acc[m][3] = fmaf(av[u], bv[u].w, acc[m][3]);
        }
      }
    }
  }

  // Across the warps of this CTA.
#pragma unroll
  for (int m = 0; m < MR; ++m) {
    *reinterpret_cast<float4*>(partial + (warp * MR + m) * kCols + lane * 4) =
        make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < MR * kCols; e += kThreads) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += partial[w * MR * kCols + e];
    cta_sum[e] = sum;
  }
  cluster.sync();

  // Across the cluster: CTA `rank` finishes a contiguous share of the outputs.
  const int share = MR * kCols / ranks;
  for (int e = rank * share + threadIdx.x; e < (rank + 1) * share; e += kThreads) {
    float sum = 0.f;
    for (int peer = 0; peer < ranks; ++peer) sum += cluster.map_shared_rank(cta_sum, peer)[e];
    const int m = e / kCols, n = col0 + e % kCols;
    if (m < p.m && n < p.n) {
      float v = p.alpha * sum;
      if (p.c != nullptr) v = fmaf(p.beta, __ldg(p.c + static_cast<int64_t>(m) * p.ldc + n), v);
      if (p.bias != nullptr) v += __ldg(p.bias + n);
      p.d[static_cast<int64_t>(m) * p.ldd + n] = activate<kAct>(v);
    }
  }
  cluster.sync();  // no CTA leaves while a peer may still read its sums
}

template <int MR, int kAct>
int launch_rows(const SkinnyParams& p, int ranks, cudaStream_t stream) {
  auto kernel = skinny_gemm_kernel<MR, kAct>;
  constexpr size_t smem = skinny_smem_bytes<MR>();
  if (!ensure_dynamic_smem<skinny_gemm_kernel<MR, kAct>, smem>()) return B200_ERR_LAUNCH_FAILED;
  const int64_t column_blocks = (p.n + kCols - 1) / kCols;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(column_blocks * ranks));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(ranks);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_failed();
  return launch_status();
}

template <int kAct>
int launch_act(const SkinnyParams& p, int ranks, cudaStream_t stream) {
  if (p.m <= 1) return launch_rows<1, kAct>(p, ranks, stream);
  if (p.m <= 2) return launch_rows<2, kAct>(p, ranks, stream);
  if (p.m <= 4) return launch_rows<4, kAct>(p, ranks, stream);
  if (p.m <= 8) return launch_rows<8, kAct>(p, ranks, stream);
  return launch_rows<16, kAct>(p, ranks, stream);
}

}  // namespace

int launch_skinny(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  if (peers.count > 0) return B200_ERR_NOT_SUPPORTED;
  if (q.m > kSkinnyMaxRows || q.n % 4 != 0) return B200_ERR_INVALID_PROBLEM;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t column_blocks = (static_cast<int64_t>(q.n) + kCols - 1) / kCols;
  if (column_blocks * 8 > 0x7fffffffLL) return B200_ERR_INVALID_PROBLEM;
  // Cluster size: cover the SMs about twice, but keep at least kUnroll K rows per warp.
  int ranks = 1;
  while (ranks < 8 && column_blocks * ranks < 2LL * sms && q.k / (kWarps * ranks * 2) >= kUnroll) ranks *= 2;
  SkinnyParams p;
  p.a = q.a, p.b = q.b, p.d = q.d;
  p.c = q.beta != 0.f ? q.c : nullptr;
  p.bias = q.bias;
  p.lda = q.lda, p.ldb = q.ldb, p.ldc = q.ldc, p.ldd = q.ldd;
  p.m = q.m, p.n = q.n, p.k = q.k;
  const int splits = kWarps * ranks;
  const int per = (q.k + splits - 1) / splits;
  p.k_per_split = (per + kUnroll - 1) / kUnroll * kUnroll;
  p.alpha = q.alpha, p.beta = q.beta;
  switch (q.epilogue) {
    case B200_EPILOGUE_LINEAR: return launch_act<B200_EPILOGUE_LINEAR>(p, ranks, stream);
    case B200_EPILOGUE_RELU: return launch_act<B200_EPILOGUE_RELU>(p, ranks, stream);
    case B200_EPILOGUE_GELU: return launch_act<B200_EPILOGUE_GELU>(p, ranks, stream);
    default: return B200_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace b200
