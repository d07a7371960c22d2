// RMSNorm and softmax over the last dimension of a row-major FP32 matrix.
//
// Both operators are HBM-bound: the algorithmic traffic is one read of x and
// one write of y. Every fast path therefore keeps a whole row on chip (in
// registers, long rows in shared memory) between the reduction and the scaling
// pass (the reference re-reads x from
// global memory, csrc/rmsnorm/rmsnorm_naive.cu:70-89, or round-trips it through
// shared memory, csrc/rmsnorm/rmsnorm_cache_x.cu; its softmax makes three
// passes, csrc/softmax/softmax.cu:25-121). Paths, chosen by row length:
//
//   warp   : one warp per row, up to 8 x 128-bit vectors per lane
//            (rows of <= 1024 floats); shuffle reductions only.
//   block  : one CTA per row, up to 4 vectors per thread: 256 or 512 threads
//            (<= 4096 / 8192 floats); shuffle + one shared-memory hop.
//   staged : rows of more than 8192 floats. The copy engine brings a row (up to
//            28 672 floats: one CTA per row) or a CTA's share of it (beyond:
//            clusters of 2/4/8 CTAs per row, partial statistics exchanged
//            through distributed shared memory; up to 401 408 floats) into
//            shared memory with one bulk copy, the threads take their
//            statistics from there, overwrite the data in place with the
//            result, and one bulk copy writes it out. The memory system is kept
//            busy by the copy engine whatever phase the threads are in, and two
//            or three CTAs per SM are in flight (a register-resident cluster
//            path, tried first, ran such rows at 65-72 % of the copy bandwidth
//            and 131 072-float rows at 32-39 %; this one 70-97 % and 61-69 %).
//   stream : any length / any alignment; re-reads the row (normally from L2).
//
// All offsets are 64-bit. 128-bit accesses are used only when the row length
// is a multiple of four and the base pointers are 16-byte aligned.
#include <cooperative_groups.h>
#include <float.h>

#include <type_traits>

#include "host_common.h"
#include "ptx_sm100.cuh"

namespace cg = cooperative_groups;

namespace b200 {

cudaError_t rowops_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

constexpr int kMaxVec = 8;        // 128-bit vectors held per thread
constexpr int kBlockThreads = 256;
constexpr int kWarpsPerBlock = kBlockThreads / 32;

__device__ __forceinline__ float4 load_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void store_stream(float4* p, float4 v) { __stcs(p, v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct SumOp {
  static __device__ __forceinline__ float identity() { return 0.f; }
  static __device__ __forceinline__ float combine(float a, float b) { return a + b; }
  static __device__ __forceinline__ float warp(float v) { return warp_sum(v); }
};

struct MaxOp {
  static __device__ __forceinline__ float identity() { return -FLT_MAX; }
  static __device__ __forceinline__ float combine(float a, float b) { return fmaxf(a, b); }
  static __device__ __forceinline__ float warp(float v) { return warp_max(v); }
};

// Reduction scopes. Every thread receives the result.
struct WarpScope {
  template <class Op>
  __device__ __forceinline__ float reduce(float v) const {
    return Op::warp(v);
  }
};

template <int kWarps>
struct BlockScope {
  float* scratch;  // kWarps floats per reduction, two slots
  int slot = 0;
  template <class Op>
  __device__ __forceinline__ float reduce(float v) {
    v = Op::warp(v);
    float* s = scratch + slot * kWarps;
    slot ^= 1;  // the next reduction uses the other slot: no trailing barrier needed
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = Op::identity();
#pragma unroll
    for (int w = 0; w < kWarps; ++w) r = Op::combine(r, s[w]);
    return r;
  }
};

template <int kWarps>
struct ClusterScope {
  float* scratch;   // kWarps floats + 1 per slot, two slots
  int slot = 0;
  template <class Op>
  __device__ __forceinline__ float reduce(float v) {
    cg::cluster_group cluster = cg::this_cluster();
    v = Op::warp(v);
    float* s = scratch + slot * (kWarps + 1);
    slot ^= 1;
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float r = Op::identity();
#pragma unroll
      for (int w = 0; w < kWarps; ++w) r = Op::combine(r, s[w]);
      s[kWarps] = r;  // this CTA's partial, read by its peers
    }
    cluster.sync();
    float r = Op::identity();
    const unsigned ranks = cluster.num_blocks();
    for (unsigned peer = 0; peer < ranks; ++peer) {
      const float* remote = cluster.map_shared_rank(s, peer);
      r = Op::combine(r, remote[kWarps]);
    }
    return r;
  }
  // Peers may still be reading this CTA's shared memory: leave together.
  __device__ __forceinline__ void finish() const { cg::this_cluster().sync(); }
};

// ---------------------------------------------------------------- row bodies
// `x_row`/`y_row` point at the part of the row this scope's threads own,
// `nvec` 128-bit vectors long; thread `t` of `nthreads` handles vectors
// t, t + nthreads, ...; `row_len` is the full row length for the mean.

template <int VPT, class Scope>
__device__ __forceinline__ void rmsnorm_row(const float4* __restrict__ x_row, const float4* __restrict__ w_row,
                                            float4* __restrict__ y_row, int nvec, int t, int nthreads,
                                            int64_t row_len, double eps, Scope& scope) {
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * nthreads;
    if (idx < nvec) {
      v[i] = load_stream(x_row + idx);
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = scope.template reduce<SumOp>(ss);
  // Same arithmetic as the reference: FP32 mean, epsilon added in double,
  // single-precision reciprocal square root (csrc/rmsnorm/rmsnorm_naive.cu:62-65).
  const float inv_rms = rsqrtf(static_cast<float>(static_cast<double>(ss / static_cast<float>(row_len)) + eps));
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * nthreads;
    if (idx < nvec) {
      const float4 w = __ldg(w_row + idx);
      store_stream(y_row + idx, make_float4(v[i].x * w.x * inv_rms, v[i].y * w.y * inv_rms,
                                            v[i].z * w.z * inv_rms, v[i].w * w.w * inv_rms));
    }
  }
}

template <int VPT, class Scope>
__device__ __forceinline__ void softmax_row(const float4* __restrict__ x_row, float4* __restrict__ y_row, int nvec,
                                            int t, int nthreads, Scope& scope) {
  float4 v[VPT];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * nthreads;
    if (idx < nvec) {
      v[i] = load_stream(x_row + idx);
      mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
  }
  mx = scope.template reduce<MaxOp>(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * nthreads;
    if (idx < nvec) {
      v[i].x = __expf(v[i].x - mx), v[i].y = __expf(v[i].y - mx);
      v[i].z = __expf(v[i].z - mx), v[i].w = __expf(v[i].w - mx);
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  sum = scope.template reduce<SumOp>(sum);
  const float inv = __frcp_rn(sum);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * nthreads;
    if (idx < nvec) store_stream(y_row + idx, make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv));
  }
}

// -------------------------------------------------------------------- kernels

enum class RowOp { kRmsNorm, kSoftmax };

struct RowArgs {
  const float* x;
  const float* w;  // RMSNorm only
  float* y;
  int64_t rows;
  int64_t cols;
  double eps;      // RMSNorm only
};

template <RowOp kOp, int VPT>
__global__ void __launch_bounds__(kBlockThreads) row_warp_kernel(const RowArgs a) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int nvec = static_cast<int>(a.cols / 4);
  const float4* x_row = reinterpret_cast<const float4*>(a.x + row * a.cols);
  float4* y_row = reinterpret_cast<float4*>(a.y + row * a.cols);
  WarpScope scope;
  if constexpr (kOp == RowOp::kRmsNorm) {
    rmsnorm_row<VPT>(x_row, reinterpret_cast<const float4*>(a.w), y_row, nvec, threadIdx.x & 31, 32, a.cols, a.eps,
                     scope);
  } else {
    softmax_row<VPT>(x_row, y_row, nvec, threadIdx.x & 31, 32, scope);
  }
}

template <RowOp kOp, int VPT, int kThreads>
__global__ void __launch_bounds__(kThreads) row_block_kernel(const RowArgs a) {
  __shared__ float scratch[2 * (kThreads / 32)];
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = blockIdx.x;
  const int nvec = static_cast<int>(a.cols / 4);
  const float4* x_row = reinterpret_cast<const float4*>(a.x + row * a.cols);
  float4* y_row = reinterpret_cast<float4*>(a.y + row * a.cols);
  BlockScope<kThreads / 32> scope{scratch};
  if constexpr (kOp == RowOp::kRmsNorm) {
    rmsnorm_row<VPT>(x_row, reinterpret_cast<const float4*>(a.w), y_row, nvec, threadIdx.x, kThreads, a.cols, a.eps,
                     scope);
  } else {
    softmax_row<VPT>(x_row, y_row, nvec, threadIdx.x, kThreads, scope);
  }
}

// A row (or, with kCluster, a CTA's share of a row whose CTAs form a cluster and exchange their
// partial statistics through distributed shared memory) staged in shared memory by the copy
// engine (see the file header).
constexpr int kStagedThreads = 512;
constexpr int64_t kStagedMaxFloats = 50176;   // 196 KiB of row + barrier and reduction scratch inside 227 KiB
constexpr int64_t kStagedPartFloats = 24576;  // largest preferred share per CTA of a cluster: 96 KiB, two CTAs per SM
constexpr int64_t kStagedAloneFloats = 28672; // largest row one CTA takes alone: 112 KiB, two such CTAs still share an SM
                                              // (2048 x 28672 softmax: 6200 GB/s alone, 4435 as clusters of two; at
                                              // 32768 floats only one CTA fits an SM and the cluster form is ahead,
                                              // 4500 against 4120)

template <RowOp kOp, bool kCluster>
__global__ void __launch_bounds__(kStagedThreads) row_staged_kernel(const RowArgs a) {
  extern __shared__ __align__(128) uint8_t staged_raw[];
  grid_launch_dependents();
  grid_dependency_wait();
  // This CTA's vectors [begin, begin + nvec) of row r.
  int64_t r = blockIdx.x;
  int begin = 0;
  int nvec = static_cast<int>(a.cols / 4);
  if constexpr (kCluster) {
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned ranks = cluster.num_blocks();
    r = blockIdx.x / ranks;
    const int per_cta = (nvec + ranks - 1) / ranks;
    begin = min(static_cast<int>(cluster.block_rank()) * per_cta, nvec);
    nvec = min(per_cta, nvec - begin);
  }
  float4* row = reinterpret_cast<float4*>(staged_raw);
  const uint32_t bytes = static_cast<uint32_t>(nvec) * 16u;
  // Barrier and scratch sit behind the largest share any CTA of this launch can have.
  const uint32_t share_bytes = kCluster ? static_cast<uint32_t>((a.cols / 4 + gridDim.x / a.rows - 1) / (gridDim.x / a.rows)) * 16u
                                        : bytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(staged_raw + ((share_bytes + 127u) & ~127u));
  float* scratch = reinterpret_cast<float*>(bar + 2);
  const float* x_part = a.x + r * a.cols + 4 * static_cast<int64_t>(begin);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
    if (bytes > 0) {
      mbar_expect_tx(bar, bytes);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(row)), "l"(reinterpret_cast<uint64_t>(x_part)), "r"(bytes), "r"(smem_u32(bar))
                   : "memory");
    } else {
      mbar_arrive(bar);
    }
  }
  __syncthreads();   // the barrier exists before anybody polls it
  const bool arrived = mbar_wait(bar, 0, kSiteRowStaged);   // on failure the statistics below are garbage, nothing is stored
  using Scope = typename std::conditional<kCluster, ClusterScope<kStagedThreads / 32>, BlockScope<kStagedThreads / 32>>::type;
  Scope scope{scratch};
  if constexpr (kOp == RowOp::kRmsNorm) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < nvec; i += kStagedThreads) {
      const float4 v = row[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = scope.template reduce<SumOp>(ss);
    const float inv_rms = rsqrtf(static_cast<float>(static_cast<double>(ss / static_cast<float>(a.cols)) + a.eps));
    const float4* w = reinterpret_cast<const float4*>(a.w) + begin;
    for (int i = threadIdx.x; i < nvec; i += kStagedThreads) {
      const float4 v = row[i], g = __ldg(w + i);
      row[i] = make_float4(v.x * g.x * inv_rms, v.y * g.y * inv_rms, v.z * g.z * inv_rms, v.w * g.w * inv_rms);
    }
  } else {
    // Maximum and sum of exponentials of THIS CTA's share first (block-wide reductions only); a
    // cluster then exchanges the (maximum, sum) pairs once and rescales: exp(x - m_i) is already in
    // shared memory and only needs the factor exp(m_i - M) / S. One cluster barrier instead of two.
    BlockScope<kStagedThreads / 32> local{scratch};
    float mx = -FLT_MAX;
    for (int i = threadIdx.x; i < nvec; i += kStagedThreads) {
      const float4 v = row[i];
      mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
    mx = local.template reduce<MaxOp>(mx);
    float sum = 0.f;
    for (int i = threadIdx.x; i < nvec; i += kStagedThreads) {   // a thread revisits only its own vectors
      float4 v = row[i];
      v.x = __expf(v.x - mx), v.y = __expf(v.y - mx), v.z = __expf(v.z - mx), v.w = __expf(v.w - mx);
      sum += (v.x + v.y) + (v.z + v.w);
      row[i] = v;
    }
    sum = local.template reduce<SumOp>(sum);
    float factor;
    if constexpr (kCluster) {
      cg::cluster_group cluster = cg::this_cluster();
      float* pair = scratch + 2 * (kStagedThreads / 32);   // behind the two reduction slots
      if (threadIdx.x == 0) pair[0] = mx, pair[1] = sum;
      cluster.sync();
      float row_max = -FLT_MAX;
      const unsigned ranks = cluster.num_blocks();
      for (unsigned peer = 0; peer < ranks; ++peer) row_max = fmaxf(row_max, cluster.map_shared_rank(pair, peer)[0]);
      float total = 0.f;
      for (unsigned peer = 0; peer < ranks; ++peer) {
        const float* remote = cluster.map_shared_rank(pair, peer);
        total += remote[1] * __expf(remote[0] - row_max);   // an empty share contributes 0 * exp(-FLT_MAX - M) = 0
      }
      factor = __expf(mx - row_max) * __frcp_rn(total);
    } else {
      factor = __frcp_rn(sum);
    }
    for (int i = threadIdx.x; i < nvec; i += kStagedThreads) {
      const float4 v = row[i];
      row[i] = make_float4(v.x * factor, v.y * factor, v.z * factor, v.w * factor);
    }
  }
  fence_proxy_async_smem();   // the row was rewritten through the generic proxy, the copy engine reads it
  __syncthreads();
  if (threadIdx.x == 0 && arrived && bytes > 0) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(reinterpret_cast<uint64_t>(a.y + r * a.cols + 4 * static_cast<int64_t>(begin))), "r"(smem_u32(row)),
                 "r"(bytes)
                 : "memory");
    tma_store_commit();
    tma_store_wait_read<0>();   // shared memory must outlive the copy's reads; the writes drain after the CTA has gone
  }
  if constexpr (kCluster) scope.finish();
}

// Shared memory of a staged launch whose largest share is `share_floats`.
constexpr size_t staged_smem_bytes(int64_t share_floats) {
  return ((static_cast<size_t>(share_floats) * sizeof(float) + 127) & ~size_t{127}) + 16 +
         2 * (kStagedThreads / 32 + 1) * sizeof(float);
}

// Any length, any alignment: scalar accesses, the row is re-read.
template <RowOp kOp>
__global__ void __launch_bounds__(kBlockThreads) row_stream_kernel(const RowArgs a) {
  __shared__ float scratch[2 * kWarpsPerBlock];
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = blockIdx.x;
  const float* x_row = a.x + row * a.cols;
  float* y_row = a.y + row * a.cols;
  BlockScope<kWarpsPerBlock> scope{scratch};
  if constexpr (kOp == RowOp::kRmsNorm) {
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < a.cols; c += kBlockThreads) {
      const float v = x_row[c];
      ss += v * v;
    }
    ss = scope.template reduce<SumOp>(ss);
    const float inv_rms = rsqrtf(static_cast<float>(static_cast<double>(ss / static_cast<float>(a.cols)) + a.eps));
    for (int64_t c = threadIdx.x; c < a.cols; c += kBlockThreads) y_row[c] = x_row[c] * a.w[c] * inv_rms;
  } else {
    // Online maximum / rescaled sum: one read for both statistics.
    float mx = -FLT_MAX, sum = 0.f;
    for (int64_t c = threadIdx.x; c < a.cols; c += kBlockThreads) {
      const float v = x_row[c];
      const float m2 = fmaxf(mx, v);
      sum = sum * __expf(mx - m2) + __expf(v - m2);
      mx = m2;
    }
    const float row_max = scope.template reduce<MaxOp>(mx);
    sum = scope.template reduce<SumOp>(sum * __expf(mx - row_max));
    const float inv = __frcp_rn(sum);
    for (int64_t c = threadIdx.x; c < a.cols; c += kBlockThreads) y_row[c] = __expf(x_row[c] - row_max) * inv;
  }
}

// ------------------------------------------------------------------- dispatch

// Launch under programmatic stream serialization: the CTAs of a kernel that follows another of
// these in the stream are scheduled as that kernel's last CTAs drain, and wait (first statement of
// the kernels) until it has completed, instead of being launched only then.
template <typename Kernel>
int launch_serialized(Kernel kernel, int64_t blocks, int threads, const RowArgs& a, cudaStream_t s, size_t smem = 0,
                      unsigned cluster = 1) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  const GemmLaunchAttributes attrs = gemm_launch_attributes(cluster);   // serialization, and the cluster if there is one
  cfg.attrs = const_cast<cudaLaunchAttribute*>(attrs.list);
  cfg.numAttrs = attrs.count;
  if (cudaLaunchKernelEx(&cfg, kernel, a) != cudaSuccess) return launch_failed();
  return launch_status();
}

template <RowOp kOp, int VPT>
int launch_warp(const RowArgs& a, cudaStream_t s) {
  return launch_serialized(row_warp_kernel<kOp, VPT>, (a.rows + kWarpsPerBlock - 1) / kWarpsPerBlock, kBlockThreads, a, s);
}

template <RowOp kOp, int VPT, int kThreads>
int launch_block(const RowArgs& a, cudaStream_t s) {
  return launch_serialized(row_block_kernel<kOp, VPT, kThreads>, a.rows, kThreads, a, s);
}

template <RowOp kOp>
int launch_by_vectors_warp(int vpt, const RowArgs& a, cudaStream_t s) {
  switch (vpt) {
    case 1: return launch_warp<kOp, 1>(a, s);
    case 2: return launch_warp<kOp, 2>(a, s);
    case 3: case 4: return launch_warp<kOp, 4>(a, s);
    case 5: case 6: return launch_warp<kOp, 6>(a, s);
    default: return launch_warp<kOp, 8>(a, s);
  }
}

template <RowOp kOp, int kThreads>
int launch_by_vectors_block(int vpt, const RowArgs& a, cudaStream_t s) {
  switch (vpt) {
    case 1: return launch_block<kOp, 1, kThreads>(a, s);
    case 2: return launch_block<kOp, 2, kThreads>(a, s);
    case 3: case 4: return launch_block<kOp, 4, kThreads>(a, s);
    case 5: case 6: return launch_block<kOp, 6, kThreads>(a, s);
    default: return launch_block<kOp, 8, kThreads>(a, s);
  }
}

template <RowOp kOp>
int launch_rows(const RowArgs& a, cudaStream_t s) {
  if (a.rows == 0 || a.cols == 0) return B200_OK;
  if (a.rows > 0x7fffffffLL / 8) return B200_ERR_INVALID_PROBLEM;  // grid.x with an 8-CTA cluster per row
  const bool vector_ok = a.cols % 4 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(a.y) % 16 == 0 &&
                         (kOp == RowOp::kSoftmax || reinterpret_cast<uintptr_t>(a.w) % 16 == 0);
  const int64_t nvec = a.cols / 4;
  if (vector_ok && nvec <= 32 * kMaxVec) {
    return launch_by_vectors_warp<kOp>(static_cast<int>((nvec + 31) / 32), a, s);
  }
  // Beyond one warp per row, many small CTAs work best: with at most four
  // vectors per thread 2048 threads stay resident per SM, and the load phase of
  // one CTA overlaps the store phase of another. Rows too long for that are
  // staged in shared memory by the copy engine instead of being held in registers.
  constexpr int kLightVec = 4;
  if (vector_ok && nvec <= 256 * kLightVec) return launch_by_vectors_block<kOp, 256>(static_cast<int>((nvec + 255) / 256), a, s);
  if (vector_ok && nvec <= 512 * kLightVec) return launch_by_vectors_block<kOp, 512>(static_cast<int>((nvec + 511) / 512), a, s);
  if (vector_ok && a.cols <= 8 * kStagedMaxFloats) {
    // One CTA per row while two rows fit an SM side by side (28 672 floats); beyond that a cluster of
    // 2, 4 or 8 CTAs per row, with shares of at most 16 384 floats where eight CTAs allow it.
    constexpr size_t kMaxSmem = staged_smem_bytes(kStagedMaxFloats);
    if (a.cols <= kStagedAloneFloats) {
      if (!ensure_dynamic_smem<row_staged_kernel<kOp, false>, kMaxSmem>()) return B200_ERR_LAUNCH_FAILED;
      return launch_serialized(row_staged_kernel<kOp, false>, a.rows, kStagedThreads, a, s, staged_smem_bytes(a.cols));
    }
    int ranks = 2;
    while (ranks < 8 && (a.cols + ranks - 1) / ranks > kStagedPartFloats) ranks *= 2;
    const int64_t share_vectors = (nvec + ranks - 1) / ranks;
    if (!ensure_dynamic_smem<row_staged_kernel<kOp, true>, kMaxSmem>()) return B200_ERR_LAUNCH_FAILED;
    return launch_serialized(row_staged_kernel<kOp, true>, a.rows * ranks, kStagedThreads, a, s,
                             staged_smem_bytes(4 * share_vectors), static_cast<unsigned>(ranks));
  }
  return launch_serialized(row_stream_kernel<kOp>, a.rows, kBlockThreads, a, s);
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_rmsnorm(int impl, const float* x, const float* weight, float* y, int64_t rows, int64_t hidden, double eps,
                 b200_stream_t stream) {
  if (impl != B200_RMSNORM_NAIVE && impl != B200_RMSNORM_CACHE_X) return B200_ERR_INVALID_ARGUMENT;
  if (rows < 0 || hidden < 0) return B200_ERR_INVALID_ARGUMENT;
  if (rows > 0 && hidden > 0 && (x == nullptr || weight == nullptr || y == nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (impl == B200_RMSNORM_CACHE_X && hidden > 4096) return B200_ERR_NOT_SUPPORTED;
  const b200::RowArgs args{x, weight, y, rows, hidden, eps};
  return b200::launch_rows<b200::RowOp::kRmsNorm>(args, static_cast<cudaStream_t>(stream));
}

int b200_softmax(int impl, const float* x, float* y, int64_t rows, int64_t cols, b200_stream_t stream) {
  if (impl != B200_SOFTMAX_NAIVE) return B200_ERR_INVALID_ARGUMENT;
  if (rows < 0 || cols < 0) return B200_ERR_INVALID_ARGUMENT;
  if (rows > 0 && cols > 0 && (x == nullptr || y == nullptr)) return B200_ERR_INVALID_ARGUMENT;
  const b200::RowArgs args{x, nullptr, y, rows, cols, 0.0};
  return b200::launch_rows<b200::RowOp::kSoftmax>(args, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
