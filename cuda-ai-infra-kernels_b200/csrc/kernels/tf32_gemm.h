// Launch functions of the TF32 tensor-core GEMM kernels, one group per kernel translation unit, as
// the registry (tf32_registry.cu) calls them. All take the problem, the peer outputs of a fused
// all-gather (usually none) and the stream, and return a b200_status.
#pragma once

#include <cuda_runtime.h>

#include "b200_kernels.h"
#include "host_common.h"

namespace b200 {

// tf32_tile_kernels.cu: one CTA per 128 x tile_n tile, persistent. `stages` counts 32-wide K blocks
// of shared memory. TMA-fed (16-byte aligned operands) or fed by loader warps (any operands).
int launch_tf32_tile(int tile_n, int stages, int act, const b200_gemm_problem& q, const PeerOutputs& peers,
                     cudaStream_t stream);
int launch_tf32_generic(int tile_n, int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);
cudaError_t tf32_tile_status_read_clear(uint32_t* word);

// tf32_pair_kernel.cu: 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2).
int launch_tf32_pair(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);
// The same on 256 x 128 tiles with two MMA issuers per pair.
int launch_tf32_pair_mid(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);
cudaError_t tf32_pair_status_read_clear(uint32_t* word);

// tf32_cluster_kernels.cu: K split over a thread-block cluster. `tf32_splitk_plan` is the cost model
// the dispatcher's gate consults: the cluster size the split-K entry would use for `q` (1 = it would
// not split) and the modelled duration in microseconds.
int launch_tf32_splitk(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);
// The same on CTA pairs with two MMA issuers: 256 x 128 tiles, clusters of 2, 4 or 8 CTAs.
// `tf32_pair_splitk_plan` returns the K ranges it would use for `q` (0 = the occupancy query failed),
// the modelled duration in microseconds and the number of waves of clusters that choice needs.
int launch_tf32_pair_splitk(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);
int tf32_pair_splitk_plan(const b200_gemm_problem& q, float* estimate_us, int* waves);
int launch_tf32_swap(int act, const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);
int tf32_splitk_plan(const b200_gemm_problem& q, int sms, float* estimate_us);
cudaError_t tf32_cluster_status_read_clear(uint32_t* word);

// skinny_gemm.cu. Rows the skinny kernel accepts (one FP32 accumulator set per row and lane).
constexpr int kSkinnyMaxRows = 16;

// D = act(alpha * A @ B + beta * C + bias) for M <= kSkinnyMaxRows, N % 4 == 0,
// B 16-byte aligned with ldb % 4 == 0; FP32 FMA arithmetic, B streamed once.
// Returns B200_ERR_INVALID_PROBLEM for shapes outside that range.
// Cannot store to peer outputs: B200_ERR_NOT_SUPPORTED when `peers` is not empty.
int launch_skinny(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);

}  // namespace b200
