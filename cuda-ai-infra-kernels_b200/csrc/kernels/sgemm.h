// Internal interface between the C ABI of the FP32 ladder and its two kernel
// translation units.
#pragma once

#include "host_common.h"

namespace b200 {

// Stages 1-5 (ids B200_SGEMM_NAIVE .. B200_SGEMM_WARP_TILE).
int sgemm_ladder_launch(int impl, const float* a, const float* b, float* c, int m, int n, int k,
                        cudaStream_t stream);

// Stages 6-8 (B200_SGEMM_PREFETCH_SMEM, _PREFETCH_REG, _SPLIT_K): persistent
// TMA + mbarrier pipeline kernels.
// `peers` lists further buffers that receive every output tile at the same
// offsets as `c` (count 0 for a plain GEMM); split_k cannot serve them.
int sgemm_pipeline_launch(int impl, const float* a, const float* b, float* c, const PeerOutputs& peers, int m, int n,
                          int k, cudaStream_t stream);

}  // namespace b200
