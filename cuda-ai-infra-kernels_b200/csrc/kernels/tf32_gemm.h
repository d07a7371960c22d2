// Launchers of the adaptive (row-major, alpha/beta/epilogue) GEMM registry that
// live outside the translation unit holding the registry table.
#pragma once

#include <cuda_runtime.h>

#include "b200_kernels.h"
#include "host_common.h"

namespace b200 {

// Rows the skinny kernel accepts (one FP32 accumulator set per row and lane).
constexpr int kSkinnyMaxRows = 16;

// D = act(alpha * A @ B + beta * C + bias) for M <= kSkinnyMaxRows, N % 4 == 0,
// B 16-byte aligned with ldb % 4 == 0; FP32 FMA arithmetic, B streamed once.
// Returns B200_ERR_INVALID_PROBLEM for shapes outside that range.
// Cannot store to peer outputs: B200_ERR_NOT_SUPPORTED when `peers` is not empty.
int launch_skinny(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream);

}  // namespace b200
