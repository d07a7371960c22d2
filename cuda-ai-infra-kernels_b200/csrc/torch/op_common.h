// Shared pieces of the PyTorch-facing launchers: argument checks with the
// reference's message texts (csrc/common/tensor_check.h:5-10), and the bridge
// from C-ABI status codes to c10::Error.
#pragma once

#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "b200_kernels.h"

#define B200_CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
#define B200_CHECK_CONTIGUOUS(x) TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")
#define B200_CHECK_FLOAT32(x) TORCH_CHECK((x).scalar_type() == torch::kFloat32, #x " must be float32")
#define B200_CHECK_INPUT(x) \
  B200_CHECK_CUDA(x);       \
  B200_CHECK_CONTIGUOUS(x)

namespace b200_torch {

inline b200_stream_t current_stream(const torch::Tensor& t) {
  return static_cast<b200_stream_t>(c10::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

// Any non-zero status from a launch is a hard error for the operators that
// validated their arguments beforehand.
inline void check_status(int status, const char* what) {
  TORCH_CHECK(status == B200_OK, what, " failed: ", b200_status_string(status));
}

}  // namespace b200_torch
