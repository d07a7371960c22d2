// PyTorch-facing launchers of `cuda_ai_kernels.rmsnorm` / `softmax`, plus the
// two operators the reference only declares (RoPE, attention decode).
#include "op_common.h"
#include "ops.h"

namespace {

using b200_torch::check_status;
using b200_torch::current_stream;

// Argument rules of csrc/rmsnorm/rmsnorm_naive.cu:95-101 (same for cache_x).
void check_rmsnorm_inputs(const torch::Tensor& x, const torch::Tensor& weight) {
  B200_CHECK_INPUT(x);
  B200_CHECK_INPUT(weight);
  B200_CHECK_FLOAT32(x);
  B200_CHECK_FLOAT32(weight);
  TORCH_CHECK(x.dim() == 2, "x must be [rows, hidden]");
  TORCH_CHECK(weight.dim() == 1, "weight must be [hidden]");
  TORCH_CHECK(x.size(1) == weight.size(0), "hidden size mismatch");
  TORCH_CHECK(x.device() == weight.device(), "x and weight must be on the same CUDA device");
}

torch::Tensor run_rmsnorm(int impl, const torch::Tensor& x, const torch::Tensor& weight, double eps) {
  check_rmsnorm_inputs(x, weight);
  // The reference launches on the legacy default stream of whatever device is
  // current; here the inputs' device and its current stream are used.
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  const int status = b200_rmsnorm(impl, x.data_ptr<float>(), weight.data_ptr<float>(), out.data_ptr<float>(),
                                  x.size(0), x.size(1), eps, current_stream(x));
  TORCH_CHECK(status != B200_ERR_NOT_SUPPORTED, "hidden size too large for naive implementation");
  check_status(status, "rmsnorm");
  return out;
}

}  // namespace

torch::Tensor rmsnorm_naive(torch::Tensor x, torch::Tensor weight, double eps) {
  return run_rmsnorm(B200_RMSNORM_NAIVE, x, weight, eps);
}

torch::Tensor rmsnorm_cache_x(torch::Tensor x, torch::Tensor weight, double eps) {
  return run_rmsnorm(B200_RMSNORM_CACHE_X, x, weight, eps);
}

// csrc/softmax/softmax.cu:124-133.
torch::Tensor softmax_naive(torch::Tensor x) {
  B200_CHECK_INPUT(x);
  B200_CHECK_FLOAT32(x);
  TORCH_CHECK(x.dim() == 2, "softmax expects a 2D tensor [rows, cols]");
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  check_status(b200_softmax(B200_SOFTMAX_NAIVE, x.data_ptr<float>(), out.data_ptr<float>(), x.size(0), x.size(1),
                            current_stream(x)),
               "softmax");
  return out;
}

// Declared but not implemented by the reference (csrc/rope/rope.cu:4-9,
// csrc/attention/attention_decode.cu:4-9): same checks, same refusal.
torch::Tensor rope_forward(torch::Tensor x, torch::Tensor cos, torch::Tensor sin) {
  B200_CHECK_INPUT(x);
  B200_CHECK_INPUT(cos);
  B200_CHECK_INPUT(sin);
  TORCH_CHECK(false, "rope_forward is planned for v0.2");
}

torch::Tensor attention_decode_forward(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache) {
  B200_CHECK_INPUT(q);
  B200_CHECK_INPUT(k_cache);
  B200_CHECK_INPUT(v_cache);
  TORCH_CHECK(false, "attention_decode_forward is planned for v0.3");
}
