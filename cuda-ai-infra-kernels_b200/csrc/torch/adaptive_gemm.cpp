// PyTorch-facing launcher of `cuda_ai_kernels.adaptive_gemm`:
//   D = act(alpha * A @ B + beta * C [+ bias]),  act in {identity, ReLU, GELU},
// all operands row-major FP32, products on the tensor cores in TF32.
// Validation order, accepted strings and error texts follow
// csrc/adaptive_gemm/adaptive_gemm.cu:14-174; the kernel choice is delegated to
// the registry behind b200_tf32_gemm_dispatch (first compatible entry wins).
#include <ATen/cuda/CUDAContext.h>
#include <cublasLt.h>
#include <cublas_v2.h>

#include <cstdint>
#include <limits>
#include <map>
#include <tuple>
#include <vector>

#include "op_common.h"
#include "ops.h"

namespace {

using b200_torch::current_stream;

thread_local std::string g_last_kernel;

// Epilogue spellings the reference parses (adaptive_gemm.cu:39-59). The
// reference runs only "linear" and "relu" and refuses the rest at run time
// (adaptive_gemm.cu:124-133); here all six run: the bias term and the GELU are
// applied in the same TMEM -> register pass as the scaling.
struct ParsedEpilogue {
  int activation;   // b200_epilogue
  bool wants_bias;
};

ParsedEpilogue parse_epilogue(const std::string& value) {
  if (value == "linear") return {B200_EPILOGUE_LINEAR, false};
  if (value == "relu") return {B200_EPILOGUE_RELU, false};
  if (value == "gelu") return {B200_EPILOGUE_GELU, false};
  if (value == "bias") return {B200_EPILOGUE_LINEAR, true};
  if (value == "bias_relu") return {B200_EPILOGUE_RELU, true};
  if (value == "bias_gelu") return {B200_EPILOGUE_GELU, true};
  TORCH_CHECK(false, "unsupported epilogue: ", value);
}

// kernel="cublaslt": library baseline with the epilogue fused by the library (no registry id).
constexpr int kKernelCublasLt = -2;

int parse_kernel(const std::string& value) {
  if (value == "cublaslt") return kKernelCublasLt;
  const int id = b200_tf32_kernel_from_name(value.c_str());
  TORCH_CHECK(id >= 0, "unsupported adaptive_gemm kernel: ", value,
              "; expected one of: auto, cublas, fast, fallback, fast_mwarp, "
              "fallback_mwarp, fast_stage3, fast_stage2, fast_relu, fallback_relu");
  return id;
}

void check_ab(const torch::Tensor& a, const torch::Tensor& b) {
  B200_CHECK_INPUT(a);
  B200_CHECK_INPUT(b);
  B200_CHECK_FLOAT32(a);
  B200_CHECK_FLOAT32(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "A and B must be 2D tensors");
  TORCH_CHECK(a.size(1) == b.size(0), "Matrix multiplication shape mismatch: A has ", a.size(1),
              " columns, but B has ", b.size(0), " rows");
  TORCH_CHECK(a.device() == b.device(), "A and B must be on the same CUDA device");
  TORCH_CHECK(a.size(0) > 0 && a.size(1) > 0 && b.size(1) > 0, "M, N, and K must be positive");
  constexpr int64_t kIntMax = std::numeric_limits<int>::max();
  TORCH_CHECK(a.size(0) <= kIntMax && a.size(1) <= kIntMax && b.size(1) <= kIntMax,
              "M, N, and K must fit in the int32 problem size");
}

void check_source(const torch::Tensor& c, const torch::Tensor& a, int64_t m, int64_t n) {
  B200_CHECK_INPUT(c);
  B200_CHECK_FLOAT32(c);
  TORCH_CHECK(c.device() == a.device(), "C must be on the same CUDA device as A");
  TORCH_CHECK(c.dim() == 2, "C must be a 2D tensor");
  TORCH_CHECK(c.size(0) == m && c.size(1) == n, "C must have shape [", m, ", ", n, "] but got ", c.sizes());
}

// Library baseline: cuBLAS with TF32 tensor-op math. The classic interface
// updates its C operand in place, so a separate source is copied into D first
// (csrc/adaptive_gemm/cublas_reference.cu:20-61).
void launch_cublas_tf32(const b200_gemm_problem& q, cudaStream_t stream) {
  if (q.beta != 0.f && q.c != q.d) {
    const size_t bytes = static_cast<size_t>(q.m) * static_cast<size_t>(q.n) * sizeof(float);
    const cudaError_t rc = cudaMemcpyAsync(q.d, q.c, bytes, cudaMemcpyDeviceToDevice, stream);
    TORCH_CHECK(rc == cudaSuccess, "CUDA error: ", cudaGetErrorString(rc));
  }
  // Row-major D[M,N] is column-major D^T[N,M] = alpha * B^T * A^T + beta * D^T.
  const cublasStatus_t rc =
      cublasGemmEx(at::cuda::getCurrentCUDABlasHandle(), CUBLAS_OP_N, CUBLAS_OP_N, q.n, q.m, q.k, &q.alpha, q.b,
                   CUDA_R_32F, static_cast<int>(q.ldb), q.a, CUDA_R_32F, static_cast<int>(q.lda), &q.beta, q.d,
                   CUDA_R_32F, static_cast<int>(q.ldd), CUBLAS_COMPUTE_32F_FAST_TF32, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
  TORCH_CHECK(rc == CUBLAS_STATUS_SUCCESS, "cublasGemmEx failed with cuBLAS status ", static_cast<int>(rc));
}

// Library baseline with a FUSED epilogue: one cublasLtMatmul computes act(alpha * A @ B + beta * C
// [+ bias]) with C as the library's own C operand and ReLU / bias as its epilogue, in TF32. This is
// the fair competitor of the fused tcgen05 kernels (the reference ships only the unfused cuBLAS
// baseline above and applies ReLU in a second pass, benchmarks/bench_adaptive_gemm.py:47-51).
// Row-major D[M,N] is handed over as column-major D^T[N,M] = B^T[N,K] * A^T[K,M].
struct LtPlan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr, d = nullptr;
  cublasLtMatmulAlgo_t algo;
};

void lt_check(cublasStatus_t rc, const char* what) {
  TORCH_CHECK(rc == CUBLAS_STATUS_SUCCESS, "cuBLASLt ", what, " failed with status ", static_cast<int>(rc));
}

void launch_cublaslt_tf32(const b200_gemm_problem& q, int device, cudaStream_t stream) {
  using Key = std::tuple<int, int, int, int, int64_t, int64_t, int64_t, int64_t, int, bool>;
  thread_local std::map<Key, LtPlan> plans;   // descriptors and the heuristic's choice, per shape
  cublasLtHandle_t handle = at::cuda::getCurrentCUDABlasLtHandle();
  const size_t workspace_bytes = at::cuda::getCUDABlasLtWorkspaceSize();
  void* workspace = at::cuda::getCUDABlasLtWorkspace();
  const Key key{device, q.m, q.n, q.k, q.lda, q.ldb, q.ldc, q.ldd, q.epilogue, q.bias != nullptr};
  auto it = plans.find(key);
  if (it == plans.end()) {
    LtPlan plan;
    lt_check(cublasLtMatmulDescCreate(&plan.op, CUBLAS_COMPUTE_32F_FAST_TF32, CUDA_R_32F), "descriptor creation");
    cublasLtEpilogue_t epilogue = CUBLASLT_EPILOGUE_DEFAULT;
    if (q.epilogue == B200_EPILOGUE_RELU) epilogue = q.bias ? CUBLASLT_EPILOGUE_RELU_BIAS : CUBLASLT_EPILOGUE_RELU;
    else if (q.bias) epilogue = CUBLASLT_EPILOGUE_BIAS;
    lt_check(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epilogue, sizeof(epilogue)), "epilogue");
    lt_check(cublasLtMatrixLayoutCreate(&plan.a, CUDA_R_32F, q.n, q.k, q.ldb), "layout");
    lt_check(cublasLtMatrixLayoutCreate(&plan.b, CUDA_R_32F, q.k, q.m, q.lda), "layout");
    lt_check(cublasLtMatrixLayoutCreate(&plan.c, CUDA_R_32F, q.n, q.m, q.ldc), "layout");
    lt_check(cublasLtMatrixLayoutCreate(&plan.d, CUDA_R_32F, q.n, q.m, q.ldd), "layout");
    cublasLtMatmulPreference_t pref = nullptr;
    lt_check(cublasLtMatmulPreferenceCreate(&pref), "preference");
    lt_check(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes,
                                                  sizeof(workspace_bytes)), "preference");
    cublasLtMatmulHeuristicResult_t result;
    int found = 0;
    const cublasStatus_t rc = cublasLtMatmulAlgoGetHeuristic(handle, plan.op, plan.a, plan.b, plan.c, plan.d, pref, 1,
                                                             &result, &found);
    cublasLtMatmulPreferenceDestroy(pref);
    TORCH_CHECK(rc == CUBLAS_STATUS_SUCCESS && found > 0, "cuBLASLt has no algorithm for this problem");
    plan.algo = result.algo;
    it = plans.emplace(key, plan).first;
  }
  const LtPlan& plan = it->second;
  if (q.bias != nullptr) {
    lt_check(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &q.bias, sizeof(q.bias)), "bias");
  }
  // With beta == 0 the library must still be given a valid C; D stands in and is never read.
  const float* c_operand = q.beta != 0.f ? q.c : q.d;
  lt_check(cublasLtMatmul(handle, plan.op, &q.alpha, q.b, plan.a, q.a, plan.b, &q.beta, c_operand, plan.c, q.d, plan.d,
                          &plan.algo, workspace, workspace_bytes, stream), "matmul");
}

const char* registry_name(int id) {
  b200_tf32_kernel_meta meta;
  for (int i = 0; i < b200_tf32_registry_size(); ++i) {
    if (b200_tf32_registry_entry(i, &meta) == B200_OK && meta.id == id) return meta.name;
  }
  return "unknown";
}

}  // namespace

std::string adaptive_gemm_last_kernel() { return g_last_kernel; }

namespace {

// Shared body of adaptive_gemm and adaptive_gemm_gather. Without `out` the
// result is a fresh tensor; with it the result is written there and fanned out
// to `peer_ptrs` by the kernel's epilogue.
torch::Tensor run_adaptive(const torch::Tensor& a, const torch::Tensor& b, const c10::optional<at::Tensor>& c,
                           const c10::optional<at::Tensor>& bias, double alpha, double beta,
                           const std::string& epilogue, const std::string& kernel, const c10::optional<at::Tensor>& out,
                           const std::vector<int64_t>& peer_ptrs) {
  check_ab(a, b);
  const ParsedEpilogue parsed = parse_epilogue(epilogue);
  const int requested = parse_kernel(kernel);
  const bool has_bias = bias.has_value() && bias->defined();
  TORCH_CHECK(requested != B200_TF32_KERNEL_CUBLAS || (parsed.activation == B200_EPILOGUE_LINEAR && !parsed.wants_bias),
              "adaptive_gemm kernel='cublas' supports only the linear epilogue; "
              "apply torch.relu to its output for an unfused ReLU baseline");
  TORCH_CHECK(requested != kKernelCublasLt || parsed.activation != B200_EPILOGUE_GELU,
              "adaptive_gemm kernel='cublaslt' has linear, ReLU and bias epilogues (the library's GELU is the tanh form)");
  TORCH_CHECK(has_bias == parsed.wants_bias,
              parsed.wants_bias ? "bias is required by the '" : "a bias tensor needs a bias epilogue, not '", epilogue,
              "' epilogue");

  const int64_t m = a.size(0), n = b.size(1);
  const bool has_c = c.has_value() && c->defined();
  TORCH_CHECK(has_c || beta == 0.0, "C is required when beta is non-zero");
  if (has_c) check_source(*c, a, m, n);
  if (has_bias) {
    B200_CHECK_INPUT((*bias));
    B200_CHECK_FLOAT32((*bias));
    TORCH_CHECK(bias->device() == a.device(), "bias must be on the same CUDA device as A");
    TORCH_CHECK(bias->dim() == 1 && bias->size(0) == n, "bias must have shape [", n, "] but got ", bias->sizes());
  }

  const c10::cuda::CUDAGuard guard(a.device());
  if (out.has_value()) {
    B200_CHECK_CUDA((*out));
    B200_CHECK_FLOAT32((*out));
    TORCH_CHECK(out->device() == a.device(), "out must be on the same CUDA device as A");
    TORCH_CHECK(out->dim() == 2 && out->size(0) == m && out->size(1) == n, "out must have shape [", m, ", ", n,
                "] but got ", out->sizes());
    TORCH_CHECK(out->stride(1) == 1 && out->stride(0) >= n, "out must be row-major");
    TORCH_CHECK(requested != B200_TF32_KERNEL_CUBLAS && requested != kKernelCublasLt,
                "adaptive_gemm_gather has no cuBLAS arm");
    TORCH_CHECK(peer_ptrs.size() <= B200_MAX_PEERS, "at most ", B200_MAX_PEERS, " peer destinations");
    for (const int64_t ptr : peer_ptrs) TORCH_CHECK(ptr != 0, "peer destination pointers must not be null");
  }
  auto d = out.has_value() ? *out : torch::empty({m, n}, a.options());

  b200_gemm_problem q{};
  q.m = static_cast<int>(m), q.n = static_cast<int>(n), q.k = static_cast<int>(a.size(1));
  q.a = a.data_ptr<float>(), q.b = b.data_ptr<float>(), q.d = d.data_ptr<float>();
  // Without a source the destination stands in for it; beta is zero then, so
  // it is never read (adaptive_gemm.cu:152-154).
  q.c = has_c ? c->data_ptr<float>() : d.data_ptr<float>();
  q.lda = a.stride(0), q.ldb = b.stride(0), q.ldd = d.stride(0);
  q.ldc = has_c ? c->stride(0) : d.stride(0);
  q.alpha = static_cast<float>(alpha), q.beta = static_cast<float>(beta);
  q.epilogue = parsed.activation;
  q.bias = has_bias ? bias->data_ptr<float>() : nullptr;
  constexpr int64_t kIntMax = std::numeric_limits<int>::max();
  TORCH_CHECK(q.lda <= kIntMax && q.ldb <= kIntMax && q.ldc <= kIntMax && q.ldd <= kIntMax,
              "leading dimension exceeds the int32 range");

  if (requested == B200_TF32_KERNEL_CUBLAS) {
    launch_cublas_tf32(q, static_cast<cudaStream_t>(current_stream(a)));
    g_last_kernel = "cublas";
    return d;
  }

  if (requested == kKernelCublasLt) {
    q.c = has_c ? c->data_ptr<float>() : d.data_ptr<float>();
    launch_cublaslt_tf32(q, a.get_device(), static_cast<cudaStream_t>(current_stream(a)));
    g_last_kernel = "cublaslt";
    return d;
  }

  float* peers[B200_MAX_PEERS] = {};
  for (size_t i = 0; i < peer_ptrs.size(); ++i) peers[i] = reinterpret_cast<float*>(static_cast<std::uintptr_t>(peer_ptrs[i]));
  int chosen = -1;
  const int status = b200_tf32_gemm_dispatch_gather(requested, &q, peers, static_cast<int>(peer_ptrs.size()), &chosen,
                                                    current_stream(a));
  TORCH_CHECK(status == B200_OK, "adaptive GEMM dispatch failed: ", b200_status_string(status));
  g_last_kernel = registry_name(chosen);
  return d;
}

}  // namespace

torch::Tensor adaptive_gemm(const torch::Tensor& a, const torch::Tensor& b, const c10::optional<at::Tensor>& c,
                            const c10::optional<at::Tensor>& bias, double alpha, double beta,
                            const std::string& epilogue, const std::string& kernel) {
  return run_adaptive(a, b, c, bias, alpha, beta, epilogue, kernel, c10::nullopt, {});
}

torch::Tensor adaptive_gemm_gather(const torch::Tensor& a, const torch::Tensor& b, const c10::optional<at::Tensor>& c,
                                   const c10::optional<at::Tensor>& bias, double alpha, double beta,
                                   const std::string& epilogue, const std::string& kernel, torch::Tensor out,
                                   std::vector<int64_t> peer_ptrs) {
  return run_adaptive(a, b, c, bias, alpha, beta, epilogue, kernel, out, peer_ptrs);
}
