// PyTorch-facing launchers of `cuda_ai_kernels.gemm`: the FP32 SIMT ladder, the
// strict-FP32 cuBLAS baseline and the two row-major TF32 side entries. Each
// validates on the host in the order and with the messages of the reference
// launcher it replaces, allocates the output with the caching allocator, and
// hands raw pointers to the C ABI on the current stream of the inputs' device.
#include <ATen/cuda/CUDAContext.h>
#include <cublas_v2.h>

#include <cstdint>
#include <limits>
#include <string>

#include "op_common.h"
#include "ops.h"

namespace {

using b200_torch::check_status;
using b200_torch::current_stream;

// A logical [M,K] tensor whose storage is a dense [K,M] array
// (csrc/gemm/gemm_layout.h:7-9).
bool is_column_major_a(const torch::Tensor& a) {
  return a.dim() == 2 && a.stride(0) == 1 && a.stride(1) == a.size(0);
}

// Device, dtype, rank, shape and layout rules shared by every ladder entry, in
// the order of check_column_major_gemm_inputs (csrc/gemm/gemm_layout.h:11-26).
void check_ladder_layout(const torch::Tensor& a, const torch::Tensor& b) {
  B200_CHECK_CUDA(a);
  B200_CHECK_CUDA(b);
  B200_CHECK_FLOAT32(a);
  B200_CHECK_FLOAT32(b);
  TORCH_CHECK(a.device() == b.device(), "A and B must be on the same CUDA device");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm expects 2D tensors");
  TORCH_CHECK(a.size(1) == b.size(0), "shape mismatch: A[M,K] @ B[K,N]");
  TORCH_CHECK(is_column_major_a(a), "A must be column-major [M,K] with strides (1,M)");
  TORCH_CHECK(b.is_contiguous(), "B must be row-major contiguous");
  constexpr int64_t kIntMax = std::numeric_limits<int>::max();
  TORCH_CHECK(a.size(0) <= kIntMax, "M is too large");
  TORCH_CHECK(a.size(1) <= kIntMax, "K is too large");
  TORCH_CHECK(b.size(1) <= kIntMax, "N is too large");
}

// Row-major contract of the cuBLAS row-major branch and of the TF32 side
// entries (check_gemm_inputs, csrc/gemm/gemm_naive.cu:3-14).
void check_row_major_inputs(const torch::Tensor& a, const torch::Tensor& b) {
  B200_CHECK_INPUT(a);
  B200_CHECK_INPUT(b);
  B200_CHECK_FLOAT32(a);
  B200_CHECK_FLOAT32(b);
  TORCH_CHECK(a.device() == b.device(), "A and B must be on the same CUDA device");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm expects 2D tensors");
  TORCH_CHECK(a.size(1) == b.size(0), "shape mismatch: A[M,K] @ B[K,N]");
  constexpr int64_t kIntMax = std::numeric_limits<int>::max();
  TORCH_CHECK(a.size(0) <= kIntMax, "M is too large for this reference kernel");
  TORCH_CHECK(a.size(1) <= kIntMax, "K is too large for this reference kernel");
  TORCH_CHECK(b.size(1) <= kIntMax, "N is too large for this reference kernel");
}

// Size rules of one ladder entry, phrased as the reference phrases them.
// `label` is "GEMM" for stages 1-5 (csrc/gemm/gemm_regular.cuh:15-25) and the
// impl name for stages 6-8 (e.g. csrc/gemm/gemm_prefetchSmem.cu:184-189).
void check_ladder_sizes(int impl, const char* label, bool named_stage, const torch::Tensor& a,
                        const torch::Tensor& b) {
  int bm = 0, bn = 0, bk = 0, vectorized = 0;
  TORCH_CHECK(b200_sgemm_tile(impl, &bm, &bn, &bk, &vectorized) == B200_OK, "unknown GEMM ladder entry");
  const int64_t m = a.size(0), k = a.size(1), n = b.size(1);
  if (named_stage) {
    TORCH_CHECK(m % bm == 0 && n % bn == 0 && k % bk == 0, label, " requires M and N divisible by ", bm,
                " and K divisible by ", bk);
  } else {
    TORCH_CHECK(m % bm == 0 && n % bn == 0 && k % bk == 0, label, " requires M divisible by ", bm,
                ", N divisible by ", bn, " and K divisible by ", bk);
  }
  TORCH_CHECK(m / bm <= 65535, label, " grid.y exceeds 65535");
  if (vectorized) {
    TORCH_CHECK(reinterpret_cast<std::uintptr_t>(a.data_ptr<float>()) % 16 == 0 &&
                    reinterpret_cast<std::uintptr_t>(b.data_ptr<float>()) % 16 == 0,
                label, " requires 16-byte aligned A and B pointers");
  }
}

torch::Tensor launch_ladder(int impl, const torch::Tensor& a, const torch::Tensor& b) {
  const int m = static_cast<int>(a.size(0)), k = static_cast<int>(a.size(1)), n = static_cast<int>(b.size(1));
  const c10::cuda::CUDAGuard guard(a.device());
  // split_k reduces into its output; the C ABI clears it on the same stream
  // first, so plain `empty` is enough here and recycled storage is harmless.
  auto c = torch::empty({m, n}, a.options());
  const int status =
      b200_sgemm(impl, a.data_ptr<float>(), b.data_ptr<float>(), c.data_ptr<float>(), m, n, k, current_stream(a));
  check_status(status, b200_sgemm_impl_name(impl));
  return c;
}

// Stages 1-5: layout first, then positivity, tiles, grid, alignment.
torch::Tensor run_regular(int impl, const torch::Tensor& a, const torch::Tensor& b) {
  check_ladder_layout(a, b);
  TORCH_CHECK(a.size(0) > 0 && b.size(1) > 0 && a.size(1) > 0, "GEMM requires positive M, N and K");
  check_ladder_sizes(impl, "GEMM", false, a, b);
  return launch_ladder(impl, a, b);
}

// Stages 6-8: rank and positivity are reported before the layout rules.
torch::Tensor run_named(int impl, const torch::Tensor& a, const torch::Tensor& b) {
  const char* label = b200_sgemm_impl_name(impl);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm expects 2D tensors");
  TORCH_CHECK(a.size(0) > 0 && a.size(1) > 0 && b.size(1) > 0, label, " requires positive M, N and K");
  check_ladder_layout(a, b);
  check_ladder_sizes(impl, label, true, a, b);
  return launch_ladder(impl, a, b);
}

// Destination checks shared by the fused all-gather entries: `out` is where
// this rank's rows live inside its copy of the gathered matrix.
void check_gather_output(const torch::Tensor& out, const torch::Tensor& a, int64_t m, int64_t n,
                         const std::vector<int64_t>& peer_ptrs) {
  B200_CHECK_CUDA(out);
  B200_CHECK_FLOAT32(out);
  TORCH_CHECK(out.device() == a.device(), "out must be on the same CUDA device as A");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == m && out.size(1) == n, "out must have shape [", m, ", ", n, "] but got ",
              out.sizes());
  TORCH_CHECK(out.stride(1) == 1 && out.stride(0) == n, "out must be a dense row-major block of rows");
  TORCH_CHECK(peer_ptrs.size() <= B200_MAX_PEERS, "at most ", B200_MAX_PEERS, " peer destinations");
  for (const int64_t ptr : peer_ptrs) TORCH_CHECK(ptr != 0, "peer destination pointers must not be null");
}

// alpha = 1, beta = 0 TF32 product of two row-major matrices through the
// tcgen05 registry. Degenerate sizes never reach a kernel.
// `compensated`: above 128 floats of K use the three-product form whose error is that of FP32
// (b200_tf32x3_gemm); up to there one TF32 pass is well inside the entry's 3e-2 bound.
torch::Tensor run_tf32_row_major(const torch::Tensor& a, const torch::Tensor& b, const char* what,
                                 bool compensated = false) {
  check_row_major_inputs(a, b);
  const int64_t m = a.size(0), k = a.size(1), n = b.size(1);
  const c10::cuda::CUDAGuard guard(a.device());
  auto d = torch::empty({m, n}, a.options());
  if (m == 0 || n == 0) return d;
  if (k == 0) return d.zero_();
  b200_gemm_problem q{};
  q.m = static_cast<int>(m), q.n = static_cast<int>(n), q.k = static_cast<int>(k);
  q.a = a.data_ptr<float>(), q.b = b.data_ptr<float>(), q.c = nullptr, q.d = d.data_ptr<float>();
  q.lda = a.stride(0), q.ldb = b.stride(0), q.ldc = d.stride(0), q.ldd = d.stride(0);
  q.alpha = 1.f, q.beta = 0.f, q.epilogue = B200_EPILOGUE_LINEAR;
  if (compensated && k > 128) {
    const size_t bytes = b200_tf32x3_scratch_bytes(q.m, q.n, q.k);
    auto scratch = torch::empty({static_cast<int64_t>(bytes / sizeof(float))}, a.options());   // freed in stream order
    check_status(b200_tf32x3_gemm(&q, scratch.data_ptr<float>(), bytes, current_stream(a)), what);
    return d;
  }
  check_status(b200_tf32_gemm_dispatch(B200_TF32_KERNEL_AUTO, &q, nullptr, current_stream(a)), what);
  return d;
}

}  // namespace

torch::Tensor gemm_naive(torch::Tensor a, torch::Tensor b) { return run_regular(B200_SGEMM_NAIVE, a, b); }
torch::Tensor gemm_block_tile(torch::Tensor a, torch::Tensor b) { return run_regular(B200_SGEMM_BLOCK_TILE, a, b); }
torch::Tensor gemm_block_tile_float4_16x16(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_BLOCK_TILE_F4_16x16, a, b);
}
torch::Tensor gemm_block_tile_float4_16x32(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_BLOCK_TILE_F4_16x32, a, b);
}
torch::Tensor gemm_block_tile_float4_32x32(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_BLOCK_TILE_F4_32x32, a, b);
}
torch::Tensor gemm_thread_tile_4x4(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_THREAD_TILE_4x4, a, b);
}
torch::Tensor gemm_thread_tile_4x8(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_THREAD_TILE_4x8, a, b);
}
torch::Tensor gemm_thread_tile_8x8(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_THREAD_TILE_8x8, a, b);
}
torch::Tensor gemm_thread_tile_8x8_warp4x8(torch::Tensor a, torch::Tensor b) {
  return run_regular(B200_SGEMM_THREAD_TILE_8x8_WARP4x8, a, b);
}
// "thread_tile" is the 4x4 variant under its older name (csrc/gemm/gemm_thread_tile.cu:102-104).
torch::Tensor gemm_thread_tile(torch::Tensor a, torch::Tensor b) { return gemm_thread_tile_4x4(a, b); }
torch::Tensor gemm_warp_tile(torch::Tensor a, torch::Tensor b) { return run_regular(B200_SGEMM_WARP_TILE, a, b); }
torch::Tensor gemm_prefetch_smem(torch::Tensor a, torch::Tensor b) { return run_named(B200_SGEMM_PREFETCH_SMEM, a, b); }
torch::Tensor gemm_prefetch_reg(torch::Tensor a, torch::Tensor b) { return run_named(B200_SGEMM_PREFETCH_REG, a, b); }
torch::Tensor gemm_split_k(torch::Tensor a, torch::Tensor b) { return run_named(B200_SGEMM_SPLIT_K, a, b); }

torch::Tensor gemm_gather(torch::Tensor a, torch::Tensor b, torch::Tensor out, std::vector<int64_t> peer_ptrs,
                          const std::string& impl) {
  const int id = b200_sgemm_impl_from_name(impl.c_str());
  TORCH_CHECK(id == B200_SGEMM_PREFETCH_SMEM || id == B200_SGEMM_PREFETCH_REG,
              "gemm_gather supports impl='prefetch_smem' or 'prefetch_reg', got '", impl, "'");
  const char* label = b200_sgemm_impl_name(id);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm expects 2D tensors");
  TORCH_CHECK(a.size(0) > 0 && a.size(1) > 0 && b.size(1) > 0, label, " requires positive M, N and K");
  check_ladder_layout(a, b);
  check_ladder_sizes(id, label, true, a, b);
  const int m = static_cast<int>(a.size(0)), k = static_cast<int>(a.size(1)), n = static_cast<int>(b.size(1));
  check_gather_output(out, a, m, n, peer_ptrs);
  const c10::cuda::CUDAGuard guard(a.device());
  float* peers[B200_MAX_PEERS] = {};
  for (size_t i = 0; i < peer_ptrs.size(); ++i) peers[i] = reinterpret_cast<float*>(static_cast<std::uintptr_t>(peer_ptrs[i]));
  const int status = b200_sgemm_gather(id, a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(), peers,
                                       static_cast<int>(peer_ptrs.size()), m, n, k, current_stream(a));
  check_status(status, label);
  return out;
}

// Library baseline: strict FP32 cuBLAS irrespective of the process-wide TF32
// switches, on PyTorch's handle for the current device and stream. Accepts the
// ladder's column-major A as well as a contiguous row-major A, and empty
// dimensions (csrc/gemm/gemm_cublas.cu:8-61).
torch::Tensor gemm_cublas(torch::Tensor a, torch::Tensor b) {
  const bool column_major_a = is_column_major_a(a);
  if (column_major_a) {
    check_ladder_layout(a, b);
  } else {
    check_row_major_inputs(a, b);
  }
  const c10::cuda::CUDAGuard guard(a.device());
  const int m = static_cast<int>(a.size(0)), k = static_cast<int>(a.size(1)), n = static_cast<int>(b.size(1));
  auto c = torch::empty({m, n}, a.options());
  if (m == 0 || n == 0) return c;
  if (k == 0) return c.zero_();
  // Row-major C[M,N] is column-major C^T[N,M] = B^T * A^T. B's storage already
  // is column-major B^T; a row-major A is column-major A^T, a column-major A
  // must be transposed by cuBLAS (lda = M).
  const float one = 1.f, zero = 0.f;
  const cublasStatus_t rc = cublasGemmEx(
      at::cuda::getCurrentCUDABlasHandle(), CUBLAS_OP_N, column_major_a ? CUBLAS_OP_T : CUBLAS_OP_N, n, m, k, &one,
      b.data_ptr<float>(), CUDA_R_32F, n, a.data_ptr<float>(), CUDA_R_32F, column_major_a ? m : k, &zero,
      c.data_ptr<float>(), CUDA_R_32F, n, CUBLAS_COMPUTE_32F_PEDANTIC, CUBLAS_GEMM_DEFAULT);
  TORCH_CHECK(rc == CUBLAS_STATUS_SUCCESS, "cublasGemmEx (FP32) failed");
  return c;
}

// Row-major TF32 side entries (csrc/gemm/gemm_tensor_core.cu:111-137,
// csrc/gemm/gemm_cutlass.cu:76-126): any shape, tensor cores.
torch::Tensor gemm_tensor_core(torch::Tensor a, torch::Tensor b) {
  return run_tf32_row_major(a, b, "gemm_tensor_core", /*compensated=*/true);
}
torch::Tensor gemm_cutlass(torch::Tensor a, torch::Tensor b) { return run_tf32_row_major(a, b, "gemm_cutlass"); }
