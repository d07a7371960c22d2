// Error-compensated TF32 GEMM ("3xTF32"): FP32-class accuracy from TF32 tensor-core products.
//
// tcgen05.mma kind::tf32 reads FP32 operands and ignores their 13 low mantissa bits. Writing an
// operand as x = hi + lo with hi = x with those bits cleared (what the MMA unit sees anyway) and
// lo = x - hi (exact in FP32), the product is
//   A * B = A_hi * B_hi + A_lo * B_hi + A_hi * B_lo + A_lo * B_lo,
// and the first three terms are three ordinary TF32 products: MMA(A, B), MMA(A_lo, B), MMA(A, B_lo).
// What is left (A_lo * B_lo and the truncation of the lo operands themselves) is about 2^-20 of
// the result, against 2^-10 per operand for a single TF32 pass.
//
// The reference's row-major tensor-core entry (csrc/gemm/gemm_tensor_core.cu:18-137) is plain TF32
// with round-to-nearest operand conversion; its own test bounds the element-wise error at 3e-2
// for K = 1024 (tests/test_gemm.py:23-35), which single-pass TF32 noise (sigma about
// 4e-4 * sqrt(K) for N(0,1) operands) reaches in the tail of a million outputs. This path keeps
// that bound with a wide margin at three times the tensor work.
//
// Scratch: the two lo matrices, dense, rows padded to four floats (so that the TMA-fed kernels
// can take them): the caller passes b200_tf32x3_scratch_bytes(m, n, k) bytes of device memory.
#include <atomic>
#include <mutex>

#include "host_common.h"
#include "tf32_gemm.h"

namespace b200 {
namespace {

// Scratch for callers that cannot hand any over (b200_tf32x3_gemm_static): a fixed array that is part
// of the library image, 8 MiB on every GPU that loads the library, for as long as the library stays
// loaded. In host code this name is only a handle for the symbol, not a device address: the address
// a kernel can use is asked for once per device with cudaGetSymbolAddress (static_scratch below).
constexpr size_t kStaticScratchBytes = size_t{8} << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

__host__ __device__ inline int64_t padded4(int64_t cols) { return (cols + 3) / 4 * 4; }

// lo[r][c] = x[r][c] - tf32_truncate(x[r][c]) for both operands in one launch; padding columns are
// written as zeros (they are never multiplied with anything, K and N bound the products, but a
// TMA box may read them). Non-finite inputs get lo = 0 (inf - inf would be NaN); an infinite
// operand still turns its whole row or column of D into NaN, because the correction products
// multiply it with lo terms that are zero. A single pass would give +-inf there.
__global__ void split_lo_kernel(const float* __restrict__ a, int64_t lda, int m, int k, float* __restrict__ a_lo,
                                const float* __restrict__ b, int64_t ldb, int n, float* __restrict__ b_lo) {
  const int64_t ka = padded4(k), nb = padded4(n);
  const int64_t total_a = static_cast<int64_t>(m) * ka, total = total_a + static_cast<int64_t>(k) * nb;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const bool in_a = i < total_a;
    const int64_t j = in_a ? i : i - total_a;
    const int64_t pitch = in_a ? ka : nb;
    const int64_t row = j / pitch, col = j - row * pitch;
    const int cols = in_a ? k : n;
    float lo = 0.f;
    if (col < cols) {
      const float x = in_a ? a[row * lda + col] : b[row * ldb + col];
      const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
      lo = isfinite(x) ? x - hi : 0.f;
    }
    (in_a ? a_lo : b_lo)[j] = lo;
  }
}

// Device address of g_static_scratch on the CURRENT device, looked up on the first call for that
// device (with that device current) and remembered. nullptr when the look-up failed.
float* static_scratch() {
  constexpr int kMaxDevices = 64;
  static std::mutex mutex;
  static float* address[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  const std::lock_guard<std::mutex> lock(mutex);
  if (address[device] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    address[device] = static_cast<float*>(ptr);
  }
  return address[device];
}

}  // namespace
}  // namespace b200

extern "C" {

size_t b200_tf32x3_scratch_bytes(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  return (static_cast<size_t>(m) * b200::padded4(k) + static_cast<size_t>(k) * b200::padded4(n)) * sizeof(float);
}

int b200_tf32x3_gemm(const b200_gemm_problem* q, void* scratch, size_t scratch_bytes, b200_stream_t stream) {
  if (q == nullptr || q->a == nullptr || q->b == nullptr || q->d == nullptr) return B200_ERR_INVALID_ARGUMENT;
  if (q->m <= 0 || q->n <= 0 || q->k <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (q->beta != 0.f && q->c == nullptr) return B200_ERR_INVALID_ARGUMENT;
  const size_t need = b200_tf32x3_scratch_bytes(q->m, q->n, q->k);
  if (scratch == nullptr || scratch_bytes < need || reinterpret_cast<uintptr_t>(scratch) % 16 != 0) {
    return B200_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t ka = b200::padded4(q->k), nb = b200::padded4(q->n);
  float* a_lo = static_cast<float*>(scratch);
  float* b_lo = a_lo + static_cast<size_t>(q->m) * ka;   // m * ka is a multiple of four floats: 16-byte aligned
  const int64_t total = static_cast<int64_t>(q->m) * ka + static_cast<int64_t>(q->k) * nb;
  const int sms = b200::sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t want = (total + 255) / 256;
  const int grid = static_cast<int>(want < 8LL * sms ? want : 8LL * sms);
  b200::split_lo_kernel<<<grid, 256, 0, s>>>(q->a, q->lda, q->m, q->k, a_lo, q->b, q->ldb, q->n, b_lo);
  int status = b200::launch_status();
  if (status != B200_OK) return status;

  // Pass 1: D = alpha * A_hi B_hi + beta * C. Passes 2 and 3 accumulate into D (source = D, beta = 1;
  // a kernel reads a source element and writes the same element from the same thread). Bias and
  // activation belong to the last pass only.
  b200_gemm_problem pass = *q;
  pass.epilogue = B200_EPILOGUE_LINEAR;
  pass.bias = nullptr;
  status = b200_tf32_gemm_dispatch(B200_TF32_KERNEL_AUTO, &pass, nullptr, stream);
  if (status != B200_OK) return status;
  pass.c = q->d, pass.ldc = q->ldd, pass.beta = 1.f;
  pass.a = a_lo, pass.lda = ka;
  status = b200_tf32_gemm_dispatch(B200_TF32_KERNEL_AUTO, &pass, nullptr, stream);
  if (status != B200_OK) return status;
  pass.a = q->a, pass.lda = q->lda;
  pass.b = b_lo, pass.ldb = nb;
  pass.epilogue = q->epilogue;
  pass.bias = q->bias;
  return b200_tf32_gemm_dispatch(B200_TF32_KERNEL_AUTO, &pass, nullptr, stream);
}

size_t b200_tf32x3_static_scratch_bytes(void) { return b200::kStaticScratchBytes; }

int b200_tf32x3_gemm_static(const b200_gemm_problem* q, b200_stream_t stream) {
  if (q == nullptr || q->m <= 0 || q->n <= 0 || q->k <= 0) return B200_ERR_INVALID_ARGUMENT;
  // Too large for the fixed array: refused before anything is launched or looked up.
  if (b200_tf32x3_scratch_bytes(q->m, q->n, q->k) > b200::kStaticScratchBytes) return B200_ERR_NOT_SUPPORTED;
  float* scratch = b200::static_scratch();   // the first call on a device resolves the symbol's address
  if (scratch == nullptr) return B200_ERR_INTERNAL;
  // The splitting pass rewrites every element of the scratch that the products read (padding columns
  // included), so whatever an earlier call left in the array does not matter and nothing is cleared.
  return b200_tf32x3_gemm(q, scratch, b200::kStaticScratchBytes, stream);
}

}  // extern "C"
