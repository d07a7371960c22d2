// C ABI of the FP32 SIMT GEMM ladder: name and tile tables, host validation,
// launch routing.
#include <cstring>

#include "sgemm.h"

namespace {

struct LadderEntry {
  const char* name;
  int bm, bn, bk;
  int vectorized;  // needs 16-byte aligned A and B
};

// Order and tile multiples follow the ladder table of the reference
// (python/cuda_ai_kernels/gemm_stages.py:4-19).
constexpr LadderEntry kLadder[B200_SGEMM_IMPL_COUNT] = {
    {"naive", 16, 16, 1, 0},
    {"block_tile", 16, 16, 8, 0},
    {"block_tile_float4_16x16", 16, 16, 8, 1},
    {"block_tile_float4_16x32", 16, 32, 8, 1},
    {"block_tile_float4_32x32", 32, 32, 8, 1},
    {"thread_tile_4x4", 128, 128, 8, 1},
    {"thread_tile_4x8", 128, 128, 8, 1},
    {"thread_tile_8x8", 128, 128, 8, 1},
    {"thread_tile_8x8_warp4x8", 128, 128, 8, 1},
    {"warp_tile", 128, 128, 8, 1},
    {"prefetch_smem", 128, 128, 8, 1},
    {"prefetch_reg", 128, 128, 8, 1},
    {"split_k", 128, 128, 16, 1},
};

bool valid_impl(int impl) { return impl >= 0 && impl < B200_SGEMM_IMPL_COUNT; }

// Every vectorised entry stores C with 128-bit accesses (split_k reduces into it with
// red.global.add.v4.f32). The reference never meets a misaligned C because its launchers allocate
// the output themselves; a caller of this ABI can pass one, so it is refused before any launch.
bool output_misaligned(int impl, const float* c) {
  return kLadder[impl].vectorized && reinterpret_cast<uintptr_t>(c) % 16 != 0;
}

}  // namespace

extern "C" {

const char* b200_sgemm_impl_name(int impl) { return valid_impl(impl) ? kLadder[impl].name : nullptr; }

int b200_sgemm_impl_from_name(const char* name) {
  if (name == nullptr) return -1;
  for (int i = 0; i < B200_SGEMM_IMPL_COUNT; ++i) {
    if (std::strcmp(name, kLadder[i].name) == 0) return i;
  }
  // The reference keeps "thread_tile" as an alias of the 4x4 variant
  // (csrc/gemm/gemm_thread_tile.cu:102-104).
  if (std::strcmp(name, "thread_tile") == 0) return B200_SGEMM_THREAD_TILE_4x4;
  return -1;
}

int b200_sgemm_tile(int impl, int* bm, int* bn, int* bk, int* needs_16b_alignment) {
  if (!valid_impl(impl)) return B200_ERR_INVALID_ARGUMENT;
  if (bm) *bm = kLadder[impl].bm;
  if (bn) *bn = kLadder[impl].bn;
  if (bk) *bk = kLadder[impl].bk;
  if (needs_16b_alignment) *needs_16b_alignment = kLadder[impl].vectorized;
  return B200_OK;
}

int b200_sgemm_check(int impl, const void* a, const void* b, int64_t m, int64_t n, int64_t k) {
  if (!valid_impl(impl)) return B200_ERR_INVALID_ARGUMENT;
  const LadderEntry& e = kLadder[impl];
  if (m <= 0 || n <= 0 || k <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return B200_ERR_INVALID_ARGUMENT;
  if (m % e.bm != 0 || n % e.bn != 0 || k % e.bk != 0) return B200_ERR_INVALID_PROBLEM;
  if (m / e.bm > 65535) return B200_ERR_INVALID_PROBLEM;
  if (e.vectorized &&
      (reinterpret_cast<uintptr_t>(a) % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  return B200_OK;
}

int b200_sgemm(int impl, const float* a_colmajor, const float* b, float* c, int m, int n, int k,
               b200_stream_t stream) {
  if (a_colmajor == nullptr || b == nullptr || c == nullptr) return B200_ERR_INVALID_ARGUMENT;
  const int check = b200_sgemm_check(impl, a_colmajor, b, m, n, k);
  if (check != B200_OK) return check;
  if (output_misaligned(impl, c)) return B200_ERR_MISALIGNED_OPERAND;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (impl <= B200_SGEMM_WARP_TILE) return b200::sgemm_ladder_launch(impl, a_colmajor, b, c, m, n, k, s);
  b200::PeerOutputs none;
  b200::make_peer_outputs(&none, nullptr, 0);
  return b200::sgemm_pipeline_launch(impl, a_colmajor, b, c, none, m, n, k, s);
}

int b200_sgemm_gather(int impl, const float* a_colmajor, const float* b, float* c, float* const* peer_c, int n_peers,
                      int m, int n, int k, b200_stream_t stream) {
  if (a_colmajor == nullptr || b == nullptr || c == nullptr) return B200_ERR_INVALID_ARGUMENT;
  b200::PeerOutputs peers;
  if (!b200::make_peer_outputs(&peers, peer_c, n_peers)) return B200_ERR_INVALID_ARGUMENT;
  const int check = b200_sgemm_check(impl, a_colmajor, b, m, n, k);
  if (check != B200_OK) return check;
  if (output_misaligned(impl, c)) return B200_ERR_MISALIGNED_OPERAND;
  // Only the persistent pipeline kernels that store finished tiles once can fan them out.
  if (impl != B200_SGEMM_PREFETCH_SMEM && impl != B200_SGEMM_PREFETCH_REG) return B200_ERR_NOT_SUPPORTED;
  for (int i = 0; i < n_peers; ++i) {
    if (reinterpret_cast<uintptr_t>(peer_c[i]) % 16 != 0) return B200_ERR_MISALIGNED_OPERAND;
  }
  return b200::sgemm_pipeline_launch(impl, a_colmajor, b, c, peers, m, n, k, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
