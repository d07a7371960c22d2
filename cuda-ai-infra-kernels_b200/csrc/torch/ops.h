// Operator entry points exported by the `cuda_ai_kernels._C` module. Names,
// argument order and defaults are those of the reference module
// (csrc/bindings.cpp:10-45).
#pragma once

#include <string>
#include <vector>

#include <c10/util/Optional.h>
#include <torch/extension.h>

torch::Tensor gemm_naive(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_cublas(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_block_tile(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_thread_tile(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_block_tile_float4_16x16(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_block_tile_float4_16x32(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_block_tile_float4_32x32(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_thread_tile_4x4(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_thread_tile_4x8(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_thread_tile_8x8(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_thread_tile_8x8_warp4x8(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_warp_tile(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_prefetch_smem(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_prefetch_reg(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_split_k(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_tensor_core(torch::Tensor a, torch::Tensor b);
torch::Tensor gemm_cutlass(torch::Tensor a, torch::Tensor b);

torch::Tensor adaptive_gemm(const torch::Tensor& a, const torch::Tensor& b, const c10::optional<at::Tensor>& c,
                            const c10::optional<at::Tensor>& bias, double alpha, double beta,
                            const std::string& epilogue, const std::string& kernel);
// Name of the registry entry the last adaptive_gemm call of this thread ran
// ("cublas" for the library baseline). Not part of the reference module.
std::string adaptive_gemm_last_kernel();

// Sharded GEMM fused with the all-gather of its output (not part of the
// reference module, which is single-GPU): the product is written into `out`, a
// [M, N] row-major view of this rank's rows inside its copy of the gathered
// matrix, and every finished tile is also stored to `peer_ptrs[i]`, the address
// of the same rows in peer i's copy (mapped into this process by the caller).
torch::Tensor gemm_gather(torch::Tensor a, torch::Tensor b, torch::Tensor out, std::vector<int64_t> peer_ptrs,
                          const std::string& impl);
torch::Tensor adaptive_gemm_gather(const torch::Tensor& a, const torch::Tensor& b, const c10::optional<at::Tensor>& c,
                                   const c10::optional<at::Tensor>& bias, double alpha, double beta,
                                   const std::string& epilogue, const std::string& kernel, torch::Tensor out,
                                   std::vector<int64_t> peer_ptrs);

torch::Tensor rmsnorm_naive(torch::Tensor x, torch::Tensor weight, double eps);
torch::Tensor rmsnorm_cache_x(torch::Tensor x, torch::Tensor weight, double eps);
torch::Tensor softmax_naive(torch::Tensor x);
torch::Tensor rope_forward(torch::Tensor x, torch::Tensor cos, torch::Tensor sin);
torch::Tensor attention_decode_forward(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache);
