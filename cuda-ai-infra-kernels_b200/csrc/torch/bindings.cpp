// pybind11 module `cuda_ai_kernels._C`: the 23 functions of the reference
// module (csrc/bindings.cpp:10-45) with identical names, positional order,
// keyword names and defaults, plus one introspection helper and the two fused all-gather entries of the
// multi-GPU path.
#include <torch/extension.h>

#include "ops.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "B200 (sm_100a) kernels behind the cuda_ai_kernels operator API";
  const char* ladder_doc = "FP32 SIMT GEMM: column-major A, row-major B/C, full tiles";
  m.def("gemm_naive", &gemm_naive, ladder_doc);
  m.def("gemm_cublas", &gemm_cublas, "cuBLAS strict-FP32 GEMM baseline");
  m.def("gemm_block_tile", &gemm_block_tile, ladder_doc);
  m.def("gemm_thread_tile", &gemm_thread_tile, ladder_doc);
  m.def("gemm_block_tile_float4_16x16", &gemm_block_tile_float4_16x16, ladder_doc);
  m.def("gemm_block_tile_float4_16x32", &gemm_block_tile_float4_16x32, ladder_doc);
  m.def("gemm_block_tile_float4_32x32", &gemm_block_tile_float4_32x32, ladder_doc);
  m.def("gemm_thread_tile_4x4", &gemm_thread_tile_4x4, ladder_doc);
  m.def("gemm_thread_tile_4x8", &gemm_thread_tile_4x8, ladder_doc);
  m.def("gemm_thread_tile_8x8", &gemm_thread_tile_8x8, ladder_doc);
  m.def("gemm_thread_tile_8x8_warp4x8", &gemm_thread_tile_8x8_warp4x8, ladder_doc);
  m.def("gemm_warp_tile", &gemm_warp_tile, ladder_doc);
  m.def("gemm_prefetch_smem", &gemm_prefetch_smem, "FP32 SIMT GEMM fed by a TMA + mbarrier ring");
  m.def("gemm_prefetch_reg", &gemm_prefetch_reg, "TMA ring + register double buffer + packed FMAs");
  m.def("gemm_split_k", &gemm_split_k, "K split across CTAs (stream-K), partial sums reduced into a cleared output");
  m.def("gemm_tensor_core", &gemm_tensor_core, "Row-major TF32 GEMM on tcgen05 tensor cores");
  m.def("gemm_cutlass", &gemm_cutlass, "Row-major TF32 GEMM on tcgen05 tensor cores");
  m.def("rmsnorm_naive", &rmsnorm_naive, "RMSNorm forward");
  m.def("rmsnorm_cache_x", &rmsnorm_cache_x, "RMSNorm forward (hidden <= 4096)");
  m.def("softmax_naive", &softmax_naive, "Row softmax forward");
  m.def("rope_forward", &rope_forward, "RoPE forward (not implemented)");
  m.def("attention_decode_forward", &attention_decode_forward, "Attention decode forward (not implemented)");
  m.def("adaptive_gemm", &adaptive_gemm, "TF32 GEMM with fused epilogue behind a compatibility registry",
        py::arg("a"), py::arg("b"), py::arg("c") = py::none(), py::arg("bias") = py::none(), py::arg("alpha") = 1.0,
        py::arg("beta") = 0.0, py::arg("epilogue") = "linear", py::arg("kernel") = "auto");
  m.def("gemm_gather", &gemm_gather, "FP32 SIMT GEMM whose epilogue also stores every tile to peer GPUs (fused all-gather)",
        py::arg("a"), py::arg("b"), py::arg("out"), py::arg("peer_ptrs"), py::arg("impl") = "prefetch_reg");
  m.def("adaptive_gemm_gather", &adaptive_gemm_gather,
        "TF32 GEMM + fused epilogue whose stores also go to peer GPUs (fused all-gather)", py::arg("a"), py::arg("b"),
        py::arg("c") = py::none(), py::arg("bias") = py::none(), py::arg("alpha") = 1.0, py::arg("beta") = 0.0,
        py::arg("epilogue") = "linear", py::arg("kernel") = "auto", py::arg("out"), py::arg("peer_ptrs"));
  m.def("adaptive_gemm_last_kernel", &adaptive_gemm_last_kernel,
        "Registry name chosen by this thread's last adaptive_gemm call");
}
