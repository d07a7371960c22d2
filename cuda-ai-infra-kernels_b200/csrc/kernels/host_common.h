// Host-side helpers shared by the launchers of libb200_kernels.so: status
// plumbing, cached device attributes and TMA tensor-map construction.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "b200_kernels.h"

namespace b200 {

// Destinations of a fused "GEMM + all-gather" store: besides its own output a
// kernel writes every finished tile to the same position of up to
// B200_MAX_PEERS other buffers (peer GPUs' memory mapped into this process,
// plain st.global over NVLink; never loaded from, never handed to TMA).
struct PeerOutputs {
  float* ptr[B200_MAX_PEERS];
  int count;
};

inline bool make_peer_outputs(PeerOutputs* out, float* const* peers, int n_peers) {
  out->count = 0;
  for (int i = 0; i < B200_MAX_PEERS; ++i) out->ptr[i] = nullptr;
  if (n_peers < 0 || n_peers > B200_MAX_PEERS || (n_peers > 0 && peers == nullptr)) return false;
  for (int i = 0; i < n_peers; ++i) {
    if (peers[i] == nullptr) return false;
    out->ptr[i] = peers[i];
  }
  out->count = n_peers;
  return true;
}

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// Status of the launch just made. cudaGetLastError reads AND clears the runtime's per-thread error
// slot: this library links its own (static) CUDA runtime, so nobody else would ever clear it, and a
// single refused launch (a non-sticky error such as an invalid configuration) would otherwise make
// every later call on the thread report failure.
inline int launch_status() {
  return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH_FAILED;
}

// For runtime calls that returned their own error code (cudaLaunchKernelEx, cudaFuncSetAttribute):
// the same code also sits in the per-thread slot; clear it and report the failure.
inline int launch_failed() {
  (void)cudaGetLastError();
  return B200_ERR_LAUNCH_FAILED;
}

// Launch attributes of the GEMM and row kernels: a cluster of `cluster_x` CTAs (1: none) and
// programmatic stream serialization. With the latter a kernel may start while the kernel before it
// in the stream is still running, once all CTAs of that kernel have executed
// griddepcontrol.launch_dependents (the kernels here do after their set-up) or exited; the kernels
// execute griddepcontrol.wait after their own set-up (barriers, TMEM, descriptor prefetch) and before
// their first access to global memory, which returns when the earlier kernel has completed and
// its writes are visible. Back-to-back calls overlap by about a microsecond that way.
struct GemmLaunchAttributes {
  cudaLaunchAttribute list[2];
  unsigned count;
};
inline GemmLaunchAttributes gemm_launch_attributes(unsigned cluster_x) {
  GemmLaunchAttributes a = {};
  a.list[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.list[0].val.programmaticStreamSerializationAllowed = 1;
  a.count = 1;
  if (cluster_x > 1) {
    a.list[1].id = cudaLaunchAttributeClusterDimension;
    a.list[1].val.clusterDim.x = cluster_x;
    a.list[1].val.clusterDim.y = 1;
    a.list[1].val.clusterDim.z = 1;
    a.count = 2;
  }
  return a;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize for kernel `kKernel`, set once per device and process
// (the attribute is per device; the call costs a few microseconds, which small problems notice).
template <auto kKernel, size_t kBytes>
inline bool ensure_dynamic_smem() {
  static std::atomic<uint64_t> done{0};   // bit d: set on device ordinal d
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return false;
  const uint64_t bit = (device >= 0 && device < 64) ? (uint64_t{1} << device) : 0;
  if (bit != 0 && (done.load(std::memory_order_acquire) & bit) != 0) return true;
  if (cudaFuncSetAttribute(kKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBytes)) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  if (bit != 0) done.fetch_or(bit, std::memory_order_release);
  return true;
}

// Device status words of the translation units that contain bounded waits.
cudaError_t sgemm_status_read_clear(uint32_t* word);
cudaError_t umma_status_read_clear(uint32_t* word);
cudaError_t selftest_status_read_clear(uint32_t* word);
cudaError_t peer_sync_status_read_clear(uint32_t* word);
cudaError_t rowops_status_read_clear(uint32_t* word);

// k128BAtom32B: 128-byte span swizzled in 32-byte granules (what an MN-major
// 32-bit tcgen05 operand needs); k128B: the usual 16-byte granules.
enum class Swizzle { kNone, k128B, k128BAtom32B };

// Row-major FP32 matrix [rows][cols] with a row pitch of `ld` elements, tiled
// in boxes of box_rows x box_cols (cols innermost). Out-of-range parts of a box
// read as zero and are clipped on store. Requirements (checked, false on
// failure): base 16-byte aligned, ld * 4 a multiple of 16, box_cols * 4 a
// multiple of 16 (and <= 128 bytes with either 128-byte swizzle), boxes <= 256.
bool make_tensor_map_2d(CUtensorMap* out, const float* base, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols, Swizzle swizzle);

// Row-major FP32 matrix [rows][cols] (cols a multiple of 32) viewed as
// [cols / 32][rows][32]: a box of `box_groups` x `box_rows` x 32 gathers
// `box_groups` adjacent 32-column strips of the same rows with ONE copy and
// lays them out strip after strip (box_rows * 128 bytes each) in shared memory.
bool make_tensor_map_strips(CUtensorMap* out, const float* base, uint64_t rows, uint64_t cols, uint64_t ld,
                            uint32_t box_rows, uint32_t box_groups, Swizzle swizzle);

}  // namespace b200
