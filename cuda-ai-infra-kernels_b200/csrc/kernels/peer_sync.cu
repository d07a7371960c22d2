// Device-side barrier between the GPUs of a fused "GEMM + all-gather" step. Every rank owns a
// small array of 32-bit flags in memory that all ranks have mapped (flag s of rank r = "rank s has
// finished step e"). The barrier kernel of rank r stores the step number into slot r of every
// other rank's array (st.release.sys over NVLink) and then waits until every slot of its own array
// has reached that number. Peer memory is only stored to; the waiting loads are local.
//
// The wait is bounded: after `max_polls` polls per peer the kernel records kSitePeerBarrier in the
// status word and returns, so a rank whose partner died or skipped the step does not spin on a
// shared GPU; the host learns of it through b200_device_status_read.
#include "host_common.h"
#include "ptx_sm100.cuh"

namespace b200 {

cudaError_t peer_sync_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

struct BarrierParams {
  uint32_t* flags[B200_MAX_PEERS + 1];   // by rank; entry `rank` is this device's own array
  int world, rank;
  uint32_t epoch, max_polls;
};

__device__ __forceinline__ void store_release_sys(uint32_t* addr, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__global__ void peer_barrier_kernel(const BarrierParams p) {
  const int peer = threadIdx.x;
  if (peer >= p.world || peer == p.rank) return;
  // Everything earlier kernels of this stream stored to the peers is ordered before the flag.
  __threadfence_system();
  store_release_sys(p.flags[peer] + p.rank, p.epoch);
  const uint32_t* mine = p.flags[p.rank] + peer;
  for (uint32_t i = 0; i < p.max_polls; ++i) {
    // Step numbers only grow; the signed difference tolerates wrap-around.
    if (static_cast<int32_t>(load_acquire_sys(mine) - p.epoch) >= 0) return;
    __nanosleep(256);
  }
  atomicOr(&g_device_status, kSitePeerBarrier);
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_peer_barrier(uint32_t* const* flags_by_rank, int world, int rank, uint32_t epoch, uint32_t max_polls,
                      b200_stream_t stream) {
  if (flags_by_rank == nullptr || world < 1 || world > B200_MAX_PEERS + 1 || rank < 0 || rank >= world) {
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (max_polls == 0 || max_polls > (1u << 24)) return B200_ERR_INVALID_ARGUMENT;
  b200::BarrierParams p = {};
  for (int r = 0; r < world; ++r) {
    if (flags_by_rank[r] == nullptr || reinterpret_cast<uintptr_t>(flags_by_rank[r]) % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
    p.flags[r] = flags_by_rank[r];
  }
  p.world = world, p.rank = rank, p.epoch = epoch, p.max_polls = max_polls;
  b200::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return b200::launch_status();
}

}  // extern "C"
