// Thin inline-PTX wrappers for the sm_100a features the kernels use:
// mbarrier phases with bounded waits, TMA bulk-tensor copies (never multicast),
// tcgen05 tensor-memory allocation / MMA / commit / load, and the proxy fences
// that order generic-proxy and async-proxy accesses to shared memory.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

namespace b200 {

// One status word per translation unit that contains bounded waits (the
// library is built without relocatable device code, so each such unit owns its
// copy). A kernel whose wait expired ORs a site code into it; the host gathers
// and clears the words with b200_device_status_read.
static __device__ uint32_t g_device_status = 0;

// Reads and clears this translation unit's word on the current device. The
// caller has synchronised the streams it cares about.
static inline cudaError_t status_word_read_clear(uint32_t* word) {
  *word = 0;
  cudaError_t rc = cudaMemcpyFromSymbol(word, g_device_status, sizeof(uint32_t));
  if (rc == cudaSuccess && *word != 0) {
    const uint32_t zero = 0;
    rc = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
  }
  return rc;
}

enum WaitSite : uint32_t {
  kSiteSgemmFull = 1u << 0,
  kSiteSgemmEmpty = 1u << 1,
  kSiteUmmaFull = 1u << 2,
  kSiteUmmaEmpty = 1u << 3,
  kSiteUmmaAccFull = 1u << 4,
  kSiteUmmaAccEmpty = 1u << 5,
  kSiteUmmaStore = 1u << 6,
  kSiteSelfTest = 1u << 7,
  kSitePeerBarrier = 1u << 8,
  kSiteRowStaged = 1u << 9,   // row operators: the staged row never arrived
  kSiteBounds = 1u << 10,   // debug build only: an index check failed and the access was skipped
};

// Debug build (-DB200_DEBUG_BOUNDS, a separate library; never the shipped one): the stores and the
// unpredicated loads of the kernels are wrapped in index checks against the extents the launcher
// passed. A failing check records kSiteBounds in the status word and SKIPS the access; nothing
// traps. The stand-in, on a shared GPU, for running the kernels under a memory checker.
#ifdef B200_DEBUG_BOUNDS
#define B200_IN_BOUNDS(cond) ((cond) ? true : (atomicOr(&::b200::g_device_status, ::b200::kSiteBounds), false))
#else
#define B200_IN_BOUNDS(cond) true
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  // Makes the initialised barriers visible to the async proxy (TMA, tcgen05).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// An arrival that only counts: no ordering of the thread's earlier accesses (the release form's
// fence waits for the thread's queued tcgen05 operations, which stalls an MMA-issuing thread).
__device__ __forceinline__ void mbar_arrive_relaxed(uint64_t* bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Upper bound on polls of one barrier phase. try_wait itself blocks for a
// hardware-defined interval (on the order of a microsecond) per poll, so the
// cap is seconds of wall time: far beyond any legitimate wait, short enough
// that a broken pipeline ends on its own.
constexpr uint32_t kMaxWaitPolls = 1u << 22;

// Waits for the phase with the given parity. Returns false (after recording
// `site`) when the cap was reached; callers must then stop issuing work and
// fall through to their teardown.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t site,
                                          uint32_t max_polls = kMaxWaitPolls) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < max_polls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  atomicOr(&g_device_status, site);
  return false;
}

// ------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while the
// kernel before it in the stream is still running: once every CTA of that kernel has executed
// launch_dependents (or exited). It must then execute `wait` before its first access to global
// memory: the wait returns when the earlier kernel has completed and its writes are visible. What
// runs before the wait (barrier set-up, TMEM allocation, descriptor prefetch) overlaps the earlier
// kernel's tail. Without the attribute, or after a kernel that never signals, both are no-ops.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ----------------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load global -> this CTA's shared memory, completion on `bar`.
// x is the innermost (contiguous) coordinate and must keep x * 4 bytes a
// multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// 3-D form of the same load (x innermost).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// 2-D tiled store shared -> global (bulk-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Orders this thread's generic-proxy writes to shared memory before later
// async-proxy reads of it (TMA store, tcgen05.mma operand fetch).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------- tcgen05

template <uint32_t kCols>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result) {
  static_assert(kCols >= 32 && kCols <= 512 && (kCols & (kCols - 1)) == 0, "power of two in [32, 512]");
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_result)), "n"(kCols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

template <uint32_t kCols>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], TF32 inputs, FP32 accumulate.
// Issued by a single thread. `accumulate` == 0 overwrites D.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Makes `bar` receive one arrival once every tcgen05.mma this thread issued so
// far has finished reading its operands and writing its accumulator.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 columns of 32-bit accumulators: thread t of the warp receives
// TMEM lane (base lane + t), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i, 2i + 1) drive one 256-row MMA: each holds
// its 128 rows of A, half of B's columns and its 128 rows of the accumulator.
// Nothing here uses cluster multicast: a signal for both CTAs is sent twice.

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared-window address of `local_addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}

// 128-bit store to the shared memory of a CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void st_shared_cluster_v4(uint32_t cluster_addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <uint32_t kCols>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_result)), "n"(kCols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <uint32_t kCols>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols) : "memory");
}

// Issued by one thread of the even-ranked CTA; operands are read from both
// CTAs' shared memory at the same offsets, accumulators land in both TMEMs.
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One arrival on the barrier at `cluster_addr` (this CTA's or the peer's) once
// the pair MMAs issued so far have completed in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

// TMA load into this CTA's shared memory whose completion bytes are counted on
// a barrier that may live in the peer CTA (`bar_cluster_addr`).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Shared-memory matrix descriptor (64-bit) for tcgen05.mma operands.
//   bits  0-13  start address  >> 4
//   bits 16-29  leading-dimension byte offset >> 4
//   bits 32-45  stride-dimension  byte offset >> 4
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  swizzle mode
enum UmmaSwizzle : uint32_t {
  kUmmaSwizzleNone = 0,
  kUmmaSwizzle128B32BAtom = 1,  // 128-byte span, 32-byte granules, 4-row period
  kUmmaSwizzle128B = 2,         // 128-byte span, 16-byte granules, 8-row period
};

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   UmmaSwizzle swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(swizzle) << 61;
  return d;
}

// The descriptor of the same matrix `bytes` further on in shared memory (bytes a multiple of 16).
// Only the start-address field changes, and it cannot carry out of its 14 bits while the operand
// stays inside shared memory, so this is one 32-bit addition on the low word: the MMA-issuing
// thread is a lone thread whose every instruction costs several cycles, and composing a descriptor
// from scratch per instruction made it, not the tensor pipe, the limit of the main loops.
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t desc, uint32_t bytes) {
  const uint32_t lo = static_cast<uint32_t>(desc) + (bytes >> 4);
  return (desc & 0xFFFFFFFF00000000ull) | lo;
}

// Instruction descriptor (32-bit) for kind::tf32 with FP32 accumulation.
//   bits  4-5   accumulator format (1 = F32)
//   bits  7-9   A format (2 = TF32)      bits 10-12  B format (2 = TF32)
//   bit  15     A major (0 = K, 1 = MN)  bit  16     B major
//   bits 17-22  N >> 3                   bits 24-28  M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace b200
