// Shared device code and launch helpers of the TF32 tensor-core GEMM kernels (tcgen05, sm_100a):
// the operand layouts in shared memory, the kernel parameter block, the epilogues, and the
// producer-independent roles (MMA issuer, epilogue warps) of the single-CTA persistent kernels.
// Included by the kernel translation units only; everything here has internal linkage.
//
// TF32 tensor-core GEMM with a fused epilogue, written for sm_100a:
//   D = epilogue(alpha * A * B + beta * C),  A [M,K], B [K,N], C/D [M,N],
// all row-major FP32; products in TF32 on tcgen05.mma, accumulation in FP32 in
// tensor memory (TMEM); epilogue (scale, source add, bias, optional ReLU or
// GELU) applied on the TMEM -> register -> global path, so the accumulator
// never touches HBM.
//
// It stands in for the CUTLASS device::Gemm instantiations of the reference
// (csrc/adaptive_gemm/kernel_sm80.h:4-171, launched through
// csrc/adaptive_gemm/kernel_launcher.h:7-29).
//
// Operand staging. One pipeline stage holds a 128 x 32 slab of A and a
// 32 x BN slab of B in swizzled layouts that both TMA and the MMA unit
// understand:
//   A is K-major for the MMA (K contiguous in memory). The slab is one TMA box
//     {32 (k), 128 (m)}: 128 rows of 128 bytes, 128-byte swizzle in 16-byte
//     granules (period 8 rows), 8-row groups 1024 bytes apart.
//   B is N-major for the MMA (N contiguous in memory). A 32-bit N-major operand
//     must use the 128-byte swizzle with 32-byte granules (period 4 rows). The
//     slab is BN/32 TMA boxes {32 (n), 32 (k)}: each 32 rows (k) of 128 bytes
//     (32 n), boxes 4096 bytes apart; inside a box, 4-row k groups are 512
//     bytes apart.
// One tcgen05.mma consumes 8 floats of K: the A descriptor advances 32 bytes
// inside the swizzled row, the B descriptor advances two 4-row groups.
//
// Two loaders feed that layout:
//   TMA     - needs 16-byte aligned pointers and leading dimensions that are
//             multiples of four floats; persistent, warp-specialised kernels
//             (producer / MMA issuer / epilogue warps), double-buffered TMEM
//             accumulator so the epilogue of one tile overlaps the main loop of
//             the next. Two forms: one CTA per 128 x BN tile, and CTA pairs
//             (cta_group::2) that share a 256 x 256 tile and halve the B bytes
//             each CTA pulls through L2. A third form gives one 128 x 128 tile
//             to a cluster whose CTAs split K and exchange their partial tiles
//             through distributed shared memory (few tiles, long K).
//   generic - any pointers, any sizes; eight loader warps of a persistent CTA
//             write predicated scalar loads into the same swizzled layout.
// Nothing here uses cluster multicast. Every kernel can also store its finished
// output to peer GPUs' copies of D (PeerOutputs: a GEMM fused with the
// all-gather of its result); peer memory is only ever stored to.
#pragma once

#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "host_common.h"
#include "ptx_sm100.cuh"
#include "tf32_gemm.h"

namespace b200 {
namespace {

constexpr int kTileM = 128;
constexpr int kStageK = 32;                       // floats of K per stage (one 128-byte swizzle row)
constexpr int kInstK = 8;                         // K of one tcgen05.mma kind::tf32
constexpr uint32_t kASlabBytes = kTileM * kStageK * 4;  // 16 KiB
constexpr uint32_t kBBoxBytes = 32 * kStageK * 4;       // 4 KiB: 32 (n) x 32 (k)

// Build-time instrumentation (-DB200_PROBE_TIMING, never in the shipped library):
// one thread per CTA stamps the global timer at the phase boundaries of a kernel.
#ifdef B200_PROBE_TIMING
#define B200_PROBE(params, slot)                                                              \
  do {                                                                                        \
    if ((params).probe != nullptr && threadIdx.x == 64) {                                     \
      uint64_t t_;                                                                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
      (params).probe[static_cast<size_t>(blockIdx.x) * 16 + (slot)] = t_;                      \
      (params).probe[4096 + static_cast<size_t>(blockIdx.x) * 16 + (slot)] = clock64();        \
    }                                                                                         \
  } while (0)
extern "C" uint64_t* b200_probe_buffer;   // [2][256][16], defined and set by the instrumented build's driver
#else
#define B200_PROBE(params, slot) do { } while (0)
#endif

struct UmmaParams {
  CUtensorMap map_a;   // [M][K] boxes {32, 128}, 128-byte swizzle   (TMA loader only)
  CUtensorMap map_b;   // [K][N] boxes {32, 32},  128-byte swizzle, 32-byte granules
  CUtensorMap map_b_strips;  // [N/32][K][32] boxes {32, 32, strips}: a whole B slab in one copy (N % 32 == 0)
  int b_strips;        // strips per map_b_strips box, 0 when that map is not usable
  CUtensorMap map_d;   // [M][N] boxes {32, 32}, 128-byte swizzle: the output, written by TMA stores
  int tma_store;       // map_d is usable (D 16-byte aligned, ldd a multiple of four floats)
  const float* a;      // generic loader only
  const float* b;
  const float* c;      // source, may be null when beta == 0
  const float* bias;   // [N] added to every row before the activation, or null
  float* d;
  int64_t lda, ldb, ldc, ldd;
  int m, n, k;
  float alpha, beta;
  int vector_io;       // C/D rows allow 128-bit accesses
  PeerOutputs peers;   // further destinations of every finished element (fused all-gather), usually none
  int pair_full_tiles;  // CTA-pair kernel: work items [0, full) are whole 256 x 256 tiles, the rest
                        // are the two 256 x 128 halves of the tiles after them (see launch_pair)
#ifdef B200_PROBE_TIMING
  uint64_t* probe;     // [2][256][16] time stamps, or null
#endif
};

// The epilogue's view of the problem, copied into registers once per thread. The kernel parameter
// block is memory as far as the compiler can tell, memory that the epilogue's own stores might
// alias: reading it inside the store loops would reload every field after every store, a chain of
// dependent loads that the few epilogue warps cannot hide.
struct EpilogueArgs {
  const float* c;      // null when beta == 0
  const float* bias;   // or null
  float* d;
  int64_t ldc, ldd;
  int m, n;
  float alpha, beta;
  int vector_io;
  PeerOutputs peers;
};

__device__ __forceinline__ EpilogueArgs epilogue_args(const UmmaParams& p) {
  return EpilogueArgs{p.c, p.bias, p.d, p.ldc, p.ldd, p.m, p.n, p.alpha, p.beta, p.vector_io, p.peers};
}

// The same element(s) of every peer's copy of the output (fused all-gather).
// (Unrolled with constant indices: a run-time index would put the whole argument block in local memory.)
__device__ __forceinline__ void store_peers(const EpilogueArgs& p, int64_t offset, float4 v) {
#pragma unroll
  for (int i = 0; i < B200_MAX_PEERS; ++i) {
    if (i < p.peers.count) *reinterpret_cast<float4*>(p.peers.ptr[i] + offset) = v;
  }
}
__device__ __forceinline__ void store_peers(const EpilogueArgs& p, int64_t offset, float v) {
#pragma unroll
  for (int i = 0; i < B200_MAX_PEERS; ++i) {
    if (i < p.peers.count) p.peers.ptr[i][offset] = v;
  }
}

template <int BN>
__host__ __device__ constexpr uint32_t stage_bytes() {
  return kASlabBytes + (BN / 32) * kBBoxBytes;
}

// Staging of the epilogues: 32 KiB of 32 x 32 FP32 boxes (4 KiB each) in the 128-byte swizzle, shared
// out evenly among the epilogue warps of a kernel (two boxes per warp with four warps, one with eight).
//   - Ordinary epilogue: a warp turns each 32 x 32 chunk through a box, from which one TMA store
//     writes the output in whole 128-byte row segments.
//   - Fused all-gather: the finished chunk (one row per lane in registers) is turned through a box
//     so that peer copies are written in 128-byte row segments, four rows per instruction, instead
//     of 32 scattered 16-byte pieces (NVLink moves those poorly).
// A launch uses one or the other.
constexpr uint32_t kOutBoxBytes = 32 * 32 * sizeof(float);
constexpr size_t kStagingBytes = 8 * kOutBoxBytes;   // 32 KiB, 1024-byte aligned

// ring | 1 KiB of barriers and the TMEM pointer | staging; the base is rounded up to 1 KiB.
template <int BN, int STAGES>
__host__ __device__ constexpr size_t smem_bytes() {
  return static_cast<size_t>(STAGES) * stage_bytes<BN>() + 1024 /*alignment slack*/ + 1024 /*barriers + tmem ptr*/ +
         kStagingBytes;
}

// Two accumulator buffers of kIssuers partial accumulators each, BN columns apart; the allocation
// is the next power of two (a 192-wide tile's two buffers take 384 of 512 columns).
template <int BN, int kIssuers = 1>
__host__ __device__ constexpr uint32_t tmem_columns() {
  uint32_t columns = 32;
  while (columns < 2u * kIssuers * BN) columns *= 2;
  return columns;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int* tm, int* tn) {
  constexpr int kBand = 8;   // bands of 1, 2, 4 and 16 tile rows measured within noise of this at 3072^3 .. 8192^3
  const int per_band = kBand * tiles_n;
  const int band = tile / per_band;
  const int first_m = band * kBand;
  const int band_rows = min(kBand, tiles_m - first_m);
  const int in_band = tile - band * per_band;
  *tm = first_m + in_band % band_rows;
  *tn = in_band / band_rows;
}

// Descriptors of the first MMA of a 32-wide K sub-block whose A slab starts at `a_addr` (B slab
// right behind it).
//   A: K-major, 8-row groups 1024 bytes apart (SBO); LBO is not used by the swizzled K-major form
//      and carries the customary 16 bytes.
//   B: N-major, 32-column groups 4096 bytes apart (LBO), 4-row k groups 512 bytes apart (SBO);
//      one MMA spans two of them.
struct SubBlockDescs {
  uint64_t a, b;
};
__device__ __forceinline__ SubBlockDescs sub_block_descs(uint32_t a_addr) {
  return SubBlockDescs{umma_smem_desc(a_addr, 16, 1024, kUmmaSwizzle128B),
                       umma_smem_desc(a_addr + kASlabBytes, kBBoxBytes, 512, kUmmaSwizzle128B32BAtom)};
}

// Issues the four MMAs of one 32-wide K sub-block. `accumulate_first` is 0 only for the very
// first MMA of an output tile. Successive MMAs advance 32 bytes along a row of A and eight rows
// (1024 bytes) of B.
template <int BN>
__device__ __forceinline__ void issue_stage_mmas(uint32_t tmem_acc, const SubBlockDescs& first, uint32_t accumulate_first) {
  constexpr uint32_t idesc = umma_idesc_tf32(kTileM, BN, /*a_mn_major=*/false, /*b_mn_major=*/true);
#pragma unroll
  for (int j = 0; j < kStageK / kInstK; ++j) {
    umma_tf32(tmem_acc, umma_desc_advance(first.a, j * (kInstK * 4)), umma_desc_advance(first.b, j * (kInstK * 128)), idesc,
              j == 0 ? accumulate_first : 1u);
  }
}

// Activation applied last: after scaling, source add and bias.
template <int kAct>
__device__ __forceinline__ float activate(float v) {
  if constexpr (kAct == B200_EPILOGUE_RELU) return fmaxf(v, 0.f);
  if constexpr (kAct == B200_EPILOGUE_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));  // exact (erf) GELU
  return v;
}

// ------------------------------------------------- epilogue through shared memory and TMA stores
// A thread owns one ROW of the accumulator (that is how tcgen05.ld hands it out), so storing
// straight from registers makes every warp-wide 128-bit access touch 32 different 128-byte lines:
// the load/store unit handles one line per cycle, and a 256-column tile cost about 16 000 of those
// cycles in reads of C and writes of D - 15 us that nothing hides for a CTA's last tile (in-kernel
// time stamps at 1024^3 .. 4096^3). Here the warp turns each 32 x 32 chunk through a swizzled box in
// shared memory instead: C arrives with coalesced loads (a lane holds column quad l % 8 of rows
// 4 j + l / 8, four whole 128-byte rows per instruction) and is turned into row ownership in the box;
// the finished chunk is written into the box row by row and leaves as ONE TMA store, which also
// clips the edges of the matrix. Arithmetic and its order are those of every other epilogue path
// (alpha * acc rounded, then one FMA with the source, then the bias): all paths give the same bits.

// Source values of a 32 x 32 chunk in coalesced ownership.
struct SourceQuads {
  float4 v[8];   // v[j]: row 4 j + lane / 8, columns 4 (lane % 8) .. + 3
};

__device__ __forceinline__ void fetch_source_coalesced(const EpilogueArgs& p, SourceQuads& out, int row0, int col0, int lane) {
  const bool want = p.beta != 0.f && col0 + 4 * (lane & 7) < p.n;
  const float* c_ptr = p.c + static_cast<int64_t>(row0 + (lane >> 3)) * p.ldc + col0 + 4 * (lane & 7);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    out.v[j] = (want && row0 + 4 * j + (lane >> 3) < p.m) ? __ldg(reinterpret_cast<const float4*>(c_ptr + static_cast<int64_t>(4 * j) * p.ldc))
                                                          : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Byte offset of the 16-byte granule (row, quad) of a 32 x 32 FP32 box in the 128-byte swizzle.
__device__ __forceinline__ uint32_t box_offset(int row, int quad) {
  return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(quad ^ (row & 7)) << 4);
}

// First half of a chunk: waits until `box` (one of the warp's kBoxes boxes, used in turn) is free - at
// most kBoxes - 1 earlier stores may still be reading the others - and turns the source values into
// row ownership through it. After this the registers of `cq` are free for the next chunk's source.
template <int kBoxes>
__device__ __forceinline__ void stage_source_boxed(const EpilogueArgs& ep, const SourceQuads& cq, int lane, uint8_t* box) {
  if (lane == 0) tma_store_wait_read<kBoxes - 1>();   // the store that used this box kBoxes chunks ago has read it
  __syncwarp();
  if (ep.beta != 0.f) {
    // Row 4 j + lane / 8: the swizzle term (row % 8) takes two values, for even and for odd j, so
    // every store is one of two per-lane bases plus a constant.
    const uint32_t r = static_cast<uint32_t>(lane >> 3), quad = static_cast<uint32_t>(lane & 7);
    uint8_t* even = box + r * 128u + ((quad ^ r) << 4);
    uint8_t* odd = box + r * 128u + ((quad ^ (r + 4u)) << 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(((j & 1) ? odd : even) + j * 512) = cq.v[j];
    __syncwarp();
  }
}

// Second half: alpha * acc + beta * C + bias, activation, into the box, TMA store.
template <int kAct>
__device__ __forceinline__ void finish_chunk_boxed(const UmmaParams& p, const EpilogueArgs& ep, const uint32_t (&raw)[32],
                                                   int row0, int col0, int lane, uint8_t* box) {
  const bool use_source = ep.beta != 0.f;
  // From here on a lane touches its own row of the box only: it reads the granules of C and puts
  // the finished values in their place. Four granules at a time, all loads before the first store:
  // the compiler cannot tell the swizzled slots apart, so a store between two loads would order
  // them, and a lone warp then pays the shared-memory latency once per granule (880 cycles a chunk).
  const bool use_bias = ep.bias != nullptr;
  uint8_t* row_base = box + static_cast<uint32_t>(lane) * 128u;
  const uint32_t swz = static_cast<uint32_t>(lane & 7);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int g = 4 * h + q;
      v[q] = use_source ? *reinterpret_cast<const float4*>(row_base + ((static_cast<uint32_t>(g) ^ swz) << 4))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int g = 4 * h + q;
      v[q] = make_float4(fmaf(ep.beta, v[q].x, ep.alpha * __uint_as_float(raw[4 * g + 0])),
                         fmaf(ep.beta, v[q].y, ep.alpha * __uint_as_float(raw[4 * g + 1])),
                         fmaf(ep.beta, v[q].z, ep.alpha * __uint_as_float(raw[4 * g + 2])),
                         fmaf(ep.beta, v[q].w, ep.alpha * __uint_as_float(raw[4 * g + 3])));
      if (use_bias && col0 + 4 * g < ep.n) {
        const float4 bv = __ldg(reinterpret_cast<const float4*>(ep.bias + col0 + 4 * g));
        v[q].x += bv.x, v[q].y += bv.y, v[q].z += bv.z, v[q].w += bv.w;
      }
      v[q] = make_float4(activate<kAct>(v[q].x), activate<kAct>(v[q].y), activate<kAct>(v[q].z), activate<kAct>(v[q].w));
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int g = 4 * h + q;
      *reinterpret_cast<float4*>(row_base + ((static_cast<uint32_t>(g) ^ swz) << 4)) = v[q];
    }
  }
  fence_proxy_async_smem();   // the box was written through the generic proxy, the store reads through the async one
  __syncwarp();
  if (lane == 0) {
    if (row0 < ep.m && col0 < ep.n) tma_store_2d(&p.map_d, box, col0, row0);   // rows and columns past the matrix are clipped
    tma_store_commit();   // one group per use of a box, stored or not: the wait above counts groups
  }
}

// Epilogue of one 128 x BN tile for one warp through its boxes. kShare warps serve each quarter of
// the accumulator's rows (TMEM lanes); warp `part` of them takes the 32-column chunks part,
// part + kShare, ... Software-pipelined: two named register sets of accumulator values alternate and
// the source registers are refilled as soon as their values sit in the box, so while a chunk is
// finished the warp's next chunk is on its way from TMEM and its source values from memory.
// `src` arrives holding the source of the warp's first chunk (fetched by the caller before it
// waited for the accumulator); `uses` counts the warp's box uses across tiles.
// kIssuers == 2: the tile's accumulator is the sum of two partial ones, BN columns apart (mma_role).
__device__ __forceinline__ void add_partial_accumulator(uint32_t (&raw)[32], uint32_t taddr) {
  uint32_t other[32];
  tmem_ld_32x32(taddr, other);
  tmem_ld_wait();
#pragma unroll
  for (int e = 0; e < 32; ++e) raw[e] = __float_as_uint(__uint_as_float(raw[e]) + __uint_as_float(other[e]));
}

// `first_box`, when not null, is the box in which the caller has already staged the source of the
// warp's first chunk (before it waited for the accumulator: the source does not depend on the
// product, and a CTA with a single tile has nothing else to hide that step behind).
template <int kShare>
__host__ __device__ constexpr int boxes_per_warp() { return 2 / kShare; }

template <int BN, int kAct, int kShare, int kIssuers = 1>
__device__ __forceinline__ void epilogue_tile_boxed(const UmmaParams& p, const EpilogueArgs& ep, uint32_t tmem_acc, int quarter,
                                                    int part, int lane, int m0, int n0, SourceQuads& src, uint8_t* boxes,
                                                    uint32_t& uses, uint8_t* first_box = nullptr) {
  constexpr int kChunks = BN / 32;
  constexpr int kMine = (kChunks + kShare - 1) / kShare;   // chunks of this warp; one fewer for the later warps of a
                                                            // quarter when the tile's chunks do not divide evenly
  constexpr int kBoxes = boxes_per_warp<kShare>();
  static_assert(kShare == 1 || kShare == 2, "four or eight epilogue warps");
  static_assert(BN % 32 == 0 && kChunks >= 1, "whole 32-column chunks (a 32-wide tile leaves the later warps of a quarter idle)");
  const int row0 = m0 + quarter * 32;
  const uint32_t tmem_row = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16);
  uint32_t raw_even[32], raw_odd[32];
  if (kChunks % kShare != 0 && part >= kChunks) return;   // a 32-wide tile: nothing for the later warps of a quarter
  tmem_ld_32x32(tmem_row + part * 32, raw_even);
  if constexpr (kIssuers == 2) tmem_ld_32x32(tmem_row + BN + part * 32, raw_odd);   // the first chunk's other partial sum
#pragma unroll
  for (int i = 0; i < kMine; i += 2) {
    const int chunk = part + i * kShare;
    constexpr bool kEven = kChunks % kShare == 0;   // then every warp of a quarter has kMine chunks
    if ((!kEven && chunk >= kChunks) || n0 + chunk * 32 >= ep.n) break;   // uniform across the warp
    const bool second = i + 1 < kMine && (kEven || chunk + kShare < kChunks);       // the warp has a chunk after this one
    const bool third = i + 2 < kMine && (kEven || chunk + 2 * kShare < kChunks);    // and one after that
    uint8_t* box = first_box;
    if (i > 0 || first_box == nullptr) {
      box = boxes + (uses++ % kBoxes) * kOutBoxBytes;
      stage_source_boxed<kBoxes>(ep, src, lane, box);
    }
    tmem_ld_wait();
    if constexpr (kIssuers == 2) {
      if (i == 0) {
#pragma unroll
        for (int e = 0; e < 32; ++e) raw_even[e] = __float_as_uint(__uint_as_float(raw_even[e]) + __uint_as_float(raw_odd[e]));
      } else {
        add_partial_accumulator(raw_even, tmem_row + BN + chunk * 32);
      }
    }
    if (second) {
      tmem_ld_32x32(tmem_row + (chunk + kShare) * 32, raw_odd);
      fetch_source_coalesced(ep, src, row0, n0 + (chunk + kShare) * 32, lane);
    }
    finish_chunk_boxed<kAct>(p, ep, raw_even, row0, n0 + chunk * 32, lane, box);
    if (second) {
      box = boxes + (uses++ % kBoxes) * kOutBoxBytes;
      stage_source_boxed<kBoxes>(ep, src, lane, box);
      tmem_ld_wait();
      if constexpr (kIssuers == 2) add_partial_accumulator(raw_odd, tmem_row + BN + (chunk + kShare) * 32);
      if (third) {
        tmem_ld_32x32(tmem_row + (chunk + 2 * kShare) * 32, raw_even);
        fetch_source_coalesced(ep, src, row0, n0 + (chunk + 2 * kShare) * 32, lane);
      }
      finish_chunk_boxed<kAct>(p, ep, raw_odd, row0, n0 + (chunk + kShare) * 32, lane, box);
    }
  }
  tmem_ld_wait();   // nothing from TMEM is in flight when the accumulator is handed back
}

// Epilogue of one 128 x BN tile for one warp, straight from registers: TMEM lanes [32 * quarter, +32)
// are rows m0 + 32 * quarter + lane. Each thread owns one row and walks it in chunks of 32 columns;
// warp `part` of the kShare that serve the quarter takes chunks part, part + kShare, ...
template <int BN, int kAct, int kShare, int kIssuers = 1>
__device__ __forceinline__ void epilogue_tile(const EpilogueArgs& p, uint32_t tmem_acc, int quarter, int part, int lane,
                                              int m0, int n0, uint8_t* stage) {
  const int row = m0 + quarter * 32 + lane;
  const bool stage_peers = p.peers.count > 0 && p.vector_io;   // `stage`: one of this warp's boxes
  const bool row_ok = row < p.m;
  const bool use_c = p.beta != 0.f;
  const bool use_bias = p.bias != nullptr;
  const float* c_row = p.c + static_cast<int64_t>(row) * p.ldc;
  float* d_row = p.d + static_cast<int64_t>(row) * p.ldd;
#pragma unroll 1
  for (int chunk = part; chunk < BN / 32; chunk += kShare) {
    const int col0 = n0 + chunk * 32;
    if (col0 >= p.n) break;  // uniform across the warp
    uint32_t raw[32];
    tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 32, raw);
    tmem_ld_wait();
    if constexpr (kIssuers == 2) add_partial_accumulator(raw, tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + BN + chunk * 32);
    if (!row_ok && !stage_peers) continue;
    if (stage_peers) {
      // Local copy straight from registers; peer copies row-wise from the staged chunk.
      if (row_ok) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int col = col0 + 4 * g;
          if (col < p.n) {
            float4 v = make_float4(p.alpha * __uint_as_float(raw[4 * g + 0]), p.alpha * __uint_as_float(raw[4 * g + 1]),
                                   p.alpha * __uint_as_float(raw[4 * g + 2]), p.alpha * __uint_as_float(raw[4 * g + 3]));
            if (use_c) {
              const float4 s = __ldg(reinterpret_cast<const float4*>(c_row + col));
              v.x = fmaf(p.beta, s.x, v.x), v.y = fmaf(p.beta, s.y, v.y);
              v.z = fmaf(p.beta, s.z, v.z), v.w = fmaf(p.beta, s.w, v.w);
            }
            if (use_bias) {
              const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col));
              v.x += bv.x, v.y += bv.y, v.z += bv.z, v.w += bv.w;
            }
            v = make_float4(activate<kAct>(v.x), activate<kAct>(v.y), activate<kAct>(v.z), activate<kAct>(v.w));
            *reinterpret_cast<float4*>(d_row + col) = v;
            *reinterpret_cast<float4*>(stage + box_offset(lane, g)) = v;
          }
        }
      }
      __syncwarp();
      // Lane l takes column quad l % 8 of rows 4 j + l / 8.
      const int quad_col = col0 + 4 * (lane & 7);
      if (quad_col < p.n) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = 4 * j + (lane >> 3);
          const int out_row = m0 + quarter * 32 + r;
          if (out_row < p.m) {
            const float4 v = *reinterpret_cast<const float4*>(stage + box_offset(r, lane & 7));
            store_peers(p, static_cast<int64_t>(out_row) * p.ldd + quad_col, v);
          }
        }
      }
      __syncwarp();   // the chunk is reused by the next iteration
      continue;
    }
    if (p.vector_io) {
      // n % 4 == 0 here, so a 4-wide group is entirely inside or outside.
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int col = col0 + 4 * g;
        if (col < p.n) {
          float4 v = make_float4(p.alpha * __uint_as_float(raw[4 * g + 0]), p.alpha * __uint_as_float(raw[4 * g + 1]),
                                 p.alpha * __uint_as_float(raw[4 * g + 2]), p.alpha * __uint_as_float(raw[4 * g + 3]));
          if (use_c) {
            const float4 s = __ldg(reinterpret_cast<const float4*>(c_row + col));
            v.x = fmaf(p.beta, s.x, v.x), v.y = fmaf(p.beta, s.y, v.y);
            v.z = fmaf(p.beta, s.z, v.z), v.w = fmaf(p.beta, s.w, v.w);
          }
          if (use_bias) {
            const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col));
            v.x += bv.x, v.y += bv.y, v.z += bv.z, v.w += bv.w;
          }
          v = make_float4(activate<kAct>(v.x), activate<kAct>(v.y), activate<kAct>(v.z), activate<kAct>(v.w));
          if (!B200_IN_BOUNDS(row >= 0 && row < p.m && col >= 0 && col + 4 <= p.n && p.ldd >= p.n)) continue;
          *reinterpret_cast<float4*>(d_row + col) = v;
        }
      }
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int col = col0 + e;
        if (col < p.n) {
          float v = p.alpha * __uint_as_float(raw[e]);
          if (use_c) v = fmaf(p.beta, __ldg(c_row + col), v);
          if (use_bias) v += __ldg(p.bias + col);
          v = activate<kAct>(v);
          if (!B200_IN_BOUNDS(row >= 0 && row < p.m && col >= 0 && col < p.n)) continue;
          d_row[col] = v;
          store_peers(p, static_cast<int64_t>(row) * p.ldd + col, v);
        }
      }
    }
  }
}

struct SmemCarve {
  uint8_t* stages;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* acc_full;
  uint64_t* acc_empty;
  uint32_t* tmem_ptr;
  float* peer_stage;   // kStagingBytes, 1024-byte aligned: fused all-gather staging or output boxes
};

template <int BN, int STAGES>
__device__ __forceinline__ SmemCarve carve(uint8_t* raw) {
  SmemCarve s;
  s.stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.full = reinterpret_cast<uint64_t*>(s.stages + static_cast<size_t>(STAGES) * stage_bytes<BN>());
  s.empty = s.full + STAGES;
  s.acc_full = s.empty + STAGES;
  s.acc_empty = s.acc_full + 2;
  s.tmem_ptr = reinterpret_cast<uint32_t*>(s.acc_empty + 2);
  s.peer_stage = reinterpret_cast<float*>(s.stages + static_cast<size_t>(STAGES) * stage_bytes<BN>() + 1024);
  return s;
}

// MMA issuer of the persistent single-CTA kernels (one thread): for every tile
// of this CTA, waits until the epilogue has drained the accumulator buffer,
// then consumes the operand ring stage by stage.
// `KSUB` 32-wide K sub-blocks share one pipeline stage (one barrier wait, one commit): the ring has
// STAGES / KSUB stages, and `k_blocks` counts stages.
// With kIssuers == 2 two threads (of different warps) run this role side by side, each with its own
// accumulator (columns [i BN, (i + 1) BN) of the buffer; the epilogue adds the two):
//   KSUB even: issuer i takes the sub-blocks i, i + 2, ... of every stage, both commit every stage
//              (`empty` barriers count two arrivals);
//   KSUB == 1: issuer i takes the stages i, i + 2, ... of the ring (an even number of stages, and the
//              caller passes an even `k_blocks`, padding K with a block that reads as zeros, so that
//              the assignment is the same for every tile), one commit per stage.
// An issuing thread is alone on its scheduler; the tensor pipe takes an MMA only when it has room,
// so the pipe stands idle while its only issuer waits on a barrier or commits (about 300 of the 820
// cycles of a 128 x 128 stage of two sub-blocks, and a 128 x 64 MMA costs the thread the same 58
// cycles as a 128 x 128 one for half the pipe time). Two issuers fill each other's gaps. They must
// not share an accumulator: MMAs of different threads are not ordered with respect to each other.
template <int KSUB, int kIssuers>
__host__ __device__ constexpr int empty_barrier_arrivals() {
  return (kIssuers == 2 && KSUB > 1) ? 2 : 1;
}

template <int BN, int STAGES, int KSUB = 1, int kIssuers = 1>
__device__ __forceinline__ void mma_role(const SmemCarve& sm, uint32_t tmem_base, int tiles, int k_blocks, int issuer = 0) {
  static_assert(STAGES % KSUB == 0, "whole stages");
  static_assert(kIssuers == 1 || (kIssuers == 2 && (KSUB % 2 == 0 || (KSUB == 1 && STAGES % 2 == 0))),
                "every issuer has work in every stage, or every other stage");
  constexpr int kRing = STAGES / KSUB;
  constexpr bool kAlternate = kIssuers == 2 && KSUB == 1;   // issuers take alternate stages
  constexpr int kStep = kAlternate ? 2 : 1;
  const SubBlockDescs ring = sub_block_descs(smem_u32(sm.stages));   // of the ring's first sub-block
  int stage = kAlternate ? issuer : 0;
  uint32_t phase = 0;
  bool ok = true;
  int local = 0;
  for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
    const int buf = local & 1;
    const uint32_t use_parity = (local >> 1) & 1u;
    // The epilogue must have drained this accumulator buffer.
    if (!mbar_wait(&sm.acc_empty[buf], use_parity ^ 1u, kSiteUmmaAccEmpty)) { ok = false; break; }
    tcgen05_fence_after_sync();
    const uint32_t tmem_acc = tmem_base + (buf * kIssuers + issuer) * BN;
    const int kb_first = kAlternate ? issuer : 0;
    for (int kb = kb_first; kb < k_blocks; kb += kStep) {
      if (!mbar_wait(&sm.full[stage], phase, kSiteUmmaFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
      const uint32_t stage_offset = static_cast<uint32_t>(stage * KSUB + (kAlternate ? 0 : issuer)) * stage_bytes<BN>();
#pragma unroll
      for (int sub = 0; sub < KSUB; sub += (kAlternate ? 1 : kIssuers)) {
        const SubBlockDescs descs{umma_desc_advance(ring.a, stage_offset + sub * stage_bytes<BN>()),
                                  umma_desc_advance(ring.b, stage_offset + sub * stage_bytes<BN>())};
        issue_stage_mmas<BN>(tmem_acc, descs, (kb > kb_first || sub > 0) ? 1u : 0u);
      }
      umma_commit(&sm.empty[stage]);  // stage reusable once these MMAs have read it
      stage += kStep;
      if (stage >= kRing) stage -= kRing, phase ^= 1u;
    }
    if (ok) umma_commit(&sm.acc_full[buf]);   // one arrival per issuer
  }
}

// One of the 4 * kShare epilogue warps of the persistent single-CTA kernels: `quarter` is the warp's
// quarter of the accumulator rows (its hardware warp index modulo four, which is what tcgen05.ld
// lets it read), `part` in [0, kShare) its place among the warps of that quarter.
template <int BN, int kAct, bool kPipelinedEpilogue, int kShare, int kIssuers = 1>
__device__ __forceinline__ void epilogue_role(const UmmaParams& p, const SmemCarve& sm, uint32_t tmem_base, int quarter,
                                              int part, int lane, int tiles, int tiles_m, int tiles_n) {
  const EpilogueArgs ep = epilogue_args(p);
  bool ok = true;
  int local = 0;
  const bool boxed = kPipelinedEpilogue && p.tma_store != 0 && ep.vector_io && ep.peers.count == 0;
  uint8_t* boxes = reinterpret_cast<uint8_t*>(sm.peer_stage) + (part * 4 + quarter) * (kStagingBytes / (4 * kShare));
  uint32_t box_uses = 0;
  for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
    const int buf = local & 1;
    const uint32_t use_parity = (local >> 1) & 1u;
    int tm, tn;
    tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
    // Before the wait for the accumulator: the source of the warp's first chunk is fetched and turned
    // into row ownership in its box.
    SourceQuads first;
    uint8_t* first_box = nullptr;
    if (boxed && part < BN / 32) {   // (a 32-wide tile has a chunk for the first warp of each quarter only)
      fetch_source_coalesced(ep, first, tm * kTileM + quarter * 32, tn * BN + part * 32, lane);
      first_box = boxes + (box_uses++ % boxes_per_warp<kShare>()) * kOutBoxBytes;
      stage_source_boxed<boxes_per_warp<kShare>()>(ep, first, lane, first_box);
    }
    B200_PROBE(p, 2);
    if (!mbar_wait(&sm.acc_full[buf], use_parity, kSiteUmmaAccFull)) { ok = false; break; }
    tcgen05_fence_after_sync();
    B200_PROBE(p, 3);
    if (boxed) {
      epilogue_tile_boxed<BN, kAct, kShare, kIssuers>(p, ep, tmem_base + buf * kIssuers * BN, quarter, part, lane, tm * kTileM,
                                                      tn * BN, first, boxes, box_uses, first_box);
    } else {
      epilogue_tile<BN, kAct, kShare, kIssuers>(ep, tmem_base + buf * kIssuers * BN, quarter, part, lane, tm * kTileM, tn * BN,
                                                boxes);
    }
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
    B200_PROBE(p, 4);
  }
  if (boxed && lane == 0) tma_store_wait_read<0>();   // every store has read its box (the writes land before the grid completes)
  B200_PROBE(p, 5);
}

// Threads of the cluster kernels (split-K, operand-swapped): warp 0 producer, warp 1 TMEM owner +
// MMA issuer, warps 2-5 epilogue.
constexpr int kTmaThreads = 6 * 32;

// Threads of the persistent TMA-fed tile kernels and the CTA-pair kernel: the same two warps and
// eight epilogue warps, two per quarter of the accumulator rows. An epilogue warp has its
// scheduler to itself and issues one dependent instruction every few cycles, so the epilogue of a
// tile is bound by its instruction count per warp: with four warps a 32-column chunk took about
// 1500 cycles (in-kernel time stamps: 2900 cycles for a 128 x 64 tile, 6400 for 128 x 128), all of
// it exposed when a CTA has a single tile. Eight warps halve the chunks per warp.
constexpr int kTileEpilogueShare = 2;
constexpr int kTileThreads = (2 + 4 * kTileEpilogueShare) * 32;
// The tile kernels with two MMA issuers (mma_role) add one warp for the second.
constexpr int kTileThreadsTwoIssuers = kTileThreads + 32;

// ------------------------------------------------------------- host-side helpers

bool aligned16(const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; }

void fill_common(UmmaParams* p, const b200_gemm_problem& q, const PeerOutputs& peers) {
  std::memset(p, 0, sizeof(*p));
  p->peers = peers;
  p->a = q.a, p->b = q.b, p->d = q.d;
  p->c = q.beta != 0.f ? q.c : nullptr;
  p->bias = q.bias;
  p->lda = q.lda, p->ldb = q.ldb, p->ldc = q.ldc, p->ldd = q.ldd;
  p->m = q.m, p->n = q.n, p->k = q.k;
  p->alpha = q.alpha, p->beta = q.beta;
  const bool c_ok = q.beta == 0.f || (aligned16(q.c) && q.ldc % 4 == 0);
  const bool bias_ok = q.bias == nullptr || aligned16(q.bias);
  bool peers_ok = true;   // peer copies share the row pitch of D, only their bases can differ in alignment
  for (int i = 0; i < peers.count; ++i) peers_ok = peers_ok && aligned16(peers.ptr[i]);
  p->vector_io = (q.n % 4 == 0 && aligned16(q.d) && q.ldd % 4 == 0 && c_ok && bias_ok && peers_ok) ? 1 : 0;
#ifdef B200_PROBE_TIMING
  p->probe = b200_probe_buffer;
#endif
}

}  // namespace
}  // namespace b200
