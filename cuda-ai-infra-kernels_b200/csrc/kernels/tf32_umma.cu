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
#include <cooperative_groups.h>

#include <atomic>
#include <cstring>

#include "host_common.h"
#include "tf32_gemm.h"
#include "ptx_sm100.cuh"

namespace b200 {

cudaError_t umma_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

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
      (params).probe[static_cast<size_t>(blockIdx.x) * 8 + (slot)] = t_;                      \
      (params).probe[2048 + static_cast<size_t>(blockIdx.x) * 8 + (slot)] = clock64();        \
    }                                                                                         \
  } while (0)
#else
#define B200_PROBE(params, slot) do { } while (0)
#endif

struct UmmaParams {
  CUtensorMap map_a;   // [M][K] boxes {32, 128}, 128-byte swizzle   (TMA loader only)
  CUtensorMap map_b;   // [K][N] boxes {32, 32},  128-byte swizzle, 32-byte granules
  CUtensorMap map_b_strips;  // [N/32][K][32] boxes {32, 32, strips}: a whole B slab in one copy (N % 32 == 0)
  int b_strips;        // strips per map_b_strips box, 0 when that map is not usable
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
  uint64_t* probe;     // [grid][8] time stamps, or null
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

// Staging of the fused all-gather: an epilogue warp turns its 32 x 32 chunk (one row per lane in
// registers) by way of shared memory so that peer copies are written in 128-byte row segments, four
// rows per instruction, instead of 32 scattered 16-byte pieces (NVLink moves those poorly). The
// pitch of 36 floats keeps both the row-per-lane writes and the row-wise reads free of conflicts.
constexpr int kPeerStagePitch = 36;
constexpr size_t kPeerStageBytesPerWarp = 32 * kPeerStagePitch * sizeof(float);
constexpr size_t kPeerStageBytes = 4 * kPeerStageBytesPerWarp;   // four epilogue warps

template <int BN, int STAGES>
__host__ __device__ constexpr size_t smem_bytes() {
  return static_cast<size_t>(STAGES) * stage_bytes<BN>() + 1024 /*alignment slack*/ + 256 /*barriers + tmem ptr*/ +
         kPeerStageBytes;
}

template <int BN>
__host__ __device__ constexpr uint32_t tmem_columns() {
  return 2 * BN < 32 ? 32 : 2 * BN;  // two accumulator buffers; BN in {64,128,256} keeps this a power of two
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int* tm, int* tn) {
  constexpr int kBand = 8;
  const int per_band = kBand * tiles_n;
  const int band = tile / per_band;
  const int first_m = band * kBand;
  const int band_rows = min(kBand, tiles_m - first_m);
  const int in_band = tile - band * per_band;
  *tm = first_m + in_band % band_rows;
  *tn = in_band / band_rows;
}

// Issues the four MMAs of one stage. `accumulate_first` is 0 only for the very
// first MMA of an output tile.
template <int BN>
__device__ __forceinline__ void issue_stage_mmas(uint32_t tmem_acc, uint32_t a_addr, uint32_t b_addr,
                                                 uint32_t accumulate_first) {
  constexpr uint32_t idesc = umma_idesc_tf32(kTileM, BN, /*a_mn_major=*/false, /*b_mn_major=*/true);
#pragma unroll
  for (int j = 0; j < kStageK / kInstK; ++j) {
    // A: K-major, 8-row groups 1024 bytes apart (SBO); LBO is not used by the
    //    swizzled K-major form and carries the customary 16 bytes.
    // B: N-major, 32-column groups 4096 bytes apart (LBO), 4-row k groups
    //    512 bytes apart (SBO); one MMA spans two of them.
    const uint64_t desc_a = umma_smem_desc(a_addr + j * (kInstK * 4), 16, 1024, kUmmaSwizzle128B);
    const uint64_t desc_b = umma_smem_desc(b_addr + j * (kInstK * 128), kBBoxBytes, 512, kUmmaSwizzle128B32BAtom);
    umma_tf32(tmem_acc, desc_a, desc_b, idesc, j == 0 ? accumulate_first : 1u);
  }
}

// Activation applied last: after scaling, source add and bias.
template <int kAct>
__device__ __forceinline__ float activate(float v) {
  if constexpr (kAct == B200_EPILOGUE_RELU) return fmaxf(v, 0.f);
  if constexpr (kAct == B200_EPILOGUE_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));  // exact (erf) GELU
  return v;
}

// Source values of one 32-column chunk of a thread's row (zeros when there is no source).
struct SourceChunk {
  float4 v[8];
};

// C of chunk `chunk` for the row of this thread. Issued well before the values are needed:
// for the first chunk of a tile even before the accumulator is ready.
__device__ __forceinline__ void fetch_source(const EpilogueArgs& p, SourceChunk& out, int row, int col0) {
  const bool want = p.beta != 0.f && row < p.m;
  const float* c_row = p.c + static_cast<int64_t>(row) * p.ldc;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int col = col0 + 4 * g;
    out.v[g] = (want && col < p.n) ? __ldg(reinterpret_cast<const float4*>(c_row + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// One chunk of the vectorised epilogue: alpha * acc + beta * C + bias, activation, 128-bit stores.
template <int kAct>
__device__ __forceinline__ void finish_chunk(const EpilogueArgs& p, const uint32_t (&raw)[32], const SourceChunk& src, int row,
                                             int col0) {
  if (row >= p.m) return;
  const bool use_bias = p.bias != nullptr;
  float* d_row = p.d + static_cast<int64_t>(row) * p.ldd;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int col = col0 + 4 * g;
    if (col < p.n) {   // n % 4 == 0 on this path: a quad is inside or outside as a whole
      // Same operation order as every other epilogue path (alpha * acc rounded, then one FMA with
      // the source), so that all paths give identical bits. Without a source src is zero and beta finite.
      float4 v = make_float4(fmaf(p.beta, src.v[g].x, p.alpha * __uint_as_float(raw[4 * g + 0])),
                             fmaf(p.beta, src.v[g].y, p.alpha * __uint_as_float(raw[4 * g + 1])),
                             fmaf(p.beta, src.v[g].z, p.alpha * __uint_as_float(raw[4 * g + 2])),
                             fmaf(p.beta, src.v[g].w, p.alpha * __uint_as_float(raw[4 * g + 3])));
      if (use_bias) {
        const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col));
        v.x += bv.x, v.y += bv.y, v.z += bv.z, v.w += bv.w;
      }
      *reinterpret_cast<float4*>(d_row + col) =
          make_float4(activate<kAct>(v.x), activate<kAct>(v.y), activate<kAct>(v.z), activate<kAct>(v.w));
    }
  }
}

// Vectorised epilogue of one 128 x BN tile for one warp, software-pipelined: while a chunk is
// scaled and stored, the next chunk's accumulators are on their way from TMEM and its source
// values from memory. `first` holds the source of chunk 0 (fetched by the caller before it waited
// for the accumulator). Two named register sets alternate so that both stay in registers.
template <int BN, int kAct>
__device__ __forceinline__ void epilogue_tile_pipelined(const EpilogueArgs& p, uint32_t tmem_acc, int quarter, int lane,
                                                        int m0, int n0, const SourceChunk& first) {
  constexpr int kChunks = BN / 32;
  static_assert(kChunks % 2 == 0, "chunks are handled in pairs");
  const int row = m0 + quarter * 32 + lane;
  const uint32_t tmem_row = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16);
  uint32_t raw_even[32], raw_odd[32];
  SourceChunk src_even = first, src_odd;
  tmem_ld_32x32(tmem_row, raw_even);
#pragma unroll
  for (int chunk = 0; chunk < kChunks; chunk += 2) {
    if (n0 + chunk * 32 >= p.n) break;   // uniform across the warp
    tmem_ld_wait();
    tmem_ld_32x32(tmem_row + (chunk + 1) * 32, raw_odd);
    fetch_source(p, src_odd, row, n0 + (chunk + 1) * 32);
    finish_chunk<kAct>(p, raw_even, src_even, row, n0 + chunk * 32);
    tmem_ld_wait();
    if (chunk + 2 < kChunks) {
      tmem_ld_32x32(tmem_row + (chunk + 2) * 32, raw_even);
      fetch_source(p, src_even, row, n0 + (chunk + 2) * 32);
    }
    finish_chunk<kAct>(p, raw_odd, src_odd, row, n0 + (chunk + 1) * 32);
  }
  tmem_ld_wait();   // nothing from TMEM is in flight when the accumulator is handed back
}

// Epilogue of one 128 x BN tile for one warp: TMEM lanes [32 * quarter, +32)
// are rows m0 + 32 * quarter + lane. Each thread owns one row and walks it in
// chunks of 32 columns.
template <int BN, int kAct>
__device__ __forceinline__ void epilogue_tile(const EpilogueArgs& p, uint32_t tmem_acc, int quarter, int lane, int m0,
                                              int n0, float* stage) {
  const int row = m0 + quarter * 32 + lane;
  const bool stage_peers = p.peers.count > 0 && p.vector_io;   // `stage`: this warp's kPeerStageBytesPerWarp
  const bool row_ok = row < p.m;
  const bool use_c = p.beta != 0.f;
  const bool use_bias = p.bias != nullptr;
  const float* c_row = p.c + static_cast<int64_t>(row) * p.ldc;
  float* d_row = p.d + static_cast<int64_t>(row) * p.ldd;
#pragma unroll 1
  for (int chunk = 0; chunk < BN / 32; ++chunk) {
    const int col0 = n0 + chunk * 32;
    if (col0 >= p.n) break;  // uniform across the warp
    uint32_t raw[32];
    tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 32, raw);
    tmem_ld_wait();
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
            *reinterpret_cast<float4*>(stage + lane * kPeerStagePitch + 4 * g) = v;
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
            const float4 v = *reinterpret_cast<const float4*>(stage + r * kPeerStagePitch + 4 * (lane & 7));
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
  float* peer_stage;   // kPeerStageBytes, 16-byte aligned
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
  s.peer_stage = reinterpret_cast<float*>(s.tmem_ptr + 4);
  return s;
}

// MMA issuer of the persistent single-CTA kernels (one thread): for every tile
// of this CTA, waits until the epilogue has drained the accumulator buffer,
// then consumes the operand ring stage by stage.
// `KSUB` 32-wide K sub-blocks share one pipeline stage (one barrier wait, one commit): the ring has
// STAGES / KSUB stages, and `k_blocks` counts stages.
template <int BN, int STAGES, int KSUB = 1>
__device__ __forceinline__ void mma_role(const SmemCarve& sm, uint32_t tmem_base, int tiles, int k_blocks) {
  static_assert(STAGES % KSUB == 0, "whole stages");
  constexpr int kRing = STAGES / KSUB;
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  int local = 0;
  for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
    const int buf = local & 1;
    const uint32_t use_parity = (local >> 1) & 1u;
    // The epilogue must have drained this accumulator buffer.
    if (!mbar_wait(&sm.acc_empty[buf], use_parity ^ 1u, kSiteUmmaAccEmpty)) { ok = false; break; }
    tcgen05_fence_after_sync();
    const uint32_t tmem_acc = tmem_base + buf * BN;
    for (int kb = 0; kb < k_blocks; ++kb) {
      if (!mbar_wait(&sm.full[stage], phase, kSiteUmmaFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
#pragma unroll
      for (int sub = 0; sub < KSUB; ++sub) {
        const uint32_t a_addr = smem_u32(sm.stages + static_cast<size_t>(stage * KSUB + sub) * stage_bytes<BN>());
        issue_stage_mmas<BN>(tmem_acc, a_addr, a_addr + kASlabBytes, (kb > 0 || sub > 0) ? 1u : 0u);
      }
      umma_commit(&sm.empty[stage]);  // stage reusable once these MMAs have read it
      if (++stage == kRing) stage = 0, phase ^= 1u;
    }
    if (ok) umma_commit(&sm.acc_full[buf]);
  }
}

// One of the four epilogue warps of the persistent single-CTA kernels.
template <int BN, int kAct, bool kPipelinedEpilogue>
__device__ __forceinline__ void epilogue_role(const UmmaParams& p, const SmemCarve& sm, uint32_t tmem_base, int quarter,
                                              int lane, int tiles, int tiles_m, int tiles_n) {
  const EpilogueArgs ep = epilogue_args(p);
  bool ok = true;
  int local = 0;
  for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
    const int buf = local & 1;
    const uint32_t use_parity = (local >> 1) & 1u;
    int tm, tn;
    tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
    const bool pipelined = kPipelinedEpilogue && ep.vector_io && ep.peers.count == 0;
    SourceChunk first;
    if (pipelined) fetch_source(ep, first, tm * kTileM + quarter * 32 + lane, tn * BN);   // before the wait
    if (!mbar_wait(&sm.acc_full[buf], use_parity, kSiteUmmaAccFull)) { ok = false; break; }
    tcgen05_fence_after_sync();
    if (pipelined) {
      epilogue_tile_pipelined<BN, kAct>(ep, tmem_base + buf * BN, quarter, lane, tm * kTileM, tn * BN, first);
    } else {
      epilogue_tile<BN, kAct>(ep, tmem_base + buf * BN, quarter, lane, tm * kTileM, tn * BN,
                              sm.peer_stage + quarter * (kPeerStageBytesPerWarp / sizeof(float)));
    }
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
  }
}

// ------------------------------------------------------- TMA, persistent kernel
// warp 0: TMA producer (one lane)      warp 1: TMEM owner + MMA issuer (one lane)
// warps 2-5: epilogue; warp w reads the TMEM lane quarter w % 4.
constexpr int kTmaThreads = 6 * 32;

// STAGES counts 32-wide K blocks of shared memory; KSUB of them form one pipeline stage (the MMA
// thread's barrier wait and commit cost about as much as four small MMAs, so narrow tiles, whose
// MMAs are short, run two sub-blocks per stage).
template <int BN, int STAGES, int kAct, int KSUB = 1>
__global__ void __launch_bounds__(kTmaThreads, 1) umma_tma_kernel(const __grid_constant__ UmmaParams p) {
  constexpr int kRing = STAGES / KSUB;
  extern __shared__ uint8_t smem_raw[];
  const SmemCarve sm = carve<BN, STAGES>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], 1);
      mbar_init(&sm.acc_empty[b], 4);  // one arrive per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc<tmem_columns<BN>()>(sm.tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;

  const int tiles_m = (p.m + kTileM - 1) / kTileM;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  const int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages per tile; K past the end reads as zeros

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&p.map_a);
      prefetch_tensormap(&p.map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sm.empty[stage], phase ^ 1u, kSiteUmmaEmpty)) { ok = false; break; }
          mbar_expect_tx(&sm.full[stage], KSUB * stage_bytes<BN>());
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const int k0 = (kb * KSUB + sub) * kStageK;
            uint8_t* a_dst = sm.stages + static_cast<size_t>(stage * KSUB + sub) * stage_bytes<BN>();
            uint8_t* b_dst = a_dst + kASlabBytes;
            tma_load_2d(a_dst, &p.map_a, &sm.full[stage], k0, tm * kTileM);
            if (p.b_strips == BN / 32) {
              // The producer thread's issue rate matters: one copy instead of BN / 32.
              tma_load_3d(b_dst, &p.map_b_strips, &sm.full[stage], 0, k0, tn * (BN / 32));
            } else {
#pragma unroll
              for (int j = 0; j < BN / 32; ++j) {
                tma_load_2d(b_dst + j * kBBoxBytes, &p.map_b, &sm.full[stage], tn * BN + j * 32, k0);
              }
            }
          }
          if (++stage == kRing) stage = 0, phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) mma_role<BN, STAGES, KSUB>(sm, tmem_base, tiles, k_blocks);
  } else {
    epilogue_role<BN, kAct, true>(p, sm, tmem_base, warp & 3, lane, tiles, tiles_m, tiles_n);
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<tmem_columns<BN>()>(tmem_base);
  }
}

// ---------------------------------------------------- TMA, CTA-pair kernel
// Two CTAs of a cluster share one 256 x 256 output tile through
// tcgen05.mma.cta_group::2: CTA r of the pair holds rows [128 r, 128 r + 128) of
// A, columns [128 r, 128 r + 128) of B and the accumulator rows [128 r, +128)
// (all 256 columns). Per CTA a stage is 16 KiB of A + 16 KiB of B for a
// 256 x 256 x 32 product, a third fewer operand bytes through L2 per flop than
// the single-CTA 128 x 256 tile. The even CTA issues the MMAs for both.
// Signals that both CTAs need (stage free, accumulator ready) are committed
// twice, once per CTA; no multicast form is used anywhere.
constexpr int kPairN = 256;
constexpr uint32_t kPairSubBytes = kASlabBytes + (kPairN / 2 / 32) * kBBoxBytes;  // 32 floats of K: 32 KiB per CTA

// A pipeline stage holds KSUB such 32-wide K sub-blocks behind one pair of barriers: the MMA
// thread's barrier wait, fence and commits are paid per stage, and they cost about as much as two
// of the eight instructions of a two-sub-block stage.
template <int STAGES, int KSUB>
__host__ __device__ constexpr size_t pair_smem_bytes() {
  return static_cast<size_t>(STAGES) * KSUB * kPairSubBytes + 1024 + 256 + kPeerStageBytes;
}

// Work item of the CTA-pair kernel: a whole 256 x 256 tile, or (for the last, partial round of
// tiles) one 256 x 128 half of one, so that twice as many pairs share the tail.
struct PairItem {
  int tile;
  int half;   // -1: whole tile; 0 / 1: left / right 128 columns
};
__device__ __forceinline__ PairItem pair_item(int item, int full_tiles) {
  if (item < full_tiles) return PairItem{item, -1};
  const int h = item - full_tiles;
  return PairItem{full_tiles + (h >> 1), h & 1};
}

template <int STAGES, int KSUB, int kAct>
__global__ void __launch_bounds__(kTmaThreads, 1) umma_pair_kernel(const __grid_constant__ UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Same carve-up in both CTAs: the MMA addresses the peer's shared memory by
  // the same offsets as its own.
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t kPairStageBytes = KSUB * kPairSubBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(STAGES) * kPairStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* peer_stage = reinterpret_cast<float*>(tmem_ptr + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0: issues the MMAs, 1: peer

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);   // used in CTA 0 only: one expect_tx arrival, bytes of both CTAs
      mbar_init(&empty[s], 1);  // one tcgen05.commit per use, sent to each CTA
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // used in CTA 0 only: four epilogue warps of each CTA
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair<512>(tmem_ptr);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any remote arrival
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;

  const int tiles_m = (p.m + 2 * kTileM - 1) / (2 * kTileM);
  const int tiles_n = (p.n + kPairN - 1) / kPairN;
  const int tiles = tiles_m * tiles_n;
  const int items = p.pair_full_tiles + 2 * (tiles - p.pair_full_tiles);   // whole tiles, then halves
  const int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages per tile; K past the end reads as zeros
  const int first_tile = blockIdx.x >> 1, tile_stride = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&p.map_a);
      prefetch_tensormap(&p.map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = first_tile; item < items && ok; item += tile_stride) {
        const PairItem it = pair_item(item, p.pair_full_tiles);
        int tm, tn;
        tile_coords(it.tile, tiles_m, tiles_n, &tm, &tn);
        const int row0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
        // This CTA's share of the B columns: 128 of a whole tile, 64 of a half tile.
        const int cta_cols = it.half < 0 ? kPairN / 2 : kPairN / 4;
        const int col0 = tn * kPairN + (it.half < 0 ? 0 : it.half * (kPairN / 2)) + static_cast<int>(rank) * cta_cols;
        const uint32_t sub_tx = kASlabBytes + (cta_cols / 32) * kBBoxBytes;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, kSiteUmmaEmpty)) { ok = false; break; }
          // Completion bytes of both CTAs are counted on CTA 0's barrier.
          const uint32_t full_addr = map_to_cta(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * KSUB * sub_tx);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const int k0 = (kb * KSUB + sub) * kStageK;
            uint8_t* a_dst = stages + static_cast<size_t>(stage) * kPairStageBytes + sub * kPairSubBytes;
            uint8_t* b_dst = a_dst + kASlabBytes;
            tma_load_2d_pair(a_dst, &p.map_a, full_addr, k0, row0);
            if (it.half < 0 && p.b_strips == kPairN / 2 / 32) {
              tma_load_3d_pair(b_dst, &p.map_b_strips, full_addr, 0, k0, col0 / 32);
            } else {
              for (int j = 0; j < cta_cols / 32; ++j) {
                tma_load_2d_pair(b_dst + j * kBBoxBytes, &p.map_b, full_addr, col0 + j * 32, k0);
              }
            }
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_whole = umma_idesc_tf32(2 * kTileM, kPairN, /*a_mn_major=*/false, /*b_mn_major=*/true);
      constexpr uint32_t idesc_half = umma_idesc_tf32(2 * kTileM, kPairN / 2, /*a_mn_major=*/false, /*b_mn_major=*/true);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int item = first_tile; item < items && ok; item += tile_stride, ++local) {
        const uint32_t idesc = item < p.pair_full_tiles ? idesc_whole : idesc_half;
        const int buf = local & 1;
        const uint32_t use_parity = (local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], use_parity ^ 1u, kSiteUmmaAccEmpty)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + buf * kPairN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) { ok = false; break; }
          tcgen05_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const uint32_t a_addr = smem_u32(stages + static_cast<size_t>(stage) * kPairStageBytes + sub * kPairSubBytes);
            const uint32_t b_addr = a_addr + kASlabBytes;
#pragma unroll
            for (int j = 0; j < kStageK / kInstK; ++j) {
              const uint64_t desc_a = umma_smem_desc(a_addr + j * (kInstK * 4), 16, 1024, kUmmaSwizzle128B);
              const uint64_t desc_b = umma_smem_desc(b_addr + j * (kInstK * 128), kBBoxBytes, 512, kUmmaSwizzle128B32BAtom);
              umma_tf32_pair(tmem_acc, desc_a, desc_b, idesc, (kb > 0 || sub > 0 || j > 0) ? 1u : 0u);
            }
          }
          // The stage is reusable in both CTAs once these MMAs have read it.
          umma_commit_pair(smem_u32(&empty[stage]));
          umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 1));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) {
          umma_commit_pair(smem_u32(&acc_full[buf]));
          umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 1));
        }
      }
    }
  } else {
    const EpilogueArgs ep = epilogue_args(p);
    const int quarter = warp & 3;
    bool ok = true;
    int local = 0;
    for (int item = first_tile; item < items && ok; item += tile_stride, ++local) {
      const PairItem it = pair_item(item, p.pair_full_tiles);
      const int buf = local & 1;
      const uint32_t use_parity = (local >> 1) & 1u;
      int tm, tn;
      tile_coords(it.tile, tiles_m, tiles_n, &tm, &tn);
      const int n0 = tn * kPairN + (it.half < 0 ? 0 : it.half * (kPairN / 2));
      const int m0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
      const bool pipelined = ep.vector_io && ep.peers.count == 0;
      SourceChunk first;
      if (pipelined) fetch_source(ep, first, m0 + quarter * 32 + lane, n0);   // before the wait
      if (!mbar_wait(&acc_full[buf], use_parity, kSiteUmmaAccFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
      float* stage_area = peer_stage + quarter * (kPeerStageBytesPerWarp / sizeof(float));
      if (it.half < 0) {
        if (pipelined) {
          epilogue_tile_pipelined<kPairN, kAct>(ep, tmem_base + buf * kPairN, quarter, lane, m0, n0, first);
        } else {
          epilogue_tile<kPairN, kAct>(ep, tmem_base + buf * kPairN, quarter, lane, m0, n0, stage_area);
        }
      } else if (pipelined) {
        epilogue_tile_pipelined<kPairN / 2, kAct>(ep, tmem_base + buf * kPairN, quarter, lane, m0, n0, first);
      } else {
        epilogue_tile<kPairN / 2, kAct>(ep, tmem_base + buf * kPairN, quarter, lane, m0, n0, stage_area);
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      // The MMA issuer (CTA 0) waits for the epilogues of both CTAs.
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer may still be signalling this CTA's barriers or reading its operands
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair<512>(tmem_base);
  }
}

// ------------------------------------------------ TMA, split-K cluster kernel
// For problems with too few 128 x 128 output tiles to occupy the SMs (few rows,
// or small M x N with a long K): the 1, 2, 4 or 8 CTAs of a cluster share one
// output tile and each reduces a contiguous range of K blocks into its own TMEM
// accumulator (same producer / MMA roles as above, one tile per CTA, up to
// two CTAs per SM). The partial tiles then meet in shared memory across the cluster:
//   1. cluster barrier: every main loop is finished, so every operand ring is
//      idle and becomes the exchange buffer;
//   2. each epilogue thread (one accumulator row) sends the columns
//      [r * W, (r + 1) * W), W = 128 / cluster, of its partial row to CTA r
//      (distributed-shared-memory stores), rows outside the matrix are skipped;
//   3. cluster barrier; CTA r adds the partials of its W columns in rank order
//      (a fixed order: results do not depend on timing) and applies the fused
//      epilogue. No scratch buffer, no atomics, no second launch.
namespace cg = cooperative_groups;

constexpr int kSplitN = 128;

// Scaling, source, bias and activation for four adjacent outputs of one row.
template <int kAct>
__device__ __forceinline__ void finish_quad(const EpilogueArgs& p, int row, int col, float4 acc) {
  float v[4] = {p.alpha * acc.x, p.alpha * acc.y, p.alpha * acc.z, p.alpha * acc.w};
  const float* c_row = p.c + static_cast<int64_t>(row) * p.ldc;
  float* d_row = p.d + static_cast<int64_t>(row) * p.ldd;
  if (p.vector_io) {  // n % 4 == 0: the quad is inside the matrix as a whole
    if (p.beta != 0.f) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(c_row + col));
      v[0] = fmaf(p.beta, s.x, v[0]), v[1] = fmaf(p.beta, s.y, v[1]);
      v[2] = fmaf(p.beta, s.z, v[2]), v[3] = fmaf(p.beta, s.w, v[3]);
    }
    if (p.bias != nullptr) {
      const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col));
      v[0] += bv.x, v[1] += bv.y, v[2] += bv.z, v[3] += bv.w;
    }
    const float4 out = make_float4(activate<kAct>(v[0]), activate<kAct>(v[1]), activate<kAct>(v[2]), activate<kAct>(v[3]));
    *reinterpret_cast<float4*>(d_row + col) = out;
    store_peers(p, static_cast<int64_t>(row) * p.ldd + col, out);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (col + e < p.n) {
        float out = v[e];
        if (p.beta != 0.f) out = fmaf(p.beta, __ldg(c_row + col + e), out);
        if (p.bias != nullptr) out += __ldg(p.bias + col + e);
        out = activate<kAct>(out);
        d_row[col + e] = out;
        store_peers(p, static_cast<int64_t>(row) * p.ldd + col + e, out);
      }
    }
  }
}

// Exchange buffer of a CTA: float4 elements [source][column quad of its share][row], kExchangePitch
// elements per (source, quad). Senders own a row each, so a warp writes 32 consecutive elements;
// the finishing pass reads row-wise (lanes = adjacent quads of one row) and the odd pitch spreads
// those reads over the banks.
constexpr int kExchangePitch = kTileM + 1;

// Step 2 of the split-K kernels for one epilogue thread (one accumulator row of kCols columns in
// TMEM at `tmem_row`): the columns of share s go to the CTA with cluster rank
// s * rank_stride + rank_offset, into that CTA's buffer for source `my_slice`. The next 32 columns
// are fetched from TMEM while the current ones are being sent; a share is at least 16 columns
// wide, so each half chunk (four quads) has a single destination. `send_chunk` sends one chunk.
__device__ __forceinline__ void send_chunk(cg::cluster_group& cluster, const uint32_t (&cur)[32], int chunk, float4* exchange,
                                           int my_slice, int quads_log2, int rank_stride, int rank_offset,
                                           int row_in_tile) {
  const int quads = 1 << quads_log2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int quad0 = chunk * 8 + half * 4;
    const int dest_slice = quad0 >> quads_log2, local_quad0 = quad0 & (quads - 1);
    float4* dst = cluster.map_shared_rank(exchange, dest_slice * rank_stride + rank_offset) +
                  (my_slice * quads + local_quad0) * kExchangePitch + row_in_tile;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = half * 16 + j * 4;
      dst[j * kExchangePitch] = make_float4(__uint_as_float(cur[e + 0]), __uint_as_float(cur[e + 1]),
                                            __uint_as_float(cur[e + 2]), __uint_as_float(cur[e + 3]));
    }
  }
}

template <int kCols>
__device__ __forceinline__ void send_partial_row(cg::cluster_group& cluster, uint32_t tmem_row, bool have_acc,
                                                 float4* exchange, int my_slice, int quads_log2, int rank_stride,
                                                 int rank_offset, int row_in_tile) {
  constexpr int kChunks = kCols / 32;
  static_assert(kChunks % 2 == 0, "chunks are handled in pairs");
  // Two register sets, named rather than indexed so that both stay in registers.
  uint32_t even[32], odd[32];
  if (have_acc) {
    tmem_ld_32x32(tmem_row, even);
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) even[e] = odd[e] = 0u;   // an empty K range contributes zeros
  }
#pragma unroll
  for (int chunk = 0; chunk < kChunks; chunk += 2) {
    if (have_acc) {
      tmem_ld_wait();
      tmem_ld_32x32(tmem_row + (chunk + 1) * 32, odd);
    }
    send_chunk(cluster, even, chunk, exchange, my_slice, quads_log2, rank_stride, rank_offset, row_in_tile);
    if (have_acc) {
      tmem_ld_wait();
      if (chunk + 2 < kChunks) tmem_ld_32x32(tmem_row + (chunk + 2) * 32, even);
    }
    send_chunk(cluster, odd, chunk + 1, exchange, my_slice, quads_log2, rank_stride, rank_offset, row_in_tile);
  }
}

// Step 3 of the split-K kernels for thread t of `threads`: adds the partials of this CTA's column
// share in source order and writes finished rows with lanes along the row, so that C is read and
// D is written in contiguous segments. Only a few warps run this, so four outputs per thread are
// kept in flight to cover the latencies.
template <int kAct>
__device__ __forceinline__ void exchange_finish(const EpilogueArgs& p, const float4* exchange, int sources, int quads_log2,
                                                int row0, int col_base, int t, int threads) {
  constexpr int kBatch = 4;
  const int quads = 1 << quads_log2;
  const int items = kTileM << quads_log2;
  for (int base = t; base < items; base += kBatch * threads) {
    float4 sum[kBatch];
    const float4* src_ptr[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int item = min(base + u * threads, items - 1);   // clamped: a duplicate read, no duplicate write below
      src_ptr[u] = exchange + (item & (quads - 1)) * kExchangePitch + (item >> quads_log2);
      sum[u] = *src_ptr[u];
    }
    for (int src = 1; src < sources; ++src) {
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const float4 v = src_ptr[u][src * quads * kExchangePitch];
        sum[u].x += v.x, sum[u].y += v.y, sum[u].z += v.z, sum[u].w += v.w;
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int item = base + u * threads;
      const int row = row0 + (item >> quads_log2), col = col_base + 4 * (item & (quads - 1));
      if (item < items && row < p.m && col < p.n) finish_quad<kAct>(p, row, col, sum[u]);
    }
  }
}

template <int STAGES, int kAct>
__global__ void __launch_bounds__(kTmaThreads, 2) umma_splitk_kernel(const __grid_constant__ UmmaParams p) {
  constexpr int BN = kSplitN;
  static_assert(static_cast<size_t>(STAGES) * stage_bytes<BN>() >= sizeof(float4) * kExchangePitch * (BN / 4),
                "the idle operand ring must hold one exchanged tile");
  cg::cluster_group cluster = cg::this_cluster();
  const int ranks = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  extern __shared__ uint8_t smem_raw[];
  const SmemCarve sm = carve<BN, STAGES>(smem_raw);
  B200_PROBE(p, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.acc_full[0], 1);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc<BN>(sm.tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;
  B200_PROBE(p, 1);

  const int tiles_m = (p.m + kTileM - 1) / kTileM;
  const int tiles_n = (p.n + BN - 1) / BN;
  int tm, tn;
  tile_coords(static_cast<int>(blockIdx.x) / ranks, tiles_m, tiles_n, &tm, &tn);
  const int k_blocks = (p.k + kStageK - 1) / kStageK;
  const int per_rank = (k_blocks + ranks - 1) / ranks;
  const int kb_begin = min(k_blocks, rank * per_rank);
  const int kb_end = min(k_blocks, kb_begin + per_rank);
  const bool has_work = kb_begin < kb_end;   // an empty range contributes zeros
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&p.map_a);
      prefetch_tensormap(p.b_strips == BN / 32 ? &p.map_b_strips : &p.map_b);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&sm.empty[stage], phase ^ 1u, kSiteUmmaEmpty)) break;
        uint8_t* a_dst = sm.stages + static_cast<size_t>(stage) * stage_bytes<BN>();
        uint8_t* b_dst = a_dst + kASlabBytes;
        mbar_expect_tx(&sm.full[stage], stage_bytes<BN>());
        tma_load_2d(a_dst, &p.map_a, &sm.full[stage], kb * kStageK, tm * kTileM);
        if (p.b_strips == BN / 32) {
          tma_load_3d(b_dst, &p.map_b_strips, &sm.full[stage], 0, kb * kStageK, tn * (BN / 32));
        } else {
#pragma unroll
          for (int j = 0; j < BN / 32; ++j) {
            tma_load_2d(b_dst + j * kBBoxBytes, &p.map_b, &sm.full[stage], tn * BN + j * 32, kb * kStageK);
          }
        }
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      int stage = 0;
      uint32_t phase = 0;
      bool fed = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&sm.full[stage], phase, kSiteUmmaFull)) { fed = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t a_addr = smem_u32(sm.stages + static_cast<size_t>(stage) * stage_bytes<BN>());
        issue_stage_mmas<BN>(tmem_base, a_addr, a_addr + kASlabBytes, kb > kb_begin ? 1u : 0u);
        umma_commit(&sm.empty[stage]);
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
      if (fed) umma_commit(&sm.acc_full[0]);
    }
  } else if (has_work) {
    ok = mbar_wait(&sm.acc_full[0], 0, kSiteUmmaAccFull);
    tcgen05_fence_after_sync();
  }

  B200_PROBE(p, 2);
  // 1. Every CTA of the cluster is past its main loop.
  tcgen05_fence_before_sync();
  cluster.sync();
  tcgen05_fence_after_sync();

  B200_PROBE(p, 3);
  // Exchange buffer of a CTA: float4 elements [source rank][column quad of its W columns][row]. Rows are
  // innermost so that the 32 lanes of a warp (32 rows) touch 512 contiguous bytes: no bank conflicts
  // on either side.
  float4* exchange = reinterpret_cast<float4*>(sm.stages);
  const int width = BN / ranks;                            // W: 128, 64, 32 or 16 columns per CTA
  const int quads = width / 4;
  const int quarter = warp & 3;
  const int row_in_tile = quarter * 32 + lane;
  const bool warp_rows = tm * kTileM + quarter * 32 < p.m;   // any row of this warp inside the matrix
  const int quads_log2 = 31 - __clz(quads);
  if (warp >= 2 && warp_rows) {
    // 2. Send this CTA's partial row, W columns to each CTA.
    send_partial_row<BN>(cluster, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16), has_work && ok, exchange,
                         rank, quads_log2, 1, 0, row_in_tile);
  }
  B200_PROBE(p, 4);
  tcgen05_fence_before_sync();
  cluster.sync();
  B200_PROBE(p, 5);

  // 3. Add the partials of this CTA's columns in rank order and finish them.
  exchange_finish<kAct>(epilogue_args(p), exchange, ranks, quads_log2, tm * kTileM, tn * BN + rank * width, threadIdx.x, kTmaThreads);

  B200_PROBE(p, 6);
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<BN>(tmem_base);
  }
}

// ---------------------------------------- TMA, operand-swapped kernel for few rows
// Up to 64 rows (decode-like shapes): computing D^T = B^T * A^T puts the long
// dimension N on the 128 rows of the MMA and the few rows of A on its N side, so
// an instruction is 128 x NM x 8 with NM = 16 or 64 instead of 128 x 128 x 8 with
// most rows zero. What the tensor pipe reads from shared memory per K block drops
// from 32 KiB to 16 KiB + NM * 128 B, and that, not the arithmetic, is what the
// K-block time of the 128 x 128 form consists of.
//   MMA operand A = B^T: M-major, i.e. exactly the B slab of the other kernels
//     (32-column boxes of 32 K rows, 128-byte swizzle in 32-byte granules).
//   MMA operand B = A^T: K-major, i.e. the A slab of the other kernels with NM
//     rows (8-row groups 1024 bytes apart, 128-byte swizzle).
// The accumulator holds D^T: TMEM lane = column n of the tile, TMEM column = row
// m, so an epilogue thread owns one output column and a warp writes 32 adjacent
// floats of a row of D. A cluster of 1/2/4/8 CTAs splits K as in the split-K
// kernel; CTA r finishes the 128 / cluster columns it owns.
constexpr int kSwapTileN = 128;   // columns of D per CTA (the M side of the MMA)

// One 32-wide K sub-block: the B slab and NM rows of A.
template <int NM>
__host__ __device__ constexpr uint32_t swap_sub_bytes() {
  return (kSwapTileN / 32) * kBBoxBytes + NM * kStageK * 4;
}

// A pipeline stage holds KSUB sub-blocks: the small MMAs of this kernel (54 cycles each in
// isolation) are cheap next to the 380 cycles of a stage's barrier wait and commit.
template <int NM, int KSUB>
__host__ __device__ constexpr uint32_t swap_stage_bytes() {
  return KSUB * swap_sub_bytes<NM>();
}

template <int NM, int STAGES, int KSUB>
__host__ __device__ constexpr size_t swap_smem_bytes() {
  return static_cast<size_t>(STAGES) * swap_stage_bytes<NM, KSUB>() + 1024 + 256;
}

template <int NM, int STAGES, int KSUB, int kAct>
__global__ void __launch_bounds__(kTmaThreads, 1) umma_swap_kernel(const __grid_constant__ UmmaParams p) {
  static_assert(NM % 16 == 0 && NM >= 16 && NM <= 64, "rows of A per tile");
  static_assert(static_cast<size_t>(STAGES) * swap_stage_bytes<NM, KSUB>() >= sizeof(float) * NM * kSwapTileN,
                "the idle operand ring must hold one exchanged tile");
  constexpr uint32_t kTmemCols = NM < 32 ? 32 : NM;
  cg::cluster_group cluster = cg::this_cluster();
  const int ranks = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(STAGES) * swap_stage_bytes<NM, KSUB>());
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_full + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_PROBE(p, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  B200_PROBE(p, 1);

  // Tiles: blocks of NM rows of A by 128 columns of B; row blocks innermost.
  const int tiles_m = (p.m + NM - 1) / NM;
  const int tile = static_cast<int>(blockIdx.x) / ranks;
  const int m0 = (tile % tiles_m) * NM, n0 = (tile / tiles_m) * kSwapTileN;
  const int k_blocks = (p.k + KSUB * kStageK - 1) / (KSUB * kStageK);   // stages; K past the end reads as zeros
  const int per_rank = (k_blocks + ranks - 1) / ranks;
  const int kb_begin = min(k_blocks, rank * per_rank);
  const int kb_end = min(k_blocks, kb_begin + per_rank);
  const bool has_work = kb_begin < kb_end;   // an empty K range contributes zeros
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&p.map_a);
      prefetch_tensormap(p.b_strips == kSwapTileN / 32 ? &p.map_b_strips : &p.map_b);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, kSiteUmmaEmpty)) break;
        mbar_expect_tx(&full[stage], swap_stage_bytes<NM, KSUB>());
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          const int k0 = (kb * KSUB + sub) * kStageK;
          uint8_t* b_dst = stages + static_cast<size_t>(stage) * swap_stage_bytes<NM, KSUB>() + sub * swap_sub_bytes<NM>();
          uint8_t* a_dst = b_dst + (kSwapTileN / 32) * kBBoxBytes;                // B slab first, then NM rows of A
          tma_load_2d(a_dst, &p.map_a, &full[stage], k0, m0);
          if (p.b_strips == kSwapTileN / 32) {
            tma_load_3d(b_dst, &p.map_b_strips, &full[stage], 0, k0, n0 / 32);
          } else {
#pragma unroll
            for (int j = 0; j < kSwapTileN / 32; ++j) {
              tma_load_2d(b_dst + j * kBBoxBytes, &p.map_b, &full[stage], n0 + j * 32, k0);
            }
          }
        }
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      // M = 128 (columns of D), N = NM (rows of D); operand A M-major, operand B K-major.
      constexpr uint32_t idesc = umma_idesc_tf32(kSwapTileN, NM, /*a_mn_major=*/true, /*b_mn_major=*/false);
      int stage = 0;
      uint32_t phase = 0;
      bool fed = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&full[stage], phase, kSiteUmmaFull)) { fed = false; break; }
        tcgen05_fence_after_sync();
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          const uint32_t b_addr =
              smem_u32(stages + static_cast<size_t>(stage) * swap_stage_bytes<NM, KSUB>() + sub * swap_sub_bytes<NM>());
          const uint32_t a_addr = b_addr + (kSwapTileN / 32) * kBBoxBytes;
#pragma unroll
          for (int j = 0; j < kStageK / kInstK; ++j) {
            const uint64_t desc_mma_a = umma_smem_desc(b_addr + j * (kInstK * 128), kBBoxBytes, 512, kUmmaSwizzle128B32BAtom);
            const uint64_t desc_mma_b = umma_smem_desc(a_addr + j * (kInstK * 4), 16, 1024, kUmmaSwizzle128B);
            umma_tf32(tmem_base, desc_mma_a, desc_mma_b, idesc, (kb > kb_begin || sub > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty[stage]);
        if (++stage == STAGES) stage = 0, phase ^= 1u;
      }
      if (fed) umma_commit(&acc_full[0]);
    }
  } else if (has_work) {
    ok = mbar_wait(&acc_full[0], 0, kSiteUmmaAccFull);
    tcgen05_fence_after_sync();
  }

  B200_PROBE(p, 2);
  // 1. Every CTA of the cluster is past its main loop: the rings are idle.
  tcgen05_fence_before_sync();
  cluster.sync();
  tcgen05_fence_after_sync();

  B200_PROBE(p, 3);
  // Exchange buffer of a CTA: floats [source rank][row m][column of its share]; a thread owns one
  // column n of the tile, so all its values go to the one CTA that owns that column.
  float* exchange = reinterpret_cast<float*>(stages);
  const int width = kSwapTileN / ranks;                 // columns per CTA
  if (warp >= 2) {
    const int quarter = warp & 3;
    const int n_local = quarter * 32 + lane;
    float* remote = cluster.map_shared_rank(exchange, n_local / width) +
                    static_cast<size_t>(rank) * NM * width + (n_local % width);
#pragma unroll
    for (int chunk = 0; chunk < kTmemCols / 32; ++chunk) {
      uint32_t raw[32];
      if (has_work && ok) {
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 32, raw);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) raw[e] = 0u;
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int m = chunk * 32 + e;
        if (m < NM) remote[m * width] = __uint_as_float(raw[e]);   // columns past NM were never accumulated
      }
    }
  }
  B200_PROBE(p, 4);
  tcgen05_fence_before_sync();
  cluster.sync();
  B200_PROBE(p, 5);

  // 3. Add the partials of this CTA's columns in rank order, apply the epilogue, lanes along a row of D.
  {
    const EpilogueArgs ep = epilogue_args(p);
    const int col_base = n0 + rank * width;
    for (int item = threadIdx.x; item < NM * width; item += kTmaThreads) {
      const int m = item / width, nl = item % width;
      const int row = m0 + m, col = col_base + nl;
      if (row >= ep.m || col >= ep.n) continue;
      float sum = 0.f;
      for (int src = 0; src < ranks; ++src) sum += exchange[(src * NM + m) * width + nl];
      float v = ep.alpha * sum;
      if (ep.beta != 0.f) v = fmaf(ep.beta, __ldg(ep.c + static_cast<int64_t>(row) * ep.ldc + col), v);
      if (ep.bias != nullptr) v += __ldg(ep.bias + col);
      v = activate<kAct>(v);
      const int64_t offset = static_cast<int64_t>(row) * ep.ldd + col;
      ep.d[offset] = v;
      store_peers(ep, offset, v);
    }
  }

  B200_PROBE(p, 6);
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// ------------------------------------------------------- generic loader kernel
// For operands TMA cannot describe (base not 16-byte aligned, leading dimension
// not a multiple of four floats). Persistent like the TMA kernel, same MMA and
// epilogue roles, but the operand ring is filled by eight loader warps with
// predicated scalar loads (zeros outside the matrix):
//   warp 0: TMEM owner + MMA issuer     warps 1-4: epilogue     warps 5-12: loaders
// A loader warp moves one 128-byte row of a slab per instruction: coalesced in
// global memory, and conflict-free in shared memory because the swizzle only
// permutes the 16- or 32-byte granules inside that row. Each thread keeps the
// values of the next stage in registers while it stores the current one, so
// 32 loads per thread are in flight across the wait for a free slot.
constexpr int kLoaderWarps = 8;
constexpr int kGenericThreads = (1 + 4 + kLoaderWarps) * 32;
constexpr int kGenericARows = kTileM / kLoaderWarps;  // A rows per loader warp and stage

// Work split of one stage over the loader warps. Warp lw owns
//   A rows  m = lw + 8 i                      (m % 8 == lw for all of them),
//   B rows  k = lw % 4 + 4 (i % 8) of strips j = (lw / 4) * (BN / 64) + i / 8   (k % 4 == lw % 4),
// so the swizzle term of every store is a per-thread constant and the stores
// are a base address plus immediates.
template <int BN>
struct StageRegs {
  static constexpr int kBRows = kStageK * (BN / 32) / kLoaderWarps;  // 128-byte B rows per loader warp and stage
  float a[kGenericARows];
  float b[kBRows];
};

// Loads this thread's share of stage (m0, n0, k0) into registers.
template <int BN>
__device__ __forceinline__ void load_stage_regs(const UmmaParams& p, StageRegs<BN>& r, int lw, int lane, int m0, int n0,
                                                int k0) {
  constexpr int kStripsPerWarpHalf = BN / 64;
  const float* a_ptr = p.a + static_cast<int64_t>(m0 + lw) * p.lda + k0 + lane;
  const int kb0 = k0 + (lw & 3), nb0 = n0 + (lw >> 2) * kStripsPerWarpHalf * 32 + lane;
  const float* b_ptr = p.b + static_cast<int64_t>(kb0) * p.ldb + nb0;
  const int64_t a_step = static_cast<int64_t>(kLoaderWarps) * p.lda, b_step = 4 * p.ldb;
  if (m0 + kTileM <= p.m && n0 + BN <= p.n && k0 + kStageK <= p.k) {  // interior stage: no predicates
#pragma unroll
    for (int i = 0; i < kGenericARows; ++i) r.a[i] = __ldg(a_ptr + i * a_step);
#pragma unroll
    for (int i = 0; i < StageRegs<BN>::kBRows; ++i) r.b[i] = __ldg(b_ptr + (i & 7) * b_step + (i >> 3) * 32);
  } else {
    const bool k_ok = k0 + lane < p.k;
#pragma unroll
    for (int i = 0; i < kGenericARows; ++i) {
      r.a[i] = (k_ok && m0 + lw + kLoaderWarps * i < p.m) ? __ldg(a_ptr + i * a_step) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < StageRegs<BN>::kBRows; ++i) {
      const bool ok = kb0 + 4 * (i & 7) < p.k && nb0 + (i >> 3) * 32 < p.n;
      r.b[i] = ok ? __ldg(b_ptr + (i & 7) * b_step + (i >> 3) * 32) : 0.f;
    }
  }
}

// Stores them into the swizzled slabs.
//   A: element (m, k) at m * 128 + ((k / 4) ^ (m % 8)) * 16 + (k % 4) * 4.
//   B: box j = n / 32; element (k, n) at j * 4096 + k * 128 + (((n % 32) / 8) ^ (k % 4)) * 32 + (n % 8) * 4.
template <int BN>
__device__ __forceinline__ void store_stage_regs(const StageRegs<BN>& r, uint8_t* a_dst, uint8_t* b_dst, int lw, int lane) {
  constexpr int kStripsPerWarpHalf = BN / 64;
  float* a_base = reinterpret_cast<float*>(a_dst + lw * 128 + (((lane >> 2) ^ lw) << 4) + ((lane & 3) << 2));
#pragma unroll
  for (int i = 0; i < kGenericARows; ++i) a_base[i * (kLoaderWarps * 128 / 4)] = r.a[i];
  float* b_base = reinterpret_cast<float*>(b_dst + (lw >> 2) * kStripsPerWarpHalf * kBBoxBytes + (lw & 3) * 128 +
                                           (((lane >> 3) ^ (lw & 3)) << 5) + ((lane & 7) << 2));
#pragma unroll
  for (int i = 0; i < StageRegs<BN>::kBRows; ++i) b_base[(i >> 3) * (kBBoxBytes / 4) + (i & 7) * (4 * 128 / 4)] = r.b[i];
}

// Position of a loader in the (tile, k block) sequence of its CTA.
struct LoaderCursor {
  int tile, kb, tm, tn;
  __device__ __forceinline__ bool valid(int tiles) const { return tile < tiles; }
  __device__ __forceinline__ void advance(int tiles, int tiles_m, int tiles_n, int k_blocks) {
    if (++kb == k_blocks) {
      kb = 0;
      tile += gridDim.x;
      if (tile < tiles) tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
    }
  }
};

template <int BN, int STAGES, int kAct>
__global__ void __launch_bounds__(kGenericThreads, 1) umma_generic_kernel(const __grid_constant__ UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemCarve sm = carve<BN, STAGES>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], kLoaderWarps);  // one arrive per loader warp
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], 1);
      mbar_init(&sm.acc_empty[b], 4);
    }
    mbar_init_fence();
  }
  if (warp == 0) {
    tmem_alloc<tmem_columns<BN>()>(sm.tmem_ptr);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;

  const int tiles_m = (p.m + kTileM - 1) / kTileM;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  const int k_blocks = (p.k + kStageK - 1) / kStageK;

  if (warp == 0) {
    if (lane == 0) mma_role<BN, STAGES>(sm, tmem_base, tiles, k_blocks);
  } else if (warp <= 4) {
    epilogue_role<BN, kAct, false>(p, sm, tmem_base, warp & 3, lane, tiles, tiles_m, tiles_n);   // 416 threads: no room for two register sets
  } else {
    const int lw = warp - 5;
    LoaderCursor cursor{static_cast<int>(blockIdx.x), 0, 0, 0};  // the next stage to load
    if (cursor.valid(tiles)) tile_coords(cursor.tile, tiles_m, tiles_n, &cursor.tm, &cursor.tn);
    int stage = 0;
    uint32_t phase = 0;
    auto load = [&](StageRegs<BN>& r) {
      const bool have = cursor.valid(tiles);
      if (have) {
        load_stage_regs<BN>(p, r, lw, lane, cursor.tm * kTileM, cursor.tn * BN, cursor.kb * kStageK);
        cursor.advance(tiles, tiles_m, tiles_n, k_blocks);
      }
      return have;
    };
    auto commit = [&](const StageRegs<BN>& r) {
      if (!mbar_wait(&sm.empty[stage], phase ^ 1u, kSiteUmmaEmpty)) return false;
      uint8_t* a_dst = sm.stages + static_cast<size_t>(stage) * stage_bytes<BN>();
      store_stage_regs<BN>(r, a_dst, a_dst + kASlabBytes, lw, lane);
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the MMA unit
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.full[stage]);
      if (++stage == STAGES) stage = 0, phase ^= 1u;
      return true;
    };
    // Two register sets alternate, written out rather than copied, so that the
    // loads of one stage stay in flight while the other is being stored.
    StageRegs<BN> r0, r1;
    bool have0 = load(r0);
    while (have0) {
      const bool have1 = load(r1);
      if (!commit(r0)) break;
      if (!have1) break;
      have0 = load(r0);
      if (!commit(r1)) break;
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after_sync();
    tmem_dealloc<tmem_columns<BN>()>(tmem_base);
  }
}

// ------------------------------------------------------------------ launchers

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
}

template <int BN, int STAGES, int kAct>
int launch_tma(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  // Two sub-blocks per stage where the ring has room for at least two such stages and the tile is
  // not already bound by what an SM can pull from L2 (the 128 x 256 tile is).
  constexpr int KSUB = (BN <= 128 && STAGES % 2 == 0 && STAGES >= 4) ? 2 : 1;
  auto kernel = umma_tma_kernel<BN, STAGES, kAct, KSUB>;
  constexpr size_t smem = smem_bytes<BN, STAGES>();
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
    return B200_ERR_LAUNCH_FAILED;
  }
  // The staging area of the fused all-gather is only asked for when there are peers: a plain GEMM
  // keeps the larger L1 for its epilogue's source reads.
  const size_t launch_smem = smem - (peers.count > 0 ? 0 : kPeerStageBytes);
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  // One copy per B slab when the columns split into whole 32-wide strips.
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, BN / 32,
                                                        Swizzle::k128BAtom32B))
                   ? BN / 32
                   : 0;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kernel<<<grid, kTmaThreads, launch_smem, stream>>>(p);
  return launch_status();
}

template <int STAGES, int kAct>
int launch_pair(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  constexpr int KSUB = 2;                       // 64 floats of K per stage
  static_assert(STAGES % KSUB == 0, "the registry states the ring depth in 32-wide K blocks");
  auto kernel = umma_pair_kernel<STAGES / KSUB, KSUB, kAct>;
  constexpr size_t smem = pair_smem_bytes<STAGES / KSUB, KSUB>();
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
    return B200_ERR_LAUNCH_FAILED;
  }
  const size_t launch_smem = smem - (peers.count > 0 ? 0 : kPeerStageBytes);
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK,
                                                        kPairN / 2 / 32, Swizzle::k128BAtom32B))
                   ? kPairN / 2 / 32
                   : 0;
  const int sms = sm_count();
  if (sms < 2) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + 2 * kTileM - 1) / (2 * kTileM)) * ((q.n + kPairN - 1) / kPairN);
  const int64_t all_pairs = sms / 2;
  // A last round that occupies at most half the pairs is run as 256 x 128 half tiles on twice as
  // many pairs: a half tile streams 24 instead of 32 KiB per K block and CTA and takes about 0.6 of
  // a whole tile's time (4096^3: 34 left-over tiles become 68 halves on 74 pairs). A problem with
  // no more tiles than half the pairs is such a last round from the start.
  const int64_t remainder = tiles % all_pairs;
  p.pair_full_tiles = static_cast<int>((remainder != 0 && 2 * remainder <= all_pairs) ? tiles - remainder : tiles);
  const int64_t items = p.pair_full_tiles + 2 * (tiles - p.pair_full_tiles);
  const int64_t pairs = items < all_pairs ? items : all_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(kTmaThreads);
  cfg.dynamicSmemBytes = launch_smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  return launch_status();
}

// Most clusters of `cluster_size` CTAs of the split-K kernel that the device keeps resident at once
// (cached per device; clusters of eight fit far fewer CTAs than the SM count suggests).
int splitk_max_clusters(int cluster_size) {
  static std::atomic<int> cache[64][4];   // [device][log2 cluster size], 0 = not asked yet
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  const int slot = cluster_size == 1 ? 0 : cluster_size == 2 ? 1 : cluster_size == 4 ? 2 : 3;
  const int cached = cache[device][slot].load(std::memory_order_relaxed);
  if (cached != 0) return cached;
  auto kernel = umma_splitk_kernel<3, B200_EPILOGUE_LINEAR>;   // the activation does not change the footprint
  constexpr size_t smem = smem_bytes<kSplitN, 3>() - kPeerStageBytes;   // no staging: two CTAs fit an SM
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(cluster_size) * 64);
  cfg.blockDim = dim3(kTmaThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(cluster_size);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) clusters = 0;
  const int result = clusters > 0 ? clusters : -1;   // concurrent first calls compute the same value
  cache[device][slot].store(result, std::memory_order_relaxed);
  return result;
}

// Cluster size of the split-K kernel, from a cost model fitted to phase timings of the kernel on a
// B200 (microseconds): a K block costs 0.34 with one CTA per SM and 0.53 per CTA with two (the
// four 128 x 128 x 8 MMAs of a block take that long however few bytes the block loads: with 16 of
// 128 rows present it is still 0.29, and a six-stage ring instead of three changes nothing, so it
// is the SM's MMA rate at this tile shape, not memory, that a second CTA has to share); barriers,
// exchange and the finishing pass cost 4.5 / 6.0 / 7.2 for clusters of 2 / 4 / 8 (half as much again when
// two CTAs share an SM). A candidate must keep
// two K blocks per range and fit the device in one wave (two CTAs per SM: twice the cluster count the
// occupancy query reports for one). `estimate_us` receives the modelled time of the choice.
int splitk_ranks(const b200_gemm_problem& q, int sms, float* estimate_us = nullptr) {
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + kSplitN - 1) / kSplitN);
  const int k_blocks = (q.k + kStageK - 1) / kStageK;
  constexpr float kExchangeUs[4] = {4.7f, 4.5f, 6.0f, 7.2f};
  int best = 1;
  float best_us = 1e30f;
  for (int log2r = 0; log2r < 4; ++log2r) {
    const int ranks = 1 << log2r;
    const int64_t ctas = tiles * ranks;
    if (ctas > 2LL * sms) break;
    if (ranks > 1 && (k_blocks / ranks < 2 || tiles > 2LL * splitk_max_clusters(ranks))) break;
    const bool shared_sm = ctas > sms;   // two CTAs per SM also share its exchange and store bandwidth
    const float us = static_cast<float>((k_blocks + ranks - 1) / ranks) * (shared_sm ? 0.53f : 0.34f) +
                     kExchangeUs[log2r] * (shared_sm ? 1.5f : 1.0f);
    if (us < best_us) best_us = us, best = ranks;
  }
  if (estimate_us != nullptr) *estimate_us = best_us;
  return best;
}

template <int STAGES, int kAct>
int launch_splitk(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  auto kernel = umma_splitk_kernel<STAGES, kAct>;
  constexpr size_t smem = smem_bytes<kSplitN, STAGES>() - kPeerStageBytes;   // its finishing pass needs no staging
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
    return B200_ERR_LAUNCH_FAILED;
  }
  UmmaParams p;
  fill_common(&p, q, peers);
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, kTileM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, kSplitN / 32,
                                                        Swizzle::k128BAtom32B))
                   ? kSplitN / 32
                   : 0;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int ranks = splitk_ranks(q, sms);
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + kSplitN - 1) / kSplitN);
  if (tiles * ranks > 0x7fffffffLL) return B200_ERR_INVALID_PROBLEM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * ranks));
  cfg.blockDim = dim3(kTmaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(ranks);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  return launch_status();
}

// Cluster size of the operand-swapped kernel: as many K ranges as keep every cluster resident at
// once (one CTA per SM) with at least two pipeline stages each.
int swap_ranks(int64_t tiles, int k_stages, int sms) {
  int ranks = 1;
  while (ranks < 8 && tiles * (ranks * 2) <= sms && k_stages / (ranks * 2) >= 2 &&
         tiles <= splitk_max_clusters(ranks * 2)) {
    ranks *= 2;
  }
  return ranks;
}

template <int NM, int kAct>
int run_swap(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  // About 144 KiB of ring either way: 2 stages x 4 sub-blocks of 18 KiB, or 3 x 2 of 24 KiB.
  constexpr int KSUB = NM <= 16 ? 4 : 2, STAGES = NM <= 16 ? 2 : 3;
  auto kernel = umma_swap_kernel<NM, STAGES, KSUB, kAct>;
  constexpr size_t smem = swap_smem_bytes<NM, STAGES, KSUB>();
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
    return B200_ERR_LAUNCH_FAILED;
  }
  UmmaParams p;
  fill_common(&p, q, peers);
  // A: boxes of NM rows x 32 floats of K; B as in the other kernels.
  if (!make_tensor_map_2d(&p.map_a, q.a, q.m, q.k, q.lda, NM, kStageK, Swizzle::k128B) ||
      !make_tensor_map_2d(&p.map_b, q.b, q.k, q.n, q.ldb, kStageK, 32, Swizzle::k128BAtom32B)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  p.b_strips = (q.n % 32 == 0 && make_tensor_map_strips(&p.map_b_strips, q.b, q.k, q.n, q.ldb, kStageK, kSwapTileN / 32,
                                                        Swizzle::k128BAtom32B))
                   ? kSwapTileN / 32
                   : 0;
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + NM - 1) / NM) * ((q.n + kSwapTileN - 1) / kSwapTileN);
  const int ranks = swap_ranks(tiles, (q.k + KSUB * kStageK - 1) / (KSUB * kStageK), sms);
  if (tiles * ranks > 0x7fffffffLL) return B200_ERR_INVALID_PROBLEM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * ranks));
  cfg.blockDim = dim3(kTmaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(ranks);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  return launch_status();
}

template <int kAct>
int launch_swap(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return q.m <= 16 ? run_swap<16, kAct>(q, peers, stream) : run_swap<64, kAct>(q, peers, stream);
}

template <int BN, int STAGES, int kAct>
int launch_generic(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  auto kernel = umma_generic_kernel<BN, STAGES, kAct>;
  constexpr size_t smem = smem_bytes<BN, STAGES>();
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
    return B200_ERR_LAUNCH_FAILED;
  }
  const size_t launch_smem = smem - (peers.count > 0 ? 0 : kPeerStageBytes);
  UmmaParams p;
  fill_common(&p, q, peers);
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_INTERNAL;
  const int64_t tiles = static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kernel<<<grid, kGenericThreads, launch_smem, stream>>>(p);
  return launch_status();
}

// ------------------------------------------------------------------- registry

using LaunchFn = int (*)(const b200_gemm_problem&, const PeerOutputs&, cudaStream_t);
// Shape heuristic consulted only by automatic dispatch; a forced kernel runs
// whatever the shape.
using AutoGateFn = bool (*)(const b200_gemm_problem&, int sms);

struct RegistryEntry {
  b200_tf32_kernel_meta meta;
  LaunchFn launch;
  AutoGateFn auto_gate;
};

constexpr b200_tf32_kernel_meta meta(int id, const char* name, const char* alias, int epilogue, int tile_n, int stages,
                                     int alignment) {
  return b200_tf32_kernel_meta{id,     name,       alias,     epilogue,  kTileM,    tile_n, kStageK,
                               kTileM, tile_n,     kInstK,    stages,    alignment, alignment, alignment, 0};
}

// A CTA pair: 256 x 256 tile and a 256 x 256 x 8 instruction across two CTAs.
constexpr b200_tf32_kernel_meta meta_pair(int id, const char* name, const char* alias, int epilogue, int stages) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, 2 * kTileM, kPairN, kStageK, 2 * kTileM, kPairN, kInstK,
                               stages, 4, 4, 4, 0};
}

// One 128 x 128 tile per cluster, K split over the cluster's CTAs.
constexpr b200_tf32_kernel_meta meta_splitk(int id, const char* name, const char* alias, int epilogue, int stages) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, kTileM, kSplitN, kStageK, kTileM, kSplitN, kInstK, stages, 4, 4, 4, 1};
}

// Few rows on the tensor cores: D^T = B^T A^T, 128 columns of D per CTA, K split over a cluster.
constexpr b200_tf32_kernel_meta meta_swap(int id, const char* name, const char* alias, int epilogue) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, 64, kSwapTileN, kStageK, kSwapTileN, 64, kInstK, 4, 4, 4, 4, 1};
}

// Skinny rows: FP32 FMA stream over B, 16 x 128 outputs per CTA, K split over warps and a cluster.
constexpr b200_tf32_kernel_meta meta_skinny(int id, const char* name, const char* alias, int epilogue) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, kSkinnyMaxRows, 128, 64, kSkinnyMaxRows, 128, 1, 1, 1, 4, 1, 0};
}

int64_t tiles_of(const b200_gemm_problem& q, int tile_n) {
  return static_cast<int64_t>((q.m + kTileM - 1) / kTileM) * ((q.n + tile_n - 1) / tile_n);
}

bool gate_always(const b200_gemm_problem&, int) { return true; }
// 128 x 256 tiles move a third fewer operand bytes per flop through L2, which
// is what bounds this kernel; worth it once they occupy three quarters of the
// SMs (measured at 2048^3: 128 tiles on 148 SMs beat both 128 x 128 tiles and
// 64 CTA pairs).
bool gate_wide(const b200_gemm_problem& q, int sms) { return tiles_of(q, 256) * 4 >= sms * 3; }
// 128 x 64 tiles when 128-wide ones would leave more than half the SMs idle.
// CTA pairs (256 x 256 per pair) when they fill at least one round of pairs.
// (Half tiles filling one round, e.g. 1536^3 with 72 halves on 74 pairs, measured level with the
// 128 x 128 tile kernel, 21.7 against 20.6 us, and stay a matter of the forced "pair" entry.)
bool gate_pair(const b200_gemm_problem& q, int sms) {
  const int64_t tiles = static_cast<int64_t>((q.m + 255) / 256) * ((q.n + 255) / 256);
  return tiles >= sms / 2;
}
// Up to four rows the FP32 stream over B is the fastest entry (1 x 4096 x 4096:
// 8.0 us against 17.1 us for the split-K tensor-core tile); from eight rows on
// its FMA work per byte of B exceeds what hides behind the memory stream and the
// tensor-core split-K entry takes over (16 x 4096 x 4096: 22.1 vs 14.7 us).
bool gate_skinny(const b200_gemm_problem& q, int) { return q.m <= 4; }
// Split K when the model above predicts a shorter run than the unsplit tile kernels, which stream a
// 32-wide K block in about 0.18 us (128 x 64 tiles, two sub-blocks per stage, when those fit the
// SMs in one round) or 0.29 us (128 x 128) on top of 3.5 us of prologue and epilogue. Measured on a
// B200: 1024 x 1024 x 8192 40.7 us split four ways against 61.0 us unsplit, 64 x 4096 x 4096 17.8
// against 31.7, while 512^3, 1024^3 and 512 x 2048 x 2048 are within 1 us either way.
bool gate_splitk(const b200_gemm_problem& q, int sms) {
  float split_us = 0.f;
  if (splitk_ranks(q, sms, &split_us) < 2) return false;
  const int k_blocks = (q.k + kStageK - 1) / kStageK;
  const float unsplit_us = static_cast<float>(k_blocks) * (tiles_of(q, 64) <= sms ? 0.18f : 0.29f) + 3.5f;
  return split_us + 1.0f < unsplit_us;   // ties go to the simpler kernel (1024^3 with a source: 17.6 vs 16.6 us)
}
// Measured against the split-K tile kernel: ahead up to 16 rows (16 x 8192 x 1024: 11.7 vs 16.5 us,
// 16 x 4096 x 4096: 12.7 vs 16.8, cuBLAS 12.9), level or behind from 32 rows on (64 x 4096 x 4096: 19.7 vs 18.2).
bool gate_swap(const b200_gemm_problem& q, int) { return q.m <= 16; }
bool gate_narrow(const b200_gemm_problem& q, int sms) { return tiles_of(q, 128) * 2 <= sms && q.n > 64; }

// Dispatch order. Entries with ids >= 16 exist only here and are tried first by
// automatic dispatch when their shape gate accepts the problem. The eight
// entries after them carry the ids, alias names and the order of the reference
// registry (csrc/adaptive_gemm/kernel_dispatch.cu:46-103, parse_kernel in
// csrc/adaptive_gemm/adaptive_gemm.cu:61-97): "fast" entries require 4-element
// alignment (here: the TMA loader), "fallback" entries accept anything (here:
// the generic loader). What distinguished the reference's variants (warp
// shape, stage count) maps onto tile width and pipeline depth.
const RegistryEntry kRegistry[] = {
    {meta_skinny(27, "simt16x128splitk", "skinny", B200_EPILOGUE_LINEAR), &launch_skinny, &gate_skinny},
    {meta_skinny(28, "simt16x128splitkRelu", "skinny_relu", B200_EPILOGUE_RELU), &launch_skinny, &gate_skinny},
    {meta_skinny(29, "simt16x128splitkGelu", "skinny_gelu", B200_EPILOGUE_GELU), &launch_skinny, &gate_skinny},
    {meta_swap(36, "umma64x128swap", "swap", B200_EPILOGUE_LINEAR), &launch_swap<B200_EPILOGUE_LINEAR>, &gate_swap},
    {meta_swap(37, "umma64x128swapRelu", "swap_relu", B200_EPILOGUE_RELU), &launch_swap<B200_EPILOGUE_RELU>, &gate_swap},
    {meta_swap(38, "umma64x128swapGelu", "swap_gelu", B200_EPILOGUE_GELU), &launch_swap<B200_EPILOGUE_GELU>, &gate_swap},
    {meta_splitk(30, "umma128x128stage3splitk", "splitk", B200_EPILOGUE_LINEAR, 3), &launch_splitk<3, B200_EPILOGUE_LINEAR>, &gate_splitk},
    {meta_splitk(31, "umma128x128stage3splitkRelu", "splitk_relu", B200_EPILOGUE_RELU, 3), &launch_splitk<3, B200_EPILOGUE_RELU>, &gate_splitk},
    {meta_splitk(32, "umma128x128stage3splitkGelu", "splitk_gelu", B200_EPILOGUE_GELU, 3), &launch_splitk<3, B200_EPILOGUE_GELU>, &gate_splitk},
    {meta_pair(20, "umma256x256stage6pair", "pair", B200_EPILOGUE_LINEAR, 6), &launch_pair<6, B200_EPILOGUE_LINEAR>, &gate_pair},
    {meta_pair(21, "umma256x256stage6pairRelu", "pair_relu", B200_EPILOGUE_RELU, 6), &launch_pair<6, B200_EPILOGUE_RELU>, &gate_pair},
    {meta(16, "umma128x256stage4tma", "wide", B200_EPILOGUE_LINEAR, 256, 4, 4), &launch_tma<256, 4, B200_EPILOGUE_LINEAR>, &gate_wide},
    {meta(17, "umma128x256stage4tmaRelu", "wide_relu", B200_EPILOGUE_RELU, 256, 4, 4), &launch_tma<256, 4, B200_EPILOGUE_RELU>, &gate_wide},
    {meta(18, "umma128x64stage6tma", "narrow", B200_EPILOGUE_LINEAR, 64, 6, 4), &launch_tma<64, 6, B200_EPILOGUE_LINEAR>, &gate_narrow},
    {meta(19, "umma128x64stage6tmaRelu", "narrow_relu", B200_EPILOGUE_RELU, 64, 6, 4), &launch_tma<64, 6, B200_EPILOGUE_RELU>, &gate_narrow},
    {meta_pair(22, "umma256x256stage6pairGelu", "pair_gelu", B200_EPILOGUE_GELU, 6), &launch_pair<6, B200_EPILOGUE_GELU>, &gate_pair},
    {meta(23, "umma128x256stage4tmaGelu", "wide_gelu", B200_EPILOGUE_GELU, 256, 4, 4), &launch_tma<256, 4, B200_EPILOGUE_GELU>, &gate_wide},
    {meta(24, "umma128x64stage6tmaGelu", "narrow_gelu", B200_EPILOGUE_GELU, 64, 6, 4), &launch_tma<64, 6, B200_EPILOGUE_GELU>, &gate_narrow},
    {meta(2, "umma128x128stage4tma", "fast", B200_EPILOGUE_LINEAR, 128, 4, 4), &launch_tma<128, 4, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(3, "umma128x128stage4generic", "fallback", B200_EPILOGUE_LINEAR, 128, 4, 1), &launch_generic<128, 4, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(4, "umma128x64stage4tma", "fast_mwarp", B200_EPILOGUE_LINEAR, 64, 4, 4), &launch_tma<64, 4, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(5, "umma128x64stage4generic", "fallback_mwarp", B200_EPILOGUE_LINEAR, 64, 4, 1), &launch_generic<64, 4, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(6, "umma128x128stage3tma", "fast_stage3", B200_EPILOGUE_LINEAR, 128, 3, 4), &launch_tma<128, 3, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(7, "umma128x128stage2tma", "fast_stage2", B200_EPILOGUE_LINEAR, 128, 2, 4), &launch_tma<128, 2, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(8, "umma128x128stage4tmaRelu", "fast_relu", B200_EPILOGUE_RELU, 128, 4, 4), &launch_tma<128, 4, B200_EPILOGUE_RELU>, &gate_always},
    {meta(9, "umma128x128stage4genericRelu", "fallback_relu", B200_EPILOGUE_RELU, 128, 4, 1), &launch_generic<128, 4, B200_EPILOGUE_RELU>, &gate_always},
    // GELU has no entry in the reference registry (the epilogue is parsed but refused there).
    {meta(25, "umma128x128stage4tmaGelu", "fast_gelu", B200_EPILOGUE_GELU, 128, 4, 4), &launch_tma<128, 4, B200_EPILOGUE_GELU>, &gate_always},
    {meta(26, "umma128x128stage4genericGelu", "fallback_gelu", B200_EPILOGUE_GELU, 128, 4, 1), &launch_generic<128, 4, B200_EPILOGUE_GELU>, &gate_always},
};
constexpr int kRegistrySize = sizeof(kRegistry) / sizeof(kRegistry[0]);

const RegistryEntry* find_entry(int id) {
  for (const RegistryEntry& e : kRegistry)
    if (e.meta.id == id) return &e;
  return nullptr;
}

bool operand_aligned(const void* ptr, int64_t ld, int alignment_elements) {
  if (alignment_elements <= 1) return true;
  return reinterpret_cast<uintptr_t>(ptr) % (static_cast<uintptr_t>(alignment_elements) * sizeof(float)) == 0 &&
         ld % alignment_elements == 0;
}

int check_problem(const b200_gemm_problem* q) {
  if (q == nullptr || q->a == nullptr || q->b == nullptr || q->d == nullptr) return B200_ERR_INVALID_ARGUMENT;
  if (q->m <= 0 || q->n <= 0 || q->k <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (q->lda < q->k || q->ldb < q->n || q->ldd < q->n) return B200_ERR_INVALID_ARGUMENT;
  if (q->beta != 0.f && (q->c == nullptr || q->ldc < q->n)) return B200_ERR_INVALID_ARGUMENT;
  if (q->epilogue != B200_EPILOGUE_LINEAR && q->epilogue != B200_EPILOGUE_RELU && q->epilogue != B200_EPILOGUE_GELU) {
    return B200_ERR_INVALID_ARGUMENT;
  }
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_tf32_registry_size(void) { return b200::kRegistrySize; }

int b200_tf32_registry_entry(int index, b200_tf32_kernel_meta* out) {
  if (index < 0 || index >= b200::kRegistrySize || out == nullptr) return B200_ERR_INVALID_ARGUMENT;
  *out = b200::kRegistry[index].meta;
  return B200_OK;
}

int b200_tf32_kernel_from_name(const char* name) {
  if (name == nullptr) return -1;
  if (std::strcmp(name, "auto") == 0) return B200_TF32_KERNEL_AUTO;
  if (std::strcmp(name, "cublas") == 0) return B200_TF32_KERNEL_CUBLAS;
  // The reference also accepts a capitalised spelling of the two ReLU kernels.
  if (std::strcmp(name, "fast_Relu") == 0) name = "fast_relu";
  if (std::strcmp(name, "fallback_Relu") == 0) name = "fallback_relu";
  for (const b200::RegistryEntry& e : b200::kRegistry) {
    if (std::strcmp(name, e.meta.alias) == 0 || std::strcmp(name, e.meta.name) == 0) return e.meta.id;
  }
  return -1;
}

int b200_tf32_can_implement(int kernel_id, const b200_gemm_problem* q) {
  const b200::RegistryEntry* e = b200::find_entry(kernel_id);
  if (e == nullptr) return B200_ERR_INVALID_ARGUMENT;
  const int basic = b200::check_problem(q);
  if (basic != B200_OK) return basic;
  if (e->meta.epilogue != q->epilogue) return B200_ERR_NOT_SUPPORTED;
  // Without a source the reference aliases C to D (adaptive_gemm.cu:152-154),
  // so the source alignment test degenerates to the destination's.
  const void* c_ptr = q->c != nullptr ? static_cast<const void*>(q->c) : static_cast<const void*>(q->d);
  const int64_t ldc = q->c != nullptr ? q->ldc : q->ldd;
  if (!b200::operand_aligned(q->a, q->lda, e->meta.alignment_a) ||
      !b200::operand_aligned(q->b, q->ldb, e->meta.alignment_b) ||
      !b200::operand_aligned(c_ptr, ldc, e->meta.alignment_c) ||
      !b200::operand_aligned(q->d, q->ldd, e->meta.alignment_c)) {
    return B200_ERR_MISALIGNED_OPERAND;
  }
  return B200_OK;
}

int b200_tf32_gemm_launch(int kernel_id, const b200_gemm_problem* q, b200_stream_t stream) {
  const int status = b200_tf32_can_implement(kernel_id, q);
  if (status != B200_OK) return status;
  b200::PeerOutputs none;
  b200::make_peer_outputs(&none, nullptr, 0);
  return b200::find_entry(kernel_id)->launch(*q, none, static_cast<cudaStream_t>(stream));
}

int b200_tf32_gemm_dispatch_gather(int requested, const b200_gemm_problem* q, float* const* peer_d, int n_peers,
                                   int* chosen, b200_stream_t stream) {
  const int basic = b200::check_problem(q);
  if (basic != B200_OK) return basic;
  b200::PeerOutputs peers;
  if (!b200::make_peer_outputs(&peers, peer_d, n_peers)) return B200_ERR_INVALID_ARGUMENT;
  if (requested == B200_TF32_KERNEL_CUBLAS) return B200_ERR_INVALID_ARGUMENT;  // library baseline lives in the caller
  const int sms = requested == B200_TF32_KERNEL_AUTO ? b200::sm_count() : 0;
  for (const b200::RegistryEntry& e : b200::kRegistry) {
    if (requested != B200_TF32_KERNEL_AUTO && e.meta.id != requested) continue;
    if (requested == B200_TF32_KERNEL_AUTO && !e.auto_gate(*q, sms)) continue;
    int status = b200_tf32_can_implement(e.meta.id, q);
    if (status == B200_OK) status = e.launch(*q, peers, static_cast<cudaStream_t>(stream));
    if (status == B200_OK) {
      if (chosen != nullptr) *chosen = e.meta.id;
      return B200_OK;
    }
    // Only "does not fit this kernel" moves on to the next entry; anything
    // else is reported as is (kernel_dispatch.cu:125-132). An epilogue
    // mismatch is a skipped entry in the reference, not an error.
    if (status != B200_ERR_MISALIGNED_OPERAND && status != B200_ERR_INVALID_PROBLEM &&
        status != B200_ERR_NOT_SUPPORTED) {
      return status;
    }
  }
  return B200_ERR_NOT_SUPPORTED;
}

int b200_tf32_gemm_dispatch(int requested, const b200_gemm_problem* q, int* chosen, b200_stream_t stream) {
  return b200_tf32_gemm_dispatch_gather(requested, q, nullptr, 0, chosen, stream);
}

}  // extern "C"
