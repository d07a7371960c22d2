// Registry, automatic dispatch and C ABI of the TF32 tensor-core GEMM (b200_tf32_*). The kernels
// live in tf32_tile_kernels.cu (single-CTA tiles, TMA or loader warps), tf32_pair_kernel.cu (CTA
// pairs), tf32_cluster_kernels.cu (K split over a cluster; operands swapped for few rows) and
// skinny_gemm.cu (FP32 stream for a few rows); this file only knows their launch functions.
// It stands in for the registry and dispatcher of the reference
// (csrc/adaptive_gemm/kernel_dispatch.cu:13-136, kernel_entry.h:7-61).
#include <cstring>

#include "host_common.h"
#include "tf32_gemm.h"

namespace b200 {

cudaError_t umma_status_read_clear(uint32_t* word) {
  // One status word per kernel translation unit; a set bit in any of them is reported.
  uint32_t tile = 0, pair = 0, cluster = 0;
  cudaError_t rc = tf32_tile_status_read_clear(&tile);
  if (rc == cudaSuccess) rc = tf32_pair_status_read_clear(&pair);
  if (rc == cudaSuccess) rc = tf32_cluster_status_read_clear(&cluster);
  *word = tile | pair | cluster;
  return rc;
}

namespace {

// Tile geometry of the kernels, as the registry records state it.
constexpr int kTileM = 128;       // rows of a single-CTA tile
constexpr int kStageK = 32;       // floats of K per 32-wide block of a pipeline stage
constexpr int kInstK = 8;         // K of one tcgen05.mma kind::tf32
constexpr int kPairN = 256;       // columns of a CTA pair's tile
constexpr int kSplitN = 128;      // columns of the split-K tile
constexpr int kSwapTileN = 128;   // columns of D per CTA of the operand-swapped kernel

template <int BN, int STAGES, int kAct>
int tile_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_tile(BN, STAGES, kAct, q, peers, stream);
}
template <int BN, int kAct>
int generic_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_generic(BN, kAct, q, peers, stream);
}
template <int kAct>
int pair_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_pair(kAct, q, peers, stream);
}
template <int kAct>
int pair_mid_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_pair_mid(kAct, q, peers, stream);
}
template <int kAct>
int splitk_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_splitk(kAct, q, peers, stream);
}
template <int kAct>
int pair_splitk_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_pair_splitk(kAct, q, peers, stream);
}
template <int kAct>
int swap_entry(const b200_gemm_problem& q, const PeerOutputs& peers, cudaStream_t stream) {
  return launch_tf32_swap(kAct, q, peers, stream);
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

// A CTA pair on 256 x 128 tiles (256 x 128 x 8 instructions), two MMA issuers.
constexpr b200_tf32_kernel_meta meta_pair_mid(int id, const char* name, const char* alias, int epilogue) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, 2 * kTileM, 128, kStageK, 2 * kTileM, 128, kInstK, 8, 4, 4, 4, 0};
}

// One 128 x 128 tile per cluster, K split over the cluster's CTAs.
constexpr b200_tf32_kernel_meta meta_splitk(int id, const char* name, const char* alias, int epilogue, int stages) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, kTileM, kSplitN, kStageK, kTileM, kSplitN, kInstK, stages, 4, 4, 4, 1};
}

// One 256 x 128 tile per cluster of CTA pairs, K split over the pairs.
constexpr b200_tf32_kernel_meta meta_pair_splitk(int id, const char* name, const char* alias, int epilogue) {
  return b200_tf32_kernel_meta{id, name, alias, epilogue, 2 * kTileM, kSplitN, kStageK, 2 * kTileM, kSplitN, kInstK, 8, 4, 4, 4, 1};
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
// 128 x 256 tiles move a third fewer operand bytes per flop through L2 and take about 1.45 times as
// long as a 128 x 128 tile; they pay when they save a round: measured at 2048^3 (128 tiles in one
// round against 256 in two: 27.9 against 34.2 us, and ahead of 64 CTA pairs) and at
// 1792 x 1792 x 2048 (98 tiles in one round against 196 in two: 27.2 against 33.7 us).
bool gate_wide(const b200_gemm_problem& q, int sms) {
  const int64_t rounds_128 = (tiles_of(q, 128) + sms - 1) / sms, rounds_256 = (tiles_of(q, 256) + sms - 1) / sms;
  return 100 * rounds_128 > 145 * rounds_256;
}
// Tile widths between the reference's: at sizes that run in one round a CTA's time is set by the
// operand bytes it takes in per K block (16 KiB of A + 128 bytes per column of B), so of the widths
// that fit one round the narrowest wins (128 x 32: 20 KiB, 64: 24, 96: 28, 128: 32, 160: 36, 192: 40,
// 224: 44, 256: 48). 128 x 32 / 128 x 64 / cuBLASLt fused: 256^3 4.4 / 4.8 / 5.1-5.4 us, 512^3 5.5 / 6.0 / 5.7-5.8,
// 640^3 6.1 / 6.7 / 6.4, 768^3 6.75 / 7.3 / 7.5.
// Graph-timed with a source and ReLU, 128 x 192 / 128 x 256 / CTA pairs / cuBLASLt fused: 1792^3
// 22.1 / 25.0 / 26.2 / 24.1 us, 1664^3 21.2 / 23.7 / 24.9 / 23.2, 1536 x 2048 x 2048 24.3 / 27.5 / 28.6 / 26.3,
// 1280 x 2688 x 1024 15.7 / 17.7 / 18.9 / 17.7, 1792 x 1792 x 4096 46.7 / 50.0 / 50.0 / 46.6 (tried before
// the CTA pairs for that reason).
int narrowest_one_round_width(const b200_gemm_problem& q, int sms) {
  for (int width = 32; width <= 256; width += 32)
    if (tiles_of(q, width) <= sms) return width;
  return 0;
}
bool gate_width32(const b200_gemm_problem& q, int sms) { return narrowest_one_round_width(q, sms) == 32; }
bool gate_width96(const b200_gemm_problem& q, int sms) { return narrowest_one_round_width(q, sms) == 96; }
bool gate_width160(const b200_gemm_problem& q, int sms) { return narrowest_one_round_width(q, sms) == 160; }
bool gate_medium(const b200_gemm_problem& q, int sms) { return narrowest_one_round_width(q, sms) == 192; }
bool gate_width224(const b200_gemm_problem& q, int sms) { return narrowest_one_round_width(q, sms) == 224; }
// CTA pairs (256 x 256 per pair) when they fill at least one round of pairs.
// (Half tiles filling one round, e.g. 1536^3 with 72 halves on 74 pairs, measured level with the
// 128 x 128 tile kernel, 21.7 against 20.6 us, and stay a matter of the forced "pair" entry.)
// With K of 4096 or more they are also ahead of the 128 x 256 tile kernel when they fill two thirds
// of one round (the wide tile streams half as many bytes again per flop, and with long K that is
// what counts): 1280 x 2560 x 4096 (50 tiles) 49.1 against 56.5 us, 1792 x 1792 x 8192 (49) 99.6 / 111.2,
// 1024 x 4096 x 4096 (64) 57.8 / 70.5, 2048 x 2048 x 8192 (64) 96.2 / 101.1; at K = 2048 the wide tile
// is level or ahead (1024 x 4096 x 2048 28.0 against 29, 2048^3 27.6 / 29.5).
bool gate_pair(const b200_gemm_problem& q, int sms) {
  const int64_t tiles = static_cast<int64_t>((q.m + 255) / 256) * ((q.n + 255) / 256);
  const int64_t pairs = sms / 2;
  return tiles >= pairs || (q.k >= 4096 && 20 * tiles >= 13 * pairs);
}
// Up to four rows the FP32 stream over B is the fastest entry (1 x 4096 x 4096:
// 8.0 us against 17.1 us for the split-K tensor-core tile); from eight rows on
// its FMA work per byte of B exceeds what hides behind the memory stream and the
// tensor-core split-K entry takes over (16 x 4096 x 4096: 22.1 vs 14.7 us).
bool gate_skinny(const b200_gemm_problem& q, int) { return q.m <= 4; }
// Split K when the split-K kernel's model predicts a shorter run than the unsplit tile kernels. Those
// take, graph-timed with a source and ReLU, about 0.136 us per 32-wide K block on top of 5.4 us
// (128 x 64 tiles, when they fit the SMs in one round: 1024 x 1024 x K 9.8 / 14.2 / 22.8 / 41.5 us at
// K = 1024 / 2048 / 4096 / 8192) or 0.22 us on top of 5.2 us (128 x 128: 1536^3 15.8, 512 x 4096 x 4096
// 34.4, 1280 x 1280 x 8192 60.6). Split against unsplit, measured: 1024 x 1024 x 4096 20.5 / 22.8 us,
// 1024 x 1024 x 8192 38.7 / 41.5, 1024 x 1024 x 16384 72.2 / 92.2, 512 x 512 x 2048 10.8 / 13.4,
// 768 x 768 x 4096 20.8 / 22.0, 768 x 768 x 8192 30.8 / 40.5, 64 x 4096 x 4096 15.1 / 22.1; unsplit is
// ahead at 1024^3 (9.8 against 11.5), 1536^3 (15.8 / 18.6), 512 x 4096 x 4096 (34.4 / 40.0), 512^3 and
// 768^3, and level at 1024 x 1024 x 2048, 256 x 4096 x 4096 and 1280 x 1280 x 8192.
bool gate_splitk(const b200_gemm_problem& q, int sms) {
  float split_us = 0.f;
  if (tf32_splitk_plan(q, sms, &split_us) < 2) return false;
  const int k_blocks = (q.k + kStageK - 1) / kStageK;
  const bool narrow = tiles_of(q, 64) <= sms;
  const float unsplit_us = static_cast<float>(k_blocks) * (narrow ? 0.136f : 0.22f) + (narrow ? 5.4f : 5.2f);
  return split_us + 1.0f < unsplit_us;   // near ties go to the simpler kernel
}
// The CTA-pair form of the split (two MMA issuers): when it splits K at all (two ranges or more), all
// its clusters are resident at once, both CTAs of a pair have rows to compute, and either the
// single-CTA split would be chosen (the pair form was ahead of it or level in every such case
// measured) or its own model predicts a shorter run than the unsplit tile kernels. Graph-timed with a
// source and ReLU, pair split / single-CTA split / best unsplit: 1024 x 1024 x 8192 33.3 / 37.4 / 41.5 us,
// 768 x 768 x 4096 18.6 / 20.7 / 22.1, 768 x 768 x 8192 28.2 / 30.8 / 40.5, 256 x 4096 x 4096 19.6 / 23.6 / 22.9,
// 512 x 512 x 2048 10.8 / 13.4 / 13.7, 1024 x 1024 x 16384 62.9 / 68.7 / 92.2; level at 1024 x 1024 x 4096
// (19.8 / 19.6) and 512 x 2048 x 4096 (19.1 / 19.8).
bool gate_pair_splitk(const b200_gemm_problem& q, int sms) {
  if (q.m <= kTileM) return false;
  float pair_us = 0.f;
  int waves = 0;
  if (tf32_pair_splitk_plan(q, &pair_us, &waves) < 2 || waves != 1) return false;
  if (gate_splitk(q, sms)) return true;
  const int k_blocks = (q.k + kStageK - 1) / kStageK;
  const bool narrow = tiles_of(q, 64) <= sms;
  const float unsplit_us = static_cast<float>(k_blocks) * (narrow ? 0.136f : 0.22f) + (narrow ? 5.4f : 5.2f);
  return pair_us + 1.0f < unsplit_us;
}
// CTA pairs on 256 x 128 tiles with two MMA issuers: where the 128 x 128 tile kernel would run one
// round (more than half the SMs, so not the 128 x 64 tile's territory) and K is long enough for the
// quarter fewer operand bytes per flop to outweigh the pair's start-up. Graph-timed with a source and
// ReLU, against the 128 x 128 tile kernel: 1280 x 1280 x 4096 27.4 / 31.4 us, 1280 x 1280 x 8192 53.0 / 60.5,
// 1536 x 1536 x 3072 24.3 / 26.0, 1536 x 1536 x 4096 32.3 / 39.0, 1024 x 2048 x 4096 30.0 / 33.3,
// 512 x 4096 x 4096 32.8 / 33.7, 192 x 6144 x 6144 44.9 / 51.3; at K = 2048 and below the 128 x 128
// tile is level or ahead (1536 x 1536 x 2048 19.0 against 18.7, 1536^3 15.7).
bool gate_pair_mid(const b200_gemm_problem& q, int sms) {
  const int64_t pair_tiles = static_cast<int64_t>((q.m + 2 * kTileM - 1) / (2 * kTileM)) * ((q.n + 127) / 128);
  return q.k >= 2560 && q.m > kTileM && tiles_of(q, 128) * 2 > sms && pair_tiles <= sms / 2;
}
// Measured against the split-K tile kernel: ahead up to 16 rows (16 x 8192 x 1024: 11.7 vs 16.5 us,
// 16 x 4096 x 4096: 12.7 vs 16.8, cuBLAS 12.9), level or behind from 32 rows on (64 x 4096 x 4096: 19.7 vs 18.2).
bool gate_swap(const b200_gemm_problem& q, int) { return q.m <= 16; }
// 128 x 64 tiles when 128-wide ones would leave more than half the SMs idle, or by the one-round rule above.
bool gate_narrow(const b200_gemm_problem& q, int sms) {
  return (tiles_of(q, 128) * 2 <= sms && q.n > 64) || narrowest_one_round_width(q, sms) == 64;
}

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
    {meta_swap(36, "umma64x128swap", "swap", B200_EPILOGUE_LINEAR), &swap_entry<B200_EPILOGUE_LINEAR>, &gate_swap},
    {meta_swap(37, "umma64x128swapRelu", "swap_relu", B200_EPILOGUE_RELU), &swap_entry<B200_EPILOGUE_RELU>, &gate_swap},
    {meta_swap(38, "umma64x128swapGelu", "swap_gelu", B200_EPILOGUE_GELU), &swap_entry<B200_EPILOGUE_GELU>, &gate_swap},
    {meta_pair_splitk(42, "umma256x128pairsplitk", "pair_splitk", B200_EPILOGUE_LINEAR), &pair_splitk_entry<B200_EPILOGUE_LINEAR>, &gate_pair_splitk},
    {meta_pair_splitk(43, "umma256x128pairsplitkRelu", "pair_splitk_relu", B200_EPILOGUE_RELU), &pair_splitk_entry<B200_EPILOGUE_RELU>, &gate_pair_splitk},
    {meta_pair_splitk(44, "umma256x128pairsplitkGelu", "pair_splitk_gelu", B200_EPILOGUE_GELU), &pair_splitk_entry<B200_EPILOGUE_GELU>, &gate_pair_splitk},
    {meta_splitk(30, "umma128x128stage3splitk", "splitk", B200_EPILOGUE_LINEAR, 3), &splitk_entry<B200_EPILOGUE_LINEAR>, &gate_splitk},
    {meta_splitk(31, "umma128x128stage3splitkRelu", "splitk_relu", B200_EPILOGUE_RELU, 3), &splitk_entry<B200_EPILOGUE_RELU>, &gate_splitk},
    {meta_splitk(32, "umma128x128stage3splitkGelu", "splitk_gelu", B200_EPILOGUE_GELU, 3), &splitk_entry<B200_EPILOGUE_GELU>, &gate_splitk},
    {meta_pair_mid(39, "umma256x128stage8pair", "pair_mid", B200_EPILOGUE_LINEAR), &pair_mid_entry<B200_EPILOGUE_LINEAR>, &gate_pair_mid},
    {meta_pair_mid(40, "umma256x128stage8pairRelu", "pair_mid_relu", B200_EPILOGUE_RELU), &pair_mid_entry<B200_EPILOGUE_RELU>, &gate_pair_mid},
    {meta_pair_mid(41, "umma256x128stage8pairGelu", "pair_mid_gelu", B200_EPILOGUE_GELU), &pair_mid_entry<B200_EPILOGUE_GELU>, &gate_pair_mid},
    {meta(57, "umma128x32stage8tma", "width32", B200_EPILOGUE_LINEAR, 32, 8, 4), &tile_entry<32, 8, B200_EPILOGUE_LINEAR>, &gate_width32},
    {meta(58, "umma128x32stage8tmaRelu", "width32_relu", B200_EPILOGUE_RELU, 32, 8, 4), &tile_entry<32, 8, B200_EPILOGUE_RELU>, &gate_width32},
    {meta(59, "umma128x32stage8tmaGelu", "width32_gelu", B200_EPILOGUE_GELU, 32, 8, 4), &tile_entry<32, 8, B200_EPILOGUE_GELU>, &gate_width32},
    {meta(48, "umma128x96stage6tma", "width96", B200_EPILOGUE_LINEAR, 96, 6, 4), &tile_entry<96, 6, B200_EPILOGUE_LINEAR>, &gate_width96},
    {meta(49, "umma128x96stage6tmaRelu", "width96_relu", B200_EPILOGUE_RELU, 96, 6, 4), &tile_entry<96, 6, B200_EPILOGUE_RELU>, &gate_width96},
    {meta(50, "umma128x96stage6tmaGelu", "width96_gelu", B200_EPILOGUE_GELU, 96, 6, 4), &tile_entry<96, 6, B200_EPILOGUE_GELU>, &gate_width96},
    {meta(51, "umma128x160stage5tma", "width160", B200_EPILOGUE_LINEAR, 160, 5, 4), &tile_entry<160, 5, B200_EPILOGUE_LINEAR>, &gate_width160},
    {meta(52, "umma128x160stage5tmaRelu", "width160_relu", B200_EPILOGUE_RELU, 160, 5, 4), &tile_entry<160, 5, B200_EPILOGUE_RELU>, &gate_width160},
    {meta(53, "umma128x160stage5tmaGelu", "width160_gelu", B200_EPILOGUE_GELU, 160, 5, 4), &tile_entry<160, 5, B200_EPILOGUE_GELU>, &gate_width160},
    {meta(54, "umma128x224stage4tma", "width224", B200_EPILOGUE_LINEAR, 224, 4, 4), &tile_entry<224, 4, B200_EPILOGUE_LINEAR>, &gate_width224},
    {meta(55, "umma128x224stage4tmaRelu", "width224_relu", B200_EPILOGUE_RELU, 224, 4, 4), &tile_entry<224, 4, B200_EPILOGUE_RELU>, &gate_width224},
    {meta(56, "umma128x224stage4tmaGelu", "width224_gelu", B200_EPILOGUE_GELU, 224, 4, 4), &tile_entry<224, 4, B200_EPILOGUE_GELU>, &gate_width224},
    {meta(45, "umma128x192stage4tma", "medium", B200_EPILOGUE_LINEAR, 192, 4, 4), &tile_entry<192, 4, B200_EPILOGUE_LINEAR>, &gate_medium},
    {meta(46, "umma128x192stage4tmaRelu", "medium_relu", B200_EPILOGUE_RELU, 192, 4, 4), &tile_entry<192, 4, B200_EPILOGUE_RELU>, &gate_medium},
    {meta(47, "umma128x192stage4tmaGelu", "medium_gelu", B200_EPILOGUE_GELU, 192, 4, 4), &tile_entry<192, 4, B200_EPILOGUE_GELU>, &gate_medium},
    {meta_pair(20, "umma256x256stage6pair", "pair", B200_EPILOGUE_LINEAR, 6), &pair_entry<B200_EPILOGUE_LINEAR>, &gate_pair},
    {meta_pair(21, "umma256x256stage6pairRelu", "pair_relu", B200_EPILOGUE_RELU, 6), &pair_entry<B200_EPILOGUE_RELU>, &gate_pair},
    {meta(16, "umma128x256stage4tma", "wide", B200_EPILOGUE_LINEAR, 256, 4, 4), &tile_entry<256, 4, B200_EPILOGUE_LINEAR>, &gate_wide},
    {meta(17, "umma128x256stage4tmaRelu", "wide_relu", B200_EPILOGUE_RELU, 256, 4, 4), &tile_entry<256, 4, B200_EPILOGUE_RELU>, &gate_wide},
    {meta(18, "umma128x64stage8tma", "narrow", B200_EPILOGUE_LINEAR, 64, 8, 4), &tile_entry<64, 8, B200_EPILOGUE_LINEAR>, &gate_narrow},
    {meta(19, "umma128x64stage8tmaRelu", "narrow_relu", B200_EPILOGUE_RELU, 64, 8, 4), &tile_entry<64, 8, B200_EPILOGUE_RELU>, &gate_narrow},
    {meta_pair(22, "umma256x256stage6pairGelu", "pair_gelu", B200_EPILOGUE_GELU, 6), &pair_entry<B200_EPILOGUE_GELU>, &gate_pair},
    {meta(23, "umma128x256stage4tmaGelu", "wide_gelu", B200_EPILOGUE_GELU, 256, 4, 4), &tile_entry<256, 4, B200_EPILOGUE_GELU>, &gate_wide},
    {meta(24, "umma128x64stage8tmaGelu", "narrow_gelu", B200_EPILOGUE_GELU, 64, 8, 4), &tile_entry<64, 8, B200_EPILOGUE_GELU>, &gate_narrow},
    {meta(2, "umma128x128stage6tma", "fast", B200_EPILOGUE_LINEAR, 128, 6, 4), &tile_entry<128, 6, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(3, "umma128x128stage4generic", "fallback", B200_EPILOGUE_LINEAR, 128, 4, 1), &generic_entry<128, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(4, "umma128x64stage4tma", "fast_mwarp", B200_EPILOGUE_LINEAR, 64, 4, 4), &tile_entry<64, 4, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(5, "umma128x64stage4generic", "fallback_mwarp", B200_EPILOGUE_LINEAR, 64, 4, 1), &generic_entry<64, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(6, "umma128x128stage3tma", "fast_stage3", B200_EPILOGUE_LINEAR, 128, 3, 4), &tile_entry<128, 3, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(7, "umma128x128stage2tma", "fast_stage2", B200_EPILOGUE_LINEAR, 128, 2, 4), &tile_entry<128, 2, B200_EPILOGUE_LINEAR>, &gate_always},
    {meta(8, "umma128x128stage6tmaRelu", "fast_relu", B200_EPILOGUE_RELU, 128, 6, 4), &tile_entry<128, 6, B200_EPILOGUE_RELU>, &gate_always},
    {meta(9, "umma128x128stage4genericRelu", "fallback_relu", B200_EPILOGUE_RELU, 128, 4, 1), &generic_entry<128, B200_EPILOGUE_RELU>, &gate_always},
    // GELU has no entry in the reference registry (the epilogue is parsed but refused there).
    {meta(25, "umma128x128stage6tmaGelu", "fast_gelu", B200_EPILOGUE_GELU, 128, 6, 4), &tile_entry<128, 6, B200_EPILOGUE_GELU>, &gate_always},
    {meta(26, "umma128x128stage4genericGelu", "fallback_gelu", B200_EPILOGUE_GELU, 128, 4, 1), &generic_entry<128, B200_EPILOGUE_GELU>, &gate_always},
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
