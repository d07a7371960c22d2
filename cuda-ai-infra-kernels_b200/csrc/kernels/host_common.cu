// Status strings, device attribute cache, tensor-map construction, the device
// status word and the row-shard planner.
#include "host_common.h"

#include <atomic>
#include <cstring>
#include <mutex>

namespace b200 {

namespace {

constexpr int kMaxDevices = 64;
std::atomic<int> g_sm_count[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  // The driver entry point is resolved through the runtime so that the library
  // does not link libcuda directly.
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Encoded tensor maps, remembered per host thread. A map is a pure function of (base address,
// extents, pitch, box, swizzle, rank): encoding it through the driver costs a few microseconds,
// which a 10-microsecond GEMM launched over and over on the same buffers (a serving loop, a
// benchmark) notices. Direct-mapped, thread-local: no locks, no invalidation needed (a stale entry
// can only be returned for an identical key, for which the encoding is identical).
struct MapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_a, box_b;
  int32_t swizzle, kind;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_a == o.box_a && box_b == o.box_b &&
           swizzle == o.swizzle && kind == o.kind;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapSlots = 64;

MapSlot* map_slot(const MapKey& key) {
  thread_local MapSlot slots[kMapSlots] = {};
  uint64_t h = reinterpret_cast<uintptr_t>(key.base) >> 4;
  h ^= key.rows * 0x9E3779B97F4A7C15ull;
  h ^= (key.cols + (static_cast<uint64_t>(key.box_a) << 32)) * 0xC2B2AE3D27D4EB4Full;
  h ^= (key.ld + (static_cast<uint64_t>(key.box_b) << 40) + (static_cast<uint64_t>(key.kind) << 20) +
        static_cast<uint64_t>(key.swizzle)) * 0x165667B19E3779F9ull;
  h ^= h >> 29;
  return &slots[h % kMapSlots];
}

}  // namespace

int sm_count() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 0;
  int cached = g_sm_count[device].load(std::memory_order_relaxed);
  if (cached > 0) return cached;
  int count = 0;
  if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  g_sm_count[device].store(count, std::memory_order_relaxed);
  return count;
}

bool make_tensor_map_2d(CUtensorMap* out, const float* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols, Swizzle swizzle) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
  if ((ld * sizeof(float)) % 16 != 0 || (box_cols * sizeof(float)) % 16 != 0) return false;
  if (box_rows == 0 || box_cols == 0 || box_rows > 256 || box_cols > 256) return false;
  if (swizzle != Swizzle::kNone && box_cols * sizeof(float) > 128) return false;
  const MapKey key{base, rows, cols, ld, box_rows, box_cols, static_cast<int32_t>(swizzle), 2};
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *out = slot->map;
    return true;
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * sizeof(float)};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
                             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swizzle == Swizzle::k128B          ? CU_TENSOR_MAP_SWIZZLE_128B
                             : swizzle == Swizzle::k128BAtom32B ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                                : CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return false;
  slot->key = key, slot->map = *out, slot->used = true;
  return true;
}

bool make_tensor_map_strips(CUtensorMap* out, const float* base, uint64_t rows, uint64_t cols, uint64_t ld,
                            uint32_t box_rows, uint32_t box_groups, Swizzle swizzle) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (ld * sizeof(float)) % 16 != 0) return false;
  if (cols == 0 || cols % 32 != 0 || box_rows == 0 || box_rows > 256 || box_groups == 0 || box_groups > 256) return false;
  const MapKey key{base, rows, cols, ld, box_rows, box_groups, static_cast<int32_t>(swizzle), 3};
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *out = slot->map;
    return true;
  }
  const cuuint64_t dims[3] = {32, rows, cols / 32};
  const cuuint64_t strides[2] = {ld * sizeof(float), 32 * sizeof(float)};
  const cuuint32_t box[3] = {32, box_rows, box_groups};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box,
                             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swizzle == Swizzle::k128B          ? CU_TENSOR_MAP_SWIZZLE_128B
                             : swizzle == Swizzle::k128BAtom32B ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                                : CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return false;
  slot->key = key, slot->map = *out, slot->used = true;
  return true;
}

}  // namespace b200

extern "C" {

const char* b200_status_string(int status) {
  switch (status) {
    case B200_OK: return "Success";
    case B200_ERR_MISALIGNED_OPERAND: return "Error Misaligned Operand";
    case B200_ERR_INVALID_PROBLEM: return "Error Invalid Problem";
    case B200_ERR_NOT_SUPPORTED: return "Error Not Supported";
    case B200_ERR_INVALID_ARGUMENT: return "Error Invalid Argument";
    case B200_ERR_LAUNCH_FAILED: return "Error Kernel Launch Failed";
    case B200_ERR_DEVICE_TIMEOUT: return "Error Device Wait Timed Out";
    case B200_ERR_INTERNAL: return "Error Internal";
    default: return "Error Unknown Status";
  }
}

const char* b200_build_info(void) {
  return "b200_kernels 0.1 (sm_100a; FP32 SIMT ladder, TF32 tcgen05 GEMM, RMSNorm, softmax)";
}

int b200_device_status_read(uint32_t* host_word, b200_stream_t stream) {
  if (host_word == nullptr) return B200_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaStreamSynchronize(s) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  uint32_t sgemm_word = 0, umma_word = 0, selftest_word = 0;
  if (b200::sgemm_status_read_clear(&sgemm_word) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  if (b200::umma_status_read_clear(&umma_word) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  if (b200::selftest_status_read_clear(&selftest_word) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  uint32_t peer_word = 0;
  if (b200::peer_sync_status_read_clear(&peer_word) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  uint32_t row_word = 0;
  if (b200::rowops_status_read_clear(&row_word) != cudaSuccess) return B200_ERR_LAUNCH_FAILED;
  *host_word = sgemm_word | umma_word | selftest_word | peer_word | row_word;
  return *host_word == 0 ? B200_OK : B200_ERR_DEVICE_TIMEOUT;
}

int b200_shard_rows(int64_t m, int parts, int granule, int64_t* row_begin, int64_t* row_count) {
  if (m < 0 || parts <= 0 || granule <= 0 || row_begin == nullptr || row_count == nullptr) {
    return B200_ERR_INVALID_ARGUMENT;
  }
  // Whole granules are dealt out as evenly as possible, earlier parts first;
  // a ragged remainder (m % granule) goes to the last part that owns rows.
  const int64_t granules = m / granule;
  const int64_t remainder = m % granule;
  const int64_t base = granules / parts;
  const int64_t extra = granules % parts;
  int64_t begin = 0;
  int last_owner = -1;
  for (int p = 0; p < parts; ++p) {
    const int64_t count = (base + (p < extra ? 1 : 0)) * granule;
    row_begin[p] = begin;
    row_count[p] = count;
    if (count > 0) last_owner = p;
    begin += count;
  }
  if (remainder > 0) {
    if (last_owner < 0) last_owner = 0;
    // Later parts own nothing, so extending this one keeps the ranges contiguous.
    row_count[last_owner] += remainder;
    for (int p = last_owner + 1; p < parts; ++p) row_begin[p] = row_begin[last_owner] + row_count[last_owner];
  }
  return B200_OK;
}

}  // extern "C"
