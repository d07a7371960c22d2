/*
 * b200_kernels.h — C ABI of libb200_kernels.so.
 *
 * Hand-written sm_100a kernels for the operator set of the
 * "cuda-ai-infra-kernels" project: the FP32 SIMT GEMM ladder, the TF32
 * tensor-core GEMM with fused LinearCombination / ReLU epilogues and its
 * compatibility registry, and the RMSNorm / softmax row operators.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; nothing in this header depends on PyTorch
 *     or on the CUDA headers (a stream is passed as an opaque pointer that is
 *     bit-identical to cudaStream_t);
 *   - the caller has made the target device current; all pointers are device
 *     pointers on that device unless a parameter says "host";
 *   - work is enqueued on `stream` and the call returns without synchronising;
 *     no entry point allocates or frees device memory, copies to the host or
 *     synchronises, so every launch may be captured in a CUDA graph
 *     (b200_device_status_read is the one exception and says so);
 *   - the return value is a b200_status; nothing throws;
 *   - inputs are never written.
 *
 * Each declaration names the reference interface it stands in for
 * (path:line inside the cuda-ai-infra-kernels source tree).
 */
#ifndef B200_KERNELS_H_
#define B200_KERNELS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b200_stream_t; /* cudaStream_t */

/* ------------------------------------------------------------------ status */

/*
 * Status codes. The adaptive dispatcher of the reference walks its registry
 * and moves on to the next entry only for "misaligned operand" and "invalid
 * problem" (csrc/adaptive_gemm/kernel_dispatch.cu:125-132); the same two
 * codes exist here with the same meaning, and the string forms match
 * cutlassGetStatusString for the three codes the reference can surface
 * (csrc/adaptive_gemm/adaptive_gemm.cu:169-172).
 */
typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_MISALIGNED_OPERAND = 1,
  B200_ERR_INVALID_PROBLEM = 2,
  B200_ERR_NOT_SUPPORTED = 3,
  B200_ERR_INVALID_ARGUMENT = 4,
  B200_ERR_LAUNCH_FAILED = 5,
  B200_ERR_DEVICE_TIMEOUT = 6,
  B200_ERR_INTERNAL = 7
} b200_status;

/* Human-readable form of a status code (never NULL). */
const char* b200_status_string(int status);

/* Library version and the architecture the kernels were compiled for. */
const char* b200_build_info(void);

/*
 * Every device-side wait in this library (mbarrier phases fed by TMA or by
 * tcgen05.commit) is bounded. A kernel whose wait ran out records a non-zero
 * word and returns instead of spinning. This call copies the word of the
 * current device to *host_word and clears it. It synchronises `stream` and is
 * therefore NOT capturable; call it from tests and after failures, not per
 * launch. No reference counterpart (the reference has no device-side waits).
 */
int b200_device_status_read(uint32_t* host_word, b200_stream_t stream);

/*
 * Bits of the status word: which wait gave up.
 */
enum {
  B200_WAIT_SGEMM_FULL = 1 << 0,    /* FP32 pipeline: consumer waiting for a TMA stage */
  B200_WAIT_SGEMM_EMPTY = 1 << 1,   /* FP32 pipeline: producer waiting for a free stage */
  B200_WAIT_UMMA_FULL = 1 << 2,     /* TF32: MMA issuer waiting for operands */
  B200_WAIT_UMMA_EMPTY = 1 << 3,    /* TF32: producer waiting for a free stage */
  B200_WAIT_UMMA_ACC_FULL = 1 << 4, /* TF32: epilogue waiting for an accumulator */
  B200_WAIT_UMMA_ACC_EMPTY = 1 << 5,/* TF32: MMA issuer waiting for a drained accumulator */
  B200_WAIT_UMMA_STORE = 1 << 6,
  B200_WAIT_SELFTEST = 1 << 7,      /* b200_selftest_wait_gives_up */
  B200_WAIT_PEER_BARRIER = 1 << 8,  /* b200_peer_barrier: a peer never signalled the step */
  B200_WAIT_ROW_STAGED = 1 << 9     /* row operators: a row staged by the copy engine never arrived */
};

/*
 * Self tests of the safety plumbing; no reference counterpart. Neither faults,
 * traps or hangs anything.
 *   b200_selftest_wait_gives_up: one thread waits, with the library's bounded
 *     wait capped at `max_polls` (1 .. 2^20) polls, on a barrier that nothing
 *     completes. The kernel returns normally; *outcome (device memory, may be
 *     NULL) receives 2 ("gave up") and the next b200_device_status_read returns
 *     B200_ERR_DEVICE_TIMEOUT with B200_WAIT_SELFTEST set, the one after that
 *     B200_OK.
 *   b200_selftest_refused_launch: asks for a launch configuration the CUDA
 *     runtime refuses on the host; returns B200_ERR_LAUNCH_FAILED. The refusal
 *     must not outlive the call: the next valid launch returns B200_OK.
 */
int b200_selftest_wait_gives_up(uint32_t max_polls, uint32_t* outcome, b200_stream_t stream);
int b200_selftest_refused_launch(b200_stream_t stream);

/* ----------------------------------------------------- FP32 SIMT GEMM ladder */

/*
 * Ladder entries. C[M,N] = A[M,K] * B[K,N] in FP32 on the FMA pipe.
 * A is logical [M,K] stored column-major (element (m,k) at A[k*M + m], i.e.
 * a contiguous [K,M] array), B is row-major [K,N], C is row-major [M,N]
 * (csrc/gemm/gemm_layout.h:5-9). Full tiles only: M % bm == 0, N % bn == 0,
 * K % bk == 0 with (bm,bn,bk) from b200_sgemm_tile, all positive.
 *
 * ids 0..12 are the thirteen hand-written stages of the reference in ladder
 * order (python/cuda_ai_kernels/gemm_stages.py:4-19; launchers declared in
 * csrc/gemm/gemm.h:9-27).
 */
typedef enum b200_sgemm_impl {
  B200_SGEMM_NAIVE = 0,                  /* gemm_naive            csrc/gemm/gemm_naive.cu:36-46 */
  B200_SGEMM_BLOCK_TILE = 1,             /* gemm_block_tile       csrc/gemm/gemm_block_tile.cu:38-48 */
  B200_SGEMM_BLOCK_TILE_F4_16x16 = 2,    /* gemm_block_tile_float4_16x16  gemm_block_tile_float4.cu:38-59 */
  B200_SGEMM_BLOCK_TILE_F4_16x32 = 3,    /* gemm_block_tile_float4_16x32 */
  B200_SGEMM_BLOCK_TILE_F4_32x32 = 4,    /* gemm_block_tile_float4_32x32 */
  B200_SGEMM_THREAD_TILE_4x4 = 5,        /* gemm_thread_tile_4x4  csrc/gemm/gemm_thread_tile.cu:77-104 */
  B200_SGEMM_THREAD_TILE_4x8 = 6,        /* gemm_thread_tile_4x8 */
  B200_SGEMM_THREAD_TILE_8x8 = 7,        /* gemm_thread_tile_8x8 */
  B200_SGEMM_THREAD_TILE_8x8_WARP4x8 = 8,/* gemm_thread_tile_8x8_warp4x8 */
  B200_SGEMM_WARP_TILE = 9,              /* gemm_warp_tile        csrc/gemm/gemm_warp_tile.cu:108-119 */
  B200_SGEMM_PREFETCH_SMEM = 10,         /* gemm_prefetchSmem     csrc/gemm/gemm_prefetchSmem.cu:176-199 */
  B200_SGEMM_PREFETCH_REG = 11,          /* gemm_prefetchReg      csrc/gemm/gemm_prefetchRegister.cu:197-220 */
  B200_SGEMM_SPLIT_K = 12,               /* gemm_splictK          csrc/gemm/gemm_splictK.cu:185-209 */
  B200_SGEMM_IMPL_COUNT = 13
} b200_sgemm_impl;

/* Ladder name ("naive", "block_tile", ..., "split_k") or NULL. */
const char* b200_sgemm_impl_name(int impl);
/* Inverse of b200_sgemm_impl_name; -1 when unknown. */
int b200_sgemm_impl_from_name(const char* name);

/*
 * Tile multiples an entry requires, and whether it needs 16-byte aligned A
 * and B (all but naive and block_tile). Mirrors the (BM,BN,BK) column of
 * python/cuda_ai_kernels/gemm_stages.py:4-19 and the `vectorized` flag of
 * check_regular_gemm_inputs (csrc/gemm/gemm_regular.cuh:10-26).
 */
int b200_sgemm_tile(int impl, int* bm, int* bn, int* bk, int* needs_16b_alignment);

/*
 * Host-only validation in the order of csrc/gemm/gemm_regular.cuh:15-25:
 * positive sizes -> B200_ERR_INVALID_ARGUMENT, divisibility or grid limit ->
 * B200_ERR_INVALID_PROBLEM, pointer alignment -> B200_ERR_MISALIGNED_OPERAND.
 * Does not touch the GPU.
 */
int b200_sgemm_check(int impl, const void* a, const void* b,
                     int64_t m, int64_t n, int64_t k);

/*
 * Launch one ladder entry. For B200_SGEMM_SPLIT_K the output is cleared on
 * `stream` inside the call before the K slices are reduced into it, which is
 * what the reference does with torch::zeros (csrc/gemm/gemm_splictK.cu:201-202).
 */
int b200_sgemm(int impl, const float* a_colmajor, const float* b, float* c,
               int m, int n, int k, b200_stream_t stream);

/* ------------------------------------------- TF32 tensor-core GEMM + epilogue */

/*
 * Epilogues of csrc/adaptive_gemm/gemm_problem.h:6-15 that have kernels. With
 * z = alpha * A*B + beta * C (+ bias[n] when the problem carries a bias):
 * Linear, Relu are the two the reference implements; Gelu (exact, erf-based)
 * and the bias term are declared by the reference (EpilogueKind::Gelu, ::Bias,
 * ::BiasRelu, ::BiasGelu, parse_epilogue in adaptive_gemm.cu:39-59) but refused
 * at run time there (adaptive_gemm.cu:124-133).
 */
typedef enum b200_epilogue {
  B200_EPILOGUE_LINEAR = 0, /* D = z            */
  B200_EPILOGUE_RELU = 1,   /* D = max(0, z)    */
  B200_EPILOGUE_GELU = 2    /* D = 0.5 z (1 + erf(z / sqrt 2)) */
} b200_epilogue;

/*
 * Problem description: the POD part of GemmProblem + EpilogueDesc
 * (csrc/adaptive_gemm/gemm_problem.h:17-57). All matrices are row-major FP32:
 * A [M,K] with leading dimension lda, B [K,N] ldb, C [M,N] ldc (source, read
 * only, never dereferenced when beta == 0), D [M,N] ldd (destination).
 * `bias` is NULL or a vector of N floats added to every row before the
 * activation (EpilogueDesc::bias, gemm_problem.h:17-23).
 */
typedef struct b200_gemm_problem {
  int m, n, k;
  const float* a;
  const float* b;
  const float* c;
  float* d;
  int64_t lda, ldb, ldc, ldd;
  float alpha, beta;
  int epilogue; /* b200_epilogue */
  const float* bias;
} b200_gemm_problem;

/*
 * Registry record: KernelEntry + KernelMeta of
 * csrc/adaptive_gemm/kernel_entry.h:7-61. `id` values 2..9 are the reference's
 * KernelId enumerators in declaration order (0 = Auto, 1 = Cublas); ids >= 16
 * are configurations that exist only here: 16-19 wider / narrower tiles,
 * 20-22 CTA pairs (256 x 256), 23-26 GELU forms, 27-29 "skinny" (up to 16 rows,
 * FP32 FMA stream over B; inst_* = 1), 30-32 "splitk" (one 128 x 128 tile per
 * cluster, K split over its CTAs; supports_split_k = 1), 36-38 "swap" (operands
 * swapped for up to 16 rows), 39-41 "pair_mid" (CTA pairs on 256 x 128 tiles),
 * 42-44 "pair_splitk" (one 256 x 128 tile per cluster of CTA pairs, K split over
 * the pairs; supports_split_k = 1), 45-47 "medium" (128 x 192 tiles), 48-56
 * "width96" / "width160" / "width224" (128 x 96, 160 and 224 tiles), 57-59 "width32"
 * (128 x 32 tiles). Automatic dispatch
 * tries them first, each behind a shape gate, and then walks the reference's
 * eight entries in the reference's order.
 */
typedef struct b200_tf32_kernel_meta {
  int id;
  const char* name;       /* registry name string */
  const char* alias;      /* name accepted by the kernel= argument */
  int epilogue;           /* b200_epilogue */
  int tile_m, tile_n, tile_k;   /* CTA tile (tile_k = one pipeline stage of K) */
  int inst_m, inst_n, inst_k;   /* tcgen05.mma instruction shape */
  int stages;                   /* shared-memory pipeline depth */
  int alignment_a, alignment_b, alignment_c; /* in elements: 4 = TMA path, 1 = any */
  int supports_split_k;
} b200_tf32_kernel_meta;

enum { B200_TF32_KERNEL_AUTO = 0, B200_TF32_KERNEL_CUBLAS = 1 };

/* Number of registry entries, in dispatch order (kKernelRegistry, kernel_dispatch.cu:46-103). */
int b200_tf32_registry_size(void);
/* Fill *out with entry `index`. */
int b200_tf32_registry_entry(int index, b200_tf32_kernel_meta* out);
/* Kernel id for a kernel= string (parse_kernel, adaptive_gemm.cu:61-97); -1 when unknown. */
int b200_tf32_kernel_from_name(const char* name);

/*
 * Host-only compatibility test of one registry entry against a problem:
 * epilogue kind, then pointer / leading-dimension alignment exactly as
 * is_aligned / is_compatible do (kernel_dispatch.cu:13-44). Returns B200_OK,
 * B200_ERR_MISALIGNED_OPERAND, B200_ERR_INVALID_PROBLEM or
 * B200_ERR_NOT_SUPPORTED (epilogue mismatch). Does not touch the GPU.
 */
int b200_tf32_can_implement(int kernel_id, const b200_gemm_problem* problem);

/*
 * Launch exactly one registry entry (launch_gemm<Gemm>, kernel_launcher.h:7-29).
 * Stream order holds as for any kernel. The tensor-core entries are launched with
 * programmatic stream serialization: after another such kernel in the same stream
 * their CTAs may become resident and set themselves up early, but they touch global
 * memory only once that kernel has completed and its writes are visible, so a call
 * may consume what the call before it produced.
 */
int b200_tf32_gemm_launch(int kernel_id, const b200_gemm_problem* problem,
                          b200_stream_t stream);

/*
 * First-compatible-wins dispatch in registry order (dispatch_gemm,
 * kernel_dispatch.cu:107-136). `requested` is B200_TF32_KERNEL_AUTO or a
 * registry id. On success *chosen (may be NULL) receives the id that ran.
 */
int b200_tf32_gemm_dispatch(int requested, const b200_gemm_problem* problem,
                            int* chosen, b200_stream_t stream);

/*
 * Error-compensated TF32 ("3xTF32"): the same D = act(alpha * A*B + beta * C
 * [+ bias]) with FP32-class accuracy, as three TF32 tensor-core products
 * A*B + A_lo*B + A*B_lo where x_lo = x - (x with its 13 low mantissa bits
 * cleared, which is what the MMA unit reads). Stands in for the reference's
 * row-major tensor-core entry gemm_tensor_core (csrc/gemm/gemm_tensor_core.cu:
 * 111-137) where its element-wise bound of 3e-2 (tests/test_gemm.py:23-35) is
 * out of reach of one TF32 pass (K above about 128).
 * `scratch` is device memory of at least b200_tf32x3_scratch_bytes(m, n, k)
 * bytes, 16-byte aligned, owned by the caller (it holds A_lo and B_lo for the
 * duration of the call's work on `stream`). Four launches: one splitting pass,
 * then three dispatches through the registry. C may not alias D unless it is D.
 */
size_t b200_tf32x3_scratch_bytes(int m, int n, int k);
int b200_tf32x3_gemm(const b200_gemm_problem* problem, void* scratch,
                     size_t scratch_bytes, b200_stream_t stream);

/*
 * b200_tf32x3_gemm for callers that have no device memory to lend and may not
 * allocate any. This entry point has no counterpart in the reference. It is
 * meant for hosts whose memory is spoken for before they load this library: a
 * serving process whose framework allocator has claimed the whole GPU (a direct
 * cudaMalloc then fails or fights that allocator), a plugin that is given
 * buffers for inputs and outputs and nothing else, a latency-bound loop in
 * which the device-wide synchronisation of cudaMalloc / cudaFree is not
 * acceptable. The two lo matrices live in a fixed array inside the library
 * image instead: b200_tf32x3_static_scratch_bytes() = 8 MiB, held by every GPU
 * that loads the library until the process exits.
 *   - The caller still passes A, B, C, D as for b200_tf32x3_gemm; results are
 *     bit-identical to it.
 *   - A problem whose b200_tf32x3_scratch_bytes(m, n, k) exceeds the array
 *     (e.g. anything beyond m = n = k = 1024) returns B200_ERR_NOT_SUPPORTED
 *     and launches nothing.
 *   - The call, and everything below it, calls no cudaMalloc, cudaFree or other
 *     allocating routine.
 *   - The FIRST call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and remembers it. Make
 *     that first call during set-up, before any stream capture begins.
 *   - All calls on a device share the one array, which keeps whatever the last
 *     call wrote; nothing in it needs to start at zero (each call rewrites all
 *     it reads). Two calls whose work overlaps on the GPU (different streams, or
 *     different host threads' streams) race on it: serialise them, or use
 *     b200_tf32x3_gemm with scratch of your own.
 */
size_t b200_tf32x3_static_scratch_bytes(void);
int b200_tf32x3_gemm_static(const b200_gemm_problem* problem, b200_stream_t stream);

/* ------------------------------------------------------------ row operators */

typedef enum b200_rmsnorm_impl {
  B200_RMSNORM_NAIVE = 0,   /* rmsnorm_naive    csrc/rmsnorm/rmsnorm_naive.cu:94-109 */
  B200_RMSNORM_CACHE_X = 1  /* rmsnorm_cache_x  csrc/rmsnorm/rmsnorm_cache_x.cu:97-117 */
} b200_rmsnorm_impl;

/*
 * y[r,:] = x[r,:] * w * rsqrt(mean(x[r,:]^2) + eps), FP32, x and y row-major
 * [rows, hidden], w [hidden]. Both impl ids run single-pass kernels that read x
 * once; B200_RMSNORM_CACHE_X keeps the reference's limit of hidden <= 4096
 * (rmsnorm_cache_x.cu:110-115) and returns B200_ERR_NOT_SUPPORTED beyond it.
 */
int b200_rmsnorm(int impl, const float* x, const float* weight, float* y,
                 int64_t rows, int64_t hidden, double eps, b200_stream_t stream);

typedef enum b200_softmax_impl {
  B200_SOFTMAX_NAIVE = 0    /* softmax_naive    csrc/softmax/softmax.cu:124-133 */
} b200_softmax_impl;

/* y[r,:] = softmax(x[r,:]) over the last dimension, FP32, row-major [rows, cols]. */
int b200_softmax(int impl, const float* x, float* y,
                 int64_t rows, int64_t cols, b200_stream_t stream);

/* ------------------------------------------------------ M-sharded large GEMM */

/*
 * Row partition of an M-row GEMM over `parts` devices: part p owns rows
 * [row_begin[p], row_begin[p] + row_count[p]). Counts are multiples of
 * `granule` (the CTA tile height) except possibly the last non-empty part.
 * Host-only. The reference is single-GPU (README.md:34); this is new.
 */
int b200_shard_rows(int64_t m, int parts, int granule,
                    int64_t* row_begin, int64_t* row_count);

/*
 * Sharded GEMM fused with the all-gather of its output. Each device computes
 * its row block and the kernel's epilogue stores every finished tile not only
 * to the local output but also, with plain global stores over NVLink, to the
 * same position of up to B200_MAX_PEERS other buffers: `peer_c[i]` /
 * `peer_d[i]` is the address, in peer i's copy of the full output, where this
 * device's element (0, 0) belongs (same row pitch as the local output; the
 * caller maps the peers' buffers into this process, e.g. CUDA IPC or symmetric
 * memory, and owns the synchronisation: a peer may read its buffer once every
 * device's call has completed). Peer buffers are only ever stored to: no loads,
 * no TMA, no multicast. With n_peers == 0 the calls equal b200_sgemm and
 * b200_tf32_gemm_dispatch. The reference is single-GPU (README.md:34) and has
 * no counterpart; the partition and the optional all-gather of C are the
 * multi-GPU configuration of the benchmark.
 *   b200_sgemm_gather: impl must be B200_SGEMM_PREFETCH_SMEM or _PREFETCH_REG
 *     (B200_ERR_NOT_SUPPORTED otherwise); peer addresses 16-byte aligned.
 *   b200_tf32_gemm_dispatch_gather: registry entries that cannot fan out
 *     (the skinny FP32 entries) are skipped by automatic dispatch and refuse
 *     a forced call with B200_ERR_NOT_SUPPORTED.
 */
#define B200_MAX_PEERS 7
int b200_sgemm_gather(int impl, const float* a_colmajor, const float* b, float* c,
                      float* const* peer_c, int n_peers,
                      int m, int n, int k, b200_stream_t stream);
int b200_tf32_gemm_dispatch_gather(int requested, const b200_gemm_problem* problem,
                                   float* const* peer_d, int n_peers,
                                   int* chosen, b200_stream_t stream);

/*
 * Device-side barrier between the ranks of a fused step: "every rank's launches
 * enqueued before its barrier have completed, and their stores to the peers'
 * copies are visible". flags_by_rank[r] (host array of `world` device
 * pointers, world <= B200_MAX_PEERS + 1) is rank r's array of `world` 32-bit
 * flags, mapped into this process and zeroed once before first use;
 * flags_by_rank[rank] is this device's own. `epoch` is the step number: every
 * rank passes the same value, larger at every call (wrap-around is fine).
 * The kernel stores `epoch` into slot `rank` of every other array and waits,
 * at most `max_polls` polls (1 .. 2^24, about a third of a microsecond each)
 * per peer, for its own slots to reach it. A wait that runs out sets
 * B200_WAIT_PEER_BARRIER in the status word and the kernel returns: a rank
 * whose partner died or skipped the step does not spin on the GPU. Peer memory
 * is only stored to. One launch, capturable. No reference counterpart (the
 * reference is single-GPU, README.md:34).
 */
int b200_peer_barrier(uint32_t* const* flags_by_rank, int world, int rank,
                      uint32_t epoch, uint32_t max_polls, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_KERNELS_H_ */
