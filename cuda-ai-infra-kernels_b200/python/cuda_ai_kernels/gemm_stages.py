"""The FP32 GEMM optimisation ladder: (stage, impl name, (BM, BN, BK)).

Same names, order and tile multiples as the reference table
(python/cuda_ai_kernels/gemm_stages.py:4-21); M, N and K must be positive
multiples of the triple. The kernels behind stages 6-8 are sm_100a designs (TMA
+ mbarrier ring, packed FMAs) that keep the reference's size contract.
"""

GEMM_STAGES = (
    (1, "naive", (16, 16, 1)),
    (2, "block_tile", (16, 16, 8)),
    (3, "block_tile_float4_16x16", (16, 16, 8)),
    (3, "block_tile_float4_16x32", (16, 32, 8)),
    (3, "block_tile_float4_32x32", (32, 32, 8)),
    (4, "thread_tile_4x4", (128, 128, 8)),
    (4, "thread_tile_4x8", (128, 128, 8)),
    (4, "thread_tile_8x8", (128, 128, 8)),
    (4, "thread_tile_8x8_warp4x8", (128, 128, 8)),
    (5, "warp_tile", (128, 128, 8)),
    (6, "prefetch_smem", (128, 128, 8)),
    (7, "prefetch_reg", (128, 128, 8)),
    (8, "split_k", (128, 128, 16)),
    (9, "cublas", (1, 1, 1)),
)
GEMM_STAGE_IMPLS = tuple(name for _, name, _ in GEMM_STAGES)
# Entries that take A as a column-major [M,K] view and must receive the
# caller's tensors untouched.
COLUMN_MAJOR_IMPLS = frozenset(GEMM_STAGE_IMPLS) | {"thread_tile"}
