"""M-sharded large GEMM across the GPUs of one node.

C[r0:r1, :] = A[r0:r1, :] @ B needs nothing from other rows, so the rows of A
are dealt out to the ranks (one process per GPU), B is replicated, and C stays
sharded: there is no collective on the data path. Gathering the shards of C on
every rank is optional and separate (`all_gather_rows`, NCCL over NVLink on
GPUs, gloo on CPU for tests). The reference is single-GPU; this module is new.

The row plan comes from the C ABI (`b200_shard_rows`), so that a C++ host that
drives the kernels directly partitions exactly like this module does.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Callable, Optional, Sequence

import torch

_LIB: Optional[ctypes.CDLL] = None


def _abi() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parents[2] / "lib" / "libb200_kernels.so"
        lib = ctypes.CDLL(str(path))
        lib.b200_shard_rows.argtypes = [ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int64),
                                        ctypes.POINTER(ctypes.c_int64)]
        _LIB = lib
    return _LIB


def shard_rows(m: int, parts: int, granule: int = 128) -> list[tuple[int, int]]:
    """(first row, row count) per part; counts are multiples of `granule` except a ragged tail."""
    begin = (ctypes.c_int64 * parts)()
    count = (ctypes.c_int64 * parts)()
    status = _abi().b200_shard_rows(m, parts, granule, begin, count)
    if status != 0:
        raise ValueError(f"invalid shard request: m={m}, parts={parts}, granule={granule}")
    return [(int(b), int(c)) for b, c in zip(begin, count)]


def column_major_shard(a_storage: torch.Tensor, first_row: int, rows: int) -> torch.Tensor:
    """Rows [first_row, first_row + rows) of A as a column-major [rows, K] view.

    `a_storage` is the ladder's storage of A, a contiguous [K, M] array. A
    column slice of it is strided with the wrong pitch for the kernels, so the
    shard is materialised once (outside any timed region).
    """
    if a_storage.dim() != 2 or not a_storage.is_contiguous():
        raise ValueError("a_storage must be the contiguous [K, M] storage of a column-major A")
    return a_storage[:, first_row:first_row + rows].contiguous().t()


def sharded_gemm(a_shard: torch.Tensor, b: torch.Tensor, impl: str = "prefetch_reg",
                 compute: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None) -> torch.Tensor:
    """This rank's rows of C. `compute` replaces the GPU operator in CPU tests."""
    if compute is not None:
        return compute(a_shard, b)
    from cuda_ai_kernels import ops

    return ops.gemm(a_shard, b, impl=impl)


def all_gather_rows(c_shard: torch.Tensor, row_counts: Sequence[int], group=None) -> torch.Tensor:
    """Concatenates every rank's row shard of C, in rank order, on every rank."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if len(row_counts) != world:
        raise ValueError("one row count per rank is required")
    n = c_shard.shape[1]
    if len(set(row_counts)) == 1:
        out = torch.empty(sum(row_counts), n, dtype=c_shard.dtype, device=c_shard.device)
        dist.all_gather_into_tensor(out, c_shard.contiguous(), group=group)
        return out
    # Uneven shards: collectives want equal pieces, so pad to the tallest shard
    # and drop the padding after the exchange.
    tallest = max(row_counts)
    padded = torch.zeros(tallest, n, dtype=c_shard.dtype, device=c_shard.device)
    padded[:c_shard.shape[0]] = c_shard
    out = torch.empty(world * tallest, n, dtype=c_shard.dtype, device=c_shard.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * tallest:r * tallest + rows] for r, rows in enumerate(row_counts)], dim=0)
