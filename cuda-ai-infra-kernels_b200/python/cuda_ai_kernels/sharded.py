"""M-sharded large GEMM across the GPUs of one node.

C[r0:r1, :] = A[r0:r1, :] @ B needs nothing from other rows, so the rows of A
are dealt out to the ranks (one process per GPU), B is replicated, and C stays
sharded: there is no collective on the data path. Gathering the shards of C on
every rank is optional: either as a separate collective (`all_gather_rows`,
NCCL over NVLink on GPUs, gloo on CPU for tests) or fused into the GEMM
(`GatheredOutput` + `sharded_gemm_gather` / `sharded_adaptive_gemm_gather`:
the kernel's epilogue stores every finished tile into every rank's copy of C
with plain stores over NVLink, so the transfer overlaps the remaining tiles).
The reference is single-GPU; this module is new.

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
        lib.b200_peer_barrier.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_uint32,
                                          ctypes.c_uint32, ctypes.c_void_p]
        lib.b200_device_status_read.argtypes = [ctypes.POINTER(ctypes.c_uint32), ctypes.c_void_p]
        _LIB = lib
    return _LIB


def init_distributed(backend: str = "nccl", timeout_s: float = 120.0, device: Optional[torch.device] = None, **kwargs):
    """`torch.distributed.init_process_group` with every wait bounded.

    Rendezvous and communicator set-up give up after `timeout_s` instead of
    waiting for a rank that never joins, and so does every later collective of
    the group: gloo raises on the calling rank; with NCCL the process group's
    watchdog thread polls the communicator's asynchronous error state
    (`ncclCommGetAsyncError`) and, once a collective has been pending for
    `timeout_s`, aborts the communicator and ends the process with an error
    instead of leaving a kernel waiting on the GPU (PyTorch's default handling,
    `TORCH_NCCL_ASYNC_ERROR_HANDLING`, left as the caller set it).
    Rank, world size and master address come from the environment or `kwargs`.
    """
    import datetime

    import torch.distributed as dist

    if backend == "nccl" and device is not None:
        kwargs.setdefault("device_id", device)
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return dist.group.WORLD


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


# ------------------------------------------------- GEMM fused with the all-gather


def peer_row_pointers(base_ptrs: Sequence[int], rank: int, first_row: int, n: int, itemsize: int = 4) -> list[int]:
    """Addresses of row `first_row` in every OTHER rank's copy of a gathered [M, n] matrix.

    `base_ptrs[r]` is the address, valid in this process, of rank r's copy.
    These are the `peer_ptrs` the fused kernels store to (at most 7: 8 GPUs).
    """
    if not 0 <= rank < len(base_ptrs):
        raise ValueError("rank outside the pointer table")
    if len(base_ptrs) - 1 > 7:
        raise ValueError("at most 8 ranks can be gathered by the fused kernels")
    if first_row < 0 or n <= 0:
        raise ValueError("invalid row offset or width")
    offset = first_row * n * itemsize
    return [int(ptr) + offset for r, ptr in enumerate(base_ptrs) if r != rank]


WAIT_PEER_BARRIER = 1 << 8   # bit of the device status word set by a barrier that gave up


def all_ranks_ok(ok: bool, group=None) -> bool:
    """Host-side agreement: True only if every rank of `group` passed True.

    Call it (on a CPU/gloo group, or any group) with the outcome of the work
    done since the last barrier, before enqueuing the next device-side barrier:
    if a rank failed, every rank skips the barrier instead of waiting for a
    partner that will never arrive.
    """
    import torch.distributed as dist

    backend = dist.get_backend(group)
    device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


class GatheredOutput:
    """Every rank's copy of the gathered C[M, N] (FP32), mapped into every process.

    Built on torch symmetric memory (CUDA virtual-memory handles exchanged
    through the process group's store), which is plumbing only: the kernels see
    raw device addresses. Multicast (NVLS) bindings are switched off before the
    first allocation; the fused kernels use plain peer stores. Collective: every
    rank of `group` must construct it with the same shape.

    The barrier between steps is this library's own kernel (`b200_peer_barrier`):
    flag stores to the peers, bounded local waits, and a status bit instead of a
    spin when a partner never arrives.
    """

    def __init__(self, m: int, n: int, plan: Sequence[tuple[int, int]], group=None, device=None):
        import os

        import torch.distributed as dist

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if len(plan) != self.world or sum(count for _, count in plan) != m:
            raise ValueError("the row plan must cover M with one entry per rank")
        self.m, self.n, self.plan = m, n, list(plan)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.full = symm_mem.empty((m, n), dtype=torch.float32, device=device)
        self._handle = symm_mem.rendezvous(self.full, self.group)
        self.base_ptrs = [int(p) for p in self._handle.buffer_ptrs]
        first, rows = self.plan[self.rank]
        self.local_rows = self.full[first:first + rows]
        self.peer_ptrs = peer_row_pointers(self.base_ptrs, self.rank, first, n)
        # Barrier flags: one 32-bit slot per source rank, zeroed before any peer can reach them
        # (the rendezvous below is a host-side collective that follows this rank's synchronize).
        self.flags = symm_mem.empty((8,), dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._flag_handle = symm_mem.rendezvous(self.flags, self.group)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self._flag_handle.buffer_ptrs])
        self._epoch = 0

    def barrier(self, max_polls: int = 1 << 21) -> None:
        """All ranks' launches so far have completed: every copy of C is whole.

        A device-side barrier on the current stream, so no host synchronisation
        is needed between the GEMM and a consumer kernel on the same stream.
        Every rank must call it the same number of times. The wait is bounded
        (`max_polls` polls per peer, of the order of a second by default); when
        it runs out the kernel returns and `check()` reports it.
        """
        self._epoch = (self._epoch + 1) & 0xFFFFFFFF
        stream = torch.cuda.current_stream(self.full.device).cuda_stream
        status = _abi().b200_peer_barrier(self._flag_ptrs, self.world, self.rank, self._epoch, max_polls,
                                          ctypes.c_void_p(stream))
        if status != 0:
            raise RuntimeError(f"b200_peer_barrier failed with status {status}")

    def check(self) -> None:
        """Synchronises the current stream and raises if a device-side wait gave up since the last check."""
        word = ctypes.c_uint32(0)
        stream = torch.cuda.current_stream(self.full.device).cuda_stream
        status = _abi().b200_device_status_read(ctypes.byref(word), ctypes.c_void_p(stream))
        if status != 0 or word.value != 0:
            what = "a peer never reached the barrier" if word.value & WAIT_PEER_BARRIER else "a device-side wait gave up"
            raise RuntimeError(f"{what} (status {status}, wait sites {word.value:#x})")


def sharded_gemm_gather(a_shard: torch.Tensor, b: torch.Tensor, out: GatheredOutput, impl: str = "prefetch_reg") -> torch.Tensor:
    """FP32 SIMT: this rank's rows of C, written into every rank's copy. Returns the local copy.

    The copy is complete only after `out.barrier()`.
    """
    from cuda_ai_kernels import _C

    _C.gemm_gather(a_shard, b, out.local_rows, out.peer_ptrs, impl)
    return out.full


def sharded_adaptive_gemm_gather(a_rows: torch.Tensor, b: torch.Tensor, out: GatheredOutput, c: Optional[torch.Tensor] = None,
                                 bias: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
                                 epilogue: str = "linear", kernel: str = "auto") -> torch.Tensor:
    """TF32 + fused epilogue: this rank's rows of D, written into every rank's copy. Returns the local copy."""
    from cuda_ai_kernels import _C

    _C.adaptive_gemm_gather(a_rows, b, c, bias, alpha, beta, epilogue, kernel, out=out.local_rows, peer_ptrs=out.peer_ptrs)
    return out.full
