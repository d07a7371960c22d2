"""Shared pytest setup.

Markers: ``gpu`` - needs a CUDA device (skipped without one). Everything else
runs on a CPU-only machine: the oracle against its golden vectors, the host
logic of the C ABI (the library loads without a GPU), the Python wrappers
against a stub native module, and world-size-2 gloo runs of the sharded path.
"""
import ctypes
import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parents[1]
PACKAGE = REPO / "cuda-ai-infra-kernels_b200"
for path in (PACKAGE / "python", REPO):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))

KERNEL_LIB = PACKAGE / "lib" / "libb200_kernels.so"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA-capable GPU (B200)")


def pytest_runtest_setup(item):
    if "gpu" in item.keywords and not torch.cuda.is_available():
        pytest.skip("no CUDA device")


class GemmProblem(ctypes.Structure):
    """ctypes mirror of ``b200_gemm_problem`` (include/b200_kernels.h)."""

    _fields_ = [
        ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int),
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p), ("d", ctypes.c_void_p),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64), ("ldd", ctypes.c_int64),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("epilogue", ctypes.c_int),
        ("bias", ctypes.c_void_p),
    ]


class KernelMeta(ctypes.Structure):
    """ctypes mirror of ``b200_tf32_kernel_meta``."""

    _fields_ = [
        ("id", ctypes.c_int), ("name", ctypes.c_char_p), ("alias", ctypes.c_char_p), ("epilogue", ctypes.c_int),
        ("tile_m", ctypes.c_int), ("tile_n", ctypes.c_int), ("tile_k", ctypes.c_int),
        ("inst_m", ctypes.c_int), ("inst_n", ctypes.c_int), ("inst_k", ctypes.c_int),
        ("stages", ctypes.c_int),
        ("alignment_a", ctypes.c_int), ("alignment_b", ctypes.c_int), ("alignment_c", ctypes.c_int),
        ("supports_split_k", ctypes.c_int),
    ]


def load_abi() -> ctypes.CDLL:
    """Loads libb200_kernels.so and declares the signatures of its entry points."""
    if not KERNEL_LIB.exists():
        raise RuntimeError(f"{KERNEL_LIB} is missing: run `python __graft_entry__.py build` first")
    lib = ctypes.CDLL(str(KERNEL_LIB))
    c_int, c_int64, c_void_p, c_char_p = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_char_p
    int_p = ctypes.POINTER(c_int)
    lib.b200_status_string.restype = c_char_p
    lib.b200_status_string.argtypes = [c_int]
    lib.b200_build_info.restype = c_char_p
    lib.b200_device_status_read.argtypes = [ctypes.POINTER(ctypes.c_uint32), c_void_p]
    lib.b200_selftest_wait_gives_up.argtypes = [ctypes.c_uint32, c_void_p, c_void_p]
    lib.b200_selftest_refused_launch.argtypes = [c_void_p]
    lib.b200_peer_barrier.argtypes = [ctypes.POINTER(c_void_p), c_int, c_int, ctypes.c_uint32, ctypes.c_uint32, c_void_p]
    lib.b200_sgemm_impl_name.restype = c_char_p
    lib.b200_sgemm_impl_name.argtypes = [c_int]
    lib.b200_sgemm_impl_from_name.argtypes = [c_char_p]
    lib.b200_sgemm_tile.argtypes = [c_int, int_p, int_p, int_p, int_p]
    lib.b200_sgemm_check.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64]
    lib.b200_sgemm.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.b200_tf32_registry_entry.argtypes = [c_int, ctypes.POINTER(KernelMeta)]
    lib.b200_tf32_kernel_from_name.argtypes = [c_char_p]
    lib.b200_tf32_can_implement.argtypes = [c_int, ctypes.POINTER(GemmProblem)]
    lib.b200_tf32_gemm_launch.argtypes = [c_int, ctypes.POINTER(GemmProblem), c_void_p]
    lib.b200_tf32_gemm_dispatch.argtypes = [c_int, ctypes.POINTER(GemmProblem), int_p, c_void_p]
    lib.b200_tf32x3_scratch_bytes.restype = ctypes.c_size_t
    lib.b200_tf32x3_scratch_bytes.argtypes = [c_int, c_int, c_int]
    lib.b200_tf32x3_gemm.argtypes = [ctypes.POINTER(GemmProblem), c_void_p, ctypes.c_size_t, c_void_p]
    lib.b200_tf32x3_static_scratch_bytes.restype = ctypes.c_size_t
    lib.b200_tf32x3_gemm_static.argtypes = [ctypes.POINTER(GemmProblem), c_void_p]
    lib.b200_rmsnorm.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, ctypes.c_double, c_void_p]
    lib.b200_softmax.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    lib.b200_shard_rows.argtypes = [c_int64, c_int, c_int, ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]
    lib.b200_sgemm_gather.argtypes = [c_int, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_int, c_int, c_int,
                                      c_int, c_void_p]
    lib.b200_tf32_gemm_dispatch_gather.argtypes = [c_int, ctypes.POINTER(GemmProblem), ctypes.POINTER(c_void_p), c_int,
                                                   int_p, c_void_p]
    return lib


@pytest.fixture(scope="session")
def abi() -> ctypes.CDLL:
    return load_abi()


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def assert_device_clean(lib) -> None:
    """Synchronises and fails if any kernel recorded an expired device-side wait."""
    word = ctypes.c_uint32(0)
    status = lib.b200_device_status_read(ctypes.byref(word), ctypes.c_void_p(current_stream_ptr()))
    assert status == 0 and word.value == 0, f"device wait timed out, site mask {word.value:#x}"
