"""The index-checking debug build of the kernel library (`build.py --debug-bounds`).

In that build the kernels' stores and unpredicated loads are wrapped in checks
against the extents the launcher passed; a failing check sets a bit in the device
status word and skips the access. Here the small exact cases run against it: the
results must equal the release library's bit for bit, and no check may fire. It is
the stand-in, on a shared GPU, for running the kernels under a memory checker."""
import ctypes

import pytest
import torch

import conftest
from conftest import GemmProblem, PACKAGE, current_stream_ptr
from oracle import oracle

pytestmark = pytest.mark.gpu

DEBUG_LIB = PACKAGE / "lib" / "libb200_kernels_debug.so"
BOUNDS_BIT = 1 << 10


@pytest.fixture(scope="module")
def debug_abi():
    if not DEBUG_LIB.exists():
        pytest.skip("debug library not built (python build.py --debug-bounds)")
    original = conftest.KERNEL_LIB
    conftest.KERNEL_LIB = DEBUG_LIB
    try:
        return conftest.load_abi()
    finally:
        conftest.KERNEL_LIB = original


def status_word(lib):
    word = ctypes.c_uint32(0)
    lib.b200_device_status_read(ctypes.byref(word), ctypes.c_void_p(current_stream_ptr()))
    return word.value


def sgemm(lib, name, a, b):
    m, k = a.shape
    n = b.shape[1]
    c = torch.full((m, n), float("nan"), device="cuda")
    impl = lib.b200_sgemm_impl_from_name(name.encode())
    assert lib.b200_sgemm(impl, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, current_stream_ptr()) == 0
    return c


def tf32(lib, kernel, a, b, c, epilogue):
    m, k = a.shape
    n = b.shape[1]
    d = torch.full((m, n), float("nan"), device="cuda")
    q = GemmProblem(m, n, k, a.data_ptr(), b.data_ptr(), c.data_ptr(), d.data_ptr(), k, n, n, n, 1.0, 0.5, epilogue, None)
    chosen = ctypes.c_int(-1)
    status = lib.b200_tf32_gemm_dispatch(kernel, ctypes.byref(q), ctypes.byref(chosen), current_stream_ptr())
    assert status == 0, lib.b200_status_string(status)
    return d


@pytest.mark.parametrize("impl", ["prefetch_smem", "prefetch_reg", "split_k"])
@pytest.mark.parametrize("shape", [(256, 384, 80), (128, 128, 1024), (640, 768, 1104)])
def test_fp32_pipeline_under_index_checks(abi, debug_abi, impl, shape):
    m, n, k = shape
    g = torch.Generator().manual_seed(m + k)
    a = torch.randint(-3, 4, (k, m), generator=g).float().cuda().t()
    b = torch.randint(-3, 4, (k, n), generator=g).float().cuda()
    checked = sgemm(debug_abi, impl, a, b)
    assert status_word(debug_abi) & BOUNDS_BIT == 0
    assert torch.equal(checked, sgemm(abi, impl, a, b))
    torch.testing.assert_close(checked.cpu(), oracle.gemm_fp64(a, b), atol=0, rtol=0)


@pytest.mark.parametrize("kernel,shape", [(0, (256, 256, 96)), (20, (700, 1000, 1100)), (3, (33, 65, 17)), (3, (300, 270, 130)),
                                          (16, (256, 512, 96)), (18, (200, 264, 100)), (30, (64, 256, 1024))])
def test_tf32_kernels_under_index_checks(abi, debug_abi, kernel, shape):
    m, n, k = shape
    g = torch.Generator().manual_seed(m + 3 * n + k)
    a = torch.randint(-3, 4, (m, k), generator=g).float().cuda()
    b = torch.randint(-3, 4, (k, n), generator=g).float().cuda()
    c = torch.randint(-8, 9, (m, n), generator=g).float().cuda()
    checked = tf32(debug_abi, kernel, a, b, c, 0)
    assert status_word(debug_abi) & BOUNDS_BIT == 0
    assert torch.equal(checked, tf32(abi, kernel, a, b, c, 0))
    torch.testing.assert_close(checked.cpu(), oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, "linear"), atol=0, rtol=0)
