"""The entry point that allocates nothing: `b200_tf32x3_gemm_static`.

Some hosts of this library cannot give it device memory and cannot let it take any:
the framework around them has already claimed the GPU's memory for its own allocator,
or they are handed input and output buffers and nothing more, or they run a loop in
which the device-wide synchronisation of cudaMalloc / cudaFree has no place. For them
the error-compensated TF32 GEMM keeps its two scratch matrices in a fixed 8 MiB array
inside the library image. This file calls that entry point through the C ABI, twice in
a row on different problems (the array keeps the first call's contents, which must not
matter), and checks each result against the ordinary entry point, which takes scratch
from the caller: same kernels, same arithmetic, so the bits must be equal - far inside
the FP32 bar (1e-4 * sqrt(K) * max|A| * max|B|) that the compensated path is held to.

Collected last (the file name sorts after every other test file), so that a run that
stops at the first failure has already run everything else; it also passes on its own
in a fresh process."""
import ctypes

import pytest
import torch

from conftest import GemmProblem, assert_device_clean, current_stream_ptr
from oracle import oracle

pytestmark = pytest.mark.gpu

LINEAR, RELU = 0, 1
NOT_SUPPORTED, INVALID_ARGUMENT = 3, 4


def problem(a, b, c, d, alpha, beta, epilogue):
    m, k = a.shape
    n = b.shape[1]
    return GemmProblem(m, n, k, a.data_ptr(), b.data_ptr(), c.data_ptr() if c is not None else None, d.data_ptr(),
                       a.stride(0), b.stride(0), c.stride(0) if c is not None else n, d.stride(0), alpha, beta, epilogue, None)


def with_callers_scratch(abi, a, b, c, alpha, beta, epilogue):
    d = torch.full((a.shape[0], b.shape[1]), float("nan"), device="cuda")
    q = problem(a, b, c, d, alpha, beta, epilogue)
    need = abi.b200_tf32x3_scratch_bytes(q.m, q.n, q.k)
    scratch = torch.empty(need // 4, device="cuda")
    assert abi.b200_tf32x3_gemm(ctypes.byref(q), scratch.data_ptr(), need, current_stream_ptr()) == 0
    return d


def with_static_scratch(abi, a, b, c, alpha, beta, epilogue):
    d = torch.full((a.shape[0], b.shape[1]), float("nan"), device="cuda")
    q = problem(a, b, c, d, alpha, beta, epilogue)
    status = abi.b200_tf32x3_gemm_static(ctypes.byref(q), current_stream_ptr())
    assert status == 0, abi.b200_status_string(status)
    return d


def test_static_scratch_entry_matches_the_ordinary_one_on_two_calls_in_a_row(abi):
    assert abi.b200_tf32x3_static_scratch_bytes() == 8 << 20
    # Two different problems back to back: the second finds the first one's lo matrices in the array.
    cases = [((1024, 1024, 1024), 1.0, 0.5, RELU, 21), ((333, 520, 777), 0.75, 0.0, LINEAR, 22)]
    for (m, n, k), alpha, beta, epilogue, seed in cases:
        a, b, c = oracle.adaptive_inputs(m, n, k, seed=seed)
        a_dev, b_dev, c_dev = a.cuda(), b.cuda(), (c.cuda() if beta != 0.0 else None)
        got = with_static_scratch(abi, a_dev, b_dev, c_dev, alpha, beta, epilogue)
        want = with_callers_scratch(abi, a_dev, b_dev, c_dev, alpha, beta, epilogue)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        expected = oracle.adaptive_gemm_fp64(a, b, c if beta != 0.0 else None, alpha, beta, "relu" if epilogue == RELU else "linear")
        err = (got.cpu() - expected).abs().max().item()
        assert err <= oracle.sgemm_abs_tolerance(a, b), err
    assert_device_clean(abi)


def test_static_scratch_entry_refuses_what_does_not_fit(abi):
    a = torch.zeros(1024, 1028, device="cuda")          # one column quad too many for 8 MiB
    b = torch.zeros(1028, 1024, device="cuda")
    d = torch.full((1024, 1024), 7.0, device="cuda")
    q = problem(a, b, None, d, 1.0, 0.0, LINEAR)
    assert abi.b200_tf32x3_scratch_bytes(q.m, q.n, q.k) > abi.b200_tf32x3_static_scratch_bytes()
    assert abi.b200_tf32x3_gemm_static(ctypes.byref(q), current_stream_ptr()) == NOT_SUPPORTED
    torch.cuda.synchronize()
    assert bool((d == 7.0).all())                        # nothing was launched
    assert abi.b200_tf32x3_gemm_static(None, current_stream_ptr()) == INVALID_ARGUMENT
    assert_device_clean(abi)
